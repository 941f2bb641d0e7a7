// Split-sign product of bounds with a constant weight, exact-fp32 path (CUDA-core FFMA).
//
//   y_lw = x_lw W+ + x_uw W-        y_uw = x_lw W- + x_uw W+       (Bounds.py:403-412)
//
// is evaluated in centre/radius form, which needs half the multiply-adds:
//   c = (x_lw + x_uw)/2, r = (x_uw - x_lw)/2,  y_c = c W,  y_r = r |W|,
//   y_lw = y_c - y_r,  y_uw = y_c + y_r.
// Every product and accumulation is fp32, so the result has the error class of the reference's
// fp32 GEMMs (different summation order, one extra rounding for c and r).
//
// Tiling: 128 x 128 output tile per block, K in steps of 16, 256 threads with an 8 x 8 micro
// tile and two accumulators (centre, radius) each; global loads of the next K step are issued
// into registers before the current step is computed (two shared-memory stages).
#include <cooperative_groups.h>

#include "common.cuh"

namespace fb {
namespace {

constexpr int BM = 128, BN = 128, BK = 16;
constexpr int LD = BM + 4;  // padded leading dimension of the k-major shared tiles
constexpr int kThreads = 256;
constexpr int kStageFloats = 3 * BK * LD;  // centre, radius, weight

// A: [M, K] row-major (two of them: lower and upper side); W: [N, K] row-major.
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
split_sign_gemm_ffma(const float* __restrict__ a_lo, const float* __restrict__ a_up,
                     const float* __restrict__ W, const float* __restrict__ bias,
                     float* __restrict__ c_lo, float* __restrict__ c_up, int64_t M, int N, int K, int split_rows,
                     int split_d) {
  extern __shared__ __align__(16) float smem[];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = (int64_t)blockIdx.x * BM;
  const int n0 = blockIdx.y * BN;

  float acc_c[8][8], acc_r[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc_c[i][j] = 0.f; acc_r[i][j] = 0.f; }

  // global -> register staging: 2 float4 per thread per operand
  float4 g_lo[2], g_up[2], g_w[2];
  auto load_tile = [&](int k0) {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int f = tid + kThreads * q;
      const int r = f >> 2, kk = k0 + (f & 3) * 4;
      const int64_t m = m0 + r;
      const int n = n0 + r;
      float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), up = lo, w = lo;
      if (VEC) {
        if (kk < K) {
          if (m < M) {
            lo = __ldg(reinterpret_cast<const float4*>(a_lo + m * K + kk));
            up = __ldg(reinterpret_cast<const float4*>(a_up + m * K + kk));
          }
          if (n < N) w = __ldg(reinterpret_cast<const float4*>(W + (int64_t)n * K + kk));
        }
      } else {
        float tl[4] = {0.f, 0.f, 0.f, 0.f}, tu[4] = {0.f, 0.f, 0.f, 0.f}, tw[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (kk + e < K) {
            if (m < M) { tl[e] = __ldg(a_lo + m * K + kk + e); tu[e] = __ldg(a_up + m * K + kk + e); }
            if (n < N) tw[e] = __ldg(W + (int64_t)n * K + kk + e);
          }
        }
        lo = make_float4(tl[0], tl[1], tl[2], tl[3]);
        up = make_float4(tu[0], tu[1], tu[2], tu[3]);
        w = make_float4(tw[0], tw[1], tw[2], tw[3]);
      }
      g_lo[q] = lo; g_up[q] = up; g_w[q] = w;
    }
  };
  auto store_tile = [&](int stage) {
    float* s_c = smem + stage * kStageFloats;
    float* s_r = s_c + BK * LD;
    float* s_w = s_r + BK * LD;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int f = tid + kThreads * q;
      const int r = f >> 2, kq = (f & 3) * 4;
      const float lo[4] = {g_lo[q].x, g_lo[q].y, g_lo[q].z, g_lo[q].w};
      const float up[4] = {g_up[q].x, g_up[q].y, g_up[q].z, g_up[q].w};
      const float w[4] = {g_w[q].x, g_w[q].y, g_w[q].z, g_w[q].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s_c[(kq + e) * LD + r] = fmul(fadd(lo[e], up[e]), 0.5f);
        s_r[(kq + e) * LD + r] = fmul(fsub(up[e], lo[e]), 0.5f);
        s_w[(kq + e) * LD + r] = w[e];
      }
    }
  };

  const int ktiles = (K + BK - 1) / BK;
  load_tile(0);
  store_tile(0);
  __syncthreads();
  for (int t = 0; t < ktiles; ++t) {
    const int cur = t & 1;
    if (t + 1 < ktiles) load_tile((t + 1) * BK);
    const float* s_c = smem + cur * kStageFloats;
    const float* s_r = s_c + BK * LD;
    const float* s_w = s_r + BK * LD;
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float ac[8], ar[8], w[8], wa[8];
      *reinterpret_cast<float4*>(ac) = *reinterpret_cast<const float4*>(s_c + k * LD + ty * 4);
      *reinterpret_cast<float4*>(ac + 4) = *reinterpret_cast<const float4*>(s_c + k * LD + 64 + ty * 4);
      *reinterpret_cast<float4*>(ar) = *reinterpret_cast<const float4*>(s_r + k * LD + ty * 4);
      *reinterpret_cast<float4*>(ar + 4) = *reinterpret_cast<const float4*>(s_r + k * LD + 64 + ty * 4);
      *reinterpret_cast<float4*>(w) = *reinterpret_cast<const float4*>(s_w + k * LD + tx * 4);
      *reinterpret_cast<float4*>(w + 4) = *reinterpret_cast<const float4*>(s_w + k * LD + 64 + tx * 4);
#pragma unroll
      for (int j = 0; j < 8; ++j) wa[j] = fabsf(w[j]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc_c[i][j] = fmaf(ac[i], w[j], acc_c[i][j]);
          acc_r[i][j] = fmaf(ar[i], wa[j], acc_r[i][j]);
        }
    }
    if (t + 1 < ktiles) store_tile(cur ^ 1);
    __syncthreads();
  }

  // epilogue: y_lo = centre - radius, y_up = centre + radius (+ bias)
  // split_rows > 0: head-split store, element (m, n) goes to [(g * H + h), r, f] with g = m / split_rows,
  // r = m % split_rows, h = n / split_d, f = n % split_d (H = N / split_d)
  const bool vec_out = split_rows == 0 && (N % 4 == 0) && aligned16(c_lo) && aligned16(c_up);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = n0 + h * 64 + tx * 4;
      float lo[4], up[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float b = (bias != nullptr && n + e < N) ? bias[n + e] : 0.f;
        lo[e] = fsub(acc_c[i][h * 4 + e], acc_r[i][h * 4 + e]);
        up[e] = fadd(acc_c[i][h * 4 + e], acc_r[i][h * 4 + e]);
        if (bias != nullptr) { lo[e] = fadd(lo[e], b); up[e] = fadd(up[e], b); }
      }
      if (vec_out && n + 3 < N) {
        *reinterpret_cast<float4*>(c_lo + m * N + n) = make_float4(lo[0], lo[1], lo[2], lo[3]);
        *reinterpret_cast<float4*>(c_up + m * N + n) = make_float4(up[0], up[1], up[2], up[3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (n + e < N) {
            int64_t o = m * N + n + e;
            if (split_rows > 0) {
              const int64_t g = m / split_rows, r = m % split_rows;
              const int hh = (n + e) / split_d, f = (n + e) % split_d;
              o = ((g * (N / split_d) + hh) * split_rows + r) * split_d + f;
            }
            c_lo[o] = lo[e];
            c_up[o] = up[e];
          }
      }
    }
  }
}

// Narrow outputs (N <= 16, e.g. a classifier head): one warp per row of A, lanes across K,
// each lane accumulates all N outputs; HBM-bound on reading A once.
template <int NMAX>
__global__ void __launch_bounds__(kThreads)
split_sign_gemv_rows(const float* __restrict__ a_lo, const float* __restrict__ a_up,
                     const float* __restrict__ W, const float* __restrict__ bias,
                     float* __restrict__ c_lo, float* __restrict__ c_up, int64_t M, int N, int K) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t m = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); m < M; m += warps) {
    float sc[NMAX], sr[NMAX];
#pragma unroll
    for (int n = 0; n < NMAX; ++n) { sc[n] = 0.f; sr[n] = 0.f; }
    for (int k = lane; k < K; k += 32) {
      const float lo = __ldg(a_lo + m * K + k), up = __ldg(a_up + m * K + k);
      const float c = fmul(fadd(lo, up), 0.5f), r = fmul(fsub(up, lo), 0.5f);
#pragma unroll
      for (int n = 0; n < NMAX; ++n) {
        if (n < N) {
          const float w = __ldg(W + (int64_t)n * K + k);
          sc[n] = fmaf(c, w, sc[n]);
          sr[n] = fmaf(r, fabsf(w), sr[n]);
        }
      }
    }
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) {
        sc[n] += __shfl_xor_sync(0xffffffffu, sc[n], s);
        sr[n] += __shfl_xor_sync(0xffffffffu, sr[n], s);
      }
    }
    if (lane == 0) {
#pragma unroll
      for (int n = 0; n < NMAX; ++n) {
        if (n < N) {
          float lo = fsub(sc[n], sr[n]), up = fadd(sc[n], sr[n]);
          if (bias != nullptr) { lo = fadd(lo, bias[n]); up = fadd(up, bias[n]); }
          c_lo[m * N + n] = lo;
          c_up[m * N + n] = up;
        }
      }
    }
  }
}

// Narrow outputs with a long contraction (e.g. the 8192 -> 10 head of the CNN): a block owns eight
// rows of A (one per warp) and walks K in chunks of 512.  The chunk of W is staged in shared memory once per block
// (cp.async into the other of two buffers while the current chunk is computed) and read by all eight warps; the
// rows of A are read with 128-bit loads, the next chunk's into registers before the current one is used, so that a
// warp keeps 8 KB of loads in flight.  Dynamic shared memory: 2 * NMAX * 512 floats.
constexpr int kGemvChunk = 512;
__device__ __forceinline__ void gemv_cp16(float* dst, const float* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are zero-filled and nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
template <int NMAX>
__global__ void __launch_bounds__(kThreads)
split_sign_gemv_tiled(const float* __restrict__ a_lo, const float* __restrict__ a_up,
                      const float* __restrict__ W, const float* __restrict__ bias,
                      float* __restrict__ c_lo, float* __restrict__ c_up, int64_t M, int N, int K) {
  extern __shared__ __align__(16) float gemv_sw[];   // [2][NMAX][kGemvChunk]
  constexpr int J = kGemvChunk / 128;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t m = (int64_t)blockIdx.x * (kThreads / 32) + warp;
  auto stage_w = [&](int buf, int k0) {
    const int kc = min(kGemvChunk, K - k0);   // multiple of 4
    for (int f = threadIdx.x; f < NMAX * (kGemvChunk / 4); f += kThreads) {
      const int n = f / (kGemvChunk / 4), k4 = (f % (kGemvChunk / 4)) * 4;
      const bool ok = n < N && k4 < kc;
      gemv_cp16(gemv_sw + ((size_t)buf * NMAX + n) * kGemvChunk + k4, ok ? W + (int64_t)n * K + k0 + k4 : W, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto load_a = [&](float4 (&lo)[J], float4 (&up)[J], int k0) {
    const int kc = min(kGemvChunk, K - k0);
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int k4 = lane * 4 + j * 128;
      if (m < M && k0 < K && k4 < kc) {
        lo[j] = __ldg(reinterpret_cast<const float4*>(a_lo + m * K + k0 + k4));
        up[j] = __ldg(reinterpret_cast<const float4*>(a_up + m * K + k0 + k4));
      } else {
        lo[j] = make_float4(0.f, 0.f, 0.f, 0.f);   // exact zeros: they leave the sums as they are
        up[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  };
  float sc[NMAX], sr[NMAX];
#pragma unroll
  for (int n = 0; n < NMAX; ++n) { sc[n] = 0.f; sr[n] = 0.f; }
  float4 lo[J], up[J], nlo[J], nup[J];
  stage_w(0, 0);
  load_a(lo, up, 0);
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += kGemvChunk, buf ^= 1) {
    const bool more = k0 + kGemvChunk < K;
    if (more) stage_w(buf ^ 1, k0 + kGemvChunk);
    load_a(nlo, nup, k0 + kGemvChunk);
    if (more) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const float* sw = gemv_sw + (size_t)buf * NMAX * kGemvChunk;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int k4 = lane * 4 + j * 128;
      const float c[4] = {fmul(fadd(lo[j].x, up[j].x), 0.5f), fmul(fadd(lo[j].y, up[j].y), 0.5f),
                          fmul(fadd(lo[j].z, up[j].z), 0.5f), fmul(fadd(lo[j].w, up[j].w), 0.5f)};
      const float r[4] = {fmul(fsub(up[j].x, lo[j].x), 0.5f), fmul(fsub(up[j].y, lo[j].y), 0.5f),
                          fmul(fsub(up[j].z, lo[j].z), 0.5f), fmul(fsub(up[j].w, lo[j].w), 0.5f)};
#pragma unroll
      for (int n = 0; n < NMAX; ++n) {
        if (n < N) {
          const float4 w = *reinterpret_cast<const float4*>(sw + n * kGemvChunk + k4);
          sc[n] = fmaf(c[0], w.x, sc[n]); sr[n] = fmaf(r[0], fabsf(w.x), sr[n]);
          sc[n] = fmaf(c[1], w.y, sc[n]); sr[n] = fmaf(r[1], fabsf(w.y), sr[n]);
          sc[n] = fmaf(c[2], w.z, sc[n]); sr[n] = fmaf(r[2], fabsf(w.z), sr[n]);
          sc[n] = fmaf(c[3], w.w, sc[n]); sr[n] = fmaf(r[3], fabsf(w.w), sr[n]);
        }
      }
    }
    __syncthreads();   // everyone is done with this buffer before the chunk after next is staged into it
#pragma unroll
    for (int j = 0; j < J; ++j) { lo[j] = nlo[j]; up[j] = nup[j]; }
  }
  if (m >= M) return;
#pragma unroll
  for (int n = 0; n < NMAX; ++n) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      sc[n] += __shfl_xor_sync(0xffffffffu, sc[n], s);
      sr[n] += __shfl_xor_sync(0xffffffffu, sr[n], s);
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      if (n < N) {
        float lo1 = fsub(sc[n], sr[n]), up1 = fadd(sc[n], sr[n]);
        if (bias != nullptr) { lo1 = fadd(lo1, bias[n]); up1 = fadd(up1, bias[n]); }
        c_lo[m * N + n] = lo1;
        c_up[m * N + n] = up1;
      }
    }
  }
}

// A few rows with a long contraction (the bias row of the CNN head, M = 1): a cluster of kGemvSplit blocks per row, each
// taking a contiguous part of K interleaved over its threads; partial sums are combined inside each warp, over the
// warps in warp order, and over the blocks in block order by block 0 through distributed shared memory.
constexpr int kGemvSplit = 8;
template <int NMAX>
__global__ void __launch_bounds__(kThreads)
split_sign_gemv_block(const float* __restrict__ a_lo, const float* __restrict__ a_up, const float* __restrict__ W,
                      const float* __restrict__ bias, float* __restrict__ c_lo, float* __restrict__ c_up, int N, int K) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float s_red[2][kThreads / 32][NMAX];
  __shared__ float s_part[2][NMAX];
  const unsigned cr = cluster.block_rank();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t m = blockIdx.x / kGemvSplit;
  const int chunk = (K + kGemvSplit - 1) / kGemvSplit;
  const int k_begin = min(K, (int)cr * chunk), k_end = min(K, k_begin + chunk);
  float sc[NMAX], sr[NMAX];
#pragma unroll
  for (int n = 0; n < NMAX; ++n) { sc[n] = 0.f; sr[n] = 0.f; }
#pragma unroll 4
  for (int k = k_begin + threadIdx.x; k < k_end; k += kThreads) {
    const float lo = __ldg(a_lo + m * K + k), up = __ldg(a_up + m * K + k);
    const float c = fmul(fadd(lo, up), 0.5f), r = fmul(fsub(up, lo), 0.5f);
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      if (n < N) {
        const float w = __ldg(W + (int64_t)n * K + k);
        sc[n] = fmaf(c, w, sc[n]);
        sr[n] = fmaf(r, fabsf(w), sr[n]);
      }
    }
  }
#pragma unroll
  for (int n = 0; n < NMAX; ++n) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      sc[n] += __shfl_xor_sync(0xffffffffu, sc[n], s);
      sr[n] += __shfl_xor_sync(0xffffffffu, sr[n], s);
    }
    if (lane == 0) { s_red[0][warp][n] = sc[n]; s_red[1][warp][n] = sr[n]; }
  }
  __syncthreads();
  if (threadIdx.x < NMAX) {
    const int n = threadIdx.x;
    float c = s_red[0][0][n], r = s_red[1][0][n];
    for (int w = 1; w < kThreads / 32; ++w) { c = fadd(c, s_red[0][w][n]); r = fadd(r, s_red[1][w][n]); }
    s_part[0][n] = c;
    s_part[1][n] = r;
  }
  cluster.sync();
  if (cr == 0 && threadIdx.x < N) {
    const int n = threadIdx.x;
    float c = s_part[0][n], r = s_part[1][n];
    for (unsigned b = 1; b < kGemvSplit; ++b) {
      const float* rp = cluster.map_shared_rank(&s_part[0][0], b);
      c = fadd(c, rp[n]);
      r = fadd(r, rp[NMAX + n]);
    }
    float lo = fsub(c, r), up = fadd(c, r);
    if (bias != nullptr) { lo = fadd(lo, bias[n]); up = fadd(up, bias[n]); }
    c_lo[m * N + n] = lo;
    c_up[m * N + n] = up;
  }
  cluster.sync();   // the other blocks' shared memory stays alive until block 0 has read it
}

}  // namespace

// One split-sign GEMM: (a_lo, a_up) [M, K] x W[N, K]^T (+ bias) -> (c_lo, c_up) [M, N].
int launch_split_sign_ffma(const float* a_lo, const float* a_up, const float* W, const float* bias, float* c_lo,
                           float* c_up, int64_t M, int N, int K, cudaStream_t st, int split_rows, int split_d) {
  if (M == 0 || N == 0) return FB_OK;
  if (N <= 16 && split_rows == 0 && K >= 2048 && M <= 32) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(M * kGemvSplit));
    cfg.blockDim = dim3(kThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kGemvSplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FB_CUDA_OK(cudaLaunchKernelEx(&cfg, split_sign_gemv_block<16>, a_lo, a_up, W, bias, c_lo, c_up, N, K));
    count_launches(1);
    return FB_OK;
  }
  if (N <= 16 && split_rows == 0 && K >= 1024 && K % 4 == 0 && aligned16(a_lo) && aligned16(a_up) && aligned16(W) &&
      ceil_div(M, kThreads / 32) <= 0x7fffffff) {
    const size_t gemv_smem = sizeof(float) * 2 * 16 * kGemvChunk;
    if (int rc = ensure_dynamic_smem(split_sign_gemv_tiled<16>, gemv_smem)) return rc;
    split_sign_gemv_tiled<16><<<(unsigned)ceil_div(M, kThreads / 32), kThreads, gemv_smem, st>>>(a_lo, a_up, W, bias, c_lo, c_up, M, N, K);
    FB_LAUNCH_OK();
    return FB_OK;
  }
  if (N <= 16 && split_rows == 0) {
    const int64_t want = ceil_div(M, kThreads / 32);
    const int64_t cap = (int64_t)device_info().sms * 16;
    const unsigned blocks = (unsigned)(want < cap ? want : cap);
    split_sign_gemv_rows<16><<<blocks, kThreads, 0, st>>>(a_lo, a_up, W, bias, c_lo, c_up, M, N, K);
    FB_LAUNCH_OK();
    return FB_OK;
  }
  const int64_t gm = ceil_div(M, BM);
  const int gn = (int)ceil_div(N, BN);
  if (gm > 0x7fffffff || gn > 65535) return FB_ERR_SHAPE;
  const size_t smem = sizeof(float) * 2 * kStageFloats;
  const bool vec = K % 4 == 0 && aligned16(a_lo) && aligned16(a_up) && aligned16(W);
  if (vec) {
    if (int rc = ensure_dynamic_smem(split_sign_gemm_ffma<true>, smem)) return rc;
    split_sign_gemm_ffma<true><<<dim3((unsigned)gm, gn), kThreads, smem, st>>>(a_lo, a_up, W, bias, c_lo, c_up, M, N, K, split_rows, split_d);
  } else {
    if (int rc = ensure_dynamic_smem(split_sign_gemm_ffma<false>, smem)) return rc;
    split_sign_gemm_ffma<false><<<dim3((unsigned)gm, gn), kThreads, smem, st>>>(a_lo, a_up, W, bias, c_lo, c_up, M, N, K, split_rows, split_d);
  }
  FB_LAUNCH_OK();
  return FB_OK;
}

}  // namespace fb
