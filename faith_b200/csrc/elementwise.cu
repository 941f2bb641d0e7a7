// Exact (relaxation-free) operators on bounds: add, scalar multiply, feature-axis sum,
// layer normalisation without variance, head split / merge.  All are single-pass HBM-bound
// kernels with 128-bit accesses where the shapes allow.
#include "common.cuh"

namespace fb {
namespace {

constexpr int kThreads = 256;

inline unsigned stream_blocks(int64_t work_items) {
  // enough blocks to fill the machine a few times over; grid-stride loops cover the rest
  const int64_t want = ceil_div(work_items, kThreads);
  const int64_t cap = (int64_t)device_info().sms * 16;
  return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
}

// z = x + y over two (pointer, count) segments per side: the weight tensors and the bias tensors.
template <int VEC>
__global__ void __launch_bounds__(kThreads)
add_kernel(const float* __restrict__ xa, const float* __restrict__ ya, float* __restrict__ za,
           const float* __restrict__ xb, const float* __restrict__ yb, float* __restrict__ zb,
           int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i * VEC < n; i += stride) {
    if (VEC == 4) {
      const float4 a = reinterpret_cast<const float4*>(xa)[i], b = reinterpret_cast<const float4*>(ya)[i];
      const float4 c = reinterpret_cast<const float4*>(xb)[i], d = reinterpret_cast<const float4*>(yb)[i];
      reinterpret_cast<float4*>(za)[i] = make_float4(fadd(a.x, b.x), fadd(a.y, b.y), fadd(a.z, b.z), fadd(a.w, b.w));
      reinterpret_cast<float4*>(zb)[i] = make_float4(fadd(c.x, d.x), fadd(c.y, d.y), fadd(c.z, d.z), fadd(c.w, d.w));
    } else {
      za[i] = fadd(xa[i], ya[i]);
      zb[i] = fadd(xb[i], yb[i]);
    }
  }
}

// za = c * xa, zb = c * xb (the caller swaps the sides for c <= 0)
template <int VEC>
__global__ void __launch_bounds__(kThreads)
scale_kernel(const float* __restrict__ xa, float* __restrict__ za, const float* __restrict__ xb,
             float* __restrict__ zb, float c, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i * VEC < n; i += stride) {
    if (VEC == 4) {
      const float4 a = reinterpret_cast<const float4*>(xa)[i], b = reinterpret_cast<const float4*>(xb)[i];
      reinterpret_cast<float4*>(za)[i] = make_float4(fmul(a.x, c), fmul(a.y, c), fmul(a.z, c), fmul(a.w, c));
      reinterpret_cast<float4*>(zb)[i] = make_float4(fmul(b.x, c), fmul(b.y, c), fmul(b.z, c), fmul(b.w, c));
    } else {
      za[i] = fmul(xa[i], c);
      zb[i] = fmul(xb[i], c);
    }
  }
}

// One warp per feature row of length Do.  Rows [0, n_w) come from the weight tensors (lw, uw),
// rows [n_w, n_w + n_b) from the bias tensors (lb, ub).
struct RowPtrs {
  const float *x_l, *x_u, *r_l, *r_u;
  float *z_l, *z_u;
};

__device__ __forceinline__ RowPtrs pick_rows(int64_t row, int64_t n_w, int Do,
                                             const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                             const float* r_lw, const float* r_uw, const float* r_lb, const float* r_ub,
                                             float* z_lw, float* z_uw, float* z_lb, float* z_ub, bool& is_bias) {
  RowPtrs q;
  is_bias = row >= n_w;
  const size_t o = (size_t)(is_bias ? row - n_w : row) * Do;
  q.x_l = (is_bias ? x_lb : x_lw) + o;
  q.x_u = (is_bias ? x_ub : x_uw) + o;
  q.r_l = r_lw ? (is_bias ? r_lb : r_lw) + o : nullptr;
  q.r_u = r_uw ? (is_bias ? r_ub : r_uw) + o : nullptr;
  q.z_l = (is_bias ? z_lb : z_lw) + o;
  q.z_u = (is_bias ? z_ub : z_uw) + o;
  return q;
}

__global__ void __launch_bounds__(kThreads)
rowsum_kernel(const float* __restrict__ x_lw, const float* __restrict__ x_uw, const float* __restrict__ x_lb,
              const float* __restrict__ x_ub, float* __restrict__ z_lw, float* __restrict__ z_uw,
              float* __restrict__ z_lb, float* __restrict__ z_ub, int64_t n_w, int64_t n_b, int Do) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); row < n_w + n_b; row += warps) {
    bool is_bias;
    const RowPtrs q = pick_rows(row, n_w, Do, x_lw, x_uw, x_lb, x_ub, nullptr, nullptr, nullptr, nullptr,
                                z_lw, z_uw, z_lb, z_ub, is_bias);
    float sl = 0.f, su = 0.f;
    for (int j = lane; j < Do; j += 32) { sl += q.x_l[j]; su += q.x_u[j]; }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      sl += __shfl_xor_sync(0xffffffffu, sl, s);
      su += __shfl_xor_sync(0xffffffffu, su, s);
    }
    for (int j = lane; j < Do; j += 32) { q.z_l[j] = sl; q.z_u[j] = su; }
  }
}

__global__ void __launch_bounds__(kThreads)
layernorm_novar_kernel(const float* __restrict__ x_lw, const float* __restrict__ x_uw,
                       const float* __restrict__ x_lb, const float* __restrict__ x_ub,
                       const float* __restrict__ r_lw, const float* __restrict__ r_uw,
                       const float* __restrict__ r_lb, const float* __restrict__ r_ub,
                       const float* __restrict__ gamma, const float* __restrict__ beta,
                       float* __restrict__ z_lw, float* __restrict__ z_uw, float* __restrict__ z_lb,
                       float* __restrict__ z_ub, int64_t n_w, int64_t n_b, int Do) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  const float inv_n = 1.0f / (float)Do;
  for (int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); row < n_w + n_b; row += warps) {
    bool is_bias;
    const RowPtrs q = pick_rows(row, n_w, Do, x_lw, x_uw, x_lb, x_ub, r_lw, r_uw, r_lb, r_ub,
                                z_lw, z_uw, z_lb, z_ub, is_bias);
    // mean of each side: sum_k t_k * (1/n), as the reference's product with a constant 1/n matrix
    float ml = 0.f, mu = 0.f;
    for (int j = lane; j < Do; j += 32) {
      float a = q.x_l[j], b = q.x_u[j];
      if (q.r_l) { a = fadd(a, q.r_l[j]); b = fadd(b, q.r_u[j]); }
      ml = fmaf(a, inv_n, ml);
      mu = fmaf(b, inv_n, mu);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      ml += __shfl_xor_sync(0xffffffffu, ml, s);
      mu += __shfl_xor_sync(0xffffffffu, mu, s);
    }
    for (int j = lane; j < Do; j += 32) {
      float a = q.x_l[j], b = q.x_u[j];
      if (q.r_l) { a = fadd(a, q.r_l[j]); b = fadd(b, q.r_u[j]); }
      const float cl = fsub(a, mu);  // lower line minus the mean of the upper line
      const float cu = fsub(b, ml);
      const float g = gamma[j];
      const float gp = (g > 0.f) ? g : 0.f;
      const float gn = fsub(g, gp);
      float ol = fadd(fmul(cl, gp), fmul(cu, gn));
      float ou = fadd(fmul(cl, gn), fmul(cu, gp));
      if (is_bias) { ol = fadd(ol, beta[j]); ou = fadd(ou, beta[j]); }
      q.z_l[j] = ol;
      q.z_u[j] = ou;
    }
  }
}

// The same operator for Do == 128 (the model width of the headline encoder): a warp owns a row, every lane
// four consecutive features, so each tensor is touched by one 128-bit access per lane and the row stays in
// registers between the mean and the rescale (the general kernel reads it twice with 32-bit accesses).
template <bool kResidual>
__global__ void __launch_bounds__(kThreads)
layernorm_novar_row128_kernel(const float* __restrict__ x_lw, const float* __restrict__ x_uw,
                              const float* __restrict__ x_lb, const float* __restrict__ x_ub,
                              const float* __restrict__ r_lw, const float* __restrict__ r_uw,
                              const float* __restrict__ r_lb, const float* __restrict__ r_ub,
                              const float* __restrict__ gamma, const float* __restrict__ beta,
                              float* __restrict__ z_lw, float* __restrict__ z_uw, float* __restrict__ z_lb,
                              float* __restrict__ z_ub, int64_t n_w, int64_t n_b, float* __restrict__ rowsum) {
  constexpr int Do = 128;
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  const float inv_n = 1.0f / (float)Do;
  const float4 g4 = __ldg(reinterpret_cast<const float4*>(gamma) + lane);
  const float4 b4 = __ldg(reinterpret_cast<const float4*>(beta) + lane);
  const float g[4] = {g4.x, g4.y, g4.z, g4.w}, be[4] = {b4.x, b4.y, b4.z, b4.w};
  float gp[4], gn[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) { gp[e] = (g[e] > 0.f) ? g[e] : 0.f; gn[e] = fsub(g[e], gp[e]); }
  for (int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); row < n_w + n_b; row += warps) {
    bool is_bias;
    const RowPtrs q = pick_rows(row, n_w, Do, x_lw, x_uw, x_lb, x_ub, r_lw, r_uw, r_lb, r_ub,
                                z_lw, z_uw, z_lb, z_ub, is_bias);
    const float4 a4 = reinterpret_cast<const float4*>(q.x_l)[lane];
    const float4 c4 = reinterpret_cast<const float4*>(q.x_u)[lane];
    float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {c4.x, c4.y, c4.z, c4.w};
    if (kResidual) {
      const float4 ra = reinterpret_cast<const float4*>(q.r_l)[lane];
      const float4 rb = reinterpret_cast<const float4*>(q.r_u)[lane];
      a[0] = fadd(a[0], ra.x); a[1] = fadd(a[1], ra.y); a[2] = fadd(a[2], ra.z); a[3] = fadd(a[3], ra.w);
      b[0] = fadd(b[0], rb.x); b[1] = fadd(b[1], rb.y); b[2] = fadd(b[2], rb.z); b[3] = fadd(b[3], rb.w);
    }
    // mean of each side: sum_k t_k * (1/n), as the reference's product with a constant 1/n matrix
    float ml = 0.f, mu = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) { ml = fmaf(a[e], inv_n, ml); mu = fmaf(b[e], inv_n, mu); }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      ml += __shfl_xor_sync(0xffffffffu, ml, s);
      mu += __shfl_xor_sync(0xffffffffu, mu, s);
    }
    float ol[4], ou[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float cl = fsub(a[e], mu);  // lower line minus the mean of the upper line
      const float cu = fsub(b[e], ml);
      ol[e] = fadd(fmul(cl, gp[e]), fmul(cu, gn[e]));
      ou[e] = fadd(fmul(cl, gn[e]), fmul(cu, gp[e]));
      if (is_bias) { ol[e] = fadd(ol[e], be[e]); ou[e] = fadd(ou[e], be[e]); }
    }
    reinterpret_cast<float4*>(q.z_l)[lane] = make_float4(ol[0], ol[1], ol[2], ol[3]);
    reinterpret_cast<float4*>(q.z_u)[lane] = make_float4(ou[0], ou[1], ou[2], ou[3]);
    if (rowsum != nullptr) {
      // row sums of the result, for a product that takes it as its residual and applies the next layer norm in its
      // epilogue: [2 lines][4 partial sums][n_w + n_b], the whole sum in the first partial sum of each line (the other
      // three are not written: the caller keeps them zero)
      float sl = fadd(fadd(ol[0], ol[1]), fadd(ol[2], ol[3])), su = fadd(fadd(ou[0], ou[1]), fadd(ou[2], ou[3]));
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) {
        sl += __shfl_xor_sync(0xffffffffu, sl, s);
        su += __shfl_xor_sync(0xffffffffu, su, s);
      }
      if (lane == 0) {   // (the other three partial sums of each line stay zero: the caller cleared them)
        rowsum[row] = sl;
        rowsum[4 * (n_w + n_b) + row] = su;
      }
    }
  }
}

// Head split / merge: pure index permutations with the head dimension d contiguous on both
// sides.  One thread per group of VEC consecutive features.
//   split: src [B, L, M, H, d] -> dst [B, H, L, M, d]      (M = Di for weights, 1 for biases)
//   merge: the inverse.
template <int VEC, bool SPLIT>
__global__ void __launch_bounds__(kThreads)
heads_permute_kernel(const float* __restrict__ src, float* __restrict__ dst, int B, int L, int M, int H, int d) {
  const int dv = d / VEC;
  const int64_t total = (int64_t)B * L * M * H * dv;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    // i enumerates the [B, H, L, M, d/VEC] side
    int64_t t = i;
    const int f = (int)(t % dv); t /= dv;
    const int m = (int)(t % M); t /= M;
    const int l = (int)(t % L); t /= L;
    const int h = (int)(t % H); t /= H;
    const int b = (int)t;
    const int64_t packed = ((((int64_t)b * L + l) * M + m) * H + h) * dv + f;  // [B, L, M, H, d/VEC]
    const int64_t s = SPLIT ? packed : i, o = SPLIT ? i : packed;
    if (VEC == 4) reinterpret_cast<float4*>(dst)[o] = reinterpret_cast<const float4*>(src)[s];
    else dst[o] = src[s];
  }
}

// Split with the position and feature axes swapped: src [B, L, M, H, d] -> dst [B, H, d, M, L].
// One block per (b, h, m): a [L, d] tile goes through shared memory so that both the reads
// (along d) and the writes (along L) are contiguous.
__global__ void __launch_bounds__(kThreads)
heads_split_transpose_kernel(const float* __restrict__ src, float* __restrict__ dst, int B, int L, int M, int H, int d) {
  __shared__ float tile[32][33];
  const int64_t bid = blockIdx.x;
  const int m = (int)(bid % M);
  const int h = (int)((bid / M) % H);
  const int b = (int)(bid / ((int64_t)M * H));
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int l0 = 0; l0 < L; l0 += 32) {
    for (int f0 = 0; f0 < d; f0 += 32) {
      for (int yy = ty; yy < 32; yy += 8) {
        const int l = l0 + yy, f = f0 + tx;
        if (l < L && f < d) tile[yy][tx] = src[((((int64_t)b * L + l) * M + m) * H + h) * d + f];
      }
      __syncthreads();
      for (int yy = ty; yy < 32; yy += 8) {
        const int f = f0 + yy, l = l0 + tx;
        if (l < L && f < d) dst[((((int64_t)b * H + h) * d + f) * M + m) * L + l] = tile[tx][yy];
      }
      __syncthreads();
    }
  }
}

// z_l = x_l * w+ + x_u * w-,  z_u = x_l * w- + x_u * w+ with w a vector over the feature axis (Bounds.py:653-664);
// n elements of rows of length Do.
__global__ void __launch_bounds__(kThreads)
mul_features_kernel(const float* xl, const float* xu, const float* __restrict__ w, float* zl, float* zu, int64_t n, int Do) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float wv = w[i % Do];
    const float wp = wv > 0.f ? wv : 0.f;
    const float wn = fsub(wv, wp);
    const float a = xl[i], b = xu[i];   // both read before either is written: z may alias x
    zl[i] = fadd(fmul(a, wp), fmul(b, wn));
    zu[i] = fadd(fmul(a, wn), fmul(b, wp));
  }
}

// Interval product of two boxes, elementwise (Bounds.get_bounds_xy in `ibp` mode, Bounds.py:667-678).
__global__ void __launch_bounds__(kThreads)
interval_mul_kernel(const float* __restrict__ xl, const float* __restrict__ xu, const float* __restrict__ yl,
                    const float* __restrict__ yu, float* __restrict__ zl, float* __restrict__ zu, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float p1 = fmul(xl[i], yl[i]), p2 = fmul(xl[i], yu[i]), p3 = fmul(xu[i], yl[i]), p4 = fmul(xu[i], yu[i]);
    zl[i] = fminf(p1, fminf(p2, fminf(p3, p4)));
    zu[i] = fmaxf(p1, fmaxf(p2, fmaxf(p3, p4)));
  }
}

// Interval dot product z[b, i, j] = sum_k [x[b, i, k]] * [y[b, j, k]] (Bounds.py:711-721): one warp per (b, i, j),
// the lanes stride over k; the partial sums are added in a fixed tree, k ascending within a lane.
__global__ void __launch_bounds__(kThreads)
interval_dot_kernel(const float* __restrict__ xl, const float* __restrict__ xu, const float* __restrict__ yl,
                    const float* __restrict__ yu, float* __restrict__ zl, float* __restrict__ zu, int64_t n_out, int Lx,
                    int Ly, int K) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t o = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; o < n_out; o += warps) {
    const int j = (int)(o % Ly);
    const int64_t bi = o / Ly;          // b * Lx + i
    const int64_t b = bi / Lx;
    const float* pxl = xl + bi * K;
    const float* pxu = xu + bi * K;
    const float* pyl = yl + (b * Ly + j) * K;
    const float* pyu = yu + (b * Ly + j) * K;
    float lo = 0.f, hi = 0.f;
    for (int k = lane; k < K; k += 32) {
      const float p1 = fmul(pxl[k], pyl[k]), p2 = fmul(pxl[k], pyu[k]), p3 = fmul(pxu[k], pyl[k]), p4 = fmul(pxu[k], pyu[k]);
      lo = fadd(lo, fminf(fminf(p1, p2), fminf(p3, p4)));
      hi = fadd(hi, fmaxf(fmaxf(p1, p2), fmaxf(p3, p4)));
    }
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) {
      lo = fadd(lo, __shfl_xor_sync(0xffffffffu, lo, sft));
      hi = fadd(hi, __shfl_xor_sync(0xffffffffu, hi, sft));
    }
    if (lane == 0) {
      zl[o] = lo;
      zu[o] = hi;
    }
  }
}

}  // namespace
}  // namespace fb

using namespace fb;

#define FB_REQUIRE(cond, code) do { if (!(cond)) return (code); } while (0)

extern "C" int fb_add_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                          const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                          float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                          int64_t rows, int Di, int Do, void* stream) {
  FB_REQUIRE(x_lw && x_uw && x_lb && x_ub && y_lw && y_uw && y_lb && y_ub && z_lw && z_uw && z_lb && z_ub, FB_ERR_ARG);
  FB_REQUIRE(rows >= 0 && Di > 0 && Do >= 0, FB_ERR_ARG);
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t nw = rows * Di * Do, nb = rows * Do;
  if (nw == 0) return FB_OK;
  ProfileScope prof(PK_ELEMENTWISE, 2.0 * (nw + nb), 4.0 * 6 * (nw + nb), stream);
  const bool vw = nw % 4 == 0 && aligned16(x_lw) && aligned16(x_uw) && aligned16(y_lw) && aligned16(y_uw) &&
                  aligned16(z_lw) && aligned16(z_uw);
  if (vw) add_kernel<4><<<stream_blocks(nw / 4), kThreads, 0, st>>>(x_lw, y_lw, z_lw, x_uw, y_uw, z_uw, nw);
  else add_kernel<1><<<stream_blocks(nw), kThreads, 0, st>>>(x_lw, y_lw, z_lw, x_uw, y_uw, z_uw, nw);
  add_kernel<1><<<stream_blocks(nb), kThreads, 0, st>>>(x_lb, y_lb, z_lb, x_ub, y_ub, z_ub, nb);
  FB_LAUNCH_OK_N(2);
  return FB_OK;
}

extern "C" int fb_scale_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                            float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                            int64_t rows, int Di, int Do, float c, void* stream) {
  FB_REQUIRE(x_lw && x_uw && x_lb && x_ub && z_lw && z_uw && z_lb && z_ub, FB_ERR_ARG);
  FB_REQUIRE(rows >= 0 && Di > 0 && Do >= 0, FB_ERR_ARG);
  FB_REQUIRE(z_lw != x_lw && z_lw != x_uw && z_uw != x_lw && z_uw != x_uw && z_lb != x_lb && z_lb != x_ub &&
             z_ub != x_lb && z_ub != x_ub, FB_ERR_ARG);
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t nw = rows * Di * Do, nb = rows * Do;
  if (nw == 0) return FB_OK;
  ProfileScope prof(PK_ELEMENTWISE, 2.0 * (nw + nb), 4.0 * 4 * (nw + nb), stream);
  // a positive scalar keeps the sides, any other swaps them (Bounds.py:596-607)
  const float* s_lw = c > 0.f ? x_lw : x_uw;
  const float* s_uw = c > 0.f ? x_uw : x_lw;
  const float* s_lb = c > 0.f ? x_lb : x_ub;
  const float* s_ub = c > 0.f ? x_ub : x_lb;
  const bool vw = nw % 4 == 0 && aligned16(x_lw) && aligned16(x_uw) && aligned16(z_lw) && aligned16(z_uw);
  if (vw) scale_kernel<4><<<stream_blocks(nw / 4), kThreads, 0, st>>>(s_lw, z_lw, s_uw, z_uw, c, nw);
  else scale_kernel<1><<<stream_blocks(nw), kThreads, 0, st>>>(s_lw, z_lw, s_uw, z_uw, c, nw);
  scale_kernel<1><<<stream_blocks(nb), kThreads, 0, st>>>(s_lb, z_lb, s_ub, z_ub, c, nb);
  FB_LAUNCH_OK_N(2);
  return FB_OK;
}

extern "C" int fb_rowsum_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                             float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                             int64_t rows, int Di, int Do, void* stream) {
  FB_REQUIRE(x_lw && x_uw && x_lb && x_ub && z_lw && z_uw && z_lb && z_ub, FB_ERR_ARG);
  FB_REQUIRE(rows >= 0 && Di > 0 && Do >= 0, FB_ERR_ARG);
  if (rows == 0 || Do == 0) return FB_OK;
  const int64_t n_w = rows * Di, n_b = rows;
  ProfileScope prof(PK_ELEMENTWISE, 2.0 * (n_w + n_b) * Do, 4.0 * 4 * (n_w + n_b) * Do, stream);
  rowsum_kernel<<<stream_blocks((n_w + n_b) * 32), kThreads, 0, (cudaStream_t)stream>>>(
      x_lw, x_uw, x_lb, x_ub, z_lw, z_uw, z_lb, z_ub, n_w, n_b, Do);
  FB_LAUNCH_OK();
  return FB_OK;
}

// fb_layernorm_novar_f32 that can also leave the row sums of its result behind (rowsum, may be null).
int fb::layernorm_novar_rowsum(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                      const float* r_lw, const float* r_uw, const float* r_lb, const float* r_ub,
                                      const float* gamma, const float* beta,
                                      float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                                      int64_t rows, int Di, int Do, float* rowsum, void* stream) {
  FB_REQUIRE(x_lw && x_uw && x_lb && x_ub && gamma && beta && z_lw && z_uw && z_lb && z_ub, FB_ERR_ARG);
  const bool any_r = r_lw || r_uw || r_lb || r_ub, all_r = r_lw && r_uw && r_lb && r_ub;
  FB_REQUIRE(any_r == all_r, FB_ERR_ARG);
  FB_REQUIRE(rows >= 0 && Di > 0 && Do >= 0, FB_ERR_ARG);
  FB_REQUIRE(z_lw != x_uw && z_uw != x_lw && z_lb != x_ub && z_ub != x_lb, FB_ERR_ARG);
  if (rows == 0 || Do == 0) return FB_OK;
  const int64_t n_w = rows * Di, n_b = rows;
  ProfileScope prof(PK_ELEMENTWISE, 8.0 * (n_w + n_b) * Do, 4.0 * (r_lw ? 6 : 4) * (n_w + n_b) * Do, stream);
  const bool row128 = Do == 128 && aligned16(x_lw) && aligned16(x_uw) && aligned16(x_lb) && aligned16(x_ub) &&
                      aligned16(z_lw) && aligned16(z_uw) && aligned16(z_lb) && aligned16(z_ub) && aligned16(gamma) &&
                      aligned16(beta) &&
                      (!r_lw || (aligned16(r_lw) && aligned16(r_uw) && aligned16(r_lb) && aligned16(r_ub)));
  if (rowsum != nullptr && !row128) return FB_ERR_SHAPE;   // row sums come from the 128-feature kernel only
  const unsigned blocks = stream_blocks((n_w + n_b) * 32);
  cudaStream_t st = (cudaStream_t)stream;
  if (row128 && r_lw)
    layernorm_novar_row128_kernel<true><<<blocks, kThreads, 0, st>>>(x_lw, x_uw, x_lb, x_ub, r_lw, r_uw, r_lb, r_ub, gamma,
                                                                      beta, z_lw, z_uw, z_lb, z_ub, n_w, n_b, rowsum);
  else if (row128)
    layernorm_novar_row128_kernel<false><<<blocks, kThreads, 0, st>>>(x_lw, x_uw, x_lb, x_ub, r_lw, r_uw, r_lb, r_ub, gamma,
                                                                       beta, z_lw, z_uw, z_lb, z_ub, n_w, n_b, rowsum);
  else
    layernorm_novar_kernel<<<blocks, kThreads, 0, st>>>(x_lw, x_uw, x_lb, x_ub, r_lw, r_uw, r_lb, r_ub, gamma, beta, z_lw,
                                                        z_uw, z_lb, z_ub, n_w, n_b, Do);
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_layernorm_novar_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                      const float* r_lw, const float* r_uw, const float* r_lb, const float* r_ub,
                                      const float* gamma, const float* beta,
                                      float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                                      int64_t rows, int Di, int Do, void* stream) {
  return fb::layernorm_novar_rowsum(x_lw, x_uw, x_lb, x_ub, r_lw, r_uw, r_lb, r_ub, gamma, beta, z_lw, z_uw, z_lb, z_ub, rows, Di,
                                    Do, nullptr, stream);
}

extern "C" int fb_split_heads_f32(const float* x_w, const float* x_b, float* z_w, float* z_b,
                                  int B, int L, int Di, int H, int d, int transpose_ld, void* stream) {
  FB_REQUIRE(x_w && x_b && z_w && z_b, FB_ERR_ARG);
  FB_REQUIRE(B >= 0 && L > 0 && Di > 0 && H > 0 && d > 0, FB_ERR_ARG);
  if (B == 0) return FB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  ProfileScope prof(PK_ELEMENTWISE, 0.0, 4.0 * 2 * ((double)B * L * (Di + 1) * H * d), stream);
  if (transpose_ld) {
    const int64_t bw = (int64_t)B * H * Di, bb = (int64_t)B * H;
    FB_REQUIRE(bw <= 0x7fffffff, FB_ERR_SHAPE);
    heads_split_transpose_kernel<<<(unsigned)bw, kThreads, 0, st>>>(x_w, z_w, B, L, Di, H, d);
    heads_split_transpose_kernel<<<(unsigned)bb, kThreads, 0, st>>>(x_b, z_b, B, L, 1, H, d);
  } else {
    const bool vec = d % 4 == 0 && aligned16(x_w) && aligned16(z_w);
    const int64_t nw = (int64_t)B * L * Di * H * d, nb = (int64_t)B * L * H * d;
    if (vec) heads_permute_kernel<4, true><<<stream_blocks(nw / 4), kThreads, 0, st>>>(x_w, z_w, B, L, Di, H, d);
    else heads_permute_kernel<1, true><<<stream_blocks(nw), kThreads, 0, st>>>(x_w, z_w, B, L, Di, H, d);
    heads_permute_kernel<1, true><<<stream_blocks(nb), kThreads, 0, st>>>(x_b, z_b, B, L, 1, H, d);
  }
  FB_LAUNCH_OK_N(2);
  return FB_OK;
}

extern "C" int fb_merge_heads_f32(const float* x_w, const float* x_b, float* z_w, float* z_b,
                                  int B, int L, int Di, int H, int d, void* stream) {
  FB_REQUIRE(x_w && x_b && z_w && z_b, FB_ERR_ARG);
  FB_REQUIRE(B >= 0 && L > 0 && Di > 0 && H > 0 && d > 0, FB_ERR_ARG);
  if (B == 0) return FB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  ProfileScope prof(PK_ELEMENTWISE, 0.0, 4.0 * 2 * ((double)B * L * (Di + 1) * H * d), stream);
  const bool vec = d % 4 == 0 && aligned16(x_w) && aligned16(z_w);
  const int64_t nw = (int64_t)B * L * Di * H * d, nb = (int64_t)B * L * H * d;
  if (vec) heads_permute_kernel<4, false><<<stream_blocks(nw / 4), kThreads, 0, st>>>(x_w, z_w, B, L, Di, H, d);
  else heads_permute_kernel<1, false><<<stream_blocks(nw), kThreads, 0, st>>>(x_w, z_w, B, L, Di, H, d);
  heads_permute_kernel<1, false><<<stream_blocks(nb), kThreads, 0, st>>>(x_b, z_b, B, L, 1, H, d);
  FB_LAUNCH_OK_N(2);
  return FB_OK;
}

extern "C" int fb_mul_features_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                   const float* w, float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                                   int64_t rows, int Di, int Do, void* stream) {
  FB_REQUIRE(x_lw && x_uw && x_lb && x_ub && w && z_lw && z_uw && z_lb && z_ub, FB_ERR_ARG);
  FB_REQUIRE(rows >= 0 && Di > 0 && Do >= 0, FB_ERR_ARG);
  const int64_t nw = rows * Di * Do, nb = rows * Do;
  if (nb == 0) return FB_OK;
  ProfileScope prof(PK_ELEMENTWISE, 4.0 * (nw + nb), 4.0 * 4 * (nw + nb), stream);
  cudaStream_t st = (cudaStream_t)stream;
  mul_features_kernel<<<stream_blocks(nw), kThreads, 0, st>>>(x_lw, x_uw, w, z_lw, z_uw, nw, Do);
  mul_features_kernel<<<stream_blocks(nb), kThreads, 0, st>>>(x_lb, x_ub, w, z_lb, z_ub, nb, Do);
  FB_LAUNCH_OK_N(2);
  return FB_OK;
}

extern "C" int fb_interval_mul_f32(const float* x_l, const float* x_u, const float* y_l, const float* y_u,
                                   float* z_l, float* z_u, int64_t n, void* stream) {
  FB_REQUIRE(x_l && x_u && y_l && y_u && z_l && z_u && n >= 0, FB_ERR_ARG);
  if (n == 0) return FB_OK;
  ProfileScope prof(PK_MUL, 4.0 * n, 4.0 * 6 * n, stream);
  interval_mul_kernel<<<stream_blocks(n), kThreads, 0, (cudaStream_t)stream>>>(x_l, x_u, y_l, y_u, z_l, z_u, n);
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_interval_dot_f32(const float* x_l, const float* x_u, const float* y_l, const float* y_u,
                                   float* z_l, float* z_u, int B, int Lx, int Ly, int K, void* stream) {
  FB_REQUIRE(x_l && x_u && y_l && y_u && z_l && z_u, FB_ERR_ARG);
  FB_REQUIRE(B >= 0 && Lx > 0 && Ly > 0 && K > 0, FB_ERR_ARG);
  const int64_t n_out = (int64_t)B * Lx * Ly;
  if (n_out == 0) return FB_OK;
  ProfileScope prof(PK_DOT, 8.0 * n_out * K, 4.0 * (2.0 * B * (Lx + Ly) * K + 2.0 * n_out), stream);
  interval_dot_kernel<<<stream_blocks(n_out * 32), kThreads, 0, (cudaStream_t)stream>>>(x_l, x_u, y_l, y_u, z_l, z_u, n_out,
                                                                                         Lx, Ly, K);
  FB_LAUNCH_OK();
  return FB_OK;
}
