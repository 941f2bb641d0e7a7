// Bound x bound dot product  z[b,i,j] = sum_k x[b,i,k] * y[b,j,k]  (attention scores, and the
// attention context when y is the transposed value operand).
//
// With (l_x, u_x), (l_y, u_y) the concretised operand ranges, the reference (Bounds.py:680-688,
// 710-823) relaxes each product x*y by the planes
//     lower:  l_y * x + l_x * y - l_x * l_y        upper:  u_y * x + l_x * y - l_x * u_y
// and substitutes, per slope sign, the lower or upper line of the operand:
//   z_lw[b,i,:,j] = sum_k  ly+[j,k] x_lw[i,:,k] + ly-[j,k] x_uw[i,:,k] + lx+[i,k] y_lw[j,:,k] + lx-[i,k] y_uw[j,:,k]
//   z_uw[b,i,:,j] = sum_k  uy+[j,k] x_uw[i,:,k] + uy-[j,k] x_lw[i,:,k] + lx+[i,k] y_uw[j,:,k] + lx-[i,k] y_lw[j,:,k]
// (same for lb/ub with the constant sum_k -alpha*beta).  The first two terms are a GEMM of x
// against the ranges of y, the last two a GEMM of y against the ranges of x whose result lands
// transposed; both are fused here so that x and y are read once per tile and z is written once.
//
// Three launches: concretise x, concretise y (column kernels), then one kernel for the bias
// part and one for the weight part.
#include <mutex>

#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace fb {
namespace {

constexpr int kThreads = 256;

// ---------------------------------------------------------------- bias part
// One warp per output element (b, i, j); lanes across k.
__global__ void __launch_bounds__(kThreads)
dot_bias_kernel(const float* __restrict__ x_lb, const float* __restrict__ x_ub, const float* __restrict__ y_lb,
                const float* __restrict__ y_ub, const float* __restrict__ x_l, const float* __restrict__ y_l,
                const float* __restrict__ y_u, float* __restrict__ z_lb, float* __restrict__ z_ub,
                int64_t total, int Lx, int Ly, int K, float out_scale, int heads) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t o = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); o < total; o += warps) {
    const int j = (int)(o % Ly);
    const int64_t bi = o / Ly;          // b * Lx + i
    const int64_t b = bi / Lx;
    const float* xr_lb = x_lb + bi * K;
    const float* xr_ub = x_ub + bi * K;
    const float* xr_l = x_l + bi * K;
    const int64_t bj = b * Ly + j;
    const float* yr_lb = y_lb + bj * K;
    const float* yr_ub = y_ub + bj * K;
    const float* yr_l = y_l + bj * K;
    const float* yr_u = y_u + bj * K;
    // five partial sums per side, kept apart and added in the reference's order
    float gl = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f, l4 = 0.f;
    float gu = 0.f, u1 = 0.f, u2 = 0.f, u3 = 0.f, u4 = 0.f;
    for (int k = lane; k < K; k += 32) {
      const float lx = xr_l[k], ly = yr_l[k], uy = yr_u[k];
      const float xl = xr_lb[k], xu = xr_ub[k], yl = yr_lb[k], yu = yr_ub[k];
      const float lxp = lx > 0.f ? lx : 0.f, lxn = lx < 0.f ? lx : 0.f;
      const float lyp = ly > 0.f ? ly : 0.f, lyn = ly < 0.f ? ly : 0.f;
      const float uyp = uy > 0.f ? uy : 0.f, uyn = uy < 0.f ? uy : 0.f;
      gl = fadd(gl, fmul(-ly, lx));
      gu = fadd(gu, fmul(-uy, lx));
      l1 = fmaf(xl, lyp, l1); l2 = fmaf(xu, lyn, l2); l3 = fmaf(yl, lxp, l3); l4 = fmaf(yu, lxn, l4);
      u1 = fmaf(xu, uyp, u1); u2 = fmaf(xl, uyn, u2); u3 = fmaf(yu, lxp, u3); u4 = fmaf(yl, lxn, u4);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      gl += __shfl_xor_sync(0xffffffffu, gl, s); gu += __shfl_xor_sync(0xffffffffu, gu, s);
      l1 += __shfl_xor_sync(0xffffffffu, l1, s); u1 += __shfl_xor_sync(0xffffffffu, u1, s);
      l2 += __shfl_xor_sync(0xffffffffu, l2, s); u2 += __shfl_xor_sync(0xffffffffu, u2, s);
      l3 += __shfl_xor_sync(0xffffffffu, l3, s); u3 += __shfl_xor_sync(0xffffffffu, u3, s);
      l4 += __shfl_xor_sync(0xffffffffu, l4, s); u4 += __shfl_xor_sync(0xffffffffu, u4, s);
    }
    if (lane == 0) {
      // heads > 1: head-merged output [S, Lx, heads * Ly]
      const int64_t i_ = bi % Lx, od = (((b / heads) * Lx + i_) * heads + b % heads) * Ly + j;
      z_lb[od] = fmul(fadd(fadd(fadd(fadd(gl, l1), l2), l3), l4), out_scale);
      z_ub[od] = fmul(fadd(fadd(fadd(fadd(gu, u1), u2), u3), u4), out_scale);
    }
  }
}

// Tiled version of the bias part: one block per (b, 32 i, 32 j) tile; the seven row tiles are staged
// in shared memory (row stride 33 floats: conflict-free both for the row-wise fill and for the
// column-wise reads), K in chunks of 32; thread (i, jq) owns the outputs (i, jq + 8 c), c = 0..3.
// Same partial sums and the same final order of additions as dot_bias_kernel.
__global__ void __launch_bounds__(kThreads)
dot_bias_tiled(const float* __restrict__ x_lb, const float* __restrict__ x_ub, const float* __restrict__ y_lb,
               const float* __restrict__ y_ub, const float* __restrict__ x_l, const float* __restrict__ y_l,
               const float* __restrict__ y_u, float* __restrict__ z_lb, float* __restrict__ z_ub,
               int Lx, int Ly, int K, int n_it, int n_jt, float out_scale, int heads, int y_kmajor) {
  __shared__ float sm[7][32][33];   // x_lb, x_ub, x_l, y_lb, y_ub, y_l, y_u
  int w = blockIdx.x;
  const int jt = w % n_jt; w /= n_jt;
  const int it = w % n_it;
  const int64_t b = w / n_it;
  const int i0 = it * 32, j0 = jt * 32;
  const int tid = threadIdx.x, ti = tid >> 3, tj = tid & 7;
  float gl[4], gu[4], l1[4], l2[4], l3[4], l4[4], u1[4], u2[4], u3[4], u4[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) gl[c] = gu[c] = l1[c] = l2[c] = l3[c] = l4[c] = u1[c] = u2[c] = u3[c] = u4[c] = 0.f;
  for (int k0 = 0; k0 < K; k0 += 32) {
    const float* src[7] = {x_lb, x_ub, x_l, y_lb, y_ub, y_l, y_u};
#pragma unroll
    for (int a = 0; a < 7; ++a) {
      const bool isx = a < 3;
      const int L = isx ? Lx : Ly, r0 = isx ? i0 : j0;
      for (int f = tid; f < 32 * 32; f += kThreads) {
        const int r = f >> 5, k = f & 31;
        const bool ok = r0 + r < L && k0 + k < K;
        // y_kmajor: y_lb / y_ub (a = 3, 4) are stored [b, k, j] instead of [b, j, k]
        const bool km = y_kmajor && (a == 3 || a == 4);
        const int64_t idx = km ? ((int64_t)b * K + k0 + k) * L + r0 + r : ((int64_t)b * L + r0 + r) * K + k0 + k;
        sm[a][r][k] = ok ? src[a][idx] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int k = 0; k < 32; ++k) {
      const float xl = sm[0][ti][k], xu = sm[1][ti][k], lx = sm[2][ti][k];
      const float lxp = lx > 0.f ? lx : 0.f, lxn = lx < 0.f ? lx : 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = tj + 8 * c;
        const float yl = sm[3][j][k], yu = sm[4][j][k], ly = sm[5][j][k], uy = sm[6][j][k];
        const float lyp = ly > 0.f ? ly : 0.f, lyn = ly < 0.f ? ly : 0.f;
        const float uyp = uy > 0.f ? uy : 0.f, uyn = uy < 0.f ? uy : 0.f;
        gl[c] = fadd(gl[c], fmul(-ly, lx));
        gu[c] = fadd(gu[c], fmul(-uy, lx));
        l1[c] = fmaf(xl, lyp, l1[c]); l2[c] = fmaf(xu, lyn, l2[c]); l3[c] = fmaf(yl, lxp, l3[c]); l4[c] = fmaf(yu, lxn, l4[c]);
        u1[c] = fmaf(xu, uyp, u1[c]); u2[c] = fmaf(xl, uyn, u2[c]); u3[c] = fmaf(yu, lxp, u3[c]); u4[c] = fmaf(yl, lxn, u4[c]);
      }
    }
    __syncthreads();
  }
  const int i = i0 + ti;
  if (i < Lx) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int j = j0 + tj + 8 * c;
      if (j < Ly) {
        // heads > 1: head-merged output [S, Lx, heads * Ly]
        const int64_t od = (((b / heads) * Lx + i) * heads + b % heads) * Ly + j;
        z_lb[od] = fmul(fadd(fadd(fadd(fadd(gl[c], l1[c]), l2[c]), l3[c]), l4[c]), out_scale);
        z_ub[od] = fmul(fadd(fadd(fadd(fadd(gu[c], u1[c]), u2[c]), u3[c]), u4[c]), out_scale);
      }
    }
  }
}

// ------------------------------------------------- weight part, native layout
// x [B, Lx, Di, K], y [B, Ly, Di, K] -> z [B, Lx, Di, Ly].
// Block tile: TI = 32 rows of x, TJ = 32 rows of y, TM = 4 symbolic coordinates, K in chunks of
// 32.  Thread (tj, ti, tm) owns i = ti + 8a, j = tj + 8c (a, c < 4) for one m: 16 outputs per
// side.  Shared tiles are k-contiguous with a 4-float pad per row so that the 128-bit reads of a
// quarter warp (8 consecutive tj) hit 32 distinct banks.
constexpr int TI = 32, TJ = 32, TM = 4, TK = 32;
constexpr int ROW = TK + 4;                       // padded k-row
constexpr int XT = TI * TM * ROW;                 // floats per x (or y) tile
constexpr int ST = TI * ROW;                      // floats per range tile (TI == TJ)
constexpr int kDotSmemFloats = 4 * XT + 3 * ST;   // x_l, x_u, y_l, y_u tiles + lx, ly, uy

// Copies an [nouter, ninner, TK] tile into shared memory as (nouter * ninner) padded k-rows.
// Source element (o, n, k) lives at src + o * outer_stride + n * inner_stride + k0 + k; rows with
// o >= outer_valid or n >= inner_valid and columns beyond K are zero-filled.
template <bool VEC>
__device__ __forceinline__ void fill_tile(float* __restrict__ dst, const float* __restrict__ src, int nouter,
                                          int ninner, int outer_valid, int inner_valid, int64_t outer_stride,
                                          int64_t inner_stride, int k0, int K) {
  const int total = nouter * ninner * (TK / 4);
  for (int f = threadIdx.x; f < total; f += kThreads) {
    const int r = f / (TK / 4), kq = (f % (TK / 4)) * 4;
    const int o = r / ninner, n = r % ninner;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (o < outer_valid && n < inner_valid) {
      const float* p = src + o * outer_stride + n * inner_stride + k0 + kq;
      if (VEC) {
        if (k0 + kq < K) v = __ldg(reinterpret_cast<const float4*>(p));
      } else {
        if (k0 + kq + 0 < K) v.x = __ldg(p + 0);
        if (k0 + kq + 1 < K) v.y = __ldg(p + 1);
        if (k0 + kq + 2 < K) v.z = __ldg(p + 2);
        if (k0 + kq + 3 < K) v.w = __ldg(p + 3);
      }
    }
    *reinterpret_cast<float4*>(dst + r * ROW + kq) = v;
  }
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
dot_weight_native(const float* __restrict__ x_lw, const float* __restrict__ x_uw, const float* __restrict__ y_lw,
                  const float* __restrict__ y_uw, const float* __restrict__ x_l, const float* __restrict__ y_l,
                  const float* __restrict__ y_u, float* __restrict__ z_lw, float* __restrict__ z_uw,
                  int Lx, int Ly, int Di, int K, int n_it, int n_jt, int n_mt, float out_scale) {
  extern __shared__ __align__(16) float smem[];
  float* s_xl = smem;
  float* s_xu = s_xl + XT;
  float* s_yl = s_xu + XT;
  float* s_yu = s_yl + XT;
  float* s_lx = s_yu + XT;
  float* s_ly = s_lx + ST;
  float* s_uy = s_ly + ST;

  int64_t bid = blockIdx.x;
  const int mt = (int)(bid % n_mt); bid /= n_mt;
  const int jt = (int)(bid % n_jt); bid /= n_jt;
  const int it = (int)(bid % n_it); bid /= n_it;
  const int64_t b = bid;
  const int i0 = it * TI, j0 = jt * TJ, m0 = mt * TM;
  const int tid = threadIdx.x;
  const int tj = tid & 7, ti = (tid >> 3) & 7, tm = tid >> 6;

  float acc_l[4][4], acc_u[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int c = 0; c < 4; ++c) { acc_l[a][c] = 0.f; acc_u[a][c] = 0.f; }

  const int ni = min(TI, Lx - i0), nj = min(TJ, Ly - j0), nm = min(TM, Di - m0);
  for (int k0 = 0; k0 < K; k0 += TK) {
    // x / y tiles: rows (i, m) resp. (j, m) of the operands; range tiles: rows i resp. j
    const int64_t xb = ((b * Lx + i0) * (int64_t)Di + m0) * K, yb = ((b * Ly + j0) * (int64_t)Di + m0) * K;
    fill_tile<VEC>(s_xl, x_lw + xb, TI, TM, ni, nm, (int64_t)Di * K, K, k0, K);
    fill_tile<VEC>(s_xu, x_uw + xb, TI, TM, ni, nm, (int64_t)Di * K, K, k0, K);
    fill_tile<VEC>(s_yl, y_lw + yb, TJ, TM, nj, nm, (int64_t)Di * K, K, k0, K);
    fill_tile<VEC>(s_yu, y_uw + yb, TJ, TM, nj, nm, (int64_t)Di * K, K, k0, K);
    fill_tile<VEC>(s_lx, x_l + (b * Lx + i0) * (int64_t)K, TI, 1, ni, 1, K, 0, k0, K);
    fill_tile<VEC>(s_ly, y_l + (b * Ly + j0) * (int64_t)K, TJ, 1, nj, 1, K, 0, k0, K);
    fill_tile<VEC>(s_uy, y_u + (b * Ly + j0) * (int64_t)K, TJ, 1, nj, 1, K, 0, k0, K);
    __syncthreads();
#pragma unroll 2
    for (int kq = 0; kq < TK; kq += 4) {
      float xl[4][4], xu[4][4], yl[4][4], yu[4][4], lx[4][4], ly[4][4], uy[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int i = ti + 8 * a, j = tj + 8 * a;
        *reinterpret_cast<float4*>(xl[a]) = *reinterpret_cast<const float4*>(s_xl + (i * TM + tm) * ROW + kq);
        *reinterpret_cast<float4*>(xu[a]) = *reinterpret_cast<const float4*>(s_xu + (i * TM + tm) * ROW + kq);
        *reinterpret_cast<float4*>(yl[a]) = *reinterpret_cast<const float4*>(s_yl + (j * TM + tm) * ROW + kq);
        *reinterpret_cast<float4*>(yu[a]) = *reinterpret_cast<const float4*>(s_yu + (j * TM + tm) * ROW + kq);
        *reinterpret_cast<float4*>(lx[a]) = *reinterpret_cast<const float4*>(s_lx + i * ROW + kq);
        *reinterpret_cast<float4*>(ly[a]) = *reinterpret_cast<const float4*>(s_ly + j * ROW + kq);
        *reinterpret_cast<float4*>(uy[a]) = *reinterpret_cast<const float4*>(s_uy + j * ROW + kq);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float lyp[4], lyn[4], uyp[4], uyn[4], lxp[4], lxn[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          lyp[a] = fmaxf(ly[a][e], 0.f); lyn[a] = fminf(ly[a][e], 0.f);
          uyp[a] = fmaxf(uy[a][e], 0.f); uyn[a] = fminf(uy[a][e], 0.f);
          lxp[a] = fmaxf(lx[a][e], 0.f); lxn[a] = fminf(lx[a][e], 0.f);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float l = acc_l[a][c], u = acc_u[a][c];
            l = fmaf(xl[a][e], lyp[c], l); l = fmaf(xu[a][e], lyn[c], l);
            l = fmaf(yl[c][e], lxp[a], l); l = fmaf(yu[c][e], lxn[a], l);
            u = fmaf(xu[a][e], uyp[c], u); u = fmaf(xl[a][e], uyn[c], u);
            u = fmaf(yu[c][e], lxp[a], u); u = fmaf(yl[c][e], lxn[a], u);
            acc_l[a][c] = l; acc_u[a][c] = u;
          }
      }
    }
    __syncthreads();
  }
  const int m = m0 + tm;
  if (m >= Di) return;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = i0 + ti + 8 * a;
    if (i >= Lx) continue;
    const int64_t row = ((b * Lx + i) * (int64_t)Di + m) * Ly;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int j = j0 + tj + 8 * c;
      if (j < Ly) {
        z_lw[row + j] = fmul(acc_l[a][c], out_scale);
        z_uw[row + j] = fmul(acc_u[a][c], out_scale);
      }
    }
  }
}

#include "dot_product_pipelined.cuh"
// Few query rows (Lx <= kFewRows; a last layer run for the first token only has Lx = 1): the tiled kernels would spend 31
// of the 32 rows of every x tile on padding.  One thread per output element (b, i, m, j), lanes along j, the products
// accumulated over k in the order of dot_weight_native; y is read once, in its native layout [B, Ly, Di, K] (a thread
// walks K consecutive values) or as [B, K, Di, Ly] (y_kmajor: the value tensor as the projection writes it; the lanes
// read consecutive words).
constexpr int kFewRows = 4;
__global__ void __launch_bounds__(256)
dot_weight_rows_kernel(const float* __restrict__ x_lw, const float* __restrict__ x_uw, const float* __restrict__ y_lw,
                       const float* __restrict__ y_uw, const float* __restrict__ x_l, const float* __restrict__ y_l,
                       const float* __restrict__ y_u, float* __restrict__ z_lw, float* __restrict__ z_uw, int64_t total,
                       int Lx, int Ly, int Di, int K, float out_scale, int merge_heads, int y_kmajor) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int j = (int)(t % Ly), m = (int)((t / Ly) % Di), i = (int)((t / ((int64_t)Ly * Di)) % Lx);
    const int64_t b = t / ((int64_t)Ly * Di * Lx);
    const float* xl = x_lw + ((b * Lx + i) * (int64_t)Di + m) * K;
    const float* xu = x_uw + ((b * Lx + i) * (int64_t)Di + m) * K;
    const float* lx = x_l + (b * Lx + i) * (int64_t)K;
    const float* ly = y_l + (b * Ly + j) * (int64_t)K;
    const float* uy = y_u + (b * Ly + j) * (int64_t)K;
    const int64_t y0 = y_kmajor ? (b * K * (int64_t)Di + m) * Ly + j : ((b * Ly + j) * (int64_t)Di + m) * K;
    const int64_t ys = y_kmajor ? (int64_t)Di * Ly : 1;
    float l = 0.f, u = 0.f;
#pragma unroll 4
    for (int k = 0; k < K; ++k) {
      const float yl = __ldg(y_lw + y0 + k * ys), yu = __ldg(y_uw + y0 + k * ys);
      const float a = __ldg(xl + k), c = __ldg(xu + k);
      const float vly = __ldg(ly + k), vuy = __ldg(uy + k), vlx = __ldg(lx + k);
      const float lyp = fmaxf(vly, 0.f), lyn = fminf(vly, 0.f), uyp = fmaxf(vuy, 0.f), uyn = fminf(vuy, 0.f);
      const float lxp = fmaxf(vlx, 0.f), lxn = fminf(vlx, 0.f);
      l = fmaf(a, lyp, l); l = fmaf(c, lyn, l);
      l = fmaf(yl, lxp, l); l = fmaf(yu, lxn, l);
      u = fmaf(c, uyp, u); u = fmaf(a, uyn, u);
      u = fmaf(yu, lxp, u); u = fmaf(yl, lxn, u);
    }
    int64_t o = ((b * Lx + i) * (int64_t)Di + m) * Ly + j;
    if (merge_heads > 1) {
      const int64_t sidx = b / merge_heads;
      const int h = (int)(b % merge_heads);
      o = ((sidx * Lx + i) * (int64_t)Di + m) * ((int64_t)merge_heads * Ly) + (int64_t)h * Ly + j;
    }
    z_lw[o] = fmul(l, out_scale);
    z_uw[o] = fmul(u, out_scale);
  }
}

int launch_dot_weight_rows(const float* x_lw, const float* x_uw, const float* y_lw, const float* y_uw, const float* x_l,
                           const float* y_l, const float* y_u, float* z_lw, float* z_uw, int B, int Lx, int Ly, int Di, int K,
                           float out_scale, int merge_heads, int y_kmajor, cudaStream_t st) {
  const int64_t total = (int64_t)B * Lx * Di * Ly;
  const int64_t want = ceil_div(total, 256), cap = (int64_t)device_info().sms * 64;
  dot_weight_rows_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(x_lw, x_uw, y_lw, y_uw, x_l, y_l, y_u, z_lw, z_uw, total,
                                                                             Lx, Ly, Di, K, out_scale, merge_heads, y_kmajor);
  FB_LAUNCH_OK();
  return FB_OK;
}


// --------------------------------------------- weight part, transposed layout
// x [B, Lx, K, Di], y [B, Ly, K, Di] -> z [B, Lx, Ly, Di]   (Di contiguous).
// One thread per symbolic coordinate m (coalesced along Di), 4 x 4 (i, j) outputs per thread;
// the operand ranges of the tile live in shared memory and are broadcast.
constexpr int TTI = 4, TTJ = 4, TTK = 128, TThreads = 128;

__global__ void __launch_bounds__(TThreads)
dot_weight_transposed(const float* __restrict__ x_lw, const float* __restrict__ x_uw, const float* __restrict__ y_lw,
                      const float* __restrict__ y_uw, const float* __restrict__ x_l, const float* __restrict__ y_l,
                      const float* __restrict__ y_u, float* __restrict__ z_lw, float* __restrict__ z_uw,
                      int Lx, int Ly, int Di, int K, int n_it, int n_jt, float out_scale) {
  __shared__ float s_lx[TTI][TTK], s_ly[TTJ][TTK], s_uy[TTJ][TTK];
  int64_t bid = blockIdx.x;
  const int jt = (int)(bid % n_jt); bid /= n_jt;
  const int it = (int)(bid % n_it); bid /= n_it;
  const int64_t b = bid;
  const int i0 = it * TTI, j0 = jt * TTJ;
  const int m = blockIdx.y * TThreads + threadIdx.x;
  const bool m_ok = m < Di;
  float acc_l[TTI][TTJ], acc_u[TTI][TTJ];
#pragma unroll
  for (int a = 0; a < TTI; ++a)
#pragma unroll
    for (int c = 0; c < TTJ; ++c) { acc_l[a][c] = 0.f; acc_u[a][c] = 0.f; }
  for (int k0 = 0; k0 < K; k0 += TTK) {
    const int nk = min(TTK, K - k0);
    for (int f = threadIdx.x; f < TTI * TTK; f += TThreads) {
      const int r = f / TTK, k = f % TTK;
      const bool kin = k < nk;
      s_lx[r][k] = (kin && i0 + r < Lx) ? x_l[(b * Lx + i0 + r) * (int64_t)K + k0 + k] : 0.f;
      s_ly[r][k] = (kin && j0 + r < Ly) ? y_l[(b * Ly + j0 + r) * (int64_t)K + k0 + k] : 0.f;
      s_uy[r][k] = (kin && j0 + r < Ly) ? y_u[(b * Ly + j0 + r) * (int64_t)K + k0 + k] : 0.f;
    }
    __syncthreads();
    if (m_ok) {
      for (int k = 0; k < nk; ++k) {
        float xl[TTI], xu[TTI], yl[TTJ], yu[TTJ];
#pragma unroll
        for (int a = 0; a < TTI; ++a) {
          const bool ok = i0 + a < Lx;
          const int64_t o = ((b * Lx + i0 + a) * (int64_t)K + k0 + k) * Di + m;
          xl[a] = ok ? __ldg(x_lw + o) : 0.f;
          xu[a] = ok ? __ldg(x_uw + o) : 0.f;
        }
#pragma unroll
        for (int c = 0; c < TTJ; ++c) {
          const bool ok = j0 + c < Ly;
          const int64_t o = ((b * Ly + j0 + c) * (int64_t)K + k0 + k) * Di + m;
          yl[c] = ok ? __ldg(y_lw + o) : 0.f;
          yu[c] = ok ? __ldg(y_uw + o) : 0.f;
        }
#pragma unroll
        for (int a = 0; a < TTI; ++a) {
          const float lx = s_lx[a][k];
          const float lxp = fmaxf(lx, 0.f), lxn = fminf(lx, 0.f);
#pragma unroll
          for (int c = 0; c < TTJ; ++c) {
            const float ly = s_ly[c][k], uy = s_uy[c][k];
            float l = acc_l[a][c], u = acc_u[a][c];
            l = fmaf(xl[a], fmaxf(ly, 0.f), l); l = fmaf(xu[a], fminf(ly, 0.f), l);
            l = fmaf(yl[c], lxp, l);            l = fmaf(yu[c], lxn, l);
            u = fmaf(xu[a], fmaxf(uy, 0.f), u); u = fmaf(xl[a], fminf(uy, 0.f), u);
            u = fmaf(yu[c], lxp, u);            u = fmaf(yl[c], lxn, u);
            acc_l[a][c] = l; acc_u[a][c] = u;
          }
        }
      }
    }
    __syncthreads();
  }
  if (!m_ok) return;
#pragma unroll
  for (int a = 0; a < TTI; ++a)
#pragma unroll
    for (int c = 0; c < TTJ; ++c)
      if (i0 + a < Lx && j0 + c < Ly) {
        const int64_t o = ((b * Lx + i0 + a) * (int64_t)Ly + j0 + c) * Di + m;
        z_lw[o] = fmul(acc_l[a][c], out_scale);
        z_uw[o] = fmul(acc_u[a][c], out_scale);
      }
}

}  // namespace
}  // namespace fb

namespace fb {
// dot_product_tc.cu
bool dot_tc_supported(const float* x_lw, const float* x_uw, const float* y_lw, const float* y_uw, const float* x_l,
                      const float* y_l, const float* y_u, const float* z_lw, const float* z_uw, int B, int Lx, int Ly,
                      int Di, int K, int heads);
int launch_dot_weight_tc(const float* x_lw, const float* x_uw, const float* y_lw, const float* y_uw, const float* x_l,
                         const float* y_l, const float* y_u, float* z_lw, float* z_uw, int B, int Lx, int Ly, int Di,
                         float out_scale, int heads, int y_kmajor, cudaStream_t st);
namespace {
// FB_DOT_IMPL=ffma in the environment keeps the dot product on the CUDA-core kernels (exact fp32 products)
bool dot_force_cuda_cores() {
  static const bool v = [] {
    const char* e = getenv("FB_DOT_IMPL");
    return e != nullptr && strcmp(e, "ffma") == 0;
  }();
  return v;
}
}  // namespace
}  // namespace fb

using namespace fb;

// given: bit 0 = x_l / x_u already hold the concretised range of x, bit 1 = y_l / y_u that of y
// (e.g. from fb_matmul_heads_ranges_f32); the corresponding concretisation pass is skipped.
static int dot_heads_impl(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                          const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                          float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                          float* x_l, float* x_u, float* y_l, float* y_u,
                          int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                          float out_scale, int layout, int merge_heads, int given, void* stream) {
  if (given < 0 || given > 3) return FB_ERR_ARG;
  if (merge_heads < 1 || (merge_heads > 1 && (layout != FB_NATIVE || B % merge_heads != 0 || K % 4 != 0))) return FB_ERR_ARG;
  if (!x_lw || !x_uw || !x_lb || !x_ub || !y_lw || !y_uw || !y_lb || !y_ub || !z_lw || !z_uw || !z_lb || !z_ub ||
      !x_l || !x_u || !y_l || !y_u)
    return FB_ERR_ARG;
  if (B < 0 || Lx <= 0 || Ly <= 0 || Di <= 0 || K <= 0 || words <= 0 || !valid_norm(p)) return FB_ERR_ARG;
  if (layout != FB_NATIVE && layout != FB_TRANSPOSED) return FB_ERR_ARG;
  if (!(out_scale > 0.f)) return FB_ERR_ARG;
  if (Di % words != 0) return FB_ERR_SHAPE;
  // The reference's Di == 1 branch (interval product, Bounds.py:711-721) is a different
  // operator that none of the forward-verifier configurations reaches.
  if (Di == 1) return FB_ERR_SHAPE;
  if (B == 0) return FB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const double d1 = (double)Di + 1;
  ProfileScope prof(PK_DOT, 16.0 * B * Lx * Ly * d1 * K,
                    4.0 * (2.0 * B * Lx * d1 * K + 2.0 * B * Ly * d1 * K + 2.0 * B * Lx * Ly * d1), stream);
  int rc = FB_OK;
  if (!(given & 1)) rc = fb_concretize_f32(x_lw, x_uw, x_lb, x_ub, x_l, x_u, (int64_t)B * Lx, Di, K, words, p, eps, layout, stream);
  if (rc != FB_OK) return rc;
  if (!(given & 2)) rc = fb_concretize_f32(y_lw, y_uw, y_lb, y_ub, y_l, y_u, (int64_t)B * Ly, Di, K, words, p, eps, layout, stream);
  if (rc != FB_OK) return rc;
  {
    const int n_it = (int)ceil_div(Lx, 32), n_jt = (int)ceil_div(Ly, 32);
    const int64_t blocks = (int64_t)B * n_it * n_jt;
    if (blocks <= 0x7fffffff) {
      dot_bias_tiled<<<(unsigned)blocks, kThreads, 0, st>>>(x_lb, x_ub, y_lb, y_ub, x_l, y_l, y_u, z_lb, z_ub, Lx, Ly, K,
                                                           n_it, n_jt, out_scale, merge_heads, 0);
    } else {
      const int64_t total = (int64_t)B * Lx * Ly;
      const int64_t want = ceil_div(total, kThreads / 32);
      const int64_t cap = (int64_t)device_info().sms * 32;
      dot_bias_kernel<<<(unsigned)(want < cap ? want : cap), kThreads, 0, st>>>(x_lb, x_ub, y_lb, y_ub, x_l, y_l, y_u,
                                                                                 z_lb, z_ub, total, Lx, Ly, K, out_scale, merge_heads);
    }
    FB_LAUNCH_OK();
  }
  if (layout == FB_NATIVE && !dot_force_cuda_cores() &&
      dot_tc_supported(x_lw, x_uw, y_lw, y_uw, x_l, y_l, y_u, z_lw, z_uw, B, Lx, Ly, Di, K, merge_heads)) {
    // attention shapes: tensor-core kernel
    return launch_dot_weight_tc(x_lw, x_uw, y_lw, y_uw, x_l, y_l, y_u, z_lw, z_uw, B, Lx, Ly, Di, out_scale, merge_heads, 0, st);
  }
  if (layout == FB_NATIVE && Lx <= kFewRows)
    return launch_dot_weight_rows(x_lw, x_uw, y_lw, y_uw, x_l, y_l, y_u, z_lw, z_uw, B, Lx, Ly, Di, K, out_scale, merge_heads, 0, st);
  if (layout == FB_NATIVE) {
    const int n_it = (int)ceil_div(Lx, TI), n_jt = (int)ceil_div(Ly, TJ), n_mt = (int)ceil_div(Di, TM);
    const int64_t blocks = (int64_t)B * n_it * n_jt * n_mt;
    if (blocks > 0x7fffffff) return FB_ERR_SHAPE;
    const size_t smem = sizeof(float) * kDotSmemFloats;
    const bool vec = K % 4 == 0 && aligned16(x_lw) && aligned16(x_uw) && aligned16(y_lw) && aligned16(y_uw) &&
                     aligned16(x_l) && aligned16(y_l) && aligned16(y_u);
    if (!vec && merge_heads > 1) return FB_ERR_ALIGN;
    if (vec) {
      // persistent, cp.async-pipelined kernel: one block per SM walks the (tile, k-chunk) items
      const int n_kc = (int)ceil_div(K, TK);
      const int64_t n_items = blocks * n_kc;
      const size_t psmem = sizeof(float) * kDotPipeSmemFloats;
      if (int rc = ensure_dynamic_smem(dot_weight_native_pipelined, psmem)) return rc;
      const int64_t sms = device_info().sms;
      dot_weight_native_pipelined<<<(unsigned)(blocks < sms ? blocks : sms), kThreads, psmem, st>>>(
          x_lw, x_uw, y_lw, y_uw, x_l, y_l, y_u, z_lw, z_uw, Lx, Ly, Di, K, n_it, n_jt, n_mt, n_kc, n_items, out_scale, merge_heads);
    } else {
      if (int rc = ensure_dynamic_smem(dot_weight_native<false>, smem)) return rc;
      dot_weight_native<false><<<(unsigned)blocks, kThreads, smem, st>>>(x_lw, x_uw, y_lw, y_uw, x_l, y_l, y_u, z_lw,
                                                                         z_uw, Lx, Ly, Di, K, n_it, n_jt, n_mt, out_scale);
    }
  } else {
    const int n_it = (int)ceil_div(Lx, TTI), n_jt = (int)ceil_div(Ly, TTJ);
    const int64_t blocks = (int64_t)B * n_it * n_jt;
    const int64_t my = ceil_div(Di, TThreads);
    if (blocks > 0x7fffffff || my > 65535) return FB_ERR_SHAPE;
    dot_weight_transposed<<<dim3((unsigned)blocks, (unsigned)my), TThreads, 0, st>>>(
        x_lw, x_uw, y_lw, y_uw, x_l, y_l, y_u, z_lw, z_uw, Lx, Ly, Di, K, n_it, n_jt, out_scale);
  }
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_dot_product_heads_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                  const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                                  float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                                  float* x_l, float* x_u, float* y_l, float* y_u,
                                  int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                                  float out_scale, int layout, int merge_heads, void* stream) {
  return dot_heads_impl(x_lw, x_uw, x_lb, x_ub, y_lw, y_uw, y_lb, y_ub, z_lw, z_uw, z_lb, z_ub, x_l, x_u, y_l, y_u, B, Lx,
                        Ly, Di, K, words, p, eps, out_scale, layout, merge_heads, 0, stream);
}

// fb_dot_product_heads_f32 for operands whose concretised ranges the caller already has (written by the
// kernel that produced the operand): `given` bit 0 = x_l / x_u are inputs, bit 1 = y_l / y_u are inputs.
extern "C" int fb_dot_product_given_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                  const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                                  float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                                  float* x_l, float* x_u, float* y_l, float* y_u,
                                  int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                                  float out_scale, int layout, int merge_heads, int given, void* stream) {
  return dot_heads_impl(x_lw, x_uw, x_lb, x_ub, y_lw, y_uw, y_lb, y_ub, z_lw, z_uw, z_lb, z_ub, x_l, x_u, y_l, y_u, B, Lx,
                        Ly, Di, K, words, p, eps, out_scale, layout, merge_heads, given, stream);
}

extern "C" int fb_dot_product_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                  const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                                  float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                                  float* x_l, float* x_u, float* y_l, float* y_u,
                                  int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                                  float out_scale, int layout, void* stream) {
  return fb_dot_product_heads_f32(x_lw, x_uw, x_lb, x_ub, y_lw, y_uw, y_lb, y_ub, z_lw, z_uw, z_lb, z_ub, x_l, x_u, y_l,
                                  y_u, B, Lx, Ly, Di, K, words, p, eps, out_scale, layout, 1, stream);
}

namespace fb {
namespace {
// In-place transposition of [B][R][C] -> [B][C][R] for small matrices (R * C <= 4096): one block per b.
__global__ void __launch_bounds__(256) transpose_small_inplace(float* a, float* b2, int R, int C) {
  __shared__ float t[2][4096];
  float* pa = a + (int64_t)blockIdx.x * R * C;
  float* pb = b2 + (int64_t)blockIdx.x * R * C;
  for (int f = threadIdx.x; f < R * C; f += 256) { t[0][f] = pa[f]; t[1][f] = pb[f]; }
  __syncthreads();
  for (int f = threadIdx.x; f < R * C; f += 256) {
    const int c = f / R, r = f % R;      // output element (c, r)
    pa[f] = t[0][r * C + c];
    pb[f] = t[1][r * C + c];
  }
}
}  // namespace
}  // namespace fb

// Context product of the attention block (Bounds.context, Bounds.py:843-850: dot_product with V.t()) that
// takes the values as the projection writes them, v_lw / v_uw [B, K, Di, Ly], v_lb / v_ub [B, K, Ly] (K = key
// positions, Ly = head features), instead of the transposed copy [B, Ly, Di, K]; z as in
// fb_dot_product_heads_f32.  Only the shapes of the tensor-core kernel (K = Ly = 32, Lx % 32 == 0,
// Di % 4 == 0, 16-byte aligned pointers); otherwise FB_ERR_SHAPE and nothing is launched.
// y_l / y_u receive the concretised value ranges as [B, Ly, K].
// `given` as in fb_dot_product_given_f32; given ranges of the values are expected as [B, K, Ly] (the layout
// of v_lb / v_ub) and are transposed in place like computed ones.
extern "C" int fb_context_given_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                    const float* v_lw, const float* v_uw, const float* v_lb, const float* v_ub,
                                    float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                                    float* x_l, float* x_u, float* y_l, float* y_u,
                                    int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                                    float out_scale, int merge_heads, int given, void* stream) {
  if (given < 0 || given > 3) return FB_ERR_ARG;
  if (!x_lw || !x_uw || !x_lb || !x_ub || !v_lw || !v_uw || !v_lb || !v_ub || !z_lw || !z_uw || !z_lb || !z_ub ||
      !x_l || !x_u || !y_l || !y_u)
    return FB_ERR_ARG;
  if (B < 0 || Lx <= 0 || Ly <= 0 || Di <= 0 || K <= 0 || words <= 0 || !valid_norm(p) || merge_heads < 1) return FB_ERR_ARG;
  if (!(out_scale > 0.f)) return FB_ERR_ARG;
  if (Di % words != 0 || Di == 1) return FB_ERR_SHAPE;
  if (B == 0) return FB_OK;
  const bool tc = !dot_force_cuda_cores() &&
                  dot_tc_supported(x_lw, x_uw, v_lw, v_uw, x_l, y_l, y_u, z_lw, z_uw, B, Lx, Ly, Di, K, merge_heads);
  // (a few query rows go through the thread-per-output kernel, which reads the values in this layout as well)
  const bool rows_kernel = !tc && Lx <= kFewRows && (int64_t)K * Ly <= 4096;
  if (!tc && !rows_kernel) return FB_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const double d1 = (double)Di + 1;
  ProfileScope prof(PK_DOT, 16.0 * B * Lx * Ly * d1 * K,
                    4.0 * (2.0 * B * Lx * d1 * K + 2.0 * B * Ly * d1 * K + 2.0 * B * Lx * Ly * d1), stream);
  int rc = FB_OK;
  if (!(given & 1)) rc = fb_concretize_f32(x_lw, x_uw, x_lb, x_ub, x_l, x_u, (int64_t)B * Lx, Di, K, words, p, eps, FB_NATIVE, stream);
  if (rc != FB_OK) return rc;
  // ranges of the values in their own layout [B, K, Ly], then transposed in place to [B, Ly, K]
  if (!(given & 2)) rc = fb_concretize_f32(v_lw, v_uw, v_lb, v_ub, y_l, y_u, (int64_t)B * K, Di, Ly, words, p, eps, FB_NATIVE, stream);
  if (rc != FB_OK) return rc;
  transpose_small_inplace<<<(unsigned)B, 256, 0, st>>>(y_l, y_u, K, Ly);
  FB_LAUNCH_OK();
  {
    const int n_it = (int)ceil_div(Lx, 32), n_jt = (int)ceil_div(Ly, 32);
    dot_bias_tiled<<<(unsigned)((int64_t)B * n_it * n_jt), kThreads, 0, st>>>(x_lb, x_ub, v_lb, v_ub, x_l, y_l, y_u, z_lb, z_ub,
                                                                            Lx, Ly, K, n_it, n_jt, out_scale, merge_heads, 1);
    FB_LAUNCH_OK();
  }
  if (rows_kernel)
    return launch_dot_weight_rows(x_lw, x_uw, v_lw, v_uw, x_l, y_l, y_u, z_lw, z_uw, B, Lx, Ly, Di, K, out_scale, merge_heads, 1, st);
  return launch_dot_weight_tc(x_lw, x_uw, v_lw, v_uw, x_l, y_l, y_u, z_lw, z_uw, B, Lx, Ly, Di, out_scale, merge_heads, 1, st);
}

extern "C" int fb_context_heads_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                    const float* v_lw, const float* v_uw, const float* v_lb, const float* v_ub,
                                    float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                                    float* x_l, float* x_u, float* y_l, float* y_u,
                                    int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                                    float out_scale, int merge_heads, void* stream) {
  return fb_context_given_f32(x_lw, x_uw, x_lb, x_ub, v_lw, v_uw, v_lb, v_ub, z_lw, z_uw, z_lb, z_ub, x_l, x_u, y_l, y_u, B,
                              Lx, Ly, Di, K, words, p, eps, out_scale, merge_heads, 0, stream);
}

// ---------------------------------------------------------------------------
// Variant for callers that must not allocate: the concretised operand ranges go to a fixed
// array that lives in the library image instead of caller-provided scratch.
namespace fb {
namespace {
constexpr int64_t kStaticScratchFloats = 4ll * 1024 * 1024;  // 16 MiB, held by every GPU that loads the library
static __device__ __align__(256) float g_dot_static_scratch[kStaticScratchFloats];

constexpr int kMaxStaticDevices = 64;
float* g_static_ptr[kMaxStaticDevices] = {nullptr};
std::mutex g_static_mu;

// Device address of the array on the current device.  The symbol name is only a host-side
// handle, so the address is asked from the runtime once per device and remembered.
int static_scratch_address(float** out) {
  int dev = 0;
  FB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxStaticDevices) return FB_ERR_ARG;
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    FB_CUDA_OK(cudaGetSymbolAddress(&p, g_dot_static_scratch));
    if (p == nullptr) return FB_ERR_CUDA;
    g_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_ptr[dev];
  return FB_OK;
}
}  // namespace
}  // namespace fb

extern "C" int64_t fb_dot_product_noalloc_max_floats(void) { return fb::kStaticScratchFloats; }

extern "C" int fb_dot_product_noalloc_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                          const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                                          float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                                          int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                                          float out_scale, int layout, void* stream) {
  if (B < 0 || Lx <= 0 || Ly <= 0 || K <= 0 || Di <= 0 || words <= 0 || Di % words != 0 || !fb::valid_norm(p) ||
      (layout != FB_NATIVE && layout != FB_TRANSPOSED))
    return FB_ERR_ARG;
  // Each factor is bounded by the capacity before the products are formed, so that three large sizes cannot wrap
  // around 64 bits and slip under the limit: this check is all that stands between a caller and a write past the array.
  const int64_t cap = fb::kStaticScratchFloats;
  if (B > cap || Lx > cap || Ly > cap || K > cap) return FB_ERR_WORKSPACE;
  if ((int64_t)B * Lx > cap || (int64_t)B * Ly > cap) return FB_ERR_WORKSPACE;       // each product below 2^44
  if ((int64_t)B * Lx * K > cap || (int64_t)B * Ly * K > cap) return FB_ERR_WORKSPACE;  // (B * L <= 2^22) * (K <= 2^22) < 2^63
  // ranges of x: 2 * B * Lx * K floats, ranges of y: 2 * B * Ly * K floats (each part padded to 64 floats)
  const int64_t nx = ((int64_t)B * Lx * K + 63) / 64 * 64, ny = ((int64_t)B * Ly * K + 63) / 64 * 64;
  if (2 * nx + 2 * ny > cap) return FB_ERR_WORKSPACE;
  float* base = nullptr;
  const int rc = fb::static_scratch_address(&base);
  if (rc != FB_OK) return rc;
  return fb_dot_product_f32(x_lw, x_uw, x_lb, x_ub, y_lw, y_uw, y_lb, y_ub, z_lw, z_uw, z_lb, z_ub,
                            base, base + nx, base + 2 * nx, base + 2 * nx + ny,
                            B, Lx, Ly, Di, K, words, p, eps, out_scale, layout, stream);
}
