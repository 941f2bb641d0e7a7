// Weight part of the bound x bound dot product, native layout, software-pipelined version.
// Included by dot_product.cu (inside namespace fb, anonymous namespace).
//
//   z_lw[b,i,m,j] = sum_k  x_c ly - x_r |ly| + y_c lx - y_r |lx|
//   z_uw[b,i,m,j] = sum_k  x_c uy + x_r |uy| + y_c lx + y_r |lx|
// with x_c = (x_lw + x_uw)/2, x_r = (x_uw - x_lw)/2 (same for y): the centre/radius form of the
// sign-split sums, 6 instead of 8 multiply-adds per product because the y-terms are shared by
// the two sides.
//
// A block is persistent: it walks work items (b, i-tile, j-tile, m-tile, k-chunk) and prefetches
// the tiles of the next item with cp.async into the second half of shared memory while it
// computes the current one, so global-load latency is hidden behind the FMAs.  Tiles are stored
// [m][row][k] with a 4-float pad per k-row: consecutive rows are 36 floats apart, which makes the
// 128/64-bit reads of a quarter warp (8 consecutive rows) hit distinct banks.
constexpr int PXT = TM * TI * ROW;                  // floats per operand tile ([m][row][k])
constexpr int PBUF = 4 * PXT + 3 * ST;              // one pipeline stage
constexpr int kDotPipeSmemFloats = 2 * PBUF;

__device__ __forceinline__ void cp_async16(float* dst, const float* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct DotItem {
  int64_t b;
  int i0, j0, m0, k0;
};

__device__ __forceinline__ DotItem dot_item(int64_t w, int n_it, int n_jt, int n_mt, int n_kc) {
  DotItem t;
  t.k0 = (int)(w % n_kc) * TK; w /= n_kc;
  t.m0 = (int)(w % n_mt) * TM; w /= n_mt;
  t.j0 = (int)(w % n_jt) * TJ; w /= n_jt;
  t.i0 = (int)(w % n_it) * TI; w /= n_it;
  t.b = w;
  return t;
}

// Asynchronous fill of one [TM][rows][TK] operand tile: element (m, r, k) comes from
// src + r * row_stride + m * K + k0 + k.  Invalid rows / m / k are zero-filled.
__device__ __forceinline__ void fill_operand_async(float* dst, const float* src, int rows_valid, int m_valid,
                                                   int64_t row_stride, int k0, int K) {
  for (int f = threadIdx.x; f < TM * TI * (TK / 4); f += kThreads) {
    const int kq = (f & 7) * 4, r = (f >> 3) % TI, m = f / (8 * TI);
    const bool ok = r < rows_valid && m < m_valid && k0 + kq < K;
    const float* p = ok ? src + r * row_stride + (int64_t)m * K + k0 + kq : src;
    cp_async16(dst + (m * TI + r) * ROW + kq, p, ok);
  }
}
__device__ __forceinline__ void fill_range_async(float* dst, const float* src, int rows_valid, int k0, int K) {
  for (int f = threadIdx.x; f < TI * (TK / 4); f += kThreads) {
    const int kq = (f & 7) * 4, r = f >> 3;
    const bool ok = r < rows_valid && k0 + kq < K;
    cp_async16(dst + r * ROW + kq, ok ? src + (int64_t)r * K + k0 + kq : src, ok);
  }
}

__global__ void __launch_bounds__(kThreads, 1)
dot_weight_native_pipelined(const float* __restrict__ x_lw, const float* __restrict__ x_uw,
                            const float* __restrict__ y_lw, const float* __restrict__ y_uw,
                            const float* __restrict__ x_l, const float* __restrict__ y_l,
                            const float* __restrict__ y_u, float* __restrict__ z_lw, float* __restrict__ z_uw,
                            int Lx, int Ly, int Di, int K, int n_it, int n_jt, int n_mt, int n_kc, int64_t n_items,
                            float out_scale, int heads) {
  extern __shared__ __align__(16) float smem[];
  const int tid = threadIdx.x;
  const int tj = tid & 7, ti = (tid >> 3) & 7, tm = tid >> 6;

  auto prefetch = [&](int64_t w, int buf) {
    const DotItem t = dot_item(w, n_it, n_jt, n_mt, n_kc);
    float* s = smem + buf * PBUF;
    const int ni = min(TI, Lx - t.i0), nj = min(TJ, Ly - t.j0), nm = min(TM, Di - t.m0);
    const int64_t xb = ((t.b * Lx + t.i0) * (int64_t)Di + t.m0) * K, yb = ((t.b * Ly + t.j0) * (int64_t)Di + t.m0) * K;
    fill_operand_async(s + 0 * PXT, x_lw + xb, ni, nm, (int64_t)Di * K, t.k0, K);
    fill_operand_async(s + 1 * PXT, x_uw + xb, ni, nm, (int64_t)Di * K, t.k0, K);
    fill_operand_async(s + 2 * PXT, y_lw + yb, nj, nm, (int64_t)Di * K, t.k0, K);
    fill_operand_async(s + 3 * PXT, y_uw + yb, nj, nm, (int64_t)Di * K, t.k0, K);
    fill_range_async(s + 4 * PXT + 0 * ST, x_l + (t.b * Lx + t.i0) * (int64_t)K, ni, t.k0, K);
    fill_range_async(s + 4 * PXT + 1 * ST, y_l + (t.b * Ly + t.j0) * (int64_t)K, nj, t.k0, K);
    fill_range_async(s + 4 * PXT + 2 * ST, y_u + (t.b * Ly + t.j0) * (int64_t)K, nj, t.k0, K);
    cp_async_commit();
  };

  // L = x-terms of the lower side, U = x-terms of the upper side, P / Q = centre / radius y-terms
  float aL[4][4], aU[4][4], aP[4][4], aQ[4][4];
  // Whole output tiles are assigned to blocks (tile = blockIdx.x + q * gridDim.x), their k-chunks
  // are walked consecutively: local step n -> item (tile, n % n_kc).
  const int64_t n_tiles = n_items / n_kc;
  const int64_t my_tiles = n_tiles > blockIdx.x ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int64_t my_steps = my_tiles * n_kc;
  auto item_of = [&](int64_t n) { return (blockIdx.x + (n / n_kc) * gridDim.x) * n_kc + n % n_kc; };
  if (my_steps > 0) prefetch(item_of(0), 0);
  int buf = 0;
  for (int64_t n = 0; n < my_steps; ++n, buf ^= 1) {
    const int64_t w = item_of(n);
    if (n + 1 < my_steps) { prefetch(item_of(n + 1), buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const DotItem t = dot_item(w, n_it, n_jt, n_mt, n_kc);
    if (t.k0 == 0) {
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) { aL[a][c] = 0.f; aU[a][c] = 0.f; aP[a][c] = 0.f; aQ[a][c] = 0.f; }
    }
    const float* s = smem + buf * PBUF;
    const float* s_xl = s + (tm * TI) * ROW;
    const float* s_xu = s_xl + PXT;
    const float* s_yl = s_xu + PXT;
    const float* s_yu = s_yl + PXT;
    const float* s_lx = s + 4 * PXT;
    const float* s_ly = s_lx + ST;
    const float* s_uy = s_ly + ST;
#pragma unroll 4
    for (int kq = 0; kq < TK; kq += 2) {
      float2 xl[4], xu[4], yl[4], yu[4], lx[4], ly[4], uy[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int i = ti + 8 * a, j = tj + 8 * a;
        xl[a] = *reinterpret_cast<const float2*>(s_xl + i * ROW + kq);
        xu[a] = *reinterpret_cast<const float2*>(s_xu + i * ROW + kq);
        yl[a] = *reinterpret_cast<const float2*>(s_yl + j * ROW + kq);
        yu[a] = *reinterpret_cast<const float2*>(s_yu + j * ROW + kq);
        lx[a] = *reinterpret_cast<const float2*>(s_lx + i * ROW + kq);
        ly[a] = *reinterpret_cast<const float2*>(s_ly + j * ROW + kq);
        uy[a] = *reinterpret_cast<const float2*>(s_uy + j * ROW + kq);
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float xc[4], xr[4], yc[4], yr[4], vlx[4], alx[4], vly[4], naly[4], vuy[4], auy[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const float xlo = e ? xl[a].y : xl[a].x, xup = e ? xu[a].y : xu[a].x;
          const float ylo = e ? yl[a].y : yl[a].x, yup = e ? yu[a].y : yu[a].x;
          xc[a] = 0.5f * (xlo + xup); xr[a] = 0.5f * (xup - xlo);
          yc[a] = 0.5f * (ylo + yup); yr[a] = 0.5f * (yup - ylo);
          vlx[a] = e ? lx[a].y : lx[a].x; alx[a] = fabsf(vlx[a]);
          vly[a] = e ? ly[a].y : ly[a].x; naly[a] = -fabsf(vly[a]);
          vuy[a] = e ? uy[a].y : uy[a].x; auy[a] = fabsf(vuy[a]);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            aL[a][c] = fmaf(xc[a], vly[c], aL[a][c]);
            aL[a][c] = fmaf(xr[a], naly[c], aL[a][c]);
            aU[a][c] = fmaf(xc[a], vuy[c], aU[a][c]);
            aU[a][c] = fmaf(xr[a], auy[c], aU[a][c]);
            aP[a][c] = fmaf(yc[c], vlx[a], aP[a][c]);
            aQ[a][c] = fmaf(yr[c], alx[a], aQ[a][c]);
          }
      }
    }
    if (t.k0 + TK >= K) {  // last k-chunk of this output tile
      const int m = t.m0 + tm;
      if (m < Di) {
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const int i = t.i0 + ti + 8 * a;
          if (i >= Lx) continue;
          // heads > 1: b = s * heads + h and the output is written head-merged, [S, Lx, Di, heads * Ly]
          const int64_t sb = t.b / heads, hb = t.b % heads;
          const int64_t row = (((sb * Lx + i) * (int64_t)Di + m) * heads + hb) * Ly;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int j = t.j0 + tj + 8 * c;
            if (j < Ly) {
              z_lw[row + j] = fmul(fadd(aL[a][c], fsub(aP[a][c], aQ[a][c])), out_scale);
              z_uw[row + j] = fmul(fadd(aU[a][c], fadd(aP[a][c], aQ[a][c])), out_scale);
            }
          }
        }
      }
    }
    __syncthreads();  // every thread is done with `buf` before the next prefetch overwrites it
  }
}
