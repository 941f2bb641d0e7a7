// Compact rows for the convolutions behind an identity input.
//
// When every pixel of an H0 x W0 image is perturbed, row r of the weight tensors stands for pixel (ci, yi, xi) =
// unravel(r) and, after a chain of convolutions, is zero outside the window that pixel reaches (conv_window.cuh).
// The dense-row kernels of conv.cu still write and read those zeros: [rows, C, H, W] per tensor, 98 % zeros for the
// benchmark CNN.  Here a row is kept as its window only:
//
//     z[r, c, dy, dx] = row r at (c, wy.lo(r) + dy, wx.lo(r) + dx),   dy < wh, dx < ww,
//
// with (wh, ww) the largest window over all pixels (fb_cw_extent) and zeros where a pixel's own window is smaller.
// The origin (wy.lo, wx.lo) is recomputed from the pixel and the chain wherever it is needed.  Every operator of the
// CNN pass has a compact form: first convolution + relaxation, later convolutions, the column norms over dim_in
// (a gather over the rows whose window holds the column, in row order: deterministic), the rescale of a relaxation,
// and the linear layer that ends the spatial part (its output is dense, [rows, N]).  fb_cw_expand_f32 writes the dense
// rows for callers that need them.  Accumulation orders follow the dense kernels, so a compact convolution expands
// to the dense kernel's values bit for bit.
//
// The reference has no counterpart (HandTunedKernels/convolution_verification.cu:228-238 is a benchmark stub); the
// operator semantics are Bounds.matmul / Bounds.relu with dim_in as batch axis (Bounds.py:397-413, :921-963).
#include <algorithm>
#include <cstdint>

#include "common.cuh"
#include "conv_window.cuh"

namespace fb {
namespace {

// Geometry of a compact tensor: the chain that leads to it and its dense shape.
struct CwShape {
  ConvChain ch;
  int H0, W0, C, H, W, wh, ww;
};

__device__ __forceinline__ void pixel_of_row(int64_t r, int H0, int W0, int& yi, int& xi) {
  xi = (int)(r % W0);
  yi = (int)((r / W0) % H0);
}

// First convolution (+ relaxation) of the identity input, compact: one thread per element of z.
__global__ void __launch_bounds__(256)
cw_identity_rows_kernel(const float* __restrict__ Wt, const float* __restrict__ k_l, const float* __restrict__ k_u,
                        float* __restrict__ z_lw, float* __restrict__ z_uw, float scale, int64_t rows, int64_t row_start,
                        int Cin, int H, int W, int Cout, int Kh, int Kw, int stride, int pad, int Ho, int Wo, int wh, int ww) {
  const int64_t per_row = (int64_t)Cout * wh * ww;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < rows * per_row; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t lr = t / per_row;
    const int e = (int)(t - lr * per_row);
    const int dx = e % ww, dy = (e / ww) % wh, co = e / (ww * wh);
    const int64_t r = row_start + lr;
    const int xi = (int)(r % W), yi = (int)((r / W) % H), ci = (int)(r / ((int64_t)W * H));
    Span sy = {yi, yi}, sx = {xi, xi};
    sy = span_after_conv(sy, Kh, stride, pad, Ho);
    sx = span_after_conv(sx, Kw, stride, pad, Wo);
    const int y = sy.lo + dy, x = sx.lo + dx;
    float lo = 0.f, up = 0.f;
    if (sy.lo <= sy.hi && sx.lo <= sx.hi && y <= sy.hi && x <= sx.hi) {
      const int ky = yi - (y * stride - pad), kx = xi - (x * stride - pad);
      if (ky >= 0 && ky < Kh && kx >= 0 && kx < Kw) {
        const float tap = fmul(scale, __ldg(Wt + (((int64_t)co * Cin + ci) * Kh + ky) * Kw + kx));
        const int64_t col = ((int64_t)co * Ho + y) * Wo + x;
        lo = fmul(tap, k_l[col]);
        up = fmul(tap, k_u[col]);
      }
    }
    z_lw[t] = lo;
    z_uw[t] = up;
  }
}

// A later convolution, compact -> compact.  A block takes kCwRows consecutive rows: the filter is staged in shared
// memory once per block with the output channel innermost ([Cin, Kh, Kw, Cout]: the lanes of a warp, which differ in the
// output channel, read consecutive words), the compact inputs of the rows as (centre, radius) pairs.  A work item is one
// output element; items are ordered (row, y, x, channel), so with Cout a multiple of 32 a warp shares its row and its
// output pixel, its tap loops are uniform and its input reads are broadcasts.  Every output accumulates over (input
// channel, tap row, tap column) in that order, as the dense kernel does.
// Shared memory: Cin*Kh*Kw*(Cout+1) + 2 * kCwRows * Cin*iwh*iww floats (the filter rows are padded by one word, so that
// both the staging stores, whose lanes differ in the tap, and the reads, whose lanes differ in the channel, are free of
// bank conflicts).
constexpr int kCwRows = 8;
// CPT: output channels per work item (4 when Cout is a multiple of 4: the four weights of a tap are one 128-bit read and
// the input pair is read once for four channels, which halves the instructions per multiply-add; else 1).
template <int CPT>
__global__ void __launch_bounds__(256)
cw_conv_kernel(const float* __restrict__ x_lo, const float* __restrict__ x_up, const float* __restrict__ Wt,
               float* __restrict__ y_lo, float* __restrict__ y_up, int64_t rows, int64_t row_start, int H0, int W0,
               const ConvChain ch, int Cin, int Cout, int Kh, int Kw, int stride, int pad, int Ho, int Wo, int iwh, int iww,
               int owh, int oww) {
  extern __shared__ __align__(16) float cw_smem[];
  const int ldw = Cout + (CPT == 4 ? 4 : 1), ctaps = Cin * Kh * Kw;   // padded: staging stores and reads spread over the banks
  const int n_in = Cin * iwh * iww, n_out = Cout * owh * oww, n_w = ctaps * ldw;
  float* s_w = cw_smem;                                        // [Cin][Kh][Kw][ldw]
  float2* s_x = reinterpret_cast<float2*>(cw_smem + n_w + (n_w & 1));   // [kCwRows][Cin][iwh][iww] (centre, radius)
  __shared__ int s_geo[kCwRows][8];   // wy.lo, wx.lo, ah, aw, oy.lo, ox.lo, bh, bw (bh = 0: nothing to compute)
  const int64_t lr0 = (int64_t)blockIdx.x * kCwRows;
  const int nr = (int)min((int64_t)kCwRows, rows - lr0);
  for (int f = threadIdx.x; f < ctaps * Cout; f += blockDim.x) {   // coalesced read of [Cout][Cin*Kh*Kw]
    const int t = f % ctaps, co = f / ctaps;        // t = (c * Kh + ky) * Kw + kx
    s_w[t * ldw + co] = __ldg(Wt + f);
  }
  for (int f = threadIdx.x; f < nr * n_in; f += blockDim.x) {
    const float lo = __ldg(x_lo + lr0 * n_in + f), up = __ldg(x_up + lr0 * n_in + f);
    s_x[f] = make_float2(fmul(fadd(lo, up), 0.5f), fmul(fsub(up, lo), 0.5f));
  }
  if (threadIdx.x < nr) {
    int yi, xi;
    pixel_of_row(row_start + lr0 + threadIdx.x, H0, W0, yi, xi);
    Span wy, wx;
    chain_window(ch, H0, W0, yi, xi, wy, wx);
    const Span oy = span_after_conv(wy, Kh, stride, pad, Ho), ox = span_after_conv(wx, Kw, stride, pad, Wo);
    const bool empty = wy.lo > wy.hi || wx.lo > wx.hi || oy.lo > oy.hi || ox.lo > ox.hi;
    int* gq = s_geo[threadIdx.x];
    gq[0] = wy.lo, gq[1] = wx.lo, gq[2] = wy.hi - wy.lo + 1, gq[3] = wx.hi - wx.lo + 1;
    gq[4] = oy.lo, gq[5] = ox.lo, gq[6] = empty ? 0 : oy.hi - oy.lo + 1, gq[7] = empty ? 0 : ox.hi - ox.lo + 1;
  }
  __syncthreads();
  const int taps = Kh * Kw, cgroups = Cout / CPT;
  for (int i = threadIdx.x; i < nr * owh * oww * cgroups; i += blockDim.x) {
    const int co = (i % cgroups) * CPT, q = i / cgroups;
    const int x = q % oww, y = (q / oww) % owh, lr = q / (oww * owh);
    const int* gq = s_geo[lr];
    float ac[CPT], ar[CPT];
#pragma unroll
    for (int e = 0; e < CPT; ++e) { ac[e] = 0.f; ar[e] = 0.f; }
    const bool live = y < gq[6] && x < gq[7];
    if (live) {
      const int iy0 = (gq[4] + y) * stride - pad - gq[0], ix0 = (gq[5] + x) * stride - pad - gq[1];   // window coordinates
      const int ky0 = max(0, -iy0), ky1 = min(Kh, gq[2] - iy0), kx0 = max(0, -ix0), kx1 = min(Kw, gq[3] - ix0);
      const float2* xp = s_x + (lr * Cin * iwh + iy0) * iww + ix0;
      const float* wp = s_w + co;
      for (int c = 0; c < Cin; ++c, xp += iwh * iww, wp += taps * ldw)
        for (int ky = ky0; ky < ky1; ++ky)
          for (int kx = kx0; kx < kx1; ++kx) {
            const float2 v = xp[ky * iww + kx];
            if (CPT == 4) {
              const float4 w = *reinterpret_cast<const float4*>(wp + (ky * Kw + kx) * ldw);
              ac[0] = fmaf(v.x, w.x, ac[0]); ar[0] = fmaf(v.y, fabsf(w.x), ar[0]);
              ac[1 % CPT] = fmaf(v.x, w.y, ac[1 % CPT]); ar[1 % CPT] = fmaf(v.y, fabsf(w.y), ar[1 % CPT]);
              ac[2 % CPT] = fmaf(v.x, w.z, ac[2 % CPT]); ar[2 % CPT] = fmaf(v.y, fabsf(w.z), ar[2 % CPT]);
              ac[3 % CPT] = fmaf(v.x, w.w, ac[3 % CPT]); ar[3 % CPT] = fmaf(v.y, fabsf(w.w), ar[3 % CPT]);
            } else {
              const float w = wp[(ky * Kw + kx) * ldw];
              ac[0] = fmaf(v.x, w, ac[0]);
              ar[0] = fmaf(v.y, fabsf(w), ar[0]);
            }
          }
    }
#pragma unroll
    for (int e = 0; e < CPT; ++e) {
      const int64_t o = (lr0 + lr) * n_out + ((int64_t)(co + e) * owh + y) * oww + x;
      y_lo[o] = live ? fsub(ac[e], ar[e]) : 0.f;
      y_up[o] = live ? fadd(ac[e], ar[e]) : 0.f;
    }
  }
}

// Unfinished dual-norm accumulation of every column (c, y, x) over the rows [row_start, row_start + rows): a gather over
// the pixels whose window holds (y, x).  The spans of all pixel coordinates are tabulated in shared memory first
// (H0 + W0 entries); a warp takes a column, its lanes interleave over the candidate pixels (the pixel rows and columns
// between the first and the last whose span holds y resp. x), and the lane sums are combined by a butterfly: the order
// of the additions is fixed by the geometry alone, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256)
cw_norm_partials_kernel(const float* __restrict__ z_lw, const float* __restrict__ z_uw, float* __restrict__ part_l,
                        float* __restrict__ part_u, int64_t rows, int64_t row_start, int Cin0, const CwShape g, int p) {
  extern __shared__ int cw_spans[];   // ylo[H0], yhi[H0], xlo[W0], xhi[W0], then ya[H], yb[H], xa[W], xb[W]
  int* ylo = cw_spans;
  int* yhi = ylo + g.H0;
  int* xlo = yhi + g.H0;
  int* xhi = xlo + g.W0;
  int* t_ya = xhi + g.W0;
  int* t_yb = t_ya + g.H;
  int* t_xa = t_yb + g.H;
  int* t_xb = t_xa + g.W;
  for (int i = threadIdx.x; i < g.H0 + g.W0; i += blockDim.x) {
    Span wy, wx;
    if (i < g.H0) {
      chain_window(g.ch, g.H0, g.W0, i, 0, wy, wx);
      ylo[i] = wy.lo, yhi[i] = wy.hi;
    } else {
      chain_window(g.ch, g.H0, g.W0, 0, i - g.H0, wy, wx);
      xlo[i - g.H0] = wx.lo, xhi[i - g.H0] = wx.hi;
    }
  }
  __syncthreads();
  // per dense coordinate: first and last pixel row / column whose span holds it
  for (int i = threadIdx.x; i < g.H + g.W; i += blockDim.x) {
    const bool is_y = i < g.H;
    const int v = is_y ? i : i - g.H, n0 = is_y ? g.H0 : g.W0;
    const int* lo = is_y ? ylo : xlo;
    const int* hi = is_y ? yhi : xhi;
    int a = n0, b = -1;
    for (int k = 0; k < n0; ++k)
      if (v >= lo[k] && v <= hi[k]) { a = min(a, k); b = k; }
    (is_y ? t_ya : t_xa)[v] = a;
    (is_y ? t_yb : t_xb)[v] = b;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t ncol = (int64_t)g.C * g.H * g.W, per_row = (int64_t)g.C * g.wh * g.ww;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t t = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < ncol; t += warps) {
    const int x = (int)(t % g.W), y = (int)((t / g.W) % g.H), c = (int)(t / ((int64_t)g.W * g.H));
    const int ya = t_ya[y], yb = t_yb[y], xa = t_xa[x], xb = t_xb[x];
    float al = 0.f, au = 0.f;
    if (yb >= ya && xb >= xa) {
      const int ny = yb - ya + 1, nx = xb - xa + 1, cand = Cin0 * ny * nx;
      for (int k = lane; k < cand; k += 32) {
        const int xi = xa + k % nx, yi = ya + (k / nx) % ny, ci = k / (nx * ny);
        if (y < ylo[yi] || y > yhi[yi] || x < xlo[xi] || x > xhi[xi]) continue;
        const int64_t lr = ((int64_t)ci * g.H0 + yi) * g.W0 + xi - row_start;
        if (lr < 0 || lr >= rows) continue;
        const int64_t o = lr * per_row + ((int64_t)c * g.wh + (y - ylo[yi])) * g.ww + (x - xlo[xi]);
        al = norm_accum(p, al, __ldg(z_lw + o));
        au = norm_accum(p, au, __ldg(z_uw + o));
      }
    }
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) {
      al = norm_combine(p, al, __shfl_xor_sync(0xffffffffu, al, sft));
      au = norm_combine(p, au, __shfl_xor_sync(0xffffffffu, au, sft));
    }
    if (lane == 0) {
      part_l[t] = al;
      part_u[t] = au;
    }
  }
}

// Relaxation coefficients per column from the (reduced) norms; the relaxed bias terms are written to out_lb / out_ub.
__global__ void __launch_bounds__(256)
cw_relax_columns_kernel(int op, const float* __restrict__ lb, const float* __restrict__ ub, const float* __restrict__ norm_l,
                        const float* __restrict__ norm_u, float* __restrict__ out_lb, float* __restrict__ out_ub,
                        float* __restrict__ coef /* [4][ncol] */, int64_t ncol, int p, float eps, int* __restrict__ violation) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < ncol; t += (int64_t)gridDim.x * blockDim.x) {
    const float lbv = lb[t], ubv = ub[t];
    const float l = fadd(lbv, fmul(-eps, norm_finish(p, norm_l[t])));
    const float u = fadd(ubv, fmul(eps, norm_finish(p, norm_u[t])));
    bool bad = false;
    const ColCoef c = relax_column(op, l, u, lbv, ubv, bad);
    if (bad && violation != nullptr) *violation = 1;
    out_lb[t] = c.nlb;
    out_ub[t] = c.nub;
    coef[t] = c.c_ll;
    coef[ncol + t] = c.c_lu;
    coef[2 * ncol + t] = c.c_ul;
    coef[3 * ncol + t] = c.c_uu;
  }
}

// Rescale of a relaxation on compact rows: out_lw = c_ll lw + c_lu uw, out_uw = c_uu uw + c_ul lw (the expressions of
// the dense kernel).  A warp per row: the window is worked out once, the lanes interleave over its elements.
__global__ void __launch_bounds__(256)
cw_rescale_kernel(const float* __restrict__ z_lw, const float* __restrict__ z_uw, const float* __restrict__ coef,
                  float* __restrict__ o_lw, float* __restrict__ o_uw, int64_t rows, int64_t row_start, const CwShape g) {
  const int lane = threadIdx.x & 31;
  const int64_t lr = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (lr >= rows) return;
  const int per_row = g.C * g.wh * g.ww;
  const int64_t ncol = (int64_t)g.C * g.H * g.W;
  int yi, xi;
  pixel_of_row(row_start + lr, g.H0, g.W0, yi, xi);
  Span wy, wx;
  chain_window(g.ch, g.H0, g.W0, yi, xi, wy, wx);
  const bool empty = wy.lo > wy.hi || wx.lo > wx.hi;
  const int ah = wy.hi - wy.lo + 1, aw = wx.hi - wx.lo + 1;
  for (int e = lane; e < per_row; e += 32) {
    const int dx = e % g.ww, dy = (e / g.ww) % g.wh, c = e / (g.ww * g.wh);
    float lo = 0.f, up = 0.f;
    if (!empty && dy < ah && dx < aw) {
      const int64_t col = ((int64_t)c * g.H + wy.lo + dy) * g.W + wx.lo + dx;
      const float a = z_lw[lr * per_row + e], b = z_uw[lr * per_row + e];
      lo = fmaf(coef[col], a, fmul(coef[ncol + col], b));
      up = fmaf(coef[3 * ncol + col], b, fmul(coef[2 * ncol + col], a));
    }
    o_lw[lr * per_row + e] = lo;
    o_uw[lr * per_row + e] = up;
  }
}

// Linear layer on compact rows (weight part): y[r, n] = sum_e c_e W[n, col(e)] -/+ r_e |W[n, col(e)]|.  One warp per
// (row, group of kCwNB outputs): the lanes interleave over the elements, partial sums are combined by shuffles.
// The weight is read as WT [F, N] (the transpose of the nn.Linear layout, made once per call by cw_transpose_kernel): the
// kCwNB weights of an element are then consecutive words, while in the [N, F] layout every one of them is a sector of
// its own (measured on the 8192 -> 10 head: 37 us against 9 us).
constexpr int kCwNB = 16;
__global__ void __launch_bounds__(256)
cw_linear_kernel(const float* __restrict__ z_lw, const float* __restrict__ z_uw, const float* __restrict__ WT,
                 float* __restrict__ y_lw, float* __restrict__ y_uw, int64_t rows, int64_t row_start, const CwShape g, int N) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int groups = (N + kCwNB - 1) / kCwNB;
  const int64_t lr = warp / groups;
  if (lr >= rows) return;
  const int n0 = (int)(warp % groups) * kCwNB;
  const int per_row = g.C * g.wh * g.ww;
  int yi, xi;
  pixel_of_row(row_start + lr, g.H0, g.W0, yi, xi);
  Span wy, wx;
  chain_window(g.ch, g.H0, g.W0, yi, xi, wy, wx);
  const int ah = wy.hi - wy.lo + 1, aw = wx.hi - wx.lo + 1;
  float sc[kCwNB], sr[kCwNB];
#pragma unroll
  for (int j = 0; j < kCwNB; ++j) { sc[j] = 0.f; sr[j] = 0.f; }
  if (wy.lo <= wy.hi && wx.lo <= wx.hi) {
    const float* zl = z_lw + lr * per_row;
    const float* zu = z_uw + lr * per_row;
#pragma unroll 3
    for (int e = lane; e < per_row; e += 32) {
      const int dx = e % g.ww, dy = (e / g.ww) % g.wh, c = e / (g.ww * g.wh);
      if (dy >= ah || dx >= aw) continue;
      const float lo = zl[e], up = zu[e];
      const float vc = fmul(fadd(lo, up), 0.5f), vr = fmul(fsub(up, lo), 0.5f);
      const int64_t col = ((int64_t)c * g.H + wy.lo + dy) * g.W + wx.lo + dx;
      const float* wp = WT + col * N + n0;
#pragma unroll
      for (int j = 0; j < kCwNB; ++j) {
        if (n0 + j < N) {
          const float w = __ldg(wp + j);
          sc[j] = fmaf(vc, w, sc[j]);
          sr[j] = fmaf(vr, fabsf(w), sr[j]);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kCwNB; ++j) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      sc[j] += __shfl_xor_sync(0xffffffffu, sc[j], s);
      sr[j] += __shfl_xor_sync(0xffffffffu, sr[j], s);
    }
    if (lane == 0 && n0 + j < N) {
      y_lw[lr * N + n0 + j] = fsub(sc[j], sr[j]);
      y_uw[lr * N + n0 + j] = fadd(sc[j], sr[j]);
    }
  }
}

// [N, F] -> [F, N] through a 32 x 32 shared-memory tile.
__global__ void __launch_bounds__(256)
cw_transpose_kernel(const float* __restrict__ W, float* __restrict__ WT, int N, int64_t F) {
  __shared__ float tile[32][33];
  const int64_t f0 = (int64_t)blockIdx.x * 32;
  const int n0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8)
    if (n0 + j < N && f0 + tx < F) tile[j][tx] = W[(int64_t)(n0 + j) * F + f0 + tx];
  __syncthreads();
  for (int j = ty; j < 32; j += 8)
    if (f0 + j < F && n0 + tx < N) WT[(f0 + j) * N + n0 + tx] = tile[tx][j];
}

// Dense rows from compact ones: one block per row, zeros outside the window.
__global__ void __launch_bounds__(256)
cw_expand_kernel(const float* __restrict__ z_lw, const float* __restrict__ z_uw, float* __restrict__ y_lw,
                 float* __restrict__ y_uw, int64_t row_start, const CwShape g) {
  const int64_t r = row_start + blockIdx.x;
  int yi, xi;
  pixel_of_row(r, g.H0, g.W0, yi, xi);
  Span wy, wx;
  chain_window(g.ch, g.H0, g.W0, yi, xi, wy, wx);
  const bool empty = wy.lo > wy.hi || wx.lo > wx.hi;
  const int per_row = g.C * g.wh * g.ww;
  const unsigned n = (unsigned)g.C * g.H * g.W, uW = g.W, uH = g.H;
  const float* zl = z_lw + (int64_t)blockIdx.x * per_row;
  const float* zu = z_uw + (int64_t)blockIdx.x * per_row;
  float* ol = y_lw + (int64_t)blockIdx.x * n;
  float* ou = y_uw + (int64_t)blockIdx.x * n;
  for (unsigned t = threadIdx.x; t < n; t += blockDim.x) {
    const unsigned q = t / uW, x = t - q * uW, c = q / uH, y = q - c * uH;
    float lo = 0.f, up = 0.f;
    if (!empty && (int)y >= wy.lo && (int)y <= wy.hi && (int)x >= wx.lo && (int)x <= wx.hi) {
      const int e = ((int)c * g.wh + ((int)y - wy.lo)) * g.ww + ((int)x - wx.lo);
      lo = zl[e];
      up = zu[e];
    }
    ol[t] = lo;
    ou[t] = up;
  }
}

int make_shape(const int* chain, int n_chain, int H0, int W0, int C, int H, int W, CwShape& g) {
  int h, w;
  int rc = chain_from_host(chain, n_chain, H0, W0, g.ch, h, w);
  if (rc != FB_OK) return rc;
  if (n_chain == 0 || C <= 0 || h != H || w != W) return FB_ERR_SHAPE;
  g.H0 = H0, g.W0 = W0, g.C = C, g.H = H, g.W = W;
  chain_extent(g.ch, H0, W0, g.wh, g.ww);
  if ((int64_t)C * H * W > 0x7fffffff || (int64_t)C * g.wh * g.ww > 0x7fffffff) return FB_ERR_SHAPE;
  return FB_OK;
}

inline unsigned grid_for(int64_t items, int per_block) {
  const int64_t want = ceil_div(items, per_block), cap = (int64_t)device_info().sms * 16;
  return (unsigned)std::max<int64_t>(1, std::min(want, cap));
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" int fb_cw_extent(int H0, int W0, const int* chain, int n_chain, int* wh, int* ww) {
  if (!wh || !ww) return FB_ERR_ARG;
  ConvChain ch;
  int h, w;
  int rc = chain_from_host(chain, n_chain, H0, W0, ch, h, w);
  if (rc != FB_OK) return rc;
  chain_extent(ch, H0, W0, *wh, *ww);
  return FB_OK;
}

extern "C" int fb_cw_identity_relax_f32(int op, const float* x_lb, const float* x_ub, const float* Wt, const float* bias,
                                        float scale, float* z_lw, float* z_uw, float* y_lb, float* y_ub, float* col_ws,
                                        int64_t rows, int64_t row_start, int Cin, int H, int W, int Cout, int Kh, int Kw,
                                        int stride, int pad, int p, float eps, int* violation, void* stream) {
  if (!x_lb || !x_ub || !Wt || !z_lw || !z_uw || !y_lb || !y_ub || !col_ws) return FB_ERR_ARG;
  if (rows < 0 || row_start < 0 || Cin <= 0 || H <= 0 || W <= 0 || Cout <= 0 || Kh <= 0 || Kw <= 0 || stride <= 0 || pad < 0 ||
      !valid_norm(p) || row_start + rows > (int64_t)Cin * H * W)
    return FB_ERR_ARG;
  if (op >= 0 && !(op >= FB_RELU && op <= FB_SQRT)) return FB_ERR_ARG;
  const int chain[4] = {Kh, Kw, stride, pad};
  CwShape g;
  const int Ho = (H + 2 * pad - Kh) / stride + 1, Wo = (W + 2 * pad - Kw) / stride + 1;
  if (Ho <= 0 || Wo <= 0) return FB_ERR_SHAPE;
  int rc = make_shape(chain, 1, H, W, Cout, Ho, Wo, g);
  if (rc != FB_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t ncol = (int64_t)Cout * Ho * Wo;
  ProfileScope prof(PK_CONV, 2.0 * rows * Cout * g.wh * g.ww, 4.0 * 2.0 * rows * Cout * g.wh * g.ww, stream);
  // bias part: an ordinary convolution of one image (x_lb doubles as the unused weight operand: Di = 0)
  rc = fb_conv2d_f32(x_lb, x_ub, x_lb, x_ub, Wt, bias, y_lb, y_ub, y_lb, y_ub, 1, 0, Cin, H, W, Cout, Kh, Kw, stride, pad, stream);
  if (rc != FB_OK) return rc;
  float* k_l = col_ws;
  float* k_u = col_ws + ncol;
  rc = launch_identity_columns(op, Wt, y_lb, y_ub, k_l, k_u, scale, Cin, H, W, Cout, Kh, Kw, stride, pad, Ho, Wo, p, eps, violation,
                               st);
  if (rc != FB_OK || rows == 0) return rc;
  cw_identity_rows_kernel<<<grid_for(rows * Cout * g.wh * g.ww, 256), 256, 0, st>>>(Wt, k_l, k_u, z_lw, z_uw, scale, rows, row_start,
                                                                                   Cin, H, W, Cout, Kh, Kw, stride, pad, Ho, Wo,
                                                                                   g.wh, g.ww);
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_cw_conv2d_f32(const float* x_lw, const float* x_uw, const float* Wt, float* y_lw, float* y_uw, int64_t rows,
                                int64_t row_start, int H0, int W0, const int* chain, int n_chain, int Cin, int H, int W,
                                int Cout, int Kh, int Kw, int stride, int pad, void* stream) {
  if (!x_lw || !x_uw || !Wt || !y_lw || !y_uw) return FB_ERR_ARG;
  if (rows < 0 || row_start < 0 || Cin <= 0 || Cout <= 0 || Kh <= 0 || Kw <= 0 || stride <= 0 || pad < 0 || n_chain < 1)
    return FB_ERR_ARG;
  if (n_chain >= kMaxChain) return FB_ERR_SHAPE;
  CwShape gi, go;
  int rc = make_shape(chain, n_chain, H0, W0, Cin, H, W, gi);
  if (rc != FB_OK) return rc;
  const int Ho = (H + 2 * pad - Kh) / stride + 1, Wo = (W + 2 * pad - Kw) / stride + 1;
  if (Ho <= 0 || Wo <= 0) return FB_ERR_SHAPE;
  int out_chain[4 * kMaxChain];
  std::copy(chain, chain + 4 * n_chain, out_chain);
  out_chain[4 * n_chain] = Kh, out_chain[4 * n_chain + 1] = Kw, out_chain[4 * n_chain + 2] = stride, out_chain[4 * n_chain + 3] = pad;
  rc = make_shape(out_chain, n_chain + 1, H0, W0, Cout, Ho, Wo, go);
  if (rc != FB_OK) return rc;
  if (rows == 0) return FB_OK;
  if (rows > 0x7fffffff) return FB_ERR_SHAPE;
  const bool by4 = Cout % 4 == 0;
  const size_t n_w = (size_t)Cin * Kh * Kw * (Cout + (by4 ? 4 : 1));
  const size_t smem = sizeof(float) * (n_w + (n_w & 1) + 2 * (size_t)kCwRows * Cin * gi.wh * gi.ww);
  if (smem > (size_t)device_info().smem_optin) return FB_ERR_SHAPE;
  auto kern = by4 ? cw_conv_kernel<4> : cw_conv_kernel<1>;
  if (int rc = ensure_dynamic_smem(kern, smem)) return rc;
  ProfileScope prof(PK_CONV, 8.0 * rows * Cout * go.wh * go.ww * Cin * Kh * Kw,
                    4.0 * 2.0 * rows * ((double)Cin * gi.wh * gi.ww + (double)Cout * go.wh * go.ww), stream);
  kern<<<(unsigned)ceil_div(rows, kCwRows), 256, smem, (cudaStream_t)stream>>>(
      x_lw, x_uw, Wt, y_lw, y_uw, rows, row_start, H0, W0, gi.ch, Cin, Cout, Kh, Kw, stride, pad, Ho, Wo, gi.wh, gi.ww, go.wh, go.ww);
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_cw_norm_partials_f32(const float* z_lw, const float* z_uw, float* part_l, float* part_u, int64_t rows,
                                       int64_t row_start, int Cin0, int H0, int W0, const int* chain, int n_chain, int C, int H,
                                       int W, int p, void* stream) {
  if (!z_lw || !z_uw || !part_l || !part_u) return FB_ERR_ARG;
  if (rows < 0 || row_start < 0 || Cin0 <= 0 || !valid_norm(p) || row_start + rows > (int64_t)Cin0 * H0 * W0) return FB_ERR_ARG;
  CwShape g;
  int rc = make_shape(chain, n_chain, H0, W0, C, H, W, g);
  if (rc != FB_OK) return rc;
  const int64_t ncol = (int64_t)C * H * W;
  const size_t smem = sizeof(int) * 2 * ((size_t)H0 + W0 + H + W);
  if (smem > 48 * 1024) return FB_ERR_SHAPE;
  ProfileScope prof(PK_RELAX, 4.0 * rows * C * g.wh * g.ww, 4.0 * (2.0 * rows * C * g.wh * g.ww + 2.0 * ncol), stream);
  cw_norm_partials_kernel<<<grid_for(ncol, 8), 256, smem, (cudaStream_t)stream>>>(z_lw, z_uw, part_l, part_u, rows, row_start, Cin0,
                                                                                    g, p);
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_cw_relax_apply_f32(int op, const float* z_lw, const float* z_uw, const float* lb, const float* ub,
                                     const float* norm_l, const float* norm_u, float* out_lw, float* out_uw, float* out_lb,
                                     float* out_ub, float* coef_ws, int64_t rows, int64_t row_start, int H0, int W0,
                                     const int* chain, int n_chain, int C, int H, int W, int p, float eps, int* violation,
                                     void* stream) {
  if (op < FB_RELU || op > FB_SQRT) return FB_ERR_ARG;
  if (!z_lw || !z_uw || !lb || !ub || !norm_l || !norm_u || !out_lw || !out_uw || !out_lb || !out_ub || !coef_ws) return FB_ERR_ARG;
  if (rows < 0 || row_start < 0 || !valid_norm(p)) return FB_ERR_ARG;
  CwShape g;
  int rc = make_shape(chain, n_chain, H0, W0, C, H, W, g);
  if (rc != FB_OK) return rc;
  const int64_t ncol = (int64_t)C * H * W, per_row = (int64_t)C * g.wh * g.ww;
  cudaStream_t st = (cudaStream_t)stream;
  ProfileScope prof(PK_RELAX, 4.0 * rows * per_row, 4.0 * (4.0 * rows * per_row + 10.0 * ncol), stream);
  cw_relax_columns_kernel<<<grid_for(ncol, 256), 256, 0, st>>>(op, lb, ub, norm_l, norm_u, out_lb, out_ub, coef_ws, ncol, p, eps,
                                                               violation);
  FB_LAUNCH_OK();
  if (rows == 0) return FB_OK;
  cw_rescale_kernel<<<(unsigned)ceil_div(rows, 8), 256, 0, st>>>(z_lw, z_uw, coef_ws, out_lw, out_uw, rows, row_start, g);
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_cw_linear_f32(const float* z_lw, const float* z_uw, const float* Wl, float* y_lw, float* y_uw, float* wt_ws,
                                int64_t rows, int64_t row_start, int H0, int W0, const int* chain, int n_chain, int C, int H,
                                int W, int N, void* stream) {
  if (!z_lw || !z_uw || !Wl || !y_lw || !y_uw || !wt_ws) return FB_ERR_ARG;
  if (rows < 0 || row_start < 0 || N <= 0) return FB_ERR_ARG;
  CwShape g;
  int rc = make_shape(chain, n_chain, H0, W0, C, H, W, g);
  if (rc != FB_OK) return rc;
  if (rows == 0) return FB_OK;
  const int64_t warps = rows * ceil_div(N, kCwNB), F = (int64_t)C * H * W;
  if (ceil_div(warps, 8) > 0x7fffffff || ceil_div(N, 32) > 65535) return FB_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  ProfileScope prof(PK_MATMUL, 8.0 * rows * C * g.wh * g.ww * N, 4.0 * (2.0 * rows * C * g.wh * g.ww + 2.0 * rows * N + 2.0 * F * N),
                    stream);
  cw_transpose_kernel<<<dim3((unsigned)ceil_div(F, 32), (unsigned)ceil_div(N, 32)), 256, 0, st>>>(Wl, wt_ws, N, F);
  FB_LAUNCH_OK();
  cw_linear_kernel<<<(unsigned)ceil_div(warps, 8), 256, 0, st>>>(z_lw, z_uw, wt_ws, y_lw, y_uw, rows, row_start, g, N);
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_cw_expand_f32(const float* z_lw, const float* z_uw, float* y_lw, float* y_uw, int64_t rows, int64_t row_start,
                                int H0, int W0, const int* chain, int n_chain, int C, int H, int W, void* stream) {
  if (!z_lw || !z_uw || !y_lw || !y_uw) return FB_ERR_ARG;
  if (rows < 0 || row_start < 0) return FB_ERR_ARG;
  CwShape g;
  int rc = make_shape(chain, n_chain, H0, W0, C, H, W, g);
  if (rc != FB_OK) return rc;
  if (rows == 0) return FB_OK;
  if (rows > 0x7fffffff) return FB_ERR_SHAPE;
  ProfileScope prof(PK_ELEMENTWISE, 0.0, 4.0 * 2.0 * rows * C * H * W, stream);
  cw_expand_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(z_lw, z_uw, y_lw, y_uw, row_start, g);
  FB_LAUNCH_OK();
  return FB_OK;
}
