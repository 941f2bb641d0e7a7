// Bound of a 2-D convolution with constant weights: the split-sign rule of the linear layer
// applied to a convolution whose batch axis is dim_in (every symbolic coordinate is an image),
// evaluated in centre/radius form like the FFMA GEMM:
//   c = (x_lw + x_uw)/2, r = (x_uw - x_lw)/2, y_c = conv(c, W), y_r = conv(r, |W|),
//   y_lw = y_c - y_r, y_uw = y_c + y_r.
// Direct convolution on CUDA cores: a block owns one image, a TH x TW tile of output pixels
// (8 x 32, or 16 x 16 for narrow outputs such as the 16 x 16 map of a stride-2 layer) and CO
// output channels (16 or 32); input channels are staged through shared memory four at a time
// (centre and radius planes with halo), the weights of the chunk are broadcast from shared memory.
#include <algorithm>
#include <cstdint>
#include "common.cuh"
#include "conv_window.cuh"

namespace fb {
namespace {

constexpr int kThreads = 256;
constexpr int CC = 4;            // input channels per shared-memory stage
constexpr int kStageBatch = 6;   // input elements per thread whose global loads are in flight together

// KS: filter size when it is the same in both directions and known at compile time (3), 0 = taken from the
// arguments; with KS the tap loops are unrolled and their index arithmetic disappears.
template <int TH, int TW, int CO, int KS>
__global__ void __launch_bounds__(kThreads, 2)
conv_bounds_kernel(const float* __restrict__ x_lo, const float* __restrict__ x_up, const float* __restrict__ Wt,
                   const float* __restrict__ bias, float* __restrict__ y_lo, float* __restrict__ y_up,
                   int Cin, int H, int W, int Cout, int Kh_arg, int Kw_arg, int stride, int pad, int Ho, int Wo,
                   int tiles_h, int tiles_w, int co_chunks) {
  const int Kh = KS ? KS : Kh_arg, Kw = KS ? KS : Kw_arg;
  extern __shared__ __align__(16) float smem[];
  const int in_h = (TH - 1) * stride + Kh, in_w = (TW - 1) * stride + Kw;
  const int plane = in_h * in_w;
  float* s_c = smem;                        // [CC][in_h][in_w]
  float* s_r = s_c + CC * plane;            // [CC][in_h][in_w]
  float* s_w = s_r + CC * plane;            // [CC][Kh][Kw][CO]

  int64_t bid = blockIdx.x;
  const int tw_i = (int)(bid % tiles_w); bid /= tiles_w;
  const int th_i = (int)(bid % tiles_h); bid /= tiles_h;
  const int cq = (int)(bid % co_chunks); bid /= co_chunks;
  const int64_t n = bid;  // image index
  const int tid = threadIdx.x;
  const int tw = tid % TW, th = tid / TW;
  const int oh = th_i * TH + th, ow = tw_i * TW + tw;
  const int ih0 = th_i * TH * stride - pad, iw0 = tw_i * TW * stride - pad;
  const int co0 = cq * CO;

  float acc_c[CO], acc_r[CO];
#pragma unroll
  for (int o = 0; o < CO; ++o) { acc_c[o] = 0.f; acc_r[o] = 0.f; }

  const float* img_lo = x_lo + n * (int64_t)Cin * H * W;
  const float* img_up = x_up + n * (int64_t)Cin * H * W;
  for (int c0 = 0; c0 < Cin; c0 += CC) {
    // staged in batches of kStageBatch elements per thread: all global loads of a batch are issued before
    // the first of them is used, so their latencies overlap instead of adding up
    for (int f0 = tid; f0 < CC * plane; f0 += kThreads * kStageBatch) {
      float lo[kStageBatch], up[kStageBatch];
#pragma unroll
      for (int b = 0; b < kStageBatch; ++b) {
        const int f = f0 + b * kThreads;
        const int c = f / plane, rem = f - c * plane;
        const int rh = rem / in_w;
        const int ih = ih0 + rh, iw = iw0 + rem - rh * in_w;
        lo[b] = 0.f;
        up[b] = 0.f;
        if (f < CC * plane && c0 + c < Cin && ih >= 0 && ih < H && iw >= 0 && iw < W) {
          const int64_t o = ((int64_t)(c0 + c) * H + ih) * W + iw;
          lo[b] = __ldg(img_lo + o);
          up[b] = __ldg(img_up + o);
        }
      }
#pragma unroll
      for (int b = 0; b < kStageBatch; ++b) {
        const int f = f0 + b * kThreads;
        if (f < CC * plane) {
          s_c[f] = fmul(fadd(lo[b], up[b]), 0.5f);
          s_r[f] = fmul(fsub(up[b], lo[b]), 0.5f);
        }
      }
    }
    for (int f = tid; f < CC * Kh * Kw * CO; f += kThreads) {
      const int o = f % CO, t = f / CO;
      const int kw = t % Kw, kh = (t / Kw) % Kh, c = t / (Kw * Kh);
      float w = 0.f;
      if (c0 + c < Cin && co0 + o < Cout) w = __ldg(Wt + (((int64_t)(co0 + o) * Cin + c0 + c) * Kh + kh) * Kw + kw);
      s_w[f] = w;
    }
    __syncthreads();
    const int s0 = th * stride * in_w + tw * stride;   // this thread's window in a staged plane
#pragma unroll(KS ? CC : 1)
    for (int c = 0; c < CC; ++c) {
#pragma unroll
      for (int kh = 0; kh < (KS ? KS : Kh); ++kh) {
#pragma unroll
        for (int kw = 0; kw < (KS ? KS : Kw); ++kw) {
          const int si = s0 + c * plane + kh * in_w + kw;
          const float vc = s_c[si], vr = s_r[si];
          const float* wp = s_w + ((c * Kh + kh) * Kw + kw) * CO;
#pragma unroll
          for (int o4 = 0; o4 < CO; o4 += 4) {
            const float4 w = *reinterpret_cast<const float4*>(wp + o4);
            acc_c[o4 + 0] = fmaf(vc, w.x, acc_c[o4 + 0]); acc_r[o4 + 0] = fmaf(vr, fabsf(w.x), acc_r[o4 + 0]);
            acc_c[o4 + 1] = fmaf(vc, w.y, acc_c[o4 + 1]); acc_r[o4 + 1] = fmaf(vr, fabsf(w.y), acc_r[o4 + 1]);
            acc_c[o4 + 2] = fmaf(vc, w.z, acc_c[o4 + 2]); acc_r[o4 + 2] = fmaf(vr, fabsf(w.z), acc_r[o4 + 2]);
            acc_c[o4 + 3] = fmaf(vc, w.w, acc_c[o4 + 3]); acc_r[o4 + 3] = fmaf(vr, fabsf(w.w), acc_r[o4 + 3]);
          }
        }
      }
    }
    __syncthreads();
  }
  if (oh >= Ho || ow >= Wo) return;
#pragma unroll
  for (int o = 0; o < CO; ++o) {
    if (co0 + o < Cout) {
      float lo = fsub(acc_c[o], acc_r[o]), up = fadd(acc_c[o], acc_r[o]);
      if (bias != nullptr) { lo = fadd(lo, bias[co0 + o]); up = fadd(up, bias[co0 + o]); }
      const int64_t off = ((n * Cout + co0 + o) * (int64_t)Ho + oh) * Wo + ow;
      y_lo[off] = lo;
      y_up[off] = up;
    }
  }
}

// A few images only (the bias part of a bound: one image per batch element): the tiled kernel above would occupy a
// handful of SMs and run at the latency of its staging loop (51 us for one 16 -> 32 channel image of 32 x 32).  Here a
// thread owns one output element and accumulates in the same order (input channel, tap row, tap column; taps outside
// the image are the exact zeros the tiled kernel multiplies), so the value is the tiled kernel's bit for bit.
// KS: filter size when it is the same in both directions and known at compile time (3), 0 = from the arguments.  With KS
// every tap is visited (those outside the image with a zero input: fmaf(0, w, acc) leaves the sum as it is), so the tap
// loops unroll and the loads of a channel are in flight together.
template <int KS>
__global__ void __launch_bounds__(128)
conv_bounds_small_kernel(const float* __restrict__ x_lo, const float* __restrict__ x_up, const float* __restrict__ Wt,
                         const float* __restrict__ bias, float* __restrict__ y_lo, float* __restrict__ y_up, int64_t total,
                         int Cin, int H, int W, int Cout, int Kh_arg, int Kw_arg, int stride, int pad, int Ho, int Wo) {
  const int Kh = KS ? KS : Kh_arg, Kw = KS ? KS : Kw_arg;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const int ow = (int)(t % Wo), oh = (int)((t / Wo) % Ho), co = (int)((t / ((int64_t)Wo * Ho)) % Cout);
  const int64_t n = t / ((int64_t)Wo * Ho * Cout);
  const int ih0 = oh * stride - pad, iw0 = ow * stride - pad;
  const float* il = x_lo + n * (int64_t)Cin * H * W;
  const float* iu = x_up + n * (int64_t)Cin * H * W;
  float ac = 0.f, ar = 0.f;
  if (KS) {
    for (int c = 0; c < Cin; ++c) {
      const float* wp = Wt + ((int64_t)co * Cin + c) * KS * KS;
      float lo[KS ? KS * KS : 1], up[KS ? KS * KS : 1], w[KS ? KS * KS : 1];
#pragma unroll
      for (int kh = 0; kh < KS; ++kh)
#pragma unroll
        for (int kw = 0; kw < KS; ++kw) {
          const int ih = ih0 + kh, iw = iw0 + kw;
          const bool in = ih >= 0 && ih < H && iw >= 0 && iw < W;
          const int64_t o = ((int64_t)c * H + ih) * W + iw;
          lo[kh * KS + kw] = in ? __ldg(il + o) : 0.f;
          up[kh * KS + kw] = in ? __ldg(iu + o) : 0.f;
          w[kh * KS + kw] = __ldg(wp + kh * KS + kw);
        }
#pragma unroll
      for (int k = 0; k < KS * KS; ++k) {
        ac = fmaf(fmul(fadd(lo[k], up[k]), 0.5f), w[k], ac);
        ar = fmaf(fmul(fsub(up[k], lo[k]), 0.5f), fabsf(w[k]), ar);
      }
    }
  } else {
    const int kh0 = max(0, -ih0), kh1 = min(Kh, H - ih0), kw0 = max(0, -iw0), kw1 = min(Kw, W - iw0);
    for (int c = 0; c < Cin; ++c) {
      const float* wp = Wt + ((int64_t)co * Cin + c) * Kh * Kw;
      const int64_t ib = ((int64_t)c * H + ih0) * W + iw0;
      for (int kh = kh0; kh < kh1; ++kh)
        for (int kw = kw0; kw < kw1; ++kw) {
          const float lo = __ldg(il + ib + (int64_t)kh * W + kw), up = __ldg(iu + ib + (int64_t)kh * W + kw);
          const float w = __ldg(wp + kh * Kw + kw);
          ac = fmaf(fmul(fadd(lo, up), 0.5f), w, ac);
          ar = fmaf(fmul(fsub(up, lo), 0.5f), fabsf(w), ar);
        }
    }
  }
  float lo = fsub(ac, ar), up = fadd(ac, ar);
  if (bias != nullptr) { lo = fadd(lo, bias[co]); up = fadd(up, bias[co]); }
  y_lo[t] = lo;
  y_up[t] = up;
}

template <int TH, int TW, int CO, int KS>
int launch_conv_t(const float* x_lo, const float* x_up, const float* Wt, const float* bias, float* y_lo, float* y_up,
                  int64_t N, int Cin, int H, int W, int Cout, int Kh, int Kw, int stride, int pad, int Ho, int Wo,
                  cudaStream_t st) {
  static_assert(TH * TW == kThreads, "one thread per output pixel of the tile");
  const int in_h = (TH - 1) * stride + Kh, in_w = (TW - 1) * stride + Kw;
  const size_t smem = sizeof(float) * ((size_t)2 * CC * in_h * in_w + (size_t)CC * Kh * Kw * CO);
  if (smem > (size_t)device_info().smem_optin) return FB_ERR_SHAPE;
  const int tiles_h = (int)ceil_div(Ho, TH), tiles_w = (int)ceil_div(Wo, TW), co_chunks = (int)ceil_div(Cout, CO);
  const int64_t blocks = N * co_chunks * tiles_h * tiles_w;
  if (blocks > 0x7fffffff) return FB_ERR_SHAPE;
  if (int rc = ensure_dynamic_smem(conv_bounds_kernel<TH, TW, CO, KS>, smem)) return rc;
  conv_bounds_kernel<TH, TW, CO, KS><<<(unsigned)blocks, kThreads, smem, st>>>(x_lo, x_up, Wt, bias, y_lo, y_up, Cin, H, W, Cout,
                                                                         Kh, Kw, stride, pad, Ho, Wo, tiles_h, tiles_w,
                                                                         co_chunks);
  FB_LAUNCH_OK();
  return FB_OK;
}

int launch_conv(const float* x_lo, const float* x_up, const float* Wt, const float* bias, float* y_lo, float* y_up,
                int64_t N, int Cin, int H, int W, int Cout, int Kh, int Kw, int stride, int pad, int Ho, int Wo,
                cudaStream_t st) {
  if (N == 0) return FB_OK;
  {
    // blocks the tiled kernel would launch (its smallest tile: 256 pixels x 16 or 32 channels); fewer than one per
    // SM and it is latency-bound
    const int64_t tiled = N * ceil_div(Cout, Cout > 16 ? 32 : 16) * ceil_div((int64_t)Ho * Wo, 256);
    const int64_t total = N * (int64_t)Cout * Ho * Wo;
    if (tiled < device_info().sms && ceil_div(total, 128) <= 0x7fffffff) {
      if (Kh == 3 && Kw == 3)
        conv_bounds_small_kernel<3><<<(unsigned)ceil_div(total, 128), 128, 0, st>>>(x_lo, x_up, Wt, bias, y_lo, y_up, total, Cin, H,
                                                                                    W, Cout, Kh, Kw, stride, pad, Ho, Wo);
      else
        conv_bounds_small_kernel<0><<<(unsigned)ceil_div(total, 128), 128, 0, st>>>(x_lo, x_up, Wt, bias, y_lo, y_up, total, Cin, H,
                                                                                    W, Cout, Kh, Kw, stride, pad, Ho, Wo);
      FB_LAUNCH_OK();
      return FB_OK;
    }
  }
  const bool narrow = Wo <= 16, wide_co = Cout > 16;
#define FB_CONV_ARGS x_lo, x_up, Wt, bias, y_lo, y_up, N, Cin, H, W, Cout, Kh, Kw, stride, pad, Ho, Wo, st
  if (Kh == 3 && Kw == 3) {
    if (narrow) return wide_co ? launch_conv_t<16, 16, 32, 3>(FB_CONV_ARGS) : launch_conv_t<16, 16, 16, 3>(FB_CONV_ARGS);
    return wide_co ? launch_conv_t<8, 32, 32, 3>(FB_CONV_ARGS) : launch_conv_t<8, 32, 16, 3>(FB_CONV_ARGS);
  }
  if (narrow) return wide_co ? launch_conv_t<16, 16, 32, 0>(FB_CONV_ARGS) : launch_conv_t<16, 16, 16, 0>(FB_CONV_ARGS);
  return wide_co ? launch_conv_t<8, 32, 32, 0>(FB_CONV_ARGS) : launch_conv_t<8, 32, 16, 0>(FB_CONV_ARGS);
#undef FB_CONV_ARGS
}

// ------------------------------------------------------------------------------------------------
// Convolutions behind an identity input.  When every pixel of an image is perturbed, dim_in = Cin * H * W and the
// input bound is lw = uw = scale * I: row r of the weight tensors is the image with the single pixel
// (ci, yi, xi) = unravel(r) set.  Two consequences are used here:
//  * the first convolution needs no input at all: y_lw[r, co, y, x] is scale * W[co, ci, ky, kx] where the tap
//    (ky, kx) of output pixel (y, x) falls on (yi, xi), else zero, and the dual norm of output column (co, y, x)
//    over ALL rows is the norm of the taps of W[co] that fall inside the image -- so the concretised range, the
//    relaxation that follows and its rescale are computed from W alone and the relaxed rows are written directly;
//  * further layers keep the rows local: row r is zero outside a small window around its pixel, so a later
//    convolution only has to compute the outputs whose taps reach into that window and store zeros elsewhere.

// Per output column (co, y, x): slopes and bias terms of the relaxation `op` of conv(identity input) (op < 0: no
// relaxation).  col_ws: k_l, k_u, then the bias terms are written to y_lb, y_ub in place (they hold the conv of
// the bias part on entry).
__global__ void __launch_bounds__(256)
identity_conv_columns_kernel(int op, const float* __restrict__ Wt, float* __restrict__ y_lb, float* __restrict__ y_ub,
                             float* __restrict__ k_l, float* __restrict__ k_u, float scale, int Cin, int H, int W,
                             int Cout, int Kh, int Kw, int stride, int pad, int Ho, int Wo, int p, float eps,
                             int* __restrict__ violation) {
  const int64_t n = (int64_t)Cout * Ho * Wo;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x) {
    const int x = (int)(t % Wo), y = (int)((t / Wo) % Ho), co = (int)(t / ((int64_t)Wo * Ho));
    float acc = 0.f;
    for (int ci = 0; ci < Cin; ++ci)
      for (int ky = 0; ky < Kh; ++ky) {
        const int iy = y * stride - pad + ky;
        if (iy < 0 || iy >= H) continue;
        for (int kx = 0; kx < Kw; ++kx) {
          const int ix = x * stride - pad + kx;
          if (ix < 0 || ix >= W) continue;
          acc = norm_accum(p, acc, fmul(scale, Wt[(((int64_t)co * Cin + ci) * Kh + ky) * Kw + kx]));
        }
      }
    const float nrm = norm_finish(p, acc);
    const float lbv = y_lb[t], ubv = y_ub[t];
    if (op < 0) {
      k_l[t] = 1.f;
      k_u[t] = 1.f;
      continue;
    }
    const float l = fadd(lbv, fmul(-eps, nrm)), u = fadd(ubv, fmul(eps, nrm));
    bool bad = false;
    const ColCoef c = relax_column(op, l, u, lbv, ubv, bad);
    if (bad && violation != nullptr) *violation = 1;
    // both lines of the input coincide, so own-side and cross coefficients apply to the same numbers; for a
    // well-formed column one of each pair is zero and the sum is exact
    k_l[t] = fadd(c.c_ll, c.c_lu);
    k_u[t] = fadd(c.c_ul, c.c_uu);
    y_lb[t] = c.nlb;
    y_ub[t] = c.nub;
  }
}

__device__ __forceinline__ void store_elems(float* p, const float (&v)[4], int n) {
  if (n == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else p[0] = v[0];
}

// One block per row r = row_start + blockIdx.x: zeros everywhere, k * scale * W at the (at most Kh * Kw * Cout)
// positions whose tap falls on the row's pixel.  A thread owns output elements (V in a row of the image at a time:
// 4 when the width allows 16-byte stores, else 1), so nothing is written twice.
template <int V>
__global__ void __launch_bounds__(256)
identity_conv_rows_kernel(const float* __restrict__ Wt, const float* __restrict__ k_l, const float* __restrict__ k_u,
                          float* __restrict__ y_lw, float* __restrict__ y_uw, float scale, int64_t row_start, int Cin,
                          int H, int W, int Cout, int Kh, int Kw, int stride, int pad, int Ho, int Wo) {
  const int64_t r = row_start + blockIdx.x;
  const int xi = (int)(r % W), yi = (int)((r / W) % H), ci = (int)(r / ((int64_t)W * H));
  const unsigned n = (unsigned)Cout * Ho * Wo, uWo = Wo, uHo = Ho;
  float* zl = y_lw + (int64_t)blockIdx.x * n;
  float* zu = y_uw + (int64_t)blockIdx.x * n;
  for (unsigned t = threadIdx.x * V; t < n; t += blockDim.x * V) {
    const unsigned q = t / uWo, x0 = t - q * uWo, co = q / uHo, y = q - co * uHo;
    const int ky = yi - ((int)y * stride - pad);
    float lo[4] = {0.f, 0.f, 0.f, 0.f}, up[4] = {0.f, 0.f, 0.f, 0.f};
    if (ky >= 0 && ky < Kh) {
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const int kx = xi - ((int)(x0 + e) * stride - pad);
        if (kx >= 0 && kx < Kw) {
          const float tap = fmul(scale, __ldg(Wt + (((int64_t)co * Cin + ci) * Kh + ky) * Kw + kx));
          lo[e] = fmul(tap, k_l[t + e]);
          up[e] = fmul(tap, k_u[t + e]);
        }
      }
    }
    store_elems(zl + t, lo, V);
    store_elems(zu + t, up, V);
  }
}

// Split-sign convolution of rows that are zero outside a window (the window follows from the row's pixel and the chain
// of convolutions before this one).  One block per row: the window of the input is staged in shared memory as
// centre and radius, the outputs whose taps reach it are accumulated there in the order of the dense kernel (input
// channel, then tap row, then tap column; the skipped terms are exact zeros, so the value is the dense kernel's bit
// for bit), and the row is then streamed out, zeros outside the output window.
// Shared memory: centre and radius [Cin, win_h, win_w], then lower and upper [Cout, out_h, out_w].
template <int V>
__global__ void __launch_bounds__(256)
conv_window_kernel(const float* __restrict__ x_lo, const float* __restrict__ x_up, const float* __restrict__ Wt,
                   float* __restrict__ y_lo, float* __restrict__ y_up, int64_t row_start, int H0, int W0,
                   const ConvChain ch, int Cin, int H, int W, int Cout, int Kh, int Kw, int stride, int pad, int Ho,
                   int Wo, int win_h, int win_w, int out_h, int out_w) {
  extern __shared__ float win_smem[];
  float* s_c = win_smem;
  float* s_r = s_c + Cin * win_h * win_w;
  float* s_ol = s_r + Cin * win_h * win_w;
  float* s_ou = s_ol + Cout * out_h * out_w;
  const int64_t r = row_start + blockIdx.x;
  const int xi = (int)(r % W0), yi = (int)((r / W0) % H0);
  Span wy, wx;
  chain_window(ch, H0, W0, yi, xi, wy, wx);
  const Span oy = span_after_conv(wy, Kh, stride, pad, Ho), ox = span_after_conv(wx, Kw, stride, pad, Wo);
  const bool empty = wy.lo > wy.hi || wx.lo > wx.hi || oy.lo > oy.hi || ox.lo > ox.hi;
  const int ah = wy.hi - wy.lo + 1, aw = wx.hi - wx.lo + 1, bh = oy.hi - oy.lo + 1, bw = ox.hi - ox.lo + 1;
  const unsigned n_out = (unsigned)Cout * Ho * Wo;
  const int64_t n_in = (int64_t)Cin * H * W;
  const float* il = x_lo + (int64_t)blockIdx.x * n_in;
  const float* iu = x_up + (int64_t)blockIdx.x * n_in;
  float* zl = y_lo + (int64_t)blockIdx.x * n_out;
  float* zu = y_up + (int64_t)blockIdx.x * n_out;
  // 1. zeros everywhere outside the output window: these stores depend on nothing and drain while the window is
  //    computed (a thread owns whole groups of V elements, so nothing is written twice).  The position (y, x0) of a
  //    thread's group is stepped without divisions: one step is blockDim.x * V elements = dq image rows and dx columns.
  {
    const unsigned uWo = Wo, uHo = Ho, step = blockDim.x * V;
    const unsigned dq = step / uWo, dx = step - dq * uWo, dy = dq % uHo;
    unsigned t = threadIdx.x * V;
    unsigned q = t / uWo, x0 = t - q * uWo, y = q % uHo;
    const float zero[4] = {0.f, 0.f, 0.f, 0.f};
    for (; t < n_out; t += step) {
      if (empty || (int)y < oy.lo || (int)y > oy.hi || (int)x0 + V - 1 < ox.lo || (int)x0 > ox.hi) {
        store_elems(zl + t, zero, V);
        store_elems(zu + t, zero, V);
      }
      x0 += dx;
      y += dy;
      if (x0 >= uWo) { x0 -= uWo; ++y; }
      if (y >= uHo) y -= uHo;
    }
  }
  if (empty) return;
  // 2. the window of the input, as centre and radius
  for (int i = threadIdx.x; i < Cin * ah * aw; i += blockDim.x) {
    const int x = i % aw, y = (i / aw) % ah, c = i / (aw * ah);
    const int64_t o = ((int64_t)c * H + wy.lo + y) * W + wx.lo + x;
    const float lo = __ldg(il + o), up = __ldg(iu + o);
    s_c[(c * win_h + y) * win_w + x] = fmul(fadd(lo, up), 0.5f);
    s_r[(c * win_h + y) * win_w + x] = fmul(fsub(up, lo), 0.5f);
  }
  __syncthreads();
  // 3. the outputs that reach it (the taps inside the window are a contiguous range per axis)
  for (int i = threadIdx.x; i < Cout * bh * bw; i += blockDim.x) {
    const int x = i % bw, y = (i / bw) % bh, co = i / (bw * bh);
    const int iy0 = (oy.lo + y) * stride - pad - wy.lo, ix0 = (ox.lo + x) * stride - pad - wx.lo;  // window coordinates
    const int ky0 = max(0, -iy0), ky1 = min(Kh, ah - iy0), kx0 = max(0, -ix0), kx1 = min(Kw, aw - ix0);
    float ac = 0.f, ar = 0.f;
    for (int c = 0; c < Cin; ++c) {
      const float* wp = Wt + ((int64_t)co * Cin + c) * Kh * Kw;
      const int sb = (c * win_h + iy0) * win_w + ix0;
      for (int ky = ky0; ky < ky1; ++ky)
        for (int kx = kx0; kx < kx1; ++kx) {
          const float w = __ldg(wp + ky * Kw + kx);
          ac = fmaf(s_c[sb + ky * win_w + kx], w, ac);
          ar = fmaf(s_r[sb + ky * win_w + kx], fabsf(w), ar);
        }
    }
    s_ol[(co * out_h + y) * out_w + x] = fsub(ac, ar);
    s_ou[(co * out_h + y) * out_w + x] = fadd(ac, ar);
  }
  __syncthreads();
  // 4. the groups of V elements that touch the output window
  const int g0 = ox.lo / V, ng = ox.hi / V - g0 + 1;
  for (int i = threadIdx.x; i < Cout * bh * ng; i += blockDim.x) {
    const int gx = i % ng, y = (i / ng) % bh, co = i / (ng * bh);
    const int x0 = (g0 + gx) * V;
    float lo[4] = {0.f, 0.f, 0.f, 0.f}, up[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const int x = x0 + e;
      if (x >= ox.lo && x <= ox.hi) {
        const int o = (co * out_h + y) * out_w + (x - ox.lo);
        lo[e] = s_ol[o];
        up[e] = s_ou[o];
      }
    }
    const int64_t t = ((int64_t)co * Ho + oy.lo + y) * Wo + x0;
    store_elems(zl + t, lo, V);
    store_elems(zu + t, up, V);
  }
}

}  // namespace

int launch_identity_columns(int op, const float* Wt, float* y_lb, float* y_ub, float* k_l, float* k_u, float scale, int Cin,
                            int H, int W, int Cout, int Kh, int Kw, int stride, int pad, int Ho, int Wo, int p, float eps,
                            int* violation, cudaStream_t st) {
  const int64_t ncol = (int64_t)Cout * Ho * Wo;
  const int64_t want = ceil_div(ncol, 256), cap = (int64_t)device_info().sms * 8;
  identity_conv_columns_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(
      op, Wt, y_lb, y_ub, k_l, k_u, scale, Cin, H, W, Cout, Kh, Kw, stride, pad, Ho, Wo, p, eps, violation);
  FB_LAUNCH_OK();
  return FB_OK;
}

}  // namespace fb

extern "C" int fb_conv2d_identity_relax_f32(int op, const float* x_lb, const float* x_ub, const float* Wt,
                                            const float* bias, float scale, float* y_lw, float* y_uw, float* y_lb,
                                            float* y_ub, float* col_ws, int64_t rows, int64_t row_start, int Cin, int H,
                                            int W, int Cout, int Kh, int Kw, int stride, int pad, int p, float eps,
                                            int* violation, void* stream) {
  if (!x_lb || !x_ub || !Wt || !y_lw || !y_uw || !y_lb || !y_ub || !col_ws) return FB_ERR_ARG;
  if (rows < 0 || row_start < 0 || Cin <= 0 || H <= 0 || W <= 0 || Cout <= 0 || Kh <= 0 || Kw <= 0 || stride <= 0 || pad < 0 ||
      !fb::valid_norm(p) || row_start + rows > (int64_t)Cin * H * W)
    return FB_ERR_ARG;
  if (op >= 0 && !((op >= FB_RELU && op <= FB_SQRT))) return FB_ERR_ARG;
  const int Ho = (H + 2 * pad - Kh) / stride + 1, Wo = (W + 2 * pad - Kw) / stride + 1;
  if (Ho <= 0 || Wo <= 0) return FB_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t ncol = (int64_t)Cout * Ho * Wo;
  fb::ProfileScope prof(fb::PK_CONV, 8.0 * (rows + 1) * ncol * Cin * Kh * Kw, 4.0 * (2.0 * (rows + 1) * ncol), stream);
  // bias part: an ordinary convolution of one image
  int rc = fb::launch_conv(x_lb, x_ub, Wt, bias, y_lb, y_ub, 1, Cin, H, W, Cout, Kh, Kw, stride, pad, Ho, Wo, st);
  if (rc != FB_OK) return rc;
  float* k_l = col_ws;
  float* k_u = col_ws + ncol;
  rc = fb::launch_identity_columns(op, Wt, y_lb, y_ub, k_l, k_u, scale, Cin, H, W, Cout, Kh, Kw, stride, pad, Ho, Wo, p, eps,
                                   violation, st);
  if (rc != FB_OK) return rc;
  if (rows == 0) return FB_OK;
  if (rows > 0x7fffffff) return FB_ERR_SHAPE;
  if (ncol > 0x7fffffff) return FB_ERR_SHAPE;
  if (Wo % 4 == 0 && fb::aligned16(y_lw) && fb::aligned16(y_uw))
    fb::identity_conv_rows_kernel<4><<<(unsigned)rows, 256, 0, st>>>(Wt, k_l, k_u, y_lw, y_uw, scale, row_start, Cin, H, W,
                                                                       Cout, Kh, Kw, stride, pad, Ho, Wo);
  else
    fb::identity_conv_rows_kernel<1><<<(unsigned)rows, 256, 0, st>>>(Wt, k_l, k_u, y_lw, y_uw, scale, row_start, Cin, H, W,
                                                                       Cout, Kh, Kw, stride, pad, Ho, Wo);
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_conv2d_windowed_f32(const float* x_lw, const float* x_uw, const float* Wt, float* y_lw, float* y_uw,
                                      int64_t rows, int64_t row_start, int H0, int W0, const int* chain, int n_chain,
                                      int Cin, int H, int W, int Cout, int Kh, int Kw, int stride, int pad,
                                      void* stream) {
  if (!x_lw || !x_uw || !Wt || !y_lw || !y_uw || (n_chain > 0 && !chain)) return FB_ERR_ARG;
  if (rows < 0 || row_start < 0 || H0 <= 0 || W0 <= 0 || n_chain < 0 || Cin <= 0 || H <= 0 || W <= 0 || Cout <= 0 || Kh <= 0 ||
      Kw <= 0 || stride <= 0 || pad < 0)
    return FB_ERR_ARG;
  if (n_chain > fb::kMaxChain) return FB_ERR_SHAPE;
  fb::ConvChain ch;
  ch.n = n_chain;
  int h = H0, w = W0;
  for (int i = 0; i < n_chain; ++i) {
    ch.kh[i] = chain[4 * i], ch.kw[i] = chain[4 * i + 1], ch.stride[i] = chain[4 * i + 2], ch.pad[i] = chain[4 * i + 3];
    if (ch.kh[i] <= 0 || ch.kw[i] <= 0 || ch.stride[i] <= 0 || ch.pad[i] < 0) return FB_ERR_ARG;
    h = (h + 2 * ch.pad[i] - ch.kh[i]) / ch.stride[i] + 1;
    w = (w + 2 * ch.pad[i] - ch.kw[i]) / ch.stride[i] + 1;
  }
  if (h != H || w != W) return FB_ERR_SHAPE;   // the chain must lead from the H0 x W0 image to this layer's input
  const int Ho = (H + 2 * pad - Kh) / stride + 1, Wo = (W + 2 * pad - Kw) / stride + 1;
  if (Ho <= 0 || Wo <= 0) return FB_ERR_SHAPE;
  if (rows == 0) return FB_OK;
  const double ncol = (double)Cout * Ho * Wo;
  if (rows > 0x7fffffff || ncol > 0x7fffffff) return FB_ERR_SHAPE;
  // the largest window any pixel reaches, in and out (the kernel sizes its shared memory by it)
  int win_h = 1, win_w = 1, out_h = 1, out_w = 1;
  for (int yi = 0; yi < H0; ++yi) {
    fb::Span wy, wx;
    fb::chain_window(ch, H0, W0, yi, 0, wy, wx);
    const fb::Span oy = fb::span_after_conv(wy, Kh, stride, pad, Ho);
    win_h = std::max(win_h, wy.hi - wy.lo + 1);
    out_h = std::max(out_h, oy.hi - oy.lo + 1);
  }
  for (int xi = 0; xi < W0; ++xi) {
    fb::Span wy, wx;
    fb::chain_window(ch, H0, W0, 0, xi, wy, wx);
    const fb::Span ox = fb::span_after_conv(wx, Kw, stride, pad, Wo);
    win_w = std::max(win_w, wx.hi - wx.lo + 1);
    out_w = std::max(out_w, ox.hi - ox.lo + 1);
  }
  const size_t smem = sizeof(float) * 2 * ((size_t)Cin * win_h * win_w + (size_t)Cout * out_h * out_w);
  if (smem > (size_t)fb::device_info().smem_optin) return FB_ERR_SHAPE;   // windows too large to pay: use fb_conv2d_f32
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = Wo % 4 == 0 && fb::aligned16(y_lw) && fb::aligned16(y_uw);
  auto kern = vec ? fb::conv_window_kernel<4> : fb::conv_window_kernel<1>;
  if (int rc = fb::ensure_dynamic_smem(kern, smem)) return rc;
  fb::ProfileScope prof(fb::PK_CONV, 8.0 * rows * Cout * out_h * out_w * Cin * Kh * Kw,
                        4.0 * (2.0 * rows * Cin * win_h * win_w + 2.0 * rows * ncol), stream);
  kern<<<(unsigned)rows, 256, smem, st>>>(x_lw, x_uw, Wt, y_lw, y_uw, row_start, H0, W0, ch, Cin, H, W, Cout, Kh, Kw, stride, pad,
                                          Ho, Wo, win_h, win_w, out_h, out_w);
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_conv2d_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                             const float* Wt, const float* bias, float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                             int B, int Di, int Cin, int H, int W, int Cout, int Kh, int Kw, int stride, int pad,
                             void* stream) {
  if (!x_lw || !x_uw || !x_lb || !x_ub || !Wt || !y_lw || !y_uw || !y_lb || !y_ub) return FB_ERR_ARG;
  // (Di == 0: the bias part alone)
  if (B < 0 || Di < 0 || Cin <= 0 || H <= 0 || W <= 0 || Cout <= 0 || Kh <= 0 || Kw <= 0 || stride <= 0 || pad < 0)
    return FB_ERR_ARG;
  const int Ho = (H + 2 * pad - Kh) / stride + 1, Wo = (W + 2 * pad - Kw) / stride + 1;
  if (Ho <= 0 || Wo <= 0) return FB_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const double n1 = (double)B * (Di + 1);
  fb::ProfileScope prof(fb::PK_CONV, 8.0 * n1 * Cout * Ho * Wo * Cin * Kh * Kw,
                        4.0 * (2 * n1 * Cin * H * W + 2 * n1 * Cout * Ho * Wo + (double)Cout * Cin * Kh * Kw), stream);
  int rc = fb::launch_conv(x_lw, x_uw, Wt, nullptr, y_lw, y_uw, (int64_t)B * Di, Cin, H, W, Cout, Kh, Kw, stride, pad,
                           Ho, Wo, st);
  if (rc != FB_OK) return rc;
  return fb::launch_conv(x_lb, x_ub, Wt, bias, y_lb, y_ub, B, Cin, H, W, Cout, Kh, Kw, stride, pad, Ho, Wo, st);
}
