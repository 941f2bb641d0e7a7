// Bound of a 2-D convolution with constant weights: the split-sign rule of the linear layer
// applied to a convolution whose batch axis is dim_in (every symbolic coordinate is an image),
// evaluated in centre/radius form like the FFMA GEMM:
//   c = (x_lw + x_uw)/2, r = (x_uw - x_lw)/2, y_c = conv(c, W), y_r = conv(r, |W|),
//   y_lw = y_c - y_r, y_uw = y_c + y_r.
// Direct convolution on CUDA cores: a block owns one image, a TH x TW tile of output pixels
// (8 x 32, or 16 x 16 for narrow outputs such as the 16 x 16 map of a stride-2 layer) and CO
// output channels (16 or 32); input channels are staged through shared memory four at a time
// (centre and radius planes with halo), the weights of the chunk are broadcast from shared memory.
#include "common.cuh"

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
  if (smem > 48 * 1024)
    FB_CUDA_OK(cudaFuncSetAttribute(conv_bounds_kernel<TH, TW, CO, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
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

}  // namespace
}  // namespace fb

extern "C" int fb_conv2d_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                             const float* Wt, const float* bias, float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                             int B, int Di, int Cin, int H, int W, int Cout, int Kh, int Kw, int stride, int pad,
                             void* stream) {
  if (!x_lw || !x_uw || !x_lb || !x_ub || !Wt || !y_lw || !y_uw || !y_lb || !y_ub) return FB_ERR_ARG;
  if (B < 0 || Di <= 0 || Cin <= 0 || H <= 0 || W <= 0 || Cout <= 0 || Kh <= 0 || Kw <= 0 || stride <= 0 || pad < 0)
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
