// Window arithmetic of the convolutions behind an identity input (all pixels of an H0 x W0 image perturbed): row r of
// the weight tensors stands for one pixel, and after a chain of convolutions it is zero outside the window that pixel
// reaches.  Shared by the dense-row kernels (conv.cu) and the compact-row kernels (conv_compact.cu).
#pragma once
#include <algorithm>

#include "common.cuh"

namespace fb {

// The convolutions a row has been through before the one being computed: enough to know, from the row's pixel alone,
// the window outside of which the row is zero.
constexpr int kMaxChain = 8;
struct ConvChain {
  int n;
  int kh[kMaxChain], kw[kMaxChain], stride[kMaxChain], pad[kMaxChain];
};

struct Span { int lo, hi; };   // inclusive; lo > hi: empty

// Outputs (along one axis) of a convolution (k, stride, pad, n_out outputs) that have a tap inside the input span.
__host__ __device__ inline Span span_after_conv(Span s, int k, int stride, int pad, int n_out) {
  if (s.lo > s.hi) return s;
  const int a = s.lo + pad - (k - 1);
  Span o;
  o.lo = a > 0 ? (a + stride - 1) / stride : 0;
  o.hi = (s.hi + pad) / stride;
  if (o.hi > n_out - 1) o.hi = n_out - 1;
  return o;
}

// Window (in the coordinates of the chain's last output) reached by pixel (yi, xi) of the H0 x W0 image.
__host__ __device__ inline void chain_window(const ConvChain& ch, int H0, int W0, int yi, int xi, Span& wy, Span& wx) {
  wy.lo = wy.hi = yi;
  wx.lo = wx.hi = xi;
  int h = H0, w = W0;
  for (int i = 0; i < ch.n; ++i) {
    h = (h + 2 * ch.pad[i] - ch.kh[i]) / ch.stride[i] + 1;
    w = (w + 2 * ch.pad[i] - ch.kw[i]) / ch.stride[i] + 1;
    wy = span_after_conv(wy, ch.kh[i], ch.stride[i], ch.pad[i], h);
    wx = span_after_conv(wx, ch.kw[i], ch.stride[i], ch.pad[i], w);
  }
}


// Host side: the chain as the C ABI passes it (n x 4 ints: kernel height, kernel width, stride, padding).  Fills `ch`
// and the size (h, w) of the chain's last output; FB_ERR_ARG / FB_ERR_SHAPE on malformed input.
inline int chain_from_host(const int* chain, int n_chain, int H0, int W0, ConvChain& ch, int& h, int& w) {
  if (n_chain < 0 || (n_chain > 0 && !chain) || H0 <= 0 || W0 <= 0) return FB_ERR_ARG;
  if (n_chain > kMaxChain) return FB_ERR_SHAPE;
  ch.n = n_chain;
  h = H0, w = W0;
  for (int i = 0; i < n_chain; ++i) {
    ch.kh[i] = chain[4 * i], ch.kw[i] = chain[4 * i + 1], ch.stride[i] = chain[4 * i + 2], ch.pad[i] = chain[4 * i + 3];
    if (ch.kh[i] <= 0 || ch.kw[i] <= 0 || ch.stride[i] <= 0 || ch.pad[i] < 0) return FB_ERR_ARG;
    h = (h + 2 * ch.pad[i] - ch.kh[i]) / ch.stride[i] + 1;
    w = (w + 2 * ch.pad[i] - ch.kw[i]) / ch.stride[i] + 1;
    if (h <= 0 || w <= 0) return FB_ERR_SHAPE;
  }
  return FB_OK;
}

// Largest window any pixel reaches through the chain (at least 1 x 1).
inline void chain_extent(const ConvChain& ch, int H0, int W0, int& win_h, int& win_w) {
  win_h = 1, win_w = 1;
  for (int yi = 0; yi < H0; ++yi) {
    Span wy, wx;
    chain_window(ch, H0, W0, yi, 0, wy, wx);
    win_h = std::max(win_h, wy.hi - wy.lo + 1);
  }
  for (int xi = 0; xi < W0; ++xi) {
    Span wy, wx;
    chain_window(ch, H0, W0, 0, xi, wy, wx);
    win_w = std::max(win_w, wx.hi - wx.lo + 1);
  }
}

// Slopes and bias terms of the relaxation behind the first convolution, per output column (defined in conv.cu).
int launch_identity_columns(int op, const float* Wt, float* y_lb, float* y_ub, float* k_l, float* k_u, float scale, int Cin,
                            int H, int W, int Cout, int Kh, int Kw, int stride, int pad, int Ho, int Wo, int p, float eps,
                            int* violation, cudaStream_t st);

}  // namespace fb
