// Whole-model driver for a small CNN whose whole image is perturbed (dim_in = Cin * H * W, input bound lw = uw = I):
// conv -> [relu] -> (conv | relu)* -> linear -> (relu | linear)* -> concretised output range, for the rows
// [row_start, row_start + rows) of dim_in (all of them, or the shard of one rank).  One call enqueues every launch of
// the pass on the caller's stream; with a communicator the dual norms of each relaxation and of the final
// concretisation are all-reduced over the ranks (the first convolution's relaxation needs no exchange: its norms
// follow from the filter alone).  The reference has no CNN verifier (HandTunedKernels/convolution_verification.cu is a
// benchmark stub, kernel_test/cnn_forward_test_bound.py is commented out); the layer semantics are those of
// Bounds.matmul / Bounds.relu (Transformer_Verification_Code/Verifiers/Bounds.py:397-413, :921-963) with dim_in as
// the batch axis of every convolution.
#include <algorithm>
#include <cstdint>

#include "common.cuh"

namespace fb {
namespace {

struct Geometry {
  int64_t wt;      // elements of the weight of the linear layer that ends the spatial part (transposed copy), or 0
  int64_t f_max;   // widest layer output (features of one row)
  int n_out;       // features of the last layer
  bool ok;
};

Geometry walk(const fb_cnn* net) {
  Geometry g = {0, 0, 0, false};
  if (!net || net->n_layers <= 0 || !net->layer || net->cin <= 0 || net->h <= 0 || net->w <= 0) return g;
  if (net->layer[0].kind != FB_CNN_CONV) return g;
  int c = net->cin, h = net->h, w = net->w;
  int64_t feat = (int64_t)c * h * w;
  bool spatial = true;
  for (int i = 0; i < net->n_layers; ++i) {
    const fb_cnn_layer& ly = net->layer[i];
    if (ly.kind == FB_CNN_CONV) {
      if (!spatial || !ly.weight || ly.cout <= 0 || ly.kh <= 0 || ly.kw <= 0 || ly.stride <= 0 || ly.pad < 0) return g;
      h = (h + 2 * ly.pad - ly.kh) / ly.stride + 1;
      w = (w + 2 * ly.pad - ly.kw) / ly.stride + 1;
      c = ly.cout;
      if (h <= 0 || w <= 0) return g;
      feat = (int64_t)c * h * w;
    } else if (ly.kind == FB_CNN_LINEAR) {
      if (!ly.weight || ly.n_out <= 0) return g;
      if (spatial) g.wt = feat * ly.n_out;
      spatial = false;
      feat = ly.n_out;
    } else if (ly.kind != FB_CNN_RELU) {
      return g;
    }
    if (feat > 0x7fffffff) return g;
    g.f_max = std::max(g.f_max, feat);
  }
  g.n_out = (int)feat;
  g.ok = true;
  return g;
}

struct Set { float *lw, *uw, *lb, *ub; };

inline int64_t round_up(int64_t n) { return (n + 63) / 64 * 64; }   // floats: keeps every buffer 256-byte aligned

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" int64_t fb_cnn_workspace_bytes(const fb_cnn* net, int64_t rows) {
  const Geometry g = walk(net);
  if (!g.ok || rows < 0) return -1;
  // two bound sets (lw, uw [rows, f_max]; lb, ub [f_max]), the column scratch of the first convolution and the norm
  // partials (2 * f_max each), the relaxation coefficients of the compact route (4 * f_max)
  const int64_t per_set = 2 * round_up(rows * g.f_max) + 2 * round_up(g.f_max);
  return 4 * (2 * per_set + 8 * round_up(g.f_max) + round_up(g.wt));
}

extern "C" int fb_cnn_forward_f32(const fb_cnn* net, const float* image, int p, float eps, int64_t row_start, int64_t rows,
                                  fb_comm* comm, int algo, int compact, float* out_l, float* out_u, int* violation,
                                  void* workspace, int64_t workspace_bytes, void* stream) {
  if (!net || !image || !out_l || !out_u || !workspace) return FB_ERR_ARG;
  const Geometry g = walk(net);
  if (!g.ok) return FB_ERR_SHAPE;
  const int64_t di = (int64_t)net->cin * net->h * net->w;
  if (!valid_norm(p) || rows <= 0 || row_start < 0 || row_start + rows > di || rows > 0x7fffffff) return FB_ERR_ARG;
  if (!aligned16(workspace)) return FB_ERR_ALIGN;
  if (workspace_bytes < fb_cnn_workspace_bytes(net, rows)) return FB_ERR_WORKSPACE;

  float* base = static_cast<float*>(workspace);
  const int64_t wsz = round_up(rows * g.f_max), bsz = round_up(g.f_max);
  Set set[2];
  for (int s = 0; s < 2; ++s) {
    set[s].lw = base; base += wsz;
    set[s].uw = base; base += wsz;
    set[s].lb = base; base += bsz;
    set[s].ub = base; base += bsz;
  }
  float* col_ws = base; base += 2 * bsz;
  float* part_ws = base; base += 2 * bsz;
  float* coef_ws = base; base += 4 * bsz;
  float* wt_ws = base;

  int c = net->cin, h = net->h, w = net->w;
  int64_t feat = di;
  int chain[4 * 8];
  int n_chain = 0;
  int cur = 0;
  int i = 0;
  bool cw = compact != 0;   // rows still kept as their windows (compact route, until the first linear layer)
  {
    // the first convolution (and the relaxation behind it, if any) from the filter alone
    const fb_cnn_layer& ly = net->layer[0];
    const bool fuse = net->n_layers > 1 && net->layer[1].kind == FB_CNN_RELU;
    int rc = (cw ? fb_cw_identity_relax_f32 : fb_conv2d_identity_relax_f32)(
        fuse ? FB_RELU : -1, image, image, ly.weight, ly.bias, 1.0f, set[0].lw, set[0].uw, set[0].lb, set[0].ub, col_ws, rows,
        row_start, c, h, w, ly.cout, ly.kh, ly.kw, ly.stride, ly.pad, p, eps, violation, stream);
    if (rc != FB_OK) return rc;
    chain[0] = ly.kh, chain[1] = ly.kw, chain[2] = ly.stride, chain[3] = ly.pad;
    n_chain = 1;
    h = (h + 2 * ly.pad - ly.kh) / ly.stride + 1;
    w = (w + 2 * ly.pad - ly.kw) / ly.stride + 1;
    c = ly.cout;
    feat = (int64_t)c * h * w;
    i = fuse ? 2 : 1;
  }
  // leaves the compact route: dense rows from here on (a layer the compact operators do not cover)
  auto expand = [&]() -> int {
    const Set& x = set[cur];
    const Set& y = set[cur ^ 1];
    int rc = fb_cw_expand_f32(x.lw, x.uw, y.lw, y.uw, rows, row_start, net->h, net->w, chain, n_chain, c, h, w, stream);
    if (rc != FB_OK) return rc;
    FB_CUDA_OK(cudaMemcpyAsync(y.lb, x.lb, sizeof(float) * feat, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    FB_CUDA_OK(cudaMemcpyAsync(y.ub, x.ub, sizeof(float) * feat, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    cur ^= 1;
    cw = false;
    return FB_OK;
  };
  for (; i < net->n_layers; ++i) {
    const fb_cnn_layer& ly = net->layer[i];
    int rc = FB_OK;
    if (cw && ly.kind == FB_CNN_CONV && n_chain + 1 > 8) {
      rc = expand();
      if (rc != FB_OK) return rc;
    }
    const Set& x = set[cur];
    const Set& y = set[cur ^ 1];
    if (ly.kind == FB_CNN_CONV) {
      const int ho = (h + 2 * ly.pad - ly.kh) / ly.stride + 1, wo = (w + 2 * ly.pad - ly.kw) / ly.stride + 1;
      if (cw) {
        rc = fb_cw_conv2d_f32(x.lw, x.uw, ly.weight, y.lw, y.uw, rows, row_start, net->h, net->w, chain, n_chain, c, h, w, ly.cout,
                              ly.kh, ly.kw, ly.stride, ly.pad, stream);
        if (rc == FB_OK)
          rc = fb_conv2d_f32(x.lb, x.ub, x.lb, x.ub, ly.weight, ly.bias, y.lb, y.ub, y.lb, y.ub, 1, 0, c, h, w, ly.cout, ly.kh,
                             ly.kw, ly.stride, ly.pad, stream);
      } else {
        rc = n_chain < 8 ? fb_conv2d_windowed_f32(x.lw, x.uw, ly.weight, y.lw, y.uw, rows, row_start, net->h, net->w, chain,
                                                  n_chain, c, h, w, ly.cout, ly.kh, ly.kw, ly.stride, ly.pad, stream)
                         : FB_ERR_SHAPE;
        if (rc == FB_ERR_SHAPE)   // windows too large to pay (or too long a chain): the dense kernel on the same rows
          rc = fb_conv2d_f32(x.lw, x.uw, x.lb, x.ub, ly.weight, ly.bias, y.lw, y.uw, y.lb, y.ub, 1, (int)rows, c, h, w, ly.cout,
                             ly.kh, ly.kw, ly.stride, ly.pad, stream);
        else if (rc == FB_OK)     // bias part: an ordinary convolution of one image
          rc = fb_conv2d_f32(x.lw, x.uw, x.lb, x.ub, ly.weight, ly.bias, y.lw, y.uw, y.lb, y.ub, 1, 0, c, h, w, ly.cout, ly.kh,
                             ly.kw, ly.stride, ly.pad, stream);
      }
      if (n_chain < 8) {
        chain[4 * n_chain] = ly.kh, chain[4 * n_chain + 1] = ly.kw, chain[4 * n_chain + 2] = ly.stride;
        chain[4 * n_chain + 3] = ly.pad;
      }
      ++n_chain;
      h = ho, w = wo, c = ly.cout;
      feat = (int64_t)c * h * w;
    } else if (ly.kind == FB_CNN_RELU) {
      if (cw) {
        float* part_l = part_ws;
        float* part_u = part_ws + feat;
        rc = fb_cw_norm_partials_f32(x.lw, x.uw, part_l, part_u, rows, row_start, net->cin, net->h, net->w, chain, n_chain, c, h, w,
                                     p, stream);
        if (rc == FB_OK && comm != nullptr) rc = fb_allreduce_f32(comm, part_ws, 2 * feat, p == FB_P1 ? 1 : 0, algo, stream);
        if (rc == FB_OK)   // relaxation coefficients in their own scratch
          rc = fb_cw_relax_apply_f32(FB_RELU, x.lw, x.uw, x.lb, x.ub, part_l, part_u, y.lw, y.uw, y.lb, y.ub, coef_ws, rows,
                                     row_start, net->h, net->w, chain, n_chain, c, h, w, p, eps, violation, stream);
      } else {
        rc = fb_relax_sharded_f32(comm, algo, FB_RELU, x.lw, x.uw, x.lb, x.ub, y.lw, y.uw, y.lb, y.ub, part_ws, 1, (int)rows,
                                  (int)feat, 1, p, eps, violation, stream);
      }
    } else {
      if (cw) {
        rc = fb_cw_linear_f32(x.lw, x.uw, ly.weight, y.lw, y.uw, wt_ws, rows, row_start, net->h, net->w, chain, n_chain, c, h, w, ly.n_out,
                              stream);
        if (rc == FB_OK)
          rc = fb_matmul_f32(x.lb, x.ub, x.lb, x.ub, ly.weight, ly.bias, y.lb, y.ub, y.lb, y.ub, 1, 0, (int)feat, ly.n_out, stream);
        cw = false;
      } else {
        rc = fb_matmul_f32(x.lw, x.uw, x.lb, x.ub, ly.weight, ly.bias, y.lw, y.uw, y.lb, y.ub, 1, (int)rows, (int)feat, ly.n_out,
                           stream);
      }
      feat = ly.n_out;
    }
    if (rc != FB_OK) return rc;
    cur ^= 1;
  }
  if (cw) {   // the network ended on a feature map
    int rc = expand();
    if (rc != FB_OK) return rc;
  }
  const Set& z = set[cur];
  return fb_concretize_sharded_f32(comm, algo, z.lw, z.uw, z.lb, z.ub, out_l, out_u, part_ws, 1, (int)rows, (int)feat, 1, p,
                                   eps, stream);
}
