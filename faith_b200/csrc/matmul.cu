// fb_matmul_f32: bounds x constant weight.  Dispatches to the split-sign GEMM kernels.
#include "common.cuh"

#include <cstdlib>
#include <cstring>

namespace fb {
bool tc_gemm_supported(const float* a_lo, const float* a_up, const float* W, const float* c_lo, const float* c_up,
                       int64_t M, int N, int K);
bool tc_split_supported(int64_t M, int N, int split_rows, int split_d);
int launch_split_sign_tc(const float* a_lo, const float* a_up, const float* W, const float* bias, float* c_lo,
                         float* c_up, int64_t M, int N, int K, cudaStream_t st, int split_rows, int split_d,
                         const float* coef_l = nullptr, const float* coef_u = nullptr, int coef_di = 1,
                         float* norm_lo = nullptr, float* norm_up = nullptr, int norm_p = 0,
                         const float* res_lo = nullptr, const float* res_up = nullptr, const TcBiasRows* br = nullptr,
                         const TcLnArgs* ln = nullptr);
bool tc_bias_rows_mergeable(const float* a_lo, const float* a_up, const float* b_lo, const float* b_up, const float* W,
                            const float* cb_lo, const float* cb_up, int64_t Mb, int N, int K, bool with_norms);
int launch_split_sign_ffma(const float* a_lo, const float* a_up, const float* W, const float* bias, float* c_lo,
                           float* c_up, int64_t M, int N, int K, cudaStream_t st, int split_rows, int split_d);

// FB_MATMUL_IMPL=ffma forces the CUDA-core kernel (exact fp32 products); default: tensor cores
// (3xTF32) for the large weight GEMM when the shape allows it.
static bool use_tensor_cores() {
  static const bool v = []() {
    const char* e = std::getenv("FB_MATMUL_IMPL");
    return !(e && std::strcmp(e, "ffma") == 0);
  }();
  return v;
}

// split_rows > 0: head-split store of the result, [group * H + head][row in group][feature in head]
// with groups of split_rows consecutive rows and heads of split_d consecutive columns.
static int split_sign_gemm(const float* a_lo, const float* a_up, const float* W, const float* bias, float* c_lo,
                           float* c_up, int64_t M, int N, int K, cudaStream_t st, int split_rows = 0, int split_d = 0) {
  if (use_tensor_cores() && tc_gemm_supported(a_lo, a_up, W, c_lo, c_up, M, N, K) &&
      (split_rows == 0 || tc_split_supported(M, N, split_rows, split_d)))
    return launch_split_sign_tc(a_lo, a_up, W, bias, c_lo, c_up, M, N, K, st, split_rows, split_d);
  return launch_split_sign_ffma(a_lo, a_up, W, bias, c_lo, c_up, M, N, K, st, split_rows, split_d);
}

// Ranges of a (head-split) product from the per-word-block column norms that the GEMM epilogue wrote:
//   l[g, l, j] = lb[g, l, j] - eps * sum_w norm_lo[(row * words + w), h * d + j],   g = s * heads + h, row = s * L + l
// and the mirror for u (Bounds.py:311-326).  With plain_lb / plain_ub != nullptr the bias terms come from
// there in the unsplit layout [rows, heads * d] and are written to lb / ub in the head-split layout on the way
// (the head split of the bias rows, VerifierForward.py:208-229, folded into this kernel).
// VEC = 4: a thread handles four consecutive features (d % 4 == 0, 16-byte aligned pointers), 128-bit accesses.
template <int VEC>
__global__ void __launch_bounds__(256)
ranges_from_norms_kernel(float* __restrict__ lb, float* __restrict__ ub, const float* __restrict__ plain_lb,
                         const float* __restrict__ plain_ub, const float* __restrict__ norm_lo,
                         const float* __restrict__ norm_up, float* __restrict__ out_l, float* __restrict__ out_u,
                         int64_t total, int L, int heads, int d, int words, float eps) {
  const int Dy = heads * d;
  const int dv = d / VEC;
  for (int64_t tv = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; tv < total / VEC; tv += (int64_t)gridDim.x * blockDim.x) {
    const int j = (int)(tv % dv) * VEC;
    const int l = (int)((tv / dv) % L);
    const int64_t g = tv / ((int64_t)dv * L);
    const int h = (int)(g % heads);
    const int64_t row = (g / heads) * L + l;
    const int64_t t = tv * VEC;
    const int64_t src = row * Dy + h * d + j;
    float lo[VEC], up[VEC];
    if (VEC == 4) {
      const float4 a = *reinterpret_cast<const float4*>((plain_lb != nullptr ? plain_lb + src : lb + t));
      const float4 b = *reinterpret_cast<const float4*>((plain_ub != nullptr ? plain_ub + src : ub + t));
      lo[0] = a.x; lo[VEC > 1 ? 1 : 0] = a.y; lo[VEC > 2 ? 2 : 0] = a.z; lo[VEC > 3 ? 3 : 0] = a.w;
      up[0] = b.x; up[VEC > 1 ? 1 : 0] = b.y; up[VEC > 2 ? 2 : 0] = b.z; up[VEC > 3 ? 3 : 0] = b.w;
    } else {
      lo[0] = plain_lb != nullptr ? plain_lb[src] : lb[t];
      up[0] = plain_ub != nullptr ? plain_ub[src] : ub[t];
    }
    if (plain_lb != nullptr) {
      if (VEC == 4) {
        *reinterpret_cast<float4*>(lb + t) = make_float4(lo[0], lo[VEC > 1 ? 1 : 0], lo[VEC > 2 ? 2 : 0], lo[VEC > 3 ? 3 : 0]);
        *reinterpret_cast<float4*>(ub + t) = make_float4(up[0], up[VEC > 1 ? 1 : 0], up[VEC > 2 ? 2 : 0], up[VEC > 3 ? 3 : 0]);
      } else {
        lb[t] = lo[0];
        ub[t] = up[0];
      }
    }
    for (int w = 0; w < words; ++w) {
      const int64_t o = (row * words + w) * Dy + h * d + j;
      if (VEC == 4) {
        const float4 nl = *reinterpret_cast<const float4*>(norm_lo + o);
        const float4 nu = *reinterpret_cast<const float4*>(norm_up + o);
        const float n_l[4] = {nl.x, nl.y, nl.z, nl.w}, n_u[4] = {nu.x, nu.y, nu.z, nu.w};
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          lo[e] = fadd(lo[e], fmul(-eps, n_l[e]));
          up[e] = fadd(up[e], fmul(eps, n_u[e]));
        }
      } else {
        lo[0] = fadd(lo[0], fmul(-eps, norm_lo[o]));
        up[0] = fadd(up[0], fmul(eps, norm_up[o]));
      }
    }
    if (VEC == 4) {
      *reinterpret_cast<float4*>(out_l + t) = make_float4(lo[0], lo[VEC > 1 ? 1 : 0], lo[VEC > 2 ? 2 : 0], lo[VEC > 3 ? 3 : 0]);
      *reinterpret_cast<float4*>(out_u + t) = make_float4(up[0], up[VEC > 1 ? 1 : 0], up[VEC > 2 ? 2 : 0], up[VEC > 3 ? 3 : 0]);
    } else {
      out_l[t] = lo[0];
      out_u[t] = up[0];
    }
  }
}
}  // namespace fb

static int matmul_impl(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub, const float* W,
                       const float* bias, float* y_lw, float* y_uw, float* y_lb, float* y_ub, int64_t rows, int Di,
                       int Do, int Dy, int L, int heads, void* stream) {
  if (!x_lw || !x_uw || !x_lb || !x_ub || !W || !y_lw || !y_uw || !y_lb || !y_ub) return FB_ERR_ARG;
  if (rows < 0 || Di < 0 || Do <= 0 || Dy <= 0) return FB_ERR_ARG;   // Di == 0: the bias rows alone
  if (heads > 1 && (L <= 0 || rows % L != 0 || Dy % heads != 0)) return FB_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const double M = (double)rows * (Di + 1);
  fb::ProfileScope prof(fb::PK_MATMUL, 8.0 * M * Do * Dy, 4.0 * (2 * M * Do + 2 * M * Dy + (double)Do * Dy + Dy), stream);
  const int d = heads > 1 ? Dy / heads : 0;
  const int64_t Mw = rows * (int64_t)Di;
  if (heads <= 1 && Di > 0 && fb::use_tensor_cores() && fb::tc_gemm_supported(x_lw, x_uw, W, y_lw, y_uw, Mw, Dy, Do) &&
      fb::tc_bias_rows_mergeable(x_lw, x_uw, x_lb, x_ub, W, y_lb, y_ub, rows, Dy, Do, false)) {
    // both parts on the tensor cores: the bias rows are extra tiles of the weight rows' launch
    const fb::TcBiasRows br = {x_lb, x_ub, bias, y_lb, y_ub, rows, nullptr, nullptr};
    return fb::launch_split_sign_tc(x_lw, x_uw, W, nullptr, y_lw, y_uw, Mw, Dy, Do, st, 0, 0, nullptr, nullptr, 1, nullptr,
                                    nullptr, 0, nullptr, nullptr, &br);
  }
  // weight rows: [rows * Di, Do] -> [rows * Di, Dy]; no bias on the symbolic part
  int rc = fb::split_sign_gemm(x_lw, x_uw, W, nullptr, y_lw, y_uw, rows * (int64_t)Di, Dy, Do, st,
                               heads > 1 ? L * Di : 0, d);
  if (rc != FB_OK) return rc;
  // bias rows: [rows, Do] -> [rows, Dy], + bias
  return fb::split_sign_gemm(x_lb, x_ub, W, bias, y_lb, y_ub, rows, Dy, Do, st, heads > 1 ? L : 0, d);
}

extern "C" int fb_matmul_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                             const float* W, const float* bias, float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                             int64_t rows, int Di, int Do, int Dy, void* stream) {
  return matmul_impl(x_lw, x_uw, x_lb, x_ub, W, bias, y_lw, y_uw, y_lb, y_ub, rows, Di, Do, Dy, 0, 1, stream);
}

extern "C" int fb_matmul_heads_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                   const float* W, const float* bias, float* y_lw, float* y_uw, float* y_lb,
                                   float* y_ub, int64_t rows, int Di, int Do, int Dy, int L, int heads, void* stream) {
  return matmul_impl(x_lw, x_uw, x_lb, x_ub, W, bias, y_lw, y_uw, y_lb, y_ub, rows, Di, Do, Dy, L, heads, stream);
}

// Product of a relaxed bound with a constant weight, the relaxation given by its column slopes
// (fb_relax_coef_f32): y = matmul((c_l * x_lw, c_u * x_uw, x_lb, x_ub), W) + bias, where c_l, c_u are
// [rows, Do] and x_lb, x_ub are the relaxed bias terms.  The slopes are applied by the GEMM while it
// reads the weights, so dense(relu(x)) needs no pass that writes relu(x) (Bounds.py:921-963 followed by
// :397-413).  Tensor-core shapes with Di a multiple of 128 and Do a multiple of 32 only; otherwise
// FB_ERR_SHAPE and nothing is launched (run fb_relax_f32 and fb_matmul_f32).
extern "C" int fb_matmul_coef_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                  const float* c_l, const float* c_u, const float* W, const float* bias,
                                  float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                                  int64_t rows, int Di, int Do, int Dy, void* stream) {
  if (!x_lw || !x_uw || !x_lb || !x_ub || !c_l || !c_u || !W || !y_lw || !y_uw || !y_lb || !y_ub) return FB_ERR_ARG;
  if (rows < 0 || Di <= 0 || Do <= 0 || Dy <= 0) return FB_ERR_ARG;
  const int64_t M = rows * (int64_t)Di;
  if (!fb::use_tensor_cores() || Di % 128 != 0 || Do % 32 != 0 || !fb::aligned16(c_l) || !fb::aligned16(c_u) ||
      !fb::tc_gemm_supported(x_lw, x_uw, W, y_lw, y_uw, M, Dy, Do))
    return FB_ERR_SHAPE;
  if (rows == 0) return FB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const double Mt = (double)rows * (Di + 1);
  fb::ProfileScope prof(fb::PK_MATMUL, 8.0 * Mt * Do * Dy, 4.0 * (2 * Mt * Do + 2 * Mt * Dy + (double)Do * Dy + Dy), stream);
  const fb::TcBiasRows br = {x_lb, x_ub, bias, y_lb, y_ub, rows, nullptr, nullptr};
  const bool merged = fb::tc_bias_rows_mergeable(x_lw, x_uw, x_lb, x_ub, W, y_lb, y_ub, rows, Dy, Do, false);
  int rc = fb::launch_split_sign_tc(x_lw, x_uw, W, nullptr, y_lw, y_uw, M, Dy, Do, st, 0, 0, c_l, c_u, Di, nullptr, nullptr, 0,
                                    nullptr, nullptr, merged ? &br : nullptr);
  if (rc != FB_OK || merged) return rc;
  return fb::split_sign_gemm(x_lb, x_ub, W, bias, y_lb, y_ub, rows, Dy, Do, st);
}

// fb_matmul_heads_f32 that also returns the concretised range of its result, y_l / y_u in the layout of
// y_lb / y_ub: the column norms over dim_in are taken by the GEMM epilogue from the tile it is about to
// store (one word block of dim_in per 128-row tile), so the dot product that consumes y needs no pass of
// its own over y_lw / y_uw (Bounds.py:311-326 fused into :397-413).  norm_ws: 2 * rows * (words + 1) * Dy
// floats of scratch.  Tensor-core shapes with Di == 128 * words only; otherwise FB_ERR_SHAPE and nothing is
// launched (run fb_matmul_heads_f32 and fb_concretize_f32).
extern "C" int fb_matmul_heads_ranges_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                          const float* W, const float* bias, float* y_lw, float* y_uw, float* y_lb,
                                          float* y_ub, float* y_l, float* y_u, float* norm_ws, int64_t rows, int Di,
                                          int Do, int Dy, int L, int heads, int words, int p, float eps, void* stream) {
  if (!x_lw || !x_uw || !x_lb || !x_ub || !W || !y_lw || !y_uw || !y_lb || !y_ub || !y_l || !y_u || !norm_ws)
    return FB_ERR_ARG;
  if (rows < 0 || Di <= 0 || Do <= 0 || Dy <= 0 || words <= 0 || heads < 1 || !fb::valid_norm(p)) return FB_ERR_ARG;
  if (L <= 0 || rows % L != 0 || Dy % heads != 0) return FB_ERR_ARG;
  const int64_t M = rows * (int64_t)Di;
  const int d = Dy / heads;
  if (!fb::use_tensor_cores() || Di != 128 * words || !fb::tc_gemm_supported(x_lw, x_uw, W, y_lw, y_uw, M, Dy, Do) ||
      (heads > 1 && !fb::tc_split_supported(M, Dy, L * Di, d)))
    return FB_ERR_SHAPE;
  if (rows == 0) return FB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const double Mt = (double)rows * (Di + 1);
  fb::ProfileScope prof(fb::PK_MATMUL, 8.0 * Mt * Do * Dy, 4.0 * (2 * Mt * Do + 2 * Mt * Dy + (double)Do * Dy + Dy), stream);
  float* norm_lo = norm_ws;
  float* norm_up = norm_ws + rows * words * Dy;
  // Bias rows.  A head-split store of [rows, Dy] does not fit the tensor-core kernel's output boxes (L rows per
  // group), and the CUDA-core kernel has too few tiles to fill the machine at this size: with heads > 1 the
  // tensor-core kernel writes them unsplit into the scratch and the range kernel splits them on the way.  Where
  // the shapes allow, they are extra tiles of the weight rows' launch.
  float* plain_lb = nullptr;
  float* plain_ub = nullptr;
  float* const b_lo = heads > 1 ? norm_ws + 2 * rows * words * Dy : y_lb;
  float* const b_up = heads > 1 ? b_lo + rows * Dy : y_ub;
  const bool merged = fb::tc_bias_rows_mergeable(x_lw, x_uw, x_lb, x_ub, W, b_lo, b_up, rows, Dy, Do, true);
  const fb::TcBiasRows br = {x_lb, x_ub, bias, b_lo, b_up, rows, nullptr, nullptr};
  int rc = fb::launch_split_sign_tc(x_lw, x_uw, W, nullptr, y_lw, y_uw, M, Dy, Do, st, heads > 1 ? L * Di : 0,
                                    heads > 1 ? d : 0, nullptr, nullptr, 1, norm_lo, norm_up, p, nullptr, nullptr,
                                    merged ? &br : nullptr);
  if (rc != FB_OK) return rc;
  if (merged) {
    if (heads > 1) { plain_lb = b_lo; plain_ub = b_up; }
  } else if (heads > 1 && fb::tc_gemm_supported(x_lb, x_ub, W, norm_ws, norm_ws, rows, Dy, Do)) {
    plain_lb = b_lo;
    plain_ub = b_up;
    rc = fb::launch_split_sign_tc(x_lb, x_ub, W, bias, plain_lb, plain_ub, rows, Dy, Do, st, 0, 0);
  } else {
    rc = fb::split_sign_gemm(x_lb, x_ub, W, bias, y_lb, y_ub, rows, Dy, Do, st, heads > 1 ? L : 0, heads > 1 ? d : 0);
  }
  if (rc != FB_OK) return rc;
  const int64_t total = rows * Dy;
  const bool vec = d % 4 == 0 && fb::aligned16(y_lb) && fb::aligned16(y_ub) && fb::aligned16(y_l) && fb::aligned16(y_u) &&
                   fb::aligned16(norm_ws) && (rows * words * Dy) % 4 == 0;
  const int64_t want = fb::ceil_div(vec ? total / 4 : total, 256), cap = (int64_t)fb::device_info().sms * 8;
  const unsigned blocks = (unsigned)(want < cap ? want : cap);
  if (vec)
    fb::ranges_from_norms_kernel<4><<<blocks, 256, 0, st>>>(y_lb, y_ub, plain_lb, plain_ub, norm_lo, norm_up, y_l, y_u, total, L,
                                                            heads, d, words, eps);
  else
    fb::ranges_from_norms_kernel<1><<<blocks, 256, 0, st>>>(y_lb, y_ub, plain_lb, plain_ub, norm_lo, norm_up, y_l, y_u, total, L,
                                                            heads, d, words, eps);
  FB_LAUNCH_OK();
  return FB_OK;
}

// dense (optionally of a relaxed bound given by its slopes, as fb_matmul_coef_f32) followed by the residual add
// of the encoder blocks (Bounds.add, Bounds.py:383-395, after :397-413): y = matmul(x, W) + bias + r.  The
// residual tile is fetched into the epilogue's staging buffer while the tile is computed and added before the
// store, bit-identical to fb_matmul_f32 followed by fb_add_f32; the layer norm that follows then reads one
// bound instead of two.  c_l / c_u may be NULL (plain dense).  Tensor-core shapes for both the weight rows and
// the bias rows (rows >= 256) only, otherwise FB_ERR_SHAPE and nothing is launched.
extern "C" int fb_matmul_residual_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                      const float* c_l, const float* c_u, const float* W, const float* bias,
                                      const float* r_lw, const float* r_uw, const float* r_lb, const float* r_ub,
                                      float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                                      int64_t rows, int Di, int Do, int Dy, void* stream) {
  if (!x_lw || !x_uw || !x_lb || !x_ub || !W || !r_lw || !r_uw || !r_lb || !r_ub || !y_lw || !y_uw || !y_lb || !y_ub)
    return FB_ERR_ARG;
  if ((c_l == nullptr) != (c_u == nullptr)) return FB_ERR_ARG;
  if (rows < 0 || Di <= 0 || Do <= 0 || Dy <= 0) return FB_ERR_ARG;
  if (y_lw == r_lw || y_lw == r_uw || y_uw == r_lw || y_uw == r_uw || y_lb == r_lb || y_lb == r_ub || y_ub == r_lb ||
      y_ub == r_ub)
    return FB_ERR_ARG;
  const int64_t M = rows * (int64_t)Di;
  if (!fb::use_tensor_cores() || !fb::tc_gemm_supported(x_lw, x_uw, W, y_lw, y_uw, M, Dy, Do) ||
      !fb::tc_gemm_supported(x_lb, x_ub, W, y_lb, y_ub, rows, Dy, Do) || !fb::aligned16(r_lw) || !fb::aligned16(r_uw) ||
      !fb::aligned16(r_lb) || !fb::aligned16(r_ub))
    return FB_ERR_SHAPE;
  if (c_l != nullptr && (Di % 128 != 0 || Do % 32 != 0 || !fb::aligned16(c_l) || !fb::aligned16(c_u))) return FB_ERR_SHAPE;
  if (rows == 0) return FB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const double Mt = (double)rows * (Di + 1);
  fb::ProfileScope prof(fb::PK_MATMUL, 8.0 * Mt * Do * Dy, 4.0 * (2 * Mt * Do + 4 * Mt * Dy + (double)Do * Dy + Dy), stream);
  const fb::TcBiasRows br = {x_lb, x_ub, bias, y_lb, y_ub, rows, r_lb, r_ub};
  const bool merged = fb::tc_bias_rows_mergeable(x_lw, x_uw, x_lb, x_ub, W, y_lb, y_ub, rows, Dy, Do, false);
  int rc = fb::launch_split_sign_tc(x_lw, x_uw, W, nullptr, y_lw, y_uw, M, Dy, Do, st, 0, 0, c_l, c_u, Di, nullptr, nullptr, 0,
                                    r_lw, r_uw, merged ? &br : nullptr);
  if (rc != FB_OK || merged) return rc;
  return fb::launch_split_sign_tc(x_lb, x_ub, W, bias, y_lb, y_ub, rows, Dy, Do, st, 0, 0, nullptr, nullptr, 1, nullptr,
                                  nullptr, 0, r_lb, r_ub);
}

// fb_matmul_residual_f32 followed by the layer norm of the encoder blocks (mode no_var, Bounds.layer_norm,
// Bounds.py:1111-1131), applied by the GEMM epilogue before the store: z = layer_norm(matmul(x, W) + bias + r).  The
// row means the norm needs are not taken from the result (a tile holds half of a row): those of the product come
// from the operand and the column means of W, those of the residual from r_rowsum, which the producer of r left
// behind, and z_rowsum (may be NULL) receives those of z for the next product that takes z as its residual.  Row sums:
// [2 lines][4 partial sums][rows * (Di + 1)] floats, weight rows first, then the bias rows; a reader adds the four
// partial sums of a line in order (a producer that has whole rows writes the sum into the first and zeros into the
// others).  The means are rounded in a different order than fb_layernorm_novar_f32 rounds them, so the result equals
// the separate operators to rounding, not bit for bit.  Dy == 128, Do a multiple of 64 up to 512, Di a multiple of
// 128 / gcd and tensor-core shapes with at least 256 bias rows only; otherwise FB_ERR_SHAPE and nothing is launched.
extern "C" int fb_matmul_residual_ln_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                         const float* c_l, const float* c_u, const float* W, const float* bias,
                                         const float* r_lw, const float* r_uw, const float* r_lb, const float* r_ub,
                                         const float* r_rowsum, const float* gamma, const float* beta,
                                         float* z_lw, float* z_uw, float* z_lb, float* z_ub, float* z_rowsum,
                                         int64_t rows, int Di, int Do, int Dy, void* stream) {
  if (!x_lw || !x_uw || !x_lb || !x_ub || !W || !r_lw || !r_uw || !r_lb || !r_ub || !r_rowsum || !gamma || !beta || !z_lw ||
      !z_uw || !z_lb || !z_ub)
    return FB_ERR_ARG;
  if ((c_l == nullptr) != (c_u == nullptr)) return FB_ERR_ARG;
  if (rows < 0 || Di <= 0 || Do <= 0 || Dy <= 0) return FB_ERR_ARG;
  if (z_lw == r_lw || z_lw == r_uw || z_uw == r_lw || z_uw == r_uw || z_lb == r_lb || z_lb == r_ub || z_ub == r_lb ||
      z_ub == r_ub || z_rowsum == r_rowsum)
    return FB_ERR_ARG;
  const int64_t M = rows * (int64_t)Di;
  if (!fb::use_tensor_cores() || Dy != 128 || Do % 64 != 0 || Do > 512 || M % 128 != 0 ||
      !fb::tc_gemm_supported(x_lw, x_uw, W, z_lw, z_uw, M, Dy, Do) ||
      !fb::tc_bias_rows_mergeable(x_lw, x_uw, x_lb, x_ub, W, z_lb, z_ub, rows, Dy, Do, false) || !fb::aligned16(r_lw) ||
      !fb::aligned16(r_uw) || !fb::aligned16(r_lb) || !fb::aligned16(r_ub))
    return FB_ERR_SHAPE;
  if (c_l != nullptr && (Di % 128 != 0 || !fb::aligned16(c_l) || !fb::aligned16(c_u))) return FB_ERR_SHAPE;
  if (rows == 0) return FB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const double Mt = (double)rows * (Di + 1);
  fb::ProfileScope prof(fb::PK_MATMUL, 8.0 * Mt * Do * Dy, 4.0 * (2 * Mt * Do + 4 * Mt * Dy + (double)Do * Dy + Dy), stream);
  const fb::TcBiasRows br = {x_lb, x_ub, bias, z_lb, z_ub, rows, r_lb, r_ub};
  const fb::TcLnArgs ln = {gamma, beta, W, r_rowsum, z_rowsum, M + rows};
  return fb::launch_split_sign_tc(x_lw, x_uw, W, nullptr, z_lw, z_uw, M, Dy, Do, st, 0, 0, c_l, c_u, Di, nullptr, nullptr, 0,
                                  r_lw, r_uw, &br, &ln);
}
