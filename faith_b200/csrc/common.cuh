// Shared host/device helpers of libfaith_b200 (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "faith_b200.h"

namespace fb {

// ---------------------------------------------------------------- host side
void set_last_cuda_error(int e);

struct DeviceInfo {
  int sms;
  int smem_optin;  // max dynamic shared memory per block (opt-in), bytes
};
// Properties of the current device, queried once per device and cached.
const DeviceInfo& device_info();

#define FB_CUDA_OK(expr)                                   \
  do {                                                     \
    cudaError_t fb_e_ = (expr);                            \
    if (fb_e_ != cudaSuccess) {                            \
      fb::set_last_cuda_error((int)fb_e_);                 \
      return FB_ERR_CUDA;                                  \
    }                                                      \
  } while (0)

// Checks the launches just enqueued (n of them, for the launch counter of fb_profile_*).
#define FB_LAUNCH_OK_N(n)                \
  do {                                   \
    fb::count_launches(n);               \
    FB_CUDA_OK(cudaGetLastError());      \
  } while (0)
#define FB_LAUNCH_OK() FB_LAUNCH_OK_N(1)

void count_launches(int n);

// Hint for the tensor-core GEMM (thread-local, set by the encoder driver around the projections of the first layer):
// the operand has M rows in blocks of Di per (sentence, position) pair, L positions per sentence, and only the
// blocks of the perturbed positions are non-zero (the input bound is an identity at those positions and zero
// elsewhere, VerifierForward.py:127-156).  Positions: `pos` (one set for all sentences) or `inst_pos` (device,
// [sentences, words]).  The zero-radius GEMM then writes zeros for the other blocks without reading or multiplying.
struct LiveRows {
  int L, Di, words;
  int pos[4];
  const int* inst_pos;
  int64_t M;
};
void tc_set_live_rows(const LiveRows* lr);   // nullptr clears

// The bias terms of a bound riding in the GEMM launch of its weight rows (extra tiles at the end of the grid):
// operand a_lo / a_up [M, K], the layer bias (may be null), results c_lo / c_up [M, N] stored plain, and the
// residual res_lo / res_up [M, N] when the weight rows add one.
struct TcBiasRows {
  const float* a_lo;
  const float* a_up;
  const float* bias;
  float* c_lo;
  float* c_up;
  int64_t M;
  const float* res_lo;
  const float* res_up;
};

// Layer norm (mode no_var) applied by the epilogue of a product with residual: gain and shift [N], the weight itself
// (its column means give the row means of the product), the row sums of the residual as its producer left them and
// those of the result for the next consumer: [2 lines][4 partial sums][rs_stride rows], weight rows first, then bias rows.
struct TcLnArgs {
  const float* gamma;
  const float* beta;
  const float* w_raw;
  const float* rs_in;
  float* rs_out;
  int64_t rs_stride;
};

// fb_layernorm_novar_f32 that can also leave the row sums of its result behind (rowsum, may be null; 128 features
// only): [2 lines][4 partial sums][rows * (Di + 1)], of which it writes the first partial sum of each line.
int layernorm_novar_rowsum(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub, const float* r_lw,
                           const float* r_uw, const float* r_lb, const float* r_ub, const float* gamma, const float* beta,
                           float* z_lw, float* z_uw, float* z_lb, float* z_ub, int64_t rows, int Di, int Do, float* rowsum,
                           void* stream);

// Opts `kernel` in to `bytes` of dynamic shared memory on the current device (nothing to do up to 48 KB, or when it
// already has that much): FB_OK or FB_ERR_CUDA.
int ensure_dynamic_smem_impl(const void* func, size_t bytes);
template <typename K>
inline int ensure_dynamic_smem(K kernel, size_t bytes) {
  return ensure_dynamic_smem_impl(reinterpret_cast<const void*>(kernel), bytes);
}

// Optional per-operator timing (fb_profile_enable): the outermost C-ABI operator call on a thread
// brackets its launches with a pair of CUDA events on the caller's stream and records the
// algorithmic work of the call.  Disabled (the default), a scope costs one branch.
enum ProfileKind { PK_MATMUL = 0, PK_RELAX = 1, PK_DOT = 2, PK_MUL = 3, PK_ELEMENTWISE = 4, PK_CONV = 5, PK_COUNT = 6 };
class ProfileScope {
 public:
  ProfileScope(int kind, double flops, double bytes, void* stream);
  ~ProfileScope();
 private:
  int slot_;
  void* stream_;
};

__host__ __device__ inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool valid_norm(int p) { return p == FB_P1 || p == FB_P2 || p == FB_PINF; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// -------------------------------------------------------------- device side
// Scalar arithmetic with the rounding of the reference's PyTorch expressions: one rounding
// per operation, no contraction into fused multiply-adds.
__device__ __forceinline__ float fadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float fsub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float fmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float fdiv(float a, float b) { return __fdiv_rn(a, b); }

constexpr float kGuard = 1e-12f;  // additive guard of every chord slope (Bounds.py:27)

// Accumulation of the dual norm over dim_in: sum |x| (p = inf), sum x^2 (p = 2), max |x| (p = 1).
__device__ __forceinline__ float norm_accum(int p, float acc, float x) {
  if (p == FB_PINF) return acc + fabsf(x);
  if (p == FB_P2) return fmaf(x, x, acc);
  return fmaxf(acc, fabsf(x));
}
__device__ __forceinline__ float norm_combine(int p, float a, float b) {
  return (p == FB_P1) ? fmaxf(a, b) : a + b;
}
__device__ __forceinline__ float norm_finish(int p, float acc) {
  return (p == FB_P2) ? sqrtf(acc) : acc;
}

// Coefficients of one column after a relaxation:
//   out_lw = c_ll * lw + c_lu * uw      out_lb = nlb
//   out_uw = c_ul * lw + c_uu * uw      out_ub = nub
// For every well-formed column (l <= u) exactly one coefficient per line is non-zero, so the
// rescale is a single rounded product as in the reference.
struct ColCoef {
  float c_ll, c_lu, c_ul, c_uu, nlb, nub;
};

// One call of the reference's add_linear (Bounds.py:362-381) at the level of a column:
// adds mask * (line with slope k through (x0, y0) applied to the input bound) to the lower
// (lower = true) or upper output line.  A positive slope keeps the side, any other swaps it.
__device__ __forceinline__ void add_line(ColCoef& c, float mask, bool lower, float k, float x0, float y0,
                                         float lb, float ub) {
  const float kp = (k > 0.f) ? 1.f : 0.f;
  const float kn = 1.f - kp;
  const float own_b = lower ? lb : ub;
  const float oth_b = lower ? ub : lb;
  const float t_own = fmul(fmul(mask, kp), fadd(fmul(fsub(own_b, x0), k), y0));
  const float t_oth = fmul(fmul(mask, kn), fadd(fmul(fsub(oth_b, x0), k), y0));
  const float w_own = fmul(fmul(mask, kp), k);
  const float w_oth = fmul(fmul(mask, kn), k);
  if (lower) {
    c.c_ll = fadd(c.c_ll, w_own);
    c.c_lu = fadd(c.c_lu, w_oth);
    c.nlb = fadd(fadd(c.nlb, t_own), t_oth);
  } else {
    c.c_uu = fadd(c.c_uu, w_own);
    c.c_ul = fadd(c.c_ul, w_oth);
    c.nub = fadd(fadd(c.nub, t_own), t_oth);
  }
}

__device__ __forceinline__ float dtanh_ref(float x) {
  const float ch = coshf(x);
  return fdiv(1.f, fmul(ch, ch));
}

// exp continued linearly above 12 (Bounds.py:984-989)
__device__ __forceinline__ float exp_capped(float x) {
  const float thres = 12.f;
  if (x < thres) return expf(fminf(x, thres));
  return fmul(expf(thres), fadd(fsub(x, thres), 1.f));
}

// Per-column relaxation: from the concretised range (l, u) and the bias terms (lb, ub) to
// the column coefficients.  `bad` is set when FB_RECIPROCAL sees l < 1e-12.
__device__ inline ColCoef relax_column(int op, float l, float u, float lb, float ub, bool& bad) {
  ColCoef c = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (op >= FB_INTERVAL) {
    // interval form (the reference's `ibp` branches): constant bounds, no dependence on the weights
    switch (op - FB_INTERVAL) {
      case FB_RELU: c.nlb = fmaxf(l, 0.f); c.nub = fmaxf(u, 0.f); break;       // Bounds.py:924-926
      case FB_TANH: c.nlb = tanhf(l); c.nub = tanhf(u); break;                  // :1030-1032
      case FB_EXP: c.nlb = expf(l); c.nub = expf(u); break;                     // :973-975
      case FB_RECIPROCAL: c.nlb = fdiv(1.f, u); c.nub = fdiv(1.f, l); break;    // :1139-1143
      case FB_SQR: {                                                            // :863-866
        const float a = fmul(l, l), b = fmul(u, u);
        const float both = 1.f - ((l > 0.f) ? 1.f : 0.f) - ((u < 0.f) ? 1.f : 0.f);
        const float lo = fminf(a, b);
        c.nlb = fsub(lo, fmul(both, lo));   // zero when the range crosses zero
        c.nub = fmaxf(a, b);
        break;
      }
      default:                                                                  // FB_SQRT, :894-898
        if (!(l > 0.f)) bad = true;
        c.nlb = sqrtf(l);
        c.nub = sqrtf(u);
        break;
    }
    return c;
  }
  if (op == FB_SQR) {  // Bounds.py:867-885: chord above; tangent below, placed so that it never goes negative
    add_line(c, 1.f, false, fadd(u, l), l, fmul(l, l), lb, ub);
    if (u < 0.f) {
      const float m = fmaxf(fmul(fadd(l, u), 0.5f), fmul(2.f, u));
      add_line(c, 1.f, true, fmul(2.f, m), m, fmul(m, m), lb, ub);
    }
    if (l > 0.f) {
      const float m = fminf(fmul(fadd(l, u), 0.5f), fmul(2.f, l));
      add_line(c, 1.f, true, fmul(2.f, m), m, fmul(m, m), lb, ub);
    }
    return c;
  }
  if (op == FB_SQRT) {  // Bounds.py:892-913: chord below, tangent at the midpoint above
    if (!(l > 0.f)) bad = true;
    const float sl = sqrtf(l);
    add_line(c, 1.f, true, fdiv(fsub(sqrtf(u), sl), fadd(fsub(u, l), kGuard)), l, sl, lb, ub);
    const float m = fmul(fadd(l, u), 0.5f);
    const float sm = sqrtf(m);
    add_line(c, 1.f, false, fdiv(0.5f, sm), m, sm, lb, ub);
    return c;
  }
  if (op == FB_EXP) {  // Bounds.py:982-997; both slopes are applied to the own side
    const float m = fminf(fmul(fadd(l, u), 0.5f), fadd(l, 0.99f));
    const float kl = expf(fminf(m, 12.f));
    const float el = exp_capped(l);
    const float ku = fdiv(fsub(exp_capped(u), el), fadd(fsub(u, l), kGuard));
    c.c_ll = kl;
    c.nlb = fmul(kl, fadd(fsub(lb, m), 1.f));
    c.c_uu = ku;
    c.nub = fadd(fsub(fmul(ub, ku), fmul(ku, l)), el);
    return c;
  }
  if (op == FB_RECIPROCAL) {  // Bounds.py:1145-1155; both slopes negative: sides swap
    if (!(l >= kGuard)) bad = true;
    const float m = fmul(fadd(l, u), 0.5f);
    const float kl = fdiv(-1.f, fmul(m, m));
    const float ku = fdiv(-1.f, fmul(l, u));
    c.c_lu = kl;
    c.nlb = fadd(fmul(ub, kl), fdiv(2.f, m));
    c.c_ul = ku;
    c.nub = fadd(fsub(fmul(lb, ku), fmul(ku, l)), fdiv(1.f, l));
    return c;
  }
  const float pos = (l > 0.f) ? 1.f : 0.f;
  const float neg = (u < 0.f) ? 1.f : 0.f;
  const float both = 1.f - pos - neg;
  if (op == FB_RELU) {  // Bounds.py:921-963
    if (pos != 0.f) {
      add_line(c, pos, true, 1.f, 0.f, 0.f, lb, ub);
      add_line(c, pos, false, 1.f, 0.f, 0.f, lb, ub);
    }
    if (both != 0.f) {
      const float k_up = fdiv(u, fadd(fsub(u, l), kGuard));
      add_line(c, both, false, k_up, l, 0.f, lb, ub);
      const float k_lo = (fabsf(u) > fabsf(l)) ? 1.f : 0.f;
      add_line(c, both, true, k_lo, 0.f, 0.f, lb, ub);
    }
    return c;
  }
  // FB_TANH, Bounds.py:1027-1103
  if (pos != 0.f || neg != 0.f) {
    const float m = fmul(fadd(l, u), 0.5f);
    const float k_tan = dtanh_ref(m);
    const float y_tan = tanhf(m);
    const float tl = tanhf(l);
    const float k_chd = fdiv(fsub(tanhf(u), tl), fadd(fsub(u, l), kGuard));
    if (neg != 0.f) {
      add_line(c, neg, true, k_tan, m, y_tan, lb, ub);
      add_line(c, neg, false, k_chd, l, tl, lb, ub);
    }
    if (pos != 0.f) {
      add_line(c, pos, false, k_tan, m, y_tan, lb, ub);
      add_line(c, pos, true, k_chd, l, tl, lb, ub);
    }
  }
  if (both != 0.f) {
    const float tu = tanhf(u), tl = tanhf(l);
    // lower line: tangent point in [l, 0] whose tangent passes through (u, tanh u)
    float d = fmul(l, 0.5f), lo = l, hi = 0.f;
#pragma unroll 1
    for (int t = 0; t < 10; ++t) {
      const float v = fsub(fdiv(fsub(tu, tanhf(d)), fadd(fsub(u, d), kGuard)), dtanh_ref(d));
      if (v > 0.f) { lo = d; d = fmul(fadd(d, hi), 0.5f); }
      else         { hi = d; d = fmul(fadd(d, lo), 0.5f); }
    }
    float td = tanhf(d);
    float k = fdiv(fsub(td, tu), fadd(fsub(d, u), kGuard));
    add_line(c, both, true, k, d, td, lb, ub);
    // upper line: tangent point in [0, u] whose tangent passes through (l, tanh l)
    d = fmul(u, 0.5f); lo = 0.f; hi = u;
#pragma unroll 1
    for (int t = 0; t < 10; ++t) {
      const float v = fsub(fdiv(fsub(tanhf(d), tl), fadd(fsub(d, l), kGuard)), dtanh_ref(d));
      if (v > 0.f) { hi = d; d = fmul(fadd(d, lo), 0.5f); }
      else         { lo = d; d = fmul(fadd(d, hi), 0.5f); }
    }
    td = tanhf(d);
    k = fdiv(fsub(td, tl), fadd(fsub(d, l), kGuard));
    add_line(c, both, false, k, d, td, lb, ub);
  }
  return c;
}

}  // namespace fb
