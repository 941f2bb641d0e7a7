// Fused softmax bound: exp -> feature-axis sum -> reciprocal -> McCormick product, the chain of
// Bounds.softmax (Bounds.py:1005-1014 with exp :970-1003, reciprocal :1136-1161, multiply(Bounds)
// :608-651), for rows whose feature axis fits one 32-column tile (attention scores, Do = length).
//
// One block owns one (b, l) row: the [Di, Do] tiles of lw and uw are read from HBM once, kept in
// shared memory through every stage, and the result is written once: 4 tensor passes instead of
// the 18 of the four separate kernels.  Intermediate bounds are never materialised; each stage
// recomputes the rescaled values (lw * k) with the same single-rounding product the separate
// kernels use, so the result matches the unfused chain bit for bit up to the order of the sums.
#include "common.cuh"

namespace fb {
namespace {

constexpr int kThreads = 256;
constexpr int kCW = 32;

// Block-wide reduction of one value per thread (sum or max); result valid in every thread.
__device__ __forceinline__ float block_reduce(float v, int p, float* s_tmp) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = norm_combine(p, v, __shfl_xor_sync(0xffffffffu, v, s));
  __syncthreads();  // s_tmp may still be read from a previous call
  if ((threadIdx.x & 31) == 0) s_tmp[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = s_tmp[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) r = norm_combine(p, r, s_tmp[w]);
  return r;
}

// kP: the norm of the perturbation (FB_P1, FB_P2, FB_PINF) as a template parameter, so that the per-element
// accumulation of the dual norms compiles to one or two instructions instead of a chain of tests.
template <int kP>
__global__ void __launch_bounds__(kThreads)
softmax_bounds_kernel(const float* __restrict__ lw, const float* __restrict__ uw, const float* __restrict__ lb,
                      const float* __restrict__ ub, float* __restrict__ o_lw, float* __restrict__ o_uw,
                      float* __restrict__ o_lb, float* __restrict__ o_ub, float* __restrict__ o_l,
                      float* __restrict__ o_u, int Di, int Do, int words, float eps,
                      int* __restrict__ violation) {
  constexpr int p = kP;
  extern __shared__ __align__(16) float smem[];
  float* s_l = smem;                       // [Di][32] scores lw
  float* s_u = s_l + (size_t)Di * kCW;     // [Di][32] scores uw
  float* s_sl = s_u + (size_t)Di * kCW;    // [Di] row sum of exp.lw
  float* s_su = s_sl + Di;                 // [Di] row sum of exp.uw
  float* s_red = s_su + Di;                // [2][8][32] column partials
  float* s_col = s_red + 2 * 8 * kCW;      // [8][32] per-column scalars
  float* s_tmp = s_col + 8 * kCW;          // [8] block-reduce scratch, [8..16) scalars
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cvl = tid & 7, rg = tid >> 3;   // 8 column lanes (float4) x 32 row groups
  const int col = cvl * 4;
  const bool col_ok = col < Do;             // Do % 4 == 0
  const int blk = Di / words;
  const float* gl = lw + (size_t)row * Di * Do;
  const float* gu = uw + (size_t)row * Di * Do;

  // column-wise dual norm of (a[r][c] * ka[c], b[r][c] * kb[c]) over the rows of every word block,
  // added word by word onto the start values in nl / nu (the bias terms), as the reference's
  // concretize does; result for threads tid < 32 (column tid)
  // With row_sums (second pass only) the same scaled values also give the sums over the features of every
  // row, s_sl / s_su: the denominator of the softmax.
  auto column_norms = [&](bool from_global, bool row_sums, const float* ka, const float* kb, float& nl, float& nu) {
    float tl = nl, tu = nu;
    for (int w = 0; w < words; ++w) {
      float al[4] = {0.f, 0.f, 0.f, 0.f}, au[4] = {0.f, 0.f, 0.f, 0.f};
      for (int r = w * blk + rg; r < (w + 1) * blk; r += 32) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (from_global) {
          if (col_ok) {
            a = __ldg(reinterpret_cast<const float4*>(gl + (size_t)r * Do + col));
            b = __ldg(reinterpret_cast<const float4*>(gu + (size_t)r * Do + col));
          }
          *reinterpret_cast<float4*>(s_l + r * kCW + col) = a;
          *reinterpret_cast<float4*>(s_u + r * kCW + col) = b;
        } else {
          a = *reinterpret_cast<const float4*>(s_l + r * kCW + col);
          b = *reinterpret_cast<const float4*>(s_u + r * kCW + col);
          a.x = fmul(a.x, ka[col + 0]); a.y = fmul(a.y, ka[col + 1]); a.z = fmul(a.z, ka[col + 2]); a.w = fmul(a.w, ka[col + 3]);
          b.x = fmul(b.x, kb[col + 0]); b.y = fmul(b.y, kb[col + 1]); b.z = fmul(b.z, kb[col + 2]); b.w = fmul(b.w, kb[col + 3]);
          if (row_sums) {
            // the eight lanes that share a row (cvl = 0..7) add their four columns each
            const unsigned group = 0xffu << (lane & 24);
            float sa = fadd(fadd(a.x, a.y), fadd(a.z, a.w));
            float sb = fadd(fadd(b.x, b.y), fadd(b.z, b.w));
#pragma unroll
            for (int s = 1; s < 8; s <<= 1) {
              sa += __shfl_xor_sync(group, sa, s);
              sb += __shfl_xor_sync(group, sb, s);
            }
            if (cvl == 0) { s_sl[r] = sa; s_su[r] = sb; }
          }
        }
        al[0] = norm_accum(p, al[0], a.x); al[1] = norm_accum(p, al[1], a.y); al[2] = norm_accum(p, al[2], a.z); al[3] = norm_accum(p, al[3], a.w);
        au[0] = norm_accum(p, au[0], b.x); au[1] = norm_accum(p, au[1], b.y); au[2] = norm_accum(p, au[2], b.z); au[3] = norm_accum(p, au[3], b.w);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int s = 8; s < 32; s <<= 1) {
          al[e] = norm_combine(p, al[e], __shfl_xor_sync(0xffffffffu, al[e], s));
          au[e] = norm_combine(p, au[e], __shfl_xor_sync(0xffffffffu, au[e], s));
        }
      __syncthreads();
      if (lane < 8) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s_red[warp * kCW + lane * 4 + e] = al[e];
          s_red[8 * kCW + warp * kCW + lane * 4 + e] = au[e];
        }
      }
      __syncthreads();
      if (tid < kCW) {
        float sl = s_red[tid], su = s_red[8 * kCW + tid];
#pragma unroll
        for (int k = 1; k < 8; ++k) {
          sl = norm_combine(p, sl, s_red[k * kCW + tid]);
          su = norm_combine(p, su, s_red[8 * kCW + k * kCW + tid]);
        }
        tl = fadd(tl, fmul(-eps, norm_finish(p, sl)));
        tu = fadd(tu, fmul(eps, norm_finish(p, su)));
      }
    }
    nl = tl;
    nu = tu;
  };

  // ---- stage 1: concretise the scores, exp relaxation per column (Bounds.py:970-1003)
  const bool mine = tid < kCW && tid < Do;
  float lbv = 0.f, ubv = 0.f;
  if (mine) { lbv = lb[row * Do + tid]; ubv = ub[row * Do + tid]; }
  float l = lbv, u = ubv;
  column_norms(true, false, nullptr, nullptr, l, u);
  float* c_kl = s_col + 0 * kCW;   // exp slope on lw
  float* c_ku = s_col + 1 * kCW;   // exp slope on uw
  float* c_elb = s_col + 2 * kCW;  // exp.lb
  float* c_eub = s_col + 3 * kCW;  // exp.ub
  float* c_la = s_col + 4 * kCW;   // concretised lower bound of exp
  if (tid < kCW) {
    ColCoef c = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bool bad = false;
    if (mine) c = relax_column(FB_EXP, l, u, lbv, ubv, bad);
    c_kl[tid] = c.c_ll; c_ku[tid] = c.c_uu; c_elb[tid] = c.nlb; c_eub[tid] = c.nub;
  }
  __syncthreads();
  // ---- stage 2: row sums of exp.lw / exp.uw over the features, and the lower range of exp (one pass over
  // the tiles: the scaled values feed both)
  float la = mine ? c_elb[tid] : 0.f, ua_unused = mine ? c_eub[tid] : 0.f;
  column_norms(false, true, c_kl, c_ku, la, ua_unused);
  if (tid < kCW) c_la[tid] = la;
  // ---- stage 3: bounds of the sum, reciprocal relaxation (Bounds.py:1136-1161), range of 1/sum
  float s_lb = 0.f, s_ub = 0.f;
  if (warp == 0) {
    float vlb = mine ? c_elb[tid] : 0.f, vub = mine ? c_eub[tid] : 0.f;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) { vlb += __shfl_xor_sync(0xffffffffu, vlb, s); vub += __shfl_xor_sync(0xffffffffu, vub, s); }
    if (lane == 0) { s_tmp[8] = vlb; s_tmp[9] = vub; }
  }
  __syncthreads();
  s_lb = s_tmp[8]; s_ub = s_tmp[9];
  float ls = s_lb, us = s_ub;
  for (int w = 0; w < words; ++w) {
    float al = 0.f, au = 0.f;
    for (int r = w * blk + tid; r < (w + 1) * blk; r += kThreads) { al = norm_accum(p, al, s_sl[r]); au = norm_accum(p, au, s_su[r]); }
    al = block_reduce(al, p, s_tmp);
    au = block_reduce(au, p, s_tmp);
    ls = fadd(ls, fmul(-eps, norm_finish(p, al)));
    us = fadd(us, fmul(eps, norm_finish(p, au)));
  }
  bool bad = false;
  const ColCoef rc = relax_column(FB_RECIPROCAL, ls, us, s_lb, s_ub, bad);   // same in every thread
  if (bad && tid == 0 && violation != nullptr) *violation = 1;
  const float kl_r = rc.c_lu, ku_r = rc.c_ul;    // 1/sum: lower line = kl_r * sum.uw, upper = ku_r * sum.lw
  float lr = rc.nlb, ur = rc.nub;
  for (int w = 0; w < words; ++w) {
    float al = 0.f, au = 0.f;
    for (int r = w * blk + tid; r < (w + 1) * blk; r += kThreads) {
      al = norm_accum(p, al, fmul(s_su[r], kl_r));
      au = norm_accum(p, au, fmul(s_sl[r], ku_r));
    }
    al = block_reduce(al, p, s_tmp);
    au = block_reduce(au, p, s_tmp);
    lr = fadd(lr, fmul(-eps, norm_finish(p, al)));
    ur = fadd(ur, fmul(eps, norm_finish(p, au)));
  }
  // ---- stage 4: McCormick product exp * (1/sum)  (Bounds.py:608-651, 680-688)
  // lower plane: alpha = l(1/sum) on exp, beta = l(exp) on 1/sum; upper plane: alpha = u(1/sum), beta = l(exp)
  const float al_ = lr, au_ = ur;
  __syncthreads();
  float res_lb = 0.f, res_ub = 0.f;   // bias terms of the result, column tid
  if (mine) {
    const float be = c_la[tid];
    const float gl_ = fmul(-al_, be), gu_ = fmul(-au_, be);
    const float tl = fadd(fmul(al_ > 0.f ? c_elb[tid] : c_eub[tid], al_), gl_);
    const float tu = fadd(fmul(au_ > 0.f ? c_eub[tid] : c_elb[tid], au_), gu_);
    res_lb = fadd(tl, fmul(be > 0.f ? rc.nlb : rc.nub, be));
    res_ub = fadd(tu, fmul(be > 0.f ? rc.nub : rc.nlb, be));
    o_lb[row * Do + tid] = res_lb;
    o_ub[row * Do + tid] = res_ub;
  }
  const bool want_ranges = o_l != nullptr;   // uniform
  if (!col_ok && !want_ranges) return;
  float kl[4] = {0.f, 0.f, 0.f, 0.f}, ku[4] = {0.f, 0.f, 0.f, 0.f}, be[4] = {0.f, 0.f, 0.f, 0.f};
  if (col_ok) {
#pragma unroll
    for (int e = 0; e < 4; ++e) { kl[e] = c_kl[col + e]; ku[e] = c_ku[col + e]; be[e] = c_la[col + e]; }
  }
  float* ol = o_lw + (size_t)row * Di * Do;
  float* ou = o_uw + (size_t)row * Di * Do;
  // The rows are walked word block by word block, so that the dual norms of the result (its concretised
  // range, for the product that consumes the probabilities) can be accumulated on the way out.
  for (int w = 0; w < words; ++w) {
    float nl[4] = {0.f, 0.f, 0.f, 0.f}, nu[4] = {0.f, 0.f, 0.f, 0.f};
    if (col_ok) {
      for (int r = w * blk + rg; r < (w + 1) * blk; r += 32) {
        const float4 a4 = *reinterpret_cast<const float4*>(s_l + r * kCW + col);
        const float4 b4 = *reinterpret_cast<const float4*>(s_u + r * kCW + col);
        const float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
        const float r_l = fmul(s_su[r], kl_r), r_u = fmul(s_sl[r], ku_r);
        float yl[4], yu[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float e_l = fmul(a[e], kl[e]), e_u = fmul(b[e], ku[e]);
          yl[e] = fadd(fmul(al_ > 0.f ? e_l : e_u, al_), fmul(be[e] > 0.f ? r_l : r_u, be[e]));
          yu[e] = fadd(fmul(au_ > 0.f ? e_u : e_l, au_), fmul(be[e] > 0.f ? r_u : r_l, be[e]));
          nl[e] = norm_accum(p, nl[e], yl[e]);
          nu[e] = norm_accum(p, nu[e], yu[e]);
        }
        *reinterpret_cast<float4*>(ol + (size_t)r * Do + col) = make_float4(yl[0], yl[1], yl[2], yl[3]);
        *reinterpret_cast<float4*>(ou + (size_t)r * Do + col) = make_float4(yu[0], yu[1], yu[2], yu[3]);
      }
    }
    if (want_ranges) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int s = 8; s < 32; s <<= 1) {
          nl[e] = norm_combine(p, nl[e], __shfl_xor_sync(0xffffffffu, nl[e], s));
          nu[e] = norm_combine(p, nu[e], __shfl_xor_sync(0xffffffffu, nu[e], s));
        }
      __syncthreads();
      if (lane < 8) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s_red[warp * kCW + lane * 4 + e] = nl[e];
          s_red[8 * kCW + warp * kCW + lane * 4 + e] = nu[e];
        }
      }
      __syncthreads();
      if (tid < kCW) {
        float sl = s_red[tid], su = s_red[8 * kCW + tid];
#pragma unroll
        for (int k = 1; k < 8; ++k) {
          sl = norm_combine(p, sl, s_red[k * kCW + tid]);
          su = norm_combine(p, su, s_red[8 * kCW + k * kCW + tid]);
        }
        res_lb = fadd(res_lb, fmul(-eps, norm_finish(p, sl)));
        res_ub = fadd(res_ub, fmul(eps, norm_finish(p, su)));
      }
    }
  }
  if (want_ranges && mine) {
    o_l[row * Do + tid] = res_lb;
    o_u[row * Do + tid] = res_ub;
  }
}

}  // namespace
}  // namespace fb

using namespace fb;

// out_l / out_u (both or neither): concretised range of the result, [rows, Do], as fb_concretize_f32 would return
// it for the written bounds; the kernel accumulates the dual norms while it writes the result.
extern "C" int fb_softmax_ranges_f32(const float* lw, const float* uw, const float* lb, const float* ub, float* out_lw,
                                     float* out_uw, float* out_lb, float* out_ub, float* out_l, float* out_u,
                                     int64_t rows, int Di, int Do, int words, int p, float eps, int* violation,
                                     void* stream) {
  if ((out_l == nullptr) != (out_u == nullptr)) return FB_ERR_ARG;
  if (rows == 0) return FB_OK;
  if (!lw || !uw || !lb || !ub || !out_lw || !out_uw || !out_lb || !out_ub) return FB_ERR_ARG;
  if (rows < 0 || Di <= 0 || Do <= 0 || words <= 0 || !valid_norm(p)) return FB_ERR_ARG;
  if (Di % words != 0) return FB_ERR_SHAPE;
  const size_t smem = sizeof(float) * ((size_t)2 * Di * kCW + 2 * Di + 2 * 8 * kCW + 8 * kCW + 16);
  // the fused kernel needs the whole feature axis in one 32-column tile and the tiles in shared memory
  if (Do > kCW || Do % 4 != 0 || smem > (size_t)device_info().smem_optin || rows > 0x7fffffff) return FB_ERR_SHAPE;
  if (!aligned16(lw) || !aligned16(uw) || !aligned16(out_lw) || !aligned16(out_uw)) return FB_ERR_ALIGN;
  const double mw = (double)rows * Di * Do, mb = (double)rows * Do;
  ProfileScope prof(PK_RELAX, 30.0 * mw, 4.0 * (4 * mw + 4 * mb), stream);
#define FB_SOFTMAX_LAUNCH(P)                                                                                          \
  do {                                                                                                                \
    if (int rc_ = ensure_dynamic_smem(softmax_bounds_kernel<P>, smem)) return rc_;                                     \
    softmax_bounds_kernel<P><<<(unsigned)rows, kThreads, smem, (cudaStream_t)stream>>>(                                \
        lw, uw, lb, ub, out_lw, out_uw, out_lb, out_ub, out_l, out_u, Di, Do, words, eps, violation);                  \
  } while (0)
  if (p == FB_PINF) FB_SOFTMAX_LAUNCH(FB_PINF);
  else if (p == FB_P2) FB_SOFTMAX_LAUNCH(FB_P2);
  else FB_SOFTMAX_LAUNCH(FB_P1);
#undef FB_SOFTMAX_LAUNCH
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_softmax_f32(const float* lw, const float* uw, const float* lb, const float* ub, float* out_lw,
                              float* out_uw, float* out_lb, float* out_ub, int64_t rows, int Di, int Do, int words,
                              int p, float eps, int* violation, void* stream) {
  return fb_softmax_ranges_f32(lw, uw, lb, ub, out_lw, out_uw, out_lb, out_ub, nullptr, nullptr, rows, Di, Do, words, p,
                               eps, violation, stream);
}
