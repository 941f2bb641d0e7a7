// Whole-model driver: forward linear-bound propagation through a BERT-style encoder for a batch
// of sentences, as one chain of kernel launches on the caller's stream (no host synchronisation,
// no allocation: all intermediates live in a caller-provided arena of four rotating slots).
//
// Stage order follows the reference verifier (VerifierForward.py:93-319): input bounds ->
// embedding layer norm -> per layer [Q,K,V dense -> head split -> scores = Q.K^T / sqrt(d) ->
// softmax (exp, row sum, reciprocal, McCormick product) -> context = probs . V -> head merge ->
// dense -> +residual -> layer norm -> dense -> relu -> dense -> +residual -> layer norm] ->
// first token -> dense -> tanh -> classifier folded to logit0 - logit1 -> concretise.
#include <math.h>

#include <utility>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace fb {
void tc_set_status_sink(int* status);

namespace {

// While a pass is being enqueued, the tensor-core kernels of this thread report an expired wait into the pass's
// status word (bit 2 of `violation`).
struct StatusSinkScope {
  explicit StatusSinkScope(int* status) { tc_set_status_sink(status); }
  ~StatusSinkScope() { tc_set_status_sink(nullptr); }
};

// Around the projections of the first layer: tells the tensor-core GEMM which row blocks of the layer input are zero.
struct LiveRowsScope {
  explicit LiveRowsScope(const LiveRows* lr) { tc_set_live_rows(lr); }
  ~LiveRowsScope() { tc_set_live_rows(nullptr); }
};

struct BoundSet {
  float *lw, *uw, *lb, *ub;
};

inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

struct Plan {
  int64_t cap_w, cap_b;      // floats per lw (resp. lb) tensor of a slot
  int64_t slot_bytes;        // one slot: lw, uw, lb, ub
  int64_t range_floats;      // one operand-range scratch tensor of the dot product
  int64_t small_bytes;       // folded classifier weight + bias
  int64_t norm_floats;       // column norms that the projection GEMMs hand to the range kernel (lower + upper)
  int64_t rowsum_floats;     // row sums of the layer input for the layer norm in a GEMM epilogue: [2 lines][4 partial sums][rows * (Di + 1)]
  int64_t total;
};

Plan make_plan(const fb_encoder* e, int S, int L, int words) {
  Plan p;
  const int64_t D = e->d_model, F = e->ffn, H = e->heads, Di = (int64_t)words * D;
  int64_t feat = D > F ? D : F;
  if (H * L > feat) feat = H * L;
  p.cap_w = (int64_t)S * L * Di * feat;
  p.cap_b = (int64_t)S * L * feat;
  p.slot_bytes = 2 * align_up(p.cap_w * 4, 256) + 2 * align_up(p.cap_b * 4, 256);
  const int64_t d = D / H;
  p.range_floats = (int64_t)S * H * (L > d ? L : d) * (L > d ? L : d);
  p.small_bytes = align_up((D + 1) * 4, 256);
  p.norm_floats = 2 * (int64_t)S * L * (words + 1) * (D > F ? D : F);
  p.rowsum_floats = 8 * (int64_t)S * L * (Di + 1);
  p.total = 4 * p.slot_bytes + 4 * align_up(p.range_floats * 4, 256) + p.small_bytes + align_up(p.norm_floats * 4, 256) +
            align_up(p.rowsum_floats * 4, 256);
  return p;
}

BoundSet carve_slot(char* base, const Plan& p) {
  BoundSet b;
  b.lw = reinterpret_cast<float*>(base);
  b.uw = reinterpret_cast<float*>(base + align_up(p.cap_w * 4, 256));
  b.lb = reinterpret_cast<float*>(base + 2 * align_up(p.cap_w * 4, 256));
  b.ub = reinterpret_cast<float*>(base + 2 * align_up(p.cap_w * 4, 256) + align_up(p.cap_b * 4, 256));
  return b;
}

// lw = uw = identity block at the perturbed positions, lb = ub = embeddings
// (VerifierForward.py:127-152).  positions are packed into `pos` (up to 4 words).
struct Positions { int v[4]; };

// With inst_pos / inst_eps != nullptr every sentence is a verification instance of its own: its perturbed positions
// are inst_pos[s * words + w] and its identity block carries inst_eps[s] instead of 1 (the perturbation radius
// folded into the weights: the dual norm is homogeneous, eps * ||lw|| = ||eps * lw||, so the pass then runs with
// radius 1 for every instance).
__global__ void __launch_bounds__(256)
input_bounds_kernel(const float* __restrict__ emb, float* __restrict__ lw, float* __restrict__ uw,
                    float* __restrict__ lb, float* __restrict__ ub, int64_t n_w, int64_t n_b, int L, int D, int words,
                    Positions pos, const int* __restrict__ inst_pos, const float* __restrict__ inst_eps) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int Di = words * D;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_w; i += stride) {
    const int j = (int)(i % D);
    const int m = (int)((i / D) % Di);
    const int l = (int)((i / ((int64_t)D * Di)) % L);
    const int w = m / D;
    const int64_t sidx = i / ((int64_t)D * Di * L);
    const int pw = inst_pos != nullptr ? inst_pos[sidx * words + w] : pos.v[w];
    const float one = inst_eps != nullptr ? inst_eps[sidx] : 1.f;
    const float v = (l == pw && (m - w * D) == j) ? one : 0.f;
    lw[i] = v;
    uw[i] = v;
  }
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_b; i += stride) {
    const float v = emb[i];
    lb[i] = v;
    ub[i] = v;
  }
}

// Input bounds and the embedding layer norm in one pass for d_model == 128 (a warp per row, four features per
// lane): the rows of lw = uw are generated in registers (one-hot at the perturbed positions, zero elsewhere)
// instead of being written by input_bounds_kernel and read back by the layer norm; same arithmetic as
// fb_layernorm_novar_f32 (Bounds.py:1111-1131 on the bounds of VerifierForward.py:127-152).
__global__ void __launch_bounds__(256)
input_bounds_norm128_kernel(const float* __restrict__ emb, const float* __restrict__ gamma, const float* __restrict__ beta,
                            float* __restrict__ lw, float* __restrict__ uw, float* __restrict__ lb, float* __restrict__ ub,
                            int64_t n_w_rows, int64_t n_b_rows, int L, int words, Positions pos,
                            const int* __restrict__ inst_pos, const float* __restrict__ inst_eps, float* __restrict__ rowsum) {
  constexpr int D = 128;
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * 8;
  const float inv_n = 1.0f / (float)D;
  const float4 g4 = __ldg(reinterpret_cast<const float4*>(gamma) + lane);
  const float4 b4 = __ldg(reinterpret_cast<const float4*>(beta) + lane);
  const float g[4] = {g4.x, g4.y, g4.z, g4.w}, be[4] = {b4.x, b4.y, b4.z, b4.w};
  float gp[4], gn[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) { gp[e] = (g[e] > 0.f) ? g[e] : 0.f; gn[e] = fsub(g[e], gp[e]); }
  const int Di = words * D;
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < n_w_rows + n_b_rows; row += warps) {
    const bool is_bias = row >= n_w_rows;
    float a[4];
    if (is_bias) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(emb + (row - n_w_rows) * D) + lane);
      a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
    } else {
      const int m = (int)(row % Di);
      const int l = (int)((row / Di) % L);
      const int w = m / D;
      const int64_t sidx = row / ((int64_t)Di * L);
      const int pw = inst_pos != nullptr ? inst_pos[sidx * words + w] : pos.v[w];
      const float one = inst_eps != nullptr ? inst_eps[sidx] : 1.f;
      const int hot = (l == pw) ? m - w * D : -1;
#pragma unroll
      for (int e = 0; e < 4; ++e) a[e] = (4 * lane + e == hot) ? one : 0.f;
    }
    float mean = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) mean = fmaf(a[e], inv_n, mean);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mean += __shfl_xor_sync(0xffffffffu, mean, s);
    float ol[4], ou[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float c = fsub(a[e], mean);     // lower and upper line coincide
      ol[e] = fadd(fmul(c, gp[e]), fmul(c, gn[e]));
      ou[e] = fadd(fmul(c, gn[e]), fmul(c, gp[e]));
      if (is_bias) { ol[e] = fadd(ol[e], be[e]); ou[e] = fadd(ou[e], be[e]); }
    }
    float* zl = is_bias ? lb + (row - n_w_rows) * D : lw + row * D;
    float* zu = is_bias ? ub + (row - n_w_rows) * D : uw + row * D;
    reinterpret_cast<float4*>(zl)[lane] = make_float4(ol[0], ol[1], ol[2], ol[3]);
    reinterpret_cast<float4*>(zu)[lane] = make_float4(ou[0], ou[1], ou[2], ou[3]);
    if (rowsum != nullptr) {
      // row sums of the result for a product that applies the next layer norm in its epilogue: the whole sum in the
      // first of the four partial sums of each line (the others were cleared at the start of the pass)
      float sl = fadd(fadd(ol[0], ol[1]), fadd(ol[2], ol[3])), su = fadd(fadd(ou[0], ou[1]), fadd(ou[2], ou[3]));
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) {
        sl += __shfl_xor_sync(0xffffffffu, sl, s);
        su += __shfl_xor_sync(0xffffffffu, su, s);
      }
      const int64_t stride = n_w_rows + n_b_rows;
      if (lane == 0) {
        rowsum[row] = sl;
        rowsum[4 * stride + row] = su;
      }
    }
  }
}

// Mean over the positions: z[s, r] = (sum_l x[s, l, r]) / L for the inner[-sized] slab r of every sentence (r runs over
// Di * D weight entries resp. D bias entries); lanes along r, the L terms added in order.
__global__ void __launch_bounds__(256)
mean_pool_kernel(const float* __restrict__ x_lo, const float* __restrict__ x_up, float* __restrict__ z_lo,
                 float* __restrict__ z_up, int64_t total, int64_t inner, int L) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t sidx = t / inner, r = t - sidx * inner;
    const float* pl = x_lo + sidx * L * inner + r;
    const float* pu = x_up + sidx * L * inner + r;
    float al = 0.f, au = 0.f;
#pragma unroll 4
    for (int l = 0; l < L; ++l) { al = fadd(al, __ldg(pl + (int64_t)l * inner)); au = fadd(au, __ldg(pu + (int64_t)l * inner)); }
    z_lo[t] = __fdiv_rn(al, (float)L);
    z_up[t] = __fdiv_rn(au, (float)L);
  }
}

// classifier folded to one row: w = cls_w[0] - cls_w[1], b = cls_b[0] - cls_b[1]
// (VerifierForward.py:289-292)
__global__ void fold_classifier_kernel(const float* __restrict__ cls_w, const float* __restrict__ cls_b,
                                       float* __restrict__ w, float* __restrict__ b, int D) {
  for (int j = threadIdx.x; j < D; j += blockDim.x) w[j] = fsub(cls_w[j], cls_w[D + j]);
  if (threadIdx.x == 0) b[0] = fsub(cls_b[0], cls_b[1]);
}

#define FB_TRY(expr) do { int rc_ = (expr); if (rc_ != FB_OK) return rc_; } while (0)

int dense(const BoundSet& x, const float* W, const float* bias, const BoundSet& y, int64_t rows, int Di, int Do, int Dy,
          void* st) {
  return fb_matmul_f32(x.lw, x.uw, x.lb, x.ub, W, bias, y.lw, y.uw, y.lb, y.ub, rows, Di, Do, Dy, st);
}

int relax(int op, const BoundSet& x, const BoundSet& y, int64_t rows, int Di, int Do, int words, int p, float eps,
          int* violation, void* st) {
  return fb_relax_f32(op, x.lw, x.uw, x.lb, x.ub, y.lw, y.uw, y.lb, y.ub, rows, Di, Do, words, p, eps, FB_NATIVE,
                      violation, st);
}

// y = layer_norm(x + r) (mode no_var) or y = x + r (mode "no"); r may be null-valued (no residual)
int norm_residual(const fb_encoder* e, const BoundSet& x, const BoundSet* r, const float* g, const float* b,
                  const BoundSet& y, int64_t rows, int Di, int Do, void* st) {
  if (e->layer_norm == 1) {
    return fb_layernorm_novar_f32(x.lw, x.uw, x.lb, x.ub, r ? r->lw : nullptr, r ? r->uw : nullptr,
                                  r ? r->lb : nullptr, r ? r->ub : nullptr, g, b, y.lw, y.uw, y.lb, y.ub, rows, Di, Do, st);
  }
  if (r) return fb_add_f32(x.lw, x.uw, x.lb, x.ub, r->lw, r->uw, r->lb, r->ub, y.lw, y.uw, y.lb, y.ub, rows, Di, Do, st);
  // no norm, no residual: plain copy
  cudaStream_t s = (cudaStream_t)st;
  const size_t nw = (size_t)rows * Di * Do * 4, nb = (size_t)rows * Do * 4;
  FB_CUDA_OK(cudaMemcpyAsync(y.lw, x.lw, nw, cudaMemcpyDeviceToDevice, s));
  FB_CUDA_OK(cudaMemcpyAsync(y.uw, x.uw, nw, cudaMemcpyDeviceToDevice, s));
  FB_CUDA_OK(cudaMemcpyAsync(y.lb, x.lb, nb, cudaMemcpyDeviceToDevice, s));
  FB_CUDA_OK(cudaMemcpyAsync(y.ub, x.ub, nb, cudaMemcpyDeviceToDevice, s));
  return FB_OK;
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" int64_t fb_encoder_workspace_bytes(const fb_encoder* enc, int S, int L, int words) {
  if (!enc || S <= 0 || L <= 0 || words <= 0 || enc->heads <= 0 || enc->d_model % enc->heads != 0) return -1;
  return make_plan(enc, S, L, words).total;
}

// positions (host, one set for all sentences) or inst_pos / inst_eps (device, one set and one radius per sentence)
static int encoder_forward_impl(const fb_encoder* enc, const float* emb, int S, int L, const int* positions,
                                const int* inst_pos, const float* inst_eps, int words, int p, float eps, float* out_l,
                                float* out_u, int* violation, void* workspace, int64_t workspace_bytes, void* stream) {
  if (!enc || !emb || !out_l || !out_u || !violation || !workspace) return FB_ERR_ARG;
  if ((positions == nullptr) == (inst_pos == nullptr) || (inst_pos == nullptr) != (inst_eps == nullptr)) return FB_ERR_ARG;
  if (S <= 0 || L <= 0 || words <= 0 || words > 4 || !valid_norm(p)) return FB_ERR_ARG;
  if (enc->layers < 0 || enc->heads <= 0 || enc->d_model <= 0 || enc->d_model % enc->heads != 0 || enc->ffn <= 0)
    return FB_ERR_ARG;
  if (enc->layer_norm != 0 && enc->layer_norm != 1) return FB_ERR_ARG;
  if (enc->pooling != 0 && enc->pooling != 1) return FB_ERR_ARG;
  for (int w = 0; positions != nullptr && w < words; ++w)
    if (positions[w] < 0 || positions[w] >= L) return FB_ERR_ARG;
  if (!aligned16(workspace)) return FB_ERR_ALIGN;
  const Plan plan = make_plan(enc, S, L, words);
  if (workspace_bytes < plan.total) return FB_ERR_WORKSPACE;

  cudaStream_t st = (cudaStream_t)stream;
  const int D = enc->d_model, H = enc->heads, F = enc->ffn, d = D / H, Di = words * D;
  const int64_t rows = (int64_t)S * L;
  char* base = static_cast<char*>(workspace);
  BoundSet slot[4];
  for (int i = 0; i < 4; ++i) slot[i] = carve_slot(base + i * plan.slot_bytes, plan);
  float* range[4];
  for (int i = 0; i < 4; ++i)
    range[i] = reinterpret_cast<float*>(base + 4 * plan.slot_bytes + i * align_up(plan.range_floats * 4, 256));
  float* fold_w = reinterpret_cast<float*>(base + 4 * plan.slot_bytes + 4 * align_up(plan.range_floats * 4, 256));
  float* fold_b = fold_w + D;
  float* norm_ws = reinterpret_cast<float*>(base + 4 * plan.slot_bytes + 4 * align_up(plan.range_floats * 4, 256) +
                                            plan.small_bytes);
  // row sums of the layer input, for the layer norm applied in the epilogue of the attention output product
  float* rs_in = norm_ws + align_up(plan.norm_floats * 4, 256) / 4;
  // The first layer norm of a block is applied by the epilogue of the attention output product where the shapes allow it
  // (128 features, at least 256 rows): the row sums of the residual (the layer input) are left behind by the kernel
  // that wrote it.  FB_ENCODER_SEPARATE_LN in the environment keeps the norm as a launch of its own (the results
  // differ in the rounding of the row means).  The second norm stays a launch of its own: behind a product with
  // K = 512 the converters' share of the row means costs more than the norm (2.66 against 1.98 + 0.34 ms).
  bool fuse_ln = enc->layer_norm == 1 && D == 128 && rows >= 256 && enc->layers > 0 && getenv("FB_ENCODER_SEPARATE_LN") == nullptr;

  FB_CUDA_OK(cudaMemsetAsync(violation, 0, sizeof(int), st));
  const StatusSinkScope sink(violation);
  // (the producers of the row sums write the first of the four partial sums of a line; the rest stays zero)
  if (fuse_ln) FB_CUDA_OK(cudaMemsetAsync(rs_in, 0, (size_t)plan.rowsum_floats * 4, st));

  // slot roles rotate; names follow the walk-through in the file header
  int A = 0, B = 1, C = 2, Dd = 3;
  {
    Positions pos = {{0, 0, 0, 0}};
    for (int w = 0; positions != nullptr && w < words; ++w) pos.v[w] = positions[w];
    // (lw == uw at the input: the first layer reads the lw buffer as both lines, so the fused kernel is given
    // that buffer twice and the uw buffer of the slot stays unwritten)
    if (enc->layer_norm == 1 && D == 128 && aligned16(emb) && aligned16(enc->emb_ln_g) && aligned16(enc->emb_ln_b)) {
      const int64_t n_w_rows = rows * Di, n_b_rows = rows;
      const int64_t want = ceil_div(n_w_rows + n_b_rows, 8), cap = (int64_t)device_info().sms * 16;
      // (without encoder layers the pooler reads both buffers, so both are written)
      input_bounds_norm128_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(
          emb, enc->emb_ln_g, enc->emb_ln_b, slot[A].lw, enc->layers == 0 ? slot[A].uw : slot[A].lw, slot[A].lb, slot[A].ub,
          n_w_rows, n_b_rows, L, words, pos, inst_pos, inst_eps, fuse_ln ? rs_in : nullptr);
      FB_LAUNCH_OK();
    } else {
      fuse_ln = false;   // (the row sums of the layer input come from the fused input kernel)
      const int64_t n_w = rows * Di * D, n_b = rows * D;
      const int64_t want = ceil_div(n_w, 256), cap = (int64_t)device_info().sms * 16;
      input_bounds_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(emb, slot[B].lw, slot[B].uw, slot[B].lb,
                                                                               slot[B].ub, n_w, n_b, L, D, words, pos, inst_pos, inst_eps);
      FB_LAUNCH_OK();
      FB_TRY(norm_residual(enc, slot[B], nullptr, enc->emb_ln_g, enc->emb_ln_b, slot[A], rows, Di, D, stream));
    }
  }
  const float inv_sqrt_d = (float)(1.0 / sqrt((double)d));
  BoundSet first_token = {nullptr, nullptr, nullptr, nullptr};   // [S, 1, Di, D] output of a last layer run for token 0 only
  for (int li = 0; li < enc->layers; ++li) {
    const fb_encoder_layer& ly = enc->layer[li];
    if (enc->first_token_only != 0 && enc->pooling == 0 && li == enc->layers - 1 && L > 1 && d % 4 == 0) {
      // ---- last layer, first token only (the pooler reads nothing else of its output, VerifierForward.py:269-287).
      // Keys and values at every position; query, attention row, attention output, feed-forward block at position 0.
      // Plain operator calls throughout: the tensors on the query side are 1/L of the usual size.
      const BoundSet X = slot[A];
      char* bump = reinterpret_cast<char*>(slot[B].lw);
      char* const bump_end = bump + plan.slot_bytes;
      bool fits = true;
      auto take = [&](int64_t r, int64_t feat) -> BoundSet {
        BoundSet b;
        const int64_t nw = align_up(r * Di * feat * 4, 256), nb = align_up(r * feat * 4, 256);
        b.lw = reinterpret_cast<float*>(bump); bump += nw;
        b.uw = reinterpret_cast<float*>(bump); bump += nw;
        b.lb = reinterpret_cast<float*>(bump); bump += nb;
        b.ub = reinterpret_cast<float*>(bump); bump += nb;
        if (bump > bump_end) fits = false;
        return b;
      };
      const int64_t SH = (int64_t)S * H;
      const BoundSet Xq = take(S, D), Qh = take(S, D), Sc = take(SH, L), Pr = take(SH, L), E1 = take(SH, L), E2 = take(SH, L),
                     Vt = take(rows, D), Cx = take(S, D), Ao = take(S, D), H3 = take(S, D), Hd = take(S, F), Hr = take(S, F),
                     F2 = take(S, D), Out = take(S, D);
      if (fits) {
        const BoundSet Kh = slot[Dd], Vd = slot[C];
        // the first token's rows of the layer input
        FB_CUDA_OK(cudaMemcpy2DAsync(Xq.lw, (size_t)Di * D * 4, X.lw, (size_t)L * Di * D * 4, (size_t)Di * D * 4, S,
                                     cudaMemcpyDeviceToDevice, st));
        FB_CUDA_OK(cudaMemcpy2DAsync(Xq.uw, (size_t)Di * D * 4, X.uw, (size_t)L * Di * D * 4, (size_t)Di * D * 4, S,
                                     cudaMemcpyDeviceToDevice, st));
        FB_CUDA_OK(cudaMemcpy2DAsync(Xq.lb, (size_t)D * 4, X.lb, (size_t)L * D * 4, (size_t)D * 4, S, cudaMemcpyDeviceToDevice, st));
        FB_CUDA_OK(cudaMemcpy2DAsync(Xq.ub, (size_t)D * 4, X.ub, (size_t)L * D * 4, (size_t)D * 4, S, cudaMemcpyDeviceToDevice, st));
        // query of token 0 [S*H, 1, Di, d], keys of every token [S*H, L, Di, d] (with their ranges from the GEMM's
        // epilogue where the shapes allow it), scores [S*H, 1, Di, L]
        FB_TRY(fb_matmul_heads_f32(Xq.lw, Xq.uw, Xq.lb, Xq.ub, ly.q_w, ly.q_b, Qh.lw, Qh.uw, Qh.lb, Qh.ub, S, Di, D, D, 1, H, stream));
        int kgiven = 0;
        const int krc = fb_matmul_heads_ranges_f32(X.lw, X.uw, X.lb, X.ub, ly.k_w, ly.k_b, Kh.lw, Kh.uw, Kh.lb, Kh.ub, range[2],
                                                   range[3], norm_ws, rows, Di, D, D, L, H, words, p, eps, stream);
        if (krc == FB_OK) kgiven = 2;
        else if (krc == FB_ERR_SHAPE)
          FB_TRY(fb_matmul_heads_f32(X.lw, X.uw, X.lb, X.ub, ly.k_w, ly.k_b, Kh.lw, Kh.uw, Kh.lb, Kh.ub, rows, Di, D, D, L, H, stream));
        else return krc;
        FB_TRY(fb_dot_product_given_f32(Qh.lw, Qh.uw, Qh.lb, Qh.ub, Kh.lw, Kh.uw, Kh.lb, Kh.ub, Sc.lw, Sc.uw, Sc.lb, Sc.ub, range[0],
                                        range[1], range[2], range[3], S * H, 1, L, Di, d, words, p, eps, inv_sqrt_d, FB_NATIVE, 1,
                                        kgiven, stream));
        // probabilities of that row
        int src = fb_softmax_f32(Sc.lw, Sc.uw, Sc.lb, Sc.ub, Pr.lw, Pr.uw, Pr.lb, Pr.ub, SH, Di, L, words, p, eps, violation, stream);
        if (src == FB_ERR_SHAPE || src == FB_ERR_ALIGN) {
          FB_TRY(relax(FB_EXP, Sc, E1, SH, Di, L, words, p, eps, nullptr, stream));
          FB_TRY(fb_rowsum_f32(E1.lw, E1.uw, E1.lb, E1.ub, Sc.lw, Sc.uw, Sc.lb, Sc.ub, SH, Di, L, stream));
          FB_TRY(relax(FB_RECIPROCAL, Sc, E2, SH, Di, L, words, p, eps, violation, stream));
          src = fb_mul_bounds_f32(E1.lw, E1.uw, E1.lb, E1.ub, E2.lw, E2.uw, E2.lb, E2.ub, Pr.lw, Pr.uw, Pr.lb, Pr.ub, SH, Di, L, words,
                                  p, eps, stream);
        }
        if (src != FB_OK) return src;
        // values of every token, split into heads as the projection writes them [S*H, L, Di, d]; context of token 0,
        // head-merged [S, 1, Di, D].  (Other shapes: the transposed copy [S*H, d, Di, L] and the general product.)
        int vgiven = 0;
        const int vrc = fb_matmul_heads_ranges_f32(X.lw, X.uw, X.lb, X.ub, ly.v_w, ly.v_b, Vd.lw, Vd.uw, Vd.lb, Vd.ub, range[2],
                                                   range[3], norm_ws, rows, Di, D, D, L, H, words, p, eps, stream);
        if (vrc == FB_OK) vgiven = 2;
        else if (vrc == FB_ERR_SHAPE)
          FB_TRY(fb_matmul_heads_f32(X.lw, X.uw, X.lb, X.ub, ly.v_w, ly.v_b, Vd.lw, Vd.uw, Vd.lb, Vd.ub, rows, Di, D, D, L, H, stream));
        else return vrc;
        const int crc = fb_context_given_f32(Pr.lw, Pr.uw, Pr.lb, Pr.ub, Vd.lw, Vd.uw, Vd.lb, Vd.ub, Cx.lw, Cx.uw, Cx.lb, Cx.ub,
                                             range[0], range[1], range[2], range[3], S * H, 1, d, Di, L, words, p, eps, 1.0f, H,
                                             vgiven, stream);
        if (crc == FB_ERR_SHAPE) {
          FB_TRY(dense(X, ly.v_w, ly.v_b, Vd, rows, Di, D, D, stream));
          FB_TRY(fb_split_heads_f32(Vd.lw, Vd.lb, Vt.lw, Vt.lb, S, L, Di, H, d, 1, stream));
          FB_TRY(fb_split_heads_f32(Vd.uw, Vd.ub, Vt.uw, Vt.ub, S, L, Di, H, d, 1, stream));
          FB_TRY(fb_dot_product_heads_f32(Pr.lw, Pr.uw, Pr.lb, Pr.ub, Vt.lw, Vt.uw, Vt.lb, Vt.ub, Cx.lw, Cx.uw, Cx.lb, Cx.ub, range[0],
                                          range[1], range[2], range[3], S * H, 1, d, Di, L, words, p, eps, 1.0f, FB_NATIVE, H, stream));
        } else if (crc != FB_OK) {
          return crc;
        }
        // attention output + residual, layer norm; feed-forward block + residual, layer norm
        FB_TRY(dense(Cx, ly.ao_w, ly.ao_b, Ao, S, Di, D, D, stream));
        FB_TRY(norm_residual(enc, Ao, &Xq, ly.ln1_g, ly.ln1_b, H3, S, Di, D, stream));
        FB_TRY(dense(H3, ly.f1_w, ly.f1_b, Hd, S, Di, D, F, stream));
        FB_TRY(relax(FB_RELU, Hd, Hr, S, Di, F, words, p, eps, nullptr, stream));
        FB_TRY(dense(Hr, ly.f2_w, ly.f2_b, F2, S, Di, F, D, stream));
        FB_TRY(norm_residual(enc, F2, &H3, ly.ln2_g, ly.ln2_b, Out, S, Di, D, stream));
        first_token = Out;
        break;
      }
    }
    const BoundSet X = slot[A], T3 = slot[Dd];
    BoundSet T1 = slot[B], T2 = slot[C];
    // Xin: the layer input as the products read it.  Before the first relaxation the two lines of the bound
    // coincide (lw == uw, VerifierForward.py:127-152 through an exact layer norm); handing the GEMM one
    // tensor as both lines selects its zero-radius instantiation.  (X itself keeps both buffers: they serve
    // as scratch later in the layer.)
    BoundSet Xin = X;
    if (li == 0) { Xin.uw = Xin.lw; Xin.ub = Xin.lb; }   // (the bias terms coincide as well: their rows then ride in the same launch)
    // The projections of such an input have coinciding lines as well: in the first layer Q, K and V are kept
    // once (both line pointers name the lw buffer; the zero-radius GEMM stores the same tile through both),
    // so the products that read them fetch every tile from HBM once.
    BoundSet Qh = T2, Kh = T3;
    if (li == 0) { Qh.uw = Qh.lw; Kh.uw = Kh.lw; }
    // The layer input of the first layer is zero in the weight rows of every position that is not perturbed (identity
    // rows at the perturbed positions only, and the exact layer norm keeps zero rows zero): the three projections of
    // this layer need not read or multiply those row blocks.
    LiveRows live_in = {L, Di, words, {0, 0, 0, 0}, inst_pos, rows * (int64_t)Di};
    for (int w = 0; positions != nullptr && w < words; ++w) live_in.pos[w] = positions[w];
    // (FB_ENCODER_NO_ZERO_SKIP in the environment switches this off: the tests compare both ways bit for bit)
    const LiveRowsScope live_scope(li == 0 && getenv("FB_ENCODER_NO_ZERO_SKIP") == nullptr ? &live_in : nullptr);
    // queries and keys, split into heads: [S*H, L, Di, d].  Where the shapes allow it the projection also
    // returns the concretised range of its result (column norms taken in the GEMM epilogue), which the
    // product below would otherwise compute in a pass of its own over the operand.
    int given = 0;
    int qrc = fb_matmul_heads_ranges_f32(Xin.lw, Xin.uw, Xin.lb, Xin.ub, ly.q_w, ly.q_b, Qh.lw, Qh.uw, T2.lb, T2.ub, range[0],
                                         range[1], norm_ws, rows, Di, D, D, L, H, words, p, eps, stream);
    if (qrc == FB_OK) {
      given |= 1;
    } else if (qrc == FB_ERR_SHAPE) {
      Qh = T2;
      FB_TRY(fb_matmul_heads_f32(Xin.lw, Xin.uw, Xin.lb, Xin.ub, ly.q_w, ly.q_b, T2.lw, T2.uw, T2.lb, T2.ub, rows, Di, D, D, L, H,
                                 stream));
    } else {
      return qrc;
    }
    qrc = fb_matmul_heads_ranges_f32(Xin.lw, Xin.uw, Xin.lb, Xin.ub, ly.k_w, ly.k_b, Kh.lw, Kh.uw, T3.lb, T3.ub, range[2], range[3],
                                     norm_ws, rows, Di, D, D, L, H, words, p, eps, stream);
    if (qrc == FB_OK) {
      given |= 2;
    } else if (qrc == FB_ERR_SHAPE) {
      Kh = T3;
      FB_TRY(fb_matmul_heads_f32(Xin.lw, Xin.uw, Xin.lb, Xin.ub, ly.k_w, ly.k_b, T3.lw, T3.uw, T3.lb, T3.ub, rows, Di, D, D, L, H,
                                 stream));
    } else {
      return qrc;
    }
    // scores [S*H, L, Di, L], scaled by 1/sqrt(d) -> T1
    FB_TRY(fb_dot_product_given_f32(Qh.lw, Qh.uw, T2.lb, T2.ub, Kh.lw, Kh.uw, T3.lb, T3.ub, T1.lw, T1.uw, T1.lb, T1.ub,
                                    range[0], range[1], range[2], range[3], S * H, L, L, Di, d, words, p, eps, inv_sqrt_d,
                                    FB_NATIVE, 1, given, stream));
    const int64_t hrows = (int64_t)S * H * L;
    // softmax: fused kernel when the score row fits one tile, else exp / row sum / reciprocal / product
    // (the fused kernel also returns the concretised range of the probabilities for the context product)
    int pgiven = 0;
    int src = fb_softmax_ranges_f32(T1.lw, T1.uw, T1.lb, T1.ub, T2.lw, T2.uw, T2.lb, T2.ub, range[0], range[1], hrows, Di,
                                    L, words, p, eps, violation, stream);
    if (src == FB_OK) {
      pgiven = 1;
      // probabilities are in T2; the stages below expect them in T1
      std::swap(T1, T2);
      std::swap(B, C);
    } else if (src == FB_ERR_SHAPE || src == FB_ERR_ALIGN) {
      FB_TRY(relax(FB_EXP, T1, T2, hrows, Di, L, words, p, eps, nullptr, stream));                     // E  -> T2
      FB_TRY(fb_rowsum_f32(T2.lw, T2.uw, T2.lb, T2.ub, T1.lw, T1.uw, T1.lb, T1.ub, hrows, Di, L, stream));  // sum -> T1
      FB_TRY(relax(FB_RECIPROCAL, T1, T3, hrows, Di, L, words, p, eps, violation, stream));             // 1/sum -> T3
      FB_TRY(fb_mul_bounds_f32(T2.lw, T2.uw, T2.lb, T2.ub, T3.lw, T3.uw, T3.lb, T3.ub, T1.lw, T1.uw, T1.lb, T1.ub,
                               hrows, Di, L, words, p, eps, stream));                                   // probs -> T1
    } else {
      return src;
    }
    // values, split into heads [S*H, L, Di, d]; the tensor-core context product reads them in this layout
    int crc = FB_ERR_SHAPE;
    if (L % 4 == 0) {
      int vgiven = pgiven;
      BoundSet Vh = T3;
      if (li == 0) Vh.uw = Vh.lw;
      const int vrc = fb_matmul_heads_ranges_f32(Xin.lw, Xin.uw, Xin.lb, Xin.ub, ly.v_w, ly.v_b, Vh.lw, Vh.uw, T3.lb, T3.ub, range[2],
                                                 range[3], norm_ws, rows, Di, D, D, L, H, words, p, eps, stream);
      if (vrc == FB_OK) {
        vgiven |= 2;
      } else if (vrc == FB_ERR_SHAPE) {
        Vh = T3;
        FB_TRY(fb_matmul_heads_f32(Xin.lw, Xin.uw, Xin.lb, Xin.ub, ly.v_w, ly.v_b, T3.lw, T3.uw, T3.lb, T3.ub, rows, Di, D, D, L, H,
                                   stream));
      } else {
        return vrc;
      }
      // context, written head-merged as [S, L, Di, D] -> T2
      crc = fb_context_given_f32(T1.lw, T1.uw, T1.lb, T1.ub, Vh.lw, Vh.uw, T3.lb, T3.ub, T2.lw, T2.uw, T2.lb, T2.ub,
                                 range[0], range[1], range[2], range[3], S * H, L, d, Di, L, words, p, eps, 1.0f, H, vgiven,
                                 stream);
      if (crc != FB_OK && crc != FB_ERR_SHAPE) return crc;
    }
    if (crc == FB_ERR_SHAPE) {
      // other shapes: values with position/feature swapped, [S*H, d, Di, L], and the general dot product
      FB_TRY(dense(Xin, ly.v_w, ly.v_b, T2, rows, Di, D, D, stream));
      FB_TRY(fb_split_heads_f32(T2.lw, T2.lb, T3.lw, T3.lb, S, L, Di, H, d, 1, stream));
      FB_TRY(fb_split_heads_f32(T2.uw, T2.ub, T3.uw, T3.ub, S, L, Di, H, d, 1, stream));
      FB_TRY(fb_dot_product_heads_f32(T1.lw, T1.uw, T1.lb, T1.ub, T3.lw, T3.uw, T3.lb, T3.ub, T2.lw, T2.uw, T2.lb, T2.ub,
                                      range[0], range[1], range[2], range[3], S * H, L, d, Di, L, words, p, eps, 1.0f,
                                      FB_NATIVE, (L % 4 == 0) ? H : 1, stream));
    }
    if (L % 4 != 0) {  // unvectorised path: merge with the permute kernel
      FB_TRY(fb_merge_heads_f32(T2.lw, T2.lb, T1.lw, T1.lb, S, L, Di, H, d, stream));
      FB_TRY(fb_merge_heads_f32(T2.uw, T2.ub, T1.uw, T1.ub, S, L, Di, H, d, stream));
      FB_CUDA_OK(cudaMemcpyAsync(T2.lw, T1.lw, (size_t)rows * Di * D * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
      FB_CUDA_OK(cudaMemcpyAsync(T2.uw, T1.uw, (size_t)rows * Di * D * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
      FB_CUDA_OK(cudaMemcpyAsync(T2.lb, T1.lb, (size_t)rows * D * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
      FB_CUDA_OK(cudaMemcpyAsync(T2.ub, T1.ub, (size_t)rows * D * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    }
    // attention output: dense, + residual, layer norm -> T3
    // (the residual is added by the GEMM epilogue where the shapes allow it: the layer norm then reads one bound)
    int arc = FB_ERR_SHAPE;
    bool ln1_done = false;
    if (fuse_ln) {
      arc = fb_matmul_residual_ln_f32(T2.lw, T2.uw, T2.lb, T2.ub, nullptr, nullptr, ly.ao_w, ly.ao_b, Xin.lw, Xin.uw, X.lb, X.ub,
                                      rs_in, ly.ln1_g, ly.ln1_b, T3.lw, T3.uw, T3.lb, T3.ub, nullptr, rows, Di, D, D, stream);
      if (arc == FB_OK) ln1_done = true;
      else if (arc == FB_ERR_SHAPE) fuse_ln = false;   // from here on the norms are launches of their own
      else return arc;
    }
    if (!ln1_done)
      arc = fb_matmul_residual_f32(T2.lw, T2.uw, T2.lb, T2.ub, nullptr, nullptr, ly.ao_w, ly.ao_b, Xin.lw, Xin.uw, X.lb, X.ub, T1.lw,
                                   T1.uw, T1.lb, T1.ub, rows, Di, D, D, stream);
    if (ln1_done) {
      // (T3 holds the normalised output of the attention block)
    } else if (arc == FB_OK) {
      FB_TRY(norm_residual(enc, T1, nullptr, ly.ln1_g, ly.ln1_b, T3, rows, Di, D, stream));
    } else if (arc == FB_ERR_SHAPE) {
      FB_TRY(dense(T2, ly.ao_w, ly.ao_b, T1, rows, Di, D, D, stream));
      FB_TRY(norm_residual(enc, T1, &Xin, ly.ln1_g, ly.ln1_b, T3, rows, Di, D, stream));
    } else {
      return arc;
    }
    // feed-forward: dense, relu, dense, + residual, layer norm
    // Where the shapes allow it the relu is not materialised: its column slopes go to the (now unused)
    // slot of the layer input and the second product applies them while it reads the hidden bounds.  The
    // first product hands over the concretised range of the hidden bounds (into the unused lb / ub of
    // that slot), so the slopes need no pass over the hidden weights either.
    int frc = fb_matmul_heads_ranges_f32(T3.lw, T3.uw, T3.lb, T3.ub, ly.f1_w, ly.f1_b, T1.lw, T1.uw, T1.lb, T1.ub, X.lb, X.ub,
                                         norm_ws, rows, Di, D, F, L, 1, words, p, eps, stream);
    if (frc == FB_OK) {
      frc = fb_relax_coef_given_f32(FB_RELU, T1.lb, T1.ub, X.lb, X.ub, X.lw, X.uw, T2.lb, T2.ub, rows, F, violation, stream);
    } else if (frc == FB_ERR_SHAPE) {
      FB_TRY(dense(T3, ly.f1_w, ly.f1_b, T1, rows, Di, D, F, stream));
      frc = fb_relax_coef_f32(FB_RELU, T1.lw, T1.uw, T1.lb, T1.ub, X.lw, X.uw, T2.lb, T2.ub, rows, Di, F, words, p, eps,
                              violation, stream);
    }
    bool residual_added = false;
    if (frc == FB_OK) {
      frc = fb_matmul_residual_f32(T1.lw, T1.uw, T2.lb, T2.ub, X.lw, X.uw, ly.f2_w, ly.f2_b, T3.lw, T3.uw, T3.lb, T3.ub, T2.lw,
                                   T2.uw, X.lb, X.ub, rows, Di, F, D, stream);
      if (frc == FB_OK)
        residual_added = true;
      else if (frc == FB_ERR_SHAPE)
        frc = fb_matmul_coef_f32(T1.lw, T1.uw, T2.lb, T2.ub, X.lw, X.uw, ly.f2_w, ly.f2_b, T2.lw, T2.uw, X.lb, X.ub, rows, Di,
                                 F, D, stream);
    }
    if (frc == FB_OK) {
      const BoundSet Y = {T2.lw, T2.uw, X.lb, X.ub};
      if (fuse_ln) {
        // (the norm also leaves the row sums of the layer output behind, for the next layer's attention output product)
        const BoundSet* r2 = residual_added ? nullptr : &T3;
        const int lrc = layernorm_novar_rowsum(Y.lw, Y.uw, Y.lb, Y.ub, r2 ? r2->lw : nullptr, r2 ? r2->uw : nullptr,
                                               r2 ? r2->lb : nullptr, r2 ? r2->ub : nullptr, ly.ln2_g, ly.ln2_b, T1.lw, T1.uw, T1.lb,
                                               T1.ub, rows, Di, D, rs_in, stream);
        if (lrc == FB_ERR_SHAPE) {
          fuse_ln = false;
          FB_TRY(norm_residual(enc, Y, r2, ly.ln2_g, ly.ln2_b, T1, rows, Di, D, stream));
        } else if (lrc != FB_OK) {
          return lrc;
        }
      } else {
        FB_TRY(norm_residual(enc, Y, residual_added ? nullptr : &T3, ly.ln2_g, ly.ln2_b, T1, rows, Di, D, stream));
      }
      // the layer output (slot B) becomes the next layer's input
      const int newA = B;
      B = A;
      A = newA;
      continue;
    }
    if (frc != FB_ERR_SHAPE) return frc;
    FB_TRY(relax(FB_RELU, T1, T2, rows, Di, F, words, p, eps, nullptr, stream));
    FB_TRY(dense(T2, ly.f2_w, ly.f2_b, T1, rows, Di, F, D, stream));
    FB_TRY(norm_residual(enc, T1, &T3, ly.ln2_g, ly.ln2_b, T2, rows, Di, D, stream));
    fuse_ln = false;
    // the layer output becomes the next layer's input
    const int newA = C;
    C = A;
    A = newA;
  }
  if (first_token.lw != nullptr) {
    // the last layer was run for the first token only: its output is the pooler's input (it lives in slot B; the two
    // scratch sets below are taken from slots C and D)
    const BoundSet &T1 = slot[C], &T2 = slot[Dd];
    FB_TRY(dense(first_token, enc->pool_w, enc->pool_b, T2, S, Di, D, D, stream));
    FB_TRY(relax(FB_TANH, T2, T1, S, Di, D, words, p, eps, nullptr, stream));
    fold_classifier_kernel<<<1, 128, 0, st>>>(enc->cls_w, enc->cls_b, fold_w, fold_b, D);
    FB_LAUNCH_OK();
    FB_TRY(dense(T1, fold_w, fold_b, T2, S, Di, D, 1, stream));
    FB_TRY(fb_concretize_f32(T2.lw, T2.uw, T2.lb, T2.ub, out_l, out_u, S, Di, 1, words, p, eps, FB_NATIVE, stream));
  } else {
    const BoundSet &X = slot[A], &T1 = slot[B], &T2 = slot[C];
    if (enc->pooling == 1) {
      // mean over the positions: [S, 1, Di, D]
      const int64_t nw = (int64_t)S * Di * D, nb = (int64_t)S * D, cap = (int64_t)device_info().sms * 32;
      mean_pool_kernel<<<(unsigned)std::min(ceil_div(nw, 256), cap), 256, 0, st>>>(X.lw, X.uw, T1.lw, T1.uw, nw, (int64_t)Di * D, L);
      FB_LAUNCH_OK();
      mean_pool_kernel<<<(unsigned)std::min(ceil_div(nb, 256), cap), 256, 0, st>>>(X.lb, X.ub, T1.lb, T1.ub, nb, (int64_t)D, L);
      FB_LAUNCH_OK();
    } else {
    // first token of every sentence: [S, 1, Di, D]
    FB_CUDA_OK(cudaMemcpy2DAsync(T1.lw, (size_t)Di * D * 4, X.lw, (size_t)L * Di * D * 4, (size_t)Di * D * 4, S,
                                 cudaMemcpyDeviceToDevice, st));
    FB_CUDA_OK(cudaMemcpy2DAsync(T1.uw, (size_t)Di * D * 4, X.uw, (size_t)L * Di * D * 4, (size_t)Di * D * 4, S,
                                 cudaMemcpyDeviceToDevice, st));
    FB_CUDA_OK(cudaMemcpy2DAsync(T1.lb, (size_t)D * 4, X.lb, (size_t)L * D * 4, (size_t)D * 4, S,
                                 cudaMemcpyDeviceToDevice, st));
    FB_CUDA_OK(cudaMemcpy2DAsync(T1.ub, (size_t)D * 4, X.ub, (size_t)L * D * 4, (size_t)D * 4, S,
                                 cudaMemcpyDeviceToDevice, st));
    }
    FB_TRY(dense(T1, enc->pool_w, enc->pool_b, T2, S, Di, D, D, stream));
    FB_TRY(relax(FB_TANH, T2, T1, S, Di, D, words, p, eps, nullptr, stream));
    fold_classifier_kernel<<<1, 128, 0, st>>>(enc->cls_w, enc->cls_b, fold_w, fold_b, D);
    FB_LAUNCH_OK();
    FB_TRY(dense(T1, fold_w, fold_b, T2, S, Di, D, 1, stream));
    FB_TRY(fb_concretize_f32(T2.lw, T2.uw, T2.lb, T2.ub, out_l, out_u, S, Di, 1, words, p, eps, FB_NATIVE, stream));
  }
  return FB_OK;
}

extern "C" int fb_encoder_forward_f32(const fb_encoder* enc, const float* emb, int S, int L, const int* positions,
                                      int words, int p, float eps, float* out_l, float* out_u, int* violation,
                                      void* workspace, int64_t workspace_bytes, void* stream) {
  if (!positions) return FB_ERR_ARG;
  return encoder_forward_impl(enc, emb, S, L, positions, nullptr, nullptr, words, p, eps, out_l, out_u, violation, workspace,
                              workspace_bytes, stream);
}

extern "C" int fb_encoder_forward_instances_f32(const fb_encoder* enc, const float* emb, int S, int L,
                                                const int* positions, const float* eps, int words, int p,
                                                float* out_l, float* out_u, int* violation, void* workspace,
                                                int64_t workspace_bytes, void* stream) {
  if (!positions || !eps) return FB_ERR_ARG;
  // the radius of every instance sits in its identity block: the pass itself runs with radius 1
  return encoder_forward_impl(enc, emb, S, L, nullptr, positions, eps, words, p, 1.0f, out_l, out_u, violation, workspace,
                              workspace_bytes, stream);
}
