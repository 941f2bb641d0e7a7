/*
 * faith_b200 -- forward linear-bound propagation operators for NVIDIA B200 (sm_100a).
 *
 * C ABI of the shared library libfaith_b200.so.  Every entry point
 *   - takes plain device pointers (fp32) and sizes, plus a CUDA stream passed as void*
 *     (a cudaStream_t; NULL = the legacy default stream),
 *   - enqueues its kernels on that stream and returns without synchronising,
 *   - never allocates or frees device memory: outputs and scratch belong to the caller,
 *   - returns an fb_status code instead of aborting.
 *
 * A bound object carries four tensors (reference: Transformer_Verification_Code/Verifiers/
 * Bounds.py:270-297):
 *     lw, uw : [rows, Di, Do]      rows = batch * length (row-major, Do contiguous)
 *     lb, ub : [rows, Do]
 * This is the reference's PyTorch layout ("native").  The reference's pybind entry points
 * (HandTunedKernels/kernel.cpp:69-241) pass lw/uw transposed, [rows, Do, Di] with Di
 * contiguous (Bounds.py:1203-1211); entry points that accept it take `layout`.
 *
 * The dual norm is selected by `p` (Bounds.py:277): FB_P1 -> max-abs, FB_P2 -> Euclidean,
 * FB_PINF -> sum-abs.  `words` is the number of perturbed words: the Di axis is split into
 * `words` equal blocks whose norms are added (Bounds.py:319-326).  `eps` is the perturbation
 * radius.
 */
#ifndef FAITH_B200_H
#define FAITH_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum fb_status {
  FB_OK = 0,
  FB_ERR_ARG = 1,     /* null pointer, negative size, unknown enum value */
  FB_ERR_SHAPE = 2,   /* sizes the kernels do not support (documented per function) */
  FB_ERR_ALIGN = 3,   /* pointer not aligned to 16 bytes where the vector path needs it */
  FB_ERR_CUDA = 4,    /* a CUDA runtime call or launch failed; see fb_last_cuda_error() */
  FB_ERR_WORKSPACE = 5, /* caller-provided scratch too small */
  FB_ERR_TIMEOUT = 6,   /* a bounded wait inside a kernel (or on a peer) expired; results are not valid */
  FB_ERR_NCCL = 7       /* a collective failed; see fb_comm_last_error() */
};

enum fb_norm { FB_P1 = 1, FB_P2 = 2, FB_PINF = 3 };
enum fb_layout { FB_NATIVE = 0 /* [rows, Di, Do] */, FB_TRANSPOSED = 1 /* [rows, Do, Di] */ };

/* Relaxation selector of fb_relax_f32.  FB_INTERVAL added to an operator selects its interval form (the
 * reference's `ibp` branches: constant bounds, zero weights). */
enum fb_relax_op { FB_RELU = 0, FB_TANH = 1, FB_EXP = 2, FB_RECIPROCAL = 3, FB_SQR = 4, FB_SQRT = 5, FB_INTERVAL = 8 };

const char* fb_status_string(int status);
/* cudaError_t (as int) of the most recent FB_ERR_CUDA on the calling thread. */
int fb_last_cuda_error(void);
int fb_version(void);

/* l = lb - eps * sum_w ||lw_w||_q,  u = ub + eps * sum_w ||uw_w||_q      (out: [rows, Do]).
 * Replaces Bounds.concretize (Bounds.py:311-326) and the reference kernel `concretize`
 * (HandTunedKernels/dot_product_verification.cu:47-105). */
int fb_concretize_f32(const float* lw, const float* uw, const float* lb, const float* ub,
                      float* l, float* u,
                      int64_t rows, int Di, int Do, int words, int p, float eps, int layout,
                      void* stream);

/* Fused concretise + per-column linear relaxation + column rescale of lw/uw.
 *   op = FB_RELU        Bounds.ori_relu  (Bounds.py:921-963); kernel.cpp:69-99 c_relu_verification
 *   op = FB_TANH        Bounds.ori_tanh  (Bounds.py:1027-1103); kernel.cpp:101-131 c_tanh_verification
 *   op = FB_EXP         Bounds.exp       (Bounds.py:970-1003)
 *   op = FB_RECIPROCAL  Bounds.reciprocal (Bounds.py:1136-1161)
 *   op = FB_SQR         Bounds.sqr        (Bounds.py:860-890)
 *   op = FB_SQRT        Bounds.sqrt       (Bounds.py:892-919)
 *   op + FB_INTERVAL    the `ibp` branch of the same operator (Bounds.py:863-866, 896-898, 924-926, 973-975,
 *                       1030-1032, 1139-1143): out_lb / out_ub are the images of the concretised range, out_lw and
 *                       out_uw are zero
 * Outputs have the shape and layout of the inputs and must not alias them.
 * `violation` (device int, may be NULL) is set to 1 by FB_RECIPROCAL when some concretised
 * lower bound is below 1e-12, the condition the reference asserts on (Bounds.py:1147), and by FB_SQRT
 * (both forms) when some lower bound is not positive (Bounds.py:894); the caller zeroes it beforehand. */
int fb_relax_f32(int op,
                 const float* lw, const float* uw, const float* lb, const float* ub,
                 float* out_lw, float* out_uw, float* out_lb, float* out_ub,
                 int64_t rows, int Di, int Do, int words, int p, float eps, int layout,
                 int* violation, void* stream);

/* The same relaxation when the dim_in axis is sharded over several GPUs (each device holds
 * Di_local rows of lw/uw of every column; lb/ub are replicated).  The reference is single-GPU;
 * the split follows from Bounds.concretize (Bounds.py:311-326): the dual norm of a column is a
 * sum (p = inf: sum |w|, p = 2: sum w^2 before the root) or a maximum (p = 1) over dim_in.
 *   1. fb_norm_partials_f32 writes the unfinished accumulation of the local rows, [rows, Do] each;
 *   2. the caller reduces part_l / part_u over the devices (all-reduce SUM, or MAX for FB_P1);
 *   3. fb_relax_with_norms_f32 finishes the norm, concretises, relaxes and rescales the local rows.
 * One perturbed word (words = 1).  Native layout. */
int fb_norm_partials_f32(const float* lw, const float* uw, float* part_l, float* part_u,
                         int64_t rows, int Di_local, int Do, int p, void* stream);
int fb_relax_with_norms_f32(int op, const float* lw, const float* uw, const float* lb, const float* ub,
                            const float* norm_l, const float* norm_u,
                            float* out_lw, float* out_uw, float* out_lb, float* out_ub,
                            int64_t rows, int Di_local, int Do, int p, float eps,
                            int* violation, void* stream);

/* Product with a constant weight W [Dy, Do] (nn.Linear layout) and optional bias [Dy]
 * (NULL = none): y_lw = x_lw W+ + x_uw W-, y_uw = x_lw W- + x_uw W+, same for lb/ub, then
 * + bias.  Replaces Bounds.ori_matmul / dense (Bounds.py:397-413, 1016-1025) and the
 * commented-out c_matmul_verification (kernel.cpp:243-266).  Native layout only.
 * x_lw, x_uw: [rows, Di, Do]; y_lw, y_uw: [rows, Di, Dy]. */
int fb_matmul_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                  const float* W, const float* bias,
                  float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                  int64_t rows, int Di, int Do, int Dy, void* stream);

/* fb_matmul_f32 with the head split of the attention projections folded into the store
 * (VerifierForward.py:208-229): rows = S * L; with heads = H > 1 and d = Dy / H the outputs are written as
 * y_lw, y_uw [S * H, L, Di, d] and y_lb, y_ub [S * H, L, d]. */
int fb_matmul_heads_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                        const float* W, const float* bias,
                        float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                        int64_t rows, int Di, int Do, int Dy, int L, int heads, void* stream);

/* fb_matmul_heads_f32 that also returns the concretised range of its result (Bounds.py:311-326 on the
 * output of :397-413): y_l, y_u in the layout of y_lb, y_ub.  The dual norms over dim_in are taken by the
 * GEMM epilogue from the tile it is about to store, so the dot product that consumes y
 * (fb_dot_product_given_f32, fb_context_given_f32) needs no pass of its own over y_lw / y_uw.
 * x_uw may be the same pointer as x_lw (a bound whose two lines coincide, as everywhere before the first
 * relaxation): the kernel then skips the radius half of the work, and y_uw may be the same pointer as y_lw
 * (both lines of the result are equal; the tile is stored through both).
 * norm_ws: 2 * rows * (words + 1) * Dy floats of scratch.  Tensor-core shapes with Di == 128 * words only,
 * otherwise FB_ERR_SHAPE and nothing is launched.  No counterpart in the reference's extension module. */
int fb_matmul_heads_ranges_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                               const float* W, const float* bias,
                               float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                               float* y_l, float* y_u, float* norm_ws,
                               int64_t rows, int Di, int Do, int Dy, int L, int heads,
                               int words, int p, float eps, void* stream);

/* A relaxation without its rescale pass, and the product that applies it while reading (dense after relu
 * of the feed-forward block, Bounds.py:921-963 + :397-413; also tanh and exp, whose slopes are positive).
 * fb_relax_coef_f32 writes, instead of rescaled weights, the own-side slopes c_l, c_u [rows, Do]
 * (out_lw = c_l * lw, out_uw = c_u * uw) and the relaxed bias terms out_lb, out_ub; a column that would
 * need a cross term (inverted range l > u) sets bit 1 of *violation, FB_RECIPROCAL is not accepted.
 * fb_matmul_coef_f32 computes matmul((c_l * x_lw, c_u * x_uw, x_lb, x_ub), W) + bias with x_lb, x_ub the
 * relaxed bias terms; results equal fb_relax_f32 followed by fb_matmul_f32 bit for bit.  Tensor-core
 * shapes with Di a multiple of 128 and Do a multiple of 32 only, otherwise FB_ERR_SHAPE and nothing is
 * launched.  No counterpart in the reference's extension module. */
int fb_relax_coef_f32(int op, const float* lw, const float* uw, const float* lb, const float* ub,
                      float* c_l, float* c_u, float* out_lb, float* out_ub,
                      int64_t rows, int Di, int Do, int words, int p, float eps,
                      int* violation, void* stream);
/* fb_relax_coef_f32 for a bound whose concretised range l, u [rows, Do] the caller already holds (e.g. from
 * fb_matmul_heads_ranges_f32 with heads = 1): no pass over lw / uw. */
int fb_relax_coef_given_f32(int op, const float* lb, const float* ub, const float* l, const float* u,
                            float* c_l, float* c_u, float* out_lb, float* out_ub,
                            int64_t rows, int Do, int* violation, void* stream);
int fb_matmul_coef_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                       const float* c_l, const float* c_u, const float* W, const float* bias,
                       float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                       int64_t rows, int Di, int Do, int Dy, void* stream);

/* dense followed by the residual add of the encoder blocks: y = matmul(x, W) + bias + r (Bounds.py:397-413 and
 * :383-395), optionally of a relaxed bound given by its slopes c_l, c_u as in fb_matmul_coef_f32 (both NULL:
 * plain dense).  The GEMM epilogue fetches the residual tile while the tile is computed and adds it before the
 * store; bit-identical to fb_matmul_f32 (fb_matmul_coef_f32) followed by fb_add_f32.  Tensor-core shapes for
 * the weight rows and the bias rows (rows >= 256) only, otherwise FB_ERR_SHAPE and nothing is launched.  No
 * counterpart in the reference's extension module. */
int fb_matmul_residual_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                           const float* c_l, const float* c_u, const float* W, const float* bias,
                           const float* r_lw, const float* r_uw, const float* r_lb, const float* r_ub,
                           float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                           int64_t rows, int Di, int Do, int Dy, void* stream);

/* fb_matmul_residual_f32 followed by the layer norm of the encoder blocks (mode no_var, Bounds.py:1111-1131), applied
 * by the GEMM epilogue: z = layer_norm(matmul(x, W) + bias + r).  r_rowsum: row sums of the residual as its producer
 * left them, z_rowsum (may be NULL): those of z for the next consumer; each [2 lines][4 partial sums][rows * (Di + 1)] floats (weight
 * rows first, then the bias rows; a reader adds the four partial sums in order).  Equals the separate operators to
 * rounding (the row means are rounded in another order).  Dy == 128, Do % 64 == 0, Do <= 512, rows * Di % 128 == 0,
 * rows >= 256; otherwise FB_ERR_SHAPE and nothing is launched.  Replaces Bounds.matmul + Bounds.add +
 * Bounds.layer_norm (Bounds.py:397-413, :383-395, :1111-1131). */
int fb_matmul_residual_ln_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                              const float* c_l, const float* c_u, const float* W, const float* bias,
                              const float* r_lw, const float* r_uw, const float* r_lb, const float* r_ub,
                              const float* r_rowsum, const float* gamma, const float* beta,
                              float* z_lw, float* z_uw, float* z_lb, float* z_ub, float* z_rowsum,
                              int64_t rows, int Di, int Do, int Dy, void* stream);

/* The tensor-core kernels behind fb_matmul_f32 and fb_dot_product_f32 bound every wait inside the kernel; if a
 * wait ever expires, the kernel raises a device-side flag, frees its tensor memory and returns, leaving its
 * outputs partly written.  fb_tc_error_flag synchronises the device, returns the flag in *flag (0 = never
 * raised) and clears it; fb_tc_check does the same and returns FB_ERR_TIMEOUT when the flag was raised.
 * fb_encoder_forward_f32 reports the same condition without a synchronisation of its own: bit 2 of its
 * `violation` word.  No counterpart in the reference (its kernels have no waits). */
int fb_tc_error_flag(int* flag);
int fb_tc_check(void);

/* Self-test of that give-up path (the reference has nothing comparable): the product of x [M, K] with W [N, K]
 * is launched once with the operand loads of k-block `skip_kblock` of the first thread block left out and every
 * wait limited to `tries` tries of about 20 microseconds.  The block runs out of patience, drains, frees its
 * tensor memory and returns; the expected return value is FB_ERR_TIMEOUT, and the device stays usable.  y is
 * scratch (garbage afterwards).  `status` (device int, may be NULL) receives bit 2 the way the `violation` word of
 * fb_encoder_forward_f32 does.  Not to be run concurrently with other products of the same process. */
int fb_tc_selftest_timeout(const float* x_lw, const float* x_uw, const float* W, float* y_lw, float* y_uw,
                           int64_t M, int N, int K, int skip_kblock, int tries, int* status, void* stream);

/* Bound x bound dot product  z[b,i,j] = sum_k x[b,i,k] * y[b,j,k]  (attention scores and,
 * with y = transposed values, the attention context).  Replaces Bounds.ori_dot_product
 * (Bounds.py:710-823) and c_dot_product_verification_QK / _V (kernel.cpp:133-241).
 *   native:      x_lw,x_uw [B,Lx,Di,K]  y_lw,y_uw [B,Ly,Di,K]  z_lw,z_uw [B,Lx,Di,Ly]
 *   transposed:  x_lw,x_uw [B,Lx,K,Di]  y_lw,y_uw [B,Ly,K,Di]  z_lw,z_uw [B,Lx,Ly,Di]
 *   x_lb,x_ub [B,Lx,K]   y_lb,y_ub [B,Ly,K]   z_lb,z_ub [B,Lx,Ly]
 * x_l,x_u [B,Lx,K] and y_l,y_u [B,Ly,K] are caller-provided scratch that receives the
 * concretised ranges of the operands (as in the reference, Bounds.py:1274-1277).
 * Every output is multiplied by `out_scale` (1/sqrt(d) of the attention scores,
 * VerifierForward.py:232-233; must be > 0; pass 1.0f for the plain operator). */
int fb_dot_product_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                       const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                       float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                       float* x_l, float* x_u, float* y_l, float* y_u,
                       int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                       float out_scale, int layout, void* stream);

/* fb_dot_product_f32 with the head merge of the attention context folded into the store
 * (VerifierForward.py:253-265): with merge_heads = H > 1 (native layout, B = S * H), z is written as
 * [S, Lx, Di, H * Ly] / [S, Lx, H * Ly] instead of [B, Lx, Di, Ly] / [B, Lx, Ly]. */
int fb_dot_product_heads_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                             const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                             float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                             float* x_l, float* x_u, float* y_l, float* y_u,
                             int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                             float out_scale, int layout, int merge_heads, void* stream);

/* fb_dot_product_heads_f32 for operands whose concretised ranges the caller already holds (written by
 * the kernel that produced the operand, e.g. fb_matmul_heads_ranges_f32): bit 0 of `given` makes
 * x_l / x_u inputs, bit 1 y_l / y_u; the corresponding concretisation pass is skipped. */
int fb_dot_product_given_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                             const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                             float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                             float* x_l, float* x_u, float* y_l, float* y_u,
                             int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                             float out_scale, int layout, int merge_heads, int given, void* stream);

/* Context product of the attention block, Bounds.context (Bounds.py:843-850: dot_product with V.t()),
 * taking the values in the layout the projection writes, v_lw / v_uw [B, K, Di, Ly] and v_lb / v_ub
 * [B, K, Ly] (K = key positions, Ly = head features), so that no transposed copy of V is needed
 * (the reference's transpose_for_scores + .t() are permute copies, VerifierForward.py:208-229).
 * x = attention probabilities [B, Lx, Di, K]; z, merge_heads and the scratch tensors as in
 * fb_dot_product_heads_f32 (y_l, y_u receive the value ranges as [B, Ly, K]).
 * Tensor-core shapes only: K = Ly = 32, Lx a multiple of 32, Di a multiple of 4, 16-byte aligned
 * pointers; otherwise FB_ERR_SHAPE and nothing is launched (transpose V and call
 * fb_dot_product_heads_f32). */
int fb_context_heads_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                         const float* v_lw, const float* v_uw, const float* v_lb, const float* v_ub,
                         float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                         float* x_l, float* x_u, float* y_l, float* y_u,
                         int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                         float out_scale, int merge_heads, void* stream);

/* fb_context_heads_f32 with `given` as in fb_dot_product_given_f32; given value ranges are expected as
 * [B, K, Ly] (the layout of v_lb / v_ub) and are transposed in place to [B, Ly, K] like computed ones. */
int fb_context_given_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                         const float* v_lw, const float* v_uw, const float* v_lb, const float* v_ub,
                         float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                         float* x_l, float* x_u, float* y_l, float* y_u,
                         int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                         float out_scale, int merge_heads, int given, void* stream);

/* The same operator for callers that cannot allocate device memory.  (No counterpart in the
 * reference, whose callers always allocate the scratch tensors themselves.)
 *
 * Some hosts of this library are not in a position to call cudaMalloc or to hand over scratch
 * buffers: code that runs inside someone else's memory plan (a serving process with a fixed
 * arena, a plugin that only receives its input and output pointers), or a region where an
 * allocation would synchronise the device.  For them the four operand-range tensors
 * (x_l, x_u, y_l, y_u) live in a 16 MiB array that is part of the library image on every GPU
 * that loads it, from load until process exit.  The caller passes inputs and outputs only.
 *
 *  - Limit: 2*B*Lx*K + 2*B*Ly*K floats (each operand's share rounded up to 64 floats) must fit
 *    in fb_dot_product_noalloc_max_floats() = 4 Mi floats; larger problems return
 *    FB_ERR_WORKSPACE and launch nothing.  256 sentences x 4 heads at L = K = 32 fit exactly.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *    with that device current); make that first call outside any stream capture.
 *  - The call itself performs no cudaMalloc / cudaFree and calls no allocating library routine.
 *  - Every call on a device shares the one array.  The ranges are fully rewritten by each call
 *    before they are read, so nothing needs clearing and stale contents are harmless, but two
 *    calls that overlap on the GPU (different streams, or different host threads) race on it:
 *    serialise them.
 *  - The concretised ranges are not returned; use fb_dot_product_f32 when they are needed.
 * All other arguments, results and error codes are those of fb_dot_product_f32. */
int fb_dot_product_noalloc_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                               const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                               float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                               int B, int Lx, int Ly, int Di, int K, int words, int p, float eps,
                               float out_scale, int layout, void* stream);
int64_t fb_dot_product_noalloc_max_floats(void);

/* Elementwise product of two bounded quantities (McCormick planes), fused with the
 * concretisation of both operands.  Replaces Bounds.multiply(Bounds) (Bounds.py:608-651). */
int fb_mul_bounds_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                      const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                      float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                      int64_t rows, int Di, int Do, int words, int p, float eps, void* stream);

/* z = x + y on all four tensors (Bounds.add with a Bounds argument, Bounds.py:383-389).
 * In-place (z == x) is allowed. */
int fb_add_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
               const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
               float* z_lw, float* z_uw, float* z_lb, float* z_ub,
               int64_t rows, int Di, int Do, void* stream);

/* Multiplication by a scalar; a non-positive scalar swaps the two sides
 * (Bounds.multiply(float), Bounds.py:594-607).  In-place is NOT allowed. */
int fb_scale_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                 float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                 int64_t rows, int Di, int Do, float c, void* stream);

/* Multiplication by a constant vector over the feature axis, split by sign (Bounds.multiply with a tensor,
 * Bounds.py:653-664; the gain of a layer norm): z_l = x_l w+ + x_u w-, z_u = x_l w- + x_u w+ on the weights and on
 * the bias terms.  w [Do].  z may alias x. */
int fb_mul_features_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                        const float* w, float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                        int64_t rows, int Di, int Do, void* stream);

/* Interval arithmetic of the reference's `ibp` mode, where a bound is a box [lb, ub] with zero weights:
 * elementwise product of two boxes (Bounds.get_bounds_xy, Bounds.py:667-678, inside Bounds.multiply) over n
 * elements, and the dot product z[b,i,j] = sum_k [x[b,i,k]] * [y[b,j,k]] of two boxes (the dim_in == 1 branch of
 * Bounds.dot_product, Bounds.py:711-721): x [B, Lx, K], y [B, Ly, K], z [B, Lx, Ly]. */
int fb_interval_mul_f32(const float* x_l, const float* x_u, const float* y_l, const float* y_u,
                        float* z_l, float* z_u, int64_t n, void* stream);
int fb_interval_dot_f32(const float* x_l, const float* x_u, const float* y_l, const float* y_u,
                        float* z_l, float* z_u, int B, int Lx, int Ly, int K, void* stream);

/* Sum over the feature axis, broadcast back to every feature: the denominator of the softmax
 * (Bounds.softmax, Bounds.py:1007-1013).  Shapes as the input. */
int fb_rowsum_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                  float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                  int64_t rows, int Di, int Do, void* stream);

/* Fused softmax bound: exp, feature-axis sum, reciprocal and McCormick product in one kernel
 * (Bounds.softmax, Bounds.py:1005-1014).  Needs the feature axis in one tile: Do <= 32, Do % 4 == 0
 * and the two [Di, 32] tiles in shared memory; other shapes return FB_ERR_SHAPE (callers then run the
 * chain fb_relax_f32(FB_EXP) / fb_rowsum_f32 / fb_relax_f32(FB_RECIPROCAL) / fb_mul_bounds_f32).
 * `violation` as in fb_relax_f32(FB_RECIPROCAL). */
int fb_softmax_f32(const float* lw, const float* uw, const float* lb, const float* ub,
                   float* out_lw, float* out_uw, float* out_lb, float* out_ub,
                   int64_t rows, int Di, int Do, int words, int p, float eps, int* violation, void* stream);

/* fb_softmax_f32 that also returns the concretised range of its result, out_l / out_u [rows, Do] (what
 * fb_concretize_f32 returns for the written bounds): the dual norms are accumulated while the result is
 * written, so the context product that consumes the probabilities (fb_context_given_f32) needs no pass
 * of its own over them.  out_l and out_u may both be NULL (= fb_softmax_f32). */
int fb_softmax_ranges_f32(const float* lw, const float* uw, const float* lb, const float* ub,
                          float* out_lw, float* out_uw, float* out_lb, float* out_ub, float* out_l, float* out_u,
                          int64_t rows, int Di, int Do, int words, int p, float eps, int* violation, void* stream);

/* Layer normalisation without the variance ("no_var", Bounds.py:1111-1131), optionally fused
 * with a preceding residual add: t = x (+ r); t -= mean over features of the opposite side;
 * out = t * gamma (split by sign of gamma) + beta on lb/ub.  r_* may all be NULL. */
int fb_layernorm_novar_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                           const float* r_lw, const float* r_uw, const float* r_lb, const float* r_ub,
                           const float* gamma, const float* beta,
                           float* z_lw, float* z_uw, float* z_lb, float* z_ub,
                           int64_t rows, int Di, int Do, void* stream);

/* Head split [B, L, Di, H*d] -> [B*H, L, Di, d] (VerifierForward.py:208-229) and its inverse
 * (VerifierForward.py:253-265).  With transpose_ld != 0 the split additionally swaps the
 * position and feature axes, giving [B*H, d, Di, L]: the operand `value.t()` of the attention
 * context (Bounds.py:843-850) in contiguous form. */
int fb_split_heads_f32(const float* x_w, const float* x_b, float* z_w, float* z_b,
                       int B, int L, int Di, int H, int d, int transpose_ld, void* stream);
int fb_merge_heads_f32(const float* x_w, const float* x_b, float* z_w, float* z_b,
                       int B, int L, int Di, int H, int d, void* stream);

/* Bound of a 2-D convolution with constant weights (split by sign like fb_matmul_f32); dim_in
 * is the batch axis of the convolution.  Replaces the commented-out
 * c_convolution_verification (kernel.cpp:268-295).
 * x_lw,x_uw [B, Di, Cin, H, W]; x_lb,x_ub [B, Cin, H, W]; Wt [Cout, Cin, Kh, Kw]; bias [Cout] or
 * NULL; y_lw,y_uw [B, Di, Cout, Ho, Wo]; y_lb,y_ub [B, Cout, Ho, Wo].  Di may be 0 (bias part alone; so may it
 * in fb_matmul_f32). */
int fb_conv2d_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                  const float* Wt, const float* bias,
                  float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                  int B, int Di, int Cin, int H, int W, int Cout, int Kh, int Kw,
                  int stride, int pad, void* stream);

/* Convolutions behind an identity input: every pixel of a [Cin, H, W] image perturbed, dim_in = Cin * H * W, input
 * bound lw = uw = scale * I, lb / ub = the image (the convention of fb_conv2d_f32 with dim_in as batch axis; the
 * reference's stub, HandTunedKernels/convolution_verification.cu:228-238, has no such shortcut).
 *
 * fb_conv2d_identity_relax_f32: first convolution and the relaxation `op` that follows it (op < 0: convolution
 * only) for the rows [row_start, row_start + rows) of dim_in (a shard; all of them: 0, Cin*H*W).  Nothing is read
 * but the filter: row r of the result is scale * W at the taps that fall on pixel r and zero elsewhere, and the
 * dual norm of every output column over ALL of dim_in is the norm of the filter taps inside the image, so the
 * concretisation needs no reduction over rows (or ranks).  y_lw, y_uw [rows, Cout, Ho, Wo]; y_lb, y_ub
 * [Cout, Ho, Wo]; col_ws: 2 * Cout * Ho * Wo floats of scratch.  Equals fb_conv2d_f32 on the materialised identity
 * followed by fb_relax_f32 up to the summation order of the column norms.
 *
 * fb_conv2d_windowed_f32: a later convolution of such rows (weight part only).  Row r stands for pixel
 * (yi, xi) = ((r / W0) % H0, r % W0) of the original H0 x W0 image and is zero outside the window that pixel reaches
 * through the convolutions before this one: `chain` is a HOST array of n_chain x 4 ints (kernel height, kernel width,
 * stride, padding), first convolution first (n_chain <= 8; it must lead from H0 x W0 to this layer's H x W, else
 * FB_ERR_SHAPE).  Outputs whose taps miss the window are stored as zero, the others equal fb_conv2d_f32's bit for
 * bit.  FB_ERR_SHAPE when the largest window does not fit in shared memory (use fb_conv2d_f32 then). */
int fb_conv2d_identity_relax_f32(int op, const float* x_lb, const float* x_ub, const float* Wt, const float* bias,
                                 float scale, float* y_lw, float* y_uw, float* y_lb, float* y_ub, float* col_ws,
                                 int64_t rows, int64_t row_start, int Cin, int H, int W, int Cout, int Kh, int Kw,
                                 int stride, int pad, int p, float eps, int* violation, void* stream);
int fb_conv2d_windowed_f32(const float* x_lw, const float* x_uw, const float* Wt, float* y_lw, float* y_uw,
                           int64_t rows, int64_t row_start, int H0, int W0, const int* chain, int n_chain,
                           int Cin, int H, int W, int Cout, int Kh, int Kw, int stride, int pad, void* stream);

/* ---- whole-model driver: forward bound pass of a BERT-style encoder ---------------------
 * Follows VerifierForward.verify_safety (VerifierForward.py:93-119) for a batch of S
 * sentences with one set of perturbed positions; no epsilon search.  Weights are device
 * pointers in nn.Linear layout. */
typedef struct fb_encoder_layer {
  const float *q_w, *q_b, *k_w, *k_b, *v_w, *v_b, *ao_w, *ao_b, *ln1_g, *ln1_b;
  const float *f1_w, *f1_b, *f2_w, *f2_b, *ln2_g, *ln2_b;
} fb_encoder_layer;

typedef struct fb_encoder {
  int layers, d_model, heads, ffn;
  int layer_norm;                 /* 0 = "no", 1 = "no_var" */
  const float *emb_ln_g, *emb_ln_b;
  const fb_encoder_layer* layer;  /* host array of `layers` entries */
  const float *pool_w, *pool_b;   /* [d_model, d_model], [d_model] */
  const float *cls_w, *cls_b;     /* [2, d_model], [2] */
  int first_token_only;           /* 0: every layer is propagated at every position, as the reference does
                                     (VerifierForward.py:93-119); != 0: the last layer is propagated for the first token
                                     only.  The pooler reads nothing else of it (VerifierForward.py:269-287), so keys
                                     and values are still formed at every position but the query, the attention row,
                                     the attention output and the feed-forward block only at position 0.  Same bounds
                                     up to the rounding of other kernel shapes; about a quarter less work for three
                                     layers. */
  int pooling;                    /* 0: the reference's pooler, first token -> dense -> tanh (VerifierForward.py:269-287);
                                     1: mean over the positions -> dense -> tanh (the pooling the benchmark description
                                     names; no reference implementation, exact for linear bounds: every line is
                                     averaged with the positive weight 1/L).  With 1, first_token_only is ignored. */
} fb_encoder;

/* Bytes of scratch fb_encoder_forward_f32 needs for S sentences of length L. */
int64_t fb_encoder_workspace_bytes(const fb_encoder* enc, int S, int L, int words);

/* emb [S, L, d_model] (device); positions[words] (host) = perturbed token indices;
 * out_l, out_u [S] (device) = concretised bounds of logit0 - logit1;
 * violation [1] (device int, zeroed by the call), a bit set the caller must read together with out_l / out_u:
 *   bit 0  a softmax denominator was not provably positive (the reference's assertion, Bounds.py:1147);
 *   bit 1  a hidden unit had an inverted range (l > u) where the feed-forward relu is applied through its slopes:
 *          the result then differs from the reference's add_linear (Bounds.py:362-381) for that unit;
 *   bit 2  a bounded wait inside a tensor-core kernel of this pass expired: out_l / out_u are NOT valid.
 * Any non-zero value means the bounds must not be used as a proof. */
int fb_encoder_forward_f32(const fb_encoder* enc, const float* emb, int S, int L,
                           const int* positions, int words, int p, float eps,
                           float* out_l, float* out_u, int* violation,
                           void* workspace, int64_t workspace_bytes, void* stream);

/* The same pass for S independent verification instances: instance s has its own perturbed positions
 * positions[s * words + w] and its own radius eps[s] (both DEVICE arrays; positions must lie in [0, L), which
 * the caller guarantees).  This is how the reference's search over the radius (Verifier.py:106-147: per word a
 * probe at max_eps and num_verify_iters bisection steps, each a call of verify_safety) is batched: the probes of
 * all words and sentences of a round are instances of one call.  The radius is folded into the identity block of the
 * input bound (the dual norm is homogeneous), so results agree with fb_encoder_forward_f32 up to rounding, not bit for
 * bit.  emb [S, L, d_model]: the embeddings of instance s (instances of one sentence repeat its rows). */
int fb_encoder_forward_instances_f32(const fb_encoder* enc, const float* emb, int S, int L,
                                     const int* positions, const float* eps, int words, int p,
                                     float* out_l, float* out_u, int* violation,
                                     void* workspace, int64_t workspace_bytes, void* stream);

/* ---- dim_in sharded over several GPUs: communicator and fused steps (no counterpart in the reference, which is
 * single-GPU; the split follows from Bounds.concretize, Bounds.py:311-326, see fb_norm_partials_f32) -------------
 *
 * fb_comm wraps an NCCL communicator (one process per GPU; NCCL is bound at run time by dlopen, the environment
 * variable FB_NCCL_LIB overrides the library name).  Rank 0 obtains a 128-byte id with fb_comm_unique_id and
 * hands it to the other ranks by any means; every rank then calls fb_comm_create with its device current.
 * oneshot_floats > 0 additionally sets up the one-shot all-reduce over NVLink for vectors of up to that many
 * floats: this is the one place where the library allocates device memory (2 * world * oneshot_floats floats plus
 * flags per rank, freed by fb_comm_destroy) and maps it into the peers through CUDA IPC.  world <= 8.
 *
 * Errors: FB_ERR_NCCL when a NCCL call fails or ncclCommGetAsyncError reports an asynchronous error (polled
 * after every collective and by fb_comm_check); fb_comm_last_error() gives the text.  The one-shot path never
 * blocks for ever: a wait for a peer is bounded (2 s, fb_comm_set_wait_ns), on expiry the kernel sets a status
 * word and returns, and fb_comm_check(c, 1) -- which synchronises the device -- reports FB_ERR_TIMEOUT. */
typedef struct fb_comm fb_comm;
int fb_comm_unique_id(void* id128);
int fb_comm_create(fb_comm** out, const void* id128, int rank, int world, int64_t oneshot_floats);
int fb_comm_destroy(fb_comm* c);
int fb_comm_abort(fb_comm* c);
int fb_comm_info(const fb_comm* c, int* rank, int* world, int64_t* oneshot_floats);
int fb_comm_set_wait_ns(fb_comm* c, uint64_t ns);
int fb_comm_check(fb_comm* c, int sync);
const char* fb_comm_last_error(void);

enum fb_reduce_op { FB_SUM = 0, FB_MAX = 1 };
enum fb_allreduce_algo { FB_ALGO_NCCL = 0, FB_ALGO_ONESHOT = 1 };
/* In-place all-reduce of n floats on `stream`.  FB_ALGO_ONESHOT: every rank stores its vector into all peers'
 * receive slots with ordinary stores over NVLink, publishes a flag, waits (bounded) for the others and sums the
 * slots in rank order (bit-identical on all ranks); n must not exceed oneshot_floats, else FB_ERR_WORKSPACE.
 * Calls on one communicator must not overlap on the GPU. */
int fb_allreduce_f32(fb_comm* c, float* buf, int64_t n, int op, int algo, void* stream);

/* fb_relax_f32 and fb_concretize_f32 for a dim_in shard: partial norms of the local rows, all-reduce over the
 * ranks (SUM, or MAX for FB_P1), relaxation of the local rows / concretisation, all enqueued on `stream` with no
 * host round trip.  lb, ub are replicated; part_ws: 2 * rows * Do floats of scratch.  c may be NULL (single
 * rank).  One perturbed word only: words != 1 returns FB_ERR_SHAPE (several word blocks would need one partial
 * per block and shards aligned to the blocks). */
int fb_relax_sharded_f32(fb_comm* c, int algo, int op,
                         const float* lw, const float* uw, const float* lb, const float* ub,
                         float* out_lw, float* out_uw, float* out_lb, float* out_ub, float* part_ws,
                         int64_t rows, int Di_local, int Do, int words, int p, float eps,
                         int* violation, void* stream);
int fb_concretize_sharded_f32(fb_comm* c, int algo,
                              const float* lw, const float* uw, const float* lb, const float* ub,
                              float* l, float* u, float* part_ws,
                              int64_t rows, int Di_local, int Do, int words, int p, float eps, void* stream);

/* ---- compact rows for the convolutions behind an identity input ---------------------------
 * Row r of such a CNN is zero outside the window its pixel reaches (fb_conv2d_windowed_f32 above); here a row is stored
 * as that window only, z [rows, C, wh, ww] with z[r, c, dy, dx] = row r at (c, y_lo(r) + dy, x_lo(r) + dx) and zeros
 * where the pixel's own window is smaller than (wh, ww), the largest window over all pixels (fb_cw_extent).  `chain`
 * (host, n_chain x 4 ints: kernel height, kernel width, stride, padding) always lists the convolutions that lead from
 * the H0 x W0 image to the tensor in question, whose dense shape is [C, H, W].  For the benchmark CNN a row shrinks
 * from 16 384 resp. 8 192 values to 144 resp. 288.  No counterpart in the reference.
 *
 * fb_cw_identity_relax_f32  first convolution + relaxation (op < 0: none), the compact form of
 *                           fb_conv2d_identity_relax_f32 (same arguments; z instead of y_lw / y_uw).
 * fb_cw_conv2d_f32          a later convolution, compact -> compact (weight part; the bias part is fb_conv2d_f32 with
 *                           Di = 0).  `chain` leads to the input [Cin, H, W]; the output's chain is that plus this layer.
 *                           Expands to fb_conv2d_f32's values bit for bit.
 * fb_cw_norm_partials_f32   unfinished dual-norm accumulation of every dense column over the rows of the shard
 *                           (the counterpart of fb_norm_partials_f32): part_l, part_u [C*H*W]; Cin0 = channels of the
 *                           original image (dim_in = Cin0 * H0 * W0).  Gathered in row order: deterministic.
 * fb_cw_relax_apply_f32     relaxation from (all-reduced) norms, the counterpart of fb_relax_with_norms_f32: rescaled
 *                           compact rows, relaxed bias terms out_lb / out_ub [C*H*W]; coef_ws: 4*C*H*W floats of scratch.
 * fb_cw_linear_f32          the linear layer that ends the spatial part, weight rows only: Wl [N, C*H*W] (nn.Linear
 *                           layout) -> y_lw, y_uw [rows, N] dense (bias rows: fb_matmul_f32 with Di = 0); wt_ws: N*C*H*W
 *                           floats of scratch (the call transposes the weight once so that its reads coalesce).
 * fb_cw_expand_f32          dense rows [rows, C, H, W] from compact ones. */
int fb_cw_extent(int H0, int W0, const int* chain, int n_chain, int* wh, int* ww);
int fb_cw_identity_relax_f32(int op, const float* x_lb, const float* x_ub, const float* Wt, const float* bias,
                             float scale, float* z_lw, float* z_uw, float* y_lb, float* y_ub, float* col_ws,
                             int64_t rows, int64_t row_start, int Cin, int H, int W, int Cout, int Kh, int Kw,
                             int stride, int pad, int p, float eps, int* violation, void* stream);
int fb_cw_conv2d_f32(const float* x_lw, const float* x_uw, const float* Wt, float* y_lw, float* y_uw,
                     int64_t rows, int64_t row_start, int H0, int W0, const int* chain, int n_chain,
                     int Cin, int H, int W, int Cout, int Kh, int Kw, int stride, int pad, void* stream);
int fb_cw_norm_partials_f32(const float* z_lw, const float* z_uw, float* part_l, float* part_u,
                            int64_t rows, int64_t row_start, int Cin0, int H0, int W0, const int* chain, int n_chain,
                            int C, int H, int W, int p, void* stream);
int fb_cw_relax_apply_f32(int op, const float* z_lw, const float* z_uw, const float* lb, const float* ub,
                          const float* norm_l, const float* norm_u, float* out_lw, float* out_uw,
                          float* out_lb, float* out_ub, float* coef_ws, int64_t rows, int64_t row_start,
                          int H0, int W0, const int* chain, int n_chain, int C, int H, int W,
                          int p, float eps, int* violation, void* stream);
int fb_cw_linear_f32(const float* z_lw, const float* z_uw, const float* Wl, float* y_lw, float* y_uw, float* wt_ws,
                     int64_t rows, int64_t row_start, int H0, int W0, const int* chain, int n_chain,
                     int C, int H, int W, int N, void* stream);
int fb_cw_expand_f32(const float* z_lw, const float* z_uw, float* y_lw, float* y_uw,
                     int64_t rows, int64_t row_start, int H0, int W0, const int* chain, int n_chain,
                     int C, int H, int W, void* stream);

/* ---- whole-model driver: CNN with every pixel of the image perturbed ----------------------
 * conv -> [relu] -> (conv | relu)* -> linear -> (relu | linear)*, dim_in = cin * h * w, input bound lw = uw = I,
 * lb = ub = image [cin, h, w] (device).  Computes the rows [row_start, row_start + rows) of dim_in (a rank's shard, or
 * 0 and cin*h*w) and writes the concretised range of the last layer, out_l / out_u [features of the last layer]; with a
 * communicator (world > 1) the dual norms are all-reduced over the ranks by `algo` (fb_allreduce_algo) and every rank
 * gets the same range, with comm == NULL nothing is exchanged.  One call enqueues the whole pass on `stream`.
 * The first layer must be a convolution (its output, and the relaxation behind it, are written from the filter alone).
 * compact != 0 (the default of the Python layer): rows are kept as their windows only (the fb_cw_* operators above)
 * until the first linear layer; compact == 0: dense rows, fb_conv2d_identity_relax_f32 and fb_conv2d_windowed_f32.  The reference has no CNN
 * verifier to mirror (HandTunedKernels/convolution_verification.cu:228-238 is a benchmark stub); layer semantics are
 * Bounds.matmul / Bounds.relu (Bounds.py:397-413, :921-963) with dim_in as the batch axis of the convolutions.
 * Weights are device pointers: conv [cout, cin, kh, kw], linear [n_out, features] (nn.Linear layout), bias or NULL. */
typedef enum fb_cnn_kind { FB_CNN_CONV = 0, FB_CNN_RELU = 1, FB_CNN_LINEAR = 2 } fb_cnn_kind;
typedef struct fb_cnn_layer {
  int kind;
  const float* weight;
  const float* bias;
  int cout, kh, kw, stride, pad;   /* FB_CNN_CONV */
  int n_out;                       /* FB_CNN_LINEAR */
} fb_cnn_layer;
typedef struct fb_cnn {
  int n_layers;
  const fb_cnn_layer* layer;       /* host array */
  int cin, h, w;
} fb_cnn;
int64_t fb_cnn_workspace_bytes(const fb_cnn* net, int64_t rows);   /* -1: malformed network */
int fb_cnn_forward_f32(const fb_cnn* net, const float* image, int p, float eps, int64_t row_start, int64_t rows,
                       fb_comm* comm, int algo, int compact, float* out_l, float* out_u, int* violation,
                       void* workspace, int64_t workspace_bytes, void* stream);

/* ---- measurement hooks (no counterpart in the reference) --------------------------------
 * fb_profile_enable(1) clears the records and makes every outermost operator call bracket its
 * launches with a pair of CUDA events on the caller's stream; fb_profile_read() waits for the
 * recorded events and returns, per operator kind (0 matmul, 1 relax/concretize, 2 dot product,
 * 3 bound x bound multiply, 4 exact elementwise ops, 5 conv), the summed device time in ms, the
 * number of calls and their algorithmic flops and bytes.  fb_launch_count() is the number of
 * kernels this library has launched in the process so far. */
int fb_profile_enable(int on);
int fb_profile_read(int kind, double* ms, int64_t* calls, double* flops, double* bytes);
int64_t fb_launch_count(void);
/* Launches a register-only chain of fp32 multiply-adds on every SM (scratch: one device float)
 * and returns in *flops the floating-point operations it performs; timed by the caller with
 * CUDA events it gives the CUDA-core fp32 peak used as the roof of the FFMA kernels. */
int fb_bench_ffma(float* scratch, int iters, double* flops, void* stream);
/* The same for the tensor pipe with kind::tf32 operands: every SM issues 128 x 256 x 8 tcgen05.mma instructions back
 * to back (8 * iters per SM); *flops receives the floating-point operations performed.  The rate is the roof of the
 * 3xTF32 kernels (which execute three such products per fp32 product). */
int fb_bench_tf32(int iters, double* flops, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FAITH_B200_H */
