// Split-sign product of bounds with a constant weight on the 5th-generation tensor cores
// (tcgen05 / TMEM), fp32-accurate through a 3xTF32 split.
//
//   y_c = c W^T,  y_r = r |W|^T,  y_lw = y_c - y_r,  y_uw = y_c + y_r,
//   c = (x_lw + x_uw)/2,  r = (x_uw - x_lw)/2          (centre/radius form of Bounds.py:403-412)
//
// Every fp32 operand v is split into hi = v with the 13 low mantissa bits cleared and lo = v - hi
// (exact); a product a*b is evaluated as a_hi*b_hi + a_hi*b_lo + a_lo*b_hi with fp32 accumulation in
// tensor memory.  The tensor core reads the leading 11 significant bits of lo; what is dropped per
// operand is below 2^-20 |v| (2^-22 |v| on average) and the dropped lo*lo term is below 2^-20.
//
// The tensor cores add into their fp32 accumulator with truncation, a bias that grows with the
// number of accumulating instructions; the two small cross terms therefore go to accumulators of
// their own (their truncation is negligible at 2^-10 of the magnitude) and the leading hi*hi term
// is the only one that touches the main accumulators.  The four partial results are summed with
// round-to-nearest in registers in the epilogue.
//
// One CTA computes a 128 x 64 tile of both outputs (four accumulators of 64 columns and two
// operand buffers of 128 columns fill the 512 columns of tensor memory, which is what limits the
// tile to 64 columns).  K is walked in blocks of 32.  Warp roles (28 warps):
//   warp 0       TMA producer: raw fp32 tiles of x_lw, x_uw (128 rows x 32) and of W (64 rows x 32)
//                into a two-stage shared-memory ring (128-byte swizzle).
//   warps 1-3    MMA issuers, one per accumulator set (main centre + main radius / centre
//                correction / radius correction), 8 tcgen05.mma.kind::tf32 per k-block each.  One
//                thread sustains one MMA per 50-110 cycles whatever its size (measured), a
//                128 x 64 x 8 MMA occupies the tensor core for 32: three issuers keep it fed, and
//                as no accumulator is shared between them they need no order among themselves.
//   warps 4-11   epilogue, two warps per tensor-memory lane quarter (32 columns each): tcgen05.ld the accumulators,
//                y_c -/+ y_r (+ bias), stage the two output tiles in shared memory (swizzled) and
//                write them with TMA stores (full 128-byte lines).
//   warps 12-27  converters, two groups of eight; group g handles the k-blocks it = g (mod 2):
//                read the raw tiles, form c, r, split hi/lo, and
//                - store the four A planes (c_hi, c_lo, r_hi, r_lo) of the block into TENSOR MEMORY
//                  (tcgen05.st; the A operand of the MMAs comes from TMEM, lane = tile row),
//                - store the four B planes (W_hi, W_lo, |W|_hi, |W|_lo) into shared memory in the
//                  K-major 128B-swizzled layout the MMA descriptor expects.
// TMEM columns: [0,64) centre main, [64,128) radius main, [128,192) centre correction,
// [192,256) radius correction, [256,512) two buffers of the four A planes.  No cluster launch
// and no multicast is used.
//
// The kernel is persistent: a CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  with one
// running k-block counter, so the producer and the converters run ahead into the next tile while
// the MMAs of the current one finish and the epilogue warps write it out; the tensor cores idle
// only while the accumulators are read out of tensor memory.
//
// Every wait on an mbarrier is bounded; on expiry the kernel raises a device-side flag
// (fb_tc_error_flag, and bit 2 of the caller's status word where one is registered), drains, frees its
// tensor memory and returns.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace fb {
namespace {

constexpr int BM = 128, BN = 64, BK = 32;
constexpr int kGroupWarps = 8;                           // converter warps per group: 4 row quarters x 2 k halves of a k-block
constexpr int kConvGroups = 2;                           // group g converts the k-blocks it = g (mod 2)
constexpr int kConvWarps = kConvGroups * kGroupWarps;
constexpr int kIssuers = 3;                              // MMA-issuing warps, each owning accumulators of its own
constexpr int kEpiWarps = 8;                             // epilogue warps: 4 tensor-memory lane quarters x 2 column halves
constexpr int kCtrlWarps = 1 + kIssuers;                 // TMA producer + issuers
constexpr int kFirstConvWarp = kCtrlWarps + kEpiWarps;
constexpr int kThreads = 32 * (kFirstConvWarp + kConvWarps);
static_assert(kCtrlWarps % 4 == 0, "epilogue warp e must be the warp of lane quarter e");
constexpr uint32_t kTileBytes = BM * BK * 4;             // one 128 x 32 fp32 tile of x = 16 KB
constexpr uint32_t kWTileBytes = BN * BK * 4;            // one 64 x 32 fp32 tile of W = 8 KB
constexpr uint32_t kRawStageBytes = 2 * kTileBytes + kWTileBytes;  // x_lw, x_uw, W
constexpr uint32_t kPlaneStageBytes = 4 * kWTileBytes;   // W_hi, W_lo, |W|_hi, |W|_lo
constexpr int kRawStages = 2;                            // TMA runs two k-blocks ahead
constexpr int kLiveWords = 128;                          // bitmap of the CTA's tiles that are not known to be zero (4096 tiles)
constexpr uint32_t kOutBoxBytes = BM * 32 * 4;            // one 128-row x 32-column fp32 box of an output tile = 16 KB
constexpr uint32_t kOutStageBytes = 4 * kOutBoxBytes;    // lower and upper output tile, two boxes each
constexpr uint32_t kSmemBytes = kRawStages * kRawStageBytes + 2 * kPlaneStageBytes + kOutStageBytes + 1024 /*align*/ + 256 /*barriers*/ +
                                kLiveWords * 4 /*live-tile bitmap*/;
constexpr uint32_t kTmemCols = 512;
// Extra shared memory of the instantiations that apply the layer norm in the epilogue (kLN), behind the live-tile bitmap:
// column means of W and |W| [512 + 512], gain split by sign [128 + 128], shift [128], mean of the layer bias [4], and the
// row means handed from the converters to the epilogue, [2 tiles][4 partial sums][128 rows] x (centre, radius).
constexpr uint32_t kLnOffWbar = 0, kLnOffAbar = 2048, kLnOffGp = 4096, kLnOffGn = 4608, kLnOffBeta = 5120, kLnOffBiasMean = 5632,
                   kLnOffMu = 5648, kLnSmemBytes = 5648 + 2 * 4 * 128 * 8;
constexpr int kLnMaxK = 512, kLnN = 128;
constexpr uint32_t kAccC = 0, kAccR = 64, kCorC = 128, kCorR = 192, kABase = 256;  // TMEM column map



#include "tc_common.cuh"

// The MMAs of one k-block (4 k steps x 6), split over three issuing warps by accumulator, so that
// no accumulator is shared between issuers and no ordering between them is needed:
//   role 0: the two main accumulators,   acc_c += c_hi W_hi,  acc_r += r_hi |W|_hi
//   role 1: centre correction,           cor_c += c_lo W_hi + c_hi W_lo
//   role 2: radius correction,           cor_r += r_lo |W|_hi + r_hi |W|_lo
// One issuing thread sustains one MMA per ~50-90 cycles whatever the MMA's size; a 128 x 64 x 8 MMA
// keeps the tensor core busy for 32, so a single issuer leaves it idle most of the time.
// kFirst: this k-block starts a tile, so the first MMA into each accumulator overwrites.
// planes of B: 0 W_hi, 1 W_lo, 2 |W|_hi, 3 |W|_lo;  planes of A: 0 c_hi, 1 c_lo, 2 r_hi, 3 r_lo
template <int kRole, bool kFirst, bool kPoint>
__device__ __forceinline__ void issue_kblock(const uint32_t (&blo)[4][4], const uint32_t (&acol)[4][4], uint32_t b_hi,
                                             uint32_t d0, uint32_t d1, uint32_t idesc) {
  constexpr int kSteps = (kPoint && kRole == 2) ? 0 : 4;   // zero radius: no radius products at all
#pragma unroll
  for (int j = 0; j < kSteps; ++j) {
    if (kRole == 0) {
      if (j == 0 && kFirst) {
        mma_tf32_ts_lean<false>(d0, acol[0][j], blo[0][j], b_hi, idesc);
        if (!kPoint) mma_tf32_ts_lean<false>(d1, acol[2][j], blo[2][j], b_hi, idesc);
      } else {
        mma_tf32_ts_lean<true>(d0, acol[0][j], blo[0][j], b_hi, idesc);
        if (!kPoint) mma_tf32_ts_lean<true>(d1, acol[2][j], blo[2][j], b_hi, idesc);
      }
    } else {
      constexpr int lo = kRole == 1 ? 1 : 3, hi = kRole == 1 ? 0 : 2;   // A planes; B planes are hi, lo the other way round
      if (j == 0 && kFirst) mma_tf32_ts_lean<false>(d0, acol[lo][j], blo[hi][j], b_hi, idesc);
      else mma_tf32_ts_lean<true>(d0, acol[lo][j], blo[hi][j], b_hi, idesc);
      mma_tf32_ts_lean<true>(d0, acol[hi][j], blo[lo][j], b_hi, idesc);
    }
  }
}
template <int kRole, bool kPoint>
__device__ __forceinline__ void issue_kblock_role(bool first, const uint32_t (&blo)[4][4], const uint32_t (&acol)[4][4],
                                                  uint32_t b_hi, uint32_t d0, uint32_t d1, uint32_t idesc) {
  if (first) issue_kblock<kRole, true, kPoint>(blo, acol, b_hi, d0, d1, idesc);
  else issue_kblock<kRole, false, kPoint>(blo, acol, b_hi, d0, d1, idesc);
}

// Instruction descriptor: D fp32, A and B tf32, both K-major, M = 128, N = 64.
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

struct SharedLayout {
  // offsets from the 1024-byte aligned base
  __host__ __device__ static constexpr uint32_t raw(int s) { return (uint32_t)s * kRawStageBytes; }
  __host__ __device__ static constexpr uint32_t planes(int s) { return kRawStages * kRawStageBytes + (uint32_t)s * kPlaneStageBytes; }
  __host__ __device__ static constexpr uint32_t out() { return kRawStages * kRawStageBytes + 2 * kPlaneStageBytes; }
  __host__ __device__ static constexpr uint32_t bars() { return out() + kOutStageBytes; }
};

// kCoef: column slopes of a relaxation are applied to the operands on the fly (a separate instantiation, so
// that the plain kernel keeps its register allocation).
// kNorm: the epilogue also writes the dual norm over the 128 rows of every output column of the tile,
// norm_lo / norm_up [M / 128][N] (norm_p as in the concretisation: sum |x|, sqrt(sum x^2) or max |x|).  With one
// word block of dim_in per tile that is the concretisation term of the result, so the product that
// consumes it needs no pass of its own over y_lw / y_uw.
// kResid: a residual bound (same shape and layout as the result, plain store only) is added to the result in
// the epilogue: its tile is fetched by TMA into the staging buffer while the k-blocks of the tile are still
// running, so the layer norm that follows reads one tensor pair instead of two.
// kPoint: x_lw and x_uw are the same tensor (every stage before the first relaxation): the radius is zero, so
// x_uw is not loaded, no radius planes are written, the radius products are not issued and the epilogue reads
// two accumulators; the results equal those of the general kernel bit for bit.
//
// Bias rows in the same grid: tiles main_tiles .. total_tiles-1 belong to a second operand (the bias terms
// x_lb, x_ub [rows, K] of the bound whose weight rows are the first operand): the same W, maps of their own
// (tm_b_*, tm_bout_*, tm_bres_*), the layer bias bias_b added, plain store, no slopes and no column norms.  Every tile is
// computed exactly as a launch of its own would compute it.  main_tiles == total_tiles: no such tiles.
//
// kLN (with kResid, N = 128, bias rows in the same grid): the layer norm that follows the product (mode no_var,
// Bounds.py:1111-1131: lw - mean(uw), uw - mean(lw) over the features, then the gain with its sign split, the shift
// on the bias rows) is applied before the store.  A tile holds 64 of the 128 features of a row, so the row means
// come from elsewhere: the mean over n of (x W^T)[r, n] is x[r, :] . mean_n W[n, :], which the converters accumulate from
// the centres and radii they hold anyway (column means of W and |W| in shared memory; four partial sums per row, added
// by the epilogue in a fixed order); the row sums of the residual were left behind by whoever wrote it (ln_args.rs_in:
// [2 lines][4 partial sums][rows of the bound, weight rows first]), and this launch leaves those of its own result in
// ln_args.rs_out for the next one.
//
// status: device word of the caller (may be null); bit 2 is set when a bounded wait of this launch expired.
// wait_tries: bound of every mbarrier wait in tries of ~20 us.  skip_it >= 0 makes the producer of CTA 0 leave
// out the loads of that k-block: the self-test of the give-up path (fb_tc_selftest_timeout), never set otherwise.
template <bool kCoef, bool kNorm, bool kResid, bool kPoint, bool kLN>
__global__ void __launch_bounds__(kThreads, 1)
split_sign_gemm_tc(const __grid_constant__ CUtensorMap tm_lo, const __grid_constant__ CUtensorMap tm_up,
                   const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_out_lo,
                   const __grid_constant__ CUtensorMap tm_out_up, const __grid_constant__ CUtensorMap tm_res_lo,
                   const __grid_constant__ CUtensorMap tm_res_up, const __grid_constant__ CUtensorMap tm_b_lo,
                   const __grid_constant__ CUtensorMap tm_b_up, const __grid_constant__ CUtensorMap tm_bout_lo,
                   const __grid_constant__ CUtensorMap tm_bout_up, const __grid_constant__ CUtensorMap tm_bres_lo,
                   const __grid_constant__ CUtensorMap tm_bres_up, const float* __restrict__ bias,
                   const float* __restrict__ bias_b, int main_tiles, int same_out_b, int64_t M, int N, int K,
                   int n_tiles_n, int64_t total_tiles, int split_rows, int split_d,
                   const float* __restrict__ coef_l, const float* __restrict__ coef_u, int coef_di,
                   float* __restrict__ norm_lo, float* __restrict__ norm_up, int norm_p,
                   int* __restrict__ status, uint32_t wait_tries, int skip_it, const LiveRows live_rows, int same_out,
                   const TcLnArgs ln_args, int64_t Mb) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  // Row blocks known to be zero (live_rows.L > 0; zero-radius instantiation only): a tile of such a block is not
  // loaded, converted or multiplied; the issuers only signal "ready" and the epilogue stores zeros (and zero norms).
  const bool use_live = kPoint && kNorm && !kCoef && !kResid && live_rows.L > 0;
  auto tile_live_slow = [&](int tile) -> bool {
    if (tile >= main_tiles) return true;   // bias rows are never known to be zero
    const unsigned bl = ((unsigned)(tile / n_tiles_n) * (unsigned)BM) / (unsigned)live_rows.Di;   // M < 2^31
    const int l = (int)(bl % (unsigned)live_rows.L), b = (int)(bl / (unsigned)live_rows.L);
    bool live = false;
#pragma unroll
    for (int w = 0; w < 4; ++w)
      if (w < live_rows.words)
        live |= (live_rows.inst_pos != nullptr ? __ldg(live_rows.inst_pos + b * live_rows.words + w) : live_rows.pos[w]) == l;
    return live;
  };
  // barriers: full[2], raw_empty[2], ops_ready[2], mma_done[2], acc_ready, acc_free; then the TMEM base slot and the abort flag
  const uint32_t bar0 = base + SharedLayout::bars();
  const uint32_t bar_full = bar0 + 0;            // [kRawStages]
  const uint32_t bar_raw_empty = bar0 + 32;      // [kRawStages]
  const uint32_t bar_ops_ready = bar0 + 64;      // [2]   (addresses are computed, never indexed from
  const uint32_t bar_mma_done = bar0 + 80;       // [2]    an array: that would live in local memory)
  const uint32_t bar_acc_ready = bar0 + 96;
  const uint32_t bar_acc_free = bar0 + 104;
  const uint32_t bar_conv = bar0 + 128;          // rendezvous of the converter warps in the epilogue (bounded, unlike bar.sync)
  const uint32_t bar_res = bar0 + 136;           // residual tile has landed in the staging buffer (kResid)
  const uint32_t bar_mu = bar0 + 144;            // [2] row means of a tile are in shared memory (kLN)
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + SharedLayout::bars() + 112);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(base_ptr + SharedLayout::bars() + 120);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (K + BK - 1) / BK;
  // tiles of this CTA: blockIdx.x + i * gridDim.x, i = 0 .. my_tiles-1; n is the fast tile index
  // (the host side guarantees that tile and k-block counts fit 32 bits: 64-bit loop counters and a
  // 64-bit division per k-block cost more instructions than the conversion itself)
  const int my_tiles = (int)((total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x);
  const int total_it = my_tiles * nkb;   // k-blocks this CTA walks, across all its tiles

  // Liveness of this CTA's tiles, worked out once by all threads into a bitmap (every role of every tile asks; the
  // divisions and the position loads of the direct form, 28 warps x 100+ tiles, cost more than the zero tiles themselves).
  uint32_t* live_bits = reinterpret_cast<uint32_t*>(base_ptr + SharedLayout::bars() + 256);
  const bool live_map = use_live && my_tiles <= 32 * kLiveWords;
  if (live_map) {
    for (int w = threadIdx.x; w < (my_tiles + 31) / 32; w += blockDim.x) {
      uint32_t bits = 0;
      for (int k = 0; k < 32; ++k) {
        const int ti = w * 32 + k;
        if (ti < my_tiles && tile_live_slow((int)blockIdx.x + ti * (int)gridDim.x)) bits |= 1u << k;
      }
      live_bits[w] = bits;
    }
  }
  // ti: index among this CTA's tiles (tile = blockIdx.x + ti * gridDim.x)
  auto tile_live = [&](int ti) -> bool {
    if (!use_live) return true;
    if (live_map) return (live_bits[ti >> 5] >> (ti & 31)) & 1u;
    return tile_live_slow((int)blockIdx.x + ti * (int)gridDim.x);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_raw_empty + 8 * s, kGroupWarps);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_ops_ready + 8 * s, kGroupWarps);
      mbar_init(bar_mma_done + 8 * s, kIssuers);
    }
    mbar_init(bar_acc_ready, kIssuers);
    mbar_init(bar_acc_free, kEpiWarps);
    mbar_init(bar_conv, kEpiWarps);
    mbar_init(bar_res, 1);
    mbar_init(bar_mu, kConvWarps);
    mbar_init(bar_mu + 8, kConvWarps);
    *cta_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  float* const ln_smem = reinterpret_cast<float*>(base_ptr + SharedLayout::bars() + 256 + kLiveWords * 4);
  if (kLN) {
    // column means of W and |W|, the gain split by sign as the layer-norm kernel splits it.  The rows of W are dealt
    // out to as many threads per group of four columns as the block has (a single thread per column walks 128 rows one
    // load after the other: 40 us); the partial sums go through the output staging buffer, which is idle until the first
    // tile is done, and are added in a fixed order.
    const float inv_n = 1.0f / (float)N;
    {
      float* scratch = reinterpret_cast<float*>(base_ptr + SharedLayout::out());
      const int groups = K >> 2;
      int parts = (int)blockDim.x / groups;
      if (parts > N) parts = N;
      const int gidx = (int)threadIdx.x % groups, part = (int)threadIdx.x / groups;
      if (part < parts) {
        float4 sw = make_float4(0.f, 0.f, 0.f, 0.f), sa = sw;
        for (int n = part; n < N; n += parts) {
          const float4 w = __ldg(reinterpret_cast<const float4*>(ln_args.w_raw + (size_t)n * K) + gidx);
          sw.x = fmaf(w.x, inv_n, sw.x); sw.y = fmaf(w.y, inv_n, sw.y); sw.z = fmaf(w.z, inv_n, sw.z); sw.w = fmaf(w.w, inv_n, sw.w);
          sa.x = fmaf(fabsf(w.x), inv_n, sa.x); sa.y = fmaf(fabsf(w.y), inv_n, sa.y);
          sa.z = fmaf(fabsf(w.z), inv_n, sa.z); sa.w = fmaf(fabsf(w.w), inv_n, sa.w);
        }
        reinterpret_cast<float4*>(scratch + (size_t)(2 * part) * K)[gidx] = sw;
        reinterpret_cast<float4*>(scratch + (size_t)(2 * part + 1) * K)[gidx] = sa;
      }
      __syncthreads();
      for (int k = threadIdx.x; k < K; k += blockDim.x) {
        float a = 0.f, b = 0.f;
        for (int q = 0; q < parts; ++q) {
          a = fadd(a, scratch[(size_t)(2 * q) * K + k]);
          b = fadd(b, scratch[(size_t)(2 * q + 1) * K + k]);
        }
        ln_smem[kLnOffWbar / 4 + k] = a;
        ln_smem[kLnOffAbar / 4 + k] = b;
      }
    }
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
      const float gv = __ldg(ln_args.gamma + n);
      const float gpv = gv > 0.f ? gv : 0.f;
      ln_smem[kLnOffGp / 4 + n] = gpv;
      ln_smem[kLnOffGn / 4 + n] = fsub(gv, gpv);
      ln_smem[kLnOffBeta / 4 + n] = __ldg(ln_args.beta + n);
    }
    if (threadIdx.x == 0) {
      float sb = 0.f;
      for (int n = 0; n < N && bias_b != nullptr; ++n) sb = fmaf(__ldg(bias_b + n), inv_n, sb);
      ln_smem[kLnOffBiasMean / 4] = sb;
    }
  }
  if (warp == 1) {  // one warp allocates all of tensor memory for this CTA
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx wc = {cta_abort, wait_tries};

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // the whole warp walks the loop convergently (a lone thread looping while its 31 siblings sit at
    // the final barrier runs much slower); only the copy instructions are issued by lane 0
    int it = 0;
    bool ok = true;
    for (int ti = 0; ti < my_tiles && ok; ++ti) {
      const int tile = blockIdx.x + ti * gridDim.x;
      if (!tile_live(ti)) continue;
      const bool bseg = tile >= main_tiles;            // a tile of the bias rows
      const int stile = bseg ? tile - main_tiles : tile;
      const int m0 = (int)(stile / n_tiles_n) * BM, n0 = (int)(stile % n_tiles_n) * BN;
      const CUtensorMap* const map_lo = bseg ? &tm_b_lo : &tm_lo;
      const CUtensorMap* const map_up = bseg ? &tm_b_up : &tm_up;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int rs = (int)(it % kRawStages);
        const uint32_t full = bar_full + 8 * rs;
        if (it >= kRawStages &&
            !mbar_wait_warp(bar_raw_empty + 8 * rs, (uint32_t)((it / kRawStages - 1) & 1), wc)) { ok = false; break; }
        if (lane == 0 && !(blockIdx.x == 0 && it == skip_it)) {
          mbar_arrive_expect_tx(full, kPoint ? kRawStageBytes - kTileBytes : kRawStageBytes);
          const uint32_t dst = base + SharedLayout::raw(rs);
          tma_load_2d(dst, map_lo, kb * BK, m0, full);
          if (!kPoint) tma_load_2d(dst + kTileBytes, map_up, kb * BK, m0, full);
          tma_load_2d(dst + 2 * kTileBytes, &tm_w, kb * BK, n0, full);
        }
        __syncwarp();
      }
    }
  } else if (warp < kCtrlWarps) {
    // ------------------------------------------------------------------ MMA issuers (warps 1-3)
    // Each warp walks the loop convergently; lane 0 issues.  Descriptors are built once and only
    // advanced by compile-time constants inside the loop: every operand of a warp's 2 x 8 MMAs
    // (two operand stages) lives in a loop-invariant register.
    const int role = warp - 1;
    bool ok = true;
    int it = 0;
    const uint64_t bdesc0 = smem_desc_sw128(base + SharedLayout::planes(0));
    const uint32_t b_hi = (uint32_t)(bdesc0 >> 32);
    const uint32_t d0 = tmem_base + (role == 0 ? kAccC : role == 1 ? kCorC : kCorR), d1 = tmem_base + kAccR;
    uint32_t blo[2][4][4], acol[2][4][4];
#pragma unroll
    for (int st = 0; st < 2; ++st)
#pragma unroll
      for (int pl = 0; pl < 4; ++pl)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // descriptor address field is in 16-byte units: stage, plane, k step -> byte offset / 16
          blo[st][pl][j] = (uint32_t)bdesc0 + ((st * kPlaneStageBytes + pl * kWTileBytes + j * 32) >> 4);
          acol[st][pl][j] = tmem_base + kABase + st * 128 + pl * 32 + j * 8;
        }
    int lt = 0;   // tiles multiplied so far: the accumulator hand-shake with the epilogue counts these only
    for (int ti = 0; ti < my_tiles && ok; ++ti) {
      if (!tile_live(ti)) continue;   // a zero row block: nothing to multiply, nothing to signal
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = (int)(it & 1);
        ok = mbar_wait_warp(bar_ops_ready + 8 * s, (uint32_t)((it >> 1) & 1), wc);
        // the first MMA of a tile overwrites the accumulators: the previous tile must have been read out
        if (ok && kb == 0 && lt > 0) ok = mbar_wait_warp(bar_acc_free, (uint32_t)((lt - 1) & 1), wc);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          if (s == 0) {
            if (role == 0) issue_kblock_role<0, kPoint>(kb == 0, blo[0], acol[0], b_hi, d0, d1, kInstrDesc);
            else if (role == 1) issue_kblock_role<1, kPoint>(kb == 0, blo[0], acol[0], b_hi, d0, d1, kInstrDesc);
            else issue_kblock_role<2, kPoint>(kb == 0, blo[0], acol[0], b_hi, d0, d1, kInstrDesc);
          } else {
            if (role == 0) issue_kblock_role<0, kPoint>(kb == 0, blo[1], acol[1], b_hi, d0, d1, kInstrDesc);
            else if (role == 1) issue_kblock_role<1, kPoint>(kb == 0, blo[1], acol[1], b_hi, d0, d1, kInstrDesc);
            else issue_kblock_role<2, kPoint>(kb == 0, blo[1], acol[1], b_hi, d0, d1, kInstrDesc);
          }
          tc_commit(bar_mma_done + 8 * s);
          if (kb == nkb - 1) tc_commit(bar_acc_ready);
        }
        __syncwarp();
      }
      ++lt;
    }
  } else if (warp < kFirstConvWarp) {
    // ------------------------------------------------------------------ epilogue (warps 4-11)
    // Warp (q, h) reads rows q*32.. and columns h*32.. of the four accumulators, 8 columns at a time, combines them
    // (y_c -/+ y_r, + bias), stages the two output tiles in shared memory in the 128-byte-swizzled
    // box layout and has them written by TMA, so that global memory sees whole 128-byte lines.
    // Rows and columns beyond M and N are clipped by the tensor map.  The accumulators are handed
    // back to the MMA issuers as soon as the last column is in registers; the converters never
    // stop for an epilogue.
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const bool leader = threadIdx.x == 32 * kCtrlWarps;
    bool ok = true;
    uint32_t epi_phase = 0;
    // rendezvous of the epilogue warps through an mbarrier, so that the wait is bounded
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_conv);
      const bool r = mbar_wait_warp(bar_conv, epi_phase & 1u, wc);
      ++epi_phase;
      return r;
    };
    const int chalf = (warp - kCtrlWarps) >> 2;   // which 32 of the 64 tile columns (= which output box)
    bool staging_zero = false;   // the staging buffer holds zeros (left there by a tile of a zero row block)
    int le = 0;                  // tiles read out of tensor memory so far (the issuers count the same tiles)
    for (int e = 0; e < my_tiles && ok; ++e) {
      const int etile = blockIdx.x + e * gridDim.x;
      const bool elive = tile_live(e);
      const bool bseg = etile >= main_tiles;           // a tile of the bias rows: maps and bias of its own, plain store, no norms
      const int stile = bseg ? etile - main_tiles : etile;
      const int my = (stile / n_tiles_n) * BM, nx = (stile % n_tiles_n) * BN;
      const float* const tbias = bseg ? bias_b : bias;
      const CUtensorMap* const map_out_lo = bseg ? &tm_bout_lo : &tm_out_lo;
      const CUtensorMap* const map_out_up = bseg ? &tm_bout_up : &tm_out_up;
      const int t_split_rows = bseg ? 0 : split_rows;
      const bool t_same_out = (bseg ? same_out_b : same_out) != 0;
      if (!elive) {
        // A zero row block (kPoint and kNorm only): the result is +0 everywhere and so are its column norms.  The
        // accumulators play no part (the issuers skip the tile as well); the staging buffer is zeroed once and then
        // stored from for every such tile in a row, without being touched again, so these tiles cost their stores and
        // little else.
        if (!staging_zero) {
          if (leader) tma_store_wait_read();
          ok = epi_sync();
          if (!ok) break;
          float4* sz = reinterpret_cast<float4*>(base_ptr + SharedLayout::out());
          for (uint32_t i = threadIdx.x - 32 * kCtrlWarps; i < kOutStageBytes / 16; i += 32 * kEpiWarps)
            sz[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          fence_async_smem();
          ok = epi_sync();
          if (!ok) break;
          staging_zero = true;
        }
        if (leader) {
          const uint32_t so = base + SharedLayout::out();
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            int cx = nx + 32 * q, cy = my, cz = 0;
            if (t_split_rows > 0) {
              const int heads = N / split_d;
              cz = (my / t_split_rows) * heads + cx / split_d;
              cy = my % t_split_rows;
              cx = cx % split_d;
            }
            tma_store_3d(map_out_lo, cx, cy, cz, so + q * kOutBoxBytes);
            // (zero radius and one buffer named as both outputs: the two tiles are the same numbers, stored once)
            if (!(kPoint && t_same_out)) tma_store_3d(map_out_up, cx, cy, cz, so + (2 + q) * kOutBoxBytes);
          }
          tma_store_commit();
        }
        if (kNorm) {
          const int i = (int)threadIdx.x - 32 * kCtrlWarps;   // 0..255: 64 lower and 64 upper norms
          const int n = nx + (i & 63);
          if (i < 128 && n < N) (i < 64 ? norm_lo : norm_up)[(int64_t)(my / BM) * N + n] = 0.f;
        }
        continue;
      }
      staging_zero = false;
      // the staging buffer is free once the previous tile's stores have read it: settle that before
      // the accumulators become ready, so that nothing stands between "ready" and the read-out
      if (leader) tma_store_wait_read();
      ok = epi_sync();
      if (!ok) break;
      if (kResid && leader) {
        // the staging buffer is free now: fetch the residual tile into it (same boxes as the store below)
        const uint32_t so = base + SharedLayout::out();
        mbar_arrive_expect_tx(bar_res, kOutStageBytes);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          tma_load_3d(so + q * kOutBoxBytes, bseg ? &tm_bres_lo : &tm_res_lo, nx + 32 * q, my, 0, bar_res);
          tma_load_3d(so + (2 + q) * kOutBoxBytes, bseg ? &tm_bres_up : &tm_res_up, nx + 32 * q, my, 0, bar_res);
        }
      }
      // kLN: the row sums of the residual do not depend on the accumulators: their loads go out before the wait
      int64_t grow = 0;                                // row of the bound: weight rows first, then the bias rows
      bool rvalid = false;
      float rsl[4] = {0.f, 0.f, 0.f, 0.f}, rsu[4] = {0.f, 0.f, 0.f, 0.f};
      if (kLN) {
        grow = (bseg ? M : 0) + my + row;
        rvalid = my + row < (bseg ? Mb : M);
        if (rvalid) {
#pragma unroll
          for (int sl = 0; sl < 4; ++sl) {
            rsl[sl] = __ldg(ln_args.rs_in + (int64_t)sl * ln_args.rs_stride + grow);
            rsu[sl] = __ldg(ln_args.rs_in + (int64_t)(4 + sl) * ln_args.rs_stride + grow);
          }
        }
      }
      ok = mbar_wait_warp(bar_acc_ready, (uint32_t)(le & 1), wc);
      if (!ok) break;
      ++le;
      tc_fence_after();
      if (kResid) {
        ok = mbar_wait_warp(bar_res, (uint32_t)(e & 1), wc);
        if (!ok) break;
      }
      // kLN: the means over all 128 features of this thread's row of y_lw and of y_uw (product + bias + residual)
      uint64_t mlo2 = 0, mup2 = 0, sl2 = 0, su2 = 0;   // the means as pairs; running sums of the normalised row
      if (kLN) {
        ok = mbar_wait_warp(bar_mu + 8 * (e & 1), (uint32_t)((e >> 1) & 1), wc);
        if (!ok) break;
        const float2* mu = reinterpret_cast<const float2*>(ln_smem + kLnOffMu / 4) + ((e & 1) * 4) * 128 + row;
        const float2 p0 = mu[0], p1 = mu[128], p2 = mu[256], p3 = mu[384];
        const float mc = fadd(fadd(fadd(p0.x, p1.x), p2.x), p3.x), mr = fadd(fadd(fadd(p0.y, p1.y), p2.y), p3.y);
        const float rl = fadd(fadd(fadd(fadd(0.f, rsl[0]), rsl[1]), rsl[2]), rsl[3]);
        const float ru = fadd(fadd(fadd(fadd(0.f, rsu[0]), rsu[1]), rsu[2]), rsu[3]);
        const float inv_n = 1.0f / (float)N;
        float mlo = fadd(fsub(mc, mr), fmul(rl, inv_n)), mup = fadd(fadd(mc, mr), fmul(ru, inv_n));
        if (bseg) {
          mlo = fadd(mlo, ln_smem[kLnOffBiasMean / 4]);
          mup = fadd(mup, ln_smem[kLnOffBiasMean / 4]);
        }
        mlo2 = pack2(__float_as_uint(mlo), __float_as_uint(mlo));
        mup2 = pack2(__float_as_uint(mup), __float_as_uint(mup));
      }
#pragma unroll
      for (int cq = 4 * chalf; cq < 4 * chalf + 4; ++cq) {
        const int ncol = cq * 8;
        uint32_t t0[8], t1[8], t2[8], t3[8];
        tmem_ld8(tmem_base + lane_addr + kAccC + ncol, t0);
        tmem_ld8(tmem_base + lane_addr + kCorC + ncol, t1);
        if (!kPoint) {
          tmem_ld8(tmem_base + lane_addr + kAccR + ncol, t2);
          tmem_ld8(tmem_base + lane_addr + kCorR + ncol, t3);
        }
        tmem_wait_ld();
        if (cq == 4 * chalf + 3) {
          // the accumulators are in registers now: hand tensor memory back to the MMA issuers
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_acc_free);
        }
        uint8_t* so = base_ptr + SharedLayout::out() + (uint32_t)(cq >> 2) * kOutBoxBytes;
        // (pairs of fp32 values per instruction, as in the converters; the order of the additions is that of the
        // scalar form: (y_c -/+ y_r) + bias + residual, each rounded to nearest)
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint64_t lo2[2], up2[2];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int k = q * 4 + 2 * i;
            const uint64_t yc = add2(pack2(t0[k], t0[k + 1]), pack2(t1[k], t1[k + 1]));
            if (kPoint) {
              lo2[i] = yc;
              up2[i] = yc;
            } else {
              const uint64_t yr = add2(pack2(t2[k], t2[k + 1]), pack2(t3[k], t3[k + 1]));
              lo2[i] = sub2(yc, yr);
              up2[i] = add2(yc, yr);
            }
            if (tbias != nullptr) {
              const int n = nx + ncol + k;   // even, and N is a multiple of four: n and n + 1 are inside or outside together
              const uint64_t bv = n < N ? pack2(__float_as_uint(tbias[n]), __float_as_uint(tbias[n + 1])) : 0ull;
              lo2[i] = add2(lo2[i], bv);
              up2[i] = add2(up2[i], bv);
            }
          }
          const uint32_t off = swz(row, (cq & 3) * 2 + q);
          if (kResid) {
            const ulonglong2 rl = *reinterpret_cast<const ulonglong2*>(so + off);
            const ulonglong2 ru = *reinterpret_cast<const ulonglong2*>(so + 2 * kOutBoxBytes + off);
            lo2[0] = add2(lo2[0], rl.x); lo2[1] = add2(lo2[1], rl.y);
            up2[0] = add2(up2[0], ru.x); up2[1] = add2(up2[1], ru.y);
          }
          if (kLN) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const int n = nx + ncol + q * 4 + 2 * i;
              const uint64_t gp2 = *reinterpret_cast<const uint64_t*>(ln_smem + kLnOffGp / 4 + n);
              const uint64_t gn2 = *reinterpret_cast<const uint64_t*>(ln_smem + kLnOffGn / 4 + n);
              const uint64_t dl = sub2(lo2[i], mup2), du = sub2(up2[i], mlo2);   // each line minus the mean of the other
              uint64_t zl = add2(mul2(dl, gp2), mul2(du, gn2)), zu = add2(mul2(dl, gn2), mul2(du, gp2));
              if (bseg) {
                const uint64_t b2 = *reinterpret_cast<const uint64_t*>(ln_smem + kLnOffBeta / 4 + n);
                zl = add2(zl, b2);
                zu = add2(zu, b2);
              }
              sl2 = add2(sl2, zl);
              su2 = add2(su2, zu);
              lo2[i] = zl;
              up2[i] = zu;
            }
          }
          *reinterpret_cast<ulonglong2*>(so + off) = make_ulonglong2(lo2[0], lo2[1]);
          *reinterpret_cast<ulonglong2*>(so + 2 * kOutBoxBytes + off) = make_ulonglong2(up2[0], up2[1]);
        }
      }
      if (kLN && rvalid && ln_args.rs_out != nullptr) {
        // sums of this thread's row over the 32 columns it handled: partial sum (n tile, column half) of the result's row
        const int sl = (nx / BN) * 2 + chalf;
        ln_args.rs_out[(int64_t)sl * ln_args.rs_stride + grow] =
            fadd(__uint_as_float((uint32_t)sl2), __uint_as_float((uint32_t)(sl2 >> 32)));
        ln_args.rs_out[(int64_t)(4 + sl) * ln_args.rs_stride + grow] =
            fadd(__uint_as_float((uint32_t)su2), __uint_as_float((uint32_t)(su2 >> 32)));
      }
      fence_async_smem();
      ok = epi_sync();
      if (!ok) break;
      if (leader) {
        // The output tensor map is 3-D.  Plain store: (column, row, 0).  Head-split store
        // (split_rows > 0): the output is [group * heads + head][row in group][feature in head], a
        // 32-column box lies inside one head and its 128 rows inside one group.
        const uint32_t so = base + SharedLayout::out();
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          int cx = nx + 32 * q, cy = my, cz = 0;
          if (t_split_rows > 0) {
            const int heads = N / split_d;
            cz = (my / t_split_rows) * heads + cx / split_d;
            cy = my % t_split_rows;
            cx = cx % split_d;
          }
          tma_store_3d(map_out_lo, cx, cy, cz, so + q * kOutBoxBytes);
          if (!(kPoint && t_same_out)) tma_store_3d(map_out_up, cx, cy, cz, so + (2 + q) * kOutBoxBytes);
        }
        tma_store_commit();
      }
      if (kNorm && !bseg) {
        // Column norms of the staged tile.  Warp w reads 16 columns of box w / 2 (lower q0, lower q1, upper q0,
        // upper q1): lanes 0-15 the rows with bit 2 clear, lanes 16-31 those with bit 2 set, which the
        // swizzle puts into the other half of the banks.  The next tile overwrites the staging buffer
        // only behind the rendezvous at the top of the loop.
        const int ew = warp - kCtrlWarps;
        const int box = ew >> 1;
        const int c = (ew & 1) * 16 + (lane & 15);
        const int rsel = (lane >> 4) * 4;
        const uint8_t* sb = base_ptr + SharedLayout::out() + (uint32_t)box * kOutBoxBytes + (c & 3) * 4;
        float acc = 0.f;
        for (int i8 = 0; i8 < 16; ++i8) {
          // rows 8 * i8 + rsel + {0, 1, 2, 3}: the four loads first, then the four accumulations
          float v[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) v[k] = *reinterpret_cast<const float*>(sb + swz(8 * i8 + rsel + k, c >> 2));
#pragma unroll
          for (int k = 0; k < 4; ++k) acc = norm_accum(norm_p, acc, v[k]);
        }
        acc = norm_finish(norm_p, norm_combine(norm_p, acc, __shfl_xor_sync(0xffffffffu, acc, 16)));
        const int n = nx + (box & 1) * 32 + c;
        if (lane < 16 && n < N) (box < 2 ? norm_lo : norm_up)[(int64_t)(my / BM) * N + n] = acc;
      }
    }
  } else {
    // ------------------------------------------------- converters
    // Two groups of eight warps; group g converts the k-blocks it = g (mod 2) into operand stage g
    // (raw stage g, plane stage g, A buffer g).  The conversion of a k-block is a chain of
    // latencies (shared-memory loads, arithmetic, tensor-memory stores, barrier hand-overs) longer
    // than the MMAs of a k-block; with two groups half a period apart the chains overlap.
    const int cw = warp - kFirstConvWarp;  // 0..15
    const int g = cw >> 3;             // converter group
    const int gt = (threadIdx.x - 32 * kFirstConvWarp) & 255;   // thread index inside the group
    const int quarter = warp & 3;      // TMEM lane quarter this warp may access
    const int half = (cw >> 2) & 1;    // which 16 of the 32 k values of a block
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    bool ok = true;
    int c_ti = 0, c_kb = g;   // tile and k-block of `it`, kept incrementally (used by the coefficient loads and by kLN)
    uint64_t mc2 = 0, mr2 = 0;   // kLN: partial row means of the product, centre and radius part (pairs)
    int conv_it = total_it;   // k-blocks to convert: those of the live tiles
    if (use_live) {
      int live_tiles = 0;
      for (int ti = 0; ti < my_tiles; ++ti) live_tiles += tile_live(ti) ? 1 : 0;
      conv_it = live_tiles * nkb;
    }
    for (int it = g; it < conv_it && ok; it += 2, c_kb += 2) {
      // Column coefficients of a relaxation applied on the fly (coef_l != nullptr): x_lw is read as
      // coef_l[row block, k] * x_lw and x_uw as coef_u[row block, k] * x_uw, the row block being the
      // (b, l) row of the bound (tile row / coef_di; a tile never straddles two row blocks).  The 16
      // values per side are the same for every thread of the CTA; they are fetched first so that their
      // latency hides behind the wait and the shared-memory loads.
      ulonglong2 kl[4], ku[4];   // pairs of fp32 slopes
      if (kLN && !kCoef) {
        while (c_kb >= nkb) { c_kb -= nkb; ++c_ti; }
      }
      if (kCoef) {
        while (c_kb >= nkb) { c_kb -= nkb; ++c_ti; }
        const int tile = blockIdx.x + c_ti * gridDim.x;
        if (tile >= main_tiles) {
          // bias rows carry no slopes (the relaxed bias terms are given as they are): a factor of one is exact
#pragma unroll
          for (int q = 0; q < 4; ++q) kl[q] = ku[q] = make_ulonglong2(kOne2, kOne2);
        } else {
          const int64_t rb = ((int64_t)(tile / n_tiles_n) * BM) / coef_di;
          const float* pl = coef_l + rb * K + c_kb * BK + half * 16;
          const float* pu = coef_u + rb * K + c_kb * BK + half * 16;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            kl[q] = __ldg(reinterpret_cast<const ulonglong2*>(pl) + q);
            ku[q] = __ldg(reinterpret_cast<const ulonglong2*>(pu) + q);
          }
        }
      }
      ok = mbar_wait_warp(bar_full + 8 * g, (uint32_t)((it >> 1) & 1), wc);
      if (!ok) break;
      const uint8_t* raw = base_ptr + SharedLayout::raw(g);
      // W tile: 64 rows x 8 chunks; this thread converts two adjacent chunks of one row
      const int wrow = gt >> 2, wchunk = (gt & 3) * 2;
      // The arithmetic below runs on pairs of fp32 values (fma / mul / sub .f32x2: one instruction for two
      // round-to-nearest results, bit for bit those of the scalar forms): the converters are bound by the number of
      // instructions they issue, not by the fp32 pipe.  c2[i], r2[i]: elements 2i, 2i+1 of this thread's 16 centres / radii.
      uint64_t c2[8], r2[8], w2[4];
      {
        ulonglong2 vl[4], vu[4], vw[2];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t off = swz(row, half * 4 + q);
          vl[q] = *reinterpret_cast<const ulonglong2*>(raw + off);
          vu[q] = kPoint ? vl[q] : *reinterpret_cast<const ulonglong2*>(raw + kTileBytes + off);
        }
#pragma unroll
        for (int q = 0; q < 2; ++q) vw[q] = *reinterpret_cast<const ulonglong2*>(raw + 2 * kTileBytes + swz(wrow, wchunk + q));
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint64_t l2[2] = {vl[q].x, vl[q].y}, u2[2] = {vu[q].x, vu[q].y};
          if (kCoef) {   // one rounded product per side, as the rescale pass of the relaxation kernels
            l2[0] = mul2(kl[q].x, l2[0]); l2[1] = mul2(kl[q].y, l2[1]);
            u2[0] = mul2(ku[q].x, u2[0]); u2[1] = mul2(ku[q].y, u2[1]);
          }
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            // centre (l + u) / 2 and radius (u - l) / 2, each rounded once
            const uint64_t hu = mul2(u2[i], kHalf2);
            c2[q * 2 + i] = fma2(l2[i], kHalf2, hu);
            r2[q * 2 + i] = fma2(l2[i], kMinusHalf2, hu);
          }
        }
        w2[0] = vw[0].x; w2[1] = vw[0].y; w2[2] = vw[1].x; w2[3] = vw[1].y;
      }
      uint64_t whi2[4], wlo2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) split_tf32_pair(w2[i], whi2[i], wlo2[i]);
      // The raw stage goes back to the TMA producer only when every value loaded from it has been
      // used: a shared-memory load completes asynchronously and the hardware only waits for it at
      // the first instruction that reads its result.  (With the arrive placed directly behind the
      // loads, k-block it+2 was seen overwriting rows of k-block it that were still being read.)
      // The empty asm statements keep the arithmetic above from being moved below the arrive.
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (kPoint) asm volatile("" : "+l"(c2[i]));
        else asm volatile("" : "+l"(c2[i]), "+l"(r2[i]));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) asm volatile("" : "+l"(whi2[i]), "+l"(wlo2[i]));
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_raw_empty + 8 * g);
      if (kLN) {
        // this thread's share of the row means of the product: its 16 centres and radii against the column means of
        // W and |W| (nkb is even here, so the group sees nkb / 2 k-blocks of every tile, the last one at nkb - 2 + g)
        const ulonglong2* wq = reinterpret_cast<const ulonglong2*>(ln_smem + kLnOffWbar / 4 + c_kb * BK + half * 16);
        const ulonglong2* aq = reinterpret_cast<const ulonglong2*>(ln_smem + kLnOffAbar / 4 + c_kb * BK + half * 16);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const ulonglong2 w = wq[q], a = aq[q];
          mc2 = fma2(c2[2 * q], w.x, mc2);
          mc2 = fma2(c2[2 * q + 1], w.y, mc2);
          mr2 = fma2(r2[2 * q], a.x, mr2);
          mr2 = fma2(r2[2 * q + 1], a.y, mr2);
        }
      }
      if (it >= 2) {
        ok = mbar_wait_warp(bar_mma_done + 8 * g, (uint32_t)(((it >> 1) - 1) & 1), wc);
        if (!ok) break;
        tc_fence_after();
      }
      if (kLN && c_kb >= nkb - 2) {
        // Last k-block of the tile for this group: hand the partial row means to the epilogue.  Only now: the MMAs of
        // this group's previous k-block have retired, so the tile before this one has been read out of tensor memory,
        // which the epilogue does after it has read that tile's means; the buffer of the tile two back is free.
        float2* mu = reinterpret_cast<float2*>(ln_smem + kLnOffMu / 4) + (((c_ti & 1) * 4 + g * 2 + half) * 128 + row);
        *mu = make_float2(fadd(__uint_as_float((uint32_t)mc2), __uint_as_float((uint32_t)(mc2 >> 32))),
                          fadd(__uint_as_float((uint32_t)mr2), __uint_as_float((uint32_t)(mr2 >> 32))));
        mc2 = 0;
        mr2 = 0;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_mu + 8 * (c_ti & 1));
      }
      {
        const uint32_t a_cols = tmem_base + lane_addr + kABase + (uint32_t)g * 128u + (uint32_t)half * 16u;
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint64_t h2, l2;
          split_tf32_pair(c2[i], h2, l2);
          hi[2 * i] = (uint32_t)h2; hi[2 * i + 1] = (uint32_t)(h2 >> 32);
          lo[2 * i] = (uint32_t)l2; lo[2 * i + 1] = (uint32_t)(l2 >> 32);
        }
        tmem_st16(a_cols + 0, hi);
        tmem_st16(a_cols + 32, lo);
        if (!kPoint) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint64_t h2, l2;
            split_tf32_pair(r2[i], h2, l2);
            hi[2 * i] = (uint32_t)h2; hi[2 * i + 1] = (uint32_t)(h2 >> 32);
            lo[2 * i] = (uint32_t)l2; lo[2 * i + 1] = (uint32_t)(l2 >> 32);
          }
          tmem_st16(a_cols + 64, hi);
          tmem_st16(a_cols + 96, lo);
        }
        uint8_t* pl = base_ptr + SharedLayout::planes(g);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint32_t off = swz(wrow, wchunk + q);
          // |w| = sgn(w) * (hi + lo); hi and lo both carry the sign of w (lo may be zero)
          const uint64_t m = 0x7fffffff7fffffffull;
          *reinterpret_cast<ulonglong2*>(pl + 0 * kWTileBytes + off) = make_ulonglong2(whi2[2 * q], whi2[2 * q + 1]);
          *reinterpret_cast<ulonglong2*>(pl + 1 * kWTileBytes + off) = make_ulonglong2(wlo2[2 * q], wlo2[2 * q + 1]);
          if (!kPoint) {
            *reinterpret_cast<ulonglong2*>(pl + 2 * kWTileBytes + off) = make_ulonglong2(whi2[2 * q] & m, whi2[2 * q + 1] & m);
            *reinterpret_cast<ulonglong2*>(pl + 3 * kWTileBytes + off) = make_ulonglong2(wlo2[2 * q] & m, wlo2[2 * q + 1] & m);
          }
        }
      }
      fence_async_smem();   // B planes were written through the generic proxy; the MMA reads them through the async proxy
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ops_ready + 8 * g);
    }
  }
  if (threadIdx.x == 32 * kCtrlWarps) tma_store_wait_all();   // this thread issued the bulk stores of the epilogues
  // Tear-down.  On the error path, give outstanding bulk copies time to land before the shared
  // memory is released (bounded), then free the tensor memory.
  if (*cta_abort) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status != nullptr) atomicOr(status, 4);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------ host side
// 2-D fp32 row-major [rows, cols] tensor, box `box_rows` rows x 32 columns.
bool make_map(CUtensorMap* map, const float* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  return get_map(map, ptr, 2, cols, rows, 1, cols * sizeof(float), 0, BK, box_rows);
}

// Output map, always 3-D: plain [1][rows][cols], or head-split [groups * heads][split_rows][split_d].
bool make_out_map(CUtensorMap* map, const float* ptr, uint64_t M, uint64_t N, int split_rows, int split_d) {
  if (split_rows > 0)
    return get_map(map, ptr, 3, (uint64_t)split_d, (uint64_t)split_rows, (M / split_rows) * (N / split_d),
                   (uint64_t)split_d * sizeof(float), (uint64_t)split_rows * split_d * sizeof(float), 32, BM);
  return get_map(map, ptr, 3, N, M, 1, N * sizeof(float), M * N * sizeof(float), 32, BM);
}

thread_local int* t_status_sink = nullptr;
thread_local LiveRows t_live_rows = {0, 0, 0, {0, 0, 0, 0}, nullptr, 0};
uint32_t g_wait_tries = kMaxTries;
int g_skip_it = -1;

}  // namespace

// The encoder driver registers its status word here around a pass: a tensor-core kernel whose bounded wait
// expires sets bit 2 of it (besides the flag behind fb_tc_error_flag).
void tc_set_status_sink(int* status) { t_status_sink = status; }
void tc_set_live_rows(const LiveRows* lr) {
  if (lr != nullptr) t_live_rows = *lr;
  else t_live_rows.L = 0;
}
int* tc_status_sink() { return t_status_sink; }

// Whether the bias rows [Mb, K] of a bound can ride in the grid of its weight rows: tensor-core shapes, and the
// same choice of zero radius on both sides when the weight rows take the zero-radius instantiation.
// FB_TC_SEPARATE_BIAS_ROWS=1 keeps them in a launch of their own (for comparisons).
bool tc_bias_rows_mergeable(const float* a_lo, const float* a_up, const float* b_lo, const float* b_up, const float* W,
                            const float* cb_lo, const float* cb_up, int64_t Mb, int N, int K, bool with_norms) {
  const char* e = std::getenv("FB_TC_SEPARATE_BIAS_ROWS");   // read per call, so that a test can compare the two forms
  const bool separate = e != nullptr && e[0] == '1';
  if (separate || Mb < 256 || Mb >= (1ll << 31)) return false;   // below 256 rows the bias terms take the CUDA-core kernel
  if (!aligned16(b_lo) || !aligned16(b_up) || !aligned16(cb_lo) || !aligned16(cb_up) || !aligned16(W)) return false;
  if (N < 32 || N % 4 != 0 || K < 8 || K % 4 != 0) return false;
  if (with_norms && (a_lo == a_up) != (b_lo == b_up)) return false;
  return true;
}

// Head-split store is possible when a 128-row tile stays inside one group and a 32-column box inside one head.
bool tc_split_supported(int64_t M, int N, int split_rows, int split_d) {
  return split_rows > 0 && split_d > 0 && split_rows % BM == 0 && M % split_rows == 0 && split_d % 32 == 0 &&
         N % split_d == 0;
}

bool tc_gemm_supported(const float* a_lo, const float* a_up, const float* W, const float* c_lo, const float* c_up,
                       int64_t M, int N, int K) {
  // the kernel counts tiles and k-blocks in 32 bits
  const int64_t k_blocks = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * ((K + BK - 1) / BK);
  return M >= 256 && M < (1ll << 31) && k_blocks < (1ll << 31) && N >= 32 && N % 4 == 0 && K >= 8 && K % 4 == 0 && aligned16(a_lo) &&
         aligned16(a_up) && aligned16(W) && aligned16(c_lo) && aligned16(c_up) && encode_fn() != nullptr;
}

int launch_split_sign_tc(const float* a_lo, const float* a_up, const float* W, const float* bias, float* c_lo,
                         float* c_up, int64_t M, int N, int K, cudaStream_t st, int split_rows, int split_d,
                         const float* coef_l, const float* coef_u, int coef_di, float* norm_lo, float* norm_up,
                         int norm_p, const float* res_lo, const float* res_up, const TcBiasRows* br, const TcLnArgs* ln) {
  // Bias rows in the same grid (br != nullptr): they must take the same instantiation as the weight rows (zero
  // radius or not, residual or not); the caller checks tc_bias_rows_mergeable first.
  if (br != nullptr && ((br->res_lo != nullptr) != (res_lo != nullptr) || (br->res_lo != nullptr) != (br->res_up != nullptr) ||
                        ((br->a_lo == br->a_up) != (a_lo == a_up) && norm_lo != nullptr) || br->M <= 0))
    return FB_ERR_ARG;
  if (ln != nullptr && (br == nullptr || res_lo == nullptr || N != kLnN || K % (2 * BK) != 0 || K > kLnMaxK || M % BM != 0 ||
                        ln->gamma == nullptr || ln->beta == nullptr || ln->rs_in == nullptr ||
                        ln->rs_stride < M + br->M))
    return FB_ERR_ARG;
  if (norm_lo != nullptr && (coef_l != nullptr || norm_up == nullptr || M % BM != 0)) return FB_ERR_ARG;
  if (res_lo != nullptr && (res_up == nullptr || norm_lo != nullptr || split_rows > 0 || !aligned16(res_lo) || !aligned16(res_up)))
    return FB_ERR_ARG;
  CUtensorMap tm_lo, tm_up, tm_w, tm_out_lo, tm_out_up, tm_res_lo, tm_res_up;
  if (!make_map(&tm_lo, a_lo, (uint64_t)M, (uint64_t)K, BM) || !make_map(&tm_up, a_up, (uint64_t)M, (uint64_t)K, BM) ||
      !make_map(&tm_w, W, (uint64_t)N, (uint64_t)K, BN) ||
      !make_out_map(&tm_out_lo, c_lo, (uint64_t)M, (uint64_t)N, split_rows, split_d) ||
      !make_out_map(&tm_out_up, c_up, (uint64_t)M, (uint64_t)N, split_rows, split_d))
    return FB_ERR_CUDA;
  // the residual maps are only read by the kResid instantiations; elsewhere they are copies of the output maps
  tm_res_lo = tm_out_lo;
  tm_res_up = tm_out_up;
  if (res_lo != nullptr && (!make_out_map(&tm_res_lo, res_lo, (uint64_t)M, (uint64_t)N, 0, 0) ||
                            !make_out_map(&tm_res_up, res_up, (uint64_t)M, (uint64_t)N, 0, 0)))
    return FB_ERR_CUDA;
  const int64_t gm = ceil_div(M, BM);
  const int gn = (int)ceil_div(N, BN);
  const int64_t main_tiles = gm * gn;
  // the maps of the bias rows are only read for tiles beyond main_tiles; without such tiles they are copies
  CUtensorMap tm_b_lo = tm_lo, tm_b_up = tm_up, tm_bout_lo = tm_out_lo, tm_bout_up = tm_out_up, tm_bres_lo = tm_res_lo,
              tm_bres_up = tm_res_up;
  int64_t total_tiles = main_tiles;
  if (br != nullptr) {
    if (!make_map(&tm_b_lo, br->a_lo, (uint64_t)br->M, (uint64_t)K, BM) || !make_map(&tm_b_up, br->a_up, (uint64_t)br->M, (uint64_t)K, BM) ||
        !make_out_map(&tm_bout_lo, br->c_lo, (uint64_t)br->M, (uint64_t)N, 0, 0) ||
        !make_out_map(&tm_bout_up, br->c_up, (uint64_t)br->M, (uint64_t)N, 0, 0))
      return FB_ERR_CUDA;
    tm_bres_lo = tm_bout_lo;
    tm_bres_up = tm_bout_up;
    if (br->res_lo != nullptr && (!make_out_map(&tm_bres_lo, br->res_lo, (uint64_t)br->M, (uint64_t)N, 0, 0) ||
                                  !make_out_map(&tm_bres_up, br->res_up, (uint64_t)br->M, (uint64_t)N, 0, 0)))
      return FB_ERR_CUDA;
    total_tiles += ceil_div(br->M, BM) * gn;
    if (total_tiles * ((K + BK - 1) / BK) >= (1ll << 31)) return FB_ERR_SHAPE;
  }
  const float* bias_b = br != nullptr ? br->bias : nullptr;
  const int same_b = (br != nullptr && br->c_lo == br->c_up) ? 1 : 0;
  static std::once_flag attr_once[64];
  int dev = 0;
  FB_CUDA_OK(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once[dev & 63], [&]() {
    const int bytes = (int)kSmemBytes;
    attr_err = cudaFuncSetAttribute(split_sign_gemm_tc<false, false, false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(split_sign_gemm_tc<true, false, false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(split_sign_gemm_tc<false, true, false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(split_sign_gemm_tc<false, false, true, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(split_sign_gemm_tc<true, false, true, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(split_sign_gemm_tc<false, true, false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    const int ln_bytes = (int)(kSmemBytes + kLnSmemBytes);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(split_sign_gemm_tc<false, false, true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ln_bytes);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(split_sign_gemm_tc<true, false, true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ln_bytes);
  });
  FB_CUDA_OK(attr_err);
  // persistent: one CTA per SM (tensor memory and shared memory allow exactly one)
  const int64_t sms = device_info().sms;
  const unsigned grid = (unsigned)(total_tiles < sms ? total_tiles : sms);
  int* status = t_status_sink;
  const uint32_t tries = g_wait_tries;
  const int skip = g_skip_it;
  // zero row blocks: only for the zero-radius products of the operand the hint was set for (weight rows, no bias)
  LiveRows no_live = {0, 0, 0, {0, 0, 0, 0}, nullptr, 0};
  LiveRows live = no_live;
  if (t_live_rows.L > 0 && t_live_rows.M == M && bias == nullptr && t_live_rows.Di > 0 && t_live_rows.Di % BM == 0 &&
      t_live_rows.words >= 1 && t_live_rows.words <= 4 && M % ((int64_t)t_live_rows.Di * t_live_rows.L) == 0)
    live = t_live_rows;
  TcLnArgs ln_args = {nullptr, nullptr, nullptr, nullptr, nullptr, 0};
  if (ln != nullptr) {
    ln_args = *ln;
    ln_args.w_raw = W;
  }
  const int64_t Mb = br != nullptr ? br->M : 0;
#define FB_TC_TAIL ln_args, Mb
#define FB_TC_ARGS tm_lo, tm_up, tm_w, tm_out_lo, tm_out_up, tm_res_lo, tm_res_up, tm_b_lo, tm_b_up, tm_bout_lo, tm_bout_up, tm_bres_lo, \
                   tm_bres_up, bias, bias_b, (int)main_tiles, same_b, M, N, K, gn, total_tiles, split_rows, split_d
  if (ln != nullptr && coef_l != nullptr)
    split_sign_gemm_tc<true, false, true, false, true><<<grid, kThreads, kSmemBytes + kLnSmemBytes, st>>>(FB_TC_ARGS, coef_l, coef_u, coef_di, nullptr, nullptr, 0, status, tries, skip, no_live, 0, FB_TC_TAIL);
  else if (ln != nullptr)
    split_sign_gemm_tc<false, false, true, false, true><<<grid, kThreads, kSmemBytes + kLnSmemBytes, st>>>(FB_TC_ARGS, nullptr, nullptr, 1, nullptr, nullptr, 0, status, tries, skip, no_live, 0, FB_TC_TAIL);
  else if (coef_l != nullptr && res_lo != nullptr)
    split_sign_gemm_tc<true, false, true, false, false><<<grid, kThreads, kSmemBytes, st>>>(FB_TC_ARGS, coef_l, coef_u, coef_di, nullptr, nullptr, 0, status, tries, skip, no_live, 0, FB_TC_TAIL);
  else if (coef_l != nullptr)
    split_sign_gemm_tc<true, false, false, false, false><<<grid, kThreads, kSmemBytes, st>>>(FB_TC_ARGS, coef_l, coef_u, coef_di, nullptr, nullptr, 0, status, tries, skip, no_live, 0, FB_TC_TAIL);
  else if (norm_lo != nullptr && a_lo == a_up)   // one tensor as both lines: zero radius
    split_sign_gemm_tc<false, true, false, true, false><<<grid, kThreads, kSmemBytes, st>>>(FB_TC_ARGS, nullptr, nullptr, 1, norm_lo, norm_up, norm_p, status, tries, skip, live, c_lo == c_up ? 1 : 0, FB_TC_TAIL);
  else if (norm_lo != nullptr)
    split_sign_gemm_tc<false, true, false, false, false><<<grid, kThreads, kSmemBytes, st>>>(FB_TC_ARGS, nullptr, nullptr, 1, norm_lo, norm_up, norm_p, status, tries, skip, no_live, 0, FB_TC_TAIL);
  else if (res_lo != nullptr)
    split_sign_gemm_tc<false, false, true, false, false><<<grid, kThreads, kSmemBytes, st>>>(FB_TC_ARGS, nullptr, nullptr, 1, nullptr, nullptr, 0, status, tries, skip, no_live, 0, FB_TC_TAIL);
  else
    split_sign_gemm_tc<false, false, false, false, false><<<grid, kThreads, kSmemBytes, st>>>(FB_TC_ARGS, nullptr, nullptr, 1, nullptr, nullptr, 0, status, tries, skip, no_live, 0, FB_TC_TAIL);
#undef FB_TC_ARGS
#undef FB_TC_TAIL
  FB_LAUNCH_OK();
  return FB_OK;
}

}  // namespace fb


// Reads (and clears) the device-side flag that the tensor-core kernels raise when one of their bounded
// waits expires.  Synchronises the device.
namespace fb { int dot_tc_error_flag(int* flag); }

extern "C" int fb_tc_error_flag(int* flag) {
  if (!flag) return FB_ERR_ARG;
  int v = 0;
  FB_CUDA_OK(cudaDeviceSynchronize());
  FB_CUDA_OK(cudaMemcpyFromSymbol(&v, fb::g_tc_error, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    FB_CUDA_OK(cudaMemcpyToSymbol(fb::g_tc_error, &zero, sizeof(int)));
  }
  int v2 = 0;
  const int rc = fb::dot_tc_error_flag(&v2);   // the tensor-core dot product keeps a flag of its own
  if (rc != FB_OK) return rc;
  *flag = (v != 0 || v2 != 0) ? 1 : 0;
  return FB_OK;
}

// ------------------------------------------------------------------------------------------------
// Measurement aid: the rate of the tensor pipe for kind::tf32, the roof of the 3xTF32 kernels above.  Every SM runs
// one CTA whose single issuing thread feeds 128 x 256 x 8 MMAs (operands in shared memory, two accumulators of 256
// columns alternating so that consecutive instructions do not depend on each other) as fast as the pipe takes them.
namespace fb {
namespace {
constexpr uint32_t kPeakSmem = 48 * 1024 + 1024 + 64;   // A 128 x 32, B 256 x 32 fp32 (128-byte rows, swizzled), barrier
constexpr uint32_t kPeakIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(0u)
      : "memory");
}

__global__ void __launch_bounds__(128, 1) tf32_peak_kernel(int iters, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar = base + 48 * 1024;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + 48 * 1024 + 16);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(base_ptr + 48 * 1024 + 24);
  for (uint32_t i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) reinterpret_cast<float*>(base_ptr)[i] = 0.f;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    *cta_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 32) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  fence_async_smem();   // the zero fill went through the generic proxy; the MMAs read through the async proxy
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (threadIdx.x == 0) {
    const uint64_t ad = smem_desc_sw128(base), bd = smem_desc_sw128(base + 16 * 1024);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {   // four k steps of a 32-wide tile, two accumulators
        mma_tf32_ss(tmem, ad + 2 * j, bd + 2 * j, kPeakIdesc, 1u);
        mma_tf32_ss(tmem + 256, ad + 2 * j, bd + 2 * j, kPeakIdesc, 1u);
      }
    }
    tc_commit(bar);
    const WaitCtx wc = {cta_abort, kMaxTries};
    if (!mbar_wait(bar, 0, wc) && status != nullptr) atomicOr(status, 4);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}
}  // namespace
}  // namespace fb

extern "C" int fb_bench_tf32(int iters, double* flops, void* stream) {
  if (iters <= 0 || !flops) return FB_ERR_ARG;
  static std::once_flag once[64];
  int dev = 0;
  FB_CUDA_OK(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[dev & 63], [&]() {
    attr_err = cudaFuncSetAttribute(fb::tf32_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fb::kPeakSmem);
  });
  FB_CUDA_OK(attr_err);
  const int blocks = fb::device_info().sms;
  fb::tf32_peak_kernel<<<blocks, 128, fb::kPeakSmem, (cudaStream_t)stream>>>(iters, fb::t_status_sink);
  FB_LAUNCH_OK();
  *flops = 2.0 * 128.0 * 256.0 * 8.0 * 8.0 * (double)iters * blocks;
  return FB_OK;
}

extern "C" int fb_tc_check(void) {
  int flag = 0;
  const int rc = fb_tc_error_flag(&flag);
  if (rc != FB_OK) return rc;
  return flag ? FB_ERR_TIMEOUT : FB_OK;
}

// Self-test of the give-up path: runs the product once with the loads of one k-block of CTA 0 left out and every
// wait limited to `tries` tries of ~20 us.  The CTA's converters run out of patience, the CTA drains, frees its tensor
// memory and returns; the call then reports FB_ERR_TIMEOUT (anything else means the path is broken).  Results of this
// call are garbage by construction.  Not thread-safe against concurrent products (process-wide switches).
extern "C" int fb_tc_selftest_timeout(const float* x_lw, const float* x_uw, const float* W, float* y_lw, float* y_uw,
                                      int64_t M, int N, int K, int skip_kblock, int tries, int* status, void* stream) {
  if (!x_lw || !x_uw || !W || !y_lw || !y_uw || skip_kblock < 0 || tries <= 0) return FB_ERR_ARG;
  if (!fb::tc_gemm_supported(x_lw, x_uw, W, y_lw, y_uw, M, N, K)) return FB_ERR_SHAPE;
  int flag = 0;
  int rc = fb_tc_error_flag(&flag);   // start from a clean flag
  if (rc != FB_OK) return rc;
  fb::g_wait_tries = (uint32_t)tries;
  fb::g_skip_it = skip_kblock;
  int* const saved_sink = fb::t_status_sink;
  fb::t_status_sink = status;
  rc = fb::launch_split_sign_tc(x_lw, x_uw, W, nullptr, y_lw, y_uw, M, N, K, (cudaStream_t)stream, 0, 0, nullptr, nullptr, 1,
                                nullptr, nullptr, 0, nullptr, nullptr, nullptr, nullptr);
  fb::t_status_sink = saved_sink;
  fb::g_wait_tries = fb::kMaxTries;
  fb::g_skip_it = -1;
  if (rc != FB_OK) return rc;
  return fb_tc_check();
}
