// Weight part of the bound x bound dot product on the 5th-generation tensor cores (tcgen05 / TMEM),
// fp32-accurate through the 3xTF32 split, for the attention shapes (K = 32, Ly = 32, Lx a multiple
// of 32, Di a multiple of 4, native layout).  Other shapes stay on the CUDA-core kernels.
//
//   z_lw[b,i,m,j] = sum_k  x_c ly - x_r |ly| + y_c lx - y_r |lx|          (Bounds.py:710-823 in
//   z_uw[b,i,m,j] = sum_k  x_c uy + x_r |uy| + y_c lx + y_r |lx|           centre/radius form)
//   x_c = (x_lw + x_uw)/2, x_r = (x_uw - x_lw)/2 at [b,i,m,k];  y_c, y_r at [b,j,m,k];
//   lx = x_l[b,i,k];  ly = y_l[b,j,k], uy = y_u[b,j,k]  (concretised operand ranges)
// With y_kmajor the weights of y are given as [b,k,m,j] (contraction axis first), which is how the
// value projection writes them: the context product then needs no transposed copy of V.
//
// One tile = one b, 32 values of i, 4 values of m, all 32 values of j.  It is made of four GEMMs with
// M = 128, K = 32:
//   X_c [128 x 64] = x_c[(i,m), k] * [ly; uy][j, k]^T        rows (i,m), columns j (lower) and 32+j (upper)
//   X_r [128 x 64] = x_r[(i,m), k] * [|ly|; |uy|][j, k]^T
//   P   [128 x 32] = y_c[(j,m), k] * lx[i, k]^T               rows (j,m), columns i
//   Q   [128 x 32] = y_r[(j,m), k] * |lx|[i, k]^T
// and z_lw = X_c[:, j] - X_r[:, j] + (P - Q)^T,  z_uw = X_c[:, 32+j] + X_r[:, 32+j] + (P + Q)^T, where
// the transposition (j,m),i -> (i,m),j goes through shared memory in the epilogue.
//
// Every product is evaluated as hi*hi + hi*lo + lo*hi on TF32 parts (hi = 13 low mantissa bits
// cleared, lo = v - hi); the two small products are issued first, so that only four MMAs add to an
// accumulator of full magnitude (the tensor core truncates when it adds to the accumulator).
// The A operands (x_c, x_r, y_c, y_r, hi and lo: eight planes of 32 columns) live in tensor memory, the
// B operands in shared memory: the raw range tiles as loaded by TMA serve as the hi planes (the
// tensor core reads the leading 19 bits of an fp32 word), the lo and absolute-value planes are written
// by the converter warps.
//
// Warp roles (24 warps, one persistent CTA per SM):
//   warp 0       TMA producer (two raw stages) and MMA issuer of Q
//   warps 1-3    MMA issuers of X_c, X_r, P (12 MMAs per tile each; one accumulator per issuer)
//   warps 4-7    epilogue, one warp per tensor-memory lane quarter
//   warps 8-15   converters of the x tile, warps 16-23 converters of the y tile
// TMEM columns: [0,64) X_c, [64,128) X_r, [128,160) P, [160,192) Q, [256,512) the eight A planes.
// Every mbarrier wait is bounded; on expiry the kernel raises a device-side flag, drains, frees its
// tensor memory and returns.  No cluster launch and no multicast is used.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace fb {
namespace {

#include "tc_common.cuh"

constexpr int kDtThreads = 768;
constexpr int kDtConvWarps = 16, kDtEpiWarps = 4, kDtIssuers = 4;
constexpr int kDtFirstEpiWarp = 4, kDtFirstConvWarp = 8;
constexpr uint32_t kDtTile = 128 * 32 * 4;                 // one 128-row x 32-k fp32 tile = 16 KB
constexpr uint32_t kDtLY = 64 * 32 * 4, kDtLX = 32 * 32 * 4;   // [ly; uy] and lx range tiles
// raw stage: x_lw, x_uw, y_lw, y_uw tiles, then [ly; uy], then lx
constexpr uint32_t kDtRawXl = 0, kDtRawXu = kDtTile, kDtRawYl = 2 * kDtTile, kDtRawYu = 3 * kDtTile;
constexpr uint32_t kDtRawLY = 4 * kDtTile, kDtRawLX = 4 * kDtTile + kDtLY;
constexpr uint32_t kDtRawStage = 4 * kDtTile + kDtLY + kDtLX;   // 76 KB
// planes written by the converters: LY_lo, |LY|_hi, |LY|_lo, LX_lo, |LX|_hi, |LX|_lo
constexpr uint32_t kDtPlLYlo = 0, kDtPlALYhi = kDtLY, kDtPlALYlo = 2 * kDtLY;
constexpr uint32_t kDtPlLXlo = 3 * kDtLY, kDtPlALXhi = 3 * kDtLY + kDtLX, kDtPlALXlo = 3 * kDtLY + 2 * kDtLX;
constexpr uint32_t kDtPlanes = 3 * kDtLY + 3 * kDtLX;            // 36 KB
constexpr int kDtTStride = 36;                                   // floats per row of the transposition buffer
constexpr uint32_t kDtTBytes = 128 * kDtTStride * 4;             // 18 KB per side (lower / upper); aliases the 16 KB store staging
constexpr uint32_t kDtOffPlanes = 2 * kDtRawStage, kDtOffT = kDtOffPlanes + kDtPlanes, kDtOffBars = kDtOffT + 2 * kDtTBytes;
constexpr uint32_t kDtSmemBytes = kDtOffBars + 1024 /*align*/ + 256 /*barriers*/;
static_assert(kDtSmemBytes <= 232448, "shared memory budget");
constexpr uint32_t kDtXc = 0, kDtXr = 64, kDtP = 128, kDtQ = 160, kDtA = 256;   // TMEM column map
constexpr uint32_t kDtIdesc64 = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
constexpr uint32_t kDtIdesc32 = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(32 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

// The 12 MMAs of one accumulator: A planes at a_hi / a_lo (TMEM columns), B planes by descriptor
// (low words; the high word is common).  Small products first, the first MMA overwrites.
__device__ __forceinline__ void issue_product(uint32_t d, uint32_t a_hi, uint32_t a_lo, uint32_t b_hi_lo32,
                                              uint32_t b_lo_lo32, uint32_t desc_hi32, uint32_t idesc) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j == 0) mma_tf32_ts_lean<false>(d, a_lo + 8 * j, b_hi_lo32 + 2 * j, desc_hi32, idesc);
    else mma_tf32_ts_lean<true>(d, a_lo + 8 * j, b_hi_lo32 + 2 * j, desc_hi32, idesc);
    mma_tf32_ts_lean<true>(d, a_hi + 8 * j, b_lo_lo32 + 2 * j, desc_hi32, idesc);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) mma_tf32_ts_lean<true>(d, a_hi + 8 * j, b_hi_lo32 + 2 * j, desc_hi32, idesc);
}

__global__ void __launch_bounds__(kDtThreads, 1)
dot_weight_tc(const __grid_constant__ CUtensorMap tm_xl, const __grid_constant__ CUtensorMap tm_xu,
              const __grid_constant__ CUtensorMap tm_yl, const __grid_constant__ CUtensorMap tm_yu,
              const __grid_constant__ CUtensorMap tm_lx, const __grid_constant__ CUtensorMap tm_ly,
              const __grid_constant__ CUtensorMap tm_uy, const __grid_constant__ CUtensorMap tm_zl,
              const __grid_constant__ CUtensorMap tm_zu, int Lx, int Ly, int n_ib, int n_mb, int total_tiles,
              float out_scale, int heads, int y_kmajor, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar0 = base + kDtOffBars;
  const uint32_t bar_full = bar0 + 0;          // [2] raw stage loaded
  const uint32_t bar_raw_empty = bar0 + 16;    // [2] raw x/y tiles and range tiles read by the converters
  const uint32_t bar_ops_ready = bar0 + 32;    // operands of the tile converted
  const uint32_t bar_mma_done = bar0 + 40;     // all MMAs of the tile complete (operands free, accumulators ready)
  const uint32_t bar_acc_free = bar0 + 48;     // accumulators read out
  const uint32_t bar_epi = bar0 + 56;          // rendezvous of the epilogue warps
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kDtOffBars + 64);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(base_ptr + kDtOffBars + 72);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int my_tiles = (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_raw_empty + 8 * s, kDtConvWarps);
    }
    mbar_init(bar_ops_ready, kDtConvWarps);
    mbar_init(bar_mma_done, kDtIssuers);
    mbar_init(bar_acc_free, kDtEpiWarps);
    mbar_init(bar_epi, kDtEpiWarps);
    *cta_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // one warp allocates all of tensor memory for this CTA
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // coordinates of tile t of this CTA
  auto tile_coords = [&](int t, int& b, int& i0, int& m0) {
    const int tile = (int)blockIdx.x + t * (int)gridDim.x;
    const int mb = tile % n_mb, rest = tile / n_mb;
    m0 = mb * 4;
    i0 = (rest % n_ib) * 32;
    b = rest / n_ib;
  };

  if (warp < kDtIssuers) {
    // ------------------------------------------------------------------ MMA issuers; warp 0 also loads
    // role 0 (warp 0): Q = y_r |lx|;  1: X_c = x_c [ly;uy];  2: X_r = x_r [|ly|;|uy|];  3: P = y_c lx
    const int role = warp;
    bool ok = true;
    const uint64_t dsc = smem_desc_sw128(base);
    const uint32_t desc_hi32 = (uint32_t)(dsc >> 32), desc_lo0 = (uint32_t)dsc;   // descriptor of offset 0; + (bytes >> 4)
    const uint32_t a_base = tmem_base + kDtA;
    // per role: accumulator, A planes (hi, lo), B planes (hi: in the raw stage for roles 1 and 3, else in the planes)
    uint32_t d, a_hi, a_lo, b_lo_off, idesc;
    uint32_t b_hi_off[2];   // per raw stage
    if (role == 1) {
      d = tmem_base + kDtXc; a_hi = a_base + 0; a_lo = a_base + 32; idesc = kDtIdesc64;
      b_hi_off[0] = kDtRawLY; b_hi_off[1] = kDtRawStage + kDtRawLY; b_lo_off = kDtOffPlanes + kDtPlLYlo;
    } else if (role == 2) {
      d = tmem_base + kDtXr; a_hi = a_base + 64; a_lo = a_base + 96; idesc = kDtIdesc64;
      b_hi_off[0] = b_hi_off[1] = kDtOffPlanes + kDtPlALYhi; b_lo_off = kDtOffPlanes + kDtPlALYlo;
    } else if (role == 3) {
      d = tmem_base + kDtP; a_hi = a_base + 128; a_lo = a_base + 160; idesc = kDtIdesc32;
      b_hi_off[0] = kDtRawLX; b_hi_off[1] = kDtRawStage + kDtRawLX; b_lo_off = kDtOffPlanes + kDtPlLXlo;
    } else {
      d = tmem_base + kDtQ; a_hi = a_base + 192; a_lo = a_base + 224; idesc = kDtIdesc32;
      b_hi_off[0] = b_hi_off[1] = kDtOffPlanes + kDtPlALXhi; b_lo_off = kDtOffPlanes + kDtPlALXlo;
    }
    auto load_tile = [&](int t) {   // warp 0, lane 0
      int b, i0, m0;
      tile_coords(t, b, i0, m0);
      const int s = t & 1;
      const uint32_t full = bar_full + 8 * s, dst = base + s * kDtRawStage;
      mbar_arrive_expect_tx(full, kDtRawStage);
      tma_load_3d(dst + kDtRawXl, &tm_xl, 0, m0, b * Lx + i0, full);
      tma_load_3d(dst + kDtRawXu, &tm_xu, 0, m0, b * Lx + i0, full);
      tma_load_3d(dst + kDtRawYl, &tm_yl, 0, m0, b * Ly, full);
      tma_load_3d(dst + kDtRawYu, &tm_yu, 0, m0, b * Ly, full);
      tma_load_2d(dst + kDtRawLY, &tm_ly, 0, b * Ly, full);
      tma_load_2d(dst + kDtRawLY + kDtLX, &tm_uy, 0, b * Ly, full);
      tma_load_2d(dst + kDtRawLX, &tm_lx, 0, b * Lx + i0, full);
    };
    if (role == 0 && my_tiles > 0) {
      if (lane == 0) load_tile(0);
      __syncwarp();
    }
    for (int t = 0; t < my_tiles && ok; ++t) {
      if (role == 0 && t + 1 < my_tiles) {
        // The stage of tile t+1 was used by tile t-1: its x/y tiles have been read by the converters
        // and its range tiles by the MMAs of tile t-1.
        if (t >= 1) {
          ok = mbar_wait_warp(bar_raw_empty + 8 * ((t + 1) & 1), (uint32_t)(((t - 1) >> 1) & 1), cta_abort);
          if (ok) ok = mbar_wait_warp(bar_mma_done, (uint32_t)((t - 1) & 1), cta_abort);
          if (!ok) break;
        }
        if (lane == 0) load_tile(t + 1);
        __syncwarp();
      }
      ok = mbar_wait_warp(bar_ops_ready, (uint32_t)(t & 1), cta_abort);
      // the first MMA of a tile overwrites the accumulators: the previous tile must have been read out
      if (ok && t > 0) ok = mbar_wait_warp(bar_acc_free, (uint32_t)((t - 1) & 1), cta_abort);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        issue_product(d, a_hi, a_lo, desc_lo0 + (b_hi_off[t & 1] >> 4), desc_lo0 + (b_lo_off >> 4), desc_hi32, idesc);
        tc_commit(bar_mma_done);
      }
      __syncwarp();
    }
  } else if (warp < kDtFirstConvWarp) {
    // ------------------------------------------------------------------ epilogue (warps 4-7)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;            // TMEM lane = accumulator row
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const bool leader = threadIdx.x == 32 * kDtFirstEpiWarp;
    float* T = reinterpret_cast<float*>(base_ptr + kDtOffT);   // [2][128][kDtTStride]
    bool ok = true;
    uint32_t epi_phase = 0;
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_epi);
      const bool r = mbar_wait_warp(bar_epi, epi_phase & 1u, cta_abort);
      ++epi_phase;
      return r;
    };
    for (int t = 0; t < my_tiles && ok; ++t) {
      ok = mbar_wait_warp(bar_mma_done, (uint32_t)(t & 1), cta_abort);
      if (!ok) break;
      tc_fence_after();
      int b, i0, m0;
      tile_coords(t, b, i0, m0);
      if (leader) tma_store_wait_read();      // the previous tile's stores have read the staging buffer
      ok = epi_sync();
      if (!ok) break;
      // ---- P -/+ Q of row (j, m), columns i  ->  T[side][(i, m)][j]
      {
        const int j = row >> 2, m = row & 3;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t tp[16], tq[16];
          tmem_ld16(tmem_base + lane_addr + kDtP + 16 * h, tp);
          tmem_ld16(tmem_base + lane_addr + kDtQ + 16 * h, tq);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const uint64_t pv = pack2(tp[i], tp[i + 1]), qv = pack2(tq[i], tq[i + 1]);
            const uint64_t d = sub2(pv, qv), a = add2(pv, qv);
            const int r = (16 * h + i) * 4 + m;
            T[r * kDtTStride + j] = __uint_as_float((uint32_t)d);
            T[(r + 4) * kDtTStride + j] = __uint_as_float((uint32_t)(d >> 32));
            T[128 * kDtTStride + r * kDtTStride + j] = __uint_as_float((uint32_t)a);
            T[128 * kDtTStride + (r + 4) * kDtTStride + j] = __uint_as_float((uint32_t)(a >> 32));
          }
        }
      }
      ok = epi_sync();
      if (!ok) break;
      // ---- X_c -/+ X_r of row (i, m), columns j, plus the transposed term; lower side, then upper side.
      // The store staging of a side takes the place of that side's transposition buffer, so it is
      // written only after every thread has read its row of the buffer.
#pragma unroll
      for (int side = 0; side < 2; ++side) {
        uint64_t z2[16];
        const uint64_t scale2 = pack2(__float_as_uint(out_scale), __float_as_uint(out_scale));
        const float* Ts = T + side * 128 * kDtTStride + row * kDtTStride;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t cc[16], rr[16];
          tmem_ld16(tmem_base + lane_addr + kDtXc + 32 * side + 16 * h, cc);
          tmem_ld16(tmem_base + lane_addr + kDtXr + 32 * side + 16 * h, rr);
          tmem_wait_ld();
          if (side == 1 && h == 1) {
            // the accumulators are in registers now: hand tensor memory back to the MMA issuers
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_free);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const ulonglong2 tv = *reinterpret_cast<const ulonglong2*>(Ts + 16 * h + 4 * q);
            const uint64_t t2[2] = {tv.x, tv.y};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int i = 4 * q + 2 * e;
              const uint64_t cv = pack2(cc[i], cc[i + 1]), rv = pack2(rr[i], rr[i + 1]);
              const uint64_t xv = side == 0 ? sub2(cv, rv) : add2(cv, rv);
              z2[(16 * h + i) >> 1] = mul2(add2(xv, t2[e]), scale2);
            }
          }
        }
        ok = epi_sync();
        if (!ok) break;
        uint8_t* so = base_ptr + kDtOffT + side * kDtTBytes;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<ulonglong2*>(so + swz(row, q)) = make_ulonglong2(z2[2 * q], z2[2 * q + 1]);
      }
      if (!ok) break;
      fence_async_smem();
      ok = epi_sync();
      if (!ok) break;
      if (leader) {
        // output [S, Lx, Di, heads * Ly] with b = s * heads + h: box (32 j, 4 m, 32 i) at (h * Ly, m0, s * Lx + i0)
        const int sb = b / heads, hb = b % heads;
        tma_store_3d(&tm_zl, hb * Ly, m0, sb * Lx + i0, base + kDtOffT);
        tma_store_3d(&tm_zu, hb * Ly, m0, sb * Lx + i0, base + kDtOffT + kDtTBytes);
        tma_store_commit();
      }
    }
  } else {
    // ------------------------------------------------------------------ converters
    const int cw = warp - kDtFirstConvWarp;   // 0..15
    const int grp = cw >> 3;                   // 0: x tile, 1: y tile
    const int gt = (threadIdx.x - 32 * kDtFirstConvWarp) & 255;
    const int quarter = warp & 3;
    const int half = (cw >> 2) & 1;            // which 16 of the 32 k values
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    bool ok = true;
    for (int t = 0; t < my_tiles && ok; ++t) {
      const int s = t & 1;
      ok = mbar_wait_warp(bar_full + 8 * s, (uint32_t)((t >> 1) & 1), cta_abort);
      if (!ok) break;
      const uint8_t* raw = base_ptr + s * kDtRawStage;
      const uint8_t* tl = raw + (grp == 0 ? kDtRawXl : kDtRawYl);
      const uint8_t* tu = raw + (grp == 0 ? kDtRawXu : kDtRawYu);
      // (arithmetic on pairs of fp32 values, fma / mul / sub .f32x2: each half rounded as the scalar instruction rounds it)
      uint64_t c2[8], r2[8];
      if (grp == 1 && y_kmajor) {
        // y given as [b, k, m, j] (the value tensor as the projection writes it): the tile is
        // [k][m][j]; this thread's row (j, m) is gathered element by element
        const int j = row >> 2, m = row & 3;
#pragma unroll
        for (int kk = 0; kk < 16; kk += 2) {
          const int k = half * 16 + kk;
          const uint32_t off0 = swz(k * 4 + m, j >> 2) + (uint32_t)(j & 3) * 4u;
          const uint32_t off1 = swz((k + 1) * 4 + m, j >> 2) + (uint32_t)(j & 3) * 4u;
          const uint64_t lo = pack2(*reinterpret_cast<const uint32_t*>(tl + off0), *reinterpret_cast<const uint32_t*>(tl + off1));
          const uint64_t up = pack2(*reinterpret_cast<const uint32_t*>(tu + off0), *reinterpret_cast<const uint32_t*>(tu + off1));
          const uint64_t hu = mul2(up, kHalf2);
          c2[kk >> 1] = fma2(lo, kHalf2, hu);
          r2[kk >> 1] = fma2(lo, kMinusHalf2, hu);
        }
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t off = swz(row, half * 4 + q);
          const ulonglong2 vl = *reinterpret_cast<const ulonglong2*>(tl + off);
          const ulonglong2 vu = *reinterpret_cast<const ulonglong2*>(tu + off);
          const uint64_t l2[2] = {vl.x, vl.y}, u2[2] = {vu.x, vu.y};
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const uint64_t hu = mul2(u2[i], kHalf2);
            c2[q * 2 + i] = fma2(l2[i], kHalf2, hu);
            r2[q * 2 + i] = fma2(l2[i], kMinusHalf2, hu);
          }
        }
      }
      // range tiles: group 0 converts [ly; uy] (64 rows x 8 chunks, two chunks per thread), group 1 lx
      // (32 rows x 8 chunks, one chunk per thread)
      const int nch = grp == 0 ? 2 : 1;
      const uint8_t* rsrc = raw + (grp == 0 ? kDtRawLY : kDtRawLX);
      uint32_t blo[8], bah[8], bal[8];
      uint32_t roff[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int id = gt * nch + q;
        roff[q] = swz(id >> 3, id & 7);
        if (q < nch) {
          const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(rsrc + roff[q]);
          const uint64_t v2[2] = {v.x, v.y};
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            uint64_t hi, lo;
            split_tf32_pair(v2[i], hi, lo);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const uint32_t h = (uint32_t)(hi >> (32 * e)), l = (uint32_t)(lo >> (32 * e));
              blo[q * 4 + 2 * i + e] = l;
              bah[q * 4 + 2 * i + e] = h & 0x7fffffffu;    // |v| = sgn(v) (hi + lo); hi and lo carry the sign of v
              bal[q * 4 + 2 * i + e] = l & 0x7fffffffu;
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) blo[q * 4 + i] = bah[q * 4 + i] = bal[q * 4 + i] = 0u;
        }
      }
      // The raw stage goes back to the producer only when every value loaded from it has been used
      // (a shared-memory load completes asynchronously); the empty asm statements keep the arithmetic
      // above from being moved below the arrive.
#pragma unroll
      for (int i = 0; i < 8; ++i) asm volatile("" : "+l"(c2[i]), "+l"(r2[i]));
#pragma unroll
      for (int i = 0; i < 8; ++i) asm volatile("" : "+r"(blo[i]), "+r"(bah[i]), "+r"(bal[i]));
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_raw_empty + 8 * s);
      if (t >= 1) {
        // tensor memory planes and shared-memory planes are still read by the MMAs of tile t-1
        ok = mbar_wait_warp(bar_mma_done, (uint32_t)((t - 1) & 1), cta_abort);
        if (!ok) break;
        tc_fence_after();
      }
      {
        const uint32_t a_cols = tmem_base + lane_addr + kDtA + (uint32_t)grp * 128u + (uint32_t)half * 16u;
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
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint64_t h2, l2;
          split_tf32_pair(r2[i], h2, l2);
          hi[2 * i] = (uint32_t)h2; hi[2 * i + 1] = (uint32_t)(h2 >> 32);
          lo[2 * i] = (uint32_t)l2; lo[2 * i + 1] = (uint32_t)(l2 >> 32);
        }
        tmem_st16(a_cols + 64, hi);
        tmem_st16(a_cols + 96, lo);
        uint8_t* pl = base_ptr + kDtOffPlanes;
        const uint32_t o_lo = grp == 0 ? kDtPlLYlo : kDtPlLXlo, o_ah = grp == 0 ? kDtPlALYhi : kDtPlALXhi,
                       o_al = grp == 0 ? kDtPlALYlo : kDtPlALXlo;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          if (q < nch) {
            *reinterpret_cast<uint4*>(pl + o_lo + roff[q]) = make_uint4(blo[q * 4], blo[q * 4 + 1], blo[q * 4 + 2], blo[q * 4 + 3]);
            *reinterpret_cast<uint4*>(pl + o_ah + roff[q]) = make_uint4(bah[q * 4], bah[q * 4 + 1], bah[q * 4 + 2], bah[q * 4 + 3]);
            *reinterpret_cast<uint4*>(pl + o_al + roff[q]) = make_uint4(bal[q * 4], bal[q * 4 + 1], bal[q * 4 + 2], bal[q * 4 + 3]);
          }
        }
      }
      fence_async_smem();   // planes were written through the generic proxy; the MMA reads them through the async proxy
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ops_ready);
    }
  }
  if (threadIdx.x == 32 * kDtFirstEpiWarp) tma_store_wait_all();   // this thread issued the bulk stores
  // Tear-down.  On the error path, give outstanding bulk copies time to land before the shared
  // memory is released (bounded), then free the tensor memory.
  if (*cta_abort) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status != nullptr) atomicOr(status, 4);   // bit 2 of the caller's status word
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------ host side

// 3-D fp32 tensor [d2][d1][d0] (d0 contiguous), box 32 x 4 x 32 (d0 x d1 x d2), 128-byte swizzle, zero fill.
bool make_map3(CUtensorMap* map, const float* ptr, uint64_t d0, uint64_t d1, uint64_t d2) {
  return get_map(map, ptr, 3, d0, d1, d2, d0 * sizeof(float), d0 * d1 * sizeof(float), 32, 4, 32);
}
// 2-D fp32 row-major [rows, 32], box 32 rows x 32 columns, 128-byte swizzle.
bool make_map2(CUtensorMap* map, const float* ptr, uint64_t rows) {
  return get_map(map, ptr, 2, 32, rows, 1, 32 * sizeof(float), 0, 32, 32);
}

}  // namespace

// Shapes the tensor-core dot product covers: the attention products of the forward verifier.
bool dot_tc_supported(const float* x_lw, const float* x_uw, const float* y_lw, const float* y_uw, const float* x_l,
                      const float* y_l, const float* y_u, const float* z_lw, const float* z_uw, int B, int Lx, int Ly,
                      int Di, int K, int heads) {
  if (K != 32 || Ly != 32 || Lx % 32 != 0 || Di % 4 != 0 || B < 1 || heads < 1 || B % heads != 0) return false;
  const int64_t tiles = (int64_t)B * (Lx / 32) * (Di / 4);
  if (tiles >= (1ll << 31) || (int64_t)B * Lx >= (1ll << 31)) return false;
  return aligned16(x_lw) && aligned16(x_uw) && aligned16(y_lw) && aligned16(y_uw) && aligned16(x_l) && aligned16(y_l) &&
         aligned16(y_u) && aligned16(z_lw) && aligned16(z_uw) && encode_fn() != nullptr;
}

int* tc_status_sink();

int launch_dot_weight_tc(const float* x_lw, const float* x_uw, const float* y_lw, const float* y_uw, const float* x_l,
                         const float* y_l, const float* y_u, float* z_lw, float* z_uw, int B, int Lx, int Ly, int Di,
                         float out_scale, int heads, int y_kmajor, cudaStream_t st) {
  CUtensorMap tm_xl, tm_xu, tm_yl, tm_yu, tm_lx, tm_ly, tm_uy, tm_zl, tm_zu;
  const uint64_t S = (uint64_t)(B / heads);
  if (!make_map3(&tm_xl, x_lw, 32, (uint64_t)Di, (uint64_t)B * Lx) || !make_map3(&tm_xu, x_uw, 32, (uint64_t)Di, (uint64_t)B * Lx) ||
      !make_map3(&tm_yl, y_lw, 32, (uint64_t)Di, (uint64_t)B * Ly) || !make_map3(&tm_yu, y_uw, 32, (uint64_t)Di, (uint64_t)B * Ly) ||
      !make_map2(&tm_lx, x_l, (uint64_t)B * Lx) || !make_map2(&tm_ly, y_l, (uint64_t)B * Ly) ||
      !make_map2(&tm_uy, y_u, (uint64_t)B * Ly) ||
      !make_map3(&tm_zl, z_lw, (uint64_t)heads * Ly, (uint64_t)Di, S * Lx) ||
      !make_map3(&tm_zu, z_uw, (uint64_t)heads * Ly, (uint64_t)Di, S * Lx))
    return FB_ERR_CUDA;
  const int n_ib = Lx / 32, n_mb = Di / 4;
  const int total = B * n_ib * n_mb;
  static std::once_flag attr_once[64];
  int dev = 0;
  FB_CUDA_OK(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once[dev & 63], [&]() {
    attr_err = cudaFuncSetAttribute(dot_weight_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDtSmemBytes);
  });
  FB_CUDA_OK(attr_err);
  const int sms = device_info().sms;
  dot_weight_tc<<<(unsigned)(total < sms ? total : sms), kDtThreads, kDtSmemBytes, st>>>(
      tm_xl, tm_xu, tm_yl, tm_yu, tm_lx, tm_ly, tm_uy, tm_zl, tm_zu, Lx, Ly, n_ib, n_mb, total, out_scale, heads, y_kmajor, tc_status_sink());
  FB_LAUNCH_OK();
  return FB_OK;
}

// Reads (and clears) this file's copy of the flag raised by an expired bounded wait.
int dot_tc_error_flag(int* flag) {
  int v = 0;
  FB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    FB_CUDA_OK(cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int)));
  }
  *flag = v;
  return FB_OK;
}

}  // namespace fb
