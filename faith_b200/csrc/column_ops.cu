// Column operators: concretisation (dual norm over dim_in) fused with the per-column linear
// relaxation and the rescale of lw/uw.  HBM-bound: every element of lw/uw is read from DRAM
// once and written once; the tile a block reduces over is kept in shared memory between the
// norm pass and the rescale pass (or, when it does not fit, re-read through L2).
//
// Native layout [rows, Di, Do]: a block owns one row (b,l) and a tile of CW = 32 columns;
// its 256 threads are (column lanes) x (row groups); the reduction over Di runs down the
// row groups, then across them by warp shuffles and a small shared-memory tree.
// Transposed layout [rows, Do, Di] (the reference's pybind layout): one warp per column.
#include <cooperative_groups.h>

#include "common.cuh"

namespace fb {
namespace {

constexpr int kThreads = 256;
constexpr int kCW = 32;  // columns per block tile

constexpr int OP_CONCRETIZE = -1;
constexpr int OP_COEF_ONLY = 16;   // added to a relaxation op: write the column coefficients instead of rescaling

// ---------------------------------------------------------------------------
// Norm pass over one operand pair (lw, uw) of a tile.  Returns, for threads tid < kCW, the
// concretised l and u of column c0 + tid (given lb/ub of that column).
// VEC = 4: thread = (cvl = tid & 7, rg = tid >> 3), float4 loads; VEC = 1: (tid & 31, tid >> 5).
template <int VEC, bool STAGED>
__device__ __forceinline__ void tile_concretize(const float* __restrict__ gl, const float* __restrict__ gu,
                                                int Di, int Do, int c0, int words, int p, float eps,
                                                float* s_l, float* s_u,      // staged tile [Di][kCW] each
                                                float* s_red,                // [2][8][kCW]
                                                float lbv, float ubv, float& l_out, float& u_out,
                                                bool raw = false) {
  constexpr int CVL = kCW / VEC;
  constexpr int RG = kThreads / CVL;
  const int tid = threadIdx.x;
  const int cvl = tid % CVL;
  const int rg = tid / CVL;
  const int col = c0 + cvl * VEC;
  const bool col_ok = col < Do;  // with VEC = 4, Do % 4 == 0, so a vector is all-valid or all-invalid
  const int blk = Di / words;
  const int warp = tid >> 5, lane = tid & 31;
  float l_run = lbv, u_run = ubv;
  for (int w = 0; w < words; ++w) {
    float al[VEC], au[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) { al[e] = 0.f; au[e] = 0.f; }
    const int r_end = (w + 1) * blk;
#pragma unroll 4
    for (int r = w * blk + rg; r < r_end; r += RG) {
      float vl[VEC], vu[VEC];
      if (col_ok) {
        const size_t off = (size_t)r * Do + col;
        if (VEC == 4) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(gl + off));
          const float4 b = __ldg(reinterpret_cast<const float4*>(gu + off));
          vl[0] = a.x; vl[1 % VEC] = a.y; vl[2 % VEC] = a.z; vl[3 % VEC] = a.w;
          vu[0] = b.x; vu[1 % VEC] = b.y; vu[2 % VEC] = b.z; vu[3 % VEC] = b.w;
        } else {
          vl[0] = __ldg(gl + off);
          vu[0] = __ldg(gu + off);
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) { vl[e] = 0.f; vu[e] = 0.f; }
      }
      if (STAGED) {
        if (VEC == 4) {
          *reinterpret_cast<float4*>(s_l + r * kCW + cvl * 4) = make_float4(vl[0], vl[1 % VEC], vl[2 % VEC], vl[3 % VEC]);
          *reinterpret_cast<float4*>(s_u + r * kCW + cvl * 4) = make_float4(vu[0], vu[1 % VEC], vu[2 % VEC], vu[3 % VEC]);
        } else {
          s_l[r * kCW + cvl] = vl[0];
          s_u[r * kCW + cvl] = vu[0];
        }
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        al[e] = norm_accum(p, al[e], vl[e]);
        au[e] = norm_accum(p, au[e], vu[e]);
      }
    }
    // across the row groups of a warp (lanes that share cvl), then across warps
    if (VEC == 4) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
#pragma unroll
        for (int s = 8; s < 32; s <<= 1) {
          al[e] = norm_combine(p, al[e], __shfl_xor_sync(0xffffffffu, al[e], s));
          au[e] = norm_combine(p, au[e], __shfl_xor_sync(0xffffffffu, au[e], s));
        }
      }
      if (lane < 8) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          s_red[warp * kCW + lane * 4 + e] = al[e];
          s_red[8 * kCW + warp * kCW + lane * 4 + e] = au[e];
        }
      }
    } else {
      s_red[warp * kCW + lane] = al[0];
      s_red[8 * kCW + warp * kCW + lane] = au[0];
    }
    __syncthreads();
    if (tid < kCW) {
      float sl = s_red[tid], su = s_red[8 * kCW + tid];
#pragma unroll
      for (int k = 1; k < 8; ++k) {
        sl = norm_combine(p, sl, s_red[k * kCW + tid]);
        su = norm_combine(p, su, s_red[8 * kCW + k * kCW + tid]);
      }
      if (raw) {  // unfinished accumulation (sum |w|, sum w^2 or max |w|) for a cross-device reduction
        l_run = sl;
        u_run = su;
      } else {
        l_run = fadd(l_run, fmul(-eps, norm_finish(p, sl)));
        u_run = fadd(u_run, fmul(eps, norm_finish(p, su)));
      }
    }
    __syncthreads();
  }
  l_out = l_run;
  u_out = u_run;
}

// Rescale pass: out_lw = c_ll*lw + c_lu*uw, out_uw = c_ul*lw + c_uu*uw for the tile.
template <int VEC, bool STAGED>
__device__ __forceinline__ void tile_rescale(const float* __restrict__ gl, const float* __restrict__ gu,
                                             float* __restrict__ ol, float* __restrict__ ou,
                                             int Di, int Do, int c0, const float* s_l, const float* s_u,
                                             const float* s_coef /* [4][kCW] */) {
  constexpr int CVL = kCW / VEC;
  constexpr int RG = kThreads / CVL;
  const int tid = threadIdx.x;
  const int cvl = tid % CVL;
  const int rg = tid / CVL;
  const int col = c0 + cvl * VEC;
  if (col >= Do) return;
  float cll[VEC], clu[VEC], cul[VEC], cuu[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    cll[e] = s_coef[0 * kCW + cvl * VEC + e];
    clu[e] = s_coef[1 * kCW + cvl * VEC + e];
    cul[e] = s_coef[2 * kCW + cvl * VEC + e];
    cuu[e] = s_coef[3 * kCW + cvl * VEC + e];
  }
#pragma unroll 4
  for (int r = rg; r < Di; r += RG) {
    const size_t off = (size_t)r * Do + col;
    float vl[VEC], vu[VEC], rl[VEC], ru[VEC];
    if (VEC == 4) {
      float4 a, b;
      if (STAGED) {
        a = *reinterpret_cast<const float4*>(s_l + r * kCW + cvl * 4);
        b = *reinterpret_cast<const float4*>(s_u + r * kCW + cvl * 4);
      } else {
        a = *reinterpret_cast<const float4*>(gl + off);
        b = *reinterpret_cast<const float4*>(gu + off);
      }
      vl[0] = a.x; vl[1 % VEC] = a.y; vl[2 % VEC] = a.z; vl[3 % VEC] = a.w;
      vu[0] = b.x; vu[1 % VEC] = b.y; vu[2 % VEC] = b.z; vu[3 % VEC] = b.w;
    } else {
      vl[0] = STAGED ? s_l[r * kCW + cvl] : gl[off];
      vu[0] = STAGED ? s_u[r * kCW + cvl] : gu[off];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      rl[e] = fmaf(cll[e], vl[e], fmul(clu[e], vu[e]));
      ru[e] = fmaf(cuu[e], vu[e], fmul(cul[e], vl[e]));
    }
    if (VEC == 4) {
      *reinterpret_cast<float4*>(ol + off) = make_float4(rl[0], rl[1 % VEC], rl[2 % VEC], rl[3 % VEC]);
      *reinterpret_cast<float4*>(ou + off) = make_float4(ru[0], ru[1 % VEC], ru[2 % VEC], ru[3 % VEC]);
    } else {
      ol[off] = rl[0];
      ou[off] = ru[0];
    }
  }
}

template <int VEC, bool STAGED>
__global__ void __launch_bounds__(kThreads)
col_relax_native(int op, const float* __restrict__ lw, const float* __restrict__ uw,
                 const float* __restrict__ lb, const float* __restrict__ ub,
                 float* __restrict__ o_lw, float* __restrict__ o_uw, float* __restrict__ o_lb,
                 float* __restrict__ o_ub, int Di, int Do, int ntiles, int words, int p, float eps,
                 int* __restrict__ violation) {
  extern __shared__ __align__(16) float smem[];
  float* s_red = smem;                    // [2][8][kCW]
  float* s_coef = s_red + 2 * 8 * kCW;    // [4][kCW]
  float* s_l = s_coef + 4 * kCW;          // [Di][kCW] when STAGED
  float* s_u = s_l + (STAGED ? (size_t)Di * kCW : 0);
  const int64_t row = blockIdx.x / ntiles;
  const int c0 = (int)(blockIdx.x % ntiles) * kCW;
  const int tid = threadIdx.x;
  const float* gl = lw + (size_t)row * Di * Do;
  const float* gu = uw + (size_t)row * Di * Do;
  const bool mine = tid < kCW && c0 + tid < Do;
  float lbv = 0.f, ubv = 0.f;
  if (mine) {
    lbv = lb[(size_t)row * Do + c0 + tid];
    ubv = ub[(size_t)row * Do + c0 + tid];
  }
  float l, u;
  tile_concretize<VEC, STAGED>(gl, gu, Di, Do, c0, words, p, eps, s_l, s_u, s_red, lbv, ubv, l, u);
  if (op == OP_CONCRETIZE) {
    if (mine) {
      o_lb[(size_t)row * Do + c0 + tid] = l;
      o_ub[(size_t)row * Do + c0 + tid] = u;
    }
    return;
  }
  if (op >= OP_COEF_ONLY) {
    // coefficients only: o_lw / o_uw are [rows, Do] arrays that receive the own-side slopes; a column
    // with a cross term (possible only for an inverted range l > u) raises bit 1 of the flag
    if (mine) {
      bool bad = false;
      const ColCoef c = relax_column(op - OP_COEF_ONLY, l, u, lbv, ubv, bad);
      if (violation != nullptr && (bad || c.c_lu != 0.f || c.c_ul != 0.f)) atomicOr(violation, bad ? 1 : 2);
      const size_t o = (size_t)row * Do + c0 + tid;
      o_lw[o] = c.c_ll;
      o_uw[o] = c.c_uu;
      o_lb[o] = c.nlb;
      o_ub[o] = c.nub;
    }
    return;
  }
  if (tid < kCW) {
    ColCoef c = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (mine) {
      bool bad = false;
      c = relax_column(op, l, u, lbv, ubv, bad);
      if (bad && violation != nullptr) *violation = 1;
      o_lb[(size_t)row * Do + c0 + tid] = c.nlb;
      o_ub[(size_t)row * Do + c0 + tid] = c.nub;
    }
    s_coef[0 * kCW + tid] = c.c_ll;
    s_coef[1 * kCW + tid] = c.c_lu;
    s_coef[2 * kCW + tid] = c.c_ul;
    s_coef[3 * kCW + tid] = c.c_uu;
  }
  __syncthreads();
  tile_rescale<VEC, STAGED>(gl, gu, o_lw + (size_t)row * Di * Do, o_uw + (size_t)row * Di * Do, Di, Do, c0,
                            s_l, s_u, s_coef);
}

// McCormick product of two bounded operands: both are concretised in the same block, the four
// input tiles stay in shared memory (or are re-read) for the combination pass.
template <int VEC, bool STAGED>
__global__ void __launch_bounds__(kThreads)
col_mul_bounds_native(const float* __restrict__ x_lw, const float* __restrict__ x_uw,
                      const float* __restrict__ x_lb, const float* __restrict__ x_ub,
                      const float* __restrict__ y_lw, const float* __restrict__ y_uw,
                      const float* __restrict__ y_lb, const float* __restrict__ y_ub,
                      float* __restrict__ z_lw, float* __restrict__ z_uw, float* __restrict__ z_lb,
                      float* __restrict__ z_ub, int Di, int Do, int ntiles, int words, int p, float eps) {
  extern __shared__ __align__(16) float smem[];
  float* s_red = smem;
  float* s_coef = s_red + 2 * 8 * kCW;  // [8][kCW]: lower (x own, x other, y own, y other), upper (same)
  float* s_xl = s_coef + 8 * kCW;
  const size_t tile = STAGED ? (size_t)Di * kCW : 0;
  float* s_xu = s_xl + tile;
  float* s_yl = s_xu + tile;
  float* s_yu = s_yl + tile;
  const int64_t row = blockIdx.x / ntiles;
  const int c0 = (int)(blockIdx.x % ntiles) * kCW;
  const int tid = threadIdx.x;
  const size_t wbase = (size_t)row * Di * Do;
  const bool mine = tid < kCW && c0 + tid < Do;
  float xlb = 0.f, xub = 0.f, ylb = 0.f, yub = 0.f;
  if (mine) {
    const size_t o = (size_t)row * Do + c0 + tid;
    xlb = x_lb[o]; xub = x_ub[o]; ylb = y_lb[o]; yub = y_ub[o];
  }
  float lx, ux, ly, uy;
  tile_concretize<VEC, STAGED>(x_lw + wbase, x_uw + wbase, Di, Do, c0, words, p, eps, s_xl, s_xu, s_red, xlb, xub, lx, ux);
  tile_concretize<VEC, STAGED>(y_lw + wbase, y_uw + wbase, Di, Do, c0, words, p, eps, s_yl, s_yu, s_red, ylb, yub, ly, uy);
  if (tid < kCW) {
    // lower plane: alpha = l_y on x, beta = l_x on y, constant -alpha*beta   (Bounds.py:680-688)
    // upper plane: alpha = u_y on x, beta = l_x on y
    float co[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) co[i] = 0.f;
    if (mine) {
      const float al = ly, be = lx, au = uy;
      const float gl_ = fmul(-al, be), gu_ = fmul(-au, be);
      const bool alp = al > 0.f, bep = be > 0.f, aup = au > 0.f;
      co[alp ? 0 : 1] = al;   // lower: x.lw (own) or x.uw
      co[bep ? 2 : 3] = be;   // lower: y.lw (own) or y.uw
      co[aup ? 4 : 5] = au;   // upper: x.uw (own) or x.lw
      co[bep ? 6 : 7] = be;   // upper: y.uw (own) or y.lw
      const float tl = fadd(fmul(alp ? xlb : xub, al), gl_);
      const float tu = fadd(fmul(aup ? xub : xlb, au), gu_);
      const size_t o = (size_t)row * Do + c0 + tid;
      z_lb[o] = fadd(tl, fmul(bep ? ylb : yub, be));
      z_ub[o] = fadd(tu, fmul(bep ? yub : ylb, be));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) s_coef[i * kCW + tid] = co[i];
  }
  __syncthreads();
  constexpr int CVL = kCW / VEC;
  constexpr int RG = kThreads / CVL;
  const int cvl = tid % CVL, rg = tid / CVL;
  const int col = c0 + cvl * VEC;
  if (col >= Do) return;
  float co[8][VEC];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int e = 0; e < VEC; ++e) co[i][e] = s_coef[i * kCW + cvl * VEC + e];
  for (int r = rg; r < Di; r += RG) {
    const size_t off = wbase + (size_t)r * Do + col;
    float a[VEC], b[VEC], c[VEC], d[VEC], rl[VEC], ru[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      if (STAGED) {
        a[e] = s_xl[r * kCW + cvl * VEC + e]; b[e] = s_xu[r * kCW + cvl * VEC + e];
        c[e] = s_yl[r * kCW + cvl * VEC + e]; d[e] = s_yu[r * kCW + cvl * VEC + e];
      } else {
        a[e] = x_lw[off + e]; b[e] = x_uw[off + e]; c[e] = y_lw[off + e]; d[e] = y_uw[off + e];
      }
      // (alpha term) + (beta term); in each pair one coefficient is zero
      const float tl = fmaf(co[0][e], a[e], fmul(co[1][e], b[e]));
      const float sl = fmaf(co[2][e], c[e], fmul(co[3][e], d[e]));
      const float tu = fmaf(co[4][e], b[e], fmul(co[5][e], a[e]));
      const float su = fmaf(co[6][e], d[e], fmul(co[7][e], c[e]));
      rl[e] = fadd(tl, sl);
      ru[e] = fadd(tu, su);
    }
    if (VEC == 4) {
      *reinterpret_cast<float4*>(z_lw + off) = make_float4(rl[0], rl[1 % VEC], rl[2 % VEC], rl[3 % VEC]);
      *reinterpret_cast<float4*>(z_uw + off) = make_float4(ru[0], ru[1 % VEC], ru[2 % VEC], ru[3 % VEC]);
    } else {
      z_lw[off] = rl[0];
      z_uw[off] = ru[0];
    }
  }
}

// ------------------------------------------------- dim_in-sharded relaxation
// When the dim_in axis is split over several GPUs, the dual norm of a column needs the rows of
// every shard.  Pass 1 (this kernel) writes the unfinished accumulation of the local rows, the
// caller reduces it across devices (sum for p = inf and p = 2, max for p = 1), pass 2 applies the
// relaxation to the local rows from the reduced values.  One perturbed word.
template <int VEC>
__global__ void __launch_bounds__(kThreads)
col_norm_partials_native(const float* __restrict__ lw, const float* __restrict__ uw, float* __restrict__ part_l,
                         float* __restrict__ part_u, int Di, int Do, int ntiles, int p) {
  extern __shared__ __align__(16) float smem[];
  const int64_t row = blockIdx.x / ntiles;
  const int c0 = (int)(blockIdx.x % ntiles) * kCW;
  const int tid = threadIdx.x;
  float l, u;
  tile_concretize<VEC, false>(lw + (size_t)row * Di * Do, uw + (size_t)row * Di * Do, Di, Do, c0, 1, p, 0.f, nullptr,
                              nullptr, smem, 0.f, 0.f, l, u, true);
  if (tid < kCW && c0 + tid < Do) {
    part_l[(size_t)row * Do + c0 + tid] = l;
    part_u[(size_t)row * Do + c0 + tid] = u;
  }
}

// The same for a tall operand with few column tiles (the CNN: one image, dim_in = 3072 rows): a cluster of kSplit
// blocks shares a column tile, each block accumulates a contiguous range of the rows, and block 0 of the cluster
// combines the kSplit partial results through distributed shared memory, in block order (so the value does not
// depend on scheduling).
constexpr int kSplit = 8;
template <int VEC>
__global__ void __launch_bounds__(kThreads)
col_norm_partials_split(const float* __restrict__ lw, const float* __restrict__ uw, float* __restrict__ part_l,
                        float* __restrict__ part_u, int Di, int Do, int ntiles, int p) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ __align__(16) float s_red[2 * 8 * kCW];
  __shared__ float s_part[2 * kCW];
  const unsigned cr = cluster.block_rank();
  const int64_t tile = blockIdx.x / kSplit;
  const int64_t row = tile / ntiles;
  const int c0 = (int)(tile % ntiles) * kCW;
  const int tid = threadIdx.x;
  const int chunk = (Di + kSplit - 1) / kSplit;
  const int r0 = min(Di, (int)cr * chunk), r1 = min(Di, r0 + chunk);
  float l, u;
  const size_t base = (size_t)row * Di * Do + (size_t)r0 * Do;
  tile_concretize<VEC, false>(lw + base, uw + base, r1 - r0, Do, c0, 1, p, 0.f, nullptr, nullptr, s_red, 0.f, 0.f, l, u, true);
  if (tid < kCW) {
    s_part[tid] = l;
    s_part[kCW + tid] = u;
  }
  cluster.sync();
  if (cr == 0 && tid < kCW && c0 + tid < Do) {
    float sl = l, su = u;
    for (unsigned k = 1; k < kSplit; ++k) {
      const float* rp = cluster.map_shared_rank(s_part, k);
      sl = norm_combine(p, sl, rp[tid]);
      su = norm_combine(p, su, rp[kCW + tid]);
    }
    part_l[(size_t)row * Do + c0 + tid] = sl;
    part_u[(size_t)row * Do + c0 + tid] = su;
  }
  cluster.sync();   // the other blocks' shared memory stays alive until block 0 has read it
}

// Few columns, many rows (the final concretisation of the CNN head: [3072, 10]): a column tile of 32 would leave
// two thirds of the lanes idle and make every load a partial sector.  Here the [Di, Do] slab of a (b, l) row is read
// as the flat array it is: a cluster of kSplit blocks splits the rows, in a block thread t < S (S = the largest
// multiple of Do within the block) owns column t % Do and walks the rows t / Do, t / Do + S / Do, ..., so a warp reads
// consecutive words; the S / Do partial results of a column are added in thread order by one thread per column, the
// kSplit block results in block order by block 0 through distributed shared memory.
__global__ void __launch_bounds__(kThreads)
col_norm_partials_narrow(const float* __restrict__ lw, const float* __restrict__ uw, float* __restrict__ part_l,
                         float* __restrict__ part_u, int Di, int Do, int p) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float s_l[kThreads], s_u[kThreads];
  __shared__ float s_part[2 * 64];
  const unsigned cr = cluster.block_rank();
  const int64_t row = blockIdx.x / kSplit;
  const int tid = threadIdx.x;
  const int per = kThreads / Do, S = per * Do;       // rows in flight per step, active threads
  const int chunk = (Di + kSplit - 1) / kSplit;
  const int r0 = min(Di, (int)cr * chunk), r1 = min(Di, r0 + chunk);
  const float* gl = lw + (size_t)row * Di * Do;
  const float* gu = uw + (size_t)row * Di * Do;
  float al = 0.f, au = 0.f;
  if (tid < S) {
    const int col = tid % Do;
#pragma unroll 4
    for (int r = r0 + tid / Do; r < r1; r += per) {
      al = norm_accum(p, al, __ldg(gl + (size_t)r * Do + col));
      au = norm_accum(p, au, __ldg(gu + (size_t)r * Do + col));
    }
  }
  s_l[tid] = al;
  s_u[tid] = au;
  __syncthreads();
  if (tid < Do) {
    float sl = s_l[tid], su = s_u[tid];
    for (int k = 1; k < per; ++k) {
      sl = norm_combine(p, sl, s_l[k * Do + tid]);
      su = norm_combine(p, su, s_u[k * Do + tid]);
    }
    s_part[tid] = sl;
    s_part[64 + tid] = su;
  }
  cluster.sync();
  if (cr == 0 && tid < Do) {
    float sl = s_part[tid], su = s_part[64 + tid];
    for (unsigned k = 1; k < kSplit; ++k) {
      const float* rp = cluster.map_shared_rank(s_part, k);
      sl = norm_combine(p, sl, rp[tid]);
      su = norm_combine(p, su, rp[64 + tid]);
    }
    part_l[(size_t)row * Do + tid] = sl;
    part_u[(size_t)row * Do + tid] = su;
  }
  cluster.sync();   // the other blocks' shared memory stays alive until block 0 has read it
}

template <int VEC>
__global__ void __launch_bounds__(kThreads)
col_relax_apply_native(int op, const float* __restrict__ lw, const float* __restrict__ uw,
                       const float* __restrict__ lb, const float* __restrict__ ub,
                       const float* __restrict__ norm_l, const float* __restrict__ norm_u,
                       float* __restrict__ o_lw, float* __restrict__ o_uw, float* __restrict__ o_lb,
                       float* __restrict__ o_ub, int Di, int Do, int ntiles, int p, float eps,
                       int* __restrict__ violation) {
  __shared__ float s_coef[4 * kCW];
  const int64_t row = blockIdx.x / ntiles;
  const int c0 = (int)(blockIdx.x % ntiles) * kCW;
  const int tid = threadIdx.x;
  if (tid < kCW) {
    ColCoef c = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (c0 + tid < Do) {
      const size_t o = (size_t)row * Do + c0 + tid;
      const float lbv = lb[o], ubv = ub[o];
      const float l = fadd(lbv, fmul(-eps, norm_finish(p, norm_l[o])));
      const float u = fadd(ubv, fmul(eps, norm_finish(p, norm_u[o])));
      bool bad = false;
      c = relax_column(op, l, u, lbv, ubv, bad);
      if (bad && violation != nullptr) *violation = 1;
      o_lb[o] = c.nlb;
      o_ub[o] = c.nub;
    }
    s_coef[0 * kCW + tid] = c.c_ll;
    s_coef[1 * kCW + tid] = c.c_lu;
    s_coef[2 * kCW + tid] = c.c_ul;
    s_coef[3 * kCW + tid] = c.c_uu;
  }
  __syncthreads();
  const size_t wb = (size_t)row * Di * Do;
  tile_rescale<VEC, false>(lw + wb, uw + wb, o_lw + wb, o_uw + wb, Di, Do, c0, nullptr, nullptr, s_coef);
}

// ------------------------------------------------------------ transposed layout
// [rows, Do, Di]: the Di values of a column are contiguous; one warp per column, two passes
// (the second is served by L1/L2, a column is at most a few KB).
template <int VEC>
__global__ void __launch_bounds__(kThreads)
col_relax_transposed(int op, const float* __restrict__ lw, const float* __restrict__ uw,
                     const float* __restrict__ lb, const float* __restrict__ ub,
                     float* __restrict__ o_lw, float* __restrict__ o_uw, float* __restrict__ o_lb,
                     float* __restrict__ o_ub, int64_t ncols, int Di, int words, int p, float eps,
                     int* __restrict__ violation) {
  const int lane = threadIdx.x & 31;
  const int64_t col = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  if (col >= ncols) return;
  const float* gl = lw + (size_t)col * Di;
  const float* gu = uw + (size_t)col * Di;
  const int blk = Di / words;
  const float lbv = lb[col], ubv = ub[col];
  float l = lbv, u = ubv;
  for (int w = 0; w < words; ++w) {
    float al = 0.f, au = 0.f;
    for (int r = w * blk + lane * VEC; r < (w + 1) * blk; r += 32 * VEC) {
      if (VEC == 4) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(gl + r));
        const float4 b = __ldg(reinterpret_cast<const float4*>(gu + r));
        al = norm_accum(p, norm_accum(p, norm_accum(p, norm_accum(p, al, a.x), a.y), a.z), a.w);
        au = norm_accum(p, norm_accum(p, norm_accum(p, norm_accum(p, au, b.x), b.y), b.z), b.w);
      } else {
        al = norm_accum(p, al, __ldg(gl + r));
        au = norm_accum(p, au, __ldg(gu + r));
      }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      al = norm_combine(p, al, __shfl_xor_sync(0xffffffffu, al, s));
      au = norm_combine(p, au, __shfl_xor_sync(0xffffffffu, au, s));
    }
    l = fadd(l, fmul(-eps, norm_finish(p, al)));
    u = fadd(u, fmul(eps, norm_finish(p, au)));
  }
  if (op == OP_CONCRETIZE) {
    if (lane == 0) { o_lb[col] = l; o_ub[col] = u; }
    return;
  }
  bool bad = false;
  const ColCoef c = relax_column(op, l, u, lbv, ubv, bad);  // every lane computes the same scalars
  if (lane == 0) {
    if (bad && violation != nullptr) *violation = 1;
    o_lb[col] = c.nlb;
    o_ub[col] = c.nub;
  }
  float* ol = o_lw + (size_t)col * Di;
  float* ou = o_uw + (size_t)col * Di;
  for (int r = lane * VEC; r < Di; r += 32 * VEC) {
    if (VEC == 4) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(gl + r));
      const float4 b = __ldg(reinterpret_cast<const float4*>(gu + r));
      float4 x, y;
      x.x = fmaf(c.c_ll, a.x, fmul(c.c_lu, b.x)); y.x = fmaf(c.c_uu, b.x, fmul(c.c_ul, a.x));
      x.y = fmaf(c.c_ll, a.y, fmul(c.c_lu, b.y)); y.y = fmaf(c.c_uu, b.y, fmul(c.c_ul, a.y));
      x.z = fmaf(c.c_ll, a.z, fmul(c.c_lu, b.z)); y.z = fmaf(c.c_uu, b.z, fmul(c.c_ul, a.z));
      x.w = fmaf(c.c_ll, a.w, fmul(c.c_lu, b.w)); y.w = fmaf(c.c_uu, b.w, fmul(c.c_ul, a.w));
      *reinterpret_cast<float4*>(ol + r) = x;
      *reinterpret_cast<float4*>(ou + r) = y;
    } else {
      const float a = __ldg(gl + r), b = __ldg(gu + r);
      ol[r] = fmaf(c.c_ll, a, fmul(c.c_lu, b));
      ou[r] = fmaf(c.c_uu, b, fmul(c.c_ul, a));
    }
  }
}

size_t relax_smem_bytes(int Di, bool staged, int tiles) {
  return sizeof(float) * ((2 * 8 + (tiles == 4 ? 8 : 4)) * kCW + (staged ? (size_t)tiles * Di * kCW : 0));
}

template <typename K>
int ensure_smem(K kernel, size_t bytes) {
  return ensure_dynamic_smem(kernel, bytes);
}

int launch_relax(int op, const float* lw, const float* uw, const float* lb, const float* ub,
                 float* o_lw, float* o_uw, float* o_lb, float* o_ub, int64_t rows, int Di, int Do,
                 int words, int p, float eps, int layout, int* violation, cudaStream_t st) {
  if (rows == 0 || Do == 0) return FB_OK;
  if (layout == FB_TRANSPOSED) {
    const int64_t ncols = rows * Do;
    const int64_t blocks = ceil_div(ncols, kThreads / 32);
    if (blocks > 0x7fffffff) return FB_ERR_SHAPE;
    const bool vec = (Di / words) % 4 == 0 && aligned16(lw) && aligned16(uw) &&
                     (op == OP_CONCRETIZE || (aligned16(o_lw) && aligned16(o_uw)));
    if (vec)
      col_relax_transposed<4><<<(unsigned)blocks, kThreads, 0, st>>>(op, lw, uw, lb, ub, o_lw, o_uw, o_lb, o_ub,
                                                                      ncols, Di, words, p, eps, violation);
    else
      col_relax_transposed<1><<<(unsigned)blocks, kThreads, 0, st>>>(op, lw, uw, lb, ub, o_lw, o_uw, o_lb, o_ub,
                                                                      ncols, Di, words, p, eps, violation);
    FB_LAUNCH_OK();
    return FB_OK;
  }
  const int ntiles = (int)ceil_div(Do, kCW);
  const int64_t blocks = rows * ntiles;
  if (blocks > 0x7fffffff) return FB_ERR_SHAPE;
  const bool vec = Do % 4 == 0 && aligned16(lw) && aligned16(uw) &&
                   (op == OP_CONCRETIZE || op >= OP_COEF_ONLY || (aligned16(o_lw) && aligned16(o_uw)));
  // Keep the tile in shared memory when a few blocks per SM still fit; concretise alone and the
  // coefficient-only mode have no second pass and never stage.
  const size_t staged_bytes = relax_smem_bytes(Di, true, 2);
  // (40 KB: dim_in up to 128 + the scratch.  A 64 KB tile, dim_in 256, leaves three blocks per SM and was slower staged than
  // re-read through L2: tanh on [8, 64, 256, 256] 0.172 ms staged, 0.137 ms not, 0.48 -> 0.60 of the HBM roof.)
  const bool staged = op != OP_CONCRETIZE && op < OP_COEF_ONLY && staged_bytes <= 40 * 1024;
  const size_t smem = staged ? staged_bytes : relax_smem_bytes(Di, false, 2);
#define FB_RELAX_LAUNCH(V, S)                                                                              \
  do {                                                                                                     \
    int rc_ = ensure_smem(col_relax_native<V, S>, smem);                                                   \
    if (rc_ != FB_OK) return rc_;                                                                          \
    col_relax_native<V, S><<<(unsigned)blocks, kThreads, smem, st>>>(op, lw, uw, lb, ub, o_lw, o_uw, o_lb, \
                                                                     o_ub, Di, Do, ntiles, words, p, eps,  \
                                                                     violation);                           \
  } while (0)
  if (vec && staged) FB_RELAX_LAUNCH(4, true);
  else if (vec) FB_RELAX_LAUNCH(4, false);
  else if (staged) FB_RELAX_LAUNCH(1, true);
  else FB_RELAX_LAUNCH(1, false);
#undef FB_RELAX_LAUNCH
  FB_LAUNCH_OK();
  return FB_OK;
}


// Slopes and relaxed bias terms of a relaxation whose concretised ranges are already known (written by
// the kernel that produced the bound): one thread per (row, column), no access to lw / uw.
__global__ void __launch_bounds__(256)
relax_coef_given_kernel(int op, const float* __restrict__ lb, const float* __restrict__ ub, const float* __restrict__ l,
                        const float* __restrict__ u, float* __restrict__ c_l, float* __restrict__ c_u,
                        float* __restrict__ o_lb, float* __restrict__ o_ub, int64_t n, int* __restrict__ violation) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x) {
    bool bad = false;
    const ColCoef c = relax_column(op, l[t], u[t], lb[t], ub[t], bad);
    if (violation != nullptr && (bad || c.c_lu != 0.f || c.c_ul != 0.f)) atomicOr(violation, bad ? 1 : 2);
    c_l[t] = c.c_ll;
    c_u[t] = c.c_uu;
    o_lb[t] = c.nlb;
    o_ub[t] = c.nub;
  }
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" int fb_concretize_f32(const float* lw, const float* uw, const float* lb, const float* ub, float* l,
                                 float* u, int64_t rows, int Di, int Do, int words, int p, float eps, int layout,
                                 void* stream) {
  if (rows == 0 || Do == 0) return FB_OK;
  if (!lw || !uw || !lb || !ub || !l || !u) return FB_ERR_ARG;
  if (rows < 0 || Di <= 0 || Do < 0 || words <= 0 || !valid_norm(p)) return FB_ERR_ARG;
  if (layout != FB_NATIVE && layout != FB_TRANSPOSED) return FB_ERR_ARG;
  if (Di % words != 0) return FB_ERR_SHAPE;
  const double mw = (double)rows * Di * Do, mb = (double)rows * Do;
  ProfileScope prof(PK_RELAX, 4.0 * mw, 4.0 * (2 * mw + 4 * mb), stream);
  return launch_relax(OP_CONCRETIZE, lw, uw, lb, ub, nullptr, nullptr, l, u, rows, Di, Do, words, p, eps, layout,
                      nullptr, (cudaStream_t)stream);
}

extern "C" int fb_relax_f32(int op, const float* lw, const float* uw, const float* lb, const float* ub,
                            float* out_lw, float* out_uw, float* out_lb, float* out_ub, int64_t rows, int Di, int Do,
                            int words, int p, float eps, int layout, int* violation, void* stream) {
  const bool known_op = (op >= FB_RELU && op <= FB_SQRT) || (op >= FB_INTERVAL + FB_RELU && op <= FB_INTERVAL + FB_SQRT);
  if (rows == 0 || Do == 0) return known_op ? FB_OK : FB_ERR_ARG;
  if (!lw || !uw || !lb || !ub || !out_lw || !out_uw || !out_lb || !out_ub) return FB_ERR_ARG;
  if (!known_op) return FB_ERR_ARG;
  if (rows < 0 || Di <= 0 || Do < 0 || words <= 0 || !valid_norm(p)) return FB_ERR_ARG;
  if (layout != FB_NATIVE && layout != FB_TRANSPOSED) return FB_ERR_ARG;
  if (Di % words != 0) return FB_ERR_SHAPE;
  if (out_lw == lw || out_lw == uw || out_uw == lw || out_uw == uw) return FB_ERR_ARG;
  const double mw = (double)rows * Di * Do, mb = (double)rows * Do;
  ProfileScope prof(PK_RELAX, 6.0 * mw, 4.0 * (4 * mw + 4 * mb), stream);
  return launch_relax(op, lw, uw, lb, ub, out_lw, out_uw, out_lb, out_ub, rows, Di, Do, words, p, eps, layout,
                      violation, (cudaStream_t)stream);
}

extern "C" int fb_mul_bounds_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                                 const float* y_lw, const float* y_uw, const float* y_lb, const float* y_ub,
                                 float* z_lw, float* z_uw, float* z_lb, float* z_ub, int64_t rows, int Di, int Do,
                                 int words, int p, float eps, void* stream) {
  if (!x_lw || !x_uw || !x_lb || !x_ub || !y_lw || !y_uw || !y_lb || !y_ub || !z_lw || !z_uw || !z_lb || !z_ub)
    return FB_ERR_ARG;
  if (rows < 0 || Di <= 0 || Do < 0 || words <= 0 || !valid_norm(p)) return FB_ERR_ARG;
  if (Di % words != 0) return FB_ERR_SHAPE;
  if (rows == 0 || Do == 0) return FB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const double mw = (double)rows * Di * Do, mb = (double)rows * Do;
  ProfileScope prof(PK_MUL, 12.0 * mw, 4.0 * (6 * mw + 6 * mb), stream);
  const int ntiles = (int)ceil_div(Do, kCW);
  const int64_t blocks = rows * ntiles;
  if (blocks > 0x7fffffff) return FB_ERR_SHAPE;
  const bool vec = Do % 4 == 0 && aligned16(x_lw) && aligned16(x_uw) && aligned16(y_lw) && aligned16(y_uw) &&
                   aligned16(z_lw) && aligned16(z_uw);
  const size_t staged_bytes = relax_smem_bytes(Di, true, 4);
  const bool staged = staged_bytes <= 100 * 1024;
  const size_t smem = staged ? staged_bytes : relax_smem_bytes(Di, false, 4);
#define FB_MUL_LAUNCH(V, S)                                                                                  \
  do {                                                                                                       \
    int rc_ = ensure_smem(col_mul_bounds_native<V, S>, smem);                                                \
    if (rc_ != FB_OK) return rc_;                                                                            \
    col_mul_bounds_native<V, S><<<(unsigned)blocks, kThreads, smem, st>>>(x_lw, x_uw, x_lb, x_ub, y_lw, y_uw, \
                                                                          y_lb, y_ub, z_lw, z_uw, z_lb, z_ub, \
                                                                          Di, Do, ntiles, words, p, eps);     \
  } while (0)
  if (vec && staged) FB_MUL_LAUNCH(4, true);
  else if (vec) FB_MUL_LAUNCH(4, false);
  else if (staged) FB_MUL_LAUNCH(1, true);
  else FB_MUL_LAUNCH(1, false);
#undef FB_MUL_LAUNCH
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_norm_partials_f32(const float* lw, const float* uw, float* part_l, float* part_u, int64_t rows,
                                    int Di_local, int Do, int p, void* stream) {
  if (rows == 0 || Do == 0) return FB_OK;
  if (!lw || !uw || !part_l || !part_u) return FB_ERR_ARG;
  if (rows < 0 || Di_local <= 0 || Do < 0 || !valid_norm(p)) return FB_ERR_ARG;
  const int ntiles = (int)ceil_div(Do, kCW);
  const int64_t blocks = rows * ntiles;
  if (blocks > 0x7fffffff) return FB_ERR_SHAPE;
  const double mw = (double)rows * Di_local * Do;
  ProfileScope prof(PK_RELAX, 4.0 * mw, 4.0 * (2 * mw + 2.0 * rows * Do), stream);
  const size_t smem = sizeof(float) * 2 * 8 * kCW;
  const bool vec = Do % 4 == 0 && aligned16(lw) && aligned16(uw);
  if (blocks < 2 * (int64_t)device_info().sms && Di_local >= 64 * kSplit) {
    // few column tiles, many rows: split the rows over a cluster
    const bool narrow = Do <= 64 && Do % 32 != 0 && rows * kSplit <= 0x7fffffff;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((narrow ? rows : blocks) * kSplit));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kSplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (narrow)
      FB_CUDA_OK(cudaLaunchKernelEx(&cfg, col_norm_partials_narrow, lw, uw, part_l, part_u, Di_local, Do, p));
    else
      FB_CUDA_OK(cudaLaunchKernelEx(&cfg, vec ? col_norm_partials_split<4> : col_norm_partials_split<1>, lw, uw, part_l, part_u,
                                    Di_local, Do, ntiles, p));
    count_launches(1);
    return FB_OK;
  }
  if (vec) col_norm_partials_native<4><<<(unsigned)blocks, kThreads, smem, (cudaStream_t)stream>>>(lw, uw, part_l, part_u, Di_local, Do, ntiles, p);
  else col_norm_partials_native<1><<<(unsigned)blocks, kThreads, smem, (cudaStream_t)stream>>>(lw, uw, part_l, part_u, Di_local, Do, ntiles, p);
  FB_LAUNCH_OK();
  return FB_OK;
}

extern "C" int fb_relax_with_norms_f32(int op, const float* lw, const float* uw, const float* lb, const float* ub,
                                       const float* norm_l, const float* norm_u, float* out_lw, float* out_uw,
                                       float* out_lb, float* out_ub, int64_t rows, int Di_local, int Do, int p,
                                       float eps, int* violation, void* stream) {
  if (op < FB_RELU || op > FB_RECIPROCAL) return FB_ERR_ARG;
  if (rows == 0 || Do == 0) return FB_OK;
  if (!lw || !uw || !lb || !ub || !norm_l || !norm_u || !out_lw || !out_uw || !out_lb || !out_ub) return FB_ERR_ARG;
  if (rows < 0 || Di_local <= 0 || Do < 0 || !valid_norm(p)) return FB_ERR_ARG;
  if (out_lw == lw || out_lw == uw || out_uw == lw || out_uw == uw) return FB_ERR_ARG;
  const int ntiles = (int)ceil_div(Do, kCW);
  const int64_t blocks = rows * ntiles;
  if (blocks > 0x7fffffff) return FB_ERR_SHAPE;
  const double mw = (double)rows * Di_local * Do;
  ProfileScope prof(PK_RELAX, 2.0 * mw, 4.0 * (4 * mw + 6.0 * rows * Do), stream);
  const bool vec = Do % 4 == 0 && aligned16(lw) && aligned16(uw) && aligned16(out_lw) && aligned16(out_uw);
  cudaStream_t st = (cudaStream_t)stream;
  if (vec) col_relax_apply_native<4><<<(unsigned)blocks, kThreads, 0, st>>>(op, lw, uw, lb, ub, norm_l, norm_u, out_lw, out_uw, out_lb, out_ub, Di_local, Do, ntiles, p, eps, violation);
  else col_relax_apply_native<1><<<(unsigned)blocks, kThreads, 0, st>>>(op, lw, uw, lb, ub, norm_l, norm_u, out_lw, out_uw, out_lb, out_ub, Di_local, Do, ntiles, p, eps, violation);
  FB_LAUNCH_OK();
  return FB_OK;
}

// Relaxation without the rescale pass: the dual norms, the relaxed bias terms and, instead of the
// rescaled weights, the own-side slopes of every column, c_l and c_u [rows, Do] (out_lw = c_l * lw,
// out_uw = c_u * uw).  For relu, tanh and exp (positive slopes, Bounds.py:921-1103) these are the only
// non-zero coefficients of a well-formed column; a column that would need a cross term (inverted range)
// sets bit 1 of *violation.  The consumer applies the slopes while it reads the weights
// (fb_matmul_coef_f32), which saves one write and one read of lw / uw.  Native layout only.
extern "C" int fb_relax_coef_f32(int op, const float* lw, const float* uw, const float* lb, const float* ub,
                                 float* c_l, float* c_u, float* out_lb, float* out_ub, int64_t rows, int Di, int Do,
                                 int words, int p, float eps, int* violation, void* stream) {
  if (op != FB_RELU && op != FB_TANH && op != FB_EXP) return FB_ERR_ARG;
  if (rows == 0 || Do == 0) return FB_OK;
  if (!lw || !uw || !lb || !ub || !c_l || !c_u || !out_lb || !out_ub) return FB_ERR_ARG;
  if (rows < 0 || Di <= 0 || Do < 0 || words <= 0 || !valid_norm(p)) return FB_ERR_ARG;
  if (Di % words != 0) return FB_ERR_SHAPE;
  const double mw = (double)rows * Di * Do, mb = (double)rows * Do;
  ProfileScope prof(PK_RELAX, 4.0 * mw, 4.0 * (2 * mw + 6 * mb), stream);
  return launch_relax(op + OP_COEF_ONLY, lw, uw, lb, ub, c_l, c_u, out_lb, out_ub, rows, Di, Do, words, p, eps,
                      FB_NATIVE, violation, (cudaStream_t)stream);
}

// fb_relax_coef_f32 for a bound whose concretised range l, u [rows, Do] the caller already holds (e.g. from
// fb_matmul_heads_ranges_f32): no pass over lw / uw at all.  out_lb / out_ub may alias lb / ub.
extern "C" int fb_relax_coef_given_f32(int op, const float* lb, const float* ub, const float* l, const float* u,
                                       float* c_l, float* c_u, float* out_lb, float* out_ub, int64_t rows, int Do,
                                       int* violation, void* stream) {
  if (op != FB_RELU && op != FB_TANH && op != FB_EXP) return FB_ERR_ARG;
  if (rows == 0 || Do == 0) return FB_OK;
  if (!lb || !ub || !l || !u || !c_l || !c_u || !out_lb || !out_ub) return FB_ERR_ARG;
  if (rows < 0 || Do < 0) return FB_ERR_ARG;
  const int64_t n = rows * Do;
  ProfileScope prof(PK_RELAX, 8.0 * n, 4.0 * 8 * n, stream);
  const int64_t want = ceil_div(n, 256), cap = (int64_t)device_info().sms * 16;
  relax_coef_given_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, (cudaStream_t)stream>>>(op, lb, ub, l, u, c_l, c_u,
                                                                                                out_lb, out_ub, n, violation);
  FB_LAUNCH_OK();
  return FB_OK;
}
