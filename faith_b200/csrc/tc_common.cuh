// Inline-PTX wrappers shared by the tcgen05 kernels (mbarrier, TMA, tensor memory, tcgen05.mma) and the
// host helper that resolves cuTensorMapEncodeTiled.  Included inside namespace fb, anonymous namespace,
// after <cuda.h>, <mutex>, <unordered_map> and common.cuh; every including file gets its own copy of the error
// flag and of the tensor-map cache.

constexpr uint32_t kTryNs = 20000;       // suspend-time hint of one mbarrier try (ns)
constexpr uint32_t kMaxTries = 100000;  // x 20 us = 2 s upper bound for any single wait

static __device__ int g_tc_error = 0;

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One try: the hardware suspends the thread until the phase completes or ~`ns` nanoseconds pass, so a
// waiting warp does not compete for issue slots with the MMA issuer and the converters.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Non-blocking test of a phase.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: at most `tries` suspended tries of ~kTryNs each (kMaxTries: a couple of seconds in total).
// Returns false (and raises the error flags) when the limit is hit or another role of this CTA has
// already given up.
struct WaitCtx {
  volatile int* cta_abort;
  uint32_t tries;
};
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& wc) {
  // fast path: in a well-fed pipeline the phase is usually complete already, and the non-blocking
  // test answers much sooner than a suspending try
  for (int i = 0; i < 4; ++i)
    if (mbar_test_wait(bar, parity)) return true;
  for (uint32_t i = 0; i < wc.tries; ++i) {
    if (mbar_try_wait(bar, parity, kTryNs)) return true;
    if (*wc.cta_abort) return false;
  }
  *wc.cta_abort = 1;
  atomicExch(&g_tc_error, 1);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* cta_abort) {
  const WaitCtx wc = {cta_abort, kMaxTries};
  return mbar_wait(bar, parity, wc);
}

// Same, for a whole warp: every lane waits, and the outcome is made uniform so that the
// .sync.aligned tensor-memory instructions that follow are executed convergently.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const WaitCtx& wc) {
  const bool ok = mbar_wait(bar, parity, wc);
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* cta_abort) {
  const bool ok = mbar_wait(bar, parity, cta_abort);
  return __all_sync(0xffffffffu, ok);
}

// Bounded wait by polling (no suspension): for the few warps whose wake-up latency is on the critical path.
// About 40 cycles per round; 512 rounds per try of the suspending wait keep the two bounds comparable.
__device__ __forceinline__ bool mbar_poll_warp(uint32_t bar, uint32_t parity, const WaitCtx& wc) {
  bool ok = false;
  const uint32_t rounds = wc.tries > (0xffffffffu >> 9) ? 0xffffffffu : wc.tries << 9;
  for (uint32_t i = 0; i < rounds; ++i) {
    if (mbar_test_wait(bar, parity)) { ok = true; break; }
    if ((i & 255u) == 255u && *wc.cta_abort) break;
  }
  if (!ok && !*wc.cta_abort) {
    *wc.cta_abort = 1;
    atomicExch(&g_tc_error, 1);
  }
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int x, int y, int z, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
               ::"l"(map), "r"(x), "r"(y), "r"(z), "r"(src) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until the bulk stores committed so far have finished READING shared memory
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem descriptor]^T, tf32 inputs, fp32 accumulate, M = 128; the
// descriptor is given as two 32-bit halves and the accumulate flag is a compile-time constant, so
// that the issuing thread spends one instruction per MMA (operands are loop-invariant registers).
template <bool kAccumulate>
__device__ __forceinline__ void mma_tf32_ts_lean(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                                 uint32_t idesc) {
  if (kAccumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "mov.b64 bd, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], bd, %4, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(0u)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\t"
        "setp.ne.b32 p, 0, 0;\n\t"
        "mov.b64 bd, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], bd, %4, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(0u)
        : "memory");
  }
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }


__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* v) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}

// Split of an fp32 value for the 3xTF32 product: hi = v with the 13 low mantissa bits cleared (the
// value the tensor core reads from an fp32 word anyway), lo = v - hi, exact in fp32 and below
// 2^-10 |v|.  lo is handed over as it is; the tensor core reads its leading 11 significant bits.
// What is lost per operand is below 2^-20 |v| (2^-22 |v| on average), against 2^-24 |v| for a
// rounded fp32 operation.  One logic and one floating-point instruction per value: the integer
// pipe is half as wide as the fp32 pipe on this architecture and an integer round-to-nearest of
// both parts (four integer instructions) made the conversion the bottleneck of the whole kernel.
__device__ __forceinline__ void split_tf32(float v, uint32_t& hi, uint32_t& lo) {
  hi = __float_as_uint(v) & 0xffffe000u;
  lo = __float_as_uint(fsub(v, __uint_as_float(hi)));
}

// Two fp32 values in one 64-bit register (element 0 in the low half) and the packed arithmetic of sm_100: each
// half is rounded to nearest exactly as the scalar instruction rounds it.
constexpr uint64_t kHalf2 = 0x3f0000003f000000ull;        // {0.5f, 0.5f}
constexpr uint64_t kMinusHalf2 = 0xbf000000bf000000ull;   // {-0.5f, -0.5f}
constexpr uint64_t kOne2 = 0x3f8000003f800000ull;         // {1.0f, 1.0f}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t pack2(uint32_t e0, uint32_t e1) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(e0), "r"(e1));
  return d;
}
// split_tf32 of both halves
__device__ __forceinline__ void split_tf32_pair(uint64_t v, uint64_t& hi, uint64_t& lo) {
  hi = v & 0xffffe000ffffe000ull;
  lo = sub2(v, hi);
}

// Byte offset of (row, 16-byte chunk) inside a 128-row x 128-byte tile with the 128-byte swizzle
// (chunk index XOR row mod 8); tiles are 1024-byte aligned.
__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);        // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                         // leading byte offset (unused with swizzle), bits [16,30)
  d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                         // descriptor version (Blackwell), bits [46,48)
  d |= (uint64_t)2 << 61;                         // layout type SWIZZLE_128B, bits [61,64)
  return d;
}

// ------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Encoded tensor maps are kept per (pointer, shape, box): a bound pass calls the same products on the same
// arena addresses over and over, and an encode costs a driver call each.
struct MapKey {
  const void* ptr;
  uint64_t d0, d1, d2, s0, s1;
  uint32_t b0, b1, b2, rank;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s0 == o.s0 && s1 == o.s1 && b0 == o.b0 && b1 == o.b1 &&
           b2 == o.b2 && rank == o.rank;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
    h ^= (k.d0 + 0x632BE59BD9B4E019ull) * 0xFF51AFD7ED558CCDull + (k.d1 << 17) + (k.d2 << 40) + k.s0 * 31 + k.s1 * 131 + k.b1 * 7 + k.b2 * 3 + k.rank;
    return (size_t)(h ^ (h >> 29));
  }
};
std::mutex g_map_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// fp32 tensor of up to three dimensions (innermost first; s0, s1: byte strides of dimensions 1 and 2), box
// {b0, b1, b2}, 128-byte swizzle, zero fill.
bool get_map(CUtensorMap* out, const float* ptr, uint32_t rank, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s0, uint64_t s1,
             uint32_t b0, uint32_t b1, uint32_t b2 = 1) {
  const MapKey key = {ptr, d0, d1, d2, s0, s1, b0, b1, b2, rank};
  {
    std::lock_guard<std::mutex> lk(g_map_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return true; }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {s0, s1};
  const cuuint32_t box[3] = {b0, b1, b2};
  const cuuint32_t estr[3] = {1, 1, 1};
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank, const_cast<float*>(ptr), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  std::lock_guard<std::mutex> lk(g_map_mu);
  if (g_maps.size() > 4096) g_maps.clear();   // callers with ever-changing addresses: start over
  g_maps.emplace(key, *out);
  return true;
}

