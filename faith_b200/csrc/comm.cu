// Collective layer of the dim_in-sharded mode: an opaque communicator around ncclComm_t, the sharded
// relaxation (partial norms -> all-reduce -> apply, enqueued on one stream with no host round trip), and a
// one-shot all-reduce over NVLink for the small messages of that mode.
//
// The reference has no distributed code at all (it is single-GPU, single-process); the split itself follows
// from Bounds.concretize (Bounds.py:311-326): the dual norm of a column is a sum (p = inf: sum |w|, p = 2:
// sum w^2 before the root) or a maximum (p = 1) over dim_in, so each device reduces its own rows and the
// partial results are combined.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy already loaded into the process if there is one;
// FB_NCCL_LIB overrides the name), so the library has no link-time dependency on it and single-GPU users never
// touch it.
//
// One-shot all-reduce: the partial norms are 64-128 KB, far below the size at which a ring or tree pays; what
// counts is latency.  Every rank owns a receive area that its peers map through CUDA IPC.  A call writes the
// local vector into slot [rank] of EVERY peer's area with ordinary stores over NVLink (no multicast object, no
// TMA), publishes a flag per thread block behind a system-wide fence, waits -- bounded -- for the flags of all
// ranks in its own memory and sums the slots in rank order, which makes the result bit-identical on all ranks.
// Two slot sets alternate between calls: a rank can be at most one call ahead of its slowest peer, because it
// cannot finish call k+1 before that peer has entered it.
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "common.cuh"

namespace fb {
namespace {

// ---- the handful of NCCL entry points used here (ABI of nccl.h, stable across 2.x) ----------------------------
typedef void* ncclComm_t;
struct NcclUniqueId { char internal[128]; };
enum { kNcclSuccess = 0, kNcclInProgress = 7 };
enum { kNcclFloat32 = 7, kNcclChar = 0 };
enum { kNcclSum = 0, kNcclMax = 2 };
struct NcclApi {
  int (*GetUniqueId)(NcclUniqueId*);
  int (*CommInitRank)(ncclComm_t*, int, NcclUniqueId, int);
  int (*CommDestroy)(ncclComm_t);
  int (*CommAbort)(ncclComm_t);
  int (*CommGetAsyncError)(ncclComm_t, int*);
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t);
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t);
  const char* (*GetErrorString)(int);
  bool ok;
};

thread_local std::string t_comm_error;

const NcclApi& nccl() {
  static NcclApi api = {};
  static std::once_flag once;
  std::call_once(once, []() {
    const char* name = std::getenv("FB_NCCL_LIB");
    void* h = nullptr;
    if (name == nullptr || name[0] == 0) {
      name = "libnccl.so.2";
      h = dlopen(name, RTLD_NOW | RTLD_NOLOAD);   // the copy the process already uses, if any
    }
    if (h == nullptr) h = dlopen(name, RTLD_NOW);
    if (h == nullptr) return;
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(dlsym(h, "ncclCommAbort"));
    api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(dlsym(h, "ncclCommGetAsyncError"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(h, "ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.CommAbort && api.CommGetAsyncError &&
             api.AllReduce && api.AllGather && api.GetErrorString;
  });
  return api;
}

int nccl_fail(const char* what, int rc) {
  const NcclApi& n = nccl();
  t_comm_error = std::string(what) + ": " + (n.ok && n.GetErrorString ? n.GetErrorString(rc) : "NCCL error") + " (" +
                 std::to_string(rc) + ")";
  return FB_ERR_NCCL;
}
#define FB_NCCL_OK(what, expr)                       \
  do {                                               \
    const int fb_n_ = (expr);                        \
    if (fb_n_ != kNcclSuccess) return nccl_fail(what, fb_n_); \
  } while (0)

constexpr int kMaxRanks = 8;
constexpr int kMaxBlocks = 64;          // thread blocks of the one-shot kernel = flags per (slot set, rank)
constexpr int kOneShotThreads = 256;

struct PeerPtrs {
  float* recv[kMaxRanks];
  unsigned int* flags[kMaxRanks];
};

// One-shot all-reduce (see the file header).  in / out: n floats (may alias); slot layout of a receive area:
// [set (2)][source rank (world)][cap floats]; flags: [set][source rank][kMaxBlocks].  op: 0 sum, 1 max.
// A wait that runs out (wait_ns) sets bit 3 of *status and the block returns without writing its part of `out`.
__global__ void __launch_bounds__(kOneShotThreads)
oneshot_allreduce_kernel(const float* in, float* out, int64_t n, int op, PeerPtrs peers, int rank, int world,
                         unsigned int epoch, int64_t cap, int* __restrict__ status, unsigned long long wait_ns) {
  __shared__ int s_fail;
  const int b = blockIdx.x;
  const int set = (int)(epoch & 1u);
  int64_t chunk = (n + gridDim.x - 1) / gridDim.x;
  chunk = (chunk + 3) / 4 * 4;
  const int64_t lo = (int64_t)b * chunk;
  const int64_t hi = lo + chunk < n ? lo + chunk : n;
  if (threadIdx.x == 0) s_fail = 0;
  // 1. my chunk into slot [rank] of every rank's area (my own included)
  for (int r = 0; r < world; ++r) {
    float* dst = peers.recv[r] + ((int64_t)set * world + rank) * cap;
    for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) dst[i] = in[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) {
    volatile unsigned int* f = peers.flags[threadIdx.x] + ((int64_t)set * world + rank) * kMaxBlocks + b;
    *f = epoch;
  }
  // 2. wait for chunk b of every rank in my own memory (bounded)
  if (threadIdx.x < world) {
    volatile unsigned int* f = peers.flags[rank] + ((int64_t)set * world + threadIdx.x) * kMaxBlocks + b;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    bool ok = false;
    for (;;) {
      if (*f == epoch) { ok = true; break; }
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > wait_ns) break;
      __nanosleep(200);
    }
    if (!ok) s_fail = 1;
  }
  __syncthreads();
  if (s_fail) {
    if (threadIdx.x == 0 && status != nullptr) atomicOr(status, 8);
    return;
  }
  __threadfence_system();
  // 3. reduce in rank order (the same order on every rank: identical bits everywhere)
  const float* mine = peers.recv[rank] + (int64_t)set * world * cap;
  for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float acc = __ldcg(mine + i);
    for (int r = 1; r < world; ++r) {
      const float v = __ldcg(mine + (int64_t)r * cap + i);
      acc = op == 0 ? acc + v : fmaxf(acc, v);
    }
    out[i] = acc;
  }
}

// l = lb - eps * finish(norm_l), u = ub + eps * finish(norm_u) from all-reduced unfinished norms (one word block).
__global__ void __launch_bounds__(256)
concretize_from_partials_kernel(const float* __restrict__ lb, const float* __restrict__ ub, const float* __restrict__ nl,
                                const float* __restrict__ nu, float* __restrict__ l, float* __restrict__ u, int64_t n,
                                int p, float eps) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    l[i] = fadd(lb[i], fmul(-eps, norm_finish(p, nl[i])));
    u[i] = fadd(ub[i], fmul(eps, norm_finish(p, nu[i])));
  }
}

}  // namespace
}  // namespace fb

struct fb_comm {
  fb::ncclComm_t nccl;
  int rank, world, device;
  // one-shot exchange (optional)
  int64_t cap;                 // floats per slot; 0 = not set up
  char* base;                  // own allocation: receive area, flags, staging
  fb::PeerPtrs peers;
  void* peer_base[fb::kMaxRanks];
  unsigned int epoch;
  int* status;                 // device word inside the allocation (bit 3: a peer wait expired)
  unsigned long long wait_ns;
};

using namespace fb;

extern "C" const char* fb_comm_last_error(void) { return t_comm_error.c_str(); }

extern "C" int fb_comm_unique_id(void* id128) {
  if (!id128) return FB_ERR_ARG;
  const NcclApi& n = nccl();
  if (!n.ok) {
    t_comm_error = "libnccl.so.2 could not be loaded";
    return FB_ERR_NCCL;
  }
  NcclUniqueId id;
  FB_NCCL_OK("ncclGetUniqueId", n.GetUniqueId(&id));
  std::memcpy(id128, &id, sizeof(id));
  return FB_OK;
}

namespace {
int64_t align_up64(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Receive area + flags + status word + staging for the handle exchange, mapped into every peer through CUDA IPC.
int setup_oneshot(fb_comm* c, int64_t cap) {
  const NcclApi& n = nccl();
  const int64_t recv_bytes = align_up64(2 * (int64_t)c->world * cap * 4, 256);
  const int64_t flag_bytes = align_up64(2 * (int64_t)c->world * kMaxBlocks * 4, 256);
  const int64_t stage_bytes = align_up64((int64_t)c->world * sizeof(cudaIpcMemHandle_t), 256);
  FB_CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&c->base), recv_bytes + flag_bytes + 256 + stage_bytes));
  FB_CUDA_OK(cudaMemset(c->base, 0, recv_bytes + flag_bytes + 256 + stage_bytes));
  c->status = reinterpret_cast<int*>(c->base + recv_bytes + flag_bytes);
  char* stage = c->base + recv_bytes + flag_bytes + 256;
  cudaIpcMemHandle_t mine;
  FB_CUDA_OK(cudaIpcGetMemHandle(&mine, c->base));
  FB_CUDA_OK(cudaMemcpy(stage + (size_t)c->rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice));
  FB_NCCL_OK("ncclAllGather (IPC handles)",
             n.AllGather(stage + (size_t)c->rank * sizeof(mine), stage, sizeof(mine), kNcclChar, c->nccl, nullptr));
  FB_CUDA_OK(cudaStreamSynchronize(nullptr));
  cudaIpcMemHandle_t all[kMaxRanks];
  FB_CUDA_OK(cudaMemcpy(all, stage, (size_t)c->world * sizeof(mine), cudaMemcpyDeviceToHost));
  for (int r = 0; r < c->world; ++r) {
    void* p = c->base;
    if (r != c->rank) FB_CUDA_OK(cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess));
    c->peer_base[r] = p;
    c->peers.recv[r] = reinterpret_cast<float*>(p);
    c->peers.flags[r] = reinterpret_cast<unsigned int*>(static_cast<char*>(p) + recv_bytes);
  }
  // nobody may write into a peer before every rank has zeroed its area and mapped the others: one more collective
  FB_NCCL_OK("ncclAllReduce (setup barrier)",
             n.AllReduce(stage, stage, 1, kNcclFloat32, kNcclMax, c->nccl, nullptr));
  FB_CUDA_OK(cudaStreamSynchronize(nullptr));
  c->cap = cap;
  c->epoch = 0;
  return FB_OK;
}
}  // namespace

extern "C" int fb_comm_create(fb_comm** out, const void* id128, int rank, int world, int64_t oneshot_floats) {
  if (!out || !id128 || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || oneshot_floats < 0) return FB_ERR_ARG;
  const NcclApi& n = nccl();
  if (!n.ok) {
    t_comm_error = "libnccl.so.2 could not be loaded";
    return FB_ERR_NCCL;
  }
  fb_comm* c = new fb_comm();
  std::memset(c, 0, sizeof(*c));
  c->rank = rank;
  c->world = world;
  c->wait_ns = 2000000000ull;   // 2 s
  NcclUniqueId id;
  std::memcpy(&id, id128, sizeof(id));
  int rc = n.CommInitRank(&c->nccl, world, id, rank);
  if (rc != kNcclSuccess) {
    delete c;
    return nccl_fail("ncclCommInitRank", rc);
  }
  cudaGetDevice(&c->device);
  if (oneshot_floats > 0 && world > 1) {
    const int s = setup_oneshot(c, align_up64(oneshot_floats, 64));
    if (s != FB_OK) {
      n.CommAbort(c->nccl);
      if (c->base) cudaFree(c->base);
      delete c;
      return s;
    }
  }
  *out = c;
  return FB_OK;
}

extern "C" int fb_comm_destroy(fb_comm* c) {
  if (!c) return FB_ERR_ARG;
  const NcclApi& n = nccl();
  if (c->base) {
    cudaDeviceSynchronize();
    for (int r = 0; r < c->world; ++r)
      if (r != c->rank && c->peer_base[r]) cudaIpcCloseMemHandle(c->peer_base[r]);
    cudaFree(c->base);
  }
  const int rc = c->nccl ? n.CommDestroy(c->nccl) : kNcclSuccess;
  delete c;
  return rc == kNcclSuccess ? FB_OK : nccl_fail("ncclCommDestroy", rc);
}

extern "C" int fb_comm_abort(fb_comm* c) {
  if (!c) return FB_ERR_ARG;
  const NcclApi& n = nccl();
  const int rc = c->nccl ? n.CommAbort(c->nccl) : kNcclSuccess;
  c->nccl = nullptr;
  return rc == kNcclSuccess ? FB_OK : nccl_fail("ncclCommAbort", rc);
}

extern "C" int fb_comm_info(const fb_comm* c, int* rank, int* world, int64_t* oneshot_floats) {
  if (!c) return FB_ERR_ARG;
  if (rank) *rank = c->rank;
  if (world) *world = c->world;
  if (oneshot_floats) *oneshot_floats = c->cap;
  return FB_OK;
}

extern "C" int fb_comm_set_wait_ns(fb_comm* c, uint64_t ns) {
  if (!c || ns == 0) return FB_ERR_ARG;
  c->wait_ns = ns;
  return FB_OK;
}

// Non-blocking health check of the NCCL side; with `sync` != 0 also waits for the stream-ordered work of the
// device and reads (and clears) the status word of the one-shot path.
extern "C" int fb_comm_check(fb_comm* c, int sync) {
  if (!c) return FB_ERR_ARG;
  const NcclApi& n = nccl();
  if (c->nccl == nullptr) {
    t_comm_error = "communicator was aborted";
    return FB_ERR_NCCL;
  }
  int async = kNcclSuccess;
  FB_NCCL_OK("ncclCommGetAsyncError", n.CommGetAsyncError(c->nccl, &async));
  if (async != kNcclSuccess && async != kNcclInProgress) return nccl_fail("asynchronous NCCL error", async);
  if (sync && c->status != nullptr) {
    FB_CUDA_OK(cudaDeviceSynchronize());
    int v = 0;
    FB_CUDA_OK(cudaMemcpy(&v, c->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) {
      FB_CUDA_OK(cudaMemset(c->status, 0, sizeof(int)));
      t_comm_error = "one-shot all-reduce: the wait for a peer expired";
      return FB_ERR_TIMEOUT;
    }
  }
  return FB_OK;
}

// buf: n floats, reduced in place over the ranks.  op: 0 sum, 1 max.  algo: 0 NCCL, 1 one-shot over NVLink
// (needs oneshot_floats >= n at creation, else FB_ERR_WORKSPACE).
extern "C" int fb_allreduce_f32(fb_comm* c, float* buf, int64_t n, int op, int algo, void* stream) {
  if (!c || !buf || n < 0 || (op != 0 && op != 1) || (algo != 0 && algo != 1)) return FB_ERR_ARG;
  if (n == 0 || c->world == 1) return FB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (algo == 1) {
    if (c->cap < n) return FB_ERR_WORKSPACE;
    ++c->epoch;
    if (c->epoch == 0) ++c->epoch;
    int64_t blocks = ceil_div(n, 4 * kOneShotThreads);
    if (blocks > kMaxBlocks) blocks = kMaxBlocks;
    oneshot_allreduce_kernel<<<(unsigned)blocks, kOneShotThreads, 0, st>>>(buf, buf, n, op, c->peers, c->rank, c->world,
                                                                           c->epoch, c->cap, c->status, c->wait_ns);
    FB_LAUNCH_OK();
    return FB_OK;
  }
  const NcclApi& nc = nccl();
  if (c->nccl == nullptr) {
    t_comm_error = "communicator was aborted";
    return FB_ERR_NCCL;
  }
  FB_NCCL_OK("ncclAllReduce", nc.AllReduce(buf, buf, (size_t)n, kNcclFloat32, op == 0 ? kNcclSum : kNcclMax, c->nccl, st));
  fb::count_launches(1);
  int async = kNcclSuccess;
  FB_NCCL_OK("ncclCommGetAsyncError", nc.CommGetAsyncError(c->nccl, &async));
  if (async != kNcclSuccess && async != kNcclInProgress) return nccl_fail("asynchronous NCCL error", async);
  return FB_OK;
}

extern "C" int fb_relax_sharded_f32(fb_comm* c, int algo, int op, const float* lw, const float* uw, const float* lb,
                                    const float* ub, float* out_lw, float* out_uw, float* out_lb, float* out_ub,
                                    float* part_ws, int64_t rows, int Di_local, int Do, int words, int p, float eps,
                                    int* violation, void* stream) {
  if (!part_ws) return FB_ERR_ARG;
  if (words != 1) return FB_ERR_SHAPE;   // one norm over the whole dim_in axis: several word blocks would need one partial each
  const int64_t n = rows * Do;
  float* part_l = part_ws;
  float* part_u = part_ws + n;
  int rc = fb_norm_partials_f32(lw, uw, part_l, part_u, rows, Di_local, Do, p, stream);
  if (rc != FB_OK) return rc;
  if (c != nullptr) {
    rc = fb_allreduce_f32(c, part_ws, 2 * n, p == FB_P1 ? 1 : 0, algo, stream);
    if (rc != FB_OK) return rc;
  }
  return fb_relax_with_norms_f32(op, lw, uw, lb, ub, part_l, part_u, out_lw, out_uw, out_lb, out_ub, rows, Di_local, Do, p,
                                 eps, violation, stream);
}

extern "C" int fb_concretize_sharded_f32(fb_comm* c, int algo, const float* lw, const float* uw, const float* lb,
                                         const float* ub, float* l, float* u, float* part_ws, int64_t rows,
                                         int Di_local, int Do, int words, int p, float eps, void* stream) {
  if (!part_ws || !lb || !ub || !l || !u) return FB_ERR_ARG;
  if (words != 1) return FB_ERR_SHAPE;
  const int64_t n = rows * Do;
  int rc = fb_norm_partials_f32(lw, uw, part_ws, part_ws + n, rows, Di_local, Do, p, stream);
  if (rc != FB_OK) return rc;
  if (c != nullptr) {
    rc = fb_allreduce_f32(c, part_ws, 2 * n, p == FB_P1 ? 1 : 0, algo, stream);
    if (rc != FB_OK) return rc;
  }
  if (n == 0) return FB_OK;
  const int64_t want = ceil_div(n, 256), cap = (int64_t)device_info().sms * 8;
  concretize_from_partials_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, (cudaStream_t)stream>>>(
      lb, ub, part_ws, part_ws + n, l, u, n, p, eps);
  FB_LAUNCH_OK();
  return FB_OK;
}
