/* A stand-in for libnccl.so.2 for tests on machines without a GPU: the eight entry points the library binds,
 * doing nothing, with failures injected through environment variables.  Built by tests/test_comm_cpu.py with gcc.
 *   FAKE_NCCL_FAIL=init|allreduce|allgather   that call returns ncclSystemError (2)
 *   FAKE_NCCL_ASYNC_AFTER=n                   ncclCommGetAsyncError reports ncclRemoteError (6) from its n-th call on
 */
#include <stdlib.h>
#include <string.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef void* ncclComm_t;
static int polls = 0;
static int dummy_comm;

static int fails(const char* what) {
  const char* f = getenv("FAKE_NCCL_FAIL");
  return f != NULL && strcmp(f, what) == 0;
}

int ncclGetUniqueId(ncclUniqueId* id) {
  memset(id, 0, sizeof(*id));
  memcpy(id->internal, "FAKE-NCCL-ID", 12);
  return 0;
}
int ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank) {
  if (fails("init")) return 2;
  if (memcmp(id.internal, "FAKE-NCCL-ID", 12) != 0 || rank < 0 || rank >= nranks) return 4; /* ncclInvalidArgument */
  *comm = &dummy_comm;
  return 0;
}
int ncclCommDestroy(ncclComm_t comm) { return comm == &dummy_comm ? 0 : 4; }
int ncclCommAbort(ncclComm_t comm) { return comm == &dummy_comm ? 0 : 4; }
int ncclCommGetAsyncError(ncclComm_t comm, int* async) {
  const char* a = getenv("FAKE_NCCL_ASYNC_AFTER");
  ++polls;
  *async = (a != NULL && polls >= atoi(a)) ? 6 : 0;
  return comm == &dummy_comm ? 0 : 4;
}
int ncclAllReduce(const void* s, void* r, size_t n, int dt, int op, ncclComm_t comm, void* stream) {
  (void)s; (void)r; (void)n; (void)dt; (void)op; (void)stream;
  if (fails("allreduce")) return 2;
  return comm == &dummy_comm ? 0 : 4;
}
int ncclAllGather(const void* s, void* r, size_t n, int dt, ncclComm_t comm, void* stream) {
  (void)s; (void)r; (void)n; (void)dt; (void)stream;
  if (fails("allgather")) return 2;
  return comm == &dummy_comm ? 0 : 4;
}
const char* ncclGetErrorString(int rc) {
  switch (rc) {
    case 0: return "no error";
    case 2: return "unhandled system error";
    case 4: return "invalid argument";
    case 6: return "remote process exited or there was a network error";
    default: return "unknown result code";
  }
}
