/* A stand-in for libnccl used by the CPU tests of the gradient exchange
 * (libferro_b200 loads whatever FB_NCCL_LIBRARY names).  It exports the NCCL
 * entry points the library binds, works on HOST memory so no GPU is needed,
 * and fails on request: fake_nccl_fail(which, code) arms one entry point.
 *
 * ncclAllReduce "sums" as if every rank held the caller's values: each
 * element is multiplied by the world size, which lets a test check the
 * pointer / count plumbing and the sum-then-divide contract.
 *
 * Test infrastructure only: nothing in the product loads this file unless
 * the environment variable says so. */
#include <stddef.h>
#include <string.h>

typedef int ncclResult_t; /* 0 = ncclSuccess */
typedef struct fake_comm { int world, rank; } fake_comm;
typedef struct { char internal[128]; } ncclUniqueId;

enum { F_INIT = 1, F_ALLREDUCE = 2, F_ASYNC = 3, F_GROUP_END = 4, F_UNIQUE_ID = 5 };
static int g_fail_which = 0, g_fail_code = 0;
static int g_allreduce_calls = 0, g_aborts = 0, g_destroys = 0;
static fake_comm g_comms[16];
static int g_ncomms = 0;

__attribute__((visibility("default"))) void fake_nccl_fail(int which, int code) { g_fail_which = which; g_fail_code = code; }
__attribute__((visibility("default"))) int fake_nccl_count(int what) {
  return what == 0 ? g_allreduce_calls : what == 1 ? g_aborts : g_destroys;
}

#define API __attribute__((visibility("default")))
API ncclResult_t ncclGetVersion(int* v) { *v = 99999; return 0; }
API ncclResult_t ncclGetUniqueId(ncclUniqueId* id) {
  if (g_fail_which == F_UNIQUE_ID) return g_fail_code;
  memset(id, 0x5a, sizeof(*id));
  return 0;
}
API ncclResult_t ncclCommInitRank(void** comm, int nranks, ncclUniqueId id, int rank) {
  (void)id;
  if (g_fail_which == F_INIT) return g_fail_code;
  if (g_ncomms >= 16) return 3;
  g_comms[g_ncomms].world = nranks;
  g_comms[g_ncomms].rank = rank;
  *comm = &g_comms[g_ncomms++];
  return 0;
}
API ncclResult_t ncclCommDestroy(void* comm) { (void)comm; ++g_destroys; return 0; }
API ncclResult_t ncclCommAbort(void* comm) { (void)comm; ++g_aborts; return 0; }
API ncclResult_t ncclCommGetAsyncError(void* comm, ncclResult_t* async) {
  (void)comm;
  *async = (g_fail_which == F_ASYNC) ? g_fail_code : 0;
  return 0;
}
API ncclResult_t ncclAllReduce(const void* send, void* recv, size_t count, int dtype, int op, void* comm, void* stream) {
  (void)stream;
  if (g_fail_which == F_ALLREDUCE) return g_fail_code;
  if (dtype != 7 /* ncclFloat32 */ || op != 0 /* ncclSum */) return 4;
  const float* s = (const float*)send;
  float* r = (float*)recv;
  const int world = ((fake_comm*)comm)->world;
  for (size_t i = 0; i < count; ++i) r[i] = s[i] * (float)world;
  ++g_allreduce_calls;
  return 0;
}
API ncclResult_t ncclGroupStart(void) { return 0; }
API ncclResult_t ncclGroupEnd(void) { return g_fail_which == F_GROUP_END ? g_fail_code : 0; }
API const char* ncclGetErrorString(ncclResult_t r) {
  switch (r) {
    case 0: return "no error";
    case 1: return "unhandled cuda error";
    case 2: return "unhandled system error";
    case 3: return "internal error";
    case 4: return "invalid argument";
    case 5: return "invalid usage";
    case 6: return "remote process exited or there was a network error";
    case 7: return "NCCL operation in progress";
    default: return "unknown result code";
  }
}
