// The gradient exchange of the data-parallel step: an NCCL communicator handle
// and the bucket all-reduce behind ferro's one collective seam, Ddp::average
// (crates/ferro-core/src/ddp.rs:127-160), which today pulls every replica's
// gradients to the host, sums them and divides by the replica count.
//
// One process per GPU.  The exchange is ncclAllReduce(sum) in place on a flat
// f32 bucket, on the stream the caller gives (a side stream, so that it
// overlaps the rest of backward); the division by the replica count is either
// folded into the fused optimizer (fb_adamw_multi's g_scale) or done here
// with an IEEE divide, which is ferro's `s / n` (ddp.rs:154).  NCCL moves the
// data over NVLink / NVSwitch and lands it in this GPU's memory: no kernel of
// this library reads a peer's memory.
//
// NCCL is bound at run time (dlopen), not at link time: the library loads and
// every other entry point works on a machine without NCCL, a world of one
// needs no NCCL at all, and a host process that already carries a libnccl
// (torch does) shares that copy instead of loading a second one.  The
// FB_NCCL_LIBRARY environment variable names the file to load instead of
// "libnccl.so.2"; the tests use it to put a stand-in behind this code that
// returns error codes on request, so every failure path runs without a GPU.
//
// Failure handling: nothing here waits on the device or on a peer.  A failed
// NCCL call returns FB_ERR_COMM with NCCL's own text and marks the handle
// broken, after which every exchange on it is refused before any launch;
// fb_ddp_poll() reads ncclCommGetAsyncError so the host can notice a dead
// peer between steps and call fb_ddp_comm_abort() instead of enqueueing a
// collective that would never finish.
#include <dlfcn.h>
#include <nccl.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace fb {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetVersion)(int*) = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  char path[256] = "";
};

static NcclApi g_nccl;
static std::mutex g_nccl_mu;

// Binds the NCCL entry points once per process.  Returns FB_OK or FB_ERR_COMM.
static int nccl_api(const NcclApi** out) {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (!g_nccl.handle) {
    const char* env = getenv("FB_NCCL_LIBRARY");
    const char* name = (env && *env) ? env : "libnccl.so.2";
    void* h = dlopen(name, RTLD_NOW | RTLD_LOCAL);
    if (!h) return fail(FB_ERR_COMM, "fb_ddp: cannot load %s: %s", name, dlerror());
    NcclApi a;
    a.handle = h;
    snprintf(a.path, sizeof(a.path), "%s", name);
    bool ok = true;
    auto sym = [&](const char* s) {
      void* p = dlsym(h, s);
      if (!p) ok = false;
      return p;
    };
    a.GetVersion = reinterpret_cast<decltype(a.GetVersion)>(sym("ncclGetVersion"));
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
    a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(sym("ncclCommAbort"));
    a.CommGetAsyncError = reinterpret_cast<decltype(a.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
    a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(sym("ncclGroupStart"));
    a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(sym("ncclGroupEnd"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
    if (!ok) {
      dlclose(h);
      return fail(FB_ERR_COMM, "fb_ddp: %s lacks an NCCL entry point this library needs", name);
    }
    g_nccl = a;
  }
  *out = &g_nccl;
  return FB_OK;
}

static int nccl_fail(const NcclApi* api, ncclResult_t r, const char* what) {
  return fail(FB_ERR_COMM, "NCCL error: %s (%d) at %s", api->GetErrorString(r), (int)r, what);
}

// out[i] = out[i] / d with an IEEE divide: ferro's `s / n` (ddp.rs:154).
__global__ void __launch_bounds__(256) divide_kernel(float* __restrict__ p, float d, uint64_t n) {
  const uint64_t n4 = n / 4;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 v = reinterpret_cast<float4*>(p)[i];
    v.x = __fdiv_rn(v.x, d); v.y = __fdiv_rn(v.y, d); v.z = __fdiv_rn(v.z, d); v.w = __fdiv_rn(v.w, d);
    reinterpret_cast<float4*>(p)[i] = v;
  }
  for (uint64_t i = n4 * 4 + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    p[i] = __fdiv_rn(p[i], d);
}
__global__ void __launch_bounds__(256) divide_scalar_kernel(float* __restrict__ p, float d, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = __fdiv_rn(p[i], d);
}

}  // namespace fb

// The handle.  `broken` is sticky: set by the first NCCL failure seen on this
// communicator (a failed call or an asynchronous error found by a poll).
struct fb_ddp_comm {
  ncclComm_t comm;
  int rank, world;
  std::atomic<int> broken;
  const fb::NcclApi* api;
};

using namespace fb;

extern "C" {

int fb_ddp_unique_id(void* id) {
  if (!id) return fail(FB_ERR_INVALID_ARG, "fb_ddp_unique_id: null id");
  const NcclApi* api;
  if (int rc = nccl_api(&api)) return rc;
  static_assert(sizeof(ncclUniqueId) == FB_DDP_UNIQUE_ID_BYTES, "unique id size");
  ncclUniqueId u;
  const ncclResult_t r = api->GetUniqueId(&u);
  if (r != ncclSuccess) return nccl_fail(api, r, "ncclGetUniqueId");
  memcpy(id, &u, sizeof(u));
  return FB_OK;
}

int fb_ddp_comm_init(const void* id, int rank, int world, fb_ddp_comm** out) {
  if (!out) return fail(FB_ERR_INVALID_ARG, "fb_ddp_comm_init: null handle slot");
  *out = nullptr;
  if (world < 1 || rank < 0 || rank >= world)
    return fail(FB_ERR_INVALID_ARG, "fb_ddp_comm_init: rank %d of %d", rank, world);
  fb_ddp_comm* c = new fb_ddp_comm{nullptr, rank, world, {0}, nullptr};
  if (world > 1) {
    if (!id) {
      delete c;
      return fail(FB_ERR_INVALID_ARG, "fb_ddp_comm_init: null id");
    }
    if (int rc = nccl_api(&c->api)) {
      delete c;
      return rc;
    }
    ncclUniqueId u;
    memcpy(&u, id, sizeof(u));
    const ncclResult_t r = c->api->CommInitRank(&c->comm, world, u, rank);
    if (r != ncclSuccess) {
      const int rc = nccl_fail(c->api, r, "ncclCommInitRank");
      delete c;
      return rc;
    }
  }
  *out = c;
  return FB_OK;
}

int fb_ddp_rank(const fb_ddp_comm* c) { return c ? c->rank : -1; }
int fb_ddp_world(const fb_ddp_comm* c) { return c ? c->world : 0; }

int fb_ddp_nccl_version(void) {
  const NcclApi* api;
  if (nccl_api(&api)) return -1;
  int v = 0;
  return api->GetVersion(&v) == ncclSuccess ? v : -1;
}

static int ddp_usable(const char* name, fb_ddp_comm* c) {
  if (!c) return fail(FB_ERR_INVALID_ARG, "%s: null communicator", name);
  if (c->broken.load(std::memory_order_acquire))
    return fail(FB_ERR_COMM, "%s: the communicator has failed before (see fb_ddp_poll); abort it and build a new one", name);
  return FB_OK;
}

int fb_ddp_allreduce_bucket(fb_ddp_comm* c, fb_stream_t stream, float* bucket, uint64_t n) {
  const char* name = "fb_ddp_allreduce_bucket";
  if (int rc = ddp_usable(name, c)) return rc;
  if (n == 0 || c->world == 1) return FB_OK;  // the sum over one replica is the gradient itself
  if (!bucket) return fail(FB_ERR_INVALID_ARG, "%s: null bucket", name);
  const ncclResult_t r = c->api->AllReduce(bucket, bucket, (size_t)n, ncclFloat32, ncclSum, c->comm, stream);
  if (r != ncclSuccess) {
    c->broken.store(1, std::memory_order_release);
    return nccl_fail(c->api, r, "ncclAllReduce");
  }
  count_launch();
  return FB_OK;
}

int fb_ddp_allreduce_buckets(fb_ddp_comm* c, fb_stream_t stream, float* const* buckets, const uint64_t* lens,
                             int n_buckets) {
  const char* name = "fb_ddp_allreduce_buckets";
  if (int rc = ddp_usable(name, c)) return rc;
  if (n_buckets < 0 || (n_buckets > 0 && (!buckets || !lens)))
    return fail(FB_ERR_INVALID_ARG, "%s: bad bucket list", name);
  for (int i = 0; i < n_buckets; ++i)
    if (lens[i] && !buckets[i]) return fail(FB_ERR_INVALID_ARG, "%s: null bucket %d", name, i);
  if (c->world == 1 || n_buckets == 0) return FB_OK;
  // One NCCL group: the collectives are fused into one launch where NCCL can.
  ncclResult_t r = c->api->GroupStart();
  const char* where = "ncclGroupStart";
  int issued = 0;
  if (r == ncclSuccess) {
    for (int i = 0; i < n_buckets && r == ncclSuccess; ++i) {
      if (!lens[i]) continue;
      r = c->api->AllReduce(buckets[i], buckets[i], (size_t)lens[i], ncclFloat32, ncclSum, c->comm, stream);
      where = "ncclAllReduce";
      ++issued;
    }
    const ncclResult_t e = c->api->GroupEnd();
    if (r == ncclSuccess && e != ncclSuccess) {
      r = e;
      where = "ncclGroupEnd";
    }
  }
  if (r != ncclSuccess) {
    c->broken.store(1, std::memory_order_release);
    return nccl_fail(c->api, r, where);
  }
  if (issued) count_launch();
  return FB_OK;
}

int fb_ddp_average_bucket(fb_ddp_comm* c, fb_stream_t stream, float* bucket, uint64_t n) {
  const char* name = "fb_ddp_average_bucket";
  if (int rc = ddp_usable(name, c)) return rc;
  if (n == 0 || c->world == 1) return FB_OK;  // x / 1 = x
  if (int rc = fb_ddp_allreduce_bucket(c, stream, bucket, n)) return rc;
  const unsigned grid = grid_for((n / 4 + 255) / 256 + 1, 8);
  if (aligned16(bucket)) divide_kernel<<<grid, 256, 0, stream>>>(bucket, (float)c->world, n);
  else divide_scalar_kernel<<<grid, 256, 0, stream>>>(bucket, (float)c->world, n);
  FB_LAUNCHED(name);
  return FB_OK;
}

int fb_ddp_poll(fb_ddp_comm* c) {
  if (!c) return fail(FB_ERR_INVALID_ARG, "fb_ddp_poll: null communicator");
  if (c->world == 1) return FB_OK;
  if (c->broken.load(std::memory_order_acquire))
    return fail(FB_ERR_COMM, "fb_ddp_poll: the communicator has failed before");
  ncclResult_t async = ncclSuccess;
  const ncclResult_t r = c->api->CommGetAsyncError(c->comm, &async);
  if (r != ncclSuccess) {
    c->broken.store(1, std::memory_order_release);
    return nccl_fail(c->api, r, "ncclCommGetAsyncError");
  }
  if (async == ncclInProgress) return FB_OK;  // a non-blocking operation still running is not a failure
  if (async != ncclSuccess) {
    c->broken.store(1, std::memory_order_release);
    return nccl_fail(c->api, async, "an earlier collective (asynchronous error)");
  }
  return FB_OK;
}

int fb_ddp_comm_abort(fb_ddp_comm* c) {
  if (!c) return FB_OK;
  int rc = FB_OK;
  if (c->world > 1 && c->comm) {
    const ncclResult_t r = c->api->CommAbort(c->comm);
    if (r != ncclSuccess) rc = nccl_fail(c->api, r, "ncclCommAbort");
  }
  delete c;
  return rc;
}

int fb_ddp_comm_destroy(fb_ddp_comm* c) {
  if (!c) return FB_OK;
  int rc = FB_OK;
  if (c->world > 1 && c->comm) {
    // A communicator that has failed cannot be flushed; tear it down instead.
    const bool broken = c->broken.load(std::memory_order_acquire) != 0;
    const ncclResult_t r = broken ? c->api->CommAbort(c->comm) : c->api->CommDestroy(c->comm);
    if (r != ncclSuccess) rc = nccl_fail(c->api, r, broken ? "ncclCommAbort" : "ncclCommDestroy");
  }
  delete c;
  return rc;
}

}  // extern "C"
