// Thread block clusters: the pieces shared by the row kernels that spread one
// row over several co-scheduled CTAs (layer_norm_cluster.cuh,
// softmax_cluster.cuh).
//
// The exchange: every warp adds up its lanes, then lane r < CL sends the
// warp's pair to CTA r's slot table ([rank][warp]) with st.async, the store
// that completes 8 bytes on CTA r's transaction barrier when it lands; every
// thread then waits on its own CTA's barrier (armed for CL * warps * 8 bytes)
// and adds the CL * warps pairs in table order.  Every CTA of a cluster adds
// the same table in the same order, so the sums are identical in all slices
// and from run to run.
//
// st.async is what makes this cheap.  The first version stored with
// st.shared::cluster and arrived with mbarrier.arrive.release.cluster (also
// tried: one message per CTA after a CTA-level reduction, and the hardware
// barrier.cluster.arrive.release / wait.acquire).  A release at cluster scope
// orders everything the thread has written before it, including the previous
// row's streaming stores to global memory, which under full HBM load take
// microseconds to be acknowledged: all three forms ran the LayerNorm kernels
// at 45-55 % of the copy rate, against 80-89 % with the exchange removed
// (wrong results, timing only).  The asynchronous store needs no fence - its
// data and its signal travel together.
//
// Slot tables and barriers are double buffered; a CTA can run at most one
// exchange ahead of the slowest CTA of its cluster (it needs that CTA's signal
// to pass its own wait), so a table is never overwritten before it has been
// read and a signal never lands in the wrong phase.
//
// Only this GPU's memory is touched; no multicast.  Every wait is bounded.
#pragma once
#include <mutex>

#include "common.cuh"
#include "pipe.cuh"

namespace fb {

constexpr int kClusterMax = 8;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of this CTA's shared-memory location `saddr` in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
// Asynchronous store of a pair into a peer's shared memory that signals 8 bytes on the peer's barrier when it lands.
__device__ __forceinline__ void cluster_store2_signal(uint32_t raddr, float a, float b, uint32_t rbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];" ::"r"(raddr),
               "f"(a), "f"(b), "r"(rbar)
               : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}

// Sums of a pair of floats over every thread of every CTA of the cluster.
// slots: [2][kClusterMax * T / 32] pairs and bars: [2] barriers in this CTA's shared memory.
template <int T>
struct ClusterSum {
  static constexpr int NW = T / 32;
  uint32_t to_slot;  // lane r < cl: shared::cluster address of row [my rank] of table 0 in CTA r
  uint32_t to_bar;   // lane r < cl: shared::cluster address of barrier 0 in CTA r

  __device__ __forceinline__ void init(float2* slots, uint64_t* bars, uint32_t cl) {
    const uint32_t lane = threadIdx.x & 31, me = cluster_ctarank();
    if (threadIdx.x == 0) {
      mbar_init(&bars[0], 1);
      mbar_init(&bars[1], 1);
      mbar_fence_init();
    }
    const uint32_t peer = lane < cl ? lane : 0;
    to_slot = cluster_map(smem_addr(slots + me * NW), peer);
    to_bar = cluster_map(smem_addr(bars), peer);
    cluster_barrier();  // every CTA's barriers exist before anyone signals them
  }
  // `count`: how many sums this CTA has taken before this one (the same number in every CTA of the
  // cluster).  Returns false when the wait gave up (a fault has been recorded).
  __device__ __forceinline__ bool sum(float2* slots, uint64_t* bars, uint32_t cl, uint32_t count, float& a, float& b,
                                      unsigned int* faults) const {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    const uint32_t buf = count & 1, parity = (count >> 1) & 1;
    if (threadIdx.x == 0) mbar_expect_tx(&bars[buf], cl * NW * (uint32_t)sizeof(float2));
    if (lane < cl)
      cluster_store2_signal(to_slot + (buf * kClusterMax * NW + warp) * (uint32_t)sizeof(float2), a, b,
                            to_bar + buf * (uint32_t)sizeof(uint64_t));
    if (!__all_sync(0xffffffffu, mbar_wait(&bars[buf], parity, faults))) return false;
    const float2* tab = slots + buf * kClusterMax * NW;
    float2 t = make_float2(0.0f, 0.0f);
    for (uint32_t j = lane; j < cl * NW; j += 32) {
      const float2 u = tab[j];
      t.x += u.x;
      t.y += u.y;
    }
    a = warp_sum(t.x);
    b = warp_sum(t.y);
    return true;
  }
  // The same exchange for the (maximum, sum of exponentials relative to it) pair of a softmax row:
  // pairs are merged as M = max(m1, m2), S = s1 exp(m1 - M) + s2 exp(m2 - M), with M taken as 0 in
  // the exponents while it is still -inf (an all -inf part contributes nothing instead of a NaN).
  // fmaxf semantics for the maximum: a NaN is dropped there and comes back through the sum.
  static __device__ __forceinline__ void merge_max_sum(float& m, float& s, float mo, float so) {
    const float mx = fmaxf(m, mo);
    const float ref = mx == -INFINITY ? 0.0f : mx;
    s = s * __expf(m - ref) + so * __expf(mo - ref);
    m = mx;
  }
  __device__ __forceinline__ bool max_sum(float2* slots, uint64_t* bars, uint32_t cl, uint32_t count, float& m, float& s,
                                          unsigned int* faults) const {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      merge_max_sum(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
    const uint32_t buf = count & 1, parity = (count >> 1) & 1;
    if (threadIdx.x == 0) mbar_expect_tx(&bars[buf], cl * NW * (uint32_t)sizeof(float2));
    if (lane < cl)
      cluster_store2_signal(to_slot + (buf * kClusterMax * NW + warp) * (uint32_t)sizeof(float2), m, s,
                            to_bar + buf * (uint32_t)sizeof(uint64_t));
    if (!__all_sync(0xffffffffu, mbar_wait(&bars[buf], parity, faults))) return false;
    const float2* tab = slots + buf * kClusterMax * NW;
    m = -INFINITY;
    s = 0.0f;
    for (uint32_t j = lane; j < cl * NW; j += 32) {
      const float2 u = tab[j];
      merge_max_sum(m, s, u.x, u.y);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      merge_max_sum(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
    return true;
  }
};

// Clusters of `cl` CTAs of `kernel` that fit the device at once: asked of the runtime the first
// time a (kernel, shared memory, cluster size) combination is launched on a device, then remembered.
static cudaError_t resident_clusters(const void* kernel, int threads, size_t smem, int cl, int* out) {
  struct Entry { const void* k; size_t smem; int cl, dev, n; };
  static std::mutex mu;
  static Entry table[64];
  static int used = 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  {
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i)
      if (table[i].k == kernel && table[i].smem == smem && table[i].cl == cl && table[i].dev == dev) {
        *out = table[i].n;
        return cudaSuccess;
      }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(device_info().sm_count * 8 / cl * cl));
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cl;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
  if (e != cudaSuccess) return e;
  if (n < 1) return cudaErrorLaunchOutOfResources;
  std::lock_guard<std::mutex> lock(mu);
  if (used < 64) table[used++] = Entry{kernel, smem, cl, dev, n};
  *out = n;
  return cudaSuccess;
}

template <typename... KArgs, typename... Args>
static cudaError_t launch_cluster(void (*kernel)(KArgs...), unsigned grid, int threads, size_t smem, int cl,
                                  bool pdl, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cl;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace fb
