// Row staging through shared memory with bulk asynchronous copies (the 1-D
// form of TMA, cp.async.bulk) and mbarrier completion, for kernels that walk
// rows with a persistent CTA.  One elected thread keeps STAGES rows in flight
// per CTA, so the number of bytes outstanding to HBM does not depend on how
// many registers the compute part needs or which phase it is in.
//
// No multicast, no cluster: every copy is global -> this CTA's shared memory.
// Every wait is bounded: a barrier that does not complete within the spin
// limit records a fault in a device status word and makes the kernel stop
// issuing work and return (fb_device_faults() reads the word).
#pragma once
#include "common.cuh"

namespace fb {

// Device status word (one per device, owned by api.cu): number of bounded
// waits that gave up.  Kernels receive its address as an argument.
unsigned int* fault_word();  // host: device address of the word on the current device, or nullptr

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  // Make the initialised barriers visible to the async proxy.
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity), "r"(20000u)  // may sleep up to ~20 us in hardware
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up `limit_ns` (wall clock; two seconds by default, far
// beyond any legitimate HBM latency) after the first failed try.  Returns
// false (after recording a fault) if the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int* faults,
                                          uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (global_ns() - t0 > limit_ns) break;
  }
  if (faults) atomicAdd(faults, 1u);
  return false;
}

// global -> shared bulk copy; `bytes` a multiple of 16, both addresses 16-byte aligned.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_addr(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}

}  // namespace fb
