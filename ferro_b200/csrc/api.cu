// Library-level plumbing: error text, device facts, launch counter.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "pipe.cuh"

namespace fb {

static thread_local char g_error[512] = "";
std::atomic<uint64_t> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(FB_ERR_CUDA, "CUDA error: %s (%s) at %s", cudaGetErrorString(e), cudaGetErrorName(e),
              what);
}

const DeviceInfo& device_info() {
  // One slot per device ordinal; filled on first use on that device.
  static DeviceInfo info[64];
  static std::atomic<int> ready[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!ready[dev].load(std::memory_order_acquire)) {
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!ready[dev].load(std::memory_order_relaxed)) {
      int sms = 0, smem = 0;
      if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        sms = 148;
      if (cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess ||
          smem <= 0)
        smem = 48 * 1024;
      info[dev].sm_count = sms;
      info[dev].max_smem_optin = smem;
      ready[dev].store(1, std::memory_order_release);
    }
  }
  return info[dev];
}

cudaError_t allow_dyn_smem(const void* kernel, size_t bytes) {
  struct Entry { const void* k; int dev; size_t bytes; };
  static std::mutex mu;
  static Entry table[256];
  static int n = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  int slot = -1;
  for (int i = 0; i < n; ++i)
    if (table[i].k == kernel && table[i].dev == dev) { slot = i; break; }
  if (slot >= 0 && table[slot].bytes >= bytes) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return e;
  if (slot < 0 && n < 256) slot = n++;
  if (slot >= 0) table[slot] = Entry{kernel, dev, bytes};  // a full table only costs the call again next time
  return cudaSuccess;
}

// Counts bounded device-side waits that gave up (see pipe.cuh).
__device__ unsigned int g_device_faults = 0;

unsigned int* fault_word() {
  static unsigned int* ptr[64];
  static std::atomic<int> ready[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ready[dev].load(std::memory_order_acquire)) {
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!ready[dev].load(std::memory_order_relaxed)) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_device_faults) != cudaSuccess) return nullptr;
      ptr[dev] = static_cast<unsigned int*>(p);
      ready[dev].store(1, std::memory_order_release);
    }
  }
  return ptr[dev];
}

}  // namespace fb

namespace fb {
// The wait path of the pipelined kernels on a barrier that nothing will ever complete: one
// transaction is expected and never issued, so the wait runs into its time limit, records a
// fault and the kernel returns.  The barrier is invalidated before exit.
__global__ void bounded_wait_selftest_kernel(unsigned int* faults, uint64_t limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_wait(&bar, 0, faults, limit_ns);
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_addr(&bar)) : "memory");
  }
}
}  // namespace fb

extern "C" {

int fb_device_faults(int reset) {
  unsigned int* p = fb::fault_word();
  if (!p) return -1;
  unsigned int v = 0;
  if (cudaMemcpy(&v, p, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (reset && v) {
    const unsigned int zero = 0;
    cudaMemcpy(p, &zero, sizeof(zero), cudaMemcpyHostToDevice);
  }
  return (int)v;
}

int fb_selftest_bounded_wait(fb_stream_t stream, uint32_t limit_ms) {
  if (limit_ms == 0 || limit_ms > 1000)
    return fb::fail(FB_ERR_INVALID_ARG, "fb_selftest_bounded_wait: limit must be 1 .. 1000 ms");
  unsigned int* faults = fb::fault_word();
  if (!faults) return fb::fail(FB_ERR_CUDA, "fb_selftest_bounded_wait: no device status word");
  fb::bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(faults, (uint64_t)limit_ms * 1000000ull);
  FB_LAUNCHED("fb_selftest_bounded_wait");
  return FB_OK;
}

int fb_version(void) { return FB_VERSION; }
const char* fb_last_error(void) { return fb::g_error; }
uint64_t fb_launch_count(void) { return fb::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
