// Shared device / host helpers for every kernel file of libferro_b200.
//
// Build rule: the translation units whose results are compared bitwise with
// ferro's CPU path (elementwise, the strided engine, the optimizers, the MLP
// glue) are compiled with -fmad=false, because that path never contracts
// a*b+c (Rust has no implicit fma).  The row kernels (softmax, LayerNorm,
// reductions) are held to a relative tolerance and keep the contraction.
// Division and square root stay IEEE everywhere (nvcc defaults
// -prec-div=true -prec-sqrt=true -ftz=false) unless a kernel asks for an
// approximation by name (math.cuh).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ferro_b200.h"

namespace fb {

// ---- host: errors -------------------------------------------------------
int fail(int code, const char* fmt, ...);   // sets fb_last_error(), returns code
int cuda_fail(cudaError_t e, const char* what);

#define FB_CUDA(expr)                                      \
  do {                                                     \
    cudaError_t fb_e_ = (expr);                            \
    if (fb_e_ != cudaSuccess) return ::fb::cuda_fail(fb_e_, #expr); \
  } while (0)

// After a <<<>>> launch: report a launch-configuration error without
// synchronising (ops are asynchronous on the caller's stream).
#define FB_LAUNCHED(name)                                  \
  do {                                                     \
    cudaError_t fb_e_ = cudaGetLastError();                \
    if (fb_e_ != cudaSuccess) return ::fb::cuda_fail(fb_e_, name); \
    ::fb::count_launch();                                  \
  } while (0)
void count_launch();  // bumps fb_launch_count()

// Per-device facts, read once per device and cached (no CUDA call on the
// steady-state launch path, so launches stay legal during stream capture).
struct DeviceInfo {
  int sm_count;
  int max_smem_optin;
};
const DeviceInfo& device_info();

// Opts `kernel` in to `bytes` of dynamic shared memory on the current device.
// The runtime call is made the first time and whenever a larger size is asked
// for; later launches find the answer in a table (no CUDA call on the
// steady-state launch path).
cudaError_t allow_dyn_smem(const void* kernel, size_t bytes);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// True when a*b overflows uint64.
inline bool mul_overflows(uint64_t a, uint64_t b, uint64_t* out) {
  return __builtin_mul_overflow(a, b, out);
}

// Grid for a grid-stride kernel: enough CTAs to fill every SM `per_sm` times,
// never more than the work needs.
inline unsigned grid_for(uint64_t work_items, int per_sm) {
  const uint64_t cap = (uint64_t)device_info().sm_count * (uint64_t)per_sm;
  if (work_items <= cap) return (unsigned)(work_items ? work_items : 1);
  // Balance: every CTA gets the same number of items (to within one), instead
  // of `cap` CTAs of which some run one item more than the rest.
  const uint64_t iters = (work_items + cap - 1) / cap;
  return (unsigned)((work_items + iters - 1) / iters);
}

// Grid for a streaming kernel that reads and writes in equal measure and keeps
// no per-CTA state: one CTA per work item, issued in address order by the
// hardware scheduler.  Measured on a 1 GiB float4 copy: 6.7 TB/s this way
// against 5.8 to 6.1 TB/s for a persistent grid-stride loop of any depth, and
// 6.46 TB/s for a device-to-device cudaMemcpy.  The kernels keep their
// stride loop, so the clamp to the grid limit is harmless.
inline unsigned grid_full(uint64_t work_items) {
  if (work_items == 0) return 1;
  return (unsigned)(work_items < 0x7fffffffull ? work_items : 0x7fffffffull);
}

// ---- programmatic dependent launch ------------------------------------------
// Short kernels (tens of microseconds) lose a tenth of their time to the gap
// between one kernel's last CTA and the next kernel's first instruction.  A
// kernel launched with launch_pdl() may be made resident while the kernel
// before it in the stream drains: it runs its set-up (shared-memory barriers,
// index arithmetic) and then blocks in pdl_wait() until that kernel has
// completed and its writes are visible.  Rules: pdl_wait() comes before the
// first access to global memory of any kind (a predecessor may still be
// writing this kernel's inputs or reading its outputs); pdl_trigger() tells
// the scheduler that the next kernel may start to launch once every CTA of
// this one has passed it (or exited), so it costs this kernel nothing.  A
// kernel that never triggers releases its dependents when it ends, and a
// predecessor that is not ours behaves exactly like that: ordering is never
// weaker than plain stream order.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- device: memory access ---------------------------------------------
// Streaming (evict-first) accesses for data touched once per kernel.
__device__ __forceinline__ float4 ld_stream4(const float* p) {
  return __ldcs(reinterpret_cast<const float4*>(p));
}
__device__ __forceinline__ float ld_stream(const float* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream4(float* p, float4 v) {
  __stcs(reinterpret_cast<float4*>(p), v);
}
__device__ __forceinline__ void st_stream(float* p, float v) { __stcs(p, v); }

// ---- device: reductions --------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sums (or maxima) of RW values over the LPR lanes that hold one row (LPR a power of two, 4..32,
// rows aligned to LPR inside the warp), transposed: each step halves the values a lane carries (a
// lane keeps the half its own bit selects and sends the other half across), so RW results cost
// RW - 1 + log2(LPR / RW) shuffles instead of RW * log2(LPR).  Lane l of the row's lanes ends with
// the result of value l / (LPR / RW); the LPR / RW lanes that share a value hold the same result.
// `a` is consumed.
template <int LPR, int RW, bool MAX>
__device__ __forceinline__ float lanes_transpose_reduce(float (&a)[RW], int l) {
  static_assert((RW & (RW - 1)) == 0 && RW <= LPR, "RW is a power of two, at most LPR");
  int o = LPR / 2;
#pragma unroll
  for (int n = RW; n > 1; n >>= 1, o >>= 1) {
    const bool upper = (l & o) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float send = upper ? a[i] : a[i + n / 2];
      const float keep = upper ? a[i + n / 2] : a[i];
      const float got = __shfl_xor_sync(0xffffffffu, send, o);
      a[i] = MAX ? fmaxf(keep, got) : keep + got;
    }
  }
#pragma unroll
  for (; o > 0; o >>= 1) {
    const float got = __shfl_xor_sync(0xffffffffu, a[0], o);
    a[0] = MAX ? fmaxf(a[0], got) : a[0] + got;
  }
  return a[0];
}
template <int LPR, int RW>
__device__ __forceinline__ float lanes_transpose_sum(float (&a)[RW], int l) {
  return lanes_transpose_reduce<LPR, RW, false>(a, l);
}
template <int LPR, int RW>
__device__ __forceinline__ float lanes_transpose_max(float (&a)[RW], int l) {
  return lanes_transpose_reduce<LPR, RW, true>(a, l);
}

// Sum over a group of G consecutive threads (G a power of two, 32..1024,
// groups aligned to G inside the CTA).  `scratch` holds blockDim.x/32 floats
// and must not be reused until the next __syncthreads() the caller issues
// (callers alternate between two scratch arrays).  Every thread of the CTA
// must call this (it contains __syncthreads when G > 32).
template <int G>
__device__ __forceinline__ float group_sum(float v, float* scratch) {
  v = warp_sum(v);
  if constexpr (G > 32) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    constexpr int W = G / 32;  // warps per group
    const int first = (warp / W) * W;
    float t = (lane < W) ? scratch[first + lane] : 0.0f;
#pragma unroll
    for (int o = W / 2; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    v = __shfl_sync(0xffffffffu, t, 0);
  }
  return v;
}
template <int G>
__device__ __forceinline__ float group_max(float v, float* scratch) {
  v = warp_max(v);
  if constexpr (G > 32) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    constexpr int W = G / 32;
    const int first = (warp / W) * W;
    float t = (lane < W) ? scratch[first + lane] : -INFINITY;
#pragma unroll
    for (int o = W / 2; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    v = __shfl_sync(0xffffffffu, t, 0);
  }
  return v;
}

// Whole-CTA sum for kernels whose CTA works on one row (any blockDim that is
// a multiple of 32, up to 1024).  Contains two __syncthreads.
__device__ __forceinline__ float block_sum(float v, float* scratch /*[32]*/) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? scratch[lane] : 0.0f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch /*[32]*/) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? scratch[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

// ---- row-in-registers geometry -------------------------------------------
// A row of `cols` floats (cols % 4 == 0, 16-byte aligned rows) is held by a
// group of G threads, each owning ITEMS float4s laid out so that one group
// load instruction covers G*16 contiguous bytes.
struct RowCfg {
  int group;  // threads per row: 32, 64, ..., 1024
  int items;  // float4 per thread: 1, 2, 4 or 8
};
// Smallest group that holds the row with at most 8 float4 per thread; items
// rounded up to a power of two.  group == 0 when the row does not fit
// (cols > 32768) or is not vectorisable.
inline RowCfg row_cfg(uint64_t cols) {
  RowCfg c{0, 0};
  if (cols == 0 || (cols & 3)) return c;
  const uint64_t v = cols / 4;
  for (int g = 32; g <= 1024; g <<= 1) {
    if (v <= (uint64_t)g * 8) {
      uint64_t it = (v + g - 1) / g;
      int p = 1;
      while ((uint64_t)p < it) p <<= 1;
      c.group = g;
      c.items = p;
      return c;
    }
  }
  return c;
}

}  // namespace fb
