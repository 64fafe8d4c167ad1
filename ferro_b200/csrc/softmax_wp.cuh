// Warp-pipelined softmax backward for rows of 256 .. 1024 columns.
//
// At these widths a problem of a few thousand rows lives for ten to thirty
// microseconds, so what decides the time is how soon every SM has its share of
// the reads in flight and whether reads, arithmetic and writes overlap at all.
// Design: one CTA of eight warps per SM, each CTA owning a contiguous, balanced
// range of rows.  A warp is a pipeline of its own: lane 0 keeps STAGES rows of
// every input array in flight into the warp's private shared-memory slots with
// 1-D bulk asynchronous copies (cp.async.bulk + mbarrier; no multicast, no
// cluster); the warp takes a finished row out of shared memory, re-arms the
// slot at once, reduces with shuffles only and stores with streaming float4
// stores.  Nothing in the row loop synchronises the CTA, so the eight warps
// drift apart and the SM always has loads, math and stores going at once.
// Every barrier wait is bounded (pipe.cuh).
//
// The fused form also stages x for the relu mask and keeps the bias-gradient
// column sums in registers across the warp's rows; at the end the CTA folds
// its warps in warp order into one partial row (at most one per SM), which a
// second, dependent launch adds up in row order: results are bit-identical
// from run to run.
//
// Measured against the register kernels of softmax.cu (B200, buffers rotated
// so that nothing is served from L2): fused backward 24.7 us against 29.7 us
// at [8192, 1024] and 330 us against 390 us at [131072, 1024]; plain backward
// 17.5 us against 19.0 us at [8192, 1024] but 256 us against 234 us at
// [131072, 1024], so the plain form is used for small problems only.  The same
// pipeline as a forward kernel lost everywhere (17.5 us against 15.0 us at
// [8192, 1024]; 57 - 87 % of the register kernel's rate on large inputs, where
// one array in flight per row is too little for the bulk copies to pay) and is
// not kept.
#pragma once
#include "common.cuh"
#include "pipe.cuh"

namespace fb {

constexpr int kWpWarps = 8;
constexpr int kWpThreads = kWpWarps * 32;

struct WpPlan {
  int items;   // float4 per lane per array (0: not eligible)
  int stages;
  unsigned grid;
  size_t smem;
};

// narr: arrays staged per row.  extra_floats: shared memory the kernel keeps besides the stages.
static inline WpPlan wp_plan(uint64_t rows, uint64_t cols, int narr, uint64_t extra_floats) {
  WpPlan p{0, 0, 0, 0};
  if ((cols & 3) || cols < 256 || cols > 1024 || rows >= (1ull << 31)) return p;
  const uint64_t v = cols / 4;
  int items = 1;
  while ((uint64_t)items * 32 < v) items <<= 1;
  const size_t stage_set = (size_t)kWpWarps * narr * cols * 4;  // one stage of every warp
  const size_t fixed = (size_t)extra_floats * 4 + 1024;
  const size_t budget = 208 * 1024;
  if (budget < fixed + 2 * stage_set) return p;
  int stages = (int)((budget - fixed) / stage_set);
  if (stages > 6) stages = 6;
  p.items = items;
  p.stages = stages;
  p.smem = fixed + (size_t)stages * stage_set;
  const uint64_t sms = (uint64_t)device_info().sm_count;
  const uint64_t want = (rows + kWpWarps - 1) / kWpWarps;
  p.grid = (unsigned)(want < sms ? want : sms);
  return p;
}

// Rows [r0, r1) of CTA b of G: contiguous and balanced to within one row.
__device__ __forceinline__ void wp_rows(uint32_t rows, uint32_t& r0, uint32_t& r1) {
  r0 = (uint32_t)(((uint64_t)blockIdx.x * rows) / gridDim.x);
  r1 = (uint32_t)(((uint64_t)(blockIdx.x + 1) * rows) / gridDim.x);
}

// Shared-memory layout: [bias: cols floats (FUSED)] [slots: warp-major] [barriers].
// NARR = 2: g, y.  NARR = 3 (FUSED): g, y, x with dx = relu_backward(dt * scale, x + bias); when
// `part` is given, CTA b leaves the column sums of its rows of dx in part[b][cols].
template <int ITEMS, bool LOG, bool FUSED>
__global__ void __launch_bounds__(kWpThreads, 1)
softmax_bwd_wp_kernel(const float* __restrict__ g, const float* __restrict__ y, const float* __restrict__ x,
                      const float* __restrict__ bias, float scale, int relu, uint32_t rows, uint32_t cols,
                      int stages, float* __restrict__ dx, float* __restrict__ part, unsigned int* faults) {
  constexpr int NARR = FUSED ? 3 : 2;
  extern __shared__ __align__(128) unsigned char wp_smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t cols4 = cols / 4, row_bytes = cols * 4;
  float* sbias = reinterpret_cast<float*>(wp_smem);
  float* stage0 = sbias + (FUSED ? cols : 0);
  float* mine = stage0 + (size_t)warp * stages * NARR * cols;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage0 + (size_t)kWpWarps * stages * NARR * cols) + warp * 8;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  uint32_t r0, r1;
  wp_rows(rows, r0, r1);
  const uint32_t first = r0 + warp;
  const uint32_t n_my = first < r1 ? (r1 - first + kWpWarps - 1) / kWpWarps : 0;
  const bool masked = FUSED && relu;
  __syncwarp();  // the warp's barriers are initialised
  pdl_wait();    // from here on global memory may be touched
  uint32_t armed = 0;
  auto arm = [&](int s) {  // lane 0 only
    const uint64_t off = (uint64_t)(first + armed * kWpWarps) * cols;
    float* dst = mine + (size_t)s * NARR * cols;
    mbar_expect_tx(&bars[s], (masked ? 3 : 2) * row_bytes);
    bulk_load(dst, g + off, row_bytes, &bars[s]);
    bulk_load(dst + cols, y + off, row_bytes, &bars[s]);
    if (masked) bulk_load(dst + 2 * cols, x + off, row_bytes, &bars[s]);
    ++armed;
  };
  if (lane == 0)
    for (int s = 0; s < stages && armed < n_my; ++s) arm(s);
  // The bias is fetched behind the first rows, so that its latency hides under theirs.
  if constexpr (FUSED) {
    for (uint32_t c = tid; c < cols4; c += kWpThreads)
      reinterpret_cast<float4*>(sbias)[c] =
          bias ? __ldg(reinterpret_cast<const float4*>(bias) + c) : make_float4(0, 0, 0, 0);
    __syncthreads();
  }
  pdl_trigger();
  float4 acc[FUSED ? ITEMS : 1];
#pragma unroll
  for (int k = 0; k < (FUSED ? ITEMS : 1); ++k) acc[k] = make_float4(0, 0, 0, 0);
  int s = 0;
  uint32_t parity = 0;
  bool gave_up = false;
  for (uint32_t i = 0; i < n_my; ++i) {
    if (!mbar_wait(&bars[s], parity, faults)) { gave_up = true; break; }
    const float4* sg = reinterpret_cast<const float4*>(mine + (size_t)s * NARR * cols);
    const float4* sy = sg + cols4;
    const float4* sx = sy + cols4;
    float4 gv[ITEMS], yv[ITEMS];
    float4 mv[FUSED ? ITEMS : 1];  // x + bias, the relu mask's input
    float dot = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * 32;
      if (c < cols4) {
        gv[k] = sg[c];
        yv[k] = sy[c];
        if constexpr (FUSED) {
          if (masked) {
            const float4 a = sx[c], b = reinterpret_cast<const float4*>(sbias)[c];
            mv[k] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
          }
        }
      } else {
        gv[k] = yv[k] = make_float4(0, 0, 0, 0);
      }
      if constexpr (LOG) dot += (gv[k].x + gv[k].y) + (gv[k].z + gv[k].w);
      else dot += (gv[k].x * yv[k].x + gv[k].y * yv[k].y) + (gv[k].z * yv[k].z + gv[k].w * yv[k].w);
    }
    __syncwarp();
    if (lane == 0 && armed < n_my) arm(s);
    dot = warp_sum(dot);
    float* dr = dx + (uint64_t)(first + i * kWpWarps) * cols;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * 32;
      if (c < cols4) {
        float4 o;
        if constexpr (LOG) {
          o.x = gv[k].x - __expf(yv[k].x) * dot; o.y = gv[k].y - __expf(yv[k].y) * dot;
          o.z = gv[k].z - __expf(yv[k].z) * dot; o.w = gv[k].w - __expf(yv[k].w) * dot;
        } else {
          o.x = yv[k].x * (gv[k].x - dot); o.y = yv[k].y * (gv[k].y - dot);
          o.z = yv[k].z * (gv[k].z - dot); o.w = yv[k].w * (gv[k].w - dot);
        }
        if constexpr (FUSED) {
          o.x *= scale; o.y *= scale; o.z *= scale; o.w *= scale;
          if (masked) {
            o.x = mv[k].x <= 0.0f ? 0.0f : o.x; o.y = mv[k].y <= 0.0f ? 0.0f : o.y;
            o.z = mv[k].z <= 0.0f ? 0.0f : o.z; o.w = mv[k].w <= 0.0f ? 0.0f : o.w;
          }
          acc[k].x += o.x; acc[k].y += o.y; acc[k].z += o.z; acc[k].w += o.w;
        }
        st_stream4(dr + c * 4, o);
      }
    }
    if (++s == stages) { s = 0; parity ^= 1; }
  }
  if constexpr (FUSED) {
    if (part) {
      // Fold the eight warps in warp order, then one partial row per CTA.  The fold reuses the
      // slot memory ([kWpWarps][cols] floats fit in it for any stage count): after the barrier every
      // warp has left its row loop and nothing is in flight into the slots.  (A warp that gave up a
      // wait has recorded a fault; the outputs are undefined then, the kernel still ends in order.)
      __syncthreads();
      float* comb = stage0;
      if (!gave_up) {
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
          const uint32_t c = lane + k * 32;
          if (c < cols4) reinterpret_cast<float4*>(comb + (size_t)warp * cols)[c] = acc[k];
        }
      }
      __syncthreads();
      float* pr = part + (size_t)blockIdx.x * cols;
      for (uint32_t c = tid; c < cols4; c += kWpThreads) {
        float4 t = reinterpret_cast<const float4*>(comb)[c];
#pragma unroll
        for (int w = 1; w < kWpWarps; ++w) {
          const float4 u = reinterpret_cast<const float4*>(comb + (size_t)w * cols)[c];
          t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        reinterpret_cast<float4*>(pr)[c] = t;
      }
    }
  }
}

}  // namespace fb
