// LayerNorm forward / backward for rows of 8 KB .. 64 KB, staged through
// shared memory by bulk asynchronous copies (pipe.cuh).  Included by
// layer_norm.cu only.
//
// One thread keeps STAGES rows in flight per CTA while all threads work on the
// row that has landed, so HBM always has STAGES * row bytes outstanding per
// CTA whatever phase the arithmetic is in.  A stage is re-armed right after
// the first block reduction of its row: that reduction's __syncthreads proves
// every thread has moved its part of the row into registers.
//
// These kernels are bound by instruction issue before they are bound by HBM
// unless the per-element work is kept small, hence: 16 elements per thread
// (the two block reductions per row are a fixed cost per thread), multiply by
// 1/std instead of dividing, fused multiply-add allowed in this translation
// unit (parity here is the 2e-4 bar, not bitwise), waits that suspend in
// hardware instead of spinning.
#pragma once
#include "common.cuh"
#include "pipe.cuh"

namespace fb {

struct PipePlan {
  int threads;  // 256, 512 or 1024 (0: row not eligible)
  int items;    // float4 per thread: 2 or 4
  int stages;
  unsigned grid;
  size_t smem;
};

// narr = arrays staged per row (1 forward, 2 backward); ctas_per_sm at 256 threads.
// Shortest rows the backward pipeline takes (FB_LN_PIPE_MIN=<cols> overrides it for A/B measurements).  Measured
// against the register kernel, % of the copy rate: 1536 columns 91 against 73, 1024 columns 90 against 87, 1000
// columns 88 against 83, 896 columns 97 against 81, 768 columns 90 against 78, 640 columns 84 against 69, 512
// columns 89 against 75, 448 columns 95 against 50, 384 columns 85 against 59, 320 columns 79 against 54 (64
// threads up to 512 columns, 128 up to 1024, 256 up to 2044); 256 columns 72 against 90.
static uint64_t pipe_min_cols() {
  static const uint64_t v = [] { const char* e = getenv("FB_LN_PIPE_MIN"); return e ? (uint64_t)atoll(e) : 260ull; }();
  return v;
}
// FB_LN_PIPE_ODD=0 keeps the backward on power-of-two CTA sizes (A/B measurements).
static bool pipe_odd_threads() {
  static const int on = [] { const char* e = getenv("FB_LN_PIPE_ODD"); return (e && e[0] == '0') ? 0 : 1; }();
  return on != 0;
}
constexpr int ln_bwd_pipe_per_sm(int t, int items);
static PipePlan pipe_plan(uint64_t rows, uint64_t cols, int narr) {
  PipePlan p{0, 0, 0, 0, 0};
  if ((cols & 3) || cols < (narr == 2 ? pipe_min_cols() : 2048u) || cols > 16384) return p;
  const uint64_t v = cols / 4;
  if (v < 512) {  // short rows (backward only): 64, 128 or 256 threads x 2 float4, 1024 threads per SM
    const int threads = v <= 128 ? 64 : (v <= 256 ? 128 : 256), per_sm = 1024 / threads;
    const size_t row_bytes = (size_t)cols * 4 * narr;
    int stages = (int)(((size_t)(200 * 1024) / per_sm - 256) / row_bytes);
    if (stages > 4) stages = 4;
    if (stages < 1) return p;
    p.threads = threads;
    p.items = 2;
    p.stages = stages;
    p.smem = (size_t)stages * row_bytes + 64;
    const uint64_t cap = (uint64_t)device_info().sm_count * per_sm;
    p.grid = (unsigned)(rows < cap ? rows : cap);
    return p;
  }
  int threads = 256;
  while ((uint64_t)threads * 4 < v) threads <<= 1;  // at most 4 float4 per thread
  // Backward: CTA sizes between the powers of two where the row fills them better.  A row padded to the next
  // power of two leaves threads idle and, worse, ends on one CTA per SM (or on 1024 threads x 4 float4, which
  // does not fit 64 registers): 5120 columns on 512 x 4 ran at 73 % of the copy rate, 10240 and 12288 columns on
  // 1024 x 4 at 56 and 59 %.
  if (narr == 2 && pipe_odd_threads()) {
    int t = 0, it = 0;
    if (v > 512 && v <= 640) { t = 320; it = 2; }
    else if (v > 640 && v <= 768) { t = 384; it = 2; }
    else if (v > 1024 && v <= 1280) { t = 320; it = 4; }
    else if (v > 1280 && v <= 1536) { t = 384; it = 4; }
    else if (v > 2048 && v <= 2560) { t = 640; it = 4; }
    else if (v > 2560 && v <= 3072) { t = 768; it = 4; }
    if (t) {
      const int per_sm = ln_bwd_pipe_per_sm(t, it);
      const size_t row_bytes = (size_t)cols * 4 * narr;
      int stages = (int)(((size_t)(200 * 1024) / per_sm - 256) / row_bytes);
      if (stages > 4) stages = 4;
      if (stages >= 1) {
        p.threads = t;
        p.items = it;
        p.stages = stages;
        p.smem = (size_t)stages * row_bytes + 64;
        const uint64_t cap = (uint64_t)device_info().sm_count * per_sm;
        p.grid = (unsigned)(rows < cap ? rows : cap);
        return p;
      }
    }
  }
  // Backward rows of 2049 .. 4096 columns: 512 threads x 2 float4 instead of 256 x 4.  The backward
  // keeps four float4 arrays per item (g, h, two column accumulators); with 2 items it fits 64
  // registers and 1024 threads stay resident per SM, where the 4-item form needs 80 and leaves 768.
  // Measured at 4096 columns: 255 us against 264 us.  The same trade loses at 2048 columns
  // (256 x 2 either way; a fourth CTA per SM: 267 us against 253 us) and at 8192 (1024 x 2 against
  // 512 x 4: 308 us against 286 us), so it stays a special case.
  const bool wide2 = narr == 2 && v > 512 && v <= 1024;
  if (wide2) threads = 512;
  const int items = (uint64_t)threads * 2 >= v ? 2 : 4;
  // Threads per SM: 1024 for the forward and the 512 x 2 backward, 768 for the rest of the backward.
  int per_sm = (narr == 1 || wide2 ? 1024 : 768) / threads;
  if (per_sm < 1) per_sm = 1;
  const size_t row_bytes = (size_t)cols * 4 * narr;
  const size_t budget = (size_t)(200 * 1024) / per_sm - 256;
  int stages = (int)(budget / row_bytes);
  if (stages > 4) stages = 4;
  if (stages < 1) return p;  // one stage still overlaps the next row's load with the second half of this row's work
  p.threads = threads;
  p.items = items;
  p.stages = stages;
  p.smem = (size_t)stages * row_bytes + 64;
  const uint64_t cap = (uint64_t)device_info().sm_count * per_sm;
  p.grid = (unsigned)(rows < cap ? rows : cap);
  return p;
}

template <int T, int ITEMS, bool RMS>
__global__ void __launch_bounds__(T, 1024 / T)
ln_fwd_pipe_kernel(const float* __restrict__ x, const float* __restrict__ w,
                   const float* __restrict__ b, uint64_t rows, uint32_t cols, int stages, float eps,
                   float* __restrict__ y, float* __restrict__ h, float* __restrict__ stds,
                   float* __restrict__ mean, float* __restrict__ rstd, unsigned int* faults) {
  extern __shared__ __align__(128) unsigned char pipe_smem[];
  float* stage = reinterpret_cast<float*>(pipe_smem);
  uint64_t* full = reinterpret_cast<uint64_t*>(pipe_smem + (size_t)stages * cols * 4);
  __shared__ float red_a[T / 32], red_b[T / 32];
  const uint32_t cols4 = cols / 4, row_bytes = cols * 4;
  const int tid = threadIdx.x;
  const float inv_d = 1.0f / (float)cols;
  const uint64_t mine = rows > blockIdx.x ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const uint64_t step = (uint64_t)gridDim.x * cols;  // elements between consecutive rows of this CTA
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  const float* next = x + (uint64_t)blockIdx.x * cols;  // next row to request (thread 0 only)
  uint64_t requested = 0;
  if (tid == 0) {
    for (int s = 0; s < stages && requested < mine; ++s, ++requested, next += step) {
      mbar_expect_tx(&full[s], row_bytes);
      bulk_load(stage + (size_t)s * cols, next, row_bytes, &full[s]);
    }
  }
  int s = 0;
  uint32_t parity = 0;
  float* yrow = y + (uint64_t)blockIdx.x * cols;
  float* hrow = h ? h + (uint64_t)blockIdx.x * cols : nullptr;
  uint64_t row = blockIdx.x;
  for (uint64_t i = 0; i < mine; ++i, row += gridDim.x, yrow += step) {
    if (!mbar_wait(&full[s], parity, faults)) return;
    const float4* sr = reinterpret_cast<const float4*>(stage + (size_t)s * cols);
    const float x0 = RMS ? 0.0f : stage[(size_t)s * cols];
    float4 v[ITEMS];
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      v[k] = c < cols4 ? sr[c] : make_float4(x0, x0, x0, x0);
      v[k].x -= x0; v[k].y -= x0; v[k].z -= x0; v[k].w -= x0;
      sum += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    }
    // RMS normalisation has no mean; the reduction still runs: its barrier is what licenses the re-arm.
    const float row_sum = group_sum<T>(sum, red_a);
    const float md = RMS ? 0.0f : row_sum * inv_d;
    if (tid == 0 && requested < mine) {  // every thread holds its part of the row: re-arm the stage
      mbar_expect_tx(&full[s], row_bytes);
      bulk_load(stage + (size_t)s * cols, next, row_bytes, &full[s]);
      ++requested;
      next += step;
    }
    float q = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      v[k].x -= md; v[k].y -= md; v[k].z -= md; v[k].w -= md;
      if (c < cols4) q += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    }
    const float var = group_sum<T>(q, red_b) * inv_d;
    const float sd = sqrtf(var + eps);
    const float rs = 1.0f / sd;
    if (tid == 0) {
      if (stds) stds[row] = sd;
      if (mean) mean[row] = x0 + md;
      if (rstd) rstd[row] = rs;
    }
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      if (c < cols4) {
        float4 o = make_float4(v[k].x * rs, v[k].y * rs, v[k].z * rs, v[k].w * rs);
        if (hrow) st_stream4(hrow + c * 4, o);
        if (w) {
          const float4 wv = __ldg(reinterpret_cast<const float4*>(w) + c);
          o.x *= wv.x; o.y *= wv.y; o.z *= wv.z; o.w *= wv.w;
        }
        if (b) {
          const float4 bv = __ldg(reinterpret_cast<const float4*>(b) + c);
          o.x += bv.x; o.y += bv.y; o.z += bv.z; o.w += bv.w;
        }
        st_stream4(yrow + c * 4, o);
      }
    }
    if (hrow) hrow += step;
    if (++s == stages) { s = 0; parity ^= 1; }
  }
}

// MODE 0: saved (h, stds); 1: saved (x, mean, rstd); 2: RMS normalisation, saved (x, rstd), no mean.
// CTAs per SM of the backward: 1024 threads' worth with 2 float4 per thread (64 registers), except 256 x 2 where a
// fourth CTA was measured behind; 768 threads' worth with 4 float4 per thread (80 registers); never less than one.
constexpr int ln_bwd_pipe_per_sm(int t, int items) {
  const int budget = (items == 2 && t != 256) ? 1024 : 768;
  return budget / t ? budget / t : 1;
}

template <int T, int ITEMS, int MODE>
__global__ void __launch_bounds__(T, ln_bwd_pipe_per_sm(T, ITEMS))
ln_bwd_pipe_kernel(const float* __restrict__ g, const float* __restrict__ hx,
                   const float* __restrict__ stat_a, const float* __restrict__ stat_b,
                   const float* __restrict__ w, uint64_t rows, uint32_t cols, int stages,
                   float* __restrict__ dx, float* __restrict__ part, int want_dw, int want_db,
                   unsigned int* faults) {
  constexpr bool FROM_X = MODE != 0, RMS = MODE == 2;
  extern __shared__ __align__(128) unsigned char pipe_smem[];
  float* stage = reinterpret_cast<float*>(pipe_smem);  // [stages][2][cols]: g row, then h (or x) row
  uint64_t* full = reinterpret_cast<uint64_t*>(pipe_smem + (size_t)stages * cols * 8);
  __shared__ float2 red2[2][T / 32];
  const uint32_t cols4 = cols / 4, row_bytes = cols * 4;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float inv_d = 1.0f / (float)cols;
  const uint64_t mine = rows > blockIdx.x ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const uint64_t step = (uint64_t)gridDim.x * cols;
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait();     // launched with launch_pdl: everything before this kernel in the stream is complete from here on
  pdl_trigger();  // the finalize launch that follows may take its place on the SMs now; it waits for this grid to end
  uint64_t next = (uint64_t)blockIdx.x * cols, requested = 0;  // thread 0 only
  auto arm = [&](int s) {
    mbar_expect_tx(&full[s], 2 * row_bytes);
    bulk_load(stage + (size_t)s * 2 * cols, g + next, row_bytes, &full[s]);
    bulk_load(stage + (size_t)s * 2 * cols + cols, hx + next, row_bytes, &full[s]);
    ++requested;
    next += step;
  };
  if (tid == 0)
    for (int s = 0; s < stages && requested < mine; ++s) arm(s);
  float4 aw[ITEMS], ab[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) aw[k] = ab[k] = make_float4(0, 0, 0, 0);
  int s = 0;
  uint32_t parity = 0;
  float* dxrow = dx + (uint64_t)blockIdx.x * cols;
  uint64_t row = blockIdx.x;
  for (uint64_t i = 0; i < mine; ++i, row += gridDim.x, dxrow += step) {
    float mu = 0.0f, rs;
    if constexpr (FROM_X) {
      mu = RMS ? 0.0f : __ldg(stat_a + row);
      rs = __ldg(stat_b + row);
    } else {
      rs = 1.0f / __ldg(stat_a + row);
    }
    if (!mbar_wait(&full[s], parity, faults)) return;
    const float4* sg = reinterpret_cast<const float4*>(stage + (size_t)s * 2 * cols);
    const float4* sh = sg + cols4;
    float4 gv[ITEMS], hv[ITEMS];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      float4 wv = make_float4(1, 1, 1, 1);
      if (c < cols4) {
        gv[k] = sg[c];
        hv[k] = sh[c];
        if (w) wv = __ldg(reinterpret_cast<const float4*>(w) + c);
      } else {
        gv[k] = hv[k] = make_float4(0, 0, 0, 0);
      }
      if constexpr (FROM_X) {
        if (c < cols4) {
          hv[k].x = (hv[k].x - mu) * rs; hv[k].y = (hv[k].y - mu) * rs;
          hv[k].z = (hv[k].z - mu) * rs; hv[k].w = (hv[k].w - mu) * rs;
        }
      }
      aw[k].x += gv[k].x * hv[k].x; aw[k].y += gv[k].y * hv[k].y;
      aw[k].z += gv[k].z * hv[k].z; aw[k].w += gv[k].w * hv[k].w;
      ab[k].x += gv[k].x; ab[k].y += gv[k].y; ab[k].z += gv[k].z; ab[k].w += gv[k].w;
      // From here on gv holds dxh = g * w.
      gv[k].x *= wv.x; gv[k].y *= wv.y; gv[k].z *= wv.z; gv[k].w *= wv.w;
      s1 += (gv[k].x + gv[k].y) + (gv[k].z + gv[k].w);
      s2 += (gv[k].x * hv[k].x + gv[k].y * hv[k].y) + (gv[k].z * hv[k].z + gv[k].w * hv[k].w);
    }
    // Both row sums in one block reduction.
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    float2* red = red2[i & 1];  // alternate, so one barrier per row is enough
    if (lane == 0) red[warp] = make_float2(s1, s2);
    __syncthreads();
    if (tid == 0 && requested < mine) arm(s);
    float2 t = lane < T / 32 ? red[lane] : make_float2(0.0f, 0.0f);
    constexpr int kNw = T / 32;  // any warp count up to 32: the butterfly spans the next power of two
    constexpr int kSpan = kNw <= 1 ? 1 : kNw <= 2 ? 2 : kNw <= 4 ? 4 : kNw <= 8 ? 8 : kNw <= 16 ? 16 : 32;
#pragma unroll
    for (int o = kSpan / 2; o > 0; o >>= 1) {
      t.x += __shfl_xor_sync(0xffffffffu, t.x, o);
      t.y += __shfl_xor_sync(0xffffffffu, t.y, o);
    }
    const float m1 = RMS ? 0.0f : __shfl_sync(0xffffffffu, t.x, 0) * inv_d;
    const float m2 = __shfl_sync(0xffffffffu, t.y, 0) * inv_d;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      if (c < cols4) {
        float4 o;
        o.x = (gv[k].x - m1 - hv[k].x * m2) * rs;
        o.y = (gv[k].y - m1 - hv[k].y * m2) * rs;
        o.z = (gv[k].z - m1 - hv[k].z * m2) * rs;
        o.w = (gv[k].w - m1 - hv[k].w * m2) * rs;
        st_stream4(dxrow + c * 4, o);
      }
    }
    if (++s == stages) { s = 0; parity ^= 1; }
  }
  if (want_dw | want_db) {
    float* pw = part + (uint64_t)blockIdx.x * 2 * cols;
    float* pb = pw + cols;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      if (c < cols4) {
        if (want_dw) *reinterpret_cast<float4*>(pw + c * 4) = aw[k];
        if (want_db) *reinterpret_cast<float4*>(pb + c * 4) = ab[k];
      }
    }
  }
}

}  // namespace fb
