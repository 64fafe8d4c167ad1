// Reduction building blocks shared by reduce.cu, softmax.cu and mlp.cu.
//
// Column reduction ("sum over rows of a [red, inner] slab, inner contiguous"):
// a CTA owns a strip of 32*VEC columns and a slice of the rows; its 8 warps
// take rows round-robin, every lane keeps VEC running sums, the warps are
// combined through shared memory in warp order, and the slice result goes
// either to the output (one slice) or to a partial row that a finalize kernel
// adds up in slice order.  No atomics: the summation order is a function of
// the shape only, as ferro requires of its reductions
// (crates/ferro-core/src/reduce.rs:11-14).
#pragma once
#include "common.cuh"

namespace fb {

// (value, index) with ferro's argmax order (ops_ext/argmax.rs:50-60): the
// first NaN wins; otherwise the greatest value, the lowest index among equals.
struct Best {
  float v;
  uint64_t i;
};
__device__ __forceinline__ bool beats(const Best& a, const Best& b) {
  const bool an = isnan(a.v), bn = isnan(b.v);
  if (an) return !bn || a.i < b.i;
  if (bn) return false;
  return a.v > b.v || (a.v == b.v && a.i < b.i);
}
__device__ __forceinline__ Best best_of(const Best& a, const Best& b) { return beats(b, a) ? b : a; }
__device__ __forceinline__ Best best_identity() { return Best{-INFINITY, UINT64_MAX}; }
__device__ __forceinline__ Best warp_best(Best b) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best t;
    t.v = __shfl_xor_sync(0xffffffffu, b.v, o);
    t.i = __shfl_xor_sync(0xffffffffu, b.i, o);
    b = best_of(b, t);
  }
  return b;
}

// Per-thread running scan used in the hot loops.  Three instructions per
// element: a strictly-greater compare that moves the index (so the first of
// equal values is kept; indices arrive in increasing order per thread) and a
// NaN-propagating maximum, which doubles as the NaN detector.  Once a NaN has
// been folded in, the running maximum stays NaN and the index stops moving;
// the caller then finds the first NaN by walking its elements again (rows
// with a NaN are the rare case), which is what ferro's argmax returns.
__device__ __forceinline__ float fmax_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
// I is the index type of the hot loop: uint32_t when the reduced extent fits.
template <class I>
struct Scan {
  float m;  // maximum so far, NaN once a NaN was seen
  I i;      // index of the first element equal to m (meaningless once m is NaN)
};
template <class I>
__device__ __forceinline__ Scan<I> scan_init(I first_index) { return Scan<I>{-INFINITY, first_index}; }
template <class I>
__device__ __forceinline__ void scan_step(Scan<I>& s, float v, I k) {
  if (v > s.m) s.i = k;
  s.m = fmax_nan(s.m, v);
}
// `first_nan` is the caller's second walk; only evaluated for a poisoned scan.
template <class I, class FirstNan>
__device__ __forceinline__ Best scan_finish(const Scan<I>& s, FirstNan first_nan) {
  if (s.m != s.m) return Best{__int_as_float(0x7fc00000), first_nan()};
  return Best{s.m, (uint64_t)s.i};
}

// Best over a group of G consecutive threads; same calling rules as group_sum.
template <int G>
__device__ __forceinline__ Best group_best(Best b, float* sv, unsigned long long* si) {
  b = warp_best(b);
  if constexpr (G > 32) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = b.v; si[warp] = b.i; }
    __syncthreads();
    constexpr int W = G / 32;
    const int first = (warp / W) * W;
    Best t = lane < W ? Best{sv[first + lane], si[first + lane]} : best_identity();
    t = warp_best(t);
    b = t;
  }
  return b;
}

constexpr int kColWarps = 8;
constexpr int kColThreads = kColWarps * 32;

// Geometry of a column reduction over x[outer][red][inner].
struct ColPlan {
  int vec;          // 4 or 1 floats per lane
  uint32_t strips;  // column strips per outer slab
  uint32_t splits;  // row slices per (outer, strip)
  uint64_t rows_per_split;
};

inline ColPlan col_plan(uint64_t outer, uint64_t red, uint64_t inner, bool aligned) {
  ColPlan p;
  p.vec = (aligned && inner % 4 == 0) ? 4 : 1;
  const uint64_t strip_cols = 32ull * p.vec;
  p.strips = (uint32_t)((inner + strip_cols - 1) / strip_cols);
  const uint64_t ctas = outer * p.strips;
  const uint64_t target = (uint64_t)device_info().sm_count * 8;
  uint64_t splits = 1;
  if (ctas < target) {
    splits = (target + ctas - 1) / ctas;
    // Keep at least 4 rows per warp in a slice, otherwise the slice is all overhead.
    const uint64_t max_splits = red / (kColWarps * 4) ? red / (kColWarps * 4) : 1;
    if (splits > max_splits) splits = max_splits;
    if (splits > 512) splits = 512;
  }
  p.rows_per_split = (red + splits - 1) / splits;
  p.splits = (uint32_t)((red + p.rows_per_split - 1) / p.rows_per_split);
  if (p.splits == 0) p.splits = 1;
  return p;
}

// Scratch a column reduction with `nout` simultaneous outputs may need.
inline uint64_t col_scratch_bytes(const ColPlan& p, uint64_t outer, uint64_t inner, int nout) {
  if (p.splits <= 1) return 0;
  return (uint64_t)p.splits * outer * inner * nout * sizeof(float);
}

// Src: struct with
//   template<int VEC> __device__ void load(uint64_t o, uint64_t r, uint64_t c, float (&v)[NOUT][VEC]) const
// giving the NOUT values to be summed at (outer o, row r, columns c..c+VEC).
// Output n lands in dst + n * outer * inner (dst = out when splits == 1, else
// the partial buffer laid out [split][n][outer][inner]).
template <int VEC, int NOUT, class Src>
__global__ void __launch_bounds__(kColThreads)
col_sum_kernel(Src src, uint64_t outer, uint64_t red, uint64_t inner, uint32_t strips,
               uint32_t splits, uint64_t rows_per_split, float* __restrict__ out0,
               float* __restrict__ out1, float* __restrict__ part, float scale) {
  pdl_trigger();  // the dependent finalize launch may become resident while this grid runs
  __shared__ float sm[kColWarps][NOUT][32 * VEC + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t tiles = outer * strips * splits;
  for (uint64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
    const uint32_t split = (uint32_t)(t % splits);
    const uint64_t os = t / splits;
    const uint32_t strip = (uint32_t)(os % strips);
    const uint64_t o = os / strips;
    const uint64_t c = ((uint64_t)strip * 32 + lane) * VEC;
    const uint64_t r0 = (uint64_t)split * rows_per_split;
    const uint64_t r1 = (r0 + rows_per_split < red) ? r0 + rows_per_split : red;
    float acc[NOUT][VEC];
#pragma unroll
    for (int n = 0; n < NOUT; ++n)
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[n][j] = 0.0f;
    if (c < inner) {
      uint64_t r = r0 + warp;
      // Two rows in flight per warp.
      for (; r + kColWarps < r1; r += 2 * kColWarps) {
        float a[NOUT][VEC], b[NOUT][VEC];
        src.template load<VEC>(o, r, c, a);
        src.template load<VEC>(o, r + kColWarps, c, b);
#pragma unroll
        for (int n = 0; n < NOUT; ++n)
#pragma unroll
          for (int j = 0; j < VEC; ++j) acc[n][j] = (acc[n][j] + a[n][j]) + b[n][j];
      }
      for (; r < r1; r += kColWarps) {
        float a[NOUT][VEC];
        src.template load<VEC>(o, r, c, a);
#pragma unroll
        for (int n = 0; n < NOUT; ++n)
#pragma unroll
          for (int j = 0; j < VEC; ++j) acc[n][j] += a[n][j];
      }
    }
    __syncthreads();  // previous tile's readers are done with sm
#pragma unroll
    for (int n = 0; n < NOUT; ++n)
#pragma unroll
      for (int j = 0; j < VEC; ++j) sm[warp][n][lane * VEC + j] = acc[n][j];
    __syncthreads();
    // Thread i of the first NOUT*32*VEC threads finishes one (output, column).
    for (int i = threadIdx.x; i < NOUT * 32 * VEC; i += kColThreads) {
      const int n = i / (32 * VEC), cc = i % (32 * VEC);
      float s = sm[0][n][cc];
#pragma unroll
      for (int w = 1; w < kColWarps; ++w) s += sm[w][n][cc];
      const uint64_t col = (uint64_t)strip * 32 * VEC + cc;
      if (col < inner) {
        if (splits == 1) {
          float* dst = n == 0 ? out0 : out1;
          if (dst) dst[o * inner + col] = s * scale;
        } else {
          part[(((uint64_t)split * NOUT + n) * outer + o) * inner + col] = s;
        }
      }
    }
  }
}

// out_n[j] = scale * sum_s part[s][n][j], s in order; j over outer*inner.
template <int NOUT>
__global__ void __launch_bounds__(256)
col_finalize_kernel(const float* __restrict__ part, uint32_t splits, uint64_t count,
                    float* __restrict__ out0, float* __restrict__ out1, float scale) {
  pdl_wait();  // launched as a dependent (launch_pdl) of the kernel that writes its input
  pdl_trigger();
  for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < count;
       j += (uint64_t)gridDim.x * blockDim.x) {
#pragma unroll
    for (int n = 0; n < NOUT; ++n) {
      float* dst = n == 0 ? out0 : out1;
      if (!dst) continue;
      float s = 0.0f;
      for (uint32_t k = 0; k < splits; ++k) s += part[((uint64_t)k * NOUT + n) * count + j];
      dst[j] = s * scale;
    }
  }
}

// Host driver.  Returns an fb_status.
template <int NOUT, class Src>
int run_col_sum(cudaStream_t stream, const Src& src, uint64_t outer, uint64_t red, uint64_t inner,
                bool aligned, float* out0, float* out1, float scale, void* workspace,
                uint64_t workspace_bytes, const char* name) {
  const ColPlan p = col_plan(outer, red, inner, aligned);
  const uint64_t need = col_scratch_bytes(p, outer, inner, NOUT);
  if (need && (!workspace || workspace_bytes < need))
    return fail(FB_ERR_WORKSPACE, "%s: needs %llu bytes of scratch", name, (unsigned long long)need);
  float* part = static_cast<float*>(workspace);
  const uint64_t tiles = outer * p.strips * (uint64_t)p.splits;
  // Tiles are few and long (col_plan aims at eight per SM): a balanced persistent grid avoids a ragged last wave.
  const unsigned grid = grid_for(tiles, 8);
  if (p.vec == 4)
    col_sum_kernel<4, NOUT, Src><<<grid, kColThreads, 0, stream>>>(
        src, outer, red, inner, p.strips, p.splits, p.rows_per_split, out0, out1, part, scale);
  else
    col_sum_kernel<1, NOUT, Src><<<grid, kColThreads, 0, stream>>>(
        src, outer, red, inner, p.strips, p.splits, p.rows_per_split, out0, out1, part, scale);
  FB_LAUNCHED(name);
  if (p.splits > 1) {
    const uint64_t count = outer * inner;
    FB_CUDA(launch_pdl(col_finalize_kernel<NOUT>, dim3(grid_for((count + 255) / 256, 8)), dim3(256), 0, stream,
                       (const float*)part, p.splits, count, out0, out1, scale));
    FB_LAUNCHED(name);
  }
  return FB_OK;
}

// The plain source: x[o][r][c].
struct PlainColSrc {
  const float* x;
  uint64_t red, inner;
  template <int VEC>
  __device__ __forceinline__ void load(uint64_t o, uint64_t r, uint64_t c, float (&v)[1][VEC]) const {
    const float* p = x + (o * red + r) * inner + c;
    if constexpr (VEC == 4) {
      const float4 t = ld_stream4(p);
      v[0][0] = t.x; v[0][1] = t.y; v[0][2] = t.z; v[0][3] = t.w;
    } else {
      v[0][0] = ld_stream(p);
    }
  }
};

}  // namespace fb
