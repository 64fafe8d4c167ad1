// softmax / log_softmax for rows wider than 16384 columns: a thread block
// cluster per row.  Included by softmax.cu only.  Backward first:
//
// Up to 16384 columns a 1024-thread CTA holds g and y of a row in registers
// (4 float4 of each per thread) or the two-sweep kernel finds its second sweep
// in L2.  Beyond that neither works: 8 float4 of each per thread spill, and
// the rows in flight no longer fit L2, so the second sweep reads HBM again
// (70 % of the copy rate at 32768 columns, 63 % at 65536).  Here CL CTAs of
// 1024 threads each keep a slice of at most 16384 columns in registers, read
// from HBM exactly once, and add their partial dot products through
// distributed shared memory (ClusterSum, cluster.cuh): one exchange per row.
// With one CTA of 1024 threads on an SM (slices of 16384 columns) that is a
// modest gain, 73 % and 68 % at 32768 and 65536 columns: nothing covers the
// exchange or the next row's loads.  With 512 threads and 4 float4 of each
// array per thread (slices of 8192 columns on twice the CTAs, two CTAs per SM)
// it is 94 / 87 / 91 % at 32768 / 50000 / 65536 columns; the 1024-thread form
// is kept for rows wider than that.
#pragma once
#include "cluster.cuh"
#include "common.cuh"

namespace fb {

struct SmClusterPlan {
  int cl;           // CTAs per row (0: shape not eligible)
  int threads;      // 1024 (one CTA per SM) or 512 (two)
  int items;        // float4 of g and of y per thread: 2 or 4
  uint32_t slice4;  // float4 per slice (the last slice may be shorter)
};

// threads: 1024 -> slices of at most 16384 columns, 512 -> at most 8192.
static SmClusterPlan sm_cluster_plan(uint64_t cols, int force_cl, int threads) {
  SmClusterPlan p{0, 0, 0, 0};
  const uint64_t cap4 = (uint64_t)threads * 4;  // float4 per slice at 4 items per thread
  if ((cols & 3) || cols <= 16384 || cols > cap4 * 4 * kClusterMax) return p;
  const uint64_t v = cols / 4;
  int cl = force_cl;
  const bool choose = cl == 0;
  if (choose) cl = v <= 2 * cap4 ? 2 : (v <= 4 * cap4 ? 4 : 8);
  if (cl != 2 && cl != 4 && cl != 8) return p;
  const uint64_t slice4 = (v + cl - 1) / cl;
  if (slice4 > cap4 || slice4 * (uint64_t)(cl - 1) >= v) return p;
  // Measured (512 MB per array, % of the copy rate, against the two-sweep kernel): 32768 columns 73 against 70,
  // 65536 columns 68 against 63, but 50000 columns (4 slices of 3125 float4, a quarter of the threads' last
  // item idle) 62 against 63: only slices that fill the threads take this path by default.
  if (choose && threads == 1024 && slice4 * 8 < 7 * cap4) return p;
  p.cl = cl;
  p.threads = threads;
  p.items = slice4 <= cap4 / 2 ? 2 : 4;
  p.slice4 = (uint32_t)slice4;
  return p;
}

// Cluster `cid` of `ncl` walks rows cid, cid + ncl, ...; CTA `rank` of it owns float4 columns
// [rank * slice4, rank * slice4 + my4) of each.
template <int T, int ITEMS, bool LOG>
__global__ void __launch_bounds__(T, 1024 / T)
softmax_bwd_cluster_kernel(const float* __restrict__ g, const float* __restrict__ y, uint64_t rows, uint32_t cols,
                           uint32_t cl, uint32_t slice4, float* __restrict__ dx, unsigned int* faults) {
  __shared__ float2 slots[2 * kClusterMax * (T / 32)];
  __shared__ __align__(8) uint64_t xbar[2];
  const int tid = threadIdx.x;
  const uint32_t rank = cluster_ctarank();
  const uint32_t cols4 = cols / 4, first4 = rank * slice4;
  const uint32_t my4 = first4 + slice4 <= cols4 ? slice4 : cols4 - first4;
  ClusterSum<T> xs;
  xs.init(slots, xbar, cl);
  pdl_wait();
  pdl_trigger();
  const uint64_t cid = blockIdx.x / cl, ncl = gridDim.x / cl;
  uint32_t count = 0;
  for (uint64_t row = cid; row < rows; row += ncl, ++count) {
    const float* gr = g + row * cols + (uint64_t)first4 * 4;
    const float* yr = y + row * cols + (uint64_t)first4 * 4;
    float4 gv[ITEMS], yv[ITEMS];
    float s = 0.0f, unused = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      if (c < my4) {
        gv[k] = ld_stream4(gr + c * 4);
        yv[k] = ld_stream4(yr + c * 4);
      } else {
        gv[k] = yv[k] = make_float4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      if constexpr (LOG) s += (gv[k].x + gv[k].y) + (gv[k].z + gv[k].w);
      else s += (gv[k].x * yv[k].x + gv[k].y * yv[k].y) + (gv[k].z * yv[k].z + gv[k].w * yv[k].w);
    }
    if (!xs.sum(slots, xbar, cl, count, s, unused, faults)) break;
    float* dr = dx + row * cols + (uint64_t)first4 * 4;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      if (c < my4) {
        float4 o;
        if constexpr (LOG) {
          o.x = gv[k].x - __expf(yv[k].x) * s; o.y = gv[k].y - __expf(yv[k].y) * s;
          o.z = gv[k].z - __expf(yv[k].z) * s; o.w = gv[k].w - __expf(yv[k].w) * s;
        } else {
          o.x = yv[k].x * (gv[k].x - s); o.y = yv[k].y * (gv[k].y - s);
          o.z = yv[k].z * (gv[k].z - s); o.w = yv[k].w * (gv[k].w - s);
        }
        st_stream4(dr + c * 4, o);
      }
    }
  }
  cluster_barrier();  // nobody leaves while a peer may still store into its tables
}

// Two-sweep forward over a cluster.  The two-sweep kernel (softmax.cu) counts on its second sweep
// finding the row in L2; with one 512-thread CTA per row and four CTAs per SM, 592 rows are in flight,
// and at 128 KB per row (32000 columns) a fifth of the second sweep misses.  Here CL CTAs share a row
// (each sweeps its own slice twice), so the rows in flight, and the L2 they need, shrink by CL; the
// (maximum, sum of exponentials) pairs cross the cluster once per row, between the sweeps
// (ClusterSum::max_sum).  88 / 83 / 83 / 83 % of the copy rate at 32768 / 50000 / 65536 / 262144 columns
// (clusters of 2 / 2 / 4 / 8) against 85 / 72 / 69 / - % for one CTA per row.
// Measured and dropped: a forward that keeps its slices in registers like the backward above (512
// threads x 4 or 8 float4, two CTAs per SM): 66 / 49 / 58 % at 32768 / 50000 / 65536 columns with one
// exchange of (max, sum) pairs, 68 / 50 / 60 % with two exchanges, 66 / 46 / 56 % with the next row
// prefetched, 49 / 34 / 43 % with one cluster per row on a full grid; 73 % at 131072 columns (this
// kernel: 75.5 %).  A register-resident cluster pays where a kernel writes half of what it reads.
template <bool LOG>
__global__ void __launch_bounds__(512)
softmax_fwd_stream_cluster_kernel(const float* __restrict__ x, uint64_t rows, uint32_t cols, uint32_t cl,
                                  uint32_t slice4, float* __restrict__ y, unsigned int* faults) {
  constexpr int T = 512;
  __shared__ float2 slots[2 * kClusterMax * (T / 32)];
  __shared__ __align__(8) uint64_t xbar[2];
  const int tid = threadIdx.x;
  const uint32_t rank = cluster_ctarank();
  const uint32_t cols4 = cols / 4, first4 = rank * slice4;
  const uint32_t cv = first4 + slice4 <= cols4 ? slice4 : cols4 - first4;  // float4 in this CTA's slice
  ClusterSum<T> xs;
  xs.init(slots, xbar, cl);
  pdl_wait();
  pdl_trigger();
  const uint64_t cid = blockIdx.x / cl, ncl = gridDim.x / cl;
  uint32_t count = 0;
  for (uint64_t row = cid; row < rows; row += ncl, ++count) {
    const float4* xr = reinterpret_cast<const float4*>(x + row * cols) + first4;
    float4* yr = reinterpret_cast<float4*>(y + row * cols) + first4;
    float m = -INFINITY, ms = 0.0f, s = 0.0f;  // ms: the maximum the exponentials are taken against (0 while m is -inf)
    auto fold = [&](float4 v) {
      const float m4 = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
      if (m4 > m) {
        s *= __expf(ms - m4);
        m = ms = m4;
      }
      s += (__expf(v.x - ms) + __expf(v.y - ms)) + (__expf(v.z - ms) + __expf(v.w - ms));
    };
    uint32_t c = tid;
    for (; c + 3 * T < cv; c += 4 * T) {
      const float4 v0 = __ldcg(xr + c), v1 = __ldcg(xr + c + T), v2 = __ldcg(xr + c + 2 * T), v3 = __ldcg(xr + c + 3 * T);
      fold(v0); fold(v1); fold(v2); fold(v3);
    }
    for (; c < cv; c += T) fold(__ldcg(xr + c));
    float M = m, S = s;
    if (!xs.max_sum(slots, xbar, cl, count, M, S, faults)) break;
    const float ls = LOG ? logf(S) : 0.0f;
    const float inv = 1.0f / S;
    auto emit = [&](float4 v, uint32_t cc) {
      float4 o;
      if constexpr (LOG) o = make_float4((v.x - M) - ls, (v.y - M) - ls, (v.z - M) - ls, (v.w - M) - ls);
      else o = make_float4(__expf(v.x - M) * inv, __expf(v.y - M) * inv, __expf(v.z - M) * inv, __expf(v.w - M) * inv);
      __stcs(yr + cc, o);
    };
    c = tid;
    for (; c + 3 * T < cv; c += 4 * T) {
      const float4 v0 = __ldcs(xr + c), v1 = __ldcs(xr + c + T), v2 = __ldcs(xr + c + 2 * T), v3 = __ldcs(xr + c + 3 * T);
      emit(v0, c); emit(v1, c + T); emit(v2, c + 2 * T); emit(v3, c + 3 * T);
    }
    for (; c < cv; c += T) emit(__ldcs(xr + c), c);
  }
  cluster_barrier();
}

}  // namespace fb
