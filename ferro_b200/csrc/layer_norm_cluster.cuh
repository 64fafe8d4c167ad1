// LayerNorm forward / backward for rows of 16384 columns and more: a thread
// block cluster per row.  Included by layer_norm.cu only.
//
// A row that wide needs 1024 threads if one CTA is to hold it in registers.
// That leaves one CTA on an SM, so nothing runs while it sits in its two
// reductions, and the backward (four float4 arrays per item) does not fit 64
// registers at all.  Here CL co-scheduled CTAs (2, 4 or 8) each take a slice
// of the row no wider than the widths the single-CTA pipeline is good at
// (4096 / 8192 columns), stage it with the same bulk-copy pipeline
// (pipe.cuh), and exchange their partial row sums through distributed shared
// memory once per reduction (ClusterSum, cluster.cuh).
//
// The exchange's barrier wait replaces the CTA-wide __syncthreads of the
// single-CTA form: all local warps have signalled, so all have moved their
// part of the slice to registers and the stage can be re-armed.
//
// Also measured and dropped: a backward that works one row ahead (rows stay
// in shared memory; the first pass over row i + 1 - column sums, row sums
// sent - runs before the wait for row i's sums, the dx pass reads row i from
// its stage again).  It hides the exchange but holds every stage two passes
// longer, so fewer rows are in flight: 68 / 62 / 55 % at 16384 / 32768 / 65536
// columns against 83 / 74 / 66 % for the form below.
//
// Only this GPU's memory is touched; no multicast.  Every wait is bounded; a
// wait that gives up records a fault, the CTA stops working on rows and goes
// to the closing cluster barrier (which every CTA reaches, since each of its
// waits is bounded too), so no CTA is left writing into the shared memory of
// one that has exited.
#pragma once
#include "cluster.cuh"
#include "common.cuh"
#include "pipe.cuh"

namespace fb {

struct ClusterPlan {
  int cl;           // CTAs per row (0: shape not eligible)
  int threads;      // 256 or 512
  int items;        // float4 per thread: 2 or 4
  int stages;
  int per_sm;       // CTAs per SM the slice geometry is sized for
  uint32_t slice4;  // float4 per slice (the last slice may be shorter)
  size_t smem;
};

// narr = arrays staged per row (1 forward, 2 backward); force_cl: 0 = choose.
static ClusterPlan cluster_plan(uint64_t cols, int narr, int force_cl) {
  ClusterPlan p{0, 0, 0, 0, 0, 0, 0};
  if ((cols & 3) || cols < 16384 || cols > 8192ull * kClusterMax) return p;
  const uint64_t v = cols / 4;
  int cl = force_cl;
  if (cl == 0) {
    // Measured on rows of 16384 / 32768 / 50000 / 65536 columns (512 MB per array, % of the copy rate; the
    // single-CTA backward forms: 61 / 54 / 44 / 46): 2 CTAs 80-83 / - / - / -; 4 CTAs 69 / 70-74 / - / -;
    // 8 CTAs 69 / 61 / 52-54 / 63-66: the fewest CTAs whose slices fit (8192 columns).
    cl = v <= 2 * 2048 ? 2 : (v <= 4 * 2048 ? 4 : 8);
  }
  if (cl != 2 && cl != 4 && cl != 8) return p;
  const uint64_t slice4 = (v + cl - 1) / cl;
  if (slice4 > 2048 || slice4 * (uint64_t)(cl - 1) >= v) return p;
  int threads, items;
  if (slice4 <= 512) { threads = 256; items = 2; }
  else if (slice4 <= 1024) { threads = narr == 2 ? 512 : 256; items = narr == 2 ? 2 : 4; }
  else { threads = 512; items = 4; }
  const int threads_per_sm = (narr == 1 || (threads == 512 && items == 2) || (threads == 256 && items == 2)) ? 1024 : 768;
  int per_sm = threads_per_sm / threads;
  if (per_sm < 1) per_sm = 1;
  const size_t slice_bytes = (size_t)slice4 * 16 * narr;
  const size_t budget = (size_t)(200 * 1024) / per_sm - 256;
  int stages = (int)(budget / slice_bytes);
  if (stages > 4) stages = 4;
  if (stages < 1) return p;
  p.cl = cl;
  p.threads = threads;
  p.items = items;
  p.stages = stages;
  p.per_sm = per_sm;
  p.slice4 = (uint32_t)slice4;
  p.smem = (size_t)stages * slice_bytes + 64;
  return p;
}

// Upper bound of the clusters a launch of `p` can have resident (what the scratch is sized for).
static uint32_t cluster_plan_max_clusters(const ClusterPlan& p) {
  return p.cl ? (uint32_t)(device_info().sm_count * p.per_sm / p.cl) : 0;
}

// Forward, slices in registers.  The single-CTA forward is at its best with 8 float4 per thread,
// loaded straight from global memory, on 256 threads (8192 columns: 97 % of the copy rate) or 512
// (16384 columns: 90 %, against 71 % for the staged 1024-thread form); this is the same kernel with
// the row spread over CL such CTAs: two exchanges per row (mean, then centred sum of squares),
// clusters walking the rows.  Measured at 32768 / 50000 / 65536 / 131072 columns: 73 / 64 / 70.5 / 63 %
// (slices of 8192 columns on 256 threads up to 65536, of 16384 on 512 threads beyond; the single-CTA
// forms: 72 / 47 / 46 / -), so it takes over above 32768.
// Measured and dropped: a forward with its slices staged in shared memory like the backward's
// (62 / 46 / 56-61 %); slices of 8192 columns on twice the CTAs (64 / 49 / 54 %), the same with the
// next row's loads issued before this row's exchanges (69 / 52 / 62 %), and one cluster per row on
// a full grid instead of resident clusters walking the rows (41 / 28 / 36 %); one exchange per row
// instead of two, each CTA finishing its slice's mean and M2 and the slices merged like the
// partitions of a parallel variance (75 / 60 / 67 / 63 %: a gain at 32768 columns only); and, for the
// backward, slices of 4096 columns in registers on two CTAs per SM (72 / 64 % at 16384 / 32768
// columns against 83 / 74 % for the staged form below), and slices of 8192 columns in registers with
// the two column accumulators in shared memory, the geometry of the cluster softmax backward
// (75 / 68 / 62 % at 16384 / 32768 / 65536 columns; ahead of the staged form only at widths whose
// slices do not fill its stages: 61 against 53 % at 50000 columns).  With the weight slice in shared
// memory as well it drops to 64 / 59 / 54 %: loads that go to registers need room in L1 for their
// lines in flight, and every KB of shared memory a CTA takes comes out of that (128 KB of
// accumulators leave about 100 KB, 192 KB leave about 30); bulk copies into shared memory do not,
// which is why the staged form below can afford 200 KB of stages.  Last, a backward in two sweeps
// (row sums first, the slice left in L2; dx and the column sums, accumulators in registers, from a
// second sweep over it; 512 threads, two CTAs per SM, no shared memory): 70 / 63 / 56 %, with spills.
template <int T, int ITEMS, bool RMS>
__global__ void __launch_bounds__(T, 1024 / T)
ln_fwd_cluster_reg_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                          uint64_t rows, uint32_t cols, uint32_t cl, uint32_t slice4, float eps,
                          float* __restrict__ y, float* __restrict__ h, float* __restrict__ stds,
                          float* __restrict__ mean, float* __restrict__ rstd, unsigned int* faults) {
  __shared__ float2 slots[2 * kClusterMax * (T / 32)];
  __shared__ __align__(8) uint64_t xbar[2];
  const int tid = threadIdx.x;
  const uint32_t rank = cluster_ctarank();
  const uint32_t cols4 = cols / 4, first4 = rank * slice4;
  const uint32_t my4 = first4 + slice4 <= cols4 ? slice4 : cols4 - first4;
  ClusterSum<T> xs;
  xs.init(slots, xbar, cl);
  const uint64_t cid = blockIdx.x / cl, ncl = gridDim.x / cl;
  const float inv_d = 1.0f / (float)cols;
  uint32_t count = 0;
  for (uint64_t row = cid; row < rows; row += ncl) {
    const float* xr = x + row * cols;
    const float x0 = RMS ? 0.0f : __ldg(xr);  // the row's first element, the same shift in every slice
    xr += (uint64_t)first4 * 4;
    float4 v[ITEMS];
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      v[k] = c < my4 ? ld_stream4(xr + c * 4) : make_float4(x0, x0, x0, x0);
    }
    float sum = 0.0f, zero = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      v[k].x -= x0; v[k].y -= x0; v[k].z -= x0; v[k].w -= x0;
      sum += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    }
    float md = 0.0f;
    if constexpr (!RMS) {
      if (!xs.sum(slots, xbar, cl, count++, sum, zero, faults)) break;
      md = sum * inv_d;
    }
    float q = 0.0f;
    zero = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      v[k].x -= md; v[k].y -= md; v[k].z -= md; v[k].w -= md;
      if (c < my4) q += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    }
    if (!xs.sum(slots, xbar, cl, count++, q, zero, faults)) break;
    const float sd = sqrtf(q * inv_d + eps);
    const float rs = 1.0f / sd;
    if (tid == 0 && rank == 0) {
      if (stds) stds[row] = sd;
      if (mean) mean[row] = x0 + md;
      if (rstd) rstd[row] = rs;
    }
    float* yr = y + row * cols + (uint64_t)first4 * 4;
    float* hr = h ? h + row * cols + (uint64_t)first4 * 4 : nullptr;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      if (c < my4) {
        float4 o = make_float4(v[k].x * rs, v[k].y * rs, v[k].z * rs, v[k].w * rs);
        if (hr) st_stream4(hr + c * 4, o);
        if (w) {
          const float4 wv = __ldg(reinterpret_cast<const float4*>(w) + first4 + c);
          o.x *= wv.x; o.y *= wv.y; o.z *= wv.z; o.w *= wv.w;
        }
        if (b) {
          const float4 bv = __ldg(reinterpret_cast<const float4*>(b) + first4 + c);
          o.x += bv.x; o.y += bv.y; o.z += bv.z; o.w += bv.w;
        }
        st_stream4(yr + c * 4, o);
      }
    }
  }
  cluster_barrier();  // nobody leaves while a peer may still store into its tables
}

// MODE 0: saved (h, stds); 1: saved (x, mean, rstd); 2: RMS normalisation, saved (x, rstd), no mean.
// part: [clusters][2][cols] partial dweight / dbias rows, each CTA writing its slice.
template <int T, int ITEMS, int MODE>
__global__ void __launch_bounds__(T, ((ITEMS == 2 ? 1024 : 768) / T) ? ((ITEMS == 2 ? 1024 : 768) / T) : 1)
ln_bwd_cluster_kernel(const float* __restrict__ g, const float* __restrict__ hx,
                      const float* __restrict__ stat_a, const float* __restrict__ stat_b,
                      const float* __restrict__ w, uint64_t rows, uint32_t cols, uint32_t cl, uint32_t slice4,
                      int stages, float* __restrict__ dx, float* __restrict__ part, int want_dw, int want_db,
                      unsigned int* faults) {
  constexpr bool FROM_X = MODE != 0, RMS = MODE == 2;
  extern __shared__ __align__(128) unsigned char pipe_smem[];
  __shared__ float2 slots[2 * kClusterMax * (T / 32)];
  __shared__ __align__(8) uint64_t xbar[2];
  const int tid = threadIdx.x;
  const uint32_t rank = cluster_ctarank();
  const uint32_t cols4 = cols / 4, first4 = rank * slice4;
  const uint32_t my4 = first4 + slice4 <= cols4 ? slice4 : cols4 - first4;
  const uint32_t my_bytes = my4 * 16;
  float* stage = reinterpret_cast<float*>(pipe_smem);  // [stages][2][slice4 * 4]: g slice, then h (or x) slice
  uint64_t* full = reinterpret_cast<uint64_t*>(pipe_smem + (size_t)stages * slice4 * 32);
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  ClusterSum<T> xs;
  xs.init(slots, xbar, cl);
  __syncthreads();
  pdl_wait();
  pdl_trigger();
  const uint64_t cid = blockIdx.x / cl, ncl = gridDim.x / cl;
  const uint64_t mine = rows > cid ? (rows - cid + ncl - 1) / ncl : 0;
  const uint64_t step = ncl * cols;
  const float inv_d = 1.0f / (float)cols;
  uint64_t next = cid * cols + (uint64_t)first4 * 4, requested = 0;  // thread 0 only
  auto arm = [&](int s) {
    float* dst = stage + (size_t)s * slice4 * 8;
    mbar_expect_tx(&full[s], 2 * my_bytes);
    bulk_load(dst, g + next, my_bytes, &full[s]);
    bulk_load(dst + slice4 * 4, hx + next, my_bytes, &full[s]);
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
  float* dxrow = dx + cid * cols + (uint64_t)first4 * 4;
  uint64_t row = cid;
  for (uint64_t i = 0; i < mine; ++i, row += ncl, dxrow += step) {
    float mu = 0.0f, rs;
    if constexpr (FROM_X) {
      mu = RMS ? 0.0f : __ldg(stat_a + row);
      rs = __ldg(stat_b + row);
    } else {
      rs = 1.0f / __ldg(stat_a + row);
    }
    if (!__all_sync(0xffffffffu, mbar_wait(&full[s], parity, faults))) break;
    const float4* sg = reinterpret_cast<const float4*>(stage + (size_t)s * slice4 * 8);
    const float4* sh = sg + slice4;
    float4 gv[ITEMS], hv[ITEMS];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      float4 wv = make_float4(1, 1, 1, 1);
      if (c < my4) {
        gv[k] = sg[c];
        hv[k] = sh[c];
        if (w) wv = __ldg(reinterpret_cast<const float4*>(w) + first4 + c);
      } else {
        gv[k] = hv[k] = make_float4(0, 0, 0, 0);
      }
      if constexpr (FROM_X) {
        if (c < my4) {
          hv[k].x = (hv[k].x - mu) * rs; hv[k].y = (hv[k].y - mu) * rs;
          hv[k].z = (hv[k].z - mu) * rs; hv[k].w = (hv[k].w - mu) * rs;
        }
      }
      aw[k].x += gv[k].x * hv[k].x; aw[k].y += gv[k].y * hv[k].y;
      aw[k].z += gv[k].z * hv[k].z; aw[k].w += gv[k].w * hv[k].w;
      ab[k].x += gv[k].x; ab[k].y += gv[k].y; ab[k].z += gv[k].z; ab[k].w += gv[k].w;
      gv[k].x *= wv.x; gv[k].y *= wv.y; gv[k].z *= wv.z; gv[k].w *= wv.w;  // from here on: dxh = g * w
      s1 += (gv[k].x + gv[k].y) + (gv[k].z + gv[k].w);
      s2 += (gv[k].x * hv[k].x + gv[k].y * hv[k].y) + (gv[k].z * hv[k].z + gv[k].w * hv[k].w);
    }
    if (!xs.sum(slots, xbar, cl, (uint32_t)i, s1, s2, faults)) break;
    if (tid == 0 && requested < mine) arm(s);
    const float m1 = RMS ? 0.0f : s1 * inv_d;
    const float m2 = s2 * inv_d;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      if (c < my4) {
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
    float* pw = part + cid * 2 * cols + (uint64_t)first4 * 4;
    float* pb = pw + cols;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = tid + k * T;
      if (c < my4) {
        if (want_dw) *reinterpret_cast<float4*>(pw + c * 4) = aw[k];
        if (want_db) *reinterpret_cast<float4*>(pb + c * 4) = ab[k];
      }
    }
  }
  cluster_barrier();
}

}  // namespace fb
