// Row softmax / log_softmax forward and backward, their fused forms with a
// bias+relu+scale prologue, and the fused log_softmax + NLL over i64 targets.
//
// Roofline: HBM.  Algorithmic bytes per row of `cols` f32:
//   softmax / log_softmax forward      read x, write y            8 * cols
//   their backward                     read g, y, write dx        12 * cols
//   prologue forward                   read x, write y            8 * cols (+ bias once)
//   prologue backward                  read g, y, x, write dx     16 * cols (+ dbias partials)
//   log_softmax+NLL forward            read logits                4 * cols (+ 3 row scalars)
//   log_softmax+NLL backward           read logits, write dlogits 8 * cols
// The exponentials of these kernels use the exp2-based __expf (relative error
// about |x| * 1e-7, far inside the 2e-4 bar of this family) and the softmax
// divides by multiplying with 1/sum: both keep the kernels from being bound
// by instruction issue at short rows.
// Fast path: the row sits in the registers of G threads (forward up to 16384
// columns, backward up to 8192), one row block per CTA on a full grid, giving
// the exact max-then-sum of ferro's host loop (ops_ext/softmax.rs:68-88) at
// one read of x; the reference kernels read x three times in two launches
// (crates/ferro-cuda/src/kernels.rs:536-588).  Longer rows: one CTA per row
// and two sweeps, the second served by L2 for the rows that are still there.
// Generic path (widths that are not a multiple of 4, unaligned buffers): one
// CTA per row, scalar accesses, re-reading the row through L2.
#include <cstdlib>

#include "common.cuh"
#include "reduce.cuh"
#include "softmax_wp.cuh"
#include "softmax_cluster.cuh"
#include "softmax_rows.cuh"

namespace fb {

// FB_SOFTMAX_WP=0 in the environment keeps rows of 256 .. 1024 columns on the register kernels
// (for A/B measurements); anything else, or nothing, uses the warp-pipelined kernels there.
static bool wp_enabled() {
  static const int on = [] {
    const char* e = getenv("FB_SOFTMAX_WP");
    return (e && e[0] == '0') ? 0 : 1;
  }();
  return on != 0;
}

// FB_SM_ROWS=0 keeps rows shorter than 256 columns on the one-row-per-warp kernels (A/B measurements).
static bool rows_enabled() {
  static const int on = [] { const char* e = getenv("FB_SM_ROWS"); return (e && e[0] == '0') ? 0 : 1; }();
  return on != 0;
}

// FB_SM_CLUSTER in the environment: 0 keeps rows wider than 16384 columns on the two-sweep kernel,
// 2 / 4 / 8 fixes the cluster size (for A/B measurements); anything else, or nothing, lets the plan choose.
static int sm_cluster_choice() {
  static const int v = [] {
    const char* e = getenv("FB_SM_CLUSTER");
    if (!e || !*e) return -1;
    const int n = atoi(e);
    return (n == 0 || n == 2 || n == 4 || n == 8) ? n : -1;
  }();
  return v;
}

// Cluster size for the two-sweep forward (softmax_fwd_stream_cluster_kernel), 0 = one CTA per row.
// FB_SM_STREAM_CLUSTER=0|2|4|8 overrides the choice (A/B measurements).  Measured, % of the copy rate,
// one CTA per row / clusters of 2 / of 4: 20000 columns 94 / 73 / 46, 32000 columns 90 / 89 / 66,
// 32768 columns 85 / 89 / 68, 50000 columns 72 / 84 / 66, 65536 columns 69 / 78 / 83.
static int sm_stream_cluster(uint64_t cols) {
  static const int v = [] {
    const char* e = getenv("FB_SM_STREAM_CLUSTER");
    if (!e || !*e) return -1;
    const int n = atoi(e);
    return (n == 0 || n == 2 || n == 4 || n == 8) ? n : -1;
  }();
  if (v >= 0) return v;
  if (cols < 32768) return 0;
  return cols < 57344 ? 2 : (cols < 114688 ? 4 : 8);
}
static int sm_cluster_threads() {
  static const int v = [] { const char* e = getenv("FB_SM_CLUSTER_T"); return (e && atoi(e) == 1024) ? 1024 : 512; }();
  return v;
}

template <int G>
constexpr int sm_threads() { return G < 256 ? 256 : G; }

struct Prologue {  // v = act(x + bias[c]) * scale
  const float* bias;
  float scale;
  int relu;
  int on;
  int smem;  // the forward register kernel finds the bias in dynamic shared memory (set by the launcher)
};

// v when v > 0 or v is NaN, else +0: one ordered compare (a short-circuit `||` here compiles to a branch).
__device__ __forceinline__ float relu_nan(float v) { return !(v <= 0.0f) ? v : 0.0f; }

__device__ __forceinline__ float4 apply_prologue(const Prologue& p, float4 v, uint32_t c4) {
  if (p.bias) {
    const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias) + c4);
    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
  }
  if (p.relu) { v.x = relu_nan(v.x); v.y = relu_nan(v.y); v.z = relu_nan(v.z); v.w = relu_nan(v.w); }
  v.x *= p.scale; v.y *= p.scale; v.z *= p.scale; v.w *= p.scale;
  return v;
}

// ------------------------------------------------------------------ forward
// PRO: the bias / relu / scale prologue is present.  It is applied in a pass
// of its own after every load of the row has been issued, so the loads stay
// back to back whatever the prologue's flags are.
template <int G, int ITEMS, bool LOG, bool PRO>
__global__ void __launch_bounds__(sm_threads<G>())
softmax_fwd_reg_kernel(const float* __restrict__ x, Prologue pro, uint64_t rows, uint32_t cols,
                       float* __restrict__ y) {
  constexpr int T = sm_threads<G>();
  constexpr int R = T / G;
  __shared__ float red_a[T / 32], red_b[T / 32];
  const uint32_t cols4 = cols / 4;
  const int grp = threadIdx.x / G, lane = threadIdx.x % G;
  const uint64_t nblk = (rows + R - 1) / R;
  // The bias is staged in shared memory once per CTA: read from global inside the
  // prologue loop, its loads sit behind that loop's uniform branches and are
  // issued one after the other, ITEMS cache latencies in a row on the critical
  // path of a kernel that lives for a few microseconds.
  extern __shared__ __align__(16) float4 bias_smem[];
  pdl_wait();     // launched with launch_pdl: the kernel before this one in the stream is complete from here on
  pdl_trigger();
  bool bias_staged = false;
  for (uint64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
    const uint64_t row = blk * R + grp;
    const bool live = row < rows;
    float4 v[ITEMS];
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      v[k] = (live && c < cols4) ? ld_stream4(x + row * cols + c * 4)
                                 : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
    if constexpr (PRO) {
      // Staged behind the first block's row loads, so that its latency hides under theirs
      // (a CTA of a full grid has one block only).
      if (pro.smem && !bias_staged) {
        for (uint32_t c = threadIdx.x; c < cols4; c += T) bias_smem[c] = __ldg(reinterpret_cast<const float4*>(pro.bias) + c);
        __syncthreads();
        bias_staged = true;
      }
    }
    if constexpr (PRO) {
      if (pro.smem) {
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
          const uint32_t c = lane + k * G;
          if (c < cols4) {  // the -inf padding must stay -inf through the relu
            const float4 b = bias_smem[c];
            float4 t = make_float4(v[k].x + b.x, v[k].y + b.y, v[k].z + b.z, v[k].w + b.w);
            if (pro.relu) { t.x = relu_nan(t.x); t.y = relu_nan(t.y); t.z = relu_nan(t.z); t.w = relu_nan(t.w); }
            v[k] = make_float4(t.x * pro.scale, t.y * pro.scale, t.z * pro.scale, t.w * pro.scale);
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
          const uint32_t c = lane + k * G;
          if (c < cols4) v[k] = apply_prologue(pro, v[k], c);
        }
      }
    }
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) m = fmaxf(m, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
    m = group_max<G>(m, red_a);
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      float4 e;
      v[k].x -= m; v[k].y -= m; v[k].z -= m; v[k].w -= m;
      e.x = __expf(v[k].x); e.y = __expf(v[k].y); e.z = __expf(v[k].z); e.w = __expf(v[k].w);
      if (c < cols4) s += (e.x + e.y) + (e.z + e.w);
      if constexpr (!LOG) v[k] = e;
    }
    s = group_sum<G>(s, red_b);
    const float ls = LOG ? logf(s) : 0.0f;
    const float inv = 1.0f / s;
    if (live) {
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = lane + k * G;
        if (c < cols4) {
          float4 o;
          if constexpr (LOG) {
            o = make_float4(v[k].x - ls, v[k].y - ls, v[k].z - ls, v[k].w - ls);
          } else {
            o = make_float4(v[k].x * inv, v[k].y * inv, v[k].z * inv, v[k].w * inv);
          }
          st_stream4(y + row * cols + c * 4, o);
        }
      }
    }
  }
}

// Streaming form for rows too long to hold in registers with more than one
// CTA per SM (cols > 16384): one CTA per row and two sweeps.  The first folds
// the row into a running (max, sum of exp(x - max)) per thread as the float4s
// arrive from HBM, with loads that leave the lines in L2; the second re-reads
// the row, which the CTA has just pulled through L2, and writes the result
// with streaming stores.  Several CTAs per SM keep loads in flight across the
// reductions between the sweeps.  The running max of a thread moves only a
// handful of times per row, so the rescale branch is cold.
template <bool LOG, int T>
__global__ void __launch_bounds__(T)
softmax_fwd_stream_kernel(const float* __restrict__ x, Prologue pro, uint64_t rows, uint32_t cols,
                          float* __restrict__ y) {
  __shared__ float red_a[T / 32], red_b[T / 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t cv = cols / 4;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float4* xr = reinterpret_cast<const float4*>(x + row * cols);
    float4* yr = reinterpret_cast<float4*>(y + row * cols);
    // `ms` is the max the exponentials are taken against: m once an element
    // above -inf has been seen, 0 until then, so that leading -inf elements
    // add exp(-inf - 0) = 0 instead of exp(-inf - -inf) = NaN.
    float m = -INFINITY, ms = 0.0f, s = 0.0f;
    auto fold = [&](float4 v, uint32_t c) {
      if (pro.on) v = apply_prologue(pro, v, c);
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
      fold(v0, c); fold(v1, c + T); fold(v2, c + 2 * T); fold(v3, c + 3 * T);
    }
    for (; c < cv; c += T) fold(__ldcg(xr + c), c);
    // Row max, then the threads' sums rescaled to it.  exp(-inf - M) = 0 drops a
    // thread that saw nothing; M = -inf (a row of -inf) gives NaN like the host loop.
    float M = warp_max(m);
    if (lane == 0) red_a[warp] = M;
    __syncthreads();
    M = warp_max(lane < T / 32 ? red_a[lane] : -INFINITY);
    float S = warp_sum(s * __expf(m - M));
    if (lane == 0) red_b[warp] = S;
    __syncthreads();
    S = warp_sum(lane < T / 32 ? red_b[lane] : 0.0f);
    const float ls = LOG ? logf(S) : 0.0f;
    const float inv = 1.0f / S;
    auto emit = [&](float4 v, uint32_t c) {
      if (pro.on) v = apply_prologue(pro, v, c);
      float4 o;
      if constexpr (LOG) {
        o = make_float4((v.x - M) - ls, (v.y - M) - ls, (v.z - M) - ls, (v.w - M) - ls);
      } else {
        o = make_float4(__expf(v.x - M) * inv, __expf(v.y - M) * inv, __expf(v.z - M) * inv, __expf(v.w - M) * inv);
      }
      __stcs(yr + c, o);
    };
    c = tid;
    for (; c + 3 * T < cv; c += 4 * T) {
      const float4 v0 = __ldcs(xr + c), v1 = __ldcs(xr + c + T), v2 = __ldcs(xr + c + 2 * T), v3 = __ldcs(xr + c + 3 * T);
      emit(v0, c); emit(v1, c + T); emit(v2, c + 2 * T); emit(v3, c + 3 * T);
    }
    for (; c < cv; c += T) emit(__ldcs(xr + c), c);
    // red_a / red_b are rewritten only after the next row's sweep, which every
    // warp enters after passing the second barrier above.
  }
}

template <bool LOG>
__global__ void __launch_bounds__(256)
softmax_fwd_generic_kernel(const float* __restrict__ x, Prologue pro, uint64_t rows, uint64_t cols,
                           float* __restrict__ y) {
  __shared__ float red[32];
  auto pre = [&](uint64_t c, float v) {
    if (!pro.on) return v;
    if (pro.bias) v += pro.bias[c];
    if (pro.relu) v = relu_nan(v);
    return v * pro.scale;
  };
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    float m = -INFINITY;
    for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, pre(c, xr[c]));
    m = block_max(m, red);
    float s = 0.0f;
    for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) s += expf(pre(c, xr[c]) - m);
    s = block_sum(s, red);
    const float ls = LOG ? logf(s) : 0.0f;
    for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float d = pre(c, xr[c]) - m;
      y[row * cols + c] = LOG ? d - ls : expf(d) / s;
    }
  }
}

// ----------------------------------------------------------------- backward
// Geometry with at most 2 float4 per thread per array (three arrays and the
// dbias accumulators live at once; more would halve the CTAs per SM, and these
// kernels need the warps to hide latency).
static RowCfg bwd_cfg(uint64_t cols) {
  RowCfg c{0, 0};
  if (cols == 0 || (cols & 3)) return c;
  const uint64_t v = cols / 4;
  for (int g = 32; g <= 1024; g <<= 1) {
    const int cap = (g == 1024) ? 8 : 2;
    if (v <= (uint64_t)g * cap) {
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

// FUSED: dx = relu_backward(dt * scale, x + bias) and per-CTA dbias partials.
// Persistent grid (gridDim.x CTAs); `part` is [gridDim.x][cols].
template <int G, int ITEMS, bool LOG, bool FUSED>
__global__ void __launch_bounds__(sm_threads<G>())
softmax_bwd_reg_kernel(const float* __restrict__ g, const float* __restrict__ y,
                       const float* __restrict__ x, Prologue pro, uint64_t rows, uint32_t cols,
                       float* __restrict__ dx, float* __restrict__ part) {
  constexpr int T = sm_threads<G>();
  constexpr int R = T / G;
  __shared__ float red_a[T / 32];
  __shared__ __align__(16) float comb[FUSED && R > 1 ? 4096 : 4];
  const uint32_t cols4 = cols / 4;
  const int grp = threadIdx.x / G, lane = threadIdx.x % G;
  const uint64_t nblk = (rows + R - 1) / R;
  float4 acc[FUSED ? ITEMS : 1];
  extern __shared__ __align__(16) float4 bias_smem[];  // the bias, staged once per CTA (see the forward kernel)
  pdl_wait();
  pdl_trigger();
  if constexpr (FUSED) {
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) acc[k] = make_float4(0, 0, 0, 0);
    if (pro.smem) {
      for (uint32_t c = threadIdx.x; c < cols4; c += T) bias_smem[c] = __ldg(reinterpret_cast<const float4*>(pro.bias) + c);
      __syncthreads();
    }
  }
  for (uint64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
    const uint64_t row = blk * R + grp;
    const bool live = row < rows;
    float4 gv[ITEMS], yv[ITEMS];
    float4 xv[FUSED ? ITEMS : 1];  // the relu mask's input, fetched with g and y: one memory latency per row, not two
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      if (live && c < cols4) {
        gv[k] = ld_stream4(g + row * cols + c * 4);
        yv[k] = ld_stream4(y + row * cols + c * 4);
        if constexpr (FUSED) {
          if (pro.relu) xv[k] = ld_stream4(x + row * cols + c * 4);
        }
      } else {
        gv[k] = yv[k] = make_float4(0, 0, 0, 0);
      }
      if constexpr (LOG) s += (gv[k].x + gv[k].y) + (gv[k].z + gv[k].w);
      else s += (gv[k].x * yv[k].x + gv[k].y * yv[k].y) + (gv[k].z * yv[k].z + gv[k].w * yv[k].w);
    }
    __syncthreads();  // red_a is reused every iteration
    s = group_sum<G>(s, red_a);
    if (live) {
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = lane + k * G;
        if (c < cols4) {
          float4 o;
          if constexpr (LOG) {
            o.x = gv[k].x - __expf(yv[k].x) * s; o.y = gv[k].y - __expf(yv[k].y) * s;
            o.z = gv[k].z - __expf(yv[k].z) * s; o.w = gv[k].w - __expf(yv[k].w) * s;
          } else {
            o.x = yv[k].x * (gv[k].x - s); o.y = yv[k].y * (gv[k].y - s);
            o.z = yv[k].z * (gv[k].z - s); o.w = yv[k].w * (gv[k].w - s);
          }
          if constexpr (FUSED) {
            o.x *= pro.scale; o.y *= pro.scale; o.z *= pro.scale; o.w *= pro.scale;
            if (pro.relu) {
              float4 a = xv[k];
              if (pro.bias) {
                const float4 b = pro.smem ? bias_smem[c] : __ldg(reinterpret_cast<const float4*>(pro.bias) + c);
                a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
              }
              o.x = a.x <= 0.0f ? 0.0f : o.x; o.y = a.y <= 0.0f ? 0.0f : o.y;
              o.z = a.z <= 0.0f ? 0.0f : o.z; o.w = a.w <= 0.0f ? 0.0f : o.w;
            }
            acc[k].x += o.x; acc[k].y += o.y; acc[k].z += o.z; acc[k].w += o.w;
          }
          st_stream4(dx + row * cols + c * 4, o);
        }
      }
    }
  }
  if constexpr (FUSED) {
    if (part) {
      float* pr = part + (uint64_t)blockIdx.x * cols;
      if constexpr (R > 1) {
        // Fold the R row groups of the CTA in group order, then write one row.
        __syncthreads();
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
          const uint32_t c = lane + k * G;
          if (c < cols4) *reinterpret_cast<float4*>(comb + (size_t)grp * cols + c * 4) = acc[k];
        }
        __syncthreads();
        for (uint32_t c = threadIdx.x; c < cols; c += T) {
          float t = comb[c];
#pragma unroll
          for (int r = 1; r < R; ++r) t += comb[(size_t)r * cols + c];
          pr[c] = t;
        }
      } else {
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
          const uint32_t c = lane + k * G;
          if (c < cols4) *reinterpret_cast<float4*>(pr + c * 4) = acc[k];
        }
      }
    }
  }
}

// (Two-sweep forward: L2 residency hints - createpolicy evict_last on the first sweep's loads,
// evict_first on the second's - were measured and change nothing: log_softmax of [16384, 32000]
// 721 us with, 713 us without; 32768 / 50000 / 65536 columns 84 / 72 / 70 % either way.)
//
// Streaming backward for long rows (cols > 8192, float4-addressable): one CTA
// per row on a full grid and two sweeps.  The first adds up the row's dot
// product (softmax: sum g*y, reading both arrays; log_softmax: sum g, reading
// g only) with loads that leave the lines in L2; the second re-reads what the
// first pulled in, touches the rest for the first time and writes dx.
template <bool LOG, int T>
__global__ void __launch_bounds__(T)
softmax_bwd_stream_kernel(const float* __restrict__ g, const float* __restrict__ y, uint64_t rows,
                          uint32_t cols, float* __restrict__ dx) {
  __shared__ float red[T / 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t cv = cols / 4;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float4* gr = reinterpret_cast<const float4*>(g + row * cols);
    const float4* yr = reinterpret_cast<const float4*>(y + row * cols);
    float4* dr = reinterpret_cast<float4*>(dx + row * cols);
    float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
    uint32_t c = tid;
    if constexpr (LOG) {
      for (; c + 3 * T < cv; c += 4 * T) {
        const float4 v0 = __ldcg(gr + c), v1 = __ldcg(gr + c + T), v2 = __ldcg(gr + c + 2 * T), v3 = __ldcg(gr + c + 3 * T);
        a0 += (v0.x + v0.y) + (v0.z + v0.w);
        a1 += (v1.x + v1.y) + (v1.z + v1.w);
        a2 += (v2.x + v2.y) + (v2.z + v2.w);
        a3 += (v3.x + v3.y) + (v3.z + v3.w);
      }
      for (; c < cv; c += T) {
        const float4 v0 = __ldcg(gr + c);
        a0 += (v0.x + v0.y) + (v0.z + v0.w);
      }
    } else {
      for (; c + T < cv; c += 2 * T) {
        const float4 v0 = __ldcg(gr + c), w0 = __ldcg(yr + c), v1 = __ldcg(gr + c + T), w1 = __ldcg(yr + c + T);
        a0 += (v0.x * w0.x + v0.y * w0.y) + (v0.z * w0.z + v0.w * w0.w);
        a1 += (v1.x * w1.x + v1.y * w1.y) + (v1.z * w1.z + v1.w * w1.w);
      }
      for (; c < cv; c += T) {
        const float4 v0 = __ldcg(gr + c), w0 = __ldcg(yr + c);
        a0 += (v0.x * w0.x + v0.y * w0.y) + (v0.z * w0.z + v0.w * w0.w);
      }
    }
    float s = warp_sum((a0 + a1) + (a2 + a3));
    __syncthreads();  // the previous row's readers are done with red
    if (lane == 0) red[warp] = s;
    __syncthreads();
    s = warp_sum(lane < T / 32 ? red[lane] : 0.0f);
    auto emit = [&](uint32_t k) {
      const float4 gg = __ldcs(gr + k), yy = __ldcs(yr + k);
      float4 o;
      if constexpr (LOG) {
        o = make_float4(gg.x - __expf(yy.x) * s, gg.y - __expf(yy.y) * s, gg.z - __expf(yy.z) * s, gg.w - __expf(yy.w) * s);
      } else {
        o = make_float4(yy.x * (gg.x - s), yy.y * (gg.y - s), yy.z * (gg.z - s), yy.w * (gg.w - s));
      }
      __stcs(dr + k, o);
    };
    for (c = tid; c + T < cv; c += 2 * T) {
      emit(c);
      emit(c + T);
    }
    for (; c < cv; c += T) emit(c);
  }
}

template <bool LOG, bool FUSED>
__global__ void __launch_bounds__(256)
softmax_bwd_generic_kernel(const float* __restrict__ g, const float* __restrict__ y,
                           const float* __restrict__ x, Prologue pro, uint64_t rows, uint64_t cols,
                           float* __restrict__ dx, float* __restrict__ part) {
  __shared__ float red[32];
  float* pr = (FUSED && part) ? part + (uint64_t)blockIdx.x * cols : nullptr;
  if (pr)
    for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) pr[c] = 0.0f;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* gr = g + row * cols;
    const float* yr = y + row * cols;
    float s = 0.0f;
    for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) s += LOG ? gr[c] : gr[c] * yr[c];
    s = block_sum(s, red);
    for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      float o = LOG ? gr[c] - expf(yr[c]) * s : yr[c] * (gr[c] - s);
      if constexpr (FUSED) {
        o *= pro.scale;
        if (pro.relu) {
          float a = x[row * cols + c];
          if (pro.bias) a += pro.bias[c];
          o = a <= 0.0f ? 0.0f : o;
        }
        if (pr) pr[c] += o;
      }
      dx[row * cols + c] = o;
    }
  }
}

// --------------------------------------------------- log_softmax + NLL fused
template <int G, int ITEMS>
__global__ void __launch_bounds__(sm_threads<G>())
nll_fwd_reg_kernel(const float* __restrict__ x, const int64_t* __restrict__ targets, uint64_t rows,
                   uint32_t cols, float* __restrict__ row_loss, float* __restrict__ row_max,
                   float* __restrict__ row_lse, int64_t* __restrict__ argmax,
                   int64_t* __restrict__ bad) {
  constexpr int T = sm_threads<G>();
  constexpr int R = T / G;
  __shared__ float red_a[T / 32], red_b[T / 32], red_v[T / 32];
  __shared__ unsigned long long red_i[T / 32];
  const uint32_t cols4 = cols / 4;
  const int grp = threadIdx.x / G, lane = threadIdx.x % G;
  const uint64_t nblk = (rows + R - 1) / R;
  for (uint64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
    const uint64_t row = blk * R + grp;
    const bool live = row < rows;
    float4 v[ITEMS];
    float m = -INFINITY;
    Best best = best_identity();
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      if (live && c < cols4) {
        v[k] = ld_stream4(x + row * cols + c * 4);
        if (argmax) {
          const uint64_t e = (uint64_t)c * 4;
          best = best_of(best, Best{v[k].x, e});
          best = best_of(best, Best{v[k].y, e + 1});
          best = best_of(best, Best{v[k].z, e + 2});
          best = best_of(best, Best{v[k].w, e + 3});
        }
      } else {
        v[k] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
      m = fmaxf(m, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
    }
    m = group_max<G>(m, red_a);
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      if (c < cols4)
        s += (expf(v[k].x - m) + expf(v[k].y - m)) + (expf(v[k].z - m) + expf(v[k].w - m));
    }
    s = group_sum<G>(s, red_b);
    if (argmax) best = group_best<G>(best, red_v, red_i);
    if (live && lane == 0) {
      const float lse = logf(s);
      row_max[row] = m;
      row_lse[row] = lse;
      if (argmax) argmax[row] = (int64_t)best.i;
      const int64_t t = targets[row];
      float l = 0.0f;
      if (t >= 0 && (uint64_t)t < cols) {
        l = -((__ldg(x + row * cols + t) - m) - lse);
      } else if (bad) {
        *bad = (int64_t)row + 1;
      }
      row_loss[row] = l;
    }
  }
}

// Streaming form for long rows: one CTA per row, every thread folds its share
// of the row into a running (max, sum of exp(x - max), index of the max) as
// the float4s arrive, so the row is read once and never held.  The running
// max only moves a handful of times per thread (the chance that element k
// beats the k-1 before it is 1/k), so the rescale branch is cold and the hot
// path is one subtract, one exp2-based exp and one add per element.
// NaN handling: a NaN never wins the `>` that moves the max, but it poisons
// the sum; a NaN sum sends the CTA (uniformly) to a rescan that finds the
// first NaN, which is what ferro's argmax returns (ops_ext/argmax.rs:50-60).
template <int VEC, int T>
__global__ void __launch_bounds__(T)
nll_fwd_stream_kernel(const float* __restrict__ x, const int64_t* __restrict__ targets, uint64_t rows,
                      uint32_t cols, float* __restrict__ row_loss, float* __restrict__ row_max,
                      float* __restrict__ row_lse, int64_t* __restrict__ argmax,
                      int64_t* __restrict__ bad) {
  __shared__ float red_f[T / 32];
  __shared__ uint32_t red_u[T / 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t cv = cols / VEC;
  auto block_maxf = [&](float v) {
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red_f[warp] = v;
    __syncthreads();
    float t = lane < T / 32 ? red_f[lane] : -INFINITY;
    return warp_max(t);
  };
  auto block_sumf = [&](float v) {
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red_f[warp] = v;
    __syncthreads();
    float t = lane < T / 32 ? red_f[lane] : 0.0f;
    return warp_sum(t);
  };
  auto block_minu = [&](uint32_t v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) red_u[warp] = v;
    __syncthreads();
    uint32_t t = lane < T / 32 ? red_u[lane] : 0xffffffffu;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
    return t;
  };
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    // `ms` stands in for m in the exponentials: 0 while the thread has seen
    // nothing above -inf (so -inf elements add 0, not exp(-inf - -inf) = NaN).
    float m = -INFINITY, ms = 0.0f, s = 0.0f;
    uint32_t bi = (uint32_t)tid * VEC;  // index of the first element equal to m among this thread's
    auto fold = [&](float a, float b, float c, float d, uint32_t e) {
      const float m4 = fmaxf(fmaxf(a, b), fmaxf(c, d));
      if (m4 > m) {
        s *= __expf(ms - m4);
        m = ms = m4;
        bi = e + (a == m4 ? 0u : (b == m4 ? 1u : (c == m4 ? 2u : 3u)));
      }
      s += (__expf(a - ms) + __expf(b - ms)) + (__expf(c - ms) + __expf(d - ms));
    };
    if constexpr (VEC == 4) {
      uint32_t c = tid;
      for (; c + 3 * T < cv; c += 4 * T) {
        const float4 v0 = ld_stream4(xr + (uint64_t)c * 4), v1 = ld_stream4(xr + (uint64_t)(c + T) * 4);
        const float4 v2 = ld_stream4(xr + (uint64_t)(c + 2 * T) * 4), v3 = ld_stream4(xr + (uint64_t)(c + 3 * T) * 4);
        fold(v0.x, v0.y, v0.z, v0.w, c * 4);
        fold(v1.x, v1.y, v1.z, v1.w, (c + T) * 4);
        fold(v2.x, v2.y, v2.z, v2.w, (c + 2 * T) * 4);
        fold(v3.x, v3.y, v3.z, v3.w, (c + 3 * T) * 4);
      }
      for (; c < cv; c += T) {
        const float4 v0 = ld_stream4(xr + (uint64_t)c * 4);
        fold(v0.x, v0.y, v0.z, v0.w, c * 4);
      }
    } else {
      for (uint32_t c = tid; c < cols; c += T) {
        const float v = xr[c];
        if (v > m) {
          s *= __expf(ms - v);
          m = ms = v;
          bi = c;
        }
        s += __expf(v - ms);
      }
    }
    const float M = block_maxf(m);
    // exp(-inf - M) = 0 drops threads that saw nothing; M = -inf gives NaN like the host loop.
    const float S = block_sumf(s * __expf(m - M));
    uint32_t best = 0;
    if (argmax) {
      if (isnan(S)) {  // uniform: some element is NaN (or the row is all -inf / has +inf)
        uint32_t first = 0xffffffffu;
        for (uint32_t c = tid; c < cols; c += T)
          if (isnan(xr[c])) { first = c; break; }
        best = block_minu(first);
        if (best == 0xffffffffu) best = block_minu(m == M ? bi : 0xffffffffu);  // no NaN element after all
      } else {
        best = block_minu(m == M ? bi : 0xffffffffu);
      }
    }
    if (tid == 0) {
      const float lse = logf(S);
      row_max[row] = M;
      row_lse[row] = lse;
      if (argmax) argmax[row] = (int64_t)best;
      const int64_t t = targets[row];
      float l = 0.0f;
      if (t >= 0 && (uint64_t)t < cols) l = -((__ldg(xr + t) - M) - lse);
      else if (bad) *bad = (int64_t)row + 1;
      row_loss[row] = l;
    }
  }
}

__global__ void __launch_bounds__(256)
nll_fwd_generic_kernel(const float* __restrict__ x, const int64_t* __restrict__ targets,
                       uint64_t rows, uint64_t cols, float* __restrict__ row_loss,
                       float* __restrict__ row_max, float* __restrict__ row_lse,
                       int64_t* __restrict__ argmax, int64_t* __restrict__ bad) {
  __shared__ float red[32];
  __shared__ float sv[32];
  __shared__ unsigned long long si[32];
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    float m = -INFINITY;
    Best best = best_identity();
    for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float v = xr[c];
      m = fmaxf(m, v);
      best = best_of(best, Best{v, c});
    }
    m = block_max(m, red);
    float s = 0.0f;
    for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) s += expf(xr[c] - m);
    s = block_sum(s, red);
    if (argmax) {
      best = warp_best(best);
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
      __syncthreads();
      if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
      __syncthreads();
      best = lane < nw ? Best{sv[lane], si[lane]} : best_identity();
      best = warp_best(best);
    }
    if (threadIdx.x == 0) {
      const float lse = logf(s);
      row_max[row] = m;
      row_lse[row] = lse;
      if (argmax) argmax[row] = (int64_t)best.i;
      const int64_t t = targets[row];
      float l = 0.0f;
      if (t >= 0 && (uint64_t)t < cols) l = -((xr[t] - m) - lse);
      else if (bad) *bad = (int64_t)row + 1;
      row_loss[row] = l;
    }
  }
}

// dlogits = exp(lp) * k - onehot * k with lp = (x - max) - lse, k = grad_scale / rows.
__device__ __forceinline__ float nll_grad1(float x, float m, float lse, float k, bool hot) {
  return expf((x - m) - lse) * k - (hot ? k : 0.0f);
}
template <int VEC>
__global__ void __launch_bounds__(256)
nll_bwd_kernel(const float* __restrict__ x, const int64_t* __restrict__ targets,
               const float* __restrict__ row_max, const float* __restrict__ row_lse, float k,
               uint64_t rows, uint64_t cols, float* __restrict__ dx) {
  const uint64_t cv = cols / VEC;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float m = __ldg(row_max + row), lse = __ldg(row_lse + row);
    const int64_t t64 = __ldg(targets + row);
    // Out-of-range targets (reported by the forward) match no column.
    const uint64_t t = (t64 >= 0 && (uint64_t)t64 < cols) ? (uint64_t)t64 : UINT64_MAX;
    const float* xr = x + row * cols;
    float* dr = dx + row * cols;
    if constexpr (VEC == 4) {
      uint64_t c = threadIdx.x;
      for (; c + 256 < cv; c += 512) {
        float4 a = ld_stream4(xr + c * 4), b = ld_stream4(xr + (c + 256) * 4);
        const uint64_t ea = c * 4, eb = (c + 256) * 4;
        a.x = nll_grad1(a.x, m, lse, k, ea == t); a.y = nll_grad1(a.y, m, lse, k, ea + 1 == t);
        a.z = nll_grad1(a.z, m, lse, k, ea + 2 == t); a.w = nll_grad1(a.w, m, lse, k, ea + 3 == t);
        b.x = nll_grad1(b.x, m, lse, k, eb == t); b.y = nll_grad1(b.y, m, lse, k, eb + 1 == t);
        b.z = nll_grad1(b.z, m, lse, k, eb + 2 == t); b.w = nll_grad1(b.w, m, lse, k, eb + 3 == t);
        st_stream4(dr + ea, a);
        st_stream4(dr + eb, b);
      }
      for (; c < cv; c += 256) {
        float4 a = ld_stream4(xr + c * 4);
        const uint64_t ea = c * 4;
        a.x = nll_grad1(a.x, m, lse, k, ea == t); a.y = nll_grad1(a.y, m, lse, k, ea + 1 == t);
        a.z = nll_grad1(a.z, m, lse, k, ea + 2 == t); a.w = nll_grad1(a.w, m, lse, k, ea + 3 == t);
        st_stream4(dr + ea, a);
      }
    } else {
      for (uint64_t c = threadIdx.x; c < cols; c += 256) dr[c] = nll_grad1(xr[c], m, lse, k, c == t);
    }
  }
}

// Adds the per-CTA partial rows of the fused backward: out[c] = sum_p part[p][c].
// A CTA owns 8 columns (one 32-byte sector per row) and spreads the rows over
// 128 row lanes, each with up to 8 independent loads in flight, so the whole
// scratch (a few MB, still in L2) is pulled in about one memory latency; the
// lanes are then added in lane order.  The order depends on `parts` only.
__global__ void __launch_bounds__(1024)
part_rows_sum_kernel(const float* __restrict__ part, uint32_t parts, uint64_t cols,
                     float* __restrict__ out) {
  __shared__ float lane_sum[128][9];
  pdl_wait();  // launched as a dependent of the kernel that writes `part`
  pdl_trigger();
  const int cx = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const uint64_t c = (uint64_t)blockIdx.x * 8 + cx;
  float a = 0.0f;
  if (c < cols) {
    uint32_t p = rl;
    for (; p + 7 * 128 < parts; p += 8 * 128) {
      float v[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = part[(uint64_t)(p + q * 128) * cols + c];
#pragma unroll
      for (int q = 0; q < 8; ++q) a += v[q];
    }
    float v[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = (p + q * 128 < parts) ? part[(uint64_t)(p + q * 128) * cols + c] : 0.0f;
#pragma unroll
    for (int q = 0; q < 8; ++q) a += v[q];
  }
  lane_sum[rl][cx] = a;
  __syncthreads();
  // Warp w < 8 finishes column w: 4 lanes-of-rows per thread, then a shuffle tree.
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (w < 8) {
    float r = (lane_sum[l][w] + lane_sum[l + 32][w]) + (lane_sum[l + 64][w] + lane_sum[l + 96][w]);
    r = warp_sum(r);
    const uint64_t oc = (uint64_t)blockIdx.x * 8 + w;
    if (l == 0 && oc < cols) out[oc] = r;
  }
}

static int check_rc(const char* name, uint64_t rows, uint64_t cols) {
  uint64_t t;
  if (mul_overflows(rows, cols, &t) || t > (UINT64_MAX >> 3))
    return fail(FB_ERR_INVALID_SHAPE, "%s: rows * cols overflows", name);
  return FB_OK;
}

template <bool LOG>
static int softmax_fwd_impl(cudaStream_t stream, const char* name, const float* x, Prologue pro,
                            uint64_t rows, uint64_t cols, float* y) {
  if (int rc = check_rc(name, rows, cols)) return rc;
  if (rows == 0 || cols == 0) return FB_OK;
  if (!x || !y) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  const RowCfg c = row_cfg(cols);
  const bool vec_ok = cols % 4 == 0 && aligned16(x) && aligned16(y) && (!pro.bias || aligned16(pro.bias));
  if (vec_ok && !pro.on && cols > 16384 && cols <= (1u << 20) && sm_stream_cluster(cols)) {
    const int cl = sm_stream_cluster(cols);
    const uint64_t v4 = cols / 4, slice4 = (v4 + cl - 1) / cl;
    if (slice4 * (uint64_t)(cl - 1) < v4) {
      unsigned int* faults = fault_word();
      int fit = 0;
      auto k = softmax_fwd_stream_cluster_kernel<LOG>;
      FB_CUDA(resident_clusters(reinterpret_cast<const void*>(k), 512, 0, cl, &fit));
      const uint64_t ncl = rows < (uint64_t)fit ? rows : (uint64_t)fit;
      const cudaError_t le = launch_cluster(k, (unsigned)(ncl * cl), 512, 0, cl, true, stream, x, rows, (uint32_t)cols,
                                            (uint32_t)cl, (uint32_t)slice4, y, faults);
      if (le != cudaSuccess) return cuda_fail(le, name);
      count_launch();
      return FB_OK;
    }
  }
  if (vec_ok && cols > 16384 && cols < (1ull << 31)) {
    softmax_fwd_stream_kernel<LOG, 512><<<grid_full(rows), 512, 0, stream>>>(x, pro, rows, (uint32_t)cols, y);
    FB_LAUNCHED(name);
    return FB_OK;
  }
  const bool fast = c.group != 0 && vec_ok;
  if (!fast) {
    softmax_fwd_generic_kernel<LOG><<<grid_for(rows, 8), 256, 0, stream>>>(x, pro, rows, cols, y);
    FB_LAUNCHED(name);
    return FB_OK;
  }
  const uint32_t cc = (uint32_t)cols;
  if ((LOG || !pro.on) && cols < 256 && rows_enabled()) {
    // Several rows per warp (softmax_rows.cuh).  Lanes per row x float4 per lane, by the row's float4 count:
    // 4 x 2 (up to 8), 8 x 2 (16), 8 x 3 (24), 16 x 2 (32), 16 x 3 (48), 16 x 4 (63).
    const uint32_t c4 = cc / 4;
    cudaError_t le = cudaSuccess;
#define FB_SM_ROWS(L, I)                                                                                     \
  {                                                                                                          \
    const uint64_t per = 8 * 4 * (32 / L);                                                                   \
    le = launch_pdl(softmax_fwd_rows_kernel<L, I, 4, LOG>, dim3(grid_full((rows + per - 1) / per)), dim3(256), 0, \
                    stream, x, rows, cc, y);                                                                 \
  }
    if (c4 <= 8) FB_SM_ROWS(4, 2)
    else if (c4 <= 16) FB_SM_ROWS(8, 2)
    else if (c4 <= 24) FB_SM_ROWS(8, 3)
    else if (c4 <= 32) FB_SM_ROWS(16, 2)
    else if (c4 <= 48) FB_SM_ROWS(16, 3)
    else FB_SM_ROWS(16, 4)
#undef FB_SM_ROWS
    if (le != cudaSuccess) return cuda_fail(le, name);
    FB_LAUNCHED(name);
    return FB_OK;
  }
  const int threads = c.group < 256 ? 256 : c.group;
  const int r = threads / c.group;
  const unsigned grid = grid_full((rows + r - 1) / r);
  // Up to 48 KB of bias fits the default dynamic shared memory limit; wider rows read it from global.
  const size_t bias_bytes = (pro.on && pro.bias && cols * 4 <= 48 * 1024) ? (size_t)cols * 4 : 0;
  pro.smem = bias_bytes ? 1 : 0;
  cudaError_t le = cudaSuccess;
#define FB_SM_FWD(G, I)                                                                                          \
  if (c.group == G && c.items == I) {                                                                            \
    if (LOG || !pro.on)                                                                                          \
      le = launch_pdl(softmax_fwd_reg_kernel<G, I, LOG, false>, dim3(grid), dim3(sm_threads<G>()), 0, stream, x, \
                      pro, rows, cc, y);                                                                         \
    else                                                                                                         \
      le = launch_pdl(softmax_fwd_reg_kernel<G, I, false, true>, dim3(grid), dim3(sm_threads<G>()), bias_bytes,  \
                      stream, x, pro, rows, cc, y);                                                              \
  } else
  FB_SM_FWD(32, 1) FB_SM_FWD(32, 2) FB_SM_FWD(32, 4) FB_SM_FWD(32, 8) FB_SM_FWD(64, 8)
  FB_SM_FWD(128, 8) FB_SM_FWD(256, 8) FB_SM_FWD(512, 8) FB_SM_FWD(1024, 8) {
    return fail(FB_ERR_UNSUPPORTED, "%s: no kernel for group %d items %d", name, c.group, c.items);
  }
#undef FB_SM_FWD
  if (le != cudaSuccess) return cuda_fail(le, name);
  FB_LAUNCHED(name);
  return FB_OK;
}

// Launches the backward; *parts_out (FUSED only) is the number of partial
// dbias rows written, one per CTA.
template <bool LOG, bool FUSED>
static int softmax_bwd_impl(cudaStream_t stream, const char* name, const float* g, const float* y,
                            const float* x, Prologue pro, uint64_t rows, uint64_t cols, float* dx,
                            float* part, unsigned* parts_out) {
  const RowCfg c = bwd_cfg(cols);
  const bool fast = c.group != 0 && aligned16(g) && aligned16(y) && aligned16(dx) &&
                    (!FUSED || ((!x || aligned16(x)) && (!pro.bias || aligned16(pro.bias)) &&
                                (!part || aligned16(part))));
  if constexpr (!FUSED) {
    const int choice = sm_cluster_choice();
    const SmClusterPlan sp = choice == 0 ? SmClusterPlan{0, 0, 0, 0}
                                         : sm_cluster_plan(cols, choice < 0 ? 0 : choice,
                                                           cols <= 65536 ? sm_cluster_threads() : 1024);
    if (sp.cl && aligned16(g) && aligned16(y) && aligned16(dx)) {
      unsigned int* faults = fault_word();
      cudaError_t le = cudaErrorInvalidValue;
      int fit = 0;
#define FB_SM_CL_BWD(TT, I)                                                                                 \
  if (sp.threads == TT && sp.items == I) {                                                                  \
    auto k = softmax_bwd_cluster_kernel<TT, I, LOG>;                                                        \
    FB_CUDA(resident_clusters(reinterpret_cast<const void*>(k), TT, 0, sp.cl, &fit));                       \
    const uint64_t ncl = rows < (uint64_t)fit ? rows : (uint64_t)fit;                                       \
    le = launch_cluster(k, (unsigned)(ncl * sp.cl), TT, 0, sp.cl, true, stream, g, y, rows,                 \
                        (uint32_t)cols, (uint32_t)sp.cl, sp.slice4, dx, faults);                            \
  }
      FB_SM_CL_BWD(1024, 2) FB_SM_CL_BWD(1024, 4) FB_SM_CL_BWD(512, 2) FB_SM_CL_BWD(512, 4)
#undef FB_SM_CL_BWD
      if (le != cudaSuccess) return cuda_fail(le, name);
      count_launch();
      return FB_OK;
    }
    if (cols > 8192 && cols % 4 == 0 && cols < (1ull << 31) && aligned16(g) && aligned16(y) && aligned16(dx)) {
      // Capping the rows in flight so that every second sweep hits L2 (fewer CTAs per SM) was
      // measured slower at every width than letting part of it miss: occupancy matters more.
      softmax_bwd_stream_kernel<LOG, 512><<<grid_full(rows), 512, 0, stream>>>(g, y, rows, (uint32_t)cols, dx);
      FB_LAUNCHED(name);
      return FB_OK;
    }
  }
  if (!fast) {
    const unsigned grid = grid_for(rows, FUSED ? 4 : 8);
    softmax_bwd_generic_kernel<LOG, FUSED><<<grid, 256, 0, stream>>>(g, y, x, pro, rows, cols, dx, part);
    FB_LAUNCHED(name);
    if (parts_out) *parts_out = grid;
    return FB_OK;
  }
  if constexpr (!FUSED) {
    if (cols < 256 && rows_enabled()) {
      // Several rows per warp (softmax_rows.cuh), the forward's geometry.
      const uint32_t cc = (uint32_t)cols, c4 = cc / 4;
      cudaError_t le = cudaSuccess;
#define FB_SM_ROWS(L, I, R)                                                                                  \
  {                                                                                                          \
    const uint64_t per = 8 * R * (32 / L);                                                                   \
    le = launch_pdl(softmax_bwd_rows_kernel<L, I, R, LOG>, dim3(grid_full((rows + per - 1) / per)), dim3(256), 0, \
                    stream, g, y, rows, cc, dx);                                                             \
  }
      if (c4 <= 8) FB_SM_ROWS(4, 2, 4)
      else if (c4 <= 16) FB_SM_ROWS(8, 2, 4)
      else if (c4 <= 24) FB_SM_ROWS(8, 3, 2)
      else if (c4 <= 32) FB_SM_ROWS(16, 2, 4)
      else if (c4 <= 48) FB_SM_ROWS(16, 3, 2)
      else FB_SM_ROWS(16, 4, 2)
#undef FB_SM_ROWS
      if (le != cudaSuccess) return cuda_fail(le, name);
      FB_LAUNCHED(name);
      return FB_OK;
    }
  }
  // Warp-pipelined form (softmax_wp.cuh): always for the fused backward, for the plain one only
  // while the problem is small (it loses to the register kernel on large inputs).
  if (wp_enabled() && (FUSED || rows * cols <= (1ull << 24))) {
    const WpPlan wp = wp_plan(rows, cols, FUSED ? 3 : 2, FUSED ? cols : 0);
    unsigned int* faults = wp.items ? fault_word() : nullptr;
    if (wp.items && faults) {
      cudaError_t e = cudaSuccess;
#define FB_SM_WP_BWD(I)                                                                                 \
  if (wp.items == I) {                                                                                  \
    auto k = softmax_bwd_wp_kernel<I, LOG, FUSED>;                                                      \
    if ((e = allow_dyn_smem(reinterpret_cast<const void*>(k), wp.smem)) == cudaSuccess)                 \
      e = launch_pdl(k, dim3(wp.grid), dim3(kWpThreads), wp.smem, stream, g, y, x, pro.bias, pro.scale, \
                     pro.relu, (uint32_t)rows, (uint32_t)cols, wp.stages, dx, part, faults);            \
  }
      FB_SM_WP_BWD(2) FB_SM_WP_BWD(4) FB_SM_WP_BWD(8)
#undef FB_SM_WP_BWD
      if (e != cudaSuccess) return cuda_fail(e, name);
      FB_LAUNCHED(name);
      if (parts_out) *parts_out = wp.grid;
      return FB_OK;
    }
  }
  const int threads = c.group < 256 ? 256 : c.group;
  const int r = threads / c.group;
  const int per_sm = (c.items <= 2 ? 1536 : 1024) / threads;
  const unsigned grid = FUSED ? grid_for((rows + r - 1) / r, per_sm < 1 ? 1 : per_sm)
                              : grid_full((rows + r - 1) / r);
  const uint32_t cc = (uint32_t)cols;
  // 16 KB of static shared memory are taken by the dbias fold: 32 KB of bias still fit the default limit.
  const size_t bias_bytes = (FUSED && pro.relu && pro.bias && cols * 4 <= 32 * 1024) ? (size_t)cols * 4 : 0;
  pro.smem = bias_bytes ? 1 : 0;
  cudaError_t le = cudaSuccess;
#define FB_SM_BWD(G, I)                                                                                        \
  if (c.group == G && c.items == I) {                                                                          \
    le = launch_pdl(softmax_bwd_reg_kernel<G, I, LOG, FUSED>, dim3(grid), dim3(sm_threads<G>()), bias_bytes,   \
                    stream, g, y, x, pro, rows, cc, dx, part);                                                 \
  } else
  FB_SM_BWD(32, 1) FB_SM_BWD(32, 2) FB_SM_BWD(64, 2) FB_SM_BWD(128, 2) FB_SM_BWD(256, 2)
  FB_SM_BWD(512, 2) FB_SM_BWD(1024, 2) FB_SM_BWD(1024, 4) FB_SM_BWD(1024, 8) {
    return fail(FB_ERR_UNSUPPORTED, "%s: no kernel for group %d items %d", name, c.group, c.items);
  }
#undef FB_SM_BWD
  if (le != cudaSuccess) return cuda_fail(le, name);
  FB_LAUNCHED(name);
  if (parts_out) *parts_out = grid;
  return FB_OK;
}

// Upper bound of the partial rows either path of the fused backward writes.
static unsigned fused_bwd_max_parts(uint64_t rows) {
  return grid_for(rows, 6);  // both paths launch at most 6 CTAs per SM, never more than `rows`
}

}  // namespace fb

using namespace fb;

extern "C" {

int fb_softmax_fwd(fb_stream_t stream, const float* x, uint64_t rows, uint64_t cols, float* y) {
  return softmax_fwd_impl<false>(stream, "fb_softmax_fwd", x, Prologue{nullptr, 1.0f, 0, 0}, rows, cols, y);
}
int fb_log_softmax_fwd(fb_stream_t stream, const float* x, uint64_t rows, uint64_t cols, float* y) {
  return softmax_fwd_impl<true>(stream, "fb_log_softmax_fwd", x, Prologue{nullptr, 1.0f, 0, 0}, rows, cols, y);
}
int fb_bias_act_scale_softmax_fwd(fb_stream_t stream, const float* x, const float* bias, int relu,
                                  float scale, uint64_t rows, uint64_t cols, float* y) {
  return softmax_fwd_impl<false>(stream, "fb_bias_act_scale_softmax_fwd", x,
                                 Prologue{bias, scale, relu ? 1 : 0, 1}, rows, cols, y);
}

int fb_softmax_bwd(fb_stream_t stream, const float* g, const float* y, uint64_t rows, uint64_t cols,
                   float* dx) {
  if (int rc = check_rc("fb_softmax_bwd", rows, cols)) return rc;
  if (rows == 0 || cols == 0) return FB_OK;
  if (!g || !y || !dx) return fail(FB_ERR_INVALID_ARG, "fb_softmax_bwd: null buffer");
  return softmax_bwd_impl<false, false>(stream, "fb_softmax_bwd", g, y, nullptr, Prologue{nullptr, 1.0f, 0, 0},
                                        rows, cols, dx, nullptr, nullptr);
}
int fb_log_softmax_bwd(fb_stream_t stream, const float* g, const float* y, uint64_t rows,
                       uint64_t cols, float* dx) {
  if (int rc = check_rc("fb_log_softmax_bwd", rows, cols)) return rc;
  if (rows == 0 || cols == 0) return FB_OK;
  if (!g || !y || !dx) return fail(FB_ERR_INVALID_ARG, "fb_log_softmax_bwd: null buffer");
  return softmax_bwd_impl<true, false>(stream, "fb_log_softmax_bwd", g, y, nullptr, Prologue{nullptr, 1.0f, 0, 0},
                                       rows, cols, dx, nullptr, nullptr);
}

uint64_t fb_softmax_fused_bwd_workspace_bytes(uint64_t rows, uint64_t cols) {
  if (rows == 0 || cols == 0) return 0;
  return (uint64_t)fused_bwd_max_parts(rows) * cols * sizeof(float);
}

int fb_bias_act_scale_softmax_bwd(fb_stream_t stream, const float* g, const float* y, const float* x,
                                  const float* bias, int relu, float scale, uint64_t rows,
                                  uint64_t cols, float* dx, float* dbias, void* workspace,
                                  uint64_t workspace_bytes) {
  const char* name = "fb_bias_act_scale_softmax_bwd";
  if (int rc = check_rc(name, rows, cols)) return rc;
  if (cols == 0) return FB_OK;
  if (rows == 0) return dbias ? fb_fill(stream, dbias, 0.0f, cols) : FB_OK;
  if (!g || !y || !dx || (relu && !x)) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  const Prologue pro{bias, scale, relu ? 1 : 0, 1};
  float* part = nullptr;
  if (dbias) {
    const uint64_t need = fb_softmax_fused_bwd_workspace_bytes(rows, cols);
    if (!workspace || workspace_bytes < need || !aligned16(workspace))
      return fail(FB_ERR_WORKSPACE, "%s: needs %llu bytes of 16-byte aligned scratch", name, (unsigned long long)need);
    part = static_cast<float*>(workspace);
  }
  unsigned parts = 0;
  if (int rc = softmax_bwd_impl<false, true>(stream, name, g, y, x, pro, rows, cols, dx, part, &parts)) return rc;
  if (dbias) {
    // A dependent launch: its CTAs are made resident while the backward drains and start the
    // moment its partial rows are complete.
    const cudaError_t e = launch_pdl(part_rows_sum_kernel, dim3((unsigned)((cols + 7) / 8)), dim3(1024), 0, stream,
                                     (const float*)part, (uint32_t)parts, cols, dbias);
    if (e != cudaSuccess) return cuda_fail(e, name);
    FB_LAUNCHED(name);
  }
  return FB_OK;
}

uint64_t fb_nll_workspace_bytes(uint64_t rows) {
  if (rows == 0) return 0;
  // [rows] per-row losses (rounded up to 16 bytes) + the scalar-reduce scratch.
  return ((rows * sizeof(float) + 15) / 16) * 16 + fb_reduce_workspace_bytes(rows);
}

int fb_log_softmax_nll_fwd(fb_stream_t stream, const float* logits, const int64_t* targets,
                           uint64_t rows, uint64_t cols, float* loss, float* row_max, float* row_lse,
                           int64_t* argmax, int64_t* bad_target, void* workspace,
                           uint64_t workspace_bytes) {
  const char* name = "fb_log_softmax_nll_fwd";
  if (int rc = check_rc(name, rows, cols)) return rc;
  if (!loss) return fail(FB_ERR_INVALID_ARG, "%s: null loss", name);
  if (rows == 0) return fb_reduce(stream, FB_RED_MEAN, nullptr, 0, loss, nullptr, 0);  // empty mean = NaN
  if (cols == 0) return fail(FB_ERR_INVALID_SHAPE, "%s: no classes", name);
  if (!logits || !targets || !row_max || !row_lse) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  const uint64_t need = fb_nll_workspace_bytes(rows);
  if (!workspace || workspace_bytes < need || !aligned16(workspace))
    return fail(FB_ERR_WORKSPACE, "%s: needs %llu bytes of 16-byte aligned scratch", name, (unsigned long long)need);
  float* row_loss = static_cast<float*>(workspace);
  const uint64_t off = ((rows * sizeof(float) + 15) / 16) * 16;
  void* red_ws = static_cast<char*>(workspace) + off;
  const RowCfg c = row_cfg(cols);
  const bool fast = c.group != 0 && aligned16(logits);
  if (cols >= 2048 && cols < (1ull << 31)) {
    const bool v4 = cols % 4 == 0 && aligned16(logits);
    const uint32_t cc = (uint32_t)cols;
    if (cols >= 8192) {
      const unsigned grid = grid_full(rows);
      if (v4) nll_fwd_stream_kernel<4, 512><<<grid, 512, 0, stream>>>(logits, targets, rows, cc, row_loss, row_max, row_lse, argmax, bad_target);
      else nll_fwd_stream_kernel<1, 512><<<grid, 512, 0, stream>>>(logits, targets, rows, cc, row_loss, row_max, row_lse, argmax, bad_target);
    } else {
      const unsigned grid = grid_full(rows);
      if (v4) nll_fwd_stream_kernel<4, 256><<<grid, 256, 0, stream>>>(logits, targets, rows, cc, row_loss, row_max, row_lse, argmax, bad_target);
      else nll_fwd_stream_kernel<1, 256><<<grid, 256, 0, stream>>>(logits, targets, rows, cc, row_loss, row_max, row_lse, argmax, bad_target);
    }
  } else if (!fast) {
    nll_fwd_generic_kernel<<<grid_for(rows, 8), 256, 0, stream>>>(logits, targets, rows, cols, row_loss, row_max,
                                                                row_lse, argmax, bad_target);
  } else {
    const int threads = c.group < 256 ? 256 : c.group;
    const int r = threads / c.group;
  const unsigned grid = grid_full((rows + r - 1) / r);
    const uint32_t cc = (uint32_t)cols;
#define FB_NLL(G, I)                                                                          \
  if (c.group == G && c.items == I) {                                                         \
    nll_fwd_reg_kernel<G, I><<<grid, sm_threads<G>(), 0, stream>>>(logits, targets, rows, cc, row_loss, \
                                                                  row_max, row_lse, argmax, bad_target); \
  } else
    FB_NLL(32, 1) FB_NLL(32, 2) FB_NLL(32, 4) FB_NLL(32, 8) FB_NLL(64, 8) FB_NLL(128, 8)
    FB_NLL(256, 8) FB_NLL(512, 8) FB_NLL(1024, 8) {
      return fail(FB_ERR_UNSUPPORTED, "%s: no kernel for group %d items %d", name, c.group, c.items);
    }
#undef FB_NLL
  }
  FB_LAUNCHED(name);
  return fb_reduce(stream, FB_RED_MEAN, row_loss, rows, loss, red_ws, workspace_bytes - off);
}

int fb_log_softmax_nll_bwd(fb_stream_t stream, const float* logits, const int64_t* targets,
                           const float* row_max, const float* row_lse, float grad_scale,
                           uint64_t rows, uint64_t cols, float* dlogits) {
  const char* name = "fb_log_softmax_nll_bwd";
  if (int rc = check_rc(name, rows, cols)) return rc;
  if (rows == 0 || cols == 0) return FB_OK;
  if (!logits || !targets || !row_max || !row_lse || !dlogits) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  const float k = grad_scale * (1.0f / (float)rows);
  if (cols % 4 == 0 && aligned16(logits) && aligned16(dlogits))
    nll_bwd_kernel<4><<<grid_full(rows), 256, 0, stream>>>(logits, targets, row_max, row_lse, k, rows, cols, dlogits);
  else
    nll_bwd_kernel<1><<<grid_full(rows), 256, 0, stream>>>(logits, targets, row_max, row_lse, k, rows, cols, dlogits);
  FB_LAUNCHED(name);
  return FB_OK;
}

}  // extern "C"
