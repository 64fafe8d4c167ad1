// Full-tensor sum / mean and the axis reductions sum_dim / mean_dim / max_dim
// over x[outer][red][inner].
//
// Roofline: HBM.  Algorithmic bytes: 4 * outer*red*inner read + the output
// (f32, plus i64 indices for max_dim).
//  - inner >= 32: column kernel (reduce.cuh): lanes run along `inner`, so the
//    loads are coalesced, rows are split over warps / CTAs.
//  - inner < 32 (including the last-dim case inner == 1): one warp or one CTA
//    per output; lanes run along `red` (contiguous when inner == 1).
// The reference kernel gives every output to a single thread that walks `red`
// serially (crates/ferro-cuda/src/kernels.rs:319-332).
#include "common.cuh"
#include "reduce.cuh"

namespace fb {

// ------------------------------------------------------------ full reduce
constexpr int kRedThreads = 256;

__global__ void __launch_bounds__(kRedThreads)
reduce_partial_kernel(const float* __restrict__ x, uint64_t n, int vec, float* __restrict__ part) {
  pdl_trigger();  // the dependent finalize launch may become resident while this grid runs
  __shared__ float red[32];
  float a0 = 0, a1 = 0, a2 = 0, a3 = 0;
  const uint64_t stride = (uint64_t)gridDim.x * kRedThreads;
  const uint64_t tid = (uint64_t)blockIdx.x * kRedThreads + threadIdx.x;
  if (vec) {
    const uint64_t nv = n / 4;
    uint64_t i = tid;
    for (; i + 3 * stride < nv; i += 4 * stride) {  // four 16-byte loads in flight per thread
      const float4 u = ld_stream4(x + i * 4), v = ld_stream4(x + (i + stride) * 4);
      const float4 p = ld_stream4(x + (i + 2 * stride) * 4), q = ld_stream4(x + (i + 3 * stride) * 4);
      a0 += u.x; a1 += u.y; a2 += u.z; a3 += u.w;
      a0 += v.x; a1 += v.y; a2 += v.z; a3 += v.w;
      a0 += p.x; a1 += p.y; a2 += p.z; a3 += p.w;
      a0 += q.x; a1 += q.y; a2 += q.z; a3 += q.w;
    }
    for (; i < nv; i += stride) {
      const float4 u = ld_stream4(x + i * 4);
      a0 += u.x; a1 += u.y; a2 += u.z; a3 += u.w;
    }
    if (tid < n - nv * 4) a0 += x[nv * 4 + tid];
  } else {
    for (uint64_t i = tid; i < n; i += stride) a0 += x[i];
  }
  const float s = block_sum((a0 + a1) + (a2 + a3), red);
  if (threadIdx.x == 0) part[blockIdx.x] = s;
}

// One CTA adds the partials (at most a few thousand) and applies the kind.
__global__ void __launch_bounds__(kRedThreads)
reduce_final_kernel(const float* __restrict__ part, uint32_t parts, float divisor,
                    float* __restrict__ out) {
  pdl_wait();  // launched as a dependent (launch_pdl) of the kernel that writes its input
  pdl_trigger();
  __shared__ float red[32];
  float a = 0.0f;
  for (uint32_t i = threadIdx.x; i < parts; i += kRedThreads) a += part[i];
  const float s = block_sum(a, red);
  if (threadIdx.x == 0) out[0] = divisor == 1.0f ? s : s / divisor;  // mean = sum / n, ops.rs:173-175
}

__global__ void store_scalar_kernel(float* out, float v) { out[0] = v; }

static uint32_t reduce_parts(uint64_t n) {
  const uint64_t per_cta = (uint64_t)kRedThreads * 4 * 8;
  return grid_for((n + per_cta - 1) / per_cta, 8);
}

// --------------------------------------------- row-wise sum (inner < 32)
// GROUP = 32: one warp per output; GROUP = 0: one CTA per output.
template <int GROUP>
__global__ void __launch_bounds__(256)
row_sum_kernel(const float* __restrict__ x, uint64_t outer, uint64_t red, uint64_t inner, int vec,
               float* __restrict__ out, float scale) {
  __shared__ float sred[32];
  const uint64_t nout = outer * inner;
  const int lanes = GROUP ? 32 : blockDim.x;
  const int lane = GROUP ? (threadIdx.x & 31) : threadIdx.x;
  const uint64_t first = GROUP ? (uint64_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5) : blockIdx.x;
  const uint64_t step = GROUP ? (uint64_t)gridDim.x * (blockDim.x / 32) : gridDim.x;
  for (uint64_t j = first; j < nout; j += step) {
    const uint64_t o = j / inner, i = j % inner;
    const float* base = x + o * red * inner + i;
    float a0 = 0, a1 = 0, a2 = 0, a3 = 0;
    if (vec) {  // inner == 1, red % 4 == 0, 16-byte aligned rows
      const uint64_t nv = red / 4;
      uint64_t k = lane;
      for (; k + lanes < nv; k += 2 * lanes) {
        const float4 u = ld_stream4(base + k * 4), v = ld_stream4(base + (k + lanes) * 4);
        a0 += u.x; a1 += u.y; a2 += u.z; a3 += u.w;
        a0 += v.x; a1 += v.y; a2 += v.z; a3 += v.w;
      }
      for (; k < nv; k += lanes) {
        const float4 u = ld_stream4(base + k * 4);
        a0 += u.x; a1 += u.y; a2 += u.z; a3 += u.w;
      }
    } else {
      uint64_t k = lane;
      for (; k + lanes < red; k += 2 * lanes) {
        a0 += base[k * inner];
        a1 += base[(k + lanes) * inner];
      }
      for (; k < red; k += lanes) a0 += base[k * inner];
    }
    float s = (a0 + a1) + (a2 + a3);
    if (GROUP) {
      s = warp_sum(s);
      if (lane == 0) out[j] = s * scale;
    } else {
      s = block_sum(s, sred);
      if (threadIdx.x == 0) out[j] = s * scale;
    }
  }
}

// ------------------------------------------------------------- max / argmax
template <int GROUP, class I>
__global__ void __launch_bounds__(256)
row_max_kernel(const float* __restrict__ x, uint64_t outer, uint64_t red, uint64_t inner, int vec,
               float* __restrict__ val, int64_t* __restrict__ idx) {
  __shared__ float sv[32];
  __shared__ unsigned long long si[32];
  const uint64_t nout = outer * inner;
  const int lanes = GROUP ? 32 : blockDim.x;
  const int lane = GROUP ? (threadIdx.x & 31) : threadIdx.x;
  const uint64_t first = GROUP ? (uint64_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5) : blockIdx.x;
  const uint64_t step = GROUP ? (uint64_t)gridDim.x * (blockDim.x / 32) : gridDim.x;
  for (uint64_t j = first; j < nout; j += step) {
    const uint64_t o = j / inner, i = j % inner;
    const float* base = x + o * red * inner + i;
    Scan<I> sc = scan_init<I>((I)(vec ? lane * 4 : lane));
    if (vec) {  // inner == 1, red % 4 == 0, 16-byte aligned rows
      const I nv = (I)(red / 4);
      I k = (I)lane;
      for (; k + lanes < nv; k += 2 * lanes) {
        const float4 u = ld_stream4(base + (uint64_t)k * 4), w = ld_stream4(base + (uint64_t)(k + lanes) * 4);
        const I k1 = k * 4, k2 = (k + lanes) * 4;
        scan_step<I>(sc, u.x, k1); scan_step<I>(sc, u.y, k1 + 1); scan_step<I>(sc, u.z, k1 + 2); scan_step<I>(sc, u.w, k1 + 3);
        scan_step<I>(sc, w.x, k2); scan_step<I>(sc, w.y, k2 + 1); scan_step<I>(sc, w.z, k2 + 2); scan_step<I>(sc, w.w, k2 + 3);
      }
      for (; k < nv; k += lanes) {
        const float4 u = ld_stream4(base + (uint64_t)k * 4);
        const I k1 = k * 4;
        scan_step<I>(sc, u.x, k1); scan_step<I>(sc, u.y, k1 + 1); scan_step<I>(sc, u.z, k1 + 2); scan_step<I>(sc, u.w, k1 + 3);
      }
    } else {
      const I n = (I)red;
      I k = (I)lane;
      for (; k + lanes < n; k += 2 * lanes) {
        const float u = ld_stream(base + (uint64_t)k * inner), w = ld_stream(base + (uint64_t)(k + lanes) * inner);
        scan_step<I>(sc, u, k);
        scan_step<I>(sc, w, k + lanes);
      }
      for (; k < n; k += lanes) scan_step<I>(sc, ld_stream(base + (uint64_t)k * inner), k);
    }
    auto first_nan = [&]() -> uint64_t {
      if (vec) {
        for (uint64_t k = lane; k < red / 4; k += lanes) {
          const float4 u = ld_stream4(base + k * 4);
          if (u.x != u.x) return k * 4;
          if (u.y != u.y) return k * 4 + 1;
          if (u.z != u.z) return k * 4 + 2;
          if (u.w != u.w) return k * 4 + 3;
        }
      } else {
        for (uint64_t k = lane; k < red; k += lanes) {
          const float u = ld_stream(base + k * inner);
          if (u != u) return k;
        }
      }
      return UINT64_MAX;
    };
    Best b = warp_best(scan_finish(sc, first_nan));
    if (!GROUP) {
      const int warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
      __syncthreads();
      if ((threadIdx.x & 31) == 0) { sv[warp] = b.v; si[warp] = b.i; }
      __syncthreads();
      b = (threadIdx.x & 31) < nw ? Best{sv[threadIdx.x & 31], si[threadIdx.x & 31]} : best_identity();
      b = warp_best(b);
    }
    if (lane == 0) {
      if (val) val[j] = b.v;
      if (idx) idx[j] = (int64_t)b.i;
    }
  }
}

struct BestPart {  // 16 bytes
  float v;
  uint32_t pad;
  uint64_t i;
};

// Column max: same tiling as col_sum_kernel; a lane owns VEC adjacent columns
// (float4 loads when VEC = 4) and keeps one running scan per column.
template <int VEC, class I>
__global__ void __launch_bounds__(kColThreads)
col_max_kernel(const float* __restrict__ x, uint64_t outer, uint64_t red, uint64_t inner,
               uint32_t strips, uint32_t splits, uint64_t rows_per_split, float* __restrict__ val,
               int64_t* __restrict__ idx, BestPart* __restrict__ part) {
  pdl_trigger();  // the dependent finalize launch may become resident while this grid runs
  __shared__ float sv[kColWarps][32 * VEC + 1];
  __shared__ unsigned long long si[kColWarps][32 * VEC + 1];
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
    Scan<I> sc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) sc[j] = scan_init<I>((I)(r0 + warp));
    if (c < inner) {
      const float* base = x + o * red * inner + c;
      auto row = [&](uint64_t r, float (&v)[VEC]) {
        if constexpr (VEC == 4) {
          const float4 q = ld_stream4(base + r * inner);
          v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
          v[0] = ld_stream(base + r * inner);
        }
      };
      uint64_t r = r0 + warp;
      // Four rows in flight per warp: the scans cost registers, so fewer CTAs
      // fit than in the sum kernel and each thread has to cover more latency.
      for (; r + 3 * kColWarps < r1; r += 4 * kColWarps) {
        float u[4][VEC];
#pragma unroll
        for (int q = 0; q < 4; ++q) row(r + q * kColWarps, u[q]);
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int j = 0; j < VEC; ++j) scan_step<I>(sc[j], u[q][j], (I)(r + q * kColWarps));
      }
      for (; r < r1; r += kColWarps) {
        float u[VEC];
        row(r, u);
#pragma unroll
        for (int j = 0; j < VEC; ++j) scan_step<I>(sc[j], u[j], (I)r);
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      auto first_nan = [&]() -> uint64_t {
        const float* col = x + o * red * inner + c + j;
        for (uint64_t r = r0 + warp; r < r1; r += kColWarps)
          if (col[r * inner] != col[r * inner]) return r;
        return UINT64_MAX;
      };
      const Best b = scan_finish(sc[j], first_nan);
      sv[warp][lane * VEC + j] = b.v;
      si[warp][lane * VEC + j] = b.i;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * VEC; i += kColThreads) {
      const uint64_t col = (uint64_t)strip * 32 * VEC + i;
      if (col >= inner) continue;
      Best r = Best{sv[0][i], si[0][i]};
#pragma unroll
      for (int w = 1; w < kColWarps; ++w) r = best_of(r, Best{sv[w][i], si[w][i]});
      if (splits == 1) {
        if (val) val[o * inner + col] = r.v;
        if (idx) idx[o * inner + col] = (int64_t)r.i;
      } else {
        part[((uint64_t)split * outer + o) * inner + col] = BestPart{r.v, 0u, r.i};
      }
    }
  }
}

__global__ void __launch_bounds__(256)
col_max_finalize_kernel(const BestPart* __restrict__ part, uint32_t splits, uint64_t count,
                        float* __restrict__ val, int64_t* __restrict__ idx) {
  pdl_wait();  // launched as a dependent (launch_pdl) of the kernel that writes its input
  pdl_trigger();
  for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < count;
       j += (uint64_t)gridDim.x * blockDim.x) {
    Best b = best_identity();
    for (uint32_t k = 0; k < splits; ++k) {
      const BestPart p = part[(uint64_t)k * count + j];
      b = best_of(b, Best{p.v, p.i});
    }
    if (val) val[j] = b.v;
    if (idx) idx[j] = (int64_t)b.i;
  }
}

static int check_dims(const char* name, uint64_t outer, uint64_t red, uint64_t inner, uint64_t* nout) {
  uint64_t t;
  if (mul_overflows(outer, inner, nout) || mul_overflows(*nout, red, &t) || t > (UINT64_MAX >> 3))
    return fail(FB_ERR_INVALID_SHAPE, "%s: outer * red * inner overflows", name);
  return FB_OK;
}

static int sum_dim_impl(cudaStream_t stream, const char* name, const float* x, uint64_t outer,
                        uint64_t red, uint64_t inner, float* out, float scale, void* workspace,
                        uint64_t workspace_bytes) {
  uint64_t nout;
  if (int rc = check_dims(name, outer, red, inner, &nout)) return rc;
  if (nout == 0) return FB_OK;
  if (!out) return fail(FB_ERR_INVALID_ARG, "%s: null output", name);
  if (red == 0) {
    // Empty reduced dim: sum is 0; mean is 0 * (1/0) = NaN (ops_ext/mean_dim.rs:17-18).
    return fb_fill(stream, out, 0.0f * scale, nout);
  }
  if (!x) return fail(FB_ERR_INVALID_ARG, "%s: null input", name);
  if (inner >= 32) {
    PlainColSrc src{x, red, inner};
    return run_col_sum<1>(stream, src, outer, red, inner, aligned16(x), out, nullptr, scale, workspace,
                          workspace_bytes, name);
  }
  const int vec = inner == 1 && red % 4 == 0 && aligned16(x);
  if (red <= 8192) {
    const uint64_t ctas = (nout + 7) / 8;
    row_sum_kernel<32><<<grid_full(ctas), 256, 0, stream>>>(x, outer, red, inner, vec, out, scale);
  } else {
    row_sum_kernel<0><<<grid_full(nout), 256, 0, stream>>>(x, outer, red, inner, vec, out, scale);
  }
  FB_LAUNCHED(name);
  return FB_OK;
}

}  // namespace fb

using namespace fb;

extern "C" {

extern "C" uint64_t fb_mse_parts(uint64_t n);  // mlp.cu: fb_mse_fwd_bwd sizes its scratch with this query too
uint64_t fb_reduce_workspace_bytes(uint64_t n) {
  if (n == 0) return 0;
  const uint64_t a = reduce_parts(n), b = fb_mse_parts(n);
  return (a > b ? a : b) * sizeof(float);
}

int fb_reduce(fb_stream_t stream, int kind, const float* x, uint64_t n, float* out, void* workspace,
              uint64_t workspace_bytes) {
  if (kind != FB_RED_SUM && kind != FB_RED_MEAN) return fail(FB_ERR_INVALID_ARG, "fb_reduce: unknown kind %d", kind);
  if (!out) return fail(FB_ERR_INVALID_ARG, "fb_reduce: null output");
  if (n == 0) {
    store_scalar_kernel<<<1, 1, 0, stream>>>(out, kind == FB_RED_MEAN ? NAN : 0.0f);
    FB_LAUNCHED("fb_reduce");
    return FB_OK;
  }
  if (!x) return fail(FB_ERR_INVALID_ARG, "fb_reduce: null input");
  const uint32_t parts = reduce_parts(n);
  if (!workspace || workspace_bytes < (uint64_t)parts * sizeof(float))
    return fail(FB_ERR_WORKSPACE, "fb_reduce: needs %llu bytes of scratch",
                (unsigned long long)((uint64_t)parts * sizeof(float)));
  float* part = static_cast<float*>(workspace);
  reduce_partial_kernel<<<parts, kRedThreads, 0, stream>>>(x, n, aligned16(x) ? 1 : 0, part);
  FB_LAUNCHED("fb_reduce");
  FB_CUDA(launch_pdl(reduce_final_kernel, dim3(1), dim3(kRedThreads), 0, stream, (const float*)part, parts,
                     kind == FB_RED_MEAN ? (float)n : 1.0f, out));
  FB_LAUNCHED("fb_reduce");
  return FB_OK;
}

uint64_t fb_reduce_dim_workspace_bytes(uint64_t outer, uint64_t red, uint64_t inner) {
  uint64_t nout, t;
  if (mul_overflows(outer, inner, &nout) || mul_overflows(nout, red, &t) || nout == 0 || red == 0) return 0;
  if (inner < 32) return 0;
  // Worst case over alignment, sized for the 16-byte max/argmax partial record.
  const ColPlan a = col_plan(outer, red, inner, true), b = col_plan(outer, red, inner, false);
  const uint32_t splits = a.splits > b.splits ? a.splits : b.splits;
  return splits > 1 ? (uint64_t)splits * nout * sizeof(BestPart) : 0;
}

int fb_sum_dim(fb_stream_t stream, const float* x, uint64_t outer, uint64_t red, uint64_t inner,
               float* out, void* workspace, uint64_t workspace_bytes) {
  return sum_dim_impl(stream, "fb_sum_dim", x, outer, red, inner, out, 1.0f, workspace, workspace_bytes);
}

int fb_mean_dim(fb_stream_t stream, const float* x, uint64_t outer, uint64_t red, uint64_t inner,
                float* out, void* workspace, uint64_t workspace_bytes) {
  return sum_dim_impl(stream, "fb_mean_dim", x, outer, red, inner, out, 1.0f / (float)red, workspace,
                      workspace_bytes);
}

int fb_max_dim(fb_stream_t stream, const float* x, uint64_t outer, uint64_t red, uint64_t inner,
               float* values, int64_t* indices, void* workspace, uint64_t workspace_bytes) {
  uint64_t nout;
  if (int rc = check_dims("fb_max_dim", outer, red, inner, &nout)) return rc;
  if (red == 0 && nout != 0)
    return fail(FB_ERR_INVALID_SHAPE, "fb_max_dim: cannot reduce an empty dimension");  // argmax.rs:36-41
  if (nout == 0) return FB_OK;
  if (!x || (!values && !indices)) return fail(FB_ERR_INVALID_ARG, "fb_max_dim: null buffer");
  const bool narrow = red < (1ull << 31);  // 32-bit indices in the hot loops
  if (inner >= 32) {
    const ColPlan p = col_plan(outer, red, inner, aligned16(x));
    const uint64_t need = p.splits > 1 ? (uint64_t)p.splits * nout * sizeof(BestPart) : 0;
    if (need && (!workspace || workspace_bytes < need || !aligned16(workspace)))
      return fail(FB_ERR_WORKSPACE, "fb_max_dim: needs %llu bytes of 16-byte aligned scratch", (unsigned long long)need);
    BestPart* part = static_cast<BestPart*>(workspace);
    const uint64_t tiles = outer * p.strips * (uint64_t)p.splits;
    const unsigned grid = grid_for(tiles, 8);
#define FB_COL_MAX(VEC, I) \
  col_max_kernel<VEC, I><<<grid, kColThreads, 0, stream>>>(x, outer, red, inner, p.strips, p.splits, p.rows_per_split, values, indices, part)
    if (narrow) {
      if (p.vec == 4) FB_COL_MAX(4, uint32_t); else FB_COL_MAX(1, uint32_t);
    } else {
      if (p.vec == 4) FB_COL_MAX(4, uint64_t); else FB_COL_MAX(1, uint64_t);
    }
#undef FB_COL_MAX
    FB_LAUNCHED("fb_max_dim");
    if (p.splits > 1) {
      FB_CUDA(launch_pdl(col_max_finalize_kernel, dim3(grid_for((nout + 255) / 256, 8)), dim3(256), 0, stream,
                         (const BestPart*)part, p.splits, nout, values, indices));
      FB_LAUNCHED("fb_max_dim");
    }
    return FB_OK;
  }
  const int mvec = inner == 1 && red % 4 == 0 && aligned16(x);
#define FB_ROW_MAX(GROUP, I, GRID) \
  row_max_kernel<GROUP, I><<<GRID, 256, 0, stream>>>(x, outer, red, inner, mvec, values, indices)
  if (red <= 8192) {
    FB_ROW_MAX(32, uint32_t, grid_full((nout + 7) / 8));
  } else if (narrow) {
    FB_ROW_MAX(0, uint32_t, grid_full(nout));
  } else {
    FB_ROW_MAX(0, uint64_t, grid_full(nout));
  }
#undef FB_ROW_MAX
  FB_LAUNCHED("fb_max_dim");
  return FB_OK;
}

}  // extern "C"
