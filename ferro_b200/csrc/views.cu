// Reductions and softmax over one dim of a tensor VIEW: (storage, shape,
// element strides, element offset), any dim, output row-major contiguous.
//
// ferro keeps such inputs off the GPU today: try_raw_sum_dim downloads every
// device tensor that is not whole and contiguous and reduces it on the host
// (crates/ferro-core/src/tensor.rs:2057-2104), and raw_row_softmax declines
// when the reduced dim is not the last one or the tensor is a view
// (tensor.rs:2124-2127), which sends softmax / log_softmax to the host loops
// of ops_ext.  Behind the same seam these entries keep them resident.
//
// Whole contiguous inputs are handed to the tuned kernels of reduce.cu and
// softmax.cu.  Everything else runs on two generic forms, chosen by where the
// unit stride is:
//   lanes along the kept dims   a warp covers 32 consecutive outputs (the
//                               innermost kept dim varies fastest, so a
//                               unit-stride kept dim gives coalesced loads),
//                               8 warps share the reduced dim round-robin and
//                               are combined in warp order;
//   lanes along the reduced dim a warp per output, for a reduced dim that is
//                               itself the contiguous one.
// Summation order is a function of the shape only (no atomics).  Roofline: HBM;
// algorithmic bytes are 4 per input element + the output for the reductions,
// 8 per element for softmax forward (two sweeps of the input, the second from
// L2 while the working set of the resident CTAs fits), 12 for the backward.
#include "chain.cuh"
#include "reduce.cuh"

namespace fb {

// Flat index over the kept dims (logical order, innermost last) -> input offset.
struct KeptIndex {
  int n;
  uint32_t ext[FB_MAX_RANK];
  FastDiv div[FB_MAX_RANK];
  int64_t stride[FB_MAX_RANK];
};
__device__ __forceinline__ int64_t kept_offset(const KeptIndex& k, uint32_t o) {
  int64_t off = 0;
  for (int d = k.n - 1; d >= 0; --d) {
    const uint32_t q = fdiv(o, k.div[d]), c = o - q * k.ext[d];
    o = q;
    off += (int64_t)c * k.stride[d];
  }
  return off;
}

constexpr int kVwThreads = 256;

// ---------------------------------------------------------------- reductions
// OP 0: sum * scale.  OP 1: maximum and its index (first NaN wins, ties keep the lowest index).
// LANES_RED: lanes along the reduced dim (one warp per output), else along the outputs.
template <int OP, bool LANES_RED>
__global__ void __launch_bounds__(kVwThreads)
view_reduce_kernel(const float* __restrict__ x, const __grid_constant__ KeptIndex kd, int64_t s_red, uint32_t red,
                   uint32_t nout, float scale, float* __restrict__ out, int64_t* __restrict__ idx) {
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  if constexpr (LANES_RED) {
    for (uint32_t o = blockIdx.x * 8 + ty; o < nout; o += gridDim.x * 8) {
      const float* p = x + kept_offset(kd, o);
      if constexpr (OP == 0) {
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        uint32_t r = tx;
        for (; r + 96 < red; r += 128) {
          const float v0 = __ldg(p + (int64_t)r * s_red), v1 = __ldg(p + (int64_t)(r + 32) * s_red);
          const float v2 = __ldg(p + (int64_t)(r + 64) * s_red), v3 = __ldg(p + (int64_t)(r + 96) * s_red);
          a0 += v0; a1 += v1; a2 += v2; a3 += v3;
        }
        for (; r < red; r += 32) a0 += __ldg(p + (int64_t)r * s_red);
        const float t = warp_sum((a0 + a1) + (a2 + a3));
        if (tx == 0) out[o] = scale == 1.0f ? t : t * scale;
      } else {
        Best b = best_identity();
        for (uint32_t r = tx; r < red; r += 32) b = best_of(b, Best{__ldg(p + (int64_t)r * s_red), r});
        b = warp_best(b);
        if (tx == 0) {
          if (out) out[o] = b.v;
          if (idx) idx[o] = (int64_t)b.i;
        }
      }
    }
  } else {
    __shared__ float sv[8][33];
    __shared__ uint32_t si[8][33];
    for (uint32_t o0 = blockIdx.x * 32; o0 < nout; o0 += gridDim.x * 32) {
      const uint32_t o = o0 + tx;
      const bool live = o < nout;
      const float* p = x + (live ? kept_offset(kd, o) : 0);
      if constexpr (OP == 0) {
        float a = 0.0f;
        if (live) {
          uint32_t r = ty;
          for (; r + 24 < red; r += 32) {
            const float v0 = __ldg(p + (int64_t)r * s_red), v1 = __ldg(p + (int64_t)(r + 8) * s_red);
            const float v2 = __ldg(p + (int64_t)(r + 16) * s_red), v3 = __ldg(p + (int64_t)(r + 24) * s_red);
            a += v0; a += v1; a += v2; a += v3;
          }
          for (; r < red; r += 8) a += __ldg(p + (int64_t)r * s_red);
        }
        sv[ty][tx] = a;
        __syncthreads();
        if (ty == 0 && live) {
          float t = sv[0][tx];
#pragma unroll
          for (int w = 1; w < 8; ++w) t += sv[w][tx];
          out[o] = scale == 1.0f ? t : t * scale;
        }
        __syncthreads();
      } else {
        Best b = best_identity();
        if (live)
          for (uint32_t r = ty; r < red; r += 8) b = best_of(b, Best{__ldg(p + (int64_t)r * s_red), r});
        sv[ty][tx] = b.v;
        si[ty][tx] = (uint32_t)b.i;
        __syncthreads();
        if (ty == 0 && live) {
          for (int w = 1; w < 8; ++w) b = best_of(b, Best{sv[w][tx], (uint64_t)si[w][tx]});
          if (out) out[o] = b.v;
          if (idx) idx[o] = (int64_t)b.i;
        }
        __syncthreads();
      }
    }
  }
}

// ------------------------------------------------------------------- softmax
// MODE 0 softmax fwd, 1 log_softmax fwd, 2 softmax bwd (a = g, b = y), 3 log_softmax bwd (a = g, b = y).
// A "column" is one slice along the softmax dim; kept index o addresses it in the input view(s),
// and its place in the row-major output is (o / inner_after) * size * inner_after + o % inner_after
// with element stride inner_after.
struct SoftmaxViewArgs {
  KeptIndex ka, kb;     // input a (x or g) and input b (y, backward only)
  int64_t sa, sb;       // strides of the softmax dim in a and b
  uint32_t size, ncols, inner_after;
  FastDiv div_inner;
};

// exp(a - m) with m = -inf read as 0 (a column that has only seen -inf so far adds nothing).
__device__ __forceinline__ void online_fold(float& m, float& s, float v) {
  if (v > m) {
    s *= __expf((m == -INFINITY ? 0.0f : m) - v);
    m = v;
  }
  s += __expf(v - (m == -INFINITY ? 0.0f : m));
}
__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float M = fmaxf(m, m2);
  const float ms = M == -INFINITY ? 0.0f : M;  // two parts that saw only -inf: exp(-inf - 0) = 0, not exp(NaN)
  s = s * __expf(m - ms) + s2 * __expf(m2 - ms);
  m = M;
}

template <int MODE, bool LANES_DIM>
__global__ void __launch_bounds__(kVwThreads)
view_softmax_kernel(const float* __restrict__ a, const float* __restrict__ b, const __grid_constant__ SoftmaxViewArgs A,
                    float* __restrict__ out) {
  constexpr bool BWD = MODE >= 2, LOG = (MODE & 1) != 0;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  __shared__ float sm_m[8][33], sm_s[8][33];
  const uint32_t size = A.size;
  // Column of this thread and its role along the softmax dim.
  const uint32_t cols_per_cta = LANES_DIM ? 8 : 32;
  for (uint32_t c0 = blockIdx.x * cols_per_cta; c0 < A.ncols; c0 += gridDim.x * cols_per_cta) {
    const uint32_t o = c0 + (LANES_DIM ? ty : tx);
    const bool live = o < A.ncols;
    const uint32_t k0 = LANES_DIM ? tx : ty, kstep = LANES_DIM ? 32 : 8;
    const float* pa = a + (live ? kept_offset(A.ka, o) : 0);
    const float* pb = BWD ? b + (live ? kept_offset(A.kb, o) : 0) : nullptr;
    const uint32_t ob = fdiv(o, A.div_inner), oi = o - ob * A.inner_after;
    float* po = out + (uint64_t)ob * size * A.inner_after + oi;
    // pass 1: the column's statistics
    float m = -INFINITY, s = 0.0f;
    if (live) {
      for (uint32_t k = k0; k < size; k += kstep) {
        const float va = __ldg(pa + (int64_t)k * A.sa);
        if constexpr (!BWD) {
          online_fold(m, s, va);
        } else {
          if constexpr (LOG) s += va;
          else s += va * __ldg(pb + (int64_t)k * A.sb);
        }
      }
    }
    // combine the partial statistics of the column
    if constexpr (LANES_DIM) {
      if constexpr (!BWD) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          const float m2 = __shfl_xor_sync(0xffffffffu, m, off), s2 = __shfl_xor_sync(0xffffffffu, s, off);
          online_merge(m, s, m2, s2);
        }
      } else {
        s = warp_sum(s);
      }
    } else {
      sm_m[ty][tx] = m;
      sm_s[ty][tx] = s;
      __syncthreads();
      m = sm_m[0][tx];
      s = sm_s[0][tx];
#pragma unroll
      for (int w = 1; w < 8; ++w) {
        if constexpr (!BWD) online_merge(m, s, sm_m[w][tx], sm_s[w][tx]);
        else s += sm_s[w][tx];
      }
      __syncthreads();
    }
    // pass 2: the outputs (the column has just been read: L2 serves most of it)
    if (live) {
      const float ls = (!BWD && LOG) ? logf(s) : 0.0f;
      const float inv = 1.0f / s;
      for (uint32_t k = k0; k < size; k += kstep) {
        const float va = __ldg(pa + (int64_t)k * A.sa);
        float r;
        if constexpr (MODE == 0) r = __expf(va - m) * inv;
        else if constexpr (MODE == 1) r = (va - m) - ls;
        else {
          const float vb = __ldg(pb + (int64_t)k * A.sb);
          if constexpr (MODE == 2) r = vb * (va - s);
          else r = va - __expf(vb) * s;
        }
        po[(uint64_t)k * A.inner_after] = r;
      }
    }
  }
}

// ---------------------------------------------------------------- host side
struct ViewPlan {
  KeptIndex kept;
  int64_t s_dim;       // stride of the reduced / softmax dim
  uint64_t size;       // its extent
  uint64_t ncols;      // product of the kept extents
  uint64_t inner_after;
  uint64_t outer, inner;  // contiguous decomposition (valid when `whole`)
  bool whole;          // the view is the whole row-major tensor at its offset
  int64_t min_kept_stride;
};

static int check_view(const char* name, const fb_view* v) {
  if (!v) return fail(FB_ERR_INVALID_ARG, "%s: null view", name);
  if (v->rank < 1 || v->rank > FB_MAX_RANK) return fail(FB_ERR_INVALID_SHAPE, "%s: rank %d not in 1..%d", name, v->rank, FB_MAX_RANK);
  uint64_t n = 1;
  for (int d = 0; d < v->rank; ++d)
    if (mul_overflows(n, v->shape[d], &n) || n > (UINT64_MAX >> 3)) return fail(FB_ERR_INVALID_SHAPE, "%s: shape overflows", name);
  if (n == 0) return FB_OK;
  if (!v->ptr) return fail(FB_ERR_INVALID_ARG, "%s: null storage", name);
  __int128 lo = v->offset, hi = v->offset;
  for (int d = 0; d < v->rank; ++d) {
    const __int128 span = (__int128)(v->shape[d] - 1) * v->strides[d];
    if (span >= 0) hi += span;
    else lo += span;
  }
  if (lo < 0 || hi >= (__int128)v->len)
    return fail(FB_ERR_INVALID_SHAPE, "%s: the view reaches outside its storage of %llu elements", name,
                (unsigned long long)v->len);
  return FB_OK;
}

static uint64_t view_numel(const fb_view* v) {
  uint64_t n = 1;
  for (int d = 0; d < v->rank; ++d) n *= v->shape[d];
  return n;
}

static int plan_view(const char* name, const fb_view* v, int dim, ViewPlan* p) {
  if (dim < 0 || dim >= v->rank) return fail(FB_ERR_INVALID_SHAPE, "%s: dim %d out of range for rank %d", name, dim, v->rank);
  *p = ViewPlan{};
  p->size = v->shape[dim];
  p->s_dim = v->strides[dim];
  p->ncols = 1;
  p->inner_after = 1;
  p->outer = 1;
  p->inner = 1;
  p->min_kept_stride = INT64_MAX;
  bool whole = true;
  int64_t expect = 1;
  for (int d = v->rank - 1; d >= 0; --d) {
    if (v->shape[d] != 1 && v->strides[d] != expect) whole = false;
    expect *= (int64_t)v->shape[d];
  }
  p->whole = whole;
  int n = 0;
  for (int d = 0; d < v->rank; ++d) {
    if (d == dim) continue;
    if (d < dim) p->outer *= v->shape[d];
    else { p->inner *= v->shape[d]; p->inner_after *= v->shape[d]; }
    if (v->shape[d] == 1) continue;
    p->kept.ext[n] = (uint32_t)v->shape[d];
    p->kept.div[n] = make_fastdiv((uint32_t)v->shape[d]);
    p->kept.stride[n] = v->strides[d];
    const int64_t as = v->strides[d] < 0 ? -v->strides[d] : v->strides[d];
    if (as < p->min_kept_stride) p->min_kept_stride = as;
    p->ncols *= v->shape[d];
    ++n;
  }
  p->kept.n = n;
  if (p->ncols >= (1ull << 31) || p->size >= (1ull << 31))
    return fail(FB_ERR_UNSUPPORTED, "%s: a view with 2^31 or more kept elements or reduced elements is not supported", name);
  return FB_OK;
}

static bool lanes_along_dim(const ViewPlan& p) {
  const int64_t as = p.s_dim < 0 ? -p.s_dim : p.s_dim;
  return p.size >= 64 && as <= 1 && (p.kept.n == 0 || p.min_kept_stride > 1);
}

template <int OP>
static int reduce_view(cudaStream_t stream, const char* name, const fb_view* x, int dim, float scale_is_mean,
                       float* out, int64_t* idx, void* workspace, uint64_t workspace_bytes) {
  if (int rc = check_view(name, x)) return rc;
  ViewPlan p;
  if (int rc = plan_view(name, x, dim, &p)) return rc;
  if (p.ncols == 0) return FB_OK;  // no outputs
  if (OP == 1 && p.size == 0) return fail(FB_ERR_INVALID_SHAPE, "%s: max over an empty dimension", name);
  if (!out && !(OP == 1 && idx)) return fail(FB_ERR_INVALID_ARG, "%s: null output", name);
  if (p.size == 0)  // the empty sum is 0; the empty mean is 0 * (1 / 0) = NaN, as in ops_ext/mean_dim.rs:24-30
    return fb_fill(stream, out, scale_is_mean != 0.0f ? NAN : 0.0f, p.ncols);
  const float* base = x->ptr + x->offset;
  if (p.whole) {
    if (OP == 0)
      return scale_is_mean != 0.0f ? fb_mean_dim(stream, base, p.outer, p.size, p.inner, out, workspace, workspace_bytes)
                                   : fb_sum_dim(stream, base, p.outer, p.size, p.inner, out, workspace, workspace_bytes);
    return fb_max_dim(stream, base, p.outer, p.size, p.inner, out, idx, workspace, workspace_bytes);
  }
  const float scale = scale_is_mean != 0.0f ? 1.0f / (float)p.size : 1.0f;  // ops_ext/mean_dim.rs:24-30: multiply by 1/n
  const uint32_t nout = (uint32_t)p.ncols, red = (uint32_t)p.size;
  if (lanes_along_dim(p)) {
    const unsigned grid = grid_for((nout + 7) / 8, 8);
    view_reduce_kernel<OP, true><<<grid, kVwThreads, 0, stream>>>(base, p.kept, p.s_dim, red, nout, scale, out, idx);
  } else {
    const unsigned grid = grid_for((nout + 31) / 32, 8);
    view_reduce_kernel<OP, false><<<grid, kVwThreads, 0, stream>>>(base, p.kept, p.s_dim, red, nout, scale, out, idx);
  }
  FB_LAUNCHED(name);
  return FB_OK;
}

template <int MODE>
static int softmax_view(cudaStream_t stream, const char* name, const fb_view* a, const fb_view* b, int dim, float* out) {
  constexpr bool BWD = MODE >= 2;
  if (int rc = check_view(name, a)) return rc;
  ViewPlan pa, pb;
  if (int rc = plan_view(name, a, dim, &pa)) return rc;
  if (BWD) {
    if (int rc = check_view(name, b)) return rc;
    if (b->rank != a->rank) return fail(FB_ERR_INVALID_SHAPE, "%s: the two views differ in rank", name);
    for (int d = 0; d < a->rank; ++d)
      if (a->shape[d] != b->shape[d]) return fail(FB_ERR_INVALID_SHAPE, "%s: the two views differ in shape", name);
    if (int rc = plan_view(name, b, dim, &pb)) return rc;
  }
  const uint64_t n = view_numel(a);
  if (n == 0) return FB_OK;
  if (!out) return fail(FB_ERR_INVALID_ARG, "%s: null output", name);
  const float* base_a = a->ptr + a->offset;
  const float* base_b = BWD ? b->ptr + b->offset : nullptr;
  // Whole row-major inputs with the softmax dim last: the row kernels of softmax.cu.
  if (pa.whole && pa.inner_after == 1 && (!BWD || pb.whole)) {
    const uint64_t rows = n / pa.size;
    if (MODE == 0) return fb_softmax_fwd(stream, base_a, rows, pa.size, out);
    if (MODE == 1) return fb_log_softmax_fwd(stream, base_a, rows, pa.size, out);
    if (MODE == 2) return fb_softmax_bwd(stream, base_a, base_b, rows, pa.size, out);
    return fb_log_softmax_bwd(stream, base_a, base_b, rows, pa.size, out);
  }
  SoftmaxViewArgs A{};
  A.ka = pa.kept;
  A.sa = pa.s_dim;
  if (BWD) {
    A.kb = pb.kept;
    A.sb = pb.s_dim;
  }
  A.size = (uint32_t)pa.size;
  A.ncols = (uint32_t)pa.ncols;
  A.inner_after = (uint32_t)pa.inner_after;
  A.div_inner = make_fastdiv((uint32_t)pa.inner_after);
  // Lanes along the softmax dim when the output is contiguous along it (it is the last dim);
  // otherwise lanes along the columns, which are then contiguous in the output.
  if (pa.inner_after == 1) {
    const unsigned grid = grid_for((A.ncols + 7) / 8, 8);
    view_softmax_kernel<MODE, true><<<grid, kVwThreads, 0, stream>>>(base_a, base_b, A, out);
  } else {
    const unsigned grid = grid_for((A.ncols + 31) / 32, 8);
    view_softmax_kernel<MODE, false><<<grid, kVwThreads, 0, stream>>>(base_a, base_b, A, out);
  }
  FB_LAUNCHED(name);
  return FB_OK;
}

}  // namespace fb

using namespace fb;

extern "C" {

uint64_t fb_reduce_view_workspace_bytes(const fb_view* x, int dim) {
  if (!x || x->rank < 1 || x->rank > FB_MAX_RANK || dim < 0 || dim >= x->rank) return 0;
  uint64_t outer = 1, inner = 1;
  for (int d = 0; d < dim; ++d) outer *= x->shape[d];
  for (int d = dim + 1; d < x->rank; ++d) inner *= x->shape[d];
  return fb_reduce_dim_workspace_bytes(outer, x->shape[dim], inner);
}

int fb_sum_dim_view(fb_stream_t stream, const fb_view* x, int dim, float* out, void* workspace, uint64_t workspace_bytes) {
  return reduce_view<0>(stream, "fb_sum_dim_view", x, dim, 0.0f, out, nullptr, workspace, workspace_bytes);
}
int fb_mean_dim_view(fb_stream_t stream, const fb_view* x, int dim, float* out, void* workspace, uint64_t workspace_bytes) {
  return reduce_view<0>(stream, "fb_mean_dim_view", x, dim, 1.0f, out, nullptr, workspace, workspace_bytes);
}
int fb_max_dim_view(fb_stream_t stream, const fb_view* x, int dim, float* values, int64_t* indices, void* workspace,
                    uint64_t workspace_bytes) {
  return reduce_view<1>(stream, "fb_max_dim_view", x, dim, 0.0f, values, indices, workspace, workspace_bytes);
}
int fb_softmax_view_fwd(fb_stream_t stream, const fb_view* x, int dim, float* y) {
  return softmax_view<0>(stream, "fb_softmax_view_fwd", x, nullptr, dim, y);
}
int fb_log_softmax_view_fwd(fb_stream_t stream, const fb_view* x, int dim, float* y) {
  return softmax_view<1>(stream, "fb_log_softmax_view_fwd", x, nullptr, dim, y);
}
int fb_softmax_view_bwd(fb_stream_t stream, const fb_view* g, const fb_view* y, int dim, float* dx) {
  return softmax_view<2>(stream, "fb_softmax_view_bwd", g, y, dim, dx);
}
int fb_log_softmax_view_bwd(fb_stream_t stream, const fb_view* g, const fb_view* y, int dim, float* dx) {
  return softmax_view<3>(stream, "fb_log_softmax_view_bwd", g, y, dim, dx);
}

}  // extern "C"
