// Index-driven ops: gather along a dim by an i64 index tensor and its
// scatter-add backward, and the CSR segment sum / softmax with their backward.
//
// ferro computes gather and its backward on the host whatever the device
// (crates/ferro-core/src/ops_ext/gather.rs:12-111 works on to_vec() copies) and
// runs the segment ops with one thread per (group, feature) that walks the
// group's edges alone (crates/ferro-cuda/src/segment.cu:1-40, launched by
// segment.rs:36-89).  All of these are bandwidth-bound and index-driven; none
// uses a float atomic here, so results do not depend on scheduling:
//   gather        one thread per output element, lanes along the innermost dim;
//   scatter-add   the thread that owns a (outer, inner) column of the gradient
//                 walks the index along the gathered dim in order and is the
//                 only writer of that column: additions land in the order of
//                 ferro's host loop (ascending flat output index), so the
//                 result is bit-identical to it;
//   segment ops   a group is owned by one warp (narrow features: by a slice of
//                 a warp), lanes along the features so that every edge row is a
//                 coalesced read, edges in CSR order, which is the ascending
//                 edge order of ferro's CPU loops (segment.rs:132-150, 217-253):
//                 sums are bit-identical to them.
// Roofline: HBM.  Algorithmic bytes: gather 4 (value) + 8 (index) + 4 (output)
// per output element; segment sum 4 * (edges + groups) * width + 8 * edges.
#include "common.cuh"

namespace fb {

struct GatherDims {
  int rank, dim;
  uint32_t out_ext[FB_MAX_RANK];
  uint64_t in_stride[FB_MAX_RANK];  // row-major element strides of the input
  uint64_t dim_size;
};

// out[c] = x[c with c[dim] replaced by index[c]]
__global__ void __launch_bounds__(256)
gather_dim_kernel(const float* __restrict__ x, const int64_t* __restrict__ index, const __grid_constant__ GatherDims G,
                  uint64_t n, float* __restrict__ out, int64_t* __restrict__ bad) {
  const uint64_t stride = (uint64_t)gridDim.x * 256;
  for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
    const int64_t id = __ldg(index + i);
    uint64_t rem = i, off = 0;
    for (int d = G.rank - 1; d >= 0; --d) {
      const uint64_t q = rem / G.out_ext[d], c = rem - q * G.out_ext[d];
      rem = q;
      if (d != G.dim) off += c * G.in_stride[d];
    }
    float v = 0.0f;
    if (id >= 0 && (uint64_t)id < G.dim_size) v = __ldg(x + off + (uint64_t)id * G.in_stride[G.dim]);
    else if (bad) *bad = (int64_t)i + 1;
    out[i] = v;
  }
}

// gx (zeroed by the caller of the kernel) += g scattered back; one thread per column.
__global__ void __launch_bounds__(256)
scatter_add_dim_kernel(const float* __restrict__ g, const int64_t* __restrict__ index, const __grid_constant__ GatherDims G,
                       uint64_t ncols, uint64_t out_dim_stride, float* __restrict__ gx, int64_t* __restrict__ bad) {
  const uint64_t stride = (uint64_t)gridDim.x * 256;
  const uint32_t J = G.out_ext[G.dim];
  for (uint64_t col = (uint64_t)blockIdx.x * 256 + threadIdx.x; col < ncols; col += stride) {
    // column index -> coordinates of every dim but `dim` -> bases in g / index and in gx
    uint64_t rem = col, in_base = 0, out_base = 0, ostr = 1;
    for (int d = G.rank - 1; d >= 0; --d) {
      if (d == G.dim) {
        ostr *= G.out_ext[d];
        continue;
      }
      const uint64_t q = rem / G.out_ext[d], c = rem - q * G.out_ext[d];
      rem = q;
      in_base += c * G.in_stride[d];
      out_base += c * ostr;
      ostr *= G.out_ext[d];
    }
    for (uint32_t j = 0; j < J; ++j) {
      const uint64_t o = out_base + (uint64_t)j * out_dim_stride;
      const int64_t id = __ldg(index + o);
      if (id >= 0 && (uint64_t)id < G.dim_size) {
        float* p = gx + in_base + (uint64_t)id * G.in_stride[G.dim];
        *p = *p + __ldg(g + o);
      } else if (bad) {
        *bad = (int64_t)o + 1;
      }
    }
  }
}

// ---------------------------------------------------------------- segments
// csr = [groups + 1 offsets][edges edge ids], as ferro's device plan (segment.rs:20-33).
// LPG lanes per group (a power of two, 1..32): a warp holds 32 / LPG groups side by side when the
// feature width is small.  Lane l of a group handles features l, l + LPG, ...
// MODE 0 sum, 1 sum backward, 2 softmax forward, 3 softmax backward.
template <int MODE>
__global__ void __launch_bounds__(256)
segment_kernel(const float* __restrict__ x, const float* __restrict__ y, const int64_t* __restrict__ csr,
               uint32_t groups, uint32_t width, int lpg, float* __restrict__ out, int* __restrict__ status) {
  const int64_t* edge = csr + groups + 1;
  const uint32_t gpw = 32 / lpg;  // groups per warp
  const uint32_t warp = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const uint32_t nwarps = gridDim.x * 8;
  const uint32_t sub = lane / lpg, fl = lane % lpg;
  for (uint64_t g0 = (uint64_t)warp * gpw; g0 < groups; g0 += (uint64_t)nwarps * gpw) {
    const uint64_t s = g0 + sub;
    if (s >= groups) continue;
    const int64_t begin = __ldg(csr + s), end = __ldg(csr + s + 1);
    for (uint32_t f = fl; f < width; f += lpg) {
      if constexpr (MODE == 0) {
        float sum = 0.0f;
        int64_t p = begin;
        for (; p + 4 <= end; p += 4) {  // four edge rows in flight, added in edge order
          const int64_t e0 = __ldg(edge + p), e1 = __ldg(edge + p + 1), e2 = __ldg(edge + p + 2), e3 = __ldg(edge + p + 3);
          const float v0 = __ldg(x + e0 * width + f), v1 = __ldg(x + e1 * width + f);
          const float v2 = __ldg(x + e2 * width + f), v3 = __ldg(x + e3 * width + f);
          sum += v0; sum += v1; sum += v2; sum += v3;
        }
        for (; p < end; ++p) sum += __ldg(x + __ldg(edge + p) * width + f);
        out[s * width + f] = sum;
      } else if constexpr (MODE == 1) {
        const float v = __ldg(x + s * width + f);
        for (int64_t p = begin; p < end; ++p) out[__ldg(edge + p) * width + f] = v;
      } else if constexpr (MODE == 2) {
        float m = -INFINITY;
        bool bad = false;
        for (int64_t p = begin; p < end; ++p) {
          const float v = __ldg(x + __ldg(edge + p) * width + f);
          bad |= !isfinite(v);
          m = fmaxf(m, v);
        }
        if (bad && status) atomicExch(status, 1);
        float denom = 0.0f;
        for (int64_t p = begin; p < end; ++p) {
          const int64_t j = __ldg(edge + p) * width + f;
          const float v = expf(__ldg(x + j) - m);
          out[j] = v;
          denom += v;
        }
        for (int64_t p = begin; p < end; ++p) {
          const int64_t j = __ldg(edge + p) * width + f;
          out[j] = out[j] / denom;
        }
      } else {
        float dot = 0.0f;
        for (int64_t p = begin; p < end; ++p) {
          const int64_t j = __ldg(edge + p) * width + f;
          dot += __ldg(x + j) * __ldg(y + j);
        }
        for (int64_t p = begin; p < end; ++p) {
          const int64_t j = __ldg(edge + p) * width + f;
          out[j] = __ldg(y + j) * (__ldg(x + j) - dot);
        }
      }
    }
  }
}

static int gather_dims(const char* name, const uint64_t* in_shape, const uint64_t* out_shape, int rank, int dim,
                       GatherDims* G, uint64_t* n_in, uint64_t* n_out) {
  if (rank < 1 || rank > FB_MAX_RANK) return fail(FB_ERR_INVALID_SHAPE, "%s: rank %d not in 1..%d", name, rank, FB_MAX_RANK);
  if (dim < 0 || dim >= rank) return fail(FB_ERR_INVALID_SHAPE, "%s: dim %d out of range for rank %d", name, dim, rank);
  if (!in_shape || !out_shape) return fail(FB_ERR_INVALID_ARG, "%s: null shape", name);
  *G = GatherDims{};
  G->rank = rank;
  G->dim = dim;
  uint64_t ni = 1, no = 1;
  for (int d = rank - 1; d >= 0; --d) {
    G->in_stride[d] = ni;
    if (mul_overflows(ni, in_shape[d], &ni) || mul_overflows(no, out_shape[d], &no) || ni > (UINT64_MAX >> 3) ||
        no > (UINT64_MAX >> 3))
      return fail(FB_ERR_INVALID_SHAPE, "%s: shape overflows", name);
    if (out_shape[d] >= (1ull << 32)) return fail(FB_ERR_UNSUPPORTED, "%s: an index extent of 2^32 or more", name);
    // gather.rs:38-48: the index may not exceed the input in any dim but `dim`
    if (d != dim && out_shape[d] > in_shape[d])
      return fail(FB_ERR_INVALID_SHAPE, "%s: index shape exceeds the input shape at dim %d", name, d);
    G->out_ext[d] = (uint32_t)out_shape[d];
  }
  G->dim_size = in_shape[dim];
  *n_in = ni;
  *n_out = no;
  return FB_OK;
}

static int segment_args(const char* name, uint64_t groups, uint64_t edges, uint64_t width, uint64_t* n_edges,
                        uint64_t* n_groups) {
  if (mul_overflows(edges, width, n_edges) || mul_overflows(groups, width, n_groups) || *n_edges > (1ull << 40) ||
      *n_groups > (1ull << 40) || groups >= (1ull << 32) || width >= (1ull << 32))
    return fail(FB_ERR_INVALID_SHAPE, "%s: invalid segment buffer or size", name);  // segment.rs:47-49
  return FB_OK;
}

static int lanes_per_group(uint64_t width) {
  int l = 1;
  while (l < 32 && (uint64_t)l < width) l <<= 1;
  return l;
}

template <int MODE>
static int run_segment(cudaStream_t stream, const char* name, const float* x, const float* y, const int64_t* csr,
                       uint64_t groups, uint64_t edges, uint64_t width, float* out, int* status) {
  uint64_t ne, ng;
  if (int rc = segment_args(name, groups, edges, width, &ne, &ng)) return rc;
  const uint64_t n_out = (MODE == 0) ? ng : ne;
  if (groups == 0 || n_out == 0) return FB_OK;
  if (!csr || !out || (ne && !x) || (MODE == 3 && ne && !y)) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  const int lpg = lanes_per_group(width);
  const uint64_t warps = (groups + (32 / lpg) - 1) / (32 / lpg);
  const unsigned grid = grid_for((warps + 7) / 8, 8);
  segment_kernel<MODE><<<grid, 256, 0, stream>>>(x, y, csr, (uint32_t)groups, (uint32_t)width, lpg, out, status);
  FB_LAUNCHED(name);
  return FB_OK;
}

}  // namespace fb

using namespace fb;

extern "C" {

int fb_gather_dim(fb_stream_t stream, const float* x, const uint64_t* in_shape, const int64_t* index,
                  const uint64_t* out_shape, int rank, int dim, float* out, int64_t* bad_index) {
  const char* name = "fb_gather_dim";
  GatherDims G;
  uint64_t ni, no;
  if (int rc = gather_dims(name, in_shape, out_shape, rank, dim, &G, &ni, &no)) return rc;
  if (no == 0) return FB_OK;
  if (ni == 0) return fail(FB_ERR_INVALID_SHAPE, "%s: indices into an empty tensor", name);
  if (!x || !index || !out) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  gather_dim_kernel<<<grid_for((no + 255) / 256, 16), 256, 0, stream>>>(x, index, G, no, out, bad_index);
  FB_LAUNCHED(name);
  return FB_OK;
}

int fb_scatter_add_dim(fb_stream_t stream, const float* g, const int64_t* index, const uint64_t* in_shape,
                       const uint64_t* out_shape, int rank, int dim, float* gx, int64_t* bad_index) {
  const char* name = "fb_scatter_add_dim";
  GatherDims G;
  uint64_t ni, no;
  if (int rc = gather_dims(name, in_shape, out_shape, rank, dim, &G, &ni, &no)) return rc;
  if (ni == 0) return FB_OK;
  if (!gx) return fail(FB_ERR_INVALID_ARG, "%s: null output", name);
  if (int rc = fb_fill(stream, gx, 0.0f, ni)) return rc;  // positions nothing was gathered from keep a zero gradient
  if (no == 0) return FB_OK;
  if (!g || !index) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  uint64_t out_dim_stride = 1;
  for (int d = rank - 1; d > dim; --d) out_dim_stride *= out_shape[d];
  const uint64_t ncols = no / out_shape[dim];
  scatter_add_dim_kernel<<<grid_for((ncols + 255) / 256, 16), 256, 0, stream>>>(g, index, G, ncols, out_dim_stride, gx,
                                                                               bad_index);
  FB_LAUNCHED(name);
  return FB_OK;
}

int fb_segment_csr_build(const uint64_t* ids, uint64_t edges, uint64_t groups, int64_t* csr) {
  const char* name = "fb_segment_csr_build";
  if ((edges && !ids) || !csr) return fail(FB_ERR_INVALID_ARG, "%s: null argument", name);
  for (uint64_t e = 0; e < edges; ++e)
    if (ids[e] >= groups) return fail(FB_ERR_INVALID_SHAPE, "%s: segment id out of bounds", name);  // segment.rs:27-29
  for (uint64_t s = 0; s <= groups; ++s) csr[s] = 0;
  for (uint64_t e = 0; e < edges; ++e) csr[ids[e] + 1] += 1;
  for (uint64_t s = 0; s < groups; ++s) csr[s + 1] += csr[s];
  // Stable fill: within a group, edges keep their ascending order (segment.rs:27-33).
  int64_t* edge = csr + groups + 1;
  int64_t* next = new int64_t[groups ? groups : 1];
  for (uint64_t s = 0; s < groups; ++s) next[s] = csr[s];
  for (uint64_t e = 0; e < edges; ++e) edge[next[ids[e]]++] = (int64_t)e;
  delete[] next;
  return FB_OK;
}

int fb_segment_sum(fb_stream_t stream, const float* x, const int64_t* csr, uint64_t groups, uint64_t edges,
                   uint64_t width, float* out) {
  return run_segment<0>(stream, "fb_segment_sum", x, nullptr, csr, groups, edges, width, out, nullptr);
}
int fb_segment_sum_bwd(fb_stream_t stream, const float* g, const int64_t* csr, uint64_t groups, uint64_t edges,
                       uint64_t width, float* dx) {
  return run_segment<1>(stream, "fb_segment_sum_bwd", g, nullptr, csr, groups, edges, width, dx, nullptr);
}
int fb_segment_softmax_fwd(fb_stream_t stream, const float* x, const int64_t* csr, uint64_t groups, uint64_t edges,
                           uint64_t width, float* y, int* not_finite) {
  return run_segment<2>(stream, "fb_segment_softmax_fwd", x, nullptr, csr, groups, edges, width, y, not_finite);
}
int fb_segment_softmax_bwd(fb_stream_t stream, const float* g, const float* y, const int64_t* csr, uint64_t groups,
                           uint64_t edges, uint64_t width, float* dx) {
  return run_segment<3>(stream, "fb_segment_softmax_bwd", g, y, csr, groups, edges, width, dx, nullptr);
}

}  // extern "C"
