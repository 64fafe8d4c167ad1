// Contiguous elementwise kernels: unary, binary, the in-place family, fill,
// copy and the i64 row gather.  All are one read and one write per element
// with 128-bit accesses whenever the pointers allow it.
//
// Roofline: HBM.  Algorithmic bytes: unary / affine / copy 8n, binary / axpy
// 12n, fill 4n (ferro's own accounting, benchmarks/README.md:28-30).
#include "common.cuh"
#include "math.cuh"

namespace fb {

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;  // independent 16-byte loads in flight per thread

// out[i] = op(in0[i], in1[i]) for NIN in {0, 1, 2}.  VEC = 4 processes float4
// groups (all pointers 16-byte aligned) plus a scalar tail; VEC = 1 is the
// fallback for unaligned buffers.  `out` may alias an input: each thread
// reads the elements it later writes, nothing else.
template <int VEC, int NIN, class Op>
__global__ void __launch_bounds__(kEwThreads) ew_kernel(Op op, const float* in0, const float* in1,
                                                        float* out, uint64_t n, int ro) {
  // ro: the output aliases no input, so the inputs may take the read-only path.
  const uint64_t nvec = n / VEC;
  const uint64_t tile = (uint64_t)kEwThreads * kEwUnroll;
  const uint64_t ntiles = (nvec + tile - 1) / tile;
  for (uint64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t base = t * tile + threadIdx.x;
    if constexpr (VEC == 4) {
      float4 a[kEwUnroll], b[kEwUnroll];
#pragma unroll
      for (int u = 0; u < kEwUnroll; ++u) {
        const uint64_t i = base + (uint64_t)u * kEwThreads;
        if (i < nvec) {
          if constexpr (NIN >= 1) a[u] = ro ? __ldg(reinterpret_cast<const float4*>(in0 + i * 4)) : ld_stream4(in0 + i * 4);
          if constexpr (NIN >= 2) b[u] = ro ? __ldg(reinterpret_cast<const float4*>(in1 + i * 4)) : ld_stream4(in1 + i * 4);
        }
      }
#pragma unroll
      for (int u = 0; u < kEwUnroll; ++u) {
        const uint64_t i = base + (uint64_t)u * kEwThreads;
        if (i < nvec) {
          float4 r;
          r.x = op(a[u].x, b[u].x);
          r.y = op(a[u].y, b[u].y);
          r.z = op(a[u].z, b[u].z);
          r.w = op(a[u].w, b[u].w);
          st_stream4(out + i * 4, r);
        }
      }
    } else {
      float a[kEwUnroll], b[kEwUnroll];
#pragma unroll
      for (int u = 0; u < kEwUnroll; ++u) {
        const uint64_t i = base + (uint64_t)u * kEwThreads;
        if (i < nvec) {
          if constexpr (NIN >= 1) a[u] = ld_stream(in0 + i);
          if constexpr (NIN >= 2) b[u] = ld_stream(in1 + i);
        }
      }
#pragma unroll
      for (int u = 0; u < kEwUnroll; ++u) {
        const uint64_t i = base + (uint64_t)u * kEwThreads;
        if (i < nvec) st_stream(out + i, op(a[u], b[u]));
      }
    }
  }
  if constexpr (VEC == 4) {
    // Scalar tail (n % 4 elements), done by the first threads of CTA 0.
    const uint64_t done = nvec * 4;
    if (blockIdx.x == 0 && threadIdx.x < n - done) {
      const uint64_t i = done + threadIdx.x;
      float a = 0.0f, b = 0.0f;
      if constexpr (NIN >= 1) a = in0[i];
      if constexpr (NIN >= 2) b = in1[i];
      out[i] = op(a, b);
    }
  }
}

template <int NIN, class Op>
static int launch_ew(cudaStream_t s, Op op, const float* in0, const float* in1, float* out,
                     uint64_t n, const char* name) {
  if (n == 0) return FB_OK;
  const bool vec = aligned16(out) && (NIN < 1 || aligned16(in0)) && (NIN < 2 || aligned16(in1));
  const uint64_t per_tile = (uint64_t)kEwThreads * kEwUnroll * (vec ? 4 : 1);
  const unsigned grid = grid_full((n + per_tile - 1) / per_tile);
  const int ro = (NIN < 1 || out != in0) && (NIN < 2 || out != in1);
  if (vec)
    ew_kernel<4, NIN, Op><<<grid, kEwThreads, 0, s>>>(op, in0, in1, out, n, ro);
  else
    ew_kernel<1, NIN, Op><<<grid, kEwThreads, 0, s>>>(op, in0, in1, out, n, ro);
  FB_LAUNCHED(name);
  return FB_OK;
}

template <int KIND>
struct UnaryOp {
  float p0, p1;
  __device__ __forceinline__ float operator()(float a, float) const {
    return unary_apply(KIND, p0, p1, a);
  }
};
template <int KIND>
struct BinaryOp {
  float p0, p1;
  __device__ __forceinline__ float operator()(float a, float b) const {
    return binary_apply(KIND, p0, p1, a, b);
  }
};
struct FillOp {
  float value;
  __device__ __forceinline__ float operator()(float, float) const { return value; }
};
struct AffineOp {  // dispatch.rs:452-457
  float mul, add;
  __device__ __forceinline__ float operator()(float d, float) const { return d * mul + add; }
};
struct AxpyOp {  // dispatch.rs:467-472: dst += alpha * src
  float alpha;
  __device__ __forceinline__ float operator()(float d, float s) const { return d + alpha * s; }
};
struct CopyOp {
  __device__ __forceinline__ float operator()(float a, float) const { return a; }
};

template <int K>
static int unary_dispatch(int kind, cudaStream_t s, float p0, float p1, const float* x, float* out,
                          uint64_t n) {
  if constexpr (K < FBI_UN_KIND_COUNT) {
    if (kind == K) return launch_ew<1>(s, UnaryOp<K>{p0, p1}, x, nullptr, out, n, "fb_unary");
    return unary_dispatch<K + 1>(kind, s, p0, p1, x, out, n);
  } else {
    return fail(FB_ERR_INVALID_ARG, "fb_unary: unknown kind %d", kind);
  }
}
template <int K>
static int binary_dispatch(int kind, cudaStream_t s, float p0, float p1, const float* a,
                           const float* b, float* out, uint64_t n, const char* name) {
  if constexpr (K < FB_BIN_KIND_COUNT) {
    if (kind == K) return launch_ew<2>(s, BinaryOp<K>{p0, p1}, a, b, out, n, name);
    return binary_dispatch<K + 1>(kind, s, p0, p1, a, b, out, n, name);
  } else {
    return fail(FB_ERR_INVALID_ARG, "%s: unknown kind %d", name, kind);
  }
}

// ---- i64 row gather --------------------------------------------------------
// One CTA-row per gathered row: out[o, :] = w[idx[o], :].
__global__ void __launch_bounds__(256) gather_rows_kernel(const float* __restrict__ w,
                                                          const int64_t* __restrict__ idx,
                                                          uint64_t n, uint64_t dim_size,
                                                          uint64_t inner, float* __restrict__ out,
                                                          int64_t* bad, int vec) {
  for (uint64_t o = blockIdx.x; o < n; o += gridDim.x) {
    const int64_t id = idx[o];
    const bool ok = id >= 0 && (uint64_t)id < dim_size;
    if (!ok && bad && threadIdx.x == 0) *bad = (int64_t)o + 1;
    const float* src = w + (ok ? (uint64_t)id : 0) * inner;
    float* dst = out + o * inner;
    if (vec) {
      for (uint64_t c = threadIdx.x; c < inner / 4; c += blockDim.x) {
        float4 v = ok ? __ldg(reinterpret_cast<const float4*>(src) + c) : make_float4(0, 0, 0, 0);
        st_stream4(dst + c * 4, v);
      }
    } else {
      for (uint64_t c = threadIdx.x; c < inner; c += blockDim.x) dst[c] = ok ? __ldg(src + c) : 0.0f;
    }
  }
}

}  // namespace fb

using namespace fb;

extern "C" {

int fb_unary(fb_stream_t stream, int kind, float p0, float p1, const float* x, float* out,
             uint64_t n) {
  if (kind < 0 || kind >= FB_UN_KIND_COUNT) return fail(FB_ERR_INVALID_ARG, "fb_unary: unknown kind %d", kind);
  if (n == 0) return FB_OK;
  if (!x || !out) return fail(FB_ERR_INVALID_ARG, "fb_unary: null buffer");
  return unary_dispatch<0>(resolve_unary_kind(kind, p0, p1), stream, p0, p1, x, out, n);
}

int fb_binary(fb_stream_t stream, int kind, float p0, float p1, const float* a, const float* b,
              float* out, uint64_t n) {
  if (kind < 0 || kind >= FB_BIN_KIND_COUNT) return fail(FB_ERR_INVALID_ARG, "fb_binary: unknown kind %d", kind);
  if (n == 0) return FB_OK;
  if (!a || !b || !out) return fail(FB_ERR_INVALID_ARG, "fb_binary: null buffer");
  return binary_dispatch<0>(kind, stream, p0, p1, a, b, out, n, "fb_binary");
}

int fb_fill(fb_stream_t stream, float* dst, float value, uint64_t n) {
  if (n == 0) return FB_OK;
  if (!dst) return fail(FB_ERR_INVALID_ARG, "fb_fill: null buffer");
  return launch_ew<0>(stream, FillOp{value}, nullptr, nullptr, dst, n, "fb_fill");
}

int fb_affine_inplace(fb_stream_t stream, float* dst, float mul, float add, uint64_t n) {
  if (n == 0) return FB_OK;
  if (!dst) return fail(FB_ERR_INVALID_ARG, "fb_affine_inplace: null buffer");
  return launch_ew<1>(stream, AffineOp{mul, add}, dst, nullptr, dst, n, "fb_affine_inplace");
}

int fb_binary_inplace(fb_stream_t stream, int kind, float* dst, const float* src, uint64_t n) {
  // ferro's in-place binary covers Add..ReluBackward (dispatch.rs:459-465).
  if (kind < 0 || kind > FB_BIN_RELU_BACKWARD)
    return fail(FB_ERR_INVALID_ARG, "fb_binary_inplace: unknown kind %d", kind);
  if (n == 0) return FB_OK;
  if (!dst || !src) return fail(FB_ERR_INVALID_ARG, "fb_binary_inplace: null buffer");
  return binary_dispatch<0>(kind, stream, 0.0f, 0.0f, dst, src, dst, n, "fb_binary_inplace");
}

int fb_axpy_inplace(fb_stream_t stream, float alpha, float* dst, const float* src, uint64_t n) {
  if (n == 0) return FB_OK;
  if (!dst || !src) return fail(FB_ERR_INVALID_ARG, "fb_axpy_inplace: null buffer");
  return launch_ew<2>(stream, AxpyOp{alpha}, dst, src, dst, n, "fb_axpy_inplace");
}

int fb_copy(fb_stream_t stream, float* dst, const float* src, uint64_t n) {
  if (n == 0) return FB_OK;
  if (!dst || !src) return fail(FB_ERR_INVALID_ARG, "fb_copy: null buffer");
  return launch_ew<1>(stream, CopyOp{}, src, nullptr, dst, n, "fb_copy");
}

int fb_gather_rows(fb_stream_t stream, const float* w, const int64_t* idx, uint64_t n,
                   uint64_t dim_size, uint64_t inner, float* out, int64_t* bad_index) {
  uint64_t total;
  if (mul_overflows(n, inner, &total) || mul_overflows(dim_size, inner, &total))
    return fail(FB_ERR_INVALID_SHAPE, "fb_gather_rows: size overflow");
  if (n == 0 || inner == 0) return FB_OK;
  if (dim_size == 0) return fail(FB_ERR_INVALID_SHAPE, "fb_gather_rows: empty table with %llu indices", (unsigned long long)n);
  if (!w || !idx || !out) return fail(FB_ERR_INVALID_ARG, "fb_gather_rows: null buffer");
  const int vec = (inner % 4 == 0) && aligned16(w) && aligned16(out);
  gather_rows_kernel<<<grid_for(n, 16), 256, 0, stream>>>(w, idx, n, dim_size, inner, out, bad_index, vec);
  FB_LAUNCHED("fb_gather_rows");
  return FB_OK;
}

}  // extern "C"
