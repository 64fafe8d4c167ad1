// Memory-bound glue of an MLP training step: the backward of bias-add (+ReLU)
// with its column-sum bias gradient, and the MSE loss with its gradient.
//
// Roofline: HBM.  Algorithmic bytes over [rows, cols]:
//   bias/relu backward   read g and x, write dx   12 * rows * cols (+ dbias)
//                        no relu: read g only, dx aliases g, 4 * rows * cols
//   mse forward+gradient read pred and target, write dpred  12 * n
// ferro today runs the bias gradient as sum_dim with one thread per column
// looping over all rows (crates/ferro-cuda/src/kernels.rs:319-332) and squares
// through a host round trip (crates/ferro-core/src/ops_ext/square.rs:16-19).
#include "common.cuh"
#include "math.cuh"
#include "reduce.cuh"

namespace fb {

// Column-sum source: value = relu_backward(g, x + bias), stored to dx on the way.
// g masked or scaled by the activation's derivative at z = x + bias: relu is the exact mask of
// ReluBackward (0 where z <= 0, g otherwise, NaN z included); gelu / silu multiply by act_grad(z).
__device__ __forceinline__ float act_bwd1(int act, float g, float z) {
  if (act == FB_ACT_RELU) return z <= 0.0f ? 0.0f : g;
  return g * act_grad(act, z);
}

struct BiasActBwdSrc {
  const float* g;
  const float* x;
  const float* bias;
  float* dx;
  uint64_t inner;
  int act;  // FB_ACT_*
  template <int VEC>
  __device__ __forceinline__ void load(uint64_t, uint64_t r, uint64_t c, float (&v)[1][VEC]) const {
    const uint64_t off = r * inner + c;
    if constexpr (VEC == 4) {
      float4 gg = ld_stream4(g + off);
      if (act) {
        float4 a = ld_stream4(x + off);
        if (bias) {
          const float4 b = __ldg(reinterpret_cast<const float4*>(bias + c));
          a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        gg.x = act_bwd1(act, gg.x, a.x); gg.y = act_bwd1(act, gg.y, a.y);
        gg.z = act_bwd1(act, gg.z, a.z); gg.w = act_bwd1(act, gg.w, a.w);
      }
      if (dx && (act || dx != g)) st_stream4(dx + off, gg);
      v[0][0] = gg.x; v[0][1] = gg.y; v[0][2] = gg.z; v[0][3] = gg.w;
    } else {
      float gg = g[off];
      if (act) {
        float a = x[off];
        if (bias) a += bias[c];
        gg = act_bwd1(act, gg, a);
      }
      if (dx && (act || dx != g)) dx[off] = gg;
      v[0][0] = gg;
    }
  }
};

// Without a bias gradient the backward is a plain masked (or scaled) copy.
__global__ void __launch_bounds__(256)
bias_act_bwd_nosum_kernel(const float* __restrict__ g, const float* __restrict__ x,
                          const float* __restrict__ bias, int act, uint64_t rows, uint64_t cols,
                          float* __restrict__ dx) {
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x)
    for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      float a = x[row * cols + c];
      if (bias) a += bias[c];
      dx[row * cols + c] = act_bwd1(act, g[row * cols + c], a);
    }
}

// Small-cols fallback for the bias gradient (cols < 32): one warp per column.
__global__ void __launch_bounds__(256)
narrow_colsum_kernel(const float* __restrict__ dxv, uint64_t rows, uint64_t cols,
                     float* __restrict__ dbias) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (uint64_t c = (uint64_t)blockIdx.x * 8 + warp; c < cols; c += (uint64_t)gridDim.x * 8) {
    float a = 0.0f;
    for (uint64_t r = lane; r < rows; r += 32) a += dxv[r * cols + c];
    a = warp_sum(a);
    if (lane == 0) dbias[c] = a;
  }
}

constexpr int kMseThreads = 256;

// diff = pred - target; partial sums of diff^2; dpred = k * (2 * diff).
// One chunk of kMseChunk elements per CTA on a full grid (the kernel writes as
// much as half of what it reads: see grid_full), four pairs of 16-byte loads
// in flight per thread, one partial per CTA added up in index order afterwards.
constexpr uint64_t kMseChunk = (uint64_t)kMseThreads * 4 * 8;  // elements per CTA
__global__ void __launch_bounds__(kMseThreads)
mse_partial_kernel(const float* __restrict__ pred, const float* __restrict__ target, uint64_t n,
                   int vec, float k, float* __restrict__ dpred, float* __restrict__ part) {
  pdl_trigger();  // the dependent finalize launch may become resident while this grid runs
  __shared__ float red[32];
  float a0 = 0, a1 = 0, a2 = 0, a3 = 0;
  const uint64_t lo = (uint64_t)blockIdx.x * kMseChunk;
  const uint64_t hi = lo + kMseChunk < n ? lo + kMseChunk : n;
  if (vec) {
    const float* p0 = pred + lo;
    const float* t0 = target + lo;
    float* d0 = dpred ? dpred + lo : nullptr;
    const uint64_t nv = (hi - lo) / 4;
    auto one = [&](uint64_t i, float4 p, float4 t) {
      const float4 d = make_float4(p.x - t.x, p.y - t.y, p.z - t.z, p.w - t.w);
      a0 += d.x * d.x; a1 += d.y * d.y; a2 += d.z * d.z; a3 += d.w * d.w;
      if (d0) st_stream4(d0 + i * 4, make_float4(k * (2.0f * d.x), k * (2.0f * d.y), k * (2.0f * d.z), k * (2.0f * d.w)));
    };
    uint64_t i = threadIdx.x;
    for (; i + 3 * kMseThreads < nv; i += 4 * kMseThreads) {
      const float4 pa = ld_stream4(p0 + i * 4), ta = ld_stream4(t0 + i * 4);
      const float4 pb = ld_stream4(p0 + (i + kMseThreads) * 4), tb = ld_stream4(t0 + (i + kMseThreads) * 4);
      const float4 pc = ld_stream4(p0 + (i + 2 * kMseThreads) * 4), tc = ld_stream4(t0 + (i + 2 * kMseThreads) * 4);
      const float4 pd = ld_stream4(p0 + (i + 3 * kMseThreads) * 4), td = ld_stream4(t0 + (i + 3 * kMseThreads) * 4);
      one(i, pa, ta); one(i + kMseThreads, pb, tb); one(i + 2 * kMseThreads, pc, tc); one(i + 3 * kMseThreads, pd, td);
    }
    for (; i < nv; i += kMseThreads) one(i, ld_stream4(p0 + i * 4), ld_stream4(t0 + i * 4));
    for (uint64_t j = lo + nv * 4 + threadIdx.x; j < hi; j += kMseThreads) {  // scalar tail of the last chunk
      const float d = pred[j] - target[j];
      a0 += d * d;
      if (dpred) dpred[j] = k * (2.0f * d);
    }
  } else {
    for (uint64_t i = lo + threadIdx.x; i < hi; i += kMseThreads) {
      const float d = pred[i] - target[i];
      a0 += d * d;
      if (dpred) dpred[i] = k * (2.0f * d);
    }
  }
  const float s = block_sum((a0 + a1) + (a2 + a3), red);
  if (threadIdx.x == 0) part[blockIdx.x] = s;
}

__global__ void __launch_bounds__(256)
mse_final_kernel(const float* __restrict__ part, uint32_t parts, float n, float* __restrict__ loss) {
  pdl_wait();  // launched as a dependent (launch_pdl) of the kernel that writes its input
  pdl_trigger();
  __shared__ float red[32];
  float a = 0.0f;
  for (uint32_t i = threadIdx.x; i < parts; i += 256) a += part[i];
  const float s = block_sum(a, red);
  if (threadIdx.x == 0) loss[0] = s / n;
}

}  // namespace fb
extern "C" uint64_t fb_mse_parts(uint64_t n) { return (n + fb::kMseChunk - 1) / fb::kMseChunk; }
namespace fb {

}  // namespace fb

using namespace fb;

extern "C" {

int fb_bias_act_bwd(fb_stream_t stream, const float* g, const float* x, const float* bias, int relu,
                    uint64_t rows, uint64_t cols, float* dx, float* dbias, void* workspace,
                    uint64_t workspace_bytes) {
  const char* name = "fb_bias_act_bwd";
  if (relu < 0 || relu > 3) return fail(FB_ERR_INVALID_ARG, "%s: unknown activation %d", name, relu);
  uint64_t n;
  if (mul_overflows(rows, cols, &n) || n > (UINT64_MAX >> 3)) return fail(FB_ERR_INVALID_SHAPE, "%s: rows * cols overflows", name);
  if (cols == 0) return FB_OK;
  if (rows == 0) return dbias ? fb_fill(stream, dbias, 0.0f, cols) : FB_OK;
  if (!g || (relu && !x)) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  if (!dx && !dbias) return FB_OK;
  if (!relu && !dx) dx = const_cast<float*>(g);  // nothing to write: dx == g suppresses the store
  if (!dbias) {
    if (!relu) return dx == g ? FB_OK : fb_copy(stream, dx, g, n);
    bias_act_bwd_nosum_kernel<<<grid_full(rows), 256, 0, stream>>>(g, x, bias, relu, rows, cols, dx);
    FB_LAUNCHED(name);
    return FB_OK;
  }
  if (cols < 32) {
    // Narrow matrices: masked copy, then a warp per column.
    const float* src = g;
    if (relu) {
      if (!dx) return fail(FB_ERR_INVALID_ARG, "%s: dx is required when cols < 32 and relu is set", name);
      bias_act_bwd_nosum_kernel<<<grid_full(rows), 256, 0, stream>>>(g, x, bias, relu, rows, cols, dx);
      FB_LAUNCHED(name);
      src = dx;
    } else if (dx != g) {
      if (int rc = fb_copy(stream, dx, g, n)) return rc;
    }
    narrow_colsum_kernel<<<(unsigned)((cols + 7) / 8), 256, 0, stream>>>(src, rows, cols, dbias);
    FB_LAUNCHED(name);
    return FB_OK;
  }
  BiasActBwdSrc src{g, x, bias, dx, cols, relu};
  const bool al = aligned16(g) && (!relu || aligned16(x)) && (!bias || aligned16(bias)) && (!dx || aligned16(dx));
  return run_col_sum<1>(stream, src, 1, rows, cols, al, dbias, nullptr, 1.0f, workspace, workspace_bytes, name);
}

int fb_mse_fwd_bwd(fb_stream_t stream, const float* pred, const float* target, uint64_t n,
                   float grad_scale, float* loss, float* dpred, void* workspace,
                   uint64_t workspace_bytes) {
  const char* name = "fb_mse_fwd_bwd";
  if (!loss) return fail(FB_ERR_INVALID_ARG, "%s: null loss", name);
  if (n == 0) return fb_reduce(stream, FB_RED_MEAN, nullptr, 0, loss, nullptr, 0);
  if (!pred || !target) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  const uint64_t parts64 = fb_mse_parts(n);
  if (parts64 > 0x7fffffffull) return fail(FB_ERR_INVALID_SHAPE, "%s: too many elements", name);
  const uint32_t parts = (uint32_t)parts64;
  if (!workspace || workspace_bytes < (uint64_t)parts * sizeof(float))
    return fail(FB_ERR_WORKSPACE, "%s: needs %llu bytes of scratch", name, (unsigned long long)((uint64_t)parts * sizeof(float)));
  float* part = static_cast<float*>(workspace);
  const int vec = aligned16(pred) && aligned16(target) && (!dpred || aligned16(dpred));
  // mean's backward multiplies by (1/n) (ops.rs:176-183); square's by 2*diff (square.rs:19).
  const float k = grad_scale * (1.0f / (float)n);
  mse_partial_kernel<<<parts, kMseThreads, 0, stream>>>(pred, target, n, vec, k, dpred, part);
  FB_LAUNCHED(name);
  FB_CUDA(launch_pdl(mse_final_kernel, dim3(1), dim3(256), 0, stream, (const float*)part, parts, (float)n, loss));
  FB_LAUNCHED(name);
  return FB_OK;
}

}  // extern "C"
