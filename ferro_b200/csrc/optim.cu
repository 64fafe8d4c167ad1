// Fused optimizer updates: Adam / AdamW and SGD with momentum, single tensor
// and whole-parameter-list ("multi") forms.
//
// Roofline: HBM.  Algorithmic bytes per parameter element: Adam 28 (read p,
// m, v, g; write p, m, v), SGD-momentum 20 (read p, v, g; write p, v).
//
// The arithmetic is ferro's host loop, one rounding per operation in the same
// order (crates/ferro-core/src/dispatch.rs:477-503); the translation unit is
// built with -fmad=false and IEEE division / square root, so results are
// bitwise equal to that loop, which is the bar ferro's own device tests set
// (crates/ferro-cuda/src/lib.rs:2214-2257).
#include "common.cuh"

namespace fb {

constexpr int kOptThreads = 256;

struct AdamConsts {
  float lr, beta1, beta2, nb1, nb2, bc1, bc2, eps, wd;
};

__device__ __forceinline__ void adam1(const AdamConsts& c, float& p, float& m, float& v, float g) {
  m = m * c.beta1 + g * c.nb1;
  v = v * c.beta2 + (g * g) * c.nb2;
  const float m_hat = m / c.bc1;
  const float denom = sqrtf(v / c.bc2);
  float upd = m_hat / (denom + c.eps);
  if (c.wd != 0.0f) upd += c.wd * p;
  p -= upd * c.lr;
}

__device__ __forceinline__ void sgd1(float lr, float mu, int nesterov, float& p, float& v, float g) {
  v = v * mu + g;
  const float d = nesterov ? v * mu + g : v;
  p -= d * lr;
}

// One tensor's range [0, n), processed by `nblocks` logical blocks of which
// this CTA is number `blk`.  VEC = 4 requires 16-byte aligned p, m, v, g.
template <int VEC, bool ADAM>
__device__ __forceinline__ void update_range(float* __restrict__ p, float* __restrict__ m,
                                             float* __restrict__ v, const float* __restrict__ g,
                                             uint64_t n, uint64_t blk, uint64_t nblocks,
                                             const AdamConsts& c, float mu, int nesterov,
                                             float g_scale, float g_scale2 = 1.0f) {
  if constexpr (VEC == 4) {
    const uint64_t nv = n / 4;
    for (uint64_t i = blk * kOptThreads + threadIdx.x; i < nv; i += nblocks * kOptThreads) {
      float4 pp = *reinterpret_cast<const float4*>(p + i * 4);
      float4 gg = ld_stream4(g + i * 4);
      float4 vv = *reinterpret_cast<const float4*>((ADAM ? v : m) + i * 4);
      gg.x = gg.x * g_scale * g_scale2; gg.y = gg.y * g_scale * g_scale2;
      gg.z = gg.z * g_scale * g_scale2; gg.w = gg.w * g_scale * g_scale2;
      if constexpr (ADAM) {
        float4 mm = *reinterpret_cast<const float4*>(m + i * 4);
        adam1(c, pp.x, mm.x, vv.x, gg.x);
        adam1(c, pp.y, mm.y, vv.y, gg.y);
        adam1(c, pp.z, mm.z, vv.z, gg.z);
        adam1(c, pp.w, mm.w, vv.w, gg.w);
        *reinterpret_cast<float4*>(m + i * 4) = mm;
        *reinterpret_cast<float4*>(v + i * 4) = vv;
      } else {
        sgd1(c.lr, mu, nesterov, pp.x, vv.x, gg.x);
        sgd1(c.lr, mu, nesterov, pp.y, vv.y, gg.y);
        sgd1(c.lr, mu, nesterov, pp.z, vv.z, gg.z);
        sgd1(c.lr, mu, nesterov, pp.w, vv.w, gg.w);
        *reinterpret_cast<float4*>(m + i * 4) = vv;
      }
      *reinterpret_cast<float4*>(p + i * 4) = pp;
    }
    // Scalar tail by logical block 0.
    if (blk == 0 && threadIdx.x < n - nv * 4) {
      const uint64_t i = nv * 4 + threadIdx.x;
      float pp = p[i], gg = g[i] * g_scale * g_scale2;
      if constexpr (ADAM) {
        float mm = m[i], vv = v[i];
        adam1(c, pp, mm, vv, gg);
        m[i] = mm;
        v[i] = vv;
      } else {
        float vv = m[i];
        sgd1(c.lr, mu, nesterov, pp, vv, gg);
        m[i] = vv;
      }
      p[i] = pp;
    }
  } else {
    for (uint64_t i = blk * kOptThreads + threadIdx.x; i < n; i += nblocks * kOptThreads) {
      float pp = p[i], gg = g[i] * g_scale * g_scale2;
      if constexpr (ADAM) {
        float mm = m[i], vv = v[i];
        adam1(c, pp, mm, vv, gg);
        m[i] = mm;
        v[i] = vv;
      } else {
        float vv = m[i];
        sgd1(c.lr, mu, nesterov, pp, vv, gg);
        m[i] = vv;
      }
      p[i] = pp;
    }
  }
}

// Single tensor.  `t` (optional) is the capturable timestep buffer
// [step, bc1, bc2]; when given, bc1 / bc2 come from it.
template <int VEC, bool ADAM>
__global__ void __launch_bounds__(kOptThreads)
step_kernel(float* p, float* m, float* v, const float* g, const float* t, uint64_t n, AdamConsts c,
            float mu, int nesterov) {
  if (t) {
    c.bc1 = t[1];
    c.bc2 = t[2];
  }
  update_range<VEC, ADAM>(p, m, v, g, n, blockIdx.x, gridDim.x, c, mu, nesterov, 1.0f);
}

// Whole parameter list.  Work is cut into chunks of kChunk elements; chunk k
// belongs to the tensor whose chunk range contains it (linear scan over the
// table: parameter lists are tens to hundreds of tensors).
constexpr uint64_t kChunk = (uint64_t)kOptThreads * 4 * 8;

template <bool ADAM>
__global__ void __launch_bounds__(kOptThreads)
multi_step_kernel(const fb_tensor_quad* __restrict__ table, int n_tensors, uint64_t total_chunks,
                  AdamConsts c, float mu, int nesterov, float g_scale, const float* __restrict__ clip) {
  // Gradient clipping: the factor is a device scalar a previous kernel wrote
  // (fb_clip_scale), folded into the gradient scale; x * 1 is exact, so the
  // unclipped update is unchanged.  Two factors that are both != 1 (a mean
  // over ranks and a clip) are applied in ferro's order, one rounding each.
  const float clip_scale = clip ? __ldg(clip) : 1.0f;
  for (uint64_t chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    uint64_t first = 0;
    int ti = 0;
    uint64_t nchunks = 0;
    for (; ti < n_tensors; ++ti) {
      nchunks = (table[ti].n + kChunk - 1) / kChunk;
      if (chunk < first + nchunks) break;
      first += nchunks;
    }
    if (ti >= n_tensors) return;
    const fb_tensor_quad q = table[ti];
    const uint64_t local = chunk - first;
    const uint64_t lo = local * kChunk;
    const uint64_t len = (q.n - lo < kChunk) ? q.n - lo : kChunk;
    float* p = q.p + lo;
    float* m = q.m + lo;
    float* v = ADAM ? q.v + lo : nullptr;
    const float* g = q.g + lo;
    const bool vec = (((uintptr_t)p | (uintptr_t)m | (uintptr_t)g | (ADAM ? (uintptr_t)v : 0)) & 15) == 0;
    if (vec)
      update_range<4, ADAM>(p, m, v, g, len, 0, 1, c, mu, nesterov, g_scale, clip_scale);
    else
      update_range<1, ADAM>(p, m, v, g, len, 0, 1, c, mu, nesterov, g_scale, clip_scale);
  }
}

// t = [step, bc1, bc2]: step += 1; bc = 1 - beta^step with the host's
// square-and-multiply powi (optim.rs:719-721), so a captured step stays
// bitwise equal to the eager one.
__device__ float powi_f32(float a, int b) {
  float r = 1.0f;
  while (true) {
    if (b & 1) r *= a;
    b /= 2;
    if (b == 0) break;
    a *= a;
  }
  return r;
}
__global__ void scalar_increment_kernel(float* t, float beta1, float beta2) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const float step = t[0] + 1.0f;
    t[0] = step;
    const int k = (int)step;
    t[1] = 1.0f - powi_f32(beta1, k);
    t[2] = 1.0f - powi_f32(beta2, k);
  }
}

// ---- global gradient norm (optim.rs:1395-1425) ---------------------------
// Sum of squares of every gradient in the table, each scaled by g_scale first.
// A fixed grid of kNormCtas CTAs takes the chunks round-robin; a thread keeps
// four accumulators, a CTA adds its threads in a fixed tree and writes one
// partial, the last kernel adds the partials in index order: the result
// depends on the shapes only.
constexpr int kNormCtas = 1184;
__global__ void __launch_bounds__(kOptThreads)
sumsq_multi_kernel(const fb_tensor_quad* __restrict__ table, int n_tensors, uint64_t total_chunks,
                   float g_scale, float* __restrict__ partial) {
  pdl_trigger();  // the dependent finalize launch may become resident while this grid runs
  __shared__ float red[32];
  float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
  for (uint64_t chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    uint64_t first = 0, nchunks = 0;
    int ti = 0;
    for (; ti < n_tensors; ++ti) {
      nchunks = (table[ti].n + kChunk - 1) / kChunk;
      if (chunk < first + nchunks) break;
      first += nchunks;
    }
    if (ti >= n_tensors) break;
    const uint64_t lo = (chunk - first) * kChunk;
    const uint64_t len = (table[ti].n - lo < kChunk) ? table[ti].n - lo : kChunk;
    const float* g = table[ti].g + lo;
    if ((((uintptr_t)g) & 15) == 0) {
      const uint64_t nv = len / 4;
      for (uint64_t i = threadIdx.x; i < nv; i += kOptThreads) {
        float4 t = ld_stream4(g + i * 4);
        t.x *= g_scale; t.y *= g_scale; t.z *= g_scale; t.w *= g_scale;
        a0 += t.x * t.x; a1 += t.y * t.y; a2 += t.z * t.z; a3 += t.w * t.w;
      }
      for (uint64_t i = nv * 4 + threadIdx.x; i < len; i += kOptThreads) {
        const float t = g[i] * g_scale;
        a0 += t * t;
      }
    } else {
      for (uint64_t i = threadIdx.x; i < len; i += kOptThreads) {
        const float t = g[i] * g_scale;
        a0 += t * t;
      }
    }
  }
  const float s = block_sum((a0 + a1) + (a2 + a3), red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void __launch_bounds__(kOptThreads)
sumsq_final_kernel(const float* __restrict__ partial, int n, float* __restrict__ out) {
  pdl_wait();  // launched as a dependent (launch_pdl) of the kernel that writes its input
  pdl_trigger();
  __shared__ float red[32];
  float a = 0.0f;
  for (int i = threadIdx.x; i < n; i += kOptThreads) a += partial[i];
  a = block_sum(a, red);
  if (threadIdx.x == 0) *out = a;
}
// clip_scale (optim.rs:1412-1425): max / norm when the norm exceeds max (and is
// not zero), else 1.  NaN norms compare false and leave the gradients alone.
__global__ void clip_scale_kernel(const float* __restrict__ sumsq, float max_norm, float* norm_out,
                                  float* scale_out) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const float norm = sqrtf(*sumsq);
    if (norm_out) *norm_out = norm;
    *scale_out = (norm > max_norm && norm > 0.0f) ? max_norm / norm : 1.0f;
  }
}

static AdamConsts consts_of(const fb_adamw_hparams& hp) {
  return AdamConsts{hp.lr, hp.beta1, hp.beta2, 1.0f - hp.beta1, 1.0f - hp.beta2,
                    hp.bc1, hp.bc2, hp.eps, hp.weight_decay};
}

static bool overlap(const void* a, const void* b, uint64_t n) {
  const uintptr_t x = (uintptr_t)a, y = (uintptr_t)b, len = n * sizeof(float);
  return x < y + len && y < x + len;
}

template <bool ADAM>
static int launch_step(cudaStream_t stream, const char* name, float* p, float* m, float* v,
                       const float* g, const float* t, uint64_t n, const AdamConsts& c, float mu,
                       int nesterov) {
  if (n == 0) return FB_OK;
  if (!p || !m || !g || (ADAM && !v)) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  // Distinct storages, as ferro's check_dst demands (inplace.rs:539-561).
  if (overlap(p, m, n) || overlap(p, g, n) || overlap(m, g, n) ||
      (ADAM && (overlap(p, v, n) || overlap(m, v, n) || overlap(v, g, n))))
    return fail(FB_ERR_INVALID_ARG, "%s: operands must not overlap", name);
  const bool vec = aligned16(p) && aligned16(m) && aligned16(g) && (!ADAM || aligned16(v));
  const uint64_t per_cta = (uint64_t)kOptThreads * (vec ? 4 : 1) * 4;
  const unsigned grid = grid_full((n + per_cta - 1) / per_cta);
  if (vec)
    step_kernel<4, ADAM><<<grid, kOptThreads, 0, stream>>>(p, m, v, g, t, n, c, mu, nesterov);
  else
    step_kernel<1, ADAM><<<grid, kOptThreads, 0, stream>>>(p, m, v, g, t, n, c, mu, nesterov);
  FB_LAUNCHED(name);
  return FB_OK;
}

}  // namespace fb

using namespace fb;

extern "C" {

int fb_sgd_step(fb_stream_t stream, float* p, float* v, const float* g, uint64_t n, float lr,
                float momentum, int nesterov) {
  AdamConsts c{};
  c.lr = lr;
  return launch_step<false>(stream, "fb_sgd_step", p, v, nullptr, g, nullptr, n, c, momentum, nesterov ? 1 : 0);
}

int fb_adamw_step(fb_stream_t stream, float* p, float* m, float* v, const float* g, uint64_t n,
                  fb_adamw_hparams hp) {
  return launch_step<true>(stream, "fb_adamw_step", p, m, v, g, nullptr, n, consts_of(hp), 0.0f, 0);
}

int fb_adamw_step_capturable(fb_stream_t stream, float* p, float* m, float* v, const float* g,
                             const float* t, uint64_t n, float lr, float beta1, float beta2,
                             float eps, float weight_decay) {
  if (!t) return fail(FB_ERR_INVALID_ARG, "fb_adamw_step_capturable: null timestep buffer");
  fb_adamw_hparams hp{lr, beta1, beta2, 1.0f, 1.0f, eps, weight_decay};
  return launch_step<true>(stream, "fb_adamw_step_capturable", p, m, v, g, t, n, consts_of(hp), 0.0f, 0);
}

int fb_scalar_increment(fb_stream_t stream, float* t, float beta1, float beta2) {
  if (!t) return fail(FB_ERR_INVALID_ARG, "fb_scalar_increment: null timestep buffer");
  scalar_increment_kernel<<<1, 1, 0, stream>>>(t, beta1, beta2);
  FB_LAUNCHED("fb_scalar_increment");
  return FB_OK;
}

int fb_adamw_multi_clipped(fb_stream_t stream, const fb_tensor_quad* table, int n_tensors,
                           uint64_t total_elems, fb_adamw_hparams hp, float g_scale,
                           const float* clip_scale) {
  if (n_tensors < 0) return fail(FB_ERR_INVALID_ARG, "fb_adamw_multi: negative tensor count");
  if (n_tensors == 0 || total_elems == 0) return FB_OK;
  if (!table) return fail(FB_ERR_INVALID_ARG, "fb_adamw_multi: null table");
  // Every tensor adds at most one partly filled chunk.
  const uint64_t chunks = total_elems / kChunk + (uint64_t)n_tensors;
  multi_step_kernel<true><<<grid_full(chunks), kOptThreads, 0, stream>>>(table, n_tensors, chunks, consts_of(hp),
                                                                          0.0f, 0, g_scale, clip_scale);
  FB_LAUNCHED("fb_adamw_multi");
  return FB_OK;
}
int fb_adamw_multi(fb_stream_t stream, const fb_tensor_quad* table, int n_tensors,
                   uint64_t total_elems, fb_adamw_hparams hp, float g_scale) {
  return fb_adamw_multi_clipped(stream, table, n_tensors, total_elems, hp, g_scale, nullptr);
}

uint64_t fb_grad_norm_workspace_bytes(void) { return (uint64_t)kNormCtas * sizeof(float); }

int fb_grad_sumsq_multi(fb_stream_t stream, const fb_tensor_quad* table, int n_tensors,
                        uint64_t total_elems, float g_scale, float* sumsq, void* workspace,
                        uint64_t workspace_bytes) {
  if (n_tensors < 0) return fail(FB_ERR_INVALID_ARG, "fb_grad_sumsq_multi: negative tensor count");
  if (!sumsq) return fail(FB_ERR_INVALID_ARG, "fb_grad_sumsq_multi: null output");
  if (n_tensors == 0 || total_elems == 0) return fb_fill(stream, sumsq, 0.0f, 1);
  if (!table) return fail(FB_ERR_INVALID_ARG, "fb_grad_sumsq_multi: null table");
  if (!workspace || workspace_bytes < fb_grad_norm_workspace_bytes())
    return fail(FB_ERR_WORKSPACE, "fb_grad_sumsq_multi: needs %llu bytes of scratch",
                (unsigned long long)fb_grad_norm_workspace_bytes());
  const uint64_t chunks = total_elems / kChunk + (uint64_t)n_tensors;
  const int grid = (int)(chunks < (uint64_t)kNormCtas ? chunks : (uint64_t)kNormCtas);
  float* partial = static_cast<float*>(workspace);
  sumsq_multi_kernel<<<grid, kOptThreads, 0, stream>>>(table, n_tensors, chunks, g_scale, partial);
  FB_LAUNCHED("fb_grad_sumsq_multi");
  FB_CUDA(launch_pdl(sumsq_final_kernel, dim3(1), dim3(kOptThreads), 0, stream, (const float*)partial, (int)grid, sumsq));
  FB_LAUNCHED("fb_grad_sumsq_multi");
  return FB_OK;
}

int fb_clip_scale(fb_stream_t stream, const float* sumsq, float max_norm, float* norm_out,
                  float* scale_out) {
  if (!sumsq || !scale_out) return fail(FB_ERR_INVALID_ARG, "fb_clip_scale: null buffer");
  clip_scale_kernel<<<1, 32, 0, stream>>>(sumsq, max_norm, norm_out, scale_out);
  FB_LAUNCHED("fb_clip_scale");
  return FB_OK;
}

int fb_sgd_multi_clipped(fb_stream_t stream, const fb_tensor_quad* table, int n_tensors,
                         uint64_t total_elems, float lr, float momentum, int nesterov, float g_scale,
                         const float* clip_scale) {
  if (n_tensors < 0) return fail(FB_ERR_INVALID_ARG, "fb_sgd_multi: negative tensor count");
  if (n_tensors == 0 || total_elems == 0) return FB_OK;
  if (!table) return fail(FB_ERR_INVALID_ARG, "fb_sgd_multi: null table");
  AdamConsts c{};
  c.lr = lr;
  const uint64_t chunks = total_elems / kChunk + (uint64_t)n_tensors;
  multi_step_kernel<false><<<grid_full(chunks), kOptThreads, 0, stream>>>(table, n_tensors, chunks, c, momentum,
                                                                           nesterov ? 1 : 0, g_scale, clip_scale);
  FB_LAUNCHED("fb_sgd_multi");
  return FB_OK;
}
int fb_sgd_multi(fb_stream_t stream, const fb_tensor_quad* table, int n_tensors,
                 uint64_t total_elems, float lr, float momentum, int nesterov, float g_scale) {
  return fb_sgd_multi_clipped(stream, table, n_tensors, total_elems, lr, momentum, nesterov, g_scale, nullptr);
}

}  // extern "C"
