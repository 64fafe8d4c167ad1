/* TEST INFRASTRUCTURE - not part of the shipped library.
 *
 * CPU restatement of the ferro code the GPU hot path must agree with: the
 * reference `CpuBackend` math, the fixed pairwise reduction tree, the host
 * loops for softmax / log_softmax / LayerNorm / argmax, the cross-entropy
 * composition, the Adam / SGD loops, the DDP mean and the `Rng` generator.
 * Every function names the ferro file:line it follows (paths are relative to
 * the ferro repository root).  Operation order and rounding follow the Rust
 * source one for one; build with -ffp-contract=off so no multiply-add is
 * contracted (Rust never contracts).  Rust's f32::exp/ln/tanh/powf/cos lower
 * to the platform libm, i.e. the very expf/logf/tanhf/powf/cosf called here.
 *
 * Parity status: pinned.  tests/test_oracle_pins.py checks this file against
 * the known-answer tests and golden tables of ferro's own test-suite.
 *
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may
 * load this library.  The `fo_*_mt` entry points are the same loops split
 * over OpenMP threads by row / by block, with the per-row operation order
 * unchanged, for the timed CPU baseline.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../include/ferro_b200_kinds.h"

#define FO_API __attribute__((visibility("default")))

FO_API int fo_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ferro's CPU path threads over available_parallelism() (workers.rs:75-78),
 * whatever OMP_NUM_THREADS says: launchers such as torchrun export
 * OMP_NUM_THREADS=1, which would turn the timed baseline into a 1-thread run. */
FO_API void fo_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------ Rng */
/* crates/ferro-core/src/rng.rs:12-70 */
typedef struct { uint64_t s0, s1; } fo_rng;

static uint64_t fo_splitmix(uint64_t *z) {
  *z += 0x9E3779B97F4A7C15ull;
  uint64_t x = *z;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

FO_API void fo_rng_seed(fo_rng *r, uint64_t seed) { /* rng.rs:12-26 */
  uint64_t z = seed + 0x9E3779B97F4A7C15ull;
  r->s0 = fo_splitmix(&z) | 1ull;
  r->s1 = fo_splitmix(&z) | 1ull;
}

static inline uint64_t fo_rng_next(fo_rng *r) { /* rng.rs:35-44 */
  uint64_t x = r->s0;
  const uint64_t y = r->s1;
  r->s0 = y;
  x ^= x << 23;
  x ^= x >> 17;
  x ^= y ^ (y >> 26);
  r->s1 = x;
  return x + y;
}

static inline float fo_rng_uniform1(fo_rng *r) { /* rng.rs:47-50 */
  return (float)(fo_rng_next(r) >> 40) / 16777216.0f;
}

static inline float fo_rng_normal1(fo_rng *r) { /* rng.rs:65-70 */
  float u1 = fo_rng_uniform1(r);
  u1 = fmaxf(u1, 1e-9f);
  const float u2 = fo_rng_uniform1(r);
  const float rad = sqrtf(-2.0f * logf(u1));
  return rad * cosf(6.28318530717958647692f * u2);
}

FO_API float fo_rng_uniform(fo_rng *r) { return fo_rng_uniform1(r); }
FO_API float fo_rng_normal(fo_rng *r) { return fo_rng_normal1(r); }

/* out[i] = shift + scale * draw, row-major, one draw after another
 * (Tensor::randn fill order, crates/ferro-core/src/tensor.rs:365-372). */
FO_API void fo_rng_fill_normal(fo_rng *r, float *out, uint64_t n, float scale, float shift) {
  for (uint64_t i = 0; i < n; ++i) out[i] = shift + scale * fo_rng_normal1(r);
}
FO_API void fo_rng_fill_uniform(fo_rng *r, float *out, uint64_t n, float scale, float shift) {
  for (uint64_t i = 0; i < n; ++i) out[i] = shift + scale * fo_rng_uniform1(r);
}
/* He initialisation: normal() * sqrt(2 / fan_in), crates/ferro-core/src/nn.rs:138-146 */
FO_API void fo_rng_fill_he(fo_rng *r, float *out, uint64_t n, uint64_t fan_in) {
  const float s = sqrtf(2.0f / (float)fan_in);
  for (uint64_t i = 0; i < n; ++i) out[i] = fo_rng_normal1(r) * s;
}
/* LayerNorm benchmark rows: one uniform row scale drawn before each row. */
FO_API void fo_rng_fill_rowscaled_normal(fo_rng *r, float *out, uint64_t rows, uint64_t cols,
                                         float lo, float span) {
  for (uint64_t i = 0; i < rows; ++i) {
    const float sc = lo + span * fo_rng_uniform1(r);
    for (uint64_t j = 0; j < cols; ++j) out[i * cols + j] = fo_rng_normal1(r) * sc;
  }
}
/* Class ids floor(uniform * classes) as i64 (ferro's Rng has no integer draw). */
FO_API void fo_rng_fill_targets(fo_rng *r, int64_t *out, uint64_t n, uint64_t classes) {
  for (uint64_t i = 0; i < n; ++i) {
    int64_t t = (int64_t)floorf(fo_rng_uniform1(r) * (float)classes);
    if (t >= (int64_t)classes) t = (int64_t)classes - 1;
    out[i] = t;
  }
}

/* ----------------------------------------------------- elementwise math */
/* crates/ferro-core/src/dispatch.rs:51-64 */
static float fo_erf_f32(float x) {
  const double A1 = 0.254829592, A2 = -0.284496736, A3 = 1.421413741, A4 = -1.453152027,
               A5 = 1.061405429, P = 0.3275911;
  const double xd = (double)x;
  const double sign = xd < 0.0 ? -1.0 : 1.0;
  const double ax = fabs(xd);
  const double t = 1.0 / (1.0 + P * ax);
  const double poly = ((((A5 * t + A4) * t + A3) * t + A2) * t + A1) * t;
  return (float)(sign * (1.0 - poly * exp(-ax * ax)));
}

/* The exponent special cases of UnaryKind::Powf, dispatch.rs:688 */
static inline float fo_powf_kind(float v, float p) {
  if (p == 0.5f) return sqrtf(v);
  if (p == -0.5f) return 1.0f / sqrtf(v);
  if (p == -1.0f) return 1.0f / v;
  if (p == -2.0f) return 1.0f / (v * v);
  if (p == 2.0f) return v * v;
  if (p == 3.0f) return (v * v) * v;
  return powf(v, p);
}

/* CpuBackend::unary, dispatch.rs:671-725 */
static inline float fo_unary1(int kind, float p0, float p1, float v) {
  switch (kind) {
    case FB_UN_NEG: return -v;
    case FB_UN_RELU: return (v > 0.0f || isnan(v)) ? v : 0.0f;
    case FB_UN_EXP: return expf(v);
    case FB_UN_SIGMOID: return 1.0f / (1.0f + expf(-v));
    case FB_UN_TANH: return tanhf(v);
    case FB_UN_SQRT: return sqrtf(v);
    case FB_UN_ABS: return fabsf(v);
    case FB_UN_SIGN: return v > 0.0f ? 1.0f : (v < 0.0f ? -1.0f : 0.0f);
    case FB_UN_LOG: return logf(v);
    case FB_UN_POWF: return fo_powf_kind(v, p0);
    case FB_UN_CLAMP: {
      if (isnan(v)) return v;
      if (isnan(p0) || isnan(p1)) return NAN;
      const float lower = v < p0 ? p0 : v;
      return lower > p1 ? p1 : lower;
    }
    case FB_UN_GTZ: return !(v <= 0.0f) ? 1.0f : 0.0f;
    case FB_UN_GELU: {
      const float u = 0.7978846f * (v + 0.044715f * v * v * v);
      return 0.5f * v * (1.0f + tanhf(u));
    }
    case FB_UN_GELU_ERF: return 0.5f * v * (1.0f + fo_erf_f32(v * 0.70710678118654752440f));
    case FB_UN_GELU_ERF_GRAD:
      return 0.5f * (1.0f + fo_erf_f32(v * 0.70710678118654752440f)) +
             v * expf(-0.5f * v * v) * 0.39894228f;
    case FB_UN_SILU: return v / (1.0f + expf(-v));
    default: return NAN;
  }
}

/* binary_scalar_fn, dispatch.rs:79-87, plus the backward closures of
 * ops_ext/{tanh,sqrt,abs,log,powf,clamp}.rs and activation_backward.rs:22-25 */
static inline float fo_binary1(int kind, float p0, float p1, float x, float y) {
  switch (kind) {
    case FB_BIN_ADD: return x + y;
    case FB_BIN_SUB: return x - y;
    case FB_BIN_MUL: return x * y;
    case FB_BIN_DIV: return x / y;
    case FB_BIN_RELU_BACKWARD: return y <= 0.0f ? 0.0f : x;
    case FB_BIN_TANH_BWD: return x * fmaf(-y, y, 1.0f);          /* activation_backward.rs:24 */
    case FB_BIN_SIGMOID_BWD: return (x * (1.0f - y)) * y;         /* activation_backward.rs:24 */
    case FB_BIN_SQRT_BWD: return x / (2.0f * y);                  /* sqrt.rs:21 */
    case FB_BIN_ABS_BWD: return x * (y > 0.0f ? 1.0f : (y < 0.0f ? -1.0f : 0.0f)); /* abs.rs:14 */
    case FB_BIN_LOG_BWD: return x / y;                            /* log.rs:15 */
    case FB_BIN_POWF_BWD: {                                       /* powf.rs:48-56 */
      if (p0 == 0.0f) return 0.0f;
      return x * (p0 * fo_powf_kind(y, p0 - 1.0f));
    }
    case FB_BIN_CLAMP_BWD: return (y >= p0 && y <= p1) ? x : 0.0f; /* clamp.rs:20-26 */
    default: return NAN;
  }
}

FO_API void fo_unary(int kind, float p0, float p1, const float *x, float *out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = fo_unary1(kind, p0, p1, x[i]);
}
FO_API void fo_unary_mt(int kind, float p0, float p1, const float *x, float *out, uint64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = fo_unary1(kind, p0, p1, x[i]);
}

FO_API void fo_binary(int kind, float p0, float p1, const float *a, const float *b, float *out,
                      uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = fo_binary1(kind, p0, p1, a[i], b[i]);
}
FO_API void fo_binary_mt(int kind, float p0, float p1, const float *a, const float *b, float *out,
                         uint64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = fo_binary1(kind, p0, p1, a[i], b[i]);
}

/* Strided binary over an output index space: out (row-major over `shape`)
 * = a[offa + sum idx*sa] kind b[offb + sum idx*sb].  With stride 0 on
 * expanded dims this is binary_bc_odometer (dispatch.rs:842-891); with
 * arbitrary element strides it is what ferro reaches after materialising a
 * view (tensor.rs:1692-1700). */
FO_API void fo_binary_strided(int kind, float p0, float p1, const float *a, const int64_t *sa,
                              int64_t offa, const float *b, const int64_t *sb, int64_t offb,
                              const uint64_t *shape, int rank, float *out) {
  uint64_t n = 1;
  for (int d = 0; d < rank; ++d) n *= shape[d];
  if (n == 0) return;
  uint64_t idx[16] = {0};
  for (uint64_t i = 0; i < n; ++i) {
    int64_t ia = offa, ib = offb;
    for (int d = 0; d < rank; ++d) {
      ia += (int64_t)idx[d] * sa[d];
      ib += (int64_t)idx[d] * sb[d];
    }
    out[i] = fo_binary1(kind, p0, p1, a[ia], b[ib]);
    for (int d = rank - 1; d >= 0; --d) {
      if (++idx[d] < shape[d]) break;
      idx[d] = 0;
    }
  }
}

/* Strided view -> row-major copy (what `materialize_dev` produces,
 * dispatch.rs:621-627; gather order of tensor.rs to_vec). */
FO_API void fo_materialize(const float *x, const int64_t *sx, int64_t off, const uint64_t *shape,
                           int rank, float *out) {
  uint64_t n = 1;
  for (int d = 0; d < rank; ++d) n *= shape[d];
  if (n == 0) return;
  uint64_t idx[16] = {0};
  for (uint64_t i = 0; i < n; ++i) {
    int64_t ix = off;
    for (int d = 0; d < rank; ++d) ix += (int64_t)idx[d] * sx[d];
    out[i] = x[ix];
    for (int d = rank - 1; d >= 0; --d) {
      if (++idx[d] < shape[d]) break;
      idx[d] = 0;
    }
  }
}

/* In-place kernels, dispatch.rs:448-472 */
FO_API void fo_affine_inplace(float *dst, float mul, float add, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) dst[i] = dst[i] * mul + add;
}
FO_API void fo_axpy_inplace(float alpha, float *dst, const float *src, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) dst[i] += alpha * src[i];
}

/* ------------------------------------------------------- pairwise tree */
/* crates/ferro-core/src/reduce.rs:16-71 */
#define FO_BASE 128
#define FO_LANES 8

static float fo_base_sum(const float *x, uint64_t offset, uint64_t n, uint64_t stride) {
  float acc[FO_LANES] = {0};
  const uint64_t chunks = n / FO_LANES;
  for (uint64_t c = 0; c < chunks; ++c)
    for (int l = 0; l < FO_LANES; ++l) acc[l] += x[offset + (c * FO_LANES + l) * stride];
  const float s01 = acc[0] + acc[1];
  const float s23 = acc[2] + acc[3];
  const float s45 = acc[4] + acc[5];
  const float s67 = acc[6] + acc[7];
  float sum = (s01 + s23) + (s45 + s67);
  for (uint64_t k = chunks * FO_LANES; k < n; ++k) sum += x[offset + k * stride];
  return sum;
}

static float fo_pairwise_strided(const float *x, uint64_t offset, uint64_t n, uint64_t stride) {
  if (n <= FO_BASE) return fo_base_sum(x, offset, n, stride);
  const uint64_t half = n / 2;
  const float left = fo_pairwise_strided(x, offset, half, stride);
  const float right = fo_pairwise_strided(x, offset + half * stride, n - half, stride);
  return left + right;
}

FO_API float fo_pairwise_sum_strided(const float *x, uint64_t offset, uint64_t n, uint64_t stride) {
  return fo_pairwise_strided(x, offset, n, stride);
}
FO_API float fo_pairwise_sum(const float *x, uint64_t n) { return fo_pairwise_strided(x, 0, n, 1); }

/* Same tree, the two top-level halves of each split handed to OpenMP tasks:
 * identical additions in identical order, any thread count. */
static float fo_pairwise_task(const float *x, uint64_t offset, uint64_t n, uint64_t stride) {
  if (n <= (1u << 16)) return fo_pairwise_strided(x, offset, n, stride);
  const uint64_t half = n / 2;
  float left, right;
#pragma omp task shared(left)
  left = fo_pairwise_task(x, offset, half, stride);
  right = fo_pairwise_task(x, offset + half * stride, n - half, stride);
#pragma omp taskwait
  return left + right;
}
FO_API float fo_pairwise_sum_mt(const float *x, uint64_t n) {
  float r = 0.0f;
#pragma omp parallel
#pragma omp single
  r = fo_pairwise_task(x, 0, n, 1);
  return r;
}

/* Tensor::sum / Tensor::mean (ops.rs:145-184): mean = tree sum / n. */
FO_API float fo_mean(const float *x, uint64_t n) { return fo_pairwise_strided(x, 0, n, 1) / (float)n; }

/* sum_dim_host, reduce.rs:41-52 */
FO_API void fo_sum_dim(const float *x, uint64_t outer, uint64_t n, uint64_t inner, float *out) {
  for (uint64_t j = 0; j < outer * inner; ++j) {
    const uint64_t o = j / inner, i = j % inner;
    out[j] = fo_pairwise_strided(x, o * n * inner + i, n, inner);
  }
}
FO_API void fo_sum_dim_mt(const float *x, uint64_t outer, uint64_t n, uint64_t inner, float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t j = 0; j < (int64_t)(outer * inner); ++j) {
    const uint64_t o = (uint64_t)j / inner, i = (uint64_t)j % inner;
    out[j] = fo_pairwise_strided(x, o * n * inner + i, n, inner);
  }
}
/* mean_dim = sum_dim * (1/n as f32), ops_ext/mean_dim.rs:24-30 */
FO_API void fo_mean_dim(const float *x, uint64_t outer, uint64_t n, uint64_t inner, float *out) {
  fo_sum_dim(x, outer, n, inner, out);
  const float scale = 1.0f / (float)n;
  for (uint64_t j = 0; j < outer * inner; ++j) out[j] = out[j] * scale;
}
FO_API void fo_mean_dim_mt(const float *x, uint64_t outer, uint64_t n, uint64_t inner, float *out) {
  fo_sum_dim_mt(x, outer, n, inner, out);
  const float scale = 1.0f / (float)n;
  for (uint64_t j = 0; j < outer * inner; ++j) out[j] = out[j] * scale;
}

/* arg_reduce with `cand > best`, ops_ext/argmax.rs:42-63: the first NaN wins
 * at once; otherwise strictly greater replaces (ties keep the lowest index).
 * The axis max is the element at that index. */
static inline uint64_t fo_argmax1(const float *x, uint64_t base, uint64_t size, uint64_t stride) {
  uint64_t arg = 0;
  for (uint64_t k = 0; k < size; ++k) {
    const float v = x[base + k * stride];
    if (isnan(v)) { arg = k; break; }
    if (v > x[base + arg * stride]) arg = k;
  }
  return arg;
}
FO_API void fo_argmax_dim(const float *x, uint64_t outer, uint64_t size, uint64_t inner,
                          int64_t *idx, float *val) {
#pragma omp parallel for schedule(static)
  for (int64_t j = 0; j < (int64_t)(outer * inner); ++j) {
    const uint64_t o = (uint64_t)j / inner, i = (uint64_t)j % inner;
    const uint64_t base = o * size * inner + i;
    const uint64_t a = fo_argmax1(x, base, size, inner);
    if (idx) idx[j] = (int64_t)a;
    if (val) val[j] = x[base + a * inner];
  }
}
/* Global max, ops_ext/max.rs:45-54 */
FO_API float fo_max_all(const float *x, uint64_t n) {
  float m = x[0];
  for (uint64_t i = 0; i < n; ++i) {
    const float v = x[i];
    if (isnan(v)) { m = v; break; }
    if (v > m) m = v;
  }
  return m;
}

/* ------------------------------------------------ softmax / log_softmax */
/* One (outer, size, stride) slice of softmax_forward, ops_ext/softmax.rs:68-88 */
static void fo_softmax_slice(const float *x, float *y, uint64_t base, uint64_t size, uint64_t stride) {
  float m = -INFINITY;
  for (uint64_t k = 0; k < size; ++k) m = fmaxf(m, x[base + k * stride]);
  for (uint64_t k = 0; k < size; ++k) y[base + k * stride] = expf(x[base + k * stride] - m);
  const float sum = fo_pairwise_strided(y, base, size, stride);
  for (uint64_t k = 0; k < size; ++k) y[base + k * stride] /= sum;
}
FO_API void fo_softmax_fwd(const float *x, uint64_t outer, uint64_t size, uint64_t stride, float *y) {
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t o = 0; o < (int64_t)outer; ++o)
    for (int64_t i = 0; i < (int64_t)stride; ++i)
      fo_softmax_slice(x, y, (uint64_t)o * size * stride + (uint64_t)i, size, stride);
}

/* softmax_backward, ops_ext/softmax.rs:90-109; `gy` is scratch of x's size */
FO_API void fo_softmax_bwd(const float *g, const float *y, uint64_t outer, uint64_t size,
                           uint64_t stride, float *gy, float *dx) {
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t o = 0; o < (int64_t)outer; ++o)
    for (int64_t i = 0; i < (int64_t)stride; ++i) {
      const uint64_t base = (uint64_t)o * size * stride + (uint64_t)i;
      for (uint64_t k = 0; k < size; ++k) {
        const uint64_t id = base + k * stride;
        gy[id] = g[id] * y[id];
      }
      const float dot = fo_pairwise_strided(gy, base, size, stride);
      for (uint64_t k = 0; k < size; ++k) {
        const uint64_t id = base + k * stride;
        dx[id] = y[id] * (g[id] - dot);
      }
    }
}

/* log_softmax_forward, ops_ext/log_softmax.rs:76-100; `exps` is scratch */
FO_API void fo_log_softmax_fwd(const float *x, uint64_t outer, uint64_t n, uint64_t stride,
                               float *exps, float *y) {
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t o = 0; o < (int64_t)outer; ++o)
    for (int64_t i = 0; i < (int64_t)stride; ++i) {
      const uint64_t base = (uint64_t)o * n * stride + (uint64_t)i;
      float m = -INFINITY;
      for (uint64_t k = 0; k < n; ++k) m = fmaxf(m, x[base + k * stride]);
      for (uint64_t k = 0; k < n; ++k) exps[base + k * stride] = expf(x[base + k * stride] - m);
      const float sum = fo_pairwise_strided(exps, base, n, stride);
      const float log_sum = logf(sum);
      for (uint64_t k = 0; k < n; ++k) y[base + k * stride] = (x[base + k * stride] - m) - log_sum;
    }
}

/* log_softmax backward closure, ops_ext/log_softmax.rs:52-72: the saved
 * softmax is exp(y); dx = g - sm * tree(g). */
FO_API void fo_log_softmax_bwd(const float *g, const float *y, uint64_t outer, uint64_t n,
                               uint64_t stride, float *dx) {
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t o = 0; o < (int64_t)outer; ++o)
    for (int64_t i = 0; i < (int64_t)stride; ++i) {
      const uint64_t base = (uint64_t)o * n * stride + (uint64_t)i;
      const float sum_g = fo_pairwise_strided(g, base, n, stride);
      for (uint64_t k = 0; k < n; ++k) {
        const uint64_t id = base + k * stride;
        dx[id] = g[id] - expf(y[id]) * sum_g;
      }
    }
}

/* cross_entropy_indices (crates/ferro-core/src/nn.rs:793-814) = one_hot
 * (nn.rs:403-432) then cross_entropy (nn.rs:380-400):
 *   lp = log_softmax(logits, 1); loss = mean(-sum_dim(lp * onehot, 1)).
 * Backward through that graph with upstream 1:
 *   mean  -> g_r = 1 * (1/N)            (ops.rs:176-183, a multiply by 1/n)
 *   neg   -> -g_r
 *   sum_dim -> broadcast over the row; mul by onehot -> glp[r,k] = -g_r * onehot[r,k]
 *   log_softmax -> d[r,k] = glp[r,k] - exp(lp[r,k]) * tree(glp[r,:]).
 * Returns 0, or 1 + the first row whose target is outside [0, C) (the
 * one_hot range error, nn.rs:419-424) with nothing written.
 * Optional outputs may be NULL.  `lp` is [rows, cols] scratch. */
FO_API int64_t fo_cross_entropy_indices(const float *logits, const int64_t *targets, uint64_t rows,
                                        uint64_t cols, float *lp, float *loss, float *dlogits,
                                        int64_t *argmax) {
  for (uint64_t r = 0; r < rows; ++r)
    if (targets[r] < 0 || (uint64_t)targets[r] >= cols) return (int64_t)r + 1;
  float *rowloss = (float *)malloc(sizeof(float) * (rows ? rows : 1));
  const float inv_n = 1.0f / (float)rows;
#pragma omp parallel
  {
    float *scratch = (float *)malloc(sizeof(float) * (cols ? cols : 1));
#pragma omp for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
      const uint64_t base = (uint64_t)r * cols;
      const float *x = logits + base;
      float *y = lp + base;
      float m = -INFINITY;
      for (uint64_t k = 0; k < cols; ++k) m = fmaxf(m, x[k]);
      for (uint64_t k = 0; k < cols; ++k) scratch[k] = expf(x[k] - m);
      const float log_sum = logf(fo_pairwise_strided(scratch, 0, cols, 1));
      for (uint64_t k = 0; k < cols; ++k) y[k] = (x[k] - m) - log_sum;
      const uint64_t t = (uint64_t)targets[r];
      /* sum_dim(lp * onehot, 1): products are lp*0 except one lp*1. */
      for (uint64_t k = 0; k < cols; ++k) scratch[k] = y[k] * (k == t ? 1.0f : 0.0f);
      rowloss[r] = -fo_pairwise_strided(scratch, 0, cols, 1);
      if (argmax) argmax[r] = (int64_t)fo_argmax1(x, 0, cols, 1);
      if (dlogits) {
        const float gr = -(1.0f * inv_n);
        for (uint64_t k = 0; k < cols; ++k) scratch[k] = gr * (k == t ? 1.0f : 0.0f);
        const float sum_g = fo_pairwise_strided(scratch, 0, cols, 1);
        for (uint64_t k = 0; k < cols; ++k) dlogits[base + k] = scratch[k] - expf(y[k]) * sum_g;
      }
    }
    free(scratch);
  }
  if (loss) *loss = fo_pairwise_strided(rowloss, 0, rows, 1) / (float)rows;
  free(rowloss);
  return 0;
}

/* ------------------------------------------------------------ LayerNorm */
/* Host forward loop, ops_ext/layer_norm.rs:184-205.  Outputs: y, yhat (h),
 * stds; `means` optional.  w / b optional (NULL). */
FO_API void fo_layer_norm_fwd(const float *x, const float *w, const float *b, uint64_t rows,
                              uint64_t d, float eps, float *y, float *yhat, float *stds,
                              float *means) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)rows; ++r) {
    const uint64_t base = (uint64_t)r * d;
    const float m = fo_pairwise_strided(x, base, d, 1) / (float)d;
    float v = 0.0f;
    for (uint64_t i = 0; i < d; ++i) {
      const float c = x[base + i] - m;
      v += c * c;
    }
    const float s = sqrtf(v / (float)d + eps);
    stds[r] = s;
    if (means) means[r] = m;
    for (uint64_t i = 0; i < d; ++i) {
      const float h = (x[base + i] - m) / s;
      yhat[base + i] = h;
      y[base + i] = h * (w ? w[i] : 1.0f) + (b ? b[i] : 0.0f);
    }
  }
}

/* host_backward, ops_ext/layer_norm.rs:28-68.  dw / db accumulate over rows
 * in row order (sequential adds), so that loop stays serial per column. */
FO_API void fo_layer_norm_bwd(const float *g, const float *yhat, const float *stds, const float *w,
                              uint64_t rows, uint64_t d, float *dx, float *dw, float *db) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)rows; ++r) {
    const uint64_t base = (uint64_t)r * d;
    const float s = stds[r];
    float sum_dxh = 0.0f, sum_dxh_h = 0.0f;
    for (uint64_t i = 0; i < d; ++i) {
      const float dxh = g[base + i] * (w ? w[i] : 1.0f);
      sum_dxh += dxh;
      sum_dxh_h += dxh * yhat[base + i];
    }
    for (uint64_t i = 0; i < d; ++i) {
      const float dxh = g[base + i] * (w ? w[i] : 1.0f);
      dx[base + i] = (dxh - sum_dxh / (float)d - yhat[base + i] * sum_dxh_h / (float)d) / s;
    }
  }
  if (dw || db) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)d; ++i) {
      float aw = 0.0f, ab = 0.0f;
      for (uint64_t r = 0; r < rows; ++r) {
        aw += g[r * d + i] * yhat[r * d + i];
        ab += g[r * d + i];
      }
      if (dw) dw[i] = aw;
      if (db) db[i] = ab;
    }
  }
}

/* ----------------------------------------------------------- optimizers */
/* f32::powi lowers to compiler-rt's __powisf2: square-and-multiply. */
FO_API float fo_powi(float a, int b) {
  const int recip = b < 0;
  float r = 1.0f;
  while (1) {
    if (b & 1) r *= a;
    b /= 2;
    if (b == 0) break;
    a *= a;
  }
  return recip ? 1.0f / r : r;
}
/* bc = 1 - beta.powi(t), optim.rs:719-721 */
FO_API float fo_bias_correction(float beta, int t) { return 1.0f - fo_powi(beta, t); }

/* Backend::adamw_step, dispatch.rs:489-503 */
FO_API void fo_adamw_step(float *p, float *m, float *v, const float *g, uint64_t n, float lr,
                          float beta1, float beta2, float bc1, float bc2, float eps, float wd) {
  const float nb1 = 1.0f - beta1, nb2 = 1.0f - beta2;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    const float gi = g[i];
    m[i] = m[i] * beta1 + gi * nb1;
    v[i] = v[i] * beta2 + (gi * gi) * nb2;
    const float m_hat = m[i] / bc1;
    const float denom = sqrtf(v[i] / bc2);
    float upd = m_hat / (denom + eps);
    if (wd != 0.0f) upd += wd * p[i];
    p[i] -= upd * lr;
  }
}

/* Backend::sgd_step, dispatch.rs:477-483 */
FO_API void fo_sgd_step(float *p, float *v, const float *g, uint64_t n, float lr, float momentum,
                        int nesterov) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    v[i] = v[i] * momentum + g[i];
    const float d = nesterov ? v[i] * momentum + g[i] : v[i];
    p[i] -= d * lr;
  }
}

/* Ddp::average, crates/ferro-core/src/ddp.rs:138-157: running sum over the
 * replicas in order, then one divide by the replica count. */
FO_API void fo_ddp_average(const float *const *grads, int replicas, uint64_t n, float *out) {
  const float cnt = (float)replicas;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    float s = grads[0][i];
    for (int r = 1; r < replicas; ++r) s += grads[r][i];
    out[i] = s / cnt;
  }
}


/* --------------------------------------------------- gather and segments */
/* Tensor::gather, crates/ferro-core/src/ops_ext/gather.rs:50-98: walk the output
 * coordinates in row-major order, substituting the gathered index along `dim`.
 * Returns 0, or 1 + the flat position of an index outside [0, in_shape[dim]). */
FO_API int64_t fo_gather(const float *x, const uint64_t *in_shape, const int64_t *index,
                         const uint64_t *out_shape, int rank, int dim, float *out, uint64_t *src) {
  uint64_t n = 1;
  for (int d = 0; d < rank; ++d) n *= out_shape[d];
  uint64_t coord[16] = {0};
  for (uint64_t i = 0; i < n; ++i) {
    const int64_t id = index[i];
    if (id < 0 || (uint64_t)id >= in_shape[dim]) return (int64_t)i + 1;
    uint64_t off = 0;
    for (int d = 0; d < rank; ++d) off = off * in_shape[d] + (d == dim ? (uint64_t)id : coord[d]);
    out[i] = x[off];
    if (src) src[i] = off;
    for (int d = rank - 1; d >= 0; --d) {
      if (++coord[d] < out_shape[d]) break;
      coord[d] = 0;
    }
  }
  return 0;
}
/* gather backward, gather.rs:103-110: gx = 0; gx[src[i]] += g[i] in output order. */
FO_API void fo_gather_bwd(const float *g, const uint64_t *src, uint64_t n_out, uint64_t n_in, float *gx) {
  memset(gx, 0, sizeof(float) * n_in);
  for (uint64_t i = 0; i < n_out; ++i) gx[src[i]] += g[i];
}
/* segment::sum and its backward, crates/ferro-core/src/segment.rs:132-150 */
FO_API void fo_segment_sum(const float *x, const uint64_t *ids, uint64_t edges, uint64_t groups, uint64_t width,
                           float *out) {
  memset(out, 0, sizeof(float) * groups * width);
  for (uint64_t e = 0; e < edges; ++e)
    for (uint64_t f = 0; f < width; ++f) out[ids[e] * width + f] += x[e * width + f];
}
FO_API void fo_segment_sum_bwd(const float *g, const uint64_t *ids, uint64_t edges, uint64_t width, float *dx) {
  for (uint64_t e = 0; e < edges; ++e)
    for (uint64_t f = 0; f < width; ++f) dx[e * width + f] = g[ids[e] * width + f];
}
/* segment::softmax, segment.rs:217-239; returns 1 when an input is not finite (the error of :222-225). */
FO_API int fo_segment_softmax(const float *x, const uint64_t *ids, uint64_t edges, uint64_t groups, uint64_t width,
                              float *maxima, float *denom, float *out) {
  for (uint64_t i = 0; i < edges * width; ++i)
    if (!isfinite(x[i])) return 1;
  for (uint64_t i = 0; i < groups * width; ++i) { maxima[i] = -INFINITY; denom[i] = 0.0f; }
  for (uint64_t e = 0; e < edges; ++e)
    for (uint64_t f = 0; f < width; ++f) {
      const uint64_t j = ids[e] * width + f;
      maxima[j] = fmaxf(maxima[j], x[e * width + f]);
    }
  for (uint64_t e = 0; e < edges; ++e)
    for (uint64_t f = 0; f < width; ++f) {
      const uint64_t j = ids[e] * width + f;
      out[e * width + f] = expf(x[e * width + f] - maxima[j]);
      denom[j] += out[e * width + f];
    }
  for (uint64_t e = 0; e < edges; ++e)
    for (uint64_t f = 0; f < width; ++f) out[e * width + f] /= denom[ids[e] * width + f];
  return 0;
}
/* its backward, segment.rs:242-253 */
FO_API void fo_segment_softmax_bwd(const float *g, const float *y, const uint64_t *ids, uint64_t edges, uint64_t groups,
                                   uint64_t width, float *dot, float *dx) {
  for (uint64_t i = 0; i < groups * width; ++i) dot[i] = 0.0f;
  for (uint64_t e = 0; e < edges; ++e)
    for (uint64_t f = 0; f < width; ++f) dot[ids[e] * width + f] += g[e * width + f] * y[e * width + f];
  for (uint64_t e = 0; e < edges; ++e)
    for (uint64_t f = 0; f < width; ++f)
      dx[e * width + f] = y[e * width + f] * (g[e * width + f] - dot[ids[e] * width + f]);
}

/* ------------------------------------------------- MLP glue (DDP config) */
/* naive_matmul, dispatch.rs:788-807 (ikj, zero-skip only for finite rhs) */
FO_API void fo_matmul(const float *a, const float *b, uint64_t m, uint64_t k, uint64_t n, float *out) {
  memset(out, 0, sizeof(float) * m * n);
  int finite_rhs = 1;
  for (uint64_t i = 0; i < k * n; ++i)
    if (!isfinite(b[i])) { finite_rhs = 0; break; }
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)m; ++i)
    for (uint64_t p = 0; p < k; ++p) {
      const float aip = a[(uint64_t)i * k + p];
      if (finite_rhs && aip == 0.0f) continue;
      for (uint64_t j = 0; j < n; ++j) out[(uint64_t)i * n + j] += aip * b[p * n + j];
    }
}

/* mse_loss = mean(square(pred - target)), ops_ext/mse_loss.rs:9-11 and
 * square.rs:16-19 (x*x; backward g * (2*x)).  Backward with upstream 1:
 * mean -> 1 * (1/n) per element; square -> gs * (2 * diff); sub -> that. */
FO_API float fo_mse_fwd_bwd(const float *pred, const float *target, uint64_t n, float *sq,
                            float *dpred) {
  const float inv = 1.0f / (float)n;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    const float diff = pred[i] - target[i];
    sq[i] = diff * diff;
    if (dpred) dpred[i] = (1.0f * inv) * (2.0f * diff);
  }
  return fo_pairwise_strided(sq, 0, n, 1) / (float)n;
}
