// Scalar device math of every unary / binary kind.  One definition serves the
// templated contiguous kernels (kind is a compile-time constant there and the
// switch folds away) and the chain interpreter (kind is warp-uniform data).
//
// Semantics follow ferro's CpuBackend (crates/ferro-core/src/dispatch.rs:79-87,
// 671-718) including the NaN / signed-zero rules its tests pin; transcendental
// kinds use CUDA's libm or the hardware approximations defined below, each
// well inside the 1e-5 relative budget: these kernels run close enough to the
// HBM rate that the issue slots of a full-precision exp or divide show.
#pragma once
#include <math_constants.h>

#include "common.cuh"

namespace fb {

// dispatch.rs:51-64: Abramowitz-Stegun 7.1.26 evaluated in f64, the exact
// formula ferro's host backends share for the erf GELU.
__device__ __forceinline__ float erf_as_f64(float x) {
  const double A1 = 0.254829592, A2 = -0.284496736, A3 = 1.421413741, A4 = -1.453152027,
               A5 = 1.061405429, P = 0.3275911;
  const double xd = (double)x;
  const double sign = xd < 0.0 ? -1.0 : 1.0;
  const double ax = fabs(xd);
  const double t = 1.0 / (1.0 + P * ax);
  const double poly = ((((A5 * t + A4) * t + A3) * t + A2) * t + A1) * t;
  return (float)(sign * (1.0 - poly * exp(-ax * ax)));
}

// ---- hardware approximations ---------------------------------------------
// Each is one special-function instruction (the forms without .ftz cost three
// or four more to rescale subnormals).  They are used only for kinds held to
// the 1e-5 relative bar, never for FB_UN_SQRT or FB_BIN_DIV, which stay IEEE.

// sqrt, relative error 2^-23.  Subnormal inputs read as zero.
__device__ __forceinline__ float sqrt_approx(float v) {
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
// 2^t, relative error 2^-22; subnormal results are kept.
__device__ __forceinline__ float ex2_approx(float t) {
  float r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}
// 2^t for results known to be normal or infinite (t >= 0 here).
__device__ __forceinline__ float ex2_approx_ftz(float t) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}
// 1/d, relative error 2^-23; subnormal results are kept.
__device__ __forceinline__ float rcp_approx(float d) {
  float r;
  asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(d));
  return r;
}
// 1/d where a result below 2^-126 may read as zero.
__device__ __forceinline__ float rcp_approx_ftz(float d) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
  return r;
}

// exp(x) = 2^(x*log2(e)).  The product is rounded once, so the relative error
// is |x| * 2^-24 plus the instruction's 2^-22: 5.5e-6 at the overflow bound
// |x| = 88.7, 5e-7 for |x| <= 4.  Overflow, underflow through the subnormals,
// NaN and the infinities behave as in libm.
__device__ __forceinline__ float exp_fast(float x) { return ex2_approx(x * 1.4426950408889634f); }

// tanh to 1.5e-6 relative in straight-line code: the odd Taylor polynomial
// through x^7 below 0.25, 1 - 2 / (exp(2x) + 1) above, both evaluated and
// selected.  The second form needs no sign handling: exp(2x) flushing to 0
// gives -1, overflowing to inf gives +1.  Preserves -0 and NaN.
__device__ __forceinline__ float tanh_fast(float x) {
  const float x2 = x * x;
  float p = fmaf(x2, -17.0f / 315.0f, 2.0f / 15.0f);
  p = fmaf(p, x2, -1.0f / 3.0f);
  const float small = fmaf(x * x2, p, x);
  const float e = ex2_approx_ftz(x * 2.885390081777927f);  // exp(2x)
  const float big = fmaf(-2.0f, rcp_approx_ftz(e + 1.0f), 1.0f);
  return fabsf(x) < 0.25f ? small : big;
}

// powf(v, 1.5) as |v| * sqrt(|v|) with the hardware square root: two
// roundings, within 2 ulp of powf, right as it stands for v >= 0, -0 (+0) and
// -inf (+inf).  Every other negative input, subnormals included, gets powf's
// NaN.  The two tests are combined with `&`: a short-circuit `&&` here is
// compiled to a branch that costs more than the rest of the function.
__device__ __forceinline__ float pow_1_5(float v) {
  const float a = fabsf(v);
  const float r = a * sqrt_approx(a);
  const bool bad = (v < 0.0f) & (v > -CUDART_INF_F);
  return bad ? CUDART_NAN_F : r;
}

// UnaryKind::Powf, dispatch.rs:688: exact-compare special cases, else powf.
__device__ __forceinline__ float powf_kind(float v, float p) {
  if (p == 0.5f) return sqrtf(v);
  if (p == -0.5f) return 1.0f / sqrtf(v);
  if (p == -1.0f) return 1.0f / v;
  if (p == -2.0f) return 1.0f / (v * v);
  if (p == 2.0f) return v * v;
  if (p == 3.0f) return (v * v) * v;
  if (p == 1.5f) return pow_1_5(v);
  return powf(v, p);
}

// Internal unary codes: FB_UN_POWF with its exponent already classified on the
// host, so the per-element exact-compare chain of powf_kind disappears from
// the kernels.  Never part of the ABI.
enum internal_unary_kind {
  FBI_POWF_SQRT = FB_UN_KIND_COUNT,  // p == 0.5
  FBI_POWF_RSQRT,                    // p == -0.5
  FBI_POWF_RCP,                      // p == -1
  FBI_POWF_RSQ,                      // p == -2
  FBI_POWF_SQ,                       // p == 2
  FBI_POWF_CUBE,                     // p == 3
  FBI_POWF_1_5,                      // p == 1.5
  FBI_POWF_GENERIC,                  // anything else: libm powf
  FBI_CLAMP_ORDERED,                 // FB_UN_CLAMP whose bounds are not NaN: two ordered selects
  FBI_UN_KIND_COUNT
};

// Host: the internal code for (kind, p0, p1).
inline int resolve_unary_kind(int kind, float p0, float p1) {
  if (kind == FB_UN_CLAMP) return (p0 == p0 && p1 == p1) ? FBI_CLAMP_ORDERED : FB_UN_CLAMP;
  if (kind != FB_UN_POWF) return kind;
  if (p0 == 0.5f) return FBI_POWF_SQRT;
  if (p0 == -0.5f) return FBI_POWF_RSQRT;
  if (p0 == -1.0f) return FBI_POWF_RCP;
  if (p0 == -2.0f) return FBI_POWF_RSQ;
  if (p0 == 2.0f) return FBI_POWF_SQ;
  if (p0 == 3.0f) return FBI_POWF_CUBE;
  if (p0 == 1.5f) return FBI_POWF_1_5;
  return FBI_POWF_GENERIC;
}

__device__ __forceinline__ float unary_apply(int kind, float p0, float p1, float v) {
  switch (kind) {
    case FBI_POWF_SQRT: return sqrtf(v);
    case FBI_POWF_RSQRT: return 1.0f / sqrtf(v);
    case FBI_POWF_RCP: return 1.0f / v;
    case FBI_POWF_RSQ: return 1.0f / (v * v);
    case FBI_POWF_SQ: return v * v;
    case FBI_POWF_CUBE: return (v * v) * v;
    case FBI_POWF_1_5: return pow_1_5(v);
    case FBI_POWF_GENERIC: return powf(v, p0);
    case FB_UN_NEG: return -v;
    case FB_UN_RELU: return !(v <= 0.0f) ? v : 0.0f;  // v when v > 0 or v is NaN, else +0
    case FB_UN_EXP: return exp_fast(v);
    case FB_UN_SIGMOID: return rcp_approx(1.0f + exp_fast(-v));
    case FB_UN_TANH: return tanh_fast(v);
    case FB_UN_SQRT: return sqrtf(v);
    case FB_UN_ABS: return fabsf(v);
    case FB_UN_SIGN: return v > 0.0f ? 1.0f : (v < 0.0f ? -1.0f : 0.0f);
    case FB_UN_LOG: return logf(v);
    case FB_UN_POWF: return powf_kind(v, p0);
    case FBI_CLAMP_ORDERED: {
      // A NaN input fails both ordered compares and passes through.
      const float lower = v < p0 ? p0 : v;
      return lower > p1 ? p1 : lower;
    }
    case FB_UN_CLAMP: {
      // A NaN input fails both ordered compares and passes through; only a
      // NaN bound needs a branch, and that one is uniform.
      if (isnan(p0) || isnan(p1)) return isnan(v) ? v : CUDART_NAN_F;
      const float lower = v < p0 ? p0 : v;
      return lower > p1 ? p1 : lower;
    }
    case FB_UN_GTZ: return !(v <= 0.0f) ? 1.0f : 0.0f;
    case FB_UN_GELU: {
      // 0.5 v (1 + tanh u) = v / (1 + exp(-2u)): the same function without the
      // cancellation of 1 + tanh(u) for u << 0, and one exponential instead of
      // the two-branch tanh.  exp(-2u) = inf gives v * 0, = 0 gives v.
      const float u = 0.7978846f * (v + 0.044715f * v * v * v);
      return v * rcp_approx(1.0f + ex2_approx(u * -2.885390081777927f));
    }
    case FB_UN_GELU_ERF: return 0.5f * v * (1.0f + erf_as_f64(v * 0.70710678118654752440f));
    case FB_UN_GELU_ERF_GRAD:
      return 0.5f * (1.0f + erf_as_f64(v * 0.70710678118654752440f)) +
             v * exp_fast(-0.5f * v * v) * 0.39894228f;
    case FB_UN_SILU: return v * rcp_approx(1.0f + exp_fast(-v));
    default: return CUDART_NAN_F;
  }
}

// d act / dz of ferro's fused bias + activation (act_bwd, crates/ferro-core/src/fused_ops.rs:31-51) for
// the two smooth activations; identity and relu are handled by their callers (relu as an exact mask).
enum { FB_ACT_IDENTITY = 0, FB_ACT_RELU = 1, FB_ACT_GELU = 2, FB_ACT_SILU = 3 };
__device__ __forceinline__ float act_grad(int act, float z) {
  if (act == FB_ACT_GELU) {
    const float t = tanh_fast(0.7978846f * (z + 0.044715f * z * z * z));
    return 0.5f * (1.0f + t) + 0.5f * z * (1.0f - t * t) * 0.7978846f * (1.0f + 3.0f * 0.044715f * z * z);
  }
  const float e = exp_fast(-z);  // FB_ACT_SILU
  const float sig = rcp_approx(1.0f + e);
  // z * e * sig, grouped so that e = inf (z very negative, sig = 0) gives 0 and not inf * 0.
  return sig * (1.0f + z * (e * sig));
}

// x is the left operand (the incoming gradient for the *_BWD kinds).
__device__ __forceinline__ float binary_apply(int kind, float p0, float p1, float x, float y) {
  switch (kind) {
    case FB_BIN_ADD: return x + y;
    case FB_BIN_SUB: return x - y;
    case FB_BIN_MUL: return x * y;
    case FB_BIN_DIV: return x / y;
    case FB_BIN_RELU_BACKWARD: return y <= 0.0f ? 0.0f : x;
    case FB_BIN_TANH_BWD: return x * fmaf(-y, y, 1.0f);
    case FB_BIN_SIGMOID_BWD: return (x * (1.0f - y)) * y;
    case FB_BIN_SQRT_BWD: return x / (2.0f * y);
    case FB_BIN_ABS_BWD: return x * (y > 0.0f ? 1.0f : (y < 0.0f ? -1.0f : 0.0f));
    case FB_BIN_LOG_BWD: return x / y;
    case FB_BIN_POWF_BWD: return p0 == 0.0f ? 0.0f : x * (p0 * powf_kind(y, p0 - 1.0f));
    case FB_BIN_CLAMP_BWD: return ((y >= p0) & (y <= p1)) ? x : 0.0f;
    default: return CUDART_NAN_F;
  }
}

}  // namespace fb
