// Scalar device math of every unary / binary kind.  One definition serves the
// templated contiguous kernels (kind is a compile-time constant there and the
// switch folds away) and the chain interpreter (kind is warp-uniform data).
//
// Semantics follow ferro's CpuBackend (crates/ferro-core/src/dispatch.rs:79-87,
// 671-718) including the NaN / signed-zero rules its tests pin; transcendental
// kinds use CUDA's full-precision libm (a few ulp from glibc's, well inside
// the 1e-5 relative budget).
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

// sqrt with the hardware approximation (relative error 2^-23, no slow path for
// negative or special inputs).  Only for kinds held to the 1e-5 bar, never for
// FB_UN_SQRT itself, which ferro's tests compare bitwise.
__device__ __forceinline__ float sqrt_approx(float v) {
  float r;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

// tanh to about 1e-6 relative in straight-line code: an odd polynomial below
// 0.55, 1 - 2 / (exp(2|x|) + 1) above, both evaluated and selected.  Preserves
// -0, NaN and the +-1 limits.
__device__ __forceinline__ float tanh_fast(float x) {
  const float ax = fabsf(x), x2 = x * x;
  float p = 21844.0f / 6081075.0f;
  p = fmaf(p, x2, -1382.0f / 155925.0f);
  p = fmaf(p, x2, 62.0f / 2835.0f);
  p = fmaf(p, x2, -17.0f / 315.0f);
  p = fmaf(p, x2, 2.0f / 15.0f);
  p = fmaf(p, x2, -1.0f / 3.0f);
  const float small = fmaf(x * x2, p, x);
  float e, r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(e) : "f"(ax * 2.885390081777927f));  // exp(2|x|)
  asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
  const float big = copysignf(fmaf(-2.0f, r, 1.0f), x);
  return ax < 0.55f ? small : big;
}

// UnaryKind::Powf, dispatch.rs:688: exact-compare special cases, else powf.
// p == 1.5 is evaluated as v*sqrt(v) (correctly rounded sqrt, one more
// rounding: within 2 ulp of powf), with powf's value at -inf restored.
__device__ __forceinline__ float powf_kind(float v, float p) {
  if (p == 0.5f) return sqrtf(v);
  if (p == -0.5f) return 1.0f / sqrtf(v);
  if (p == -1.0f) return 1.0f / v;
  if (p == -2.0f) return 1.0f / (v * v);
  if (p == 2.0f) return v * v;
  if (p == 3.0f) return (v * v) * v;
  if (p == 1.5f) return v == -CUDART_INF_F ? CUDART_INF_F : v * sqrt_approx(v);
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
  FBI_UN_KIND_COUNT
};

// Host: the internal code for (kind, p0).
inline int resolve_unary_kind(int kind, float p0) {
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
    case FBI_POWF_1_5: return v == -CUDART_INF_F ? CUDART_INF_F : v * sqrt_approx(v);
    case FBI_POWF_GENERIC: return powf(v, p0);
    case FB_UN_NEG: return -v;
    case FB_UN_RELU: return (v > 0.0f || isnan(v)) ? v : 0.0f;
    case FB_UN_EXP: return expf(v);
    case FB_UN_SIGMOID: return 1.0f / (1.0f + expf(-v));
    case FB_UN_TANH: return tanh_fast(v);
    case FB_UN_SQRT: return sqrtf(v);
    case FB_UN_ABS: return fabsf(v);
    case FB_UN_SIGN: return v > 0.0f ? 1.0f : (v < 0.0f ? -1.0f : 0.0f);
    case FB_UN_LOG: return logf(v);
    case FB_UN_POWF: return powf_kind(v, p0);
    case FB_UN_CLAMP: {
      if (isnan(v)) return v;
      if (isnan(p0) || isnan(p1)) return CUDART_NAN_F;
      const float lower = v < p0 ? p0 : v;
      return lower > p1 ? p1 : lower;
    }
    case FB_UN_GTZ: return !(v <= 0.0f) ? 1.0f : 0.0f;
    case FB_UN_GELU: {
      const float u = 0.7978846f * (v + 0.044715f * v * v * v);
      return 0.5f * v * (1.0f + tanh_fast(u));
    }
    case FB_UN_GELU_ERF: return 0.5f * v * (1.0f + erf_as_f64(v * 0.70710678118654752440f));
    case FB_UN_GELU_ERF_GRAD:
      return 0.5f * (1.0f + erf_as_f64(v * 0.70710678118654752440f)) +
             v * expf(-0.5f * v * v) * 0.39894228f;
    case FB_UN_SILU: return v / (1.0f + expf(-v));
    default: return CUDART_NAN_F;
  }
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
    case FB_BIN_CLAMP_BWD: return (y >= p0 && y <= p1) ? x : 0.0f;
    default: return CUDART_NAN_F;
  }
}

}  // namespace fb
