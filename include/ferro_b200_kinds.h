/* Kind codes shared by the C ABI and by the chain-program encoding.
 *
 * The unary and binary codes name the same kernels as ferro's `UnaryKind`
 * and `BinaryKind` (crates/ferro-core/src/dispatch.rs:18-43 and :68-76).
 * Parametrised kinds take their scalars in the (p0, p1) pair every entry
 * point carries: Powf uses p0 = exponent, Clamp uses p0 = min, p1 = max.
 *
 * The FB_BIN_*_BWD kinds are the vector-Jacobian products ferro evaluates
 * with host closures on device tensors today (crates/ferro-core/src/ops_ext/
 * {abs,sqrt,log,powf,clamp,tanh}.rs, activation_backward.rs:22-25); behind
 * the same binary entry point they stay on the GPU.  The first operand is
 * always the incoming gradient g.
 */
#ifndef FERRO_B200_KINDS_H
#define FERRO_B200_KINDS_H

enum fb_unary_kind {
  FB_UN_NEG = 0,
  FB_UN_RELU = 1,      /* v if v > 0 or v is NaN, else +0 */
  FB_UN_EXP = 2,
  FB_UN_SIGMOID = 3,   /* 1 / (1 + exp(-v)) */
  FB_UN_TANH = 4,
  FB_UN_SQRT = 5,
  FB_UN_ABS = 6,
  FB_UN_SIGN = 7,      /* -1 / 0 / +1, sign(NaN) = 0 */
  FB_UN_LOG = 8,
  FB_UN_POWF = 9,      /* p0 = exponent; exact special cases 0.5 -0.5 -1 -2 2 3 */
  FB_UN_CLAMP = 10,    /* p0 = min, p1 = max; NaN input or bound propagates */
  FB_UN_GTZ = 11,      /* 0 when v <= 0, else 1 (so 1 for NaN) */
  FB_UN_GELU = 12,     /* tanh approximation */
  FB_UN_GELU_ERF = 13,
  FB_UN_GELU_ERF_GRAD = 14,
  FB_UN_SILU = 15,
  FB_UN_KIND_COUNT = 16
};

enum fb_binary_kind {
  FB_BIN_ADD = 0,
  FB_BIN_SUB = 1,
  FB_BIN_MUL = 2,
  FB_BIN_DIV = 3,
  FB_BIN_RELU_BACKWARD = 4, /* (g, x): 0 when x <= 0, else g */
  FB_BIN_TANH_BWD = 5,      /* (g, y): g * fma(-y, y, 1) */
  FB_BIN_SIGMOID_BWD = 6,   /* (g, y): (g * (1 - y)) * y */
  FB_BIN_SQRT_BWD = 7,      /* (g, y): g / (2 * y) */
  FB_BIN_ABS_BWD = 8,       /* (g, x): g * sign(x), sign(0) = 0 */
  FB_BIN_LOG_BWD = 9,       /* (g, x): g / x */
  FB_BIN_POWF_BWD = 10,     /* (g, x): g * (p0 * x^(p0-1)); p0 == 0 gives 0 */
  FB_BIN_CLAMP_BWD = 11,    /* (g, x): g when p0 <= x <= p1, else 0 */
  FB_BIN_KIND_COUNT = 12
};

enum fb_reduce_kind { FB_RED_SUM = 0, FB_RED_MEAN = 1 };

/* Return codes.  Zero is success; everything else leaves every output and
 * in-place operand untouched ("on any Err a kernel must have mutated
 * nothing", dispatch.rs:444-446) and sets the thread-local message read by
 * fb_last_error(). */
enum fb_status {
  FB_OK = 0,
  FB_ERR_INVALID_SHAPE = 1, /* maps to ferro Error::InvalidShape */
  FB_ERR_INVALID_ARG = 2,   /* null pointer, bad kind, aliasing the op forbids */
  FB_ERR_CUDA = 3,          /* maps to Error::Unsupported{msg:"CUDA error: ..."} */
  FB_ERR_UNSUPPORTED = 4,   /* valid request this build does not implement */
  FB_ERR_WORKSPACE = 5,     /* scratch buffer missing or too small */
  FB_ERR_COMM = 6,          /* the gradient exchange failed (NCCL's message follows) */
  FB_ERR_FORMAT = 7         /* a checkpoint image is malformed (maps to ferro Error::Format) */
};

#endif
