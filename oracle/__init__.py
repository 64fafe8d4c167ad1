"""TEST INFRASTRUCTURE: numpy front-end of the CPU oracle (oracle/ferro_oracle.c).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
package.  The shipped library (`ferro_b200`) never does.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_f32p = C.POINTER(C.c_float)
_i64p = C.POINTER(C.c_int64)
_u64p = C.POINTER(C.c_uint64)
_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(_build.build())
        L = _LIB
        L.fo_max_threads.restype = C.c_int
        L.fo_rng_uniform.restype = C.c_float
        L.fo_rng_normal.restype = C.c_float
        L.fo_pairwise_sum.restype = C.c_float
        L.fo_pairwise_sum_mt.restype = C.c_float
        L.fo_pairwise_sum_strided.restype = C.c_float
        L.fo_mean.restype = C.c_float
        L.fo_max_all.restype = C.c_float
        L.fo_powi.restype = C.c_float
        L.fo_bias_correction.restype = C.c_float
        L.fo_mse_fwd_bwd.restype = C.c_float
        L.fo_cross_entropy_indices.restype = C.c_int64
    return _LIB


def max_threads() -> int:
    return int(lib().fo_max_threads())


def use_all_cores() -> int:
    """Thread the *_mt loops over every core this process may run on, as ferro does
    (available_parallelism, workers.rs:75-78), even when a launcher exported OMP_NUM_THREADS=1."""
    import os
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().fo_set_threads(C.c_int(n))
    return max_threads()


def _f(a):
    return a.ctypes.data_as(_f32p)


def _opt(a):
    return None if a is None else a.ctypes.data_as(_f32p)


def _c(a, dtype=np.float32):
    return np.ascontiguousarray(a, dtype=dtype)


class _RngState(C.Structure):
    _fields_ = [("s0", C.c_uint64), ("s1", C.c_uint64)]


class Rng:
    """ferro_core::Rng (crates/ferro-core/src/rng.rs:12-70)."""

    def __init__(self, seed: int):
        self._s = _RngState()
        lib().fo_rng_seed(C.byref(self._s), C.c_uint64(seed))

    def state(self):
        return (int(self._s.s0), int(self._s.s1))

    def uniform(self) -> float:
        return float(lib().fo_rng_uniform(C.byref(self._s)))

    def normal(self) -> float:
        return float(lib().fo_rng_normal(C.byref(self._s)))

    def fill_normal(self, shape, scale=1.0, shift=0.0):
        out = np.empty(shape, np.float32)
        lib().fo_rng_fill_normal(C.byref(self._s), _f(out), C.c_uint64(out.size),
                                 C.c_float(scale), C.c_float(shift))
        return out

    def fill_uniform(self, shape, scale=1.0, shift=0.0):
        out = np.empty(shape, np.float32)
        lib().fo_rng_fill_uniform(C.byref(self._s), _f(out), C.c_uint64(out.size),
                                  C.c_float(scale), C.c_float(shift))
        return out

    def fill_he(self, shape, fan_in):
        out = np.empty(shape, np.float32)
        lib().fo_rng_fill_he(C.byref(self._s), _f(out), C.c_uint64(out.size), C.c_uint64(fan_in))
        return out

    def fill_rowscaled_normal(self, rows, cols, lo=0.5, span=3.5):
        out = np.empty((rows, cols), np.float32)
        lib().fo_rng_fill_rowscaled_normal(C.byref(self._s), _f(out), C.c_uint64(rows),
                                           C.c_uint64(cols), C.c_float(lo), C.c_float(span))
        return out

    def fill_targets(self, n, classes):
        out = np.empty((n,), np.int64)
        lib().fo_rng_fill_targets(C.byref(self._s), out.ctypes.data_as(_i64p), C.c_uint64(n),
                                  C.c_uint64(classes))
        return out


def unary(kind, x, p0=0.0, p1=0.0, mt=False):
    x = _c(x)
    out = np.empty_like(x)
    fn = lib().fo_unary_mt if mt else lib().fo_unary
    fn(C.c_int(kind), C.c_float(p0), C.c_float(p1), _f(x), _f(out), C.c_uint64(x.size))
    return out


def binary(kind, a, b, p0=0.0, p1=0.0, mt=False):
    a, b = _c(a), _c(b)
    assert a.shape == b.shape
    out = np.empty_like(a)
    fn = lib().fo_binary_mt if mt else lib().fo_binary
    fn(C.c_int(kind), C.c_float(p0), C.c_float(p1), _f(a), _f(b), _f(out), C.c_uint64(a.size))
    return out


def _arr(vals, ct):
    return (ct * max(len(vals), 1))(*vals)


def binary_strided(kind, a, sa, offa, b, sb, offb, shape, p0=0.0, p1=0.0):
    """Row-major output over `shape`; operands addressed by element strides."""
    a, b = _c(a).ravel(), _c(b).ravel()
    out = np.empty(tuple(shape), np.float32)
    lib().fo_binary_strided(C.c_int(kind), C.c_float(p0), C.c_float(p1), _f(a),
                            _arr(list(sa), C.c_int64), C.c_int64(offa), _f(b),
                            _arr(list(sb), C.c_int64), C.c_int64(offb),
                            _arr(list(shape), C.c_uint64), C.c_int(len(shape)), _f(out))
    return out


def broadcast_strides(shape, out_shape):
    """dispatch.rs:823-835: stride 0 on padded / expanded dims."""
    own = []
    acc = 1
    for s in reversed(shape):
        own.insert(0, acc)
        acc *= s
    pad = len(out_shape) - len(shape)
    return [0 if (i < pad or shape[i - pad] != out_shape[i]) else own[i - pad]
            for i in range(len(out_shape))]


def binary_bc(kind, a, b, p0=0.0, p1=0.0):
    """Backend::binary_bc (dispatch.rs:217-227) on numpy operands of shapes sa, sb."""
    a, b = _c(a), _c(b)
    out_shape = np.broadcast_shapes(a.shape, b.shape)
    return binary_strided(kind, a, broadcast_strides(a.shape, out_shape), 0, b,
                          broadcast_strides(b.shape, out_shape), 0, out_shape, p0, p1)


def materialize(x, strides, offset, shape):
    x = _c(x).ravel()
    out = np.empty(tuple(shape), np.float32)
    lib().fo_materialize(_f(x), _arr(list(strides), C.c_int64), C.c_int64(offset),
                         _arr(list(shape), C.c_uint64), C.c_int(len(shape)), _f(out))
    return out


def affine_inplace(dst, mul, add):
    lib().fo_affine_inplace(_f(dst), C.c_float(mul), C.c_float(add), C.c_uint64(dst.size))


def axpy_inplace(alpha, dst, src):
    lib().fo_axpy_inplace(C.c_float(alpha), _f(dst), _f(_c(src)), C.c_uint64(dst.size))


def pairwise_sum(x, mt=False):
    x = _c(x).ravel()
    fn = lib().fo_pairwise_sum_mt if mt else lib().fo_pairwise_sum
    return np.float32(fn(_f(x), C.c_uint64(x.size)))


def pairwise_sum_strided(x, offset, n, stride):
    x = _c(x).ravel()
    return np.float32(lib().fo_pairwise_sum_strided(_f(x), C.c_uint64(offset), C.c_uint64(n),
                                                    C.c_uint64(stride)))


def mean(x):
    x = _c(x).ravel()
    return np.float32(lib().fo_mean(_f(x), C.c_uint64(x.size)))


def _ori(shape, dim):
    outer = int(np.prod(shape[:dim], dtype=np.int64))
    inner = int(np.prod(shape[dim + 1:], dtype=np.int64))
    return outer, int(shape[dim]), inner


def _keep(shape, dim):
    s = list(shape)
    s[dim] = 1
    return tuple(s)


def sum_dim(x, dim, mt=False):
    x = _c(x)
    o, n, i = _ori(x.shape, dim)
    out = np.empty(_keep(x.shape, dim), np.float32)
    fn = lib().fo_sum_dim_mt if mt else lib().fo_sum_dim
    fn(_f(x), C.c_uint64(o), C.c_uint64(n), C.c_uint64(i), _f(out))
    return out


def mean_dim(x, dim, mt=False):
    x = _c(x)
    o, n, i = _ori(x.shape, dim)
    out = np.empty(_keep(x.shape, dim), np.float32)
    fn = lib().fo_mean_dim_mt if mt else lib().fo_mean_dim
    fn(_f(x), C.c_uint64(o), C.c_uint64(n), C.c_uint64(i), _f(out))
    return out


def argmax_dim(x, dim):
    """(indices i64, values f32) in keepdim layout; values = x at argmax."""
    x = _c(x)
    o, n, i = _ori(x.shape, dim)
    idx = np.empty(_keep(x.shape, dim), np.int64)
    val = np.empty(_keep(x.shape, dim), np.float32)
    lib().fo_argmax_dim(_f(x), C.c_uint64(o), C.c_uint64(n), C.c_uint64(i),
                        idx.ctypes.data_as(_i64p), _f(val))
    return idx, val


def max_all(x):
    x = _c(x).ravel()
    return np.float32(lib().fo_max_all(_f(x), C.c_uint64(x.size)))


def softmax_fwd(x, dim=-1):
    x = _c(x)
    dim %= x.ndim
    o, n, i = _ori(x.shape, dim)
    y = np.empty_like(x)
    lib().fo_softmax_fwd(_f(x), C.c_uint64(o), C.c_uint64(n), C.c_uint64(i), _f(y))
    return y


def softmax_bwd(g, y, dim=-1):
    g, y = _c(g), _c(y)
    dim %= y.ndim
    o, n, i = _ori(y.shape, dim)
    gy = np.empty_like(y)
    dx = np.empty_like(y)
    lib().fo_softmax_bwd(_f(g), _f(y), C.c_uint64(o), C.c_uint64(n), C.c_uint64(i), _f(gy), _f(dx))
    return dx


def log_softmax_fwd(x, dim=-1):
    x = _c(x)
    dim %= x.ndim
    o, n, i = _ori(x.shape, dim)
    y = np.empty_like(x)
    ex = np.empty_like(x)
    lib().fo_log_softmax_fwd(_f(x), C.c_uint64(o), C.c_uint64(n), C.c_uint64(i), _f(ex), _f(y))
    return y


def log_softmax_bwd(g, y, dim=-1):
    g, y = _c(g), _c(y)
    dim %= y.ndim
    o, n, i = _ori(y.shape, dim)
    dx = np.empty_like(y)
    lib().fo_log_softmax_bwd(_f(g), _f(y), C.c_uint64(o), C.c_uint64(n), C.c_uint64(i), _f(dx))
    return dx


def cross_entropy_indices(logits, targets, want_grad=True, want_argmax=True):
    """(loss, dlogits | None, argmax | None) or raises ValueError like one_hot."""
    logits = _c(logits)
    targets = _c(targets, np.int64)
    rows, cols = logits.shape
    lp = np.empty_like(logits)
    loss = C.c_float(0.0)
    dl = np.empty_like(logits) if want_grad else None
    am = np.empty((rows,), np.int64) if want_argmax else None
    rc = lib().fo_cross_entropy_indices(
        _f(logits), targets.ctypes.data_as(_i64p), C.c_uint64(rows), C.c_uint64(cols), _f(lp),
        C.byref(loss), _opt(dl), None if am is None else am.ctypes.data_as(_i64p))
    if rc != 0:
        raise ValueError(f"id {int(targets[rc - 1])} out of range for {cols} classes")
    return np.float32(loss.value), dl, am


def layer_norm_fwd(x, w, b, eps):
    """(y, yhat, stds, means), rows = prod(shape[:-1])."""
    x = _c(x)
    d = x.shape[-1]
    rows = x.size // d if d else 0
    w = None if w is None else _c(w)
    b = None if b is None else _c(b)
    y = np.empty_like(x)
    h = np.empty_like(x)
    stds = np.empty((rows,), np.float32)
    means = np.empty((rows,), np.float32)
    lib().fo_layer_norm_fwd(_f(x), _opt(w), _opt(b), C.c_uint64(rows), C.c_uint64(d),
                            C.c_float(eps), _f(y), _f(h), _f(stds), _f(means))
    return y, h, stds, means


def layer_norm_bwd(g, yhat, stds, w, want_dw=True, want_db=True):
    g, yhat, stds = _c(g), _c(yhat), _c(stds)
    d = g.shape[-1]
    rows = g.size // d
    w = None if w is None else _c(w)
    dx = np.empty_like(g)
    dw = np.empty((d,), np.float32) if want_dw else None
    db = np.empty((d,), np.float32) if want_db else None
    lib().fo_layer_norm_bwd(_f(g), _f(yhat), _f(stds), _opt(w), C.c_uint64(rows), C.c_uint64(d),
                            _f(dx), _opt(dw), _opt(db))
    return dx, dw, db


def powi(a, b):
    return np.float32(lib().fo_powi(C.c_float(a), C.c_int(b)))


def bias_correction(beta, t):
    return np.float32(lib().fo_bias_correction(C.c_float(beta), C.c_int(t)))


def adamw_step(p, m, v, g, lr, beta1, beta2, bc1, bc2, eps, wd):
    """In place on p, m, v (contiguous float32 arrays)."""
    g = _c(g)
    lib().fo_adamw_step(_f(p), _f(m), _f(v), _f(g), C.c_uint64(p.size), C.c_float(lr),
                        C.c_float(beta1), C.c_float(beta2), C.c_float(bc1), C.c_float(bc2),
                        C.c_float(eps), C.c_float(wd))


def sgd_step(p, v, g, lr, momentum, nesterov):
    g = _c(g)
    lib().fo_sgd_step(_f(p), _f(v), _f(g), C.c_uint64(p.size), C.c_float(lr),
                      C.c_float(momentum), C.c_int(1 if nesterov else 0))


def ddp_average(grads):
    grads = [_c(g) for g in grads]
    out = np.empty_like(grads[0])
    ptrs = (_f32p * len(grads))(*[_f(g) for g in grads])
    lib().fo_ddp_average(ptrs, C.c_int(len(grads)), C.c_uint64(out.size), _f(out))
    return out


def rms_norm_fwd(x, weight, eps):
    """RmsNorm::forward (crates/ferro-core/src/nn.rs:272-279), op by op in f32:
    ms = mean_dim(x*x, last) (pairwise tree times 1/n), y = x / sqrt(ms + eps) * gamma.  Returns (y, rstd)."""
    x = _c(x)
    rows, cols = x.shape
    ms = mean_dim(np.float32(x * x), 1).reshape(rows, 1)
    den = np.sqrt(np.float32(ms + np.float32(eps)), dtype=np.float32)
    y = np.float32(x / den)
    if weight is not None:
        y = np.float32(y * _c(weight))
    return y, np.float32(1.0 / den.ravel())


def rms_norm_bwd(g, x, weight, eps):
    """Gradient of the composition above, evaluated in float64 (the tolerance of the parity test is
    2e-4, far above f32 reassociation effects): dx = r * (g*w - xh * mean(g*w*xh)), dw = sum_rows g*xh."""
    g64, x64 = np.asarray(g, np.float64), np.asarray(x, np.float64)
    w64 = np.ones(x64.shape[1]) if weight is None else np.asarray(weight, np.float64)
    r = 1.0 / np.sqrt((x64 * x64).mean(1, keepdims=True) + eps)
    xh = x64 * r
    dh = g64 * w64
    dx = r * (dh - xh * (dh * xh).mean(1, keepdims=True))
    return dx, (g64 * xh).sum(0)


def global_grad_norm(grads):
    """crates/ferro-core/src/optim.rs:1395-1408: per gradient, g*g then the pairwise-tree sum;
    the per-gradient sums are added in f32 in list order; one sqrt at the end."""
    acc = np.float32(0.0)
    for g in grads:
        g = _c(g).ravel()
        acc = np.float32(acc + np.float32(pairwise_sum(np.float32(g * g))))
    return np.float32(np.sqrt(acc))


def clip_scale(grads, max_norm):
    """optim.rs:1412-1425: max/norm when the norm exceeds max (and is not zero), else 1."""
    if max_norm is None:
        return np.float32(1.0)
    norm = global_grad_norm(grads)
    if norm > np.float32(max_norm) and norm > 0:
        return np.float32(np.float32(max_norm) / norm)
    return np.float32(1.0)


def matmul(a, b):
    a, b = _c(a), _c(b)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    out = np.empty((m, n), np.float32)
    lib().fo_matmul(_f(a), _f(b), C.c_uint64(m), C.c_uint64(k), C.c_uint64(n), _f(out))
    return out


def mse_fwd_bwd(pred, target):
    pred, target = _c(pred), _c(target)
    sq = np.empty_like(pred)
    dp = np.empty_like(pred)
    loss = lib().fo_mse_fwd_bwd(_f(pred), _f(target), C.c_uint64(pred.size), _f(sq), _f(dp))
    return np.float32(loss), dp


def gather(x, dim, index):
    """Tensor::gather (ops_ext/gather.rs:12-98): (out, src) with src the flat source offset of every output."""
    x, index = _c(x), _c(index, np.int64)
    assert x.ndim == index.ndim
    out = np.empty(index.shape, np.float32)
    src = np.empty(index.shape, np.uint64)
    ish, osh = _arr(x.shape, C.c_uint64), _arr(index.shape, C.c_uint64)
    lib().fo_gather.restype = C.c_int64
    bad = lib().fo_gather(_f(x), ish, index.ctypes.data_as(_i64p), osh, C.c_int(x.ndim), C.c_int(dim), _f(out),
                          src.ctypes.data_as(C.POINTER(C.c_uint64)))
    if bad:
        raise ValueError(f"index {int(index.ravel()[bad - 1])} out of range for dim {dim}")
    return out, src


def gather_bwd(g, src, in_shape):
    """gather's backward (gather.rs:103-110)."""
    g, src = _c(g), np.ascontiguousarray(src, np.uint64)
    gx = np.empty(in_shape, np.float32)
    lib().fo_gather_bwd(_f(g), src.ctypes.data_as(C.POINTER(C.c_uint64)), C.c_uint64(g.size), C.c_uint64(gx.size), _f(gx))
    return gx


def _ids(ids):
    ids = np.ascontiguousarray(ids, np.uint64)
    return ids, ids.ctypes.data_as(C.POINTER(C.c_uint64))


def segment_sum(x, ids, groups):
    x = _c(x)
    ids, pi = _ids(ids)
    width = int(np.prod(x.shape[1:])) if x.ndim > 1 else 1
    out = np.empty((groups, width), np.float32)
    lib().fo_segment_sum(_f(x), pi, C.c_uint64(len(ids)), C.c_uint64(groups), C.c_uint64(width), _f(out))
    return out


def segment_sum_bwd(g, ids, width):
    g = _c(g)
    ids, pi = _ids(ids)
    dx = np.empty((len(ids), width), np.float32)
    lib().fo_segment_sum_bwd(_f(g), pi, C.c_uint64(len(ids)), C.c_uint64(width), _f(dx))
    return dx


def segment_softmax(x, ids, groups):
    x = _c(x)
    ids, pi = _ids(ids)
    width = x.size // len(ids)
    out = np.empty_like(x)
    mx, dn = np.empty(groups * width, np.float32), np.empty(groups * width, np.float32)
    if lib().fo_segment_softmax(_f(x), pi, C.c_uint64(len(ids)), C.c_uint64(groups), C.c_uint64(width), _f(mx), _f(dn), _f(out)):
        raise ValueError("finite logits required")
    return out


def segment_softmax_bwd(g, y, ids, groups):
    g, y = _c(g), _c(y)
    ids, pi = _ids(ids)
    width = y.size // len(ids)
    dot = np.empty(groups * width, np.float32)
    dx = np.empty_like(y)
    lib().fo_segment_softmax_bwd(_f(g), _f(y), pi, C.c_uint64(len(ids)), C.c_uint64(groups), C.c_uint64(width), _f(dot), _f(dx))
    return dx
