"""GPU parity: every kernel, called through the C ABI (via the host mirror of
ferro's Backend seam), against the CPU oracle on the same seeded inputs.

Bars (the stated tolerances of the hot path):
  bit-exact   argmax / max indices, i64 gathers, masks (relu, clamp pass-through, NaN), exact kinds,
              fused Adam / SGD
  1e-5 rel    transcendental elementwise kinds
  2e-4 rel    reductions, softmax, log_softmax, LayerNorm (all outputs)
NaN == NaN counts as equal (crates/ferro-fastcpu/src/elementwise.rs:315-320).
"""
import json
import os

import numpy as np
import pytest
import torch

import oracle as fo
from ferro_b200 import kinds as K

pytestmark = pytest.mark.gpu

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_fixtures.json")))
ELT_RTOL = 1e-5
RED_RTOL = 2e-4


@pytest.fixture(scope="module")
def be():
    from ferro_b200.backend import CudaBackend
    return CudaBackend(0)


def B():
    import ferro_b200.backend as b
    return b


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def assert_bitwise(got, want, ctx=""):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape, ctx
    ok = (bits(got) == bits(want)) | (np.isnan(got) & np.isnan(want))
    assert ok.all(), f"{ctx}: {np.argwhere(~ok)[:5].tolist()} got {got[~ok][:5]} want {want[~ok][:5]}"


def assert_close(got, want, rtol, atol=0.0, ctx=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, ctx
    nan_g, nan_w = np.isnan(got), np.isnan(want)
    assert (nan_g == nan_w).all(), f"{ctx}: NaN masks differ"
    inf = np.isinf(want)
    assert (got[inf] == want[inf]).all(), f"{ctx}: infinities differ"
    m = ~(nan_w | inf)
    err = np.abs(got[m] - want[m])
    bound = rtol * np.abs(want[m]) + atol
    assert (err <= bound).all(), f"{ctx}: max excess {np.max(err - bound):.3e}, max rel {np.max(err / (np.abs(want[m]) + 1e-30)):.3e}"


def special_vals(seed, n):
    """Random values with +-0, NaN, +-inf, denormals planted at both ends
    (crates/ferro-fastcpu/src/elementwise.rs:289-311)."""
    sp = np.array([0.0, -0.0, np.nan, np.inf, -np.inf, 5.8e-39, -5.8e-39, 1.0, -1.0, 2.5], np.float32)
    r = np.random.default_rng(seed)
    head = min(len(sp), n)
    tail = len(sp) if n >= 2 * len(sp) else 0
    mid = ((r.random(n - head - tail) - 0.5) * 4).astype(np.float32)
    return np.concatenate([sp[:head], mid, sp[:tail]]).astype(np.float32)


LENGTHS = [0, 1, 7, 8, 9, 15, 16, 17, 1023, (1 << 20) + 3]

EXACT_UNARY = [K.UN_NEG, K.UN_RELU, K.UN_SQRT, K.UN_ABS, K.UN_SIGN, K.UN_GTZ]
TRANS_UNARY = [K.UN_EXP, K.UN_SIGMOID, K.UN_TANH, K.UN_LOG, K.UN_GELU, K.UN_GELU_ERF,
               K.UN_GELU_ERF_GRAD, K.UN_SILU]


def run_unary(be, kind, x, p0=0.0, p1=0.0):
    out = be.unary_dev(B().UnaryKind(kind, p0, p1), be.alloc_from_host(x))
    return be.copy_to_host(out)


def run_binary(be, kind, a, b, p0=0.0, p1=0.0):
    out = be.binary_dev(B().BinaryKind(kind, p0, p1), be.alloc_from_host(a), be.alloc_from_host(b))
    return be.copy_to_host(out)


# ------------------------------------------------------------------ elementwise
def test_unary_exact_kinds_bitwise_over_length_sweep(be):
    for kind in EXACT_UNARY:
        for n in LENGTHS:
            x = special_vals(n * 11 + kind, n)
            assert_bitwise(run_unary(be, kind, x), fo.unary(kind, x), f"kind {kind} n {n}")


def test_unary_powf_special_cases_bitwise(be):
    for p in (0.5, -0.5, -1.0, -2.0, 2.0, 3.0):
        for n in (17, 1023, (1 << 20) + 3):
            x = special_vals(n, n)
            assert_bitwise(run_unary(be, K.UN_POWF, x, p), fo.unary(K.UN_POWF, x, p), f"powf {p} n {n}")


def test_unary_clamp_bitwise_incl_goldens(be):
    x = np.asarray(GOLD["clamp32"]["input_bits"], np.uint32).view(np.float32)
    for case in GOLD["clamp32"]["cases"]:
        lo = np.asarray([case["min"]], np.uint32).view(np.float32)[0]
        hi = np.asarray([case["max"]], np.uint32).view(np.float32)[0]
        want = np.asarray(case["expected"], np.uint32).view(np.float32)
        assert_bitwise(run_unary(be, K.UN_CLAMP, x, lo, hi), want, f"clamp [{lo},{hi}]")
        g = np.full_like(x, 0.7)
        assert_bitwise(run_binary(be, K.BIN_CLAMP_BWD, g, x, lo, hi), fo.binary(K.BIN_CLAMP_BWD, g, x, lo, hi))
    big = special_vals(3, 100003)
    assert_bitwise(run_unary(be, K.UN_CLAMP, big, -1.0, 1.0), fo.unary(K.UN_CLAMP, big, -1.0, 1.0))


def test_special_power_goldens(be):
    rows = GOLD["power_special_f32"]["forward"]
    for p in sorted({r["p"] for r in rows}):
        sel = [r for r in rows if r["p"] == p]
        x = np.asarray([r["x"] for r in sel], np.uint32).view(np.float32)
        want = np.asarray([r["y"] for r in sel], np.uint32).view(np.float32)
        assert_bitwise(run_unary(be, K.UN_POWF, x, p), want, f"powf {p}")


def test_unary_transcendental_kinds(be):
    for kind in TRANS_UNARY:
        for n in (9, 1023, (1 << 20) + 3):
            x = special_vals(n * 7 + kind, n)
            if kind == K.UN_LOG:
                x = np.abs(x)
            # atol: GELU-type kinds cancel to ~0 for large negative inputs.
            atol = 3e-7 if kind in (K.UN_GELU, K.UN_GELU_ERF, K.UN_GELU_ERF_GRAD, K.UN_TANH) else 1e-37
            assert_close(run_unary(be, kind, x), fo.unary(kind, x), ELT_RTOL, atol, f"kind {kind} n {n}")
    x = np.abs(special_vals(5, 100003))
    for p in (1.5, 2.5, 0.3, -1.7):
        assert_close(run_unary(be, K.UN_POWF, x, p), fo.unary(K.UN_POWF, x, p), ELT_RTOL, 1e-37, f"powf {p}")
    neg = special_vals(6, 4099)
    got, want = run_unary(be, K.UN_POWF, neg, 1.5), fo.unary(K.UN_POWF, neg, 1.5)
    assert (np.isnan(got) == np.isnan(want)).all()
    assert_close(got, want, ELT_RTOL, 1e-37, "powf 1.5 on mixed signs")


def _logspace_signed(lo_exp, hi_exp, per_decade=400, seed=0):
    """Both signs of magnitudes spread evenly in the exponent from 10^lo_exp to 10^hi_exp, jittered."""
    r = np.random.default_rng(seed)
    n = int((hi_exp - lo_exp) * per_decade)
    e = np.linspace(lo_exp, hi_exp, n) + r.uniform(-0.5, 0.5, n) / per_decade
    m = (10.0 ** e).astype(np.float32)
    return np.concatenate([m, -m]).astype(np.float32)


def _assert_rel(got, want, rtol, cond_atol=None, ctx=""):
    """Relative bar with no absolute term, except (a) where the oracle's result is subnormal, which may be off
    by two subnormal quanta, and (b) an explicit per-element conditioning term for kinds whose value is a
    difference of larger terms (the oracle's own f32 result is only defined to that term's rounding)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert (np.isnan(got) == np.isnan(want)).all(), f"{ctx}: NaN masks differ"
    inf = np.isinf(want)
    assert (got[inf] == want[inf]).all(), f"{ctx}: infinities differ"
    m = ~(np.isnan(want) | inf)
    tiny = np.float64(np.finfo(np.float32).tiny)
    bound = rtol * np.abs(want) + np.where(np.abs(want) < tiny, 2 * 2.0 ** -149, 0.0)
    if cond_atol is not None:
        bound = bound + cond_atol
    err = np.abs(got - want)
    bad = m & (err > bound)
    assert not bad.any(), (f"{ctx}: {int(bad.sum())} off; worst rel {np.max(err[m] / (np.abs(want[m]) + 1e-300)):.3e} "
                           f"at want={want[bad][:3]} got={got[bad][:3]}")


def test_transcendental_kinds_over_their_whole_input_ranges(be):
    """exp to +-88 and into the subnormal results, tanh / sigmoid / silu / gelu to +-20 and across the
    0.25 switch of the two-branch tanh, log and powf(., 1.5) over 1e-38 .. 1e38: 1e-5 relative to the
    oracle with no absolute term (see _assert_rel for the two stated exceptions)."""
    f32 = np.float32
    # exp: log-spaced magnitudes up to the overflow bound, a dense sweep of the last decade, and the
    # inputs whose results are subnormal (-103.9 .. -87.3).
    x = np.concatenate([_logspace_signed(-6, np.log10(88.0)), np.linspace(-88.7, 88.7, 40001).astype(f32),
                        np.linspace(-104.0, -87.0, 4001).astype(f32)])
    _assert_rel(run_unary(be, K.UN_EXP, x), fo.unary(K.UN_EXP, x), ELT_RTOL, ctx="exp")
    # tanh-family inputs
    x = np.concatenate([_logspace_signed(-8, np.log10(20.0)), np.linspace(-20, 20, 40001).astype(f32),
                        np.linspace(0.2, 0.3, 20001).astype(f32), -np.linspace(0.2, 0.3, 20001).astype(f32),
                        f32([0.25, -0.25, np.nextafter(f32(0.25), f32(0)), np.nextafter(f32(0.25), f32(1))])])
    _assert_rel(run_unary(be, K.UN_TANH, x), fo.unary(K.UN_TANH, x), ELT_RTOL, ctx="tanh")
    _assert_rel(run_unary(be, K.UN_SIGMOID, x), fo.unary(K.UN_SIGMOID, x), ELT_RTOL, ctx="sigmoid")
    _assert_rel(run_unary(be, K.UN_SILU, x), fo.unary(K.UN_SILU, x), ELT_RTOL, ctx="silu")
    # sigmoid / silu further out: exp(-v) up to the overflow bound
    far = np.concatenate([np.linspace(-88.5, -20, 20001), np.linspace(20, 88.5, 2001)]).astype(f32)
    _assert_rel(run_unary(be, K.UN_SIGMOID, far), fo.unary(K.UN_SIGMOID, far), ELT_RTOL, ctx="sigmoid far")
    _assert_rel(run_unary(be, K.UN_SILU, far), fo.unary(K.UN_SILU, far), ELT_RTOL, ctx="silu far")
    # GELU kinds are 0.5 v (1 + t) with t -> -1 for negative v: ferro's own f32 value is quantised to
    # 0.5 |v| ulp(1), which is the conditioning term allowed on top of the relative bar.
    xd = x.astype(np.float64)
    cond = 0.5 * np.abs(xd) * 2.0 ** -23
    _assert_rel(run_unary(be, K.UN_GELU, x), fo.unary(K.UN_GELU, x), ELT_RTOL, cond, "gelu")
    _assert_rel(run_unary(be, K.UN_GELU_ERF, x), fo.unary(K.UN_GELU_ERF, x), ELT_RTOL, cond, "gelu_erf")
    # its derivative is Phi(v) + v phi(v), two terms of opposite sign for v < 0 (zero near -0.75)
    cond_g = (0.5 + np.abs(xd) * np.exp(-0.5 * xd * xd) * 0.39894228) * 2.0 ** -23
    _assert_rel(run_unary(be, K.UN_GELU_ERF_GRAD, x), fo.unary(K.UN_GELU_ERF_GRAD, x), ELT_RTOL, cond_g, "gelu_erf_grad")
    # log and powf(., 1.5) over the whole positive range, powf on both signs for the NaN mask
    pos = np.abs(_logspace_signed(-38, 38, per_decade=300, seed=3))
    near1 = np.linspace(0.5, 2.0, 30001).astype(f32)
    for arr, what in ((pos, "1e-38..1e38"), (near1, "around 1")):
        _assert_rel(run_unary(be, K.UN_LOG, arr), fo.unary(K.UN_LOG, arr), ELT_RTOL, ctx=f"log {what}")
        _assert_rel(run_unary(be, K.UN_POWF, arr, 1.5), fo.unary(K.UN_POWF, arr, 1.5), ELT_RTOL, ctx=f"powf 1.5 {what}")
    both = _logspace_signed(-38, 38, per_decade=50, seed=4)
    got, want = run_unary(be, K.UN_POWF, both, 1.5), fo.unary(K.UN_POWF, both, 1.5)
    assert (np.isnan(got) == (both < 0)).all() and (np.isnan(want) == (both < 0)).all()
    # the backward kinds that lean on the same approximations
    g = np.random.default_rng(5).standard_normal(pos.size).astype(f32)
    _assert_rel(run_binary(be, K.BIN_POWF_BWD, g, pos, 1.5), fo.binary(K.BIN_POWF_BWD, g, pos, 1.5), ELT_RTOL, ctx="powf 1.5 bwd")
    _assert_rel(run_binary(be, K.BIN_POWF_BWD, g, pos, 2.5), fo.binary(K.BIN_POWF_BWD, g, pos, 2.5), ELT_RTOL, ctx="powf 2.5 bwd")


def test_binary_kinds(be):
    for kind in (K.BIN_ADD, K.BIN_SUB, K.BIN_MUL, K.BIN_DIV, K.BIN_RELU_BACKWARD, K.BIN_SIGMOID_BWD,
                 K.BIN_SQRT_BWD, K.BIN_ABS_BWD, K.BIN_LOG_BWD, K.BIN_TANH_BWD):
        for n in LENGTHS:
            a, b = special_vals(n * 11 + kind, n), special_vals(n * 13 + kind + 1, n)
            assert_bitwise(run_binary(be, kind, a, b), fo.binary(kind, a, b), f"kind {kind} n {n}")
    incoming = np.float32([np.nan, np.inf, -np.inf, np.nan, -0.0, -7.0, np.inf, 2.0, np.nan])
    inputs = np.float32([-1.0, 0.0, -0.0, 1.0, np.nan, np.inf, -np.inf, 2.0, np.nan])
    assert_bitwise(run_binary(be, K.BIN_RELU_BACKWARD, incoming, inputs),
                   np.float32([0.0, 0.0, 0.0, np.nan, -0.0, -7.0, 0.0, 2.0, np.nan]))
    for p in (2.0, 3.0, 0.5, 1.5, 2.5, 0.0):
        a, x = special_vals(1, 4099), np.abs(special_vals(2, 4099))
        assert_close(run_binary(be, K.BIN_POWF_BWD, a, x, p), fo.binary(K.BIN_POWF_BWD, a, x, p), ELT_RTOL, 1e-37)


def test_unaligned_buffers_take_the_scalar_path(be):
    b = B()
    x = special_vals(4, 4099)
    big = be.alloc_from_host(np.concatenate([[0.0], x]).astype(np.float32))
    view = b.DeviceBuffer(big.t[1:])  # 4-byte aligned only
    assert_bitwise(be.copy_to_host(be.unary_dev(b.UnaryKind.Relu, view)), fo.unary(K.UN_RELU, x))
    assert_bitwise(be.copy_to_host(be.binary_dev(b.BinaryKind.Mul, view, view)), fo.binary(K.BIN_MUL, x, x))


def test_inplace_family(be):
    b = B()
    x, y = special_vals(1, 100003), special_vals(2, 100003)
    d = be.alloc_from_host(x)
    be.affine_inplace_dev(d, 1.5, -0.25)
    want = x.copy()
    fo.affine_inplace(want, 1.5, -0.25)
    assert_bitwise(be.copy_to_host(d), want, "affine")
    d = be.alloc_from_host(x)
    be.axpy_inplace_dev(-0.1, d, be.alloc_from_host(y))
    want = x.copy()
    fo.axpy_inplace(-0.1, want, y)
    assert_bitwise(be.copy_to_host(d), want, "axpy")
    for kind in (b.BinaryKind.Add, b.BinaryKind.Sub, b.BinaryKind.Mul, b.BinaryKind.Div, b.BinaryKind.ReluBackward):
        d = be.alloc_from_host(x)
        be.binary_inplace_dev(kind, d, be.alloc_from_host(y))
        assert_bitwise(be.copy_to_host(d), fo.binary(kind.code, x, y), f"inplace {kind.code}")
    d = be.alloc_from_host(x)
    be.binary_inplace_dev(b.BinaryKind.Add, d, d)  # dst may be src (dispatch.rs:438-441)
    assert_bitwise(be.copy_to_host(d), fo.binary(K.BIN_ADD, x, x), "aliased add")
    assert_bitwise(be.copy_to_host(be.fill_dev(3.25, 1027)), np.full(1027, 3.25, np.float32))
    assert_bitwise(be.copy_to_host(be.copy_dev(be.alloc_from_host(x))), x)
    assert len(be.unary_dev(b.UnaryKind.Exp, be.alloc_from_host(np.zeros(0, np.float32)))) == 0


def test_gather_rows_bit_exact_and_range_checked(be):
    b = B()
    r = np.random.default_rng(0)
    for inner in (1, 3, 8, 64, 300):
        w = r.standard_normal((50, inner)).astype(np.float32)
        idx = r.integers(0, 50, 1000)
        out = be.gather_rows_dev(be.alloc_from_host(w), be.alloc_i64_from_host(idx), 50, inner)
        assert_bitwise(be.copy_to_host(out).reshape(-1, inner), w[idx])
    with pytest.raises(b.InvalidShape):
        be.gather_rows_dev(be.alloc_from_host(w), be.alloc_i64_from_host([0, 50]), 50, 300)
    with pytest.raises(b.InvalidShape):
        be.gather_rows_dev(be.alloc_from_host(w), be.alloc_i64_from_host([-1]), 50, 300)


# ---------------------------------------------------------- broadcast / strided
def test_binary_bc_shapes(be):
    b = B()
    r = np.random.default_rng(1)
    cases = [((8, 1024), (1024,)), ((3, 1, 5), (4, 1)), ((), (2, 3)), ((2, 3), ()), ((64, 64), (64, 1)),
             ((2, 0, 3), (3,)), ((5, 7), (5, 7)), ((4, 3, 8), (1, 3, 1)), ((1, 1030), (6, 1)),
             ((2, 3, 4, 5, 6), (3, 1, 5, 1))]
    for sa, sb in cases:
        a = r.standard_normal(sa).astype(np.float32)
        bb = r.standard_normal(sb).astype(np.float32)
        out_shape = np.broadcast_shapes(sa, sb)
        for kind in (b.BinaryKind.Add, b.BinaryKind.Div):
            got = be.copy_to_host(be.binary_bc_dev(kind, be.alloc_from_host(a), sa, be.alloc_from_host(bb), sb, out_shape))
            assert_bitwise(got.reshape(out_shape), fo.binary_bc(kind.code, a, bb), f"{sa} {sb}")
    with pytest.raises(b.InvalidShape):
        be.binary_bc_dev(b.BinaryKind.Add, be.alloc_from_host(np.zeros(6)), (2, 3), be.alloc_from_host(np.zeros(4)), (4,), (2, 3))


def test_views_stay_on_the_device(be):
    b = B()
    r = np.random.default_rng(2)
    a = r.standard_normal((37, 53)).astype(np.float32)
    A = be.alloc_from_host(a)
    # transpose: swapped shape and strides (tensor.rs:1206-1227)
    got = be.copy_to_host(be.materialize_dev(A, (53, 37), (1, 53), 0)).reshape(53, 37)
    assert_bitwise(got, a.T)
    got = be.copy_to_host(be.unary_strided_dev(b.UnaryKind.Exp, b.View(A, (1, 53), 0), (53, 37))).reshape(53, 37)
    assert_close(got, fo.unary(K.UN_EXP, a.T), ELT_RTOL)
    # slice with an offset, rows 3..10 cols 5..25 step 2
    got = be.copy_to_host(be.materialize_dev(A, (7, 10), (53, 2), 3 * 53 + 5)).reshape(7, 10)
    assert_bitwise(got, a[3:10, 5:25:2])
    # f(a, a^T) on a square matrix, and against a column broadcast
    s = r.standard_normal((96, 96)).astype(np.float32)
    S = be.alloc_from_host(s)
    got = be.copy_to_host(be.binary_strided_dev(b.BinaryKind.Sub, b.View(S, (96, 1)), b.View(S, (1, 96)), (96, 96)))
    assert_bitwise(got.reshape(96, 96), s - s.T)
    # every rank up to 8 with odd extents and a permuted operand
    for rank in range(1, 9):
        shape = [2 + (i % 3) for i in range(rank)]
        x = r.standard_normal(shape).astype(np.float32)
        perm = list(reversed(range(rank)))
        xt = np.ascontiguousarray(x.transpose(perm))  # storage holds the permuted tensor
        st = [0] * rank
        acc = 1
        for ax in reversed(range(rank)):  # strides of xt's storage, mapped back to x's axis order
            st[perm[ax]] = acc
            acc *= xt.shape[ax]
        got = be.copy_to_host(be.materialize_dev(be.alloc_from_host(xt), shape, st, 0)).reshape(shape)
        assert_bitwise(got, x, f"rank {rank}")
    with pytest.raises(b.InvalidShape):
        be.materialize_dev(A, (53, 38), (1, 53), 0)  # reaches outside the storage


def test_chain_programs(be):
    b = B()
    S, U, Bi = b.ChainStep, b.UnaryKind, b.BinaryKind
    r = np.random.default_rng(3)
    # ferro's own chain form: relu(x)*y+z, all whole (docs/FUSION_3090.md chain)
    n = (1 << 16) + 5
    x, y, z = (r.standard_normal(n).astype(np.float32) for _ in range(3))
    prog = [S.Load(0), S.Unary(U.Relu), S.Binary(Bi.Mul, other=1), S.Binary(Bi.Add, other=2)]
    got = be.copy_to_host(be.chain_dev(prog, [be.alloc_from_host(v) for v in (x, y, z)]))
    assert_bitwise(got, fo.binary(K.BIN_ADD, fo.binary(K.BIN_MUL, fo.unary(K.UN_RELU, x), y), z))
    # relu(x + b) * s with a row-broadcast bias and an immediate scale
    rows, cols = 33, 1024
    xm, bias = r.standard_normal((rows, cols)).astype(np.float32), (0.1 * r.standard_normal(cols)).astype(np.float32)
    prog = [S.Load(0), S.Binary(Bi.Add, other=1), S.Unary(U.Relu), S.Binary(Bi.Mul, imm=0.125)]
    got = be.copy_to_host(be.chain_dev(prog, [b.View(be.alloc_from_host(xm), (cols, 1)), b.View(be.alloc_from_host(bias), (0, 1))], (rows, cols)))
    want = fo.binary(K.BIN_MUL, fo.unary(K.UN_RELU, fo.binary_bc(K.BIN_ADD, xm, bias)), np.full((rows, cols), 0.125, np.float32))
    assert_bitwise(got.reshape(rows, cols), want)
    # z = clamp(tanh(exp(-abs(a)) * sqrt(abs(b)+1)) + powf(a^T, 1.5), -1, 1), b a column, a^T a zero-copy view
    for n in (64, 100):
        a = r.uniform(-4, 4, (n, n)).astype(np.float32)
        col = r.uniform(-4, 4, (n, 1)).astype(np.float32)
        A, C_ = be.alloc_from_host(a), be.alloc_from_host(col)
        prog = [S.Load(0), S.Unary(U.Abs), S.Unary(U.Neg), S.Unary(U.Exp),
                S.Load(1, dst=b.T), S.Unary(U.Abs, dst=b.T), S.Binary(Bi.Add, imm=1.0, dst=b.T), S.Unary(U.Sqrt, dst=b.T),
                S.Binary(Bi.Mul), S.Unary(U.Tanh),
                S.Load(2, dst=b.T), S.Unary(U.Powf(1.5), dst=b.T), S.Binary(Bi.Add),
                S.Unary(U.Clamp(-1.0, 1.0))]
        got = be.copy_to_host(be.chain_dev(prog, [b.View(A, (n, 1)), b.View(C_, (1, 0)), b.View(A, (1, n))], (n, n))).reshape(n, n)
        t1 = fo.unary(K.UN_EXP, fo.unary(K.UN_NEG, fo.unary(K.UN_ABS, a)))
        t2 = fo.unary(K.UN_SQRT, fo.binary_bc(K.BIN_ADD, fo.unary(K.UN_ABS, col), np.float32(1.0).reshape(())))
        t3 = fo.unary(K.UN_TANH, fo.binary_bc(K.BIN_MUL, t1, t2))
        t4 = fo.unary(K.UN_POWF, np.ascontiguousarray(a.T), 1.5)
        want = fo.unary(K.UN_CLAMP, fo.binary(K.BIN_ADD, t3, t4), -1.0, 1.0)
        assert (np.isnan(got) == np.isnan(want)).all()  # NaN mask exact
        assert_close(got, want, ELT_RTOL, 1e-6, f"config-4 chain n={n}")
    # swap: dst = rhs - dst
    prog = [S.Load(0), S.Binary(Bi.Sub, other=1, swap=True)]
    got = be.copy_to_host(be.chain_dev(prog, [be.alloc_from_host(x), be.alloc_from_host(y)]))
    assert_bitwise(got, y - x)
    with pytest.raises(b.InvalidArgument):
        be.chain_dev([S.Unary(U.Relu)], [be.alloc_from_host(x)])


def test_compiled_chain_programs_equal_the_interpreter_bit_for_bit(be):
    """Every chain of the build-time manifest (csrc/chain_programs.def) against the same call on the
    interpreter (fb_chain_catalogue off): identical bits, on the segment kernel, the general tile
    kernel (extents that are not multiples of the tile) and its interior form (multiples of 64)."""
    b = B()
    S, U, Bi, Tr = b.ChainStep, b.UnaryKind, b.BinaryKind, b.T
    r = np.random.default_rng(33)

    def both(prog, views, shape):
        prev = be.lib.fb_chain_catalogue(1)
        try:
            fast = be.copy_to_host(be.chain_dev(prog, views, shape))
            be.lib.fb_chain_catalogue(0)
            slow = be.copy_to_host(be.chain_dev(prog, views, shape))
        finally:
            be.lib.fb_chain_catalogue(prev)
        assert_bitwise(fast, slow)
        return fast

    rows, cols = 40, 4096
    x, y, z = (be.alloc_from_host(r.standard_normal((rows, cols)).astype(np.float32) * 3) for _ in range(3))
    whole = lambda buf: b.View(buf, (cols, 1))
    gate = [S.Load(0), S.Unary(U.Sigmoid), S.Binary(Bi.Mul, other=1), S.Binary(Bi.Add, other=2)]
    got = both(gate, [whole(x), whole(y), whole(z)], (rows, cols))
    xh, yh, zh = (be.copy_to_host(v) for v in (x, y, z))
    assert_close(got, fo.binary(K.BIN_ADD, fo.binary(K.BIN_MUL, fo.unary(K.UN_SIGMOID, xh), yh), zh), ELT_RTOL, 1e-6)
    squash = [S.Load(0), S.Binary(Bi.Mul, imm=0.37), S.Binary(Bi.Add, other=1), S.Unary(U.Tanh)]
    got = both(squash, [whole(x), whole(y)], (rows, cols))
    want = fo.unary(K.UN_TANH, fo.binary(K.BIN_ADD, fo.binary(K.BIN_MUL, xh, np.full_like(xh, 0.37)), yh))
    assert_close(got, want, ELT_RTOL, 1e-7)
    for prog in ([S.Load(0), S.Unary(U.Relu), S.Binary(Bi.Mul, other=1), S.Binary(Bi.Add, other=2)],
                 [S.Load(0), S.Binary(Bi.Add, other=1), S.Unary(U.Relu), S.Binary(Bi.Mul, imm=0.125)],
                 [S.Load(0), S.Binary(Bi.Add, other=1), S.Unary(U.Relu)],
                 [S.Load(0), S.Binary(Bi.Add, other=1)], [S.Load(0), S.Binary(Bi.Mul, other=1)], [S.Load(0)]):
        both(prog, [whole(x), whole(y), whole(z)][:max(1, sum(1 for st in prog if st.opcode == 0 or st.src >= 8))], (rows, cols))
    # tile kernels: a + a^T, a^T alone, and the gate-clamp chain, at an interior size and a ragged one
    gc = [S.Load(0), S.Unary(U.Abs), S.Unary(U.Neg), S.Unary(U.Exp), S.Load(1, dst=Tr), S.Unary(U.Abs, dst=Tr),
          S.Binary(Bi.Add, imm=1.0, dst=Tr), S.Unary(U.Sqrt, dst=Tr), S.Binary(Bi.Mul), S.Unary(U.Tanh),
          S.Load(2, dst=Tr), S.Unary(U.Powf(1.5), dst=Tr), S.Binary(Bi.Add), S.Unary(U.Clamp(-1.0, 1.0))]
    for n in (256, 320, 200):
        a = r.uniform(-4, 4, (n, n)).astype(np.float32)
        col = r.uniform(-4, 4, (n, 1)).astype(np.float32)
        A, C_ = be.alloc_from_host(a), be.alloc_from_host(col)
        got = both(gc, [b.View(A, (n, 1)), b.View(C_, (1, 0)), b.View(A, (1, n))], (n, n)).reshape(n, n)
        assert (np.isnan(got) == (a.T < 0)).all()
        got = both([S.Load(0), S.Binary(Bi.Add, other=1)], [b.View(A, (n, 1)), b.View(A, (1, n))], (n, n)).reshape(n, n)
        assert_bitwise(got, a + a.T)
        got = both([S.Load(0), S.Binary(Bi.Add, other=1)], [b.View(A, (1, n)), b.View(A, (n, 1))], (n, n)).reshape(n, n)
        assert_bitwise(got, a.T + a)
        assert_bitwise(both([S.Load(0)], [b.View(A, (1, n))], (n, n)).reshape(n, n), np.ascontiguousarray(a.T))
    # a rectangular interior case: [128, 192] output, operand 1 the transposed one
    m, n = 128, 192
    p, q = r.standard_normal((m, n)).astype(np.float32), r.standard_normal((n, m)).astype(np.float32)
    got = both([S.Load(0), S.Binary(Bi.Add, other=1)], [b.View(be.alloc_from_host(p), (n, 1)), b.View(be.alloc_from_host(q), (1, m))], (m, n))
    assert_bitwise(got.reshape(m, n), p + q.T)


# ------------------------------------------------------------------- reductions
def test_full_reduce(be):
    b = B()
    r = np.random.default_rng(4)
    for n in (1, 7, 1000, 4096, (1 << 20) + 3):
        x = r.standard_normal(n).astype(np.float32)
        s = be.copy_to_host(be.reduce_dev(b.ReduceKind.Sum, be.alloc_from_host(x)))[0]
        m = be.copy_to_host(be.reduce_dev(b.ReduceKind.Mean, be.alloc_from_host(x)))[0]
        scale = np.abs(x).sum()
        assert abs(s - fo.pairwise_sum(x)) <= RED_RTOL * abs(fo.pairwise_sum(x)) + 1e-6 * scale
        assert abs(m - fo.mean(x)) <= RED_RTOL * abs(fo.mean(x)) + 1e-6 * scale / n
    empty = be.alloc_from_host(np.zeros(0, np.float32))
    assert be.copy_to_host(be.reduce_dev(b.ReduceKind.Sum, empty))[0] == 0.0
    assert np.isnan(be.copy_to_host(be.reduce_dev(b.ReduceKind.Mean, empty))[0])  # lib.rs:1197
    # adversarial magnitudes (tests/reduce_accuracy.rs): stay within 1e-4*sqrt(n) of the f64 sum like gpu_integration.rs:208-231
    mags = (10.0 ** r.uniform(-6, 6, 100000) * r.choice([-1, 1], 100000)).astype(np.float32)
    got = be.copy_to_host(be.reduce_dev(b.ReduceKind.Sum, be.alloc_from_host(mags)))[0]
    assert abs(got - mags.astype(np.float64).sum()) <= 1e-6 * np.abs(mags).sum()


def test_sum_mean_dim_every_axis(be):
    r = np.random.default_rng(5)
    shapes = [(2, 3), (4, 6, 8), (7, 130, 33), (3, 5, 64), (1, 300, 257), (33, 4100), (5, 2, 3, 4), (64, 2048),
              (2048, 64), (16, 40, 128), (9, 1), (1, 9), (3, 0, 4), (0, 5)]
    for shape in shapes:
        x = r.standard_normal(shape).astype(np.float32)
        X = be.alloc_from_host(x)
        for dim in range(len(shape)):
            for name, dev, ref in (("sum", be.sum_dim_dev, fo.sum_dim), ("mean", be.mean_dim_dev, fo.mean_dim)):
                got = be.copy_to_host(dev(X, shape, dim))
                if shape[dim] == 0 or x.size == 0:
                    want = np.zeros_like(got) if name == "sum" else np.full_like(got, np.nan)
                    assert_bitwise(got, want.ravel(), f"{name} {shape} dim {dim}")
                    continue
                want = ref(x, dim).ravel()
                atol = 1e-6 * np.abs(x).sum(axis=dim).max() / (shape[dim] if name == "mean" else 1)
                assert_close(got, want, RED_RTOL, atol, f"{name} {shape} dim {dim}")
    a = np.float32([[1, 2, 3], [4, 5, 6]])  # tests/op_sum_dim.rs:5-16
    assert_bitwise(be.copy_to_host(be.sum_dim_dev(be.alloc_from_host(a), (2, 3), 0)), np.float32([5, 7, 9]))
    assert_bitwise(be.copy_to_host(be.sum_dim_dev(be.alloc_from_host(a), (2, 3), 1)), np.float32([6, 15]))


def test_max_dim_values_and_indices_bit_exact(be):
    b = B()
    r = np.random.default_rng(6)
    shapes = [(2, 3), (4, 6, 8), (7, 130, 33), (3, 5, 64), (1, 300, 257), (33, 4100), (64, 2048), (2048, 64), (9, 1), (1, 9), (20000,)]
    for shape in shapes:
        x = r.integers(-5, 5, shape).astype(np.float32)  # many ties
        x[r.random(shape) < 0.002] = np.nan
        X = be.alloc_from_host(x)
        for dim in range(len(shape)):
            val, idx = be.max_dim_dev(X, shape, dim)
            wi, wv = fo.argmax_dim(x, dim)
            assert (be.copy_i64_to_host(idx) == wi.ravel()).all(), f"{shape} dim {dim}"
            assert_bitwise(be.copy_to_host(val), wv.ravel(), f"{shape} dim {dim}")
    # tests/op_argmax.rs:5-27
    a = np.float32([[1, 5, 3], [4, 0, 2]])
    assert be.copy_i64_to_host(be.max_dim_dev(be.alloc_from_host(a), (2, 3), 1)[1]).tolist() == [1, 0]
    assert be.copy_i64_to_host(be.max_dim_dev(be.alloc_from_host(a), (2, 3), 0)[1]).tolist() == [1, 0, 0]
    assert be.copy_i64_to_host(be.max_dim_dev(be.alloc_from_host(np.float32([2, 2, 1])), (3,), 0)[1]).tolist() == [0]
    assert be.copy_i64_to_host(be.max_dim_dev(be.alloc_from_host(np.float32([1, np.nan, 9])), (3,), 0)[1]).tolist() == [1]
    with pytest.raises(b.InvalidShape):
        be.max_dim_dev(be.alloc_from_host(np.zeros(0, np.float32)), (3, 0), 1)


# ---------------------------------------------------------------- softmax family
SOFTMAX_COLS = [1, 2, 3, 4, 8, 16, 20, 31, 32, 33, 48, 64, 96, 100, 128, 160, 192, 252, 256, 1000, 1024, 1028, 4096, 4100, 8193, 32000, 32768, 40000]


def test_softmax_and_log_softmax_forward(be):
    r = np.random.default_rng(7)
    for cols in SOFTMAX_COLS:
        rows = 3 if cols > 8192 else 37
        x = (r.standard_normal((rows, cols)) * 3).astype(np.float32)
        X = be.alloc_from_host(x)
        assert_close(be.copy_to_host(be.softmax_dev(X, rows, cols)).reshape(rows, cols), fo.softmax_fwd(x), RED_RTOL, 1e-30, f"softmax {cols}")
        assert_close(be.copy_to_host(be.log_softmax_dev(X, rows, cols)).reshape(rows, cols), fo.log_softmax_fwd(x), RED_RTOL, 1e-6, f"log_softmax {cols}")
    # tests/op_softmax.rs:5-15
    got = be.copy_to_host(be.softmax_dev(be.alloc_from_host(np.float32([1, 2, 3, 0, 0, 0])), 2, 3))
    assert abs(got[:3].sum() - 1) < 1e-5 and np.all(np.abs(got[3:] - 1 / 3) < 1e-6)
    # large common offsets keep normalisation (tests/op_log_softmax.rs:44-62, gpu_integration.rs:14-25)
    for offset in (1e8, -1e8, 3e38):
        for width in (3, 1024, 4100):
            y = be.copy_to_host(be.log_softmax_dev(be.alloc_from_host(np.full((2, width), offset, np.float32)), 2, width))
            assert np.all(np.abs(y + np.log(np.float32(width))) < 2e-6)
    # NaN and all -inf rows behave like the host loop
    x = (r.standard_normal((4, 64))).astype(np.float32)
    x[1, 5] = np.nan
    x[2, :] = -np.inf
    x[3, 7] = np.inf
    got = be.copy_to_host(be.softmax_dev(be.alloc_from_host(x), 4, 64)).reshape(4, 64)
    want = fo.softmax_fwd(x)
    assert (np.isnan(got) == np.isnan(want)).all()
    assert_close(got[0], want[0], RED_RTOL)


def test_softmax_short_rows_many_rows(be):
    """Rows shorter than 256 columns go several to a warp (4, 8 or 16 lanes per row, 2 .. 4 float4 per lane):
    enough rows for many CTAs and a ragged last block, masked (-inf) entries and a fully masked row included."""
    r = np.random.default_rng(81)
    rows = 5003
    for cols in (8, 12, 32, 64, 72, 96, 128, 192, 200, 252):
        x = (r.standard_normal((rows, cols)) * 3).astype(np.float32)
        x[7, : cols // 2] = -np.inf
        x[11, :] = -np.inf
        x[rows - 1, cols - 1] = -np.inf
        g = r.standard_normal((rows, cols)).astype(np.float32)
        X, G = be.alloc_from_host(x), be.alloc_from_host(g)
        y, ly = fo.softmax_fwd(x), fo.log_softmax_fwd(x)
        got = be.copy_to_host(be.softmax_dev(X, rows, cols)).reshape(rows, cols)
        assert (np.isnan(got) == np.isnan(y)).all(), cols
        ok = ~np.isnan(y).any(1)
        assert_close(got[ok], y[ok], RED_RTOL, 1e-30, f"softmax {rows}x{cols}")
        got = be.copy_to_host(be.log_softmax_dev(X, rows, cols)).reshape(rows, cols)
        assert (np.isnan(got) == np.isnan(ly)).all(), cols
        fin = np.isfinite(ly)
        assert (got[~fin & ~np.isnan(ly)] == -np.inf).all(), cols
        assert_close(got[fin], ly[fin], RED_RTOL, 1e-6, f"log_softmax {rows}x{cols}")
        x = (r.standard_normal((rows, cols)) * 2).astype(np.float32)
        y, ly = fo.softmax_fwd(x), fo.log_softmax_fwd(x)
        dx = be.copy_to_host(be.softmax_backward_dev(G, be.alloc_from_host(y), rows, cols)).reshape(rows, cols)
        want = fo.softmax_bwd(g, y)
        assert_close(dx, want, RED_RTOL, 2e-4 * np.abs(want).max(), f"softmax bwd {rows}x{cols}")
        dx = be.copy_to_host(be.log_softmax_backward_dev(G, be.alloc_from_host(ly), rows, cols)).reshape(rows, cols)
        want = fo.log_softmax_bwd(g, ly)
        assert_close(dx, want, RED_RTOL, 2e-4 * np.abs(g).max(), f"log_softmax bwd {rows}x{cols}")


def test_minus_inf_entries_in_rows_that_take_the_streaming_kernels(be):
    """Masked entries (-inf next to finite values: masked vocabulary, left-padded attention rows) in rows long
    enough for the one-pass streaming folds: the result is finite wherever the host loop's is.  -inf is
    planted at the row head, over the whole first float4 of every thread, and at scattered thread-leading
    positions; aligned and unaligned widths."""
    r = np.random.default_rng(21)

    def plant(x):
        cols = x.shape[1]
        x[0, 0] = -np.inf                                     # the row head
        x[1, :min(4 * 512, cols - 1)] = -np.inf               # every thread's first float4 (512 threads)
        x[2, :min(16 * 512, cols - 1)] = -np.inf              # the first unrolled round of every thread
        x[3, r.integers(0, cols, cols // 3)] = -np.inf        # scattered
        x[3, 0:8] = -np.inf
        x[4, :] = -np.inf                                     # a fully masked row: NaN, like the host loop
        x[5, 4:9] = -np.inf                                   # thread 1's leading float4, and a straddle
        return x

    for cols in (16388, 20000, 32768, 40000, 20001):
        x = plant((r.standard_normal((7, cols)) * 3).astype(np.float32))
        X = be.alloc_from_host(x)
        got = be.copy_to_host(be.softmax_dev(X, 7, cols)).reshape(7, cols)
        want = fo.softmax_fwd(x)
        assert np.isfinite(want[[0, 1, 2, 3, 5, 6]]).all() and np.isnan(want[4]).all()
        assert_close(got, want, RED_RTOL, 1e-30, f"softmax {cols}")
        got = be.copy_to_host(be.log_softmax_dev(X, 7, cols)).reshape(7, cols)
        assert_close(got, fo.log_softmax_fwd(x), RED_RTOL, 1e-6, f"log_softmax {cols}")
    for cols in (2048, 2049, 8192, 8193, 32000, 32001):
        x = plant((2 * r.standard_normal((7, cols))).astype(np.float32))
        t = np.array([int(np.flatnonzero(np.isfinite(row))[-1]) if np.isfinite(row).any() else 0 for row in x])
        L, T = be.alloc_from_host(x), be.alloc_i64_from_host(t)
        loss, saved, am = be.cross_entropy_indices_dev(L, T, 7, cols)
        be.check_targets()
        keep = [0, 1, 2, 3, 5, 6]
        _, wd, wa = fo.cross_entropy_indices(x[keep], t[keep])
        # ferro's one-hot composition (nn.rs:380-400) multiplies the -inf log-probabilities by the
        # zeros of the one-hot matrix and so reports NaN for such a batch; the gather formulation
        # (ferro's Python functional.cross_entropy, functional.py:419-444) is finite, and that is
        # what the fused entry computes: -mean(logp[r, t_r]) on the oracle's log_softmax.
        lp = fo.log_softmax_fwd(x[keep])
        wl = np.float32(-np.mean(lp[np.arange(len(keep)), t[keep]].astype(np.float64)))
        assert np.isfinite(wl) and np.isfinite(wd).all()
        # per-row statistics of the finite rows are finite and the argmax is bit-exact
        rmax, rlse = (be.copy_to_host(b) for b in saved)
        assert np.isfinite(rmax[keep]).all() and np.isfinite(rlse[keep]).all(), cols
        assert (be.copy_i64_to_host(am)[keep] == wa).all(), cols
        assert np.isnan(be.copy_to_host(loss)[0])             # the fully masked row poisons the mean, as on the host
        # the same rows without the masked one: loss and gradient against the oracle
        L2, T2 = be.alloc_from_host(x[keep]), be.alloc_i64_from_host(t[keep])
        loss2, saved2, _ = be.cross_entropy_indices_dev(L2, T2, 6, cols)
        assert abs(be.copy_to_host(loss2)[0] - wl) <= RED_RTOL * abs(wl), cols
        dl = be.copy_to_host(be.cross_entropy_indices_backward_dev(L2, T2, saved2, 6, cols)).reshape(6, cols)
        assert_close(dl, wd, RED_RTOL, 2e-4 / 6 * 1e-3, f"dlogits {cols}")
        assert (dl[np.isneginf(x[keep])] == 0).all()


def test_softmax_and_log_softmax_backward(be):
    r = np.random.default_rng(8)
    for cols in SOFTMAX_COLS:
        rows = 3 if cols > 8192 else 29
        x = (r.standard_normal((rows, cols)) * 2).astype(np.float32)
        g = r.standard_normal((rows, cols)).astype(np.float32)
        y, ly = fo.softmax_fwd(x), fo.log_softmax_fwd(x)
        G = be.alloc_from_host(g)
        dx = be.copy_to_host(be.softmax_backward_dev(G, be.alloc_from_host(y), rows, cols)).reshape(rows, cols)
        want = fo.softmax_bwd(g, y)
        assert_close(dx, want, RED_RTOL, 2e-4 * np.abs(want).max(), f"softmax bwd {cols}")
        dx = be.copy_to_host(be.log_softmax_backward_dev(G, be.alloc_from_host(ly), rows, cols)).reshape(rows, cols)
        want = fo.log_softmax_bwd(g, ly)
        assert_close(dx, want, RED_RTOL, 2e-4 * np.abs(g).max(), f"log_softmax bwd {cols}")
    # rows wider than 16384 columns are shared by a cluster of CTAs (2 x 16384, 4 x 12500, 4 x 16384, 8 x 16384
    # with a short last slice); enough rows for every cluster to take several
    for rows, cols in [(331, 32768), (200, 50000), (160, 65536), (150, 131068)]:
        x = (r.standard_normal((rows, cols)) * 2).astype(np.float32)
        g = r.standard_normal((rows, cols)).astype(np.float32)
        y, ly = fo.softmax_fwd(x), fo.log_softmax_fwd(x)
        G = be.alloc_from_host(g)
        dx = be.copy_to_host(be.softmax_backward_dev(G, be.alloc_from_host(y), rows, cols)).reshape(rows, cols)
        want = fo.softmax_bwd(g, y)
        assert_close(dx, want, RED_RTOL, 2e-4 * np.abs(want).max(), f"softmax bwd {rows}x{cols}")
        dx = be.copy_to_host(be.log_softmax_backward_dev(G, be.alloc_from_host(ly), rows, cols)).reshape(rows, cols)
        want = fo.log_softmax_bwd(g, ly)
        assert_close(dx, want, RED_RTOL, 2e-4 * np.abs(g).max(), f"log_softmax bwd {rows}x{cols}")
    assert be.lib.fb_device_faults(0) == 0
    # grads [-1, 0, 1]-style check of op_log_softmax.rs:56-60
    seed = np.array([(i % 5) - 2.0 for i in range(12)], np.float32).reshape(4, 3)
    y = fo.log_softmax_fwd(np.full((4, 3), 1e8, np.float32))
    dx = be.copy_to_host(be.log_softmax_backward_dev(be.alloc_from_host(seed), be.alloc_from_host(y), 4, 3)).reshape(4, 3)
    assert np.all(np.abs(dx - (seed - seed.sum(1, keepdims=True) / 3)) < 2e-6)


def test_fused_bias_relu_scale_softmax(be):
    r = np.random.default_rng(9)
    for rows, cols in [(64, 1024), (37, 1000), (5, 33), (300, 128), (9, 4096)]:
        x = r.standard_normal((rows, cols)).astype(np.float32)
        bias = (0.1 * r.standard_normal(cols)).astype(np.float32)
        g = r.standard_normal((rows, cols)).astype(np.float32)
        s = np.float32(0.125)
        pre = fo.binary_bc(K.BIN_ADD, x, bias)
        t = fo.binary(K.BIN_MUL, fo.unary(K.UN_RELU, pre), np.full_like(x, s))
        y_want = fo.softmax_fwd(t)
        X, Bb, G = be.alloc_from_host(x), be.alloc_from_host(bias), be.alloc_from_host(g)
        Y = be.bias_act_scale_softmax_dev(X, Bb, True, float(s), rows, cols)
        assert_close(be.copy_to_host(Y).reshape(rows, cols), y_want, RED_RTOL, 1e-30, f"fwd {rows}x{cols}")
        # backward through softmax -> mul(s) -> relu -> add(bias), unbroadcast for db (ops.rs:19-58, 99-109)
        dt = fo.softmax_bwd(g, y_want)
        dr = fo.binary(K.BIN_MUL, dt, np.full_like(x, s))
        dx_want = fo.binary(K.BIN_RELU_BACKWARD, dr, pre)
        db_want = fo.sum_dim(dx_want, 0).ravel()
        dx, db = be.bias_act_scale_softmax_backward_dev(G, be.alloc_from_host(y_want), X, Bb, True, float(s), rows, cols)
        dxh = be.copy_to_host(dx).reshape(rows, cols)
        assert ((dxh == 0) == (dx_want == 0)).all()  # relu mask exact
        assert_close(dxh, dx_want, RED_RTOL, 2e-4 * np.abs(dx_want).max(), f"dx {rows}x{cols}")
        assert_close(be.copy_to_host(db), db_want, RED_RTOL, 2e-4 * np.abs(dx_want).sum(0).max(), f"db {rows}x{cols}")


def test_cross_entropy_with_i64_targets(be):
    b = B()
    r = np.random.default_rng(10)
    for rows, cols in [(4, 2), (33, 11), (16, 1000), (7, 32000), (3, 40000), (65, 1024), (9, 4099)]:
        logits = (2 * r.standard_normal((rows, cols))).astype(np.float32)
        if cols > 5:
            logits[0, 3] = logits[0, 1] = logits[0].max() + 1  # a tie for the row maximum
        t = r.integers(0, cols, rows)
        L, T = be.alloc_from_host(logits), be.alloc_i64_from_host(t)
        loss, saved, am = be.cross_entropy_indices_dev(L, T, rows, cols)
        be.check_targets()
        wl, wd, wa = fo.cross_entropy_indices(logits, t)
        assert abs(be.copy_to_host(loss)[0] - wl) <= RED_RTOL * abs(wl), (rows, cols)
        assert (be.copy_i64_to_host(am) == wa).all(), (rows, cols)  # bit-exact argmax
        dl = be.copy_to_host(be.cross_entropy_indices_backward_dev(L, T, saved, rows, cols)).reshape(rows, cols)
        assert_close(dl, wd, RED_RTOL, 2e-4 / rows * 1e-3, f"dlogits {rows}x{cols}")
        hot = np.zeros_like(dl, bool)
        hot[np.arange(rows), t] = True
        assert (dl[hot] < 0).all() and (dl[~hot] >= 0).all()  # the one-hot column is the only negative one
    # uniform two-class logits -> ln 2 (tests/nn.rs:18-32)
    loss, _, _ = be.cross_entropy_indices_dev(be.alloc_from_host(np.zeros((4, 2), np.float32)), be.alloc_i64_from_host([0, 1, 1, 0]), 4, 2)
    assert abs(be.copy_to_host(loss)[0] - np.log(2)) < 1e-6
    # NaN in a row: first NaN wins the argmax
    x = r.standard_normal((2, 100)).astype(np.float32)
    x[1, 40] = x[1, 70] = np.nan
    _, _, am = be.cross_entropy_indices_dev(be.alloc_from_host(x), be.alloc_i64_from_host([0, 0]), 2, 100)
    assert be.copy_i64_to_host(am)[1] == 40
    # a class id outside [0, C) is reported, not trapped (nn.rs:419-424)
    be.cross_entropy_indices_dev(be.alloc_from_host(x), be.alloc_i64_from_host([0, 100]), 2, 100)
    with pytest.raises(b.InvalidShape):
        be.check_targets()


# --------------------------------------------------------------------- LayerNorm
LN_COLS = [1, 3, 4, 7, 31, 32, 33, 48, 64, 80, 96, 100, 128, 160, 192, 256, 384, 512, 513, 640, 768, 896, 1024, 1280, 1600, 2048, 2560, 3072, 4096, 4097, 4100, 5120, 6144, 8192, 8193, 8196, 10240, 12288, 16384, 20000, 20001, 32768, 33000,
           140000]


def test_layer_norm_forward_all_outputs(be):
    r = np.random.default_rng(11)
    for cols in LN_COLS:
        rows = 3 if cols > 8192 else 21
        x = (r.standard_normal((rows, cols)) * r.uniform(0.5, 4, (rows, 1))).astype(np.float32)
        w = (1 + 0.02 * r.standard_normal(cols)).astype(np.float32)
        bb = (0.02 * r.standard_normal(cols)).astype(np.float32)
        for affine in range(4):
            ww, bv = (w if affine & 1 else None), (bb if affine & 2 else None)
            W, Bv = (be.alloc_from_host(ww) if ww is not None else None), (be.alloc_from_host(bv) if bv is not None else None)
            X = be.alloc_from_host(x)
            yw, hw, sw, mw = fo.layer_norm_fwd(x, ww, bv, 1e-5)
            y, h, s = be.layer_norm_dev(X, W, Bv, rows, cols, 1e-5)
            atol = 2e-4 if cols > 1 else 1e-6
            assert_close(be.copy_to_host(y).reshape(rows, cols), yw, RED_RTOL, atol * 1e-2 + 1e-6, f"y {cols} affine {affine}")
            assert_close(be.copy_to_host(h).reshape(rows, cols), hw, RED_RTOL, 1e-6, f"h {cols}")
            assert_close(be.copy_to_host(s), sw, RED_RTOL, 0, f"stds {cols}")
            y2, mu, rs = be.layer_norm_stats_dev(X, W, Bv, rows, cols, 1e-5)
            assert_bitwise(be.copy_to_host(y2), be.copy_to_host(y), "stats form gives the same y")
            assert_close(be.copy_to_host(mu), mw, RED_RTOL, 2e-4 * np.abs(x).max() / np.sqrt(cols), f"mean {cols}")
            assert_close(be.copy_to_host(rs), 1 / sw.astype(np.float64), RED_RTOL, 0, f"rstd {cols}")
            assert_bitwise(be.copy_to_host(be.layer_norm_output_dev(X, W, Bv, rows, cols, 1e-5)), be.copy_to_host(y))
    # [1,2,3] -> +-sqrt(1.5) (tests/op_layer_norm.rs:15-22)
    y = be.copy_to_host(be.layer_norm_output_dev(be.alloc_from_host(np.float32([1, 2, 3])), None, None, 1, 3, 1e-5))
    s = np.sqrt(1.5)
    assert np.all(np.abs(y - [-s, 0, s]) < 1e-5)


def test_layer_norm_huge_offsets_match_f64_formula(be):
    """crates/ferro-cuda/tests/layer_norm_fused.rs:28-42, tolerance 2e-6."""
    for cols, offset, step in [(33, 1e8, 8.0), (4097, 1e20, 1e14), (7, 3.0, 0.0), (4096, 1e8, 8.0), (1024, 1e20, 1e14),
                               (16384, 1e8, 8.0), (50000, 1e20, 1e14), (9001, 1e8, 8.0), (140000, 1e20, 1e14)]:
        data = np.array([offset + (i % 19) * step for i in range(2 * cols)], np.float32).reshape(2, cols)
        y = be.copy_to_host(be.layer_norm_output_dev(be.alloc_from_host(data), None, None, 2, cols, 1e-5)).reshape(2, cols)
        d64 = data.astype(np.float64)
        want = (d64 - d64.mean(1, keepdims=True)) / np.sqrt(d64.var(1, keepdims=True) + 1e-5)
        assert np.all(np.abs(y - want) < 2e-6), (cols, offset)


def test_layer_norm_boundaries(be):
    """layer_norm_fused.rs:17-27: shape errors and empty inputs."""
    b = B()
    x = be.alloc_from_host(np.float32([1, 2, 3]))
    for rows, cols in [(1, 0), (2, 3), ((1 << 64) - 1, 2)]:
        with pytest.raises(b.InvalidShape):
            be.layer_norm_dev(x, None, None, rows, cols, 1e-5)
    with pytest.raises(b.InvalidShape):
        be.layer_norm_dev(x, x, None, 3, 1, 1e-5)
    e = be.alloc_from_host(np.zeros(0, np.float32))
    y, h, s = be.layer_norm_dev(e, None, None, 0, 3, 1e-5)
    assert (len(y), len(h), len(s)) == (0, 0, 0)


def test_layer_norm_backward_both_saved_forms(be):
    r = np.random.default_rng(12)
    for cols in LN_COLS:
        for rows in ((2, 5) if cols > 8192 else (1, 19, 700)):
            x = (r.standard_normal((rows, cols)) * r.uniform(0.5, 4, (rows, 1))).astype(np.float32)
            w = (1 + 0.02 * r.standard_normal(cols)).astype(np.float32)
            g = r.standard_normal((rows, cols)).astype(np.float32)
            yw, hw, sw, mw = fo.layer_norm_fwd(x, w, None, 1e-5)
            dxw, dww, dbw = fo.layer_norm_bwd(g, hw, sw, w)
            G, W = be.alloc_from_host(g), be.alloc_from_host(w)
            atol_dx = 2e-4 * np.abs(dxw).max()
            atol_dw = 2e-4 * np.abs(g * hw).sum(0).max()
            atol_db = 2e-4 * np.abs(g).sum(0).max()
            # ferro's saved tensors (h, stds)
            dx, dw, db = be.layer_norm_backward_dev(G, W, rows, cols, h=be.alloc_from_host(hw), stds=be.alloc_from_host(sw))
            assert_close(be.copy_to_host(dx).reshape(rows, cols), dxw, RED_RTOL, atol_dx, f"dx(h) {rows}x{cols}")
            assert_close(be.copy_to_host(dw), dww, RED_RTOL, atol_dw, f"dw(h) {rows}x{cols}")
            assert_close(be.copy_to_host(db), dbw, RED_RTOL, atol_db, f"db(h) {rows}x{cols}")
            # compact statistics (x, mean, rstd)
            X = be.alloc_from_host(x)
            _, mu, rs = be.layer_norm_stats_dev(X, W, None, rows, cols, 1e-5)
            dx, dw, db = be.layer_norm_backward_dev(G, W, rows, cols, x=X, mean=mu, rstd=rs)
            assert_close(be.copy_to_host(dx).reshape(rows, cols), dxw, RED_RTOL, atol_dx, f"dx(x) {rows}x{cols}")
            assert_close(be.copy_to_host(dw), dww, RED_RTOL, atol_dw, f"dw(x) {rows}x{cols}")
            assert_close(be.copy_to_host(db), dbw, RED_RTOL, atol_db, f"db(x) {rows}x{cols}")
            # no affine weight, no parameter gradients
            dxn, _, _ = fo.layer_norm_bwd(g, hw, sw, None, False, False)
            dx, dw, db = be.layer_norm_backward_dev(G, None, rows, cols, h=be.alloc_from_host(hw), stds=be.alloc_from_host(sw), want_dw=False, want_db=False)
            assert dw is None and db is None
            assert_close(be.copy_to_host(dx).reshape(rows, cols), dxn, RED_RTOL, 2e-4 * np.abs(dxn).max(), f"dx(no w) {rows}x{cols}")


def test_layer_norm_pipelined_paths(be):
    """Enough rows for the shared-memory pipeline to be chosen (it needs two rows per resident CTA): forward for
    rows wider than 8192 columns, backward from 260 columns up (64 / 128 / 256 threads below 2048 columns, which need
    up to 4800 rows to be chosen), CTAs of 320 / 384 / 640 / 768 threads where the row fills them better than a power of two: 2560, 3072, 5120,
    6144, 10240, 12288 columns), both saved forms; from 16384 columns up (backward;
    forward above 32768) a cluster of CTAs shares each row (2 x 8192, 4 x 8192, 8 x 6252 with a short last slice,
    8 x 8192 in the backward; 4 x 12500, 4 x 16384, 8 x 16384 in the forward), several rows per cluster; at 131072
    columns the backward takes the two-kernel form."""
    r = np.random.default_rng(141)
    for rows, cols in [(4800, 320), (4800, 448), (2400, 640), (2400, 1000), (1250, 1536), (900, 2048), (1000, 2560), (900, 3072), (640, 5120), (640, 6144), (900, 8192), (320, 10240), (320, 12288), (320, 16384), (301, 32768),
                       (150, 50000), (77, 65536), (33, 131072)]:
        x = (r.standard_normal((rows, cols)) * r.uniform(0.5, 4, (rows, 1))).astype(np.float32)
        w = (1 + 0.02 * r.standard_normal(cols)).astype(np.float32)
        bb = (0.02 * r.standard_normal(cols)).astype(np.float32)
        g = r.standard_normal((rows, cols)).astype(np.float32)
        yw, hw, sw, mw = fo.layer_norm_fwd(x, w, bb, 1e-5)
        dxw, dww, dbw = fo.layer_norm_bwd(g, hw, sw, w)
        X, W, Bv, G = (be.alloc_from_host(a) for a in (x, w, bb, g))
        y, h, s = be.layer_norm_dev(X, W, Bv, rows, cols, 1e-5)
        assert_close(be.copy_to_host(y).reshape(rows, cols), yw, RED_RTOL, 3e-6, f"y {rows}x{cols}")
        assert_close(be.copy_to_host(h).reshape(rows, cols), hw, RED_RTOL, 1e-6, f"h {rows}x{cols}")
        assert_close(be.copy_to_host(s), sw, RED_RTOL, 0, f"stds {rows}x{cols}")
        _, mu, rs = be.layer_norm_stats_dev(X, W, Bv, rows, cols, 1e-5)
        atol_dx = 2e-4 * np.abs(dxw).max()
        atol_dw = 2e-4 * np.abs(g * hw).sum(0).max()
        atol_db = 2e-4 * np.abs(g).sum(0).max()
        for kw in (dict(h=h, stds=s), dict(x=X, mean=mu, rstd=rs)):
            dx, dw, db = be.layer_norm_backward_dev(G, W, rows, cols, **kw)
            assert_close(be.copy_to_host(dx).reshape(rows, cols), dxw, RED_RTOL, atol_dx, f"dx {rows}x{cols} {list(kw)}")
            assert_close(be.copy_to_host(dw), dww, RED_RTOL, atol_dw, f"dw {rows}x{cols}")
            assert_close(be.copy_to_host(db), dbw, RED_RTOL, atol_db, f"db {rows}x{cols}")
        yr, rr = be.rms_norm_dev(X, W, rows, cols, 1e-5)
        assert_close(be.copy_to_host(yr).reshape(rows, cols), fo.rms_norm_fwd(x, w, 1e-5)[0], RED_RTOL, 1e-6, f"rms y {rows}x{cols}")
        dxr, dwr = be.rms_norm_backward_dev(G, X, rr, W, rows, cols)
        wx, ww_ = fo.rms_norm_bwd(g, x, w, 1e-5)
        assert_close(be.copy_to_host(dxr).reshape(rows, cols), wx, RED_RTOL, 2e-4 * np.abs(wx).max(), f"rms dx {rows}x{cols}")
        assert_close(be.copy_to_host(dwr), ww_, RED_RTOL, 2e-4 * np.abs(ww_).max() + atol_dw, f"rms dw {rows}x{cols}")
    assert be.lib.fb_device_faults(0) == 0


def test_layer_norm_short_rows_many_rows(be):
    """Short rows go several to a warp (8 or 16 lanes x 1 or x 3 float4, 32 lanes x 1 .. 4), forward up to 512
    columns and backward up to 384, the backward on a persistent grid of two CTAs per SM: 40011 rows make every CTA take more than one block of rows and leave the
    last block ragged.  Both saved forms and RMS normalisation."""
    r = np.random.default_rng(142)
    rows = 40011
    for cols in (32, 48, 64, 96, 128, 192, 196, 256, 320, 384):
        x = (r.standard_normal((rows, cols)) * r.uniform(0.5, 4, (rows, 1)) + 0.2).astype(np.float32)
        w = (1 + 0.02 * r.standard_normal(cols)).astype(np.float32)
        g = r.standard_normal((rows, cols)).astype(np.float32)
        yw, hw, sw, mw = fo.layer_norm_fwd(x, w, None, 1e-5)
        dxw, dww, dbw = fo.layer_norm_bwd(g, hw, sw, w)
        X, W, G = (be.alloc_from_host(a) for a in (x, w, g))
        y, h, s = be.layer_norm_dev(X, W, None, rows, cols, 1e-5)
        assert_close(be.copy_to_host(y).reshape(rows, cols), yw, RED_RTOL, 3e-6, f"y {rows}x{cols}")
        assert_close(be.copy_to_host(h).reshape(rows, cols), hw, RED_RTOL, 1e-6, f"h {rows}x{cols}")
        assert_close(be.copy_to_host(s), sw, RED_RTOL, 0, f"stds {rows}x{cols}")
        _, mu, rs = be.layer_norm_stats_dev(X, W, None, rows, cols, 1e-5)
        assert_close(be.copy_to_host(mu), mw, RED_RTOL, 2e-4 * np.abs(x).max() / np.sqrt(cols), f"mean {rows}x{cols}")
        assert_close(be.copy_to_host(rs), 1 / sw.astype(np.float64), RED_RTOL, 0, f"rstd {rows}x{cols}")
        atol_dx = 2e-4 * np.abs(dxw).max()
        atol_dw = 2e-4 * np.abs(g * hw).sum(0).max()
        atol_db = 2e-4 * np.abs(g).sum(0).max()
        for kw in (dict(h=h, stds=s), dict(x=X, mean=mu, rstd=rs)):
            dx, dw, db = be.layer_norm_backward_dev(G, W, rows, cols, **kw)
            assert_close(be.copy_to_host(dx).reshape(rows, cols), dxw, RED_RTOL, atol_dx, f"dx {rows}x{cols} {list(kw)}")
            assert_close(be.copy_to_host(dw), dww, RED_RTOL, atol_dw, f"dw {rows}x{cols}")
            assert_close(be.copy_to_host(db), dbw, RED_RTOL, atol_db, f"db {rows}x{cols}")
        yr, rr = be.rms_norm_dev(X, W, rows, cols, 1e-5)
        assert_close(be.copy_to_host(yr).reshape(rows, cols), fo.rms_norm_fwd(x, w, 1e-5)[0], RED_RTOL, 1e-6, f"rms y {rows}x{cols}")
        dxr, dwr = be.rms_norm_backward_dev(G, X, rr, W, rows, cols)
        wx, ww_ = fo.rms_norm_bwd(g, x, w, 1e-5)
        assert_close(be.copy_to_host(dxr).reshape(rows, cols), wx, RED_RTOL, 2e-4 * np.abs(wx).max(), f"rms dx {rows}x{cols}")
        assert_close(be.copy_to_host(dwr), ww_, RED_RTOL, 2e-4 * np.abs(ww_).max() + atol_dw, f"rms dw {rows}x{cols}")


def test_residual_layer_norm(be):
    """Tensor::residual_layernorm (crates/ferro-core/src/fused_ops.rs:106-231): LayerNorm of x + r; the oracle
    forms the sum with ferro's add and normalises it with the LayerNorm host loop."""
    r = np.random.default_rng(131)
    for cols in (7, 256, 1000, 1024, 1536, 2048, 4096, 6000, 8192, 8196, 20000):
        rows = 3 if cols > 8192 else 19
        x = (r.standard_normal((rows, cols)) * r.uniform(0.5, 4, (rows, 1))).astype(np.float32)
        res = r.standard_normal((rows, cols)).astype(np.float32)
        w = (1 + 0.02 * r.standard_normal(cols)).astype(np.float32)
        bb = (0.02 * r.standard_normal(cols)).astype(np.float32)
        sw = fo.binary(K.BIN_ADD, x, res)
        yw, hw, stw, _ = fo.layer_norm_fwd(sw, w, bb, 1e-5)
        X, R_, W, Bv = (be.alloc_from_host(a) for a in (x, res, w, bb))
        y, h, st, sm = be.residual_layer_norm_dev(X, R_, W, Bv, rows, cols, 1e-5, want_sum=True)
        assert_bitwise(be.copy_to_host(sm).reshape(rows, cols), sw, f"sum {cols}")
        assert_close(be.copy_to_host(y).reshape(rows, cols), yw, RED_RTOL, 3e-6, f"res-ln y {cols}")
        assert_close(be.copy_to_host(h).reshape(rows, cols), hw, RED_RTOL, 1e-6, f"res-ln h {cols}")
        assert_close(be.copy_to_host(st), stw, RED_RTOL, 0, f"res-ln stds {cols}")
        y2, _, _ = be.residual_layer_norm_dev(X, R_, W, Bv, rows, cols, 1e-5)  # without the sum: the wide path sums into y
        assert_close(be.copy_to_host(y2).reshape(rows, cols), yw, RED_RTOL, 3e-6, f"res-ln y (no sum) {cols}")
    b = B()
    with pytest.raises(b.InvalidShape):
        be.residual_layer_norm_dev(X, be.alloc_from_host(np.zeros(3, np.float32)), None, None, rows, cols, 1e-5)


def test_rms_norm_forward_and_backward(be):
    """RmsNorm (crates/ferro-core/src/nn.rs:255-283) as one kernel each way, against the op-by-op oracle."""
    r = np.random.default_rng(121)
    for cols in (1, 7, 64, 1000, 1024, 4096, 4100, 8192, 20000, 33000):
        for rows in ((3,) if cols > 8192 else (1, 37)):
            x = (r.standard_normal((rows, cols)) * r.uniform(0.5, 4, (rows, 1)) + 0.3).astype(np.float32)
            w = (1 + 0.1 * r.standard_normal(cols)).astype(np.float32)
            g = r.standard_normal((rows, cols)).astype(np.float32)
            X, W, G = be.alloc_from_host(x), be.alloc_from_host(w), be.alloc_from_host(g)
            for ww, Wd in ((w, W), (None, None)):
                yw, rw = fo.rms_norm_fwd(x, ww, 1e-5)
                y, rs = be.rms_norm_dev(X, Wd, rows, cols, 1e-5)
                assert_close(be.copy_to_host(y).reshape(rows, cols), yw, RED_RTOL, 1e-6, f"rms y {rows}x{cols}")
                assert_close(be.copy_to_host(rs), rw, RED_RTOL, 0, f"rstd {cols}")
                dxw, dww = fo.rms_norm_bwd(g, x, ww, 1e-5)
                dx, dw = be.rms_norm_backward_dev(G, X, rs, Wd, rows, cols)
                assert_close(be.copy_to_host(dx).reshape(rows, cols), dxw, RED_RTOL, 2e-4 * np.abs(dxw).max(), f"rms dx {rows}x{cols}")
                assert_close(be.copy_to_host(dw), dww, RED_RTOL, 2e-4 * np.abs(g * x).sum(0).max() * float(rw.max()), f"rms dw {cols}")
    # an infinite entry: finite entries of that row go to 0, the entry itself to NaN, as in the op chain
    x = np.float32([[1, 2, np.inf, 4], [1, 2, 3, 4]])
    y, _ = be.rms_norm_dev(be.alloc_from_host(x), None, 2, 4, 1e-5)
    got, want = be.copy_to_host(y).reshape(2, 4), fo.rms_norm_fwd(x, None, 1e-5)[0]
    assert (np.isnan(got) == np.isnan(want)).all()
    assert_close(got, want, RED_RTOL, 1e-6, "rms with inf")


# -------------------------------------------------------------------- optimizers
def test_fused_adam_and_sgd_bitwise_vs_host_loop(be):
    """crates/ferro-cuda/src/lib.rs:2214-2257: bitwise against the host loop."""
    b = B()
    r = np.random.default_rng(13)
    for n in (1, 5, 1023, 4096, (1 << 20) + 3):
        p, m, g = (r.standard_normal(n).astype(np.float32) for _ in range(3))
        v = np.abs(r.standard_normal(n)).astype(np.float32)
        for wd in (0.0, 0.01):
            P, M, Vv, G = (be.alloc_from_host(a) for a in (p, m, v, g))
            hp = b.AdamWStep(1e-3, 0.9, 0.999, float(fo.bias_correction(0.9, 3)), float(fo.bias_correction(0.999, 3)), 1e-8, wd)
            be.adamw_step_dev(P, M, Vv, G, hp)
            pp, mm, vv = p.copy(), m.copy(), v.copy()
            fo.adamw_step(pp, mm, vv, g, hp.lr, hp.beta1, hp.beta2, hp.bc1, hp.bc2, hp.eps, hp.weight_decay)
            assert_bitwise(be.copy_to_host(P), pp, f"adam p n={n} wd={wd}")
            assert_bitwise(be.copy_to_host(M), mm, "adam m")
            assert_bitwise(be.copy_to_host(Vv), vv, "adam v")
        for nesterov in (False, True):
            P, Vv, G = (be.alloc_from_host(a) for a in (p, m, g))
            be.sgd_step_dev(P, Vv, G, 0.1, 0.9, nesterov)
            pp, vv = p.copy(), m.copy()
            fo.sgd_step(pp, vv, g, 0.1, 0.9, nesterov)
            assert_bitwise(be.copy_to_host(P), pp, f"sgd p n={n}")
            assert_bitwise(be.copy_to_host(Vv), vv, "sgd v")
    with pytest.raises(b.InvalidArgument):  # distinct storages (inplace.rs:539-561)
        P = be.alloc_from_host(p)
        be.adamw_step_dev(P, P, be.alloc_from_host(v), be.alloc_from_host(g), hp)


def test_adam_trajectory_and_capturable_timestep(be):
    """Five steps with a per-step bias correction, eager vs capturable vs host
    (optim.rs:707-771; kernels.rs:489-530)."""
    b = B()
    r = np.random.default_rng(14)
    n = 10007
    p0 = r.standard_normal(n).astype(np.float32)
    P1, M1, V1 = be.alloc_from_host(p0), be.fill_dev(0.0, n), be.fill_dev(0.0, n)
    P2, M2, V2 = be.alloc_from_host(p0), be.fill_dev(0.0, n), be.fill_dev(0.0, n)
    t = be.alloc_from_host(np.zeros(3, np.float32))
    pp, mm, vv = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for step in range(1, 6):
        g = r.standard_normal(n).astype(np.float32)
        G = be.alloc_from_host(g)
        bc1, bc2 = float(fo.bias_correction(0.9, step)), float(fo.bias_correction(0.999, step))
        be.adamw_step_dev(P1, M1, V1, G, b.AdamWStep(1e-3, 0.9, 0.999, bc1, bc2, 1e-8, 0.0))
        be.scalar_increment_dev(t, 0.9, 0.999)
        be.adamw_step_capturable_dev(P2, M2, V2, G, t, 1e-3, 0.9, 0.999, 1e-8, 0.0)
        fo.adamw_step(pp, mm, vv, g, 1e-3, 0.9, 0.999, bc1, bc2, 1e-8, 0.0)
        assert_bitwise(be.copy_to_host(P1), pp, f"eager step {step}")
        assert_bitwise(be.copy_to_host(P2), pp, f"capturable step {step}")
    assert_bitwise(be.copy_to_host(t), np.float32([5, fo.bias_correction(0.9, 5), fo.bias_correction(0.999, 5)]))
    # first Adam step moves by -lr (tests/optim.rs:127-157)
    P, M, Vv = be.alloc_from_host([1.0]), be.fill_dev(0.0, 1), be.fill_dev(0.0, 1)
    be.adamw_step_dev(P, M, Vv, be.alloc_from_host([0.5]), b.AdamWStep(0.1, 0.9, 0.999, float(fo.bias_correction(0.9, 1)), float(fo.bias_correction(0.999, 1)), 1e-8, 0.0))
    assert abs(be.copy_to_host(P)[0] - 0.9) < 1e-4


def test_multi_tensor_steps_bitwise(be):
    b = B()
    r = np.random.default_rng(15)
    sizes = [67, 16384, 1, 40000, 4096, 9]
    ps = [r.standard_normal(n).astype(np.float32) for n in sizes]
    ms = [r.standard_normal(n).astype(np.float32) for n in sizes]
    vs = [np.abs(r.standard_normal(n)).astype(np.float32) for n in sizes]
    gs = [r.standard_normal(n).astype(np.float32) for n in sizes]
    for g_scale in (1.0, 0.25):
        dev = [[be.alloc_from_host(a) for a in arr] for arr in (ps, ms, vs, gs)]
        table = be.make_table(list(zip(*dev)))
        hp = b.AdamWStep(1e-3, 0.9, 0.999, 0.1, 0.001, 1e-8, 0.0)
        be.adamw_multi_dev(table, hp, g_scale)
        for i, n in enumerate(sizes):
            pp, mm, vv = ps[i].copy(), ms[i].copy(), vs[i].copy()
            fo.adamw_step(pp, mm, vv, gs[i] * np.float32(g_scale), 1e-3, 0.9, 0.999, 0.1, 0.001, 1e-8, 0.0)
            assert_bitwise(be.copy_to_host(dev[0][i]), pp, f"multi adam tensor {i}")
            assert_bitwise(be.copy_to_host(dev[1][i]), mm)
            assert_bitwise(be.copy_to_host(dev[2][i]), vv)
    dev = [[be.alloc_from_host(a) for a in arr] for arr in (ps, ms, gs)]
    table = be.make_table([(p, m, None, g) for p, m, g in zip(*dev)])
    be.sgd_multi_dev(table, 0.1, 0.9, True)
    for i in range(len(sizes)):
        pp, vv = ps[i].copy(), ms[i].copy()
        fo.sgd_step(pp, vv, gs[i], 0.1, 0.9, True)
        assert_bitwise(be.copy_to_host(dev[0][i]), pp, f"multi sgd tensor {i}")
        assert_bitwise(be.copy_to_host(dev[1][i]), vv)


def test_bias_add_activation_gelu_silu(be):
    """Tensor::bias_add_activation with Act::Gelu / Act::Silu (crates/ferro-core/src/fused_ops.rs:21-51, 57-104):
    forward act(x + b), backward g * act'(z) with db summed over rows."""
    r = np.random.default_rng(161)
    C, A = 0.7978846, 0.044715
    for rows, cols in [(64, 4096), (33, 100), (7, 5), (300, 36)]:
        x = (2 * r.standard_normal((rows, cols))).astype(np.float32)
        bias = r.standard_normal(cols).astype(np.float32)
        g = r.standard_normal((rows, cols)).astype(np.float32)
        X, Bb, G = be.alloc_from_host(x), be.alloc_from_host(bias), be.alloc_from_host(g)
        z = fo.binary_bc(K.BIN_ADD, x, bias)
        z64 = z.astype(np.float64)
        for act, kind in (("gelu", K.UN_GELU), ("silu", K.UN_SILU)):
            want = fo.unary(kind, z)
            got = be.copy_to_host(be.bias_act_dev(X, Bb, act, rows, cols)).reshape(rows, cols)
            # atol: gelu cancels to ~0 for very negative inputs (|z| up to 8 here), where 0.5*z*(1+tanh) keeps the absolute error of tanh
            assert_close(got, want, ELT_RTOL, 1.5e-6, f"{act} fwd {rows}x{cols}")
            if act == "gelu":
                t = np.tanh(C * (z64 + A * z64 ** 3))
                d = 0.5 * (1 + t) + 0.5 * z64 * (1 - t * t) * C * (1 + 3 * A * z64 * z64)
            else:
                s_ = np.exp(-z64)
                sig = 1 / (1 + s_)
                d = sig * (1 + z64 * s_ * sig)
            dxw = g.astype(np.float64) * d
            dx, db = be.bias_act_backward_dev(G, X, Bb, act, rows, cols)
            # atol: act' cancels for very negative z (1 + tanh and 1 - tanh^2 near 0 are multiplied by z and 1 + 3Az^2),
            # in ferro's own f32 evaluation as much as here
            assert_close(be.copy_to_host(dx).reshape(rows, cols), dxw, 2e-5, 1e-5 * np.abs(g).max(), f"{act} bwd {rows}x{cols}")
            assert_close(be.copy_to_host(db), dxw.sum(0), RED_RTOL, 2e-4 * np.abs(dxw).sum(0).max(), f"{act} db")
    b = B()
    with pytest.raises(b.InvalidArgument):
        be._check(be.lib.fb_bias_act_fwd(be._s(), X.ptr, Bb.ptr, 7, 1, 1, X.ptr))


def test_global_norm_clipping_on_device(be):
    """global_grad_norm / clip_scale (crates/ferro-core/src/optim.rs:1395-1425) with the norm, the factor and
    the clipped update all staying on the device."""
    b = B()
    r = np.random.default_rng(151)
    sizes = [67, 300000, 1, 40000, 4099, 9]
    ps = [r.standard_normal(n).astype(np.float32) for n in sizes]
    ms = [r.standard_normal(n).astype(np.float32) for n in sizes]
    vs = [np.abs(r.standard_normal(n)).astype(np.float32) for n in sizes]
    gs = [(3.0 * r.standard_normal(n)).astype(np.float32) for n in sizes]
    hp = b.AdamWStep(1e-3, 0.9, 0.999, 0.1, 0.001, 1e-8, 0.0)
    for g_scale, max_norm in [(1.0, 1.0), (0.5, 10.0), (1.0, 1e9)]:
        dev = [[be.alloc_from_host(a) for a in arr] for arr in (ps, ms, vs, gs)]
        table = be.make_table(list(zip(*dev)))
        norm, scale = be.clip_scale_dev(table, max_norm, g_scale)
        scaled = [g * np.float32(g_scale) for g in gs]
        want_norm, want_scale = fo.global_grad_norm(scaled), fo.clip_scale(scaled, max_norm)
        got_norm, got_scale = be.copy_to_host(norm)[0], be.copy_to_host(scale)[0]
        assert abs(got_norm - want_norm) <= RED_RTOL * want_norm, (got_norm, want_norm)
        assert abs(got_scale - want_scale) <= RED_RTOL * want_scale, (got_scale, want_scale)
        assert (got_scale == 1.0) == (want_scale == 1.0)
        # the update applies exactly the factor the device computed: g * g_scale * scale, one rounding each
        be.adamw_multi_dev(table, hp, g_scale, clip_scale=scale)
        for i in range(len(sizes)):
            pp, mm, vv = ps[i].copy(), ms[i].copy(), vs[i].copy()
            fo.adamw_step(pp, mm, vv, scaled[i] * np.float32(got_scale), 1e-3, 0.9, 0.999, 0.1, 0.001, 1e-8, 0.0)
            assert_bitwise(be.copy_to_host(dev[0][i]), pp, f"clipped adam tensor {i}")
            assert_bitwise(be.copy_to_host(dev[1][i]), mm)
    # SGD form, and an all-zero gradient list (norm 0 leaves the factor at 1)
    zeros = [np.zeros(n, np.float32) for n in sizes]
    dev = [[be.alloc_from_host(a) for a in arr] for arr in (ps, ms, zeros)]
    table = be.make_table([(p, m, None, g) for p, m, g in zip(*dev)])
    norm, scale = be.clip_scale_dev(table, 0.5)
    assert be.copy_to_host(norm)[0] == 0.0 and be.copy_to_host(scale)[0] == 1.0
    dev = [[be.alloc_from_host(a) for a in arr] for arr in (ps, ms, gs)]
    table = be.make_table([(p, m, None, g) for p, m, g in zip(*dev)])
    norm, scale = be.clip_scale_dev(table, 2.0)
    sc = be.copy_to_host(scale)[0]
    be.sgd_multi_dev(table, 0.1, 0.9, True, clip_scale=scale)
    for i in range(len(sizes)):
        pp, vv = ps[i].copy(), ms[i].copy()
        fo.sgd_step(pp, vv, gs[i] * np.float32(sc), 0.1, 0.9, True)
        assert_bitwise(be.copy_to_host(dev[0][i]), pp, f"clipped sgd tensor {i}")


# ---------------------------------------------------------------------- MLP glue
def test_bias_act_and_mse(be):
    r = np.random.default_rng(16)
    for rows, cols in [(64, 4096), (33, 100), (300, 36), (7, 5), (1000, 64), (2, 16384)]:
        x = r.standard_normal((rows, cols)).astype(np.float32)
        bias = r.standard_normal(cols).astype(np.float32)
        g = r.standard_normal((rows, cols)).astype(np.float32)
        X, Bb, G = be.alloc_from_host(x), be.alloc_from_host(bias), be.alloc_from_host(g)
        pre = fo.binary_bc(K.BIN_ADD, x, bias)
        for relu in (True, False):
            want = fo.unary(K.UN_RELU, pre) if relu else pre
            assert_bitwise(be.copy_to_host(be.bias_act_dev(X, Bb, relu, rows, cols)).reshape(rows, cols), want, f"fwd {rows}x{cols} relu={relu}")
            dxw = fo.binary(K.BIN_RELU_BACKWARD, g, pre) if relu else g
            dbw = fo.sum_dim(dxw, 0).ravel()
            dx, db = be.bias_act_backward_dev(G, X, Bb, relu, rows, cols)
            assert_bitwise(be.copy_to_host(dx).reshape(rows, cols), dxw, f"dx {rows}x{cols} relu={relu}")  # mask exact
            assert_close(be.copy_to_host(db), dbw, RED_RTOL, 2e-4 * np.abs(dxw).sum(0).max(), f"db {rows}x{cols}")
    for n in (1, 1000, (1 << 20) + 3):
        pred, tgt = r.standard_normal(n).astype(np.float32), r.standard_normal(n).astype(np.float32)
        loss, dp = be.mse_dev(be.alloc_from_host(pred), be.alloc_from_host(tgt))
        wl, wd = fo.mse_fwd_bwd(pred, tgt)
        assert abs(be.copy_to_host(loss)[0] - wl) <= RED_RTOL * wl
        assert_bitwise(be.copy_to_host(dp), wd, f"mse grad n={n}")
