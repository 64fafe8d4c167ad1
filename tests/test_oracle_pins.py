"""Pins the CPU oracle to the known-answer tests and golden tables of ferro's
own test-suite (file:line given per test; paths relative to the ferro
repository).  An oracle that drifts from ferro's CPU path fails here, on the
CPU, before any GPU parity test can be trusted."""
import json
import math
import os

import numpy as np
import pytest

import oracle as fo
from ferro_b200 import kinds as K

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_fixtures.json")))


def bits(a):
    return np.asarray(a, np.float32).view(np.uint32)


def from_bits(b):
    return np.asarray(b, np.uint32).view(np.float32)


def assert_bitwise(got, want_bits):
    got = np.asarray(got, np.float32)
    want = from_bits(want_bits)
    assert got.shape == want.shape
    both_nan = np.isnan(got) & np.isnan(want)
    same = bits(got) == bits(want)
    assert np.all(both_nan | same), (got, want)


# ---- Rng ---------------------------------------------------------------
def test_rng_restated_independently():
    """crates/ferro-core/src/rng.rs:12-50 restated here in Python integers."""
    M = (1 << 64) - 1

    def split(z):
        z = (z + 0x9E3779B97F4A7C15) & M
        x = z
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & M
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & M
        return z, x ^ (x >> 31)

    for seed in (0, 1, 2, 0xC0FFEE0012345678):
        z = (seed + 0x9E3779B97F4A7C15) & M
        z, a = split(z)
        z, b = split(z)
        s0, s1 = a | 1, b | 1
        r = fo.Rng(seed)
        assert r.state() == (s0, s1)
        for _ in range(100):
            x, y = s0, s1
            s0 = y
            x ^= (x << 23) & M
            x ^= x >> 17
            x ^= y ^ (y >> 26)
            s1 = x
            want = np.float32(((x + y) & M) >> 40) / np.float32(1 << 24)
            assert np.float32(r.uniform()) == want


def test_rng_normal_is_box_muller_cosine_branch():
    """rng.rs:65-70."""
    r1, r2 = fo.Rng(7), fo.Rng(7)
    for _ in range(50):
        u1 = max(np.float32(r1.uniform()), np.float32(1e-9))
        u2 = np.float32(r1.uniform())
        rad = np.sqrt(np.float32(-2.0) * np.log(u1, dtype=np.float32), dtype=np.float32)
        want = rad * np.cos(np.float32(6.2831855) * u2, dtype=np.float32)
        got = np.float32(r2.normal())
        assert abs(got - want) <= 4e-7 * max(1.0, abs(want))
    vals = fo.Rng(0).fill_normal((200000,))
    assert abs(vals.mean()) < 0.01 and abs(vals.std() - 1.0) < 0.01


# ---- elementwise -------------------------------------------------------
def test_clamp_matches_torch_goldens():
    """crates/ferro-core/tests/clamp_bounds.rs:15-18 with fixtures/clamp_bounds_goldens.rs."""
    x = from_bits(GOLD["clamp32"]["input_bits"])
    for case in GOLD["clamp32"]["cases"]:
        lo, hi = from_bits([case["min"]])[0], from_bits([case["max"]])[0]
        assert_bitwise(fo.unary(K.UN_CLAMP, x, lo, hi), case["expected"])


def test_clamp_backward_mask_is_inclusive():
    """clamp_bounds.rs:22-36: g where min <= x <= max, else +0."""
    x = from_bits(GOLD["clamp32"]["input_bits"])
    for case in GOLD["clamp32"]["cases"]:
        lo, hi = from_bits([case["min"]])[0], from_bits([case["max"]])[0]
        for value in (0.7, np.inf, np.nan, -0.0):
            g = np.full_like(x, value)
            want = np.where((x >= lo) & (x <= hi), np.float32(value), np.float32(0.0))
            assert_bitwise(fo.binary(K.BIN_CLAMP_BWD, g, x, lo, hi), bits(want))


def test_special_powers_match_torch_bits():
    """crates/ferro-core/tests/power_special.rs:22-51 (f32 rows)."""
    for row in GOLD["power_special_f32"]["forward"]:
        x = from_bits([row["x"]])
        assert_bitwise(fo.unary(K.UN_POWF, x, row["p"]), [row["y"]])
    for row in GOLD["power_special_f32"]["backward"]:
        x, g = from_bits([row["x"]]), from_bits([row["g"]])
        assert_bitwise(fo.binary(K.BIN_POWF_BWD, g, x, row["p"]), [row["dx"]])


def test_half_powers_domains_and_signed_zero():
    """crates/ferro-fastcpu/src/elementwise.rs:331-341."""
    inp = np.array([-np.inf, -4.0, -0.0, 0.0, 4.0, np.inf, np.nan], np.float32)
    assert_bitwise(fo.unary(K.UN_POWF, inp, 0.5),
                   bits(np.array([np.nan, np.nan, -0.0, 0.0, 2.0, np.inf, np.nan], np.float32)))
    assert_bitwise(fo.unary(K.UN_POWF, inp, -0.5),
                   bits(np.array([np.nan, np.nan, -np.inf, np.inf, 0.5, 0.0, np.nan], np.float32)))


def test_activation_gradient_kinds_on_nonfinite_values():
    """crates/ferro-fastcpu/src/elementwise.rs:595-604."""
    v = np.array([-np.inf, -2.0, -0.0, 0.0, 2.0, np.inf, np.nan], np.float32)
    assert_bitwise(fo.unary(K.UN_SIGN, v), bits(np.array([-1, -1, 0, 0, 1, 1, 0], np.float32)))
    assert_bitwise(fo.unary(K.UN_GTZ, v), bits(np.array([0, 0, 0, 0, 1, 1, 1], np.float32)))
    incoming = np.array([np.nan, np.inf, -np.inf, np.nan, -0.0, -7.0, np.inf, 2.0, np.nan], np.float32)
    inputs = np.array([-1.0, 0.0, -0.0, 1.0, np.nan, np.inf, -np.inf, 2.0, np.nan], np.float32)
    want = np.array([0.0, 0.0, 0.0, np.nan, -0.0, -7.0, 0.0, 2.0, np.nan], np.float32)
    assert_bitwise(fo.binary(K.BIN_RELU_BACKWARD, incoming, inputs), bits(want))


def test_relu_propagates_nan_and_flushes_negative_zero():
    """crates/ferro-core/src/dispatch.rs:674-681."""
    v = np.array([-1.0, -0.0, 0.0, 3.0, np.nan, -np.inf, np.inf], np.float32)
    assert_bitwise(fo.unary(K.UN_RELU, v), bits(np.array([0.0, 0.0, 0.0, 3.0, np.nan, 0.0, np.inf], np.float32)))


def test_unary_formulas_against_independent_numpy():
    """The expression of each kind, dispatch.rs:671-718 (and kernels.rs:639-675)."""
    r = np.random.default_rng(0)
    v = r.uniform(-4, 4, 4097).astype(np.float32)
    one = np.float32(1)
    np.testing.assert_array_equal(fo.unary(K.UN_NEG, v), -v)
    np.testing.assert_array_equal(fo.unary(K.UN_ABS, v), np.abs(v))
    np.testing.assert_array_equal(fo.unary(K.UN_SQRT, np.abs(v)), np.sqrt(np.abs(v)))
    np.testing.assert_allclose(fo.unary(K.UN_EXP, v), np.exp(v.astype(np.float64)), rtol=2e-7)
    np.testing.assert_allclose(fo.unary(K.UN_LOG, np.abs(v)), np.log(np.abs(v).astype(np.float64)), rtol=2e-7, atol=1e-7)
    np.testing.assert_allclose(fo.unary(K.UN_TANH, v), np.tanh(v.astype(np.float64)), rtol=3e-7)
    np.testing.assert_allclose(fo.unary(K.UN_SIGMOID, v), 1 / (1 + np.exp(-v.astype(np.float64))), rtol=3e-7)
    np.testing.assert_allclose(fo.unary(K.UN_SILU, v), v / (1 + np.exp(-v.astype(np.float64))), rtol=3e-7, atol=1e-7)
    np.testing.assert_array_equal(fo.unary(K.UN_POWF, v, 2.0), v * v)
    np.testing.assert_array_equal(fo.unary(K.UN_POWF, v, 3.0), (v * v) * v)
    np.testing.assert_array_equal(fo.unary(K.UN_POWF, v, -1.0), one / v)
    np.testing.assert_array_equal(fo.unary(K.UN_POWF, v, -2.0), one / (v * v))
    av = np.abs(v)
    np.testing.assert_allclose(fo.unary(K.UN_POWF, av, 1.5), av.astype(np.float64) ** 1.5, rtol=2e-7)
    assert np.isnan(fo.unary(K.UN_POWF, -av[av > 0], 1.5)).all()
    u = np.float32(0.7978846) * (v + np.float32(0.044715) * v * v * v)
    np.testing.assert_allclose(fo.unary(K.UN_GELU, v), np.float32(0.5) * v * (one + np.tanh(u)), rtol=1e-6, atol=5e-7)
    erf = np.vectorize(math.erf)
    np.testing.assert_allclose(fo.unary(K.UN_GELU_ERF, v), 0.5 * v * (1 + erf(v / math.sqrt(2))), rtol=1e-5, atol=3e-7)
    phi = np.exp(-0.5 * v.astype(np.float64) ** 2) * 0.3989422804
    np.testing.assert_allclose(fo.unary(K.UN_GELU_ERF_GRAD, v), 0.5 * (1 + erf(v / math.sqrt(2))) + v * phi, rtol=1e-5, atol=3e-7)


def test_binary_formulas():
    """dispatch.rs:79-87; backward closures of ops_ext/{sqrt,abs,log,tanh}.rs."""
    r = np.random.default_rng(1)
    a = r.uniform(-4, 4, 1025).astype(np.float32)
    b = r.uniform(-4, 4, 1025).astype(np.float32)
    np.testing.assert_array_equal(fo.binary(K.BIN_ADD, a, b), a + b)
    np.testing.assert_array_equal(fo.binary(K.BIN_SUB, a, b), a - b)
    np.testing.assert_array_equal(fo.binary(K.BIN_MUL, a, b), a * b)
    np.testing.assert_array_equal(fo.binary(K.BIN_DIV, a, b), a / b)
    np.testing.assert_array_equal(fo.binary(K.BIN_SQRT_BWD, a, b), a / (np.float32(2) * b))
    np.testing.assert_array_equal(fo.binary(K.BIN_ABS_BWD, a, b), a * np.sign(b))
    np.testing.assert_array_equal(fo.binary(K.BIN_LOG_BWD, a, b), a / b)
    np.testing.assert_array_equal(fo.binary(K.BIN_SIGMOID_BWD, a, b), (a * (np.float32(1) - b)) * b)
    y = np.tanh(b)
    want = a.astype(np.float64) * (1.0 - y.astype(np.float64) ** 2)
    np.testing.assert_allclose(fo.binary(K.BIN_TANH_BWD, a, y), want, rtol=3e-7, atol=1e-9)


def test_broadcast_odometer():
    """dispatch.rs:842-891: numpy broadcasting rules, row-major output."""
    r = np.random.default_rng(2)
    for sa, sb in [((4, 5), (5,)), ((3, 1, 5), (4, 1)), ((), (2, 3)), ((2, 3), ()), ((6,), (6,)), ((2, 0, 3), (3,))]:
        a = r.standard_normal(sa).astype(np.float32)
        b = r.standard_normal(sb).astype(np.float32)
        np.testing.assert_array_equal(fo.binary_bc(K.BIN_SUB, a, b), a - b)
        np.testing.assert_array_equal(fo.binary_bc(K.BIN_DIV, a, b), a / b)


def test_materialize_of_a_transposed_view():
    """tensor.rs:1206-1227: transpose swaps shape and stride entries."""
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    np.testing.assert_array_equal(fo.materialize(a, (1, 4), 0, (4, 3)), a.T)
    np.testing.assert_array_equal(fo.materialize(a, (4, 1), 5, (2, 2)), a[1:3, 1:3])


# ---- reductions --------------------------------------------------------
def test_pairwise_known_answers():
    """crates/ferro-core/src/reduce.rs:75-99."""
    assert fo.pairwise_sum(np.zeros(0, np.float32)) == 0.0
    assert fo.pairwise_sum(np.arange(1, 11, dtype=np.float32)) == 55.0
    x = np.arange(40, dtype=np.float32)
    assert fo.pairwise_sum_strided(x, 3, 6, 4) == sum(x[3 + k * 4] for k in range(6))


def test_pairwise_tree_shape():
    """reduce.rs:16-71 restated recursively in numpy float32."""
    def base(v):
        acc = np.zeros(8, np.float32)
        ch = len(v) // 8
        for c in range(ch):
            acc += v[c * 8:(c + 1) * 8]
        s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]))
        for k in range(ch * 8, len(v)):
            s = np.float32(s + v[k])
        return np.float32(s)

    def tree(v):
        if len(v) <= 128:
            return base(v)
        h = len(v) // 2
        return np.float32(tree(v[:h]) + tree(v[h:]))

    r = np.random.default_rng(3)
    for n in [1, 2, 7, 8, 9, 127, 128, 129, 255, 256, 257, 1000, 4096, 32000, 100003]:
        v = (r.standard_normal(n) * 10 ** r.uniform(-3, 3, n)).astype(np.float32)
        assert bits(fo.pairwise_sum(v)) == bits(tree(v)), n
        assert bits(fo.pairwise_sum(v, mt=True)) == bits(tree(v)), n
    v = r.standard_normal(1 << 20).astype(np.float32)
    assert bits(fo.pairwise_sum(v, mt=True)) == bits(fo.pairwise_sum(v))


def test_pairwise_accuracy_gate():
    """crates/ferro-core/tests/reduce_accuracy.rs:12-55 (same generator, same seed)."""
    n = 1_000_000
    rng = fo.Rng(0xC0FFEE0012345678)
    data = np.empty(n, np.float32)
    for i in range(n):
        mag = np.float32(10.0) ** np.float32(np.float32(-6.0) + np.float32(12.0) * np.float32(rng.uniform()))
        data[i] = mag if rng.uniform() < 0.5 else -mag
    ref = data.astype(np.float64).sum()
    naive = np.float32(0)
    for chunk in np.split(data, 1000):
        for v in chunk:
            naive = np.float32(naive + v)
    rel = lambda v: abs(float(v) - ref) / max(abs(ref), 1.0)
    assert rel(naive) > 1e-6
    assert rel(fo.pairwise_sum(data)) <= 1e-6


def test_cancellation_recovers_small_residual():
    """reduce_accuracy.rs:57-75 in spirit: tree keeps what a running sum loses."""
    v = np.concatenate([[1e8], np.ones(1_000_000), [-1e8]]).astype(np.float32)
    got = fo.pairwise_sum(v)
    assert abs(float(got) - 1e6) / 1e6 < 1e-3


def test_sum_dim_values():
    """crates/ferro-core/tests/op_sum_dim.rs:5-16."""
    a = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    np.testing.assert_array_equal(fo.sum_dim(a, 0).ravel(), [5, 7, 9])
    assert fo.sum_dim(a, 1).shape == (2, 1)
    np.testing.assert_array_equal(fo.sum_dim(a, 1).ravel(), [6, 15])
    np.testing.assert_array_equal(fo.mean_dim(a, 1).ravel(), np.float32([6, 15]) * np.float32(1 / 3))


def test_argmax_values_ties_and_nan():
    """crates/ferro-core/tests/op_argmax.rs:5-27."""
    a = np.array([[1, 5, 3], [4, 0, 2]], np.float32)
    np.testing.assert_array_equal(fo.argmax_dim(a, 1)[0].ravel(), [1, 0])
    np.testing.assert_array_equal(fo.argmax_dim(a, 0)[0].ravel(), [1, 0, 0])
    np.testing.assert_array_equal(fo.argmax_dim(np.float32([2, 2, 1]), 0)[0].ravel(), [0])
    np.testing.assert_array_equal(fo.argmax_dim(np.float32([1, np.nan, 9]), 0)[0].ravel(), [1])
    assert np.isnan(fo.argmax_dim(np.float32([1, np.nan, 9]), 0)[1][0])


def test_global_max_first_nan_wins():
    """crates/ferro-core/src/ops_ext/max.rs:45-54; tests/op_max.rs."""
    assert fo.max_all(np.float32([1, 7, 3])) == 7
    assert np.isnan(fo.max_all(np.float32([1, np.nan, 9])))


# ---- softmax / log_softmax --------------------------------------------
def test_softmax_values():
    """crates/ferro-core/tests/op_softmax.rs:5-15."""
    got = fo.softmax_fwd(np.float32([[1, 2, 3], [0, 0, 0]]), 1)
    assert abs(got[0].sum() - 1) < 1e-5 and abs(got[1].sum() - 1) < 1e-5
    assert np.all(np.abs(got[1] - 1 / 3) < 1e-6)


def test_log_softmax_values():
    """crates/ferro-core/tests/op_log_softmax.rs:5-26."""
    x = np.float32([[1, 2, 3], [0.5, -1, 2]])
    y = fo.log_softmax_fwd(x, 1)
    for r in range(2):
        assert abs(np.exp(y[r]).sum() - 1) < 1e-5
        m = x[r].max()
        denom = np.float32(np.exp(x[r] - m).sum())
        np.testing.assert_allclose(y[r], (x[r] - m) - np.log(denom), atol=1e-5)


def test_log_softmax_large_common_offsets():
    """op_log_softmax.rs:44-62 and crates/ferro-cuda/tests/gpu_integration.rs:14-25."""
    seed = np.array([(i % 5) - 2.0 for i in range(12)], np.float32).reshape(2, 3, 2)
    for offset in (1e8, -1e8, 3e38):
        for dim in range(3):
            x = np.full((2, 3, 2), offset, np.float32)
            y = fo.log_softmax_fwd(x, dim)
            width = x.shape[dim]
            assert np.all(np.abs(y + np.log(np.float32(width))) < 2e-6)
            dx = fo.log_softmax_bwd(seed, y, dim)
            want = seed - seed.sum(axis=dim, keepdims=True) / np.float32(width)
            assert np.all(np.abs(dx - want) < 2e-6)


def test_softmax_backward_against_finite_differences():
    """op_softmax.rs:25-34 (grad_check: eps 4e-3, tol 1e-2 + 2e-2|g|, testkit.rs:20-32)."""
    a = np.float32([[0.5, -1.0, 0.3], [1.2, 0.1, -0.4]])
    for dim in (0, 1):
        y = fo.softmax_fwd(a, dim)
        dx = fo.softmax_bwd(a.copy(), y, dim)  # loss = sum(softmax(a) * a) holding the weight fixed
        eps = 4e-3
        for i in np.ndindex(a.shape):
            ap, am = a.copy(), a.copy()
            ap[i] += eps
            am[i] -= eps
            num = ((fo.softmax_fwd(ap, dim) * a).sum() - (fo.softmax_fwd(am, dim) * a).sum()) / (2 * eps)
            assert abs(dx[i] - num) < 1e-2 + 2e-2 * abs(num)


def test_cross_entropy_known_answers():
    """crates/ferro-core/tests/nn.rs:18-32 (uniform 2-class -> ln 2) and :73-83."""
    loss, dl, am = fo.cross_entropy_indices(np.zeros((4, 2), np.float32), np.int64([0, 1, 1, 0]))
    assert abs(loss - math.log(2)) < 1e-6
    r = np.random.default_rng(5)
    logits = r.standard_normal((7, 11)).astype(np.float32) * 2
    t = r.integers(0, 11, 7)
    loss, dl, am = fo.cross_entropy_indices(logits, t)
    # indices == one-hot composition: mean(-sum(onehot * log_softmax))
    lp = fo.log_softmax_fwd(logits, 1)
    oh = np.eye(11, dtype=np.float32)[t]
    want = fo.mean(-fo.sum_dim(fo.binary(K.BIN_MUL, lp, oh), 1))
    assert bits(loss) == bits(want)
    sm = np.exp(lp.astype(np.float64))
    np.testing.assert_allclose(dl, (sm - oh) / 7, rtol=2e-6, atol=1e-8)
    np.testing.assert_array_equal(am, logits.argmax(1))
    with pytest.raises(ValueError):
        fo.cross_entropy_indices(logits, np.int64([0, 1, 2, 3, 4, 5, 11]))


# ---- LayerNorm ---------------------------------------------------------
def test_layer_norm_values():
    """crates/ferro-core/tests/op_layer_norm.rs:15-44."""
    s = np.sqrt(np.float32(1.5))
    y, h, stds, means = fo.layer_norm_fwd(np.float32([[1, 2, 3]]), None, None, 1e-5)
    assert np.all(np.abs(y - [-s, 0, s]) < 1e-5)
    w, b = np.float32([2, 0.5, -1]), np.float32([0.1, -0.2, 0.3])
    y2, *_ = fo.layer_norm_fwd(np.float32([[1, 2, 3]]), w, b, 1e-5)
    assert np.all(np.abs(y2 - (np.float32([-s, 0, s]) * w + b)) < 1e-3)
    y3, *_ = fo.layer_norm_fwd(np.float32([[10, 20, 30], [-5, 0, 5]]), None, None, 1e-5)
    for row in y3:
        assert abs(row[0] + s) < 1e-3 and abs(row[1]) < 1e-3 and abs(row[2] - s) < 1e-3


def test_layer_norm_against_f64_formula():
    """crates/ferro-cuda/tests/layer_norm_fused.rs:28-42: the moderate-offset case.
    (The 1e8 / 1e20 offsets in that test exercise the GPU kernel's f64 shifted
    sums; the CPU loop this oracle restates is only held to 2e-3 there, :79-137.)"""
    cols = 7
    data = np.array([3.0 + (i % 19) * 0.0 for i in range(2 * cols)], np.float32).reshape(2, cols)
    y, *_ = fo.layer_norm_fwd(data, None, None, 1e-5)
    assert np.all(np.abs(y) < 2e-6)
    for d in (1, 3, 31, 256, 513, 8193):
        x = np.array([1000.0 + (i % 17) * 0.125 for i in range(3 * d)], np.float32).reshape(3, d)
        y, *_ = fo.layer_norm_fwd(x, np.full(d, 1.25, np.float32), np.full(d, -0.3, np.float32), 1e-5)
        x64 = x.astype(np.float64)
        want = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * 1.25 - 0.3
        assert np.all(np.abs(y - want) < 2e-3), d


def test_layer_norm_backward_against_finite_differences():
    """op_layer_norm.rs:53-67 (weighted loss, grad_check tolerances)."""
    a = np.float32([[0.7, -1.2, 0.3], [1.4, -0.5, 0.9]])
    w, b = np.float32([1.1, 0.6, -0.8]), np.float32([0.2, -0.3, 0.5])
    c = np.array([0.15 + 0.27 * i for i in range(6)], np.float32).reshape(2, 3)
    y, h, stds, _ = fo.layer_norm_fwd(a, w, b, 1e-5)
    dx, dw, db = fo.layer_norm_bwd(c, h, stds, w)
    loss = lambda aa, ww, bb: float((fo.layer_norm_fwd(aa, ww, bb, 1e-5)[0].astype(np.float64) * c).sum())
    eps = 4e-3
    for i in np.ndindex(a.shape):
        ap, am = a.copy(), a.copy()
        ap[i] += eps
        am[i] -= eps
        num = (loss(ap, w, b) - loss(am, w, b)) / (2 * eps)
        assert abs(dx[i] - num) < 1e-2 + 2e-2 * abs(num)
    for j in range(3):
        wp, wm = w.copy(), w.copy()
        wp[j] += eps
        wm[j] -= eps
        num = (loss(a, wp, b) - loss(a, wm, b)) / (2 * eps)
        assert abs(dw[j] - num) < 1e-2 + 2e-2 * abs(num)
        assert abs(db[j] - c[:, j].sum()) < 1e-6


# ---- optimizers --------------------------------------------------------
def test_powi_is_square_and_multiply():
    assert fo.powi(0.9, 1) == np.float32(0.9)
    assert fo.powi(0.9, 2) == np.float32(0.9) * np.float32(0.9)
    a = np.float32(0.999)
    a2 = a * a
    assert fo.powi(0.999, 5) == (a * (a2 * a2)) or fo.powi(0.999, 5) == np.float32(np.float32(a) * np.float32(a2 * a2))
    assert fo.bias_correction(0.9, 1) == np.float32(1) - np.float32(0.9)


def test_first_adam_step_is_minus_lr_and_decay_is_decoupled():
    """crates/ferro-core/tests/optim.rs:127-157."""
    lr, wd = 0.1, 0.04
    outs = []
    for decay in (0.0, wd):
        p, m, v = np.float32([1.0]), np.float32([0.0]), np.float32([0.0])
        fo.adamw_step(p, m, v, np.float32([0.5]), lr, 0.9, 0.999, fo.bias_correction(0.9, 1),
                      fo.bias_correction(0.999, 1), 1e-8, decay)
        outs.append(float(p[0]))
    assert abs(outs[0] - (1 - lr)) < 1e-4
    assert abs(outs[1] - (outs[0] - lr * wd * 1.0)) < 1e-6


def test_sgd_momentum_trajectory():
    """crates/ferro-core/tests/optim_inplace.rs:111-123: p = 0.4 then 1.08."""
    p, v = np.float32([0.0]), np.float32([0.0])
    fo.sgd_step(p, v, np.float32([2 * (p[0] - 2)]), 0.1, 0.9, False)
    assert abs(p[0] - 0.4) < 1e-6
    fo.sgd_step(p, v, np.float32([2 * (p[0] - 2)]), 0.1, 0.9, False)
    assert abs(p[0] - 1.08) < 1e-6


def test_adam_step_expression_order():
    """dispatch.rs:489-503 restated op by op in numpy float32."""
    r = np.random.default_rng(9)
    n = 1000
    p, m, v, g = (r.standard_normal(n).astype(np.float32) for _ in range(4))
    v = np.abs(v)
    f = np.float32
    lr, b1, b2, eps, wd = f(1e-3), f(0.9), f(0.999), f(1e-8), f(0.01)
    bc1, bc2 = fo.bias_correction(b1, 3), fo.bias_correction(b2, 3)
    nb1, nb2 = f(1) - b1, f(1) - b2
    m2 = m * b1 + g * nb1
    v2 = v * b2 + (g * g) * nb2
    upd = (m2 / bc1) / (np.sqrt(v2 / bc2) + eps)
    upd = upd + wd * p
    p2 = p - upd * lr
    fo.adamw_step(p, m, v, g, lr, b1, b2, bc1, bc2, eps, wd)
    np.testing.assert_array_equal(bits(p), bits(p2))
    np.testing.assert_array_equal(bits(m), bits(m2))
    np.testing.assert_array_equal(bits(v), bits(v2))


def test_ddp_average_is_exact_mean():
    """crates/ferro-core/tests/ddp.rs:288-356; src/ddp.rs:138-157."""
    r = np.random.default_rng(4)
    gs = [r.standard_normal(33).astype(np.float32) for _ in range(4)]
    want = ((gs[0] + gs[1]) + gs[2] + gs[3]) / np.float32(4)
    np.testing.assert_array_equal(bits(fo.ddp_average(gs)), bits(want))


def test_mse_and_matmul_glue():
    """ops_ext/mse_loss.rs:9-11, square.rs:16-19, dispatch.rs:788-807."""
    r = np.random.default_rng(6)
    a, b = r.standard_normal((5, 7)).astype(np.float32), r.standard_normal((7, 3)).astype(np.float32)
    np.testing.assert_allclose(fo.matmul(a, b), a.astype(np.float64) @ b, rtol=1e-5, atol=1e-6)
    pred, tgt = r.standard_normal(64).astype(np.float32), r.standard_normal(64).astype(np.float32)
    loss, dp = fo.mse_fwd_bwd(pred, tgt)
    assert abs(loss - ((pred - tgt) ** 2).mean()) < 1e-6
    np.testing.assert_allclose(dp, 2 * (pred - tgt) / 64, rtol=1e-6)


def test_global_grad_norm_and_clip_scale_known_answers():
    """optim.rs:1395-1425: norm over all gradients, factor max/norm only above the budget."""
    g = [np.float32([3.0]), np.float32([0.0, 4.0])]
    assert fo.global_grad_norm(g) == np.float32(5.0)
    assert fo.clip_scale(g, 1.0) == np.float32(np.float32(1.0) / np.float32(5.0))
    assert fo.clip_scale(g, 5.0) == 1.0 and fo.clip_scale(g, 7.0) == 1.0 and fo.clip_scale(g, None) == 1.0
    assert fo.clip_scale([np.zeros(4, np.float32)], 0.5) == 1.0


def test_rms_norm_known_answers():
    """nn.rs:255-283: x / sqrt(mean(x^2) + eps) * gamma; [3, 4] has rms sqrt(12.5)."""
    y, r = fo.rms_norm_fwd(np.float32([[3, 4]]), np.float32([1, 2]), 0.0)
    s = np.sqrt(12.5)
    assert np.allclose(y, [[3 / s, 8 / s]], rtol=1e-6) and np.allclose(r, [1 / s], rtol=1e-6)
    # backward against a finite difference of the forward (float64)
    rng = np.random.default_rng(5)
    x, w, g = rng.standard_normal((2, 6)), rng.standard_normal(6), rng.standard_normal((2, 6))
    dx, dw = fo.rms_norm_bwd(g, x, w, 1e-5)
    f = lambda xx: ((xx / np.sqrt((xx * xx).mean(1, keepdims=True) + 1e-5) * w) * g).sum()
    num = np.zeros_like(x)
    for i in range(2):
        for j in range(6):
            e = np.zeros_like(x); e[i, j] = 1e-6
            num[i, j] = (f(x + e) - f(x - e)) / 2e-6
    assert np.allclose(dx, num, rtol=1e-5, atol=1e-7)


# ------------------------------------------------------------- gather and segments
def test_gather_known_answers():
    # crates/ferro-core/tests/op_gather.rs:5-19
    out, _ = fo.gather(np.float32([[1, 2], [3, 4]]), 1, np.array([[0, 0], [1, 0]]))
    assert out.tolist() == [[1, 1], [4, 3]]
    out, _ = fo.gather(np.float32([[1, 2], [3, 4], [5, 6]]), 0, np.array([[2, 0]]))
    assert out.tolist() == [[5, 2]]
    with pytest.raises(ValueError):
        fo.gather(np.float32([[1, 2], [3, 4]]), 1, np.array([[0, 2]]))  # op_gather.rs:24-25
    # op_gather.rs:35-45: duplicates accumulate in the backward
    x = np.float32([[0.7, -1.1, 0.4], [1.3, -0.6, 0.2]])
    idx = np.array([[1, 1], [0, 2]])
    out, src = fo.gather(x, 1, idx)
    gx = fo.gather_bwd(np.float32([[1, 10], [100, 1000]]), src, x.shape)
    assert gx.tolist() == [[0, 11, 0], [100, 0, 1000]]


def test_segment_known_answers():
    # crates/ferro-core/tests/foundation_segment.rs:19-27: softmax over groups {0, 1} and {2}
    logits = np.float32([[1000.0], [1001.0], [-1000.0]])
    p = fo.segment_softmax(logits, [0, 0, 1], 3).ravel()
    e = np.float32(1.0)
    want = [1 / (1 + np.exp(e)), 1 / (1 + np.exp(-e)), 1.0]
    assert np.abs(p - want).max() < 1e-6
    dp = fo.segment_softmax_bwd(np.float32([[2.0], [-1.0], [7.0]]), p.reshape(3, 1), [0, 0, 1], 3).ravel()
    assert abs(dp[0] - 3 * want[0] * want[1]) < 1e-6 and abs(dp[1] + dp[0]) < 1e-6 and dp[2] == 0
    with pytest.raises(ValueError):
        fo.segment_softmax(np.float32([[np.inf]]), [0], 1)  # foundation_segment.rs:41
    # sums: repeated ids accumulate, missing segments are zero (segment.rs:131-141)
    x = np.float32([[1, 2], [3, 4], [5, 6]])
    assert fo.segment_sum(x, [2, 0, 2], 4).tolist() == [[3, 4], [0, 0], [6, 8], [0, 0]]
    assert fo.segment_sum_bwd(np.float32([[1, 2], [3, 4], [5, 6], [7, 8]]), [2, 0, 2], 2).tolist() == [[5, 6], [1, 2], [5, 6]]


def test_layer_norm_against_the_reference_held_torch_tangents():
    """tests/fixtures/physical2_layernorm_goldens.rs (consumed by tests/physical_saved_stats.rs:16-45 with the
    tolerance used here, 5e-5 + 1e-4 rel): forward-mode tangents of layer_norm from torch.  Seed on the weight:
    seed * h; on the bias: the seed; on x: weight * dx(g = t, no weight) - the forward's normalised values and the
    backward's dx formula, pinned to values the reference holds."""
    gold = GOLD["layernorm_tangents"]
    mk = lambda n, i: (np.arange(n, dtype=np.float32) * np.float32(0.17) + np.float32(0.2) + np.float32(i) * np.float32(0.1))
    x, w, b = mk(6, 0).reshape(2, 3), mk(3, 1), mk(3, 2)
    seed = lambda n: np.arange(n, dtype=np.float32) * np.float32(0.11) - np.float32(0.3)
    y, h, stds, means = fo.layer_norm_fwd(x, w, b, 1e-5)

    def close(got, want):
        got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64)
        assert (np.abs(got - want) <= 5e-5 + 1e-4 * np.abs(want)).all(), (got, want)

    close(h * seed(3), gold["2"])
    close(np.broadcast_to(seed(3), (2, 3)), gold["4"])
    dx, _, _ = fo.layer_norm_bwd(seed(6).reshape(2, 3), h, stds, None, False, False)
    close(dx * w, gold["1"])
