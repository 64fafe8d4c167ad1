"""Reductions and softmax over one dim of tensor views (transposed, sliced, stepped, broadcast,
offset), through the C ABI, against the oracle run on the materialised input: sums / means and
softmax to 2e-4 relative, max values and argmax indices bit-exact.  These are the inputs ferro
downloads to the host today (crates/ferro-core/src/tensor.rs:2057-2104, 2124-2127)."""
import numpy as np
import pytest

import oracle as fo

pytestmark = pytest.mark.gpu
RED_RTOL = 2e-4


@pytest.fixture(scope="module")
def be():
    from ferro_b200.backend import CudaBackend
    return CudaBackend(0)


def bk():
    import ferro_b200.backend as b
    return b


def elem_strides(a):
    return [s // a.itemsize for s in a.strides]


def view_of(be, base, sub):
    """A numpy view `sub` of the contiguous array `base` as (View, shape)."""
    off = (sub.__array_interface__["data"][0] - base.__array_interface__["data"][0]) // base.itemsize
    return bk().View(view_of.buf, elem_strides(sub), off), list(sub.shape)


def cases(r):
    base = r.standard_normal((6, 40, 70)).astype(np.float32) * 2
    yield "whole", base, base
    yield "transpose 0<->2", base, base.transpose(2, 1, 0)
    yield "transpose 1<->2", base, base.transpose(0, 2, 1)
    yield "slice", base, base[1:5, 3:37, 10:60]
    yield "step", base, base[::2, ::3, ::5]
    yield "negative step", base, base[:, ::-1, :]
    yield "broadcast", base, np.broadcast_to(base[:, :1, :], (6, 33, 70))
    yield "row of a matrix", base, base[2, 7]
    big = r.standard_normal((300, 1000)).astype(np.float32)
    yield "wide transpose", big, big.T
    yield "wide slice", big, big[5:290, 100:900]
    yield "column block", big, big[:, 128:160]


def close(got, want, rtol, atol, ctx):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, ctx
    assert (np.isnan(got) == np.isnan(want)).all(), ctx
    m = ~np.isnan(want)
    err = np.abs(got[m] - want[m])
    bound = rtol * np.abs(want[m]) + atol
    assert (err <= bound).all(), f"{ctx}: max excess {float((err - bound).max()):.3e}"


def test_sum_mean_max_over_every_dim_of_views(be):
    r = np.random.default_rng(41)
    for name, base, sub in cases(r):
        view_of.buf = be.alloc_from_host(base)
        v, shape = view_of(be, base, sub)
        dense = np.ascontiguousarray(sub)
        for dim in range(sub.ndim):
            ctx = f"{name} dim {dim}"
            want = fo.sum_dim(dense, dim)
            atol = 2e-4 * np.abs(dense).sum(axis=dim).max()
            close(be.copy_to_host(be.sum_dim_view_dev(v, shape, dim)), want.ravel(), RED_RTOL, atol, "sum " + ctx)
            close(be.copy_to_host(be.mean_dim_view_dev(v, shape, dim)), fo.mean_dim(dense, dim).ravel(), RED_RTOL,
                  atol / sub.shape[dim], "mean " + ctx)
            val, idx = be.max_dim_view_dev(v, shape, dim)
            wi, wv = fo.argmax_dim(dense, dim)
            assert (be.copy_i64_to_host(idx) == wi.ravel()).all(), "argmax " + ctx
            assert (be.copy_to_host(val).view(np.uint32) == wv.ravel().view(np.uint32)).all(), "max " + ctx


def test_max_over_views_with_nan_and_ties(be):
    base = np.zeros((5, 64, 9), np.float32)
    base[:, 10, :] = 3.0
    base[:, 50, :] = 3.0          # a tie: the lower index wins
    base[2, 30, 4] = np.nan       # the first NaN wins
    base[2, 40, 4] = np.nan
    view_of.buf = be.alloc_from_host(base)
    for sub in (base.transpose(2, 0, 1), base[:, ::1, ::2].transpose(0, 2, 1)):
        v, shape = view_of(be, base, sub)
        dim = [i for i, s in enumerate(sub.shape) if s == 64][0]
        val, idx = be.max_dim_view_dev(v, shape, dim)
        wi, wv = fo.argmax_dim(np.ascontiguousarray(sub), dim)
        assert (be.copy_i64_to_host(idx) == wi.ravel()).all()
        got = be.copy_to_host(val)
        assert ((got.view(np.uint32) == wv.ravel().view(np.uint32)) | (np.isnan(got) & np.isnan(wv.ravel()))).all()


def test_softmax_and_log_softmax_over_every_dim_of_views(be):
    r = np.random.default_rng(42)
    for name, base, sub in cases(r):
        view_of.buf = be.alloc_from_host(base)
        v, shape = view_of(be, base, sub)
        dense = np.ascontiguousarray(sub)
        for dim in range(sub.ndim):
            ctx = f"{name} dim {dim}"
            got = be.copy_to_host(be.softmax_view_dev(v, shape, dim)).reshape(sub.shape)
            close(got, fo.softmax_fwd(dense, dim), RED_RTOL, 1e-30, "softmax " + ctx)
            got = be.copy_to_host(be.softmax_view_dev(v, shape, dim, log=True)).reshape(sub.shape)
            close(got, fo.log_softmax_fwd(dense, dim), RED_RTOL, 1e-6, "log_softmax " + ctx)


def test_softmax_backward_over_views(be):
    r = np.random.default_rng(43)
    base_g = r.standard_normal((6, 40, 70)).astype(np.float32)
    base_x = r.standard_normal((6, 40, 70)).astype(np.float32) * 2
    G = be.alloc_from_host(base_g)
    picks = [lambda a: a, lambda a: a.transpose(2, 1, 0), lambda a: a[1:5, ::2, 3:60], lambda a: a.transpose(0, 2, 1)]
    for pick in picks:
        gs, xs = pick(base_g), pick(base_x)
        dense_g, dense_x = np.ascontiguousarray(gs), np.ascontiguousarray(xs)
        for dim in range(gs.ndim):
            for log in (False, True):
                y = (fo.log_softmax_fwd if log else fo.softmax_fwd)(dense_x, dim)
                # g as a view of its storage, y whole (what the forward returned): different strides
                view_of.buf = G
                gv, shape = view_of(be, base_g, gs)
                Y = be.alloc_from_host(y)
                st, acc = [], 1
                for n in reversed(shape):
                    st.insert(0, acc)
                    acc *= n
                got = be.copy_to_host(be.softmax_view_backward_dev(gv, bk().View(Y, st, 0), shape, dim, log=log)).reshape(gs.shape)
                want = (fo.log_softmax_bwd if log else fo.softmax_bwd)(dense_g, y, dim)
                close(got, want, RED_RTOL, 2e-4 * np.abs(want).max(), f"bwd log={log} dim {dim}")


def test_masked_and_empty_views(be):
    b = bk()
    x = np.random.default_rng(44).standard_normal((4, 50, 6)).astype(np.float32)
    x[0, :10, 0] = -np.inf       # masked entries at the head of a column
    x[1, :, 1] = -np.inf         # a fully masked column: NaN, like the host loop
    view_of.buf = be.alloc_from_host(x)
    v, shape = view_of(be, x, x)
    got = be.copy_to_host(be.softmax_view_dev(v, shape, 1)).reshape(x.shape)
    close(got, fo.softmax_fwd(x, 1), RED_RTOL, 1e-30, "masked softmax over dim 1")
    # views outside their storage and bad dims are refused before any launch
    with pytest.raises(b.InvalidShape):
        be.sum_dim_view_dev(b.View(view_of.buf, (300, 6, 1), 0), (5, 50, 6), 1)
    with pytest.raises(b.InvalidShape):
        be.sum_dim_view_dev(v, shape, 3)
    # an empty reduced dim: sum 0, mean NaN
    e = be.alloc_from_host(np.zeros(1, np.float32))
    assert be.copy_to_host(be.sum_dim_view_dev(b.View(e, (0, 1), 0), (3, 0), 1)).tolist() == [0, 0, 0]
    assert np.isnan(be.copy_to_host(be.mean_dim_view_dev(b.View(e, (0, 1), 0), (3, 0), 1))).all()
