"""gather along a dim, its scatter-add backward, and the CSR segment sum / softmax with their
backward, through the C ABI, against the oracle's restatement of ferro's host loops
(crates/ferro-core/src/ops_ext/gather.rs:50-110, src/segment.rs:132-253).  Bars: gathers,
scatter-adds and segment sums are bit-exact (index work, and additions in the host loop's own order);
segment softmax 2e-4 relative."""
import numpy as np
import pytest

import oracle as fo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from ferro_b200.backend import CudaBackend
    return CudaBackend(0)


def bk():
    import ferro_b200.backend as b
    return b


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_gather_and_scatter_add_every_dim_bit_exact(be):
    r = np.random.default_rng(51)
    for in_shape, out_shape in [((2, 2), (2, 2)), ((3, 2), (1, 2)), ((7, 33, 40), (7, 33, 40)), ((7, 33, 40), (5, 20, 9)),
                                ((4, 1000), (4, 1000)), ((2000, 64), (3000, 64)), ((5, 6, 7, 8), (5, 6, 7, 8)), ((129,), (1000,))]:
        x = r.standard_normal(in_shape).astype(np.float32)
        X = be.alloc_from_host(x)
        for dim in range(len(in_shape)):
            osh = list(out_shape)
            if in_shape == (2000, 64) and dim != 0:
                continue  # the index may only exceed the input along `dim`
            if in_shape == (129,) and dim != 0:
                continue
            idx = r.integers(0, in_shape[dim], osh)
            if np.prod(osh) > 100:
                idx.reshape(-1)[:50] = idx.reshape(-1)[50]  # plenty of duplicates for the backward
            want, src = fo.gather(x, dim, idx)
            I = be.alloc_i64_from_host(idx)
            got = be.copy_to_host(be.gather_dev(X, in_shape, dim, I, osh)).reshape(osh)
            assert (bits(got) == bits(want)).all(), (in_shape, osh, dim)
            g = r.standard_normal(osh).astype(np.float32)
            gx = be.copy_to_host(be.gather_backward_dev(be.alloc_from_host(g), I, in_shape, osh, dim)).reshape(in_shape)
            assert (bits(gx) == bits(fo.gather_bwd(g, src, in_shape))).all(), (in_shape, osh, dim)
    # known answers of crates/ferro-core/tests/op_gather.rs:5-19 and the rejections of :21-32
    t = be.alloc_from_host(np.float32([1, 2, 3, 4]))
    assert be.copy_to_host(be.gather_dev(t, (2, 2), 1, be.alloc_i64_from_host([0, 0, 1, 0]), (2, 2))).tolist() == [1, 1, 4, 3]
    with pytest.raises(bk().InvalidShape):
        be.gather_dev(t, (2, 2), 1, be.alloc_i64_from_host([0, 2]), (1, 2))       # index out of range
    with pytest.raises(bk().InvalidShape):
        be.gather_dev(t, (2, 2), 0, be.alloc_i64_from_host([0, 0, 0]), (1, 3))    # wider than the input


def test_segment_sum_and_softmax_forward_backward(be):
    r = np.random.default_rng(52)
    for edges, groups, width in [(3, 4, 2), (1000, 37, 1), (5000, 300, 7), (20000, 1000, 64), (4000, 50, 200), (64, 64, 33),
                                 (10000, 3, 16), (0, 5, 4)]:
        ids = r.integers(0, groups, edges)
        if edges > 100:
            ids[ids == 1] = 0            # an empty group
            ids[:40] = groups - 1        # a run of edges in one group
        x = r.standard_normal((edges, width)).astype(np.float32)
        plan = be.prepare_segments(ids, groups)
        X = be.alloc_from_host(x)
        got = be.copy_to_host(be.segment_dev(plan, "sum", X, width)).reshape(groups, width)
        assert (bits(got) == bits(fo.segment_sum(x, ids, groups).reshape(groups, width))).all(), (edges, groups, width)
        g = r.standard_normal((groups, width)).astype(np.float32)
        dx = be.copy_to_host(be.segment_dev(plan, "sum_backward", be.alloc_from_host(g), width)).reshape(edges, width)
        assert (bits(dx) == bits(fo.segment_sum_bwd(g, ids, width).reshape(edges, width))).all()
        if edges == 0:
            continue
        y = fo.segment_softmax(x, ids, groups)
        Y = be.segment_dev(plan, "softmax", X, width)
        got = be.copy_to_host(Y).reshape(edges, width)
        assert np.abs(got - y).max() <= 2e-4 * np.abs(y).max()
        assert (np.abs(got - y) <= 2e-4 * np.abs(y) + 1e-30).all()
        ge = r.standard_normal((edges, width)).astype(np.float32)
        dxs = be.copy_to_host(be.segment_dev(plan, "softmax_backward", be.alloc_from_host(ge), width, saved=be.alloc_from_host(y))).reshape(edges, width)
        want = fo.segment_softmax_bwd(ge, y, ids, groups)
        assert (np.abs(dxs - want) <= 2e-4 * np.abs(want) + 2e-4 * np.abs(want).max() * 1e-2).all()
    # foundation_segment.rs:19-27 and :41: shifted logits, and the finite-logit check
    plan = be.prepare_segments([0, 0, 1], 3)
    p = be.copy_to_host(be.segment_dev(plan, "softmax", be.alloc_from_host(np.float32([1000, 1001, -1000])), 1))
    assert np.abs(p - [1 / (1 + np.e), 1 / (1 + 1 / np.e), 1.0]).max() < 1e-6
    with pytest.raises(bk().Unsupported):
        be.segment_dev(be.prepare_segments([0], 1), "softmax", be.alloc_from_host(np.float32([np.inf])), 1)
    with pytest.raises(bk().InvalidShape):
        be.prepare_segments([0, 3], 3)  # segment id out of bounds
