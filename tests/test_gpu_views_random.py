"""Randomised views through the strided pointwise engine: permuted, sliced,
stepped and broadcast operands of rank 1..6 against the oracle's odometer.
Every dispatch of the engine (segment, vector tile, scalar tile, flat, wide
and narrow index math) is reached by some case; results must be bit-exact for
the exact kinds used here."""
import numpy as np
import pytest

import oracle as fo
from ferro_b200 import kinds as K

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from ferro_b200.backend import CudaBackend
    return CudaBackend(0)


def random_view(r, shape):
    """A random ferro-style view producing `shape`: storage, element strides, offset."""
    rank = len(shape)
    perm = list(r.permutation(rank))
    steps = [int(r.integers(1, 3)) for _ in range(rank)]
    bcast = [bool(r.random() < 0.2) for _ in range(rank)]
    # storage dims in permuted order, each long enough for the stepped extent
    sdims = [1 if bcast[d] else shape[d] * steps[d] + int(r.integers(0, 2)) for d in perm]
    storage = r.standard_normal(int(np.prod(sdims)) + 8).astype(np.float32)
    sstr = [0] * rank
    acc = 1
    for pos in reversed(range(rank)):
        sstr[pos] = acc
        acc *= sdims[pos]
    strides = [0] * rank
    for pos, d in enumerate(perm):
        strides[d] = 0 if bcast[d] else sstr[pos] * steps[d]
    offset = int(r.integers(0, 8))
    return storage, strides, offset


def test_random_views_binary_and_unary(be):
    import ferro_b200.backend as b
    r = np.random.default_rng(1234)
    shapes = [(5,), (1030,), (7, 9), (64, 64), (96, 130), (3, 4, 5), (2, 130, 68), (4, 1, 260), (2, 3, 4, 5), (3, 2, 65, 66),
              (2, 2, 2, 3, 3), (2, 1, 3, 2, 2, 5), (1, 4100), (260, 1028), (128, 2048)]
    for shape in shapes:
        for trial in range(4):
            sa, sta, oa = random_view(r, shape)
            sb, stb, ob = random_view(r, shape)
            A, Bv = be.alloc_from_host(sa), be.alloc_from_host(sb)
            got = be.copy_to_host(be.binary_strided_dev(b.BinaryKind.Sub, b.View(A, sta, oa), b.View(Bv, stb, ob), shape))
            want = fo.binary_strided(K.BIN_SUB, sa, sta, oa, sb, stb, ob, shape)
            assert (got.view(np.uint32) == want.ravel().view(np.uint32)).all(), (shape, sta, stb)
            got = be.copy_to_host(be.unary_strided_dev(b.UnaryKind.Neg, b.View(A, sta, oa), shape))
            want = -fo.materialize(sa, sta, oa, shape)
            assert (got.view(np.uint32) == want.ravel().view(np.uint32)).all(), (shape, sta)


def test_random_three_operand_programs(be):
    import ferro_b200.backend as b
    S, U, Bi = b.ChainStep, b.UnaryKind, b.BinaryKind
    r = np.random.default_rng(99)
    for shape in [(33, 65), (256, 256), (8, 16, 260), (3, 5, 7, 9), (4, 4100)]:
        views = [random_view(r, shape) for _ in range(3)]
        bufs = [be.alloc_from_host(v[0]) for v in views]
        ops = [b.View(bufs[i], views[i][1], views[i][2]) for i in range(3)]
        m = [fo.materialize(v[0], v[1], v[2], shape) for v in views]
        # relu(x0) * x1 + x2 (catalogue entry when it lands on the segment kernel, interpreter otherwise)
        got = be.copy_to_host(be.chain_dev([S.Load(0), S.Unary(U.Relu), S.Binary(Bi.Mul, other=1), S.Binary(Bi.Add, other=2)], ops, shape))
        want = fo.binary(K.BIN_ADD, fo.binary(K.BIN_MUL, fo.unary(K.UN_RELU, m[0]), m[1]), m[2])
        assert (got.view(np.uint32) == want.ravel().view(np.uint32)).all(), shape
        # (x1 - |x0|) / x2 with the temporary register and a swapped operand order
        prog = [S.Load(0), S.Unary(U.Abs), S.Load(1, dst=b.T), S.Binary(Bi.Sub, swap=True), S.Binary(Bi.Div, other=2)]
        got = be.copy_to_host(be.chain_dev(prog, ops, shape))
        want = fo.binary(K.BIN_DIV, fo.binary(K.BIN_SUB, m[1], fo.unary(K.UN_ABS, m[0])), m[2])
        assert (got.view(np.uint32) == want.ravel().view(np.uint32)).all(), shape
