"""The library's host-side generator (fb_rng_*, the source of "seed k via ferro
Rng" inputs) against the oracle's restatement of ferro_core::Rng
(crates/ferro-core/src/rng.rs:12-70), bit for bit, at sizes that cross the
block boundaries of the threaded fills, and against the reference's own
determinism test values held by the oracle pins."""
import time

import numpy as np

import oracle as fo
from ferro_b200.rng import Rng


def same(a, b):
    return a.dtype == b.dtype and a.shape == b.shape and (a.view(np.uint32 if a.dtype == np.float32 else np.uint64)
                                                          == b.view(np.uint32 if b.dtype == np.float32 else np.uint64)).all()


def test_scalar_draws_and_state_follow_the_oracle():
    for seed in (0, 1, 2, 42, 2**63 + 5):
        a, b = Rng(seed), fo.Rng(seed)
        assert (a.state.s0, a.state.s1) == b.state()
        for _ in range(50):
            assert np.float32(a.uniform()).view(np.uint32) == np.float32(b.uniform()).view(np.uint32)
            assert np.float32(a.normal()).view(np.uint32) == np.float32(b.normal()).view(np.uint32)
        assert (a.state.s0, a.state.s1) == b.state()


def test_fills_are_bit_identical_across_block_boundaries_and_leave_the_same_state():
    n = (1 << 21) + 12345
    a, b = Rng(0), fo.Rng(0)
    assert same(a.fill_normal((n,)), b.fill_normal((n,)))
    assert same(a.fill_normal((3, 1000), 0.1, 1.0), b.fill_normal((3, 1000), 0.1, 1.0))
    assert same(a.fill_uniform((70001,), 8.0, -4.0), b.fill_uniform((70001,), 8.0, -4.0))
    assert same(a.fill_rowscaled_normal(1030, 4096), b.fill_rowscaled_normal(1030, 4096))   # two row blocks
    assert same(a.fill_rowscaled_normal(3, 5), b.fill_rowscaled_normal(3, 5))
    assert same(a.fill_he((64, 256), 64), b.fill_he((64, 256), 64))
    assert same(a.fill_index(5000, 32000), b.fill_targets(5000, 32000))
    assert (a.state.s0, a.state.s1) == b.state()


def test_fill_into_a_caller_buffer_and_statistics():
    import torch
    buf = torch.empty(1 << 20, dtype=torch.float32)
    t0 = time.time()
    Rng(7).fill_normal((1 << 20,), out=buf)
    assert time.time() - t0 < 5
    x = buf.numpy()
    assert abs(float(x.mean())) < 5e-3 and abs(float(x.std()) - 1) < 5e-3
    assert same(x, fo.Rng(7).fill_normal((1 << 20,)))
