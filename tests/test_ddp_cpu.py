"""Host-side logic of the data-parallel step on CPU: row sharding, bucket
layout, and the gradient mean over a world of 2 gloo ranks, checked against
the oracle of ferro's Ddp::average (crates/ferro-core/src/ddp.rs:138-157) and
its tests (crates/ferro-core/tests/ddp.rs:288-356: exact mean)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as fo
from ferro_b200 import ddp


def test_shard_rows_cover_the_batch_without_overlap():
    for world in (1, 2, 4, 8):
        spans = [ddp.shard_rows(r, world, 65536) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 65536
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    with pytest.raises(ValueError):
        ddp.shard_rows(0, 3, 65536)


def test_buckets_are_flat_aligned_views():
    buckets = ddp.make_buckets([[("W2", (6, 5)), ("b2", (5,))], [("W1", (3, 6)), ("b1", (6,))]], "cpu")
    assert [b.names for b in buckets] == [["W2", "b2"], ["W1", "b1"]]
    for b in buckets:
        for v in b.views:
            assert v.data_ptr() >= b.flat.data_ptr()
            assert (v.data_ptr() - b.flat.data_ptr()) % 16 == 0
            v.fill_(1.0)
        assert b.flat.sum().item() == sum(v.numel() for v in b.views)


def test_bias_correction_matches_the_oracle_powi():
    for beta in (0.9, 0.999):
        for t in (1, 2, 3, 7, 100, 1000):
            assert np.float32(ddp.bias_correction(beta, t)) == fo.bias_correction(beta, t)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # A tiny MLP step per rank on its shard, gradients from the oracle's formulas.
        B, din, dh, dout = 8, 5, 7, 3
        rng = fo.Rng(1)
        W1, W2 = rng.fill_he((din, dh), din), rng.fill_he((dh, dout), dh)
        data = fo.Rng(2)
        x, y = data.fill_normal((B, din)), data.fill_normal((B, dout))
        lo, hi = ddp.shard_rows(rank, world, B)
        xs, ys = x[lo:hi], y[lo:hi]
        h = np.maximum(fo.matmul(xs, W1), 0)
        yh = fo.matmul(h, W2)
        _, dy = fo.mse_fwd_bwd(yh, ys)
        dy = dy.reshape(yh.shape)
        gW2, gb2 = fo.matmul(np.ascontiguousarray(h.T), dy), dy.sum(0)
        dhid = fo.matmul(dy, np.ascontiguousarray(W2.T)) * (h > 0)
        gW1, gb1 = fo.matmul(np.ascontiguousarray(xs.T), dhid), dhid.sum(0)
        buckets = ddp.make_buckets([[("W2", (dh, dout)), ("b2", (dout,))], [("W1", (din, dh)), ("b1", (dh,))]], "cpu")
        for view, g in zip(buckets[0].views + buckets[1].views, (gW2, gb2, gW1, gb1)):
            view.copy_(torch.from_numpy(np.ascontiguousarray(g, dtype=np.float32)))
        local = [b.flat.clone().numpy() for b in buckets]
        for b in buckets:
            ddp.average_(b)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), l0=local[0], l1=local[1],
                 a0=buckets[0].flat.numpy(), a1=buckets[1].flat.numpy())
    finally:
        dist.destroy_process_group()


def test_gradient_mean_over_two_gloo_ranks_is_the_exact_mean(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    r = [np.load(tmp_path / f"rank{k}.npz") for k in range(world)]
    for key_l, key_a in (("l0", "a0"), ("l1", "a1")):
        want = fo.ddp_average([r[0][key_l], r[1][key_l]])  # sum in replica order, then divide
        for k in range(world):
            assert (r[k][key_a].view(np.uint32) == want.view(np.uint32)).all()
    # The mean of the shard gradients is the gradient of the global-batch mean loss.
    B, din, dh, dout = 8, 5, 7, 3
    rng = fo.Rng(1)
    W1, W2 = rng.fill_he((din, dh), din), rng.fill_he((dh, dout), dh)
    data = fo.Rng(2)
    x, y = data.fill_normal((B, din)), data.fill_normal((B, dout))
    h = np.maximum(fo.matmul(x, W1), 0)
    _, dy = fo.mse_fwd_bwd(fo.matmul(h, W2), y)
    gW2 = fo.matmul(np.ascontiguousarray(h.T), dy.reshape(B, dout))
    np.testing.assert_allclose(r[0]["a0"][:dh * dout].reshape(dh, dout), gW2, rtol=1e-5, atol=1e-7)
