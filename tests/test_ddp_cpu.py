"""Host-side logic of the data-parallel step on CPU: row sharding, the bucket
planner and its readiness bookkeeping, the per-step agreement that notices a
rank leaving between steps, and the gradient mean over a world of 2 gloo
ranks, checked against the oracle of ferro's Ddp::average
(crates/ferro-core/src/ddp.rs:138-157) and its tests
(crates/ferro-core/tests/ddp.rs:288-356: exact mean).  gloo stands in for the
NCCL exchange here (the product path has no gloo branch; the exchange itself
is covered in tests/test_ddp_exchange_cpu.py)."""
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


def test_planner_walks_parameters_backwards_and_closes_buckets_at_the_cap():
    mlp = [("W1", (4096, 16384)), ("b1", (16384,)), ("W2", (16384, 4096)), ("b2", (4096,))]
    names = lambda plan: [[n for n, _ in g] for g in plan]
    assert names(ddp.plan_buckets(mlp)) == [["b2", "W2"], ["b1", "W1"]]            # layer 2 first: its grads exist first
    assert names(ddp.plan_buckets(mlp, 1 << 40)) == [["b2", "W2", "b1", "W1"]]     # one bucket when the cap allows
    assert names(ddp.plan_buckets(mlp, 1)) == [["b2"], ["W2"], ["b1"], ["W1"]]
    many = [(f"p{i}", (1000,)) for i in range(10)]
    plan = ddp.plan_buckets(many, 12000)
    assert names(plan) == [["p9", "p8", "p7"], ["p6", "p5", "p4"], ["p3", "p2", "p1"], ["p0"]]
    assert sorted(n for g in plan for n, _ in g) == sorted(n for n, _ in many)     # every parameter exactly once
    with pytest.raises(ValueError):
        ddp.plan_buckets(many, 0)


def test_gradient_buckets_report_the_bucket_a_gradient_completes():
    gb = ddp.GradientBuckets([("W1", (3, 6)), ("b1", (6,)), ("W2", (6, 5)), ("b2", (5,))], "cpu", cap_bytes=4 * 30)
    assert [b.names for b in gb.buckets] == [["b2", "W2"], ["b1", "W1"]]
    assert gb.grad("W2").shape == (6, 5) and gb.grad("W2").data_ptr() % 16 == gb.buckets[0].flat.data_ptr() % 16
    assert gb.ready("b2") is None and gb.ready("W2") == 0
    assert gb.incomplete() == [1]
    with pytest.raises(RuntimeError):
        gb.ready("W2")                                   # twice in one step
    assert gb.ready("W1") is None and gb.ready("b1") == 1 and gb.incomplete() == []
    gb.begin()
    assert gb.incomplete() == [0, 1]
    with pytest.raises(ValueError):
        ddp.GradientBuckets([("a", (1,)), ("a", (2,))], "cpu")
    with pytest.raises(ValueError):
        ddp.GradientBuckets([], "cpu")


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
        gb = ddp.GradientBuckets([("W1", (din, dh)), ("b1", (dh,)), ("W2", (dh, dout)), ("b2", (dout,))], "cpu",
                                 cap_bytes=4 * dh * dout)
        buckets = gb.buckets
        assert [b.names for b in buckets] == [["b2", "W2"], ["b1", "W1"]]
        local = {}

        def exchange(bi):
            # Ddp::average for one bucket: sum over replicas, then divide by the replica count.
            local[bi] = buckets[bi].flat.clone().numpy()
            dist.all_reduce(buckets[bi].flat, op=dist.ReduceOp.SUM)
            buckets[bi].flat.div_(float(world))

        for name, g in (("b2", gb2), ("W2", gW2), ("b1", gb1), ("W1", gW1)):  # the order backward produces them
            gb.grad(name).copy_(torch.from_numpy(np.ascontiguousarray(g, dtype=np.float32)))
            done = gb.ready(name)
            if done is not None:
                exchange(done)
        assert gb.incomplete() == []
        local = [local[0], local[1]]
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
    off = (dout + 3) // 4 * 4  # bucket 0 is [b2 | W2]
    np.testing.assert_allclose(r[0]["a0"][off:off + dh * dout].reshape(dh, dout), gW2, rtol=1e-5, atol=1e-7)


def _watch_main(rank, world, port, out_dir):
    """Three steps are planned; rank 1 leaves after the first.  Rank 0 must learn of it on the
    host before it would enqueue step 1, and a rank that simply never checks in must run into
    the agreement's time limit instead of a hang."""
    import time
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=30))
    watch = ddp.PeerWatch(store, rank, world, timeout_s=20.0)
    log = []
    try:
        watch.agree(0)
        log.append("step0")
        if rank == 1:
            watch.leave(1, "preempted")
            log.append("left")
        else:
            watch.agree(1)
            log.append("step1")  # must not be reached
    except ddp.PeerLeft as e:
        log.append(f"peer_left:{e}")
    # second phase: silence instead of an announcement
    quick = ddp.PeerWatch(store, rank, world, timeout_s=1.0, prefix="silent")
    if rank == 0:
        t0 = time.time()
        try:
            quick.agree(0)
            log.append("silent-went-through")
        except ddp.PeerLeft:
            log.append(f"timeout:{time.time() - t0:.1f}")
    store.set(f"done/{rank}", "1")
    store.wait([f"done/{r}" for r in range(world)])
    with open(os.path.join(out_dir, f"watch{rank}.txt"), "w") as f:
        f.write("\n".join(log))


def test_a_rank_leaving_between_steps_is_noticed_before_the_next_collective(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_watch_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    log0 = open(tmp_path / "watch0.txt").read().split("\n")
    log1 = open(tmp_path / "watch1.txt").read().split("\n")
    assert log0[0] == "step0" and log0[1].startswith("peer_left:") and "[1] left" in log0[1]
    assert "step1" not in log0
    assert log0[2].startswith("timeout:") and float(log0[2].split(":")[1]) < 10
    assert log1 == ["step0", "left"]
