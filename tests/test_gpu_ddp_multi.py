"""The gradient exchange on real GPUs: two ranks, one process per GPU, the library's own NCCL
communicator (fb_ddp_*).  Needs at least two devices; with fewer the tests are skipped (the
host logic and every failure path are covered on CPU in test_ddp_cpu.py and
test_ddp_exchange_cpu.py).

  - Ddp.average() leaves, on every rank, exactly ferro's Ddp::average of the per-rank gradients
    (crates/ferro-core/src/ddp.rs:138-157: sum in replica order, then divide) - bitwise against the oracle.
  - Two steps of the sharded MLP on two ranks equal the same global batch on one rank.
"""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, out_dir):
    import datetime
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    import oracle as fo
    from ferro_b200 import ddp
    from ferro_b200.backend import CudaBackend
    torch.cuda.set_device(rank)
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=120))
    be = CudaBackend(rank)
    comm = ddp.NcclComm(rank, world, ddp.share_id_over_store(store, rank))
    assert be.lib.fb_ddp_nccl_version() > 20000
    # (1) exact mean of per-rank gradients
    shapes = [("W1", (37, 50)), ("b1", (50,)), ("W2", (50, 11)), ("b2", (11,))]
    with torch.cuda.stream(be.stream):
        params = [(n, torch.zeros(*s, device=be.device)) for n, s in shapes]
    d = ddp.Ddp(be, params, comm, bucket_cap_bytes=4 * 50 * 11, divide=True, watch=ddp.PeerWatch(store, rank, world))
    assert [b.names for b in d.gb.buckets] == [["b2", "W2"], ["b1", "W1"]]
    local = {}
    for n, s in reversed(shapes):
        g = fo.Rng(100 + rank * 10 + len(n) + s[0]).fill_normal(s)
        local[n] = g
        with torch.cuda.stream(be.stream):
            d.grad(n).copy_(torch.from_numpy(g).to(be.device))
        d.grad_ready(n)
    d.average()
    be.synchronize()
    np.savez(os.path.join(out_dir, f"avg{rank}.npz"), **{f"l_{n}": local[n] for n in local},
             **{f"a_{n}": d.grad(n).cpu().numpy() for n in local})
    comm.poll()
    # (2) sharded training steps against the one-rank run
    B, din, dh, dout = 128, 48, 96, 24
    init = fo.Rng(1)
    P = [init.fill_he((din, dh), din), np.zeros(dh, np.float32), init.fill_he((dh, dout), dh), np.zeros(dout, np.float32)]
    data = fo.Rng(2)
    x, y = data.fill_normal((B, din)), data.fill_normal((B, dout))
    lo, hi = ddp.shard_rows(rank, world, B)
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(be.device)
    sharded = ddp.DdpMlp(be, din, dh, dout, hi - lo, comm=comm, params=[to(p) for p in P], bucket_cap_bytes=4 * dh * dout)
    single = ddp.DdpMlp(be, din, dh, dout, B, params=[to(p) for p in P], bucket_cap_bytes=4 * dh * dout)
    xs, ys, xf, yf = to(x[lo:hi]), to(y[lo:hi]), to(x), to(y)
    for _ in range(2):
        sharded.step(xs, ys)
        single.step(xf, yf)
    sharded.synchronize()
    single.synchronize()
    np.savez(os.path.join(out_dir, f"mlp{rank}.npz"), **{f"s{i}": p.cpu().numpy() for i, p in enumerate(sharded.params)},
             **{f"o{i}": p.cpu().numpy() for i, p in enumerate(single.params)},
             **{f"g{i}": single.ddp.grad(n).cpu().numpy() for i, n in enumerate(["W1", "b1", "W2", "b2"])})
    comm.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_exchange_is_the_exact_mean_and_matches_one_rank(tmp_path):
    import torch.multiprocessing as mp
    import oracle as fo
    world, port = 2, _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    r = [np.load(tmp_path / f"avg{k}.npz") for k in range(world)]
    for n in ("W1", "b1", "W2", "b2"):
        want = fo.ddp_average([r[0][f"l_{n}"].ravel(), r[1][f"l_{n}"].ravel()])
        for k in range(world):
            assert (r[k][f"a_{n}"].ravel().view(np.uint32) == want.view(np.uint32)).all(), (n, k)
    m = [np.load(tmp_path / f"mlp{k}.npz") for k in range(world)]
    for i in range(4):
        assert (m[0][f"s{i}"] == m[1][f"s{i}"]).all()          # replicas stay identical
        a, b, g = m[0][f"s{i}"], m[0][f"o{i}"], m[0][f"g{i}"]
        live = np.abs(g) >= 1e-5 * np.abs(g).max()              # Adam's first steps are +-lr * sign(g) near g = 0
        assert (np.abs(a - b)[live] <= (1e-4 * np.abs(b) + 2e-4)[live]).all(), i
        assert np.abs(b - m[0][f"o{i}"]).max() == 0
