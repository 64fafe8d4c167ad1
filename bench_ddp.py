"""The data-parallel training step of configuration 5 as a benchmark record: the 2-layer MLP
4096 -> 16384 (ReLU) -> 4096, f32, He init from seed 1 (ferro's Rng), MSE loss against y ~ N(0,1),
global batch 65536 drawn from seed 2 and sharded by rows over the ranks (strong scaling),
gradients all-reduced over NVLink through the library's communicator (fb_ddp_*), overlapped
with backward, followed by the fused Adam (lr 1e-3, betas 0.9 / 0.999, eps 1e-8).

The GEMMs are cuBLAS f32 (out of the library's scope: ferro keeps matmul on cuBLAS too); every
memory-bound op and the exchange go through libferro_b200.
"""
import time

from bench_common import NVLINK_MEASURED_GBS, NVLINK_NOMINAL_GBS, Staging

B, DIN, DH, DOUT = 65536, 4096, 16384, 4096


def _bcast(t, dist, world):
    if world > 1:
        dist.broadcast(t, src=0)
    return t


def draw_params(be, rank, world, dist, din, dh, dout, seed=1):
    """W1, b1, W2, b2 in the order of Linear::new (crates/ferro-core/src/nn.rs:138-146): rank 0 draws,
    the others receive a copy."""
    import torch
    from ferro_b200.rng import Rng
    dev = be.device
    if rank == 0:
        st, rng = Staging(be, 1 << 24), Rng(seed)
        W1 = st.normal(rng, din * dh, float((2.0 / din) ** 0.5)).view(din, dh)
        W2 = st.normal(rng, dh * dout, float((2.0 / dh) ** 0.5)).view(dh, dout)
    else:
        with torch.cuda.stream(be.stream):
            W1, W2 = torch.empty(din, dh, device=dev), torch.empty(dh, dout, device=dev)
    be.synchronize()
    _bcast(W1, dist, world)
    _bcast(W2, dist, world)
    torch.cuda.synchronize()
    with torch.cuda.stream(be.stream):
        return [W1, torch.zeros(dh, device=dev), W2, torch.zeros(dout, device=dev)]


def draw_batch(be, lo, hi, batch, din, dout, seed=2):
    """Rows [lo, hi) of x [batch, din] and y [batch, dout], both standard normal, x drawn in full
    before y: the rank skips the draws of the rows it does not own."""
    from ferro_b200.rng import Rng
    st, rng = Staging(be, 1 << 24), Rng(seed)
    rng.skip(2 * lo * din)
    x = st.normal(rng, (hi - lo) * din).view(hi - lo, din)
    rng.skip(2 * (batch - hi) * din + 2 * lo * dout)
    y = st.normal(rng, (hi - lo) * dout).view(hi - lo, dout)
    return x, y


def parity_check(be, comm, rank, world, dist, steps=2):
    """k steps of a small MLP on `world` ranks (sharded batch, all-reduced gradients) against the same
    global batch on one rank, same code with a world of one: parameters must agree within
    1e-4 relative + 2e-4 absolute."""
    import torch
    from ferro_b200.ddp import DdpMlp, NcclComm, shard_rows
    batch, din, dh, dout = 64 * max(world, 2), 128, 512, 64
    params = draw_params(be, rank, world, dist, din, dh, dout, seed=11)
    lo, hi = shard_rows(rank, world, batch)
    xs, ys = draw_batch(be, lo, hi, batch, din, dout, seed=12)
    xf, yf = draw_batch(be, 0, batch, batch, din, dout, seed=12)
    sharded = DdpMlp(be, din, dh, dout, hi - lo, lr=1e-3, comm=comm, params=[p.clone() for p in params],
                     bucket_cap_bytes=4 * dh * dout)
    single = DdpMlp(be, din, dh, dout, batch, lr=1e-3, comm=NcclComm(0, 1), params=[p.clone() for p in params],
                    bucket_cap_bytes=4 * dh * dout)
    names = ["W1", "b1", "W2", "b2"]
    live = [torch.ones_like(p, dtype=torch.bool) for p in params]
    g_worst, g_ok = 0.0, True
    for _ in range(steps):
        sharded.step(xs, ys)
        single.step(xf, yf)
        sharded.synchronize()
        single.synchronize()
        # The averaged gradient itself: sum over ranks / N against the one-rank gradient.
        for i, n in enumerate(names):
            ga, gb = sharded.ddp.grad(n) / world, single.ddp.grad(n)
            scale = float(gb.abs().max()) + 1e-30
            err, bound = (ga - gb).abs(), 1e-4 * gb.abs() + 1e-6 * scale
            g_worst = max(g_worst, float((err / bound).max()))
            g_ok = g_ok and bool((err <= bound).all())
            # Where a gradient is within rounding of zero, Adam's early steps are +-lr * sign(g) and two
            # correct runs may differ by 2 * lr: those elements are judged on the gradient alone.
            live[i] &= gb.abs() >= 1e-5 * scale
    worst, ok = 0.0, g_ok
    for a, b, m in zip(sharded.params, single.params, live):
        err = (a - b).abs()[m]
        bound = (1e-4 * b.abs() + 2e-4)[m]
        if err.numel():
            worst = max(worst, float((err / bound).max()))
            ok = ok and bool((err <= bound).all())
    moved = float((single.params[0] - params[0]).abs().max())
    flag = torch.tensor([1.0 if ok else 0.0, worst, g_worst], device=be.device)
    if world > 1:
        dist.all_reduce(flag[:1], op=dist.ReduceOp.MIN)
        dist.all_reduce(flag[1:], op=dist.ReduceOp.MAX)
    return {"ok": bool(flag[0].item() == 1.0), "steps": steps, "world": world,
            "shape": f"batch {batch}, {din}->{dh}->{dout}",
            "params_worst_err_over_bound": float(flag[1].item()), "grads_worst_err_over_bound": float(flag[2].item()),
            "bound": "parameters: 1e-4 * |p| + 2e-4; averaged gradients: 1e-4 * |g| + 1e-6 * max|g|; N ranks vs one rank on the "
                     "same global batch (parameter elements whose gradient is below 1e-5 of the largest are judged on the gradient)",
            "max_param_change": moved}


def allreduce_probe(be, comm, world, dist, sizes_bytes, reps=5):
    """Stand-alone all-reduce of each size (nothing else on the GPU): bus bandwidth 2(N-1)/N * S / t."""
    import torch
    if world == 1:
        return None
    out = []
    s = torch.cuda.Stream(device=be.device)
    for nbytes in sizes_bytes:
        n = nbytes // 4
        with torch.cuda.stream(s):
            buf = torch.zeros(n, device=be.device)
        for _ in range(2):
            comm.allreduce_sum(buf.data_ptr(), n, s.cuda_stream)
        s.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(s)
            comm.allreduce_sum(buf.data_ptr(), n, s.cuda_stream)
            z.record(s)
            s.synchronize()
            ts.append(a.elapsed_time(z))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=be.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        bus = 2 * (world - 1) / world * nbytes / (ms * 1e-3) / 1e9
        out.append({"bytes": int(nbytes), "ms": ms, "bus_gbs": bus, "frac_of_nvlink_nominal": bus / NVLINK_NOMINAL_GBS,
                    "frac_of_nvlink_measured_copy": bus / NVLINK_MEASURED_GBS})
        del buf
    return out


def run_ddp_record(be, comm, rank, world, dist, sampler, hbm_peak, steps=5, warmup=3, check=True):
    """Returns the `ddp_mlp` record (rank 0; None elsewhere)."""
    import torch
    from ferro_b200.backend import AdamWStep
    from ferro_b200.ddp import DdpMlp, shard_rows

    def fence():
        mlp.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    chk = parity_check(be, comm, rank, world, dist) if check else None
    lo, hi = shard_rows(rank, world, B)
    R = hi - lo
    params = draw_params(be, rank, world, dist, DIN, DH, DOUT, seed=1)
    x, y = draw_batch(be, lo, hi, B, DIN, DOUT, seed=2)
    mlp = DdpMlp(be, DIN, DH, DOUT, R, lr=1e-3, comm=comm, params=params, timing=True)
    for _ in range(max(warmup, 3)):
        mlp.step(x, y)
    fence()
    mlp.ddp.timings()  # drop the warm-up log
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = be.lib.fb_launch_count()
    fence()
    host_t0 = time.time()
    a.record(be.stream)
    for _ in range(steps):
        loss = mlp.step(x, y)
    be.stream.wait_event(mlp.done)
    z.record(be.stream)
    fence()
    host_t1 = time.time()
    launches = be.lib.fb_launch_count() - launches0
    ms = a.elapsed_time(z) / steps
    tm = mlp.ddp.timings()
    # The optimizer alone (its own roofline: 28 bytes per parameter), on the optimizer stream.
    hp = be._hp(AdamWStep(1e-3, 0.9, 0.999, 0.1, 0.001, 1e-8, 0.0))
    dev_table, n_t, total = mlp.ddp.all_table
    c, d = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c.record(be.stream)
    for _ in range(5):
        be._check(be.lib.fb_adamw_multi(be._s(), dev_table.data_ptr(), n_t, total, hp, 1.0 / world))
    d.record(be.stream)
    fence()
    adam_ms = c.elapsed_time(d) / 5
    t = torch.tensor([ms, adam_ms, tm["exposed_ms"], tm["update_tail_ms"]] + tm["allreduce_ms"], device=be.device,
                     dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    vals = t.tolist()
    ms, adam_ms, exposed, tail = vals[:4]
    ar_ms = vals[4:]
    probe = allreduce_probe(be, comm, world, dist, tm["bucket_bytes"] + [sum(tm["bucket_bytes"])])
    if rank != 0:
        return None
    n_params = mlp.n_params()
    adam_gbs = 28 * n_params / (adam_ms * 1e-3) / 1e9
    buckets = []
    for names, nbytes, t_ms in zip(tm["bucket_names"], tm["bucket_bytes"], ar_ms):
        rec = {"names": names, "bytes": int(nbytes), "allreduce_ms_in_step": t_ms}
        if world > 1 and t_ms > 0:
            bus = 2 * (world - 1) / world * nbytes / (t_ms * 1e-3) / 1e9
            rec.update({"bus_gbs_in_step": bus, "frac_of_nvlink_nominal": bus / NVLINK_NOMINAL_GBS})
        buckets.append(rec)
    return {
        "metric": "ddp_mlp_step_samples_per_s", "value": B / (ms * 1e-3), "unit": "samples/s", "n_gpus": world,
        "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms, "scaling": "strong", "dtype": "f32",
        "workload": "2-layer MLP 4096->16384(relu)->4096, global batch 65536 sharded by rows, MSE, Adam; cuBLAS f32 GEMMs; "
                    "parameters from ferro Rng seed 1, batch from seed 2",
        "loss": float(loss.item()), "rows_per_rank": R,
        "grad_bytes": 4 * n_params,
        "exchange": {"via": "fb_ddp_allreduce_bucket (NCCL over NVLink) on a side stream, one call per bucket as soon as its "
                            "last gradient is enqueued; 1/N folded into fb_adamw_multi",
                     "buckets": buckets, "exposed_ms": exposed, "update_tail_ms": tail,
                     "exposed_how": "device time from the end of backward (compute stream) to the end of the last all-reduce",
                     "standalone_allreduce": probe,
                     "nvlink_roofline_gbs": {"nominal_per_direction": NVLINK_NOMINAL_GBS,
                                             "measured_peer_copy": NVLINK_MEASURED_GBS}},
        "adam": {"kernel": "multi_step_kernel (fb_adamw_multi, 134 238 208 params)", "ms": adam_ms, "gbs": adam_gbs,
                 "frac_of_peak": adam_gbs / hbm_peak, "bytes": 28 * n_params},
        "gemm_flops_per_step": 6 * B * (DIN * DH + DH * DOUT),
        "gemm_tflops_per_gpu": 6 * B * (DIN * DH + DH * DOUT) / world / (ms * 1e-3) / 1e12,
        "gpu_launches": int(launches), "clocks": sampler.window(host_t0, host_t1) if sampler else None,
        "ddp_check": chk,
    }
