"""Benchmark of the hot path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Headline workload `layernorm_fwd_bwd`: LayerNorm forward + backward over f32
rows [32768, 4096] per GPU (x ~ N(0,1) scaled per row by U(0.5, 4), gamma ~
N(1, 0.02), beta ~ N(0, 0.02), eps 1e-5, upstream gradient ~ N(0,1), drawn
with ferro's Rng from seed 0 + rank); outputs y, mean, rstd, dx, dgamma,
dbeta.  A step is one forward and one backward over the whole batch.  With N
GPUs every rank owns its own 32768 rows (weak scaling, rows are independent);
the only exchange is the sum of the [2, 4096] parameter gradients, through
the library's communicator on a side stream, overlapped with the next
forward.

Metric: HBM GB/s on the algorithmic bytes of the step (read x, write y; read
x and g, write dx: 5 passes over the batch = 2 684 354 560 bytes per GPU),
whole job.  `e2e` is the same metric with the inputs in pinned host memory
and every output read back to the host inside the timed region.

The same line carries two more records (their own timed regions, after the
headline one):
  `configs`  (1 GPU)   every kernel of configurations 1, 3, 4 and 5 at full
                       size with its own clock sample (bench_configs.py)
  `ddp_mlp`  (every N) the data-parallel MLP training step of configuration 5,
                       strong scaling, with the all-reduce figures against the
                       NVLink roofline and a parity check of N ranks against
                       one (bench_ddp.py)
`--workload ddp_mlp` prints the ddp record alone, `--workload kernels` the
wider per-kernel sweep of bench_kernels.py.

`--impl reference` times ferro's own CPU implementation of the headline step
(the C restatement under oracle/, all host threads) on a bounded row sample.
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
print_line = print  # replaced in main(): the JSON line goes to the process's original stdout

ROWS, COLS, EPS = 32768, 4096, 1e-5
FWD_BYTES_PER_ROW = 2 * COLS * 4          # read x, write y
BWD_BYTES_PER_ROW = 3 * COLS * 4          # read x, g, write dx
METRIC = "layernorm_fwd_bwd_hbm_gbs"


from bench_common import ClockSampler, peaks  # noqa: E402


def cpu_baseline(seconds_target=12.0):
    """ferro's CPU path (oracle, OpenMP over rows) on a bounded row sample; GB/s on the same byte count."""
    import numpy as np
    import oracle as fo
    fo.use_all_cores()  # torchrun exports OMP_NUM_THREADS=1; ferro's CPU path uses every core regardless
    rows = 2048
    r = np.random.default_rng(0)
    x = (r.standard_normal((rows, COLS)) * r.uniform(0.5, 4, (rows, 1))).astype(np.float32)
    w = (1 + 0.02 * r.standard_normal(COLS)).astype(np.float32)
    b = (0.02 * r.standard_normal(COLS)).astype(np.float32)
    g = r.standard_normal((rows, COLS)).astype(np.float32)

    def step():
        y, h, s, m = fo.layer_norm_fwd(x, w, b, EPS)
        fo.layer_norm_bwd(g, h, s, w)

    step()
    t0 = time.perf_counter()
    step()
    one = time.perf_counter() - t0
    reps = max(3, min(200, int(seconds_target / max(one, 1e-4))))
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t0)
    ts.sort()
    med = ts[len(ts) // 2]
    gbs = rows * (FWD_BYTES_PER_ROW + BWD_BYTES_PER_ROW) / med / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": fo.max_threads(), "kind": "port",
            "sample": f"{rows} of {ROWS} rows x {COLS} cols, fwd+bwd, median of {reps}",
            "ms_per_sample": med * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpu_baseline(seconds_target=max(5.0, 4.0 * args.steps))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": base["ms_per_sample"] * ROWS / 2048, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config(args.gpus),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print_line(json.dumps(line))


WORKLOAD = "layernorm_fwd_bwd f32 [32768,4096] per GPU, eps 1e-5, affine; outputs y, mean, rstd, dx, dgamma, dbeta"


def config(world):
    """The `config` object both arms print."""
    return {"workload": WORKLOAD, "l2": "inputs (537 MB per array) larger than L2",
            "exchange": "all-reduce(sum) of dgamma/dbeta [2,4096] (fb_ddp_allreduce_bucket, NCCL) on a side stream"
                        if world > 1 else "none",
            "inputs": "ferro Rng, seed 0 + rank, order x (row scale before each row), gamma, beta, g"}


def traffic_record():
    """DRAM bytes of one launch of the dominant kernel, from the ncu capture whose figures are kept
    beside its summary under profiles/ (None when that file is absent)."""
    path = os.path.join(ROOT, "profiles", "layer_norm_bwd_dram_traffic.json")
    try:
        rec = json.load(open(path))
        return int(rec["dram_bytes_per_launch"]), rec.get("kernel")
    except (OSError, ValueError, KeyError):
        return None, None


def setup():
    """Process group (plumbing: barrier, max over ranks), backend and the library's own communicator."""
    import torch
    import torch.distributed as dist
    from ferro_b200.backend import CudaBackend
    from ferro_b200.ddp import NcclComm, share_id_over_process_group

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    be = CudaBackend(local)
    comm = NcclComm(rank, world, share_id_over_process_group(device=be.device) if world > 1 else None)
    return torch, dist, be, comm, world, rank, local


def run_ours(args):
    torch, dist, be, comm, world, rank, local = setup()
    from ferro_b200.backend import DeviceBuffer
    from ferro_b200.rng import Rng
    from bench_common import Staging
    dev = be.device
    rows, cols = ROWS, COLS
    sampler = ClockSampler(local).start() if rank == 0 else None

    # Synthetic inputs of the configured shapes and distributions (ferro's Rng), pinned on the host.
    rng = Rng(rank)
    x_h = torch.empty(rows * cols, dtype=torch.float32).pin_memory()
    g_h = torch.empty(rows * cols, dtype=torch.float32).pin_memory()
    w_h, b_h = torch.empty(cols).pin_memory(), torch.empty(cols).pin_memory()
    rng.fill_rowscaled_normal(rows, cols, 0.5, 3.5, out=x_h)
    rng.fill_normal((cols,), 0.02, 1.0, out=w_h)
    rng.fill_normal((cols,), 0.02, 0.0, out=b_h)
    rng.fill_normal((rows * cols,), out=g_h)
    with torch.cuda.stream(be.stream):
        X = DeviceBuffer(x_h.to(dev, non_blocking=True))
        G = DeviceBuffer(g_h.to(dev, non_blocking=True))
        W = DeviceBuffer(w_h.to(dev, non_blocking=True))
        Bv = DeviceBuffer(b_h.to(dev, non_blocking=True))
        Y = DeviceBuffer(torch.empty(rows * cols, device=dev))
        DX = DeviceBuffer(torch.empty(rows * cols, device=dev))
        MU = DeviceBuffer(torch.empty(rows, device=dev))
        RS = DeviceBuffer(torch.empty(rows, device=dev))
        # dgamma | dbeta, a ring of 4: the exchange of step k runs beside the forward of step k + 1, and the
        # backward that reuses a slot only has to wait for an exchange issued four steps earlier.
        RING = 4
        DWBS = [torch.empty(2 * cols, device=dev) for _ in range(RING)]
        DWB = DWBS[0]
        ws_bytes = int(be.lib.fb_layer_norm_bwd_workspace_bytes(rows, cols))
        WS = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    be.synchronize()
    lib, s = be.lib, be._s()
    # High priority: the all-reduce's few CTAs are placed as soon as an SM has room, beside the next forward's small
    # CTAs, instead of queueing behind that grid and landing on the persistent backward (measured at 4 GPUs: the
    # backward ran 15 us longer on every rank with a default-priority exchange stream).
    xchg = torch.cuda.Stream(device=dev, priority=-1)
    ev_grads = [torch.cuda.Event() for _ in range(RING)]
    ev_summed = [torch.cuda.Event() for _ in range(RING)]
    slot = [0]

    def fwd():
        be._check(lib.fb_layer_norm_fwd(s, X.ptr, W.ptr, Bv.ptr, rows, cols, EPS, Y.ptr, None, None, MU.ptr, RS.ptr))

    def bwd():
        k = slot[0]
        if world > 1:
            be.stream.wait_event(ev_summed[k])  # the sum issued RING steps ago has left this slot
        d = DWBS[k]
        be._check(lib.fb_layer_norm_bwd(s, G.ptr, None, None, X.ptr, MU.ptr, RS.ptr, W.ptr, rows, cols, DX.ptr,
                                        d.data_ptr(), d.data_ptr() + 4 * cols, WS.data_ptr(), WS.numel()))

    def exchange():
        # The parameter gradients are summed over ranks on a side stream while the next forward runs.
        k = slot[0]
        if world > 1 and not args.no_exchange:
            ev_grads[k].record(be.stream)
            xchg.wait_event(ev_grads[k])
            comm.allreduce_sum(DWBS[k].data_ptr(), 2 * cols, xchg.cuda_stream)
            ev_summed[k].record(xchg)
        slot[0] = (k + 1) % RING

    def step():
        fwd()
        bwd()
        exchange()

    def fence():
        if world > 1:
            for e in ev_summed:
                be.stream.wait_event(e)
        be.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    fence()

    ev = lambda: torch.cuda.Event(enable_timing=True)
    marks = []
    launches0 = lib.fb_launch_count()
    t_start, t_end = ev(), ev()
    fence()
    host_t0 = time.time()
    t_start.record(be.stream)
    for _ in range(args.steps):
        e0, e1, e2 = ev(), ev(), ev()
        e0.record(be.stream)
        fwd()
        e1.record(be.stream)
        bwd()
        e2.record(be.stream)
        exchange()
        marks.append((e0, e1, e2))
    if world > 1:
        for e in ev_summed:
            be.stream.wait_event(e)  # every exchange is inside the timed region
    t_end.record(be.stream)
    fence()
    launches = lib.fb_launch_count() - launches0
    total_ms = t_start.elapsed_time(t_end)
    fwd_ms = sum(a.elapsed_time(b) for a, b, _ in marks) / args.steps
    bwd_ms = sum(b.elapsed_time(c) for _, b, c in marks) / args.steps
    # nvidia-smi samples every 50 ms and the timed region may be shorter than that: keep the
    # GPU on the very same step loop (untimed) until 1.5 s have passed since the timed region
    # began, and report the clocks seen over that window.
    # Every rank must run the same number of steps here (each step holds a collective): the count comes from
    # the slowest rank's measured step time, not from each rank's own clock.
    pace = torch.tensor([total_ms / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(pace, op=dist.ReduceOp.MAX)
    batches = int(max(0.0, 1500.0 - total_ms) / (10.0 * max(pace.item(), 1e-3))) + 1
    for _ in range(batches):
        for _ in range(10):
            step()
        be.synchronize()
    fence()
    clocks = sampler.window(host_t0, time.time()) if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "timed region plus an untimed continuation of the same step loop, 1.5 s in all"

    # End to end through the host-buffer entry point: inputs in pinned host memory, every output
    # (y, dx, mean, rstd, dgamma, dbeta) back in pinned host memory, copies inside the timed region.
    from ferro_b200.host_api import HostLayerNorm
    del Y, DX
    hln = HostLayerNorm(be, rows, cols, EPS, chunks=8)
    xh2, gh2 = x_h.view(rows, cols), g_h.view(rows, cols)
    y_h = torch.empty(rows, cols, dtype=torch.float32).pin_memory()
    dx_h = torch.empty(rows, cols, dtype=torch.float32).pin_memory()
    mu_h, rs_h = torch.empty(rows).pin_memory(), torch.empty(rows).pin_memory()
    dwb_h = torch.empty(2 * cols).pin_memory()
    dwb_d = torch.empty(2 * cols, device=dev)

    def e2e_step():
        hln(xh2, gh2, w_h, b_h, y_h, dx_h, mu_h, rs_h, dwb_h)
        if world > 1:
            hln.synchronize()
            with torch.cuda.stream(xchg):
                dwb_d.copy_(dwb_h, non_blocking=True)
                comm.allreduce_sum(dwb_d.data_ptr(), 2 * cols, xchg.cuda_stream)
                dwb_h.copy_(dwb_d, non_blocking=True)
            xchg.synchronize()

    e2e_steps = max(2, min(args.steps, 5))
    ref_dwb = DWBS[(slot[0] - 1) % RING].cpu() if world == 1 else None
    e2e_step()
    hln.synchronize()
    fence()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    hln.synchronize()
    fence()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    # The pipelined result equals the one-shot kernels' result.
    if ref_dwb is not None:
        err = (dwb_h - ref_dwb).abs().max().item()
        assert err <= 2e-4 * ref_dwb.abs().max().item() + 1e-3, f"host pipeline disagrees with the resident path: {err}"
    h2d, d2h = hln.bytes_in(), hln.bytes_out()
    hln.close()
    del hln, X, G, y_h, dx_h, x_h, g_h, xh2, gh2
    torch.cuda.empty_cache()

    # max over ranks (and every rank's own figures beside it: the GPUs of one box are not equally fast)
    t = torch.tensor([total_ms, e2e_ms, fwd_ms, bwd_ms], device=dev, dtype=torch.float64)
    per_rank = None
    if world > 1:
        every = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        per_rank = [{"rank": r, "ms_per_step": v[0].item() / args.steps, "ln_fwd_ms": v[2].item(), "ln_bwd_ms": v[3].item()}
                    for r, v in enumerate(every)]
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, fwd_ms, bwd_ms = t.tolist()

    peak, which = peaks()
    configs = ref_gpu = None
    if world == 1 and not args.no_configs:
        from bench_configs import run_configs, run_reference_gpu
        configs = run_configs(be, sampler, peak)
        ref_gpu = run_reference_gpu(be, sampler, peak)
    ddp = None
    if not args.no_ddp:
        from bench_ddp import run_ddp_record
        ddp = run_ddp_record(be, comm, rank, world, dist, sampler, peak, steps=max(3, min(args.steps, 5)),
                             warmup=args.warmup)

    if rank == 0:
        sampler.stop()
        step_bytes = rows * (FWD_BYTES_PER_ROW + BWD_BYTES_PER_ROW)
        ms_per_step = total_ms / args.steps
        value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
        bwd_bytes = rows * BWD_BYTES_PER_ROW
        achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
        fwd_gbs = rows * FWD_BYTES_PER_ROW / (fwd_ms * 1e-3) / 1e9
        base = cpu_baseline() if world == 1 and not args.no_cpu_baseline else None
        traffic, traffic_kernel = traffic_record()
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(config(world), **({"exchange": "left out (--no-exchange, diagnostic run)"}
                                             if world > 1 and args.no_exchange else {})),
            "rows_per_s": world * rows / (ms_per_step * 1e-3),
            "kernels": {"ln_fwd": {"ms": fwd_ms, "gbs": fwd_gbs, "frac_of_peak": fwd_gbs / peak},
                        "ln_bwd": {"ms": bwd_ms, "gbs": achieved, "frac_of_peak": achieved / peak}},
            "roofline": {"bound": "hbm", "kernel": traffic_kernel or "LayerNorm backward", "achieved": achieved,
                         "peak": peak, "peak_source": which, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic},
            "e2e": {"value": world * step_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "fb_host_ln_run (C ABI, host pointers in, host pointers out): 8 row chunks, upload / compute / download "
                           "overlapped on three streams inside the library; host wall clock"},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if per_rank is not None:
            line["per_rank"] = per_rank  # value / ms_per_step are the max over these
        if base:
            line["cpu_baseline"] = base
        if configs is not None:
            line["configs"] = configs
            if not args.no_cpu_baseline:
                line["configs_cpu_baseline"] = cpu_config_baselines()
            if ref_gpu is not None:
                line["reference_source_recompiled"] = ref_gpu
        if ddp is not None:
            line["ddp_mlp"] = ddp
        print_line(json.dumps(line))
    comm.close()
    if world > 1:
        dist.destroy_process_group()


def run_ddp(args):
    """--workload ddp_mlp: the data-parallel step's record alone, as the JSON line."""
    torch, dist, be, comm, world, rank, local = setup()
    from bench_ddp import run_ddp_record
    sampler = ClockSampler(local).start() if rank == 0 else None
    peak, _ = peaks()
    rec = run_ddp_record(be, comm, rank, world, dist, sampler, peak, steps=args.steps, warmup=args.warmup)
    if rank == 0:
        sampler.stop()
        rec.update({"higher_is_better": True, "vs_baseline": None, "data": "synthetic",
                    "config": {"workload": rec["workload"], "l2": "activations (1 GB and more per array) larger than L2"}})
        print_line(json.dumps(rec))
    comm.close()
    if world > 1:
        dist.destroy_process_group()


def cpu_config_baselines():
    """ferro's CPU path (oracle, all host threads) on bounded samples of configurations 1-5, in GB/s on
    the same algorithmic bytes the GPU rows use."""
    import numpy as np
    import oracle as fo
    from ferro_b200 import kinds as K
    fo.use_all_cores()
    r = np.random.default_rng(0)
    out = {}

    def timed(fn, reps=5):
        fn()
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return sorted(ts)[len(ts) // 2]

    # C1 (full size): softmax(relu(x+b)*s) forward, then backward to dx, db
    rows, cols = 8192, 1024
    x, b, g = r.standard_normal((rows, cols), np.float32), (0.1 * r.standard_normal(cols)).astype(np.float32), r.standard_normal((rows, cols), np.float32)
    sc = np.full((rows, cols), 0.125, np.float32)
    state = {}

    def c1_fwd():
        pre = fo.binary_bc(K.BIN_ADD, x, b)
        state["pre"] = pre
        state["y"] = fo.softmax_fwd(fo.binary(K.BIN_MUL, fo.unary(K.UN_RELU, pre, mt=True), sc, mt=True))

    def c1_bwd():
        dt = fo.softmax_bwd(g, state["y"])
        dx = fo.binary(K.BIN_RELU_BACKWARD, fo.binary(K.BIN_MUL, dt, sc, mt=True), state["pre"], mt=True)
        fo.sum_dim(dx, 0, mt=True)

    out["c1_fwd"] = {"gbs": 2 * x.nbytes / timed(c1_fwd) / 1e9, "sample": "full [8192,1024]"}
    out["c1_bwd"] = {"gbs": 4 * x.nbytes / timed(c1_bwd) / 1e9, "sample": "full [8192,1024]"}
    # C3: cross entropy forward+backward with argmax on 256 of 16384 rows
    rows, cols = 256, 32000
    lg, tg = (2 * r.standard_normal((rows, cols))).astype(np.float32), r.integers(0, cols, rows)
    t = timed(lambda: fo.cross_entropy_indices(lg, tg), 3)
    out["c3_fwd_bwd"] = {"gbs": 3 * lg.nbytes / t / 1e9, "sample": "256 of 16384 rows x 32000"}
    # C4: the chain on 512 of 16384 rows, and sum_dim over each axis of a [32,512,2048] block
    rows, cols = 512, 16384
    a, at, col = (8 * r.random((rows, cols), np.float32) - 4), (8 * r.random((rows, cols), np.float32) - 4), (8 * r.random((rows, 1), np.float32) - 4)
    one = np.ones((rows, 1), np.float32)

    def c4_chain():
        t1 = fo.unary(K.UN_EXP, fo.unary(K.UN_NEG, fo.unary(K.UN_ABS, a, mt=True), mt=True), mt=True)
        t2 = fo.unary(K.UN_SQRT, fo.binary(K.BIN_ADD, fo.unary(K.UN_ABS, col), one))
        t3 = fo.unary(K.UN_TANH, fo.binary_bc(K.BIN_MUL, t1, t2), mt=True)
        fo.unary(K.UN_CLAMP, fo.binary(K.BIN_ADD, t3, fo.unary(K.UN_POWF, at, 1.5, mt=True), mt=True), -1.0, 1.0, mt=True)

    out["c4_chain"] = {"gbs": 2 * a.nbytes / timed(c4_chain, 3) / 1e9, "sample": "512 of 16384 rows x 16384 (ferro runs it op by op)"}
    blk = r.standard_normal((32, 512, 2048), np.float32)
    for dim in range(3):
        out[f"c4_sum_dim{dim}"] = {"gbs": blk.nbytes / timed(lambda: fo.sum_dim(blk, dim, mt=True), 3) / 1e9,
                                   "sample": "[32,512,2048] of [256,512,2048]"}
    # C5: Adam over 16 777 216 of 134 238 208 parameters
    n = 1 << 24
    p_, m_, g_ = (r.standard_normal(n, np.float32) for _ in range(3))
    v_ = np.abs(r.standard_normal(n, np.float32))
    out["c5_adam"] = {"gbs": 28 * n / timed(lambda: fo.adamw_step(p_, m_, v_, g_, 1e-3, 0.9, 0.999, 0.1, 0.001, 1e-8, 0.0), 5) / 1e9,
                      "sample": "16 777 216 of 134 238 208 parameters"}
    return {"cores": fo.max_threads(), "kind": "port", "rows": out}


def run_kernels(args):
    """--workload kernels: the wider per-kernel sweep (bench_kernels.py) with the CPU path's figures
    for the same configurations beside it."""
    import bench_kernels as kb
    B = kb.Bench(max(5, args.steps))
    kb.cases(B, None)
    base = cpu_config_baselines() if not args.no_cpu_baseline else None
    print_line(json.dumps({"metric": "kernel_table_hbm_gbs", "unit": "GB/s", "n_gpus": 1, "peak": B.peak,
                      "peak_source": B.peak_src, "rows": B.rows, "cpu_baseline": base}))


def main():
    # Libraries below us print to stdout on their own (NCCL announces its version there): keep file
    # descriptor 1 for the one JSON line and send everything else to stderr.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    global print_line
    print_line = lambda text: os.write(json_fd, (text + "\n").encode())
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the per-configuration kernel records")
    ap.add_argument("--no-ddp", action="store_true", help="skip the data-parallel MLP record")
    ap.add_argument("--no-exchange", action="store_true",
                    help="diagnostic: leave the gradient all-reduce out of the headline step (N > 1), to separate its cost "
                         "from the spread between the GPUs of a box; the line says so in config.exchange")
    ap.add_argument("--workload", default="layernorm_fwd_bwd", choices=["layernorm_fwd_bwd", "ddp_mlp", "kernels"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "ddp_mlp":
        run_ddp(args)
    elif args.workload == "kernels":
        run_kernels(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

