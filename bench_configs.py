"""The kernels of the published configurations 1, 3, 4 and 5 at full size, one record per
kernel: algorithmic bytes, median CUDA-event time, GB/s, fraction of the measured HBM copy rate,
rows/s where a row is the unit, and the clocks sampled over that kernel's own timed loop.

Inputs are the configurations' seeded draws (seed 0 through ferro's Rng, in the order the
tensors are listed; configuration 5's parameters from seed 1).  Every kernel is one library
call through the C ABI; L2 is flushed between timed iterations.
"""
import time

from bench_common import Flusher, Staging, time_call, time_rotating


def _record(out, sampler, peak, name, kernel, nbytes, timing, rows=None, extra=None):
    med, mn, iters, launches, t0, t1 = timing
    gbs = nbytes / (med * 1e-3) / 1e9
    rec = {"kernel": kernel, "bytes": int(nbytes), "ms": med, "ms_min": mn, "iters": iters, "gbs": gbs,
           "frac_of_peak": gbs / peak, "launches": launches, "clocks": sampler.window(t0, t1)}
    if rows:
        rec["rows_per_s"] = rows / (med * 1e-3)
    if extra:
        rec.update(extra)
    out[name] = rec


def run_configs(be, sampler, peak, min_s=0.6, which=("c1", "c3", "c4", "c5")):
    import torch
    from ferro_b200.backend import AdamWStep, BinaryKind, ChainStep, DeviceBuffer, T, UnaryKind, View
    from ferro_b200.rng import Rng

    lib, S = be.lib, be._s
    flush = Flusher(be)
    stage = Staging(be)
    out = {}
    tc = lambda fn: time_call(be, fn, flush, min_s)
    empty = lambda n, dt=torch.float32: be._alloc(n, dt)

    # ---- configuration 1: y = softmax(relu(x + b) * 0.125), backward to dx, db; [8192, 1024]
    if "c1" in which:
        r, c = 8192, 1024
        rng = Rng(0)
        x = DeviceBuffer(stage.normal(rng, r * c))
        bias = DeviceBuffer(stage.normal(rng, c, 0.1))
        g = DeviceBuffer(stage.normal(rng, r * c))
        y, dx, db = empty(r * c), empty(r * c), empty(c)
        wsb = int(lib.fb_softmax_fused_bwd_workspace_bytes(r, c))
        ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=be.device)
        fwd = lambda: be._check(lib.fb_bias_act_scale_softmax_fwd(S(), x.ptr, bias.ptr, 1, 0.125, r, c, y.ptr))
        bwd = lambda: be._check(lib.fb_bias_act_scale_softmax_bwd(S(), g.ptr, y.ptr, x.ptr, bias.ptr, 1, 0.125, r, c,
                                                                  dx.ptr, db.ptr, ws.data_ptr(), ws.numel()))
        # Configuration 1 moves 67 / 134 MB per call, less than the 126 MB L2, so its figures are taken
        # over 8 rotating buffer sets (1 GB in all, each set untouched for the 7 calls in between): every
        # input comes from HBM and every output has to leave L2, as in a steady stream of such calls.
        # (Rewriting a flush buffer before each call instead leaves L2 full of that buffer's dirty lines,
        # whose write-back is then charged to the 10 - 30 us kernel under test; that figure is kept as
        # `flushed`.)
        K = 8
        with torch.cuda.stream(be.stream):
            xs = [DeviceBuffer(x.t.clone()) for _ in range(K)]
            gs = [DeviceBuffer(g.t.clone()) for _ in range(K)]
        ys, dxs = [empty(r * c) for _ in range(K)], [empty(r * c) for _ in range(K)]

        def rot(name, kernel, nbytes, fns, single):
            m = time_rotating(be, fns, min_s)
            flushed = tc(single)
            _record(out, sampler, peak, name, kernel, nbytes, (m[0], m[1], m[2], flushed[3], m[3], m[4]), r,
                    {"l2": "8 rotating buffer sets (1 GB in all), calls back to back; ms is per call",
                     "flushed": {"ms": flushed[0], "gbs": nbytes / (flushed[0] * 1e-3) / 1e9,
                                 "how": "one buffer set, a 256 MB buffer rewritten before every call"}})

        rot("c1_fwd", "fb_bias_act_scale_softmax_fwd [8192,1024]", 2 * r * c * 4,
            [(lambda i=i: be._check(lib.fb_bias_act_scale_softmax_fwd(S(), xs[i].ptr, bias.ptr, 1, 0.125, r, c, ys[i].ptr)))
             for i in range(K)], fwd)
        rot("c1_bwd", "fb_bias_act_scale_softmax_bwd dx,db [8192,1024]", 4 * r * c * 4,
            [(lambda i=i: be._check(lib.fb_bias_act_scale_softmax_bwd(
                S(), gs[i].ptr, ys[i].ptr, xs[i].ptr, bias.ptr, 1, 0.125, r, c, dxs[i].ptr, db.ptr, ws.data_ptr(), ws.numel())))
             for i in range(K)], bwd)
        rot("softmax_fwd", "fb_softmax_fwd [8192,1024]", 2 * r * c * 4,
            [(lambda i=i: be._check(lib.fb_softmax_fwd(S(), xs[i].ptr, r, c, ys[i].ptr))) for i in range(K)],
            lambda: be._check(lib.fb_softmax_fwd(S(), x.ptr, r, c, y.ptr)))
        rot("softmax_bwd", "fb_softmax_bwd [8192,1024]", 3 * r * c * 4,
            [(lambda i=i: be._check(lib.fb_softmax_bwd(S(), gs[i].ptr, ys[i].ptr, r, c, dxs[i].ptr))) for i in range(K)],
            lambda: be._check(lib.fb_softmax_bwd(S(), g.ptr, y.ptr, r, c, dx.ptr)))
        # What the same bytes cost as plain streaming kernels of this library at this size: the floor a
        # 10 - 30 us launch can reach here (launch, ramp and drain are a fifth of it).
        rot("c1_ref_copy_2_arrays", "fb_copy of 8 388 608 floats (read 33.5 MB, write 33.5 MB): reference for c1_fwd", 2 * r * c * 4,
            [(lambda i=i: be._check(lib.fb_copy(S(), ys[i].ptr, xs[i].ptr, r * c))) for i in range(K)],
            lambda: be._check(lib.fb_copy(S(), y.ptr, x.ptr, r * c)))
        rot("c1_ref_add_3_arrays", "fb_binary add of 8 388 608 floats (3 arrays of 33.5 MB): reference for the backward kernels", 3 * r * c * 4,
            [(lambda i=i: be._check(lib.fb_binary(S(), 0, 0.0, 0.0, xs[i].ptr, gs[i].ptr, ys[i].ptr, r * c))) for i in range(K)],
            lambda: be._check(lib.fb_binary(S(), 0, 0.0, 0.0, x.ptr, g.ptr, y.ptr, r * c)))
        del x, g, y, dx, xs, gs, ys, dxs

    # ---- configuration 3: log_softmax + NLL (+argmax) forward, dlogits backward; [16384, 32000]
    if "c3" in which:
        r, c = 16384, 32000
        rng = Rng(0)
        x = DeviceBuffer(stage.normal(rng, r * c, 2.0))
        t = DeviceBuffer(stage.index(rng, r, c))
        loss, rmax, rlse, am, dl = empty(1), empty(r), empty(r), empty(r, torch.int64), empty(r * c)
        ws = torch.empty(int(lib.fb_nll_workspace_bytes(r)), dtype=torch.uint8, device=be.device)
        _record(out, sampler, peak, "c3_fwd", "fb_log_softmax_nll_fwd (+argmax) [16384,32000]", r * c * 4,
                tc(lambda: be._check(lib.fb_log_softmax_nll_fwd(S(), x.ptr, t.ptr, r, c, loss.ptr, rmax.ptr, rlse.ptr, am.ptr,
                                                                None, ws.data_ptr(), ws.numel()))), r)
        _record(out, sampler, peak, "c3_bwd", "fb_log_softmax_nll_bwd dlogits [16384,32000]", 2 * r * c * 4,
                tc(lambda: be._check(lib.fb_log_softmax_nll_bwd(S(), x.ptr, t.ptr, rmax.ptr, rlse.ptr, 1.0, r, c, dl.ptr))), r)
        _record(out, sampler, peak, "c3_log_softmax_fwd", "fb_log_softmax_fwd (materialised) [16384,32000]", 2 * r * c * 4,
                tc(lambda: be._check(lib.fb_log_softmax_fwd(S(), x.ptr, r, c, dl.ptr))), r)
        out["c3_fwd"]["loss"] = float(be.copy_to_host(loss)[0])
        del x, t, dl

    # ---- configuration 4: the chain over a [16384,16384] and its transpose, then 9 axis reductions
    if "c4" in which:
        n = 16384
        rng = Rng(0)
        a = DeviceBuffer(stage.uniform(rng, n * n, 8.0, -4.0))
        col = DeviceBuffer(stage.uniform(rng, n, 8.0, -4.0))
        U, Bi, St = UnaryKind, BinaryKind, ChainStep
        prog = [St.Load(0), St.Unary(U.Abs), St.Unary(U.Neg), St.Unary(U.Exp),
                St.Load(1, dst=T), St.Unary(U.Abs, dst=T), St.Binary(Bi.Add, imm=1.0, dst=T), St.Unary(U.Sqrt, dst=T),
                St.Binary(Bi.Mul), St.Unary(U.Tanh),
                St.Load(2, dst=T), St.Unary(U.Powf(1.5), dst=T), St.Binary(Bi.Add), St.Unary(U.Clamp(-1.0, 1.0))]
        ops = [View(a, (n, 1)), View(col, (1, 0)), View(a, (1, n))]
        z = empty(n * n)
        chain = lambda: be.chain_into(prog, ops, (n, n), z)
        _record(out, sampler, peak, "c4_chain", "fb_chain clamp(tanh(exp(-|a|)*sqrt(|b|+1))+powf(a^T,1.5)) [16384,16384], compiled program",
                2 * n * n * 4, tc(chain))
        prev = lib.fb_chain_catalogue(0)
        try:
            _record(out, sampler, peak, "c4_chain_interpreted", "the same fb_chain call on the step interpreter (catalogue off)",
                    2 * n * n * 4, tc(chain))
        finally:
            lib.fb_chain_catalogue(prev)
        del z
        shape = (n * n // (512 * 2048), 512, 2048)
        for dim in range(3):
            o = 1
            for s_ in shape[:dim]:
                o *= s_
            i = 1
            for s_ in shape[dim + 1:]:
                i *= s_
            red = shape[dim]
            res, idx = empty(o * i), empty(o * i, torch.int64)
            ws = torch.empty(max(int(lib.fb_reduce_dim_workspace_bytes(o, red, i)), 16), dtype=torch.uint8, device=be.device)
            wp, wn = ws.data_ptr(), ws.numel()
            _record(out, sampler, peak, f"c4_sum_dim{dim}", f"fb_sum_dim dim {dim} of [256,512,2048]", n * n * 4 + o * i * 4,
                    tc(lambda: be._check(lib.fb_sum_dim(S(), a.ptr, o, red, i, res.ptr, wp, wn))))
            _record(out, sampler, peak, f"c4_mean_dim{dim}", f"fb_mean_dim dim {dim} of [256,512,2048]", n * n * 4 + o * i * 4,
                    tc(lambda: be._check(lib.fb_mean_dim(S(), a.ptr, o, red, i, res.ptr, wp, wn))))
            _record(out, sampler, peak, f"c4_max_dim{dim}", f"fb_max_dim (+argmax) dim {dim} of [256,512,2048]", n * n * 4 + o * i * 12,
                    tc(lambda: be._check(lib.fb_max_dim(S(), a.ptr, o, red, i, res.ptr, idx.ptr, wp, wn))))
        del a, col

    # ---- configuration 5: fused Adam over the MLP's 134 238 208 parameters (4 tensors, one launch)
    if "c5" in which:
        sizes = [4096 * 16384, 16384, 16384 * 4096, 4096]
        fan = [4096, None, 16384, None]
        rng = Rng(1)
        with torch.cuda.stream(be.stream):
            ps = [DeviceBuffer(stage.normal(rng, sz, (2.0 / f) ** 0.5)) if f else DeviceBuffer(torch.zeros(sz, device=be.device))
                  for sz, f in zip(sizes, fan)]
            ms = [DeviceBuffer(torch.zeros(sz, device=be.device)) for sz in sizes]
            vs = [DeviceBuffer(torch.zeros(sz, device=be.device)) for sz in sizes]
        g5 = Rng(3)
        gs5 = [DeviceBuffer(stage.normal(g5, sz, 1e-2)) for sz in sizes]
        table = be.make_table(list(zip(ps, ms, vs, gs5)))
        total = sum(sizes)
        hp = AdamWStep(1e-3, 0.9, 0.999, 0.1, 0.001, 1e-8, 0.0)
        _record(out, sampler, peak, "c5_adam", "fb_adamw_multi 134238208 params (W1,b1,W2,b2), one launch", 28 * total,
                tc(lambda: be.adamw_multi_dev(table, hp, 1.0)), extra={"params_per_s": None})
        out["c5_adam"]["params_per_s"] = total / (out["c5_adam"]["ms"] * 1e-3)
        del ps, ms, vs, gs5, table
    del flush, stage
    torch.cuda.empty_cache()
    return out


def run_reference_gpu(be, sampler, peak, min_s=0.5):
    """"Reference source recompiled": ferro's own CUDA kernels (crates/ferro-cuda/src/layer_norm.cu and the
    softmax kernel text of kernels.rs:536-588), built for sm_100a by oracle/build_ref_gpu.py and launched
    with the reference's geometry, timed on the same GPU next to this library's entry for the same work.
    Not ferro as shipped (no Rust host, no nvrtc); a GPU-against-GPU anchor beside the CPU baseline.
    Returns None when the recompiled kernels are not present."""
    import ctypes as C
    import os
    import torch
    from ferro_b200.backend import DeviceBuffer
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "_ref", "libferro_ref_gpu.so")
    if not os.path.exists(path):
        return None
    ref = C.CDLL(path)
    ref.ref_gpu_layer_norm.argtypes = [C.c_void_p] * 7 + [C.c_uint, C.c_uint, C.c_float]
    ref.ref_gpu_softmax.argtypes = [C.c_void_p] * 4 + [C.c_uint, C.c_uint, C.c_int]
    lib, S = be.lib, be._s
    flush = Flusher(be)
    out = {"what": "ferro's CUDA kernels recompiled for sm_100a from the reference sources, reference launch geometry; "
                   "ours = this library's entry for the same outputs; ratio = reference time / ours"}

    def pair(name, nbytes, ref_fn, our_fn, rows):
        assert ref_fn() == 0
        r_ = time_call(be, ref_fn, flush, min_s)
        o_ = time_call(be, our_fn, flush, min_s)
        out[name] = {"bytes": int(nbytes), "reference_ms": r_[0], "reference_gbs": nbytes / (r_[0] * 1e-3) / 1e9,
                     "ours_ms": o_[0], "ours_gbs": nbytes / (o_[0] * 1e-3) / 1e9, "ratio": r_[0] / o_[0],
                     "reference_rows_per_s": rows / (r_[0] * 1e-3), "ours_rows_per_s": rows / (o_[0] * 1e-3),
                     "clocks": sampler.window(r_[4], o_[5])}

    with torch.cuda.stream(be.stream):
        gen = torch.Generator(device=be.device).manual_seed(0)
        rows, cols = 32768, 4096
        x = torch.randn(rows * cols, device=be.device, generator=gen)
        w, b = torch.randn(cols, device=be.device, generator=gen), torch.randn(cols, device=be.device, generator=gen)
        y, h, sd = torch.empty_like(x), torch.empty_like(x), torch.empty(rows, device=be.device)
    P = lambda t: t.data_ptr()
    pair("layer_norm_fwd (y, h, stds) [32768,4096]", 3 * rows * cols * 4,
         lambda: ref.ref_gpu_layer_norm(be.stream.cuda_stream, P(x), P(w), P(b), P(y), P(h), P(sd), rows, cols, 1e-5),
         lambda: be._check(lib.fb_layer_norm_fwd(S(), P(x), P(w), P(b), rows, cols, 1e-5, P(y), P(h), P(sd), None, None)), rows)
    pair("layer_norm_fwd (y only) [32768,4096]", 2 * rows * cols * 4,
         lambda: ref.ref_gpu_layer_norm(be.stream.cuda_stream, P(x), P(w), P(b), P(y), None, None, rows, cols, 1e-5),
         lambda: be._check(lib.fb_layer_norm_fwd(S(), P(x), P(w), P(b), rows, cols, 1e-5, P(y), None, None, None, None)), rows)
    del h
    for (r2, c2) in ((8192, 1024), (16384, 32000)):
        n = r2 * c2
        with torch.cuda.stream(be.stream):
            xs = torch.randn(n, device=be.device, generator=gen)
            ys = torch.empty(n, device=be.device)
            stats = torch.empty(2 * r2, device=be.device)
        for log in (0, 1):
            ours = lib.fb_log_softmax_fwd if log else lib.fb_softmax_fwd
            pair(f"{'log_' if log else ''}softmax_fwd [{r2},{c2}]", 2 * n * 4,
                 lambda: ref.ref_gpu_softmax(be.stream.cuda_stream, P(xs), P(stats), P(ys), r2, c2, log),
                 lambda: be._check(ours(S(), P(xs), r2, c2, P(ys))), r2)
        del xs, ys
    del x, y, flush
    torch.cuda.empty_cache()
    return out
