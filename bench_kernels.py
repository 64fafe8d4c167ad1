"""Per-kernel HBM throughput at the shapes of the published configurations.

    python bench_kernels.py [--iters 20] [--only SUBSTR] [--json PATH] [--small]

Every case is one library call (one to three kernel launches) timed with CUDA
events on the backend's stream, after 3 warm-up calls, with a buffer larger
than L2 rewritten between iterations so the inputs come from HBM even when
they would fit in L2.  GB/s = algorithmic bytes / median time; the byte
counts are the ones stated next to each kernel in ferro_b200/csrc/*.cu.
Output: one JSON object per case and a markdown table.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from ferro_b200.backend import (AdamWStep, BinaryKind, ChainStep, CudaBackend, DeviceBuffer, T, UnaryKind,
                      View)

NOMINAL_GBS = 8000.0


def measured_peak():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class Bench:
    def __init__(self, iters):
        self.be = CudaBackend(0)
        self.iters = iters
        self.rows = []
        self.peak, self.peak_src = measured_peak()
        with torch.cuda.stream(self.be.stream):
            self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.be.device)  # 2x L2

    def randn(self, *shape, scale=1.0):
        with torch.cuda.stream(self.be.stream):
            return DeviceBuffer((torch.randn(*shape, device=self.be.device) * scale).reshape(-1))

    def rand(self, *shape, lo=0.0, hi=1.0):
        with torch.cuda.stream(self.be.stream):
            return DeviceBuffer((torch.rand(*shape, device=self.be.device) * (hi - lo) + lo).reshape(-1))

    def empty(self, n, dtype=torch.float32):
        return self.be._alloc(n, dtype)

    def run(self, name, nbytes, fn, units=None, unit_name=None):
        be = self.be
        for _ in range(3):
            fn()
        be.synchronize()
        times = []
        launches0 = be.lib.fb_launch_count()
        for _ in range(self.iters):
            with torch.cuda.stream(be.stream):
                self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(be.stream)
            fn()
            b.record(be.stream)
            be.synchronize()
            times.append(a.elapsed_time(b))
        launches = (be.lib.fb_launch_count() - launches0) // self.iters
        times.sort()
        med = times[len(times) // 2]
        gbs = nbytes / (med * 1e-3) / 1e9
        row = {"kernel": name, "bytes": int(nbytes), "us": med * 1e3, "us_min": times[0] * 1e3, "gbs": gbs,
               "frac_measured": gbs / self.peak, "frac_nominal": gbs / NOMINAL_GBS, "launches": int(launches)}
        if units:
            row[unit_name] = units / (med * 1e-3)
        self.rows.append(row)
        print(json.dumps(row), flush=True)


def _run_rotating(self, name, nbytes, fns):
    """Time len(fns) calls over distinct buffer sets inside one event pair (per-call average)."""
    be = self.be
    for fn in fns:
        fn()
    be.synchronize()
    times = []
    launches0 = be.lib.fb_launch_count()
    for _ in range(self.iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(be.stream)
        for fn in fns:
            fn()
        b.record(be.stream)
        be.synchronize()
        times.append(a.elapsed_time(b) / len(fns))
    launches = (be.lib.fb_launch_count() - launches0) // (self.iters * len(fns))
    times.sort()
    med = times[len(times) // 2]
    gbs = nbytes / (med * 1e-3) / 1e9
    row = {"kernel": name, "bytes": int(nbytes), "us": med * 1e3, "us_min": times[0] * 1e3, "gbs": gbs,
           "frac_measured": gbs / self.peak, "frac_nominal": gbs / NOMINAL_GBS, "launches": int(launches)}
    self.rows.append(row)
    print(json.dumps(row), flush=True)


Bench.run_rotating = _run_rotating


def cases(B, only, small=False, widths=None):
    be = B.be
    lib, S = be.lib, be._s

    def want(name):
        return only is None or only in name

    # ---- C1: softmax(relu(x + b) * s) fwd / bwd, [8192, 1024]
    if want("c1"):
        r, c = 8192, 1024
        x, bias, g = B.randn(r, c), B.randn(c, scale=0.1), B.randn(r, c)
        y, dx, db = B.empty(r * c), B.empty(r * c), B.empty(c)
        ws = B.empty(int(lib.fb_softmax_fused_bwd_workspace_bytes(r, c)) // 4 + 4)
        B.run("c1_fused_fwd softmax(relu(x+b)*s) [8192,1024]", 2 * r * c * 4,
              lambda: be._check(lib.fb_bias_act_scale_softmax_fwd(S(), x.ptr, bias.ptr, 1, 0.125, r, c, y.ptr)),
              r, "rows_per_s")
        B.run("c1_fused_bwd dx,db [8192,1024]", 4 * r * c * 4,
              lambda: be._check(lib.fb_bias_act_scale_softmax_bwd(S(), g.ptr, y.ptr, x.ptr, bias.ptr, 1, 0.125, r, c,
                                                                  dx.ptr, db.ptr, ws.ptr, len(ws) * 4)), r, "rows_per_s")
        B.run("softmax_fwd [8192,1024]", 2 * r * c * 4, lambda: be._check(lib.fb_softmax_fwd(S(), x.ptr, r, c, y.ptr)), r, "rows_per_s")
        B.run("softmax_bwd [8192,1024]", 3 * r * c * 4, lambda: be._check(lib.fb_softmax_bwd(S(), g.ptr, y.ptr, r, c, dx.ptr)), r, "rows_per_s")
        del x, y, dx, g
        # The same four calls back to back over 8 rotating buffer sets (8 x 33.5 MB per array,
        # more than L2 in total): the launch gap of a 10-40 us kernel is no longer in the figure.
        K = 8
        xs, gs = [B.randn(r, c) for _ in range(K)], [B.randn(r, c) for _ in range(K)]
        ys, dxs = [B.empty(r * c) for _ in range(K)], [B.empty(r * c) for _ in range(K)]
        B.run_rotating("c1_fused_fwd, 8 rotating sets [8192,1024]", 2 * r * c * 4,
                       [(lambda i=i: be._check(lib.fb_bias_act_scale_softmax_fwd(S(), xs[i].ptr, bias.ptr, 1, 0.125, r, c, ys[i].ptr)))
                        for i in range(K)])
        B.run_rotating("c1_fused_bwd, 8 rotating sets [8192,1024]", 4 * r * c * 4,
                       [(lambda i=i: be._check(lib.fb_bias_act_scale_softmax_bwd(S(), gs[i].ptr, ys[i].ptr, xs[i].ptr, bias.ptr, 1, 0.125,
                                                                                  r, c, dxs[i].ptr, db.ptr, ws.ptr, len(ws) * 4)))
                        for i in range(K)])
        B.run_rotating("softmax_fwd, 8 rotating sets [8192,1024]", 2 * r * c * 4,
                       [(lambda i=i: be._check(lib.fb_softmax_fwd(S(), xs[i].ptr, r, c, ys[i].ptr))) for i in range(K)])
        B.run_rotating("softmax_bwd, 8 rotating sets [8192,1024]", 3 * r * c * 4,
                       [(lambda i=i: be._check(lib.fb_softmax_bwd(S(), gs[i].ptr, ys[i].ptr, r, c, dxs[i].ptr))) for i in range(K)])
        del xs, gs, ys, dxs, bias, db, ws

    # ---- C2: LayerNorm [32768, 4096]
    if want("c2"):
        r, c = (4096 if small else 32768), 4096
        x, g, w, bb = B.randn(r, c), B.randn(r, c), B.randn(c), B.randn(c)
        y, dx, h = B.empty(r * c), B.empty(r * c), B.empty(r * c)
        mu, rs, sd, dw, db = B.empty(r), B.empty(r), B.empty(r), B.empty(c), B.empty(c)
        ws = B.empty(int(lib.fb_layer_norm_bwd_workspace_bytes(r, c)) // 4 + 4)
        B.run("c2_ln_fwd (y,mean,rstd) [32768,4096]", 2 * r * c * 4,
              lambda: be._check(lib.fb_layer_norm_fwd(S(), x.ptr, w.ptr, bb.ptr, r, c, 1e-5, y.ptr, None, None, mu.ptr, rs.ptr)), r, "rows_per_s")
        B.run("c2_ln_bwd (x,mean,rstd)->dx,dg,db [32768,4096]", 3 * r * c * 4,
              lambda: be._check(lib.fb_layer_norm_bwd(S(), g.ptr, None, None, x.ptr, mu.ptr, rs.ptr, w.ptr, r, c, dx.ptr, dw.ptr, db.ptr, ws.ptr, len(ws) * 4)), r, "rows_per_s")
        B.run("ln_fwd ferro form (y,h,stds) [32768,4096]", 3 * r * c * 4,
              lambda: be._check(lib.fb_layer_norm_fwd(S(), x.ptr, w.ptr, bb.ptr, r, c, 1e-5, y.ptr, h.ptr, sd.ptr, None, None)), r, "rows_per_s")
        B.run("ln_bwd ferro form (h,stds) [32768,4096]", 3 * r * c * 4,
              lambda: be._check(lib.fb_layer_norm_bwd(S(), g.ptr, h.ptr, sd.ptr, None, None, None, w.ptr, r, c, dx.ptr, dw.ptr, db.ptr, ws.ptr, len(ws) * 4)), r, "rows_per_s")
        B.run("residual_ln_fwd x+r -> (y,mean,rstd) [32768,4096]", 3 * r * c * 4,
              lambda: be._check(lib.fb_residual_layer_norm_fwd(S(), x.ptr, g.ptr, w.ptr, bb.ptr, r, c, 1e-5, y.ptr, None, None,
                                                               mu.ptr, rs.ptr, None)), r, "rows_per_s")
        B.run("rms_norm_fwd (y,rstd) [32768,4096]", 2 * r * c * 4,
              lambda: be._check(lib.fb_rms_norm_fwd(S(), x.ptr, w.ptr, r, c, 1e-5, y.ptr, rs.ptr)), r, "rows_per_s")
        B.run("rms_norm_bwd (x,rstd)->dx,dg [32768,4096]", 3 * r * c * 4,
              lambda: be._check(lib.fb_rms_norm_bwd(S(), g.ptr, x.ptr, rs.ptr, w.ptr, r, c, dx.ptr, dw.ptr, ws.ptr, len(ws) * 4)), r, "rows_per_s")
        del x, g, w, bb, y, dx, h, mu, rs, sd, dw, db, ws

    # ---- other row widths (not in the default table: run with --only widths), 512 MB per array
    if only is not None and want("widths"):
        for c in widths or (32, 64, 128, 256, 768, 1024, 1536, 2048, 3072, 5120, 8192, 16384, 32768, 65536, 1000, 50000):
            r = (1 << (24 if small else 27)) // c
            x, g, w, bb = B.randn(r, c), B.randn(r, c), B.randn(c), B.randn(c)
            y, dx = B.empty(r * c), B.empty(r * c)
            mu, rs, dw, db = B.empty(r), B.empty(r), B.empty(c), B.empty(c)
            ws = B.empty(int(lib.fb_layer_norm_bwd_workspace_bytes(r, c)) // 4 + 4)
            B.run(f"widths ln_fwd [{r},{c}]", 2 * r * c * 4,
                  lambda: be._check(lib.fb_layer_norm_fwd(S(), x.ptr, w.ptr, bb.ptr, r, c, 1e-5, y.ptr, None, None, mu.ptr, rs.ptr)))
            B.run(f"widths ln_bwd [{r},{c}]", 3 * r * c * 4,
                  lambda: be._check(lib.fb_layer_norm_bwd(S(), g.ptr, None, None, x.ptr, mu.ptr, rs.ptr, w.ptr, r, c, dx.ptr, dw.ptr, db.ptr, ws.ptr, len(ws) * 4)))
            B.run(f"widths softmax_fwd [{r},{c}]", 2 * r * c * 4, lambda: be._check(lib.fb_softmax_fwd(S(), x.ptr, r, c, y.ptr)))
            B.run(f"widths softmax_bwd [{r},{c}]", 3 * r * c * 4, lambda: be._check(lib.fb_softmax_bwd(S(), g.ptr, y.ptr, r, c, dx.ptr)))
            del x, g, w, bb, y, dx, mu, rs, dw, db, ws

    # ---- C3: cross entropy [16384, 32000]
    if want("c3"):
        r, c = (2048 if small else 16384), 32000
        x = B.randn(r, c, scale=2.0)
        with torch.cuda.stream(be.stream):
            t = DeviceBuffer(torch.randint(0, c, (r,), device=be.device, dtype=torch.int64))
        loss, rmax, rlse, am, dl = B.empty(1), B.empty(r), B.empty(r), B.empty(r, torch.int64), B.empty(r * c)
        ws = B.empty(int(lib.fb_nll_workspace_bytes(r)) // 4 + 4)
        B.run("c3_nll_fwd (+argmax) [16384,32000]", r * c * 4,
              lambda: be._check(lib.fb_log_softmax_nll_fwd(S(), x.ptr, t.ptr, r, c, loss.ptr, rmax.ptr, rlse.ptr, am.ptr, None, ws.ptr, len(ws) * 4)), r, "rows_per_s")
        B.run("c3_nll_bwd dlogits [16384,32000]", 2 * r * c * 4,
              lambda: be._check(lib.fb_log_softmax_nll_bwd(S(), x.ptr, t.ptr, rmax.ptr, rlse.ptr, 1.0, r, c, dl.ptr)), r, "rows_per_s")
        B.run("log_softmax_fwd [16384,32000]", 2 * r * c * 4, lambda: be._check(lib.fb_log_softmax_fwd(S(), x.ptr, r, c, dl.ptr)), r, "rows_per_s")
        del x, t, loss, rmax, rlse, am, dl, ws

    # ---- C4: chain over a [16384,16384] and a^T, then axis reductions of [256,512,2048]
    if want("c4"):
        n = 8192 if small else 16384
        a, col = B.rand(n, n, lo=-4, hi=4), B.rand(n, 1, lo=-4, hi=4)
        z = B.empty(n * n)
        U, Bi, St = UnaryKind, BinaryKind, ChainStep
        prog = [St.Load(0), St.Unary(U.Abs), St.Unary(U.Neg), St.Unary(U.Exp),
                St.Load(1, dst=T), St.Unary(U.Abs, dst=T), St.Binary(Bi.Add, imm=1.0, dst=T), St.Unary(U.Sqrt, dst=T),
                St.Binary(Bi.Mul), St.Unary(U.Tanh),
                St.Load(2, dst=T), St.Unary(U.Powf(1.5), dst=T), St.Binary(Bi.Add), St.Unary(U.Clamp(-1.0, 1.0))]
        ops = [View(a, (n, 1)), View(col, (1, 0)), View(a, (1, n))]
        B.run("c4_chain clamp(tanh(exp(-|a|)*sqrt(|b|+1))+powf(a^T,1.5)) [16384,16384]", 2 * n * n * 4,
              lambda: be.chain_dev(prog, ops, (n, n)))
        lib.fb_chain_catalogue(0)  # the same chain through the interpreter, as a chain outside the manifest would run
        B.run("c4_chain, interpreted [16384,16384]", 2 * n * n * 4, lambda: be.chain_dev(prog, ops, (n, n)))
        lib.fb_chain_catalogue(1)
        B.run("materialize a^T [16384,16384]", 2 * n * n * 4, lambda: be.materialize_dev(a, (n, n), (1, n), 0))
        shape = (n * n // (512 * 2048), 512, 2048)
        for dim in range(3):
            o = 1
            for s_ in shape[:dim]:
                o *= s_
            i = 1
            for s_ in shape[dim + 1:]:
                i *= s_
            red = shape[dim]
            out, idx = B.empty(o * i), B.empty(o * i, torch.int64)
            ws = B.empty(int(lib.fb_reduce_dim_workspace_bytes(o, red, i)) // 4 + 4)
            B.run(f"c4_sum_dim{dim} [256,512,2048]", n * n * 4 + o * i * 4,
                  lambda: be._check(lib.fb_sum_dim(S(), a.ptr, o, red, i, out.ptr, ws.ptr, len(ws) * 4)))
            B.run(f"c4_mean_dim{dim} [256,512,2048]", n * n * 4 + o * i * 4,
                  lambda: be._check(lib.fb_mean_dim(S(), a.ptr, o, red, i, out.ptr, ws.ptr, len(ws) * 4)))
            B.run(f"c4_max_dim{dim} (+argmax) [256,512,2048]", n * n * 4 + o * i * 12,
                  lambda: be._check(lib.fb_max_dim(S(), a.ptr, o, red, i, out.ptr, idx.ptr, ws.ptr, len(ws) * 4)))
        ws = B.empty(int(lib.fb_reduce_workspace_bytes(n * n)) // 4 + 4)
        out = B.empty(1)
        B.run("reduce sum 2^28", n * n * 4, lambda: be._check(lib.fb_reduce(S(), 0, a.ptr, n * n, out.ptr, ws.ptr, len(ws) * 4)))
        B.run("unary relu 2^28", 2 * n * n * 4, lambda: be._check(lib.fb_unary(S(), 1, 0.0, 0.0, a.ptr, z.ptr, n * n)))
        B.run("unary exp 2^28", 2 * n * n * 4, lambda: be._check(lib.fb_unary(S(), 2, 0.0, 0.0, a.ptr, z.ptr, n * n)))
        B.run("unary tanh 2^28", 2 * n * n * 4, lambda: be._check(lib.fb_unary(S(), 4, 0.0, 0.0, a.ptr, z.ptr, n * n)))
        b2 = B.randn(n * n)
        B.run("binary add 2^28", 3 * n * n * 4, lambda: be._check(lib.fb_binary(S(), 0, 0.0, 0.0, a.ptr, b2.ptr, z.ptr, n * n)))
        B.run("binary_bc [16384,16384]*[16384,1]", 2 * n * n * 4, lambda: be.binary_bc_dev(Bi.Mul, a, (n, n), col, (n, 1), (n, n)))
        B.run("copy 2^28", 2 * n * n * 4, lambda: be._check(lib.fb_copy(S(), z.ptr, a.ptr, n * n)))
        del a, col, z, b2, out, ws

    # ---- C5: optimizer over the MLP's 134 238 208 parameters, and the MLP glue at N = 1
    if want("c5"):
        sizes = [4096 * 16384, 16384, 16384 * 4096, 4096]
        if small:
            sizes = [v // 8 for v in sizes]
        total = sum(sizes)
        bufs = [[B.randn(n) for n in sizes] for _ in range(4)]
        with torch.cuda.stream(be.stream):
            for v in bufs[2]:
                v.t.abs_()
        table = be.make_table(list(zip(*bufs)))
        hp = AdamWStep(1e-3, 0.9, 0.999, 0.1, 0.001, 1e-8, 0.0)
        B.run("c5_adam_multi 134238208 params (4 tensors)", 28 * total, lambda: be.adamw_multi_dev(table, hp, 1.0))
        B.run("adam_single 67108864", 28 * sizes[0], lambda: be.adamw_step_dev(bufs[0][0], bufs[1][0], bufs[2][0], bufs[3][0], hp))
        B.run("sgd_momentum_single 67108864", 20 * sizes[0], lambda: be.sgd_step_dev(bufs[0][0], bufs[1][0], bufs[3][0], 0.01, 0.9, False))
        del bufs, table
        r, c = (4096 if small else 65536), 16384
        x, g, bias = B.randn(r, c), B.randn(r, c), B.randn(c)
        out, db = B.empty(r * c), B.empty(c)
        ws = B.empty(int(lib.fb_reduce_dim_workspace_bytes(1, r, c)) // 4 + 4)
        B.run("c5_bias_relu_fwd [65536,16384]", 2 * r * c * 4, lambda: be._check(lib.fb_bias_act_fwd(S(), x.ptr, bias.ptr, 1, r, c, out.ptr)))
        B.run("c5_bias_relu_bwd dx,db [65536,16384]", 3 * r * c * 4,
              lambda: be._check(lib.fb_bias_act_bwd(S(), g.ptr, x.ptr, bias.ptr, 1, r, c, out.ptr, db.ptr, ws.ptr, len(ws) * 4)))
        del x, g, out
        r, c = (8192 if small else 65536), 4096
        p, t = B.randn(r, c), B.randn(r, c)
        dp, loss = B.empty(r * c), B.empty(1)
        ws = B.empty(int(lib.fb_reduce_workspace_bytes(r * c)) // 4 + 4)
        B.run("c5_mse_fwd_bwd [65536,4096]", 3 * r * c * 4,
              lambda: be._check(lib.fb_mse_fwd_bwd(S(), p.ptr, t.ptr, r * c, 1.0, loss.ptr, dp.ptr, ws.ptr, len(ws) * 4)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default=None)
    ap.add_argument("--json", default=None)
    ap.add_argument("--small", action="store_true", help="1/8-size cases (still larger than L2) for profiler captures")
    ap.add_argument("--widths", default=None, help="comma-separated row widths for --only widths")
    args = ap.parse_args()
    B = Bench(args.iters)
    cases(B, args.only, args.small, [int(v) for v in args.widths.split(",")] if args.widths else None)
    print(f"\n| kernel | bytes | us (median) | GB/s | % of {B.peak:.0f} ({B.peak_src}) | % of 8000 | launches |")
    print("|---|---|---|---|---|---|---|")
    for r in B.rows:
        print(f"| {r['kernel']} | {r['bytes']} | {r['us']:.1f} | {r['gbs']:.0f} | {100 * r['frac_measured']:.1f} | {100 * r['frac_nominal']:.1f} | {r['launches']} |")
    if args.json:
        with open(args.json, "w") as f:
            json.dump(B.rows, f, indent=1)


if __name__ == "__main__":
    sys.exit(main())
