"""Shared pieces of the benchmark scripts next to this file: the measured roofline
denominators, the clock sampler, CUDA-event timing loops and seeded inputs."""
import json
import os
import subprocess
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
NOMINAL_HBM_GBS = 8000.0
NVLINK_NOMINAL_GBS = 900.0     # per direction per GPU
NVLINK_MEASURED_GBS = 770.0    # peer copy per direction measured on this pool's B200s


def peaks():
    """(HBM GB/s, "measured" | "fallback"): the STREAM-style copy figure written by the driver, else
    the pool's earlier measurement."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi in the background; `window`
    summarises the samples that fell between two host times."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index, period_ms=50):
        self.index, self.period_ms, self.proc, self.lines = index, period_ms, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def window(self, t0=None, t1=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        sm, mx, pw, reasons = [], [], [], set()
        for ts, ln in list(self.lines):
            if t0 is not None and not (t0 <= ts <= t1):
                continue
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                pw.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()


class Flusher:
    """A buffer of twice the L2 size rewritten between timed iterations, so inputs that would fit
    in L2 still come from HBM."""

    def __init__(self, be):
        import torch
        self.be = be
        with torch.cuda.stream(be.stream):
            self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=be.device)

    def __call__(self):
        import torch
        with torch.cuda.stream(self.be.stream):
            self.buf.zero_()


def time_call(be, fn, flush=None, min_s=0.6, min_iters=20, warmup=3):
    """Median / min CUDA-event time of `fn` (one library call) on the backend's stream, repeated
    until both `min_iters` and `min_s` seconds have passed so that the clock sampler sees the
    loop.  Returns (median_ms, min_ms, iters, launches_per_call, host_t0, host_t1)."""
    import torch
    for _ in range(warmup):
        fn()
    be.synchronize()
    times = []
    launches0 = be.lib.fb_launch_count()
    t0 = time.time()
    while True:
        evs = []
        for _ in range(10):
            if flush is not None:
                flush()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(be.stream)
            fn()
            b.record(be.stream)
            evs.append((a, b))
        be.synchronize()
        times += [a.elapsed_time(b) for a, b in evs]
        if len(times) >= min_iters and time.time() - t0 >= min_s:
            break
    t1 = time.time()
    launches = (be.lib.fb_launch_count() - launches0) // len(times)
    times.sort()
    return times[len(times) // 2], times[0], len(times), int(launches), t0, t1


def time_rotating(be, fns, min_s=0.6, min_iters=20):
    """Per-call average over len(fns) calls on distinct buffer sets inside one event pair (the
    sets together exceed L2): the launch gap of a 10-40 us kernel is no longer in the figure."""
    import torch
    for fn in fns:
        fn()
    be.synchronize()
    times = []
    t0 = time.time()
    while True:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(be.stream)
        for fn in fns:
            fn()
        b.record(be.stream)
        be.synchronize()
        times.append(a.elapsed_time(b) / len(fns))
        if len(times) >= min_iters and time.time() - t0 >= min_s:
            break
    t1 = time.time()
    times.sort()
    return times[len(times) // 2], times[0], len(times), t0, t1


class Staging:
    """Seeded host draws to the device through one reusable pinned buffer: the generator fills a
    chunk (ferro's Rng draws on the host), the chunk is copied up, the next chunk continues the
    same stream of draws."""

    def __init__(self, be, elems=1 << 26):
        import torch
        self.be, self.elems = be, elems
        self.pin = torch.empty(elems, dtype=torch.float32).pin_memory()

    def _pump(self, total, fill, device_flat):
        import torch
        done = 0
        while done < total:
            m = min(self.elems, total - done)
            fill(self.pin[:m], m)
            with torch.cuda.stream(self.be.stream):
                device_flat[done:done + m].copy_(self.pin[:m], non_blocking=True)
            self.be.stream.synchronize()
            done += m

    def normal(self, rng, n, scale=1.0, shift=0.0):
        import torch
        with torch.cuda.stream(self.be.stream):
            out = torch.empty(n, device=self.be.device)
        self._pump(n, lambda buf, m: rng.fill_normal((m,), scale, shift, out=buf), out)
        return out

    def uniform(self, rng, n, scale=1.0, shift=0.0):
        import torch
        with torch.cuda.stream(self.be.stream):
            out = torch.empty(n, device=self.be.device)
        self._pump(n, lambda buf, m: rng.fill_uniform((m,), scale, shift, out=buf), out)
        return out

    def rowscaled_normal(self, rng, rows, cols, lo=0.5, span=3.5):
        import torch
        with torch.cuda.stream(self.be.stream):
            out = torch.empty(rows * cols, device=self.be.device)
        per = max(1, self.elems // cols)
        r0 = 0
        while r0 < rows:
            m = min(per, rows - r0)
            rng.fill_rowscaled_normal(m, cols, lo, span, out=self.pin[:m * cols])
            with torch.cuda.stream(self.be.stream):
                out[r0 * cols:(r0 + m) * cols].copy_(self.pin[:m * cols], non_blocking=True)
            self.be.stream.synchronize()
            r0 += m
        return out

    def index(self, rng, n, classes):
        import torch
        host = torch.empty(n, dtype=torch.int64)
        rng.fill_index(n, classes, out=host)
        with torch.cuda.stream(self.be.stream):
            return host.to(self.be.device)
