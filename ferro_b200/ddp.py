"""Data-parallel training step: shard the batch over ranks, average gradients
over NCCL while the rest of backward runs, update with the fused Adam.

What this replaces in ferro: `ferro_core::ddp::Ddp` (crates/ferro-core/src/ddp.rs:23-180),
which replicates the batch, runs the replicas one after another and averages
gradients by downloading every replica's gradients to the host
(`Ddp::average`, ddp.rs:127-160).  Here there is one process per GPU, rank k
owns batch rows [k*B/N, (k+1)*B/N), and the only exchange is the all-reduce of
flat gradient buckets through the library's own communicator (`fb_ddp_*` in
include/ferro_b200.h: NCCL over NVLink), issued on a side stream as soon as a
bucket's last gradient exists and overlapped with the backward work that
remains.  The mean is "sum, then divide by the replica count" as in
ddp.rs:138-157: the all-reduce sums and the fused Adam multiplies by 1/N on
load (exact for power-of-two world sizes), or `Ddp.average()` divides.

Pieces, host side first:
  shard_rows, plan_buckets, GradientBuckets   pure host logic (no GPU needed)
  PeerWatch      per-step agreement over a key-value store, so that a rank that
                 leaves between steps is noticed before the next collective
  NcclComm       the communicator handle of the C ABI
  Ddp            buckets + communicator + streams: grad_ready(), average(), adam_step()
  DdpMlp         the 2-layer MLP step of the benchmark, written on top of Ddp
The matmuls stay on cuBLAS (torch.matmul), as in ferro; every memory-bound op
goes through libferro_b200.
"""
import ctypes as C
import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib
from .backend import CommError, FerroError


def bias_correction(beta: float, t: int) -> float:
    """1 - beta.powi(t) in f32 with the square-and-multiply order of Rust's powi
    (crates/ferro-core/src/optim.rs:719-721)."""
    import numpy as np
    a, r, b = np.float32(beta), np.float32(1.0), int(t)
    while True:
        if b & 1:
            r = np.float32(r * a)
        b //= 2
        if b == 0:
            break
        a = np.float32(a * a)
    return float(np.float32(1.0) - r)


def shard_rows(rank: int, world: int, batch: int) -> Tuple[int, int]:
    """Rows [lo, hi) of a global batch owned by `rank`.  The batch must divide evenly so
    that the mean of shard-mean gradients is the global-batch mean."""
    if batch % world:
        raise ValueError(f"global batch {batch} does not divide over {world} ranks")
    per = batch // world
    return rank * per, (rank + 1) * per


# --------------------------------------------------------------------------- buckets
NamedShape = Tuple[str, Tuple[int, ...]]
DEFAULT_BUCKET_BYTES = 256 << 20


def plan_buckets(named_shapes: Sequence[NamedShape], cap_bytes: int = DEFAULT_BUCKET_BYTES) -> List[List[NamedShape]]:
    """Groups a parameter list (given in forward order) into exchange buckets.

    Gradients appear in reverse order during backward, so the list is walked backwards and a
    bucket is closed as soon as it holds `cap_bytes` or more: the first bucket is complete
    early and its all-reduce overlaps the rest of backward.  A small parameter never gets a
    collective of its own unless it is the last one left; a parameter larger than the cap
    closes the bucket it lands in."""
    if cap_bytes <= 0:
        raise ValueError("bucket cap must be positive")
    buckets, cur, size = [], [], 0
    for name, shape in reversed(list(named_shapes)):
        cur.append((name, tuple(int(s) for s in shape)))
        size += 4 * math.prod(shape)
        if size >= cap_bytes:
            buckets.append(cur)
            cur, size = [], 0
    if cur:
        buckets.append(cur)
    return buckets


@dataclass
class Bucket:
    flat: torch.Tensor            # one contiguous gradient buffer
    views: List[torch.Tensor]     # per-parameter views into `flat`, parameter shapes
    names: List[str]
    offsets: List[int] = field(default_factory=list)  # element offset of each view in `flat`


def make_buckets(groups: Sequence[Sequence[NamedShape]], device, dtype=torch.float32) -> List[Bucket]:
    """One flat buffer per bucket, each parameter's gradient a view into it.  Offsets are
    rounded up to 4 elements so every view stays 16-byte aligned."""
    buckets = []
    for group in groups:
        offs, total = [], 0
        for _, shape in group:
            offs.append(total)
            total += (math.prod(shape) + 3) // 4 * 4
        flat = torch.zeros(total, device=device, dtype=dtype)
        views = [flat[o:o + math.prod(s)].view(*s) for o, (_, s) in zip(offs, group)]
        buckets.append(Bucket(flat, views, [n for n, _ in group], offs))
    return buckets


class GradientBuckets:
    """Bucket storage plus the bookkeeping of which gradients exist: `ready(name)` returns the
    index of the bucket that this gradient completed, or None.  Device-agnostic host logic."""

    def __init__(self, named_shapes: Sequence[NamedShape], device, cap_bytes: int = DEFAULT_BUCKET_BYTES):
        names = [n for n, _ in named_shapes]
        if len(set(names)) != len(names):
            raise ValueError("duplicate parameter name")
        if not names:
            raise ValueError("at least one parameter is required")  # ddp.rs:31-36
        self.groups = plan_buckets(named_shapes, cap_bytes)
        self.buckets = make_buckets(self.groups, device)
        self.where: Dict[str, Tuple[int, int]] = {}
        for bi, b in enumerate(self.buckets):
            for vi, n in enumerate(b.names):
                self.where[n] = (bi, vi)
        self._pending: List[set] = []
        self.begin()

    def begin(self):
        """Start of a step: no gradient exists yet."""
        self._pending = [set(b.names) for b in self.buckets]

    def grad(self, name: str) -> torch.Tensor:
        bi, vi = self.where[name]
        return self.buckets[bi].views[vi]

    def ready(self, name: str) -> Optional[int]:
        bi, _ = self.where[name]
        pend = self._pending[bi]
        if name not in pend:
            raise RuntimeError(f"gradient of {name} marked ready twice in one step")
        pend.remove(name)
        return bi if not pend else None

    def incomplete(self) -> List[int]:
        return [i for i, p in enumerate(self._pending) if p]


# --------------------------------------------------------------------------- failure detection
class PeerLeft(RuntimeError):
    """Another rank announced that it leaves (or never checked in) before this step's collectives."""


class PeerWatch:
    """Per-step agreement through a key-value store (a torch.distributed Store): before a rank
    enqueues the collectives of step k it publishes "go" under (k, rank) and reads the others'
    entries.  A rank that stops between steps publishes "left" instead, so the ranks that go on
    learn of it on the host, before their next launch, and nothing is enqueued that would wait
    on the device for a peer that is gone.  A rank that publishes nothing within `timeout_s`
    counts as gone too."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "fb_ddp"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def _key(self, step, rank):
        return f"{self.prefix}/{step}/{rank}"

    def leave(self, step: int, reason: str = ""):
        """Announce that this rank will not take part in `step` (the next one)."""
        self.store.set(self._key(step, self.rank), "left:" + reason)

    def agree(self, step: int):
        """Raises PeerLeft unless every rank goes into `step`."""
        import datetime
        self.store.set(self._key(step, self.rank), "go")
        keys = [self._key(step, r) for r in range(self.world) if r != self.rank]
        if not keys:
            return
        try:
            self.store.wait(keys, datetime.timedelta(seconds=self.timeout_s))
        except Exception as e:  # the store raises its own timeout type
            raise PeerLeft(f"step {step}: a peer did not check in within {self.timeout_s} s ({e})") from None
        gone = [r for r in range(self.world) if r != self.rank
                and self.store.get(self._key(step, r)).decode().startswith("left")]
        if gone:
            raise PeerLeft(f"step {step}: rank(s) {gone} left")


# --------------------------------------------------------------------------- communicator
def share_id_over_process_group(group=None, device=None) -> Callable[[Optional[bytes]], bytes]:
    """Carries rank 0's unique id to every rank with a torch.distributed broadcast."""
    import torch.distributed as dist

    def share(raw: Optional[bytes]) -> bytes:
        box = [raw]
        if device is not None:
            dist.broadcast_object_list(box, src=0, group=group, device=device)
        else:
            dist.broadcast_object_list(box, src=0, group=group)
        return box[0]
    return share


def share_id_over_store(store, rank: int, key: str = "fb_ddp/unique_id") -> Callable[[Optional[bytes]], bytes]:
    """Carries rank 0's unique id through a key-value store."""
    def share(raw: Optional[bytes]) -> bytes:
        if rank == 0:
            store.set(key, raw)
            return raw
        return bytes(store.get(key))
    return share


class NcclComm:
    """The communicator handle of the C ABI (fb_ddp_comm): one per process, bound to the GPU
    that is current when it is created."""

    def __init__(self, rank: int, world: int, share_id: Optional[Callable[[Optional[bytes]], bytes]] = None):
        self.lib = _lib.load()
        self.rank, self.world = rank, world
        raw = None
        if world > 1:
            if share_id is None:
                raise ValueError("a world of more than one rank needs a way to share the unique id")
            mine = None
            if rank == 0:
                buf = C.create_string_buffer(_lib.DDP_UNIQUE_ID_BYTES)
                self._check(self.lib.fb_ddp_unique_id(buf))
                mine = buf.raw
            raw = share_id(mine)
            if raw is None or len(raw) != _lib.DDP_UNIQUE_ID_BYTES:
                raise CommError("the shared unique id is missing or has the wrong size")
        h = C.c_void_p()
        self._check(self.lib.fb_ddp_comm_init(raw, rank, world, C.byref(h)))
        self.handle = h

    def _check(self, rc):
        if rc != 0:
            msg = self.lib.fb_last_error().decode()
            raise (CommError if rc == 6 else FerroError)(msg)

    def allreduce_sum(self, ptr: int, n: int, stream: int):
        self._check(self.lib.fb_ddp_allreduce_bucket(self.handle, C.c_void_p(stream), C.c_void_p(ptr), n))

    def allreduce_sum_many(self, ptrs: Sequence[int], lens: Sequence[int], stream: int):
        k = len(ptrs)
        self._check(self.lib.fb_ddp_allreduce_buckets(self.handle, C.c_void_p(stream), (C.c_void_p * max(k, 1))(*ptrs),
                                                      (C.c_uint64 * max(k, 1))(*lens), k))

    def average(self, ptr: int, n: int, stream: int):
        self._check(self.lib.fb_ddp_average_bucket(self.handle, C.c_void_p(stream), C.c_void_p(ptr), n))

    def poll(self):
        """Raises CommError once NCCL has reported a failure on this communicator."""
        self._check(self.lib.fb_ddp_poll(self.handle))

    def abort(self):
        if self.handle:
            h, self.handle = self.handle, None
            self._check(self.lib.fb_ddp_comm_abort(h))

    def close(self):
        if self.handle:
            h, self.handle = self.handle, None
            self._check(self.lib.fb_ddp_comm_destroy(h))


# --------------------------------------------------------------------------- Ddp
class Ddp:
    """Gradient buckets, their exchange and the update that follows, for one rank.

    The caller writes each parameter's gradient into `grad(name)` (a view into a flat bucket),
    calls `grad_ready(name)` on the compute stream once the kernel producing it is enqueued, and
    `release(name)` once backward no longer reads the parameter itself.  A bucket's all-reduce is
    enqueued on the exchange stream the moment its last gradient is ready; `adam_step()` enqueues,
    per bucket and on a third stream, the fused multi-tensor Adam as soon as that bucket's sum has
    arrived and its parameters are released, so the update of an early bucket overlaps the
    exchange of a later one."""

    def __init__(self, backend, named_params: Sequence[Tuple[str, torch.Tensor]], comm: NcclComm,
                 bucket_cap_bytes: int = DEFAULT_BUCKET_BYTES, watch: Optional[PeerWatch] = None,
                 divide: bool = False, timing: bool = False):
        from .backend import DeviceBuffer
        self.be, self.comm, self.watch = backend, comm, watch
        self.world = comm.world
        # divide=True: the exchange leaves the exact mean in the bucket (sum, then `/ world`);
        # divide=False: it leaves the sum and the fused optimizer applies 1/world on load.
        self.divide = divide
        # timing=True keeps a timed event pair around every bucket's all-reduce and marks the end
        # of backward and of the update, per step, for `timings()`; off, only untimed events exist.
        self.timing = timing
        self._tlog: List[dict] = []
        dev = backend.device
        self.names = [n for n, _ in named_params]
        self.params = dict(named_params)
        for n, p in named_params:
            if p.device != dev or p.dtype != torch.float32 or not p.is_contiguous():
                raise ValueError(f"parameter {n} must be a contiguous f32 tensor on {dev}")
        with torch.cuda.stream(backend.stream):
            self.gb = GradientBuckets([(n, tuple(p.shape)) for n, p in named_params], dev, bucket_cap_bytes)
            self.m = {n: torch.zeros_like(p) for n, p in named_params}
            self.v = {n: torch.zeros_like(p) for n, p in named_params}
        wrap = lambda t: DeviceBuffer(t.reshape(-1))
        self.tables = [backend.make_table([(wrap(self.params[n]), wrap(self.m[n]), wrap(self.v[n]), wrap(self.gb.grad(n)))
                                           for n in b.names]) for b in self.gb.buckets]
        self.all_table = backend.make_table([(wrap(self.params[n]), wrap(self.m[n]), wrap(self.v[n]), wrap(self.gb.grad(n)))
                                             for n in self.names])
        self.xchg = torch.cuda.Stream(device=dev, priority=-1)    # collectives: placed ahead of queued compute CTAs
        self.opt = torch.cuda.Stream(device=dev)     # optimizer
        nb = len(self.gb.buckets)
        self.ev_ready = [torch.cuda.Event() for _ in range(nb)]       # bucket's gradients complete (compute stream)
        self.ev_summed = [torch.cuda.Event() for _ in range(nb)]      # bucket's all-reduce done (exchange stream)
        self.ev_released = [torch.cuda.Event() for _ in range(nb)]    # backward no longer reads the bucket's parameters
        self.ev_updated = torch.cuda.Event()                          # last optimizer kernel of the step
        self._unreleased: List[set] = []
        self._exchanged: List[bool] = []
        self.step_no = 0
        self.t = 0
        backend.synchronize()
        self.begin_step()

    # -- per-step protocol ----------------------------------------------------------------
    def grad(self, name: str) -> torch.Tensor:
        return self.gb.grad(name)

    def n_params(self) -> int:
        return sum(p.numel() for p in self.params.values())

    def begin_step(self):
        """Host-side checks before anything of this step is enqueued: the communicator is healthy
        and (with a PeerWatch) every rank goes into the step."""
        self.comm.poll()
        if self.watch is not None and self.world > 1:
            self.watch.agree(self.step_no)
        self.gb.begin()
        if self.timing:
            self._tlog.append({"xchg": []})
        self._unreleased = [set(b.names) for b in self.gb.buckets]
        self._exchanged = [False] * len(self.gb.buckets)

    def wait_for_update(self, stream=None):
        """Make `stream` (default: the backend's) wait for the previous step's parameter update."""
        (stream or self.be.stream).wait_event(self.ev_updated)

    def grad_ready(self, *names: str):
        """The kernels writing these gradients are enqueued on the backend's stream."""
        for name in names:
            bi = self.gb.ready(name)
            if bi is not None:
                self.ev_ready[bi].record(self.be.stream)
                self._exchange(bi)

    def release(self, *names: str):
        """Backward's reads of these parameters are enqueued on the backend's stream."""
        for name in names:
            bi, _ = self.gb.where[name]
            self._unreleased[bi].discard(name)
            if not self._unreleased[bi]:
                self.ev_released[bi].record(self.be.stream)

    def _exchange(self, bi: int):
        b = self.gb.buckets[bi]
        self.xchg.wait_event(self.ev_ready[bi])
        if self.timing:
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(self.xchg)
        (self.comm.average if self.divide else self.comm.allreduce_sum)(
            b.flat.data_ptr(), b.flat.numel(), self.xchg.cuda_stream)
        if self.timing:
            z.record(self.xchg)
            self._tlog[-1]["xchg"].append((bi, a, z))
        self.ev_summed[bi].record(self.xchg)
        self._exchanged[bi] = True
        if self.timing and not self.gb.incomplete():
            # every gradient exists: backward is over on the compute stream
            e = torch.cuda.Event(enable_timing=True)
            e.record(self.be.stream)
            self._tlog[-1]["bwd_done"] = e
            self._tlog[-1]["xchg_done"] = z

    def _finish(self):
        left = self.gb.incomplete()
        if left:
            raise RuntimeError(f"buckets {left} still wait for gradients: "
                               f"{[sorted(self.gb._pending[i]) for i in left]}")
        for bi, names in enumerate(self._unreleased):
            if names:
                self.release(*list(names))

    def average(self):
        """Ddp::average (ddp.rs:127-160) for callers without a fused optimizer (build the Ddp with
        divide=True): after this, on the backend's stream, every `grad(name)` holds the exact mean
        over ranks - the sum of the all-reduce followed by an IEEE divide by the replica count."""
        if not self.divide:
            raise RuntimeError("average() needs Ddp(..., divide=True); otherwise the mean is folded into adam_step()")
        self._finish()
        for bi in range(len(self.gb.buckets)):
            self.be.stream.wait_event(self.ev_summed[bi])
        self.step_no += 1

    def adam_step(self, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, max_grad_norm=None):
        """Adam / AdamW on every parameter with the averaged gradients (optim.rs:695-771): one
        multi-tensor launch per bucket on the optimizer stream, each after its bucket's sum and
        release; 1/world is applied to the gradient on load.  With `max_grad_norm`, the global
        norm of the averaged gradients is reduced on the device first and its clipping factor is
        read by the update (optim.rs:1395-1425); that needs every bucket, so it is one launch
        over the whole list."""
        from .backend import AdamWStep
        self._finish()
        self.t += 1
        hp = self.be._hp(AdamWStep(lr, betas[0], betas[1], bias_correction(betas[0], self.t),
                                   bias_correction(betas[1], self.t), eps, weight_decay))
        lib, scale = self.be.lib, (1.0 if self.divide else 1.0 / self.world)
        o = C.c_void_p(self.opt.cuda_stream)
        if max_grad_norm is None:
            for bi in range(len(self.gb.buckets)):
                self.opt.wait_event(self.ev_summed[bi])
                self.opt.wait_event(self.ev_released[bi])
                dev_table, n, total = self.tables[bi]
                self.be._check(lib.fb_adamw_multi(o, dev_table.data_ptr(), n, total, hp, scale))
        else:
            for bi in range(len(self.gb.buckets)):
                self.opt.wait_event(self.ev_summed[bi])
                self.opt.wait_event(self.ev_released[bi])
            if getattr(self, "_norm_buf", None) is None:
                with torch.cuda.stream(self.opt):
                    self._norm_buf = torch.empty(3, device=self.be.device)  # sum of squares, norm, factor
                    self._norm_ws = torch.empty(int(lib.fb_grad_norm_workspace_bytes()), dtype=torch.uint8,
                                                device=self.be.device)
                self.grad_norm, self.clip_scale = self._norm_buf[1:2], self._norm_buf[2:3]
            dev_table, n, total = self.all_table
            self.be._check(lib.fb_grad_sumsq_multi(o, dev_table.data_ptr(), n, total, scale, self._norm_buf.data_ptr(),
                                                   self._norm_ws.data_ptr(), self._norm_ws.numel()))
            self.be._check(lib.fb_clip_scale(o, self._norm_buf.data_ptr(), float(max_grad_norm),
                                             self.grad_norm.data_ptr(), self.clip_scale.data_ptr()))
            self.be._check(lib.fb_adamw_multi_clipped(o, dev_table.data_ptr(), n, total, hp, scale,
                                                      self.clip_scale.data_ptr()))
        self.ev_updated.record(self.opt)
        if self.timing:
            e = torch.cuda.Event(enable_timing=True)
            e.record(self.opt)
            self._tlog[-1]["updated"] = e
        self.step_no += 1

    def synchronize(self):
        self.xchg.synchronize()
        self.opt.synchronize()
        self.be.synchronize()

    def timings(self, last: Optional[int] = None, clear: bool = True):
        """Averages over the logged steps (timing=True), after a synchronize():
          allreduce_ms[b]  device time of bucket b's all-reduce, from the moment the exchange
                           stream was free to start it (it includes waiting for slower ranks)
          exposed_ms       from the end of backward on the compute stream to the end of the last
                           all-reduce: the part of the exchange no compute covered
          update_tail_ms   from the end of the last all-reduce to the end of the last optimizer kernel"""
        self.synchronize()
        log = [t for t in self._tlog if "updated" in t and "bwd_done" in t]
        if last:
            log = log[-last:]
        if clear:
            self._tlog = []
        if not log:
            return None
        nb = len(self.gb.buckets)
        ar = [0.0] * nb
        exposed = tail = 0.0
        for t in log:
            for bi, a, z in t["xchg"]:
                ar[bi] += a.elapsed_time(z)
            exposed += max(0.0, t["bwd_done"].elapsed_time(t["xchg_done"]))
            tail += max(0.0, t["xchg_done"].elapsed_time(t["updated"]))
        k = float(len(log))
        return {"steps": len(log), "allreduce_ms": [v / k for v in ar], "exposed_ms": exposed / k,
                "update_tail_ms": tail / k, "bucket_bytes": [4 * b.flat.numel() for b in self.gb.buckets],
                "bucket_names": [b.names for b in self.gb.buckets]}


class DdpMlp:
    """The 2-layer MLP data-parallel step: in -> hidden (ReLU) -> out, MSE loss, Adam.

    Linear layers are `x @ W + b` with W stored [in, out] (nn.rs:157-160).  Parameters are
    declared in forward order (W1, b1, W2, b2), so the planner's first bucket holds layer 2,
    whose gradients exist first."""

    def __init__(self, backend, d_in, d_hidden, d_out, rows_per_rank, lr=1e-3, betas=(0.9, 0.999), eps=1e-8,
                 seed=1, comm: Optional[NcclComm] = None, max_grad_norm=None, bucket_cap_bytes=DEFAULT_BUCKET_BYTES,
                 watch: Optional[PeerWatch] = None, params=None, timing: bool = False):
        self.be = backend
        self.comm = comm if comm is not None else NcclComm(0, 1)
        self.world = self.comm.world
        self.d_in, self.d_hidden, self.d_out, self.rows = d_in, d_hidden, d_out, rows_per_rank
        self.lr, self.betas, self.eps = lr, betas, eps
        self.max_grad_norm = max_grad_norm
        dev = backend.device
        torch.backends.cuda.matmul.allow_tf32 = False  # f32 GEMMs, as ferro's sgemm
        with torch.cuda.stream(backend.stream):
            if params is None:
                gen = torch.Generator(device=dev).manual_seed(seed)  # same seed on every rank: replicated parameters
                self.W1 = torch.randn(d_in, d_hidden, device=dev, generator=gen) * math.sqrt(2.0 / d_in)  # He, nn.rs:138-146
                self.b1 = torch.zeros(d_hidden, device=dev)
                self.W2 = torch.randn(d_hidden, d_out, device=dev, generator=gen) * math.sqrt(2.0 / d_hidden)
                self.b2 = torch.zeros(d_out, device=dev)
            else:
                self.W1, self.b1, self.W2, self.b2 = (p.to(dev).contiguous() for p in params)
            self.h = torch.empty(rows_per_rank, d_hidden, device=dev)
            self.yhat = torch.empty(rows_per_rank, d_out, device=dev)
            self.dy = torch.empty(rows_per_rank, d_out, device=dev)
            self.dh = torch.empty(rows_per_rank, d_hidden, device=dev)
            self.loss = torch.empty(1, device=dev)
            ws_bytes = max(int(backend.lib.fb_reduce_workspace_bytes(rows_per_rank * d_out)),
                           int(backend.lib.fb_reduce_dim_workspace_bytes(1, rows_per_rank, d_hidden)),
                           int(backend.lib.fb_reduce_dim_workspace_bytes(1, rows_per_rank, d_out)), 16)
            self.ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        self.params = [self.W1, self.b1, self.W2, self.b2]
        self.ddp = Ddp(backend, [("W1", self.W1), ("b1", self.b1), ("W2", self.W2), ("b2", self.b2)], self.comm,
                       bucket_cap_bytes, watch, timing=timing)
        self.gW1, self.gb1, self.gW2, self.gb2 = (self.ddp.grad(n) for n in ("W1", "b1", "W2", "b2"))
        backend.synchronize()

    def n_params(self):
        return self.ddp.n_params()

    @property
    def done(self):
        return self.ddp.ev_updated

    def step(self, x: torch.Tensor, y: torch.Tensor):
        """One training step on this rank's shard (x [rows, d_in], y [rows, d_out], device tensors).
        Returns the device scalar holding the shard-mean loss."""
        be, lib, ddp = self.be, self.be.lib, self.ddp
        s = be._s()
        R, H, O = self.rows, self.d_hidden, self.d_out
        ws, wsn = self.ws.data_ptr(), self.ws.numel()
        ddp.begin_step()
        with torch.cuda.stream(be.stream):
            ddp.wait_for_update()  # the previous update of the parameters has finished
            # forward
            torch.matmul(x, self.W1, out=self.h)
            be._check(lib.fb_bias_act_fwd(s, self.h.data_ptr(), self.b1.data_ptr(), 1, R, H, self.h.data_ptr()))
            torch.matmul(self.h, self.W2, out=self.yhat)
            be._check(lib.fb_bias_act_fwd(s, self.yhat.data_ptr(), self.b2.data_ptr(), 0, R, O, self.yhat.data_ptr()))
            ddp.release("b1", "b2")
            # loss and its gradient in one pass
            be._check(lib.fb_mse_fwd_bwd(s, self.yhat.data_ptr(), y.data_ptr(), R * O, 1.0, self.loss.data_ptr(),
                                         self.dy.data_ptr(), ws, wsn))
            # backward, layer 2: db2 = column sums of dy, dW2 = h^T dy
            be._check(lib.fb_bias_act_bwd(s, self.dy.data_ptr(), None, None, 0, R, O, None, self.gb2.data_ptr(), ws, wsn))
            ddp.grad_ready("b2")
            torch.matmul(self.h.t(), self.dy, out=self.gW2)
            ddp.grad_ready("W2")
            # backward, layer 1 (overlaps the exchange of layer 2's bucket)
            torch.matmul(self.dy, self.W2.t(), out=self.dh)
            ddp.release("W2")
            # relu mask from the saved activation (h > 0 exactly where the pre-activation was), dx in place
            be._check(lib.fb_bias_act_bwd(s, self.dh.data_ptr(), self.h.data_ptr(), None, 1, R, H, self.dh.data_ptr(),
                                          self.gb1.data_ptr(), ws, wsn))
            ddp.grad_ready("b1")
            torch.matmul(x.t(), self.dh, out=self.gW1)
            ddp.grad_ready("W1")
            ddp.release("W1")
        ddp.adam_step(self.lr, self.betas, self.eps, 0.0, self.max_grad_norm)
        return self.loss

    @property
    def grad_norm(self):
        return getattr(self.ddp, "grad_norm", None)

    @property
    def clip_scale(self):
        return getattr(self.ddp, "clip_scale", None)

    def synchronize(self):
        self.ddp.synchronize()
