"""Data-parallel training step: shard the batch over ranks, average gradients
over NCCL while the rest of backward runs, update with the fused Adam.

What this replaces in ferro: `ferro_core::ddp::Ddp` (crates/ferro-core/src/ddp.rs:23-180),
which replicates the batch, runs the replicas one after another and averages
gradients by downloading every replica's gradients to the host
(`Ddp::average`, ddp.rs:127-160).  Here there is one process per GPU
(torch.distributed supplies the NCCL plumbing), rank k owns batch rows
[k*B/N, (k+1)*B/N), and the only exchange is the all-reduce of the flat
gradient buckets, issued on a side stream as soon as a bucket's last gradient
exists and overlapped with the backward work that remains.  The mean is
"sum, then divide by the replica count" exactly as ddp.rs:138-157: the
all-reduce sums and the fused Adam multiplies by 1/N on load (exact for the
power-of-two world sizes used here).

The host-side pieces (row sharding, bucket layout, the averaging call) do not
need a GPU and run over gloo on CPU tensors in the tests.  The matmuls stay on
cuBLAS (torch.matmul), as in ferro; every memory-bound op goes through
libferro_b200.
"""
import math
from dataclasses import dataclass
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


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


@dataclass
class Bucket:
    flat: torch.Tensor            # one contiguous gradient buffer
    views: List[torch.Tensor]     # per-parameter views into `flat`, parameter shapes
    names: List[str]


def make_buckets(named_shapes: Sequence[Sequence[Tuple[str, Tuple[int, ...]]]], device, dtype=torch.float32):
    """One flat buffer per bucket, each parameter's gradient a view into it.  Offsets are
    rounded up to 4 elements so every view stays 16-byte aligned."""
    buckets = []
    for group in named_shapes:
        offs, total = [], 0
        for _, shape in group:
            offs.append(total)
            total += (math.prod(shape) + 3) // 4 * 4
        flat = torch.zeros(total, device=device, dtype=dtype)
        views = [flat[o:o + math.prod(s)].view(*s) for o, (_, s) in zip(offs, group)]
        buckets.append(Bucket(flat, views, [n for n, _ in group]))
    return buckets


def allreduce_sum_(bucket: Bucket, group=None, async_op=False):
    """The exchange step: in-place sum over ranks of one flat bucket."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return None
    return dist.all_reduce(bucket.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)


def average_(bucket: Bucket, group=None):
    """Ddp::average (ddp.rs:127-160) for one bucket: sum over replicas, then divide by the
    replica count.  Used where no fused optimizer follows (tests, CPU)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    allreduce_sum_(bucket, group)
    if world > 1:
        bucket.flat.div_(float(world))
    return bucket


class DdpMlp:
    """The 2-layer MLP data-parallel step: in -> hidden (ReLU) -> out, MSE loss, Adam.

    Linear layers are `x @ W + b` with W stored [in, out] (nn.rs:157-160).  Buckets follow
    the order gradients become available in backward: {W2, b2} first, {W1, b1} second."""

    def __init__(self, backend, d_in, d_hidden, d_out, rows_per_rank, lr=1e-3, betas=(0.9, 0.999), eps=1e-8,
                 seed=1, group=None, max_grad_norm=None):
        from .backend import DeviceBuffer
        self.be, self.group = backend, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.d_in, self.d_hidden, self.d_out, self.rows = d_in, d_hidden, d_out, rows_per_rank
        self.lr, self.betas, self.eps, self.t = lr, betas, eps, 0
        # Optional global-norm clipping of the averaged gradients (optim.rs:1395-1425), computed on the
        # device after the last all-reduce: norm and factor of the latest step stay in these buffers.
        self.max_grad_norm, self.grad_norm, self.clip_scale = max_grad_norm, None, None
        dev = backend.device
        torch.backends.cuda.matmul.allow_tf32 = False  # f32 GEMMs, as ferro's sgemm
        gen = torch.Generator(device=dev).manual_seed(seed)  # same seed on every rank: replicated parameters
        with torch.cuda.stream(backend.stream):
            self.W1 = torch.randn(d_in, d_hidden, device=dev, generator=gen) * math.sqrt(2.0 / d_in)  # He, nn.rs:138-146
            self.b1 = torch.zeros(d_hidden, device=dev)
            self.W2 = torch.randn(d_hidden, d_out, device=dev, generator=gen) * math.sqrt(2.0 / d_hidden)
            self.b2 = torch.zeros(d_out, device=dev)
            self.params = [self.W1, self.b1, self.W2, self.b2]
            self.m = [torch.zeros_like(p) for p in self.params]
            self.v = [torch.zeros_like(p) for p in self.params]
            self.buckets = make_buckets([[("W2", (d_hidden, d_out)), ("b2", (d_out,))],
                                         [("W1", (d_in, d_hidden)), ("b1", (d_hidden,))]], dev)
            self.gW2, self.gb2 = self.buckets[0].views
            self.gW1, self.gb1 = self.buckets[1].views
            self.h = torch.empty(rows_per_rank, d_hidden, device=dev)
            self.yhat = torch.empty(rows_per_rank, d_out, device=dev)
            self.dy = torch.empty(rows_per_rank, d_out, device=dev)
            self.dh = torch.empty(rows_per_rank, d_hidden, device=dev)
            self.loss = torch.empty(1, device=dev)
            ws_bytes = max(int(backend.lib.fb_reduce_workspace_bytes(rows_per_rank * d_out)),
                           int(backend.lib.fb_reduce_dim_workspace_bytes(1, rows_per_rank, d_hidden)),
                           int(backend.lib.fb_reduce_dim_workspace_bytes(1, rows_per_rank, d_out)), 16)
            self.ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        wrap = lambda t: DeviceBuffer(t.reshape(-1))
        grads = [self.gW1, self.gb1, self.gW2, self.gb2]
        self.table = backend.make_table([(wrap(p), wrap(m), wrap(v), wrap(g))
                                         for p, m, v, g in zip(self.params, self.m, self.v, grads)])
        self.comm = torch.cuda.Stream(device=dev)
        self.ready = [torch.cuda.Event(), torch.cuda.Event()]
        self.done = torch.cuda.Event()
        backend.synchronize()

    def n_params(self):
        return sum(p.numel() for p in self.params)

    def step(self, x: torch.Tensor, y: torch.Tensor):
        """One training step on this rank's shard (x [rows, d_in], y [rows, d_out], device tensors).
        Returns the device scalar holding the shard-mean loss."""
        be, lib = self.be, self.be.lib
        s = be._s()
        R, H, O = self.rows, self.d_hidden, self.d_out
        ws, wsn = self.ws.data_ptr(), self.ws.numel()
        with torch.cuda.stream(be.stream):
            be.stream.wait_event(self.done)  # the previous update of the parameters has finished
            # forward
            torch.matmul(x, self.W1, out=self.h)
            be._check(lib.fb_bias_act_fwd(s, self.h.data_ptr(), self.b1.data_ptr(), 1, R, H, self.h.data_ptr()))
            torch.matmul(self.h, self.W2, out=self.yhat)
            be._check(lib.fb_bias_act_fwd(s, self.yhat.data_ptr(), self.b2.data_ptr(), 0, R, O, self.yhat.data_ptr()))
            # loss and its gradient in one pass
            be._check(lib.fb_mse_fwd_bwd(s, self.yhat.data_ptr(), y.data_ptr(), R * O, 1.0, self.loss.data_ptr(),
                                         self.dy.data_ptr(), ws, wsn))
            # backward, layer 2: db2 = column sums of dy, dW2 = h^T dy
            be._check(lib.fb_bias_act_bwd(s, self.dy.data_ptr(), None, None, 0, R, O, None, self.gb2.data_ptr(), ws, wsn))
            torch.matmul(self.h.t(), self.dy, out=self.gW2)
            self.ready[0].record(be.stream)
        if self.world > 1:
            with torch.cuda.stream(self.comm):
                self.comm.wait_event(self.ready[0])
                allreduce_sum_(self.buckets[0], self.group)
        with torch.cuda.stream(be.stream):
            # backward, layer 1 (overlaps the first all-reduce)
            torch.matmul(self.dy, self.W2.t(), out=self.dh)
            # relu mask from the saved activation (h > 0 exactly where the pre-activation was), dx in place
            be._check(lib.fb_bias_act_bwd(s, self.dh.data_ptr(), self.h.data_ptr(), None, 1, R, H, self.dh.data_ptr(),
                                          self.gb1.data_ptr(), ws, wsn))
            torch.matmul(x.t(), self.dh, out=self.gW1)
            self.ready[1].record(be.stream)
        self.t += 1
        bc1, bc2 = bias_correction(self.betas[0], self.t), bias_correction(self.betas[1], self.t)
        from .backend import AdamWStep
        hp = AdamWStep(self.lr, self.betas[0], self.betas[1], bc1, bc2, self.eps, 0.0)
        with torch.cuda.stream(self.comm):
            self.comm.wait_event(self.ready[1])
            if self.world > 1:
                allreduce_sum_(self.buckets[1], self.group)
            dev_table, n, total = self.table
            if self.max_grad_norm is None:
                be._check(lib.fb_adamw_multi(self.comm.cuda_stream, dev_table.data_ptr(), n, total, be._hp(hp),
                                             1.0 / self.world))
            else:
                if self.clip_scale is None:
                    self._norm_buf = torch.empty(3, device=be.device)  # sum of squares, norm, factor
                    self._norm_ws = torch.empty(int(lib.fb_grad_norm_workspace_bytes()), dtype=torch.uint8, device=be.device)
                    self.grad_norm, self.clip_scale = self._norm_buf[1:2], self._norm_buf[2:3]
                cs = self.comm.cuda_stream
                be._check(lib.fb_grad_sumsq_multi(cs, dev_table.data_ptr(), n, total, 1.0 / self.world,
                                                  self._norm_buf.data_ptr(), self._norm_ws.data_ptr(), self._norm_ws.numel()))
                be._check(lib.fb_clip_scale(cs, self._norm_buf.data_ptr(), float(self.max_grad_norm),
                                            self.grad_norm.data_ptr(), self.clip_scale.data_ptr()))
                be._check(lib.fb_adamw_multi_clipped(cs, dev_table.data_ptr(), n, total, be._hp(hp), 1.0 / self.world,
                                                     self.clip_scale.data_ptr()))
            self.done.record(self.comm)
        return self.loss

    def synchronize(self):
        self.comm.synchronize()
        self.be.synchronize()
