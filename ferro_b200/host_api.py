"""Host-buffer entry point for LayerNorm forward + backward.

ferro users who keep their tensors on the host reach the device through
`alloc_from_host` / `copy_to_host` (crates/ferro-cuda/src/lib.rs:571-588,
674-686): upload everything, compute, download everything, one after the
other.  Rows of a LayerNorm are independent, so the same request can be cut
into row chunks and run as a three-stage pipeline - upload chunk k+1 while
chunk k is computed and chunk k-1 is downloaded - which keeps both directions
of the host link busy at once.  The parameter gradients are the only values
that couple the chunks: each chunk writes its own partial dgamma / dbeta row
and one `fb_sum_dim` adds them at the end (in chunk order).
"""
import ctypes as C

import torch

from .backend import CudaBackend


class HostLayerNorm:
    """y, mean, rstd, dx, dgamma, dbeta = LN(x; gamma, beta) and its backward for upstream g,
    with x, g and every output living in pinned host memory."""

    def __init__(self, backend: CudaBackend, rows: int, cols: int, eps: float = 1e-5, chunks: int = 8):
        if rows % chunks:
            raise ValueError("rows must divide into the chunks")
        self.be, self.rows, self.cols, self.eps, self.k = backend, rows, cols, eps, chunks
        self.cr = rows // chunks
        dev = backend.device
        f = lambda *s: torch.empty(*s, device=dev, dtype=torch.float32)
        with torch.cuda.stream(backend.stream):
            self.x, self.g, self.y, self.dx = f(rows, cols), f(rows, cols), f(rows, cols), f(rows, cols)
            self.mu, self.rs = f(rows), f(rows)
            self.w, self.b = f(cols), f(cols)
            self.part = f(chunks, 2 * cols)      # per-chunk dgamma | dbeta
            self.dwb = f(2 * cols)
            ws = max(int(backend.lib.fb_layer_norm_bwd_workspace_bytes(self.cr, cols)),
                     int(backend.lib.fb_reduce_dim_workspace_bytes(1, chunks, 2 * cols)), 16)
            self.ws = torch.empty(ws, dtype=torch.uint8, device=dev)
        self.h2d, self.d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.ev_in = [torch.cuda.Event() for _ in range(chunks)]
        self.ev_out = [torch.cuda.Event() for _ in range(chunks)]
        self.ev_done, self.ev_read = torch.cuda.Event(), torch.cuda.Event()
        self.ev_done.record(backend.stream)
        self.ev_read.record(self.d2h)
        backend.synchronize()

    def bytes_in(self):
        return (2 * self.rows * self.cols + 2 * self.cols) * 4

    def bytes_out(self):
        return (2 * self.rows * self.cols + 2 * self.rows + 2 * self.cols) * 4

    def __call__(self, x_h, g_h, w_h, b_h, y_h, dx_h, mean_h, rstd_h, dwb_h):
        """All arguments are pinned host tensors; outputs are complete once `synchronize()` returns."""
        be, lib, cr, cols = self.be, self.be.lib, self.cr, self.cols
        s = C.c_void_p(be.stream.cuda_stream)
        p = lambda t: C.c_void_p(t.data_ptr())
        with torch.cuda.stream(self.h2d):
            self.h2d.wait_event(self.ev_done)  # the previous call no longer reads the device inputs
            self.w.copy_(w_h, non_blocking=True)
            self.b.copy_(b_h, non_blocking=True)
            for c in range(self.k):
                r = slice(c * cr, (c + 1) * cr)
                self.x[r].copy_(x_h[r], non_blocking=True)
                self.g[r].copy_(g_h[r], non_blocking=True)
                self.ev_in[c].record(self.h2d)
        be.stream.wait_event(self.ev_read)  # the previous call's downloads have left the device outputs
        for c in range(self.k):
            r = slice(c * cr, (c + 1) * cr)
            with torch.cuda.stream(be.stream):
                be.stream.wait_event(self.ev_in[c])
                be._check(lib.fb_layer_norm_fwd(s, p(self.x[r]), p(self.w), p(self.b), cr, cols, self.eps, p(self.y[r]),
                                                None, None, p(self.mu[r]), p(self.rs[r])))
                be._check(lib.fb_layer_norm_bwd(s, p(self.g[r]), None, None, p(self.x[r]), p(self.mu[r]), p(self.rs[r]),
                                                p(self.w), cr, cols, p(self.dx[r]), p(self.part[c]),
                                                C.c_void_p(self.part[c].data_ptr() + 4 * cols), p(self.ws), self.ws.numel()))
                self.ev_out[c].record(be.stream)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(self.ev_out[c])
                y_h[r].copy_(self.y[r], non_blocking=True)
                dx_h[r].copy_(self.dx[r], non_blocking=True)
        with torch.cuda.stream(be.stream):
            be._check(lib.fb_sum_dim(s, p(self.part), 1, self.k, 2 * cols, p(self.dwb), p(self.ws), self.ws.numel()))
            self.ev_done.record(be.stream)
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(self.ev_done)
            mean_h.copy_(self.mu, non_blocking=True)
            rstd_h.copy_(self.rs, non_blocking=True)
            dwb_h.copy_(self.dwb, non_blocking=True)
            self.ev_read.record(self.d2h)

    def synchronize(self):
        self.d2h.synchronize()
        self.be.synchronize()
