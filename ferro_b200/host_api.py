"""Host-buffer entry point for LayerNorm forward + backward.

ferro users who keep their tensors on the host reach the device through
`alloc_from_host` / `copy_to_host` (crates/ferro-cuda/src/lib.rs:571-588,
674-686): upload everything, compute, download everything, one after the
other.  `HostLayerNorm` is the Python face of the library's `fb_host_ln_*`
entry: the same request cut into row chunks and run as a three-stage pipeline
on three streams inside the library (upload chunk k + 1 / compute chunk k /
download chunk k - 1).  torch supplies the pinned host tensors and the device
staging buffer; every copy and kernel is issued by the C entry.
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
        lib = backend.lib
        torch.cuda.set_device(backend.device)
        self.handle = C.c_void_p()
        backend._check(lib.fb_host_ln_create(chunks, C.byref(self.handle)))
        nbytes = int(lib.fb_host_ln_device_bytes(rows, cols, chunks))
        with torch.cuda.stream(backend.stream):
            self.staging = torch.empty(nbytes, dtype=torch.uint8, device=backend.device)
        backend.synchronize()

    def bytes_in(self):
        return (2 * self.rows * self.cols + 2 * self.cols) * 4

    def bytes_out(self):
        return (2 * self.rows * self.cols + 2 * self.rows + 2 * self.cols) * 4

    def __call__(self, x_h, g_h, w_h, b_h, y_h, dx_h, mean_h, rstd_h, dwb_h):
        """All arguments are (pinned) host tensors; outputs are complete once `synchronize()` returns."""
        for t in (x_h, g_h, w_h, b_h, y_h, dx_h, mean_h, rstd_h, dwb_h):
            if t.is_cuda or not t.is_contiguous() or t.dtype != torch.float32:
                raise ValueError("HostLayerNorm takes contiguous f32 host tensors")
        p = lambda t: C.c_void_p(t.data_ptr())
        self.be._check(self.be.lib.fb_host_ln_run(self.handle, self.rows, self.cols, self.eps, p(x_h), p(g_h), p(w_h), p(b_h),
                                                  p(y_h), p(dx_h), p(mean_h), p(rstd_h), p(dwb_h),
                                                  C.c_void_p(self.staging.data_ptr()), self.staging.numel()))

    def synchronize(self):
        self.be._check(self.be.lib.fb_host_ln_synchronize(self.handle))

    def close(self):
        if self.handle:
            h, self.handle = self.handle, None
            self.be._check(self.be.lib.fb_host_ln_destroy(h))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
