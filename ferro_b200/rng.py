"""ferro's seeded generator (`ferro_core::Rng`, crates/ferro-core/src/rng.rs:12-70)
through the library's host-side entry points (fb_rng_*): the source of every
"seed k via ferro Rng" input.  Values land in host memory (numpy arrays, or
the pinned torch tensors passed as `out`), as ferro's Tensor::randn does
before it uploads (crates/ferro-core/src/tensor.rs:365-372)."""
import ctypes as C
import math

import numpy as np

from . import _lib


class Rng:
    def __init__(self, seed: int):
        self.lib = _lib.load()
        self.state = _lib.RngState()
        self.lib.fb_rng_seed(C.byref(self.state), int(seed))

    def _out(self, out, shape, dtype):
        n = math.prod(shape)
        if out is None:
            arr = np.empty(shape, dtype)
            return arr, arr.ctypes.data, n
        if hasattr(out, "data_ptr"):  # a (pinned) host torch tensor
            assert not out.is_cuda and out.is_contiguous() and out.numel() == n
            return out, out.data_ptr(), n
        assert out.flags["C_CONTIGUOUS"] and out.size == n and out.dtype == dtype
        return out, out.ctypes.data, n

    def _check(self, rc):
        if rc != 0:
            raise ValueError(self.lib.fb_last_error().decode())

    def skip(self, draws: int):
        """Advance by `draws` uniforms (a normal is two) without producing values."""
        self.lib.fb_rng_skip(C.byref(self.state), int(draws))

    def uniform(self) -> float:
        return float(self.lib.fb_rng_uniform(C.byref(self.state)))

    def normal(self) -> float:
        return float(self.lib.fb_rng_normal(C.byref(self.state)))

    def fill_uniform(self, shape, scale=1.0, shift=0.0, out=None):
        """shift + scale * uniform() per element, row-major."""
        arr, ptr, n = self._out(out, shape, np.float32)
        self._check(self.lib.fb_rng_fill_uniform(C.byref(self.state), ptr, n, scale, shift))
        return arr

    def fill_normal(self, shape, scale=1.0, shift=0.0, out=None):
        """shift + scale * normal() per element, row-major."""
        arr, ptr, n = self._out(out, shape, np.float32)
        self._check(self.lib.fb_rng_fill_normal(C.byref(self.state), ptr, n, scale, shift))
        return arr

    def fill_he(self, shape, fan_in, out=None):
        """normal() * sqrt(2 / fan_in): Linear::new (crates/ferro-core/src/nn.rs:138-146)."""
        s = float(np.sqrt(np.float32(2.0) / np.float32(fan_in)))
        return self.fill_normal(shape, s, 0.0, out)

    def fill_rowscaled_normal(self, rows, cols, lo=0.5, span=3.5, out=None):
        """Each row: one uniform u, then `cols` normals multiplied by (lo + span * u)."""
        arr, ptr, _ = self._out(out, (rows, cols), np.float32)
        self._check(self.lib.fb_rng_fill_rowscaled_normal(C.byref(self.state), ptr, rows, cols, lo, span))
        return arr

    def fill_index(self, n, classes, out=None):
        """floor(uniform() * classes) as i64."""
        arr, ptr, n = self._out(out, (n,), np.int64)
        self._check(self.lib.fb_rng_fill_index(C.byref(self.state), ptr, n, classes))
        return arr
