"""DLPack exchange of device buffers, the Python face of the library's `fb_dlpack_*` entries.

ferro's `Tensor.__dlpack__` / `from_dlpack` (crates/ferro-py/src/lib.rs:2071-2103,
crates/ferro-py/src/dlpack.rs) export a CUDA tensor zero-copy behind a host
synchronisation and import one through the host.  Here:

* `export(backend, buf, shape, ...)` wraps a `DeviceBuffer` (or a view of it:
  element offset and strides) in an object with `__dlpack__(stream=None)` and
  `__dlpack_device__()`; the capsule borrows the buffer, which stays alive until
  the consumer's deleter has run; the hand-off to the consumer's stream is an
  event, not a host wait;
* `from_dlpack(backend, obj)` asks `obj.__dlpack__(stream=<backend stream>)` and
  copies the tensor into a fresh contiguous `DeviceBuffer` on the device (a
  strided producer tensor is gathered by the strided-copy kernel).

The capsule is built with the CPython C API through ctypes (PyCapsule_New,
name "dltensor"; a consumer renames it "used_dltensor" and owns the deleter
call from then on).
"""
import ctypes as C

import torch

from . import _lib
from .backend import CudaBackend, DeviceBuffer

_DLTENSOR, _USED = b"dltensor", b"used_dltensor"
_api = C.pythonapi
_api.PyCapsule_New.restype = C.py_object
_api.PyCapsule_New.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p]
_api.PyCapsule_IsValid.restype = C.c_int
_api.PyCapsule_IsValid.argtypes = [C.py_object, C.c_char_p]
_api.PyCapsule_GetPointer.restype = C.c_void_p
_api.PyCapsule_GetPointer.argtypes = [C.py_object, C.c_char_p]
_api.PyCapsule_SetName.restype = C.c_int
_api.PyCapsule_SetName.argtypes = [C.py_object, C.c_char_p]

_CAPSULE_DTOR = C.CFUNCTYPE(None, C.c_void_p)
_owners = {}     # token -> object kept alive for a capsule that is out
_next_token = [1]


@_lib.DLPACK_RELEASE_FN
def _release(token):
    _owners.pop(int(token or 0), None)


@_CAPSULE_DTOR
def _capsule_destructor(capsule_ptr):
    # A capsule nobody consumed still owns its tensor: run the deleter.  A consumed one was renamed.
    cap = C.cast(capsule_ptr, C.py_object)
    if _api.PyCapsule_IsValid(cap, _DLTENSOR):
        _lib.load().fb_dlpack_delete(_api.PyCapsule_GetPointer(cap, _DLTENSOR))


class Exported:
    """A device tensor offered to other libraries: `torch.from_dlpack(Exported(...))`."""

    def __init__(self, backend: CudaBackend, buf: DeviceBuffer, shape, strides=None, offset=0):
        self.be, self.buf = backend, buf
        self.shape = [int(v) for v in shape]
        self.strides = None if strides is None else [int(v) for v in strides]
        self.offset = int(offset)
        need = 1
        for v in self.shape:
            need *= v
        if self.strides is None and self.offset + need > len(buf):
            raise ValueError("shape does not fit the buffer")

    def __dlpack_device__(self):
        return (2, self.buf.device.index or 0)  # kDLCUDA

    def __dlpack__(self, stream=None):
        if isinstance(stream, bool) or not (stream is None or isinstance(stream, int)):
            raise TypeError("CUDA DLPack stream must be None or an integer")
        lib = self.be.lib
        # The consumer's stream is made to wait for everything enqueued on the backend's stream so far.
        self.be._check(lib.fb_dlpack_handoff(self.be._s(), 0 if stream is None else 1, 0 if stream is None else stream))
        width = 8 if self.buf.is_i64 else 4
        n = len(self.shape)
        shape = (C.c_int64 * max(n, 1))(*self.shape)
        strides = None if self.strides is None else (C.c_int64 * max(n, 1))(*self.strides)
        token = _next_token[0]
        _next_token[0] += 1
        managed = C.c_void_p()
        self.be._check(lib.fb_dlpack_export(self.buf.ptr, self.offset * width, 1 if self.buf.is_i64 else 0, n, shape, strides,
                                            self.buf.device.index or 0, token, _release, C.byref(managed)))
        _owners[token] = self.buf  # the capsule borrows the storage until its deleter runs
        return _api.PyCapsule_New(managed, _DLTENSOR, C.cast(_capsule_destructor, C.c_void_p))


def export(backend, buf, shape, strides=None, offset=0):
    return Exported(backend, buf, shape, strides, offset)


def outstanding():
    """Number of exported tensors whose deleter has not run yet."""
    return len(_owners)


_pending = []    # (event, capsule, managed pointer, lib): imported tensors whose copy may still be running


def _reap(block=False):
    """Runs the deleter of every imported tensor whose copy has finished (all of them when `block`)."""
    keep = []
    for ev, cap, managed, lib in _pending:
        if block:
            ev.synchronize()
        if block or ev.query():
            lib.fb_dlpack_delete(managed)
        else:
            keep.append((ev, cap, managed, lib))
    _pending[:] = keep


def from_dlpack(backend: CudaBackend, obj):
    """A contiguous DeviceBuffer (and its shape) holding the tensor `obj` offers.  The copy runs on the
    backend's stream, after the producer has ordered its own work before that stream; nothing waits on
    the host: the producer's tensor is kept (its deleter is called) only once an event behind the copy
    has completed, at a later call of this module."""
    lib = backend.lib
    _reap()
    cap = obj.__dlpack__(stream=backend.stream.cuda_stream) if hasattr(obj, "__dlpack__") else obj
    if not _api.PyCapsule_IsValid(cap, _DLTENSOR):
        raise ValueError("expected a 'dltensor' capsule (already consumed?)")
    managed = _api.PyCapsule_GetPointer(cap, _DLTENSOR)
    # Consumed from here on: the capsule is renamed so that its destructor leaves the tensor alone; the
    # deleter is ours to call, exactly once.
    _api.PyCapsule_SetName(cap, _USED)
    try:
        desc = _lib.DlpackDesc()
        backend._check(lib.fb_dlpack_describe(managed, C.byref(desc)))
        if desc.on_device and desc.device_id != (backend.device.index or 0):
            raise ValueError(f"tensor lives on cuda:{desc.device_id}, the backend on {backend.device}")
        shape = [int(desc.shape[d]) for d in range(desc.rank)]
        dtype = torch.int64 if desc.dtype == 1 else torch.float32
        with torch.cuda.stream(backend.stream):
            out = DeviceBuffer(torch.empty(int(desc.numel), dtype=dtype, device=backend.device))
        backend._check(lib.fb_dlpack_import_into(backend._s(), managed, out.ptr, int(desc.numel) * (8 if desc.dtype == 1 else 4)))
    except Exception:
        lib.fb_dlpack_delete(managed)
        raise
    ev = torch.cuda.Event()
    ev.record(backend.stream)
    _pending.append((ev, cap, managed, lib))  # the producer's memory stays alive until the copy has run
    return out, shape


def release_imports():
    """Waits for the imports in flight and returns their tensors to their producers."""
    _reap(block=True)
