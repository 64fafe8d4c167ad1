"""Checkpoints of a device-resident training state in ferro's wire format.

ferro saves a state dict with `save_safetensors` and the optimizer state as
flat arrays named by parameter position - "m.i", "v.i", "t.i" for Adam
(crates/ferro-core/src/optim.rs:828-847), prefixed "optim." by its Checkpoint -
after downloading and re-encoding every buffer.  Here the image is laid out on
the host by the library (fb_safetensors_*), and tensor bytes go straight from
device memory into a pinned host image and back; files are interchangeable with
ferro's and with any other safetensors reader.
"""
import ctypes as C
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from .backend import FerroError, FormatError

_DT = {torch.float32: 0, torch.int64: 1, np.dtype(np.float32): 0, np.dtype(np.int64): 1}
_TORCH = {0: torch.float32, 1: torch.int64}


def _check(lib, rc):
    if rc != 0:
        raise (FormatError if rc == 7 else FerroError)(lib.fb_last_error().decode())


def _entries(named: Sequence[Tuple[str, object]]):
    arr = (_lib.StEntry * max(len(named), 1))()
    keep = []
    for i, (name, t) in enumerate(named):
        b = name.encode()
        keep.append(b)
        arr[i].name, arr[i].dtype, arr[i].rank = b, _DT[t.dtype], len(t.shape)
        for d, n in enumerate(t.shape):
            arr[i].shape[d] = int(n)
    return arr, keep


def to_safetensors_image(named: Sequence[Tuple[str, torch.Tensor]], stream=None) -> torch.Tensor:
    """to_safetensors_bytes (crates/ferro-core/src/safetensors.rs:36-94) for tensors that live on a device
    (or on the host): returns a pinned uint8 host tensor holding the whole file image.  Device tensors are
    copied on `stream` (default: the current one), which is synchronised before the image is returned."""
    lib = _lib.load()
    for _, t in named:
        if t.dtype not in _DT or not t.is_contiguous():
            raise FerroError("safetensors: tensors must be contiguous f32 or i64")
    on_dev = [t.is_cuda for _, t in named]
    if any(on_dev) and not all(on_dev):
        raise FerroError("safetensors: tensors must all live on the device or all on the host")
    arr, _keep = _entries(named)
    n = len(named)
    total = int(lib.fb_safetensors_image_bytes(arr, n, None))
    if total == 0:
        _check(lib, 2)
    image = torch.empty(total, dtype=torch.uint8)
    dev = bool(on_dev and on_dev[0])
    if dev and torch.cuda.is_available():
        image = image.pin_memory()
    srcs = (C.c_void_p * max(n, 1))(*[t.data_ptr() if t.numel() else None for _, t in named])
    s = None
    if dev:
        stream = stream or torch.cuda.current_stream(named[0][1].device)
        s = C.c_void_p(stream.cuda_stream)
    _check(lib, lib.fb_safetensors_write(s, arr, n, srcs, 1 if dev else 0, image.data_ptr(), total))
    if dev:
        stream.synchronize()
    return image


def save_safetensors(path: str, named: Sequence[Tuple[str, torch.Tensor]], stream=None):
    with open(path, "wb") as f:
        f.write(memoryview(to_safetensors_image(named, stream).numpy()))


def describe(image: torch.Tensor) -> List[Tuple[str, torch.dtype, Tuple[int, ...]]]:
    """(name, dtype, shape) of every tensor of an image, in header order."""
    lib = _lib.load()
    n = lib.fb_safetensors_count(image.data_ptr(), image.numel())
    if n < 0:
        raise FormatError(lib.fb_last_error().decode())
    out = []
    name = C.create_string_buffer(4096)
    for i in range(n):
        e = _lib.StEntry()
        _check(lib, lib.fb_safetensors_entry(image.data_ptr(), image.numel(), i, name, 4096, C.byref(e), None, None))
        if e.dtype not in _TORCH:
            raise FormatError(f"{name.value.decode()!r}: only F32 and I64 tensors are read")
        out.append((name.value.decode(), _TORCH[e.dtype], tuple(int(e.shape[d]) for d in range(e.rank))))
    return out


def from_safetensors_image(image: torch.Tensor, device=None, stream=None) -> List[Tuple[str, torch.Tensor]]:
    """from_safetensors_bytes (safetensors.rs:96-230): every tensor of the image, created on `device` (host
    when None) with its bytes copied straight from the image."""
    lib = _lib.load()
    if device is not None and not image.is_pinned() and torch.cuda.is_available():
        image = image.pin_memory()
    out = []
    dev = device is not None
    s = None
    if dev:
        device = torch.device(device)
        stream = stream or torch.cuda.current_stream(device)
        s = C.c_void_p(stream.cuda_stream)
    for name, dt, shape in describe(image):
        t = torch.empty(shape, dtype=dt, device=device if dev else "cpu")
        _check(lib, lib.fb_safetensors_read(s, image.data_ptr(), image.numel(), name.encode(), _DT[dt], t.numel(),
                                            t.data_ptr() if t.numel() else None, 1 if dev else 0))
        out.append((name, t))
    if dev:
        stream.synchronize()
    return out


def load_safetensors(path: str, device=None, stream=None) -> List[Tuple[str, torch.Tensor]]:
    raw = np.fromfile(path, dtype=np.uint8)
    return from_safetensors_image(torch.from_numpy(raw), device, stream)


def adam_state(params: Sequence[torch.Tensor], m: Sequence[torch.Tensor], v: Sequence[torch.Tensor], t: Sequence[int],
               prefix: str = "optim.") -> List[Tuple[str, torch.Tensor]]:
    """Adam::snapshot (optim.rs:828-847) as (name, tensor) pairs over the LIVE device buffers: per parameter i the
    flat first and second moments "m.i", "v.i" and the scalar step count "t.i" (f32), in that order."""
    out = []
    for i, (p, mi, vi, ti) in enumerate(zip(params, m, v, t)):
        out.append((f"{prefix}m.{i}", mi.reshape(-1)))
        out.append((f"{prefix}v.{i}", vi.reshape(-1)))
        out.append((f"{prefix}t.{i}", torch.full((), float(ti), dtype=torch.float32, device=p.device)))
    return out


def restore_adam_state(named: Dict[str, torch.Tensor], params: Sequence[torch.Tensor], m: Sequence[torch.Tensor],
                       v: Sequence[torch.Tensor], prefix: str = "optim.") -> List[int]:
    """The strict restore of optim.rs:73-80 / check_buf (:147-180): every "m.i" / "v.i" must be present as a flat
    f32 array of the parameter's element count; returns the step counts."""
    steps = []
    for i, p in enumerate(params):
        for key, dst in ((f"{prefix}m.{i}", m[i]), (f"{prefix}v.{i}", v[i])):
            if key not in named:
                raise FormatError(f"optimizer state is missing {key!r}")
            src = named[key]
            if src.dtype != torch.float32 or tuple(src.shape) != (p.numel(),):
                raise FormatError(f"{key!r}: expected flat f32 [{p.numel()}] (for {list(p.shape)}), got {src.dtype} {list(src.shape)}")
            dst.reshape(-1).copy_(src)
        key = f"{prefix}t.{i}"
        if key not in named:
            raise FormatError(f"optimizer state is missing {key!r}")
        steps.append(int(named[key].item()))
    return steps
