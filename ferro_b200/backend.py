"""Host-side mirror of ferro's device backend seam, over libferro_b200's C ABI.

`CudaBackend` carries the methods of `ferro_core::dispatch::Backend`
(crates/ferro-core/src/dispatch.rs:199-665) that `ferro_cuda::CudaBackend`
implements on the memory-bound path (crates/ferro-cuda/src/lib.rs:1032-1707),
with the same names, argument meaning and error behaviour, plus the fused
entry points the new library adds behind that seam.  A `DeviceBuffer` is what
the trait calls `&dyn DeviceBuffer`: a whole contiguous f32 (or i64) device
buffer.  torch supplies device memory and the stream, nothing else: every
operation goes through the C ABI, and there is no CPU fallback.
"""
import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from . import kinds as K


# ---- errors: ferro_core::Error variants this path can raise (error.rs) -------
class FerroError(Exception):
    pass


class InvalidShape(FerroError):
    pass


class Unsupported(FerroError):
    pass


class InvalidArgument(FerroError):
    pass


class WorkspaceError(FerroError):
    pass


class CommError(FerroError):
    """The gradient exchange failed (FB_ERR_COMM): an NCCL call or an asynchronous NCCL error."""


class FormatError(FerroError):
    """A checkpoint image is malformed (FB_ERR_FORMAT; ferro's Error::Format)."""


class DeviceFault(FerroError):
    """A kernel gave up a bounded wait (fb_device_faults() != 0): outputs of the calls since the
    last check are undefined."""


_ERRORS = {K.ERR_INVALID_SHAPE: InvalidShape, K.ERR_INVALID_ARG: InvalidArgument,
           K.ERR_CUDA: Unsupported, K.ERR_UNSUPPORTED: Unsupported, K.ERR_WORKSPACE: WorkspaceError,
           K.ERR_COMM: CommError, K.ERR_FORMAT: FormatError}


# ---- kinds (dispatch.rs:18-43, 68-76, 135-138) ------------------------------------
@dataclass(frozen=True)
class UnaryKind:
    code: int
    p0: float = 0.0
    p1: float = 0.0

    @staticmethod
    def Powf(p):
        return UnaryKind(K.UN_POWF, float(p))

    @staticmethod
    def Clamp(min, max):
        return UnaryKind(K.UN_CLAMP, float(min), float(max))


for _name, _code in [("Neg", K.UN_NEG), ("Relu", K.UN_RELU), ("Exp", K.UN_EXP),
                     ("Sigmoid", K.UN_SIGMOID), ("Tanh", K.UN_TANH), ("Sqrt", K.UN_SQRT),
                     ("Abs", K.UN_ABS), ("Sign", K.UN_SIGN), ("Log", K.UN_LOG), ("Gtz", K.UN_GTZ),
                     ("Gelu", K.UN_GELU), ("GeluErf", K.UN_GELU_ERF),
                     ("GeluErfGrad", K.UN_GELU_ERF_GRAD), ("Silu", K.UN_SILU)]:
    setattr(UnaryKind, _name, UnaryKind(_code))


@dataclass(frozen=True)
class BinaryKind:
    code: int
    p0: float = 0.0
    p1: float = 0.0

    @staticmethod
    def PowfBackward(p):
        return BinaryKind(K.BIN_POWF_BWD, float(p))

    @staticmethod
    def ClampBackward(min, max):
        return BinaryKind(K.BIN_CLAMP_BWD, float(min), float(max))


for _name, _code in [("Add", K.BIN_ADD), ("Sub", K.BIN_SUB), ("Mul", K.BIN_MUL), ("Div", K.BIN_DIV),
                     ("ReluBackward", K.BIN_RELU_BACKWARD), ("TanhBackward", K.BIN_TANH_BWD),
                     ("SigmoidBackward", K.BIN_SIGMOID_BWD), ("SqrtBackward", K.BIN_SQRT_BWD),
                     ("AbsBackward", K.BIN_ABS_BWD), ("LogBackward", K.BIN_LOG_BWD)]:
    setattr(BinaryKind, _name, BinaryKind(_code))


class ReduceKind:
    Sum = K.RED_SUM
    Mean = K.RED_MEAN


@dataclass(frozen=True)
class AdamWStep:
    """dispatch.rs:92-100."""
    lr: float
    beta1: float
    beta2: float
    bc1: float
    bc2: float
    eps: float
    weight_decay: float = 0.0


# ---- chain steps (dispatch.rs:107-121, extended with a temporary register) -------
V, T = 0, 1
SRC_OTHER, SRC_IMM, SRC_OPERAND0, SWAP = 0, 1, 8, 64


@dataclass(frozen=True)
class ChainStep:
    opcode: int
    dst: int = V
    kind: int = 0
    src: int = 0
    p0: float = 0.0
    p1: float = 0.0

    @staticmethod
    def Load(operand, dst=V):
        return ChainStep(0, dst, 0, operand)

    @staticmethod
    def Unary(kind: UnaryKind, dst=V):
        return ChainStep(1, dst, kind.code, 0, kind.p0, kind.p1)

    @staticmethod
    def Binary(kind: BinaryKind, other: Optional[int] = None, imm: Optional[float] = None,
               dst=V, swap=False):
        """dst = dst kind rhs; rhs = operand `other`, the immediate `imm`, or (neither given)
        the other register.  swap=True computes rhs kind dst."""
        if other is not None:
            src, p1 = SRC_OPERAND0 + other, kind.p1
        elif imm is not None:
            src, p1 = SRC_IMM, float(imm)
        else:
            src, p1 = SRC_OTHER, kind.p1
        return ChainStep(2, dst, kind.code, src | (SWAP if swap else 0), kind.p0, p1)

    @staticmethod
    def Imm(value, dst=V):
        return ChainStep(3, dst, 0, 0, float(value))


@dataclass
class View:
    """A ferro tensor view: (storage, shape, element strides, element offset), tensor.rs:213-227."""
    buf: "DeviceBuffer"
    strides: Sequence[int]
    offset: int = 0


class DeviceBuffer:
    """`dyn DeviceBuffer` (dispatch.rs:143-147): whole contiguous device storage."""

    def __init__(self, tensor: torch.Tensor):
        assert tensor.is_cuda and tensor.is_contiguous() and tensor.dim() == 1
        assert tensor.dtype in (torch.float32, torch.int64)
        self.t = tensor

    def __len__(self):
        return self.t.numel()

    @property
    def device(self):
        return self.t.device

    @property
    def ptr(self):
        return self.t.data_ptr() if self.t.numel() else None

    @property
    def is_i64(self):
        return self.t.dtype == torch.int64


def _u64s(vals):
    vals = [int(v) for v in vals]
    return (C.c_uint64 * max(len(vals), 1))(*vals)


def _i64s(vals):
    vals = [int(v) for v in vals]
    return (C.c_int64 * max(len(vals), 1))(*vals)


def _numel(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


class CudaBackend:
    """ferro_cuda::CudaBackend (crates/ferro-cuda/src/lib.rs:262-279) over the new kernels."""

    def __init__(self, ordinal: int = 0):
        if not torch.cuda.is_available():
            raise Unsupported("CUDA error: no CUDA device (there is no CPU fallback)")
        self.lib = _lib.load()
        self.device = torch.device("cuda", ordinal)
        torch.cuda.set_device(self.device)
        # One non-default stream per backend, like lib.rs:308-312.
        self.stream = torch.cuda.Stream(device=self.device)
        self._ws = None

    # -- plumbing ---------------------------------------------------------------
    def _s(self):
        return C.c_void_p(self.stream.cuda_stream)

    def _check(self, rc):
        if rc != 0:
            msg = self.lib.fb_last_error().decode()
            raise _ERRORS.get(rc, FerroError)(msg)

    def _own(self, *bufs):
        for b in bufs:
            if b is not None and b.device != self.device:
                raise Unsupported("buffer belongs to another device")  # lib.rs:378-386

    def _alloc(self, n, dtype=torch.float32) -> DeviceBuffer:
        with torch.cuda.stream(self.stream):
            return DeviceBuffer(torch.empty(int(n), dtype=dtype, device=self.device))

    def _workspace(self, nbytes):
        """Scratch owned by the caller side of the ABI (grown on demand, reused)."""
        nbytes = int(nbytes)
        if nbytes == 0:
            return None, 0
        if self._ws is None or self._ws.numel() < nbytes:
            with torch.cuda.stream(self.stream):
                self._ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=self.device)
        return self._ws.data_ptr(), self._ws.numel()

    def synchronize(self):
        """Wait for the backend's stream, then read the device status word: a pipelined kernel whose
        bounded wait gave up returns early and leaves its outputs incomplete, and this is where the
        host learns of it (the reference surfaces recorded driver errors the same way,
        crates/ferro-cuda/src/lib.rs:593-597, 1938-1946)."""
        self.stream.synchronize()
        self._raise_on_device_fault()

    def _raise_on_device_fault(self):
        n = self.lib.fb_device_faults(1)
        if n > 0:
            raise DeviceFault(f"{n} bounded device wait(s) gave up since the last check: the outputs of the "
                              "kernels launched since then are undefined")

    # -- transfers (lib.rs:571-588, 674-686) ---------------------------------------
    def alloc_from_host(self, data) -> DeviceBuffer:
        a = np.ascontiguousarray(data, dtype=np.float32).ravel()
        with torch.cuda.stream(self.stream):
            return DeviceBuffer(torch.from_numpy(a.copy()).to(self.device, non_blocking=False))

    def alloc_i64_from_host(self, data) -> DeviceBuffer:
        a = np.ascontiguousarray(data, dtype=np.int64).ravel()
        with torch.cuda.stream(self.stream):
            return DeviceBuffer(torch.from_numpy(a.copy()).to(self.device))

    def copy_to_host(self, buf: DeviceBuffer) -> np.ndarray:
        if buf.is_i64:
            raise Unsupported("copy_to_host on an i64 buffer")
        self.synchronize()
        return buf.t.cpu().numpy()

    def copy_i64_to_host(self, buf: DeviceBuffer) -> np.ndarray:
        if not buf.is_i64:
            raise Unsupported("copy_i64_to_host on an f32 buffer")
        self.synchronize()
        return buf.t.cpu().numpy()

    # -- elementwise ------------------------------------------------------------------
    def unary_dev(self, kind: UnaryKind, x: DeviceBuffer) -> DeviceBuffer:
        self._own(x)
        out = self._alloc(len(x))
        self._check(self.lib.fb_unary(self._s(), kind.code, kind.p0, kind.p1, x.ptr, out.ptr, len(x)))
        return out

    def binary_dev(self, kind: BinaryKind, a: DeviceBuffer, b: DeviceBuffer) -> DeviceBuffer:
        self._own(a, b)
        if len(a) != len(b):
            raise InvalidShape(f"binary_dev: {len(a)} vs {len(b)} elements")
        out = self._alloc(len(a))
        self._check(self.lib.fb_binary(self._s(), kind.code, kind.p0, kind.p1, a.ptr, b.ptr, out.ptr, len(a)))
        return out

    def binary_bc_dev(self, kind: BinaryKind, a, sa, b, sb, out_shape) -> DeviceBuffer:
        self._own(a, b)
        if _numel(sa) != len(a) or _numel(sb) != len(b):
            raise InvalidShape("binary_bc_dev: buffer length does not match its shape")
        out = self._alloc(_numel(out_shape))
        self._check(self.lib.fb_binary_bc(self._s(), kind.code, kind.p0, kind.p1, a.ptr, _u64s(sa), len(sa),
                                          b.ptr, _u64s(sb), len(sb), out.ptr, _u64s(out_shape), len(out_shape)))
        return out

    def unary_strided_dev(self, kind: UnaryKind, x: View, shape) -> DeviceBuffer:
        self._own(x.buf)
        out = self._alloc(_numel(shape))
        self._check(self.lib.fb_unary_strided(self._s(), kind.code, kind.p0, kind.p1, x.buf.ptr, len(x.buf),
                                              _i64s(x.strides), x.offset, _u64s(shape), len(shape), out.ptr))
        return out

    def binary_strided_dev(self, kind: BinaryKind, a: View, b: View, shape) -> DeviceBuffer:
        self._own(a.buf, b.buf)
        out = self._alloc(_numel(shape))
        self._check(self.lib.fb_binary_strided(self._s(), kind.code, kind.p0, kind.p1, a.buf.ptr, len(a.buf),
                                               _i64s(a.strides), a.offset, b.buf.ptr, len(b.buf),
                                               _i64s(b.strides), b.offset, _u64s(shape), len(shape), out.ptr))
        return out

    def materialize_dev(self, x: DeviceBuffer, shape, strides, offset) -> DeviceBuffer:
        self._own(x)
        out = self._alloc(_numel(shape))
        self._check(self.lib.fb_materialize(self._s(), x.ptr, len(x), _i64s(strides), offset, _u64s(shape),
                                            len(shape), out.ptr))
        return out

    def chain_dev(self, steps: Sequence[ChainStep], inputs: Sequence, shape=None) -> DeviceBuffer:
        """`inputs` are DeviceBuffers (whole, output-shaped: ferro's contract) or Views."""
        return self.chain_into(steps, inputs, shape, None)

    def chain_into(self, steps: Sequence[ChainStep], inputs: Sequence, shape=None, out: Optional[DeviceBuffer] = None):
        """chain_dev writing into a buffer the caller already holds (allocated when None)."""
        views = []
        for x in inputs:
            if isinstance(x, DeviceBuffer):
                if shape is None:
                    shape = [len(x)]
                st, acc = [], 1
                for s in reversed(list(shape)):
                    st.insert(0, acc)
                    acc *= int(s)
                if acc != len(x):
                    raise InvalidShape("chain_dev: whole operands must have the output's length")
                x = View(x, st, 0)
            views.append(x)
        if shape is None:
            raise InvalidShape("chain_dev: shape is required when every input is a view")
        self._own(*[v.buf for v in views])
        cs = (_lib.ChainStep * max(len(steps), 1))()
        for i, s in enumerate(steps[:_lib.CHAIN_MAX_STEPS]):
            cs[i] = _lib.ChainStep(s.opcode, s.dst, s.kind, s.src, s.p0, s.p1)
        co = (_lib.ChainOperand * max(len(views), 1))()
        for i, v in enumerate(views[:_lib.CHAIN_MAX_OPERANDS]):
            st = list(v.strides) + [0] * (_lib.MAX_RANK - len(v.strides))
            co[i] = _lib.ChainOperand(v.buf.ptr, len(v.buf), int(v.offset), (C.c_int64 * _lib.MAX_RANK)(*st[:_lib.MAX_RANK]))
        if out is None:
            out = self._alloc(_numel(shape))
        elif len(out) != _numel(shape):
            raise InvalidShape("chain_into: the output buffer does not have the output's length")
        self._own(out)
        self._check(self.lib.fb_chain(self._s(), cs, len(steps), co, len(views), _u64s(shape), len(shape), out.ptr))
        return out

    # -- in-place family -------------------------------------------------------------
    def fill_dev(self, value, n) -> DeviceBuffer:
        out = self._alloc(n)
        self._check(self.lib.fb_fill(self._s(), out.ptr, value, n))
        return out

    def fill_inplace_dev(self, dst: DeviceBuffer, value):
        self._own(dst)
        self._check(self.lib.fb_fill(self._s(), dst.ptr, value, len(dst)))

    def affine_inplace_dev(self, dst: DeviceBuffer, mul, add):
        self._own(dst)
        self._check(self.lib.fb_affine_inplace(self._s(), dst.ptr, mul, add, len(dst)))

    def binary_inplace_dev(self, kind: BinaryKind, dst: DeviceBuffer, src: DeviceBuffer):
        self._own(dst, src)
        if len(dst) != len(src):
            raise InvalidShape("binary_inplace_dev: length mismatch")
        self._check(self.lib.fb_binary_inplace(self._s(), kind.code, dst.ptr, src.ptr, len(dst)))

    def axpy_inplace_dev(self, alpha, dst: DeviceBuffer, src: DeviceBuffer):
        self._own(dst, src)
        if len(dst) != len(src):
            raise InvalidShape("axpy_inplace_dev: length mismatch")
        self._check(self.lib.fb_axpy_inplace(self._s(), alpha, dst.ptr, src.ptr, len(dst)))

    def copy_into_dev(self, dst: DeviceBuffer, src: DeviceBuffer):
        self._own(dst, src)
        if len(dst) != len(src):
            raise InvalidShape("copy_into_dev: length mismatch")
        self._check(self.lib.fb_copy(self._s(), dst.ptr, src.ptr, len(dst)))

    def copy_dev(self, src: DeviceBuffer) -> DeviceBuffer:
        out = self._alloc(len(src))
        self.copy_into_dev(out, src)
        return out

    def gather_rows_dev(self, w: DeviceBuffer, idx: DeviceBuffer, dim_size, inner) -> DeviceBuffer:
        self._own(w, idx)
        if not idx.is_i64:
            raise Unsupported("gather_rows_dev: indices must be an i64 buffer")
        if len(w) != dim_size * inner:
            raise InvalidShape("gather_rows_dev: table length does not match dim_size * inner")
        out = self._alloc(len(idx) * inner)
        with torch.cuda.stream(self.stream):
            bad = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._check(self.lib.fb_gather_rows(self._s(), w.ptr, idx.ptr, len(idx), dim_size, inner, out.ptr,
                                            bad.data_ptr()))
        self.stream.synchronize()
        if int(bad.item()):
            raise InvalidShape(f"gather_rows_dev: index at position {int(bad.item()) - 1} out of range")
        return out

    # -- reductions ---------------------------------------------------------------------
    def reduce_dev(self, kind, x: DeviceBuffer) -> DeviceBuffer:
        self._own(x)
        out = self._alloc(1)
        ws, nb = self._workspace(self.lib.fb_reduce_workspace_bytes(len(x)))
        self._check(self.lib.fb_reduce(self._s(), kind, x.ptr, len(x), out.ptr, ws, nb))
        return out

    @staticmethod
    def _ori(shape, dim):
        if dim >= len(shape):
            raise InvalidShape(f"dim {dim} out of range for rank {len(shape)}")
        return _numel(shape[:dim]), int(shape[dim]), _numel(shape[dim + 1:])

    def _dim_reduce(self, fn, x, shape, dim):
        self._own(x)
        o, r, i = self._ori(shape, dim)
        if o * r * i != len(x):
            raise InvalidShape("buffer length does not match its shape")
        out = self._alloc(o * i)
        ws, nb = self._workspace(self.lib.fb_reduce_dim_workspace_bytes(o, r, i))
        self._check(fn(self._s(), x.ptr, o, r, i, out.ptr, ws, nb))
        return out

    def sum_dim_dev(self, x, shape, dim) -> DeviceBuffer:
        return self._dim_reduce(self.lib.fb_sum_dim, x, shape, dim)

    def mean_dim_dev(self, x, shape, dim) -> DeviceBuffer:
        return self._dim_reduce(self.lib.fb_mean_dim, x, shape, dim)

    def max_dim_dev(self, x, shape, dim):
        """(values f32, indices i64), keepdim layout; ferro's argmax order (ops_ext/argmax.rs:42-63)."""
        self._own(x)
        o, r, i = self._ori(shape, dim)
        if o * r * i != len(x):
            raise InvalidShape("buffer length does not match its shape")
        val, idx = self._alloc(o * i), self._alloc(o * i, torch.int64)
        ws, nb = self._workspace(self.lib.fb_reduce_dim_workspace_bytes(o, r, i))
        self._check(self.lib.fb_max_dim(self._s(), x.ptr, o, r, i, val.ptr, idx.ptr, ws, nb))
        return val, idx

    # -- index-driven ops (ops_ext/gather.rs, segment.rs) -----------------------------------------------
    def _bad_word(self):
        with torch.cuda.stream(self.stream):
            return torch.zeros(1, dtype=torch.int64, device=self.device)

    def gather_dev(self, x: DeviceBuffer, in_shape, dim, index: DeviceBuffer, out_shape) -> DeviceBuffer:
        """Tensor::gather (ops_ext/gather.rs:12-98) on device buffers; raises InvalidShape on an index out of range."""
        self._own(x, index)
        if not index.is_i64 or len(index) != _numel(out_shape) or len(x) != _numel(in_shape) or len(in_shape) != len(out_shape):
            raise InvalidShape("gather_dev: buffers do not match their shapes")
        out, bad = self._alloc(len(index)), self._bad_word()
        self._check(self.lib.fb_gather_dim(self._s(), x.ptr, _u64s(in_shape), index.ptr, _u64s(out_shape), len(in_shape),
                                           dim, out.ptr, bad.data_ptr()))
        self.synchronize()
        if int(bad.item()):
            raise InvalidShape(f"gather: index at flat position {int(bad.item()) - 1} out of range for dim {dim}")
        return out

    def gather_backward_dev(self, g: DeviceBuffer, index: DeviceBuffer, in_shape, out_shape, dim) -> DeviceBuffer:
        """The scatter-add of gather's backward (ops_ext/gather.rs:103-110): a gradient over in_shape."""
        self._own(g, index)
        if not index.is_i64 or len(index) != _numel(out_shape) or len(g) != len(index):
            raise InvalidShape("gather_backward_dev: buffers do not match their shapes")
        gx = self._alloc(_numel(in_shape))
        self._check(self.lib.fb_scatter_add_dim(self._s(), g.ptr, index.ptr, _u64s(in_shape), _u64s(out_shape),
                                                len(in_shape), dim, gx.ptr, None))
        return gx

    def prepare_segments(self, ids, groups):
        """Backend::prepare_segments (dispatch.rs:383; crates/ferro-cuda/src/segment.rs:20-33): the CSR table
        on the device.  Returns (csr buffer, edges, groups)."""
        ids = np.ascontiguousarray(ids, dtype=np.uint64)
        csr = np.empty(groups + 1 + len(ids), np.int64)
        self._check(self.lib.fb_segment_csr_build(ids.ctypes.data, len(ids), groups, csr.ctypes.data))
        return self.alloc_i64_from_host(csr), len(ids), int(groups)

    def segment_dev(self, plan, op: str, x: DeviceBuffer, width, saved: Optional[DeviceBuffer] = None) -> DeviceBuffer:
        """Backend::segment_dev (dispatch.rs:388): op in "sum", "sum_backward", "softmax", "softmax_backward"."""
        csr, edges, groups = plan
        self._own(x, saved)
        n_in = groups * width if op == "sum_backward" else edges * width
        if len(x) != n_in or (op == "softmax_backward" and (saved is None or len(saved) != edges * width)):
            raise InvalidShape("segment_dev: invalid segment buffer or size")
        out = self._alloc(groups * width if op == "sum" else edges * width)
        s = self._s()
        if op == "sum":
            self._check(self.lib.fb_segment_sum(s, x.ptr, csr.ptr, groups, edges, width, out.ptr))
        elif op == "sum_backward":
            self._check(self.lib.fb_segment_sum_bwd(s, x.ptr, csr.ptr, groups, edges, width, out.ptr))
        elif op == "softmax":
            with torch.cuda.stream(self.stream):
                flag = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._check(self.lib.fb_segment_softmax_fwd(s, x.ptr, csr.ptr, groups, edges, width, out.ptr, flag.data_ptr()))
            self.synchronize()  # the four-byte control read of segment.rs:79-85
            if int(flag.item()):
                raise Unsupported("segment_softmax: finite logits required")
        elif op == "softmax_backward":
            self._check(self.lib.fb_segment_softmax_bwd(s, x.ptr, saved.ptr, csr.ptr, groups, edges, width, out.ptr))
        else:
            raise InvalidArgument(f"segment_dev: unknown op {op}")
        return out

    # -- reductions and softmax on views (tensor.rs:2057-2104, 2124-2140) --------------------------------
    @staticmethod
    def _view(v: View, shape):
        d = _lib.ViewDesc()
        d.ptr, d.len, d.offset, d.rank = v.buf.ptr, len(v.buf), int(v.offset), len(shape)
        for i, (n, st) in enumerate(zip(shape, v.strides)):
            d.shape[i], d.strides[i] = int(n), int(st)
        return d

    def _reduce_view(self, fn, x: View, shape, dim, *outs):
        self._own(x.buf)
        if len(x.strides) != len(shape) or not 0 <= dim < len(shape):
            raise InvalidShape(f"view of rank {len(x.strides)} for shape {list(shape)}, dim {dim}")
        d = self._view(x, shape)
        ws, nb = self._workspace(self.lib.fb_reduce_view_workspace_bytes(C.byref(d), dim))
        self._check(fn(self._s(), C.byref(d), dim, *[o.ptr if o is not None else None for o in outs], ws, nb))

    def sum_dim_view_dev(self, x: View, shape, dim) -> DeviceBuffer:
        """sum over `dim` of a view; the result is row-major over `shape` with `dim` set to 1."""
        out = self._alloc(_numel([s for i, s in enumerate(shape) if i != dim]))
        self._reduce_view(self.lib.fb_sum_dim_view, x, shape, dim, out)
        return out

    def mean_dim_view_dev(self, x: View, shape, dim) -> DeviceBuffer:
        out = self._alloc(_numel([s for i, s in enumerate(shape) if i != dim]))
        self._reduce_view(self.lib.fb_mean_dim_view, x, shape, dim, out)
        return out

    def max_dim_view_dev(self, x: View, shape, dim):
        """(values, i64 indices) of the maximum over `dim` of a view (first NaN wins, ties keep the lowest index)."""
        n = _numel([s for i, s in enumerate(shape) if i != dim])
        val, idx = self._alloc(n), self._alloc(n, torch.int64)
        self._reduce_view(self.lib.fb_max_dim_view, x, shape, dim, val, idx)
        return val, idx

    def softmax_view_dev(self, x: View, shape, dim, log=False) -> DeviceBuffer:
        """softmax / log_softmax over any dim of a view; the result is row-major over `shape`."""
        self._own(x.buf)
        out = self._alloc(_numel(shape))
        fn = self.lib.fb_log_softmax_view_fwd if log else self.lib.fb_softmax_view_fwd
        self._check(fn(self._s(), C.byref(self._view(x, shape)), dim, out.ptr))
        return out

    def softmax_view_backward_dev(self, g: View, y: View, shape, dim, log=False) -> DeviceBuffer:
        self._own(g.buf, y.buf)
        out = self._alloc(_numel(shape))
        fn = self.lib.fb_log_softmax_view_bwd if log else self.lib.fb_softmax_view_bwd
        self._check(fn(self._s(), C.byref(self._view(g, shape)), C.byref(self._view(y, shape)), dim, out.ptr))
        return out

    # -- softmax family ---------------------------------------------------------------------
    def _rc(self, x, rows, cols):
        if rows * cols != len(x):
            raise InvalidShape(f"rows {rows} x cols {cols} does not match {len(x)} elements")

    def softmax_dev(self, x, rows, cols) -> DeviceBuffer:
        self._own(x)
        self._rc(x, rows, cols)
        y = self._alloc(len(x))
        self._check(self.lib.fb_softmax_fwd(self._s(), x.ptr, rows, cols, y.ptr))
        return y

    def log_softmax_dev(self, x, rows, cols) -> DeviceBuffer:
        self._own(x)
        self._rc(x, rows, cols)
        y = self._alloc(len(x))
        self._check(self.lib.fb_log_softmax_fwd(self._s(), x.ptr, rows, cols, y.ptr))
        return y

    def softmax_backward_dev(self, g, y, rows, cols) -> DeviceBuffer:
        self._own(g, y)
        self._rc(g, rows, cols)
        self._rc(y, rows, cols)
        dx = self._alloc(len(y))
        self._check(self.lib.fb_softmax_bwd(self._s(), g.ptr, y.ptr, rows, cols, dx.ptr))
        return dx

    def log_softmax_backward_dev(self, g, y, rows, cols) -> DeviceBuffer:
        self._own(g, y)
        self._rc(g, rows, cols)
        self._rc(y, rows, cols)
        dx = self._alloc(len(y))
        self._check(self.lib.fb_log_softmax_bwd(self._s(), g.ptr, y.ptr, rows, cols, dx.ptr))
        return dx

    def bias_act_scale_softmax_dev(self, x, bias, relu, scale, rows, cols) -> DeviceBuffer:
        self._own(x, bias)
        self._rc(x, rows, cols)
        y = self._alloc(len(x))
        self._check(self.lib.fb_bias_act_scale_softmax_fwd(self._s(), x.ptr, bias.ptr if bias else None,
                                                           1 if relu else 0, scale, rows, cols, y.ptr))
        return y

    def bias_act_scale_softmax_backward_dev(self, g, y, x, bias, relu, scale, rows, cols, want_dbias=True):
        self._own(g, y, x, bias)
        self._rc(g, rows, cols)
        dx = self._alloc(len(g))
        db = self._alloc(cols) if want_dbias else None
        ws, nb = self._workspace(self.lib.fb_softmax_fused_bwd_workspace_bytes(rows, cols) if want_dbias else 0)
        self._check(self.lib.fb_bias_act_scale_softmax_bwd(
            self._s(), g.ptr, y.ptr, x.ptr, bias.ptr if bias else None, 1 if relu else 0, scale, rows, cols,
            dx.ptr, db.ptr if db else None, ws, nb))
        return dx, db

    def cross_entropy_indices_dev(self, logits, targets, rows, cols, want_argmax=True):
        """nn::cross_entropy_indices (crates/ferro-core/src/nn.rs:793-814) fused:
        returns (loss[1], saved (row_max, row_lse), argmax i64[rows] | None)."""
        self._own(logits, targets)
        self._rc(logits, rows, cols)
        if not targets.is_i64 or len(targets) != rows:
            raise InvalidShape(f"{len(targets)} target ids for batch of {rows}")
        loss, rmax, rlse = self._alloc(1), self._alloc(rows), self._alloc(rows)
        am = self._alloc(rows, torch.int64) if want_argmax else None
        with torch.cuda.stream(self.stream):
            bad = torch.zeros(1, dtype=torch.int64, device=self.device)
        ws, nb = self._workspace(self.lib.fb_nll_workspace_bytes(rows))
        self._check(self.lib.fb_log_softmax_nll_fwd(self._s(), logits.ptr, targets.ptr, rows, cols, loss.ptr,
                                                    rmax.ptr, rlse.ptr, am.ptr if am else None,
                                                    bad.data_ptr(), ws, nb))
        self._bad_target = bad
        return loss, (rmax, rlse), am

    def check_targets(self):
        """Raises like one_hot (nn.rs:419-424) if the last cross-entropy saw a bad class id."""
        self.stream.synchronize()
        b = int(self._bad_target.item())
        if b:
            raise InvalidShape(f"id at row {b - 1} out of range")

    def cross_entropy_indices_backward_dev(self, logits, targets, saved, rows, cols, grad_scale=1.0):
        self._own(logits, targets)
        rmax, rlse = saved
        dl = self._alloc(len(logits))
        self._check(self.lib.fb_log_softmax_nll_bwd(self._s(), logits.ptr, targets.ptr, rmax.ptr, rlse.ptr,
                                                    grad_scale, rows, cols, dl.ptr))
        return dl

    # -- LayerNorm -------------------------------------------------------------------------------
    def _ln_check(self, x, weight, bias, rows, cols):
        self._own(x, weight, bias)
        if cols == 0:
            raise InvalidShape("last dimension must be nonempty")
        if rows >= (1 << 63) or rows * cols != len(x):  # lib.rs:1264-1269
            raise InvalidShape("rows x cols does not match the buffer")
        for t in (weight, bias):
            if t is not None and len(t) != cols:
                raise InvalidShape(f"affine parameter has {len(t)} elements, expected {cols}")

    def layer_norm_dev(self, x, weight, bias, rows, cols, eps):
        """(y, h, stds), dispatch.rs:369-373."""
        self._ln_check(x, weight, bias, rows, cols)
        y, h, s = self._alloc(len(x)), self._alloc(len(x)), self._alloc(rows)
        self._check(self.lib.fb_layer_norm_fwd(self._s(), x.ptr, weight.ptr if weight else None,
                                               bias.ptr if bias else None, rows, cols, eps, y.ptr, h.ptr,
                                               s.ptr, None, None))
        return y, h, s

    def layer_norm_output_dev(self, x, weight, bias, rows, cols, eps) -> DeviceBuffer:
        self._ln_check(x, weight, bias, rows, cols)
        y = self._alloc(len(x))
        self._check(self.lib.fb_layer_norm_fwd(self._s(), x.ptr, weight.ptr if weight else None,
                                               bias.ptr if bias else None, rows, cols, eps, y.ptr, None,
                                               None, None, None))
        return y

    def layer_norm_stats_dev(self, x, weight, bias, rows, cols, eps):
        """(y, mean, rstd): the compact statistics form."""
        self._ln_check(x, weight, bias, rows, cols)
        y, mu, rs = self._alloc(len(x)), self._alloc(rows), self._alloc(rows)
        self._check(self.lib.fb_layer_norm_fwd(self._s(), x.ptr, weight.ptr if weight else None,
                                               bias.ptr if bias else None, rows, cols, eps, y.ptr, None,
                                               None, mu.ptr, rs.ptr))
        return y, mu, rs

    def layer_norm_backward_dev(self, g, weight, rows, cols, h=None, stds=None, x=None, mean=None,
                                rstd=None, want_dw=True, want_db=True):
        """(dx, dweight | None, dbias | None) from (h, stds) or from (x, mean, rstd)."""
        self._own(g, weight, h, stds, x, mean, rstd)
        self._rc(g, rows, cols)
        dx = self._alloc(len(g))
        dw = self._alloc(cols) if want_dw else None
        db = self._alloc(cols) if want_db else None
        ws, nb = self._workspace(self.lib.fb_layer_norm_bwd_workspace_bytes(rows, cols))
        p = lambda b: b.ptr if b is not None else None
        self._check(self.lib.fb_layer_norm_bwd(self._s(), g.ptr, p(h), p(stds), p(x), p(mean), p(rstd),
                                               p(weight), rows, cols, dx.ptr, p(dw), p(db), ws, nb))
        return dx, dw, db

    def residual_layer_norm_dev(self, x, residual, weight, bias, rows, cols, eps, want_sum=False):
        """Tensor::residual_layernorm (fused_ops.rs:106-231): (y, h, stds[, x + residual])."""
        self._own(x, residual, weight, bias)
        self._rc(x, rows, cols)
        if len(residual) != len(x):
            raise InvalidShape("residual_layer_norm_dev: x and residual differ in length")
        if cols == 0:
            raise InvalidShape("residual_layer_norm_dev: last dimension must be nonempty")
        for t in (weight, bias):
            if t is not None and len(t) != cols:
                raise InvalidShape("residual_layer_norm_dev: weight / bias length != cols")
        y, h, s = self._alloc(rows * cols), self._alloc(rows * cols), self._alloc(rows)
        sm = self._alloc(rows * cols) if want_sum else None
        p = lambda b: b.ptr if b is not None else None
        self._check(self.lib.fb_residual_layer_norm_fwd(self._s(), x.ptr, residual.ptr, p(weight), p(bias), rows, cols,
                                                        eps, y.ptr, h.ptr, s.ptr, None, None, p(sm)))
        return (y, h, s, sm) if want_sum else (y, h, s)

    def rms_norm_dev(self, x, weight, rows, cols, eps):
        """RmsNorm::forward (nn.rs:272-279) as one kernel: (y, rstd)."""
        self._own(x, weight)
        self._rc(x, rows, cols)
        if cols == 0:
            raise InvalidShape("rms_norm_dev: last dimension must be nonempty")
        if weight is not None and len(weight) != cols:
            raise InvalidShape("rms_norm_dev: weight length != cols")
        y, rs = self._alloc(rows * cols), self._alloc(rows)
        self._check(self.lib.fb_rms_norm_fwd(self._s(), x.ptr, weight.ptr if weight is not None else None, rows, cols,
                                             eps, y.ptr, rs.ptr))
        return y, rs

    def rms_norm_backward_dev(self, g, x, rstd, weight, rows, cols, want_dw=True):
        """(dx, dweight | None) from the saved (x, rstd)."""
        self._own(g, x, rstd, weight)
        self._rc(g, rows, cols)
        dx = self._alloc(len(g))
        dw = self._alloc(cols) if want_dw else None
        ws, nb = self._workspace(self.lib.fb_layer_norm_bwd_workspace_bytes(rows, cols))
        self._check(self.lib.fb_rms_norm_bwd(self._s(), g.ptr, x.ptr, rstd.ptr, weight.ptr if weight is not None else None,
                                             rows, cols, dx.ptr, dw.ptr if dw is not None else None, ws, nb))
        return dx, dw

    # -- optimizers -----------------------------------------------------------------------------------
    def sgd_step_dev(self, p, v, g, lr, momentum, nesterov):
        self._own(p, v, g)
        if not (len(p) == len(v) == len(g)):
            raise InvalidShape("sgd_step_dev: length mismatch")
        self._check(self.lib.fb_sgd_step(self._s(), p.ptr, v.ptr, g.ptr, len(p), lr, momentum, 1 if nesterov else 0))

    @staticmethod
    def _hp(hp: AdamWStep):
        return _lib.AdamWHparams(hp.lr, hp.beta1, hp.beta2, hp.bc1, hp.bc2, hp.eps, hp.weight_decay)

    def adamw_step_dev(self, p, m, v, g, hp: AdamWStep):
        self._own(p, m, v, g)
        if not (len(p) == len(m) == len(v) == len(g)):
            raise InvalidShape("adamw_step_dev: length mismatch")
        self._check(self.lib.fb_adamw_step(self._s(), p.ptr, m.ptr, v.ptr, g.ptr, len(p), self._hp(hp)))

    def adamw_step_capturable_dev(self, p, m, v, g, t, lr, beta1, beta2, eps, weight_decay):
        self._own(p, m, v, g, t)
        if len(t) != 3:
            raise InvalidShape("timestep buffer must hold [step, bc1, bc2]")
        self._check(self.lib.fb_adamw_step_capturable(self._s(), p.ptr, m.ptr, v.ptr, g.ptr, t.ptr, len(p), lr,
                                                      beta1, beta2, eps, weight_decay))

    def scalar_increment_dev(self, t, beta1, beta2):
        self._own(t)
        self._check(self.lib.fb_scalar_increment(self._s(), t.ptr, beta1, beta2))

    def make_table(self, quads):
        """Device table of (p, m, v, g) buffers for the multi-tensor steps."""
        arr = (_lib.TensorQuad * len(quads))()
        total = 0
        for i, (p, m, v, g) in enumerate(quads):
            arr[i] = _lib.TensorQuad(p.ptr, m.ptr, v.ptr if v is not None else None, g.ptr, len(p))
            total += len(p)
        raw = np.frombuffer(bytes(arr), dtype=np.uint8).copy()
        with torch.cuda.stream(self.stream):
            dev = torch.from_numpy(raw).to(self.device)
        return dev, len(quads), total

    def adamw_multi_dev(self, table, hp: AdamWStep, g_scale=1.0, clip_scale=None):
        """One launch over the whole parameter list; `clip_scale` is the device scalar written by
        clip_scale_dev (None: no clipping)."""
        dev, n, total = table
        self._own(clip_scale)
        self._check(self.lib.fb_adamw_multi_clipped(self._s(), dev.data_ptr(), n, total, self._hp(hp), g_scale,
                                                    clip_scale.ptr if clip_scale is not None else None))

    def sgd_multi_dev(self, table, lr, momentum, nesterov, g_scale=1.0, clip_scale=None):
        dev, n, total = table
        self._own(clip_scale)
        self._check(self.lib.fb_sgd_multi_clipped(self._s(), dev.data_ptr(), n, total, lr, momentum,
                                                  1 if nesterov else 0, g_scale,
                                                  clip_scale.ptr if clip_scale is not None else None))

    def clip_scale_dev(self, table, max_norm, g_scale=1.0):
        """Global-norm clipping for the gradients of `table` (optim.rs:1395-1425) with nothing read back:
        returns (norm, scale) as one-element device buffers; pass `scale` to the multi-tensor update."""
        dev, n, total = table
        sumsq, norm, scale = self._alloc(1), self._alloc(1), self._alloc(1)
        ws, nb = self._workspace(self.lib.fb_grad_norm_workspace_bytes())
        self._check(self.lib.fb_grad_sumsq_multi(self._s(), dev.data_ptr(), n, total, g_scale, sumsq.ptr, ws, nb))
        self._check(self.lib.fb_clip_scale(self._s(), sumsq.ptr, max_norm, norm.ptr, scale.ptr))
        return norm, scale

    # -- MLP glue -----------------------------------------------------------------------------------------
    ACTS = {"identity": 0, "relu": 1, "gelu": 2, "silu": 3}

    @classmethod
    def _act(cls, relu):
        """Activation code of bias_add_activation's Act (fused_ops.rs:10-16); True / False keep meaning relu / none."""
        if isinstance(relu, str):
            return cls.ACTS[relu]
        return 1 if relu else 0

    def bias_act_dev(self, x, bias, relu, rows, cols, out=None) -> DeviceBuffer:
        """act(x + bias); `relu` is True / False or one of "identity", "relu", "gelu", "silu"."""
        self._own(x, bias)
        self._rc(x, rows, cols)
        out = out or self._alloc(len(x))
        self._check(self.lib.fb_bias_act_fwd(self._s(), x.ptr, bias.ptr if bias else None, self._act(relu),
                                             rows, cols, out.ptr))
        return out

    def bias_act_backward_dev(self, g, x, bias, relu, rows, cols, dx=None, want_dx=True):
        """(dx | None, dbias)."""
        self._own(g, x, bias)
        self._rc(g, rows, cols)
        if want_dx and dx is None:
            dx = self._alloc(len(g))
        db = self._alloc(cols)
        ws, nb = self._workspace(self.lib.fb_reduce_dim_workspace_bytes(1, rows, cols))
        self._check(self.lib.fb_bias_act_bwd(self._s(), g.ptr, x.ptr if x is not None else None,
                                             bias.ptr if bias else None, self._act(relu), rows, cols,
                                             dx.ptr if dx is not None else None, db.ptr, ws, nb))
        return dx, db

    def mse_dev(self, pred, target, grad_scale=1.0, want_grad=True):
        """(loss[1], dpred | None): mse_loss forward and gradient in one pass."""
        self._own(pred, target)
        if len(pred) != len(target):
            raise InvalidShape("mse_dev: length mismatch")
        loss = self._alloc(1)
        dp = self._alloc(len(pred)) if want_grad else None
        ws, nb = self._workspace(self.lib.fb_reduce_workspace_bytes(len(pred)))
        self._check(self.lib.fb_mse_fwd_bwd(self._s(), pred.ptr, target.ptr, len(pred), grad_scale, loss.ptr,
                                            dp.ptr if dp else None, ws, nb))
        return loss, dp
