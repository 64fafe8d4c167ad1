"""DLPack exchange (fb_dlpack_*): descriptor rules on CPU, zero-copy export and on-device import on a GPU.

The CPU cases follow the reference's own unit tests of its importer
(crates/ferro-py/src/dlpack.rs:740-890: negative rank and extents, element-count
overflow, strides reaching outside the buffer, device type, dtype, null data,
the deleter running exactly once) and of its stream tokens
(crates/ferro-py/src/lib.rs:32-46).
"""
import ctypes as C

import numpy as np
import pytest

from ferro_b200 import _lib

i64 = C.c_int64


class DLDevice(C.Structure):
    _fields_ = [("device_type", C.c_int32), ("device_id", C.c_int32)]


class DLDataType(C.Structure):
    _fields_ = [("code", C.c_uint8), ("bits", C.c_uint8), ("lanes", C.c_uint16)]


class DLTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("device", DLDevice), ("ndim", C.c_int32), ("dtype", DLDataType),
                ("shape", C.POINTER(i64)), ("strides", C.POINTER(i64)), ("byte_offset", C.c_uint64)]


class DLManagedTensor(C.Structure):
    pass


DELETER = C.CFUNCTYPE(None, C.POINTER(DLManagedTensor))
DLManagedTensor._fields_ = [("dl_tensor", DLTensor), ("manager_ctx", C.c_void_p), ("deleter", DELETER)]


def fixture(shape, strides=None, data=0x1000, device_type=2, code=2, bits=32, lanes=1, byte_offset=0, ndim=None):
    """A hand-made DLManagedTensor (the pointer is never dereferenced by fb_dlpack_describe)."""
    n = len(shape)
    m = DLManagedTensor()
    m._shape = (i64 * max(n, 1))(*shape)
    m._strides = None if strides is None else (i64 * max(n, 1))(*strides)
    m.dl_tensor.data = data
    m.dl_tensor.device = DLDevice(device_type, 0)
    m.dl_tensor.ndim = n if ndim is None else ndim
    m.dl_tensor.dtype = DLDataType(code, bits, lanes)
    m.dl_tensor.shape = m._shape
    m.dl_tensor.strides = m._strides if m._strides is not None else C.POINTER(i64)()
    m.dl_tensor.byte_offset = byte_offset
    return m


def describe(lib, m):
    d = _lib.DlpackDesc()
    rc = lib.fb_dlpack_describe(C.byref(m), C.byref(d))
    return rc, d, lib.fb_last_error().decode()


def test_export_builds_a_cuda_descriptor_and_the_deleter_releases_the_owner_once():
    lib = _lib.load()
    calls = []

    @_lib.DLPACK_RELEASE_FN
    def release(owner):
        calls.append(int(owner))

    managed = C.c_void_p()
    shape, strides = (i64 * 2)(3, 5), (i64 * 2)(1, 3)
    assert lib.fb_dlpack_export(0x7000, 8, 0, 2, shape, strides, 3, 41, release, C.byref(managed)) == 0
    m = C.cast(managed, C.POINTER(DLManagedTensor)).contents
    t = m.dl_tensor
    assert (t.device.device_type, t.device.device_id) == (2, 3)           # kDLCUDA, ordinal passed through
    assert (t.dtype.code, t.dtype.bits, t.dtype.lanes) == (2, 32, 1)
    assert t.data == 0x7000 and t.byte_offset == 8 and t.ndim == 2
    assert [t.shape[0], t.shape[1]] == [3, 5] and [t.strides[0], t.strides[1]] == [1, 3]
    rc, d, _ = describe(lib, m)
    assert rc == 0 and d.data == 0x7008 and d.on_device == 1 and d.device_id == 3 and d.numel == 15 and d.contiguous == 0
    assert calls == []
    lib.fb_dlpack_delete(managed)
    assert calls == [41]
    # compact tensors carry no strides; i64 is the other dtype
    assert lib.fb_dlpack_export(0x7000, 0, 1, 1, (i64 * 1)(4), None, 0, None, _lib.DLPACK_RELEASE_FN(), C.byref(managed)) == 0
    m = C.cast(managed, C.POINTER(DLManagedTensor)).contents
    assert not m.dl_tensor.strides and (m.dl_tensor.dtype.code, m.dl_tensor.dtype.bits) == (0, 64)
    rc, d, _ = describe(lib, m)
    assert rc == 0 and d.contiguous == 1 and d.dtype == 1 and d.strides[0] == 1
    lib.fb_dlpack_delete(managed)
    # refused before anything is built
    for args, word in [((0x7000, 2, 0, 1, (i64 * 1)(4), None, 0), "aligned"), ((0x7000, 0, 2, 1, (i64 * 1)(4), None, 0), "dtype"),
                       ((0x7000, 0, 0, 1, (i64 * 1)(-4), None, 0), "negative"), ((None, 0, 0, 1, (i64 * 1)(4), None, 0), "null"),
                       ((0x7000, 0, 0, _lib.MAX_RANK + 1, (i64 * (_lib.MAX_RANK + 1))(*[1] * (_lib.MAX_RANK + 1)), None, 0), "rank")]:
        assert lib.fb_dlpack_export(*args, None, _lib.DLPACK_RELEASE_FN(), C.byref(managed)) != 0
        assert word in lib.fb_last_error().decode() and not managed.value


def test_describe_follows_the_reference_importers_rules():
    lib = _lib.load()
    rc, d, _ = describe(lib, fixture([2, 3]))
    assert rc == 0 and d.numel == 6 and d.contiguous == 1 and [d.strides[0], d.strides[1]] == [3, 1]
    # a transposed view reaches exactly the described span
    rc, d, _ = describe(lib, fixture([3, 2], strides=[1, 3]))
    assert rc == 0 and d.contiguous == 0
    for m, word in [
        (fixture([2, 3], ndim=-1), "negative ndim"),
        (fixture([2, -3]), "negative extent (-3) in dimension 1"),
        (fixture([1 << 40, 1 << 40]), "overflows"),
        (fixture([0, 1 << 40, 1 << 40]), "overflows"),                 # a zero axis does not mask the overflow
        (fixture([2, 3], strides=[4, 1]), "strides reach outside"),
        (fixture([2, 3], strides=[-3, 1]), "strides reach outside"),
        (fixture([2, 3], device_type=4), "kDLCUDA"),                    # kDLOneAPI
        (fixture([2, 3], code=2, bits=16), "unsupported DLPack dtype"),
        (fixture([2, 3], code=6, bits=8), "unsupported DLPack dtype"),
        (fixture([2, 3], data=None), "null data pointer"),
        (fixture([2, 3], byte_offset=2), "byte_offset is not element-aligned"),
        (fixture([2, 3], data=0x1002), "data pointer is not element-aligned"),
    ]:
        rc, _, msg = describe(lib, m)
        assert rc != 0 and word in msg, (word, msg)
    # an empty tensor has no reachable address: null data and any strides are fine
    rc, d, _ = describe(lib, fixture([0, 3], strides=[100, -7], data=None))
    assert rc == 0 and d.numel == 0 and not d.data


def test_stream_tokens_are_refused_like_ferro_without_touching_cuda():
    lib = _lib.load()
    for token, word in [(0, "ambiguous"), (-1, "no-sync (-1) is unsupported")]:
        assert lib.fb_dlpack_handoff(None, 1, token) == 2  # FB_ERR_INVALID_ARG
        assert word in lib.fb_last_error().decode()


@pytest.mark.gpu
def test_export_is_zero_copy_and_stream_ordered_and_import_stays_on_the_device():
    import torch
    from ferro_b200 import dlpack as fdl
    from ferro_b200.backend import CudaBackend, UnaryKind
    be = CudaBackend(0)
    r = np.random.default_rng(5)
    x = r.standard_normal((64, 96)).astype(np.float32)
    X = be.alloc_from_host(x.ravel())
    Y = be.unary_dev(UnaryKind.Exp, X)  # enqueued on the backend's stream, not waited for
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):  # the consumer passes its current stream to __dlpack__
        t = torch.from_dlpack(fdl.export(be, Y, (64, 96)))
        got = (t * 2).cpu().numpy()
    assert t.data_ptr() == Y.ptr and tuple(t.shape) == (64, 96) and t.device.index == 0
    np.testing.assert_allclose(got, 2 * np.exp(x), rtol=1e-5)
    assert fdl.outstanding() == 1
    del t
    import gc
    gc.collect()
    assert fdl.outstanding() == 0  # torch ran the deleter, the buffer is released
    # a view: rows 8.. of the buffer, transposed
    v = torch.from_dlpack(fdl.export(be, Y, (96, 56), strides=(1, 96), offset=8 * 96))
    torch.cuda.synchronize()
    np.testing.assert_allclose(v.cpu().numpy(), np.exp(x)[8:].T, rtol=1e-5)
    del v
    # an unconsumed capsule releases its tensor when it is dropped
    cap = fdl.export(be, Y, (64 * 96,)).__dlpack__()
    assert fdl.outstanding() == 1
    del cap
    gc.collect()
    assert fdl.outstanding() == 0
    # import: compact, transposed (gathered by the strided-copy kernel), i64; nothing goes through the host
    src = torch.randn(40, 72, device="cuda:0")
    for view in (src, src.t(), src.reshape(8, 5, 72).permute(2, 0, 1), src.unsqueeze(1)):
        buf, shape = fdl.from_dlpack(be, view)
        assert shape == list(view.shape)
        np.testing.assert_array_equal(be.copy_to_host(buf).reshape(shape), view.cpu().numpy())
    idx = torch.arange(1000, device="cuda:0") * 3
    buf, shape = fdl.from_dlpack(be, idx)
    be.synchronize()
    assert buf.is_i64 and shape == [1000] and torch.equal(buf.t, idx)
    fdl.release_imports()  # every imported tensor goes back to its producer once its copy has run
    for bad in (src[:, ::2], src[:, :1]):  # views that reach outside their own element count: refused, as in ferro
        with pytest.raises(Exception):
            fdl.from_dlpack(be, bad)
    with pytest.raises(Exception):
        fdl.from_dlpack(be, src.double())
    with pytest.raises(Exception):
        fdl.export(be, Y, (64, 96)).__dlpack__(stream=0)
    assert fdl.outstanding() == 0
