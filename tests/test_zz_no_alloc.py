"""The allocation-free LayerNorm backward (fb_layer_norm_bwd_static).

Some callers have no way to pass device scratch: their memory pool is frozen
for the duration of a step, or the allocator lives on the other side of a
plug-in boundary.  For them the library keeps the scratch in a fixed device
array of its own.  This test drives that entry point through the C ABI and
checks it against the ordinary entry point (caller scratch) on the same
inputs, twice in a row with different data, so that anything the shared array
keeps from the first call would show up in the second.  The file sorts last so
a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def test_static_scratch_backward_matches_caller_scratch_backward_twice():
    from ferro_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev)
    s = C.c_void_p(stream.cuda_stream)
    gen = torch.Generator(device=dev).manual_seed(7)
    for call, (rows, cols) in enumerate([(4096, 4096), (1500, 1000), (333, 517)]):
        x = torch.randn(rows, cols, device=dev, generator=gen) * 3 + call
        g = torch.randn(rows, cols, device=dev, generator=gen)
        w = 1 + 0.02 * torch.randn(cols, device=dev, generator=gen)
        y, mean, rstd = torch.empty_like(x), torch.empty(rows, device=dev), torch.empty(rows, device=dev)
        assert lib.fb_layer_norm_fwd(s, _ptr(x), _ptr(w), None, rows, cols, 1e-5, _ptr(y), None, None,
                                     _ptr(mean), _ptr(rstd)) == 0, lib.fb_last_error()
        # Reference result: the existing entry point with scratch the caller allocated.
        need = lib.fb_layer_norm_bwd_workspace_bytes(rows, cols)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
        dx0, dw0, db0 = torch.empty_like(x), torch.empty(cols, device=dev), torch.empty(cols, device=dev)
        assert lib.fb_layer_norm_bwd(s, _ptr(g), None, None, _ptr(x), _ptr(mean), _ptr(rstd), _ptr(w), rows, cols,
                                     _ptr(dx0), _ptr(dw0), _ptr(db0), _ptr(ws), ws.numel()) == 0, lib.fb_last_error()
        # The entry point under test: outputs poisoned first, no scratch argument at all.
        dx1 = torch.full_like(x, float("nan"))
        dw1 = torch.full((cols,), float("nan"), device=dev)
        db1 = torch.full((cols,), float("nan"), device=dev)
        torch.cuda.synchronize()
        if call == 0:
            # First use on this device: the one-time look-up of the array's address happens here,
            # outside the window in which free device memory is watched.
            assert lib.fb_layer_norm_bwd_static(s, _ptr(g), None, None, _ptr(x), _ptr(mean), _ptr(rstd), _ptr(w), rows,
                                                cols, _ptr(dx1), _ptr(dw1), _ptr(db1)) == 0, lib.fb_last_error()
            torch.cuda.synchronize()
            dx1.fill_(float("nan"))
            dw1.fill_(float("nan"))
            db1.fill_(float("nan"))
            torch.cuda.synchronize()
        # Free device memory as the driver sees it (not only torch's allocator): an allocation made
        # inside the library by any route would show here.
        before_torch, before_free = torch.cuda.memory_allocated(dev), torch.cuda.mem_get_info(dev)[0]
        assert lib.fb_layer_norm_bwd_static(s, _ptr(g), None, None, _ptr(x), _ptr(mean), _ptr(rstd), _ptr(w), rows,
                                            cols, _ptr(dx1), _ptr(dw1), _ptr(db1)) == 0, lib.fb_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before_torch
        assert torch.cuda.mem_get_info(dev)[0] == before_free
        # Same kernels, same summation order: the results are identical, which is
        # inside the 2e-4 relative bar the LayerNorm parity tests use.
        for a, b, name in ((dx1, dx0, "dx"), (dw1, dw0, "dweight"), (db1, db0, "dbias")):
            a, b = a.cpu().numpy(), b.cpu().numpy()
            assert not np.isnan(a).any(), name
            err = np.abs(a.astype(np.float64) - b)
            assert (err <= 2e-4 * np.abs(b) + 1e-12).all(), (call, name, float(err.max()))
            assert (a.view(np.uint32) == b.view(np.uint32)).all(), (call, name)
        if call == 2:
            # ... and against the CPU oracle directly on the smallest shape (2e-4 relative, as every LayerNorm test).
            import oracle as fo
            xh, gh, wh = x.cpu().numpy(), g.cpu().numpy(), w.cpu().numpy()
            _, hh, sh, _ = fo.layer_norm_fwd(xh, wh, None, 1e-5)
            dxw, dww, dbw = fo.layer_norm_bwd(gh, hh, sh, wh)
            for got, want, scale, name in ((dx1, dxw, np.abs(dxw).max(), "dx"), (dw1, dww, np.abs(gh * hh).sum(0).max(), "dweight"),
                                           (db1, dbw, np.abs(gh).sum(0).max(), "dbias")):
                err = np.abs(got.cpu().numpy().astype(np.float64) - want)
                assert (err <= 2e-4 * np.abs(want) + 2e-4 * scale).all(), name
        # The saved (h, stds) form and a call that asks for dx only go through the same entry.
        h, stds = torch.empty_like(x), torch.empty(rows, device=dev)
        assert lib.fb_layer_norm_fwd(s, _ptr(x), _ptr(w), None, rows, cols, 1e-5, _ptr(y), _ptr(h), _ptr(stds), None, None) == 0
        dx2, dw2, db2 = torch.full_like(x, float("nan")), torch.empty(cols, device=dev), torch.empty(cols, device=dev)
        dx3 = torch.full_like(x, float("nan"))
        assert lib.fb_layer_norm_bwd(s, _ptr(g), _ptr(h), _ptr(stds), None, None, None, _ptr(w), rows, cols,
                                     _ptr(dx2), _ptr(dw2), _ptr(db2), _ptr(ws), ws.numel()) == 0, lib.fb_last_error()
        dw3, db3 = torch.empty(cols, device=dev), torch.empty(cols, device=dev)
        assert lib.fb_layer_norm_bwd_static(s, _ptr(g), _ptr(h), _ptr(stds), None, None, None, _ptr(w), rows, cols,
                                            _ptr(dx3), _ptr(dw3), _ptr(db3)) == 0, lib.fb_last_error()
        dx4 = torch.full_like(x, float("nan"))
        assert lib.fb_layer_norm_bwd_static(s, _ptr(g), None, None, _ptr(x), _ptr(mean), _ptr(rstd), _ptr(w), rows, cols,
                                            _ptr(dx4), None, None) == 0, lib.fb_last_error()
        torch.cuda.synchronize()
        assert torch.equal(dx3, dx2) and torch.equal(dw3, dw2) and torch.equal(db3, db2)
        assert torch.equal(dx4, dx0)


def test_static_scratch_refuses_problems_beyond_its_fixed_size():
    from ferro_b200 import _lib
    lib = _lib.load()
    rows, cols = 1 << 20, 32768  # needs far more partial-sum space than the built-in 16 MiB
    assert lib.fb_layer_norm_bwd_workspace_bytes(rows, cols) > (16 << 20)
    one = torch.zeros(1, device="cuda:0")
    rc = lib.fb_layer_norm_bwd_static(None, _ptr(one), None, None, _ptr(one), _ptr(one), _ptr(one), None, rows, cols,
                                      _ptr(one), _ptr(one), _ptr(one))
    assert rc == 5  # FB_ERR_WORKSPACE, nothing launched
    assert b"built-in" in lib.fb_last_error()
    # A dx-only call on a shape that has no fused form (width not a multiple of 4) needs the per-row
    # statistics of the two-kernel form: beyond the fixed size it is refused by this entry, with its own message.
    rows, cols = 1 << 22, 1001
    assert lib.fb_layer_norm_bwd_workspace_bytes(rows, cols) > (16 << 20)
    rc = lib.fb_layer_norm_bwd_static(None, _ptr(one), None, None, _ptr(one), _ptr(one), _ptr(one), None, rows, cols,
                                      _ptr(one), None, None)
    assert rc == 5 and b"built-in" in lib.fb_last_error()
