"""The host-buffer LayerNorm entry (fb_host_ln_*): host pointers in, host pointers out, the chunked
upload / compute / download pipeline inside the library.  Checked against the CPU oracle and against
the resident kernels, twice in a row with different data (the handle and its staging are reused)."""
import numpy as np
import pytest
import torch

import oracle as fo

pytestmark = pytest.mark.gpu


def test_host_layer_norm_matches_the_oracle_and_the_resident_path():
    from ferro_b200.backend import CudaBackend
    from ferro_b200.host_api import HostLayerNorm
    be = CudaBackend(0)
    rows, cols, eps = 512, 1000, 1e-5
    hln = HostLayerNorm(be, rows, cols, eps, chunks=4)
    pin = lambda *s: torch.empty(*s, dtype=torch.float32).pin_memory()
    y, dx, mu, rs, dwb = pin(rows, cols), pin(rows, cols), pin(rows), pin(rows), pin(2 * cols)
    for seed in (0, 1):
        r = fo.Rng(seed)
        x = torch.from_numpy(r.fill_rowscaled_normal(rows, cols)).pin_memory()
        w = torch.from_numpy(r.fill_normal((cols,), 0.02, 1.0)).pin_memory()
        b = torch.from_numpy(r.fill_normal((cols,), 0.02, 0.0)).pin_memory()
        g = torch.from_numpy(r.fill_normal((rows, cols))).pin_memory()
        y.fill_(float("nan")); dx.fill_(float("nan")); dwb.fill_(float("nan"))
        hln(x, g, w, b, y, dx, mu, rs, dwb)
        hln.synchronize()
        yw, hw, sw, mw = fo.layer_norm_fwd(x.numpy(), w.numpy(), b.numpy(), eps)
        dxw, dww, dbw = fo.layer_norm_bwd(g.numpy(), hw, sw, w.numpy())

        def close(got, want, scale, what):
            err = np.abs(np.asarray(got, np.float64) - want)
            assert (err <= 2e-4 * np.abs(want) + 2e-4 * scale).all(), (seed, what, float(err.max()))

        close(y.numpy(), yw, 1e-2, "y")
        close(mu.numpy(), mw, np.abs(x.numpy()).mean(), "mean")
        close(rs.numpy(), 1 / sw.astype(np.float64), 0, "rstd")
        close(dx.numpy(), dxw, np.abs(dxw).max(), "dx")
        close(dwb.numpy()[:cols], dww, np.abs(g.numpy() * hw).sum(0).max(), "dgamma")
        close(dwb.numpy()[cols:], dbw, np.abs(g.numpy()).sum(0).max(), "dbeta")
        # the same rows through the resident kernels: identical y and dx (same kernels per chunk)
        X, W, B, G = (be.alloc_from_host(t.numpy()) for t in (x, w, b, g))
        Y, MU, RS = be.layer_norm_stats_dev(X, W, B, rows, cols, eps)
        DX, _, _ = be.layer_norm_backward_dev(G, W, rows, cols, x=X, mean=MU, rstd=RS)
        assert (be.copy_to_host(Y).reshape(rows, cols) == y.numpy()).all()
        assert (be.copy_to_host(DX).reshape(rows, cols) == dx.numpy()).all()
    # bad requests are refused before anything is enqueued
    assert be.lib.fb_host_ln_device_bytes(513, cols, 4) == 0          # rows do not divide into the chunks
    with pytest.raises(ValueError):
        HostLayerNorm(be, 513, cols, eps, chunks=4)
    hln.close()
