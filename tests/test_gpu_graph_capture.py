"""The library's launch path inside a CUDA graph.

ferro records its fused training steps into CUDA graphs (the capturable AdamW with a device-side
step counter exists for that: crates/ferro-cuda/src/kernels.rs:489-530).  Every entry of the
library promises the same: no allocation, no synchronisation and no module load on the launch path.
Here a step made of the kernels with the least ordinary launches - programmatic dependent launches
(LayerNorm backward + finalize, softmax), thread block cluster launches sized by an occupancy query
(wide LayerNorm backward, wide softmax forward and backward), the capturable AdamW - is captured once
and replayed on new inputs; the replays must equal eager calls on the same inputs bit for bit.
"""
import ctypes as C

import pytest
import torch

from ferro_b200.backend import CudaBackend

pytestmark = pytest.mark.gpu


def _p(t):
    return C.c_void_p(t.data_ptr())


def test_a_step_with_pdl_and_cluster_launches_replays_from_a_cuda_graph():
    be = CudaBackend(0)
    lib, s, dev = be.lib, be._s(), be.device
    gen = torch.Generator(device=dev).manual_seed(3)
    shapes = [(512, 4096), (96, 32768)]  # staged backward + dependent finalize; cluster backward and cluster softmax
    with torch.cuda.stream(be.stream):
        bufs = []
        for rows, cols in shapes:
            x = torch.randn(rows, cols, device=dev, generator=gen)
            g = torch.randn(rows, cols, device=dev, generator=gen)
            w = 1 + 0.1 * torch.randn(cols, device=dev, generator=gen)
            b = 0.1 * torch.randn(cols, device=dev, generator=gen)
            out = {k: torch.empty(rows, cols, device=dev) for k in ("y", "dx", "sm", "dsm")}
            out.update({k: torch.empty(rows, device=dev) for k in ("mu", "rs")})
            out.update({k: torch.empty(cols, device=dev) for k in ("dw", "db")})
            ws = torch.empty(int(lib.fb_layer_norm_bwd_workspace_bytes(rows, cols)) + 16, dtype=torch.uint8, device=dev)
            bufs.append((rows, cols, x, g, w, b, out, ws))
        n = 100003
        p, m, v = torch.randn(n, device=dev, generator=gen), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        grad = torch.randn(n, device=dev, generator=gen)
        t = torch.zeros(3, device=dev)

    def step():
        for rows, cols, x, g, w, b, o, ws in bufs:
            be._check(lib.fb_layer_norm_fwd(s, _p(x), _p(w), _p(b), rows, cols, 1e-5, _p(o["y"]), None, None, _p(o["mu"]), _p(o["rs"])))
            be._check(lib.fb_layer_norm_bwd(s, _p(g), None, None, _p(x), _p(o["mu"]), _p(o["rs"]), _p(w), rows, cols, _p(o["dx"]),
                                            _p(o["dw"]), _p(o["db"]), _p(ws), ws.numel()))
            be._check(lib.fb_softmax_fwd(s, _p(o["y"]), rows, cols, _p(o["sm"])))
            be._check(lib.fb_softmax_bwd(s, _p(g), _p(o["sm"]), rows, cols, _p(o["dsm"])))
        be._check(lib.fb_scalar_increment(s, _p(t), 0.9, 0.999))
        be._check(lib.fb_adamw_step_capturable(s, _p(p), _p(m), _p(v), _p(grad), _p(t), n, 1e-3, 0.9, 0.999, 1e-8, 0.01))

    def snapshot():
        be.synchronize()
        outs = [o[k].clone() for *_, o, _ws in bufs for k in ("y", "dx", "sm", "dsm", "mu", "rs", "dw", "db")]
        return outs + [p.clone(), m.clone(), v.clone(), t.clone()]

    def reset_state(state):
        with torch.cuda.stream(be.stream):
            for dst, src in zip((p, m, v, t), state):
                dst.copy_(src)

    state0 = [z.clone() for z in (p, m, v, t)]
    step()  # warm-up: first-use attribute calls and occupancy queries happen outside the capture
    be.synchronize()
    reset_state(state0)
    be.synchronize()
    launches0 = lib.fb_launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=be.stream):
        step()
    captured = lib.fb_launch_count() - launches0
    assert captured >= 11  # every entry enqueued its kernels into the capture instead of failing or running eagerly
    reset_state(state0)
    be.synchronize()
    for trial in range(2):
        # new inputs in place, then one replay against one eager step from the same state
        with torch.cuda.stream(be.stream):
            for rows, cols, x, g, w, b, o, ws in bufs:
                x.normal_(generator=gen)
                g.normal_(generator=gen)
            grad.normal_(generator=gen)
        be.synchronize()
        before = [z.clone() for z in (p, m, v, t)]
        graph.replay()
        torch.cuda.synchronize()
        from_graph = snapshot()
        reset_state(before)
        be.synchronize()
        step()
        eager = snapshot()
        for a, e in zip(from_graph, eager):
            assert torch.equal(a, e), f"replay {trial} differs from the eager step"
    assert lib.fb_device_faults(0) == 0
