"""The checkpoint wire format (fb_safetensors_*, ferro_b200/checkpoint.py): byte-for-byte the layout of ferro's
to_safetensors_bytes (crates/ferro-core/src/safetensors.rs:36-94), interchangeable with the `safetensors`
package, strict about malformed images; on a GPU, optimizer state goes from device buffers to a file and back
without a host-side re-encode and a restored run continues bit-exactly."""
import json
import struct

import numpy as np
import pytest
import torch

from ferro_b200 import checkpoint as ck
from ferro_b200.backend import FerroError, FormatError


def expected_bytes(named):
    """The layout of safetensors.rs:36-94 written out independently."""
    header, data = "{", b""
    for i, (name, a) in enumerate(named):
        start = len(data)
        data += np.ascontiguousarray(a).tobytes()
        tag = "F32" if a.dtype == np.float32 else "I64"
        esc = "".join('\\"' if c == '"' else "\\\\" if c == "\\" else f"\\u{ord(c):04x}" if ord(c) < 0x20 else c for c in name)
        header += ("," if i else "") + f'"{esc}":{{"dtype":"{tag}","shape":[{",".join(str(d) for d in a.shape)}],"data_offsets":[{start},{len(data)}]}}'
    header += "}"
    while (8 + len(header.encode())) % 8:
        header += " "
    return struct.pack("<Q", len(header.encode())) + header.encode() + data


def test_host_image_is_byte_for_byte_ferros_layout_and_round_trips():
    r = np.random.default_rng(0)
    named = [("weight", r.standard_normal((3, 5)).astype(np.float32)), ("steps", np.arange(4, dtype=np.int64)),
             ("scalar", np.array(2.5, dtype=np.float32)), ('odd "name"\\with\ttab', r.standard_normal(7).astype(np.float32)),
             ("empty", np.zeros((0, 4), np.float32))]
    image = ck.to_safetensors_image([(n, torch.from_numpy(np.array(a))) for n, a in named])
    assert bytes(image.numpy()) == expected_bytes(named)
    back = ck.from_safetensors_image(image)
    assert [n for n, _ in back] == [n for n, _ in named]
    for (_, t), (_, a) in zip(back, named):
        assert t.shape == a.shape and (t.numpy() == a).all()


def test_interchange_with_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.numpy")
    r = np.random.default_rng(1)
    tensors = {"optim.m.0": r.standard_normal(12).astype(np.float32), "optim.v.0": r.random(12).astype(np.float32),
               "optim.t.0": np.array(3, dtype=np.float32), "ids": np.arange(5, dtype=np.int64)}
    # ours -> theirs
    ck.save_safetensors(str(tmp_path / "ours.safetensors"), [(k, torch.from_numpy(v)) for k, v in tensors.items()])
    theirs = st.load_file(str(tmp_path / "ours.safetensors"))
    assert set(theirs) == set(tensors) and all((theirs[k] == tensors[k]).all() for k in tensors)
    # theirs -> ours (their header carries __metadata__ and their own key order)
    st.save_file(tensors, str(tmp_path / "theirs.safetensors"), metadata={"format": "pt"})
    ours = dict(ck.load_safetensors(str(tmp_path / "theirs.safetensors")))
    assert set(ours) == set(tensors) and all((ours[k].numpy() == tensors[k]).all() for k in tensors)


def test_malformed_images_are_format_errors_with_a_message():
    good = ck.to_safetensors_image([("a", torch.arange(6, dtype=torch.float32))])
    raw = bytes(good.numpy())
    def img(b):
        return torch.from_numpy(np.frombuffer(b, dtype=np.uint8).copy())
    for bad, what in [(raw[:5], "shorter"), (struct.pack("<Q", 1 << 40) + raw[8:], "exceeds"),
                      (raw[:8] + raw[8:].replace(b'"F32"', b'"F3" '), None),
                      (raw[:8] + raw[8:].replace(b"[0,24]", b"[0,99]"), "outside"),
                      (raw[:8] + raw[8:].replace(b'"shape":[6]', b'"shape":[7]'), "bytes for"),
                      (raw[:8] + b"[" + raw[9:], "not a JSON object")]:
        with pytest.raises(FormatError) as e:
            ck.from_safetensors_image(img(bad))
        if what:
            assert what in str(e.value), (what, str(e.value))
    with pytest.raises(FerroError):
        ck.to_safetensors_image([("a", torch.zeros(2)), ("a", torch.zeros(2))])  # duplicate name (safetensors.rs:40-45)
    with pytest.raises(FerroError):
        ck.to_safetensors_image([("h", torch.zeros(2, dtype=torch.float16))])


def test_adam_state_names_and_strict_restore():
    p = [torch.zeros(2, 3), torch.zeros(4)]
    m = [torch.full_like(t, 0.5) for t in p]
    v = [torch.full_like(t, 0.25) for t in p]
    named = ck.adam_state(p, m, v, [7, 7])
    assert [n for n, _ in named] == ["optim.m.0", "optim.v.0", "optim.t.0", "optim.m.1", "optim.v.1", "optim.t.1"]
    assert named[0][1].shape == (6,) and named[2][1].shape == ()          # flat arrays and a scalar (optim.rs:839-846)
    back = dict(ck.from_safetensors_image(ck.to_safetensors_image(named)))
    m2, v2 = [torch.zeros_like(t) for t in p], [torch.zeros_like(t) for t in p]
    assert ck.restore_adam_state(back, p, m2, v2) == [7, 7]
    assert all(torch.equal(a, b) for a, b in zip(m + v, m2 + v2))
    del back["optim.v.1"]
    with pytest.raises(FormatError):
        ck.restore_adam_state(back, p, m2, v2)


@pytest.mark.gpu
def test_device_resident_training_state_checkpoints_and_resumes_bit_exactly(tmp_path):
    """Three Adam steps of the data-parallel MLP, a checkpoint of parameters + moments taken from the device
    buffers, two more steps; a second model restored from the file and given the same two steps ends on the same bits."""
    from ferro_b200.backend import CudaBackend
    from ferro_b200.ddp import DdpMlp
    be = CudaBackend(0)
    R, din, dh, dout = 128, 32, 64, 16
    gen = torch.Generator(device=be.device).manual_seed(5)
    with torch.cuda.stream(be.stream):
        x = torch.randn(R, din, device=be.device, generator=gen)
        y = torch.randn(R, dout, device=be.device, generator=gen)
    a = DdpMlp(be, din, dh, dout, R, seed=3)
    for _ in range(3):
        a.step(x, y)
    a.synchronize()
    names = ["W1", "b1", "W2", "b2"]
    state = [(f"model.{n}", p) for n, p in zip(names, a.params)] + ck.adam_state(
        a.params, [a.ddp.m[n] for n in names], [a.ddp.v[n] for n in names], [a.ddp.t] * 4)
    path = str(tmp_path / "step3.safetensors")
    ck.save_safetensors(path, state, stream=be.stream)
    for _ in range(2):
        a.step(x, y)
    a.synchronize()
    loaded = dict(ck.load_safetensors(path, device=be.device, stream=be.stream))
    assert all(t.is_cuda for t in loaded.values())
    b = DdpMlp(be, din, dh, dout, R, params=[loaded[f"model.{n}"] for n in names])
    steps = ck.restore_adam_state(loaded, b.params, [b.ddp.m[n] for n in names], [b.ddp.v[n] for n in names])
    assert steps == [3, 3, 3, 3]
    b.ddp.t = steps[0]
    for _ in range(2):
        b.step(x, y)
    b.synchronize()
    for p, q in zip(a.params, b.params):
        assert torch.equal(p, q)
