"""Extract the golden tables of ferro's own test-suite that pin the hot path.

Run once, in a checkout that has the ferro sources next to it:

    python tests/golden/make_golden.py /path/to/ferro

It reads ferro's test fixtures AS TEXT (nothing is compiled or executed) and
writes tests/golden/reference_fixtures.json, which the CPU tests compare the
oracle against.  Tables taken:

* crates/ferro-core/tests/fixtures/clamp_bounds_goldens.rs  INPUT32 / CLAMP32
  (torch scalar-bound clamp bits; consumed by tests/clamp_bounds.rs:15-18)
* crates/ferro-core/tests/fixtures/power_special_reference.rs  FORWARD / BACKWARD
  rows with wide == false (f32 `powf` for p in {-2,-1,2,3}; consumed by
  tests/power_special.rs:22-51)

* crates/ferro-core/tests/fixtures/physical2_layernorm_goldens.rs  the rows with
  physical == false, one seeded input (mask 1, 2 or 4), gradients disabled:
  torch's forward-mode tangents of layer_norm for the inputs built in
  tests/physical_saved_stats.rs:16-27.  The tangent for a seed on the weight is
  seed * h (pins the normalised values of the forward), for a seed on x it is
  weight * (t - mean(t) - h * mean(t * h)) / std (the dx formula of the backward
  with g = t and no weight), for a seed on the bias it is the seed itself.

Not taken: adam_f64_goldens.rs and sgd_f64_goldens.rs hold f64 bit patterns only
(ferro's typed f64 optimizer path); the f32 kernels have no rows there.
crates/ferro-core/tests/fixtures/scalar_power_reference.rs is not taken: every
finite exponent in it is deliberately not an exact f32, so those rows go
through ferro's host f64 path (src/ops_ext/powf.rs:16-27), not UnaryKind::Powf.
"""
import json
import os
import re
import sys


def _read(root, rel):
    with open(os.path.join(root, rel)) as f:
        return f.read()


def clamp32(root):
    src = _read(root, "crates/ferro-core/tests/fixtures/clamp_bounds_goldens.rs")
    inp = re.search(r"INPUT32: &\[u32\] = &\[([^\]]*)\]", src).group(1)
    inputs = [int(t, 16) for t in inp.split(",") if t.strip()]
    block = src[src.index("const CLAMP32"):src.index("const INPUT64")]
    cases = []
    for m in re.finditer(r"\((0x[0-9a-f]+),(0x[0-9a-f]+),&\[([^\]]*)\]\)", block):
        cases.append({"min": int(m.group(1), 16), "max": int(m.group(2), 16),
                      "expected": [int(t, 16) for t in m.group(3).split(",") if t.strip()]})
    return {"input_bits": inputs, "cases": cases}


def power_special(root):
    src = _read(root, "crates/ferro-core/tests/fixtures/power_special_reference.rs")
    fwd_block = src[src.index("const FORWARD"):src.index("const BACKWARD")]
    bwd_block = src[src.index("const BACKWARD"):]
    fwd = [{"p": float(m.group(1)), "x": int(m.group(2)), "y": int(m.group(3))}
           for m in re.finditer(r"\(false,([-0-9.eE]+),(\d+),(\d+)\)", fwd_block)]
    bwd = [{"p": float(m.group(1)), "x": int(m.group(2)), "g": int(m.group(3)), "dx": int(m.group(4))}
           for m in re.finditer(r"\(false,([-0-9.eE]+),(\d+),(\d+),(\d+)\)", bwd_block)]
    return {"forward": fwd, "backward": bwd}


def layernorm_tangents(root):
    src = _read(root, "crates/ferro-core/tests/fixtures/physical2_layernorm_goldens.rs")
    out = {}
    for m in re.finditer(r"Golden \{ physical: false, mask: (\d), enabled: false, live: false, seed_live: false, "
                         r"requires: false, values: &\[([^\]]*)\]", src):
        mask = int(m.group(1))
        if mask in (1, 2, 4):
            out[str(mask)] = [float(t.replace("f32", "")) for t in m.group(2).split(",") if t.strip()]
    return out


def main():
    root = sys.argv[1]
    out = {
        "source": "ferro test fixtures, read as text by tests/golden/make_golden.py",
        "clamp32": clamp32(root),
        "power_special_f32": power_special(root),
        "layernorm_tangents": layernorm_tangents(root),
    }
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_fixtures.json")
    with open(dst, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print(dst, {k: (len(v) if isinstance(v, list) else {kk: len(vv) for kk, vv in v.items()})
                for k, v in out.items() if k != "source"})


if __name__ == "__main__":
    main()
