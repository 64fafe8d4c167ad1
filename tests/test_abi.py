"""CPU checks of the drop-in boundary: the C-ABI library loads, exports every
symbol include/ferro_b200.h declares, and rejects bad requests before any
launch (no compute happens here)."""
import ctypes as C
import os
import re

import pytest

from ferro_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ferro_b200.h")).read()
    return sorted(set(re.findall(r"FB_API\s+[\w\s\*]+?\b(fb_\w+)\s*\(", text)))


def test_header_declares_what_the_binding_binds():
    assert declared_symbols() == sorted(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert lib.fb_version() == 1


def test_entry_points_cite_the_reference_interface_they_replace():
    text = open(os.path.join(ROOT, "include", "ferro_b200.h")).read()
    # Every trait method on the hot path is named next to its replacement.
    for method in ["unary_dev", "binary_dev", "binary_bc_dev", "chain_dev", "reduce_dev", "sum_dim_dev",
                   "softmax_dev", "log_softmax_dev", "layer_norm_dev", "layer_norm_output_dev", "fill_dev",
                   "affine_inplace_dev", "binary_inplace_dev", "axpy_inplace_dev", "copy_into_dev",
                   "sgd_step_dev", "adamw_step_dev", "adamw_step_capturable_dev", "scalar_increment_dev",
                   "materialize_dev", "gather_rows_dev"]:
        assert method in text, method
    assert "dispatch.rs" in text and "lib.rs" in text


def test_bad_requests_fail_before_launch_with_a_message(lib):
    # Unknown kind, zero cols for LayerNorm, overflowing sizes, mixed LN backward operands:
    # all are rejected on the host, so they are safe without a GPU.
    assert lib.fb_unary(None, 99, 0.0, 0.0, None, None, 4) == 2
    assert b"unknown kind" in lib.fb_last_error()
    assert lib.fb_layer_norm_fwd(None, None, None, None, 2, 0, 1e-5, None, None, None, None, None) == 1
    assert b"nonempty" in lib.fb_last_error()
    big = (1 << 63)
    assert lib.fb_layer_norm_fwd(None, None, None, None, big, 4, 1e-5, None, None, None, None, None) == 1
    assert lib.fb_softmax_fwd(None, None, big, 8, None) == 1
    assert lib.fb_sum_dim(None, None, big, 4, 2, None, None, 0) == 1
    assert lib.fb_layer_norm_bwd(None, None, None, None, None, None, None, None, 2, 4, None, None, None, None, 0) == 2
    assert lib.fb_max_dim(None, None, 2, 0, 3, None, None, None, 0) == 1
    assert b"empty dimension" in lib.fb_last_error()


def test_zero_length_problems_succeed_without_a_device(lib):
    assert lib.fb_unary(None, 0, 0.0, 0.0, None, None, 0) == 0
    assert lib.fb_binary(None, 0, 0.0, 0.0, None, None, None, 0) == 0
    assert lib.fb_softmax_fwd(None, None, 0, 16, None) == 0
    assert lib.fb_layer_norm_fwd(None, None, None, None, 0, 3, 1e-5, None, None, None, None, None) == 0
    assert lib.fb_adamw_step(None, None, None, None, None, 0, _lib.AdamWHparams()) == 0
    assert lib.fb_sum_dim(None, None, 0, 4, 2, None, None, 0) == 0


def test_chain_program_validation(lib):
    S, O = _lib.ChainStep, _lib.ChainOperand
    shape = (C.c_uint64 * 1)(4)
    ops = (O * 1)()
    ops[0] = O(0x1000, 4, 0, (C.c_int64 * 16)(1))
    # reads T before it is written
    prog = (S * 2)(S(0, 0, 0, 0, 0, 0), S(2, 0, 0, 0, 0, 0))
    assert lib.fb_chain(None, prog, 2, ops, 1, shape, 1, 0x2000) == 2
    assert b"before it is written" in lib.fb_last_error()
    # operand index out of range
    prog = (S * 1)(S(0, 0, 0, 3, 0, 0))
    assert lib.fb_chain(None, prog, 1, ops, 1, shape, 1, 0x2000) == 2
    # view reaches outside its storage
    ops[0] = O(0x1000, 4, 1, (C.c_int64 * 16)(1))
    prog = (S * 1)(S(0, 0, 0, 0, 0, 0))
    assert lib.fb_chain(None, prog, 1, ops, 1, shape, 1, 0x2000) == 1
    assert b"outside its storage" in lib.fb_last_error()
    # shapes that do not broadcast
    sa, sb, so = (C.c_uint64 * 2)(2, 3), (C.c_uint64 * 1)(4), (C.c_uint64 * 2)(2, 3)
    assert lib.fb_binary_bc(None, 0, 0.0, 0.0, 0x1000, sa, 2, 0x1000, sb, 1, 0x2000, so, 2) == 1


def test_workspace_queries_are_consistent(lib):
    assert lib.fb_layer_norm_bwd_workspace_bytes(0, 8) == 0
    assert lib.fb_layer_norm_bwd_workspace_bytes(32768, 4096) % (2 * 4096 * 4) == 0
    assert lib.fb_nll_workspace_bytes(16384) >= 16384 * 4
    assert lib.fb_reduce_workspace_bytes(0) == 0
    assert lib.fb_reduce_dim_workspace_bytes(1, 8192, 1024) > 0
    assert lib.fb_reduce_dim_workspace_bytes(131072, 2048, 1) == 0


def test_manifest_helper_reproduces_a_line_of_the_chain_manifest():
    """`python -m ferro_b200.chain_manifest` writes what csrc/chain_programs.def holds for the gate-clamp chain."""
    import subprocess
    import sys
    out = subprocess.run([sys.executable, "-m", "ferro_b200.chain_manifest"], capture_output=True, text=True, cwd=ROOT, check=True).stdout
    manifest = open(os.path.join(ROOT, "ferro_b200", "csrc", "chain_programs.def")).read()
    squeeze = lambda t: re.sub(r"\s+", "", t)
    for line in out.strip().splitlines():
        if line.startswith("FB_CHAIN"):
            assert squeeze(line) in squeeze(manifest), line


def test_rust_bindings_follow_the_header():
    """include/ferro_b200_sys.rs is what `python -m ferro_b200.rust_bindings` prints today, declares every entry of
    the header exactly once, and lays its structs out like the ctypes binding does."""
    from ferro_b200 import rust_bindings
    committed = open(os.path.join(ROOT, "include", "ferro_b200_sys.rs")).read()
    assert committed == rust_bindings.generate()
    names = re.findall(r"pub fn (fb_\w+)\(", committed)
    assert sorted(names) == sorted(_lib.SIGNATURES) and len(set(names)) == len(names)
    # argument counts agree with the ctypes signatures
    for name, args in re.findall(r"pub fn (fb_\w+)\((.*?)\)(?: -> [^;]+)?;", committed):
        n_rust = 0 if not args.strip() else args.count(":")
        assert n_rust == len(_lib.SIGNATURES[name][1]), name
    # struct fields: same count as the ctypes mirrors
    for rust_name, ctypes_struct in [("ChainStep", _lib.ChainStep), ("ChainOperand", _lib.ChainOperand), ("View", _lib.ViewDesc),
                                     ("TensorQuad", _lib.TensorQuad), ("StEntry", _lib.StEntry), ("DlpackDesc", _lib.DlpackDesc),
                                     ("Rng", _lib.RngState), ("AdamwHparams", _lib.AdamWHparams)]:
        body = re.search(rf"pub struct {rust_name} \{{(.*?)\n\}}", committed, flags=re.S).group(1)
        assert body.count("pub ") == len(ctypes_struct._fields_), rust_name
