"""ctypes binding of libferro_b200.so (the C ABI declared in include/ferro_b200.h).

There is no fallback: if the shared library is missing, loading raises.  Build
it with `python -m ferro_b200.build`.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libferro_b200.so")

MAX_RANK = 16
CHAIN_MAX_STEPS = 32
CHAIN_MAX_OPERANDS = 6
DDP_UNIQUE_ID_BYTES = 128

c_f32p = C.c_void_p  # device pointers travel as integers
c_i64p = C.c_void_p
c_stream = C.c_void_p
u64 = C.c_uint64
i64 = C.c_int64
f32 = C.c_float
u64p = C.POINTER(C.c_uint64)
i64p = C.POINTER(C.c_int64)


class AdamWHparams(C.Structure):
    """fb_adamw_hparams == ferro's AdamWStep (crates/ferro-core/src/dispatch.rs:92-100)."""
    _fields_ = [("lr", f32), ("beta1", f32), ("beta2", f32), ("bc1", f32), ("bc2", f32),
                ("eps", f32), ("weight_decay", f32)]


class ChainStep(C.Structure):
    _fields_ = [("opcode", C.c_int32), ("dst", C.c_int32), ("kind", C.c_int32), ("src", C.c_int32),
                ("p0", f32), ("p1", f32)]


class ChainOperand(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("len", u64), ("offset", i64), ("strides", i64 * MAX_RANK)]


class StEntry(C.Structure):
    """fb_st_entry: one tensor of a safetensors image."""
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_int32), ("rank", C.c_int32), ("shape", u64 * MAX_RANK)]


class DlpackDesc(C.Structure):
    """fb_dlpack_desc: what fb_dlpack_describe reports about a DLManagedTensor."""
    _fields_ = [("data", C.c_void_p), ("on_device", C.c_int32), ("device_id", C.c_int32), ("dtype", C.c_int32),
                ("rank", C.c_int32), ("contiguous", C.c_int32), ("reserved", C.c_int32), ("numel", u64),
                ("shape", u64 * MAX_RANK), ("strides", i64 * MAX_RANK)]


DLPACK_RELEASE_FN = C.CFUNCTYPE(None, C.c_void_p)


class ViewDesc(C.Structure):
    """fb_view: a ferro tensor view (crates/ferro-core/src/tensor.rs:213-227)."""
    _fields_ = [("ptr", C.c_void_p), ("len", u64), ("offset", i64), ("rank", C.c_int32),
                ("shape", u64 * MAX_RANK), ("strides", i64 * MAX_RANK)]


class RngState(C.Structure):
    """fb_rng == the two state words of ferro's Rng (crates/ferro-core/src/rng.rs:6-9)."""
    _fields_ = [("s0", u64), ("s1", u64)]


class TensorQuad(C.Structure):
    _fields_ = [("p", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p),
                ("n", u64)]


# name -> (restype, argtypes); kept in one table so the symbol test can walk it.
SIGNATURES = {
    "fb_version": (C.c_int, []),
    "fb_last_error": (C.c_char_p, []),
    "fb_launch_count": (u64, []),
    "fb_device_faults": (C.c_int, [C.c_int]),
    "fb_selftest_bounded_wait": (C.c_int, [c_stream, C.c_uint32]),
    "fb_unary": (C.c_int, [c_stream, C.c_int, f32, f32, c_f32p, c_f32p, u64]),
    "fb_binary": (C.c_int, [c_stream, C.c_int, f32, f32, c_f32p, c_f32p, c_f32p, u64]),
    "fb_binary_bc": (C.c_int, [c_stream, C.c_int, f32, f32, c_f32p, u64p, C.c_int, c_f32p, u64p,
                               C.c_int, c_f32p, u64p, C.c_int]),
    "fb_unary_strided": (C.c_int, [c_stream, C.c_int, f32, f32, c_f32p, u64, i64p, i64, u64p,
                                   C.c_int, c_f32p]),
    "fb_binary_strided": (C.c_int, [c_stream, C.c_int, f32, f32, c_f32p, u64, i64p, i64, c_f32p,
                                    u64, i64p, i64, u64p, C.c_int, c_f32p]),
    "fb_materialize": (C.c_int, [c_stream, c_f32p, u64, i64p, i64, u64p, C.c_int, c_f32p]),
    "fb_chain": (C.c_int, [c_stream, C.POINTER(ChainStep), C.c_int, C.POINTER(ChainOperand),
                           C.c_int, u64p, C.c_int, c_f32p]),
    "fb_chain_catalogue": (C.c_int, [C.c_int]),
    "fb_fill": (C.c_int, [c_stream, c_f32p, f32, u64]),
    "fb_affine_inplace": (C.c_int, [c_stream, c_f32p, f32, f32, u64]),
    "fb_binary_inplace": (C.c_int, [c_stream, C.c_int, c_f32p, c_f32p, u64]),
    "fb_axpy_inplace": (C.c_int, [c_stream, f32, c_f32p, c_f32p, u64]),
    "fb_copy": (C.c_int, [c_stream, c_f32p, c_f32p, u64]),
    "fb_gather_rows": (C.c_int, [c_stream, c_f32p, c_i64p, u64, u64, u64, c_f32p, c_i64p]),
    "fb_reduce_workspace_bytes": (u64, [u64]),
    "fb_reduce": (C.c_int, [c_stream, C.c_int, c_f32p, u64, c_f32p, C.c_void_p, u64]),
    "fb_reduce_dim_workspace_bytes": (u64, [u64, u64, u64]),
    "fb_sum_dim": (C.c_int, [c_stream, c_f32p, u64, u64, u64, c_f32p, C.c_void_p, u64]),
    "fb_mean_dim": (C.c_int, [c_stream, c_f32p, u64, u64, u64, c_f32p, C.c_void_p, u64]),
    "fb_max_dim": (C.c_int, [c_stream, c_f32p, u64, u64, u64, c_f32p, c_i64p, C.c_void_p, u64]),
    "fb_gather_dim": (C.c_int, [c_stream, c_f32p, u64p, c_i64p, u64p, C.c_int, C.c_int, c_f32p, c_i64p]),
    "fb_scatter_add_dim": (C.c_int, [c_stream, c_f32p, c_i64p, u64p, u64p, C.c_int, C.c_int, c_f32p, c_i64p]),
    "fb_segment_csr_build": (C.c_int, [C.c_void_p, u64, u64, C.c_void_p]),
    "fb_segment_sum": (C.c_int, [c_stream, c_f32p, c_i64p, u64, u64, u64, c_f32p]),
    "fb_segment_sum_bwd": (C.c_int, [c_stream, c_f32p, c_i64p, u64, u64, u64, c_f32p]),
    "fb_segment_softmax_fwd": (C.c_int, [c_stream, c_f32p, c_i64p, u64, u64, u64, c_f32p, C.c_void_p]),
    "fb_segment_softmax_bwd": (C.c_int, [c_stream, c_f32p, c_f32p, c_i64p, u64, u64, u64, c_f32p]),
    "fb_reduce_view_workspace_bytes": (u64, [C.POINTER(ViewDesc), C.c_int]),
    "fb_sum_dim_view": (C.c_int, [c_stream, C.POINTER(ViewDesc), C.c_int, c_f32p, C.c_void_p, u64]),
    "fb_mean_dim_view": (C.c_int, [c_stream, C.POINTER(ViewDesc), C.c_int, c_f32p, C.c_void_p, u64]),
    "fb_max_dim_view": (C.c_int, [c_stream, C.POINTER(ViewDesc), C.c_int, c_f32p, c_i64p, C.c_void_p, u64]),
    "fb_softmax_view_fwd": (C.c_int, [c_stream, C.POINTER(ViewDesc), C.c_int, c_f32p]),
    "fb_log_softmax_view_fwd": (C.c_int, [c_stream, C.POINTER(ViewDesc), C.c_int, c_f32p]),
    "fb_softmax_view_bwd": (C.c_int, [c_stream, C.POINTER(ViewDesc), C.POINTER(ViewDesc), C.c_int, c_f32p]),
    "fb_log_softmax_view_bwd": (C.c_int, [c_stream, C.POINTER(ViewDesc), C.POINTER(ViewDesc), C.c_int, c_f32p]),
    "fb_softmax_fwd": (C.c_int, [c_stream, c_f32p, u64, u64, c_f32p]),
    "fb_log_softmax_fwd": (C.c_int, [c_stream, c_f32p, u64, u64, c_f32p]),
    "fb_softmax_bwd": (C.c_int, [c_stream, c_f32p, c_f32p, u64, u64, c_f32p]),
    "fb_log_softmax_bwd": (C.c_int, [c_stream, c_f32p, c_f32p, u64, u64, c_f32p]),
    "fb_bias_act_scale_softmax_fwd": (C.c_int, [c_stream, c_f32p, c_f32p, C.c_int, f32, u64, u64,
                                                c_f32p]),
    "fb_softmax_fused_bwd_workspace_bytes": (u64, [u64, u64]),
    "fb_bias_act_scale_softmax_bwd": (C.c_int, [c_stream, c_f32p, c_f32p, c_f32p, c_f32p, C.c_int,
                                                f32, u64, u64, c_f32p, c_f32p, C.c_void_p, u64]),
    "fb_nll_workspace_bytes": (u64, [u64]),
    "fb_log_softmax_nll_fwd": (C.c_int, [c_stream, c_f32p, c_i64p, u64, u64, c_f32p, c_f32p,
                                         c_f32p, c_i64p, c_i64p, C.c_void_p, u64]),
    "fb_log_softmax_nll_bwd": (C.c_int, [c_stream, c_f32p, c_i64p, c_f32p, c_f32p, f32, u64, u64,
                                         c_f32p]),
    "fb_layer_norm_fwd": (C.c_int, [c_stream, c_f32p, c_f32p, c_f32p, u64, u64, f32, c_f32p,
                                    c_f32p, c_f32p, c_f32p, c_f32p]),
    "fb_layer_norm_bwd_workspace_bytes": (u64, [u64, u64]),
    "fb_layer_norm_bwd": (C.c_int, [c_stream, c_f32p, c_f32p, c_f32p, c_f32p, c_f32p, c_f32p,
                                    c_f32p, u64, u64, c_f32p, c_f32p, c_f32p, C.c_void_p, u64]),
    "fb_residual_layer_norm_fwd": (C.c_int, [c_stream, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, u64, u64, f32,
                                             C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "fb_rms_norm_fwd": (C.c_int, [c_stream, C.c_void_p, C.c_void_p, u64, u64, f32, C.c_void_p, C.c_void_p]),
    "fb_rms_norm_bwd": (C.c_int, [c_stream, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, u64, u64, C.c_void_p,
                                  C.c_void_p, C.c_void_p, u64]),
    "fb_layer_norm_bwd_static": (C.c_int, [c_stream, c_f32p, c_f32p, c_f32p, c_f32p, c_f32p, c_f32p,
                                           c_f32p, u64, u64, c_f32p, c_f32p, c_f32p]),
    "fb_sgd_step": (C.c_int, [c_stream, c_f32p, c_f32p, c_f32p, u64, f32, f32, C.c_int]),
    "fb_adamw_step": (C.c_int, [c_stream, c_f32p, c_f32p, c_f32p, c_f32p, u64, AdamWHparams]),
    "fb_adamw_step_capturable": (C.c_int, [c_stream, c_f32p, c_f32p, c_f32p, c_f32p, c_f32p, u64,
                                           f32, f32, f32, f32, f32]),
    "fb_scalar_increment": (C.c_int, [c_stream, c_f32p, f32, f32]),
    "fb_adamw_multi": (C.c_int, [c_stream, C.c_void_p, C.c_int, u64, AdamWHparams, f32]),
    "fb_sgd_multi": (C.c_int, [c_stream, C.c_void_p, C.c_int, u64, f32, f32, C.c_int, f32]),
    "fb_grad_norm_workspace_bytes": (u64, []),
    "fb_grad_sumsq_multi": (C.c_int, [c_stream, C.c_void_p, C.c_int, u64, f32, C.c_void_p, C.c_void_p, u64]),
    "fb_clip_scale": (C.c_int, [c_stream, C.c_void_p, f32, C.c_void_p, C.c_void_p]),
    "fb_adamw_multi_clipped": (C.c_int, [c_stream, C.c_void_p, C.c_int, u64, AdamWHparams, f32, C.c_void_p]),
    "fb_sgd_multi_clipped": (C.c_int, [c_stream, C.c_void_p, C.c_int, u64, f32, f32, C.c_int, f32, C.c_void_p]),
    "fb_bias_act_fwd": (C.c_int, [c_stream, c_f32p, c_f32p, C.c_int, u64, u64, c_f32p]),
    "fb_bias_act_bwd": (C.c_int, [c_stream, c_f32p, c_f32p, c_f32p, C.c_int, u64, u64, c_f32p,
                                  c_f32p, C.c_void_p, u64]),
    "fb_mse_fwd_bwd": (C.c_int, [c_stream, c_f32p, c_f32p, u64, f32, c_f32p, c_f32p, C.c_void_p,
                                 u64]),
    "fb_host_ln_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "fb_host_ln_device_bytes": (u64, [u64, u64, C.c_int]),
    "fb_host_ln_run": (C.c_int, [C.c_void_p, u64, u64, f32] + [C.c_void_p] * 9 + [C.c_void_p, u64]),
    "fb_host_ln_synchronize": (C.c_int, [C.c_void_p]),
    "fb_host_ln_destroy": (C.c_int, [C.c_void_p]),
    "fb_safetensors_image_bytes": (u64, [C.POINTER(StEntry), C.c_int, u64p]),
    "fb_safetensors_write": (C.c_int, [c_stream, C.POINTER(StEntry), C.c_int, C.POINTER(C.c_void_p), C.c_int, C.c_void_p, u64]),
    "fb_safetensors_count": (C.c_int, [C.c_void_p, u64]),
    "fb_safetensors_entry": (C.c_int, [C.c_void_p, u64, C.c_int, C.c_char_p, u64, C.POINTER(StEntry), u64p, u64p]),
    "fb_safetensors_read": (C.c_int, [c_stream, C.c_void_p, u64, C.c_char_p, C.c_int, u64, C.c_void_p, C.c_int]),
    "fb_dlpack_export": (C.c_int, [C.c_void_p, u64, C.c_int, C.c_int, C.POINTER(i64), C.POINTER(i64), C.c_int, C.c_void_p,
                                   DLPACK_RELEASE_FN, C.POINTER(C.c_void_p)]),
    "fb_dlpack_handoff": (C.c_int, [c_stream, C.c_int, i64]),
    "fb_dlpack_describe": (C.c_int, [C.c_void_p, C.POINTER(DlpackDesc)]),
    "fb_dlpack_import_into": (C.c_int, [c_stream, C.c_void_p, C.c_void_p, u64]),
    "fb_dlpack_delete": (None, [C.c_void_p]),
    "fb_rng_seed": (None, [C.c_void_p, u64]),
    "fb_rng_skip": (None, [C.c_void_p, u64]),
    "fb_rng_uniform": (f32, [C.c_void_p]),
    "fb_rng_normal": (f32, [C.c_void_p]),
    "fb_rng_fill_uniform": (C.c_int, [C.c_void_p, C.c_void_p, u64, f32, f32]),
    "fb_rng_fill_normal": (C.c_int, [C.c_void_p, C.c_void_p, u64, f32, f32]),
    "fb_rng_fill_rowscaled_normal": (C.c_int, [C.c_void_p, C.c_void_p, u64, u64, f32, f32]),
    "fb_rng_fill_index": (C.c_int, [C.c_void_p, C.c_void_p, u64, u64]),
    "fb_ddp_unique_id": (C.c_int, [C.c_void_p]),
    "fb_ddp_comm_init": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "fb_ddp_rank": (C.c_int, [C.c_void_p]),
    "fb_ddp_world": (C.c_int, [C.c_void_p]),
    "fb_ddp_nccl_version": (C.c_int, []),
    "fb_ddp_allreduce_bucket": (C.c_int, [C.c_void_p, c_stream, c_f32p, u64]),
    "fb_ddp_allreduce_buckets": (C.c_int, [C.c_void_p, c_stream, C.POINTER(C.c_void_p), u64p, C.c_int]),
    "fb_ddp_average_bucket": (C.c_int, [C.c_void_p, c_stream, c_f32p, u64]),
    "fb_ddp_poll": (C.c_int, [C.c_void_p]),
    "fb_ddp_comm_abort": (C.c_int, [C.c_void_p]),
    "fb_ddp_comm_destroy": (C.c_int, [C.c_void_p]),
}

_LIB = None


def load():
    """Load the library once and attach the prototypes.  Raises if it is absent."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built "
            "(run `python -m ferro_b200.build`); there is no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib
