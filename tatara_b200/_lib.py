"""ctypes binding of libtatara_b200.so (the C ABI declared in include/tatara_b200.h).

Importing this module never touches the CPU oracle and has no CPU fallback: if the shared library is
missing the import of the first symbol raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtatara_b200.so")

TB_OK = 0
ARCH_LAYERSTACK, ARCH_SIMPLE = 0, 1
ACT_CRELU, ACT_SCRELU, ACT_PAIRWISE = 0, 1, 2
OPT_RANGER, OPT_RADAM, OPT_ADAMW = 0, 1, 2
LOSS_SIGMOID, LOSS_WRM = 0, 1
NUM_SLOTS = 4

f = C.c_float
i32 = C.c_int32
i64 = C.c_int64
vp = C.c_void_p


class Config(C.Structure):
    _fields_ = [
        ("struct_size", i32), ("device", i32), ("arch", i32), ("batch_capacity", i32), ("ft_in", i32),
        ("piece_inputs", i32), ("ft_factorize", i32), ("max_active", i32), ("ft_out", i32), ("l1_out", i32),
        ("l2_out", i32), ("num_buckets", i32), ("activation", i32), ("optimizer", i32), ("precision", i32),
        ("wd_ft", f), ("wd_dense", f), ("wd_bias", f), ("lr_mult_ft", f), ("lr_mult_dense", f), ("lr_mult_bias", f),
        ("world_size", i32), ("rank", i32), ("nccl_unique_id", C.c_uint8 * 128), ("nccl_ctas", i32), ("dp_exchange", i32),
    ]


class Loss(C.Structure):
    _fields_ = [
        ("kind", i32), ("scale", f), ("nnue2score", f), ("in_scaling", f), ("in_offset", f), ("target_offset", f),
        ("target_scaling", f), ("pow_exp", f), ("qp_asymmetry", f), ("weight_boost_w1", f), ("weight_boost_w2", f),
    ]


class MicrobenchResult(C.Structure):
    _fields_ = [("fwd_ms", f), ("bwd_ms", f), ("adam_ms", f), ("fwd_slice_ms", f), ("bwd_slice_ms", f), ("iters", i32)]


class Batch(C.Structure):
    _fields_ = [
        ("n_pos", i32), ("stm_indices", vp), ("nstm_indices", vp), ("nnz", vp), ("bucket_idx", vp), ("score", vp),
        ("wdl", vp), ("per_pos_norm", f),
    ]


# every symbol include/tatara_b200.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "tb_create": (C.c_int, [C.POINTER(Config), C.POINTER(vp)]),
    "tb_destroy": (None, [vp]),
    "tb_last_error": (C.c_char_p, [vp]),
    "tb_num_groups": (C.c_int, [vp]),
    "tb_group_name": (C.c_char_p, [vp, C.c_int]),
    "tb_group_len": (i64, [vp, C.c_char_p]),
    "tb_upload_group": (C.c_int, [vp, C.c_char_p, vp, vp, vp, vp, i64]),
    "tb_download_group": (C.c_int, [vp, C.c_char_p, vp, vp, vp, vp, i64]),
    "tb_get_step_count": (C.c_int, [vp, C.POINTER(C.c_uint64)]),
    "tb_set_step_count": (C.c_int, [vp, C.c_uint64]),
    "tb_train_step": (C.c_int, [vp, C.POINTER(Batch), f, f, C.POINTER(Loss), C.POINTER(C.c_double)]),
    "tb_train_step_psv": (C.c_int, [vp, C.c_int, vp, C.c_int, f, f, C.POINTER(Loss), C.POINTER(C.c_double)]),
    "tb_flush_pending_loss": (C.c_int, [vp, C.POINTER(C.c_double)]),
    "tb_validate_step": (C.c_int, [vp, C.POINTER(Batch), f, C.POINTER(Loss), C.POINTER(C.c_double), vp]),
    "tb_read_fp16_clamp_count": (C.c_int, [vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "tb_stage_batch": (C.c_int, [vp, C.c_int, C.POINTER(Batch)]),
    "tb_train_step_staged": (C.c_int, [vp, C.c_int, f, f, C.POINTER(Loss), C.POINTER(C.c_double)]),
    "tb_forward_backward": (C.c_int, [vp, C.POINTER(Batch), f, C.POINTER(Loss), C.POINTER(C.c_double)]),
    "tb_apply_optimizer": (C.c_int, [vp, f]),
    "tb_download_grad": (C.c_int, [vp, C.c_char_p, vp, i64]),
    "tb_read_buffer": (C.c_int, [vp, C.c_char_p, vp, i64]),
    "tb_timer_start": (C.c_int, [vp]),
    "tb_timer_stop": (C.c_int, [vp, C.POINTER(f)]),
    "tb_profile_enable": (C.c_int, [vp, C.c_int]),
    "tb_profile_num_phases": (C.c_int, [vp]),
    "tb_profile_read": (C.c_int, [vp, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_double), C.POINTER(i64)]),
    "tb_profile_reset": (C.c_int, [vp]),
    "tb_launch_count": (i64, [vp]),
    "tb_synchronize": (C.c_int, [vp]),
    "tb_ft_forward_bench": (C.c_int, [C.c_int, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, C.POINTER(f)]),
    "tb_ft_backward_bench": (C.c_int, [C.c_int, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, C.POINTER(f)]),
    "tb_adam_clamp_bench": (C.c_int, [C.c_int, vp, vp, vp, vp, i64, f, f, f, f, C.c_int, C.POINTER(f)]),
    "tb_ft_microbench": (C.c_int, [C.c_int, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.POINTER(MicrobenchResult)]),
    "tb_psv_extract": (C.c_int, [C.c_int, C.c_int, vp, i64, vp, vp, vp, vp, vp, vp]),
    "tb_psv_synthesize": (C.c_int, [C.c_uint64, i64, vp]),
    "tb_psv_encode": (C.c_int, [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "tb_init_sample": (C.c_int, [vp, i64, i64, i64, C.c_int, C.c_int, f, C.c_int, C.c_uint64]),
    "tb_host_alloc": (C.c_int, [C.POINTER(vp), C.c_size_t]),
    "tb_host_free": (C.c_int, [vp]),
    "tb_ft_backward_static_scratch": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp, C.c_char_p, C.c_size_t]),
    "tb_nccl_unique_id": (C.c_int, [vp]),
    "tb_device_count": (C.c_int, []),
    "tb_version": (C.c_char_p, []),
}

_lib = None


def load():
    """Loads the shared library and types every exported function.  Fails loudly when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "tatara_b200: %s is missing; build it with `python -m tatara_b200.build` (needs nvcc). "
            "There is no CPU fallback." % LIB_PATH)
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL | os.RTLD_NOW)  # RTLD_NOW: an unresolved symbol fails here, not mid-run
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError names the missing symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
