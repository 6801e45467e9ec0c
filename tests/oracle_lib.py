"""ctypes binding of the CPU oracle (oracle/libtatara_oracle.so).

Test infrastructure only: the product package never imports this module.
The library is built on demand with `make -C oracle`.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB_PATH = os.path.join(ORACLE_DIR, "libtatara_oracle.so")

f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
sz = C.c_size_t
f = C.c_float


class Board(C.Structure):
    _fields_ = [
        ("board_pt", C.c_uint8 * 81),
        ("board_color", C.c_uint8 * 81),
        ("hand", (C.c_uint8 * 7) * 2),
        ("side_to_move", C.c_uint8),
        ("black_king_sq", C.c_uint8),
        ("white_king_sq", C.c_uint8),
        ("score", C.c_int16),
        ("result", C.c_int8),
        ("ply", C.c_uint16),
    ]


class Config(C.Structure):
    _fields_ = [
        ("arch", C.c_int), ("ft_in", C.c_int), ("piece_inputs", C.c_int), ("factorize", C.c_int),
        ("max_active", C.c_int), ("ft_out", C.c_int), ("l1", C.c_int), ("l2", C.c_int),
        ("num_buckets", C.c_int), ("activation", C.c_int), ("optimizer", C.c_int),
        ("wd_ft", f), ("wd_dense", f), ("wd_bias", f),
        ("lr_mult_ft", f), ("lr_mult_dense", f), ("lr_mult_bias", f),
    ]


class Loss(C.Structure):
    _fields_ = [
        ("kind", C.c_int), ("scale", f),
        ("nnue2score", f), ("in_scaling", f), ("in_offset", f), ("target_offset", f), ("target_scaling", f),
        ("pow_exp", f), ("qp_asymmetry", f), ("weight_boost_w1", f), ("weight_boost_w2", f),
    ]


def sigmoid_loss(scale=1.0 / 290.0):
    return Loss(0, scale, 0, 0, 0, 0, 0, 2.0, 0.0, 0.0, 0.5)


def wrm_loss(nnue2score=600.0, in_scaling=340.0, in_offset=270.0, target_offset=270.0, target_scaling=380.0,
             pow_exp=2.0, qp_asymmetry=0.0, w1=0.0, w2=0.5):
    return Loss(1, 0.0, nnue2score, in_scaling, in_offset, target_offset, target_scaling, pow_exp, qp_asymmetry, w1, w2)


_lib = None


def build():
    subprocess.run(["make", "-C", ORACLE_DIR], check=True, stdout=subprocess.DEVNULL)


def lib():
    global _lib
    if _lib is not None:
        return _lib
    src = os.path.join(ORACLE_DIR, "tatara_oracle.c")
    if not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        build()
    L = C.CDLL(LIB_PATH)
    sig = {
        "ora_sparse_ft_forward": [f32p, i32p, i32p, f32p, sz, sz, sz, sz],
        "ora_sparse_ft_backward": [f32p, i32p, f32p, sz, sz, sz, sz],
        "ora_ft_fold_virtual": [f32p, f32p, sz, sz, sz],
        "ora_ft_reduce_virtual_grad": [f32p, sz, sz, sz],
        "ora_ft_post_perspective_fwd": [f32p, f32p, f32p, f32p, sz, sz, f],
        "ora_ft_post_perspective_grad": [f32p, f32p, f32p, f32p, f32p, sz, sz, sz, sz, f],
        "ora_dense_mm_fwd": [f32p, f32p, f32p, f32p, sz, sz, sz],
        "ora_dense_mm_bwd_input": [f32p, f32p, f32p, sz, sz, sz],
        "ora_dense_mm_bwd_weight": [f32p, f32p, f32p, sz, sz, sz],
        "ora_bias_grad": [f32p, f32p, sz, sz],
        "ora_dense_mm_fwd_bucket": [f32p, f32p, f32p, i32p, f32p, sz, sz, sz, sz],
        "ora_dense_mm_bwd_input_bucket": [f32p, f32p, i32p, f32p, sz, sz, sz, sz],
        "ora_dense_mm_bwd_weight_bucket": [f32p, f32p, i32p, f32p, sz, sz, sz, sz],
        "ora_bias_grad_bucket": [f32p, i32p, f32p, sz, sz, sz],
        "ora_crelu_fwd": [f32p, f32p, sz],
        "ora_crelu_grad": [f32p, f32p, f32p, sz],
        "ora_screlu_fwd": [f32p, f32p, sz],
        "ora_screlu_grad": [f32p, f32p, f32p, sz],
        "ora_abs_pow2_scale_fwd": [f32p, f32p, f, sz],
        "ora_abs_pow2_scale_grad": [f32p, f32p, f32p, f, sz],
        "ora_concat_l1sqr_main_fwd": [f32p, f32p, f32p, sz, sz, sz],
        "ora_concat_l1sqr_main_grad": [f32p, f32p, f32p, sz, sz],
        "ora_slice_extract_2d": [f32p, f32p, sz, sz, sz, sz],
        "ora_slice_scatter_2d": [f32p, f32p, sz, sz, sz, sz],
        "ora_elementwise_add": [f32p, f32p, f32p, sz],
        "ora_loss_wdl": [f32p, f32p, f32p, f32p, f32p, C.POINTER(C.c_double), f, f, sz],
        "ora_loss_wrm": [f32p, f32p, f32p, f32p, f32p, C.POINTER(C.c_double)] + [f] * 10 + [C.c_int, sz],
        "ora_radam_compute_step_size_denom": [C.c_uint64, f, f, f, C.POINTER(f), C.POINTER(C.c_int32)],
        "ora_radam_step": [f32p, f32p, f32p, f32p, f, f, C.c_int32, f, f, f, f, f, f, sz],
        "ora_ranger_lookahead_lerp": [f32p, f32p, f, sz],
        "ora_optimizer_scalars": [C.c_int, C.c_uint64, f, f, C.POINTER(f), C.POINTER(C.c_int32), C.POINTER(f)],
        "ora_init_sample": [f32p, sz, sz, sz, C.c_int, C.c_int, f, C.c_int, C.c_uint64],
        "ora_psv_decode": [u8p, C.POINTER(Board)],
        "ora_feature_dims": [C.c_int] + [C.POINTER(C.c_int)] * 4,
        "ora_extract_active_features": [C.c_int, C.POINTER(Board), i32p, i32p, C.c_int],
        "ora_kingrank9_bucket": [C.POINTER(Board)],
        "ora_psv_to_batch": [C.c_int, u8p, sz, i32p, i32p, i32p, C.c_void_p, f32p, f32p],
        "ora_loader_digest_bytes": [i32p, i32p, C.c_int32, f, f, u8p],
        "ora_psv_synthesize": [C.c_uint64, sz, u8p],
        "ora_psv_encode": [C.POINTER(Board), u8p],
    }
    for name, args in sig.items():
        getattr(L, name).argtypes = args
        getattr(L, name).restype = None
    for name in ("ora_feature_dims", "ora_extract_active_features", "ora_kingrank9_bucket", "ora_psv_to_batch",
                 "ora_psv_synthesize", "ora_psv_encode"):
        getattr(L, name).restype = C.c_int
    L.ora_loader_digest_bytes.restype = sz
    # trainer
    L.ora_trainer_create.argtypes = [C.POINTER(Config), C.c_int]
    L.ora_trainer_create.restype = C.c_void_p
    L.ora_trainer_destroy.argtypes = [C.c_void_p]
    L.ora_trainer_num_groups.argtypes = [C.c_void_p]
    L.ora_trainer_num_groups.restype = C.c_int
    L.ora_trainer_group_name.argtypes = [C.c_void_p, C.c_int]
    L.ora_trainer_group_name.restype = C.c_char_p
    L.ora_trainer_group_len.argtypes = [C.c_void_p, C.c_int]
    L.ora_trainer_group_len.restype = sz
    L.ora_trainer_group_ptr.argtypes = [C.c_void_p, C.c_int, C.c_int]
    L.ora_trainer_group_ptr.restype = C.POINTER(C.c_float)
    L.ora_trainer_init_default.argtypes = [C.c_void_p]
    L.ora_trainer_step_count.argtypes = [C.c_void_p]
    L.ora_trainer_step_count.restype = C.c_uint64
    L.ora_trainer_set_step_count.argtypes = [C.c_void_p, C.c_uint64]
    L.ora_trainer_set_threads.argtypes = [C.c_void_p, C.c_int]
    L.ora_trainer_buffer.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(sz)]
    L.ora_trainer_buffer.restype = C.POINTER(C.c_float)
    L.ora_trainer_step.argtypes = [C.c_void_p, i32p, i32p, i32p, C.c_void_p, f32p, f32p, C.c_int, f, f, f,
                                   C.POINTER(Loss), C.c_int]
    L.ora_trainer_step.restype = C.c_double
    L.ora_trainer_validate.argtypes = [C.c_void_p, i32p, i32p, i32p, C.c_void_p, f32p, f32p, C.c_int, f,
                                       C.POINTER(Loss), f32p]
    L.ora_trainer_validate.restype = C.c_double
    L.ora_trainer_set_precision.argtypes = [C.c_void_p, C.c_int]
    L.ora_trainer_clamp_count.argtypes = [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    L.ora_round_half.argtypes = [f]
    L.ora_round_half.restype = f
    L.ora_tf32.argtypes = [f]
    L.ora_tf32.restype = f
    L.ora_radam_step_f16state.argtypes = [f32p, f32p, f32p, f32p, f, f, C.c_int32, f, f, f, f, f, f, f, f, sz]
    L.ora_radam_step_f16state.restype = None
    L.ora_trainer_accumulate_grads.argtypes = [C.c_void_p, C.c_void_p]
    L.ora_trainer_apply_optimizer.argtypes = [C.c_void_p, f]
    _lib = L
    return L


FEATURE_SETS = {"halfkp": 0, "halfka-split": 1, "halfka-merged": 2, "halfka-hm-split": 3, "halfka-hm-merged": 4}
OPTIMIZERS = {"ranger": 0, "radam": 1, "adamw": 2}
WHICH = {"w": 0, "m": 1, "v": 2, "slow": 3, "grad": 4}


def feature_dims(name):
    kb, pi, n, a = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    assert lib().ora_feature_dims(FEATURE_SETS[name], kb, pi, n, a) == 0
    return dict(king_buckets=kb.value, piece_inputs=pi.value, ft_in=n.value, max_active=a.value)


def synthesize_psv(seed, n_records):
    """The benchmark's seeded synthetic records (uint8 [n, 40]), from the oracle's own generator."""
    out = np.zeros((n_records, 40), np.uint8)
    assert lib().ora_psv_synthesize(seed, n_records, out.reshape(-1)) == 0
    return out


def psv_to_batch(feature_set, psv_bytes, with_bucket=True):
    """PSV records (bytes / uint8 array, 40 B each) -> dict of the trainer's step inputs."""
    psv = np.ascontiguousarray(np.frombuffer(bytes(psv_bytes), dtype=np.uint8))
    n = psv.size // 40
    A = feature_dims(feature_set)["max_active"]
    out = dict(
        stm=np.empty((n, A), np.int32), nstm=np.empty((n, A), np.int32), nnz=np.empty(n, np.int32),
        bucket=np.empty(n, np.int32), score=np.empty(n, np.float32), wdl=np.empty(n, np.float32),
    )
    rc = lib().ora_psv_to_batch(FEATURE_SETS[feature_set], psv, n, out["stm"], out["nstm"], out["nnz"],
                                out["bucket"].ctypes.data if with_bucket else None, out["score"], out["wdl"])
    assert rc == 0, rc
    return out


class OracleTrainer:
    """Whole-step CPU oracle (LayerStack or Simple)."""

    def __init__(self, *, arch, ft_in, piece_inputs, factorize, max_active, ft_out, l1, l2, num_buckets=9,
                 activation=0, optimizer="ranger", wd=(0.01, 0.01, 0.01), lr_mult=(1.0, 1.0, 1.0), capacity=1024, precision=0):
        self.L = lib()
        self.cfg = Config(0 if arch == "layerstack" else 1, ft_in, piece_inputs, int(factorize), max_active, ft_out,
                          l1, l2, num_buckets, activation, OPTIMIZERS[optimizer], wd[0], wd[1], wd[2],
                          lr_mult[0], lr_mult[1], lr_mult[2])
        self.h = self.L.ora_trainer_create(C.byref(self.cfg), capacity)
        self.names = [self.L.ora_trainer_group_name(self.h, i).decode() for i in range(self.L.ora_trainer_num_groups(self.h))]
        if precision:
            self.L.ora_trainer_set_precision(self.h, precision)   # 1 tf32, 2 ft_fp16, 4 ft_fp16_out, 8 fp16_opt_state

    def clamp_count(self):
        a, b = C.c_uint64(), C.c_uint64()
        self.L.ora_trainer_clamp_count(self.h, C.byref(a), C.byref(b))
        return a.value, b.value

    def close(self):
        if self.h:
            self.L.ora_trainer_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def init_default(self):
        self.L.ora_trainer_init_default(self.h)

    def group(self, name, which="w"):
        """numpy view (no copy) of a parameter-group buffer."""
        gi = self.names.index(name)
        n = self.L.ora_trainer_group_len(self.h, gi)
        p = self.L.ora_trainer_group_ptr(self.h, gi, WHICH[which])
        return np.ctypeslib.as_array(p, shape=(n,))

    def buffer(self, name):
        n = sz()
        p = self.L.ora_trainer_buffer(self.h, name.encode(), C.byref(n))
        if not p:
            return None
        return np.ctypeslib.as_array(p, shape=(n.value,)).copy()

    @property
    def step_count(self):
        return self.L.ora_trainer_step_count(self.h)

    def set_threads(self, n):
        self.L.ora_trainer_set_threads(self.h, n)

    def step(self, batch, lr, wdl_lambda, loss, per_pos_norm=None, do_optimizer=True):
        n = int(batch["nnz"].shape[0])
        norm = (1.0 / n) if per_pos_norm is None else per_pos_norm
        bucket = batch.get("bucket")
        bptr = bucket.ctypes.data if bucket is not None else None
        return self.L.ora_trainer_step(self.h, batch["stm"], batch["nstm"], batch["nnz"], bptr, batch["score"],
                                       batch["wdl"], n, norm, lr, wdl_lambda, C.byref(loss), int(do_optimizer))

    def validate(self, batch, wdl_lambda, loss):
        n = int(batch["nnz"].shape[0])
        out = np.empty(n, np.float32)
        bucket = batch.get("bucket")
        bptr = bucket.ctypes.data if bucket is not None else None
        l = self.L.ora_trainer_validate(self.h, batch["stm"], batch["nstm"], batch["nnz"], bptr, batch["score"],
                                        batch["wdl"], n, wdl_lambda, C.byref(loss), out)
        return l, out

    def accumulate_grads(self, other):
        self.L.ora_trainer_accumulate_grads(self.h, other.h)

    def apply_optimizer(self, lr):
        self.L.ora_trainer_apply_optimizer(self.h, lr)
