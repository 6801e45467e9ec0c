"""Host-side mirror of tatara's trainer backends over the C ABI.

`GpuTrainer` / `SimpleGpuTrainer` take the arguments of the reference constructors
(bins/nnue_train/src/trainer_layerstack.rs:781-796, bins/nnue_train/src/trainer_simple.rs:392-402) and
expose the `TrainerBackend` methods (crates/nnue-train/src/trainer.rs:273-374): train_step,
flush_pending_loss, validate_step, read_fp16_clamp_count.  Errors of the library become `TrainerError`
(the reference maps them to io::Error::other).  All compute happens in libtatara_b200.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import numpy as np

from . import _lib as L


class TrainerError(RuntimeError):
    pass


# ---- feature sets (crates/shogi-features/src/feature_set.rs:1031-1038) --------------------------------
@dataclass(frozen=True)
class FeatureSetSpec:
    name: str
    index: int          # the library's feature-set id (tb_psv_extract)
    king_buckets: int
    piece_inputs: int
    max_active: int
    ft_factorize: bool = True   # the CLI default (bins/nnue_train/src/cli.rs:730-745)

    @property
    def ft_in(self) -> int:
        return self.king_buckets * self.piece_inputs

    @property
    def train_ft_in(self) -> int:
        return self.ft_in + (self.piece_inputs if self.ft_factorize else 0)

    def with_factorize(self, on: bool) -> "FeatureSetSpec":
        return FeatureSetSpec(self.name, self.index, self.king_buckets, self.piece_inputs, self.max_active, on)


FEATURE_SETS: Dict[str, FeatureSetSpec] = {
    "halfkp": FeatureSetSpec("halfkp", 0, 81, 1548, 38),
    "halfka-split": FeatureSetSpec("halfka-split", 1, 81, 1710, 40),
    "halfka-merged": FeatureSetSpec("halfka-merged", 2, 81, 1629, 40),
    "halfka-hm-split": FeatureSetSpec("halfka-hm-split", 3, 45, 1710, 40),
    "halfka-hm-merged": FeatureSetSpec("halfka-hm-merged", 4, 45, 1629, 40),
}


# ---- loss / optimizer kinds ------------------------------------------------------------------------------
@dataclass(frozen=True)
class LossKind:
    """nnue_train::trainer::LossKind (crates/nnue-train/src/trainer.rs:75-95)."""
    kind: int
    scale: float = 0.0
    nnue2score: float = 600.0
    in_scaling: float = 340.0
    in_offset: float = 270.0
    target_offset: float = 270.0
    target_scaling: float = 380.0
    pow_exp: float = 2.0
    qp_asymmetry: float = 0.0
    weight_boost_w1: float = 0.0
    weight_boost_w2: float = 0.5

    @staticmethod
    def sigmoid(scale: float = 1.0 / 290.0) -> "LossKind":
        return LossKind(L.LOSS_SIGMOID, scale=scale)

    @staticmethod
    def wrm(**kw) -> "LossKind":
        return LossKind(L.LOSS_WRM, **kw)

    def to_c(self) -> L.Loss:
        return L.Loss(self.kind, self.scale, self.nnue2score, self.in_scaling, self.in_offset, self.target_offset,
                      self.target_scaling, self.pow_exp, self.qp_asymmetry, self.weight_boost_w1, self.weight_boost_w2)


OPTIMIZERS = {"ranger": L.OPT_RANGER, "radam": L.OPT_RADAM, "adamw": L.OPT_ADAMW}


@dataclass(frozen=True)
class OptimGroupConfig:
    """(weight_decay, lr_mult) of the ft / dense / bias groups (trainer_layerstack.rs:640-705)."""
    ft: Tuple[float, float] = (0.01, 1.0)
    dense: Tuple[float, float] = (0.01, 1.0)
    bias: Tuple[float, float] = (0.01, 1.0)

    @staticmethod
    def resolve(global_weight_decay: float, ft_wd=None, dense_wd=None, bias_wd=None, ft_lr=None, dense_lr=None,
                bias_lr=None) -> "OptimGroupConfig":
        g = lambda wd, lm: (global_weight_decay if wd is None else wd, 1.0 if lm is None else lm)
        return OptimGroupConfig(g(ft_wd, ft_lr), g(dense_wd, dense_lr), g(bias_wd, bias_lr))


@dataclass(frozen=True)
class PrecisionFlags:
    tf32: bool = False
    ft_fp16: bool = False
    ft_fp16_out: bool = False
    fp16_opt_state: bool = False

    def mask(self) -> int:
        return (1 if self.tf32 else 0) | (2 if self.ft_fp16 else 0) | (4 if self.ft_fp16_out else 0) | \
               (8 if self.fp16_opt_state else 0)


@dataclass
class BatchData:
    """Step inputs (bins/nnue_train/src/trainer_common.rs:142-151); arrays are C-contiguous numpy arrays."""
    stm_indices: np.ndarray
    nstm_indices: np.ndarray
    nnz: np.ndarray
    score: np.ndarray
    wdl: np.ndarray
    bucket_idx: Optional[np.ndarray] = None
    per_pos_norm: float = 0.0
    _keep: list = field(default_factory=list, repr=False)

    @property
    def n_pos(self) -> int:
        return int(self.nnz.shape[0])

    def to_c(self) -> L.Batch:
        def ptr(a, dt):
            if a is None:
                return None
            if a.dtype != dt or not a.flags["C_CONTIGUOUS"]:
                raise TrainerError("batch arrays must be C-contiguous %s" % dt)
            return a.ctypes.data
        return L.Batch(self.n_pos, ptr(self.stm_indices, np.int32), ptr(self.nstm_indices, np.int32),
                       ptr(self.nnz, np.int32), ptr(self.bucket_idx, np.int32), ptr(self.score, np.float32),
                       ptr(self.wdl, np.float32), self.per_pos_norm)


# ---- default initialisation (crates/nnue-train/src/init.rs:213-316) -------------------------------------
def _sample(n, num_buckets, fan_in, dist, scale_kind, value, seed) -> np.ndarray:
    out = np.empty(n, np.float32)
    rc = L.load().tb_init_sample(out.ctypes.data, n, num_buckets, fan_in, dist, scale_kind, value, 0, seed)
    if rc != L.TB_OK:
        raise TrainerError("tb_init_sample failed (%d)" % rc)
    return out


def layerstack_default_init(fs: FeatureSetSpec, ft_out: int, l1: int, l2: int, nb: int) -> Dict[str, np.ndarray]:
    """LayerStackInit::default_uniform with the call shapes of trainer_layerstack.rs:844-878."""
    N, F, l2in = fs.ft_in, ft_out, 2 * (l1 - 1)
    ft_w = np.zeros(fs.train_ft_in * F, np.float32)
    ft_w[:N * F] = _sample(N * F, 1, N, 1, 1, 1.0, 0x100)
    z = lambda n: np.zeros(n, np.float32)
    return {
        "ft_w": ft_w, "ft_b": z(F),
        "l1_w": _sample(nb * l1 * F, nb, F, 1, 0, 0.01, 0x101), "l1_b": z(nb * l1),
        "l1_shared_weight": _sample(F * l1, 1, F, 1, 0, 0.01, 0x102), "l1_shared_bias": z(l1),
        "l2_w": _sample(nb * l2 * l2in, nb, l2in, 1, 0, 0.01, 0x103), "l2_b": z(nb * l2),
        "l3_w": _sample(nb * l2, nb, l2, 1, 0, 0.01, 0x104), "l3_b": z(nb),
    }


def simple_default_init(fs: FeatureSetSpec, ft_out: int, l1: int, l2: int, pairwise: bool = False) -> Dict[str, np.ndarray]:
    """SimpleInit::default_uniform with the call shapes of trainer_simple.rs:454-463 (the L1 input is 2 * ft_out wide,
    ft_out with the Pairwise activation)."""
    N, F = fs.ft_in, ft_out
    K1 = F if pairwise else 2 * F
    ft_w = np.zeros(fs.train_ft_in * F, np.float32)
    ft_w[:N * F] = _sample(N * F, 1, N, 1, 0, 0.01, 0x5071E001)
    return {
        "ft_w": ft_w, "ft_b": _sample(F, 1, N, 1, 0, 0.01, 0x5071E002),
        "l1_w": _sample(K1 * l1, 1, K1, 1, 0, 0.01, 0x5071E003), "l1_b": _sample(l1, 1, K1, 1, 0, 0.01, 0x5071E004),
        "l2_w": _sample(l1 * l2, 1, l1, 1, 0, 0.01, 0x5071E005), "l2_b": _sample(l2, 1, l1, 1, 0, 0.01, 0x5071E006),
        "l3_w": _sample(l2, 1, l2, 1, 0, 0.01, 0x5071E007), "l3_b": _sample(1, 1, l2, 1, 0, 0.01, 0x5071E008),
    }


# ---- trainers ------------------------------------------------------------------------------------------------
class _Trainer:
    def __init__(self, cfg: L.Config, init: Optional[Dict[str, np.ndarray]]):
        self._lib = L.load()
        self._h = L.vp()
        cfg.struct_size = C.sizeof(L.Config)
        rc = self._lib.tb_create(C.byref(cfg), C.byref(self._h))
        if rc != L.TB_OK:
            self._h = None
            raise TrainerError("tb_create failed (%d): %s" % (rc, self._lib.tb_last_error(None).decode()))
        self.cfg = cfg
        self.group_names = [self._lib.tb_group_name(self._h, i).decode() for i in range(self._lib.tb_num_groups(self._h))]
        if init is not None:
            for name in self.group_names:
                self.upload_group(name, w=init[name])

    # -- life cycle
    def close(self):
        if getattr(self, "_h", None):
            self._lib.tb_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc, what):
        if rc != L.TB_OK:
            raise TrainerError("%s failed (%d): %s" % (what, rc, self._lib.tb_last_error(self._h).decode()))

    # -- parameter groups
    def group_len(self, name: str) -> int:
        n = int(self._lib.tb_group_len(self._h, name.encode()))
        if n < 0:
            raise TrainerError("unknown group '%s'" % name)
        return n

    def upload_group(self, name, w=None, m=None, v=None, slow=None):
        n = self.group_len(name)
        arrs = []
        for a in (w, m, v, slow):
            if a is None:
                arrs.append(None)
            else:
                a = np.ascontiguousarray(a, np.float32).reshape(-1)
                if a.size != n:
                    raise TrainerError("group '%s' has %d elements, got %d" % (name, n, a.size))
                arrs.append(a)
        p = [None if a is None else a.ctypes.data for a in arrs]
        self._check(self._lib.tb_upload_group(self._h, name.encode(), p[0], p[1], p[2], p[3], n), "tb_upload_group")

    def download_group(self, name, which=("w",)) -> Dict[str, np.ndarray]:
        n = self.group_len(name)
        out = {k: np.empty(n, np.float32) for k in which}
        p = [out[k].ctypes.data if k in out else None for k in ("w", "m", "v", "slow")]
        self._check(self._lib.tb_download_group(self._h, name.encode(), p[0], p[1], p[2], p[3], n), "tb_download_group")
        return out

    def download_grad(self, name) -> np.ndarray:
        n = self.group_len(name)
        g = np.empty(n, np.float32)
        self._check(self._lib.tb_download_grad(self._h, name.encode(), g.ctypes.data, n), "tb_download_grad")
        return g

    @property
    def step_count(self) -> int:
        s = C.c_uint64()
        self._check(self._lib.tb_get_step_count(self._h, C.byref(s)), "tb_get_step_count")
        return s.value

    @step_count.setter
    def step_count(self, v: int):
        self._check(self._lib.tb_set_step_count(self._h, v), "tb_set_step_count")

    # -- TrainerBackend
    def train_step(self, batch: BatchData, lr: float, wdl_lambda: float, loss: LossKind) -> float:
        """Returns the loss sum of the previous step (0.0 on the first call)."""
        out = C.c_double()
        cb, cl = batch.to_c(), loss.to_c()
        self._check(self._lib.tb_train_step(self._h, C.byref(cb), lr, wdl_lambda, C.byref(cl), C.byref(out)), "tb_train_step")
        self._last_batch = batch  # a pinned batch stays alive until the next call returns
        return out.value

    step = train_step

    def train_step_psv(self, psv: np.ndarray, lr: float, wdl_lambda: float, loss: LossKind) -> float:
        """train_step on 40-byte PackedSfenValue records (uint8 [n, 40]); decode and feature extraction run on the GPU."""
        psv = np.ascontiguousarray(psv, np.uint8).reshape(-1, 40)
        out = C.c_double()
        cl = loss.to_c()
        self._check(self._lib.tb_train_step_psv(self._h, self.feature_set.index, psv.ctypes.data, psv.shape[0], lr, wdl_lambda,
                                                C.byref(cl), C.byref(out)), "tb_train_step_psv")
        self._last_batch = psv
        return out.value

    def flush_pending_loss(self) -> float:
        out = C.c_double()
        self._check(self._lib.tb_flush_pending_loss(self._h, C.byref(out)), "tb_flush_pending_loss")
        return out.value

    def validate_step(self, batch: BatchData, wdl_lambda: float, loss: LossKind) -> Tuple[float, np.ndarray]:
        """Forward + loss only: (sum of squared errors, net_output[n_pos])."""
        out = C.c_double()
        net = np.empty(batch.n_pos, np.float32)
        cb, cl = batch.to_c(), loss.to_c()
        self._check(self._lib.tb_validate_step(self._h, C.byref(cb), wdl_lambda, C.byref(cl), C.byref(out),
                                               net.ctypes.data), "tb_validate_step")
        return out.value, net

    validate = validate_step

    def read_fp16_clamp_count(self) -> Tuple[int, int]:
        a, b = C.c_uint64(), C.c_uint64()
        self._check(self._lib.tb_read_fp16_clamp_count(self._h, C.byref(a), C.byref(b)), "tb_read_fp16_clamp_count")
        return a.value, b.value

    # -- device-resident batches
    def stage_batch(self, slot: int, batch: BatchData):
        cb = batch.to_c()
        self._check(self._lib.tb_stage_batch(self._h, slot, C.byref(cb)), "tb_stage_batch")

    def train_step_staged(self, slot: int, lr: float, wdl_lambda: float, loss: LossKind) -> float:
        out = C.c_double()
        cl = loss.to_c()
        self._check(self._lib.tb_train_step_staged(self._h, slot, lr, wdl_lambda, C.byref(cl), C.byref(out)),
                    "tb_train_step_staged")
        return out.value

    # -- diagnostics
    def forward_backward(self, batch: BatchData, wdl_lambda: float, loss: LossKind) -> float:
        out = C.c_double()
        cb, cl = batch.to_c(), loss.to_c()
        self._check(self._lib.tb_forward_backward(self._h, C.byref(cb), wdl_lambda, C.byref(cl), C.byref(out)),
                    "tb_forward_backward")
        return out.value

    def apply_optimizer(self, lr: float):
        self._check(self._lib.tb_apply_optimizer(self._h, lr), "tb_apply_optimizer")

    def read_buffer(self, name: str, n: int) -> np.ndarray:
        out = np.empty(n, np.float32)
        self._check(self._lib.tb_read_buffer(self._h, name.encode(), out.ctypes.data, n), "tb_read_buffer")
        return out

    # -- timing
    def timer_start(self):
        self._check(self._lib.tb_timer_start(self._h), "tb_timer_start")

    def timer_stop(self) -> float:
        ms = C.c_float()
        self._check(self._lib.tb_timer_stop(self._h, C.byref(ms)), "tb_timer_stop")
        return ms.value

    def profile_enable(self, on: bool):
        self._check(self._lib.tb_profile_enable(self._h, int(on)), "tb_profile_enable")

    def profile_reset(self):
        self._check(self._lib.tb_profile_reset(self._h), "tb_profile_reset")

    def profile_read(self) -> Dict[str, Tuple[float, int]]:
        out = {}
        for i in range(self._lib.tb_profile_num_phases(self._h)):
            name, ms, n = C.c_char_p(), C.c_double(), L.i64()
            self._check(self._lib.tb_profile_read(self._h, i, C.byref(name), C.byref(ms), C.byref(n)), "tb_profile_read")
            out[name.value.decode()] = (ms.value, n.value)
        return out

    @property
    def launch_count(self) -> int:
        return int(self._lib.tb_launch_count(self._h))

    def synchronize(self):
        self._check(self._lib.tb_synchronize(self._h), "tb_synchronize")


DP_EXCHANGE = {"nccl": 0, "peer-copy": 1, "peer-kernel": 2}


def _dp(cfg: L.Config, world_size: int, rank: int, nccl_id: Optional[bytes], nccl_ctas: int = 0, dp_exchange: str = "nccl"):
    cfg.world_size, cfg.rank, cfg.nccl_ctas, cfg.dp_exchange = world_size, rank, nccl_ctas, DP_EXCHANGE[dp_exchange]
    if world_size > 1:
        if nccl_id is None or len(nccl_id) != 128:
            raise TrainerError("data parallel needs the 128-byte NCCL id of rank 0")
        C.memmove(cfg.nccl_unique_id, nccl_id, 128)


class GpuTrainer(_Trainer):
    """LayerStack trainer (bins/nnue_train/src/trainer_layerstack.rs GpuTrainer)."""

    def __init__(self, batch_size: int, ft_out: int, l1_out: int, l2_out: int, num_buckets: int,
                 feature_set: FeatureSetSpec, optimizer: str = "ranger",
                 optim_groups: OptimGroupConfig = OptimGroupConfig(), precision: PrecisionFlags = PrecisionFlags(),
                 init: Optional[Dict[str, np.ndarray]] = "default", device: int = 0, world_size: int = 1, rank: int = 0,
                 nccl_id: Optional[bytes] = None, nccl_ctas: int = 0, dp_exchange: str = "nccl"):
        cfg = L.Config()
        cfg.device, cfg.arch, cfg.batch_capacity = device, L.ARCH_LAYERSTACK, batch_size
        cfg.ft_in, cfg.piece_inputs, cfg.ft_factorize = feature_set.ft_in, feature_set.piece_inputs, int(feature_set.ft_factorize)
        cfg.max_active, cfg.ft_out, cfg.l1_out, cfg.l2_out, cfg.num_buckets = feature_set.max_active, ft_out, l1_out, l2_out, num_buckets
        cfg.activation, cfg.optimizer, cfg.precision = 0, OPTIMIZERS[optimizer], precision.mask()
        (cfg.wd_ft, cfg.lr_mult_ft), (cfg.wd_dense, cfg.lr_mult_dense), (cfg.wd_bias, cfg.lr_mult_bias) = \
            optim_groups.ft, optim_groups.dense, optim_groups.bias
        _dp(cfg, world_size, rank, nccl_id, nccl_ctas, dp_exchange)
        self.feature_set = feature_set
        if isinstance(init, str):
            init = layerstack_default_init(feature_set, ft_out, l1_out, l2_out, num_buckets)
        super().__init__(cfg, init)


class SimpleGpuTrainer(_Trainer):
    """Simple 4-layer trainer (bins/nnue_train/src/trainer_simple.rs SimpleGpuTrainer)."""

    def __init__(self, batch_size: int, ft_out: int, l1_out: int, l2_out: int, feature_set: FeatureSetSpec,
                 activation: str = "crelu", optimizer: str = "ranger", weight_decay: float = 0.01,
                 precision: PrecisionFlags = PrecisionFlags(), init: Optional[Dict[str, np.ndarray]] = "default",
                 device: int = 0, world_size: int = 1, rank: int = 0, nccl_id: Optional[bytes] = None, nccl_ctas: int = 0, dp_exchange: str = "nccl"):
        cfg = L.Config()
        cfg.device, cfg.arch, cfg.batch_capacity = device, L.ARCH_SIMPLE, batch_size
        cfg.ft_in, cfg.piece_inputs, cfg.ft_factorize = feature_set.ft_in, feature_set.piece_inputs, int(feature_set.ft_factorize)
        cfg.max_active, cfg.ft_out, cfg.l1_out, cfg.l2_out, cfg.num_buckets = feature_set.max_active, ft_out, l1_out, l2_out, 0
        cfg.activation = {"crelu": L.ACT_CRELU, "screlu": L.ACT_SCRELU, "pairwise": L.ACT_PAIRWISE}[activation]
        cfg.optimizer, cfg.precision = OPTIMIZERS[optimizer], precision.mask()
        cfg.wd_ft = cfg.wd_dense = cfg.wd_bias = weight_decay
        cfg.lr_mult_ft = cfg.lr_mult_dense = cfg.lr_mult_bias = 1.0
        _dp(cfg, world_size, rank, nccl_id, nccl_ctas, dp_exchange)
        self.feature_set = feature_set
        if isinstance(init, str):
            init = simple_default_init(feature_set, ft_out, l1_out, l2_out, pairwise=activation == "pairwise")
        super().__init__(cfg, init)
