"""tatara_b200 — the NNUE training step of SH11235/tatara as hand-written sm_100a CUDA behind a C ABI.

The package is a thin host layer over libtatara_b200.so (include/tatara_b200.h).  There is no CPU path:
constructing a trainer without the shared library or without a CUDA device raises.
"""
from ._lib import LIB_PATH, load as load_library
from .trainer import (BatchData, FEATURE_SETS, FeatureSetSpec, GpuTrainer, LossKind, OptimGroupConfig, PrecisionFlags,
                      SimpleGpuTrainer, TrainerError, layerstack_default_init, simple_default_init)
from .ckpt import RawCkptHeader, load_raw_checkpoint, read_raw_checkpoint_header, save_raw_checkpoint
from .data import PinnedArray, extract_batch, nccl_unique_id, synthesize_psv, synthetic_batch, SYNTH_SEED

__all__ = [
    "BatchData", "FEATURE_SETS", "FeatureSetSpec", "GpuTrainer", "LossKind", "OptimGroupConfig", "PrecisionFlags",
    "SimpleGpuTrainer", "TrainerError", "layerstack_default_init", "simple_default_init", "PinnedArray", "extract_batch",
    "nccl_unique_id", "synthesize_psv", "synthetic_batch", "SYNTH_SEED", "LIB_PATH", "load_library",
    "RawCkptHeader", "load_raw_checkpoint", "read_raw_checkpoint_header", "save_raw_checkpoint",
]
