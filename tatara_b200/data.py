"""Step inputs: synthetic PackedSfenValue records and their extraction into index batches on the GPU.

The reference trains on a private teacher file; the benchmark uses seeded synthetic records of the same
40-byte shape (tb_psv_synthesize) and turns them into the trainer's inputs with the device-side decoder
(tb_psv_extract), i.e. the work of the reference's dataloader workers
(crates/nnue-train/src/dataloader.rs:1303-1407).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib as L
from .trainer import BatchData, FeatureSetSpec, TrainerError

SYNTH_SEED = 0x7A7A2A  # base seed of the synthetic generator; the benchmark adds the config index and the rank


def synthesize_psv(seed: int, n_records: int) -> np.ndarray:
    """n_records seeded synthetic 40-byte records as a uint8 array [n_records, 40]."""
    out = np.zeros((n_records, 40), np.uint8)
    rc = L.load().tb_psv_synthesize(seed, n_records, out.ctypes.data)
    if rc != L.TB_OK:
        raise TrainerError("tb_psv_synthesize failed (%d)" % rc)
    return out


class PinnedArray:
    """A numpy view of page-locked host memory owned by the library (tb_host_alloc)."""

    def __init__(self, shape, dtype):
        self.dtype = np.dtype(dtype)
        n = int(np.prod(shape)) * self.dtype.itemsize
        self._p = L.vp()
        rc = L.load().tb_host_alloc(C.byref(self._p), n)
        if rc != L.TB_OK:
            raise TrainerError("tb_host_alloc failed (%d)" % rc)
        buf = (C.c_uint8 * max(n, 1)).from_address(self._p.value)
        self.array = np.frombuffer(buf, dtype=self.dtype, count=int(np.prod(shape))).reshape(shape)

    def free(self):
        if self._p is not None and self._p.value:
            self.array = None
            L.load().tb_host_free(self._p)
            self._p = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def extract_batch(psv: np.ndarray, feature_set: FeatureSetSpec, with_bucket: bool = True, device: int = 0,
                  pinned: bool = False) -> BatchData:
    """Decodes records and extracts both perspectives' active indices, nnz, kingrank9 bucket, score and wdl
    on the GPU; returns host arrays (page-locked when `pinned`)."""
    psv = np.ascontiguousarray(psv, np.uint8).reshape(-1, 40)
    n, A = psv.shape[0], feature_set.max_active
    keep = []

    def alloc(shape, dt):
        if pinned:
            p = PinnedArray(shape, dt)
            keep.append(p)
            return p.array
        return np.empty(shape, dt)

    stm, nstm = alloc((n, A), np.int32), alloc((n, A), np.int32)
    nnz, score, wdl = alloc((n,), np.int32), alloc((n,), np.float32), alloc((n,), np.float32)
    bucket = alloc((n,), np.int32) if with_bucket else None
    rc = L.load().tb_psv_extract(device, feature_set.index, psv.ctypes.data, n, stm.ctypes.data, nstm.ctypes.data,
                                 nnz.ctypes.data, bucket.ctypes.data if with_bucket else None, score.ctypes.data,
                                 wdl.ctypes.data)
    if rc != L.TB_OK:
        raise TrainerError("tb_psv_extract failed (%d): %s" % (rc, L.load().tb_last_error(None).decode()))
    return BatchData(stm, nstm, nnz, score, wdl, bucket, 0.0, keep)


def synthetic_batch(seed: int, n_pos: int, feature_set: FeatureSetSpec, with_bucket: bool = True, device: int = 0,
                    pinned: bool = False) -> BatchData:
    return extract_batch(synthesize_psv(seed, n_pos), feature_set, with_bucket, device, pinned)


def nccl_unique_id() -> bytes:
    buf = (C.c_uint8 * 128)()
    rc = L.load().tb_nccl_unique_id(buf)
    if rc != L.TB_OK:
        raise TrainerError("tb_nccl_unique_id failed (%d): %s" % (rc, L.load().tb_last_error(None).decode()))
    return bytes(buf)
