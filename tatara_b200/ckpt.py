"""Raw resume checkpoint (`RNRC` version 8) over the C ABI.

The reference writes `{net_id}-{superbatch}.ckpt`: a self-describing header followed, per parameter group in the
trainer's group order, by `len, w, m, v, slow` as little-endian f32 (bins/nnue_train/src/ckpt.rs:17-55; group order
raw_ckpt_group_sources, bins/nnue_train/src/trainer_layerstack.rs:1440; header writer ckpt.rs:269-312, reader and its
checks ckpt.rs:322-470).  Moments are true f32 values whatever precision the trainer stores them in
(MomentBuf::to_host_f32, bins/nnue_train/src/trainer_common.rs:89-126): tb_download_group / tb_upload_group do the
scaling.  This module produces and consumes the same bytes from a `GpuTrainer` / `SimpleGpuTrainer`, so that files
move freely between this library and the reference's `--resume`.
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import _lib as L
from .trainer import TrainerError

MAGIC = b"RNRC"
VERSION = 8
MAX_RUN_ID_BYTES = 256
# crates/shogi-features/src/feature_set.rs:1063-1086
FEATURE_HASH = {"halfkp": 0x5D69D5B8, "halfka-split": 0x5F134CB8, "halfka-merged": 0xACD68C97,
                "halfka-hm-split": 0x2A46AC09, "halfka-hm-merged": 0x7F134CB8}


@dataclass
class RawCkptHeader:
    version: int
    feature_set: str
    train_ft_in: int
    ft_out: int
    max_active: int
    ft_factorize: bool
    feature_hash: int
    run_id: Optional[str]
    arch_kind: str
    bucket_mode: str
    topology: tuple
    superbatch: int
    step_count: int
    lr_horizon: Optional[int]
    num_groups: int


def _identity(trainer, bucket_mode):
    cfg, fs = trainer.cfg, trainer.feature_set
    if cfg.arch == L.ARCH_LAYERSTACK:
        arch = "layerstack"
        topo = (cfg.ft_out, cfg.l1_out, cfg.l2_out, cfg.num_buckets)      # layerstack_topology, ckpt.rs:186-198
        mode = "kingrank9" if bucket_mode is None else bucket_mode
    else:
        arch = "simple"
        topo = (cfg.ft_out, cfg.l1_out, cfg.l2_out)                       # trainer_simple.rs:2881
        mode = "" if bucket_mode is None else bucket_mode
    return arch, topo, mode, fs


def save_raw_checkpoint(trainer, path: str, superbatch: int, run_id: str = "", lr_horizon: Optional[int] = None,
                        bucket_mode: Optional[str] = None) -> None:
    """Writes the trainer's state; atomic tmp + rename like the reference (crates/nnue-train/src/trainer.rs:343-345)."""
    arch, topo, mode, fs = _identity(trainer, bucket_mode)
    rid = run_id.encode()
    if len(rid) > MAX_RUN_ID_BYTES:
        raise TrainerError("run id longer than %d bytes" % MAX_RUN_ID_BYTES)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        name = fs.name.encode()
        f.write(MAGIC + struct.pack("<I", VERSION))
        f.write(struct.pack("<I", len(name)) + name)
        f.write(struct.pack("<QQQ", fs.train_ft_in, trainer.cfg.ft_out, fs.max_active))
        f.write(struct.pack("<B", 1 if fs.ft_factorize else 0))
        f.write(struct.pack("<I", FEATURE_HASH[fs.name]))
        f.write(struct.pack("<I", len(rid)) + rid)
        f.write(struct.pack("<I", len(arch)) + arch.encode())
        f.write(struct.pack("<I", len(mode)) + mode.encode())
        f.write(struct.pack("<Q", len(topo)) + struct.pack("<%dQ" % len(topo), *topo))
        f.write(struct.pack("<QQQQ", superbatch, trainer.step_count, lr_horizon or 0, len(trainer.group_names)))
        for g in trainer.group_names:
            st = trainer.download_group(g, ("w", "m", "v", "slow"))
            f.write(struct.pack("<Q", st["w"].size))
            for k in ("w", "m", "v", "slow"):
                f.write(np.ascontiguousarray(st[k], "<f4").tobytes())
    os.replace(tmp, path)


def _read(f, n, what):
    b = f.read(n)
    if len(b) != n:
        raise TrainerError("raw checkpoint is truncated at %s" % what)
    return b


def read_raw_checkpoint_header(f) -> RawCkptHeader:
    if _read(f, 4, "magic") != MAGIC:
        raise TrainerError("raw checkpoint magic mismatch")
    version, = struct.unpack("<I", _read(f, 4, "version"))
    if version != VERSION:
        raise TrainerError("raw checkpoint version %d is not supported (this reader takes %d)" % (version, VERSION))
    n, = struct.unpack("<I", _read(f, 4, "feature set name length"))
    if n > 256:
        raise TrainerError("raw checkpoint feature set name length %d is implausible (max 256)" % n)
    fs_name = _read(f, n, "feature set name").decode()
    ft_in, ft_out, max_active = struct.unpack("<QQQ", _read(f, 24, "feature set dimensions"))
    fact, = struct.unpack("<B", _read(f, 1, "ft_factorize flag"))
    fhash, = struct.unpack("<I", _read(f, 4, "feature hash"))
    n, = struct.unpack("<I", _read(f, 4, "producer run id length"))
    if n > MAX_RUN_ID_BYTES:
        raise TrainerError("raw checkpoint producer run id length %d is implausible (max %d)" % (n, MAX_RUN_ID_BYTES))
    run_id = _read(f, n, "producer run id").decode() if n else None
    n, = struct.unpack("<I", _read(f, 4, "arch kind length"))
    arch = _read(f, n, "arch kind").decode()
    n, = struct.unpack("<I", _read(f, 4, "bucket mode length"))
    mode = _read(f, n, "bucket mode").decode()
    n, = struct.unpack("<Q", _read(f, 8, "topology count"))
    if n > 16:
        raise TrainerError("raw checkpoint topology count %d is implausible" % n)
    topo = struct.unpack("<%dQ" % n, _read(f, 8 * n, "topology"))
    sb, step, horizon, groups = struct.unpack("<QQQQ", _read(f, 32, "counters"))
    return RawCkptHeader(version, fs_name, ft_in, ft_out, max_active, bool(fact), fhash, run_id, arch, mode, tuple(topo), sb,
                         step, horizon or None, groups)


def load_raw_checkpoint(trainer, path: str, bucket_mode: Optional[str] = None) -> RawCkptHeader:
    """Restores weights, moments, slow weights and the step counter; returns the header (resume from
    header.superbatch + 1).  Refuses a file of another feature set, factorizer setting, architecture, bucket mode or
    layer shape, as the reference does."""
    arch, topo, mode, fs = _identity(trainer, bucket_mode)
    with open(path, "rb") as f:
        h = read_raw_checkpoint_header(f)
        if h.feature_set != fs.name:
            raise TrainerError("raw checkpoint feature set mismatch: checkpoint is '%s', requested '%s'" % (h.feature_set, fs.name))
        if h.ft_factorize != bool(fs.ft_factorize):
            raise TrainerError("raw checkpoint ft-factorize mismatch: checkpoint %s, requested %s" % (h.ft_factorize, fs.ft_factorize))
        if h.feature_hash != FEATURE_HASH[fs.name]:
            raise TrainerError("raw checkpoint feature hash mismatch: got %#010x, want %#010x" % (h.feature_hash, FEATURE_HASH[fs.name]))
        if h.train_ft_in != fs.train_ft_in:
            raise TrainerError("raw checkpoint ft_in mismatch: got %d, want %d" % (h.train_ft_in, fs.train_ft_in))
        if h.ft_out != trainer.cfg.ft_out:
            raise TrainerError("raw checkpoint ft_out mismatch: got %d, want %d" % (h.ft_out, trainer.cfg.ft_out))
        if h.max_active != fs.max_active and not (fs.ft_factorize and h.max_active == 2 * fs.max_active):
            raise TrainerError("raw checkpoint max_active mismatch: got %d, want %d" % (h.max_active, fs.max_active))
        if h.arch_kind != arch:
            raise TrainerError("raw checkpoint arch mismatch: checkpoint is '%s', requested '%s'" % (h.arch_kind, arch))
        if h.bucket_mode != mode:
            raise TrainerError("raw checkpoint bucket mode mismatch: checkpoint is '%s', requested '%s'" % (h.bucket_mode, mode))
        if h.topology != tuple(topo):
            raise TrainerError("raw checkpoint topology mismatch: got %s, want %s" % (h.topology, tuple(topo)))
        if h.num_groups != len(trainer.group_names):
            raise TrainerError("raw checkpoint has %d groups, the trainer %d" % (h.num_groups, len(trainer.group_names)))
        for g in trainer.group_names:
            n, = struct.unpack("<Q", _read(f, 8, "group length"))
            if n != trainer.group_len(g):
                raise TrainerError("raw checkpoint group '%s' has %d elements, the trainer %d" % (g, n, trainer.group_len(g)))
            arrs = [np.frombuffer(_read(f, 4 * n, "group " + g), "<f4") for _ in range(4)]
            trainer.upload_group(g, w=arrs[0], m=arrs[1], v=arrs[2], slow=arrs[3])
    trainer.step_count = h.step_count
    return h
