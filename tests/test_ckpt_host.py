"""Raw checkpoint (RNRC v8) byte layout, without a GPU: a stand-in trainer feeds the writer and the reader.

Expected bytes are packed by hand from the layout in the reference's bins/nnue_train/src/ckpt.rs:17-55.
"""
import struct
from types import SimpleNamespace

import numpy as np
import pytest

import tatara_b200 as tb
from tatara_b200 import _lib as L


class FakeTrainer:
    def __init__(self, fs, arch, F, l1, l2, nb, groups):
        self.feature_set = fs
        self.cfg = SimpleNamespace(arch=arch, ft_out=F, l1_out=l1, l2_out=l2, num_buckets=nb)
        self.group_names = list(groups)
        self.state = {g: {k: (np.arange(n, dtype=np.float32) + i * 0.25 + j) for j, k in enumerate(("w", "m", "v", "slow"))}
                      for i, (g, n) in enumerate(groups.items())}
        self.step_count = 41

    def group_len(self, g):
        return self.state[g]["w"].size

    def download_group(self, g, which):
        return {k: self.state[g][k].copy() for k in which}

    def upload_group(self, g, w=None, m=None, v=None, slow=None):
        for k, a in (("w", w), ("m", m), ("v", v), ("slow", slow)):
            self.state[g][k] = np.array(a, np.float32)


def test_rnrc_v8_bytes_and_round_trip(tmp_path):
    fs = tb.FEATURE_SETS["halfka-hm-merged"]
    groups = {"ft_w": 6, "ft_b": 2, "l1_w": 3}
    a = FakeTrainer(fs, L.ARCH_LAYERSTACK, 1536, 16, 32, 9, groups)
    path = str(tmp_path / "x.ckpt")
    tb.save_raw_checkpoint(a, path, superbatch=7, run_id="run-1", lr_horizon=None)
    raw = open(path, "rb").read()
    name = b"halfka-hm-merged"
    want = b"RNRC" + struct.pack("<I", 8) + struct.pack("<I", len(name)) + name
    want += struct.pack("<QQQ", 74934, 1536, 40) + b"\x01" + struct.pack("<I", 0x7F134CB8)
    want += struct.pack("<I", 5) + b"run-1" + struct.pack("<I", 10) + b"layerstack" + struct.pack("<I", 9) + b"kingrank9"
    want += struct.pack("<Q", 4) + struct.pack("<4Q", 1536, 16, 32, 9) + struct.pack("<QQQQ", 7, 41, 0, 3)
    assert raw[:len(want)] == want
    body = raw[len(want):]
    n0, = struct.unpack("<Q", body[:8])
    assert n0 == 6 and np.array_equal(np.frombuffer(body[8:8 + 24], "<f4"), a.state["ft_w"]["w"])
    assert len(body) == sum(8 + 16 * n for n in groups.values())
    b = FakeTrainer(fs, L.ARCH_LAYERSTACK, 1536, 16, 32, 9, groups)
    for g in groups:
        for k in b.state[g]:
            b.state[g][k][:] = -1
    b.step_count = 0
    h = tb.load_raw_checkpoint(b, path)
    assert (h.version, h.superbatch, h.step_count, h.lr_horizon, h.run_id, h.num_groups) == (8, 7, 41, None, "run-1", 3)
    assert b.step_count == 41
    for g in groups:
        for k in ("w", "m", "v", "slow"):
            assert np.array_equal(a.state[g][k], b.state[g][k])


def test_rnrc_reader_rejects_mismatches(tmp_path):
    fs = tb.FEATURE_SETS["halfkp"]
    groups = {"ft_w": 4}
    a = FakeTrainer(fs, L.ARCH_SIMPLE, 256, 32, 32, 0, groups)
    path = str(tmp_path / "s.ckpt")
    tb.save_raw_checkpoint(a, path, superbatch=1)
    hdr = tb.read_raw_checkpoint_header(open(path, "rb"))
    assert (hdr.arch_kind, hdr.bucket_mode, hdr.topology, hdr.feature_hash) == ("simple", "", (256, 32, 32), 0x5D69D5B8)
    cases = [
        (FakeTrainer(tb.FEATURE_SETS["halfka-hm-merged"], L.ARCH_SIMPLE, 256, 32, 32, 0, groups), "feature set mismatch"),
        (FakeTrainer(fs.with_factorize(False), L.ARCH_SIMPLE, 256, 32, 32, 0, groups), "ft-factorize mismatch"),
        (FakeTrainer(fs, L.ARCH_SIMPLE, 512, 32, 32, 0, groups), "ft_out mismatch"),
        (FakeTrainer(fs, L.ARCH_LAYERSTACK, 256, 32, 32, 9, groups), "arch mismatch"),
        (FakeTrainer(fs, L.ARCH_SIMPLE, 256, 16, 32, 0, groups), "topology mismatch"),
        (FakeTrainer(fs, L.ARCH_SIMPLE, 256, 32, 32, 0, {"ft_w": 5}), "has 4 elements"),
    ]
    for t, msg in cases:
        with pytest.raises(tb.TrainerError, match=msg):
            tb.load_raw_checkpoint(t, path)
    raw = bytearray(open(path, "rb").read())
    open(path, "wb").write(bytes(raw[:-3]))
    with pytest.raises(tb.TrainerError, match="truncated"):
        tb.load_raw_checkpoint(FakeTrainer(fs, L.ARCH_SIMPLE, 256, 32, 32, 0, groups), path)
    raw[4] = 9
    open(path, "wb").write(bytes(raw))
    with pytest.raises(tb.TrainerError, match="version 9"):
        tb.load_raw_checkpoint(FakeTrainer(fs, L.ARCH_SIMPLE, 256, 32, 32, 0, groups), path)
    raw[0] = ord("X")
    open(path, "wb").write(bytes(raw))
    with pytest.raises(tb.TrainerError, match="magic"):
        tb.load_raw_checkpoint(FakeTrainer(fs, L.ARCH_SIMPLE, 256, 32, 32, 0, groups), path)
