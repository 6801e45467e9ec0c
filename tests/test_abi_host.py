"""CPU-only checks of the C-ABI library: it loads, exports every declared symbol, its host-side
functions (PSV encoder / synthetic generator / weight initialiser) agree with the oracle, and the
device entry points fail with an error value (never a crash) when no GPU is present.
"""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle_lib as O
import tatara_b200 as tb
from tatara_b200 import _lib as L
from helpers import GOLDEN, ROOT


def test_library_exports_every_declared_symbol():
    lib = tb.load_library()
    header = open(os.path.join(ROOT, "include", "tatara_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(tb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(lib, name), "library does not export %s" % name
    assert declared == set(L.SIGNATURES), declared ^ set(L.SIGNATURES)
    assert lib.tb_version().startswith(b"tatara_b200")


def test_config_struct_matches_header_layout():
    # 15 int32 + 6 float + 2 int32 + 128 bytes + 2 int32
    assert C.sizeof(L.Config) == 15 * 4 + 6 * 4 + 2 * 4 + 128 + 8
    assert C.sizeof(L.Loss) == 11 * 4


def test_synthetic_records_decode_to_full_piece_sets():
    n = 512
    psv = tb.synthesize_psv(tb.SYNTH_SEED, n)
    again = tb.synthesize_psv(tb.SYNTH_SEED, n)
    assert (psv == again).all(), "generator is not deterministic"
    assert (tb.synthesize_psv(tb.SYNTH_SEED + 1, n) != psv).any()
    for fs, nnz in (("halfkp", 38), ("halfka-hm-merged", 40)):
        b = O.psv_to_batch(fs, psv.tobytes())
        assert (b["nnz"] == nnz).all()          # 38 non-king pieces (+ 2 king features)
        assert (b["stm"] >= 0).all() and (b["nstm"] >= 0).all()
    b = O.psv_to_batch("halfka-hm-merged", psv.tobytes())
    assert np.abs(b["score"]).max() <= 3000 and 250 < b["score"].std() < 550
    assert set(np.unique(b["wdl"]).tolist()) == {0.0, 0.5, 1.0}
    assert set(np.unique(b["bucket"]).tolist()) <= set(range(9)) and len(np.unique(b["bucket"])) == 9
    ply = psv[:, 36].astype(int) + 256 * psv[:, 37].astype(int)
    assert ply.min() >= 1 and ply.max() <= 256
    assert (psv[:, 34:36] == 0).all() and (psv[:, 39] == 0).all()
    # every record uses all 256 bits: hands + board hold exactly 38 pieces
    for r in range(16):
        bd = O.Board()
        O.lib().ora_psv_decode(np.ascontiguousarray(psv[r]), C.byref(bd))
        on_board = sum(1 for s in range(81) if bd.board_pt[s] not in (0, 8))
        in_hand = sum(bd.hand[c][k] for c in range(2) for k in range(7))
        assert on_board + in_hand == 38 and bd.black_king_sq != bd.white_king_sq


def _reencode(rec):
    bd = O.Board()
    O.lib().ora_psv_decode(np.ascontiguousarray(rec), C.byref(bd))
    pt = np.array(list(bd.board_pt), np.uint8); col = np.array(list(bd.board_color), np.uint8)
    hb = np.array(list(bd.hand[0]), np.uint8); hw = np.array(list(bd.hand[1]), np.uint8)
    out = np.zeros(40, np.uint8)
    rc = tb.load_library().tb_psv_encode(pt.ctypes.data, col.ctypes.data, hb.ctypes.data, hw.ctypes.data,
                                         bd.side_to_move, bd.black_king_sq, bd.white_king_sq, bd.score, bd.ply,
                                         bd.result, out.ctypes.data)
    assert rc == 0
    return out, bd


def test_encoder_inverts_the_decoder():
    # synthetic records: decode -> encode reproduces the bytes (the generator writes hand pieces grouped by
    # owner and type only by chance, so compare decoded boards, and bytes for the board part)
    psv = tb.synthesize_psv(123, 64)
    for rec in psv:
        out, bd = _reencode(rec)
        bd2 = O.Board()
        O.lib().ora_psv_decode(out, C.byref(bd2))
        assert bytes(bd) == bytes(bd2)
        assert (out[32:] == rec[32:]).all()
    # the reference's real fixture: positions survive decode -> encode -> decode, move16 aside
    raw = np.frombuffer(open(os.path.join(GOLDEN, "sample_psv.bin"), "rb").read(), np.uint8).reshape(100, 40)
    same_bytes = 0
    for rec in raw:
        out, bd = _reencode(rec)
        bd2 = O.Board()
        O.lib().ora_psv_decode(out, C.byref(bd2))
        assert bytes(bd) == bytes(bd2)
        same_bytes += int((out[:32] == rec[:32]).all())
    assert same_bytes >= 1   # identical bit streams whenever the file's hand-piece order is the encoder's


def test_init_sampler_matches_oracle():
    lib = tb.load_library()
    for n, nb, fan, dist, kind, val, rep, seed in ((37, 1, 99, 1, 0, 0.01, 0, 0x100), (1024, 1, 73305, 1, 1, 1.0, 0, 0xABCD),
                                                   (90, 9, 5, 1, 0, 0.5, 1, 7), (16, 1, 1, 0, 0, 0.0, 0, 0)):
        a = np.full(n, 7, np.float32); b = np.full(n, 9, np.float32)
        assert lib.tb_init_sample(a.ctypes.data, n, nb, fan, dist, kind, val, rep, seed) == 0
        O.lib().ora_init_sample(b, n, nb, fan, dist, kind, val, rep, seed)
        assert (a == b).all()


def test_default_init_matches_oracle_defaults():
    fs = tb.FEATURE_SETS["halfkp"]
    fs_small = tb.FeatureSetSpec("tiny", 0, 3, 4, 38, True)
    init = tb.simple_default_init(fs_small, 128, 8, 8)
    ot = O.OracleTrainer(arch="simple", ft_in=fs_small.ft_in, piece_inputs=4, factorize=True, max_active=38, ft_out=128,
                         l1=8, l2=8, capacity=16)
    ot.init_default()
    for name in ot.names:
        assert (init[name] == ot.group(name)).all(), name
    fs_ls = tb.FeatureSetSpec("tiny", 4, 5, 6, 40, True)
    init = tb.layerstack_default_init(fs_ls, 256, 16, 32, 9)
    ot = O.OracleTrainer(arch="layerstack", ft_in=fs_ls.ft_in, piece_inputs=6, factorize=True, max_active=40, ft_out=256,
                         l1=16, l2=32, num_buckets=9, capacity=16)
    ot.init_default()
    for name in ot.names:
        assert (init[name] == ot.group(name)).all(), name
    assert fs.ft_in == 125_388 and tb.FEATURE_SETS["halfka-hm-merged"].train_ft_in == 74_934


def test_invalid_config_is_an_error_value():
    lib = tb.load_library()
    h = L.vp()
    cfg = L.Config()
    assert lib.tb_create(C.byref(cfg), C.byref(h)) != 0          # struct_size 0
    assert b"struct_size" in lib.tb_last_error(None)
    cfg.struct_size = C.sizeof(L.Config)
    cfg.arch, cfg.batch_capacity, cfg.ft_in, cfg.piece_inputs, cfg.max_active = 0, 24, 100, 10, 40
    cfg.ft_out, cfg.l1_out, cfg.l2_out, cfg.num_buckets, cfg.world_size = 256, 16, 32, 9, 1
    assert lib.tb_create(C.byref(cfg), C.byref(h)) == -1 and b"multiple of 16" in lib.tb_last_error(None)
    cfg.batch_capacity = 32
    cfg.ft_out = 200
    assert lib.tb_create(C.byref(cfg), C.byref(h)) == -1 and b"ft_out" in lib.tb_last_error(None)
    cfg.ft_out = 256
    cfg.num_buckets = 12
    assert lib.tb_create(C.byref(cfg), C.byref(h)) == -1 and b"num_buckets" in lib.tb_last_error(None)
    cfg.num_buckets = 9
    cfg.precision = 4     # ft_fp16_out without ft_fp16 (trainer_layerstack.rs:801-805)
    assert lib.tb_create(C.byref(cfg), C.byref(h)) == -1 and b"ft-fp16-out" in lib.tb_last_error(None)


@pytest.mark.skipif(tb.load_library().tb_device_count() > 0, reason="only meaningful without a GPU")
def test_no_gpu_means_error_not_fallback():
    with pytest.raises(tb.TrainerError) as e:
        tb.SimpleGpuTrainer(16, 128, 8, 8, tb.FeatureSetSpec("tiny", 0, 3, 4, 38, False), init=None)
    assert "CUDA device" in str(e.value) or "failed" in str(e.value)
    psv = tb.synthesize_psv(1, 16)
    with pytest.raises(tb.TrainerError):
        tb.extract_batch(psv, tb.FEATURE_SETS["halfkp"])
