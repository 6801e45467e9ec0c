"""The CPU oracle's decoder / feature extractors against the committed golden fixtures.

tests/golden/sample_psv.bin is the reference's real 100-record fixture; the expected outputs were
computed by the independent pure-Python implementation in tests/golden/make_golden.py (the index
formulas of the reference's own integration test).  CPU only.
"""
import os

import numpy as np

import oracle_lib as O
from helpers import GOLDEN, sort_rows

RAW = open(os.path.join(GOLDEN, "sample_psv.bin"), "rb").read()
EXP = np.load(os.path.join(GOLDEN, "sample_psv_expected.npz"))


def test_fixture_shape():
    # crates/shogi-format/tests/psv_smoke.rs: sample_has_expected_size, read_one_batch_of_psv_records
    assert len(RAW) == 100 * 40
    b = O.psv_to_batch("halfkp", RAW)
    assert (np.abs(b["score"]) <= 32600).all()
    assert set(np.unique(b["wdl"]).tolist()) <= {0.0, 0.5, 1.0}


def test_halfkp_indices_match_reference_formula():
    # crates/shogi-features/tests/feature_set.rs: halfkp matches oracle_halfkp on sample.psv (sorted sets)
    b = O.psv_to_batch("halfkp", RAW)
    assert (b["nnz"] == EXP["nnz_kp"]).all()
    assert (sort_rows(b["stm"]) == EXP["kp_stm"]).all()
    assert (sort_rows(b["nstm"]) == EXP["kp_nstm"]).all()
    assert b["stm"].max() < 125_388 and b["nstm"].max() < 125_388


def test_halfka_hm_merged_indices_match_reference_formula():
    b = O.psv_to_batch("halfka-hm-merged", RAW)
    assert (b["nnz"] == EXP["nnz_hm"]).all()
    assert (sort_rows(b["stm"]) == EXP["hm_stm"]).all()
    assert (sort_rows(b["nstm"]) == EXP["hm_nstm"]).all()
    assert b["stm"].max() < 73_305 and b["nstm"].max() < 73_305


def test_targets_and_buckets():
    b = O.psv_to_batch("halfka-hm-merged", RAW)
    assert (b["bucket"] == EXP["bucket"]).all()
    assert (b["score"] == EXP["score"]).all()
    assert (b["wdl"] == EXP["wdl"]).all()


def test_emission_order_board_then_kings_then_hands():
    # feature_set.rs:655-808: within the board phase the index order follows (piece type, colour, square);
    # king features come next; the stm row is not sorted in general
    b = O.psv_to_batch("halfka-hm-merged", RAW)
    PI = 1629
    for r in range(100):
        row = b["stm"][r, :b["nnz"][r]] % PI
        kings = np.where((row >= 1548))[0]
        assert len(kings) == 2 and kings[1] == kings[0] + 1      # friend king then (folded) enemy king
        assert (row[:kings[0]] >= 90).all() and (row[:kings[0]] < 1548).all()   # board pieces first
        assert (row[kings[1] + 1:] < 90).all()                                   # hand pieces last


def test_all_five_feature_sets_respect_their_dimensions():
    # crates/shogi-features/src/feature_set.rs: extract_active_features_matches_map_features_board runs
    # all five public sets over the fixture
    for name in O.FEATURE_SETS:
        d = O.feature_dims(name)
        b = O.psv_to_batch(name, RAW)
        assert b["nnz"].max() <= d["max_active"]
        for key in ("stm", "nstm"):
            valid = b[key][b[key] >= 0]
            assert valid.max() < d["ft_in"]


def test_synthetic_generator_of_the_oracle_equals_the_library_generator():
    """Both generators follow the same documented draw order: byte-identical records; decode(encode(x)) == x."""
    import tatara_b200 as tb
    for seed, n in ((tb.SYNTH_SEED + 3, 4096), (1, 333)):
        a = tb.synthesize_psv(seed, n)
        b = O.synthesize_psv(seed, n)
        assert np.array_equal(a, b)
    rec = O.synthesize_psv(5, 64)
    for r in rec:
        board = O.Board()
        O.lib().ora_psv_decode(np.ascontiguousarray(r), board)
        again = np.zeros(40, np.uint8)
        assert O.lib().ora_psv_encode(board, again) == 0
        assert np.array_equal(again, r)
