"""Generates the golden fixtures of tests/golden/ from the reference checkout.

    python tests/golden/make_golden.py /path/to/reference

Outputs (committed):
  sample_psv.bin          the reference's real 100-record PackedSfenValue fixture
                          (crates/shogi-format/tests/data/sample.psv), the input vector
  sample_psv_expected.npz expected outputs for it, computed HERE by an independent pure-Python
                          decoder and the index formulas that the reference's own integration test uses as
                          its oracle (crates/shogi-features/tests/feature_set.rs:125-200: halfkp =
                          king_sq * 1548 + bonapiece; the merged/mirrored variant per
                          crates/shogi-features/src/halfka_hm.rs), compared as sorted index sets like that
                          test does, plus kingrank9 buckets, scores and results.

Neither file is produced by the C oracle or the CUDA library: they pin both.
"""
import os
import sys

import numpy as np

HUFF = [(0x00, 1, 0), (0x01, 2, 1), (0x03, 4, 2), (0x0B, 4, 3), (0x07, 4, 4), (0x1F, 6, 5), (0x3F, 6, 6), (0x0F, 5, 7)]
PROMOTE = {1: 9, 2: 10, 3: 11, 4: 12, 5: 13, 6: 14}
# BonaPiece bases (crates/shogi-format/src/bona_piece.rs:13-57): (friend, enemy)
BOARD_BASE = {1: (90, 171), 2: (252, 333), 3: (414, 495), 4: (576, 657), 7: (738, 819), 5: (900, 981), 13: (1062, 1143),
              6: (1224, 1305), 14: (1386, 1467), 9: (738, 819), 10: (738, 819), 11: (738, 819), 12: (738, 819)}
HAND_BASE = {1: (1, 20), 2: (39, 44), 3: (49, 54), 4: (59, 64), 7: (69, 74), 5: (79, 82), 6: (85, 88)}
F_KING, E_KING = 1548, 1629


def decode(rec):
    bits = [(rec[i >> 3] >> (i & 7)) & 1 for i in range(256)]
    cur = 0

    def take(n):
        nonlocal cur
        v = 0
        for i in range(n):
            v |= bits[cur + i] << i if cur + i < 256 else 0
        cur += n
        return v

    def peek(n):
        v = 0
        for i in range(n):
            if cur + i < 256:
                v |= bits[cur + i] << i
        return v

    stm = take(1)
    bk, wk = take(7), take(7)
    board = {}
    for sq in range(81):
        if sq in (bk, wk):
            continue
        p = peek(6)
        for pat, ln, pt in HUFF:
            if p & ((1 << ln) - 1) == pat:
                break
        cur += ln
        if pt == 0:
            continue
        promoted = take(1) if pt != 7 else 0
        color = take(1)
        board[sq] = (PROMOTE[pt] if promoted else pt, color)
    hands = {0: {}, 1: {}}
    while cur < 256:
        p = peek(5)
        for pat, ln, pt in HUFF[1:]:
            if p & ((1 << (ln - 1)) - 1) == pat >> 1:
                break
        cur += ln - 1
        box = take(1) if pt != 7 else 0
        color = take(1)
        if not box:
            hands[color][pt] = hands[color].get(pt, 0) + 1
    score = int(np.frombuffer(bytes(rec[32:34]), "<i2")[0])
    result = int(np.frombuffer(bytes(rec[38:39]), "i1")[0])
    return stm, bk, wk, board, hands, score, result


def features(stm, bk, wk, board, hands, merged_hm):
    """Sorted (stm, nstm) index lists: halfkp, or halfka with merged king plane and file mirroring."""
    out = []
    for persp in (stm, 1 - stm):
        king = bk if persp == 0 else wk
        ksq = king if persp == 0 else 80 - king
        mirror = False
        if merged_hm:
            f, r = divmod(ksq, 9)
            mirror = f >= 5
            kb, pi = (8 - f if mirror else f) * 9 + r, 1629
        else:
            kb, pi = ksq, 1548

        def pack(bp):
            if mirror and bp >= 90:
                piece, sq = divmod(bp - 90, 81)
                bp = 90 + piece * 81 + (8 - sq // 9) * 9 + sq % 9
            if merged_hm and bp >= E_KING:
                bp -= 81
            return kb * pi + bp

        idx = []
        for sq, (pt, color) in board.items():
            base = BOARD_BASE[pt][0 if color == persp else 1]
            idx.append(pack(base + (sq if persp == 0 else 80 - sq)))
        if merged_hm:
            other = wk if persp == 0 else bk
            idx.append(pack(F_KING + ksq))
            idx.append(pack(E_KING + (other if persp == 0 else 80 - other)))
        for owner in (0, 1):
            for pt, cnt in hands[owner].items():
                for i in range(cnt):
                    idx.append(pack(HAND_BASE[pt][0 if owner == persp else 1] + i))
        out.append(sorted(idx))
    return out


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of the reference project>")
    ref = sys.argv[1]
    here = os.path.dirname(os.path.abspath(__file__))
    raw = open(os.path.join(ref, "crates/shogi-format/tests/data/sample.psv"), "rb").read()
    assert len(raw) == 4000
    open(os.path.join(here, "sample_psv.bin"), "wb").write(raw)
    recs = np.frombuffer(raw, np.uint8).reshape(100, 40)
    exp = {k: [] for k in ("kp_stm", "kp_nstm", "hm_stm", "hm_nstm", "bucket", "score", "wdl", "nnz_kp", "nnz_hm")}
    for rec in recs:
        stm, bk, wk, board, hands, score, result = decode(rec.tolist())
        kp = features(stm, bk, wk, board, hands, False)
        hm = features(stm, bk, wk, board, hands, True)
        pad = lambda l, n: l + [-1] * (n - len(l))
        exp["kp_stm"].append(pad(kp[0], 38)); exp["kp_nstm"].append(pad(kp[1], 38))
        exp["hm_stm"].append(pad(hm[0], 40)); exp["hm_nstm"].append(pad(hm[1], 40))
        exp["nnz_kp"].append(len(kp[0])); exp["nnz_hm"].append(len(hm[0]))
        friendly, enemy = (bk, 80 - wk) if stm == 0 else (80 - wk, bk)
        exp["bucket"].append((friendly % 9) // 3 * 3 + (enemy % 9) // 3)
        exp["score"].append(float(score))
        exp["wdl"].append(1.0 if result > 0 else (0.0 if result < 0 else 0.5))
    np.savez_compressed(os.path.join(here, "sample_psv_expected.npz"),
                        **{k: np.array(v, np.float32 if k in ("score", "wdl") else np.int32) for k, v in exp.items()})
    print("wrote sample_psv.bin, sample_psv_expected.npz")


if __name__ == "__main__":
    main()
