"""Pins the CPU oracle to the literal vectors of the reference's own unit tests.

Each test names the reference test it restates (file and test function, paths relative to
the reference project root).  Runs on CPU only.
"""
import ctypes as C

import numpy as np
import pytest

from oracle_lib import lib, Board

f32 = np.float32


def A(x, dt=np.float32):
    return np.ascontiguousarray(np.array(x, dtype=dt))


# ---------------------------------------------------------------- sparse forward / backward
def test_sparse_fwd_matches_reference_evaluate_test():
    # crates/gpu-kernels/src/sparse/sparse_ft_forward.rs: matches_reference_evaluate_test
    w = A([0, 1, 2, 3, 4, 5]); idx = A([0, 1, -1, -1, 2, 2, 1, 0], np.int32); out = np.zeros(4, f32)
    lib().ora_sparse_ft_forward(w, idx, A([2, 4], np.int32), out, 2, 2, 3, 4)
    assert out.tolist() == [2.0, 4.0, 10.0, 14.0]


def test_sparse_fwd_edge_cases():
    # sparse_ft_forward.rs: all_padding_yields_zero, out_of_range_index_is_silently_skipped,
    # duplicate_indices_are_summed, zero_dimension_is_no_op
    L = lib()
    out = A([999, 999])
    L.ora_sparse_ft_forward(A([1, 2, 3, 4]), A([-1] * 6, np.int32), A([6], np.int32), out, 1, 2, 2, 6)
    assert out.tolist() == [0.0, 0.0]
    out = np.zeros(2, f32)
    L.ora_sparse_ft_forward(A([1, 2, 3, 4]), A([0, 5, -1], np.int32), A([3], np.int32), out, 1, 2, 2, 3)
    assert out.tolist() == [1.0, 2.0]
    out = np.zeros(2, f32)
    L.ora_sparse_ft_forward(A([1, 10, 2, 20]), A([0, 0, 1], np.int32), A([3], np.int32), out, 1, 2, 2, 3)
    assert out.tolist() == [4.0, 40.0]
    out = A([999, 999])
    L.ora_sparse_ft_forward(A([1, 2]), np.zeros(0, np.int32), A([0], np.int32), out, 1, 2, 1, 0)
    assert out.tolist() == [0.0, 0.0]


def test_sparse_bwd_matches_reference_evaluate_bwd_test():
    # sparse_ft_backward.rs: matches_reference_evaluate_bwd_test
    g = np.zeros(9, f32)
    lib().ora_sparse_ft_backward(A([0, 1, 2, 3, 4, 5]), A([0, 1, -1, -1, 2, 2, 1, 0], np.int32), g, 2, 3, 3, 4)
    assert g.tolist() == [3, 5, 7, 3, 5, 7, 6, 8, 10]


def test_sparse_bwd_edge_cases():
    # sparse_ft_backward.rs: all_padding..., out_of_range..., duplicate..., accumulates_into_existing...
    L = lib()
    g = np.zeros(6, f32)
    L.ora_sparse_ft_backward(A([1, 2, 3]), A([-1] * 4, np.int32), g, 1, 3, 2, 4)
    assert g.tolist() == [0] * 6
    g = np.zeros(4, f32)
    L.ora_sparse_ft_backward(A([1, 1]), A([0, 5, -1], np.int32), g, 1, 2, 2, 3)
    assert g.tolist() == [1, 1, 0, 0]
    g = np.zeros(4, f32)
    L.ora_sparse_ft_backward(A([10, 20]), A([0, 0, 1], np.int32), g, 1, 2, 2, 3)
    assert g.tolist() == [20, 40, 10, 20]
    g = A([1.0])
    L.ora_sparse_ft_backward(A([5.0]), A([0], np.int32), g, 1, 1, 1, 1)
    assert g.tolist() == [6.0]


def test_sparse_forward_backward_consistency():
    # sparse_ft_backward.rs: forward_backward_consistency
    L = lib()
    w = A([0, 1, 2, 3, 4, 5]); idx = A([0, 1, -1, -1, 2, 2, 1, 0], np.int32)
    out = np.zeros(4, f32)
    L.ora_sparse_ft_forward(w, idx, A([4, 4], np.int32), out, 2, 2, 3, 4)
    g = np.zeros(6, f32)
    L.ora_sparse_ft_backward(out, idx, g, 2, 2, 3, 4)
    assert g.tolist() == [12, 18, 12, 18, 20, 28]


def test_factorizer_fold_and_reduce_equal_virtual_index_semantics():
    # crates/gpu-kernels/src/sparse/ft_factorize.rs: fold_forward_matches_virtual_index_forward and
    # reduce_backward_matches_virtual_index_backward (fixture ft_in=6 = 3 king buckets x pi=2, ft_out=4)
    L = lib()
    FT_IN, FT_OUT, PI = 6, 4, 2
    rows = FT_IN + PI
    w = A([((i * 37 % 101) - 50.0) * 0.013 for i in range(rows * FT_OUT)])
    comb = np.zeros(FT_IN * FT_OUT, f32)
    L.ora_ft_fold_virtual(w, comb, FT_IN, FT_OUT, PI)
    real = [0, 4, 5, 2, 3, -1]
    train = []
    for p in range(2):
        row = real[p * 3:(p + 1) * 3]
        train += row + [FT_IN + i % PI if i >= 0 else -1 for i in row]
    real = A(real, np.int32); train = A(train, np.int32)
    out_fold = np.zeros(2 * FT_OUT, f32); out_virt = np.zeros(2 * FT_OUT, f32)
    L.ora_sparse_ft_forward(comb, real, A([3, 3], np.int32), out_fold, 2, FT_OUT, FT_IN, 3)
    L.ora_sparse_ft_forward(w, train, A([6, 6], np.int32), out_virt, 2, FT_OUT, rows, 6)
    np.testing.assert_allclose(out_fold, out_virt, rtol=0, atol=1e-6)
    # backward: reduce(real-index backward) == virtual-index backward
    dy = A([0.1 * i - 0.3 for i in range(2 * FT_OUT)])
    g1 = np.zeros(rows * FT_OUT, f32)
    L.ora_sparse_ft_backward(dy, real, g1, 2, FT_OUT, FT_IN, 3)
    L.ora_ft_reduce_virtual_grad(g1, FT_IN, FT_OUT, PI)
    g2 = np.zeros(rows * FT_OUT, f32)
    L.ora_sparse_ft_backward(dy, train, g2, 2, FT_OUT, rows, 6)
    np.testing.assert_allclose(g1, g2, rtol=0, atol=1e-6)


def test_factorizer_fold_and_reduce_cell_by_cell():
    # crates/gpu-kernels/src/sparse/ft_factorize.rs: fold_adds_matching_virtual_row, reduce_sums_over_king_buckets
    L = lib()
    FT_IN, FT_OUT, PI = 6, 4, 2
    rows = FT_IN + PI
    w = A([((i * 37 % 101) - 50.0) * 0.013 for i in range(rows * FT_OUT)])
    comb = np.zeros(FT_IN * FT_OUT, f32)
    L.ora_ft_fold_virtual(w, comb, FT_IN, FT_OUT, PI)
    for feat in range(FT_IN):
        for ri in range(FT_OUT):
            assert comb[feat * FT_OUT + ri] == w[feat * FT_OUT + ri] + w[(FT_IN + feat % PI) * FT_OUT + ri]
    grad = A([float(i) for i in range(rows * FT_OUT)])
    real = grad[:FT_IN * FT_OUT].copy()
    L.ora_ft_reduce_virtual_grad(grad, FT_IN, FT_OUT, PI)
    assert np.array_equal(grad[:FT_IN * FT_OUT], real)                      # the real block is untouched
    for p in range(PI):
        for ri in range(FT_OUT):
            want = f32(0)
            for kb in range(FT_IN // PI):
                want = f32(want + f32((kb * PI + p) * FT_OUT + ri))
            assert grad[(FT_IN + p) * FT_OUT + ri] == want


# ---------------------------------------------------------------- pairwise FT post
SCALE = f32(127.0) / f32(128.0)


def test_ft_post_forward_hand_computed():
    # crates/gpu-kernels/src/layerstack/ft_post_perspective.rs: forward_hand_computed_scale_one,
    # forward_bias_and_clamp
    L = lib()
    c = np.zeros(4, f32)
    L.ora_ft_post_perspective_fwd(A([0.5, 0.25, 2.0, -1.0]), A([0.8, 0.1, 0.3, 0.9]), np.zeros(4, f32), c, 1, 4, 1.0)
    exp = [f32(0.5) * f32(1.0), f32(0.25) * f32(0.0), f32(0.8) * f32(0.3), f32(0.1) * f32(0.9)]
    assert c.tolist() == [float(e) for e in exp]
    bias = A([0.5, 0.5])
    c1 = np.zeros(2, f32)
    L.ora_ft_post_perspective_fwd(A([10.0, -10.0]), A([0.0, 0.0]), bias, c1, 1, 2, SCALE)
    assert c1[0] == 0.0 and c1[1] == f32(0.25) * SCALE
    c2 = np.zeros(2, f32)
    L.ora_ft_post_perspective_fwd(A([0.5, 0.5]), A([0.5, 0.5]), bias, c2, 1, 2, SCALE)
    assert c2[0] == SCALE and c2[1] == SCALE


def test_ft_post_grad_hand_computed():
    # ft_post_perspective.rs: grad_hand_computed_interior, grad_zeroed_at_saturation,
    # grad_nstm_offset_reads_second_half_of_d_combined
    L = lib()
    g = np.zeros(2, f32); gb = np.zeros(2, f32)
    L.ora_ft_post_perspective_grad(A([3.0, 999.0]), A([0.5, 0.25]), np.zeros(2, f32), g, gb, 1, 2, 0, 2, 1.0)
    assert g.tolist() == [0.75, 1.5] and gb.tolist() == [0.75, 1.5]
    g = np.zeros(2, f32); gb = A([7.0, 8.0])
    L.ora_ft_post_perspective_grad(A([10.0, 0.0]), A([-1.0, 5.0]), np.zeros(2, f32), g, gb, 1, 2, 0, 2, 1.0)
    assert g.tolist() == [0.0, 0.0] and gb.tolist() == [7.0, 8.0]
    g = np.zeros(4, f32); gb = np.zeros(4, f32)
    L.ora_ft_post_perspective_grad(A([1.0, 2.0, 10.0, 20.0]), A([0.5] * 4), np.zeros(4, f32), g, gb, 1, 4, 2, 4, 1.0)
    assert g.tolist() == [5.0, 10.0, 5.0, 10.0] and gb.tolist() == [5.0, 10.0, 5.0, 10.0]


# ---------------------------------------------------------------- dense layers
def test_dense_mm_hand_computed():
    # crates/gpu-kernels/src/layerstack/dense_mm.rs: forward_hand_computed, bwd_input_hand_computed,
    # bwd_weight_hand_computed, bias_grad_accumulates
    L = lib()
    y = np.zeros(4, f32)
    L.ora_dense_mm_fwd(A([1, 2, 3, 4]), A([5, 6, 7, 8]), A([10, 20]), y, 2, 2, 2)
    assert y.tolist() == [29, 42, 53, 70]
    dx = np.zeros(4, f32)
    L.ora_dense_mm_bwd_input(A([1, 1, 1, 1]), A([5, 6, 7, 8]), dx, 2, 2, 2)
    assert dx.tolist() == [11, 15, 11, 15]
    dw = A([999] * 4)
    L.ora_dense_mm_bwd_weight(A([1, 2, 3, 4]), A([10, 20, 30, 40]), dw, 2, 2, 2)
    assert dw.tolist() == [100, 140, 140, 200]
    gb = A([1, 2])
    L.ora_bias_grad(A([10, 20, 30, 40]), gb, 2, 2)
    assert gb.tolist() == [41, 62]


def test_dense_mm_bucket_hand_computed():
    # crates/gpu-kernels/src/layerstack/dense_mm_bucket.rs: forward_hand_computed,
    # forward_out_of_range_bucket_yields_zero, bwd_input_hand_computed, bwd_input_out_of_range_yields_zero,
    # bwd_weight_hand_computed, bwd_weight_out_of_range_position_ignored, bias_grad_bucket_*
    L = lib()
    w = A([1, 2, 3, 4]); bias = A([10, 20])
    y = np.zeros(2, f32)
    L.ora_dense_mm_fwd_bucket(A([1, 1, 2, 2]), w, bias, A([0, 1], np.int32), y, 2, 2, 1, 2)
    assert y.tolist() == [13, 34]
    for bad in (-1, 2):
        y = A([999])
        L.ora_dense_mm_fwd_bucket(A([5, 5]), w, bias, A([bad], np.int32), y, 1, 2, 1, 2)
        assert y.tolist() == [0]
    dx = np.zeros(4, f32)
    L.ora_dense_mm_bwd_input_bucket(A([1, 1]), w, A([0, 1], np.int32), dx, 2, 2, 1, 2)
    assert dx.tolist() == [1, 2, 3, 4]
    dx = A([7, 7])
    L.ora_dense_mm_bwd_input_bucket(A([1]), w, A([-5], np.int32), dx, 1, 2, 1, 2)
    assert dx.tolist() == [0, 0]
    gw = A([-1] * 4)
    L.ora_dense_mm_bwd_weight_bucket(A([1, 1, 2, 2, 3, 3]), A([10, 20, 30]), A([0, 0, 1], np.int32), gw, 3, 2, 1, 2)
    assert gw.tolist() == [50, 50, 90, 90]
    gw = np.zeros(4, f32)
    L.ora_dense_mm_bwd_weight_bucket(A([1, 1, 100, 100]), A([10, 10]), A([0, -1], np.int32), gw, 2, 2, 1, 2)
    assert gw.tolist() == [10, 10, 0, 0]
    gb = A([10, 20, 30, 40])
    L.ora_bias_grad_bucket(A([1, 2, 3, 4, 5, 6]), A([0, 1, 0], np.int32), gb, 3, 2, 2)
    assert gb.tolist() == [16, 28, 33, 44]
    gb = np.zeros(4, f32)
    L.ora_bias_grad_bucket(A([1, 2, 99, 99]), A([0, 9], np.int32), gb, 2, 2, 2)
    assert gb.tolist() == [1, 2, 0, 0]


def test_elementwise_glue():
    # crelu.rs, abs_pow2_scale.rs, concat_l1sqr_main.rs, slice2d.rs, elementwise.rs, screlu_*.rs literals
    L = lib()
    x = A([-2.0, -0.5, 0.0, 0.3, 1.0, 1.5, 7.0]); y = np.zeros(7, f32)
    L.ora_crelu_fwd(x, y, 7)
    assert y.tolist() == [0.0, 0.0, 0.0, float(f32(0.3)), 1.0, 1.0, 1.0]
    x = A([-1.0, 0.0, 0.0001, 0.5, 0.9999, 1.0, 2.0]); dx = np.zeros(7, f32)
    L.ora_crelu_grad(x, A([3.0] * 7), dx, 7)
    assert dx.tolist() == [0, 0, 3, 3, 3, 0, 0]
    dx = A([9.0]); L.ora_crelu_grad(A([np.nan]), A([5.0]), dx, 1)
    assert dx[0] == 0.0
    x = A([-3.0, 0.0, 0.5, 2.0]); y = np.zeros(4, f32)
    L.ora_abs_pow2_scale_fwd(x, y, SCALE, 4)
    assert y.tolist() == [float(f32(v) * f32(v) * SCALE) for v in x]
    dx = np.zeros(4, f32)
    L.ora_abs_pow2_scale_grad(A([1, -2, 0, 4]), A([0.5, 1, 3, -1]), dx, 2.0, 4)
    assert dx.tolist() == [2.0, -8.0, 0.0, -16.0]
    out = np.zeros(10, f32)
    L.ora_concat_l1sqr_main_fwd(A([1, 2, 3, 4, 5, 6]), A([10, 20, 30, 40]), out, 2, 3, 2)
    assert out.tolist() == [1, 2, 3, 10, 20, 4, 5, 6, 30, 40]
    da = np.zeros(6, f32); db = np.zeros(6, f32)
    L.ora_concat_l1sqr_main_grad(A(range(1, 13)), da, db, 2, 3)
    assert da.tolist() == [1, 2, 3, 7, 8, 9] and db.tolist() == [4, 5, 6, 10, 11, 12]
    src = A(range(32)); main = np.zeros(30, f32); skip = np.zeros(2, f32)
    L.ora_slice_extract_2d(src, main, 2, 16, 0, 15)
    L.ora_slice_extract_2d(src, skip, 2, 16, 15, 1)
    assert main.tolist() == list(range(15)) + list(range(16, 31)) and skip.tolist() == [15, 31]
    dst = A([9, 9, 9, 9])
    L.ora_slice_scatter_2d(A([1, 2]), dst, 1, 2, 4, 1)
    assert dst.tolist() == [9, 1, 2, 9]
    c = np.zeros(4, f32)
    L.ora_elementwise_add(A([1, -2, 3.5, 0]), A([0.5, 2, -1.5, 7]), c, 4)
    assert c.tolist() == [1.5, 0, 2, 7]
    x = A([-2.0, -0.5, 0.0, 0.3, 0.7, 1.0, 1.5]); y = np.zeros(7, f32)
    L.ora_screlu_fwd(x, y, 7)
    assert y.tolist() == [0, 0, 0, float(f32(0.3) * f32(0.3)), float(f32(0.7) * f32(0.7)), 1, 1]
    dx = np.zeros(6, f32)
    L.ora_screlu_grad(A([-0.5, 0.0, 0.3, 0.7, 1.0, 1.5]), A([1, 2, 3, 4, 5, 6]), dx, 6)
    np.testing.assert_allclose(dx, [0, 0, 3 * 0.6, 4 * 1.4, 0, 0], atol=1e-7)


# ---------------------------------------------------------------- losses
def _sig(x):
    x = f32(x)
    return f32(1.0) / (f32(1.0) + np.exp(-x, dtype=f32))


def test_loss_wdl_formula():
    # crates/gpu-kernels/src/pointwise/loss_wdl.rs tests: lambda 0 / 1 / blend against the formula in f32
    L = lib()
    out = A([120.0, -300.0, 15.0, 900.0]); score = A([200.0, -150.0, 0.0, 1200.0]); wdl = A([1.0, 0.0, 0.5, 1.0])
    norm = A([0.25] * 4); scale = f32(1.0 / 290.0)
    for lam in (0.0, 1.0, 0.3):
        dl = np.zeros(4, f32); acc = C.c_double(0.0)
        L.ora_loss_wdl(out, score, wdl, norm, dl, C.byref(acc), lam, scale, 4)
        exp_loss = 0.0
        for i in range(4):
            p = _sig(out[i] * scale); ys = _sig(score[i] * scale)
            y = f32(lam) * wdl[i] + (f32(1.0) - f32(lam)) * ys
            err = p - y
            exp_loss += float(err) * float(err)
            g = f32(2.0) * err * p * (f32(1.0) - p) * scale * norm[i]
            assert abs(float(dl[i]) - float(g)) < 1e-8  # numpy exp vs libm expf: 1 ulp
        assert abs(acc.value - exp_loss) < 1e-7


def _wrm(L, out, score, wdl, norm, lam, n2s=600.0, ins=340.0, ino=270.0, to=270.0, ts=380.0):
    dl = np.zeros(len(out), f32); acc = C.c_double(0.0)
    L.ora_loss_wrm(A(out), A(score), A(wdl), A(norm), dl, C.byref(acc), lam, n2s, ins, ino, to, ts,
                   2.0, 0.0, 0.0, 0.5, 0, len(out))
    return dl, acc.value


def test_loss_wrm_identities():
    # crates/gpu-kernels/src/pointwise/loss_wrm.rs: zero_input_yields_half_target_and_prediction_zero_loss,
    # lambda_one_uses_pure_wdl_target, matches_wrm_formula, per_pos_norm_scales_grad_but_not_loss,
    # large_score_saturates_without_nan
    L = lib()
    dl, acc = _wrm(L, [0.0], [0.0], [0.5], [1.0], 0.0)
    assert acc == 0.0 and dl[0] == 0.0
    dl, acc = _wrm(L, [0.0], [999.0], [0.5], [1.0], 1.0)
    assert acc == 0.0 and dl[0] == 0.0
    out = [0.3, -0.8, 2.5, -0.05]; score = [150.0, -1200.0, 30.0, 5000.0]; wdl = [1.0, 0.0, 0.5, 1.0]
    dl, acc = _wrm(L, out, score, wdl, [1.0] * 4, 0.0)
    exp_loss = 0.0
    for i in range(4):
        s = f32(score[i])
        tw = f32(0.5) * (f32(1.0) + _sig((s - f32(270)) / f32(380)) - _sig((-s - f32(270)) / f32(380)))
        sn = f32(out[i]) * f32(600)
        q = _sig((sn - f32(270)) / f32(340)); qm = _sig((-sn - f32(270)) / f32(340))
        qf = f32(0.5) * (f32(1.0) + q - qm)
        err = qf - tw
        exp_loss += float(err) ** 2
        g = err * (f32(600) / f32(340)) * (q * (f32(1) - q) + qm * (f32(1) - qm))
        assert abs(float(dl[i]) - float(g)) < 1e-7
    assert abs(acc - exp_loss) < 1e-7  # numpy exp vs libm expf: 1 ulp
    dl_a, acc_a = _wrm(L, [1.5] * 3, [800.0] * 3, [1.0] * 3, [1.0] * 3, 0.0)
    dl_b, acc_b = _wrm(L, [1.5] * 3, [800.0] * 3, [1.0] * 3, [0.25] * 3, 0.0)
    assert abs(acc_a - acc_b) < 1e-12
    np.testing.assert_allclose(dl_b, dl_a * f32(0.25), atol=1e-7)
    dl, acc = _wrm(L, [10.0, -10.0], [32000.0, -32000.0], [1.0, 0.0], [1.0, 1.0], 0.0)
    assert np.isfinite(dl).all() and np.isfinite(acc)


def test_loss_wrm_degenerate_equals_sigmoid():
    # with nnue2score = in_scaling = target_scaling and zero offsets, 0.5(1+s(x)-s(-x)) = s(x):
    # WRM equals the sigmoid loss except for the factor 2 the WRM gradient cancels analytically
    L = lib()
    out = A([100.0, -40.0, 5.0]); score = A([250.0, -90.0, 10.0]); wdl = A([1.0, 0.0, 0.5]); norm = A([1 / 3.0] * 3)
    dl_w, acc_w = _wrm(L, out, score, wdl, norm, 0.0, n2s=1.0, ins=290.0, ino=0.0, to=0.0, ts=290.0)
    dl_s = np.zeros(3, f32); acc_s = C.c_double(0.0)
    L.ora_loss_wdl(out, score, wdl, norm, dl_s, C.byref(acc_s), 0.0, f32(1.0 / 290.0), 3)
    assert abs(acc_w - acc_s.value) < 1e-6  # x/290 vs x*(1/290) round differently in f32
    np.testing.assert_allclose(dl_w, dl_s, rtol=2e-5, atol=1e-9)


# ---------------------------------------------------------------- optimizer
def _ssd(step, b1, b2, thr):
    ss = C.c_float(); dn = C.c_int32()
    lib().ora_radam_compute_step_size_denom(step, b1, b2, thr, C.byref(ss), C.byref(dn))
    return ss.value, dn.value


def test_radam_schedule():
    # crates/gpu-kernels/src/pointwise/radam_step.rs: step_size_denom_step_1_disables_variance,
    # step_size_denom_large_step_enables_variance
    ss, dn = _ssd(1, 0.9, 0.999, 5.0)
    assert dn == 0 and abs(ss - float(f32(1.0) / (f32(1.0) - f32(0.9)))) < 1e-6
    ss, dn = _ssd(1000, 0.9, 0.999, 5.0)
    b2 = f32(0.999); sf = f32(1000)
    b2t = f32(np.power(b2, sf, dtype=f32))
    nmax = f32(2) / (f32(1) - b2) - f32(1)
    n = nmax - f32(2) * sf * b2t / (f32(1) - b2t)
    bc1 = f32(1) - f32(np.power(f32(0.9), sf, dtype=f32))
    exp = np.sqrt((f32(1) - b2t) * ((n - f32(4)) / (nmax - f32(4))) * ((n - f32(2)) / n) * (nmax / (nmax - f32(2)))) / bc1
    assert dn == 1 and abs(ss - float(exp)) < 1e-6


def _radam(w, m, v, g, lr, ss, dn, decay, lo, hi, b1=0.9, b2=0.999, eps=1e-8):
    w, m, v, g = A(w), A(m), A(v), A(g)
    lib().ora_radam_step(w, m, v, g, lr, ss, dn, decay, b1, b2, eps, lo, hi, len(w))
    return w, m, v, g


FMAX = float(np.finfo(f32).max)


def test_radam_step_literals():
    # radam_step.rs: one_step_denom_zero_skips_variance, one_step_denom_one_applies_adam,
    # clamp_pulls_weights_into_range, nan_grad_propagates_into_weights,
    # collapsed_clip_range_pins_weights_to_single_value
    w, m, v, g = _radam([1.0], [0.0], [0.0], [0.1], 0.1, 10.0, 0, 0.0, -FMAX, FMAX)
    assert abs(w[0] - 0.99) < 1e-6 and abs(m[0] - 0.01) < 1e-7 and abs(v[0] - 1e-5) < 1e-9 and g[0] == 0.0
    w, m, v, g = _radam([1.0], [0.01], [1e-5], [0.1], 0.1, 1.0, 1, 0.0, -FMAX, FMAX)
    mi = f32(0.9) * f32(0.01) + (f32(1) - f32(0.9)) * f32(0.1)
    vi = f32(0.999) * f32(1e-5) + (f32(1) - f32(0.999)) * f32(0.1) * f32(0.1)
    exp = f32(1.0) - f32(0.1) * f32(1.0) * (mi / (np.sqrt(vi) + f32(1e-8)))
    assert abs(float(w[0]) - float(exp)) < 1e-7
    w, *_ = _radam([100.0, -100.0, 0.5], [0] * 3, [0] * 3, [0] * 3, 0.0, 1.0, 1, 0.0, -1.0, 1.0)
    assert w.tolist() == [1.0, -1.0, 0.5]
    w, m, v, g = _radam([0.5], [0.0], [0.0], [np.nan], 1e-3, 1.0, 1, 0.0, -FMAX, FMAX)
    assert np.isnan(w[0]) and np.isnan(m[0]) and np.isnan(v[0]) and g[0] == 0.0
    w, *_ = _radam([100.0, -100.0, 0.0, 0.5], [0] * 4, [0] * 4, [1] * 4, 0.1, 1.0, 1, 0.0, 0.5, 0.5)
    assert w.tolist() == [0.5] * 4


def test_adamw_scalars_reduce_to_plain_adamw():
    # crates/nnue-train/src/optimizer.rs: adamw_step_size_denom_is_constant,
    # adamw_scalars_reduce_radam_step_to_plain_adamw, ranger_and_radam_step_size_follow_rectified_schedule
    L = lib()
    for step in (1, 2, 6, 1000):
        ss, dn, b1 = C.c_float(), C.c_int32(), C.c_float()
        L.ora_optimizer_scalars(2, step, 0.999, 5.0, C.byref(ss), C.byref(dn), C.byref(b1))
        assert (ss.value, dn.value) == (1.0, 1) and abs(b1.value - 0.9) < 1e-7
    w, m, v, _ = _radam([0.5], [0.02], [3e-4], [0.1], 0.001, 1.0, 1, 0.01, -1.98, 1.98)
    m1 = f32(0.9) * f32(0.02) + (f32(1) - f32(0.9)) * f32(0.1)
    v1 = f32(0.999) * f32(3e-4) + (f32(1) - f32(0.999)) * f32(0.1) * f32(0.1)
    exp = f32(0.5) * (f32(1) - f32(0.01) * f32(0.001)) - f32(0.001) * m1 / (np.sqrt(v1) + f32(1e-8))
    assert m[0] == m1 and v[0] == v1 and abs(float(w[0]) - float(exp)) < 1e-7
    for step in (1, 10, 1000):
        for kind, beta1 in ((0, 0.99), (1, 0.9)):
            ss, dn, b1 = C.c_float(), C.c_int32(), C.c_float()
            L.ora_optimizer_scalars(kind, step, 0.999, 5.0, C.byref(ss), C.byref(dn), C.byref(b1))
            assert (ss.value, dn.value) == _ssd(step, beta1, 0.999, 5.0)


def test_ranger_lerp_literals():
    # crates/gpu-kernels/src/pointwise/ranger_step.rs: lerp_alpha_one..., lerp_alpha_zero..., lerp_alpha_half...
    L = lib()
    for alpha, ew in ((1.0, [1, 2, 3]), (0.0, [10, 20, 30])):
        w = A([1, 2, 3]); s = A([10, 20, 30])
        L.ora_ranger_lookahead_lerp(w, s, alpha, 3)
        assert w.tolist() == ew and s.tolist() == ew
    w = A([2, -4, 0]); s = A([4, 4, 10])
    L.ora_ranger_lookahead_lerp(w, s, 0.5, 3)
    assert w.tolist() == [3, 0, 5] and s.tolist() == [3, 0, 5]


def test_composed_ranger_step_lerps_only_every_kth_step():
    # crates/gpu-kernels/src/pointwise/ranger_step.rs: step_cpu_invokes_lerp_only_at_k_step, restated on the composed
    # optimizer of the oracle's trainer (RangerParams::DEFAULT: k = 6, alpha = 0.5; slow weights start at 0): steps 1..5
    # leave slow untouched, step 6 synchronises weights and slow and pulls the weights towards slow = 0
    import oracle_lib as O
    ot = O.OracleTrainer(arch="simple", ft_in=8, piece_inputs=4, factorize=False, max_active=2, ft_out=128, l1=8, l2=8,
                         optimizer="ranger", wd=(0.0, 0.0, 0.0), capacity=16)
    names = list(ot.names)
    for n in names:
        ot.group(n)[:] = 1.0
    before = None
    for step in range(1, 7):
        for n in names:
            ot.group(n, "grad")[:] = 0.1 if step == 1 else 0.0   # (the reference's kernel zeroes the gradient itself)
        if step == 6:
            before = {n: ot.group(n).copy() for n in names}
        ot.apply_optimizer(0.1)
        assert ot.step_count == step
        for n in names:
            if step < 6:
                assert not ot.group(n, "slow").any(), (n, step)
            else:
                assert np.array_equal(ot.group(n), ot.group(n, "slow")), n
                assert (np.abs(ot.group(n)) < np.abs(before[n])).all(), n


# ---------------------------------------------------------------- init
def _xorshift_uniform(seed, n, half):
    # the sequence crates/nnue-train/src/init.rs documents for uniform_abs (u64 xorshift 13/7/17, top 53 bits)
    s = max(seed, 1); M = (1 << 64) - 1; out = []
    for _ in range(n):
        s ^= (s << 13) & M; s ^= s >> 7; s ^= (s << 17) & M
        u = f32(s >> 11) / f32(1 << 53)
        out.append(float((u * f32(2.0) - f32(1.0)) * f32(half)))
    return out


def test_init_uniform_abs_bit_identical_to_xorshift():
    # crates/nnue-train/src/init.rs: uniform_abs_is_bit_identical_to_reference_xorshift
    for seed, n in ((0x100, 37), (0x5071E003, 1024), (1, 9)):
        out = np.zeros(n, f32)
        lib().ora_init_sample(out, n, 1, 99, 1, 0, 0.01, 0, seed)
        assert out.tolist() == _xorshift_uniform(seed, n, 0.01)


def test_init_fan_in_half_width():
    # init.rs: fanin_uniform_half_width_matches_sqrt_inv_fan_in
    out = np.zeros(200_000, f32)
    lib().ora_init_sample(out, out.size, 1, 73_305, 1, 1, 1.0, 0, 0xABCD)
    bound = float(np.sqrt(f32(1.0) / f32(73_305)))
    assert bound * 0.98 < out.max() <= bound and -bound <= out.min() < -bound * 0.98
    assert abs(out.astype(np.float64).std() - bound / np.sqrt(3)) / (bound / np.sqrt(3)) < 0.05


# ---------------------------------------------------------------- PSV bit patterns, BonaPiece, king buckets
def _decode(bits_bytes):
    raw = np.zeros(40, np.uint8)
    raw[:len(bits_bytes)] = bits_bytes
    b = Board()
    lib().ora_psv_decode(raw, C.byref(b))
    return b


def test_psv_accessors_and_huffman_patterns():
    # crates/shogi-format/src/packed_sfen.rs: test_packed_sfen_value_accessors, test_huffman_decode_*
    raw = np.zeros(40, np.uint8); raw[32] = 0x34; raw[33] = 0x12; raw[36] = 0x56; raw[38] = 0xFF
    b = Board(); lib().ora_psv_decode(raw, C.byref(b))
    assert (b.score, b.ply, b.result) == (0x1234, 0x56, -1)

    def first_square(code_bits):
        # stm bit + kings on squares 79/80 so that square 0 is the first Huffman symbol at bit 15
        v = 0 | (79 << 1) | (80 << 8) | (code_bits << 15)
        return _decode(list(v.to_bytes(8, "little")))
    b = first_square(0b0)
    assert b.board_pt[0] == 0
    b = first_square(0b0001)
    assert (b.board_pt[0], b.board_color[0]) == (1, 0)       # black pawn
    b = first_square(0b1101)
    assert (b.board_pt[0], b.board_color[0]) == (9, 1)       # white promoted pawn
    b = first_square(0b001111)
    assert (b.board_pt[0], b.board_color[0]) == (7, 0)       # black gold


def test_king_bucket_mirror_and_pack_literals():
    # crates/shogi-features/src/halfka_hm.rs: test_king_bucket_black_perspective, test_is_hm_mirror,
    # test_pack_bonapiece_*; crates/shogi-format/src/bona_piece.rs: test_bona_piece_from_piece_square/_from_hand
    L = lib()

    def feats(fs, bk, wk, stm=0, pieces=(), hands=()):
        b = Board()
        b.side_to_move = stm; b.black_king_sq = bk; b.white_king_sq = wk
        b.board_pt[bk] = 8; b.board_color[bk] = 0; b.board_pt[wk] = 8; b.board_color[wk] = 1
        for sq, pt, col in pieces:
            b.board_pt[sq] = pt; b.board_color[sq] = col
        for col, slot, cnt in hands:
            b.hand[col][slot] = cnt
        s = np.full(40, -1, np.int32); n = np.full(40, -1, np.int32)
        k = L.ora_extract_active_features(fs, C.byref(b), s, n, 40)
        return s[:k].tolist(), n[:k].tolist()

    PI = 1629
    # king bucket literals: black king on 5i(44)->44, 1i(8)->8, 9i(80)->8, 6i(53)->35, 5a(36)->36, 1a(0)->0.
    # the friend-king feature of halfka-hm-merged is kb*PI + F_KING(1548) + mirrored king square
    for sq, kb, mirror in ((44, 44, False), (8, 8, False), (80, 8, True), (53, 35, True), (36, 36, False), (0, 0, False)):
        wk = 40 if sq != 40 else 41
        s, _ = feats(4, sq, wk)
        ksq = sq if not mirror else (8 - sq // 9) * 9 + sq % 9
        assert s[0] == kb * PI + 1548 + ksq
        # enemy king folded onto the friend plane: E_KING(1629) + sq - 81, mirrored when the own king mirrors
        esq = wk if not mirror else (8 - wk // 9) * 9 + wk % 9
        assert s[1] == kb * PI + 1629 + esq - 81
    # board mirror: black pawn on square 0 with a mirroring king -> 90 + 72 ; on square 9 -> 90 + 63
    s, _ = feats(4, 80, 40, pieces=[(0, 1, 0)])
    assert s[0] == 8 * PI + 90 + 72
    s, _ = feats(4, 80, 40, pieces=[(9, 1, 0)])
    assert s[0] == 8 * PI + 90 + 63
    s, _ = feats(4, 8, 40, pieces=[(9, 1, 0)])
    assert s[0] == 8 * PI + 90 + 9
    # hand pieces never mirror; F_HAND_PAWN = 1, second pawn = 2, enemy pawn = E_HAND_PAWN = 20
    s, n = feats(4, 80, 40, hands=[(0, 0, 2), (1, 0, 1)])
    assert s[2:] == [8 * PI + 1, 8 * PI + 2, 8 * PI + 20]
    # halfkp: black pawn on 7g (file 6, rank 6 -> square 60): F_PAWN + 60 = 150, no king features
    s, n = feats(0, 44, 36, pieces=[(60, 1, 0)])
    assert s == [44 * 1548 + 150] and n == [(80 - 36) * 1548 + 171 + (80 - 60)]


def _board_from_sfen_kings(sfen):
    # king squares only, the way crates/shogi-features/src/kingrank9.rs tests build their boards
    placement, side = sfen.split()[:2]
    b = Board(); b.side_to_move = 0 if side == "b" else 1
    b.black_king_sq = 81; b.white_king_sq = 81
    for rank, row in enumerate(placement.split("/")):
        f = 0
        for ch in row:
            if ch.isdigit():
                f += int(ch); continue
            if ch == "+":
                continue
            file = 8 - f
            if ch == "K":
                b.black_king_sq = file * 9 + rank
            if ch == "k":
                b.white_king_sq = file * 9 + rank
            f += 1
    return b


@pytest.mark.parametrize("sfen,expected", [
    ("lnsgkgsnl/1r5b1/ppppppppp/9/9/9/PPPPPPPPP/1B5R1/LNSGKGSNL b - 1", 8),
    ("lnsg1gsnl/1r2k2b1/ppppppppp/9/9/9/PPPPPPPPP/1B2K2R1/LNSG1GSNL w - 1", 8),
    ("9/9/4K4/9/9/9/4k4/9/9 b - 1", 0),
    ("9/9/9/4K4/4k4/9/9/9/9 b - 1", 4),
    ("lnsgkgsnl/1r5b1/ppppppppp/9/9/9/PPPPPPPPP/1B5R1/LNSGKGSNL w - 1", 8),
])
def test_kingrank9_fixtures(sfen, expected):
    # crates/shogi-features/src/kingrank9.rs: oracle_fixtures_match_yaneuraou_kingrank9
    b = _board_from_sfen_kings(sfen)
    assert lib().ora_kingrank9_bucket(C.byref(b)) == expected


def test_feature_dims_table():
    # crates/shogi-features/src/feature_set.rs: spec_dimensions_match_design_table
    from oracle_lib import feature_dims
    exp = {"halfkp": (81, 1548, 125_388, 38), "halfka-split": (81, 1710, 138_510, 40),
           "halfka-merged": (81, 1629, 131_949, 40), "halfka-hm-split": (45, 1710, 76_950, 40),
           "halfka-hm-merged": (45, 1629, 73_305, 40)}
    for name, (kb, pi, n, a) in exp.items():
        d = feature_dims(name)
        assert (d["king_buckets"], d["piece_inputs"], d["ft_in"], d["max_active"]) == (kb, pi, n, a)
