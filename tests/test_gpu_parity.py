"""Parity of the CUDA path (through the C ABI) against the CPU oracle on the same seeded inputs.

Tolerances (the reference's comparison form |g - c| <= tol (1 + |c|)):
  indices / buckets      bit-exact
  FT forward sums        bit-exact (pure adds in slot order; the reference's own bar is tolerance 0)
  forward values, loss   1e-5
  gradients              1e-4 (against the tensor's scale for sums of many signed terms)
  optimizer state        1e-5 after one step
"""
import ctypes as C
import os

import numpy as np
import pytest

import oracle_lib as O
import tatara_b200 as tb
from helpers import GOLDEN, assert_close, assert_close_scaled, random_index_batch

pytestmark = pytest.mark.gpu

TOL_FWD = 1e-5
TOL_GRAD = 1e-4


def _lib():
    return tb.load_library()


# ---------------------------------------------------------------- inputs: GPU decode + extraction
@pytest.mark.parametrize("fs", ["halfkp", "halfka-hm-merged", "halfka-split", "halfka-merged", "halfka-hm-split"])
def test_psv_extract_bit_exact_synthetic(fs):
    psv = tb.synthesize_psv(tb.SYNTH_SEED, 4096 + 16)
    got = tb.extract_batch(psv, tb.FEATURE_SETS[fs])
    want = O.psv_to_batch(fs, psv.tobytes())
    assert (got.nnz == want["nnz"]).all()
    assert (got.stm_indices == want["stm"]).all() and (got.nstm_indices == want["nstm"]).all()
    assert (got.bucket_idx == want["bucket"]).all()
    assert (got.score == want["score"]).all() and (got.wdl == want["wdl"]).all()


def test_psv_extract_bit_exact_on_reference_fixture():
    raw = np.frombuffer(open(os.path.join(GOLDEN, "sample_psv.bin"), "rb").read(), np.uint8).reshape(100, 40)
    exp = np.load(os.path.join(GOLDEN, "sample_psv_expected.npz"))
    from helpers import sort_rows
    for fs, key in (("halfkp", "kp"), ("halfka-hm-merged", "hm")):
        got = tb.extract_batch(raw, tb.FEATURE_SETS[fs])
        want = O.psv_to_batch(fs, raw.tobytes())
        assert (got.stm_indices == want["stm"]).all() and (got.nstm_indices == want["nstm"]).all()   # same order
        assert (sort_rows(got.stm_indices) == exp[key + "_stm"]).all()                               # golden sets
        assert (sort_rows(got.nstm_indices) == exp[key + "_nstm"]).all()
        assert (got.nnz == exp["nnz_" + key]).all() and (got.bucket_idx == exp["bucket"]).all()
        assert (got.score == exp["score"]).all() and (got.wdl == exp["wdl"]).all()


def test_psv_extract_empty_input():
    got = tb.extract_batch(np.zeros((0, 40), np.uint8), tb.FEATURE_SETS["halfkp"])
    assert got.n_pos == 0


# ---------------------------------------------------------------- FT kernels alone
def _ft_forward(table, idx, nnz, N, F, A):
    B = nnz.shape[0]
    out = np.empty((B, F), np.float32)
    ms = C.c_float()
    rc = _lib().tb_ft_forward_bench(0, table.ctypes.data, idx.ctypes.data, nnz.ctypes.data, B, F, N, A, 1,
                                    out.ctypes.data, C.byref(ms))
    assert rc == 0, _lib().tb_last_error(None)
    return out


def test_ft_forward_reference_vectors():
    # sparse_ft_forward.rs literal cases embedded in a 128-wide table (column 0/1 carry the literals)
    F, N, A = 128, 3, 4
    table = np.zeros((N, F), np.float32)
    table[:, 0] = [0, 2, 4]; table[:, 1] = [1, 3, 5]
    idx = np.array([[0, 1, -1, -1], [2, 2, 1, 0]], np.int32); nnz = np.array([2, 4], np.int32)
    out = _ft_forward(table, idx, nnz, N, F, A)
    assert out[:, :2].reshape(-1).tolist() == [2.0, 4.0, 10.0, 14.0]
    # all padding -> 0 ; out-of-range skipped ; duplicates summed ; nnz = 0
    idx = np.array([[-1, -1, -1, -1], [0, 5, -1, 7], [0, 0, 1, -1], [1, 1, 1, 1]], np.int32)
    nnz = np.array([4, 3, 3, 0], np.int32)
    out = _ft_forward(table, idx, nnz, N, F, A)
    assert out[0, :2].tolist() == [0.0, 0.0] and out[1, :2].tolist() == [0.0, 1.0]
    assert out[2, :2].tolist() == [2.0, 5.0] and out[3, :2].tolist() == [0.0, 0.0]


@pytest.mark.parametrize("F,B,A", [(128, 48, 7), (256, 1000, 38), (768, 512, 40), (1536, 300, 40), (3072, 64, 40)])
def test_ft_forward_bit_exact(F, B, A):
    rng = np.random.default_rng(F + B)
    N = 5000
    table = (rng.standard_normal((N, F)) * 0.05).astype(np.float32)
    d = random_index_batch(rng, B, A, N, max(0, A - 10), A, with_bucket=0)
    d["stm"][::7, 0] = N + 3       # out-of-range
    d["stm"][::5, 1] = -1          # padding inside the active range
    d["stm"][::11, 2] = d["stm"][::11, 3]   # duplicate
    want = np.empty((B, F), np.float32)
    O.lib().ora_sparse_ft_forward(table.reshape(-1), d["stm"].reshape(-1), d["nnz"], want.reshape(-1), B, F, N, A)
    got = _ft_forward(table, d["stm"], d["nnz"], N, F, A)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def _ft_backward(dft, idx, nnz, N, F, A):
    B = nnz.shape[0]
    grad = np.full((N, F), 123.0, np.float32)
    ms = C.c_float()
    rc = _lib().tb_ft_backward_bench(0, dft.ctypes.data, idx.ctypes.data, nnz.ctypes.data, B, F, N, A, 1,
                                     grad.ctypes.data, C.byref(ms))
    assert rc == 0, _lib().tb_last_error(None)
    return grad


def test_ft_backward_reference_vectors():
    # sparse_ft_backward.rs: matches_reference_evaluate_bwd_test embedded in 128 columns
    F, N, A = 128, 3, 4
    dft = np.zeros((2, F), np.float32); dft[0, :3] = [0, 1, 2]; dft[1, :3] = [3, 4, 5]
    idx = np.array([[0, 1, -1, -1], [2, 2, 1, 0]], np.int32); nnz = np.array([4, 4], np.int32)
    g = _ft_backward(dft, idx, nnz, N, F, A)
    assert g[:, :3].reshape(-1).tolist() == [3, 5, 7, 3, 5, 7, 6, 8, 10]
    assert (g[:, 3:] == 0).all()       # rows are overwritten, also where nothing contributes


@pytest.mark.parametrize("F,B,A,N", [(128, 64, 6, 50), (256, 2048, 38, 3000), (1536, 512, 40, 700)])
def test_ft_backward_matches_oracle(F, B, A, N):
    rng = np.random.default_rng(F * 3 + B)
    dft = (rng.standard_normal((B, F)) * 1e-3).astype(np.float32)
    d = random_index_batch(rng, B, A, N, max(0, A - 8), A, with_bucket=0)
    d["stm"][::9, 0] = -1
    d["stm"][::13, 1] = N + 1
    masked = np.where(np.arange(A)[None, :] < d["nnz"][:, None], d["stm"], -1).astype(np.int32)
    want = np.zeros((N, F), np.float32)
    O.lib().ora_sparse_ft_backward(dft.reshape(-1), masked.reshape(-1), want.reshape(-1), B, F, N, A)
    got = _ft_backward(dft, d["stm"], d["nnz"], N, F, A)
    # lists are sorted by position, so the sums run in the oracle's order: bit-exact
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    again = _ft_backward(dft, d["stm"], d["nnz"], N, F, A)
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))


def test_ft_backward_hot_feature_long_list():
    # one feature in every position (the king feature of a king bucket): exercises the long-list path
    F, B, A, N = 256, 16384, 4, 64
    rng = np.random.default_rng(5)
    dft = (rng.standard_normal((B, F)) * 1e-3).astype(np.float32)
    idx = np.stack([np.full(B, 7), rng.integers(8, N, B), rng.integers(8, N, B), np.full(B, -1)], 1).astype(np.int32)
    nnz = np.full(B, 3, np.int32)
    want = np.zeros((N, F), np.float32)
    O.lib().ora_sparse_ft_backward(dft.reshape(-1), np.where(np.arange(A)[None] < 3, idx, -1).astype(np.int32).reshape(-1),
                                   want.reshape(-1), B, F, N, A)
    got = _ft_backward(dft, idx, nnz, N, F, A)
    # lists longer than 4096 entries are summed in parts: same terms, different association
    assert_close_scaled(got, want, 1e-5, "hot feature")
    assert np.array_equal(got[8:].view(np.uint32), want[8:].view(np.uint32))     # short lists stay bit-exact
    again = _ft_backward(dft, idx, nnz, N, F, A)
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))            # and the result is reproducible


def test_adam_clamp_matches_oracle():
    rng = np.random.default_rng(11)
    n = 128 * 1000
    w = (rng.standard_normal(n) * 0.5).astype(np.float32); m = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    v = (rng.random(n) * 1e-5).astype(np.float32); g = (rng.standard_normal(n) * 1e-2).astype(np.float32)
    w2, m2, v2, g2 = w.copy(), m.copy(), v.copy(), g.copy()
    O.lib().ora_radam_step(w2, m2, v2, g2, 1e-3, 1.0, 1, 0.01, 0.9, 0.999, 1e-8, -0.25, 0.25, n)
    ms = C.c_float()
    rc = _lib().tb_adam_clamp_bench(0, w.ctypes.data, m.ctypes.data, v.ctypes.data, g.ctypes.data, n, 1e-3, 0.01, -0.25, 0.25,
                                    1, C.byref(ms))
    assert rc == 0
    assert_close(m, m2, 1e-6, "m"); assert_close(v, v2, 1e-6, "v"); assert_close(w, w2, 1e-6, "w")
    assert w.max() <= 0.25 and w.min() >= -0.25 and (np.abs(w) == 0.25).any()


# ---------------------------------------------------------------- whole step
LS_FS = tb.FeatureSetSpec("halfka-hm-merged", 4, 45, 1629, 40, True)
KP_FS = tb.FeatureSetSpec("halfkp", 0, 81, 1548, 38, True)


def _oracle_for(tr, arch, fs, F, l1, l2, nb, optimizer, wd, cap, activation=0):
    ot = O.OracleTrainer(arch=arch, ft_in=fs.ft_in, piece_inputs=fs.piece_inputs, factorize=fs.ft_factorize,
                         max_active=fs.max_active, ft_out=F, l1=l1, l2=l2, num_buckets=nb, activation=activation,
                         optimizer=optimizer, wd=wd, capacity=cap)
    ot.set_threads(os.cpu_count() or 1)
    return ot


def _sync_weights(tr, ot, init):
    for name in ot.names:
        ot.group(name)[:] = init[name]


def _batch_dict(b):
    d = dict(stm=b.stm_indices, nstm=b.nstm_indices, nnz=b.nnz, score=b.score, wdl=b.wdl)
    if b.bucket_idx is not None:
        d["bucket"] = b.bucket_idx
    return d


def _perturb(init, rng, names):
    # biases start at zero in the reference's default init; give them values so every path carries signal
    for n in names:
        init[n] = (rng.standard_normal(init[n].size) * 0.05).astype(np.float32)
    return init


def _check_step(tr, ot, batch, loss_t, loss_o, lr, arch, B, F, l1):
    K = F if arch == "layerstack" else 2 * F
    l_gpu = tr.forward_backward(batch, 0.25, loss_t)
    l_cpu = ot.step(_batch_dict(batch), lr, 0.25, loss_o, do_optimizer=False)
    ft_stm, ft_nstm = tr.read_buffer("ft_stm", B * F), tr.read_buffer("ft_nstm", B * F)
    if arch == "layerstack":
        assert np.array_equal(ft_stm.view(np.uint32), ot.buffer("ft_stm").view(np.uint32)), "FT forward must be bit-exact"
        assert np.array_equal(ft_nstm.view(np.uint32), ot.buffer("ft_nstm").view(np.uint32))
    else:
        assert_close(ft_stm, ot.buffer("ft_stm"), 1e-6, "ft_stm (+bias)")
    assert_close(tr.read_buffer("combined", B * K), ot.buffer("combined"), TOL_FWD, "combined")
    assert_close(tr.read_buffer("l1_total", B * l1), ot.buffer("l1_total"), TOL_FWD, "l1_total")
    assert_close(tr.read_buffer("net_output", B), ot.buffer("net_output"), TOL_FWD, "net_output")
    assert abs(l_gpu - l_cpu) <= TOL_FWD * (1 + abs(l_cpu)), (l_gpu, l_cpu)
    assert_close_scaled(tr.read_buffer("dy", B), ot.buffer("dy"), TOL_GRAD, "dy")
    assert_close_scaled(tr.read_buffer("dl1_total", B * l1), ot.buffer("dl1_total"), TOL_GRAD, "dl1_total")
    assert_close_scaled(tr.read_buffer("dft_stm", B * F), ot.buffer("dft_stm"), TOL_GRAD, "dft_stm")
    assert_close_scaled(tr.read_buffer("dft_nstm", B * F), ot.buffer("dft_nstm"), TOL_GRAD, "dft_nstm")
    for name in ot.names:
        assert_close_scaled(tr.download_grad(name), ot.group(name, "grad"), TOL_GRAD, "grad " + name)
    return l_gpu


@pytest.mark.parametrize("F,l1,l2,B,optimizer,factorize", [
    (256, 16, 32, 512, "ranger", True), (768, 8, 32, 256, "adamw", True), (512, 16, 32, 496, "radam", False)])
def test_layerstack_step_matches_oracle(F, l1, l2, B, optimizer, factorize):
    fs = LS_FS.with_factorize(factorize)
    rng = np.random.default_rng(F + B)
    init = _perturb(tb.layerstack_default_init(fs, F, l1, l2, 9), rng, ["ft_b", "l1_b", "l1_shared_bias", "l2_b", "l3_b"])
    init["ft_w"][:fs.ft_in * F] *= 30.0      # pushes pre-activations across both CReLU edges
    if factorize:
        init["ft_w"][fs.ft_in * F:] = (rng.standard_normal(fs.piece_inputs * F) * 0.02).astype(np.float32)
    tr = tb.GpuTrainer(B, F, l1, l2, 9, fs, optimizer=optimizer, init=init)
    ot = _oracle_for(tr, "layerstack", fs, F, l1, l2, 9, optimizer, (0.01, 0.01, 0.01), B)
    _sync_weights(tr, ot, init)
    batch = tb.synthetic_batch(tb.SYNTH_SEED + 3, B, fs)
    lr = 8.75e-4
    _check_step(tr, ot, batch, tb.LossKind.sigmoid(), O.sigmoid_loss(), lr, "layerstack", B, F, l1)
    tr.apply_optimizer(lr); ot.apply_optimizer(lr)
    assert tr.step_count == 1 == ot.step_count
    for name in ot.names:
        got = tr.download_group(name, ("w", "m", "v"))
        assert_close(got["w"], ot.group(name, "w"), TOL_FWD, "w " + name)
        assert_close_scaled(got["m"], ot.group(name, "m"), TOL_GRAD, "m " + name)
        assert_close_scaled(got["v"], ot.group(name, "v"), TOL_GRAD, "v " + name)
    if factorize:
        w = ot.group("ft_w")
        want_comb = (w[:fs.ft_in * F].reshape(-1, fs.piece_inputs, F) + w[fs.ft_in * F:].reshape(1, fs.piece_inputs, F)).reshape(-1)
        assert_close(tr.read_buffer("comb", fs.ft_in * F), want_comb, TOL_FWD, "comb")


@pytest.mark.parametrize("F,l1,l2,B,act,factorize", [(256, 32, 32, 512, "crelu", True), (256, 32, 32, 208, "screlu", False),
                                                     (128, 8, 16, 64, "crelu", True)])
def test_simple_step_matches_oracle(F, l1, l2, B, act, factorize):
    fs = KP_FS.with_factorize(factorize)
    rng = np.random.default_rng(F + B + 1)
    init = tb.simple_default_init(fs, F, l1, l2)
    init["ft_w"][:fs.ft_in * F] *= 4.0
    for k in ("l1_w", "l2_w", "l3_w"):
        init[k] *= 8.0
    if factorize:
        init["ft_w"][fs.ft_in * F:] = (rng.standard_normal(fs.piece_inputs * F) * 0.02).astype(np.float32)
    tr = tb.SimpleGpuTrainer(B, F, l1, l2, fs, activation=act, optimizer="adamw", weight_decay=0.0, init=init)
    ot = _oracle_for(tr, "simple", fs, F, l1, l2, 0, "adamw", (0.0, 0.0, 0.0), B, activation=0 if act == "crelu" else 1)
    _sync_weights(tr, ot, init)
    batch = tb.synthetic_batch(tb.SYNTH_SEED + 1, B, fs, with_bucket=False)
    lr = 8.75e-4
    # config 0/1 of the benchmark: WRM with every scale 290 and zero offsets
    lt = tb.LossKind.wrm(nnue2score=290.0, in_scaling=290.0, in_offset=0.0, target_offset=0.0, target_scaling=290.0)
    lo = O.wrm_loss(290.0, 290.0, 0.0, 0.0, 290.0)
    _check_step(tr, ot, batch, lt, lo, lr, "simple", B, F, l1)
    tr.apply_optimizer(lr); ot.apply_optimizer(lr)
    for name in ot.names:
        got = tr.download_group(name, ("w", "m", "v"))
        assert_close(got["w"], ot.group(name, "w"), TOL_FWD, "w " + name)
        assert_close_scaled(got["m"], ot.group(name, "m"), TOL_GRAD, "m " + name)


def test_simple_pairwise_step_matches_oracle():
    """SimpleActivation::Pairwise (bins/nnue_train/src/trainer_simple.rs:1241-1262, 2008-2040): the LayerStack FT post in
    front of the Simple dense layers; the L1 input is ft_out wide."""
    F, l1, l2, B = 256, 32, 32, 272
    fs = KP_FS
    rng = np.random.default_rng(44)
    init = tb.simple_default_init(fs, F, l1, l2, pairwise=True)
    init["ft_w"][:fs.ft_in * F] *= 12.0
    for k in ("l1_w", "l2_w", "l3_w"):
        init[k] *= 8.0
    init["ft_w"][fs.ft_in * F:] = (rng.standard_normal(fs.piece_inputs * F) * 0.02).astype(np.float32)
    assert init["l1_w"].size == F * l1
    tr = tb.SimpleGpuTrainer(B, F, l1, l2, fs, activation="pairwise", optimizer="adamw", weight_decay=0.0, init=init)
    ot = _oracle_for(tr, "simple", fs, F, l1, l2, 0, "adamw", (0.0, 0.0, 0.0), B, activation=2)
    _sync_weights(tr, ot, init)
    batch = tb.synthetic_batch(tb.SYNTH_SEED + 4, B, fs, with_bucket=False)
    lt = tb.LossKind.wrm(nnue2score=290.0, in_scaling=290.0, in_offset=0.0, target_offset=0.0, target_scaling=290.0)
    lo = O.wrm_loss(290.0, 290.0, 0.0, 0.0, 290.0)
    l_gpu = tr.forward_backward(batch, 0.25, lt)
    l_cpu = ot.step(_batch_dict(batch), 8.75e-4, 0.25, lo, do_optimizer=False)
    assert np.array_equal(tr.read_buffer("ft_stm", B * F).view(np.uint32), ot.buffer("ft_stm").view(np.uint32))   # raw sums are kept
    assert_close(tr.read_buffer("combined", B * F), ot.buffer("combined"), TOL_FWD, "combined")
    assert_close(tr.read_buffer("net_output", B), ot.buffer("net_output"), TOL_FWD, "net_output")
    assert abs(l_gpu - l_cpu) <= TOL_FWD * (1 + abs(l_cpu))
    assert_close_scaled(tr.read_buffer("dft_stm", B * F), ot.buffer("dft_stm"), TOL_GRAD, "dft_stm")
    for name in ot.names:
        assert_close_scaled(tr.download_grad(name), ot.group(name, "grad"), TOL_GRAD, "grad " + name)
    tr.apply_optimizer(8.75e-4); ot.apply_optimizer(8.75e-4)
    for name in ot.names:
        assert_close(tr.download_group(name)["w"], ot.group(name, "w"), TOL_FWD, "w " + name)


@pytest.mark.parametrize("arch", ["simple", "layerstack"])
def test_extended_wrm_loss_matches_oracle(arch):
    """LossKind::Wrm with pow_exp, qp_asymmetry and the weight boost (loss_wrm extended branch + wrm_weight_sum,
    native_kernels.cu:408-545): the per-position weights are normalised by their sum over the batch."""
    B = 256
    rng = np.random.default_rng(9)
    kw = dict(nnue2score=600.0, in_scaling=340.0, in_offset=270.0, target_offset=270.0, target_scaling=380.0, pow_exp=2.5,
              qp_asymmetry=0.3, weight_boost_w1=1.5, weight_boost_w2=0.5)
    lt = tb.LossKind.wrm(**kw)
    lo = O.wrm_loss(600.0, 340.0, 270.0, 270.0, 380.0, 2.5, 0.3, 1.5, 0.5)
    if arch == "simple":
        F, l1, l2, fs = 256, 32, 32, KP_FS
        init = tb.simple_default_init(fs, F, l1, l2)
        init["ft_w"][:fs.ft_in * F] *= 4.0
        for k in ("l1_w", "l2_w", "l3_w"):
            init[k] *= 20.0
        tr = tb.SimpleGpuTrainer(B, F, l1, l2, fs, activation="crelu", optimizer="adamw", weight_decay=0.0, init=init)
        ot = _oracle_for(tr, "simple", fs, F, l1, l2, 0, "adamw", (0.0, 0.0, 0.0), B)
        batch = tb.synthetic_batch(31, B, fs, with_bucket=False)
    else:
        F, l1, l2, fs = 256, 16, 32, LS_FS
        init = _perturb(tb.layerstack_default_init(fs, F, l1, l2, 9), rng, ["ft_b", "l1_b", "l1_shared_bias", "l2_b", "l3_b"])
        init["ft_w"][:fs.ft_in * F] *= 30.0
        for k in ("l1_w", "l1_shared_weight", "l2_w", "l3_w"):
            init[k] = init[k] * np.float32(40.0)
        tr = tb.GpuTrainer(B, F, l1, l2, 9, fs, optimizer="adamw", init=init)
        ot = _oracle_for(tr, "layerstack", fs, F, l1, l2, 9, "adamw", (0.01, 0.01, 0.01), B)
        batch = tb.synthetic_batch(32, B, fs)
    _sync_weights(tr, ot, init)
    l_gpu = tr.forward_backward(batch, 0.25, lt)
    l_cpu = ot.step(_batch_dict(batch), 1e-3, 0.25, lo, do_optimizer=False)
    assert abs(l_gpu - l_cpu) <= 1e-5 * (1 + abs(l_cpu)), (l_gpu, l_cpu)
    assert_close_scaled(tr.read_buffer("dy", B), ot.buffer("dy"), TOL_GRAD, "dy")
    assert np.abs(ot.buffer("dy")).max() > 0
    for name in ot.names:
        assert_close_scaled(tr.download_grad(name), ot.group(name, "grad"), TOL_GRAD, "grad " + name)
    # the plain parameters still take the default path: same loss as the sigmoid-shaped WRM
    plain = tb.LossKind.wrm(nnue2score=600.0, in_scaling=340.0, in_offset=270.0, target_offset=270.0, target_scaling=380.0)
    assert tr.validate_step(batch, 0.25, plain)[0] != l_gpu
    tr.close()


def test_layerstack_loss_curve_and_lag():
    """8 steps on changing batches: the per-step loss follows the oracle within 1e-3 relative, the reported
    loss lags by one step, Ranger's look-ahead fires on step 6."""
    F, l1, l2, B = 256, 16, 32, 256
    fs = LS_FS
    init = tb.layerstack_default_init(fs, F, l1, l2, 9)
    init["ft_w"][:fs.ft_in * F] *= 30.0
    tr = tb.GpuTrainer(B, F, l1, l2, 9, fs, optimizer="ranger", init=init)
    ot = _oracle_for(tr, "layerstack", fs, F, l1, l2, 9, "ranger", (0.01, 0.01, 0.01), B)
    _sync_weights(tr, ot, init)
    lt, lo = tb.LossKind.sigmoid(), O.sigmoid_loss()
    want, got = [], []
    for s in range(8):
        batch = tb.synthetic_batch(100 + s, B, fs)
        want.append(ot.step(_batch_dict(batch), 1e-3, 0.0, lo))
        got.append(tr.train_step(batch, 1e-3, 0.0, lt))
    got.append(tr.flush_pending_loss())
    assert got[0] == 0.0                                   # first call reports 0.0
    for s in range(8):
        assert abs(got[s + 1] - want[s]) <= 1e-3 * abs(want[s]), (s, got[s + 1], want[s])
    assert tr.step_count == 8
    assert tr.flush_pending_loss() == 0.0                  # ring re-armed
    for name in ot.names:
        g = tr.download_group(name, ("w", "slow"))
        assert_close(g["w"], ot.group(name, "w"), 1e-4, "w after 8 steps " + name)
        assert_close(g["slow"], ot.group(name, "slow"), 1e-4, "slow " + name)


def test_step_is_deterministic_and_validate_is_pure():
    F, l1, l2, B = 256, 16, 32, 256
    fs = LS_FS
    init = tb.layerstack_default_init(fs, F, l1, l2, 9)
    batch = tb.synthetic_batch(9, B, fs)
    outs = []
    for _ in range(2):
        tr = tb.GpuTrainer(B, F, l1, l2, 9, fs, init=init)
        v0 = tr.validate_step(batch, 0.0, tb.LossKind.sigmoid())
        v1 = tr.validate_step(batch, 0.0, tb.LossKind.sigmoid())
        assert v0[0] == v1[0] and np.array_equal(v0[1], v1[1]) and tr.step_count == 0
        for _ in range(3):
            tr.train_step(batch, 1e-3, 0.0, tb.LossKind.sigmoid())
        outs.append((tr.flush_pending_loss(), tr.download_group("ft_w")["w"], tr.download_group("l1_w")["w"]))
        tr.close()
    assert outs[0][0] == outs[1][0]
    assert np.array_equal(outs[0][1].view(np.uint32), outs[1][1].view(np.uint32))
    assert np.array_equal(outs[0][2].view(np.uint32), outs[1][2].view(np.uint32))


def test_error_values_and_edge_batches():
    F, l1, l2, B = 256, 16, 32, 64
    fs = LS_FS
    tr = tb.GpuTrainer(B, F, l1, l2, 9, fs)
    good = tb.synthetic_batch(1, 64, fs)
    bad = tb.BatchData(good.stm_indices[:24], good.nstm_indices[:24], good.nnz[:24], good.score[:24], good.wdl[:24],
                       good.bucket_idx[:24])
    with pytest.raises(tb.TrainerError, match="multiple of 16"):
        tr.train_step(bad, 1e-3, 0.0, tb.LossKind.sigmoid())
    big = tb.synthetic_batch(1, 80, fs)
    with pytest.raises(tb.TrainerError, match="capacity"):
        tr.train_step(big, 1e-3, 0.0, tb.LossKind.sigmoid())
    empty = tb.BatchData(good.stm_indices[:0], good.nstm_indices[:0], good.nnz[:0], good.score[:0], good.wdl[:0],
                         good.bucket_idx[:0])
    assert tr.train_step(empty, 1e-3, 0.0, tb.LossKind.sigmoid()) == 0.0 and tr.step_count == 0
    nobucket = tb.BatchData(good.stm_indices, good.nstm_indices, good.nnz, good.score, good.wdl, None)
    with pytest.raises(tb.TrainerError, match="bucket_idx"):
        tr.train_step(nobucket, 1e-3, 0.0, tb.LossKind.sigmoid())
    with pytest.raises(tb.TrainerError, match="scale"):
        tr.train_step(good, 1e-3, 0.0, tb.LossKind.sigmoid(0.0))
    with pytest.raises(tb.TrainerError, match="unknown group"):
        tr.download_grad("nope")
    # the handle still works after every error
    tr.train_step(good, 1e-3, 0.0, tb.LossKind.sigmoid())
    assert np.isfinite(tr.flush_pending_loss())


def test_out_of_range_buckets_and_ragged_rows():
    """Rows with a bucket id outside [0, nb) get zero from the per-bucket layers (dense_mm_bucket.rs:45-73),
    ragged nnz, -1 padding and out-of-range indices are skipped."""
    F, l1, l2, B = 256, 16, 32, 128
    fs = LS_FS.with_factorize(False)
    rng = np.random.default_rng(3)
    init = _perturb(tb.layerstack_default_init(fs, F, l1, l2, 9), rng, ["ft_b", "l1_b", "l1_shared_bias", "l2_b", "l3_b"])
    init["ft_w"] *= 30.0
    d = random_index_batch(rng, B, 40, fs.ft_in, 0, 40)
    d["bucket"][::5] = -1
    d["bucket"][1::7] = 9
    d["stm"][::3, 0] = fs.ft_in + 5
    d["nstm"][::4, 1] = -1
    batch = tb.BatchData(d["stm"], d["nstm"], d["nnz"], d["score"], d["wdl"], d["bucket"])
    tr = tb.GpuTrainer(B, F, l1, l2, 9, fs, optimizer="adamw", init=init)
    ot = _oracle_for(tr, "layerstack", fs, F, l1, l2, 9, "adamw", (0.01, 0.01, 0.01), B)
    _sync_weights(tr, ot, init)
    _check_step(tr, ot, batch, tb.LossKind.sigmoid(), O.sigmoid_loss(), 1e-3, "layerstack", B, F, l1)


def test_staged_batch_equals_host_batch():
    F, l1, l2, B = 256, 16, 32, 256
    fs = LS_FS
    init = tb.layerstack_default_init(fs, F, l1, l2, 9)
    batch = tb.synthetic_batch(21, B, fs, pinned=True)
    a = tb.GpuTrainer(B, F, l1, l2, 9, fs, init=init)
    b = tb.GpuTrainer(B, F, l1, l2, 9, fs, init=init)
    b.stage_batch(0, batch)
    for _ in range(3):
        a.train_step(batch, 1e-3, 0.0, tb.LossKind.sigmoid())
        b.train_step_staged(0, 1e-3, 0.0, tb.LossKind.sigmoid())
    assert a.flush_pending_loss() == b.flush_pending_loss()
    assert np.array_equal(a.download_group("ft_w")["w"], b.download_group("ft_w")["w"])
    assert a.launch_count == b.launch_count and a.launch_count > 0


def _sequential_ft_grad(stm, nstm, nnz, dft_stm, dft_nstm, N, F):
    """Per feature row the one-by-one fp32 sum of the dft rows that hold it: stm items by ascending position, then
    nstm items (the order of sparse_ft_backward_cpu, crates/gpu-kernels/src/sparse_ft_backward.rs)."""
    grad = np.zeros((N, F), np.float32)
    for idx, dft in ((stm, dft_stm), (nstm, dft_nstm)):
        B, A = idx.shape
        live = (np.arange(A)[None, :] < nnz[:, None]) & (idx >= 0) & (idx < N)
        pos, _slot = np.nonzero(live)             # row-major: ascending position, then slot
        np.add.at(grad, idx[live], dft.reshape(B, F)[pos])   # unbuffered: adds one by one in this order
    return grad


@pytest.mark.parametrize("outside", [False, True])
def test_ft_slice_backward_many_chunks_bit_exact(outside):
    """King-sliced index lists with thousands of items in two slices: the slice-resident weight gradient walks several
    chunks per slice and must reproduce the sequential sum bit for bit (lists of 256 entries or more: to rounding);
    with one row outside its item's slice the generic kernels take over and must do the same."""
    F, l1, l2, B, A = 256, 8, 16, 2048, 40
    fs = LS_FS.with_factorize(False)
    pi, N = fs.piece_inputs, fs.ft_in
    rng = np.random.default_rng(11)
    init = _perturb(tb.layerstack_default_init(fs, F, l1, l2, 9), rng, ["ft_b", "l1_b", "l1_shared_bias", "l2_b", "l3_b"])
    init["ft_w"] *= 30.0
    d = random_index_batch(rng, B, A, pi, 25, A)
    hot = rng.integers(0, pi, 3)
    for key, slices in (("stm", (3, 44)), ("nstm", (3, 17))):
        k = np.asarray(slices)[rng.integers(0, 2, B)]
        idx = d[key]
        idx[:, 1] = np.where(rng.random(B) < 0.9, hot[0], idx[:, 1])     # a row that nearly every item holds
        idx[:, 2] = np.where(rng.random(B) < 0.5, hot[1], idx[:, 2])
        idx[::9, 5] = idx[::9, 4]                                        # the same feature twice in one item
        d[key] = np.where(idx >= 0, idx + k[:, None] * pi, idx).astype(np.int32)
    if outside:
        d["stm"][100, 7] = 20 * pi + 5
    batch = tb.BatchData(d["stm"], d["nstm"], d["nnz"], d["score"], d["wdl"], d["bucket"])
    tr = tb.GpuTrainer(B, F, l1, l2, 9, fs, optimizer="adamw", init=init)
    tr.forward_backward(batch, 0.25, tb.LossKind.sigmoid())
    dft_stm, dft_nstm = tr.read_buffer("dft_stm", B * F), tr.read_buffer("dft_nstm", B * F)
    assert np.abs(dft_stm).max() > 0
    want = _sequential_ft_grad(d["stm"], d["nstm"], d["nnz"], dft_stm, dft_nstm, N, F)
    got = tr.download_grad("ft_w").reshape(-1, F)[:N]
    # lists of 256 entries or more may be summed as four partial sums per chunk (fixed order, not the sequential one)
    live = lambda idx: idx[(np.arange(A)[None, :] < d["nnz"][:, None]) & (idx >= 0) & (idx < N)]
    count = np.bincount(np.concatenate([live(d["stm"]), live(d["nstm"])]), minlength=N)
    short = count < 256
    assert short.sum() > 1000 and (~short).sum() >= 4
    assert np.array_equal(got[short].view(np.uint32), want[short].view(np.uint32))
    assert_close_scaled(got[~short], want[~short], 1e-6, "long lists")


def test_config3_full_size_step_matches_oracle():
    """The benchmark's own shapes (LayerStack F=1536, l1=16, l2=32, halfka-hm-merged, B = 65 536, factorizer on): one
    forward/backward and one Ranger step against the oracle.  About 8 GB of host memory and 20 s of CPU time."""
    F, l1, l2, B, nb = 1536, 16, 32, 65536, 9
    fs = LS_FS
    rng = np.random.default_rng(65536)
    init = _perturb(tb.layerstack_default_init(fs, F, l1, l2, nb), rng, ["ft_b", "l1_b", "l1_shared_bias", "l2_b", "l3_b"])
    init["ft_w"][:fs.ft_in * F] *= 30.0
    init["ft_w"][fs.ft_in * F:] = (rng.standard_normal(fs.piece_inputs * F) * 0.02).astype(np.float32)
    tr = tb.GpuTrainer(B, F, l1, l2, nb, fs, optimizer="ranger", init=init)
    ot = _oracle_for(tr, "layerstack", fs, F, l1, l2, nb, "ranger", (0.01, 0.01, 0.01), B)
    _sync_weights(tr, ot, init)
    batch = tb.synthetic_batch(tb.SYNTH_SEED + 3, B, fs)
    lr = 8.75e-4
    l_gpu = tr.forward_backward(batch, 0.0, tb.LossKind.sigmoid(1.0 / 290.0))
    l_cpu = ot.step(_batch_dict(batch), lr, 0.0, O.sigmoid_loss(1.0 / 290.0), do_optimizer=False)
    for name in ("ft_stm", "ft_nstm"):
        assert np.array_equal(tr.read_buffer(name, B * F).view(np.uint32), ot.buffer(name).view(np.uint32)), name
    assert_close(tr.read_buffer("net_output", B), ot.buffer("net_output"), TOL_FWD, "net_output")
    assert abs(l_gpu - l_cpu) <= TOL_FWD * (1 + abs(l_cpu)), (l_gpu, l_cpu)
    assert_close_scaled(tr.read_buffer("dft_stm", B * F), ot.buffer("dft_stm"), TOL_GRAD, "dft_stm")
    for name in ot.names:
        assert_close_scaled(tr.download_grad(name), ot.group(name, "grad"), TOL_GRAD, "grad " + name)
    tr.apply_optimizer(lr); ot.apply_optimizer(lr)
    for name in ot.names:
        got = tr.download_group(name, ("w", "m", "v"))
        assert_close(got["w"], ot.group(name, "w"), TOL_FWD, "w " + name)
        assert_close_scaled(got["m"], ot.group(name, "m"), TOL_GRAD, "m " + name)
        assert_close_scaled(got["v"], ot.group(name, "v"), TOL_GRAD, "v " + name)
    w = ot.group("ft_w")
    want_comb = (w[:fs.ft_in * F].reshape(-1, fs.piece_inputs, F) + w[fs.ft_in * F:].reshape(1, fs.piece_inputs, F)).reshape(-1)
    assert_close(tr.read_buffer("comb", fs.ft_in * F), want_comb, TOL_FWD, "comb")


def test_ft_slice_backward_one_huge_slice_checksum():
    """Every item in one king-bucket slice: more chunks than a block stages descriptors for, one list as long as the
    batch.  Column sums of the gradient equal the dft rows weighted by their number of live features."""
    F, l1, l2, B, A = 256, 8, 16, 36864, 40
    fs = LS_FS.with_factorize(False)
    pi, N = fs.piece_inputs, fs.ft_in
    rng = np.random.default_rng(12)
    init = _perturb(tb.layerstack_default_init(fs, F, l1, l2, 9), rng, ["ft_b", "l1_b", "l1_shared_bias", "l2_b", "l3_b"])
    init["ft_w"] *= 30.0
    nnz = rng.integers(20, A + 1, B).astype(np.int32)
    def lists():
        idx = rng.integers(0, pi, (B, A)).astype(np.int32)      # duplicates inside an item are allowed
        idx[:, 0] = 7                                           # one row in every item
        idx[np.arange(A)[None, :] >= nnz[:, None]] = -1
        return np.where(idx >= 0, idx + 5 * pi, idx).astype(np.int32)
    stm, nstm = lists(), lists()
    batch = tb.BatchData(stm, nstm, nnz, np.clip(np.round(rng.normal(0, 400, B)), -3000, 3000).astype(np.float32),
                         rng.choice(np.array([0.0, 0.5, 1.0], np.float32), B), rng.integers(0, 9, B).astype(np.int32))
    tr = tb.GpuTrainer(B, F, l1, l2, 9, fs, optimizer="adamw", init=init)
    tr.forward_backward(batch, 0.25, tb.LossKind.sigmoid())
    dft = tr.read_buffer("dft_stm", B * F).reshape(B, F).astype(np.float64) + tr.read_buffer("dft_nstm", B * F).reshape(B, F)
    grad = tr.download_grad("ft_w").reshape(-1, F)[:N]
    assert not grad[:5 * pi].any() and not grad[6 * pi:].any()             # rows of the other slices stay zero
    want = (dft * nnz[:, None]).sum(axis=0)
    got = grad.astype(np.float64).sum(axis=0)
    assert_close_scaled(got, want, 1e-5, "column sums")
    live = np.arange(A)[None, :] < nnz[:, None]
    hits = ((stm == 5 * pi + 7) & live).sum(axis=1)[:, None] * tr.read_buffer("dft_stm", B * F).reshape(B, F).astype(np.float64) + \
        ((nstm == 5 * pi + 7) & live).sum(axis=1)[:, None] * tr.read_buffer("dft_nstm", B * F).reshape(B, F).astype(np.float64)
    assert_close_scaled(grad[5 * pi + 7].astype(np.float64), hits.sum(axis=0), 1e-5, "the row every item holds")
