"""Reduced-precision modes of the LayerStack trainer (--ft-fp16, --ft-fp16-out, --fp16-opt-state, --tf32; all four =
--all-optim, bins/nnue_train/src/cli.rs:623-638): CUDA path against the CPU oracle's restatement of the reference's fp16
kernels, and against those kernels themselves run on the GPU (oracle/_ref).

Tolerances (|g - c| <= tol (1 + |c|), gradient tensors against their scale), looser than fp32 where a value passes
through fp16 or TF32 storage:
  fp16 FT sums (stored pre-activations)   bit-exact: fp16 rows are summed in fp32 in slot order, then rounded once
  forward values, loss                    1e-5 without --tf32; 5e-3 with it: the reference's own bar for its TF32 products
                                          (bins/nnue_train/src/tests/gpu_cpu_equivalence_tests.rs:718, 773, 829)
  fp16 dft rows                           1e-3 (one fp16 ulp is 2^-11 relative)
  FT weight gradient                      2e-4 (a rounding flip of single fp16 terms), other gradients 1e-4 (5e-3 with --tf32)
  weights after one step                  1e-5 (1e-4 with --tf32); fp16 moments one fp16 step of the stored value
The reference's own whole-trainer bar for these modes is GPU-vs-GPU (bins/nnue_train/src/tests/native_cuda_tests.rs:24-42).
"""
import ctypes as C
import os

import numpy as np
import pytest

import oracle_lib as O
import ref_kernels as R
import tatara_b200 as tb
from helpers import assert_close, assert_close_scaled
from ref_kernels import F32, I32, U32, U64, Slice

pytestmark = pytest.mark.gpu

LS_FS = tb.FeatureSetSpec("halfka-hm-merged", 4, 45, 1629, 40, True)
LR = 8.75e-4
TF32, FT16, OUT16, STATE16 = 1, 2, 4, 8
ALL_OPTIM = TF32 | FT16 | OUT16 | STATE16


def _flags(mask):
    return tb.PrecisionFlags(tf32=bool(mask & TF32), ft_fp16=bool(mask & FT16), ft_fp16_out=bool(mask & OUT16),
                             fp16_opt_state=bool(mask & STATE16))


def _batch_dict(b):
    return dict(stm=b.stm_indices, nstm=b.nstm_indices, nnz=b.nnz, score=b.score, wdl=b.wdl, bucket=b.bucket_idx)


def _init(fs, F, l1, l2, nb, rng):
    init = tb.layerstack_default_init(fs, F, l1, l2, nb)
    for n in ("ft_b", "l1_b", "l1_shared_bias", "l2_b", "l3_b"):
        init[n] = (rng.standard_normal(init[n].size) * 0.05).astype(np.float32)
    init["ft_w"][:fs.ft_in * F] *= 30.0
    if fs.ft_factorize:
        init["ft_w"][fs.ft_in * F:] = (rng.standard_normal(fs.piece_inputs * F) * 0.02).astype(np.float32)
    return init


def _pair(fs, F, l1, l2, nb, B, mask, init, optimizer="ranger"):
    tr = tb.GpuTrainer(B, F, l1, l2, nb, fs, optimizer=optimizer, precision=_flags(mask), init=init)
    ot = O.OracleTrainer(arch="layerstack", ft_in=fs.ft_in, piece_inputs=fs.piece_inputs, factorize=fs.ft_factorize,
                         max_active=fs.max_active, ft_out=F, l1=l1, l2=l2, num_buckets=nb, optimizer=optimizer, capacity=B,
                         precision=mask)
    ot.set_threads(os.cpu_count() or 1)
    for name in ot.names:
        ot.group(name)[:] = init[name]
    return tr, ot


def _assert_close_fp16_stored(got, want, store_scale, tol, what):
    """A value kept as fp16(value * store_scale): beside the relative tolerance (against the tensor's scale) one fp16
    step of the stored value is allowed (2^-24 below the normal range), since inputs that differ in the last fp32 bits
    can round to neighbouring fp16 values."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    stored = np.abs(want) * store_scale
    ulp = np.maximum(2.0 ** -24, 2.0 ** (np.floor(np.log2(np.maximum(stored, 2.0 ** -14))) - 10)) / store_scale
    err = np.abs(got - want) - tol * (np.abs(want).max() + np.abs(want)) - 1.01 * ulp
    i = int(np.argmax(err))
    assert err[i] <= 0, "%s: element %d got %r want %r" % (what, i, got[i], want[i])


def _check_step(tr, ot, batch, B, F, l1, mask, fs):
    tf32 = bool(mask & TF32)
    tol_fwd = 5e-3 if tf32 else 1e-5
    tol_grad = 5e-3 if tf32 else 1e-4
    loss_t, loss_o = tb.LossKind.sigmoid(1.0 / 290.0), O.sigmoid_loss(1.0 / 290.0)
    l_gpu = tr.forward_backward(batch, 0.0, loss_t)
    l_cpu = ot.step(_batch_dict(batch), LR, 0.0, loss_o, do_optimizer=False)
    for name in ("ft_stm", "ft_nstm"):
        got, want = tr.read_buffer(name, B * F), ot.buffer(name)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name + " must be bit-exact"
        if mask & OUT16:
            assert np.array_equal(got, got.astype(np.float16).astype(np.float32)), "stored as fp16"
    if mask & FT16:
        comb = tr.read_buffer("comb", fs.ft_in * F)
        want = ot.buffer("comb") if fs.ft_factorize else ot.group("ft_w")
        assert np.array_equal(comb, want.astype(np.float16).astype(np.float32)), "fp16 forward table"
    assert_close(tr.read_buffer("combined", B * F), ot.buffer("combined"), 1e-5, "combined")
    assert_close(tr.read_buffer("l1_total", B * l1), ot.buffer("l1_total"), tol_fwd, "l1_total")
    assert_close(tr.read_buffer("net_output", B), ot.buffer("net_output"), tol_fwd, "net_output")
    assert abs(l_gpu - l_cpu) <= tol_fwd * (1 + abs(l_cpu)), (l_gpu, l_cpu)
    assert_close_scaled(tr.read_buffer("dy", B), ot.buffer("dy"), tol_grad, "dy")
    assert_close_scaled(tr.read_buffer("dl1_total", B * l1), ot.buffer("dl1_total"), tol_grad, "dl1_total")
    tol_dft = max(1e-3 if mask & OUT16 else 1e-4, tol_grad)
    assert_close_scaled(tr.read_buffer("dft_stm", B * F), ot.buffer("dft_stm"), tol_dft, "dft_stm")
    assert_close_scaled(tr.read_buffer("dft_nstm", B * F), ot.buffer("dft_nstm"), tol_dft, "dft_nstm")
    for name in ot.names:
        tol = max(2e-4 if (name == "ft_w" and mask & OUT16) else 1e-4, tol_grad)
        assert_close_scaled(tr.download_grad(name), ot.group(name, "grad"), tol, "grad " + name)
    if mask & OUT16:
        assert tr.read_fp16_clamp_count() == ot.clamp_count() == (0, 2 * B * F)
    tr.apply_optimizer(LR); ot.apply_optimizer(LR)
    tol_w = 1e-4 if tf32 else 1e-5
    for name in ot.names:
        got = tr.download_group(name, ("w", "m", "v"))
        assert_close(got["w"], ot.group(name, "w"), tol_w, "w " + name)
        if name == "ft_w" and mask & STATE16:
            _assert_close_fp16_stored(got["m"], ot.group(name, "m"), 2.0 ** 28, tol_grad, "m " + name)
            _assert_close_fp16_stored(got["v"], ot.group(name, "v"), 2.0 ** 40, tol_grad, "v " + name)
        else:
            assert_close_scaled(got["m"], ot.group(name, "m"), tol_grad, "m " + name)
            assert_close_scaled(got["v"], ot.group(name, "v"), tol_grad, "v " + name)
    if mask & STATE16:
        m = tr.download_group("ft_w", ("m",))["m"] * np.float32(2.0 ** 28)
        assert np.array_equal(m, m.astype(np.float16).astype(np.float32)), "moments are stored as fp16 of m * 2^28"


@pytest.mark.parametrize("mask,factorize,F,l1,B", [
    (FT16, True, 256, 16, 512), (FT16 | OUT16, True, 256, 16, 512), (STATE16, True, 256, 16, 256),
    (FT16 | OUT16 | STATE16, True, 768, 8, 256), (FT16 | OUT16 | STATE16, False, 512, 32, 496), (FT16, False, 256, 16, 256),
    (ALL_OPTIM, True, 256, 16, 512)])
def test_reduced_precision_step_matches_oracle(mask, factorize, F, l1, B):
    fs = LS_FS.with_factorize(factorize)
    rng = np.random.default_rng(F + B + mask)
    init = _init(fs, F, l1, 32, 9, rng)
    tr, ot = _pair(fs, F, l1, 32, 9, B, mask, init)
    batch = tb.synthetic_batch(tb.SYNTH_SEED + 3, B, fs)
    batch.bucket_idx[::19] = 9       # rows with an out-of-range bucket
    _check_step(tr, ot, batch, B, F, l1, mask, fs)
    tr.close()


def test_reduced_precision_with_index_lists_outside_the_king_slices():
    """Arbitrary index lists break the king-slice property: the generic fp16 kernels take over (same results)."""
    from helpers import random_index_batch
    F, l1, B = 256, 16, 128
    fs = LS_FS.with_factorize(False)
    rng = np.random.default_rng(3)
    init = _init(fs, F, l1, 32, 9, rng)
    mask = FT16 | OUT16 | STATE16
    tr, ot = _pair(fs, F, l1, 32, 9, B, mask, init, optimizer="adamw")
    d = random_index_batch(rng, B, 40, fs.ft_in, 0, 40)
    d["stm"][::3, 0] = fs.ft_in + 5
    d["nstm"][::4, 1] = -1
    batch = tb.BatchData(d["stm"], d["nstm"], d["nnz"], d["score"], d["wdl"], d["bucket"])
    _check_step(tr, ot, batch, B, F, l1, mask, fs)
    tr.close()


def test_all_optim_config3_full_size_step_matches_oracle():
    """Config 3 under --all-optim at B = 65 536: one forward/backward and one Ranger step against the oracle."""
    F, l1, l2, B, nb = 1536, 16, 32, 65536, 9
    fs = LS_FS
    init = _init(fs, F, l1, l2, nb, np.random.default_rng(65536))
    tr, ot = _pair(fs, F, l1, l2, nb, B, ALL_OPTIM, init)
    batch = tb.synthetic_batch(tb.SYNTH_SEED + 3, B, fs)
    _check_step(tr, ot, batch, B, F, l1, ALL_OPTIM, fs)
    tr.close()


def test_fp16_clamp_counter_counts_what_the_oracle_counts():
    """A per-position normaliser 2^8 too large pushes part of the loss-scaled dft rows beyond +-65504: they are clamped
    and counted (read_fp16_clamp_count, crates/nnue-train/src/trainer.rs:1100-1119)."""
    F, l1, B = 256, 16, 256
    fs = LS_FS
    init = _init(fs, F, l1, 32, 9, np.random.default_rng(1))
    for k in ("l1_w", "l1_shared_weight", "l2_w", "l3_w"):
        init[k] = init[k] * np.float32(40.0)
    mask = FT16 | OUT16
    tr, ot = _pair(fs, F, l1, 32, 9, B, mask, init)
    batch = tb.synthetic_batch(77, B, fs)
    batch.per_pos_norm = 4096.0 / B
    tr.forward_backward(batch, 0.0, tb.LossKind.sigmoid(0.5))
    ot.step(_batch_dict(batch), LR, 0.0, O.sigmoid_loss(0.5), per_pos_norm=4096.0 / B, do_optimizer=False)
    got, want = tr.read_fp16_clamp_count(), ot.clamp_count()
    assert want[0] > 100 and got[1] == want[1] == 2 * B * F
    assert abs(got[0] - want[0]) <= 0.01 * want[0] + 2, (got, want)      # elements within rounding of the limit may differ
    assert np.abs(tr.read_buffer("dft_stm", B * F)).max() <= 65504.0 / (16384.0 * B) * (1 + 1e-6)
    tr.close()


def test_all_optim_eight_steps_follow_the_oracle():
    """Eight Ranger steps under --all-optim on changing batches: per-step loss within 2e-3 relative, weights within 1e-3."""
    F, l1, l2, B, nb = 256, 16, 32, 512, 9
    fs = LS_FS
    init = _init(fs, F, l1, l2, nb, np.random.default_rng(8))
    for k in ("l1_w", "l1_shared_weight", "l2_w", "l3_w"):
        init[k] = init[k] * np.float32(60.0)
    tr, ot = _pair(fs, F, l1, l2, nb, B, ALL_OPTIM, init)
    lt, lo = tb.LossKind.sigmoid(0.5), O.sigmoid_loss(0.5)
    want, got = [], []
    for s in range(8):
        batch = tb.synthetic_batch(100 + s, B, fs)
        want.append(ot.step(_batch_dict(batch), 1e-3, 0.0, lo))
        got.append(tr.train_step(batch, 1e-3, 0.0, lt))
    got.append(tr.flush_pending_loss())
    for s in range(8):
        assert abs(got[s + 1] - want[s]) <= 2e-3 * abs(want[s]), (s, got[s + 1], want[s])
    assert want[-1] < want[0]
    for name in ot.names:
        g = tr.download_group(name, ("w", "slow"))
        assert_close(g["w"], ot.group(name, "w"), 1e-3, "w after 8 steps " + name)
        assert_close(g["slow"], ot.group(name, "slow"), 1e-3, "slow " + name)
    tr.close()


def test_unsupported_precision_combinations_are_errors():
    with pytest.raises(tb.TrainerError, match="LayerStack"):
        tb.SimpleGpuTrainer(64, 256, 32, 32, tb.FEATURE_SETS["halfkp"], precision=_flags(FT16))
    with pytest.raises(tb.TrainerError, match="requires --ft-fp16"):
        tb.GpuTrainer(64, 256, 16, 32, 9, LS_FS, precision=tb.PrecisionFlags(ft_fp16_out=True))
    with pytest.raises(tb.TrainerError, match="8, 16 or 32"):
        tb.GpuTrainer(64, 256, 12, 32, 9, LS_FS, precision=_flags(FT16))


# ---------------------------------------------------------------------------------------------- against the reference's fp16 kernels
@pytest.fixture(scope="module")
def ref():
    if not R.available():
        pytest.skip("oracle/_ref/native_kernels.fatbin is not built")
    pytest.importorskip("torch")
    return R.RefKernels(0)


def test_fp16_path_vs_reference_fp16_kernels(ref):
    """ft_fold_virtual_f16, sparse_ft_forward_fp16_out, ft_post_perspective_fwd_fp16, ft_post_perspective_grad_fused_fp16,
    gather_and_sum_per_feature_*_fp16 and radam_step_f16state of the reference, launched on the same GPU with the
    reference's launch shapes, against the buffers of one --ft-fp16 --ft-fp16-out --fp16-opt-state step."""
    t = ref.torch
    F, l1, l2, B, nb = 256, 16, 32, 512, 9
    fs = LS_FS
    N, A, pi = fs.ft_in, fs.max_active, fs.piece_inputs
    init = _init(fs, F, l1, l2, nb, np.random.default_rng(21))
    mask = FT16 | OUT16 | STATE16
    tr = tb.GpuTrainer(B, F, l1, l2, nb, fs, optimizer="ranger", precision=_flags(mask), init=init)
    batch = tb.synthetic_batch(tb.SYNTH_SEED + 9, B, fs)
    tr.forward_backward(batch, 0.0, tb.LossKind.sigmoid())
    cu = lambda a: t.from_numpy(np.ascontiguousarray(a)).cuda()
    dummy = t.zeros(1, dtype=t.int32, device="cuda")
    # fold to fp16
    comb_h = t.empty(N * F, dtype=t.float16, device="cuda")
    ref.launch_1d("ft_fold_virtual_f16", N * F, cu(init["ft_w"]), comb_h, Slice(dummy, 0), U64(N | (N << 32)), U32(F), U32(pi), U32(1))
    ref.sync()
    assert np.array_equal(comb_h.cpu().numpy().astype(np.float32), tr.read_buffer("comb", N * F))
    # forward with fp16 output, then the activation
    nnz = cu(batch.nnz)
    outs = {}
    for key, idx in (("stm", batch.stm_indices), ("nstm", batch.nstm_indices)):
        o = t.empty(B * F, dtype=t.float16, device="cuda")
        ref.sparse_ft_forward(comb_h, cu(idx), nnz, o, B, F, N, A, name="sparse_ft_forward_fp16_out")
        ref.sync()
        outs[key] = o
        assert np.array_equal(o.cpu().numpy().astype(np.float32), tr.read_buffer("ft_" + key, B * F)), key
    comb = t.empty(B * F, dtype=t.float32, device="cuda")
    ref.launch_1d("ft_post_perspective_fwd_fp16", B * F, outs["stm"], outs["nstm"], cu(init["ft_b"]), comb, U32(B), U32(F), F32(127.0 / 128.0))
    ref.sync()
    assert_close(tr.read_buffer("combined", B * F), comb.cpu().numpy(), 1e-6, "combined")
    # activation gradient to fp16: dcombined rebuilt in float64 from dl1_total and the L1 weights
    dl1 = tr.read_buffer("dl1_total", B * l1).reshape(B, l1).astype(np.float64)
    wb = init["l1_w"].reshape(nb, l1, F).astype(np.float64)
    d_bucket = np.einsum("bo,bof->bf", dl1, wb[batch.bucket_idx])
    d_shared = dl1 @ init["l1_shared_weight"].reshape(F, l1).astype(np.float64).T
    a, b_ = cu(d_bucket.astype(np.float32)), cu(d_shared.astype(np.float32))
    bias_grad = t.zeros(F, dtype=t.float32, device="cuda")
    counter = t.zeros(1, dtype=t.int64, device="cuda")
    scale = 16384.0 * B
    dfts = []
    for key, off in (("stm", 0), ("nstm", F // 2)):
        dft = t.empty(B * F, dtype=t.float16, device="cuda")
        ref.launch_1d("ft_post_perspective_grad_fused_fp16", B * F // 2, a, b_, outs[key], cu(init["ft_b"]), dft, bias_grad, counter,
                      U32(B), U32(F), U32(off), U32(F), F32(127.0 / 128.0), F32(scale))
        ref.sync()
        dfts.append(dft)
        want = dft.cpu().numpy().astype(np.float32) / np.float32(scale)
        assert_close_scaled(tr.read_buffer("dft_" + key, B * F), want, 1e-3, "dft_" + key)
    assert int(counter.cpu()[0]) == 0 == tr.read_fp16_clamp_count()[0]
    assert_close_scaled(tr.download_grad("ft_b"), bias_grad.cpu().numpy(), 1e-4, "ft_b grad")
    # FT weight gradient from the fp16 rows (the library's own rows, so that only the summation is compared)
    grad = t.zeros((N + pi) * F, dtype=t.float32, device="cuda")
    mine = [cu((tr.read_buffer("dft_" + k, B * F) * np.float32(scale)).astype(np.float16)) for k in ("stm", "nstm")]
    ref.ft_backward(mine, [cu(batch.stm_indices), cu(batch.nstm_indices)], nnz, B, A, N, F, grad, suffix="_fp16", extra=(F32(1.0 / scale),))
    ref.launch_1d("ft_reduce_virtual_grad", pi * F, grad, Slice(dummy, 0), U64(N | (N << 32)), U32(F), U32(pi), U32(1))
    ref.sync()
    g_mine = tr.download_grad("ft_w")
    assert_close_scaled(g_mine, grad.cpu().numpy(), 1e-5, "ft_w grad from fp16 rows")
    # optimizer with fp16 state: two steps, so that the second reads back stored fp16 moments
    w, m, v = cu(init["ft_w"]), t.zeros((N + pi) * F, dtype=t.float16, device="cuda"), t.zeros((N + pi) * F, dtype=t.float16, device="cuda")
    n = (N + pi) * F
    for step in (1, 2):
        step_size, denom, beta1 = C.c_float(), C.c_int32(), C.c_float()
        O.lib().ora_optimizer_scalars(0, step, 0.999, 5.0, C.byref(step_size), C.byref(denom), C.byref(beta1))
        ref.launch_1d("radam_step_f16state", n, w, m, v, cu(g_mine), F32(LR), F32(step_size.value), I32(denom.value), F32(0.01),
                      F32(beta1.value), F32(0.999), F32(1e-8), F32(-3.0e38), F32(3.0e38), F32(2.0 ** 28), F32(2.0 ** 40), U32(n))
        tr.apply_optimizer(LR)
    ref.sync()
    got = tr.download_group("ft_w", ("w", "m", "v"))
    assert_close(got["w"], w.cpu().numpy(), 1e-6, "ft_w after two fp16-state steps")
    assert_close_scaled(got["m"], m.cpu().numpy().astype(np.float32) / np.float32(2.0 ** 28), 1e-3, "m")
    assert_close_scaled(got["v"], v.cpu().numpy().astype(np.float32) / np.float32(2.0 ** 40), 1e-3, "v")
    tr.close()
