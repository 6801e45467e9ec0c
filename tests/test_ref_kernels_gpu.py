"""GPU-vs-GPU parity: this library's kernels against the reference's own CUDA kernels run on the same device.

The reference's device code (crates/cuda-native-runtime/kernels/native_kernels.cu) is compiled unchanged into
oracle/_ref/native_kernels.fatbin (`make -C oracle ref`) and launched with the reference's launch shapes and
parameter packets (tests/ref_kernels.py).  This pins the pieces that the CPU oracle restates from the .cu text
only, and the CPU oracle itself, against the reference's text as it runs.

Tolerances: the reference's own (bins/nnue_train/src/tests/gpu_cpu_equivalence_tests.rs:58-66): sparse forward
bit-exact; everything that the reference sums with atomics or with interleaved partial sums 1e-5 in the form
|g - c| <= tol (1 + |c|) (gradient sums against the tensor's scale).
"""
import ctypes as C
import os

import numpy as np
import pytest

import oracle_lib as O
import ref_kernels as R
import tatara_b200 as tb
from helpers import assert_close, assert_close_scaled, random_index_batch
from ref_kernels import F32, I32, U32, U64, Slice

pytestmark = pytest.mark.gpu

LS_FS = tb.FeatureSetSpec("halfka-hm-merged", 4, 45, 1629, 40, True)
KP_FS = tb.FeatureSetSpec("halfkp", 0, 81, 1548, 38, True)
FT_POST_SCALE = 127.0 / 128.0


@pytest.fixture(scope="module")
def ref():
    if not R.available():
        pytest.skip("oracle/_ref/native_kernels.fatbin is not built (make -C oracle ref needs the reference checkout)")
    torch = pytest.importorskip("torch")
    return R.RefKernels(0)


def _cuda(ref, a):
    return ref.torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _lib():
    return tb.load_library()


# ------------------------------------------------------------------------------------------ FT kernels alone
@pytest.mark.parametrize("F,B,A,N", [(256, 1000, 38, 5000), (1536, 300, 40, 5000)])
def test_sparse_ft_forward_bit_exact_vs_reference_kernel(ref, F, B, A, N):
    rng = np.random.default_rng(F + B)
    table = (rng.standard_normal((N, F)) * 0.05).astype(np.float32)
    d = random_index_batch(rng, B, A, N, max(0, A - 10), A, with_bucket=0)
    d["stm"][::7, 0] = N + 3
    d["stm"][::5, 1] = -1
    d["stm"][::11, 2] = d["stm"][::11, 3]
    out = ref.torch.empty((B, F), dtype=ref.torch.float32, device="cuda")
    ref.sparse_ft_forward(_cuda(ref, table), _cuda(ref, d["stm"]), _cuda(ref, d["nnz"]), out, B, F, N, A)
    ref.sync()
    want = out.cpu().numpy()
    got = np.empty((B, F), np.float32)
    ms = C.c_float()
    rc = _lib().tb_ft_forward_bench(0, table.ctypes.data, d["stm"].ctypes.data, d["nnz"].ctypes.data, B, F, N, A, 1,
                                    got.ctypes.data, C.byref(ms))
    assert rc == 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # and the CPU oracle agrees with the reference kernel bit for bit
    cpu = np.empty((B, F), np.float32)
    O.lib().ora_sparse_ft_forward(table.reshape(-1), d["stm"].reshape(-1), d["nnz"], cpu.reshape(-1), B, F, N, A)
    assert np.array_equal(cpu.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("F,B,A,N", [(256, 2048, 38, 3000), (1536, 512, 40, 700)])
def test_ft_backward_vs_reference_inverse_index_pipeline(ref, F, B, A, N):
    rng = np.random.default_rng(F * 3 + B)
    dft = (rng.standard_normal((B, F)) * 1e-3).astype(np.float32)
    d = random_index_batch(rng, B, A, N, max(0, A - 8), A, with_bucket=0)
    d["stm"][d["stm"] >= N - 40] = 6   # the last 40 rows are held by nobody
    d["stm"][::9, 0] = -1
    d["stm"][::13, 1] = N + 1
    d["stm"][::3, 2] = 5            # a list of several hundred entries
    grad = ref.torch.full((N, F), 9.0, dtype=ref.torch.float32, device="cuda")
    ref.ft_backward([_cuda(ref, dft)], [_cuda(ref, d["stm"])], _cuda(ref, d["nnz"]), B, A, N, F, grad)
    ref.sync()
    want = grad.cpu().numpy()
    got = np.empty((N, F), np.float32)
    ms = C.c_float()
    rc = _lib().tb_ft_backward_bench(0, dft.ctypes.data, d["stm"].ctypes.data, d["nnz"].ctypes.data, B, F, N, A, 1,
                                     got.ctypes.data, C.byref(ms))
    assert rc == 0
    # the reference's list order comes from atomics and it keeps four interleaved partial sums: to rounding
    assert_close_scaled(got, want, 1e-5, "ft weight gradient")
    empty = np.bincount(d["stm"][(np.arange(A)[None] < d["nnz"][:, None]) & (d["stm"] >= 0) & (d["stm"] < N)], minlength=N) == 0
    assert empty.any() and not got[empty].any() and not want[empty].any()      # rows nobody holds are overwritten with 0


def test_adam_clamp_vs_reference_radam_step(ref):
    rng = np.random.default_rng(11)
    n = 128 * 1000
    w = (rng.standard_normal(n) * 0.5).astype(np.float32); m = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    v = (rng.random(n) * 1e-5).astype(np.float32); g = (rng.standard_normal(n) * 1e-2).astype(np.float32)
    dw, dm, dv, dg = (_cuda(ref, x) for x in (w, m, v, g))
    ref.launch_1d("radam_step", n, dw, dm, dv, dg, F32(1e-3), F32(1.0), I32(1), F32(0.01), F32(0.9), F32(0.999), F32(1e-8),
                  F32(-0.25), F32(0.25), U32(n))
    ref.sync()
    assert not dg.cpu().numpy().any()              # the reference's kernel also zeroes the gradient
    ms = C.c_float()
    rc = _lib().tb_adam_clamp_bench(0, w.ctypes.data, m.ctypes.data, v.ctypes.data, g.ctypes.data, n, 1e-3, 0.01, -0.25, 0.25,
                                    1, C.byref(ms))
    assert rc == 0
    assert_close(m, dm.cpu().numpy(), 1e-6, "m"); assert_close(v, dv.cpu().numpy(), 1e-6, "v")
    assert_close(w, dw.cpu().numpy(), 1e-6, "w")


# ------------------------------------------------------------------------------------------ inside a LayerStack step
@pytest.fixture(scope="module")
def ls_step(ref):
    """One forward/backward of a small LayerStack trainer; its buffers feed the reference kernels below."""
    F, l1, l2, B, nb = 256, 16, 32, 512, 9
    fs = LS_FS
    rng = np.random.default_rng(77)
    init = tb.layerstack_default_init(fs, F, l1, l2, nb)
    for n in ("ft_b", "l1_b", "l1_shared_bias", "l2_b", "l3_b"):
        init[n] = (rng.standard_normal(init[n].size) * 0.05).astype(np.float32)
    init["ft_w"][:fs.ft_in * F] *= 30.0
    init["ft_w"][fs.ft_in * F:] = (rng.standard_normal(fs.piece_inputs * F) * 0.02).astype(np.float32)
    tr = tb.GpuTrainer(B, F, l1, l2, nb, fs, optimizer="ranger", init=init)
    batch = tb.synthetic_batch(tb.SYNTH_SEED + 5, B, fs)
    batch.bucket_idx[::17] = 9          # out-of-range bucket rows
    loss = tr.forward_backward(batch, 0.25, tb.LossKind.sigmoid())
    buf = {k: tr.read_buffer(k, n) for k, n in (("ft_stm", B * F), ("ft_nstm", B * F), ("combined", B * F), ("l1_total", B * l1),
                                                ("net_output", B), ("dy", B), ("dl1_total", B * l1), ("dft_stm", B * F),
                                                ("dft_nstm", B * F), ("comb", fs.ft_in * F))}
    grads = {n: tr.download_grad(n) for n in tr.group_names}
    yield dict(F=F, l1=l1, l2=l2, B=B, nb=nb, fs=fs, init=init, tr=tr, batch=batch, loss=loss, buf=buf, grads=grads)
    tr.close()


def test_fold_virtual_vs_reference(ref, ls_step):
    s = ls_step
    fs, F = s["fs"], s["F"]
    N = fs.ft_in
    w = _cuda(ref, s["init"]["ft_w"])
    comb = ref.torch.empty(N * F, dtype=ref.torch.float32, device="cuda")
    dummy = ref.torch.zeros(1, dtype=ref.torch.int32, device="cuda")
    # launch_ft_fold (bins/nnue_train/src/ft_factorize_host.rs:81-126): bounds = base_ft_in | ft_in << 32, mode 0, nb 1
    ref.launch_1d("ft_fold_virtual", N * F, w, comb, Slice(dummy, 0), U64(N | (N << 32)), U32(F), U32(fs.piece_inputs), U32(1))
    ref.sync()
    assert np.array_equal(comb.cpu().numpy().view(np.uint32), s["buf"]["comb"].view(np.uint32))


def test_sparse_forward_inside_the_step_vs_reference(ref, ls_step):
    s = ls_step
    fs, F, B = s["fs"], s["F"], s["B"]
    comb = _cuda(ref, s["buf"]["comb"])
    nnz = _cuda(ref, s["batch"].nnz)
    for key, idx in (("ft_stm", s["batch"].stm_indices), ("ft_nstm", s["batch"].nstm_indices)):
        out = ref.torch.empty(B * F, dtype=ref.torch.float32, device="cuda")
        ref.sparse_ft_forward(comb, _cuda(ref, idx), nnz, out, B, F, fs.ft_in, fs.max_active)
        ref.sync()
        assert np.array_equal(out.cpu().numpy().view(np.uint32), s["buf"][key].view(np.uint32)), key


def test_ft_post_perspective_fwd_vs_reference(ref, ls_step):
    s = ls_step
    F, B = s["F"], s["B"]
    out = ref.torch.empty(B * F, dtype=ref.torch.float32, device="cuda")
    ref.launch_1d("ft_post_perspective_fwd", B * F, _cuda(ref, s["buf"]["ft_stm"]), _cuda(ref, s["buf"]["ft_nstm"]),
                  _cuda(ref, s["init"]["ft_b"]), out, U32(B), U32(F), F32(FT_POST_SCALE))
    ref.sync()
    assert_close(s["buf"]["combined"], out.cpu().numpy(), 1e-6, "combined")


def test_l1_bucket_plus_shared_forward_vs_reference(ref, ls_step):
    """l1_total = dense_mm_fwd_bucket (per-bucket weights, zero for out-of-range buckets) + the shared layer (a cuBLAS
    Sgemm in the reference; here a float64 product of the same operands)."""
    s = ls_step
    F, B, l1, nb, init = s["F"], s["B"], s["l1"], s["nb"], s["init"]
    out = ref.torch.empty(B * l1, dtype=ref.torch.float32, device="cuda")
    ref.launch_1d("dense_mm_fwd_bucket", B * l1, _cuda(ref, s["buf"]["combined"]), _cuda(ref, init["l1_w"]), _cuda(ref, init["l1_b"]),
                  _cuda(ref, s["batch"].bucket_idx), out, U32(B), U32(F), U32(l1), U32(nb))
    ref.sync()
    x = s["buf"]["combined"].reshape(B, F).astype(np.float64)
    shared = x @ init["l1_shared_weight"].reshape(F, l1).astype(np.float64) + init["l1_shared_bias"].astype(np.float64)
    want = out.cpu().numpy().reshape(B, l1).astype(np.float64) + shared
    assert_close(s["buf"]["l1_total"], want, 1e-5, "l1_total")


def test_loss_wdl_vs_reference(ref, ls_step):
    s = ls_step
    B = s["B"]
    dy = ref.torch.empty(B, dtype=ref.torch.float32, device="cuda")
    acc = ref.torch.zeros(1, dtype=ref.torch.float64, device="cuda")
    ref.launch_1d("loss_wdl", B, _cuda(ref, s["buf"]["net_output"]), _cuda(ref, s["batch"].score), _cuda(ref, s["batch"].wdl),
                  F32(1.0 / B), dy, acc, F32(0.25), F32(1.0 / 290.0), U32(B))
    ref.sync()
    assert_close_scaled(s["buf"]["dy"], dy.cpu().numpy(), 1e-5, "dy")
    want = float(acc.cpu()[0])
    assert abs(s["loss"] - want) <= 1e-6 * (1 + abs(want))


def test_ft_post_grad_fused_vs_reference(ref, ls_step):
    """dcombined (never stored by this library) is rebuilt from dl1_total and the L1 weights in float64, split into the
    per-bucket and the shared part as the reference's two buffers, and fed to ft_post_perspective_grad_fused."""
    s = ls_step
    F, B, l1, nb, init = s["F"], s["B"], s["l1"], s["nb"], s["init"]
    dl1 = s["buf"]["dl1_total"].reshape(B, l1).astype(np.float64)
    bucket = s["batch"].bucket_idx
    wb = init["l1_w"].reshape(nb, l1, F).astype(np.float64)
    ws = init["l1_shared_weight"].reshape(F, l1).astype(np.float64)
    valid = (bucket >= 0) & (bucket < nb)
    d_bucket = np.zeros((B, F))
    d_bucket[valid] = np.einsum("bo,bof->bf", dl1[valid], wb[bucket[valid]])
    d_shared = dl1 @ ws.T
    a, b_ = _cuda(ref, d_bucket.astype(np.float32)), _cuda(ref, d_shared.astype(np.float32))
    bias_grad = ref.torch.zeros(F, dtype=ref.torch.float32, device="cuda")
    half = F // 2
    for key, off in (("stm", 0), ("nstm", half)):
        dft = ref.torch.empty(B * F, dtype=ref.torch.float32, device="cuda")
        ref.launch_1d("ft_post_perspective_grad_fused", B * half, a, b_, _cuda(ref, s["buf"]["ft_" + key]), _cuda(ref, init["ft_b"]),
                      dft, bias_grad, U32(B), U32(F), U32(off), U32(F), F32(FT_POST_SCALE))
        ref.sync()
        assert_close_scaled(s["buf"]["dft_" + key], dft.cpu().numpy(), 1e-4, "dft_" + key)
    assert_close_scaled(s["grads"]["ft_b"], bias_grad.cpu().numpy(), 1e-4, "ft_b grad")


def test_ft_weight_gradient_and_virtual_reduce_vs_reference(ref, ls_step):
    s = ls_step
    fs, F, B = s["fs"], s["F"], s["B"]
    N, A, pi = fs.ft_in, fs.max_active, fs.piece_inputs
    grad = ref.torch.zeros((N + pi) * F, dtype=ref.torch.float32, device="cuda")
    ref.ft_backward([_cuda(ref, s["buf"]["dft_stm"]), _cuda(ref, s["buf"]["dft_nstm"])],
                    [_cuda(ref, s["batch"].stm_indices), _cuda(ref, s["batch"].nstm_indices)], _cuda(ref, s["batch"].nnz), B, A, N, F, grad)
    dummy = ref.torch.zeros(1, dtype=ref.torch.int32, device="cuda")
    ref.launch_1d("ft_reduce_virtual_grad", pi * F, grad, Slice(dummy, 0), U64(N | (N << 32)), U32(F), U32(pi), U32(1))
    ref.sync()
    assert_close_scaled(s["grads"]["ft_w"], grad.cpu().numpy(), 1e-5, "ft_w grad incl. virtual rows")


def test_ranger_step_and_lookahead_vs_reference(ref, ls_step):
    """Six optimizer steps on a fixed gradient: radam_step per group + ranger_lookahead_lerp on the sixth, against the
    library's fused kernels (the dense group l1_w with its clamp)."""
    s = ls_step
    tr = s["tr"]
    name = "l1_w"
    n = tr.group_len(name)
    st = tr.download_group(name, ("w", "m", "v", "slow"))
    g = s["grads"][name]
    w, m, v, slow = (_cuda(ref, st[k]) for k in ("w", "m", "v", "slow"))
    lr = 8.75e-4
    for step in range(1, 7):
        step_size, denom, beta1 = C.c_float(), C.c_int32(), C.c_float()
        O.lib().ora_optimizer_scalars(0, step, 0.999, 5.0, C.byref(step_size), C.byref(denom), C.byref(beta1))
        dg = _cuda(ref, g)
        ref.launch_1d("radam_step", n, w, m, v, dg, F32(lr), F32(step_size.value), I32(denom.value), F32(0.01), F32(beta1.value),
                      F32(0.999), F32(1e-8), F32(-127.0 / 64.0), F32(127.0 / 64.0), U32(n))
        if step % 6 == 0:
            ref.launch_1d("ranger_lookahead_lerp", n, w, slow, F32(0.5), U32(n))
        tr.apply_optimizer(lr)       # the gradients held by the handle stay as they are
    ref.sync()
    got = tr.download_group(name, ("w", "m", "v", "slow"))
    assert tr.step_count == 6
    assert_close(got["w"], w.cpu().numpy(), 1e-6, "w"); assert_close(got["slow"], slow.cpu().numpy(), 1e-6, "slow")
    assert_close_scaled(got["m"], m.cpu().numpy(), 1e-5, "m"); assert_close_scaled(got["v"], v.cpu().numpy(), 1e-5, "v")


# ------------------------------------------------------------------------------------------ Simple architecture
@pytest.mark.parametrize("act", ["crelu", "screlu"])
def test_simple_ft_post_and_act_grad_vs_reference(ref, act):
    F, l1, l2, B = 256, 32, 32, 256
    fs = KP_FS
    rng = np.random.default_rng(5)
    init = tb.simple_default_init(fs, F, l1, l2)
    init["ft_w"][:fs.ft_in * F] *= 4.0
    for k in ("l1_w", "l2_w", "l3_w"):
        init[k] *= 8.0
    tr = tb.SimpleGpuTrainer(B, F, l1, l2, fs, activation=act, optimizer="adamw", weight_decay=0.0, init=init)
    batch = tb.synthetic_batch(tb.SYNTH_SEED + 1, B, fs, with_bucket=False)
    lt = tb.LossKind.wrm(nnue2score=290.0, in_scaling=290.0, in_offset=0.0, target_offset=0.0, target_scaling=290.0)
    loss = tr.forward_backward(batch, 0.25, lt)
    pre = {k: tr.read_buffer("ft_" + k, B * F) for k in ("stm", "nstm")}
    combined = tr.read_buffer("combined", B * 2 * F)
    comb_tab = _cuda(ref, tr.read_buffer("comb", fs.ft_in * F))
    nnz = _cuda(ref, batch.nnz)
    out_comb = ref.torch.zeros(B * 2 * F, dtype=ref.torch.float32, device="cuda")
    ref_pre = {}
    for key, idx, off in (("stm", batch.stm_indices, 0), ("nstm", batch.nstm_indices, F)):
        ft = ref.torch.empty(B * F, dtype=ref.torch.float32, device="cuda")
        ref.sparse_ft_forward(comb_tab, _cuda(ref, idx), nnz, ft, B, F, fs.ft_in, fs.max_active)
        ref.launch_1d("simple_ft_post_fused_" + act, B * F, ft, _cuda(ref, init["ft_b"]), out_comb, U32(B), U32(F), U32(off))
        ref.sync()
        ref_pre[key] = ft
        assert np.array_equal(ft.cpu().numpy().view(np.uint32), pre[key].view(np.uint32)), "biased pre-activation " + key
    assert_close(combined, out_comb.cpu().numpy(), 1e-6, "combined")
    # loss
    dy = ref.torch.empty(B, dtype=ref.torch.float32, device="cuda")
    acc = ref.torch.zeros(1, dtype=ref.torch.float64, device="cuda")
    wsum = ref.torch.ones(1, dtype=ref.torch.float64, device="cuda")
    ref.launch_1d("loss_wrm", B, _cuda(ref, tr.read_buffer("net_output", B)), _cuda(ref, batch.score), _cuda(ref, batch.wdl), F32(1.0 / B),
                  dy, acc, F32(0.25), F32(290.0), F32(290.0), F32(0.0), F32(0.0), F32(290.0), F32(2.0), F32(0.0), F32(0.0), F32(0.5),
                  wsum, U32(0), U32(B))
    ref.sync()
    assert_close_scaled(tr.read_buffer("dy", B), dy.cpu().numpy(), 1e-5, "dy (wrm)")
    assert abs(loss - float(acc.cpu()[0])) <= 1e-6 * (1 + abs(loss))
    # activation gradient + bias gradient: dcombined rebuilt in float64 from dl1 and the L1 weights ([2F, l1] in-major)
    dl1 = tr.read_buffer("dl1_total", B * l1).reshape(B, l1).astype(np.float64)
    dcomb = _cuda(ref, (dl1 @ init["l1_w"].reshape(2 * F, l1).astype(np.float64).T).astype(np.float32))
    dfts = []
    for key, off in (("stm", 0), ("nstm", F)):
        dft = ref.torch.empty(B * F, dtype=ref.torch.float32, device="cuda")
        ref.launch_1d("simple_bwd_ft_act_%s_fused" % act, B * F, dcomb, ref_pre[key], dft, U32(B), U32(F), U32(off))
        ref.sync()
        assert_close_scaled(tr.read_buffer("dft_" + key, B * F), dft.cpu().numpy(), 1e-4, "dft_" + key)
        dfts.append(dft)
    bias_grad = ref.torch.zeros(F, dtype=ref.torch.float32, device="cuda")
    items = 64
    ref.launch("simple_bias_grad_dual", ((B + items - 1) // items, (F + 255) // 256), 256, dfts[0], dfts[1], bias_grad, U32(B), U32(F), U32(items))
    ref.sync()
    assert_close_scaled(tr.download_grad("ft_b"), bias_grad.cpu().numpy(), 1e-4, "ft_b grad")
    tr.close()
