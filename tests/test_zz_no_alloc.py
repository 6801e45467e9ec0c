"""The allocation-free FT backward entry point (tb_ft_backward_static_scratch).

Callers with a fixed GPU memory plan (a framework allocator that owns the device, a service that may not
touch cudaMalloc after start-up) pass their own device buffers; the library's working memory for the
inverse index lives in a static device array.  This test plays such a caller: torch owns every buffer,
the result must equal the allocating entry point's (tb_ft_backward_bench) bit for bit — the FT backward
sums in a fixed order — on two calls in a row that share the static array, the second one on a different
problem so that stale contents of the array would show.  Collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

import tatara_b200 as tb

pytestmark = pytest.mark.gpu


def _reference(dft, idx, nnz, N, F, A):
    lib = tb.load_library()
    B = nnz.shape[0]
    grad = np.empty((N, F), np.float32)
    ms = C.c_float()
    rc = lib.tb_ft_backward_bench(0, dft.ctypes.data, idx.ctypes.data, nnz.ctypes.data, B, F, N, A, 1, grad.ctypes.data,
                                  C.byref(ms))
    assert rc == 0, lib.tb_last_error(None)
    return grad


def _problem(seed, B, F, N, A):
    rng = np.random.default_rng(seed)
    dft = (rng.standard_normal((B, F)) * 1e-3).astype(np.float32)
    idx = np.full((B, A), -1, np.int32)
    nnz = rng.integers(0, A + 1, B).astype(np.int32)
    for b in range(B):
        idx[b, :nnz[b]] = rng.choice(N, nnz[b], replace=False)
    idx[::7, 0] = 3            # one hot feature: a list long enough for the long-list path
    idx[::11, 1] = N + 9       # out of range: skipped
    return dft, idx, nnz


def test_static_scratch_matches_allocating_entry_point_twice():
    torch = pytest.importorskip("torch")
    lib = tb.load_library()
    torch.cuda.set_device(0)
    err = C.create_string_buffer(256)
    for call, (B, F, N, A) in enumerate([(2048, 256, 3000, 38), (1024, 512, 700, 40)]):
        dft, idx, nnz = _problem(call, B, F, N, A)
        want = _reference(dft, idx, nnz, N, F, A)
        d_dft = torch.from_numpy(dft).cuda()
        d_idx = torch.from_numpy(idx).cuda()
        d_nnz = torch.from_numpy(nnz).cuda()
        d_grad = torch.full((N, F), 7.0, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.tb_ft_backward_static_scratch(d_dft.data_ptr(), d_idx.data_ptr(), d_nnz.data_ptr(), B, F, N, A,
                                               d_grad.data_ptr(), None, err, 256)
        assert rc == 0, err.value
        torch.cuda.synchronize()
        # The CUDA runtime makes the library's static array resident when its module is first used, which can be
        # this very first call; every later call must leave the device's free memory exactly where it was.
        if call > 0:
            assert abs(torch.cuda.mem_get_info()[0] - free_before) < (1 << 20)
        got = d_grad.cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "call %d differs" % call


def test_static_scratch_long_list_is_summed_like_the_allocating_entry_point():
    """A feature held by every position: its list (16 384 entries) is cut into parts of 4096 by both entry points,
    so they agree bit for bit; against the one-by-one sum of the CPU oracle the row agrees to rounding."""
    torch = pytest.importorskip("torch")
    import oracle_lib as O
    from helpers import assert_close_scaled
    lib = tb.load_library()
    torch.cuda.set_device(0)
    B, F, N, A = 16384, 256, 64, 4
    rng = np.random.default_rng(5)
    dft = (rng.standard_normal((B, F)) * 1e-3).astype(np.float32)
    idx = np.stack([np.full(B, 7), rng.integers(8, N, B), rng.integers(8, N, B), np.full(B, -1)], 1).astype(np.int32)
    nnz = np.full(B, 3, np.int32)
    want = _reference(dft, idx, nnz, N, F, A)
    d_dft, d_idx, d_nnz = torch.from_numpy(dft).cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(nnz).cuda()
    d_grad = torch.full((N, F), 7.0, dtype=torch.float32, device="cuda")
    err = C.create_string_buffer(256)
    rc = lib.tb_ft_backward_static_scratch(d_dft.data_ptr(), d_idx.data_ptr(), d_nnz.data_ptr(), B, F, N, A,
                                           d_grad.data_ptr(), None, err, 256)
    assert rc == 0, err.value
    torch.cuda.synchronize()
    got = d_grad.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    seq = np.zeros((N, F), np.float32)
    O.lib().ora_sparse_ft_backward(dft.reshape(-1), idx.reshape(-1), seq.reshape(-1), B, F, N, A)
    assert_close_scaled(got, seq, 1e-5, "long list against the sequential sum")
    assert np.array_equal(got[8:].view(np.uint32), seq[8:].view(np.uint32))      # short lists: the sequential sum itself
    # a misaligned buffer is refused before anything is launched
    rc = lib.tb_ft_backward_static_scratch(d_dft.data_ptr() + 4, d_idx.data_ptr(), d_nnz.data_ptr(), B - 16, F, N, A,
                                           d_grad.data_ptr(), None, err, 256)
    assert rc == -1 and b"16-byte aligned" in err.value


def test_static_scratch_rejects_sizes_beyond_its_array():
    lib = tb.load_library()
    err = C.create_string_buffer(256)
    one = C.c_void_p(16)   # never dereferenced: the size checks come first
    rc = lib.tb_ft_backward_static_scratch(one, one, one, 16, 256, 131073, 40, one, None, err, 256)
    assert rc == -1 and b"static scratch limit" in err.value and b"131072" in err.value
    rc = lib.tb_ft_backward_static_scratch(one, one, one, 65536, 256, 1000, 40, one, None, err, 256)
    assert rc == -1 and b"index slots" in err.value
    rc = lib.tb_ft_backward_static_scratch(None, one, one, 16, 256, 1000, 40, one, None, err, 256)
    assert rc == -1 and b"NULL" in err.value
