"""Shared helpers of the test-suite."""
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def assert_close(got, want, tol, what=""):
    """The reference's comparison form |g - c| <= tol * (1 + |c|)
    (bins/nnue_train/src/tests/gpu_cpu_equivalence_tests.rs:155-172)."""
    got = np.asarray(got, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    assert got.shape == want.shape, "%s: shape %s vs %s" % (what, got.shape, want.shape)
    assert np.isfinite(got).all(), "%s: non-finite values" % what
    err = np.abs(got - want) - tol * (1.0 + np.abs(want))
    i = int(np.argmax(err)) if err.size else 0
    assert err.size == 0 or err[i] <= 0, "%s: element %d got %r want %r (tol %g)" % (what, i, got[i], want[i], tol)


def assert_close_scaled(got, want, tol, what=""):
    """Gradient tensors: |g - c| <= tol * (max|c| + |c|).  Sums of many terms of mixed sign are compared
    against the tensor's scale, since single cells can cancel to ~0."""
    got = np.asarray(got, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    assert got.shape == want.shape, "%s: shape %s vs %s" % (what, got.shape, want.shape)
    assert np.isfinite(got).all(), "%s: non-finite values" % what
    scale = float(np.max(np.abs(want))) if want.size else 0.0
    err = np.abs(got - want) - tol * (scale + np.abs(want))
    i = int(np.argmax(err)) if err.size else 0
    assert err.size == 0 or err[i] <= 0, "%s: element %d got %r want %r (scale %g, tol %g)" % (what, i, got[i], want[i], scale, tol)


def sort_rows(idx):
    """Sorts every row ascending with the -1 padding last."""
    big = np.where(idx < 0, 1 << 30, idx)
    big = np.sort(big, axis=1)
    big[big == (1 << 30)] = -1
    return big.astype(np.int32)


def random_index_batch(rng, B, A, N, nnz_lo, nnz_hi, with_bucket=9, pad=-1):
    """Random distinct indices per row (the FT microbenchmark's inputs) plus targets."""
    stm = np.full((B, A), pad, np.int32)
    nstm = np.full((B, A), pad, np.int32)
    nnz = rng.integers(nnz_lo, nnz_hi + 1, B).astype(np.int32)
    for b in range(B):
        stm[b, :nnz[b]] = rng.choice(N, nnz[b], replace=False)
        nstm[b, :nnz[b]] = rng.choice(N, nnz[b], replace=False)
    out = dict(stm=stm, nstm=nstm, nnz=nnz,
               score=np.clip(np.round(rng.normal(0, 400, B)), -3000, 3000).astype(np.float32),
               wdl=rng.choice(np.array([0.0, 0.5, 1.0], np.float32), B))
    if with_bucket:
        out["bucket"] = rng.integers(0, with_bucket, B).astype(np.int32)
    return out
