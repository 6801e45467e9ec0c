"""Benchmark of the NNUE training step (positions/s) on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg3|cfg2|cfg1]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

A step is one full training step (forward, loss, backward, gradient all-reduce when N > 1, optimizer) of
the workload on one batch of 65 536 synthetic positions per GPU (weak scaling).  `value` runs on batches
already resident in HBM; `e2e` passes page-locked HOST batches through tb_train_step every step (copies
inside the timed region, the lagged loss read back every step).  The timed region of K steps is repeated
(`repeats`); the line reports the median repeat.  Prints one JSON line on rank 0.

At N = 1 the line also carries `ft_microbench` (the FT kernels alone over ft_out 256..3072 x batch 4096..262 144,
HBM GB/s against the measured peak), `other_configs` (the other single-GPU configurations in short) and
`cpu_baseline`.  At N > 1 the ranks first check the data-parallel step against the CPU oracle on a small shape
(`dp_parity`) and compare their replicas after the timed steps (`replicas_identical`).

`--impl reference` times the CPU restatement of the reference's step (oracle/, OpenMP over all host
cores) on the same workload.  The reference itself is Rust and cannot be built on a box without cargo, so the
oracle port is the CPU arm; where the reference's own CUDA kernels were compiled (oracle/_ref) and a GPU is
present, their timings on the microbenchmark shapes are reported beside it (`reference_gpu_kernels`).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

BATCH = 65536
LR = 8.75e-4  # bins/nnue_train/src/cli.rs:260
SYNTH_SEED = 0x7A7A2A
WORKLOADS = {
    # the headline configuration (cfg3) and the two smaller ones the same step is checked and timed on
    "cfg3": dict(arch="layerstack", fs="halfka-hm-merged", F=1536, l1=16, l2=32, nb=9, optimizer="ranger",
                 name="LayerStack ft1536 l1=16 l2=32 halfka-hm-merged kingrank9 fp32 ranger factorizer-on"),
    "cfg2": dict(arch="layerstack", fs="halfka-hm-merged", F=768, l1=8, l2=32, nb=9, optimizer="ranger",
                 name="LayerStack ft768 l1=8 l2=32 halfka-hm-merged kingrank9 fp32 ranger factorizer-on"),
    "cfg1": dict(arch="simple", fs="halfkp", F=256, l1=32, l2=32, nb=0, optimizer="adamw",
                 name="Simple halfkp 256x2-32-32 crelu fp32 adamw wrm(290) factorizer-on"),
}
CONFIG_INDEX = {"cfg1": 1, "cfg2": 2, "cfg3": 3}
# (king buckets, piece inputs, max active): crates/shogi-features/src/feature_set.rs:1031-1038
FS_DIMS = {"halfkp": (81, 1548, 38), "halfka-hm-merged": (45, 1629, 40)}
# used only when the box has no MEASURED_PEAKS.json: an earlier STREAM-style copy measurement on B200
FALLBACK_HBM_GBS = 6650.0
SMEM_BYTES_PER_CLK_PER_SM = 128.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel of each phase, from one ncu capture of
# cfg3 at B = 65 536, fp32, on one GPU (its summary is the launch-list file under profiles/).  Reported only for that
# exact case; any other batch, precision or GPU count prints null.
NCU_TRAFFIC_BYTES = {
    ("cfg3", "ft_backward"): 1635.0e6, ("cfg3", "ft_forward"): 1750.2e6, ("cfg3", "opt_ft"): 4232.5e6,
    ("cfg3", "l1_dgrad_ftgrad"): 1583.3e6, ("cfg3", "l1_forward"): 404.8e6, ("cfg3", "l1_wgrad"): 411.2e6,
}
MICRO_F = (256, 768, 1536, 3072)
MICRO_B = (4096, 16384, 65536, 262144)


def peak_hbm():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def algorithmic_bytes(w, n_pos, all_optim=False):
    """Algorithmic bytes per launch of each kernel phase: every large tensor crosses HBM once per producer and
    once per consumer; index arrays, [B, <=32] tensors and the small parameter groups are left out.
    Under --all-optim the FT table read by the forward, the pre-activations, the dft rows and the FT moments are fp16."""
    kb, pi, _ = FS_DIMS[w["fs"]]
    F = w["F"]
    W = kb * pi * F * 4.0
    Wt = (kb + 1) * pi * F * 4.0
    X = n_pos * F * 4.0
    comb = X if w["arch"] == "layerstack" else 2 * X      # the L1 input [B, F] or [B, 2F]
    if all_optim:
        Wh, Xh = W / 2, X / 2
        d = {
            "ft_forward": Wh + 2 * Xh + comb,      # fp16 table in, fp16 pre-activations and the fp32 L1 input out
            "l1_forward": comb,
            "l1_wgrad": comb,
            "l1_dgrad_ftgrad": 4 * Xh,             # fp16 pre-activations in, fp16 dft out
            "ft_backward": 2 * Xh + W,             # fp16 dft in, fp32 gradient rows out
            "opt_ft": 5 * Wt + Wh,                 # w, g in (fp32), m, v in and out (fp16), w out; fp16 folded table out
        }
        d["step"] = sum(d.values())                # = 2W + 5Wt + 7X
        return d
    return {
        "ft_forward": W + 2 * X + comb,        # read the table once, write both pre-activations and the L1 input
        "l1_forward": comb,                    # read the L1 input
        "l1_wgrad": comb,                      # read the L1 input again
        "l1_dgrad_ftgrad": 4 * X,              # read both pre-activations, write both dft
        "ft_backward": 2 * X + W,              # read both dft, write the real gradient rows
        "opt_ft": 7 * Wt + W,                  # w, m, v, grad in; w, m, v out; folded table out
        "step": 4 * W + 7 * Wt + (13 if w["arch"] == "layerstack" else 18) * X,
    }


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.lines, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ts, line in self.lines:
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                clk, cmax = float(p[1]), float(p[2])
            except ValueError:
                continue
            mx.append(cmax)
            if t0 - 0.05 <= ts <= t1 + 0.15:
                sm.append(clk)
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        if not sm:   # a very short timed region can fall between two samples: use everything sampled
            sm = [float(l.split(",")[1]) for _, l in self.lines if len(l.split(",")) >= 9 and l.split(",")[1].strip().replace(".", "").isdigit()]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


NCCL_ENV = {"NCCL_NVLS_ENABLE": "0", "NCCL_ALGO": "Ring", "NCCL_PROTO": "Simple"}


def make_trainer(tb, w, device, world, rank, nccl_id, capacity=BATCH, precision=None, nccl_ctas=0, dp_exchange="nccl"):
    fs = tb.FEATURE_SETS[w["fs"]]
    kw = {} if precision is None else {"precision": precision}
    if nccl_ctas:
        kw["nccl_ctas"] = nccl_ctas
    if world > 1:
        kw["dp_exchange"] = dp_exchange
    if w["arch"] == "layerstack":
        tr = tb.GpuTrainer(capacity, w["F"], w["l1"], w["l2"], w["nb"], fs, optimizer=w["optimizer"], device=device,
                           world_size=world, rank=rank, nccl_id=nccl_id, **kw)
        loss = tb.LossKind.sigmoid(1.0 / 290.0)
    else:
        tr = tb.SimpleGpuTrainer(capacity, w["F"], w["l1"], w["l2"], fs, optimizer=w["optimizer"], weight_decay=0.0,
                                 device=device, world_size=world, rank=rank, nccl_id=nccl_id, **kw)
        loss = tb.LossKind.wrm(nnue2score=290.0, in_scaling=290.0, in_offset=0.0, target_offset=0.0, target_scaling=290.0)
    return tr, loss, fs


# ---------------------------------------------------------------------------------------------- CPU arm (oracle only)
def run_cpu(w, wname, threads, sample_b, steps, warmup, limit_s=None):
    """Times the oracle's whole step on `sample_b` synthetic positions; returns (pos/s, steps done, ms/step).
    Touches nothing but oracle/ (records come from the oracle's own seeded generator)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    kb, pi, A = FS_DIMS[w["fs"]]
    ot = O.OracleTrainer(arch=w["arch"], ft_in=kb * pi, piece_inputs=pi, factorize=True, max_active=A, ft_out=w["F"],
                         l1=w["l1"], l2=w["l2"], num_buckets=max(w["nb"], 1), optimizer=w["optimizer"],
                         wd=(0.01, 0.01, 0.01) if w["arch"] == "layerstack" else (0.0, 0.0, 0.0), capacity=sample_b)
    ot.init_default()
    ot.set_threads(threads)
    psv = O.synthesize_psv(SYNTH_SEED + CONFIG_INDEX[wname], sample_b)
    batch = O.psv_to_batch(w["fs"], psv.tobytes(), with_bucket=w["arch"] == "layerstack")
    if w["arch"] != "layerstack":
        batch.pop("bucket")
    loss = O.sigmoid_loss(1.0 / 290.0) if w["arch"] == "layerstack" else O.wrm_loss(290.0, 290.0, 0.0, 0.0, 290.0)
    for _ in range(warmup):
        ot.step(batch, LR, 0.0, loss)
    t0 = time.time()
    done = 0
    for _ in range(steps):
        ot.step(batch, LR, 0.0, loss)
        done += 1
        if limit_s is not None and time.time() - t0 > limit_s:
            break
    dt = time.time() - t0
    ot.close()
    return sample_b * done / dt, done, dt / done * 1e3


def micro_lists(rng, B, A, space, lo=30, hi=38, slices=0, slice_p=None):
    """Index lists of the FT microbenchmark: per position `lo..hi` distinct indices drawn uniformly from `space` rows,
    unsorted, padded with -1 to A slots.  With `slices` > 0 every position draws its rows inside one uniformly chosen
    slice of `space` rows (king-relative feature sets: `slices` king buckets x `space` piece inputs)."""
    nnz = rng.integers(lo, hi + 1, B).astype(np.int32)
    idx = rng.integers(0, space, (B, hi), dtype=np.int64)
    for _ in range(64):   # redraw the few duplicates inside a row (38^2 / 2 / space of the rows)
        order = np.argsort(idx, axis=1, kind="stable")
        srt = np.take_along_axis(idx, order, axis=1)
        dup_sorted = np.zeros_like(srt, dtype=bool)
        dup_sorted[:, 1:] = srt[:, 1:] == srt[:, :-1]
        if not dup_sorted.any():
            break
        dup = np.zeros_like(dup_sorted)
        np.put_along_axis(dup, order, dup_sorted, axis=1)
        idx[dup] = rng.integers(0, space, int(dup.sum()))
    if slices:
        pick = rng.integers(0, slices, B) if slice_p is None else rng.choice(slices, B, p=slice_p)
        idx += pick[:, None] * space
    out = np.full((B, A), -1, np.int32)
    out[:, :hi] = idx
    out[np.arange(A)[None, :] >= nnz[:, None]] = -1
    return out, nnz


def micro_bytes(B, F, N, A, U):
    """Algorithmic bytes of the three FT kernels, one perspective: forward = the distinct table rows the batch
    touches + output + index lists + counts; backward = incoming gradient rows + lists + offsets + the gradient table;
    optimizer = w, m, v, g read and w, m, v written."""
    return {"fwd": U * F * 4.0 + B * F * 4.0 + B * A * 4.0 + B * 4.0,
            "bwd": B * F * 4.0 + B * A * 4.0 + (N + 1) * 4.0 + N * F * 4.0,
            "adam": 28.0 * N * F}


def run_microbench(tb, device, peak, iters=5):
    """FT kernels alone, F x B sweep: uniform random lists (served by the generic L2-gather kernels, since they break
    the king-slice property) and king-sliced lists (served by the slice-resident kernels of the training step)."""
    from tatara_b200 import _lib as L
    lib = tb.load_library()
    kb, pi, A = FS_DIMS["halfka-hm-merged"]
    N = kb * pi
    rng = np.random.default_rng(4)
    rows = []
    for B in MICRO_B:
        uni, nnz = micro_lists(rng, B, A, N)
        sli, nnz_s = micro_lists(rng, B, A, pi, slices=kb)
        U = int(np.unique(uni[uni >= 0]).size)
        U_s = int(np.unique(sli[sli >= 0]).size)
        for F in MICRO_F:
            r, rs = L.MicrobenchResult(), L.MicrobenchResult()
            rc = lib.tb_ft_microbench(device, uni.ctypes.data, nnz.ctypes.data, B, F, N, 0, A, iters, 1, C.byref(r))
            rc2 = lib.tb_ft_microbench(device, sli.ctypes.data, nnz_s.ctypes.data, B, F, N, pi, A, iters, 1, C.byref(rs))
            if rc != 0 or rc2 != 0:
                rows.append({"F": F, "B": B, "error": int(rc or rc2)})
                continue
            by, bys = micro_bytes(B, F, N, A, U), micro_bytes(B, F, N, A, U_s)
            gbs = lambda b, ms: round(b / (ms * 1e-3) / 1e9, 1) if ms > 0 else None
            row = {"F": F, "B": B, "distinct_rows": U,
                   "fwd_ms": round(r.fwd_ms, 4), "fwd_gbs": gbs(by["fwd"], r.fwd_ms),
                   "bwd_ms": round(r.bwd_ms, 4), "bwd_gbs": gbs(by["bwd"], r.bwd_ms),
                   "adam_ms": round(r.adam_ms, 4), "adam_gbs": gbs(by["adam"], r.adam_ms),
                   "sliced": {"distinct_rows": U_s,
                              "fwd_ms": round(rs.fwd_slice_ms, 4), "fwd_gbs": gbs(bys["fwd"], rs.fwd_slice_ms),
                              "bwd_ms": round(rs.bwd_slice_ms, 4), "bwd_gbs": gbs(bys["bwd"], rs.bwd_slice_ms)}}
            for k in ("fwd", "bwd", "adam"):
                row[k + "_frac"] = round(row[k + "_gbs"] / peak, 3) if row[k + "_gbs"] else None
            for k in ("fwd", "bwd"):
                row["sliced"][k + "_frac"] = round(row["sliced"][k + "_gbs"] / peak, 3) if row["sliced"][k + "_gbs"] else None
            rows.append(row)
    return {"protocol": "one perspective, A=40 slots with 30..38 distinct indices, N=73305 rows, fp32; %d timed launches per cell, "
                        "each after a 256 MB L2 flush, CUDA events per launch; bwd includes the inverse index" % iters,
            "kernels": {"uniform": "k_ft_forward (L2 gather), k_feat_* + k_lists_sort_* + k_ft_backward_short/long, k_radam",
                        "sliced": "item sort + k_fwd_plan/k_fwd_codes + k_ft_forward_slice; k_chunk_plan + k_inv_chunk + k_ft_backward_slice"},
            "bytes": "fwd U*F*4+B*F*4+B*A*4+B*4, bwd B*F*4+B*A*4+(N+1)*4+N*F*4, adam 28*N*F; GB/s of %.1f" % peak,
            "rows": rows}


def run_reference_gpu_kernels(iters=5):
    """The reference's own CUDA kernels (oracle/_ref, compiled unchanged) on the microbenchmark shapes, on this GPU.
    Returns None when there is no GPU or no compiled reference."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    try:
        import torch
        import ref_kernels as R
        if not (R.available() and torch.cuda.is_available()):
            return None
        ref = R.RefKernels(0)
    except Exception as e:  # no cuda-python, no driver, ...
        return {"unavailable": str(e)[:200]}
    from ref_kernels import F32, I32, U32
    kb, pi, A = FS_DIMS["halfka-hm-merged"]
    N = kb * pi
    rng = np.random.default_rng(4)
    rows = []
    flush = torch.empty(64 << 20, dtype=torch.float32, device="cuda")

    def timed(fn):
        total = 0.0
        for i in range(-1, iters):
            flush.fill_(1.0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); e1.synchronize()
            if i >= 0:
                total += e0.elapsed_time(e1)
        return total / iters

    for B in MICRO_B[:3]:          # the reference's 32-bit index arithmetic ends at B * F < 2^32
        uni, nnz = micro_lists(rng, B, A, N)
        d_idx, d_nnz = torch.from_numpy(uni).cuda(), torch.from_numpy(nnz).cuda()
        for F in MICRO_F:
            table = torch.rand(N * F, device="cuda") * 0.05
            out = torch.empty(B * F, device="cuda")
            grad = torch.empty(N * F, device="cuda")
            m, v = torch.zeros(N * F, device="cuda"), torch.zeros(N * F, device="cuda")
            fwd = timed(lambda: ref.sparse_ft_forward(table, d_idx, d_nnz, out, B, F, N, A))
            bwd = timed(lambda: ref.ft_backward([out], [d_idx], d_nnz, B, A, N, F, grad))
            adam = timed(lambda: ref.launch_1d("radam_step", N * F, table, m, v, grad, F32(1e-3), F32(1.0), I32(1), F32(0.01), F32(0.9),
                                               F32(0.999), F32(1e-8), F32(-258.0), F32(258.0), U32(N * F)))
            rows.append({"F": F, "B": B, "fwd_ms": round(fwd, 4), "bwd_ms": round(bwd, 4), "adam_ms": round(adam, 4)})
            del table, out, grad, m, v
    return {"what": "sparse_ft_forward; build_feature_counts + 3 scans + scatter_positions + gather_and_sum_per_feature_overwrite; "
                    "radam_step -- the reference's kernels with its launch shapes, same lists and timing protocol as ft_microbench "
                    "(torch allocations inside the backward's timed region, as the reference allocates nothing there, favour us slightly)",
            "rows": rows}


# ---------------------------------------------------------------------------------------------- data-parallel self check
def dp_parity_check(tb, dist, device, world, rank, nccl_id, dp_exchange):
    """Before the timed region at N > 1: six pipelined data-parallel steps on a small LayerStack shape against the CPU
    oracle stepping on the concatenated batch (the check of tests/dp_worker.py), then bitwise equality of the replicas."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    F, L1, L2, NB, B = 256, 16, 32, 9, 256
    fs = tb.FEATURE_SETS["halfka-hm-merged"]
    init = tb.layerstack_default_init(fs, F, L1, L2, NB)
    init["ft_w"][:fs.ft_in * F] *= 30.0
    shards = [O.psv_to_batch(fs.name, O.synthesize_psv(SYNTH_SEED + 7919 * r, B).tobytes()) for r in range(world)]
    mine = shards[rank]
    tr = tb.GpuTrainer(B, F, L1, L2, NB, fs, optimizer="ranger", init=init, device=device, world_size=world, rank=rank, nccl_id=nccl_id,
                       dp_exchange=dp_exchange)
    batch = tb.BatchData(mine["stm"], mine["nstm"], mine["nnz"], mine["score"], mine["wdl"], mine["bucket"])
    if os.environ.get("TB_BENCH_TRACE"):
        print("[dp check rank %d] trainer created" % rank, file=sys.stderr, flush=True)
    for _ in range(6):
        tr.train_step(batch, 1e-3, 0.0, tb.LossKind.sigmoid())
    loss = tr.flush_pending_loss()
    if os.environ.get("TB_BENCH_TRACE"):
        print("[dp check rank %d] six steps done" % rank, file=sys.stderr, flush=True)
    ok = True
    if rank == 0:
        full = {k: np.concatenate([s[k] for s in shards]) for k in mine}
        ref = O.OracleTrainer(arch="layerstack", ft_in=fs.ft_in, piece_inputs=fs.piece_inputs, factorize=True, max_active=fs.max_active,
                              ft_out=F, l1=L1, l2=L2, num_buckets=NB, optimizer="ranger", capacity=world * B)
        ref.set_threads(os.cpu_count() or 1)
        for n in ref.names:
            ref.group(n)[:] = init[n]
        for _ in range(6):
            ref_loss = ref.step(full, 1e-3, 0.0, O.sigmoid_loss())
        ok = abs(loss - ref_loss) <= 1e-4 * (1 + abs(ref_loss))
        for n in ref.names:
            got, want = tr.download_group(n)["w"], ref.group(n)
            ok = ok and bool(np.all(np.abs(got - want) <= 1e-4 * (1 + np.abs(want))))
    same = replicas_identical(tr, dist, ("ft_w", "l1_w", "l2_w"))
    tr.close()
    t = torch.tensor([1 if ok else 0], dtype=torch.int32)
    dist.broadcast(t, src=0)
    return bool(t[0]), same


def replicas_identical(tr, dist, names):
    """Every rank's weights equal rank 0's, bit for bit."""
    import torch
    same = True
    for n in names:
        w = torch.from_numpy(tr.download_group(n)["w"].view(np.int32).copy())
        w0 = w.clone()
        dist.broadcast(w0, src=0)
        same = same and bool(torch.equal(w, w0))
    t = torch.tensor([1 if same else 0], dtype=torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t[0])


def skewed_run(tb, w, device, steps, uniform_ms, prec):
    """The headline workload on king-skewed batches: every position's rows lie in one king-bucket slice per perspective, the
    slice drawn from a Zipf law (p_k ~ 1 / k^1.2: the most frequent king bucket holds about 30 % of the items), as real
    game positions crowd a few king squares.  Reports the step time beside the uniform generator's."""
    kb, pi, A = FS_DIMS[w["fs"]]
    rng = np.random.default_rng(12)
    p = 1.0 / np.arange(1, kb + 1) ** 1.2
    p /= p.sum()
    tr, loss, fs = make_trainer(tb, w, device, 1, 0, None, precision=prec)
    batches = []
    for i in range(2):
        stm, nnz = micro_lists(rng, BATCH, A, pi, lo=A - 2, hi=A - 2, slices=kb, slice_p=p)
        nstm, _ = micro_lists(rng, BATCH, A, pi, lo=A - 2, hi=A - 2, slices=kb, slice_p=p)
        batches.append(tb.BatchData(stm, nstm, nnz, np.clip(np.round(rng.normal(0, 400, BATCH)), -3000, 3000).astype(np.float32),
                                    rng.choice(np.array([0.0, 0.5, 1.0], np.float32), BATCH),
                                    rng.integers(0, 9, BATCH).astype(np.int32) if w["arch"] == "layerstack" else None))
    for i, b in enumerate(batches):
        tr.stage_batch(i, b)
    for i in range(3):
        tr.train_step_staged(i % 2, LR, 0.0, loss)
    tr.synchronize()
    tr.timer_start()
    for i in range(steps):
        tr.train_step_staged(i % 2, LR, 0.0, loss)
    ms = tr.timer_stop() / steps
    tr.profile_enable(True)
    tr.profile_reset()
    for i in range(4):
        tr.train_step_staged(i % 2, LR, 0.0, loss)
    prof = {k: round(v[0] / 4, 4) for k, v in tr.profile_read().items() if v[1] > 0 and k in ("ft_forward", "ft_backward", "inverse_index")}
    tr.close()
    return {"generator": "king bucket of each perspective ~ Zipf(1.2) over %d slices (top slice %.0f %% of the items)" % (kb, 100 * p[0]),
            "ms_per_step": round(ms, 4), "uniform_ms_per_step": round(uniform_ms, 4), "slowdown": round(ms / uniform_ms, 4),
            "kernels_ms": prof}


def short_config(tb, wname, device, steps, peak):
    """pos/s and step-level roofline fraction of another single-GPU configuration (a parity-test case, not the headline)."""
    w = WORKLOADS[wname]
    tr, loss, fs = make_trainer(tb, w, device, 1, 0, None)
    batches = [tb.synthetic_batch(SYNTH_SEED + CONFIG_INDEX[wname] + 104729 * i, BATCH, fs, with_bucket=w["arch"] == "layerstack", device=device)
               for i in range(2)]
    for i, b in enumerate(batches):
        tr.stage_batch(i, b)
    for i in range(3):
        tr.train_step_staged(i % 2, LR, 0.0, loss)
    tr.synchronize()
    tr.timer_start()
    for i in range(steps):
        tr.train_step_staged(i % 2, LR, 0.0, loss)
    ms = tr.timer_stop() / steps
    tr.close()
    alg = algorithmic_bytes(w, BATCH)["step"]
    return {"workload": w["name"], "ms_per_step": round(ms, 4), "value": BATCH / (ms * 1e-3), "unit": "pos/s",
            "roofline_step_frac": round(alg / (ms * 1e-3) / 1e9 / peak, 4)}


T0 = time.time()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--precision", default="fp32", choices=["fp32", "all-optim"],
                    help="all-optim: --tf32 --ft-fp16 --ft-fp16-out --fp16-opt-state of the reference's CLI")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-microbench", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true")
    ap.add_argument("--trace", action="store_true", help="progress lines on stderr")
    ap.add_argument("--dp-exchange", default="auto", choices=["auto", "nccl", "peer-copy", "peer-kernel"],
                    help="how the gradient parts are summed over the ranks: ncclAllReduce, copy engines over peer mappings, or a "
                         "kernel over peer mappings; auto = what measured fastest: peer-copy on two GPUs, nccl on more")
    ap.add_argument("--nccl-ctas", type=int, default=0, help="fixed CTA (channel) count of the library's communicator; 0: NCCL chooses")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = WORKLOADS[args.workload]
    K, Wm = max(1, args.steps), max(3, args.warmup)
    threads = os.cpu_count() or 1

    def trace(msg):
        if args.trace:
            print("[bench rank %d %.1fs] %s" % (rank, time.time() - T0, msg), file=sys.stderr, flush=True)

    if args.impl == "reference":
        if rank != 0:
            return
        # the benchmark's own configuration (65 536 positions per step) for as many of the K steps as fit in the time
        # limit, then a small-sample figure
        value, done, ms = run_cpu(w, args.workload, threads, args.batch, K, 1, limit_s=150.0)
        v_small, done_small, ms_small = run_cpu(w, args.workload, threads, 4096, 3, 1, limit_s=20.0)
        line = {"impl": "reference", "metric": "train_positions_per_second", "value": value, "unit": "pos/s", "n_gpus": 0,
                "steps": done, "warmup": 1, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": w["name"], "positions_per_step": args.batch, "same_config": args.batch == BATCH,
                           "note": "CPU restatement of the reference step (oracle/), OpenMP; the Rust reference cannot be built without cargo"},
                "cpu_baseline": {"value": value, "unit": "pos/s", "cores": threads, "kind": "port",
                                 "sample": "%d steps of %d synthetic positions (the benchmark's step); 4096-position steps run at %.0f pos/s "
                                           "(%.0f ms/step: the optimizer and factorizer passes do not shrink with the batch)"
                                           % (done, args.batch, v_small, ms_small)},
                "e2e": {"value": value, "unit": "pos/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        ref_gpu = run_reference_gpu_kernels()
        if ref_gpu is not None:
            line["reference_gpu_kernels"] = ref_gpu
        print(json.dumps(line), flush=True)
        return

    import tatara_b200 as tb
    dist = None
    nccl_id = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # This application's NCCL settings (the library sets none): one algorithm and protocol, so that the order in which
        # the gradient sum is formed is fixed; NVLS off because the all-reduce runs next to a kernel that holds every SM.
        for k, v in NCCL_ENV.items():
            os.environ.setdefault(k, v)
        dist.init_process_group(backend="gloo", rank=rank, world_size=world)
        ids = [tb.nccl_unique_id() if rank == 0 else None for _ in range(3)]
        dist.broadcast_object_list(ids, src=0)
        nccl_id = ids[0]
        if args.dp_exchange == "auto":
            # two B200s: peer-copy 4.69 ms per step, nccl 4.82; four: 4.98 / 5.00 / peer-kernel 5.17 (fp32, config 3)
            args.dp_exchange = "peer-copy" if world == 2 else "nccl"
        if args.dp_exchange != "nccl":
            # The peer exchange needs CUDA IPC between the ranks' processes.  Its set-up fails on every rank together when one
            # rank cannot map a peer's memory; the benchmark then runs on NCCL all-reduces and says so in config.dp_exchange.
            fs0 = tb.FEATURE_SETS["halfka-hm-merged"]
            try:
                probe = tb.GpuTrainer(256, 256, 16, 32, 9, fs0, optimizer="ranger", device=local_rank, world_size=world, rank=rank,
                                      nccl_id=ids[2], dp_exchange=args.dp_exchange)
                dist.barrier()
                probe.close()
                dist.barrier()
            except tb.TrainerError as e:
                trace("peer exchange unavailable (%s): falling back to NCCL" % e)
                args.dp_exchange = "nccl"
    device = local_rank
    B = args.batch
    dp_ok = dp_same_small = None
    trace("rendezvous done")
    if world > 1:
        dp_ok, dp_same_small = dp_parity_check(tb, dist, device, world, rank, ids[1], args.dp_exchange)
        trace("dp self check done: %s %s" % (dp_ok, dp_same_small))
        if not (dp_ok and dp_same_small):
            if rank == 0:
                print(json.dumps({"error": "data-parallel self check failed", "dp_parity": dp_ok, "replicas_identical": dp_same_small}), flush=True)
            sys.exit(1)
    all_optim = args.precision == "all-optim"
    prec = tb.PrecisionFlags(tf32=True, ft_fp16=True, ft_fp16_out=True, fp16_opt_state=True) if all_optim else None
    tr, loss, fs = make_trainer(tb, w, device, world, rank, nccl_id, capacity=B, precision=prec, nccl_ctas=args.nccl_ctas, dp_exchange=args.dp_exchange)
    n_batches = 3
    seed0 = SYNTH_SEED + CONFIG_INDEX[args.workload] + 7919 * rank
    psvs = [tb.synthesize_psv(seed0 + 104729 * i, B) for i in range(n_batches)]
    batches = [tb.extract_batch(p, fs, with_bucket=w["arch"] == "layerstack", device=device, pinned=True) for p in psvs]
    for i, b in enumerate(batches):
        tr.stage_batch(i, b)
    trace("trainer and batches ready")

    def barrier():
        tr.synchronize()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---- device-resident throughput: `repeats` timed regions of exactly K steps each ---------------------------------
    for i in range(Wm):
        tr.train_step_staged(i % n_batches, LR, 0.0, loss)
    barrier()
    sampler = ClockSampler(device)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    launches0 = tr.launch_count
    rep_ms = []
    t_wall0 = time.time()
    for r in range(max(1, args.repeats)):
        barrier()
        tr.timer_start()
        for i in range(K):
            tr.train_step_staged(i % n_batches, LR, 0.0, loss)
        m = tr.timer_stop()
        tr.synchronize()
        rep_ms.append(max_over_ranks(m))
    t_wall1 = time.time()
    trace("timed repeats done: %s" % rep_ms)
    launches = (tr.launch_count - launches0) // max(1, args.repeats)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    barrier()
    ms = float(np.median(rep_ms))
    last_loss = tr.flush_pending_loss()
    value = world * B * K / (ms * 1e-3)

    # ---- end to end: page-locked host batches through tb_train_step ------------------------------------------
    def e2e_run(step_fn):
        for i in range(3):
            step_fn(i)
        barrier()
        tr.timer_start()
        acc = 0.0
        for i in range(K):
            acc += step_fn(i)   # the returned loss is a device->host read
        m = tr.timer_stop()
        tr.synchronize()
        barrier()
        tr.flush_pending_loss()
        return max_over_ranks(m)

    ms_e2e = e2e_run(lambda i: tr.train_step(batches[i % n_batches], LR, 0.0, loss))
    trace("e2e (index feed) done")
    e2e_value = world * B * K / (ms_e2e * 1e-3)
    A = fs.max_active
    h2d = 2 * B * A * 4 + (4 if w["arch"] == "layerstack" else 3) * B * 4
    # the same fed with 40-byte records: decode and feature extraction on the device, on the copy stream
    pinned_psv = []
    for p in psvs:
        pa = tb.PinnedArray(p.shape, np.uint8)
        pa.array[:] = p
        pinned_psv.append(pa)
    ms_psv = e2e_run(lambda i: tr.train_step_psv(pinned_psv[i % n_batches].array, LR, 0.0, loss))
    trace("e2e (record feed) done")

    # ---- per-kernel timing (CUDA events around every phase, on the launching stream) -----------------------------
    tr.profile_enable(True)
    tr.profile_reset()
    n_prof = min(K, 10)
    for i in range(n_prof):
        tr.train_step_staged(i % n_batches, LR, 0.0, loss)
    prof = tr.profile_read()
    tr.profile_enable(False)
    barrier()
    trace("per-phase profile done")
    same = replicas_identical(tr, dist, ("ft_w", "l1_w")) if dist is not None else None
    trace("replica comparison done")
    if dist is not None and not same:
        if rank == 0:
            print(json.dumps({"error": "replicas diverged during the timed steps"}), flush=True)
        sys.exit(1)

    if rank == 0:
        peak, peak_kind = peak_hbm()
        alg = algorithmic_bytes(w, B, all_optim)
        phases = {k: v[0] / n_prof for k, v in prof.items() if v[1] > 0}
        dominant = max((k for k in phases if k in alg), key=lambda k: phases[k])
        ach = alg[dominant] / (phases[dominant] * 1e-3) / 1e9
        step_ach = alg["step"] / (ms / K * 1e-3) / 1e9
        lookup = 2.0 * B * fs.max_active * w["F"] * (2.0 if all_optim else 4.0)   # row bytes each slice-resident FT kernel reads from shared memory
        smem_peak = None
        if clocks and clocks.get("sm_mhz"):
            smem_peak = 148 * SMEM_BYTES_PER_CLK_PER_SM * clocks["sm_mhz"] * 1e6 / 1e9     # GB/s at the sampled clock
        smem = {}
        for k in ("ft_forward", "ft_backward"):
            if k in phases and smem_peak:
                a = lookup / (phases[k] * 1e-3) / 1e9
                smem[k] = {"achieved": a, "peak": smem_peak, "unit": "GB/s", "frac": a / smem_peak}
        exact_case = args.workload == "cfg3" and B == BATCH and world == 1 and not all_optim
        line = {
            "metric": "train_positions_per_second", "value": value, "unit": "pos/s", "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16/tf32" if all_optim else "f32", "data": "synthetic",
            "config": {"workload": w["name"].replace("fp32", "all-optim (fp16 FT table/activations/moments, tf32 L1)") if all_optim else w["name"],
                       "positions_per_step_per_gpu": B, "global_batch": B * world,
                       "parallelism": "dp%d" % world, "l2": "inputs larger than L2 (tables and activations >> 126 MB), 3 rotating batches",
                       "loss_per_position": last_loss / (B * world)},
            "repeats": {"n": len(rep_ms), "steps_each": K, "ms_per_step_median": ms / K, "ms_per_step_min": min(rep_ms) / K,
                        "ms_per_step_max": max(rep_ms) / K},
            "e2e": {"value": e2e_value, "unit": "pos/s", "ms_per_step": ms_e2e / K, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8,
                    "feed": "extracted index arrays, the reference's BatchData"},
            "e2e_psv": {"value": world * B * K / (ms_psv * 1e-3), "unit": "pos/s", "ms_per_step": ms_psv / K, "h2d_bytes_per_step": 40 * B,
                        "d2h_bytes_per_step": 8, "feed": "40-byte PackedSfenValue records, decode + extraction on the device"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": dominant, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "peak_kind": peak_kind,
                         # from one ncu capture of exactly this case (cfg3, B = 65 536, one GPU); null for any other case
                         "traffic": NCU_TRAFFIC_BYTES.get((args.workload, dominant)) if exact_case else None,
                         "algorithmic_bytes": alg[dominant], "kernel_ms": phases[dominant],
                         # the bound that binds the two slice-resident FT kernels: their row reads (what a cache-less gather
                         # would move through HBM) come from shared memory at 128 B/clk/SM
                         "lookup_bytes": lookup, "smem": smem or None,
                         "step": {"algorithmic_bytes": alg["step"], "achieved": step_ach, "frac": step_ach / peak}},
            "kernels_ms": {k: round(v, 4) for k, v in phases.items()},
        }
        if world > 1:
            line["config"]["dp_exchange"] = args.dp_exchange
            line["config"]["nccl"] = dict({k: os.environ.get(k) for k in NCCL_ENV}, ctas=args.nccl_ctas or "NCCL's choice")
            line["dp_parity"] = "ok" if dp_ok else "failed"
            line["replicas_identical"] = bool(same and dp_same_small)
        if world == 1:
            tr.close()   # (with several ranks the communicator is torn down by all of them together, below)
            if not args.no_other_configs:
                line["other_configs"] = [short_config(tb, n, device, 10, peak) for n in ("cfg1", "cfg2") if n != args.workload]
            if not args.no_other_configs:
                line["skewed"] = skewed_run(tb, w, device, 10, ms / K, prec)
            if not args.no_microbench:
                line["ft_microbench"] = run_microbench(tb, device, peak)
            if not args.no_cpu_baseline:
                v, done, cms = run_cpu(w, args.workload, threads, 4096, 3, 1, limit_s=25.0)
                line["cpu_baseline"] = {"value": v, "unit": "pos/s", "cores": threads, "kind": "port",
                                        "sample": "%d steps of 4096 synthetic positions on the CPU restatement of the reference step (%.0f ms/step)" % (done, cms)}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        tr.close()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
