"""Benchmark of the NNUE training step (positions/s) on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg3|cfg2|cfg1]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

A step is one full training step (forward, loss, backward, gradient all-reduce when N > 1, optimizer) of
the workload on one batch of 65 536 synthetic positions per GPU (weak scaling).  `value` runs on batches
already resident in HBM; `e2e` passes page-locked HOST batches through tb_train_step every step (copies
inside the timed region, the lagged loss read back every step).  Prints one JSON line on rank 0.

`--impl reference` times the CPU restatement of the reference's step (oracle/, OpenMP over all host
cores) on a bounded sample of the same workload.  The reference itself is Rust and cannot be built on a
box without cargo, so the oracle port is the CPU arm.
"""
from __future__ import annotations

import argparse
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
WORKLOADS = {
    # BASELINE.json configs[3] / [2] / [1]
    "cfg3": dict(arch="layerstack", fs="halfka-hm-merged", F=1536, l1=16, l2=32, nb=9, optimizer="ranger",
                 name="LayerStack ft1536 l1=16 l2=32 halfka-hm-merged kingrank9 fp32 ranger factorizer-on"),
    "cfg2": dict(arch="layerstack", fs="halfka-hm-merged", F=768, l1=8, l2=32, nb=9, optimizer="ranger",
                 name="LayerStack ft768 l1=8 l2=32 halfka-hm-merged kingrank9 fp32 ranger factorizer-on"),
    "cfg1": dict(arch="simple", fs="halfkp", F=256, l1=32, l2=32, nb=0, optimizer="adamw",
                 name="Simple halfkp 256x2-32-32 crelu fp32 adamw wrm(290) factorizer-on"),
}
CONFIG_INDEX = {"cfg1": 1, "cfg2": 2, "cfg3": 3}
# measured peak (MEASURED_PEAKS.json: STREAM-style copy on this pool's B200s); fallback = the pool's earlier figure
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under profiles/
# (bytes at the benchmark's full size; None = not captured yet)
NCU_TRAFFIC_BYTES = {
    # profiles/step_cfg3_launch_list.md: full-size launches of the dominant kernel of each phase (the metrics take one pass)
    ("cfg3", "ft_backward"): 1635.0e6, ("cfg3", "ft_forward"): 1750.2e6, ("cfg3", "opt_ft"): 4232.5e6,
    ("cfg3", "l1_dgrad_ftgrad"): 1583.3e6, ("cfg3", "l1_forward"): 404.8e6, ("cfg3", "l1_wgrad"): 411.2e6,
}


def peak_hbm():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def algorithmic_bytes(w, n_pos):
    """Algorithmic bytes per launch of each kernel phase: every large tensor crosses HBM once per producer and
    once per consumer; index arrays, [B, <=32] tensors and the small parameter groups are left out."""
    import tatara_b200 as tb
    fs = tb.FEATURE_SETS[w["fs"]]
    F = w["F"]
    W = fs.ft_in * F * 4.0
    Wt = fs.train_ft_in * F * 4.0
    X = n_pos * F * 4.0
    comb = X if w["arch"] == "layerstack" else 2 * X      # the L1 input [B, F] or [B, 2F]
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
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
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


def make_trainer(tb, w, device, world, rank, nccl_id, capacity=BATCH):
    fs = tb.FEATURE_SETS[w["fs"]]
    if w["arch"] == "layerstack":
        tr = tb.GpuTrainer(capacity, w["F"], w["l1"], w["l2"], w["nb"], fs, optimizer=w["optimizer"], device=device,
                           world_size=world, rank=rank, nccl_id=nccl_id)
        loss = tb.LossKind.sigmoid(1.0 / 290.0)
    else:
        tr = tb.SimpleGpuTrainer(capacity, w["F"], w["l1"], w["l2"], fs, optimizer=w["optimizer"], weight_decay=0.0,
                                 device=device, world_size=world, rank=rank, nccl_id=nccl_id)
        loss = tb.LossKind.wrm(nnue2score=290.0, in_scaling=290.0, in_offset=0.0, target_offset=0.0, target_scaling=290.0)
    return tr, loss, fs


def run_cpu(w, wname, threads, sample_b, steps, warmup, limit_s=None):
    """Times the oracle's whole step on `sample_b` synthetic positions; returns (pos/s, steps done, ms/step)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    import tatara_b200 as tb
    fs = tb.FEATURE_SETS[w["fs"]]
    ot = O.OracleTrainer(arch=w["arch"], ft_in=fs.ft_in, piece_inputs=fs.piece_inputs, factorize=True,
                         max_active=fs.max_active, ft_out=w["F"], l1=w["l1"], l2=w["l2"], num_buckets=max(w["nb"], 1),
                         optimizer=w["optimizer"], wd=(0.01, 0.01, 0.01) if w["arch"] == "layerstack" else (0.0, 0.0, 0.0),
                         capacity=sample_b)
    ot.init_default()
    ot.set_threads(threads)
    psv = tb.synthesize_psv(tb.SYNTH_SEED + CONFIG_INDEX[wname], sample_b)
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
    return sample_b * done / dt, done, dt / done * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = WORKLOADS[args.workload]
    K, Wm = max(1, args.steps), max(3, args.warmup)
    threads = os.cpu_count() or 1

    if args.impl == "reference":
        if rank != 0:
            return
        sample_b = 4096
        value, done, ms = run_cpu(w, args.workload, threads, sample_b, K, min(Wm, 1), limit_s=150.0)
        line = {"impl": "reference", "metric": "train_positions_per_second", "value": value, "unit": "pos/s", "n_gpus": 0,
                "steps": done, "warmup": min(Wm, 1), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": w["name"], "positions_per_step": sample_b,
                           "note": "CPU restatement of the reference step (oracle/), OpenMP; the Rust reference cannot be built without cargo"},
                "cpu_baseline": {"value": value, "unit": "pos/s", "cores": threads, "kind": "port",
                                 "sample": "%d steps of %d synthetic positions (the optimizer and factorizer passes do not shrink with the sample)" % (done, sample_b)},
                "e2e": {"value": value, "unit": "pos/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    import tatara_b200 as tb
    dist = None
    nccl_id = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend="gloo", rank=rank, world_size=world)
        ids = [tb.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        nccl_id = ids[0]
    device = local_rank
    B = args.batch
    tr, loss, fs = make_trainer(tb, w, device, world, rank, nccl_id, capacity=B)
    n_batches = 3
    seed0 = tb.SYNTH_SEED + CONFIG_INDEX[args.workload] + 7919 * rank
    batches = [tb.synthetic_batch(seed0 + 104729 * i, B, fs, with_bucket=w["arch"] == "layerstack", device=device, pinned=True)
               for i in range(n_batches)]
    for i, b in enumerate(batches):
        tr.stage_batch(i, b)

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

    # ---- device-resident throughput ---------------------------------------------------------------------------
    for i in range(Wm):
        tr.train_step_staged(i % n_batches, LR, 0.0, loss)
    barrier()
    sampler = ClockSampler(device)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    launches0 = tr.launch_count
    barrier()
    t_wall0 = time.time()
    tr.timer_start()
    for i in range(K):
        tr.train_step_staged(i % n_batches, LR, 0.0, loss)
    ms = tr.timer_stop()
    tr.synchronize()
    t_wall1 = time.time()
    launches = tr.launch_count - launches0
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    barrier()
    ms = max_over_ranks(ms)
    last_loss = tr.flush_pending_loss()
    value = world * B * K / (ms * 1e-3)

    # ---- end to end: page-locked host batches through tb_train_step ------------------------------------------
    for i in range(3):
        tr.train_step(batches[i % n_batches], LR, 0.0, loss)
    barrier()
    tr.timer_start()
    acc = 0.0
    for i in range(K):
        acc += tr.train_step(batches[i % n_batches], LR, 0.0, loss)   # the returned loss is a device->host read
    ms_e2e = tr.timer_stop()
    tr.synchronize()
    barrier()
    ms_e2e = max_over_ranks(ms_e2e)
    tr.flush_pending_loss()
    e2e_value = world * B * K / (ms_e2e * 1e-3)
    A = fs.max_active
    h2d = 2 * B * A * 4 + (4 if w["arch"] == "layerstack" else 3) * B * 4

    # ---- per-kernel timing (CUDA events around every phase, on the launching stream) -----------------------------
    tr.profile_enable(True)
    tr.profile_reset()
    n_prof = min(K, 10)
    for i in range(n_prof):
        tr.train_step_staged(i % n_batches, LR, 0.0, loss)
    prof = tr.profile_read()
    tr.profile_enable(False)
    barrier()

    if rank == 0:
        peak, peak_kind = peak_hbm()
        alg = algorithmic_bytes(w, B)
        phases = {k: v[0] / n_prof for k, v in prof.items() if v[1] > 0}
        dominant = max((k for k in phases if k in alg), key=lambda k: phases[k])
        ach = alg[dominant] / (phases[dominant] * 1e-3) / 1e9
        step_ach = alg["step"] / (ms / K * 1e-3) / 1e9
        line = {
            "metric": "train_positions_per_second", "value": value, "unit": "pos/s", "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": w["name"], "positions_per_step_per_gpu": B, "global_batch": B * world,
                       "parallelism": "dp%d" % world, "l2": "inputs larger than L2 (tables and activations >> 126 MB), 3 rotating batches",
                       "loss_per_position": last_loss / (B * world)},
            "e2e": {"value": e2e_value, "unit": "pos/s", "ms_per_step": ms_e2e / K, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": dominant, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "peak_kind": peak_kind, "traffic": NCU_TRAFFIC_BYTES.get((args.workload, dominant)),
                         "algorithmic_bytes": alg[dominant], "kernel_ms": phases[dominant],
                         # not graded: what a cache-less gather would move; the slice-resident FT kernels serve these
                         # bytes from shared memory
                         "lookup_bytes": 2.0 * B * fs.max_active * w["F"] * 4.0 if dominant in ("ft_forward", "ft_backward") else None,
                         "step": {"algorithmic_bytes": alg["step"], "achieved": step_ach, "frac": step_ach / peak}},
            "kernels_ms": {k: round(v, 4) for k, v in phases.items()},
        }
        if world == 1 and not args.no_cpu_baseline:
            tr.close()
            v, done, cms = run_cpu(w, args.workload, threads, 4096, 3, 1, limit_s=25.0)
            line["cpu_baseline"] = {"value": v, "unit": "pos/s", "cores": threads, "kind": "port",
                                    "sample": "%d steps of 4096 synthetic positions on the CPU restatement of the reference step (%.0f ms/step)" % (done, cms)}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
