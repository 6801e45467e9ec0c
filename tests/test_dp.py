"""Data-parallel path: world_size-2 gloo ranks on CPU (host logic + oracle), NCCL ranks on GPUs."""
import json
import os
import socket
import subprocess
import sys

import pytest

import tatara_b200 as tb
from helpers import ROOT

WORKER = os.path.join(ROOT, "tests", "dp_worker.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(n, args, timeout=900, script=WORKER, extra_env=None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), script] + args
    env = dict(os.environ, OMP_NUM_THREADS="2", NCCL_NVLS_ENABLE="0")
    env.update(extra_env or {})
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


def test_dp_semantics_two_gloo_ranks_on_cpu():
    r = _torchrun(2, ["cpu"])
    assert r.returncode == 0 and "DP_WORKER_OK cpu 2" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_reference_arm_runs_on_rank0_only():
    r = _torchrun(2, ["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1", "--workload", "cfg1"],
                  script=os.path.join(ROOT, "bench.py"))
    assert r.returncode == 0, r.stderr[-3000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    j = json.loads(lines[0])
    assert j["impl"] == "reference" and j["unit"] == "pos/s" and j["value"] > 0
    assert j["cpu_baseline"]["kind"] == "port" and j["e2e"]["h2d_bytes_per_step"] == 0


@pytest.mark.gpu
def test_dp_two_gpus_nccl():
    if tb.load_library().tb_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = _torchrun(2, ["gpu"])
    assert r.returncode == 0 and "DP_WORKER_OK gpu 2" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.gpu
def test_dp_two_gpus_peer_copy():
    # the same six steps, run-to-run and replica checks with the gradient parts summed by copy engines over peer mappings
    if tb.load_library().tb_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = _torchrun(2, ["gpu-peer"])
    assert r.returncode == 0 and "DP_WORKER_OK gpu-peer 2" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
    # at the benchmark's FT width the weight gradient runs in whole waves with a one-wave last part
    r = _torchrun(2, ["gpu-peer"], extra_env={"DP_WORKER_F": "1536", "OMP_NUM_THREADS": "8"})
    assert r.returncode == 0 and "DP_WORKER_OK gpu-peer 2" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.gpu
def test_dp_two_gpus_peer_kernel():
    # the same checks with the parts summed by one kernel per part over the peer mappings
    if tb.load_library().tb_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = _torchrun(2, ["gpu-peer-kernel"])
    assert r.returncode == 0 and "DP_WORKER_OK gpu-peer-kernel 2" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
