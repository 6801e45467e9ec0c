"""Worker of the data-parallel tests: run as `python -m torch.distributed.run --nproc-per-node N tests/dp_worker.py MODE`.

MODE cpu : the host-side logic on the CPU oracle over gloo (no GPU): shard seeds per rank, gradient sum,
           identical optimizer step, loss sum — compared with one rank stepping on the concatenated batch.
MODE gpu : the same through the CUDA library and its NCCL all-reduce, one rank per GPU.
MODE gpu-peer : the same with the gradient parts summed by the copy engines over peer mappings (dp_exchange "peer-copy").
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import oracle_lib as O  # noqa: E402
import tatara_b200 as tb  # noqa: E402
from helpers import assert_close, assert_close_scaled  # noqa: E402

# DP_WORKER_F = 1536: the weight gradient is then cut into whole waves of blocks as at the benchmark size
F, L1, L2, NB, B = int(os.environ.get("DP_WORKER_F", "256")), 16, 32, 9, 256
LR = 1e-3


def oracle(fs, cap):
    ot = O.OracleTrainer(arch="layerstack", ft_in=fs.ft_in, piece_inputs=fs.piece_inputs, factorize=True,
                         max_active=fs.max_active, ft_out=F, l1=L1, l2=L2, num_buckets=NB, optimizer="ranger", capacity=cap)
    return ot


def shard(rank, fs):
    psv = tb.synthesize_psv(tb.SYNTH_SEED + 7919 * rank, B)
    return O.psv_to_batch(fs.name, psv.tobytes())


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    for k, v in (("NCCL_NVLS_ENABLE", "0"), ("NCCL_ALGO", "Ring"), ("NCCL_PROTO", "Simple")):   # a fixed summation order
        os.environ.setdefault(k, v)
    dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    fs = tb.FEATURE_SETS["halfka-hm-merged"]
    init = tb.layerstack_default_init(fs, F, L1, L2, NB)
    init["ft_w"][:fs.ft_in * F] *= 30.0
    mine = shard(rank, fs)
    # single-process answer: one oracle stepping on the concatenation of every rank's shard
    full = {k: np.concatenate([shard(r, fs)[k] for r in range(world)]) for k in mine}
    ref = oracle(fs, world * B)
    for n in ref.names:
        ref.group(n)[:] = init[n]
    ref_loss = ref.step(full, LR, 0.0, O.sigmoid_loss(), do_optimizer=False)
    ref_grads = {n: ref.group(n, "grad").copy() for n in ref.names}
    ref.apply_optimizer(LR)

    if mode == "cpu":
        ot = oracle(fs, B)
        for n in ot.names:
            ot.group(n)[:] = init[n]
        loss = ot.step(mine, LR, 0.0, O.sigmoid_loss(), per_pos_norm=1.0 / (world * B), do_optimizer=False)
        t = torch.tensor([loss], dtype=torch.float64)
        dist.all_reduce(t)
        for n in ot.names:
            g = torch.from_numpy(ot.group(n, "grad"))
            dist.all_reduce(g)          # in place on the oracle's gradient buffer
        assert abs(float(t[0]) - ref_loss) <= 1e-9 * (1 + abs(ref_loss))
        for n in ot.names:
            assert_close_scaled(ot.group(n, "grad"), ref_grads[n], 1e-5, "summed grad " + n)
        ot.apply_optimizer(LR)
        for n in ot.names:
            assert_close(ot.group(n), ref.group(n), 1e-6, "weights " + n)
            w = torch.from_numpy(ot.group(n).copy())
            w0 = w.clone()
            dist.broadcast(w0, src=0)
            assert torch.equal(w, w0), "replicas diverged in " + n
    else:
        exchange = {"gpu-peer": "peer-copy", "gpu-peer-kernel": "peer-kernel"}.get(mode, "nccl")
        ids = [tb.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        # communicators with a fixed channel count (ncclCommInitRankConfig); the benchmark covers ncclCommInitRank
        tr = tb.GpuTrainer(B, F, L1, L2, NB, fs, optimizer="ranger", init=init, device=int(os.environ["LOCAL_RANK"]),
                           world_size=world, rank=rank, nccl_id=ids[0], nccl_ctas=8, dp_exchange=exchange)
        batch = tb.BatchData(mine["stm"], mine["nstm"], mine["nnz"], mine["score"], mine["wdl"], mine["bucket"])
        loss = tr.forward_backward(batch, 0.0, tb.LossKind.sigmoid())
        assert abs(loss - ref_loss) <= 1e-5 * (1 + abs(ref_loss)), (loss, ref_loss)    # the all-reduced loss
        for n in ref.names:
            assert_close_scaled(tr.download_grad(n), ref_grads[n], 1e-4, "all-reduced grad " + n)
        tr.apply_optimizer(LR)
        for n in ref.names:
            assert_close(tr.download_group(n)["w"], ref.group(n), 1e-5, "weights " + n)
        # full steps (all-reduces and FT row updates pipelined behind the weight gradient; the sixth optimizer step is a
        # Ranger look-ahead step): still the single-process answer, and the replicas stay bitwise identical
        for s in range(5):
            tr.train_step(batch, LR, 0.0, tb.LossKind.sigmoid())
            ref.step(full, LR, 0.0, O.sigmoid_loss())
        tr.flush_pending_loss()
        assert tr.step_count == 6 == ref.step_count
        for n in ref.names:
            assert_close(tr.download_group(n)["w"], ref.group(n), 1e-4, "weights after 6 steps " + n)
        first = {}
        for n in ref.names:
            first[n] = tr.download_group(n, which=("w", "m", "v", "slow"))
            w = torch.from_numpy(first[n]["w"])
            w0 = w.clone()
            dist.broadcast(w0, src=0)
            assert torch.equal(w, w0), "replicas diverged in " + n
        dist.barrier()
        tr.close()
        dist.barrier()
        # run to run: a second communicator and trainer, the same six steps: weights and optimizer state bit for bit
        ids = [tb.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        tr = tb.GpuTrainer(B, F, L1, L2, NB, fs, optimizer="ranger", init=init, device=int(os.environ["LOCAL_RANK"]),
                           world_size=world, rank=rank, nccl_id=ids[0], nccl_ctas=8, dp_exchange=exchange)
        tr.forward_backward(batch, 0.0, tb.LossKind.sigmoid())
        tr.apply_optimizer(LR)
        for s in range(5):
            tr.train_step(batch, LR, 0.0, tb.LossKind.sigmoid())
        tr.flush_pending_loss()
        for n in ref.names:
            grp = tr.download_group(n, which=("w", "m", "v", "slow"))
            for k, v in first[n].items():
                assert np.array_equal(grp[k], v), "second run differs in %s.%s" % (n, k)
        dist.barrier()
        tr.close()
    dist.barrier()
    if rank == 0:
        print("DP_WORKER_OK", mode, world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
