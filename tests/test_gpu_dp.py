"""Data-parallel training on real GPUs: two ranks (one process per GPU, gradients summed with
fg_allreduce_sum_f32 over NCCL) must end up with the parameters a single GPU gets from the
concatenated batch.  Skipped when fewer than two GPUs are visible."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DIMS, BATCH, STEPS = [64, 256, 192, 10], 256, 3
OPT = ("adamw", 1e-3, 0.9, 0.999, 1e-8, 0.01)
WL = dict(dims=DIMS, batch=BATCH, loss="ce")


def _rank(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    from ferrograd_b200 import GpuContext, dp
    from ferrograd_b200.mlp import MLPTrainer
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)     # host plumbing only
    ctx = GpuContext(rank)
    ctx.comm_init(world, rank, dp.exchange_unique_id(ctx, dist, rank))
    tr = MLPTrainer(ctx, DIMS, BATCH, "gelu", "ce", OPT, world=world, rank=rank, gemm_mode="3xtf32")
    tr.set_params(*MLPTrainer.init_params(DIMS, "he_normal", 21))
    for s in range(STEPS):
        x, t = dp.synth_batch(WL, rank, s)
        tr.upload_batch(x, t)
        tr.step()
    ctx.sync()
    W, b = tr.get_params()
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), *W, *b)
    dist.barrier()
    dist.destroy_process_group()
    ctx.destroy()


def test_two_gpus_match_one_gpu_on_the_global_batch(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from ferrograd_b200 import GpuContext, dp
    from ferrograd_b200.mlp import MLPTrainer
    mp.spawn(_rank, args=(2, 29600 + os.getpid() % 300, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    for k in r0.files:
        assert np.array_equal(r0[k], r1[k])           # replicas stay bit-identical
    ctx = GpuContext(0)
    tr = MLPTrainer(ctx, DIMS, 2 * BATCH, "gelu", "ce", OPT, gemm_mode="3xtf32")
    tr.set_params(*MLPTrainer.init_params(DIMS, "he_normal", 21))
    for s in range(STEPS):
        x, t = dp.global_batch(WL, 2, s)
        tr.upload_batch(x, t)
        tr.step()
    ctx.sync()
    W, b = tr.get_params()
    ctx.destroy()
    for got, ref in zip([r0[k] for k in r0.files], W + b):
        # same mathematics, different summation order (per-rank partial sums); Adam steps are at most lr each
        assert np.max(np.abs(got - ref)) <= 2e-5 + 1e-4 * np.max(np.abs(ref)), float(np.max(np.abs(got - ref)))
