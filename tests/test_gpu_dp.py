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


def _rank_graph_api(rank, world, port, out_dir, plans):
    """The reference's training loop (dispatch_forward / loss / backward / optim) on two ranks: the graph engine
    itself sums the gradients over the ranks.  A small exchange threshold makes the backward pass start exchanges
    of its own, as it does for large layers; four steps cover the eager, the recorded and the replayed dispatch."""
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    from ferrograd_b200 import GpuContext, dp
    from ferrograd_b200.mlp import GraphMLP, MLPTrainer
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)     # host plumbing only
    ctx = GpuContext(rank)
    ctx.comm_init(world, rank, dp.exchange_unique_id(ctx, dist, rank))
    ctx.set_option("comm_min_exchange", 20000)
    ctx.set_option("exec_plans", plans)             # recorded and replayed dispatches, or plain launches
    net = GraphMLP(ctx, GDIMS, BATCH, "gelu", "ce", OPT)
    net.set_params(*MLPTrainer.init_params(GDIMS, "he_normal", 21))
    for s in range(GSTEPS):
        net.upload_batch(*dp.synth_batch(dict(dims=GDIMS, batch=BATCH, loss="ce"), rank, s))
        net.step()
        ctx.comm_sync(20000)          # a rank that waits for a peer that never comes ends with FG_ERR_TIMEOUT, not a hang
    ctx.sync()
    assert ctx.device_status() == 0
    W, b = net.get_params()
    np.savez(os.path.join(out_dir, f"graph_rank{rank}.npz"), *W, *b)
    dist.barrier()
    net.destroy()                 # the recorded dispatches hold the communicator: they go first
    dist.destroy_process_group()
    ctx.destroy()


GDIMS, GSTEPS = [64, 256, 192, 10], 4


@pytest.mark.parametrize("plans", ["1", "0"])
def test_graph_api_two_gpus_match_one_gpu_on_the_global_batch(tmp_path, plans):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from ferrograd_b200 import GpuContext, dp
    from ferrograd_b200.mlp import GraphMLP, MLPTrainer
    mp.spawn(_rank_graph_api, args=(2, 29900 + os.getpid() % 300 + int(plans), str(tmp_path), plans), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "graph_rank0.npz"), np.load(tmp_path / "graph_rank1.npz")
    for k in r0.files:
        assert np.array_equal(r0[k], r1[k])           # replicas stay bit-identical
    # one GPU, the concatenated batch, the same API: the loss is unreduced, so the summed gradient is the same sum
    ctx = GpuContext(0)
    net = GraphMLP(ctx, GDIMS, 2 * BATCH, "gelu", "ce", OPT)
    net.set_params(*MLPTrainer.init_params(GDIMS, "he_normal", 21))
    for s in range(GSTEPS):
        net.upload_batch(*dp.global_batch(dict(dims=GDIMS, batch=BATCH, loss="ce"), 2, s))
        net.step()
    ctx.sync()
    W, b = net.get_params()
    ctx.destroy()
    for got, ref in zip([r0[k] for k in r0.files], W + b):
        assert np.max(np.abs(got - ref)) <= 2e-5 + 1e-4 * np.max(np.abs(ref)), float(np.max(np.abs(got - ref)))


def _rank_peer_absent(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    from ferrograd_b200 import FgError, GpuContext, dp
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)     # host plumbing only
    ctx = GpuContext(rank)
    ctx.comm_init(world, rank, dp.exchange_unique_id(ctx, dist, rank))
    n = 4096
    buf = ctx.init_tensor_f32((n,), np.full(n, rank + 1.0, np.float32))
    ctx.allreduce_sum(buf, n)                 # a healthy exchange first: 1 + 2 on both ranks
    ctx.comm_sync(5000)
    ctx.sync()
    ok_first = bool((ctx.to_numpy(buf) == 3.0).all())
    dist.barrier()
    result = "none"
    if rank == 0:
        # rank 1 has stopped taking part (between steps, nothing of its own in flight): this exchange can
        # never complete; the bounded wait must report it and leave the context usable
        ctx.allreduce_sum(buf, n)
        try:
            ctx.comm_sync(1000)
            result = "completed"
        except FgError as e:
            result = e.kind
        w, g = ctx.init_tensor_f32((n,), np.full(n, 3.0, np.float32)), ctx.init_tensor_f32((n,), np.full(n, 2.0, np.float32))
        ctx.sgd_step(w, g, n, 0.5)
        ctx.sync()
        usable = bool((ctx.to_numpy(w) == 2.0).all())
        with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
            f.write(f"{ok_first} {result} {usable}")
    dist.barrier()                            # rank 1 waits here, on the host, until rank 0 is done
    if rank == 1:
        ctx.comm_abort()                      # its peer's communicator is gone: no collective teardown
    dist.destroy_process_group()
    ctx.destroy()


def test_absent_peer_ends_the_exchange_with_a_timeout(tmp_path):
    """Failure detection without a GPU fault: the failure is made on the host (a rank that does not join),
    the wait on the exchange is bounded, the communicator is aborted and the context stays usable."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_rank_peer_absent, args=(2, 29300 + os.getpid() % 300, str(tmp_path)), nprocs=2, join=True)
    ok_first, result, usable = open(tmp_path / "rank0.txt").read().split()
    assert ok_first == "True"
    assert result == "FG_ERR_TIMEOUT", result
    assert usable == "True"
