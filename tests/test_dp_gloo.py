"""Data-parallel host logic on CPU: two gloo ranks shard the batch, compute gradients with
the CPU oracle, sum them, and must reproduce the single-process gradient on the
concatenated batch.  Also covers the id exchange used to bootstrap NCCL."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import oracle
    from ferrograd_b200 import dp
    from ferrograd_b200.mlp import MLPTrainer
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    oracle.set_num_threads(2)
    wl = dict(dims=[24, 32, 10], batch=48, loss="ce")
    dims, B = wl["dims"], wl["batch"]
    W, b = MLPTrainer.init_params(dims, "he_normal", 11)

    class FakeCtx:   # stands in for the GPU context: only the id source is needed here
        def comm_unique_id(self):
            return bytes(range(128))

    uid = dp.exchange_unique_id(FakeCtx(), dist, rank)
    assert uid == bytes(range(128))

    x, t = dp.synth_batch(wl, rank, 0)
    _, gW, gb, _ = oracle.mlp_step(dims, B, "gelu", [w.copy() for w in W], [v.copy() for v in b], x, t, "ce",
                                   1.0 / (B * world), ("none",))
    flat = torch.from_numpy(np.concatenate([g.ravel() for g in gW + gb]))
    dist.all_reduce(flat)                       # the step's one exchange: a gradient sum
    if rank == 0:
        xg, tg = dp.global_batch(wl, world, 0)
        _, rW, rb, _ = oracle.mlp_step(dims, B * world, "gelu", [w.copy() for w in W], [v.copy() for v in b], xg,
                                       tg, "ce", 1.0 / (B * world), ("none",))
        ref = np.concatenate([g.ravel() for g in rW + rb])
        np.save(os.path.join(out_dir, "got.npy"), flat.numpy())
        np.save(os.path.join(out_dir, "ref.npy"), ref)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gradient_sum_equals_global_batch(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got, ref = np.load(tmp_path / "got.npy"), np.load(tmp_path / "ref.npy")
    rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    assert np.all(np.abs(got - ref) <= 1e-5 * (np.abs(ref) + rms))


def test_shards_are_disjoint_and_reproducible():
    sys.path.insert(0, ROOT)
    from ferrograd_b200 import dp
    a0, _ = dp.synth_batch("c4", 0, 0, 8)
    a0b, _ = dp.synth_batch("c4", 0, 0, 8)
    a1, _ = dp.synth_batch("c4", 1, 0, 8)
    a0s1, _ = dp.synth_batch("c4", 0, 1, 8)
    assert np.array_equal(a0, a0b) and not np.array_equal(a0, a1) and not np.array_equal(a0, a0s1)
    assert a0.min() >= 0.0 and a0.max() < 1.0
    x, t = dp.synth_batch("c1", 0, 0)
    assert x.shape == (64, 2) and t.shape == (64, 2)
    assert np.array_equal(t[:, 1] == 1.0, (x[:, 0] * x[:, 1]) > 0) and (t.sum(1) == 1.0).all()
    xg, tg = dp.global_batch("c4", 4, 0, 8)
    assert xg.shape == (32, 784) and tg.dtype == np.uint32 and tg.max() < 10


def test_arena_layout_and_buckets():
    sys.path.insert(0, ROOT)
    from ferrograd_b200.mlp import _align
    dims = [784, 4096, 4096, 10]
    off, ranges = 0, []
    for l in range(3):
        start = off
        off = _align(off + dims[l] * dims[l + 1])
        off = _align(off + dims[l + 1])
        ranges.append((start, off))
    assert ranges[0][0] == 0 and all(ranges[i][1] == ranges[i + 1][0] for i in range(2))
    assert all(r[0] % 64 == 0 for r in ranges)       # 256-byte aligned bucket starts
