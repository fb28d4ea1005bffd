"""Host-side logic of the data-parallel path: workload definitions, per-rank synthetic
data, and the exchange of the NCCL id.  Nothing here touches a GPU, so it is covered by
CPU tests with gloo ranks.

The reference is single-device (crates/fused_gpu/src/dispatch/backend/rocm/mod.rs:58-78);
data parallelism shards the batch by rank, keeps parameters and optimizer state
replicated, and sums gradients once per step.
"""
import numpy as np

# Benchmark workloads that train an MLP.  `batch` is per GPU (weak scaling).
WORKLOADS = {
    "c1": dict(name="C1: MLP 2-16-2 tanh, MSE, SGD lr 0.1, batch 64", dims=[2, 16, 2], batch=64, act="tanh",
               loss="mse", opt=("sgd", 0.1), init="xavier_uniform", seed=0, steps=1000),
    "c4": dict(name="C4: DP MLP 784-4096-4096-10 GELU, softmax-CE, AdamW, 4096 samples/GPU",
               dims=[784, 4096, 4096, 10], batch=4096, act="gelu", loss="ce",
               opt=("adamw", 1e-3, 0.9, 0.999, 1e-8, 0.01), init="he_normal", seed=7, steps=100),
    "c5": dict(name="C5: DP MLP 8x8192 tanh, MSE, AdamW, 2048 samples/GPU", dims=[8192] * 9, batch=2048,
               act="tanh", loss="mse", opt=("adamw", 1e-3, 0.9, 0.999, 1e-8, 0.01), init="normal_fan_in",
               seed=8, steps=50),
}


def batch_seed(base, rank, step):
    """Distinct, reproducible seed per (rank, step); ranks never share a stream."""
    return int(base) + 1_000_003 * int(rank) + 7919 * int(step)


def synth_batch(workload, rank, step, batch=None):
    """Synthetic inputs and targets of one rank for one step, with the shapes and value
    distributions the workload states."""
    w = WORKLOADS[workload] if isinstance(workload, str) else workload
    B = int(batch or w["batch"])
    din, dout = w["dims"][0], w["dims"][-1]
    key = workload if isinstance(workload, str) else "custom"
    r = np.random.Generator(np.random.Philox(batch_seed(100, rank, step)))
    if key == "c1":
        x = r.uniform(-1.0, 1.0, (B, din)).astype(np.float32)
        pos = (x[:, 0] * x[:, 1]) > 0
        t = np.zeros((B, dout), np.float32)
        t[np.arange(B), pos.astype(np.int64)] = 1.0
        return x, t
    if w["loss"] == "ce":
        x = r.random((B, din), np.float32)                       # uniform in [0, 1)
        t = r.integers(0, dout, B).astype(np.uint32)
        return x, t
    x = r.standard_normal((B, din), np.float32)
    t = r.standard_normal((B, dout), np.float32)
    return x, t


def global_batch(workload, world, step, batch=None):
    """Concatenation of every rank's shard: what a single device would have to process to
    produce the same summed gradient."""
    parts = [synth_batch(workload, r, step, batch) for r in range(world)]
    return np.concatenate([p[0] for p in parts]), np.concatenate([p[1] for p in parts])


def exchange_unique_id(ctx, dist, rank):
    """Rank 0 creates the NCCL id; everyone receives it through torch.distributed."""
    box = [ctx.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return box[0]
