"""Small, self-contained runs of single kernels, sized for profiler captures: inputs larger
than the 126 MB L2 so DRAM counters mean something, but well under a few GB on the device
and only a handful of launches.

    python -m ferrograd_b200.cases gemm|gemm_bwd|gemm_bf16|layer|softmax|softmax_ce|adamw|sgd|eltwise|skinny|mlp|graph_mlp [--iters N]

mlp runs training steps of a benchmark workload (--workload c4|c5|c5s) through MLPTrainer, graph_mlp the same
through the graph API (dispatch_forward / loss / backward / optim); c5s is the eight-layer workload at 4096-wide
layers and 4096 samples, small enough for a multi-pass capture.  layer runs the three GEMMs of one hidden layer on
f32 tensors with bf16 pairs as a training step launches them (forward with bias, tanh and the output's pairs; dW; dX
with the activation factor of the layer below, its pairs and its bias gradient) at --m samples, --k inputs, --nn
outputs (default 2048 x 8192 x 8192, one layer of the eight-layer workload).
"""
import argparse
import sys

import numpy as np

from . import GpuContext
from .mlp import MLPTrainer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "gemm_bwd", "gemm_bf16", "layer", "softmax", "softmax_ce", "adamw", "sgd", "eltwise", "skinny",
                                     "mlp", "graph_mlp"])
    ap.add_argument("--workload", default="c4", choices=["c4", "c5", "c5s"])
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--nn", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--n", type=int, default=0, help="override the problem size")
    ap.add_argument("--mode", default="auto", choices=["auto", "simt", "3xtf32", "tf32_bf16x2"], help="GEMM mode")
    a = ap.parse_args()
    ctx = GpuContext(0)
    r = np.random.Generator(np.random.Philox(1))
    if a.case in ("gemm", "gemm_bwd"):
        n = a.n or 4096
        A = ctx.init_tensor_f32((n, n), r.standard_normal((n, n), np.float32) / np.float32(n ** 0.5))
        B = ctx.init_tensor_f32((n, n), r.standard_normal((n, n), np.float32) / np.float32(n ** 0.5))
        bias = ctx.init_tensor_f32((n,), r.standard_normal(n, np.float32))
        Cm = ctx.new_tensor((n, n))
        if a.case == "gemm":
            for _ in range(a.iters):
                ctx.gemm(A, B, Cm, n, n, n, bias=bias, act="relu", mode=a.mode)
        else:
            dY = ctx.init_tensor_f32((n, n), r.standard_normal((n, n), np.float32))
            ctx.gemm(A, B, Cm, n, n, n, bias=bias, act="relu", mode=a.mode)
            dA, dB = ctx.new_tensor((n, n)), ctx.new_tensor((n, n))
            for _ in range(a.iters):
                ctx.gemm_bwd(A, B, dY, n, n, n, act="relu", saved=Cm, dA=dA, dB=dB, mode=a.mode)
    elif a.case == "gemm_bf16":
        n = a.n or 8192
        A = ctx.init_tensor_bf16((n, n), r.standard_normal((n, n), np.float32) / np.float32(n ** 0.5))
        B = ctx.init_tensor_bf16((n, n), r.standard_normal((n, n), np.float32) / np.float32(n ** 0.5))
        bias = ctx.init_tensor_bf16((n,), r.standard_normal(n, np.float32))
        Cm = ctx.new_tensor((n, n), np.uint16)
        for _ in range(a.iters):
            ctx.gemm_lowp(A, B, Cm, n, n, n, "bf16", bias=bias, act="relu")
    elif a.case == "layer":
        M, K, N = a.m, a.k, a.nn
        f = lambda shape, scale: ctx.init_tensor_f32(shape, r.standard_normal(shape, np.float32) * np.float32(scale))
        x, w, bias, dz, saved_below = f((M, K), 1.0), f((K, N), K ** -0.5), f((N,), 0.1), f((M, N), 1.0), f((M, K), 0.5)
        pairs = {name: ctx.new_tensor((2, rows * cols), np.uint16)
                 for name, (rows, cols) in dict(x=(M, K), w=(K, N), y=(M, N), dz=(M, N), dx=(M, K)).items()}
        ctx.pairs_from_f32(x, M * K, pairs["x"])
        ctx.pairs_from_f32(w, K * N, pairs["w"])
        ctx.pairs_from_f32(dz, M * N, pairs["dz"])
        y, dw, dx, db_below = ctx.new_tensor((M, N)), ctx.new_tensor((K, N)), ctx.new_tensor((M, K)), ctx.new_tensor((K,))
        for _ in range(a.iters):
            ctx.gemm_paired(x, w, y, M, N, K, A_pairs=pairs["x"], B_pairs=pairs["w"], bias=bias, act="tanh", C_pairs=pairs["y"])
            ctx.gemm_bwd_paired(x, w, dz, M, N, K, A_pairs=pairs["x"], B_pairs=pairs["w"], dZ_pairs=pairs["dz"], dB=dw, dA=dx,
                                below_act="tanh", below_saved=saved_below, dA_pairs=pairs["dx"], below_dbias=db_below)
    elif a.case == "softmax":
        # row softmax alone, forward and backward, on rows too short for the row-in-registers kernel
        rows, cols = a.n or 16384, 4096
        x = ctx.init_tensor_f32((rows, cols), 2.0 * r.standard_normal((rows, cols), np.float32))
        dy = ctx.init_tensor_f32((rows, cols), r.standard_normal((rows, cols), np.float32))
        y, dx = ctx.new_tensor((rows, cols)), ctx.new_tensor((rows, cols))
        for _ in range(a.iters):
            ctx.softmax_fwd(x, y, rows, cols)
            ctx.softmax_bwd(y, dy, dx, rows, cols)
    elif a.case == "softmax_ce":
        rows, cols = a.n or 2048, 32000
        x = ctx.init_tensor_f32((rows, cols), 2.0 * r.standard_normal((rows, cols), np.float32))
        lab = ctx.init_tensor_u32((rows,), r.integers(0, cols, rows).astype(np.uint32))
        dl, lr, lm = ctx.new_tensor((rows, cols)), ctx.new_tensor((rows,)), ctx.new_tensor((1,))
        for _ in range(a.iters):
            ctx.softmax_ce(x, lab, rows, cols, grad_scale=1.0 / rows, loss_row=lr, loss_mean=lm, dlogits=dl)
    elif a.case in ("adamw", "sgd"):
        n = a.n or (64 << 20)
        bufs = [ctx.new_tensor((n,), zeroed=True) for _ in range(4)]
        for i in range(a.iters):
            if a.case == "adamw":
                ctx.adamw_step(bufs[0], bufs[1], bufs[2], bufs[3], n, 1e-3, 0.9, 0.999, 1e-8, 0.01, step=i + 1,
                               zero_grad=False)
            else:
                ctx.sgd_step(bufs[0], bufs[1], n, 1e-3)
    elif a.case == "eltwise":
        # every streaming elementwise kernel once per iteration, on 32 Mi elements per tensor (128 MB)
        n = a.n or (32 << 20)
        t = [ctx.init_tensor_f32((n,), (r.random(n, np.float32) * np.float32(0.8) + np.float32(0.1))) for _ in range(2)]
        t += [ctx.new_tensor((n,)) for _ in range(2)]
        one = ctx.new_tensor((1,))
        bias = ctx.init_tensor_f32((4096,), r.standard_normal(4096, np.float32))
        chain = [("input", 0, 0, 0.0), ("input", 1, 0, 0.0), ("mul", 0, 1, 0.0), ("gelu", 2, 0, 0.0), ("add", 3, 0, 0.0)]
        for _ in range(a.iters):
            ctx.bias_act_fwd(t[0], bias, "gelu", t[2], n // 4096, 4096)
            ctx.act_bwd(t[0], t[1], t[2], n, "gelu")
            ctx.mse_loss_grad(t[0], t[1], n, 0.5, loss_elem=t[2], loss_sum=one, grad=t[3])
            ctx.bce_loss_grad(t[0], t[1], n, 0.5, loss_elem=t[2], loss_sum=one, grad=t[3])
            ctx.eltwise_chain_fwd(chain, [t[0], t[1]], t[2], n)
            ctx.eltwise_chain_bwd(chain, [t[0], t[1]], t[2], [t[3], None], n)
    elif a.case == "skinny":
        # the three kernels of a 10-class output layer on 32768 x 4096 activations (512 MB)
        M, K, N = a.n or 32768, 4096, 10
        h = ctx.init_tensor_f32((M, K), r.standard_normal((M, K), np.float32))
        w = ctx.init_tensor_f32((K, N), r.standard_normal((K, N), np.float32) * np.float32(0.02))
        dz = ctx.init_tensor_f32((M, N), r.standard_normal((M, N), np.float32))
        z, dw, dh = ctx.new_tensor((M, N)), ctx.new_tensor((K, N)), ctx.new_tensor((M, K))
        for _ in range(a.iters):
            ctx.gemm(h, w, z, M, N, K)
            ctx.gemm_bwd(h, w, dz, M, N, K, dA=dh, dB=dw)
    else:   # training steps of a benchmark workload
        from . import dp
        from .mlp import GraphMLP
        w = dict(dp.WORKLOADS["c5" if a.workload == "c5s" else a.workload])
        if a.workload == "c5s":
            w["dims"], w["batch"] = [4096] * 9, 4096
        cls = GraphMLP if a.case == "graph_mlp" else MLPTrainer
        tr = cls(ctx, w["dims"], w["batch"], w["act"], w["loss"], w["opt"])
        W, b = MLPTrainer.init_params(w["dims"], w["init"], w["seed"])
        tr.set_params(W, b)
        x, t = dp.synth_batch(w if a.workload == "c5s" else a.workload, 0, 0)
        tr.upload_batch(x, t)
        for _ in range(a.iters):
            tr.step()
    ctx.sync()
    status = ctx.device_status()
    print(f"{a.case}: done, device status {status}, launches {ctx.launch_count()}")
    ctx.destroy()
    return 0 if status == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
