"""Small, self-contained runs of single kernels, sized for profiler captures: inputs larger
than the 126 MB L2 so DRAM counters mean something, but well under a few GB on the device
and only a handful of launches.

    python -m ferrograd_b200.cases gemm|gemm_bwd|gemm_bf16|softmax_ce|adamw|sgd|mlp [--iters N]
"""
import argparse
import sys

import numpy as np

from . import GpuContext
from .mlp import MLPTrainer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "gemm_bwd", "gemm_bf16", "softmax_ce", "adamw", "sgd", "mlp"])
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
    else:   # one BASELINE config-4 sized training step per iteration
        from . import dp
        w = dp.WORKLOADS["c4"]
        tr = MLPTrainer(ctx, w["dims"], w["batch"], w["act"], w["loss"], w["opt"])
        W, b = MLPTrainer.init_params(w["dims"], w["init"], w["seed"])
        tr.set_params(W, b)
        x, t = dp.synth_batch("c4", 0, 0)
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
