#!/usr/bin/env python
"""Benchmark of the hot path: data-parallel MLP training samples/s (headline), with the
GEMM TFLOP/s and softmax-CE / AdamW GB/s of the single kernels beside it.

    python bench.py --gpus N --steps K --warmup W [--workload c4|c5] [--impl reference]

One process per GPU (torchrun for N > 1).  Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# Datasheet figures, reported beside the measured ones: HBM3e 8 TB/s, dense TF32 1.1 PFLOP/s.
NOMINAL = {"hbm_gbs": 8000.0, "tf32_tflops": 1100.0}
# DRAM bytes (read + write) per tensor-core GEMM launch of one training step come from the committed ncu
# summary of that step (a line `dram_bytes_per_gemm_launch = <bytes>`).
TRAFFIC_PROFILE = {"c4": "mlp_c4_gemm_dram_traffic.md", "c5": "mlp_c5_gemm_dram_traffic.md"}


def gemm_traffic_per_launch(workload):
    import re
    path = os.path.join(ROOT, "profiles", TRAFFIC_PROFILE.get(workload, ""))
    try:
        m = re.search(r"dram_bytes_per_gemm_launch\s*=\s*([0-9.eE+]+)", open(path).read())
        return float(m.group(1)) if m else None
    except OSError:
        return None


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def host_threads():
    """Every host core, whatever OMP_NUM_THREADS says (torchrun exports 1 to its children)."""
    n = int(os.environ.get("FG_REF_THREADS", "0")) or (os.cpu_count() or 1)
    try:
        n = min(n, len(os.sched_getaffinity(0))) if not os.environ.get("FG_REF_THREADS") else n
    except AttributeError:
        pass
    return max(1, n)


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        self.p.wait()
        self.f.flush()
        rows = [l.strip().split(",") for l in open(self.f.name) if l.strip()]
        os.unlink(self.f.name)
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1])); pw.append(float(r[2]))
                for n, v in zip(names, r[3:7]):
                    if v.strip().lower() == "active":
                        reasons.add(n)
            except Exception:
                continue
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # the timed regions are separated by short idles: only samples taken under load count (power within 40 %
        # of the highest seen)
        load = [c for c, p in zip(sm, pw) if p >= 0.6 * max(pw)]
        return {"sm_mhz": float(np.median(load)), "sm_max_mhz": float(max(mx)), "power_w_max": float(max(pw)),
                "samples": len(load), "samples_idle": len(sm) - len(load), "reasons": sorted(reasons)}


def timed(torch, stream, ctx, fn, iters):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx.sync()
    with torch.cuda.stream(stream):
        e0.record()
    for i in range(iters):
        fn(i)
    with torch.cuda.stream(stream):
        e1.record()
    ctx.sync()
    return e0.elapsed_time(e1)


def flush_l2(torch, buf):
    buf.add_(1.0)   # writes a buffer larger than L2


# --------------------------------------------------------------------------------------
def run_reference(args, rank, world):
    """The reference has no CPU execution path and cannot be built here (Rust + HIP/wgpu), so
    this arm times the CPU oracle (a port of the reference's kernel arithmetic) on the host's
    cores, on the same workload."""
    if rank != 0:
        return
    import oracle
    from ferrograd_b200 import dp
    from ferrograd_b200.mlp import MLPTrainer
    w = dp.WORKLOADS[args.workload]
    oracle.set_num_threads(host_threads())
    threads = oracle.num_threads()
    dims = w["dims"]
    W, b = MLPTrainer.init_params(dims, w["init"], w["seed"])
    state = {k: [np.zeros_like(t) for t in (W if k[1] == "W" else b)] for k in ("mW", "vW", "mb", "vb")}
    od = dims[-1]

    def one(batch, step):
        x, t = dp.synth_batch(args.workload, 0, step % 4, batch)
        gs = 1.0 / (batch * (od if w["loss"] == "mse" else 1))
        t0 = time.perf_counter()
        oracle.mlp_step(dims, batch, w["act"], W, b, x, t, w["loss"], gs, w["opt"], step=step + 1, state=state)
        return time.perf_counter() - t0

    # size the per-step sample so that the whole run takes about two minutes
    probe_b = min(256, w["batch"])
    one(probe_b, 0)
    t_probe = one(probe_b, 1)
    step_limit_s = 120.0 / max(1, args.steps + args.warmup)
    batch = probe_b
    while batch * 2 <= w["batch"] and t_probe * (batch * 2 / probe_b) <= step_limit_s:
        batch *= 2
    for s in range(args.warmup):
        one(batch, s)
    total = sum(one(batch, args.warmup + s) for s in range(args.steps))
    value = batch * args.steps / total
    sample = (f"{args.steps} steps of {batch} samples each (full batch is {w['batch']}); the optimizer pass "
              "runs over all parameters every step, so a reduced batch understates the CPU samples/s")
    line = {"impl": "reference", "metric": "mlp_train_samples_per_s", "value": value, "unit": "samples/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "note": "CPU oracle port; the reference has no CPU path and needs "
                       "Rust + HIP or wgpu (unavailable on this box)"},
            "cpu_baseline": {"value": value, "unit": "samples/s", "cores": threads, "kind": "port", "sample": sample,
                             "cpu": cpu_model()},
            "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
def kernel_lines(torch, stream, ctx, peaks):
    """Single-kernel figures: C3 GEMM (fwd, dA, dB), C2 softmax-CE, AdamW/SGD on the C5 parameter count."""
    with torch.cuda.stream(stream):   # torch's allocations and fills run on the context's stream
        return _kernel_lines(torch, stream, ctx, peaks)


def _kernel_lines(torch, stream, ctx, peaks):
    out = {}
    hbm = peaks["hbm_gbs"]
    tf32x3_burst = peaks["bf16_tflops"] / 6.0
    flush = torch.empty(64 * 1024 * 1024, device="cuda")   # 256 MiB > L2

    def per_launch(kind, fn, iters):
        ctx.timing_read(kind)
        for i in range(iters):
            flush_l2(torch, flush)
            fn()
        n, ms, work = ctx.timing_read(kind)
        return n, ms / max(n, 1), work / max(n, 1)

    # C2
    rows, cols = 8192, 32000
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(rows, cols, device="cuda", generator=g) * 2.0
    lab = torch.randint(0, cols, (rows,), device="cuda", dtype=torch.int32, generator=g)
    dl = torch.empty_like(x)
    lrow, lmean = torch.empty(rows, device="cuda"), torch.empty(1, device="cuda")
    torch.cuda.synchronize()
    fn = lambda: ctx.softmax_ce(x.data_ptr(), lab.data_ptr(), rows, cols, 1.0 / rows, lrow.data_ptr(),
                                lmean.data_ptr(), dl.data_ptr())
    for _ in range(3):
        fn()
    n, ms, work = per_launch("softmax_ce", fn, 10)
    out["softmax_ce_c2"] = {"ms": ms, "gbs": work / ms / 1e6, "frac_of_hbm": work / ms / 1e6 / hbm,
                            "frac_of_nominal_hbm": work / ms / 1e6 / NOMINAL["hbm_gbs"], "bytes": work, "shape": [rows, cols]}
    del x, dl
    # row softmax alone (forward, backward) on rows short enough to be held in registers: 16384 x 4096
    rows2, cols2 = 16384, 4096
    x2 = torch.randn(rows2, cols2, device="cuda", generator=g) * 2.0
    y2, dy2, dx2 = torch.empty_like(x2), torch.randn(rows2, cols2, device="cuda", generator=g), torch.empty_like(x2)
    torch.cuda.synchronize()
    for name, fn in (("softmax_fwd_16384x4096", lambda: ctx.softmax_fwd(x2.data_ptr(), y2.data_ptr(), rows2, cols2)),
                     ("softmax_bwd_16384x4096", lambda: ctx.softmax_bwd(y2.data_ptr(), dy2.data_ptr(), dx2.data_ptr(), rows2, cols2))):
        for _ in range(3):
            fn()
        n, ms, work = per_launch("softmax_ce", fn, 5)
        out[name] = {"ms": ms, "gbs": work / ms / 1e6, "frac_of_hbm": work / ms / 1e6 / hbm, "bytes": work}
    del x2, y2, dy2, dx2
    # AdamW / SGD on the C5 parameter count
    n_par = 8 * (8192 * 8192 + 8192)
    bufs = [torch.zeros(n_par, device="cuda") for _ in range(4)]
    torch.cuda.synchronize()
    fn = lambda: ctx.adamw_step(bufs[0].data_ptr(), bufs[1].data_ptr(), bufs[2].data_ptr(), bufs[3].data_ptr(),
                                n_par, 1e-3, 0.9, 0.999, 1e-8, 0.01, step=2, zero_grad=False)
    for _ in range(3):
        fn()
    n, ms, work = per_launch("adamw", fn, 5)
    out["adamw_c5"] = {"ms": ms, "gbs": work / ms / 1e6, "frac_of_hbm": work / ms / 1e6 / hbm,
                       "frac_of_nominal_hbm": work / ms / 1e6 / NOMINAL["hbm_gbs"], "params": n_par, "bytes_per_param": 28}
    fn = lambda: ctx.sgd_step(bufs[0].data_ptr(), bufs[1].data_ptr(), n_par, 1e-3)
    for _ in range(3):
        fn()
    n, ms, work = per_launch("sgd", fn, 5)
    out["sgd_c5"] = {"ms": ms, "gbs": work / ms / 1e6, "frac_of_hbm": work / ms / 1e6 / hbm,
                     "frac_of_nominal_hbm": work / ms / 1e6 / NOMINAL["hbm_gbs"], "bytes_per_param": 16}
    del bufs
    # C3
    N = 8192
    s = 1.0 / N ** 0.5
    A = torch.randn(N, N, device="cuda", generator=g) * s
    B = torch.randn(N, N, device="cuda", generator=g) * s
    bias = torch.randn(N, device="cuda", generator=g) * s
    dC = torch.randn(N, N, device="cuda", generator=g)
    C, dA, dB = torch.empty_like(A), torch.empty_like(A), torch.empty_like(A)
    torch.cuda.synchronize()
    # Tensor work per f32 product, in units of one TF32 MMA: 3 for the 3xTF32 split, 2 for the default
    # (TF32 main term + two bf16 cross terms at half the cost each).  peak = measured bf16 burst / 2 / units.
    for mode, units in (("auto", 2.0), ("3xtf32", 3.0)):
        peak = peaks["bf16_tflops"] / 2.0 / units
        fwd = lambda: ctx.gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), N, N, N, bias=bias.data_ptr(), act="relu",
                               mode=mode)
        bwd = lambda: ctx.gemm_bwd(A.data_ptr(), B.data_ptr(), dC.data_ptr(), N, N, N, act="relu", saved=C.data_ptr(),
                                   dA=dA.data_ptr(), dB=dB.data_ptr(), mode=mode)
        for f in (fwd, bwd):
            f(); f()
        ctx.timing_read("gemm_tc"); ctx.timing_read("split")
        e_ms = timed(torch, stream, ctx, lambda i: fwd(), 5) / 5
        n, ms, work = ctx.timing_read("gemm_tc")
        tag = "" if mode == "auto" else "_3xtf32"
        out["gemm_c3_fwd" + tag] = {"mode": "tf32+bf16x2 (default)" if mode == "auto" else mode, "kernel_ms": ms / n,
                                    "kernel_tflops": work / ms / 1e9, "tensor_units_per_product": units,
                                    "frac_of_own_tensor_peak": work / ms / 1e9 / peak,
                                    "frac_of_3xtf32_peak": work / ms / 1e9 / tf32x3_burst,
                                    "frac_of_nominal_3xtf32": work / ms / 1e9 / (NOMINAL["tf32_tflops"] / 3.0),
                                    "call_ms_with_prepass": e_ms, "call_tflops_with_prepass": 2.0 * N ** 3 / e_ms / 1e9}
        ctx.timing_read("split")
        e_ms = timed(torch, stream, ctx, lambda i: bwd(), 5) / 5
        n, ms, work = ctx.timing_read("gemm_tc")
        out["gemm_c3_bwd_dA_dB" + tag] = {"mode": "tf32+bf16x2 (default)" if mode == "auto" else mode, "kernel_ms": ms / n,
                                          "kernel_tflops": work / ms / 1e9,
                                          "frac_of_own_tensor_peak": work / ms / 1e9 / peak,
                                          "frac_of_3xtf32_peak": work / ms / 1e9 / tf32x3_burst,
                                          "call_ms_with_prepass": e_ms,
                                          "call_tflops_with_prepass": 4.0 * N ** 3 / e_ms / 1e9}
    # the same shape on bf16 tensors: 16-bit operands go to the tensor cores as they are (kind::f16)
    del dC, dA, dB
    A16, B16, C16 = A.to(torch.bfloat16), B.to(torch.bfloat16), torch.empty(N, N, device="cuda", dtype=torch.bfloat16)
    b16 = bias.to(torch.bfloat16)
    torch.cuda.synchronize()
    f16 = lambda: ctx.gemm_lowp(A16.data_ptr(), B16.data_ptr(), C16.data_ptr(), N, N, N, "bf16", bias=b16.data_ptr(),
                                act="relu")
    f16(); f16()
    ctx.timing_read("gemm_tc")
    e_ms = timed(torch, stream, ctx, lambda i: f16(), 5) / 5
    n, ms, work = ctx.timing_read("gemm_tc")
    out["gemm_c3_fwd_bf16_storage"] = {"mode": "bf16 tensors, kind::f16 MMA, f32 accumulate", "kernel_ms": ms / n,
                                       "kernel_tflops": work / ms / 1e9,
                                       "frac_of_bf16_peak": work / ms / 1e9 / peaks["bf16_tflops"],
                                       "call_ms_with_transpose": e_ms,
                                       "call_tflops_with_transpose": 2.0 * N ** 3 / e_ms / 1e9}
    del A16, B16, C16, A, B, C
    # Streaming elementwise kernels on 32 Mi elements per tensor (128 MB each, so nothing fits the L2), and the three
    # kernels of a 10-class output layer on 32768 x 4096 activations (512 MB)
    n_el = 32 << 20
    t = [torch.rand(n_el, device="cuda", generator=g) * 0.8 + 0.1 for _ in range(2)] + \
        [torch.empty(n_el, device="cuda") for _ in range(2)]
    one = torch.empty(1, device="cuda")
    bias_v = torch.randn(4096, device="cuda", generator=g)
    gelu_chain = [("input", 0, 0, 0.0), ("input", 1, 0, 0.0), ("mul", 0, 1, 0.0), ("gelu", 2, 0, 0.0),
                  ("add", 3, 0, 0.0)]                                                            # gelu(x*y) + x
    ew = {
        "bias_gelu_fwd": lambda: ctx.bias_act_fwd(t[0].data_ptr(), bias_v.data_ptr(), "gelu", t[2].data_ptr(), n_el // 4096, 4096),
        "gelu_bwd": lambda: ctx.act_bwd(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), n_el, "gelu"),
        "mse_loss_grad": lambda: ctx.mse_loss_grad(t[0].data_ptr(), t[1].data_ptr(), n_el, 0.5, loss_elem=t[2].data_ptr(),
                                                   loss_sum=one.data_ptr(), grad=t[3].data_ptr()),
        "bce_loss_grad": lambda: ctx.bce_loss_grad(t[0].data_ptr(), t[1].data_ptr(), n_el, 0.5, loss_elem=t[2].data_ptr(),
                                                   loss_sum=one.data_ptr(), grad=t[3].data_ptr()),
        "chain_fwd_5_instr": lambda: ctx.eltwise_chain_fwd(gelu_chain, [t[0].data_ptr(), t[1].data_ptr()], t[2].data_ptr(), n_el),
        "chain_bwd_5_instr": lambda: ctx.eltwise_chain_bwd(gelu_chain, [t[0].data_ptr(), t[1].data_ptr()], t[2].data_ptr(),
                                                           [t[3].data_ptr(), None], n_el),
    }
    for name, fn in ew.items():
        for _ in range(3):
            fn()
        n, ms, work = per_launch("eltwise", fn, 5)
        out[name] = {"ms": ms, "gbs": work / ms / 1e6, "frac_of_hbm": work / ms / 1e6 / hbm, "bytes": work, "elements": n_el}
    del t
    Ms, Ks, Ns = 32768, 4096, 10
    h = torch.randn(Ms, Ks, device="cuda", generator=g)
    w_s = torch.randn(Ks, Ns, device="cuda", generator=g) * 0.02
    dz = torch.randn(Ms, Ns, device="cuda", generator=g)
    z_s, dw_s, dh = torch.empty(Ms, Ns, device="cuda"), torch.empty(Ks, Ns, device="cuda"), torch.empty(Ms, Ks, device="cuda")
    sk = {
        "skinny_fwd": lambda: ctx.gemm(h.data_ptr(), w_s.data_ptr(), z_s.data_ptr(), Ms, Ns, Ks),
        "skinny_bwd_dW_dX": lambda: ctx.gemm_bwd(h.data_ptr(), w_s.data_ptr(), dz.data_ptr(), Ms, Ns, Ks, dA=dh.data_ptr(),
                                                 dB=dw_s.data_ptr()),
    }
    for name, fn in sk.items():
        for _ in range(3):
            fn()
        n, ms, work = per_launch("skinny", fn, 5)
        out[name] = {"ms_per_kernel": ms, "gbs": work / ms / 1e6, "frac_of_hbm": work / ms / 1e6 / hbm,
                     "bytes_per_kernel": work, "shape": [Ms, Ns, Ks], "kernels_per_call": n // 5}
    del h, dh
    # C1: the reference's own CPU-scale case (MLP 2-16-2, batch 64, MSE, SGD), 1000 steps replayed as a plan;
    # launch-bound, so the figure is steps per second
    from ferrograd_b200 import dp
    from ferrograd_b200.mlp import MLPTrainer
    w1 = dp.WORKLOADS["c1"]
    tr1 = MLPTrainer(ctx, w1["dims"], w1["batch"], w1["act"], w1["loss"], w1["opt"], gemm_mode="simt")
    tr1.set_params(*MLPTrainer.init_params(w1["dims"], w1["init"], w1["seed"]))
    tr1.upload_batch(*dp.synth_batch("c1", 0, 0))
    tr1.step()
    tr1.build_plan()
    for _ in range(10):
        tr1.step_plan()
    ms = timed(torch, stream, ctx, lambda i: tr1.step_plan(), w1["steps"])
    out["mlp_c1"] = {"steps": w1["steps"], "ms_total": ms, "steps_per_s": w1["steps"] / ms * 1e3,
                     "samples_per_s": w1["steps"] * w1["batch"] / ms * 1e3, "final_loss_sum": tr1.get_loss(),
                     "note": "exact SIMT GEMM path; one CUDA-graph replay per step"}
    out["peak_note"] = ("tensor peaks derive from the measured bf16 burst: TF32 runs at half the bf16 rate; the 3xTF32 "
                        "peak is that / 3, the default mode's own peak that / 2; frac_of_hbm is of the measured copy "
                        "bandwidth; frac_of_nominal_* are of the datasheet figures (HBM 8 TB/s, dense TF32 1.1 PFLOP/s / 3)")
    return out


def fused_step_line(torch, stream, ctx, workload, steps):
    """The same workload through MLPTrainer: one flat parameter arena, one update launch, the whole step one
    CUDA graph, mean-reduced loss.  A side line: how much the four separate dispatches of the reference's loop cost."""
    from ferrograd_b200 import dp
    from ferrograd_b200.mlp import MLPTrainer
    w = dp.WORKLOADS[workload]
    tr = MLPTrainer(ctx, w["dims"], w["batch"], w["act"], w["loss"], w["opt"])
    tr.set_params(*MLPTrainer.init_params(w["dims"], w["init"], w["seed"]))
    tr.upload_batch(*dp.synth_batch(workload, 0, 0))
    for _ in range(3):
        tr.step()
    tr.build_plan()
    for _ in range(3):
        tr.step_plan()
    ms = timed(torch, stream, ctx, lambda i: tr.step_plan(), steps)
    out = {"samples_per_s": w["batch"] * steps / (ms / 1e3), "ms_per_step": ms / steps,
           "note": "MLPTrainer: flat arena, one update launch, one CUDA-graph replay per step, mean-reduced loss"}
    tr.destroy()
    return out


def get_arena(torch, ctx, net):
    """All parameters of a GraphMLP as one device vector (W0, b0, W1, b1, ...)."""
    parts = []
    for l in range(net.L):
        for t in (net.W[l], net.b[l]):
            v = torch.empty(t.size, device="cuda", dtype=torch.float32)
            ctx.copy_dev_async(v.data_ptr(), t.ptr, t.size * 4)
            parts.append(v)
    ctx.sync()
    return torch.cat(parts)


def dp_parity_check(torch, dist, ctx, net, make_net, w, workload, rank, world, W0, b0):
    """One training step on `world` ranks against the same step on ONE GPU over the concatenated batch, both
    through the graph API.  Returns (on every rank) the largest parameter difference between replicas -- it must be
    0: every rank applies the same update to the same summed gradient -- and, measured on rank 0, how far the
    N-rank loss and parameters are from the single-GPU ones (summation order is the only difference)."""
    from ferrograd_b200 import dp
    net.upload_batch(*dp.synth_batch(workload, rank, 0))
    net.step()
    ctx.sync()
    mine = get_arena(torch, ctx, net)
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    diff = (mine - ref).abs().max().to(torch.float64).reshape(1)
    dist.all_reduce(diff, op=dist.ReduceOp.MAX)
    loss = torch.tensor([net.get_loss()], device="cuda", dtype=torch.float64)
    dist.all_reduce(loss, op=dist.ReduceOp.SUM)         # the loss is an unreduced sum: the global loss is the sum over ranks
    out = {"replica_max_abs_diff": float(diff.item()), "loss_sum_n_ranks": float(loss.item())}
    if rank == 0:
        from ferrograd_b200 import GpuContext
        solo = GpuContext(ctx.device)                      # a context of its own: no communicator, nothing is exchanged
        single = make_net(w["batch"] * world, on=solo)
        single.set_params(W0, b0)
        single.upload_batch(*dp.global_batch(workload, world, 0))
        single.step()
        solo.sync()
        one = get_arena(torch, solo, single)
        out["loss_sum_one_gpu_on_concatenated_batch"] = single.get_loss()
        out["params_vs_one_gpu_max_abs_diff"] = float((mine - one).abs().max().item())
        out["params_rms"] = float(one.double().pow(2).mean().sqrt().item())
        out["note"] = ("the first AdamW step moves every weight by about lr, sign(g) deciding the direction, so where "
                       "|g| is at rounding level the two summation orders may differ by up to 2*lr")
        single.destroy()
        solo.destroy()
    dist.barrier()
    return out


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from ferrograd_b200 import GpuContext, dp
    from ferrograd_b200.mlp import GraphMLP, MLPTrainer

    # Libraries (NCCL's version banner, for one) may write to stdout; the contract is ONE JSON line there.
    # Keep the real stdout aside and point fd 1 at stderr until the line is printed.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(obj) + "\n").encode())

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks, peak_src = load_peaks()
    w = dp.WORKLOADS[args.workload]
    stream = torch.cuda.Stream()
    ctx = GpuContext(local_rank, stream=stream.cuda_stream)
    if world > 1:
        uid = dp.exchange_unique_id(ctx, dist, rank)
        ctx.comm_init(world, rank, uid)

    # The training loop is the reference's: a Graph, alloc_tensors, schedule, then dispatch_forward / dispatch_loss /
    # dispatch_backward / dispatch_optim per step.  With a communicator the engine sums the gradients over the ranks.
    def make_net(batch, on=None):
        return GraphMLP(on or ctx, w["dims"], batch, w["act"], w["loss"], w["opt"])

    net = make_net(w["batch"])
    W0, b0 = MLPTrainer.init_params(w["dims"], w["init"], w["seed"])
    net.set_params(W0, b0)

    # synthetic batches in pinned host memory (rotated); shapes and distributions per the workload
    NB = 4
    xs, ts = [], []
    for s in range(NB):
        x, t = dp.synth_batch(args.workload, rank, s)
        px, pt = ctx.pinned_array(x.shape, x.dtype), ctx.pinned_array(t.shape, t.dtype)
        px[...] = x; pt[...] = t
        xs.append(px); ts.append(pt)
    loss_host = ctx.pinned_array((1,), np.float32)
    h2d = xs[0].nbytes + ts[0].nbytes

    def barrier():
        ctx.sync()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- data-parallel parity, outside every timed region: one step from the initial parameters ----
    dp_check = None
    if world > 1:
        dp_check = dp_parity_check(torch, dist, ctx, net, make_net, w, args.workload, rank, world, W0, b0)
        net.destroy()
        net = make_net(w["batch"])          # a fresh start: initial parameters, zero optimizer state
        net.set_params(W0, b0)

    # ---- warm-up: plain launches first (they size the scratch arena), then the engine's own choice between
    #      plain launches and recorded CUDA graphs per dispatch (the reference's Schedule is a captured graph:
    #      rocm/mod.rs:324-389; here only launch-bound graphs, and medium ones with a communicator, are recorded);
    #      a dispatch is recorded on its second call, so four more steps settle that ----
    ctx.set_option("exec_plans", "0")
    net.upload_batch_async(xs[0], ts[0])
    for _ in range(max(3, args.warmup)):
        net.step()
    ctx.set_option("exec_plans", "auto")
    for _ in range(4):
        net.step()
    barrier()
    mode = ("dispatch_forward + dispatch_loss + dispatch_backward + dispatch_optim through the graph API, "
            + ("each replayed as a recorded CUDA graph" if net.tensors.plans_active() else
               "plain asynchronous launches (the engine records CUDA graphs only for launch-bound graphs)")
            + ("; gradients summed over the ranks inside dispatch_backward / dispatch_optim (NCCL)" if world > 1 else ""))
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()

    # ---- timed region 1 (headline): K steps, inputs resident in HBM ----
    launches0 = ctx.launch_count()
    barrier()
    ms = timed(torch, stream, ctx, lambda i: net.step(), args.steps)
    barrier()
    launches = ctx.launch_count() - launches0
    ms = max_over_ranks(ms)

    # ---- timed region 2: end to end through the public API with host buffers ----
    # Every step's inputs travel from pinned host memory inside the timed region; the copy of batch i+1 runs
    # on the context's copy stream while step i computes, and a device-to-device move puts it in place.
    # Half a second of idle first: the headline region has just drawn the GPU into its power cap, and a region
    # that starts there would be measured at lower clocks than one that starts after a warm-up, as the headline did.
    ctx.sync()
    time.sleep(0.5)
    net.prefetch_batch(xs[0], ts[0])

    def e2e_step(i):
        net.take_prefetched()                                   # batch i is on the device
        net.prefetch_batch(xs[(i + 1) % NB], ts[(i + 1) % NB])  # start moving batch i+1
        net.step()
        ctx.download_async(loss_host.ctypes.data, net.loss_out, 4)

    for i in range(3):
        e2e_step(i)
    barrier()
    e2e_ms = timed(torch, stream, ctx, e2e_step, args.steps)
    barrier()
    e2e_ms = max_over_ranks(e2e_ms)
    ctx.sync()
    final_loss_sum = float(loss_host[0])
    net.take_prefetched()                                       # the copy started by the last step is consumed

    # ---- timed region 3: the same K steps with plain launches, every GEMM / AdamW launch bracketed by CUDA
    #      events on the context's stream, which gives the roofline figures ----
    ctx.set_option("exec_plans", "0")
    time.sleep(0.5)
    for _ in range(3):
        net.step()
    ctx.timing_enable(True)
    for k in ("gemm_tc", "split", "adamw", "softmax_ce"):
        ctx.timing_read(k)
    barrier()
    eager_ms = timed(torch, stream, ctx, lambda i: net.step(), args.steps)
    barrier()
    eager_ms = max_over_ranks(eager_ms)
    gemm_n, gemm_ms, gemm_flop = ctx.timing_read("gemm_tc")
    split_n, split_ms, split_bytes = ctx.timing_read("split")
    adam_n, adam_ms, adam_bytes = ctx.timing_read("adamw")
    ctx.timing_enable(False)
    ctx.set_option("exec_plans", "auto")
    clocks = sampler.stop() if sampler else None

    # ---- the gradient exchange of one step alone (no compute beside it): one allreduce per layer's weight range,
    #      as the backward pass issues them, on the communicator the step uses; outside every timed region ----
    exchange_alone = None
    if world > 1:
        sizes = [w["dims"][l] * w["dims"][l + 1] + w["dims"][l + 1] for l in range(len(w["dims"]) - 1)]
        with torch.cuda.stream(stream):
            gbuf = torch.zeros(sum(sizes), device="cuda")
        ctx.sync()

        def exchange_once(i):
            off = 0
            for n_el in sizes:
                ctx.allreduce_sum(gbuf.data_ptr() + 4 * off, n_el)
                off += n_el
            ctx.comm_join()

        for i in range(2):
            exchange_once(i)
        barrier()
        x_ms = max_over_ranks(timed(torch, stream, ctx, exchange_once, 5)) / 5
        barrier()
        nbytes = 4.0 * sum(sizes)
        exchange_alone = {"bytes_per_step": nbytes, "ms": x_ms, "algbw_gbs": nbytes / x_ms / 1e6,
                          "busbw_gbs": nbytes / x_ms / 1e6 * 2.0 * (world - 1) / world, "allreduces": len(sizes)}
        del gbuf
    od = w["dims"][-1]
    final_loss = final_loss_sum / (w["batch"] * (od if w["loss"] == "mse" else 1))     # per-sample mean of this rank

    if rank == 0:
        gb = w["batch"] * world
        value = gb * args.steps / (ms / 1e3)
        # The default GEMM mode spends two TF32-MMA units of tensor work per f32 product (one tf32 MMA + two
        # bf16 MMAs at half cost), so its own ceiling is the TF32 rate / 2 = bf16 / 4.  Which measured bf16
        # figure applies depends on how long the GPU has been under load: the burst figure for a timed region
        # of under a second (the clocks stay near their maximum), the sustained one for a long region.
        region_s = eager_ms / 1e3
        basis = "burst" if region_s < 1.0 else "sustained"
        bf16_peak = peaks["bf16_tflops"] if basis == "burst" else peaks["bf16_tflops_sustained"]
        own_peak = bf16_peak / 4.0
        ach = gemm_flop / gemm_ms / 1e9 if gemm_ms > 0 else 0.0
        line = {
            "metric": "mlp_train_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "global_batch": gb, "parallelism": f"dp{world}",
                       "gemm": "tcgen05 on the f32 tensors as they lie: trunc(a)*trunc(b) as kind::tf32 plus the two cross "
                               "terms as bf16 MMAs from bf16 pairs kept beside every tensor, f32 accumulate (a 3xTF32 split "
                               "in which the two 2^-11-sized terms run at bf16 precision); no operand pre-pass",
                       "l2": "per-step working set (parameters, moments, activations, pairs: >1 GB) exceeds the 126 MB L2",
                       "timed_region": mode,
                       "order": "warm-up, this region, the end-to-end region, then the per-kernel-timed region; half a second of idle "
                                "and three untimed steps before each of the latter two, so that every region starts from "
                                "the same state of the power cap",
                       "roofline_region": "the same K steps launched eagerly with per-kernel CUDA events"},
            "clocks": clocks,
            "e2e": {"value": gb * args.steps / (e2e_ms / 1e3), "unit": "samples/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "kernel": "gemm_tc_pair_kernel (+ gemm_tc_pair_fold_kernel)", "achieved": ach,
                         "peak": own_peak, "unit": "TFLOP/s", "frac": ach / own_peak if own_peak else None,
                         "traffic": gemm_traffic_per_launch(args.workload),
                         "launches": int(gemm_n), "avg_launch_ms": gemm_ms / max(gemm_n, 1),
                         "peak_basis": f"{peak_src} bf16 {basis} {bf16_peak} TF/s / 2 (tf32 rate) / 2 (tensor work per f32 "
                                       f"product: one tf32 MMA + two half-cost bf16 MMAs); {basis} because the timed region "
                                       f"lasted {region_s:.3f} s",
                         "frac_of_burst": ach / (peaks["bf16_tflops"] / 4.0),
                         "frac_of_sustained": ach / (peaks["bf16_tflops_sustained"] / 4.0),
                         "frac_of_3xtf32_peak": ach / (bf16_peak / 6.0),
                         "frac_of_nominal_3xtf32": ach / (NOMINAL["tf32_tflops"] / 3.0),
                         "flop_per_launch": gemm_flop / max(gemm_n, 1),
                         "share_of_step": gemm_ms / eager_ms if eager_ms else None},
            "eager_ms_per_step": eager_ms / args.steps,
            "other_kernels": {"pairs_of_inputs": {"launches": int(split_n), "gbs": split_bytes / split_ms / 1e6 if split_ms else None,
                                                  "share_of_step": split_ms / eager_ms if eager_ms else None},
                              "adamw": {"launches": int(adam_n), "gbs": adam_bytes / adam_ms / 1e6 if adam_ms else None,
                                        "frac_of_hbm": adam_bytes / adam_ms / 1e6 / peaks["hbm_gbs"] if adam_ms else None,
                                        "frac_of_nominal_hbm": adam_bytes / adam_ms / 1e6 / NOMINAL["hbm_gbs"] if adam_ms else None,
                                        "share_of_step": adam_ms / eager_ms if eager_ms else None}},
            "final_loss": final_loss, "peaks": peak_src, "dp_check": dp_check, "exchange_alone": exchange_alone,
            "model_tflops": net.flops_per_step() * world * args.steps / (ms / 1e3) / 1e12,
        }
        if world == 1 and not args.no_kernels:
            try:
                line["fused_step_api"] = fused_step_line(torch, stream, ctx, args.workload, args.steps)
            except Exception as e:   # reported, never hidden
                line["fused_step_api"] = f"unavailable: {e}"
            ctx.timing_enable(True)
            line["kernels"] = kernel_lines(torch, stream, ctx, peaks)
            ctx.timing_enable(False)
            if not args.no_cpu:
                line["kernels"]["cpu"] = cpu_kernel_baselines()
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(args.workload)
        emit(line)
    barrier()
    net.destroy()           # the recorded dispatches hold the communicator: they go before it
    if world > 1:
        dist.destroy_process_group()
    ctx.destroy()


def cpu_baseline(workload):
    """The CPU oracle on this host's cores, on a bounded sample: a few full-batch steps."""
    import oracle
    from ferrograd_b200 import dp
    from ferrograd_b200.mlp import MLPTrainer
    w = dp.WORKLOADS[workload]
    dims, batch = w["dims"], w["batch"]
    oracle.set_num_threads(host_threads())
    W, b = MLPTrainer.init_params(dims, w["init"], w["seed"])
    state = {k: [np.zeros_like(t) for t in (W if k[1] == "W" else b)] for k in ("mW", "vW", "mb", "vb")}
    od = dims[-1]
    gs = 1.0 / (batch * (od if w["loss"] == "mse" else 1))
    x, t = dp.synth_batch(workload, 0, 0)
    times = []
    t_start = time.perf_counter()
    for s in range(8):
        t0 = time.perf_counter()
        oracle.mlp_step(dims, batch, w["act"], W, b, x, t, w["loss"], gs, w["opt"], step=s + 1, state=state)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > 20.0 and len(times) >= 2:
            break
    use = times[1:] if len(times) > 1 else times
    return {"value": batch * len(use) / sum(use), "unit": "samples/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": f"{len(use)} full training steps of {batch} samples after one warm-up step", "cpu": cpu_model()}


def cpu_kernel_baselines():
    """The CPU oracle on this host's cores for the single-kernel figures, each on a bounded sample."""
    import oracle
    from ferrograd_b200 import dp
    from ferrograd_b200.mlp import MLPTrainer
    oracle.set_num_threads(host_threads())
    cores = oracle.num_threads()
    r = np.random.Generator(np.random.Philox(99))
    out = {"cores": cores, "cpu": cpu_model(), "kind": "port"}

    def best(fn, reps=3):
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return min(ts)

    # softmax-CE: 1024 of the 8192 rows of 32000 logits
    rows, cols = 1024, 32000
    x = (2.0 * r.standard_normal((rows, cols), np.float32)).astype(np.float32)
    lab = r.integers(0, cols, rows).astype(np.uint32)
    t = best(lambda: oracle.softmax_ce(x, lab, grad_scale=1.0 / rows))
    out["softmax_ce_c2"] = {"gbs": 2.0 * rows * cols * 4 / t / 1e9, "sample": f"{rows} of 8192 rows x {cols}",
                            "full_size_ms_estimate": t * 8192 / rows * 1e3}
    del x
    # AdamW / SGD: 32 Mi of the 537 M parameters
    n = 32 << 20
    w, g, m, v = (np.zeros(n, np.float32) for _ in range(4))
    t = best(lambda: oracle.adamw(w, g, m, v, 1e-3, 0.9, 0.999, 1e-8, 0.01, 2, zero_grad=False))
    out["adamw_c5"] = {"gbs": 28.0 * n / t / 1e9, "sample": f"{n} of 536936448 parameters",
                       "full_size_ms_estimate": t * 536936448 / n * 1e3}
    t = best(lambda: oracle.sgd(w, g, 1e-3))
    out["sgd_c5"] = {"gbs": 16.0 * n / t / 1e9, "sample": f"{n} of 536936448 parameters",
                     "full_size_ms_estimate": t * 536936448 / n * 1e3}
    del w, g, m, v
    # GEMM: a 2048^3 slice of the 8192^3 product (1/64 of the flop; same k-sequential f32 fma arithmetic)
    N = 2048
    A, B = r.standard_normal((N, N), np.float32), r.standard_normal((N, N), np.float32)
    t = best(lambda: oracle.gemm(A, B), reps=2)
    out["gemm_c3"] = {"tflops": 2.0 * N ** 3 / t / 1e12, "sample": "2048^3 slice of 8192^3 (1/64 of the work)",
                      "full_size_ms_estimate": t * 64 * 1e3}
    # the tiny MLP: 200 of its 1000 steps
    w1 = dp.WORKLOADS["c1"]
    W, b = MLPTrainer.init_params(w1["dims"], w1["init"], w1["seed"])
    xs, ts = dp.synth_batch("c1", 0, 0)
    steps = 200
    t0 = time.perf_counter()
    for s_ in range(steps):
        oracle.mlp_step(w1["dims"], w1["batch"], w1["act"], W, b, xs, ts, w1["loss"], 1.0 / (w1["batch"] * 2), w1["opt"],
                        step=s_ + 1)
    t = time.perf_counter() - t0
    out["mlp_c1"] = {"steps_per_s": steps / t, "sample": f"{steps} of 1000 steps (one ctypes call per step)"}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=["c4", "c5"])
    ap.add_argument("--no-kernels", action="store_true", help="skip the single-kernel figures")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        print(json.dumps({"error": "launch with torchrun --nproc-per-node N for N > 1"}))
        sys.exit(2)
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
