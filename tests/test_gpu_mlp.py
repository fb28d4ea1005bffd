"""GPU parity of whole training steps (forward -> loss -> backward -> update) against the CPU
oracle composing the same operations in the reference's order.  GEMM-bearing results are
held to 1e-4, as |x - ref| <= tol * (|ref| + rms(ref))."""
import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu
TOL = 1e-4


@pytest.fixture(scope="module")
def ctx():
    from ferrograd_b200 import GpuContext
    c = GpuContext(0)
    yield c
    c.sync()
    c.destroy()


def zeros_state(W, b):
    return {k: [np.zeros_like(t) for t in (W if k[1] == "W" else b)] for k in ("mW", "vW", "mb", "vb")}


def check(x, ref, tol, what):
    ok, worst = rel_err_ok(x, ref, tol)
    assert ok, f"{what}: worst error ratio {worst:.3g} x tolerance {tol}"


def param_bound(ref_p, ref_g, opt, tol):
    """Allowed |p - p_ref| after one update when the gradient itself is only known to `tol`.

    SGD is linear in g.  The first AdamW step is lr * g / (|g| + eps) (+ decay): its slope in g is
    at most lr / (|g| + eps), so a gradient error of tol * (|g| + rms g) moves the parameter by up to
    lr * tol * (|g| + rms g) / (|g| + eps), capped at 2 lr (the step itself is at most lr).  Where |g| is
    far above eps this term is about lr * tol; it only opens up for gradients near zero, where the
    Adam step is ill-conditioned by construction."""
    p = np.abs(ref_p.astype(np.float64))
    g = np.abs(ref_g.astype(np.float64))
    rms_p = np.sqrt(np.mean(p * p))
    rms_g = np.sqrt(np.mean(g * g))
    bound = tol * (p + rms_p) + 1e-30
    dg = tol * (g + rms_g)
    if opt[0] == "adamw":
        lr, eps = opt[1], opt[4]
        bound = bound + lr * np.minimum(2.0, dg / (g + eps))
    else:
        bound = bound + opt[1] * dg
    return bound


def run_case(ctx, oracle, dims, batch, act, loss, opt, init, steps, mode, tol=TOL, workload=None):
    from ferrograd_b200 import dp
    from ferrograd_b200.mlp import MLPTrainer
    tr = MLPTrainer(ctx, dims, batch, act, loss, opt, gemm_mode=mode)
    W, b = MLPTrainer.init_params(dims, init, 3)
    tr.set_params(W, b)
    state = zeros_state(W, b)
    od = dims[-1]
    gs = 1.0 / (batch * (od if loss == "mse" else 1))
    wl = workload or dict(dims=dims, batch=batch, loss=loss)
    drift = []
    for s in range(steps):
        x, t = dp.synth_batch(wl, 0, s, batch)
        tr.upload_batch(x, t)
        tr.step()
        if s == 0:
            W_prev, b_prev = [w.copy() for w in W], [v.copy() for v in b]
        ref_loss, gW, gb, out = oracle.mlp_step(dims, batch, act, W, b, x, t, loss, gs, opt, step=s + 1, state=state)
        if s == 0:
            check(tr.get_output(), out, tol, "forward output")
            got_gW, got_gb = tr.get_grads()
            for l in range(len(dims) - 1):
                check(got_gW[l], gW[l], tol, f"dW[{l}]")
                check(got_gb[l], gb[l], tol, f"db[{l}]")
            got_W, got_b = tr.get_params()
            for l in range(len(dims) - 1):
                # (1) the optimizer in isolation: the oracle's update applied to the GPU's own gradients
                for prev, g, got, name in ((W_prev[l], got_gW[l], got_W[l], "W"), (b_prev[l], got_gb[l], got_b[l], "b")):
                    p, gg = prev.copy(), g.copy()
                    if opt[0] == "adamw":
                        oracle.adamw(p, gg, np.zeros_like(p), np.zeros_like(p), *opt[1:], 1)
                    else:
                        oracle.sgd(p, gg, opt[1])
                    check(got, p, 1e-5, f"update of {name}[{l}] from the same gradients")
                # (2) end to end: the gradient tolerance propagated through the update
                for ref_p, ref_g, got, name in ((W[l], gW[l], got_W[l], "W"), (b[l], gb[l], got_b[l], "b")):
                    bound = param_bound(ref_p, ref_g, opt, tol)
                    worst = float(np.max(np.abs(got.astype(np.float64) - ref_p) / bound))
                    assert worst <= 1.0, f"updated {name}[{l}]: {worst:.3g} x the propagated bound"
        ref = ref_loss / batch if loss == "ce" else ref_loss
        drift.append(abs(tr.get_loss() - ref) / max(abs(ref), 1e-30))
    assert ctx.device_status() == 0
    return tr, W, b, drift


def test_c1_tiny_mlp_1000_steps(ctx, oracle):
    # Benchmark workload C1 (the reference's own CPU-scale case): 2 -> 16 -> 2, tanh, MSE, SGD lr 0.1, batch 64, 1000 steps.
    from ferrograd_b200 import dp
    w = dp.WORKLOADS["c1"]
    from ferrograd_b200.mlp import MLPTrainer
    dims, batch = w["dims"], w["batch"]
    tr = MLPTrainer(ctx, dims, batch, w["act"], w["loss"], w["opt"])
    W, b = MLPTrainer.init_params(dims, w["init"], w["seed"])
    tr.set_params(W, b)
    gs = 1.0 / (batch * dims[-1])
    first, last = None, None
    for s in range(1000):
        x, t = dp.synth_batch("c1", 0, s)
        tr.upload_batch(x, t)
        tr.step()
        ref_loss, gW, gb, out = oracle.mlp_step(dims, batch, "tanh", W, b, x, t, "mse", gs, w["opt"])
        if s == 0:
            got_W, got_b = tr.get_params()
            for l in range(2):
                check(got_W[l], W[l], 1e-5, f"W[{l}] after step 1")
                check(got_b[l], b[l], 1e-5, f"b[{l}] after step 1")
            first = ref_loss
        last = ref_loss
    got_W, got_b = tr.get_params()
    # after 1000 steps the two f32 trajectories may differ by accumulated ulps of tanh; stated band: 1e-3
    for l in range(2):
        check(got_W[l], W[l], 1e-3, f"W[{l}] after step 1000")
    assert abs(tr.get_loss() - last) <= 1e-3 * abs(last) + 1e-6
    assert last < first      # it trains


@pytest.mark.parametrize("mode", ["simt", "3xtf32", "tf32_bf16x2"])
def test_c4_reduced(ctx, oracle, mode):
    # Benchmark workload C4 at reduced width: GELU hidden layers, softmax-CE, AdamW.
    opt = ("adamw", 1e-3, 0.9, 0.999, 1e-8, 0.01)
    tr, W, b, drift = run_case(ctx, oracle, [784, 256, 320, 10], 512, "gelu", "ce", opt, "he_normal", 5, mode)
    assert max(drift) < 1e-4, f"loss drift over 5 steps: {drift}"


@pytest.mark.parametrize("mode", ["simt", "3xtf32", "tf32_bf16x2"])
def test_c5_reduced(ctx, oracle, mode):
    # Benchmark workload C5 at reduced width/depth: tanh, MSE, AdamW.
    opt = ("adamw", 1e-3, 0.9, 0.999, 1e-8, 0.01)
    tr, W, b, drift = run_case(ctx, oracle, [512] * 5, 256, "tanh", "mse", opt, "normal_fan_in", 3, mode)
    assert max(drift) < 1e-4, f"loss drift over 3 steps: {drift}"


def test_relu_sgd_odd_shapes(ctx, oracle):
    tr, W, b, drift = run_case(ctx, oracle, [70, 130, 33, 7], 200, "relu", "ce", ("sgd", 0.05), "he_normal", 3, "3xtf32")
    assert max(drift) < 1e-4


def test_c4_full_size_one_step(ctx, oracle):
    # Benchmark workload C4 at its real size: 784 -> 4096 -> 4096 -> 10, batch 4096, one step.
    from ferrograd_b200 import dp
    w = dp.WORKLOADS["c4"]
    tr, W, b, drift = run_case(ctx, oracle, w["dims"], w["batch"], w["act"], w["loss"], w["opt"], w["init"], 1, "auto")
    assert drift[0] < 1e-5


def test_c4_full_size_one_step_through_the_graph_api(ctx, oracle):
    # The same workload through the reference's loop (dispatch_forward / loss / backward / optim), which is what the
    # benchmark times: the loss is unreduced there, so the oracle runs with a gradient scale of one.
    from ferrograd_b200 import dp
    from ferrograd_b200.mlp import GraphMLP, MLPTrainer
    w = dp.WORKLOADS["c4"]
    dims, batch, opt = w["dims"], w["batch"], w["opt"]
    net = GraphMLP(ctx, dims, batch, w["act"], w["loss"], opt)
    W, b = MLPTrainer.init_params(dims, w["init"], 3)
    net.set_params(W, b)
    x, t = dp.synth_batch("c4", 0, 0)
    net.upload_batch(x, t)
    net.step()
    ctx.sync()
    assert ctx.device_status() == 0
    state = zeros_state(W, b)
    loss_sum, gW, gb, out = oracle.mlp_step(dims, batch, w["act"], W, b, x, t, "ce", 1.0, opt, step=1, state=state)
    check(net.get_output(), oracle.softmax_fwd(out), TOL, "forward output (probabilities)")
    assert abs(net.get_loss() - loss_sum) <= 1e-5 * abs(loss_sum)
    got_W, got_b = net.get_params()
    for l in range(len(dims) - 1):
        for ref_p, ref_g, got, name in ((W[l], gW[l], got_W[l], "W"), (b[l], gb[l], got_b[l], "b")):
            bound = param_bound(ref_p, ref_g, opt, TOL)
            worst = float(np.max(np.abs(got.astype(np.float64) - ref_p) / bound))
            assert worst <= 1.0, f"updated {name}[{l}]: {worst:.3g} x the propagated bound"
    net.destroy()


def test_c5_full_size_one_step(ctx, oracle):
    # Benchmark workload C5 at its real size: eight 8192 x 8192 layers, tanh, MSE, AdamW, batch 2048, one step
    # (6.6 TFLOP in the oracle: about a minute of host time).
    from ferrograd_b200 import dp
    w = dp.WORKLOADS["c5"]
    tr, W, b, drift = run_case(ctx, oracle, w["dims"], w["batch"], w["act"], w["loss"], w["opt"], w["init"], 1, "auto")
    assert drift[0] < 1e-5
    tr.destroy()


def test_plan_replay_matches_eager(ctx, oracle):
    from ferrograd_b200 import dp
    from ferrograd_b200.mlp import MLPTrainer
    dims, batch = [96, 256, 10], 256
    opt = ("adamw", 1e-3, 0.9, 0.999, 1e-8, 0.01)
    W, b = MLPTrainer.init_params(dims, "he_normal", 5)
    x, t = dp.synth_batch(dict(dims=dims, batch=batch, loss="ce"), 0, 0, batch)
    results = []
    for use_plan in (False, True):
        tr = MLPTrainer(ctx, dims, batch, "gelu", "ce", opt, gemm_mode="3xtf32")
        tr.set_params(W, b)
        tr.upload_batch(x, t)
        tr.step()                      # eager step 1 (sizes the scratch arena)
        if use_plan:
            tr.build_plan()
            for _ in range(3):
                tr.step_plan()
        else:
            for _ in range(3):
                tr.step()
        ctx.sync()
        results.append(tr.get_params())
    for l in range(2):
        assert np.array_equal(results[0][0][l], results[1][0][l])   # same kernels, same order: identical bits
        assert np.array_equal(results[0][1][l], results[1][1][l])
