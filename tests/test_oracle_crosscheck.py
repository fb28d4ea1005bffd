"""Cross-checks of the CPU oracle against independent float64 formulas on random inputs.

The reference's own tests pin the oracle only at constant-filled tensors
(tests/test_oracle_golden.py), which cannot see a transposition, an index or a
reduction-order error.  Here every oracle function is compared with a numpy float64
restatement of the cited definition on seeded random data, gradients are checked
against central differences, and each switch that reproduces a deviation of the
reference (REF_QUIRK_*) is exercised with values derived by hand from the lines it cites.
Tolerance: f32 arithmetic against float64, 1e-5 relative to |ref| + rms(ref) unless stated.
"""
import numpy as np
import pytest

from conftest import rel_err_ok

A_GELU, B_GELU = 0.044715, 0.7978846      # crates/ferrograd-nn/src/op/unary.rs:493-494


def rng(seed):
    return np.random.Generator(np.random.Philox(seed))


def check(x, ref, tol, what):
    ok, worst = rel_err_ok(x, ref, tol)
    assert ok, f"{what}: worst error ratio {worst:.3g} x tolerance {tol}"


def softmax64(x):
    x = np.asarray(x, np.float64)
    e = np.exp(x - x.max(axis=1, keepdims=True))
    return e / e.sum(axis=1, keepdims=True)


def act64(name, z):
    z = np.asarray(z, np.float64)
    if name == "relu":
        return np.maximum(z, 0.0)
    if name == "tanh":
        return np.tanh(z)
    if name == "gelu":
        return 0.5 * z * (1.0 + np.tanh(B_GELU * (z + A_GELU * z ** 3)))
    return z


def act_grad64(name, z):
    """d act / d z at pre-activation z."""
    z = np.asarray(z, np.float64)
    if name == "relu":
        return (z > 0).astype(np.float64)
    if name == "tanh":
        return 1.0 - np.tanh(z) ** 2
    if name == "gelu":
        t = np.tanh(B_GELU * (z + A_GELU * z ** 3))
        return 0.5 * (1.0 + t) + 0.5 * z * (1.0 - t * t) * B_GELU * (1.0 + 3.0 * A_GELU * z * z)
    return np.ones_like(z)


# ------------------------------------------------------------------ matmul
@pytest.mark.parametrize("tA,tB", [(False, False), (True, False), (False, True), (True, True)])
def test_gemm_against_float64_matmul(oracle, tA, tB):
    # distinct M, N, K and non-symmetric data: a swapped index or a missed transposition cannot cancel
    M, N, K = 37, 53, 29
    r = rng(1)
    A = r.standard_normal((K, M) if tA else (M, K), np.float32)
    B = r.standard_normal((N, K) if tB else (K, N), np.float32)
    ref = (A.T if tA else A).astype(np.float64) @ (B.T if tB else B).astype(np.float64)
    check(oracle.gemm(A, B, transA=tA, transB=tB), ref, 1e-5, "f32 fma chain")
    check(oracle.gemm(A, B, transA=tA, transB=tB, f64=True), ref, 2e-7, "f64 accumulation")


def test_colsum_and_bias_broadcast(oracle):
    r = rng(2)
    z, bias = r.standard_normal((19, 23), np.float32), r.standard_normal(23, np.float32)
    check(oracle.colsum(z), z.astype(np.float64).sum(axis=0), 1e-6, "column sums")
    for name in ("none", "relu", "tanh", "gelu"):
        y, pre = oracle.bias_act_fwd(z, bias, name)
        check(pre, z.astype(np.float64) + bias, 1e-6, f"{name} pre-activation (bias over columns)")
        check(y, act64(name, z.astype(np.float64) + bias), 1e-5, f"{name} forward")


# ------------------------------------------------------------------ activations backward
@pytest.mark.parametrize("name", ["relu", "tanh", "gelu"])
def test_activation_backward_against_formula_and_differences(oracle, name):
    r = rng(3)
    z = (1.5 * r.standard_normal(4000, np.float32)).astype(np.float32)
    z = z[np.abs(z) > 1e-3]                       # ReLU is not differentiable at 0
    dy = r.standard_normal(z.size, np.float32)
    y = act64(name, z)
    saved = z if name == "gelu" else y.astype(np.float32)     # GELU saves the pre-activation, the others the output
    got = oracle.act_bwd(dy, saved, name)
    check(got, dy * act_grad64(name, z), 2e-5, f"{name} backward vs formula")
    h = 1e-6
    fd = (act64(name, z.astype(np.float64) + h) - act64(name, z.astype(np.float64) - h)) / (2 * h)
    check(got, dy * fd, 1e-4, f"{name} backward vs central differences")


# ------------------------------------------------------------------ softmax and the losses
@pytest.mark.parametrize("rows,cols", [(5, 7), (3, 300), (2, 1000)])
def test_softmax_forward_backward(oracle, rows, cols):
    r = rng(4 + cols)
    x = (2.0 * r.standard_normal((rows, cols), np.float32)).astype(np.float32)
    y64 = softmax64(x)
    y = oracle.softmax_fwd(x)
    check(y, y64, 1e-5, "softmax forward")
    dy = r.standard_normal((rows, cols), np.float32)
    ref = y64 * (dy - (dy * y64).sum(axis=1, keepdims=True))
    check(oracle.softmax_bwd(y, dy), ref, 1e-5, "softmax backward, non-zero upstream gradient")
    base = r.standard_normal((rows, cols), np.float32)
    check(oracle.softmax_bwd(y, dy, dx=base), base + ref, 1e-5, "softmax backward, accumulate form")


def test_softmax_cross_entropy(oracle):
    rows, cols = 11, 40
    r = rng(6)
    x = (2.0 * r.standard_normal((rows, cols), np.float32)).astype(np.float32)
    labels = r.integers(0, cols, rows).astype(np.uint32)
    p = softmax64(x)
    onehot = np.zeros((rows, cols))
    onehot[np.arange(rows), labels] = 1.0
    out = oracle.softmax_ce(x, labels, grad_scale=0.25, want_probs=True)
    loss_row = -np.log(p[np.arange(rows), labels])
    check(out["loss_row"], loss_row, 1e-5, "per-row loss")
    assert abs(out["loss_mean"] - loss_row.mean()) <= 1e-5 * abs(loss_row.mean())
    check(out["probs"], p, 1e-5, "probabilities")
    check(out["dlogits"], 0.25 * (p - onehot), 1e-5, "dlogits = (p - onehot) * scale")
    assert np.array_equal(out["argmax"], x.argmax(axis=1).astype(np.uint32))
    # the reference's unfused per-element form (loss/basic_loss.rs:91-133): label indexed by ROW, compared with COLUMN
    loss, grad = oracle.ce_loss_grad(p.astype(np.float32), labels)
    check(loss, -np.log(p) * onehot, 1e-5, "elementwise loss")
    check(grad, p - onehot, 1e-5, "elementwise gradient")
    # d(mean loss)/dlogits by central differences of the float64 loss
    h, fd = 1e-6, np.zeros((rows, cols))
    for rr in range(rows):
        for cc in range(0, cols, 7):
            xp, xm = x.astype(np.float64), x.astype(np.float64)
            xp[rr, cc] += h
            xm[rr, cc] -= h
            fd[rr, cc] = (-np.log(softmax64(xp)[rr, labels[rr]]) + np.log(softmax64(xm)[rr, labels[rr]])) / (2 * h)
    got = oracle.softmax_ce(x, labels, grad_scale=1.0)["dlogits"]
    check(got[:, ::7], fd[:, ::7], 1e-4, "dlogits vs central differences")


def test_mse_and_bce(oracle):
    r = rng(7)
    p, t = r.standard_normal(1000, np.float32), r.standard_normal(1000, np.float32)
    loss, loss_sum, grad = oracle.mse(p, t, grad_scale=0.5)
    d = p.astype(np.float64) - t
    check(loss, d * d, 1e-6, "MSE loss")          # loss/basic_loss.rs:3-27, no 1/N
    check(grad, 2.0 * d * 0.5, 1e-6, "MSE gradient")
    assert abs(loss_sum - (d * d).sum()) <= 1e-5 * (d * d).sum()
    pp = r.uniform(0.02, 0.98, 1000).astype(np.float32)
    tt = (r.random(1000) > 0.5).astype(np.float32)
    loss, _, grad = oracle.bce(pp, tt)
    check(loss, -(tt * np.log(pp.astype(np.float64)) + (1 - tt) * np.log(1.0 - pp)), 1e-5, "BCE loss")
    check(grad, pp.astype(np.float64) - tt, 1e-6, "BCE gradient")


# ------------------------------------------------------------------ optimizers
def test_sgd_and_adamw_three_steps(oracle):
    n = 500
    r = rng(8)
    w = r.standard_normal(n, np.float32)
    w64, m64, v64 = w.astype(np.float64), np.zeros(n), np.zeros(n)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    # the hyper-parameters are f32 inputs: the float64 restatement starts from their f32 values
    lr, b1, b2, eps, wd, gs = (float(np.float32(h)) for h in (1e-2, 0.9, 0.999, 1e-8, 0.01, 0.5))
    for step in (1, 2, 3):
        g = r.standard_normal(n, np.float32)
        g64 = g.astype(np.float64) * gs
        m64 = b1 * m64 + (1 - b1) * g64
        v64 = b2 * v64 + (1 - b2) * g64 * g64
        mh, vh = m64 / (1 - b1 ** step), v64 / (1 - b2 ** step)
        w64 = w64 - lr * (mh / (np.sqrt(vh) + eps) + wd * w64)       # decoupled decay, bias-corrected
        oracle.adamw(w, g, m, v, lr, b1, b2, eps, wd, step, grad_scale=gs)
        assert (g == 0).all()
    check(w, w64, 1e-5, "AdamW weights after 3 steps")
    check(m, m64, 1e-5, "AdamW first moment")
    check(v, v64, 1e-5, "AdamW second moment")
    w2, g2 = r.standard_normal(n, np.float32), r.standard_normal(n, np.float32)
    ref = w2.astype(np.float64) - 0.1 * (g2.astype(np.float64) * 0.5)
    oracle.sgd(w2, g2, 0.1, grad_scale=0.5)
    check(w2, ref, 1e-6, "SGD")                                       # optim/basic_optim.rs:3-31
    assert (g2 == 0).all()


# ------------------------------------------------------------------ elementwise chains
def chain64(instrs, inputs):
    """float64 interpreter of the chain encoding (instruction i defines value i)."""
    v = []
    for op, a, b, imm in instrs:
        if op == "input":
            v.append(np.asarray(inputs[a], np.float64))
        elif op == "const":
            v.append(np.full_like(np.asarray(inputs[0], np.float64), imm))
        elif op == "add":
            v.append(v[a] + v[b])
        elif op == "sub":
            v.append(v[a] - v[b])
        elif op == "mul":
            v.append(v[a] * v[b])
        elif op == "div":
            v.append(v[a] / v[b])
        elif op == "neg":
            v.append(-v[a])
        elif op == "abs":
            v.append(np.abs(v[a]))
        elif op == "exp":
            v.append(np.exp(v[a]))
        elif op == "log":
            v.append(np.log(v[a]))
        elif op == "elu":
            v.append(np.where(v[a] > 0, v[a], np.exp(v[a]) - 1.0))
        else:
            v.append(act64(op, v[a]))
    return v[-1]


def test_chain_backward_against_central_differences(oracle):
    n = 64
    r = rng(9)
    ins = [r.uniform(0.5, 2.0, n).astype(np.float32) for _ in range(3)]
    prog = [("input", 0, 0, 0.0), ("input", 1, 0, 0.0), ("input", 2, 0, 0.0), ("mul", 0, 1, 0.0),
            ("const", 0, 0, 0.75), ("div", 3, 2, 0.0), ("sub", 5, 4, 0.0), ("tanh", 6, 0, 0.0),
            ("exp", 7, 0, 0.0), ("log", 0, 0, 0.0), ("add", 8, 9, 0.0), ("gelu", 10, 0, 0.0),
            ("neg", 11, 0, 0.0), ("abs", 12, 0, 0.0), ("elu", 6, 0, 0.0), ("add", 13, 14, 0.0)]
    out, _ = oracle.eltwise_fwd(prog, ins)
    check(out, chain64(prog, ins), 1e-5, "chain forward")
    seed = r.standard_normal(n, np.float32)
    grads = oracle.eltwise_bwd(prog, ins, seed)
    h = 1e-6
    for k in range(3):
        plus = [a.astype(np.float64) + (h if j == k else 0.0) for j, a in enumerate(ins)]
        minus = [a.astype(np.float64) - (h if j == k else 0.0) for j, a in enumerate(ins)]
        fd = seed * (chain64(prog, plus) - chain64(prog, minus)) / (2 * h)
        check(grads[k], fd, 1e-4, f"chain gradient of input {k}")


# ------------------------------------------------------------------ a whole training step
def mlp64(dims, act, W, b, x, target, loss_kind, gs):
    L = len(dims) - 1
    a, pre = [np.asarray(x, np.float64)], []
    for l in range(L):
        z = a[-1] @ W[l].astype(np.float64) + b[l]
        pre.append(z)
        a.append(act64(act, z) if l < L - 1 else z)
    if loss_kind == "ce":
        p = softmax64(a[-1])
        onehot = np.zeros_like(p)
        onehot[np.arange(p.shape[0]), target] = 1.0
        loss = -np.log(p[np.arange(p.shape[0]), target]).sum()
        dz = (p - onehot) * gs
    else:
        d = a[-1] - target
        loss = (d * d).sum()
        dz = 2.0 * d * gs
    gW, gb = [None] * L, [None] * L
    for l in range(L - 1, -1, -1):
        gW[l] = a[l].T @ dz
        gb[l] = dz.sum(axis=0)
        if l > 0:
            dz = (dz @ W[l].astype(np.float64).T) * act_grad64(act, pre[l - 1])
    return loss, gW, gb, a[-1]


@pytest.mark.parametrize("act,loss_kind", [("gelu", "ce"), ("tanh", "mse"), ("relu", "ce")])
def test_mlp_step_against_float64_network(oracle, act, loss_kind):
    dims, batch = [13, 29, 17, 7], 24
    r = rng(10)
    W = [(r.standard_normal((dims[l], dims[l + 1])) * 0.4).astype(np.float32) for l in range(3)]
    b = [(r.standard_normal(dims[l + 1]) * 0.1).astype(np.float32) for l in range(3)]
    x = r.standard_normal((batch, dims[0]), np.float32)
    target = r.integers(0, dims[-1], batch).astype(np.uint32) if loss_kind == "ce" \
        else r.standard_normal((batch, dims[-1]), np.float32)
    gs = 1.0 / batch
    loss64, gW64, gb64, out64 = mlp64(dims, act, W, b, x, target, loss_kind, gs)
    W0 = [w.copy() for w in W]
    opt = ("adamw", 1e-2, 0.9, 0.999, 1e-8, 0.01)
    state = {k: [np.zeros_like(a) for a in (W if k[1] == "W" else b)] for k in ("mW", "vW", "mb", "vb")}
    loss, gW, gb, out = oracle.mlp_step(dims, batch, act, W, b, x, target, loss_kind, gs, opt, step=1, state=state)
    assert abs(loss - loss64) <= 1e-5 * abs(loss64)
    check(out, out64, 1e-5, "network output")
    for l in range(3):
        check(gW[l], gW64[l], 2e-5, f"dW[{l}] (x^T dZ: a transposition error would show here)")
        check(gb[l], gb64[l], 2e-5, f"db[{l}]")
        # first AdamW step from zero moments: w - lr*(g/(|g| + eps') + wd*w), on the oracle's own gradient
        g = gW[l].astype(np.float64)
        mh, vh = g, g * g
        ref = W0[l] - 1e-2 * (mh / (np.sqrt(vh) + 1e-8) + 0.01 * W0[l].astype(np.float64))
        check(W[l], ref, 1e-5, f"updated W[{l}]")


# ------------------------------------------------------------------ switches that reproduce the reference's deviations
def test_quirk_relu_mask_is_ge_zero_on_the_saved_output(oracle):
    # op/unary.rs:453-472: the backward condition is `saved >= 0` (Op::Ge) and the saved tensor is the ReLU's own
    # output, which is never negative -- so with the switch every element passes the gradient through.
    z = np.array([-2.0, -0.5, 0.0, 0.5, 3.0], np.float32)
    y = np.maximum(z, 0.0).astype(np.float32)         # what the reference saves
    dy = np.array([5.0, 7.0, 9.0, 11.0, 13.0], np.float32)
    assert np.array_equal(oracle.act_bwd(dy, y, "relu"), np.array([0, 0, 0, 11, 13], np.float32))
    assert np.array_equal(oracle.act_bwd(dy, y, "relu", quirks=oracle.QUIRK_RELU_MASK_GE0), dy)
    # on a tensor that does contain negatives the switch is exactly `>= 0`
    assert np.array_equal(oracle.act_bwd(dy, z, "relu", quirks=oracle.QUIRK_RELU_MASK_GE0),
                          np.array([0, 0, 9, 11, 13], np.float32))


def test_quirk_gelu_backward_uses_tanh_where_x_is_meant(oracle):
    # op/unary.rs:588-714 computes 0.5*((1 + t) + (1 - t^2) * X * b*(1 + 3a*X^2)) with X bound to t = tanh(u)
    # instead of the pre-activation x.
    x = np.array([-1.5, -0.3, 0.2, 0.9, 2.5], np.float32)
    dy = np.ones_like(x)
    t = np.tanh(B_GELU * (x.astype(np.float64) + A_GELU * x.astype(np.float64) ** 3))
    quirk = 0.5 * ((1 + t) + (1 - t * t) * t * B_GELU * (1 + 3 * A_GELU * t * t))
    check(oracle.act_bwd(dy, x, "gelu", quirks=oracle.QUIRK_GELU_BWD_T), quirk, 1e-5, "GELU backward, reference form")
    check(oracle.act_bwd(dy, x, "gelu"), act_grad64("gelu", x), 1e-5, "GELU backward, standard form")
    assert np.abs(quirk - act_grad64("gelu", x)).max() > 1e-2          # the two settings really differ


def test_quirk_softmax_backward_touches_every_256th_column(oracle):
    # op/softmax.rs:601 resets the column counter to 0 for every thread, and the loop then strides by the block
    # size 256: only columns 0, 256, 512, ... receive a gradient.
    rows, cols = 2, 600
    r = rng(11)
    y = softmax64(r.standard_normal((rows, cols))).astype(np.float32)
    dy = r.standard_normal((rows, cols), np.float32)
    full = oracle.softmax_bwd(y, dy)
    base = np.full((rows, cols), 3.0, np.float32)
    got = oracle.softmax_bwd(y, dy, dx=base, quirks=oracle.QUIRK_SOFTMAX_BWD_COL0)
    touched = np.zeros(cols, bool)
    touched[::256] = True
    check(got[:, touched], 3.0 + full[:, touched].astype(np.float64), 1e-5, "touched columns")
    assert (got[:, ~touched] == 3.0).all()


def test_quirk_ce_gradient_goes_through_the_softmax_backward_again(oracle):
    # dispatch/mod.rs:713-718 binds the loss kernel's gradient to `seed`, the upstream gradient of the graph's last
    # node; when that node is a softmax, backward multiplies p - onehot by the softmax Jacobian once more:
    # dlogits = p * ((p - onehot) - sum_c p_c*(p_c - onehot_c)).
    rows, cols = 4, 9
    r = rng(12)
    x = r.standard_normal((rows, cols), np.float32)
    labels = r.integers(0, cols, rows).astype(np.uint32)
    p = softmax64(x)
    onehot = np.zeros((rows, cols))
    onehot[np.arange(rows), labels] = 1.0
    seed = p - onehot
    twice = p * (seed - (seed * p).sum(axis=1, keepdims=True))
    got = oracle.softmax_ce(x, labels, quirks=oracle.QUIRK_CE_THROUGH_SOFTMAX)
    check(got["dlogits"], twice, 1e-5, "reference order")
    check(oracle.softmax_ce(x, labels)["dlogits"], seed, 1e-5, "standard order")
    assert np.abs(twice - seed).max() > 1e-2


def test_quirk_bce_reference_formula(oracle):
    # loss/basic_loss.rs:47-51 builds (1 - target) where (1 - pred) is meant, and :75-79 subtracts the two terms
    # the other way round: loss_ref = (1 - t)*log(1 - t) ... is not finite for t in {0, 1}; compare on soft targets.
    r = rng(13)
    p = r.uniform(0.1, 0.9, 50).astype(np.float32)
    t = r.uniform(0.1, 0.9, 50).astype(np.float32)
    std_loss, _, std_grad = oracle.bce(p, t)
    ref_loss, _, ref_grad = oracle.bce(p, t, reference_formula=True)
    check(std_loss, -(t * np.log(p.astype(np.float64)) + (1 - t) * np.log(1.0 - p)), 1e-5, "standard BCE")
    assert np.abs(ref_loss - std_loss).max() > 1e-3
    check(ref_grad, std_grad, 1e-7, "the gradient expression p - t is the same in both")
