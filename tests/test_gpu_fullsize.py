"""The softmax-CE (8192 x 32000) and GEMM (8192^3) benchmark workloads at their full sizes, checked through size-independent
properties plus sampled rows against the CPU oracle; and the edge cases of the C ABI (empty and
degenerate inputs)."""
import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from ferrograd_b200 import GpuContext
    c = GpuContext(0)
    yield c
    c.sync()
    c.destroy()


def rng(seed):
    return np.random.Generator(np.random.Philox(seed))


def test_c2_softmax_ce_full_size(ctx, oracle):
    # f32 logits [8192, 32000] ~ N(0, 2.0), labels uniform in [0, 32000)
    rows, cols = 8192, 32000
    x = rng(1).standard_normal((rows, cols), np.float32)
    x *= np.float32(2.0)
    labels = rng(2).integers(0, cols, rows).astype(np.uint32)
    dx = ctx.init_tensor_f32(x.shape, x)
    dlab = ctx.init_tensor_u32(labels.shape, labels)
    dlog, lrow, lmean = ctx.new_tensor((rows, cols)), ctx.new_tensor((rows,)), ctx.new_tensor((1,))
    am = ctx.new_tensor((rows,), np.uint32)
    scale = 1.0 / rows
    ctx.softmax_ce(dx, dlab, rows, cols, grad_scale=scale, loss_row=lrow, loss_mean=lmean, dlogits=dlog, argmax=am)
    ctx.sync()
    assert ctx.device_status() == 0
    g = ctx.to_numpy(dlog)
    loss = ctx.to_numpy(lrow)
    # properties: every gradient row sums to zero (sum p - 1), only the label entry is negative, losses are
    # positive, the mean is the mean of the rows, the arg-max is the arg-max (index output: bit-exact)
    assert np.abs(g.sum(axis=1, dtype=np.float64)).max() <= 1e-5 * scale
    assert (g[np.arange(rows), labels] < 0).all() and (g.min(axis=1) == g[np.arange(rows), labels]).all()
    assert (loss > 0).all() and np.isfinite(loss).all()
    assert abs(float(ctx.to_numpy(lmean)[0]) - float(loss.astype(np.float64).mean())) <= 1e-5 * float(loss.mean())
    assert np.array_equal(ctx.to_numpy(am), x.argmax(axis=1).astype(np.uint32))
    # sampled rows against the oracle
    pick = rng(3).choice(rows, 48, replace=False)
    ref = oracle.softmax_ce(x[pick], labels[pick], grad_scale=scale)
    ok, worst = rel_err_ok(g[pick], ref["dlogits"], 1e-5)
    assert ok, f"dlogits rows: {worst:.3g} x 1e-5"
    ok, worst = rel_err_ok(loss[pick], ref["loss_row"], 1e-5)
    assert ok, f"loss rows: {worst:.3g} x 1e-5"


def test_c3_gemm_full_size(ctx, oracle):
    # C = ReLU(A·B + bias), 8192^3, all N(0, 1/sqrt(8192)); backward with dC ~ N(0, 1)
    N = 8192
    s = np.float32(1.0 / np.sqrt(N))
    A = rng(3).standard_normal((N, N), np.float32) * s
    B = rng(4).standard_normal((N, N), np.float32) * s
    bias = rng(5).standard_normal(N, np.float32) * s
    dC = rng(6).standard_normal((N, N), np.float32)
    dA_, dB_, dbias_ = ctx.init_tensor_f32(A.shape, A), ctx.init_tensor_f32(B.shape, B), ctx.init_tensor_f32((N,), bias)
    dCd = ctx.init_tensor_f32(dC.shape, dC)
    Cd, Pd = ctx.new_tensor((N, N)), ctx.new_tensor((N, N))
    ctx.gemm(dA_, dB_, Cd, N, N, N, bias=dbias_, act="relu", preact_out=Pd)
    gA, gB, gb = ctx.new_tensor((N, N)), ctx.new_tensor((N, N)), ctx.new_tensor((N,))
    ctx.gemm_bwd(dA_, dB_, dCd, N, N, N, act="relu", saved=Cd, dA=gA, dB=gB, dbias=gb)
    ctx.sync()
    assert ctx.device_status() == 0
    C, P = ctx.to_numpy(Cd), ctx.to_numpy(Pd)
    # properties: ReLU of the stored pre-activation, exactly
    assert np.array_equal(C, np.maximum(P, 0.0))
    # sampled rows of the forward against the f64-accumulating oracle
    pick = np.sort(rng(7).choice(N, 40, replace=False))
    pre_ref = oracle.gemm(A[pick], B, f64=True) + bias
    ok, worst = rel_err_ok(P[pick], pre_ref, 1e-4)
    assert ok, f"pre-activation rows: {worst:.3g} x 1e-4"
    clear = np.abs(pre_ref) > 1e-4 * np.sqrt(np.mean(pre_ref ** 2))
    assert np.array_equal((C[pick] > 0)[clear], (pre_ref > 0)[clear])       # the mask, where it is decidable
    # backward: dZ = dC * mask (the GPU's own mask), dA rows and dB rows against the oracle
    dZ = dC * (C > 0)
    ok, worst = rel_err_ok(ctx.to_numpy(gA)[pick], oracle.gemm(dZ[pick], B, transB=True, f64=True), 1e-4)
    assert ok, f"dA rows: {worst:.3g} x 1e-4"
    ok, worst = rel_err_ok(ctx.to_numpy(gB)[pick], oracle.gemm(np.ascontiguousarray(A[:, pick]), dZ, transA=True, f64=True), 1e-4)
    assert ok, f"dB rows: {worst:.3g} x 1e-4"
    ok, worst = rel_err_ok(ctx.to_numpy(gb), dZ.sum(axis=0, dtype=np.float64), 1e-4)
    assert ok, f"dbias: {worst:.3g} x 1e-4"
    # linearity: scaling A by a power of two scales every split plane exactly, so the result is exactly doubled
    ctx.upload(dA_, A * np.float32(2.0))
    C2 = ctx.new_tensor((N, N))
    ctx.gemm(dA_, dB_, C2, N, N, N)
    ctx.upload(dA_, A)
    C1 = ctx.new_tensor((N, N))
    ctx.gemm(dA_, dB_, C1, N, N, N)
    assert np.array_equal(ctx.to_numpy(C2), np.float32(2.0) * ctx.to_numpy(C1))


def test_adamw_c5_parameter_count_constant_fill(ctx, oracle):
    # 536,936,448 parameters (config 5): constant inputs, so every element must equal the scalar update
    n = 8 * (8192 * 8192 + 8192)
    w, g, m, v = (ctx.new_tensor((n,)) for _ in range(4))
    fills = (0.5, -0.25, 0.0, 0.0)
    one = np.empty(1 << 20, np.float32)
    for t, val in zip((w, g, m, v), fills):
        if val == 0.0:
            ctx.memset_zero(t)
        else:
            one[:] = val
            for off in range(0, n, one.size):
                k = min(one.size, n - off)
                ctx.upload(t, one[:k], dst_off=off * 4)
    ctx.adamw_step(w, g, m, v, n, 1e-3, 0.9, 0.999, 1e-8, 0.01, step=1, zero_grad=False)
    ref = [np.full(4, f, np.float32) for f in fills]
    oracle.adamw(*ref, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1, zero_grad=False)
    out = np.empty(1 << 20, np.float32)
    for t, r in zip((w, m, v), (ref[0], ref[2], ref[3])):
        for off in (0, (n // 2) & ~3, n - out.size):          # head, middle, tail (the tail covers the last element)
            ctx.download(t, out, src_off=off * 4)
            assert (out == out[0]).all() and abs(float(out[0]) - float(r[0])) <= 1e-6 * abs(float(r[0])) + 1e-12


def test_empty_and_degenerate_inputs(ctx, oracle):
    t = ctx.new_tensor((16,), zeroed=True)
    lab = ctx.init_tensor_u32((4,), np.array([0, 0, 0, 0], np.uint32))
    before = ctx.launch_count()
    ctx.sgd_step(t, t, 0, 0.1)
    ctx.adamw_step(t, t, t, t, 0, 1e-3, 0.9, 0.999, 1e-8, 0.0, step=1)
    ctx.softmax_fwd(t, t, 0, 4)
    ctx.softmax_bwd(t, t, t, 0, 4)
    ctx.softmax_ce(t, lab, 0, 4, dlogits=t)
    ctx.act_bwd(t, t, t, 0, "tanh")
    ctx.bias_act_fwd(t, None, "relu", t, 0, 4)
    ctx.sync()
    assert ctx.launch_count() == before                  # nothing to do, nothing launched
    # a single column: the softmax is 1, its gradient 0, the loss 0
    x = rng(1).standard_normal((5, 1), np.float32)
    y, dlog, lrow = ctx.new_tensor((5, 1)), ctx.new_tensor((5, 1)), ctx.new_tensor((5,))
    ctx.softmax_fwd(ctx.init_tensor_f32(x.shape, x), y, 5, 1)
    ctx.softmax_ce(ctx.init_tensor_f32(x.shape, x), ctx.init_tensor_u32((5,), np.zeros(5, np.uint32)), 5, 1, dlogits=dlog,
                   loss_row=lrow)
    assert (ctx.to_numpy(y) == 1.0).all() and (ctx.to_numpy(dlog) == 0.0).all() and (ctx.to_numpy(lrow) == 0.0).all()
    # a label outside [0, cols) contributes no one-hot and no loss, as in the oracle
    x = rng(2).standard_normal((3, 7), np.float32)
    labels = np.array([2, 99, 6], np.uint32)
    dlog, lrow = ctx.new_tensor((3, 7)), ctx.new_tensor((3,))
    ctx.softmax_ce(ctx.init_tensor_f32(x.shape, x), ctx.init_tensor_u32((3,), labels), 3, 7, dlogits=dlog, loss_row=lrow)
    ref = oracle.softmax_ce(x, labels)
    ok, _ = rel_err_ok(ctx.to_numpy(dlog), ref["dlogits"], 1e-5)
    assert ok and ctx.to_numpy(lrow)[1] == 0.0
    # K = 1 and a single output element through both GEMM paths
    for mode in ("simt", "3xtf32", "tf32_bf16x2"):
        a, b = np.float32([[1.5], [2.0], [-3.0]]), np.float32([[2.0, 0.5]])
        c = ctx.new_tensor((3, 2))
        ctx.gemm(ctx.init_tensor_f32(a.shape, a), ctx.init_tensor_f32(b.shape, b), c, 3, 2, 1, mode=mode)
        assert np.array_equal(ctx.to_numpy(c), a @ b)
