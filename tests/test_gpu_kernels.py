"""GPU parity tests: every CUDA entry point, called through the C ABI, against the CPU
oracle on the same seeded inputs.  Tolerances: 1e-5 for elementwise and softmax work,
1e-4 for GEMM-bearing results, both as |x - ref| <= tol * (|ref| + rms(ref)); integer
outputs and the exact SIMT GEMM are compared bit for bit."""
import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu

TOL_EW = 1e-5
TOL_GEMM = 1e-4


@pytest.fixture(scope="module")
def ctx():
    from ferrograd_b200 import GpuContext
    c = GpuContext(0)
    yield c
    c.sync()
    c.destroy()


def rng(seed):
    return np.random.Generator(np.random.Philox(seed))


def up(ctx, a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        return ctx.init_tensor_u32(a.shape, a)
    return ctx.init_tensor_f32(a.shape, a)


def check(x, ref, tol, what=""):
    ok, worst = rel_err_ok(x, ref, tol)
    assert ok, f"{what}: worst error ratio {worst:.3g} x tolerance {tol}"


# ---------------------------------------------------------------- optimizers
def test_sgd_reference_constants(ctx):
    # crates/ferrograd/tests/optim.rs:10-104
    f32 = np.float32
    for wv, gv, expect in ((3.0, 2.0, f32(3.0) - f32(2e-3)), (2.0, 3.0, f32(2.0) - f32(3e-3)),
                           (1.0, 1.0, f32(1.0) - f32(1e-3))):
        w, g = up(ctx, np.full(1024, wv, f32)), up(ctx, np.full(1024, gv, f32))
        ctx.sgd_step(w, g, 1024, float(f32(1e-3)))
        assert (ctx.to_numpy(w) == expect).all()
        assert (ctx.to_numpy(g) == 0.0).all()


@pytest.mark.parametrize("n", [1, 3, 1000, 4097, 1 << 20])
def test_sgd_vs_oracle(ctx, oracle, n):
    r = rng(10 + n)
    w, g = r.standard_normal(n, np.float32), r.standard_normal(n, np.float32)
    dw, dg = up(ctx, w), up(ctx, g)
    ctx.sgd_step(dw, dg, n, 0.1, grad_scale=0.5, zero_grad=False)
    oracle.sgd(w, g, 0.1, grad_scale=0.5, zero_grad=False)
    assert np.array_equal(ctx.to_numpy(dw), w)      # same operations, same rounding
    assert np.array_equal(ctx.to_numpy(dg), g)


@pytest.mark.parametrize("n", [5, 4096, (1 << 20) + 3])
def test_adamw_vs_oracle(ctx, oracle, n):
    r = rng(20 + n)
    w = r.standard_normal(n, np.float32)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    dw, dm, dv = up(ctx, w), up(ctx, m), up(ctx, v)
    hp = (1e-3, 0.9, 0.999, 1e-8, 0.01)
    for step in (1, 2, 3):
        g = r.standard_normal(n, np.float32)
        dg = up(ctx, g)
        ctx.adamw_step(dw, dg, dm, dv, n, *hp, step=step, grad_scale=0.25)
        oracle.adamw(w, g, m, v, *hp, step, grad_scale=0.25)
        assert (ctx.to_numpy(dg) == 0.0).all()
    check(ctx.to_numpy(dw), w, TOL_EW, "adamw w")
    check(ctx.to_numpy(dm), m, TOL_EW, "adamw m")
    check(ctx.to_numpy(dv), v, TOL_EW, "adamw v")


@pytest.mark.parametrize("kind", ["adamw", "sgd"])
def test_multi_tensor_update_equals_one_call_per_tensor(ctx, kind):
    # one launch over several tensors (ragged sizes, more than 16 of them): bit-identical to one call each,
    # pairs included
    from ferrograd_b200.backend import to_bf16_bits
    r = rng(404)
    sizes = [5, 4096, 8193, 1, 100003, 8192, 12] + [33] * 12
    hp = (1e-3, 0.9, 0.999, 1e-8, 0.01)
    tensors, singles = [], []
    for n in sizes:
        w, g = r.standard_normal(n, np.float32), r.standard_normal(n, np.float32)
        m, v = r.standard_normal(n, np.float32) * 0.1, np.abs(r.standard_normal(n, np.float32)) * 0.01
        stride = (n + 7) // 8 * 8
        a = dict(w=up(ctx, w), g=up(ctx, g), m=up(ctx, m), v=up(ctx, v), w_pairs=ctx.alloc_zeroed(4 * stride), pairs_stride=stride, n=n)
        b = dict(w=up(ctx, w), g=up(ctx, g), m=up(ctx, m), v=up(ctx, v), w_pairs=ctx.alloc_zeroed(4 * stride), pairs_stride=stride, n=n)
        tensors.append(a)
        singles.append(b)
    if kind == "adamw":
        ctx.adamw_step_multi(tensors, *hp, step=3, grad_scale=0.5)
        for b in singles:
            ctx.adamw_step_paired(b["w"], b["g"], b["m"], b["v"], b["n"], *hp, b["w_pairs"], b["pairs_stride"], step=3, grad_scale=0.5)
    else:
        ctx.sgd_step_multi(tensors, 0.1, grad_scale=0.5)
        for b in singles:
            ctx.sgd_step_paired(b["w"], b["g"], b["n"], 0.1, b["w_pairs"], b["pairs_stride"], grad_scale=0.5)
    ctx.sync()
    for a, b in zip(tensors, singles):
        for key in ("w", "g") + (("m", "v") if kind == "adamw" else ()):
            assert np.array_equal(ctx.to_numpy(a[key]), ctx.to_numpy(b[key])), key
        pa = ctx.download(a["w_pairs"], np.empty(2 * a["pairs_stride"], np.uint16))
        pb = ctx.download(b["w_pairs"], np.empty(2 * a["pairs_stride"], np.uint16))
        assert np.array_equal(pa, pb)
        # the pairs are those of the updated weights: plane 0 = bf16(w), plane 1 = bf16(w - trunc_tf32(w))
        w = ctx.to_numpy(a["w"])
        hi = (w.view(np.uint32) & np.uint32(0xffffe000)).view(np.float32)
        assert np.array_equal(pa[:a["n"]], to_bf16_bits(w))
        assert np.array_equal(pa[a["pairs_stride"]:a["pairs_stride"] + a["n"]], to_bf16_bits(w - hi))
        assert (ctx.to_numpy(a["g"]) == 0).all()


def test_adamw_device_step_counter(ctx, oracle):
    n = 1000
    r = rng(33)
    w, g = r.standard_normal(n, np.float32), r.standard_normal(n, np.float32)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    dw, dg, dm, dv = up(ctx, w), up(ctx, g), up(ctx, m), up(ctx, v)
    counter = up(ctx, np.array([4], np.uint32))
    ctx.counter_increment(counter)
    ctx.adamw_step(dw, dg, dm, dv, n, 1e-3, 0.9, 0.999, 1e-8, 0.0, step=0, step_dev=counter, zero_grad=False)
    oracle.adamw(w, g, m, v, 1e-3, 0.9, 0.999, 1e-8, 0.0, 5, zero_grad=False)
    check(ctx.to_numpy(dw), w, TOL_EW, "adamw w (device step)")


# ---------------------------------------------------------------- softmax family
# 1000, 2000, 4096, 6000 columns: the kernels that hold a row in registers, with 1, 2, 4 and 8 float4 per thread
SOFTMAX_SHAPES = [(1, 1), (7, 10), (64, 33), (37, 1000), (33, 2000), (5, 4096), (21, 6000), (300, 8192), (9, 12345),
                  (40, 32000), (3, 40000)]


@pytest.mark.parametrize("rows,cols", SOFTMAX_SHAPES)
def test_softmax_fwd_bwd(ctx, oracle, rows, cols):
    r = rng(rows * 100003 + cols)
    x = (2.0 * r.standard_normal((rows, cols), np.float32)).astype(np.float32)
    dx_, dy_ = up(ctx, x), ctx.new_tensor((rows, cols))
    ctx.softmax_fwd(dx_, dy_, rows, cols)
    y = ctx.to_numpy(dy_)
    yref = oracle.softmax_fwd(x)
    check(y, yref, TOL_EW, "softmax fwd")
    dy = r.standard_normal((rows, cols), np.float32)
    ddy, dgrad = up(ctx, dy), ctx.new_tensor((rows, cols))
    ctx.softmax_bwd(up(ctx, yref), ddy, dgrad, rows, cols)
    check(ctx.to_numpy(dgrad), oracle.softmax_bwd(yref, dy), TOL_EW, "softmax bwd")
    # accumulate form (the reference's +=)
    base = r.standard_normal((rows, cols), np.float32)
    dacc = up(ctx, base)
    ctx.softmax_bwd(up(ctx, yref), ddy, dacc, rows, cols, accumulate=True)
    check(ctx.to_numpy(dacc), oracle.softmax_bwd(yref, dy, dx=base), TOL_EW, "softmax bwd accumulate")


@pytest.mark.parametrize("rows,cols", SOFTMAX_SHAPES)
def test_softmax_ce(ctx, oracle, rows, cols):
    r = rng(rows * 7919 + cols)
    x = (2.0 * r.standard_normal((rows, cols), np.float32)).astype(np.float32)
    labels = r.integers(0, cols, rows).astype(np.uint32)
    scale = 1.0 / rows
    ref = oracle.softmax_ce(x, labels, grad_scale=scale, want_probs=True)
    dlog, probs = ctx.new_tensor((rows, cols)), ctx.new_tensor((rows, cols))
    lrow, lmean = ctx.new_tensor((rows,)), ctx.new_tensor((1,))
    am = ctx.new_tensor((rows,), np.uint32)
    ctx.softmax_ce(up(ctx, x), up(ctx, labels), rows, cols, grad_scale=scale, loss_row=lrow, loss_mean=lmean,
                   dlogits=dlog, probs=probs, argmax=am)
    check(ctx.to_numpy(lrow), ref["loss_row"], TOL_EW, "loss_row")
    check(ctx.to_numpy(lmean), np.array([ref["loss_mean"]], np.float32), TOL_EW, "loss_mean")
    check(ctx.to_numpy(probs), ref["probs"], TOL_EW, "probs")
    check(ctx.to_numpy(dlog), ref["dlogits"], TOL_EW, "dlogits")
    assert np.array_equal(ctx.to_numpy(am), ref["argmax"])          # index output: bit-exact
    assert ctx.device_status() == 0


def test_softmax_ce_argmax_ties_and_minimal_outputs(ctx, oracle):
    rows, cols = 4, 16384
    x = np.zeros((rows, cols), np.float32)
    x[1, 5] = x[1, 9000] = 3.0       # tie: first index wins
    x[2, cols - 1] = 1.0
    labels = np.array([0, 5, cols - 1, 7], np.uint32)
    ref = oracle.softmax_ce(x, labels)
    am, dlog = ctx.new_tensor((rows,), np.uint32), ctx.new_tensor((rows, cols))
    ctx.softmax_ce(up(ctx, x), up(ctx, labels), rows, cols, dlogits=dlog, argmax=am)
    assert np.array_equal(ctx.to_numpy(am), ref["argmax"]) and ctx.to_numpy(am)[1] == 5
    check(ctx.to_numpy(dlog), ref["dlogits"], TOL_EW, "dlogits")


def test_ce_elementwise_reference_form(ctx, oracle):
    rows, cols = 33, 48
    r = rng(5)
    p = oracle.softmax_fwd(r.standard_normal((rows, cols), np.float32))
    labels = r.integers(0, cols, rows).astype(np.uint32)
    loss, grad = ctx.new_tensor((rows, cols)), ctx.new_tensor((rows, cols))
    ctx.ce_loss_grad(up(ctx, p), up(ctx, labels), rows, cols, loss, grad)
    lref, gref = oracle.ce_loss_grad(p, labels)
    check(ctx.to_numpy(loss), lref, TOL_EW, "ce loss")
    assert np.array_equal(ctx.to_numpy(grad), gref)


# ---------------------------------------------------------------- elementwise
@pytest.mark.parametrize("n", [1, 130, 100003])
def test_mse(ctx, oracle, n):
    r = rng(40 + n)
    p, t = r.standard_normal(n, np.float32), r.standard_normal(n, np.float32)
    loss, grad, s = ctx.new_tensor((n,)), ctx.new_tensor((n,)), ctx.new_tensor((1,))
    ctx.mse_loss_grad(up(ctx, p), up(ctx, t), n, grad_scale=0.5, loss_elem=loss, loss_sum=s, grad=grad)
    lref, sref, gref = oracle.mse(p, t, grad_scale=0.5)
    assert np.array_equal(ctx.to_numpy(loss), lref) and np.array_equal(ctx.to_numpy(grad), gref)
    check(ctx.to_numpy(s), np.array([sref], np.float32), TOL_EW, "mse sum")


@pytest.mark.parametrize("n", [1, 130, 100003])
def test_bce(ctx, oracle, n):
    r = rng(45 + n)
    p = (1.0 / (1.0 + np.exp(-r.standard_normal(n) * 2.0))).astype(np.float32)
    t = (r.random(n) < 0.5).astype(np.float32)
    if n > 100:
        t[:50] = r.random(50).astype(np.float32)        # soft targets too
    loss, grad, s = ctx.new_tensor((n,)), ctx.new_tensor((n,)), ctx.new_tensor((1,))
    ctx.bce_loss_grad(up(ctx, p), up(ctx, t), n, grad_scale=0.25, loss_elem=loss, loss_sum=s, grad=grad)
    lref, sref, gref = oracle.bce(p, t, grad_scale=0.25)
    assert np.array_equal(ctx.to_numpy(grad), gref)
    check(ctx.to_numpy(loss), lref, TOL_EW, "bce loss")
    check(ctx.to_numpy(s), np.array([sref], np.float32), TOL_EW, "bce sum")
    # float64 closed form
    p64, t64 = p.astype(np.float64), t.astype(np.float64)
    check(ctx.to_numpy(loss), -(t64 * np.log(p64) + (1 - t64) * np.log1p(-p64)), TOL_EW, "bce vs float64")


@pytest.mark.parametrize("act", ["none", "relu", "tanh", "gelu"])
def test_bias_act_and_backward(ctx, oracle, act):
    rows, cols = 67, 130
    r = rng(50)
    z, b = r.standard_normal((rows, cols), np.float32), r.standard_normal(cols, np.float32)
    y = ctx.new_tensor((rows, cols))
    ctx.bias_act_fwd(up(ctx, z), up(ctx, b), act, y, rows, cols)
    yref, pre = oracle.bias_act_fwd(z, b, act)
    check(ctx.to_numpy(y), yref, TOL_EW, f"bias+{act}")
    dy = r.standard_normal((rows, cols), np.float32)
    saved = pre if act == "gelu" else yref
    dz = ctx.new_tensor((rows, cols))
    ctx.act_bwd(up(ctx, dy), up(ctx, saved), dz, rows * cols, act)
    check(ctx.to_numpy(dz), oracle.act_bwd(dy, saved, act), TOL_EW, f"{act} backward")


def test_chain_mul_add_reference_constants(ctx):
    # crates/ferrograd/tests/std_wgsl.rs:10-94: out = c + a*b.
    n = 32 * 32
    a, b, c = (up(ctx, np.full(n, v, np.float32)) for v in (3.0, 2.0, 1.0))
    prog = [("input", 0, 0, 0.0), ("input", 1, 0, 0.0), ("input", 2, 0, 0.0), ("mul", 0, 1, 0.0), ("add", 2, 3, 0.0)]
    out = ctx.new_tensor((n,))
    ctx.eltwise_chain_fwd(prog, [a, b, c], out, n)
    assert (ctx.to_numpy(out) == 7.0).all()
    grads = [ctx.new_tensor((n,)) for _ in range(3)]
    ctx.eltwise_chain_bwd(prog, [a, b, c], up(ctx, np.ones(n, np.float32)), grads, n)
    assert [float(ctx.to_numpy(g)[0]) for g in grads] == [2.0, 3.0, 1.0]
    assert all((ctx.to_numpy(g) == ctx.to_numpy(g)[0]).all() for g in grads)


def test_chain_all_ops_vs_oracle(ctx, oracle):
    n = 5000
    r = rng(60)
    x0 = r.standard_normal(n, np.float32)
    x1 = (np.abs(r.standard_normal(n, np.float32)) + 0.5).astype(np.float32)
    prog = [("input", 0, 0, 0.0), ("input", 1, 0, 0.0), ("const", 0, 0, 1.5), ("mul", 0, 1, 0.0),
            ("div", 3, 1, 0.0), ("sub", 4, 2, 0.0), ("tanh", 5, 0, 0.0), ("gelu", 0, 0, 0.0), ("add", 6, 7, 0.0),
            ("log", 1, 0, 0.0), ("exp", 6, 0, 0.0), ("mul", 9, 10, 0.0), ("neg", 11, 0, 0.0), ("abs", 0, 0, 0.0),
            ("relu", 5, 0, 0.0), ("elu", 0, 0, 0.0), ("add", 12, 13, 0.0), ("add", 14, 15, 0.0),
            ("add", 16, 17, 0.0), ("add", 18, 8, 0.0)]
    out = ctx.new_tensor((n,))
    sv = ctx.new_tensor((n,))
    ctx.eltwise_chain_fwd(prog, [up(ctx, x0), up(ctx, x1)], out, n, saved={6: sv})
    oref, saved = oracle.eltwise_fwd(prog, [x0, x1], save=(6,))
    check(ctx.to_numpy(out), oref, TOL_EW, "chain fwd")
    check(ctx.to_numpy(sv), saved[6], TOL_EW, "chain saved value")
    seed = r.standard_normal(n, np.float32)
    grads = [ctx.new_tensor((n,)) for _ in range(2)]
    ctx.eltwise_chain_bwd(prog, [up(ctx, x0), up(ctx, x1)], up(ctx, seed), grads, n)
    gref = oracle.eltwise_bwd(prog, [x0, x1], seed)
    for g, gr in zip(grads, gref):
        check(ctx.to_numpy(g), gr, TOL_EW, "chain bwd")


# ---------------------------------------------------------------- 16-bit storage
def up16(ctx, x, dtype):
    """x (float32, already representable in dtype) as a device tensor of that storage type."""
    return ctx.init_tensor_f16(x.shape, x) if dtype == "f16" else ctx.init_tensor_bf16(x.shape, x)


def down16(ctx, t, dtype):
    from ferrograd_b200.backend import from_bf16_bits
    a = ctx.to_numpy(t)
    return a.astype(np.float32) if dtype == "f16" else from_bf16_bits(a)


def new16(ctx, n, dtype):
    return ctx.new_tensor((n,), np.float16 if dtype == "f16" else np.uint16)


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_convert_round_trip(ctx, oracle, dtype):
    n = 70001
    x = (rng(70).standard_normal(n) * 37.0).astype(np.float32)
    x[:4] = [0.0, -0.0, 65504.0, 1e-7]
    d32, d16, back = up(ctx, x), new16(ctx, n, dtype), ctx.new_tensor((n,))
    ctx.convert(d32, "f32", d16, dtype, n)
    ctx.convert(d16, dtype, back, "f32", n)
    assert np.array_equal(ctx.to_numpy(back), oracle.round_to(x, dtype))        # round to nearest even, bit for bit
    assert np.array_equal(down16(ctx, d16, dtype), oracle.round_to(x, dtype))


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_chain_16bit_arithmetic_bit_exact(ctx, oracle, dtype):
    # + - * / with every result rounded to the storage type: identical to the oracle's, bit for bit
    n = 20011
    r = rng(71)
    x0 = oracle.round_to(r.standard_normal(n, np.float32), dtype)
    x1 = oracle.round_to(np.abs(r.standard_normal(n, np.float32)) + 0.5, dtype)
    prog = [("input", 0, 0, 0.0), ("input", 1, 0, 0.0), ("const", 0, 0, 1.7), ("mul", 0, 1, 0.0), ("div", 3, 2, 0.0),
            ("sub", 4, 1, 0.0), ("add", 5, 0, 0.0), ("div", 6, 1, 0.0), ("neg", 7, 0, 0.0), ("abs", 8, 0, 0.0),
            ("mul", 9, 7, 0.0)]
    a, b, out = up16(ctx, x0, dtype), up16(ctx, x1, dtype), new16(ctx, n, dtype)
    ctx.eltwise_chain_fwd(prog, [a, b], out, n, dtype=dtype)
    oref, _ = oracle.eltwise_fwd(prog, [x0, x1], dtype=dtype)
    assert np.array_equal(down16(ctx, out, dtype), oref)
    seed = oracle.round_to(r.standard_normal(n, np.float32), dtype)
    grads = [new16(ctx, n, dtype) for _ in range(2)]
    ctx.eltwise_chain_bwd(prog, [a, b], up16(ctx, seed, dtype), grads, n, dtype=dtype)
    for g, gr in zip(grads, oracle.eltwise_bwd(prog, [x0, x1], seed, dtype=dtype)):
        assert np.array_equal(down16(ctx, g, dtype), gr)


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_chain_16bit_all_ops(ctx, oracle, dtype):
    # exp/log/tanh/gelu go through float libm on both sides; a last-bit difference there can land on the
    # other side of a 16-bit rounding boundary, so the bar is one unit of the storage type's precision
    n = 5000
    tol = 2.0 ** -10 if dtype == "f16" else 2.0 ** -7
    r = rng(72)
    x0 = oracle.round_to(r.standard_normal(n, np.float32), dtype)
    x1 = oracle.round_to(np.abs(r.standard_normal(n, np.float32)) + 0.5, dtype)
    prog = [("input", 0, 0, 0.0), ("input", 1, 0, 0.0), ("const", 0, 0, 1.5), ("mul", 0, 1, 0.0),
            ("div", 3, 1, 0.0), ("sub", 4, 2, 0.0), ("tanh", 5, 0, 0.0), ("gelu", 0, 0, 0.0), ("add", 6, 7, 0.0),
            ("log", 1, 0, 0.0), ("exp", 6, 0, 0.0), ("mul", 9, 10, 0.0), ("neg", 11, 0, 0.0), ("abs", 0, 0, 0.0),
            ("relu", 5, 0, 0.0), ("elu", 0, 0, 0.0), ("add", 12, 13, 0.0), ("add", 14, 15, 0.0),
            ("add", 16, 17, 0.0), ("add", 18, 8, 0.0)]
    a, b, out = up16(ctx, x0, dtype), up16(ctx, x1, dtype), new16(ctx, n, dtype)
    ctx.eltwise_chain_fwd(prog, [a, b], out, n, dtype=dtype)
    oref, _ = oracle.eltwise_fwd(prog, [x0, x1], dtype=dtype)
    check(down16(ctx, out, dtype), oref, tol, f"{dtype} chain fwd")
    seed = oracle.round_to(r.standard_normal(n, np.float32), dtype)
    grads = [new16(ctx, n, dtype) for _ in range(2)]
    ctx.eltwise_chain_bwd(prog, [a, b], up16(ctx, seed, dtype), grads, n, dtype=dtype)
    for g, gr in zip(grads, oracle.eltwise_bwd(prog, [x0, x1], seed, dtype=dtype)):
        check(down16(ctx, g, dtype), gr, 4 * tol, f"{dtype} chain bwd")


LOWP_SHAPES = [(256, 256, 64), (512, 384, 1024), (300, 520, 1100),     # ragged: copies with padded pitch
               (130, 10, 257), (1100, 264, 4100), (600, 712, 2304)]     # narrow N; long K; split-K tail


def new16m(ctx, shape, dtype):
    return ctx.new_tensor(shape, np.float16 if dtype == "f16" else np.uint16)


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", LOWP_SHAPES)
def test_gemm_16bit_storage(ctx, oracle, dtype, M, N, K):
    # products of 16-bit values are exact in f32, so against a float64 accumulation the only visible error
    # is the final rounding to the storage type (half a unit in the last place: 2^-11 / 2^-8 relative)
    tol = 2.0 ** -10 if dtype == "f16" else 2.0 ** -7
    r = rng(M + 3 * N + 7 * K)
    A = oracle.round_to(r.standard_normal((M, K), np.float32), dtype)
    B = oracle.round_to(r.standard_normal((K, N), np.float32) / np.sqrt(K), dtype)
    bias = oracle.round_to(r.standard_normal(N, np.float32), dtype)
    Cd, Pd = new16m(ctx, (M, N), dtype), new16m(ctx, (M, N), dtype)
    ctx.gemm_lowp(up16(ctx, A, dtype), up16(ctx, B, dtype), Cd, M, N, K, dtype, bias=up16(ctx, bias, dtype), act="tanh",
                  preact_out=Pd)
    assert ctx.device_status() == 0
    y, pre = oracle.bias_act_fwd(oracle.gemm(A, B, f64=True), bias, "tanh")
    check(down16(ctx, Pd, dtype), pre, tol, f"{dtype} pre-activation")
    check(down16(ctx, Cd, dtype), y, tol, f"{dtype} output")


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K,act", [(256, 384, 512, "none"), (300, 264, 200, "tanh"), (520, 130, 1000, "gelu"),
                                       (1024, 512, 768, "relu")])
def test_gemm_16bit_storage_backward(ctx, oracle, dtype, M, N, K, act):
    tol = 2.0 ** -10 if dtype == "f16" else 2.0 ** -7
    r = rng(M + N + K)
    A = oracle.round_to(r.standard_normal((M, K), np.float32), dtype)
    B = oracle.round_to(r.standard_normal((K, N), np.float32) / np.sqrt(K), dtype)
    bias = oracle.round_to(r.standard_normal(N, np.float32) * 0.1, dtype)
    y, pre = oracle.bias_act_fwd(oracle.gemm(A, B, f64=True), bias, act)
    saved = oracle.round_to(pre if act == "gelu" else y, dtype)
    dY = oracle.round_to(r.standard_normal((M, N), np.float32), dtype)
    dA, dB, db = new16m(ctx, (M, K), dtype), new16m(ctx, (K, N), dtype), new16m(ctx, (N,), dtype)
    ctx.gemm_bwd_lowp(up16(ctx, A, dtype), up16(ctx, B, dtype), up16(ctx, dY, dtype), M, N, K, dtype, act=act,
                      saved=up16(ctx, saved, dtype) if act != "none" else None, dA=dA, dB=dB, dbias=db)
    assert ctx.device_status() == 0
    dz = oracle.round_to(oracle.act_bwd(dY, saved, act), dtype)      # dZ is rounded to the storage type
    check(down16(ctx, dA, dtype), oracle.gemm(dz, B, transB=True, f64=True), tol, f"{dtype} dA")
    check(down16(ctx, dB, dtype), oracle.gemm(A, dz, transA=True, f64=True), tol, f"{dtype} dB")
    check(down16(ctx, db, dtype), dz.astype(np.float64).sum(axis=0), 2 * tol, f"{dtype} dbias")


# ---------------------------------------------------------------- GEMM
GEMM_SHAPES = [(32, 64, 16), (1, 1, 1), (64, 2, 16), (70, 33, 45), (130, 257, 100), (256, 512, 384)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("tA,tB", [(False, False), (True, False), (False, True), (True, True)])
def test_gemm_simt_bit_exact(ctx, oracle, M, N, K, tA, tB):
    r = rng(M * 31 + N * 17 + K)
    A = r.standard_normal((K, M) if tA else (M, K), np.float32)
    B = r.standard_normal((N, K) if tB else (K, N), np.float32)
    Cd = ctx.new_tensor((M, N))
    ctx.gemm(up(ctx, A), up(ctx, B), Cd, M, N, K, transA=tA, transB=tB, mode="simt")
    assert np.array_equal(ctx.to_numpy(Cd), oracle.gemm(A, B, transA=tA, transB=tB))


TC_SHAPES = [(128, 256, 32), (128, 128, 64), (256, 512, 384), (200, 72, 100), (130, 10, 257), (1000, 300, 77),
             (64, 48, 8), (384, 1024, 1000), (128, 256, 8192), (256, 130, 4100),
             # shapes that take the CTA-pair kernel (M > 128, N > 128), with ragged edges and long K
             (256, 256, 64), (300, 520, 1000), (512, 768, 8192), (1100, 257, 333)]
TC_MODES = ["3xtf32", "tf32_bf16x2", "auto"]


@pytest.mark.parametrize("mode", TC_MODES)
@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_gemm_tensor_core_vs_oracle(ctx, oracle, M, N, K, mode):
    r = rng(M * 131 + N * 71 + K)
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32)
    Cd = ctx.new_tensor((M, N))
    ctx.gemm(up(ctx, A), up(ctx, B), Cd, M, N, K, mode=mode)
    got = ctx.to_numpy(Cd)
    assert ctx.device_status() == 0
    check(got, oracle.gemm(A, B), TOL_GEMM, f"{mode} vs f32 fma chain")
    check(got, oracle.gemm(A, B, f64=True), TOL_GEMM, f"{mode} vs f64 accumulate")


@pytest.mark.parametrize("mode", ["3xtf32", "tf32_bf16x2"])
@pytest.mark.parametrize("tile", ["128x32", "256x32", "pair"])
def test_gemm_every_tile_kernel(ctx, oracle, mode, tile):
    # The tile heuristic picks one kernel per shape; force each of them on the same ragged problem.
    ctx.set_option("gemm_tile", tile)
    M, N, K = 400, 600, 700
    r = rng(4242)
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32)
    bias = r.standard_normal(N, np.float32)
    Cd, Pd = ctx.new_tensor((M, N)), ctx.new_tensor((M, N))
    ctx.gemm(up(ctx, A), up(ctx, B), Cd, M, N, K, bias=up(ctx, bias), act="tanh", preact_out=Pd, mode=mode)
    ctx.set_option("gemm_tile", "auto")
    yref, pre = oracle.bias_act_fwd(oracle.gemm(A, B), bias, "tanh")
    assert ctx.device_status() == 0
    check(ctx.to_numpy(Pd), pre, TOL_GEMM, f"{mode}/{tile} pre-activation")
    check(ctx.to_numpy(Cd), yref, TOL_GEMM, f"{mode}/{tile} output")


@pytest.mark.parametrize("mode", ["3xtf32", "tf32_bf16x2"])
@pytest.mark.parametrize("M,N,K", [(600, 700, 2304),      # 9 tiles, no full wave: every tile in 4 K-shares
                                   (2500, 2304, 1024),    # 90 tiles: one full wave, then 16 tiles in 2 K-shares
                                   (300, 520, 1100)])     # 5 chunks in 2 uneven shares
def test_gemm_pair_split_k_tail(ctx, oracle, mode, M, N, K):
    # The pair kernel cuts the tiles of an under-filled last wave into K-shares that a second kernel folds.
    r = rng(M + N + K)
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32) * 0.1
    bias = r.standard_normal(N, np.float32)
    Ad, Bd, bd = up(ctx, A), up(ctx, B), up(ctx, bias)
    Cd, Pd = ctx.new_tensor((M, N)), ctx.new_tensor((M, N))
    ctx.set_option("gemm_tile", "pair")
    ctx.gemm(Ad, Bd, Cd, M, N, K, bias=bd, act="gelu", preact_out=Pd, mode=mode)
    got, got_pre = ctx.to_numpy(Cd), ctx.to_numpy(Pd)
    assert ctx.device_status() == 0
    yref, pre = oracle.bias_act_fwd(oracle.gemm(A, B), bias, "gelu")
    check(got_pre, pre, TOL_GEMM, f"{mode} split-K pre-activation")
    check(got, yref, TOL_GEMM, f"{mode} split-K output")
    # the same product without the split agrees to rounding, and the split is deterministic
    ctx.gemm(Ad, Bd, Cd, M, N, K, bias=bd, act="gelu", preact_out=Pd, mode=mode)
    assert np.array_equal(ctx.to_numpy(Cd), got)
    ctx.set_option("gemm_split_k", "0")
    ctx.gemm(Ad, Bd, Cd, M, N, K, bias=bd, act="gelu", preact_out=Pd, mode=mode)
    ctx.set_option("gemm_split_k", "1")
    ctx.set_option("gemm_tile", "auto")
    check(ctx.to_numpy(Pd), got_pre, TOL_EW, "split vs unsplit")


@pytest.mark.parametrize("mode", ["3xtf32", "tf32_bf16x2"])
@pytest.mark.parametrize("tA,tB", [(True, False), (False, True), (True, True)])
def test_gemm_tensor_core_transposes(ctx, oracle, tA, tB, mode):
    M, N, K = 192, 320, 200
    r = rng(77)
    A = r.standard_normal((K, M) if tA else (M, K), np.float32)
    B = r.standard_normal((N, K) if tB else (K, N), np.float32)
    Cd = ctx.new_tensor((M, N))
    ctx.gemm(up(ctx, A), up(ctx, B), Cd, M, N, K, transA=tA, transB=tB, mode=mode)
    check(ctx.to_numpy(Cd), oracle.gemm(A, B, transA=tA, transB=tB), TOL_GEMM, f"{mode} transposed")


def _pairs_of(x):
    """What the library defines as a tensor's bf16 pairs: bf16(x) and bf16(x - trunc_tf32(x))."""
    from ferrograd_b200.backend import to_bf16_bits
    x = np.ascontiguousarray(x, np.float32)
    hi = (x.view(np.uint32) & np.uint32(0xffffe000)).view(np.float32)
    return to_bf16_bits(x).reshape(x.shape), to_bf16_bits(x - hi).reshape(x.shape)


# (M, N, K): the pair kernel on the tensors themselves; a ragged shape that goes through operand planes; a narrow layer
PAIRED_SHAPES = [(512, 384, 256), (640, 520, 1032), (300, 130, 100), (512, 10, 256)]


@pytest.mark.parametrize("act", ["none", "relu", "tanh", "gelu"])
@pytest.mark.parametrize("M,N,K", PAIRED_SHAPES)
@pytest.mark.parametrize("own_pairs", [True, False])
def test_gemm_paired_forward(ctx, oracle, M, N, K, act, own_pairs):
    r = rng(M * 7 + N * 3 + K + len(act))
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32) * 0.1
    bias = r.standard_normal(N, np.float32)
    Ad, Bd, Cd, Pd = up(ctx, A), up(ctx, B), ctx.new_tensor((M, N)), ctx.new_tensor((M, N))
    sa, sb, sc = (M * K + 7) // 8 * 8, (K * N + 7) // 8 * 8, (M * N + 7) // 8 * 8
    ap = bp = None
    if own_pairs:       # the caller keeps the operands' pairs; otherwise the call makes them
        ap, bp = ctx.alloc(4 * sa), ctx.alloc(4 * sb)
        ctx.pairs_from_f32(Ad, M * K, ap, sa)
        ctx.pairs_from_f32(Bd, K * N, bp, sb)
    cp = ctx.alloc_zeroed(4 * sc)
    ctx.gemm_paired(Ad, Bd, Cd, M, N, K, A_pairs=ap, B_pairs=bp, bias=up(ctx, bias), act=act, preact_out=Pd, C_pairs=cp,
                    A_stride=sa, B_stride=sb, C_stride=sc)
    got, pre = ctx.to_numpy(Cd), ctx.to_numpy(Pd)
    assert ctx.device_status() == 0
    yref, zref = oracle.bias_act_fwd(oracle.gemm(A, B), bias, act)
    check(pre, zref, TOL_GEMM, "pre-activation")
    check(got, yref, TOL_GEMM, "output")
    pairs = ctx.download(cp, np.empty(2 * sc, np.uint16))
    hb, lo = _pairs_of(got)
    assert np.array_equal(pairs[:M * N].reshape(M, N), hb)                  # the pairs are exact functions of what was stored
    assert np.array_equal(pairs[sc:sc + M * N].reshape(M, N), lo)


@pytest.mark.parametrize("below", ["none", "relu", "tanh", "gelu"])
@pytest.mark.parametrize("M,N,K", PAIRED_SHAPES)
def test_gemm_paired_backward(ctx, oracle, M, N, K, below):
    # dB = A^T dZ; dA = (dZ B^T) * act'(saved of the layer below), with its pairs and column sums; dbias = column sums of dZ
    r = rng(M + N * 5 + K * 11 + len(below))
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32) * 0.1
    dZ = r.standard_normal((M, N), np.float32)
    z_below = r.standard_normal((M, K), np.float32)                  # pre-activation of the layer below
    y_below, _ = oracle.bias_act_fwd(z_below, None, below)
    saved = z_below if below == "gelu" else y_below                    # GELU saves the pre-activation, the others the output
    Ad, Bd, Zd = up(ctx, A), up(ctx, B), up(ctx, dZ)
    dB, dA = ctx.new_tensor((K, N)), ctx.new_tensor((M, K))
    dbias, dbias_below = ctx.new_tensor((N,)), ctx.new_tensor((K,))
    sa = (M * K + 7) // 8 * 8
    dap = ctx.alloc_zeroed(4 * sa)
    ctx.gemm_bwd_paired(Ad, Bd, Zd, M, N, K, dB=dB, dbias=dbias, dA=dA, below_act=below,
                        below_saved=up(ctx, saved) if below != "none" else None, dA_pairs=dap, dA_stride=sa,
                        below_dbias=dbias_below)
    got_dA, got_dB = ctx.to_numpy(dA), ctx.to_numpy(dB)
    assert ctx.device_status() == 0
    check(got_dB, oracle.gemm(A, dZ, transA=True), TOL_GEMM, "dB")
    ref_dA = oracle.act_bwd(oracle.gemm(dZ, B, transB=True), saved, below)
    check(got_dA, ref_dA, TOL_GEMM, "dA with the activation factor of the layer below")
    check(ctx.to_numpy(dbias), oracle.colsum(dZ), TOL_EW, "dbias")
    check(ctx.to_numpy(dbias_below), oracle.colsum(got_dA), TOL_EW, "bias gradient of the layer below = column sums of dA")
    pairs = ctx.download(dap, np.empty(2 * sa, np.uint16))
    hb, lo = _pairs_of(got_dA)
    assert np.array_equal(pairs[:M * K].reshape(M, K), hb)
    assert np.array_equal(pairs[sa:sa + M * K].reshape(M, K), lo)


@pytest.mark.parametrize("mode", ["simt", "3xtf32", "tf32_bf16x2"])
@pytest.mark.parametrize("act", ["none", "relu", "tanh", "gelu"])
def test_gemm_epilogue(ctx, oracle, mode, act):
    M, N, K = 256, 264, 96
    r = rng(88)
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32) * 0.2
    bias = r.standard_normal(N, np.float32)
    Cd, Pd = ctx.new_tensor((M, N)), ctx.new_tensor((M, N))
    ctx.gemm(up(ctx, A), up(ctx, B), Cd, M, N, K, bias=up(ctx, bias), act=act, preact_out=Pd, mode=mode)
    yref, pre = oracle.bias_act_fwd(oracle.gemm(A, B), bias, act)
    check(ctx.to_numpy(Pd), pre, TOL_GEMM, "pre-activation")
    got = ctx.to_numpy(Cd)
    if act == "relu":
        # the mask is an index-like output: wherever the reference is clearly non-zero it must agree
        clear = np.abs(pre) > 1e-3
        assert np.array_equal((got > 0)[clear], (yref > 0)[clear])
    check(got, yref, TOL_GEMM, f"epilogue {act}")


@pytest.mark.parametrize("mode", ["simt", "3xtf32", "tf32_bf16x2"])
@pytest.mark.parametrize("act", ["none", "relu", "tanh", "gelu"])
def test_gemm_backward(ctx, oracle, mode, act):
    M, N, K = 192, 136, 160
    r = rng(99)
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32) * 0.2
    bias = r.standard_normal(N, np.float32) * 0.1
    y, pre = oracle.bias_act_fwd(oracle.gemm(A, B), bias, act)
    saved = pre if act == "gelu" else y
    dY = r.standard_normal((M, N), np.float32)
    dA, dB, db, dZ = ctx.new_tensor((M, K)), ctx.new_tensor((K, N)), ctx.new_tensor((N,)), ctx.new_tensor((M, N))
    ctx.gemm_bwd(up(ctx, A), up(ctx, B), up(ctx, dY), M, N, K, act=act, saved=up(ctx, saved), dA=dA, dB=dB,
                 dbias=db, dZ_out=dZ, mode=mode)
    dz_ref = oracle.act_bwd(dY, saved, act)
    check(ctx.to_numpy(dZ), dz_ref, TOL_EW, "dZ")
    check(ctx.to_numpy(dA), oracle.gemm(dz_ref, B, transB=True), TOL_GEMM, "dA")
    check(ctx.to_numpy(dB), oracle.gemm(A, dz_ref, transA=True), TOL_GEMM, "dB")
    check(ctx.to_numpy(db), oracle.colsum(dz_ref), TOL_GEMM, "dbias")
    assert ctx.device_status() == 0
    # partial requests
    dA2 = ctx.new_tensor((M, K))
    ctx.gemm_bwd(None, up(ctx, B), up(ctx, dY), M, N, K, act=act, saved=up(ctx, saved), dA=dA2, mode=mode)
    check(ctx.to_numpy(dA2), oracle.gemm(dz_ref, B, transB=True), TOL_GEMM, "dA only")


@pytest.mark.parametrize("M,N,K", [(512, 10, 1024), (1001, 16, 517), (300, 3, 4800), (4096, 1, 1030)])
@pytest.mark.parametrize("act", ["none", "tanh"])
def test_gemm_skinny_output_layer(ctx, oracle, M, N, K, act):
    # N <= 16 in auto mode runs on plain-FMA kernels (forward, dA and dB) instead of tensor-core tiles.
    r = rng(M + 7 * N + K)
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32) * 0.1
    bias = r.standard_normal(N, np.float32)
    Cd, Pd = ctx.new_tensor((M, N)), ctx.new_tensor((M, N))
    ctx.gemm(up(ctx, A), up(ctx, B), Cd, M, N, K, bias=up(ctx, bias), act=act, preact_out=Pd, mode="auto")
    y, pre = oracle.bias_act_fwd(oracle.gemm(A, B), bias, act)
    check(ctx.to_numpy(Pd), pre, TOL_GEMM, "skinny pre-activation")
    check(ctx.to_numpy(Cd), y, TOL_GEMM, "skinny output")
    dY = r.standard_normal((M, N), np.float32)
    dz_ref = oracle.act_bwd(dY, y, act)
    dA, dB, db = ctx.new_tensor((M, K)), ctx.new_tensor((K, N)), ctx.new_tensor((N,))
    ctx.gemm_bwd(up(ctx, A), up(ctx, B), up(ctx, dY), M, N, K, act=act, saved=up(ctx, y), dA=dA, dB=dB, dbias=db,
                 mode="auto")
    check(ctx.to_numpy(dA), oracle.gemm(dz_ref, B, transB=True), TOL_GEMM, "skinny dA")
    check(ctx.to_numpy(dB), oracle.gemm(A, dz_ref, transA=True), TOL_GEMM, "skinny dB")
    check(ctx.to_numpy(db), oracle.colsum(dz_ref), TOL_GEMM, "skinny dbias")
    # dB alone, no activation: dZ is dY itself and no pre-pass runs
    dB2 = ctx.new_tensor((K, N))
    ctx.gemm_bwd(up(ctx, A), None, up(ctx, dY), M, N, K, dB=dB2, mode="auto")
    check(ctx.to_numpy(dB2), oracle.gemm(A, dY, transA=True), TOL_GEMM, "skinny dB only")
    assert ctx.device_status() == 0


def test_exchange_entry_points_without_a_communicator(ctx):
    # the data-parallel entry points refuse to run before fg_comm_init instead of launching anything
    from ferrograd_b200 import FgError
    M, N, K = 64, 32, 48
    A, B, dY = ctx.new_tensor((M, K), zeroed=True), ctx.new_tensor((K, N), zeroed=True), ctx.new_tensor((M, N), zeroed=True)
    dA, dB = ctx.new_tensor((M, K)), ctx.new_tensor((K, N))
    before = ctx.launch_count()
    with pytest.raises(FgError) as e:
        ctx.gemm_bwd_exchange(A, B, dY, M, N, K, dB, K * N, dA=dA, dB=dB)
    assert e.value.kind == "FG_ERR_NOT_INITIALIZED"
    with pytest.raises(FgError):
        ctx.allreduce_sum(dB, K * N)
    assert ctx.launch_count() == before
    ctx.comm_join()                      # nothing pending: a no-op
    ctx.comm_sync(100)                   # likewise


@pytest.mark.parametrize("mode", ["simt", "auto"])
def test_gemm_batched(ctx, oracle, mode):
    # rank-3 matmul: T independent products, every tensor stepped by one matrix per product
    T, M, N, K = 3, 136, 200, 168
    r = rng(314)
    A, B = r.standard_normal((T, M, K), np.float32), r.standard_normal((T, K, N), np.float32) * 0.2
    bias = r.standard_normal(N, np.float32)
    Cd, Pd = ctx.new_tensor((T, M, N)), ctx.new_tensor((T, M, N))
    ctx.gemm_batched(up(ctx, A), up(ctx, B), Cd, T, M, N, K, bias=up(ctx, bias), act="tanh", preact_out=Pd, mode=mode)
    got, dY = ctx.to_numpy(Cd), r.standard_normal((T, M, N), np.float32)
    dA, dB = ctx.new_tensor((T, M, K)), ctx.new_tensor((T, K, N))
    ctx.gemm_batched_bwd(up(ctx, A), up(ctx, B), up(ctx, dY), T, M, N, K, act="tanh", saved=Cd, dA=dA, dB=dB, mode=mode)
    gA, gB = ctx.to_numpy(dA), ctx.to_numpy(dB)
    for t in range(T):
        y, _ = oracle.bias_act_fwd(oracle.gemm(A[t], B[t]), bias, "tanh")
        check(got[t], y, TOL_GEMM, f"batched output {t}")
        dz = oracle.act_bwd(dY[t], y, "tanh")
        check(gA[t], oracle.gemm(dz, B[t], transB=True), TOL_GEMM, f"batched dA {t}")
        check(gB[t], oracle.gemm(A[t], dz, transA=True), TOL_GEMM, f"batched dB {t}")
    with pytest.raises(Exception):
        ctx.gemm_batched(up(ctx, A), up(ctx, B), Cd, T, M, N, K, strides=(M * K, 0, M * N))


def test_gemm_batched_small_matrices_run_as_one_launch(ctx, oracle):
    # 64 small products: one launch with the matrix index in the grid (forward), three launches for the backward
    # pass (dY * act', dB, dA); the exact path, so the results equal the oracle's sequential fma chain bit for bit
    T, M, N, K = 64, 24, 40, 56
    r = rng(2718)
    A, B = r.standard_normal((T, M, K), np.float32), r.standard_normal((T, K, N), np.float32)
    bias, dY = r.standard_normal(N, np.float32), r.standard_normal((T, M, N), np.float32)
    Ad, Bd, Cd, Pd = up(ctx, A), up(ctx, B), ctx.new_tensor((T, M, N)), ctx.new_tensor((T, M, N))
    ctx.sync()
    before = ctx.launch_count()
    ctx.gemm_batched(Ad, Bd, Cd, T, M, N, K, bias=up(ctx, bias), act="relu", preact_out=Pd)
    assert ctx.launch_count() - before == 1
    got, pre = ctx.to_numpy(Cd), ctx.to_numpy(Pd)
    dA, dB = ctx.new_tensor((T, M, K)), ctx.new_tensor((T, K, N))
    before = ctx.launch_count()
    ctx.gemm_batched_bwd(Ad, Bd, up(ctx, dY), T, M, N, K, act="relu", saved=Cd, dA=dA, dB=dB)
    assert ctx.launch_count() - before == 3
    gA, gB = ctx.to_numpy(dA), ctx.to_numpy(dB)
    for t in range(T):
        z = oracle.gemm(A[t], B[t])
        y, p = oracle.bias_act_fwd(z, bias, "relu")
        assert np.array_equal(got[t], y) and np.array_equal(pre[t], p), t
        dz = oracle.act_bwd(dY[t], y, "relu")
        assert np.array_equal(gA[t], oracle.gemm(dz, B[t], transB=True)), t
        assert np.array_equal(gB[t], oracle.gemm(A[t], dz, transA=True)), t


def test_gemm_batched_large_matrices_share_one_pairs_pass(ctx, oracle):
    # tensor-core sized products: the bf16 pairs of both operands are made once for the whole batch
    # (two launches), then one GEMM launch (+ its split-K fold, if any) per matrix
    T, M, N, K = 3, 512, 384, 256
    r = rng(1618)
    A, B = r.standard_normal((T, M, K), np.float32), r.standard_normal((T, K, N), np.float32) * 0.1
    bias = r.standard_normal(N, np.float32)
    Cd = ctx.new_tensor((T, M, N))
    Ad, Bd, bd = up(ctx, A), up(ctx, B), up(ctx, bias)
    ctx.sync()
    before = ctx.launch_count()
    ctx.gemm_batched(Ad, Bd, Cd, T, M, N, K, bias=bd, act="gelu")
    assert ctx.launch_count() - before <= 2 + 2 * T
    got = ctx.to_numpy(Cd)
    for t in range(T):
        y, _ = oracle.bias_act_fwd(oracle.gemm(A[t], B[t]), bias, "gelu")
        check(got[t], y, TOL_GEMM, f"batched output {t}")


@pytest.mark.parametrize("mode", ["simt", "3xtf32", "tf32_bf16x2"])
def test_reference_matmul_known_answers(ctx, mode):
    # crates/ferrograd/tests/std_wgsl.rs:268-373 (matmul_add) and :376-520 (matmul_chain3): constant
    # inputs, closed-form results, compared with ==.  Small integers are exact in TF32 too.
    def full(shape, v):
        return up(ctx, np.full(shape, v, np.float32))

    M, N, K = 32, 64, 16
    A, B = full((M, K), 3.0), full((K, N), 2.0)
    bias_full = np.full((M, N), 1.0, np.float32)
    X = ctx.new_tensor((M, N))
    ctx.gemm(A, B, X, M, N, K, mode=mode)
    assert (ctx.to_numpy(X) + bias_full == 97.0).all()
    dA, dB = ctx.new_tensor((M, K)), ctx.new_tensor((K, N))
    ctx.gemm_bwd(A, B, full((M, N), 1.0), M, N, K, dA=dA, dB=dB, mode=mode)
    assert (ctx.to_numpy(dA) == 128.0).all() and (ctx.to_numpy(dB) == 96.0).all()

    M, N, K, H = 32, 64, 128, 256
    A, B, Cc, D = full((M, K), 3.0), full((K, N), 2.0), full((H, M), 1.0), full((N, H), 0.5)
    X, Y, Z = ctx.new_tensor((M, N)), ctx.new_tensor((H, N)), ctx.new_tensor((H, H))
    ctx.gemm(A, B, X, M, N, K, mode=mode)
    ctx.gemm(Cc, X, Y, H, N, M, mode=mode)
    ctx.gemm(Y, D, Z, H, H, N, mode=mode)
    assert (ctx.to_numpy(X) == 768.0).all() and (ctx.to_numpy(Y) == 24576.0).all()
    assert (ctx.to_numpy(Z) == 786432.0).all()
    dY, dD = ctx.new_tensor((H, N)), ctx.new_tensor((N, H))
    ctx.gemm_bwd(Y, D, full((H, H), 1.0), H, H, N, dA=dY, dB=dD, mode=mode)
    dC, dX = ctx.new_tensor((H, M)), ctx.new_tensor((M, N))
    ctx.gemm_bwd(Cc, X, dY, H, N, M, dA=dC, dB=dX, mode=mode)
    dA, dB = ctx.new_tensor((M, K)), ctx.new_tensor((K, N))
    ctx.gemm_bwd(A, B, dX, M, N, K, dA=dA, dB=dB, mode=mode)
    y_grad, x_grad = 0.5 * H, 0.5 * H * H
    assert (ctx.to_numpy(dA) == x_grad * 2.0 * N).all() and (ctx.to_numpy(dB) == 3.0 * x_grad * M).all()
    assert (ctx.to_numpy(dC) == y_grad * 768.0 * N).all() and (ctx.to_numpy(dD) == 24576.0 * H).all()


def test_reference_softmax_known_answers(ctx):
    # std_wgsl.rs:97-187: softmax(C - A@B) = 1/64 exactly, gradients 0.
    A, B = up(ctx, np.full((16, 32), 3.0, np.float32)), up(ctx, np.full((32, 64), 2.0, np.float32))
    X = ctx.new_tensor((16, 64))
    ctx.gemm(A, B, X, 16, 64, 32, mode="simt")
    prog = [("input", 0, 0, 0.0), ("input", 1, 0, 0.0), ("sub", 0, 1, 0.0)]
    Q = ctx.new_tensor((16, 64))
    ctx.eltwise_chain_fwd(prog, [up(ctx, np.ones((16, 64), np.float32)), X], Q, 16 * 64)
    Y = ctx.new_tensor((16, 64))
    ctx.softmax_fwd(Q, Y, 16, 64)
    assert (ctx.to_numpy(Y) == np.float32(1.0) / np.float32(64.0)).all()
    dQ = ctx.new_tensor((16, 64), zeroed=True)
    ctx.softmax_bwd(Y, up(ctx, np.ones((16, 64), np.float32)), dQ, 16, 64, accumulate=True)
    assert (ctx.to_numpy(dQ) == 0.0).all()


# ---------------------------------------------------------------- boundary behaviour
def test_invalid_arguments_are_rejected(ctx):
    from ferrograd_b200 import FgError
    t = ctx.new_tensor((16,))
    with pytest.raises(FgError) as e:
        ctx.gemm(t, t, t, 0, 4, 4)
    assert e.value.kind == "FG_ERR_INVALID_ARGUMENT"
    with pytest.raises(FgError):
        ctx.sgd_step(t.ptr + 4, t, 3, 0.1)            # misaligned pointer
    with pytest.raises(FgError):
        ctx.upload(t, np.zeros(17, np.float32))        # larger than the buffer
    with pytest.raises(FgError):
        ctx.eltwise_chain_fwd([("add", 0, 1, 0.0)], [t], t, 16)   # operands name later values
    ctx.sync()


def test_plan_capture_and_replay(ctx, oracle):
    n = 4096
    r = rng(123)
    w, g = r.standard_normal(n, np.float32), r.standard_normal(n, np.float32)
    dw, dg = up(ctx, w), up(ctx, g)
    before = ctx.launch_count()
    ctx.plan_begin()
    ctx.sgd_step(dw, dg, n, 0.01, zero_grad=False)
    plan = ctx.plan_end()
    assert ctx.launch_count() == before                # recorded, not executed
    for _ in range(3):
        plan.launch()
        oracle.sgd(w, g, 0.01, zero_grad=False)
    ctx.sync()
    assert ctx.launch_count() == before + 3
    assert np.array_equal(ctx.to_numpy(dw), w)
    plan.destroy()


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_survives(ctx, oracle):
    # the wait routine of the GEMM kernels, on a barrier nobody arrives on, with a short limit: the kernel returns,
    # fg_sync reports FG_ERR_TIMEOUT once, the status word is clear afterwards and a GEMM runs normally
    from ferrograd_b200 import FgError
    assert ctx.device_status() == 0
    ctx._check(ctx.lib.fg_selftest_bounded_wait(ctx.handle, 20000))
    with pytest.raises(FgError) as e:
        ctx.sync()
    assert e.value.kind == "FG_ERR_TIMEOUT"
    ctx.sync()                                   # reported once, then clear
    assert ctx.device_status() == 0
    M, N, K = 256, 384, 512
    r = rng(9)
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32)
    Cd = ctx.new_tensor((M, N))
    ctx.gemm(up(ctx, A), up(ctx, B), Cd, M, N, K)
    check(ctx.to_numpy(Cd), oracle.gemm(A, B), TOL_GEMM, "GEMM after an expired wait")
    assert ctx.device_status() == 0


def test_a_plan_recorded_before_the_scratch_arena_moved_is_refused(oracle):
    # A recorded plan carries addresses inside the scratch arena.  A later, larger eager call reallocates the arena;
    # replaying the old plan would touch freed memory, so fg_plan_launch refuses it.
    from ferrograd_b200 import FgError, GpuContext
    c = GpuContext(0)
    try:
        r = rng(10)
        M, N, K = 200, 72, 100                                      # a shape that goes through operand planes (scratch)
        A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32)
        Ad, Bd, Cd = up(c, A), up(c, B), c.new_tensor((M, N))
        c.gemm(Ad, Bd, Cd, M, N, K, mode="3xtf32")                  # sizes the arena
        c.plan_begin()
        c.gemm(Ad, Bd, Cd, M, N, K, mode="3xtf32")
        plan = c.plan_end()
        plan.launch()
        c.sync()
        check(c.to_numpy(Cd), oracle.gemm(A, B), TOL_GEMM, "replayed GEMM")
        big = 1024
        X, Y = up(c, r.standard_normal((big, big), np.float32)), up(c, r.standard_normal((big, big), np.float32))
        c.gemm(X, Y, c.new_tensor((big, big)), big, big, big, mode="3xtf32")    # needs a larger arena: it is reallocated
        with pytest.raises(FgError) as e:
            plan.launch()
        assert e.value.kind == "FG_ERR_INCONSISTENT_CAPTURE"
        c.sync()
        assert c.device_status() == 0
        plan.destroy()
    finally:
        c.destroy()
