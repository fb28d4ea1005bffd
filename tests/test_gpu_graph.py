"""The reference's own integration tests, restated through the mirrored graph API
(Graph / define_ops / alloc_tensors / schedule / dispatch_*), with the same constant inputs and
the same closed-form expectations compared with `==`
(crates/ferrograd/tests/std_wgsl.rs, crates/ferrograd/tests/optim.rs), plus graph-level parity of
training steps against the CPU oracle."""
import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from ferrograd_b200 import GpuContext
    c = GpuContext.new()
    yield c
    c.sync()
    c.destroy()


def full(ctx, shape, v):
    return ctx.init_tensor_f32(shape, np.full(shape, v, np.float32))


def dl(ctx, buf, shape):
    return ctx.download(buf, np.empty(shape, np.float32))


def build(ctx, define, meta_vals, loss=None, optim=None, lr=1e-3, gemm_mode="auto", state=()):
    from ferrograd_b200 import MEAN_SQUARED_ERROR, Graph, Metadata, Optim, f32_bits
    meta = Metadata.new()
    fields = [meta.new_field() for _ in meta_vals]
    opt = optim or Optim.sgd()
    graph = Graph.new(MEAN_SQUARED_ERROR if loss is None else loss, opt.lower)
    define(graph.define_ops(), *fields)
    saved = graph.compute_saved_nodes()
    graph.validate(meta)
    binding = [f32_bits(lr)] + list(meta_vals)
    assert meta.validate_meta(binding)
    tensors = ctx.alloc_tensors(graph, saved, ctx.alloc_meta(binding), state or opt.state, gemm_mode=gemm_mode)
    kernels = ctx.compile(graph.lower(meta, None, saved), None)
    return graph, tensors, kernels, binding


@pytest.mark.parametrize("gemm_mode", ["auto", "simt"])
def test_mul_add_forward_backward(ctx, gemm_mode):
    # std_wgsl.rs:10-94
    def define(g, m, n):
        a, b, c = g.input([m, n]), g.input([m, n]), g.input([m, n])
        g.add(c, g.mul(a, b))
    graph, t, kernels, binding = build(ctx, define, [32, 32], gemm_mode=gemm_mode)
    ins = [full(ctx, (32, 32), 3.0), full(ctx, (32, 32), 2.0), full(ctx, (32, 32), 1.0)]
    ctx.upload(t.seed, np.ones(1024, np.float32))
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    ctx.sync()
    assert (dl(ctx, t.forward_out, 1024) == 7.0).all()
    assert (dl(ctx, t.grad_tensors[0], 1024) == 2.0).all()
    assert (dl(ctx, t.grad_tensors[1], 1024) == 3.0).all()
    assert (dl(ctx, t.grad_tensors[2], 1024) == 1.0).all()
    assert t.forward_steps() == 1          # the whole elementwise graph is one kernel
    t.destroy()


@pytest.mark.parametrize("gemm_mode", ["auto", "simt", "3xtf32", "tf32_bf16x2"])
def test_matmul_add_forward_backward(ctx, gemm_mode):
    # std_wgsl.rs:268-373
    M, N, K = 32, 64, 16

    def define(g, m, n, k):
        a, b, c = g.input([m, k]), g.input([k, n]), g.input([m, n])
        g.add(g.matmul(a, b), c)
    graph, t, kernels, binding = build(ctx, define, [M, N, K], gemm_mode=gemm_mode)
    ins = [full(ctx, (M, K), 3.0), full(ctx, (K, N), 2.0), full(ctx, (M, N), 1.0)]
    ctx.upload(t.seed, np.ones(M * N, np.float32))
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    ctx.sync()
    assert (dl(ctx, t.forward_out, M * N) == 3.0 * 2.0 * K + 1.0).all()
    assert (dl(ctx, t.grad_tensors[0], M * K) == 2.0 * N).all()
    assert (dl(ctx, t.grad_tensors[1], K * N) == 3.0 * M).all()
    assert (dl(ctx, t.grad_tensors[2], M * N) == 1.0).all()
    t.destroy()


@pytest.mark.parametrize("gemm_mode", ["auto", "simt"])
def test_matmul_sub_forward_backward(ctx, gemm_mode):
    # std_wgsl.rs:523-653: out = A@B - C@D
    M, N, K = 32, 64, 128

    def define(g, m, n, k):
        a, b, c, d = g.input([m, k]), g.input([k, n]), g.input([m, k]), g.input([k, n])
        g.sub(g.matmul(a, b), g.matmul(c, d))
    graph, t, kernels, binding = build(ctx, define, [M, N, K], gemm_mode=gemm_mode)
    ins = [full(ctx, (M, K), 3.0), full(ctx, (K, N), 2.0), full(ctx, (M, K), 1.0), full(ctx, (K, N), 0.5)]
    ctx.upload(t.seed, np.ones(M * N, np.float32))
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    ctx.sync()
    assert (dl(ctx, t.forward_saved[0], M * N) == 768.0).all()
    assert (dl(ctx, t.forward_saved[1], M * N) == 64.0).all()
    assert (dl(ctx, t.forward_out, M * N) == 704.0).all()
    for i, v in enumerate((128.0, 96.0, -32.0, -32.0)):
        g = dl(ctx, t.grad_tensors[i], ins[i].size)
        assert (g == v).all(), (i, g[:4])
    t.destroy()


@pytest.mark.parametrize("gemm_mode", ["auto", "simt", "3xtf32"])
def test_matmul_chain3_forward_backward(ctx, gemm_mode):
    # std_wgsl.rs:376-520: out = ((C @ (A @ B)) @ D) + E
    M, N, K, H = 32, 64, 128, 256

    def define(g, m, n, k, h):
        a, b, c, d, e = g.input([m, k]), g.input([k, n]), g.input([h, m]), g.input([n, h]), g.input([h, h])
        x = g.matmul(a, b)
        y = g.matmul(c, x)
        z = g.matmul(y, d)
        g.add(z, e)
    graph, t, kernels, binding = build(ctx, define, [M, N, K, H], gemm_mode=gemm_mode)
    ins = [full(ctx, (M, K), 3.0), full(ctx, (K, N), 2.0), full(ctx, (H, M), 1.0), full(ctx, (N, H), 0.5),
           full(ctx, (H, H), 1.0)]
    ctx.upload(t.seed, np.ones(H * H, np.float32))
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    ctx.sync()
    X, Y, Z = 3.0 * 2.0 * K, 1.0 * 768.0 * M, 24576.0 * 0.5 * N
    assert (dl(ctx, t.forward_saved[0], M * N) == X).all()
    assert (dl(ctx, t.forward_saved[1], H * N) == Y).all()
    assert (dl(ctx, t.forward_saved[2], H * H) == Z).all()
    assert (dl(ctx, t.forward_out, H * H) == Z + 1.0).all()
    y_grad = 0.5 * H
    x_grad = y_grad * 1.0 * H
    expect = [x_grad * 2.0 * N, 3.0 * x_grad * M, y_grad * X * N, Y * H, 1.0]   # std_wgsl.rs:387-395
    for i, v in enumerate(expect):
        assert (dl(ctx, t.grad_tensors[i], ins[i].size) == v).all(), i
    t.destroy()


def test_matmul_sub_softmax(ctx):
    # std_wgsl.rs:97-187: softmax(C - A@B) = 1/64 exactly; every gradient 0
    M, N, K = 16, 64, 32

    def define(g, m, n, k):
        a, b, c = g.input([m, k]), g.input([k, n]), g.input([m, n])
        g.softmax(g.sub(c, g.matmul(a, b)))
    graph, t, kernels, binding = build(ctx, define, [M, N, K], gemm_mode="simt")
    ins = [full(ctx, (M, K), 3.0), full(ctx, (K, N), 2.0), full(ctx, (M, N), 1.0)]
    ctx.upload(t.seed, np.ones(M * N, np.float32))
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    ctx.sync()
    assert (dl(ctx, t.forward_out, M * N) == np.float32(1.0) / np.float32(64.0)).all()
    for i in range(3):
        assert (dl(ctx, t.grad_tensors[i], ins[i].size) == 0.0).all()
    t.destroy()


def test_div_const_softmax(ctx):
    # std_wgsl.rs:190-265: softmax(2 / x) + 2 with x = 3 -> 2 + 1/32; dx = 0
    def define(g, m, n):
        x = g.input([m, n])
        two = g.constant_f32(2.0)
        g.add(g.softmax(g.div(two, x)), two)
    graph, t, kernels, binding = build(ctx, define, [16, 32])
    ins = [full(ctx, (16, 32), 3.0)]
    ctx.upload(t.seed, np.ones(512, np.float32))
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    ctx.sync()
    assert (dl(ctx, t.forward_out, 512) == np.float32(2.0) + np.float32(1.0) / np.float32(32.0)).all()
    assert (dl(ctx, t.grad_tensors[0], 512) == 0.0).all()
    t.destroy()


@pytest.mark.parametrize("separate", [False, True])
def test_mul_add_optim(ctx, separate):
    # tests/optim.rs:10-104 (dispatch_optim) and :107-207 (dispatch_single_optim)
    def define(g, m, n):
        a, b, c = g.input([m, n]), g.input([m, n]), g.input([m, n])
        g.add(c, g.mul(a, b))
    graph, t, kernels, binding = build(ctx, define, [32, 32], lr=1e-3)
    ins = [full(ctx, (32, 32), 3.0), full(ctx, (32, 32), 2.0), full(ctx, (32, 32), 1.0)]
    ctx.upload(t.seed, np.ones(1024, np.float32))
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    if separate:
        for i in range(3):
            ctx.dispatch_single_optim(sch, ins[i], i, t)
    else:
        ctx.dispatch_optim(sch)
    ctx.sync()
    f32 = np.float32
    assert (dl(ctx, t.forward_out, 1024) == 7.0).all()
    for i in range(3):
        assert (dl(ctx, t.grad_tensors[i], 1024) == 0.0).all()
    assert (ctx.to_numpy(ins[0]) == f32(3.0) - f32(2e-3)).all()
    assert (ctx.to_numpy(ins[1]) == f32(2.0) - f32(3e-3)).all()
    assert (ctx.to_numpy(ins[2]) == f32(1.0) - f32(1e-3)).all()
    t.destroy()


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_mul_add_f16(ctx, dtype):
    # crates/ferrograd/tests/nonf32.rs:10-99 (f16; the same constants are exact in bf16): inputs declared
    # with SimpleDType::F16, tensors from init_tensor_f16, the seed uploaded as f16, results compared with ==.
    from ferrograd_b200 import SimpleDType
    from ferrograd_b200.backend import from_bf16_bits, to_bf16_bits
    sd = SimpleDType.F16 if dtype == "f16" else SimpleDType.BF16

    def define(g, m, n):
        a, b, c = g.input([m, n], sd), g.input([m, n], sd), g.input([m, n], sd)
        g.add(c, g.mul(a, b))
    graph, t, kernels, binding = build(ctx, define, [32, 32])
    init = ctx.init_tensor_f16 if dtype == "f16" else ctx.init_tensor_bf16
    ins = [init((32, 32), np.full((32, 32), v, np.float32)) for v in (3.0, 2.0, 1.0)]
    ones = np.ones(1024, np.float32)
    ctx.upload(t.seed, ones.astype(np.float16) if dtype == "f16" else to_bf16_bits(ones))
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    ctx.sync()

    def dl16(buf):
        raw = ctx.download(buf, np.empty(1024, np.float16 if dtype == "f16" else np.uint16))
        return raw.astype(np.float32) if dtype == "f16" else from_bf16_bits(raw)
    assert (dl16(t.forward_out) == 7.0).all()
    assert (dl16(t.grad_tensors[0]) == 2.0).all()
    assert (dl16(t.grad_tensors[1]) == 3.0).all()
    assert (dl16(t.grad_tensors[2]) == 1.0).all()
    # SGD in the storage type: w -= lr*g with every result rounded; gradients zeroed
    ctx.dispatch_optim(sch)
    ctx.sync()
    lr = np.float32(1e-3)
    for i, (w, g) in enumerate(((3.0, 2.0), (2.0, 3.0), (1.0, 1.0))):
        if dtype == "f16":
            expect = np.float32(np.float16(w) - np.float16(np.float16(g) * np.float16(lr)))
            got = ctx.to_numpy(ins[i]).astype(np.float32)
        else:
            rb = lambda x: from_bf16_bits(to_bf16_bits(np.array([x], np.float32)))[0]
            expect = rb(np.float32(w) - rb(np.float32(g) * rb(lr)))
            got = from_bf16_bits(ctx.to_numpy(ins[i]))
        assert (got == expect).all(), (i, got.ravel()[0], expect)
        assert (dl16(t.grad_tensors[i]) == 0.0).all()
    t.destroy()


def test_16bit_graph_rejects_adamw(ctx):
    from ferrograd_b200 import FgError, Optim, SimpleDType

    def define(g, m):
        a = g.input([m, m], SimpleDType.F16)
        g.tanh(a)
    graph, t, kernels, binding = build(ctx, define, [32], optim=Optim.adamw())
    ins = [ctx.init_tensor_f16((32, 32), np.ones((32, 32), np.float32))]
    sch = ctx.schedule(kernels, binding, ins, t, [], Optim.adamw().state)
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    with pytest.raises(FgError):
        ctx.dispatch_optim(sch)
    t.destroy()


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("loss_name", ["mse", "ce"])
def test_16bit_classifier_step(ctx, oracle, dtype, loss_name):
    """softmax(x @ W + b) stored in 16 bits, loss, backward and one SGD step: softmax and the loss are computed
    in f32 on widened copies and rounded back.  Checked against the same chain in float64 on the rounded inputs;
    the bar is a few units of the storage type's precision (every stored tensor is rounded once)."""
    from ferrograd_b200 import CROSS_ENTROPY, MEAN_SQUARED_ERROR, Optim, SimpleDType
    from ferrograd_b200.backend import from_bf16_bits, to_bf16_bits
    sd = SimpleDType.F16 if dtype == "f16" else SimpleDType.BF16
    tol = 4 * (2.0 ** -10 if dtype == "f16" else 2.0 ** -7)
    Bn, I, O = 64, 40, 16
    r = np.random.Generator(np.random.Philox(91))
    x = oracle.round_to(r.standard_normal((Bn, I), np.float32), dtype)
    W = oracle.round_to(r.standard_normal((I, O), np.float32) * 0.3, dtype)
    b = oracle.round_to(r.standard_normal(O, np.float32) * 0.1, dtype)
    ce = loss_name == "ce"

    def define(g, fb, fi, fo):
        xi, w, bb = g.input([fb, fi], sd), g.input([fi, fo], sd), g.input([fo], sd)
        g.softmax(g.add(g.matmul(xi, w), bb))
    graph, t, kernels, binding = build(ctx, define, [Bn, I, O], loss=CROSS_ENTROPY if ce else MEAN_SQUARED_ERROR,
                                       optim=Optim.sgd(), lr=0.5)
    init = ctx.init_tensor_f16 if dtype == "f16" else ctx.init_tensor_bf16
    dec = (lambda a: a.astype(np.float32)) if dtype == "f16" else from_bf16_bits
    raw = np.float16 if dtype == "f16" else np.uint16
    get = lambda buf, shape: dec(ctx.download(buf, np.empty(shape, raw)))
    ins = [init(a.shape, a) for a in (x, W, b)]
    sch = ctx.schedule(kernels, binding, ins, t, [], (), trainable=[0, 1, 1])
    if ce:
        labels = r.integers(0, O, Bn).astype(np.uint32)
        target = ctx.new_onehot_init(labels)
        tgt = np.eye(O, dtype=np.float64)[labels]
    else:
        tg = oracle.round_to(r.random((Bn, O)).astype(np.float32), dtype)
        target = init(tg.shape, tg)
        tgt = tg.astype(np.float64)
    ctx.dispatch_forward(sch)
    ctx.dispatch_loss(sch, target)
    ctx.dispatch_backward(sch)
    ctx.sync()
    z = x.astype(np.float64) @ W.astype(np.float64) + b
    ez = np.exp(z - z.max(axis=1, keepdims=True))
    p = ez / ez.sum(axis=1, keepdims=True)
    if ce:
        loss = np.where(tgt > 0, -np.log(p), 0.0)
        dz = p - tgt                                     # softmax + CE: p - onehot is dL/dlogits
    else:
        loss = (p - tgt) ** 2
        seed = 2 * (p - tgt)
        dz = p * (seed - (seed * p).sum(axis=1, keepdims=True))
    grads = {n: t.grad_tensors[i] for i, n in enumerate(t.grad_nodes)}
    for got, ref, what in ((get(t.forward_out, (Bn, O)), p, "probabilities"), (get(t.loss_t, (Bn, O)), loss, "loss"),
                           (get(grads[1], (I, O)), x.astype(np.float64).T @ dz, "dW"),
                           (get(grads[2], (O,)), dz.sum(axis=0), "db")):
        ok, worst = rel_err_ok(got, ref, tol)
        assert ok, f"{what}: {worst:.3g} x {tol}"
    gW = get(grads[1], (I, O))
    ctx.dispatch_optim(sch)
    ctx.sync()
    lr = oracle.round_to(np.array([0.5], np.float32), dtype)[0]
    expect = oracle.round_to(W - oracle.round_to(gW * lr, dtype), dtype)      # SGD in the storage type, exactly
    assert np.array_equal(dec(ctx.to_numpy(ins[1])), expect)
    assert np.array_equal(dec(ctx.to_numpy(ins[0])), x)
    t.destroy()


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_16bit_dense_layer_graph(ctx, oracle, dtype):
    """tanh(x @ W + b) with every tensor stored in 16 bits: the fused GEMM runs on the 16-bit operands with f32
    accumulation; outputs and gradients are rounded once to the storage type."""
    from ferrograd_b200 import SimpleDType
    from ferrograd_b200.backend import from_bf16_bits, to_bf16_bits
    sd = SimpleDType.F16 if dtype == "f16" else SimpleDType.BF16
    tol = 2.0 ** -10 if dtype == "f16" else 2.0 ** -7
    Bn, I, O = 64, 40, 72
    r = np.random.Generator(np.random.Philox(55))
    x = oracle.round_to(r.standard_normal((Bn, I), np.float32), dtype)
    W = oracle.round_to(r.standard_normal((I, O), np.float32) * 0.2, dtype)
    b = oracle.round_to(r.standard_normal(O, np.float32) * 0.1, dtype)
    seed = oracle.round_to(r.standard_normal((Bn, O), np.float32), dtype)

    def define(g, fb, fi, fo):
        xi, w, bb = g.input([fb, fi], sd), g.input([fi, fo], sd), g.input([fo], sd)
        g.tanh(g.add(g.matmul(xi, w), bb))
    graph, t, kernels, binding = build(ctx, define, [Bn, I, O])
    assert t.forward_steps() == 1
    init = ctx.init_tensor_f16 if dtype == "f16" else ctx.init_tensor_bf16
    enc = (lambda a: a.astype(np.float16)) if dtype == "f16" else to_bf16_bits
    dec = (lambda a: a.astype(np.float32)) if dtype == "f16" else from_bf16_bits
    ins = [init(a.shape, a) for a in (x, W, b)]
    ctx.upload(t.seed, enc(seed))
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    ctx.sync()
    raw = np.float16 if dtype == "f16" else np.uint16
    get = lambda buf, shape: dec(ctx.download(buf, np.empty(shape, raw)))
    y, _ = oracle.bias_act_fwd(oracle.gemm(x, W, f64=True), b, "tanh")
    y16 = oracle.round_to(y, dtype)
    ok, worst = rel_err_ok(get(t.forward_out, (Bn, O)), y, tol)
    assert ok, f"output: {worst:.3g} x {tol}"
    dz = oracle.round_to(oracle.act_bwd(seed, get(t.forward_out, (Bn, O)), "tanh"), dtype)
    grads = {n: t.grad_tensors[i] for i, n in enumerate(t.grad_nodes)}
    for got, ref, what in ((get(grads[0], (Bn, I)), oracle.gemm(dz, W, transB=True, f64=True), "dx"),
                           (get(grads[1], (I, O)), oracle.gemm(x, dz, transA=True, f64=True), "dW"),
                           (get(grads[2], (O,)), dz.astype(np.float64).sum(axis=0), "db")):
        ok, worst = rel_err_ok(got, ref, 2 * tol)
        assert ok, f"{what}: {worst:.3g} x {2 * tol}"
    assert y16.shape == (Bn, O)
    t.destroy()


# ---------------------------------------------------------------- beyond the reference's tests
@pytest.mark.parametrize("act,loss_name", [("tanh", "mse"), ("gelu", "ce"), ("relu", "ce")])
def test_mlp_graph_matches_oracle(ctx, oracle, act, loss_name):
    """A two-layer MLP written as a graph (matmul, + bias, activation, matmul, + bias [, softmax]) takes the
    fused GEMM path and matches the oracle's forward, loss gradient, parameter gradients and SGD update."""
    from ferrograd_b200 import CROSS_ENTROPY, MEAN_SQUARED_ERROR, Optim
    B, I, Hd, O = 96, 40, 72, 10
    r = np.random.Generator(np.random.Philox(5))
    x = r.standard_normal((B, I), np.float32)
    W = [r.standard_normal((I, Hd), np.float32) * 0.3, r.standard_normal((Hd, O), np.float32) * 0.3]
    b = [r.standard_normal(Hd, np.float32) * 0.1, r.standard_normal(O, np.float32) * 0.1]
    ce = loss_name == "ce"

    def define(g, fb, fi, fh, fo):
        xi, w0, b0, w1, b1 = g.input([fb, fi]), g.input([fi, fh]), g.input([fh]), g.input([fh, fo]), g.input([fo])
        h = getattr(g, act)(g.add(g.matmul(xi, w0), b0))
        o = g.add(g.matmul(h, w1), b1)
        if ce:
            g.softmax(o)
    graph, t, kernels, binding = build(ctx, define, [B, I, Hd, O], loss=CROSS_ENTROPY if ce else MEAN_SQUARED_ERROR,
                                       optim=Optim.sgd(), lr=0.05, gemm_mode="3xtf32")
    assert t.forward_steps() == (3 if ce else 2)       # two fused GEMMs (+ softmax)
    ins = [ctx.init_tensor_f32(a.shape, a) for a in (x, W[0], b[0], W[1], b[1])]
    sch = ctx.schedule(kernels, binding, ins, t, [], (), trainable=[0, 1, 1, 1, 1])
    if ce:
        labels = r.integers(0, O, B).astype(np.uint32)
        target = ctx.new_onehot_init(labels)
    else:
        labels = r.standard_normal((B, O), np.float32)
        target = ctx.init_tensor_f32(labels.shape, labels)
    ctx.dispatch_forward(sch)
    ctx.dispatch_loss(sch, target)
    ctx.dispatch_backward(sch)
    ctx.sync()
    grads = {n: dl(ctx, t.grad_tensors[i], ins[n].size) for i, n in enumerate(t.grad_nodes) if n < 5}
    ctx.dispatch_optim(sch)
    ctx.sync()
    Wc, bc = [w.copy() for w in W], [v.copy() for v in b]
    loss, gW, gb, out = oracle.mlp_step([I, Hd, O], B, act, Wc, bc, x, labels, loss_name, 1.0, ("sgd", 0.05))
    got_out = dl(ctx, t.forward_out, B * O).reshape(B, O)
    ref_out = oracle.softmax_fwd(out) if ce else out
    for got, ref, what in ((got_out, ref_out, "output"), (grads[1].reshape(I, Hd), gW[0], "dW0"), (grads[2], gb[0], "db0"),
                           (grads[3].reshape(Hd, O), gW[1], "dW1"), (grads[4], gb[1], "db1"),
                           (ctx.to_numpy(ins[1]), Wc[0], "W0 after SGD"), (ctx.to_numpy(ins[3]), Wc[1], "W1 after SGD")):
        ok, worst = rel_err_ok(got, ref, 1e-4)
        assert ok, f"{what}: {worst:.3g} x 1e-4"
    assert np.array_equal(ctx.to_numpy(ins[0]), x)      # the data input is not trainable
    t.destroy()


def test_replayed_dispatches_equal_eager(ctx):
    """From its second call on, every dispatch_* replays a recorded CUDA graph.  Five training steps with new
    data each step end with bit-identical parameters whether the dispatches are replayed or run eagerly, also
    after the loss target moves to another buffer."""
    from ferrograd_b200 import CROSS_ENTROPY, Optim
    B, I, Hd, O = 128, 48, 136, 10
    r = np.random.Generator(np.random.Philox(77))
    W = [r.standard_normal((I, Hd), np.float32) * 0.2, r.standard_normal((Hd, O), np.float32) * 0.2]
    b = [np.zeros(Hd, np.float32), np.zeros(O, np.float32)]
    xs = [r.standard_normal((B, I), np.float32) for _ in range(5)]
    ls = [r.integers(0, O, B).astype(np.uint32) for _ in range(5)]

    def define(g, fb, fi, fh, fo):
        xi, w0, b0, w1, b1 = g.input([fb, fi]), g.input([fi, fh]), g.input([fh]), g.input([fh, fo]), g.input([fo])
        g.softmax(g.add(g.matmul(g.gelu(g.add(g.matmul(xi, w0), b0)), w1), b1))

    def train(eager):
        ctx.set_option("exec_plans", "0" if eager else "1")
        graph, t, kernels, binding = build(ctx, define, [B, I, Hd, O], loss=CROSS_ENTROPY, optim=Optim.adamw(),
                                           lr=1e-2)
        ins = [ctx.init_tensor_f32(a.shape, a) for a in (xs[0], W[0], b[0], W[1], b[1])]
        sch = ctx.schedule(kernels, binding, ins, t, [], Optim.adamw().state, trainable=[0, 1, 1, 1, 1])
        targets = [ctx.new_onehot_init(ls[0]), ctx.new_onehot_init(ls[0])]
        for step in range(5):
            ctx.upload(ins[0], xs[step])
            tgt = targets[0 if step < 3 else 1]          # the target moves: the loss plan is recorded again
            ctx.upload(tgt, ls[step])
            ctx.dispatch_forward(sch)
            ctx.dispatch_loss(sch, tgt)
            ctx.dispatch_backward(sch)
            ctx.dispatch_optim(sch)
        ctx.sync()
        out = [ctx.to_numpy(ins[i]).copy() for i in (1, 2, 3, 4)]
        t.destroy()
        return out
    try:
        for got, ref in zip(train(eager=False), train(eager=True)):
            assert np.array_equal(got, ref)
        assert not np.array_equal(train(eager=False)[0], W[0])       # and training moved the weights
    finally:
        ctx.set_option("exec_plans", "auto")


def test_binary_cross_entropy_graph(ctx, oracle):
    """p = 1 / (1 + exp(-x)) built from graph ops, BINARY_CROSS_ENTROPY against soft and hard targets:
    loss_t holds the per-element loss, the seed is p - t (loss/basic_loss.rs:81-85), and the backward
    pass carries it through the sigmoid's own derivative."""
    from ferrograd_b200 import BINARY_CROSS_ENTROPY
    R, Cn = 64, 48
    r = np.random.Generator(np.random.Philox(21))
    x = (r.standard_normal((R, Cn)) * 1.5).astype(np.float32)
    tgt = (r.random((R, Cn)) < 0.4).astype(np.float32)
    tgt[:8] = r.random((8, Cn)).astype(np.float32)

    def define(g, fr, fc):
        xi = g.input([fr, fc])
        g.div(g.constant_f32(1.0), g.add(g.constant_f32(1.0), g.exp(g.neg(xi))))
    graph, t, kernels, binding = build(ctx, define, [R, Cn], loss=BINARY_CROSS_ENTROPY)
    ins = [ctx.init_tensor_f32(x.shape, x)]
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    target = ctx.init_tensor_f32(tgt.shape, tgt)
    ctx.dispatch_forward(sch)
    ctx.dispatch_loss(sch, target)
    ctx.dispatch_backward(sch)
    ctx.sync()
    x64, t64 = x.astype(np.float64), tgt.astype(np.float64)
    p64 = 1.0 / (1.0 + np.exp(-x64))
    got_p = dl(ctx, t.forward_out, x.size).reshape(R, Cn)
    ok, worst = rel_err_ok(got_p, p64, 1e-5)
    assert ok, f"sigmoid: {worst:.3g} x 1e-5"
    lref, _, gref = oracle.bce(got_p, tgt)
    ok, worst = rel_err_ok(ctx.to_numpy(t.loss_t).reshape(R, Cn), lref, 1e-5)
    assert ok, f"loss: {worst:.3g} x 1e-5"
    ok, worst = rel_err_ok(ctx.to_numpy(t.loss_t).reshape(R, Cn), -(t64 * np.log(p64) + (1 - t64) * np.log1p(-p64)), 1e-5)
    assert ok, f"loss vs float64: {worst:.3g} x 1e-5"
    assert np.array_equal(dl(ctx, t.seed, x.size).reshape(R, Cn), gref)
    ok, worst = rel_err_ok(dl(ctx, t.grad_tensors[0], x.size).reshape(R, Cn), (p64 - t64) * p64 * (1 - p64), 1e-5)
    assert ok, f"dx: {worst:.3g} x 1e-5"
    t.destroy()


@pytest.mark.parametrize("shared_b", [False, True])
def test_rank3_matmul_graph(ctx, oracle, shared_b):
    """[T,M,K] x [T,K,N] runs one product per leading index; [T,M,K] x [K,N] is one product with T*M rows.
    Forward and both gradients against the oracle, followed by an elementwise consumer."""
    T, M, K, Nn = 3, 48, 40, 56
    r = np.random.Generator(np.random.Philox(33))
    A = r.standard_normal((T, M, K), np.float32)
    B = (r.standard_normal((K, Nn) if shared_b else (T, K, Nn), np.float32) * 0.3).astype(np.float32)

    def define(g, ft, fm, fk, fn):
        a = g.input([ft, fm, fk])
        b = g.input([fk, fn]) if shared_b else g.input([ft, fk, fn])
        g.tanh(g.matmul(a, b))
    graph, t, kernels, binding = build(ctx, define, [T, M, K, Nn], gemm_mode="simt")
    ins = [ctx.init_tensor_f32(A.shape, A), ctx.init_tensor_f32(B.shape, B)]
    seed = r.standard_normal((T, M, Nn), np.float32)
    ctx.upload(t.seed, seed)
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    ctx.sync()
    Bt = [B if shared_b else B[i] for i in range(T)]
    Y = np.stack([np.tanh(oracle.gemm(A[i], Bt[i])) for i in range(T)])
    dZ = seed * (1.0 - Y * Y)
    dA = np.stack([oracle.gemm(dZ[i], Bt[i], transB=True) for i in range(T)])
    dB = [oracle.gemm(A[i], dZ[i], transA=True) for i in range(T)]
    dB = sum(dB) if shared_b else np.stack(dB)
    for got, ref, what in ((dl(ctx, t.forward_out, Y.size).reshape(Y.shape), Y, "output"),
                           (dl(ctx, t.grad_tensors[0], A.size).reshape(A.shape), dA, "dA"),
                           (dl(ctx, t.grad_tensors[1], B.size).reshape(B.shape), dB, "dB")):
        ok, worst = rel_err_ok(got, ref, 1e-4)
        assert ok, f"{what}: {worst:.3g} x 1e-4"
    t.destroy()


def test_fan_out_accumulates_gradients(ctx, oracle):
    """y = (a @ b) * tanh(a @ b): the matmul result has two consumers, a is used by one matmul only; and
    z = a @ a (both operands the same tensor) takes the accumulate path."""
    r = np.random.Generator(np.random.Philox(9))
    A = (r.standard_normal((48, 48), np.float32) * 0.2).astype(np.float32)

    def define(g, m):
        a = g.input([m, m])
        p = g.matmul(a, a)
        g.mul(p, g.tanh(p))
    graph, t, kernels, binding = build(ctx, define, [48], gemm_mode="simt")
    ins = [ctx.init_tensor_f32(A.shape, A)]
    seed = r.standard_normal((48, 48), np.float32)
    ctx.upload(t.seed, seed)
    sch = ctx.schedule(kernels, binding, ins, t, [], ())
    ctx.dispatch_forward(sch)
    ctx.dispatch_backward(sch)
    ctx.sync()
    P = oracle.gemm(A, A)
    T = np.tanh(P)
    dP = seed * (T + P * (1.0 - T * T))
    dA = oracle.gemm(dP, A, transB=True) + oracle.gemm(A, dP, transA=True)
    ok, worst = rel_err_ok(dl(ctx, t.forward_out, A.size).reshape(48, 48), P * T, 1e-5)
    assert ok, worst
    ok, worst = rel_err_ok(dl(ctx, t.grad_tensors[0], A.size).reshape(48, 48), dA, 1e-4)
    assert ok, f"dA with fan-out: {worst:.3g} x 1e-4"
    t.destroy()


def test_graph_errors_are_values(ctx):
    from ferrograd_b200 import FgError, Graph, MEAN_SQUARED_ERROR, Optim, f32_bits
    g = Graph.new(MEAN_SQUARED_ERROR, Optim.sgd().lower)
    ops = g.define_ops()
    a = ops.input([1, 2])
    b = ops.input([2, 1])
    with pytest.raises(FgError):
        ops.add(a, 99)                         # UnresolvedInput
    ops.add(a, b)                              # shapes differ: rejected when the tensors are allocated
    with pytest.raises(FgError) as e:
        ctx.alloc_tensors(g, g.compute_saved_nodes(), [f32_bits(0.1), 4, 8])
    assert e.value.kind == "FG_ERR_INVALID_ARGUMENT"
    empty = Graph.new(MEAN_SQUARED_ERROR, Optim.sgd().lower)
    with pytest.raises(FgError):
        ctx.alloc_tensors(empty, None, [f32_bits(0.1)])
