"""Pins the CPU oracle to the known answers of the reference's own tests.

Each case rebuilds the inputs of one reference test (constant-filled tensors) and
compares with `==` against the closed-form constants that test asserts
(crates/ferrograd/tests/std_wgsl.rs, crates/ferrograd/tests/optim.rs).
"""
import numpy as np

f32 = np.float32


def full(shape, v):
    return np.full(shape, v, dtype=np.float32)


def test_mul_add(oracle):
    # std_wgsl.rs:10-94: out = c + a*b on [32,32]; seed = 1.
    a, b, c = full((32, 32), 3.0), full((32, 32), 2.0), full((32, 32), 1.0)
    prog = [("input", 0, 0, 0.0), ("input", 1, 0, 0.0), ("input", 2, 0, 0.0),
            ("mul", 0, 1, 0.0), ("add", 2, 3, 0.0)]
    out, _ = oracle.eltwise_fwd(prog, [a, b, c])
    assert (out == 7.0).all()
    da, db, dc = oracle.eltwise_bwd(prog, [a, b, c], full((32, 32), 1.0))
    assert (da == 2.0).all() and (db == 3.0).all() and (dc == 1.0).all()


def test_matmul_add(oracle):
    # std_wgsl.rs:268-373: A[32,16]=3, B[16,64]=2, C[32,64]=1; out = A@B + C.
    M, N, K = 32, 64, 16
    A, B, Cc = full((M, K), 3.0), full((K, N), 2.0), full((M, N), 1.0)
    out = oracle.gemm(A, B) + Cc
    assert (out == 3.0 * 2.0 * K + 1.0).all()
    seed = full((M, N), 1.0)
    dA = oracle.gemm(seed, B, transB=True)
    dB = oracle.gemm(A, seed, transA=True)
    assert (dA == 2.0 * N).all() and (dB == 3.0 * M).all()


def test_matmul_sub(oracle):
    # std_wgsl.rs:523-653: out = A@B - C@D.
    A, C_ = full((32, 128), 3.0), full((32, 128), 1.0)
    B, D = full((128, 64), 2.0), full((128, 64), 0.5)
    X, Y = oracle.gemm(A, B), oracle.gemm(C_, D)
    assert (X == 768.0).all() and (Y == 64.0).all() and ((X - Y) == 704.0).all()
    seed = full((32, 64), 1.0)
    assert (oracle.gemm(seed, B, transB=True) == 128.0).all()
    assert (oracle.gemm(A, seed, transA=True) == 96.0).all()
    assert (oracle.gemm(-seed, D, transB=True) == -32.0).all()
    assert (oracle.gemm(C_, -seed, transA=True) == -32.0).all()


def test_matmul_chain3(oracle):
    # std_wgsl.rs:376-520: out = ((C@(A@B))@D) + E.
    M, N, K, H = 32, 64, 128, 256
    A, B = full((M, K), 3.0), full((K, N), 2.0)
    Cc, D, E = full((H, M), 1.0), full((N, H), 0.5), full((H, H), 1.0)
    X = oracle.gemm(A, B)
    Y = oracle.gemm(Cc, X)
    Z = oracle.gemm(Y, D)
    assert (X == 768.0).all() and (Y == 24576.0).all() and (Z == 786432.0).all()
    assert ((Z + E) == 786433.0).all()
    seed = full((H, H), 1.0)
    dY = oracle.gemm(seed, D, transB=True)          # [H,N]
    dD = oracle.gemm(Y, seed, transA=True)          # [N,H]
    dX = oracle.gemm(Cc, dY, transA=True)           # [M,N]
    dC = oracle.gemm(dY, X, transB=True)            # [H,M]
    dA = oracle.gemm(dX, B, transB=True)
    dB = oracle.gemm(A, dX, transA=True)
    # Expected constants as the reference derives them (std_wgsl.rs:387-395).
    y_grad = 0.5 * H
    x_grad = y_grad * 1.0 * H
    assert (dA == x_grad * 2.0 * N).all() and (dB == 3.0 * x_grad * M).all()
    assert (dC == y_grad * 768.0 * N).all() and (dD == 24576.0 * H).all()


def test_matmul_sub_softmax(oracle):
    # std_wgsl.rs:97-187: softmax(C - A@B) is uniform -> 1/64 exactly; all grads 0.
    A, B, Cc = full((16, 32), 3.0), full((32, 64), 2.0), full((16, 64), 1.0)
    y = oracle.softmax_fwd(Cc - oracle.gemm(A, B))
    assert (y == f32(1.0) / f32(64.0)).all()
    dx = oracle.softmax_bwd(y, full((16, 64), 1.0))
    assert (dx == 0.0).all()


def test_div_const_softmax(oracle):
    # std_wgsl.rs:190-265: softmax(2/x) + 2 with x = 3 on [16,32] -> 2 + 1/32; dx = 0.
    x = full((16, 32), 3.0)
    prog = [("const", 0, 0, 2.0), ("input", 0, 0, 0.0), ("div", 0, 1, 0.0)]
    q, _ = oracle.eltwise_fwd(prog, [x])
    y = oracle.softmax_fwd(q) + f32(2.0)
    assert (y == f32(2.0) + f32(1.0) / f32(32.0)).all()
    dq = oracle.softmax_bwd(oracle.softmax_fwd(q), full((16, 32), 1.0))
    (dx,) = oracle.eltwise_bwd(prog, [x], dq)
    assert (dx == 0.0).all()


def test_mul_add_f16(oracle):
    # crates/ferrograd/tests/nonf32.rs:10-99: c + a*b in f16 with a, b, c = 3, 2, 1 -> 7; grads 2, 3, 1.
    prog = [("input", 0, 0, 0.0), ("input", 1, 0, 0.0), ("input", 2, 0, 0.0), ("mul", 0, 1, 0.0), ("add", 2, 3, 0.0)]
    for dtype in ("f16", "bf16"):
        out, _ = oracle.eltwise_fwd(prog, [full(1024, 3.0), full(1024, 2.0), full(1024, 1.0)], dtype=dtype)
        assert (out == 7.0).all()
        ga, gb, gc = oracle.eltwise_bwd(prog, [full(1024, 3.0), full(1024, 2.0), full(1024, 1.0)], full(1024, 1.0), dtype=dtype)
        assert (ga == 2.0).all() and (gb == 3.0).all() and (gc == 1.0).all()


def test_16bit_rounding(oracle):
    # the oracle's rounding against numpy's float16 cast and a bit-level bf16 rounding; and one f16 product
    # that differs from the f32 one: 0.1 * 0.3 in f16 arithmetic
    r = np.random.Generator(np.random.Philox(3))
    x = (r.standard_normal(100000) * 50).astype(np.float32)
    assert np.array_equal(oracle.round_to(x, "f16"), x.astype(np.float16).astype(np.float32))
    u = x.view(np.uint32)
    bf = (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)
    assert np.array_equal(oracle.round_to(x, "bf16"), bf)
    a, b = np.float16(0.1), np.float16(0.3)
    out, _ = oracle.eltwise_fwd([("input", 0, 0, 0.0), ("input", 1, 0, 0.0), ("mul", 0, 1, 0.0)],
                                [np.full(4, a, np.float32), np.full(4, b, np.float32)], dtype="f16")
    assert (out == np.float32(a * b)).all() and np.float32(a * b) != np.float32(a) * np.float32(b)


def test_bce_formulas(oracle):
    # loss/basic_loss.rs:29-89.  Hard targets at p = 1/2: the definition gives log 2 per element and the
    # gradient is p - t.  With reference_formula the loss is (1-t)*log(1-t) - t*log(p) as the file has it:
    # at t = 1/2, p = 1/4 that is 0.5*log(0.5) - 0.5*log(0.25) = 0.5*log 2.
    p, t = full(64, 0.5), np.concatenate([full(32, 0.0), full(32, 1.0)])
    loss, s, grad = oracle.bce(p, t)
    assert np.allclose(loss, np.log(2.0), rtol=1e-6) and abs(s - 64 * np.log(2.0)) < 1e-4
    assert (grad == p - t).all()
    loss_q, _, grad_q = oracle.bce(full(8, 0.25), full(8, 0.5), reference_formula=True)
    assert np.allclose(loss_q, 0.5 * np.log(2.0), rtol=1e-6)
    assert (grad_q == f32(-0.25)).all()


def test_mul_add_optim(oracle):
    # tests/optim.rs:10-104: SGD with lr = 1e-3 after mul_add; grads are zeroed.
    a, b, c = full(1024, 3.0), full(1024, 2.0), full(1024, 1.0)
    ga, gb, gc = full(1024, 2.0), full(1024, 3.0), full(1024, 1.0)
    lr = float(f32(1e-3))
    for w, g in ((a, ga), (b, gb), (c, gc)):
        oracle.sgd(w, g, lr)
        assert (g == 0.0).all()
    assert (a == f32(3.0) - f32(2e-3)).all()
    assert (b == f32(2.0) - f32(3e-3)).all()
    assert (c == f32(1.0) - f32(1e-3)).all()
