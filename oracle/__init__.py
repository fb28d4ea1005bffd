"""numpy front end of the CPU oracle -- TEST INFRASTRUCTURE, NOT PRODUCT.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this package.
The arithmetic lives in fg_oracle.cpp (each function cites the reference lines it
restates); this module only marshals numpy arrays through ctypes.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None

ACT = {"none": 0, "relu": 1, "tanh": 2, "gelu": 3}
QUIRK_RELU_MASK_GE0 = 1
QUIRK_GELU_BWD_T = 2
QUIRK_SOFTMAX_BWD_COL0 = 4

EW = {"input": 0, "const": 1, "add": 2, "sub": 3, "mul": 4, "div": 5, "neg": 6, "abs": 7,
      "exp": 8, "log": 9, "tanh": 10, "relu": 11, "gelu": 12, "elu": 13}


class EwInstr(C.Structure):
    _fields_ = [("op", C.c_int32), ("a", C.c_int32), ("b", C.c_int32), ("imm", C.c_float)]


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "libfg_oracle.so")
        if not os.path.exists(path):
            path = _build.build()
        _lib = C.CDLL(path)
        _lib.ref_mlp_step.restype = C.c_double
        _lib.ref_num_threads.restype = C.c_int
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_threads():
    return lib().ref_num_threads()


def set_num_threads(n):
    lib().ref_set_num_threads(C.c_int(n))


def gemm(A, B, transA=False, transB=False, f64=False):
    A, B = _f(A), _f(B)
    M, K = (A.shape[1], A.shape[0]) if transA else A.shape
    N = B.shape[0] if transB else B.shape[1]
    assert (B.shape[1] if transB else B.shape[0]) == K
    Cm = np.empty((M, N), np.float32)
    lib().ref_gemm_f32(int(transA), int(transB), C.c_uint32(M), C.c_uint32(N), C.c_uint32(K),
                       _p(A), _p(B), _p(Cm), int(f64))
    return Cm


def bias_act_fwd(z, bias, act):
    z = _f(z)
    rows, cols = z.shape
    y = np.empty_like(z)
    pre = np.empty_like(z)
    b = None if bias is None else _f(bias)
    lib().ref_bias_act_fwd(C.c_uint32(rows), C.c_uint32(cols), _p(z), _p(b), ACT[act], _p(y), _p(pre))
    return y, pre


def act_bwd(dy, saved, act, quirks=0):
    dy, saved = _f(dy), _f(saved)
    dz = np.empty_like(dy)
    lib().ref_act_bwd(C.c_uint64(dy.size), ACT[act], _p(dy), _p(saved), _p(dz), quirks)
    return dz


def colsum(x):
    x = _f(x)
    out = np.empty(x.shape[1], np.float32)
    lib().ref_colsum(C.c_uint32(x.shape[0]), C.c_uint32(x.shape[1]), _p(x), _p(out))
    return out


def softmax_fwd(x):
    x = _f(x)
    y = np.empty_like(x)
    lib().ref_softmax_fwd(C.c_uint32(x.shape[0]), C.c_uint32(x.shape[1]), _p(x), _p(y))
    return y


def softmax_bwd(y, dy, dx=None, quirks=0):
    y, dy = _f(y), _f(dy)
    acc = dx is not None
    out = _f(dx).copy() if acc else np.empty_like(y)
    lib().ref_softmax_bwd(C.c_uint32(y.shape[0]), C.c_uint32(y.shape[1]), _p(y), _p(dy), _p(out),
                          int(acc), quirks)
    return out


def ce_loss_grad(probs, labels):
    probs = _f(probs)
    labels = np.ascontiguousarray(labels, dtype=np.uint32)
    loss = np.empty_like(probs)
    grad = np.empty_like(probs)
    lib().ref_ce_loss_grad(C.c_uint32(probs.shape[0]), C.c_uint32(probs.shape[1]), _p(probs),
                           _p(labels), _p(loss), _p(grad))
    return loss, grad


QUIRK_RELU_MASK_GE0, QUIRK_GELU_BWD_T, QUIRK_SOFTMAX_BWD_COL0, QUIRK_CE_THROUGH_SOFTMAX = 1, 2, 4, 8


def softmax_ce(logits, labels, grad_scale=1.0, want_probs=False, want_dlogits=True, quirks=0):
    logits = _f(logits)
    labels = np.ascontiguousarray(labels, dtype=np.uint32)
    rows, cols = logits.shape
    loss_row = np.empty(rows, np.float32)
    mean = np.empty(1, np.float32)
    dl = np.empty_like(logits) if want_dlogits else None
    pr = np.empty_like(logits) if want_probs else None
    am = np.empty(rows, np.uint32)
    lib().ref_softmax_ce_fwd_bwd_q(C.c_uint32(rows), C.c_uint32(cols), _p(logits), _p(labels),
                                   C.c_float(grad_scale), _p(loss_row), _p(mean), _p(dl), _p(pr),
                                   _p(am), int(quirks))
    return {"loss_row": loss_row, "loss_mean": float(mean[0]), "dlogits": dl, "probs": pr,
            "argmax": am}


def mse(pred, target, grad_scale=1.0):
    pred, target = _f(pred), _f(target)
    loss = np.empty_like(pred)
    grad = np.empty_like(pred)
    s = np.empty(1, np.float32)
    lib().ref_mse_loss_grad(C.c_uint64(pred.size), _p(pred), _p(target), C.c_float(grad_scale),
                            _p(loss), _p(s), _p(grad))
    return loss, float(s[0]), grad


def bce(pred, target, grad_scale=1.0, reference_formula=False):
    pred, target = _f(pred), _f(target)
    loss = np.empty_like(pred)
    grad = np.empty_like(pred)
    s = np.empty(1, np.float32)
    lib().ref_bce_loss_grad(C.c_uint64(pred.size), _p(pred), _p(target), C.c_float(grad_scale),
                            int(reference_formula), _p(loss), _p(s), _p(grad))
    return loss, float(s[0]), grad


def sgd(w, g, lr, grad_scale=1.0, zero_grad=True):
    """In place on w and g (float32 contiguous arrays)."""
    assert w.dtype == np.float32 and g.dtype == np.float32
    lib().ref_sgd_step(C.c_uint64(w.size), _p(w), _p(g), C.c_float(lr), C.c_float(grad_scale),
                       int(zero_grad))


def adamw(w, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale=1.0, zero_grad=True):
    """In place on w, g, m, v."""
    for a in (w, g, m, v):
        assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    lib().ref_adamw_step(C.c_uint64(w.size), _p(w), _p(g), _p(m), _p(v), C.c_float(lr),
                         C.c_float(beta1), C.c_float(beta2), C.c_float(eps), C.c_float(wd),
                         C.c_uint32(step), C.c_float(grad_scale), int(zero_grad))


def make_prog(instrs):
    """instrs: list of (opname, a, b, imm)."""
    arr = (EwInstr * len(instrs))()
    for i, (op, a, b, imm) in enumerate(instrs):
        arr[i] = EwInstr(EW[op], a, b, imm)
    return arr


DTYPES = {"f32": 0, "f16": 1, "bf16": 2}


def round_to(x, dtype):
    """x rounded to the nearest f16 / bf16 value (ties to even), returned as float32."""
    x = _f(x)
    out = np.empty_like(x)
    lib().ref_round_to(DTYPES[dtype], C.c_uint64(x.size), _p(x), _p(out))
    return out


def eltwise_fwd(instrs, inputs, save=(), dtype="f32"):
    inputs = [_f(x) for x in inputs]
    n = inputs[0].size
    prog = make_prog(instrs)
    out = np.empty_like(inputs[0])
    inp = (C.c_void_p * len(inputs))(*[x.ctypes.data for x in inputs])
    saved = {k: np.empty_like(inputs[0]) for k in save}
    sv = (C.c_void_p * len(instrs))(*[saved[k].ctypes.data if k in saved else None
                                      for k in range(len(instrs))])
    lib().ref_eltwise_chain_fwd_dt(DTYPES[dtype], C.c_uint64(n), prog, len(instrs), inp, len(inputs), _p(out), sv)
    return out, saved


def eltwise_bwd(instrs, inputs, seed, quirks=0, dtype="f32"):
    inputs = [_f(x) for x in inputs]
    seed = _f(seed)
    n = inputs[0].size
    prog = make_prog(instrs)
    grads = [np.zeros_like(x) for x in inputs]
    inp = (C.c_void_p * len(inputs))(*[x.ctypes.data for x in inputs])
    gp = (C.c_void_p * len(inputs))(*[g.ctypes.data for g in grads])
    lib().ref_eltwise_chain_bwd_dt(DTYPES[dtype], C.c_uint64(n), prog, len(instrs), inp, len(inputs), _p(seed), gp,
                                   0, quirks)
    return grads


def mlp_step(dims, batch, hidden_act, W, b, x, target, loss_kind, grad_scale, opt, step=1,
             state=None):
    """One training step in place on W, b (lists of float32 arrays) and the AdamW state.

    opt = ("sgd", lr) or ("adamw", lr, beta1, beta2, eps, wd).  Returns (loss_sum, gW, gb, out).
    """
    L = len(dims) - 1
    dims_a = (C.c_uint32 * (L + 1))(*dims)
    x = _f(x)

    def arr(lst):
        return (C.c_void_p * L)(*[a.ctypes.data for a in lst])

    gW = [np.empty_like(w) for w in W]
    gb = [np.empty_like(v) for v in b]
    out = np.empty((batch, dims[-1]), np.float32)
    if loss_kind == "mse":
        tgt = _f(target)
        lk = 0
    else:
        tgt = np.ascontiguousarray(target, dtype=np.uint32)
        lk = 1
    if opt[0] == "sgd":
        ok, lr, b1, b2, eps, wd = 0, opt[1], 0.0, 0.0, 0.0, 0.0
        mW = vW = mb = vb = None
    elif opt[0] == "adamw":
        ok, lr, b1, b2, eps, wd = 1, opt[1], opt[2], opt[3], opt[4], opt[5]
        mW, vW, mb, vb = (arr(state[k]) for k in ("mW", "vW", "mb", "vb"))
    else:
        ok, lr, b1, b2, eps, wd = 2, 0.0, 0.0, 0.0, 0.0, 0.0
        mW = vW = mb = vb = None
    loss = lib().ref_mlp_step(L, dims_a, C.c_uint32(batch), ACT[hidden_act], arr(W), arr(b), _p(x),
                              _p(tgt), lk, C.c_float(grad_scale), ok, C.c_float(lr), C.c_float(b1),
                              C.c_float(b2), C.c_float(eps), C.c_float(wd), C.c_uint32(step),
                              mW, vW, mb, vb, arr(gW), arr(gb), _p(out))
    return loss, gW, gb, out
