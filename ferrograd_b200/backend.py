"""Host-side mirror of the reference's context/tensor interface, over the C ABI.

`GpuContext` keeps the reference's method names and argument meaning
(crates/fused_gpu/src/dispatch/mod.rs:352-662: alloc / alloc_zeroed / alloc_init /
upload / download / copy / sync / is_ready / init_tensor_f32 / new_tensor) and error
behaviour (errors are raised as `FgError` carrying the status code that maps onto the
reference's `ErrorKind`).  The compute methods are thin wrappers of the `fg_*` entry
points; all of them enqueue on the context's stream and return immediately.
"""
import ctypes as C

import numpy as np

from . import _lib

ACT = {"none": 0, None: 0, "relu": 1, "tanh": 2, "gelu": 3}
GEMM_MODE = {"auto": 0, "simt": 1, "3xtf32": 2, "tf32_bf16x2": 3}
KERNEL_KIND = {"gemm_tc": 0, "softmax_ce": 1, "adamw": 2, "sgd": 3, "split": 4, "eltwise": 5, "skinny": 6}
EW = {"input": 0, "const": 1, "add": 2, "sub": 3, "mul": 4, "div": 5, "neg": 6, "abs": 7,
      "exp": 8, "log": 9, "tanh": 10, "relu": 11, "gelu": 12, "elu": 13}


class FgError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"{_lib.STATUS.get(code, code)}: {msg}")
        self.code = code
        self.kind = _lib.STATUS.get(code, str(code))


class Buffer:
    """GpuBackend::Buffer: a device allocation owned by the context."""

    def __init__(self, ctx, handle):
        self.ctx = ctx
        self.handle = handle
        self.ptr = ctx.lib.fg_buf_device_ptr(handle) or 0

    def size_bytes(self):
        return int(self.ctx.lib.fg_buf_size_bytes(self.handle))

    def size(self):
        """Size in 32-bit words (GpuBufferBackend::size, dispatch/mod.rs:147-151)."""
        return self.size_bytes() // 4

    def free(self):
        if self.handle:
            self.ctx.lib.fg_free(self.ctx.handle, self.handle)
            self.handle = None
            self.ptr = 0


class Tensor:
    """Shape + device buffer (crates/fused_gpu/src/tensor.rs:125-128)."""

    def __init__(self, shape, data, dtype=np.float32):
        self.shape = tuple(int(s) for s in shape)
        self.data = data
        self.dtype = np.dtype(dtype)

    @property
    def ptr(self):
        return self.data.ptr

    @property
    def size(self):
        return int(np.prod(self.shape)) if self.shape else 1

    def as_buffer(self):
        return self.data


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, (Tensor, Buffer)):
        return x.ptr
    return int(x)


class Plan:
    """GpuBackend::Schedule: a captured CUDA graph."""

    def __init__(self, ctx, handle):
        self.ctx = ctx
        self.handle = handle

    def launch(self):
        self.ctx._check(self.ctx.lib.fg_plan_launch(self.ctx.handle, self.handle))

    def destroy(self):
        if self.handle:
            self.ctx.lib.fg_plan_destroy(self.handle)
            self.handle = None


DTYPE = {"f32": 0, "f16": 1, "bf16": 2}


def to_bf16_bits(x):
    """float32 array -> uint16 bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return np.where((u & 0x7FFFFFFF) > 0x7F800000, u >> 16, r).astype(np.uint16)


def from_bf16_bits(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


class GpuContext:
    def __init__(self, device=0, stream=None):
        self.lib = _lib.load()
        h = C.c_void_p()
        code = self.lib.fg_ctx_create_on_stream(int(device), stream, C.byref(h))
        if code != 0:
            raise FgError(code, "could not create a context on device %d" % device)
        self.handle = h
        self.device = device

    # the reference spells the constructor GpuContext::new()
    @classmethod
    def new(cls, device=0):
        return cls(device)

    def _check(self, code):
        if code != 0:
            raise FgError(code, (self.lib.fg_last_error(self.handle) or b"").decode())

    def destroy(self):
        if self.handle:
            self.lib.fg_ctx_destroy(self.handle)
            self.handle = None

    # ---- GpuBackend: memory ----
    def alloc(self, nbytes):
        b = C.c_void_p()
        self._check(self.lib.fg_alloc(self.handle, int(nbytes), C.byref(b)))
        return Buffer(self, b)

    def alloc_zeroed(self, nbytes):
        b = C.c_void_p()
        self._check(self.lib.fg_alloc_zeroed(self.handle, int(nbytes), C.byref(b)))
        return Buffer(self, b)

    def alloc_init(self, data):
        a = np.ascontiguousarray(data)
        b = C.c_void_p()
        self._check(self.lib.fg_alloc_init(self.handle, a.ctypes.data, a.nbytes, C.byref(b)))
        return Buffer(self, b)

    def upload(self, dst, data, dst_off=0):
        a = np.ascontiguousarray(data)
        buf = dst.as_buffer() if isinstance(dst, Tensor) else dst
        self._check(self.lib.fg_upload(self.handle, buf.handle, a.ctypes.data, a.nbytes, int(dst_off)))

    def download(self, src, out, src_off=0):
        assert out.flags["C_CONTIGUOUS"]
        buf = src.as_buffer() if isinstance(src, Tensor) else src
        self._check(self.lib.fg_download(self.handle, buf.handle, out.ctypes.data, out.nbytes, int(src_off)))
        return out

    def copy(self, src, dst):
        s = src.as_buffer() if isinstance(src, Tensor) else src
        d = dst.as_buffer() if isinstance(dst, Tensor) else dst
        self._check(self.lib.fg_copy(self.handle, s.handle, d.handle))

    def sync(self):
        self._check(self.lib.fg_sync(self.handle))

    def is_ready(self):
        r = C.c_int32()
        self._check(self.lib.fg_is_ready(self.handle, C.byref(r)))
        return bool(r.value)

    # ---- GpuContext helpers of the reference (dispatch/mod.rs:577-662) ----
    def init_tensor_f32(self, shape, data):
        a = np.ascontiguousarray(data, dtype=np.float32)
        assert a.size == int(np.prod(shape))
        return Tensor(shape, self.alloc_init(a), np.float32)

    def init_tensor_f16(self, shape, data):
        """GpuContext::init_tensor_f16 (exercised by crates/ferrograd/tests/nonf32.rs:57-64)."""
        a = np.ascontiguousarray(data, dtype=np.float16)
        assert a.size == int(np.prod(shape))
        return Tensor(shape, self.alloc_init(a), np.float16)

    def init_tensor_bf16(self, shape, data):
        """data: float values; stored as bf16 bit patterns (numpy has no bf16: the tensor's dtype is uint16)."""
        a = to_bf16_bits(np.ascontiguousarray(data, dtype=np.float32))
        assert a.size == int(np.prod(shape))
        return Tensor(shape, self.alloc_init(a), np.uint16)

    def init_tensor_u32(self, shape, data):
        a = np.ascontiguousarray(data, dtype=np.uint32)
        assert a.size == int(np.prod(shape))
        return Tensor(shape, self.alloc_init(a), np.uint32)

    def new_tensor(self, shape, dtype=np.float32, zeroed=False):
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        return Tensor(shape, self.alloc_zeroed(n) if zeroed else self.alloc(n), dtype)

    def to_numpy(self, t):
        out = np.empty(t.shape, t.dtype)
        return self.download(t, out)

    # ---- misc ----
    def set_option(self, name, value):
        """fg_ctx_set_option: "gemm_tile", "gemm_group", "gemm_split_k", "gemm_pairs", "exec_plans", "comm_max_ctas",
        "comm_sms", "comm_min_exchange"."""
        self._check(self.lib.fg_ctx_set_option(self.handle, name.encode(), str(value).encode()))

    def stream(self):
        return self.lib.fg_ctx_stream(self.handle)

    def launch_count(self):
        return int(self.lib.fg_ctx_launch_count(self.handle))

    def reserve_workspace(self, nbytes):
        self._check(self.lib.fg_ctx_reserve_workspace(self.handle, int(nbytes)))

    def workspace_bytes(self):
        return int(self.lib.fg_ctx_workspace_bytes(self.handle))

    def device_status(self):
        w = C.c_int32()
        self._check(self.lib.fg_ctx_device_status(self.handle, C.byref(w)))
        return w.value

    def timing_enable(self, on=True):
        self._check(self.lib.fg_ctx_timing_enable(self.handle, int(on)))

    def timing_read(self, kind):
        """(launches, total_ms, total_work) of one kernel kind since the last read."""
        n, ms, work = C.c_uint64(), C.c_double(), C.c_double()
        self._check(self.lib.fg_ctx_timing_read(self.handle, KERNEL_KIND[kind], C.byref(n), C.byref(ms),
                                                C.byref(work)))
        return n.value, ms.value, work.value

    def memset_zero(self, t, nbytes=None):
        nb = nbytes if nbytes is not None else t.size * t.dtype.itemsize
        self._check(self.lib.fg_memset_zero(self.handle, _ptr(t), int(nb)))

    def upload_async(self, dst, pinned_ptr, nbytes):
        self._check(self.lib.fg_upload_async(self.handle, _ptr(dst), pinned_ptr, int(nbytes)))

    def download_async(self, pinned_ptr, src, nbytes):
        self._check(self.lib.fg_download_async(self.handle, pinned_ptr, _ptr(src), int(nbytes)))

    def upload_prefetch(self, dst, pinned_ptr, nbytes):
        self._check(self.lib.fg_upload_prefetch(self.handle, _ptr(dst), pinned_ptr, int(nbytes)))

    def prefetch_wait(self):
        self._check(self.lib.fg_prefetch_wait(self.handle))

    def prefetch_mark(self):
        self._check(self.lib.fg_prefetch_mark(self.handle))

    def copy_dev_async(self, dst, src, nbytes):
        self._check(self.lib.fg_copy_dev_async(self.handle, _ptr(dst), _ptr(src), int(nbytes)))

    def pinned_array(self, shape, dtype=np.float32):
        """A numpy array over page-locked host memory (kept alive by the returned array)."""
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        code = self.lib.fg_host_alloc_pinned(n, C.byref(p))
        if code != 0:
            raise FgError(code, "pinned host allocation failed")
        buf = (C.c_char * max(n, 1)).from_address(p.value)
        arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
        return arr

    # ---- compute ----
    def gemm(self, A, B, Cout, M, N, K, transA=False, transB=False, bias=None, act="none", preact_out=None,
             mode="auto"):
        self._check(self.lib.fg_gemm_f32(self.handle, GEMM_MODE[mode], int(transA), int(transB), M, N, K,
                                         _ptr(A), _ptr(B), _ptr(Cout), _ptr(bias), ACT[act], _ptr(preact_out)))

    def gemm_bwd(self, A, B, dY, M, N, K, act="none", saved=None, dA=None, dB=None, dbias=None, dZ_out=None,
                 mode="auto"):
        self._check(self.lib.fg_gemm_bwd_f32(self.handle, GEMM_MODE[mode], M, N, K, _ptr(A), _ptr(B), _ptr(dY),
                                             ACT[act], _ptr(saved), _ptr(dA), _ptr(dB), _ptr(dbias), _ptr(dZ_out)))

    def gemm_bwd_exchange(self, A, B, dY, M, N, K, exch_buf, exch_count, act="none", saved=None, dA=None, dB=None,
                          dbias=None, mode="auto"):
        """gemm_bwd that starts the allreduce of exch_buf once dB and dbias are done and computes dA beside it."""
        self._check(self.lib.fg_gemm_bwd_exchange_f32(self.handle, GEMM_MODE[mode], M, N, K, _ptr(A), _ptr(B), _ptr(dY),
                                                      ACT[act], _ptr(saved), _ptr(dA), _ptr(dB), _ptr(dbias),
                                                      _ptr(exch_buf), exch_count))

    # ---- f32 tensors with bf16 pairs: no operand pre-pass (see include/ferrograd_b200.h) ----
    def pairs_from_f32(self, x, n, pairs, plane_stride=None):
        self._check(self.lib.fg_pairs_from_f32(self.handle, _ptr(x), n, _ptr(pairs), plane_stride or n))

    def gemm_paired(self, A, B, Cout, M, N, K, A_pairs=None, B_pairs=None, bias=None, act="none", preact_out=None,
                    C_pairs=None, A_stride=None, B_stride=None, C_stride=None):
        self._check(self.lib.fg_gemm_paired_f32(self.handle, M, N, K, _ptr(A), _ptr(A_pairs), A_stride or M * K, _ptr(B),
                                                _ptr(B_pairs), B_stride or K * N, _ptr(Cout), _ptr(bias), ACT[act],
                                                _ptr(preact_out), _ptr(C_pairs), C_stride or M * N))

    def gemm_bwd_paired(self, A, B, dZ, M, N, K, A_pairs=None, B_pairs=None, dZ_pairs=None, dB=None, dbias=None, dA=None,
                        below_act="none", below_saved=None, dA_pairs=None, below_dbias=None, exch_buf=None,
                        exch_count=0, A_stride=None, B_stride=None, dZ_stride=None, dA_stride=None):
        self._check(self.lib.fg_gemm_bwd_paired_f32(
            self.handle, M, N, K, _ptr(A), _ptr(A_pairs), A_stride or M * K, _ptr(B), _ptr(B_pairs), B_stride or K * N,
            _ptr(dZ), _ptr(dZ_pairs), dZ_stride or M * N, _ptr(dB), _ptr(dbias), _ptr(dA), ACT[below_act], _ptr(below_saved),
            _ptr(dA_pairs), dA_stride or M * K, _ptr(below_dbias), _ptr(exch_buf), exch_count))

    def gemm_batched(self, A, B, Cout, batch, M, N, K, bias=None, act="none", preact_out=None, mode="auto",
                     strides=None):
        sa, sb, sc = strides or (M * K, K * N, M * N)
        self._check(self.lib.fg_gemm_batched_f32(self.handle, GEMM_MODE[mode], batch, M, N, K, _ptr(A), sa, _ptr(B), sb,
                                                 _ptr(Cout), sc, _ptr(bias), ACT[act], _ptr(preact_out)))

    def gemm_batched_bwd(self, A, B, dY, batch, M, N, K, act="none", saved=None, dA=None, dB=None, mode="auto",
                         strides=None):
        sa, sb, sc = strides or (M * K, K * N, M * N)
        self._check(self.lib.fg_gemm_batched_bwd_f32(self.handle, GEMM_MODE[mode], batch, M, N, K, _ptr(A), sa,
                                                     _ptr(B), sb, _ptr(dY), sc, ACT[act], _ptr(saved), _ptr(dA),
                                                     _ptr(dB)))

    def bias_act_fwd(self, z, bias, act, y, rows, cols):
        self._check(self.lib.fg_bias_act_fwd(self.handle, rows, cols, _ptr(z), _ptr(bias), ACT[act], _ptr(y)))

    def act_bwd(self, dy, saved, dz, n, act):
        self._check(self.lib.fg_act_bwd(self.handle, n, ACT[act], _ptr(dy), _ptr(saved), _ptr(dz)))

    def softmax_fwd(self, x, y, rows, cols):
        self._check(self.lib.fg_softmax_fwd(self.handle, rows, cols, _ptr(x), _ptr(y)))

    def softmax_bwd(self, y, dy, dx, rows, cols, accumulate=False):
        self._check(self.lib.fg_softmax_bwd(self.handle, rows, cols, _ptr(y), _ptr(dy), _ptr(dx), int(accumulate)))

    def softmax_ce(self, logits, labels, rows, cols, grad_scale=1.0, loss_row=None, loss_mean=None, dlogits=None,
                   probs=None, argmax=None):
        self._check(self.lib.fg_softmax_ce_fwd_bwd(self.handle, _ptr(logits), _ptr(labels), rows, cols,
                                                   grad_scale, _ptr(loss_row), _ptr(loss_mean), _ptr(dlogits),
                                                   _ptr(probs), _ptr(argmax)))

    def ce_loss_grad(self, probs, labels, rows, cols, loss, grad):
        self._check(self.lib.fg_ce_loss_grad(self.handle, _ptr(probs), _ptr(labels), rows, cols, _ptr(loss),
                                             _ptr(grad)))

    def mse_loss_grad(self, pred, target, n, grad_scale=1.0, loss_elem=None, loss_sum=None, grad=None):
        self._check(self.lib.fg_mse_loss_grad(self.handle, _ptr(pred), _ptr(target), n, grad_scale,
                                              _ptr(loss_elem), _ptr(loss_sum), _ptr(grad)))

    def bce_loss_grad(self, pred, target, n, grad_scale=1.0, loss_elem=None, loss_sum=None, grad=None):
        self._check(self.lib.fg_bce_loss_grad(self.handle, _ptr(pred), _ptr(target), n, grad_scale,
                                              _ptr(loss_elem), _ptr(loss_sum), _ptr(grad)))

    def mse_loss_grad_noalloc(self, pred, target, n, grad_scale=1.0, loss_elem=None, loss_sum=None, grad=None):
        """fg_mse_loss_grad for hosts that must not allocate device memory: the reduction scratch is a
        fixed array inside the library (n <= 268,435,456; calls on one GPU must not overlap)."""
        self._check(self.lib.fg_mse_loss_grad_noalloc(self.handle, _ptr(pred), _ptr(target), n, grad_scale,
                                                      _ptr(loss_elem), _ptr(loss_sum), _ptr(grad)))

    def sgd_step(self, w, g, n, lr, grad_scale=1.0, zero_grad=True):
        self._check(self.lib.fg_sgd_step(self.handle, _ptr(w), _ptr(g), n, lr, grad_scale, int(zero_grad)))

    def adamw_step(self, w, g, m, v, n, lr, beta1, beta2, eps, weight_decay, step=1, step_dev=None,
                   grad_scale=1.0, zero_grad=True):
        h = _lib.AdamWHyper(lr, beta1, beta2, eps, weight_decay)
        self._check(self.lib.fg_adamw_step(self.handle, _ptr(w), _ptr(g), _ptr(m), _ptr(v), n, C.byref(h),
                                           int(step), _ptr(step_dev), grad_scale, int(zero_grad)))

    def sgd_step_paired(self, w, g, n, lr, w_pairs, pairs_stride, grad_scale=1.0, zero_grad=True):
        self._check(self.lib.fg_sgd_step_paired(self.handle, _ptr(w), _ptr(g), n, lr, grad_scale, int(zero_grad),
                                                _ptr(w_pairs), pairs_stride))

    def adamw_step_paired(self, w, g, m, v, n, lr, beta1, beta2, eps, weight_decay, w_pairs, pairs_stride, step=1,
                          step_dev=None, grad_scale=1.0, zero_grad=True):
        h = _lib.AdamWHyper(lr, beta1, beta2, eps, weight_decay)
        self._check(self.lib.fg_adamw_step_paired(self.handle, _ptr(w), _ptr(g), _ptr(m), _ptr(v), n, C.byref(h),
                                                  int(step), _ptr(step_dev), grad_scale, int(zero_grad), _ptr(w_pairs),
                                                  pairs_stride))

    def _update_tensors(self, tensors):
        arr = (_lib.UpdateTensor * len(tensors))()
        for i, t in enumerate(tensors):
            arr[i] = _lib.UpdateTensor(_ptr(t["w"]), _ptr(t["g"]), _ptr(t.get("m")), _ptr(t.get("v")), _ptr(t.get("w_pairs")),
                                       int(t.get("pairs_stride", 0)), int(t["n"]))
        return arr

    def adamw_step_multi(self, tensors, lr, beta1, beta2, eps, weight_decay, step=1, step_dev=None, grad_scale=1.0,
                         zero_grad=True):
        """tensors: dicts with w, g, m, v, n and optionally w_pairs, pairs_stride; one launch for all of them."""
        h = _lib.AdamWHyper(lr, beta1, beta2, eps, weight_decay)
        self._check(self.lib.fg_adamw_step_multi(self.handle, self._update_tensors(tensors), len(tensors), C.byref(h),
                                                 int(step), _ptr(step_dev), grad_scale, int(zero_grad)))

    def sgd_step_multi(self, tensors, lr, grad_scale=1.0, zero_grad=True):
        self._check(self.lib.fg_sgd_step_multi(self.handle, self._update_tensors(tensors), len(tensors), lr, grad_scale,
                                               int(zero_grad)))

    def counter_increment(self, counter):
        self._check(self.lib.fg_counter_increment(self.handle, _ptr(counter)))

    @staticmethod
    def _prog(instrs):
        arr = (_lib.EwInstr * len(instrs))()
        for i, (op, a, b, imm) in enumerate(instrs):
            arr[i] = _lib.EwInstr(EW[op] if isinstance(op, str) else op, a, b, imm)
        return arr

    def eltwise_chain_fwd(self, instrs, inputs, out, n, saved=None, dtype="f32"):
        prog = self._prog(instrs)
        inp = (C.c_void_p * len(inputs))(*[_ptr(x) for x in inputs])
        sv = None
        if saved:
            sv = (C.c_void_p * len(instrs))(*[_ptr(saved.get(k)) for k in range(len(instrs))])
        self._check(self.lib.fg_eltwise_chain_fwd_dt(self.handle, DTYPE[dtype], n, prog, len(instrs), inp, len(inputs),
                                                     _ptr(out), sv))

    def eltwise_chain_bwd(self, instrs, inputs, seed, grads, n, accumulate=False, dtype="f32"):
        prog = self._prog(instrs)
        inp = (C.c_void_p * len(inputs))(*[_ptr(x) for x in inputs])
        gp = (C.c_void_p * len(inputs))(*[_ptr(g) for g in grads])
        self._check(self.lib.fg_eltwise_chain_bwd_dt(self.handle, DTYPE[dtype], n, prog, len(instrs), inp, len(inputs),
                                                     _ptr(seed), gp, int(accumulate)))

    def gemm_lowp(self, A, B, Cout, M, N, K, dtype, bias=None, act="none", preact_out=None):
        """GEMM on f16 / bf16 tensors: 16-bit operands straight into the tensor cores, f32 accumulate."""
        self._check(self.lib.fg_gemm_lowp(self.handle, DTYPE[dtype], M, N, K, _ptr(A), _ptr(B), _ptr(Cout), _ptr(bias),
                                          ACT[act], _ptr(preact_out)))

    def gemm_bwd_lowp(self, A, B, dY, M, N, K, dtype, act="none", saved=None, dA=None, dB=None, dbias=None):
        self._check(self.lib.fg_gemm_bwd_lowp(self.handle, DTYPE[dtype], M, N, K, _ptr(A), _ptr(B), _ptr(dY), ACT[act],
                                              _ptr(saved), _ptr(dA), _ptr(dB), _ptr(dbias)))

    def convert(self, src, src_dtype, dst, dst_dtype, n):
        self._check(self.lib.fg_convert(self.handle, _ptr(src), DTYPE[src_dtype], _ptr(dst), DTYPE[dst_dtype], n))

    # ---- plans ----
    def plan_begin(self):
        self._check(self.lib.fg_plan_begin(self.handle))

    def plan_end(self):
        p = C.c_void_p()
        self._check(self.lib.fg_plan_end(self.handle, C.byref(p)))
        return Plan(self, p)

    # ---- data-parallel exchange ----
    def comm_unique_id(self):
        buf = (C.c_uint8 * 128)()
        code = self.lib.fg_comm_unique_id(buf)
        if code != 0:
            raise FgError(code, "NCCL unique id")
        return bytes(buf)

    def comm_init(self, nranks, rank, uid):
        buf = (C.c_uint8 * 128).from_buffer_copy(uid)
        self._check(self.lib.fg_comm_init(self.handle, nranks, rank, buf))

    def allreduce_sum(self, buf, count):
        self._check(self.lib.fg_allreduce_sum_f32(self.handle, _ptr(buf), int(count)))

    def comm_join(self):
        self._check(self.lib.fg_comm_join(self.handle))

    def comm_sync(self, timeout_ms):
        """Host wait for the exchanges in flight; raises FgError(FG_ERR_TIMEOUT) and aborts the communicator
        when they do not complete in time."""
        self._check(self.lib.fg_comm_sync(self.handle, int(timeout_ms)))

    def comm_abort(self):
        self._check(self.lib.fg_comm_abort(self.handle))

    def comm_checkpoint(self, slot):
        self._check(self.lib.fg_comm_checkpoint(self.handle, slot))

    def comm_wait(self, slot):
        self._check(self.lib.fg_comm_wait(self.handle, slot))
