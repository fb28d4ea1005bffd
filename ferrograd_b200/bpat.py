"""`.bpat` checkpoints through the C ABI: the reference's `save_tensors` / `load_tensors`
(crates/fused_gpu/src/io/mod.rs:98-159, exposed on GpuContext at crates/fused_gpu/src/dispatch/mod.rs:816-833).
"""
import ctypes as C

import numpy as np

from . import _lib
from .backend import Buffer, FgError, GpuContext, Tensor

# BpatHeader of the reference (crates/fused_gpu/src/io/mod.rs): the formats this backend can write / read
V0, V1, V1_MICRO, V2_F32, V2_F16, V2_BF16 = 0, 1, 2, 3, 4, 5
# numpy view of what fg_bpat_load_tensor returns, by fg_dtype: bf16 tensors are exposed as their uint16 bit patterns
_NP_DTYPE = {0: np.float32, 1: np.float16, 2: np.uint16}


def inspect(path):
    """Header, shapes (and checksum verification) without a device: [(shape...)], format."""
    lib = _lib.load()
    h = C.c_void_p()
    code = lib.fg_bpat_open(str(path).encode(), C.byref(h))
    if code != 0:
        raise FgError(code, f"cannot read {path}: missing, truncated, or a checksum does not match")
    try:
        shapes = []
        for i in range(lib.fg_bpat_count(h)):
            nd, dims = C.c_uint32(), (C.c_uint32 * 8)()
            lib.fg_bpat_shape(h, i, C.byref(nd), dims)
            shapes.append(tuple(dims[d] for d in range(nd.value)))
        return shapes, lib.fg_bpat_format(h)
    finally:
        lib.fg_bpat_close(h)


def save_tensors(ctx, path, tensors, header=V2_F32):
    n = len(tensors)
    bufs = (C.c_void_p * n)(*[t.as_buffer().handle for t in tensors])
    ndims = (C.c_uint32 * n)(*[len(t.shape) for t in tensors])
    shape_arrays = [(C.c_uint32 * len(t.shape))(*t.shape) for t in tensors]
    shapes = (C.POINTER(C.c_uint32) * n)(*[C.cast(a, C.POINTER(C.c_uint32)) for a in shape_arrays])
    ctx._check(ctx.lib.fg_bpat_save(ctx.handle, str(path).encode(), int(header), n, bufs, ndims, shapes))


def load_tensors(ctx, path):
    lib = ctx.lib
    h = C.c_void_p()
    code = lib.fg_bpat_open(str(path).encode(), C.byref(h))
    if code != 0:
        raise FgError(code, f"cannot read {path}: missing, truncated, or a checksum does not match")
    try:
        out = []
        dtype = _NP_DTYPE[lib.fg_bpat_dtype(h)]
        for i in range(lib.fg_bpat_count(h)):
            nd, dims = C.c_uint32(), (C.c_uint32 * 8)()
            lib.fg_bpat_shape(h, i, C.byref(nd), dims)
            b = C.c_void_p()
            ctx._check(lib.fg_bpat_load_tensor(ctx.handle, h, i, C.byref(b)))
            out.append(Tensor(tuple(dims[d] for d in range(nd.value)), Buffer(ctx, b), dtype))
        return out
    finally:
        lib.fg_bpat_close(h)


def save_adamw_state(ctx, path, m, v, step):
    """The optimizer state of a run, to be kept beside a parameter checkpoint.

    This is NOT one of the reference's formats (its SGD has no state and it has no AdamW): the container is an
    ordinary v2-f32 `.bpat` file, so every reader of the format can open it, whose tensor list is by convention
    m_0 .. m_{n-1}, v_0 .. v_{n-1} (shapes of the parameters), then one [2] tensor holding the step count as two
    16-bit halves (low, high), each exact in f32.  m and v are lists of Tensors."""
    if len(m) != len(v):
        raise ValueError("m and v must list the same tensors")
    step = int(step)
    if not 0 <= step < (1 << 32):
        raise ValueError("step count out of range")
    count = ctx.init_tensor_f32((2,), np.array([step & 0xffff, step >> 16], np.float32))
    try:
        save_tensors(ctx, path, list(m) + list(v) + [count], V2_F32)
    finally:
        count.data.free()


def load_adamw_state(ctx, path):
    """Inverse of save_adamw_state: (m, v, step)."""
    ts = load_tensors(ctx, path)
    if len(ts) % 2 != 1 or ts[-1].shape != (2,):
        for t in ts:
            t.data.free()
        raise ValueError(f"{path} is not an optimizer-state container (2n + 1 tensors, the last of shape [2])")
    n = (len(ts) - 1) // 2
    halves = ctx.to_numpy(ts[-1])
    ts[-1].data.free()
    return ts[:n], ts[n:2 * n], int(halves[0]) | (int(halves[1]) << 16)


GpuContext.save_tensors = lambda self, path, tensors, header=V2_F32: save_tensors(self, path, tensors, header)
GpuContext.load_tensors = lambda self, path: load_tensors(self, path)
