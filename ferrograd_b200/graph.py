"""Host-side mirror of the reference's graph API, over the C ABI's graph engine.

Names, call order and argument meaning follow the reference so that its tests can be
restated line by line (crates/ferrograd/tests/std_wgsl.rs:268-319 is the canonical sequence):

    meta = Metadata(); m, n, k = meta.new_field(), meta.new_field(), meta.new_field()
    graph = Graph(MEAN_SQUARED_ERROR, Optim.sgd().lower)
    g = graph.define_ops(); a = g.input([m, k]); b = g.input([k, n]); c = g.input([m, n])
    g.add(g.matmul(a, b), c)
    saved = graph.compute_saved_nodes(); graph.validate(meta)
    ctx = GpuContext.new()
    meta_binding = [f32_bits(1e-3), M, N, K]
    saved_tensors = ctx.alloc_tensors(graph, saved, meta_binding, state)
    kernels = ctx.compile(graph.lower(meta, options, saved), options)
    schedule = ctx.schedule(kernels, meta_binding, in_tensors, saved_tensors, [], state)
    ctx.dispatch_forward(schedule); ctx.dispatch_backward(schedule); ctx.dispatch_optim(schedule)

`Graph` (crates/ferrograd/src/graph.rs:15-158), `Metadata` (crates/fused_gpu/src/dispatch/backend/mod.rs:577-620),
`AllocTensors` (crates/fused_gpu/src/dispatch/mod.rs:835-845).  The lowering itself happens in C++
(csrc/graph.cu); `lower`/`compile` exist so that the call sequence reads the same and return tokens.
"""
import ctypes as C
import struct

import numpy as np

from . import _lib
from .backend import Buffer, FgError, Tensor

MEAN_SQUARED_ERROR = 0      # ferrograd_nn::loss::MEAN_SQUARED_ERROR
CROSS_ENTROPY = 1           # ferrograd_nn::loss::CROSS_ENTROPY
BINARY_CROSS_ENTROPY = 2    # ferrograd_nn::loss::BINARY_CROSS_ENTROPY
_OPS = {"add": 2, "sub": 3, "mul": 4, "div": 5, "neg": 6, "abs": 7, "exp": 8, "log": 9, "tanh": 10, "relu": 11,
        "gelu": 12, "elu": 13, "matmul": 14, "softmax": 15}


def f32_bits(x):
    """`f32::to_bits`: how the learning rate travels in metadata field 0."""
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


class SimpleDType:
    """crates/fused_gpu/src/dispatch/backend/mod.rs:337-345 (the storage types this backend takes)."""
    F32 = "f32"
    F16 = "f16"
    BF16 = "bf16"
    U32 = "u32"


_DTYPE_CODE = {SimpleDType.F32: 0, SimpleDType.F16: 1, SimpleDType.BF16: 2}


class Metadata:
    """Field 0 is reserved for the learning rate; new_field() hands out 1, 2, ..."""

    def __init__(self):
        self.fields = 1

    @classmethod
    def new(cls):
        return cls()

    def new_field(self):
        self.fields += 1
        return self.fields - 1

    def validate_meta(self, binding):
        return len(binding) == self.fields


class Optim:
    """crates/ferrograd/src/optim.rs:4-16 (sgd); adamw is this backend's addition."""

    def __init__(self, kind, state):
        self.lower = kind
        self.state = state

    @classmethod
    def sgd(cls):
        return cls(0, ())

    @classmethod
    def adamw(cls, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
        return cls(1, (beta1, beta2, eps, weight_decay))


class Graph:
    def __init__(self, loss, optim_lower):
        self.lib = _lib.load()
        h = C.c_void_p()
        code = self.lib.fg_graph_create(int(loss), int(optim_lower), C.byref(h))
        if code != 0:
            raise FgError(code, "Graph::new")
        self.handle = h
        self.loss, self.optim = loss, optim_lower

    @classmethod
    def new(cls, loss, optim_lower):
        return cls(loss, optim_lower)

    def define_ops(self):
        return DefineOps(self)

    def node_count(self):
        return self.lib.fg_graph_node_count(self.handle)

    def compute_saved_nodes(self):
        """The decision is taken by the engine when the tensors are allocated; this returns a token."""
        return ("saved", self.node_count())

    def validate(self, meta):
        if self.node_count() <= 0:
            raise FgError(1, "GraphEmpty")
        return True

    def lower(self, meta, options=None, saved=None):
        return ("ir", self)

    def __del__(self):
        try:
            if self.handle:
                self.lib.fg_graph_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


class DefineOps:
    def __init__(self, graph):
        self.graph = graph

    def _check(self, code, what):
        if code != 0:
            raise FgError(code, what)

    def input(self, shape, dtype=SimpleDType.F32):
        fields = (C.c_uint32 * len(shape))(*shape)
        node = C.c_int32()
        self._check(self.graph.lib.fg_graph_input_dt(self.graph.handle, fields, len(shape), _DTYPE_CODE[dtype],
                                                     C.byref(node)), "input")
        return node.value

    def constant_f32(self, value):
        node = C.c_int32()
        self._check(self.graph.lib.fg_graph_constant_f32(self.graph.handle, float(value), C.byref(node)), "constant_f32")
        return node.value

    def _op(self, name, a, b=-1):
        node = C.c_int32()
        self._check(self.graph.lib.fg_graph_op(self.graph.handle, _OPS[name], int(a), int(b), C.byref(node)), name)
        return node.value


for _name in ("add", "sub", "mul", "div", "matmul"):
    setattr(DefineOps, _name, (lambda n: lambda self, a, b: self._op(n, a, b))(_name))
for _name in ("abs", "exp", "gelu", "relu", "elu", "log", "neg", "tanh", "softmax"):
    setattr(DefineOps, _name, (lambda n: lambda self, x: self._op(n, x))(_name))


class _BorrowedBuffer(Buffer):
    """A buffer owned by the engine (freed with it)."""

    def free(self):
        pass


class AllocTensors:
    def __init__(self, ctx, handle, meta):
        self.ctx, self.handle, self.meta = ctx, handle, list(meta)
        lib = ctx.lib
        wrap = lambda h: _BorrowedBuffer(ctx, C.c_void_p(h))
        self.forward_out = wrap(lib.fg_exec_forward_out(handle))
        self.seed = wrap(lib.fg_exec_seed(handle))
        self.forward_saved, self.saved_nodes = [], []
        for i in range(lib.fg_exec_num_saved(handle)):
            node = C.c_int32()
            self.forward_saved.append(wrap(lib.fg_exec_saved(handle, i, C.byref(node))))
            self.saved_nodes.append(node.value)
        self.grad_tensors, self.grad_nodes = [], []
        for i in range(lib.fg_exec_num_grads(handle)):
            node = C.c_int32()
            self.grad_tensors.append(wrap(lib.fg_exec_grad(handle, i, C.byref(node))))
            self.grad_nodes.append(node.value)
        lt = wrap(lib.fg_exec_loss_t(handle))
        self.loss_t = Tensor((lt.size_bytes() // 4,), lt)
        self.loss_sum = wrap(lib.fg_exec_loss_sum(handle))      # one f32: sum over loss_t (this backend's addition)
        self.state = []

    def plans_active(self):
        """True when the engine records this graph's dispatches as CUDA graphs and replays them."""
        return bool(self.ctx.lib.fg_exec_plans_active(self.handle))

    def forward_steps(self):
        return int(self.ctx.lib.fg_exec_forward_steps(self.handle))

    def destroy(self):
        if self.handle:
            self.ctx.lib.fg_exec_destroy(self.handle)
            self.handle = None


class Schedule:
    def __init__(self, tensors):
        self.tensors = tensors


class GraphContextMixin:
    """The graph half of GpuContext (crates/fused_gpu/src/dispatch/mod.rs:369-455, :509-575, :664-814)."""

    def alloc_meta(self, binding):
        return [int(v) & 0xFFFFFFFF for v in binding]

    def alloc_tensors(self, graph, saved, meta_binding, state=(), gemm_mode="auto"):
        from .backend import GEMM_MODE
        meta = (C.c_uint32 * len(meta_binding))(*[int(v) & 0xFFFFFFFF for v in meta_binding])
        h = C.c_void_p()
        self._check(self.lib.fg_exec_create(self.handle, graph.handle, meta, len(meta_binding), GEMM_MODE[gemm_mode],
                                            C.byref(h)))
        if graph.optim == 1 and state:
            lr = struct.unpack("<f", struct.pack("<I", int(meta_binding[0]) & 0xFFFFFFFF))[0]
            hp = _lib.AdamWHyper(lr, state[0], state[1], state[2], state[3])
            self._check(self.lib.fg_exec_set_adamw(h, C.byref(hp)))
        return AllocTensors(self, h, meta_binding)

    def compile(self, ir, options=None):
        return ("kernels", ir)

    def schedule(self, kernels, meta_binding, in_tensors, saved_tensors, extra=(), state=(), trainable=None):
        arr = (C.c_void_p * len(in_tensors))(*[t.as_buffer().handle if isinstance(t, Tensor) else t.handle
                                                for t in in_tensors])
        mask = None if trainable is None else bytes(bytearray(int(bool(t)) for t in trainable))
        self._check(self.lib.fg_exec_bind(saved_tensors.handle, arr, len(in_tensors), mask))
        return Schedule(saved_tensors)

    def dispatch_forward(self, schedule):
        self._check(self.lib.fg_exec_dispatch_forward(schedule.tensors.handle))

    def dispatch_backward(self, schedule):
        self._check(self.lib.fg_exec_dispatch_backward(schedule.tensors.handle))

    def dispatch_loss(self, schedule, target):
        buf = target.as_buffer() if isinstance(target, Tensor) else target
        self._check(self.lib.fg_exec_dispatch_loss(schedule.tensors.handle, buf.handle))

    def dispatch_optim(self, schedule):
        self._check(self.lib.fg_exec_dispatch_optim(schedule.tensors.handle))

    def dispatch_single_optim(self, schedule, weight, grad, tensors=None):
        buf = weight.as_buffer() if isinstance(weight, Tensor) else weight
        self._check(self.lib.fg_exec_dispatch_single_optim(schedule.tensors.handle, buf.handle, int(grad)))

    def new_onehot_init(self, labels):
        """Labels for CROSS_ENTROPY: one u32 class index per row (dispatch/mod.rs:656-662)."""
        a = np.ascontiguousarray(labels, dtype=np.uint32)
        return self.init_tensor_u32(a.shape, a)


def _install():
    """GpuContext gets the graph methods (one class in the reference: dispatch/mod.rs:352-833)."""
    from .backend import GpuContext
    for name, fn in vars(GraphContextMixin).items():
        if callable(fn) and not name.startswith("__"):
            setattr(GpuContext, name, fn)


_install()
