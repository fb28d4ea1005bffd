"""Data-parallel MLP training on the C ABI: forward -> loss -> backward -> gradient
exchange -> update, the order of the reference's training loop
(crates/ferrograd/examples/save_load_model.rs:148-156: dispatch_forward, dispatch_loss,
dispatch_backward, dispatch_optim).

Buffer roles follow the reference's `AllocTensors` (crates/fused_gpu/src/dispatch/mod.rs:835-845):
`act[l]` / `pre[l]` are the forward_saved tensors (a matmul output is always saved,
op/matmul/mod.rs:191-202; GELU additionally needs its pre-activation), `grads` the
grad_tensors, `dact` the seed (dL/dout) and the intermediate gradients, `loss_row` /
`loss_sum` the loss tensor.  Unlike the reference, all parameters live in ONE flat arena
(W0, b0, W1, b1, ...), with gradients and optimizer moments in arenas of the same layout,
so the update is a single fused pass and each layer's gradient is one contiguous range
for the allreduce.

In the default GEMM mode every tensor a tensor-core GEMM reads (weights, activations, the
gradients dZ) keeps its bf16 pairs beside it, written by whoever writes the tensor: the
forward epilogue, the dA epilogue (which also applies the activation derivative of the
layer below and sums the columns for its bias gradient), the narrow layer's dA kernel and
the optimizer.  No operand pre-pass and no transposition is left in the step; only the
input batch, which arrives from outside, gets its pairs from a kernel of its own.
"""
import numpy as np

from .backend import GpuContext


def _align(n, a=64):
    return (n + a - 1) // a * a


class MLPTrainer:
    def __init__(self, ctx: GpuContext, dims, batch, hidden_act="gelu", loss="ce",
                 optimizer=("adamw", 1e-3, 0.9, 0.999, 1e-8, 0.01), grad_scale=None, world=1, rank=0,
                 gemm_mode="auto", overlap_comm=True):
        self.ctx = ctx
        self.dims = [int(d) for d in dims]
        self.L = len(self.dims) - 1
        self.batch = int(batch)
        self.act = hidden_act
        self.loss_kind = loss
        self.opt = optimizer
        self.world, self.rank = int(world), int(rank)
        self.mode = gemm_mode
        self.overlap = overlap_comm
        self.min_exchange = 1 << 20     # elements: smaller layers ride along with the next exchange
        od = self.dims[-1]
        if grad_scale is None:
            # mean loss over the GLOBAL batch (and over output elements for MSE)
            grad_scale = 1.0 / (self.batch * self.world * (od if loss == "mse" else 1))
        self.grad_scale = float(grad_scale)

        # ---- flat parameter arena: [W0 | b0 | W1 | b1 | ...], every tensor 256-byte aligned ----
        self.w_off, self.b_off = [], []
        off = 0
        for l in range(self.L):
            self.w_off.append(off)
            off = _align(off + self.dims[l] * self.dims[l + 1])
            self.b_off.append(off)
            off = _align(off + self.dims[l + 1])
        self.n_arena = off
        self.layer_range = [(self.w_off[l], (self.w_off[l + 1] if l + 1 < self.L else off)) for l in range(self.L)]
        self.n_params = sum(self.dims[l] * self.dims[l + 1] + self.dims[l + 1] for l in range(self.L))
        nb = self.n_arena * 4
        self.params = ctx.alloc_zeroed(nb)
        self.grads = ctx.alloc_zeroed(nb)
        self.m = ctx.alloc_zeroed(nb) if optimizer[0] == "adamw" else None
        self.v = ctx.alloc_zeroed(nb) if optimizer[0] == "adamw" else None
        self.step_counter = ctx.alloc_zeroed(256)

        # ---- activations, saved tensors, gradients of activations ----
        B = self.batch
        self.x = ctx.alloc(B * self.dims[0] * 4)
        self.act_buf = [self.x] + [ctx.alloc(B * self.dims[l + 1] * 4) for l in range(self.L)]
        self.pre_buf = [ctx.alloc(B * self.dims[l + 1] * 4) if (hidden_act == "gelu" and l < self.L - 1) else None
                        for l in range(self.L)]
        self.dact = [None] + [ctx.alloc(B * self.dims[l + 1] * 4) for l in range(self.L)]
        if loss == "ce":
            self.target = ctx.alloc(B * 4)
            self.loss_row = ctx.alloc(B * 4)
        else:
            self.target = ctx.alloc(B * od * 4)
            self.loss_row = None
        self.loss_out = ctx.alloc_zeroed(256)     # one float: mean CE loss, or summed squared error
        self.plan = None
        self.steps_done = 0
        # ---- bf16 pairs (default GEMM mode): weights [2][n_arena], activations and dZ [2][B*d] each ----
        self.paired = gemm_mode == "auto"
        if self.paired:
            self.w_pairs = ctx.alloc_zeroed(2 * self.n_arena * 2)
            self.act_pairs = [ctx.alloc(2 * B * self.dims[l] * 2) for l in range(self.L)]
            # dz[l] = dL/d(pre-activation of layer l) lives in dact[l + 1]; the top layer's comes from the loss kernel
            self.dz_pairs = [ctx.alloc(2 * B * self.dims[l + 1] * 2) if l < self.L - 1 else None for l in range(self.L)]

    # ---- parameter access ----
    def W(self, l):
        return self.params.ptr + 4 * self.w_off[l]

    def b(self, l):
        return self.params.ptr + 4 * self.b_off[l]

    def gW(self, l):
        return self.grads.ptr + 4 * self.w_off[l]

    def gb(self, l):
        return self.grads.ptr + 4 * self.b_off[l]

    def set_params(self, W, b):
        arena = np.zeros(self.n_arena, np.float32)
        for l in range(self.L):
            arena[self.w_off[l]:self.w_off[l] + W[l].size] = np.asarray(W[l], np.float32).ravel()
            arena[self.b_off[l]:self.b_off[l] + b[l].size] = np.asarray(b[l], np.float32).ravel()
        self.ctx.upload(self.params, arena)
        if self.paired:
            self.ctx.pairs_from_f32(self.params, self.n_arena, self.w_pairs, self.n_arena)

    # ---- checkpoints ----
    def _arena_tensors(self, host_arena):
        """[W0, b0, W1, b1, ...] as device tensors made from a host copy of an arena."""
        out = []
        for l in range(self.L):
            k, n = self.dims[l], self.dims[l + 1]
            out.append(self.ctx.init_tensor_f32((k, n), host_arena[self.w_off[l]:self.w_off[l] + k * n]))
            out.append(self.ctx.init_tensor_f32((n,), host_arena[self.b_off[l]:self.b_off[l] + n]))
        return out

    def save_checkpoint(self, path):
        """Parameters as a v2-f32 `.bpat` file in the reference's order (W0, b0, W1, b1, ...), readable by the
        reference's load_tensors; with AdamW, its moments and step count go to `path + ".adamw"`
        (bpat.save_adamw_state: not a reference format)."""
        from . import bpat
        self.ctx.sync()
        arena = lambda buf: self.ctx.download(buf, np.empty(self.n_arena, np.float32))
        ts = self._arena_tensors(arena(self.params))
        try:
            bpat.save_tensors(self.ctx, path, ts)
        finally:
            for t in ts:
                t.data.free()
        if self.opt[0] == "adamw":
            m, v = self._arena_tensors(arena(self.m)), self._arena_tensors(arena(self.v))
            try:
                bpat.save_adamw_state(self.ctx, str(path) + ".adamw", m, v, self.steps_done)
            finally:
                for t in m + v:
                    t.data.free()

    def load_checkpoint(self, path):
        """Inverse of save_checkpoint; training continues with the step count it had."""
        import os
        from . import bpat
        ts = bpat.load_tensors(self.ctx, path)
        try:
            if [t.shape for t in ts] != [s for l in range(self.L) for s in ((self.dims[l], self.dims[l + 1]), (self.dims[l + 1],))]:
                raise ValueError(f"{path}: tensor shapes do not match this network")
            host = [self.ctx.to_numpy(t) for t in ts]
        finally:
            for t in ts:
                t.data.free()
        self.set_params(host[0::2], host[1::2])
        if self.opt[0] == "adamw" and os.path.exists(str(path) + ".adamw"):
            m, v, step = bpat.load_adamw_state(self.ctx, str(path) + ".adamw")
            try:
                for buf, lst in ((self.m, m), (self.v, v)):
                    a = np.zeros(self.n_arena, np.float32)
                    for l in range(self.L):
                        w, bb = self.ctx.to_numpy(lst[2 * l]), self.ctx.to_numpy(lst[2 * l + 1])
                        a[self.w_off[l]:self.w_off[l] + w.size] = w.ravel()
                        a[self.b_off[l]:self.b_off[l] + bb.size] = bb.ravel()
                    self.ctx.upload(buf, a)
            finally:
                for t in m + v:
                    t.data.free()
            self.ctx.upload(self.step_counter, np.array([step], np.uint32))
            self.steps_done = step

    def destroy(self):
        """Frees every device buffer of the trainer."""
        from .backend import Buffer
        if self.plan is not None:
            self.plan.destroy()
            self.plan = None
        for v in list(vars(self).values()):
            for b in (v if isinstance(v, (list, tuple)) else [v]):
                if isinstance(b, Buffer):
                    b.free()

    def reset_state(self):
        """Zeroes gradients, optimizer moments and the step counter (a fresh start from the current parameters)."""
        nb = self.n_arena * 4
        self.ctx.memset_zero(self.grads, nb)
        if self.m is not None:
            self.ctx.memset_zero(self.m, nb)
            self.ctx.memset_zero(self.v, nb)
        self.ctx.memset_zero(self.step_counter, 256)
        self.steps_done = 0

    def _split(self, arena):
        W = [arena[self.w_off[l]:self.w_off[l] + self.dims[l] * self.dims[l + 1]]
             .reshape(self.dims[l], self.dims[l + 1]).copy() for l in range(self.L)]
        b = [arena[self.b_off[l]:self.b_off[l] + self.dims[l + 1]].copy() for l in range(self.L)]
        return W, b

    def get_params(self):
        return self._split(self.ctx.download(self.params, np.empty(self.n_arena, np.float32)))

    def get_grads(self):
        return self._split(self.ctx.download(self.grads, np.empty(self.n_arena, np.float32)))

    def get_output(self):
        return self.ctx.download(self.act_buf[self.L], np.empty((self.batch, self.dims[-1]), np.float32))

    def get_loss(self):
        return float(self.ctx.download(self.loss_out, np.empty(1, np.float32))[0])

    @staticmethod
    def init_params(dims, init="he_normal", seed=7):
        """Host-side initial weights, identical on every rank (biases zero)."""
        r = np.random.Generator(np.random.Philox(seed))
        W, b = [], []
        for l in range(len(dims) - 1):
            fi, fo = dims[l], dims[l + 1]
            if init == "he_normal":
                w = r.standard_normal((fi, fo), np.float32) * np.float32(np.sqrt(2.0 / fi))
            elif init == "xavier_uniform":
                lim = np.sqrt(6.0 / (fi + fo))
                w = r.uniform(-lim, lim, (fi, fo)).astype(np.float32)
            else:   # "normal_fan_in": N(0, 1/sqrt(fan_in))
                w = r.standard_normal((fi, fo), np.float32) * np.float32(1.0 / np.sqrt(fi))
            W.append(w.astype(np.float32))
            b.append(np.zeros(fo, np.float32))
        return W, b

    # ---- data ----
    def upload_batch(self, x, target):
        self.ctx.upload(self.x, np.ascontiguousarray(x, np.float32))
        t = np.ascontiguousarray(target, np.uint32 if self.loss_kind == "ce" else np.float32)
        self.ctx.upload(self.target, t)

    def upload_batch_async(self, x_pinned, target_pinned):
        """x_pinned / target_pinned: numpy arrays over page-locked memory (ctx.pinned_array)."""
        self.ctx.upload_async(self.x, x_pinned.ctypes.data, x_pinned.nbytes)
        self.ctx.upload_async(self.target, target_pinned.ctypes.data, target_pinned.nbytes)

    def prefetch_batch(self, x_pinned, target_pinned):
        """Starts copying the NEXT batch into staging buffers on the copy stream; it overlaps the step that
        is running.  take_prefetched() then moves it into place at device speed."""
        if not hasattr(self, "stage_x"):
            self.stage_x = self.ctx.alloc(x_pinned.nbytes)
            self.stage_t = self.ctx.alloc(target_pinned.nbytes)
        self.ctx.upload_prefetch(self.stage_x, x_pinned.ctypes.data, x_pinned.nbytes)
        self.ctx.upload_prefetch(self.stage_t, target_pinned.ctypes.data, target_pinned.nbytes)
        self._staged = (x_pinned.nbytes, target_pinned.nbytes)

    def take_prefetched(self):
        nx, nt = self._staged
        self.ctx.prefetch_wait()
        self.ctx.copy_dev_async(self.x, self.stage_x, nx)
        self.ctx.copy_dev_async(self.target, self.stage_t, nt)
        self.ctx.prefetch_mark()

    # ---- one training step, enqueued on the context's stream ----
    def Wp(self, l):
        return self.w_pairs.ptr + 2 * self.w_off[l]

    def _enqueue_step_paired(self):
        """The step on f32 tensors with bf16 pairs: no operand pre-pass between the GEMMs."""
        c, B, L, d = self.ctx, self.batch, self.L, self.dims
        c.pairs_from_f32(self.x, B * d[0], self.act_pairs[0])
        for l in range(L):
            a = self.act if l < L - 1 else "none"
            c.gemm_paired(self.act_buf[l], self.W(l), self.act_buf[l + 1], B, d[l + 1], d[l],
                          A_pairs=self.act_pairs[l], B_pairs=self.Wp(l), B_stride=self.n_arena, bias=self.b(l), act=a,
                          preact_out=self.pre_buf[l], C_pairs=self.act_pairs[l + 1] if l + 1 < L else None)
        od = d[-1]
        if self.loss_kind == "ce":
            c.softmax_ce(self.act_buf[L], self.target, B, od, grad_scale=self.grad_scale, loss_row=self.loss_row,
                         loss_mean=self.loss_out, dlogits=self.dact[L])
        else:
            c.mse_loss_grad(self.act_buf[L], self.target, B * od, grad_scale=self.grad_scale,
                            loss_sum=self.loss_out, grad=self.dact[L])
        pend_hi = self.n_arena
        exchanged = []
        for l in range(L - 1, -1, -1):
            # the layer below (l - 1) has the hidden activation; its saved tensor is its pre-activation (GELU)
            # or its output, which is this layer's input
            below = self.act if l > 0 else "none"
            below_saved = None if l == 0 else (self.pre_buf[l - 1] if self.act == "gelu" else self.act_buf[l])
            lo = self.layer_range[l][0]
            exch = self.world > 1 and self.overlap and (l == 0 or pend_hi - lo >= self.min_exchange)
            c.gemm_bwd_paired(self.act_buf[l], self.W(l), self.dact[l + 1], B, d[l + 1], d[l],
                              A_pairs=self.act_pairs[l], B_pairs=self.Wp(l), B_stride=self.n_arena,
                              dZ_pairs=self.dz_pairs[l], dB=self.gW(l), dbias=self.gb(l) if l == L - 1 else None,
                              dA=self.dact[l] if l > 0 else None, below_act=below, below_saved=below_saved,
                              dA_pairs=self.dz_pairs[l - 1] if l > 0 else None,
                              below_dbias=self.gb(l - 1) if l > 0 else None,
                              exch_buf=self.grads.ptr + 4 * lo if exch else None, exch_count=pend_hi - lo if exch else 0)
            if exch:
                # NOTE: the bias gradient of layer l - 1 is written by this call's dA epilogue, after the
                # exchange of [lo, pend_hi) has started; it belongs to the range below lo, exchanged later.
                if len(exchanged) < 7:
                    c.comm_checkpoint(len(exchanged))
                    exchanged.append((lo, pend_hi, len(exchanged)))
                else:
                    exchanged.append((lo, pend_hi, -1))
                pend_hi = lo
        return exchanged

    def enqueue_step(self):
        c, B, L = self.ctx, self.batch, self.L
        if self.paired:
            return self._finish_step(self._enqueue_step_paired())
        for l in range(L):
            a = self.act if l < L - 1 else "none"
            c.gemm(self.act_buf[l], self.W(l), self.act_buf[l + 1], B, self.dims[l + 1], self.dims[l],
                   bias=self.b(l), act=a, preact_out=self.pre_buf[l], mode=self.mode)
        od = self.dims[-1]
        if self.loss_kind == "ce":
            c.softmax_ce(self.act_buf[L], self.target, B, od, grad_scale=self.grad_scale, loss_row=self.loss_row,
                         loss_mean=self.loss_out, dlogits=self.dact[L])
        else:
            c.mse_loss_grad(self.act_buf[L], self.target, B * od, grad_scale=self.grad_scale,
                            loss_sum=self.loss_out, grad=self.dact[L])
        # Gradient exchange: layers are contiguous in the arena, so consecutive layers can share one call.
        # A layer's gradients wait for the next layer's when they are small (a 10-class head is not worth a
        # launch, and the GEMMs give up SMs while an exchange is in flight).
        pend_hi = self.n_arena
        exchanged = []      # (lo, hi, checkpoint slot) of every exchange, in issue order
        for l in range(L - 1, -1, -1):
            a = self.act if l < L - 1 else "none"
            saved = None if a == "none" else (self.pre_buf[l] if a == "gelu" else self.act_buf[l + 1])
            args = (self.act_buf[l], self.W(l), self.dact[l + 1], B, self.dims[l + 1], self.dims[l])
            kw = dict(act=a, saved=saved, dA=self.dact[l] if l > 0 else None, dB=self.gW(l), dbias=self.gb(l),
                      mode=self.mode)
            lo = self.layer_range[l][0]
            if self.world > 1 and self.overlap and (l == 0 or pend_hi - lo >= self.min_exchange):
                # weight and bias gradients first; their exchange runs beside this layer's dX GEMM and the
                # backward of the layers below
                c.gemm_bwd_exchange(*args, self.grads.ptr + 4 * lo, pend_hi - lo, **kw)
                if len(exchanged) < 7:
                    c.comm_checkpoint(len(exchanged))
                    exchanged.append((lo, pend_hi, len(exchanged)))
                else:                                   # out of checkpoint slots: this range waits for the join
                    exchanged.append((lo, pend_hi, -1))
                pend_hi = lo
            else:
                c.gemm_bwd(*args, **kw)
        self._finish_step(exchanged)

    def _finish_step(self, exchanged):
        c = self.ctx
        # gradients were computed with the global-mean scale, so the sum over ranks needs no further factor
        if self.opt[0] == "adamw":
            c.counter_increment(self.step_counter)
        if self.world > 1 and self.overlap and len(exchanged) > 1 and all(s >= 0 for _, _, s in exchanged):
            # update each exchanged range as soon as its own exchange is complete: the last layers' update
            # runs while the first layer's gradients are still on the wire
            for lo, hi, slot in exchanged[:-1]:
                c.comm_wait(slot)
                self._update(lo, hi)
            c.comm_join()
            self._update(*exchanged[-1][:2])
            return
        if self.world > 1:
            if not self.overlap:
                c.allreduce_sum(self.grads, self.n_arena)
            c.comm_join()
        self._update(0, self.n_arena)

    def _update(self, lo, hi):
        """The optimizer step on arena elements [lo, hi)."""
        c, off, n = self.ctx, 4 * lo, hi - lo
        wp = self.w_pairs.ptr + 2 * lo if self.paired else None      # the updated weights' pairs, same pass
        if self.opt[0] == "adamw":
            _, lr, b1, b2, eps, wd = self.opt
            c.adamw_step_paired(self.params.ptr + off, self.grads.ptr + off, self.m.ptr + off, self.v.ptr + off, n, lr,
                                b1, b2, eps, wd, wp, self.n_arena, step=0, step_dev=self.step_counter, zero_grad=False)
        elif self.opt[0] == "sgd":
            c.sgd_step_paired(self.params.ptr + off, self.grads.ptr + off, n, self.opt[1], wp, self.n_arena,
                              zero_grad=False)

    def step(self):
        """Eager step (one launch per kernel)."""
        self.enqueue_step()
        self.steps_done += 1

    def build_plan(self):
        """Records one step as a CUDA graph (the reference's Schedule).  Run one eager step first so
        that the scratch arena has its final size."""
        self.ctx.plan_begin()
        try:
            self.enqueue_step()
        finally:
            self.plan = self.ctx.plan_end()
        return self.plan

    def step_plan(self):
        self.plan.launch()
        self.steps_done += 1

    # flop of one step on this rank (2*M*N*K per GEMM; no dX for the first layer)
    def flops_per_step(self):
        f = 0
        for l in range(self.L):
            g = 2 * self.batch * self.dims[l] * self.dims[l + 1]
            f += g * (3 if l > 0 else 2)
        return f


class GraphMLP:
    """The same training step written against the mirrored graph API, the way a ferrograd program is
    (crates/ferrograd/examples/save_load_model.rs:148-156): Graph / define_ops / alloc_tensors / schedule, then
    dispatch_forward, dispatch_loss, dispatch_backward, dispatch_optim per step.  Reference semantics: the loss is
    unreduced (gradients are sums over the batch, not means), every weight and bias is its own tensor.  With a
    communicator on the context (ctx.comm_init) the engine sums the gradients over the ranks."""

    def __init__(self, ctx: GpuContext, dims, batch, hidden_act="gelu", loss="ce",
                 optimizer=("adamw", 1e-3, 0.9, 0.999, 1e-8, 0.01), gemm_mode="auto"):
        from .graph import CROSS_ENTROPY, MEAN_SQUARED_ERROR, Graph, Metadata, Optim, f32_bits
        self.ctx, self.dims, self.batch, self.loss_kind = ctx, [int(d) for d in dims], int(batch), loss
        self.L = L = len(self.dims) - 1
        meta = Metadata.new()
        fb = meta.new_field()
        fd = [meta.new_field() for _ in self.dims]
        self.opt = Optim.adamw(*optimizer[2:]) if optimizer[0] == "adamw" else Optim.sgd()
        self.graph = Graph.new(CROSS_ENTROPY if loss == "ce" else MEAN_SQUARED_ERROR, self.opt.lower)
        g = self.graph.define_ops()
        h = g.input([fb, fd[0]])
        for l in range(L):
            h = g.add(g.matmul(h, g.input([fd[l], fd[l + 1]])), g.input([fd[l + 1]]))
            if l < L - 1:
                h = getattr(g, hidden_act)(h)
        if loss == "ce":
            g.softmax(h)
        binding = [f32_bits(optimizer[1]), self.batch] + self.dims
        self.tensors = ctx.alloc_tensors(self.graph, self.graph.compute_saved_nodes(), ctx.alloc_meta(binding), self.opt.state,
                                         gemm_mode=gemm_mode)
        kernels = ctx.compile(self.graph.lower(meta, None, None), None)
        self.x = ctx.new_tensor((self.batch, self.dims[0]))
        self.W = [ctx.new_tensor((self.dims[l], self.dims[l + 1]), zeroed=True) for l in range(L)]
        self.b = [ctx.new_tensor((self.dims[l + 1],), zeroed=True) for l in range(L)]
        od = self.dims[-1]
        self.target = ctx.new_tensor((self.batch,), np.uint32) if loss == "ce" else ctx.new_tensor((self.batch, od))
        ins = [self.x]
        for l in range(L):
            ins += [self.W[l], self.b[l]]
        self.schedule = ctx.schedule(kernels, binding, ins, self.tensors, [], self.opt.state, trainable=[0] + [1] * (2 * L))
        self.loss_out = self.tensors.loss_sum
        self.n_params = sum(self.dims[l] * self.dims[l + 1] + self.dims[l + 1] for l in range(L))

    def set_params(self, W, b):
        for l in range(self.L):
            self.ctx.upload(self.W[l], np.asarray(W[l], np.float32))
            self.ctx.upload(self.b[l], np.asarray(b[l], np.float32))

    def get_params(self):
        return [self.ctx.to_numpy(w) for w in self.W], [self.ctx.to_numpy(v) for v in self.b]

    def upload_batch(self, x, target):
        self.ctx.upload(self.x, np.ascontiguousarray(x, np.float32))
        self.ctx.upload(self.target, np.ascontiguousarray(target, np.uint32 if self.loss_kind == "ce" else np.float32))

    def upload_batch_async(self, x_pinned, target_pinned):
        self.ctx.upload_async(self.x, x_pinned.ctypes.data, x_pinned.nbytes)
        self.ctx.upload_async(self.target, target_pinned.ctypes.data, target_pinned.nbytes)

    prefetch_batch = MLPTrainer.prefetch_batch
    take_prefetched = MLPTrainer.take_prefetched

    def step(self):
        c, s = self.ctx, self.schedule
        c.dispatch_forward(s)
        c.dispatch_loss(s, self.target)
        c.dispatch_backward(s)
        c.dispatch_optim(s)

    def get_loss(self):
        """Sum of the unreduced loss tensor (cross-entropy: over the rows; MSE: over all elements)."""
        return float(self.ctx.download(self.loss_out, np.empty(1, np.float32))[0])

    def get_output(self):
        return self.ctx.download(self.tensors.forward_out, np.empty((self.batch, self.dims[-1]), np.float32))

    def flops_per_step(self):
        return sum(2 * self.batch * self.dims[l] * self.dims[l + 1] * (3 if l > 0 else 2) for l in range(self.L))

    def destroy(self):
        self.tensors.destroy()
        for t in [self.x, self.target] + self.W + self.b:
            t.data.free()
        for name in ("stage_x", "stage_t"):
            if hasattr(self, name):
                getattr(self, name).free()
