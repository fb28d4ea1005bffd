// Graph engine: ferrograd graphs executed with the hand-written kernels.
//
// What it stands in for.  In the reference a user builds a `Graph` of nodes
// (crates/fused_gpu/src/dispatch/backend/mod.rs:500-506, :978-1316; ops from
// crates/ferrograd/src/graph.rs:111-158), `compute_saved_nodes` decides what persists between
// forward and backward (backend/mod.rs:1189-1208), `alloc_tensors` creates forward_saved /
// grad_tensors / forward_out / seed / loss_t (dispatch/mod.rs:509-575), the lowering drivers turn the
// graph into fused kernels (kernel/forward.rs:19-281, kernel/backward.rs:19-227, kernel/loss.rs,
// kernel/optim.rs) and `schedule` binds buffers (dispatch/mod.rs:664-764).  Here the same graph is
// lowered to calls of this library's entry points instead of generated code:
//   * matmul, optionally followed by `+ bias[N]` and tanh/relu/gelu with single consumers, becomes
//     one fg_gemm_f32 with a fused epilogue (the reference fuses trailing elementwise ops into the
//     matmul kernel the same way: kernel/forward.rs:373-457); its backward is one fg_gemm_bwd_f32;
//   * every maximal region of elementwise nodes becomes one fg_eltwise_chain_fwd and one
//     fg_eltwise_chain_bwd (the reference inlines elementwise producers into their consumer:
//     kernel/forward.rs:298-464);
//   * softmax is fg_softmax_fwd / fg_softmax_bwd.
// A node is materialised (gets a buffer) when it is a matmul/softmax/fused-GEMM result, the graph
// output, has more than one consumer, or feeds a matmul/softmax; everything else lives in registers
// inside a chain kernel.
//
// The default GEMM mode multiplies f32 tensors as they lie with their bf16 pairs beside them
// (fg_gemm_paired_f32): the engine keeps pairs for every tensor a matmul reads, written by whoever
// writes the tensor -- the producing GEMM's epilogue, the optimizer (weights), or one elementwise
// kernel for tensors that arrive from outside.  In the backward pass a matmul whose first operand is
// the fused result of another matmul (x·W + b, activation) applies that layer's activation derivative
// in its own dA epilogue, which also writes the pairs of the result and sums its columns into the
// layer's bias gradient; the gradient tensor of such a node therefore holds dL/d(pre-activation).
//
// Data parallelism (no counterpart in the reference, which is single device): when the context has a
// communicator (fg_comm_init), dispatch_backward sums the gradients of the trainable inputs over the
// ranks.  Those gradients live in one arena in the order in which the backward pass completes them, so
// what is complete is always a contiguous range: each matmul's backward starts the exchange of the
// range completed so far between its dB and its dA product, and dispatch_optim starts the exchange of
// the last range, updates the tensors of the earlier ranges beside it, and updates the last range when
// it has arrived.
//
// Deviations from the reference, by design: a softmax that ends the graph under the CROSS_ENTROPY
// loss is not differentiated a second time (the loss kernel's p - onehot already is dL/dlogits;
// the reference pushes it through the softmax backward again, dispatch/mod.rs:713-718); shapes
// need not be multiples of 16; `add` accepts a bias of shape [N] or [1,N] after a matmul.
#include <limits.h>
#include <stdlib.h>

#include <algorithm>
#include <functional>
#include <new>
#include <vector>

#include "fg_internal.cuh"

namespace {

enum { OP_MATMUL = FG_GRAPH_MATMUL, OP_SOFTMAX = FG_GRAPH_SOFTMAX };

struct GNode {
    int op, a, b;
    float imm;
    std::vector<uint32_t> fields;   // INPUT: one metadata field id per dimension
    int dtype = FG_DTYPE_F32;       // INPUT: storage type
};

inline bool is_ew(int op) { return op >= FG_EW_ADD && op <= FG_EW_ELU; }
inline bool is_binary(int op) { return op >= FG_EW_ADD && op <= FG_EW_DIV; }

}  // namespace

struct fg_graph {
    std::vector<GNode> nodes;
    int loss, optim;
};

namespace {

struct ENode {
    std::vector<uint32_t> dims;
    uint64_t numel = 0;
    int consumers = 0;
    bool materialized = false;   // has a value buffer
    bool absorbed = false;       // computed inside a fused GEMM epilogue, never stored on its own
    bool bias_bcast = false;     // ADD whose second operand is a [N] bias (legal only after a matmul)
    fg_buf* value = nullptr;     // owned, or the bound input tensor
    bool own_value = false;
    fg_buf* grad = nullptr;      // owned (a view into the gradient arena for inputs)
    int input_slot = -1;         // index among the graph's inputs
    fg_buf* pairs = nullptr;     // bf16 pairs of the value, for tensors a matmul reads (f32 graphs)
    int produced_by_gemm = -1;   // index of the GemmStep whose fused result this node is
};

struct GemmStep {
    int mm, a, b, bias, act, out;   // node ids; bias = -1 when absent; out = node whose buffer receives the result
    fg_buf* preact;                 // GELU needs the pre-activation
    // batch products of [M,K] x [K,N].  [T,M,K] x [T,K,N] is T products (the reference steps both operands
    // and the result by one matrix per Z index: kernel/forward.rs:159-190); [T,M,K] x [K,N] is one product
    // with T*M rows.
    uint32_t batch, M, K, N;
    fg_buf* dz_pairs = nullptr;     // pairs of dL/d(pre-activation), written by the consumer's dA epilogue
    bool dz_ready = false;          // this backward pass: grad(out) already holds dL/d(pre-activation)
    bool dbias_done = false;        // this backward pass: the bias gradient came out of the consumer's dA epilogue
};
struct ChainStep {
    int root;
    std::vector<fg_ew_instr> prog;
    std::vector<int> inputs;        // node ids of the loaded values
};
struct Step {
    int kind;   // 0 gemm, 1 chain, 2 softmax
    int idx;    // index into gemms / chains, or the softmax node id
};

}  // namespace

struct fg_exec {
    fg_ctx* ctx;
    fg_graph g;
    std::vector<uint32_t> meta;
    int gemm_mode;
    std::vector<ENode> n;
    std::vector<GemmStep> gemms;
    std::vector<ChainStep> chains;
    std::vector<Step> fwd;          // in execution order; backward walks it in reverse
    std::vector<int> inputs;        // node ids of INPUT nodes, in order
    std::vector<int> saved;         // materialised non-input nodes except the output, in node order
    std::vector<int> grads;         // nodes that own a gradient buffer, in node order
    std::vector<uint8_t> trainable;
    fg_buf *seed = nullptr, *loss_t = nullptr, *tmp = nullptr, *loss_sum = nullptr;
    fg_buf* stage[4] = {nullptr, nullptr, nullptr, nullptr};   // 16-bit graphs: f32 staging for softmax and the losses
    std::vector<fg_buf*> m, v;      // AdamW moments per input
    fg_buf* step_counter = nullptr;
    fg_adamw_hyper hyper{1e-3f, 0.9f, 0.999f, 1e-8f, 0.01f};
    bool bound = false;
    int last;                       // output node
    int dtype = FG_DTYPE_F32;       // storage type of every tensor of the graph
    uint64_t esize = 4;
    // Each dispatch_* is recorded as a CUDA graph on its second call and replayed from then on (the
    // reference's Schedule is a captured hipGraph: rocm/mod.rs:324-389).  0 forward, 1 loss, 2 backward, 3 optim.
    fg_plan* plan[4] = {nullptr, nullptr, nullptr, nullptr};
    int calls[4] = {0, 0, 0, 0};
    const void* plan_key[4] = {nullptr, nullptr, nullptr, nullptr};   // loss: the target buffer
    const void* plan_ws[4] = {nullptr, nullptr, nullptr, nullptr};    // scratch arena the plan was recorded against
    bool use_plans = true;
    bool ce_softmax_tail = false;   // graph ends in softmax and the loss is cross-entropy
    // Gradients (and AdamW moments) of the inputs: one arena each, tensors in the order in which the backward
    // pass completes them.  ready_key[slot] = 2 * (backward step that completes it) + (0: by the time the step's
    // dB is done, 1: at the end of the step).
    fg_buf *grad_arena = nullptr, *m_arena = nullptr, *v_arena = nullptr;
    uint64_t arena_elems = 0;
    std::vector<int> arena_order;          // input slots in arena order
    std::vector<uint64_t> arena_off;       // per input slot: element offset in the arenas
    std::vector<int> ready_key;            // per input slot
    std::vector<uint64_t> pairs_version;   // per input slot: version of the bound tensor its pairs were made from
    std::vector<uint8_t> pairs_fresh;      // per input slot
    bool paired = false;                   // f32 graph in the default GEMM mode: keep pairs, fuse the backward epilogues
    // data-parallel state of one step
    uint64_t exchanged_end = 0;            // arena elements whose exchange has been started by dispatch_backward
    uint64_t final_lo = 0;                 // [final_lo, arena_elems): exchanged by dispatch_optim (set by the backward pass)
    uint64_t optim_lo = 0;                 // the value dispatch_optim works with: final_lo after a backward pass, else 0
    bool backward_done = false;            // a backward pass has run since the last dispatch_optim
};

namespace {

int32_t fail(fg_exec* e, int32_t code, const char* msg) { return fg_fail(e->ctx, code, msg); }

float* vptr(fg_exec* e, int node) { return (float*)e->n[node].value->ptr; }
// Elements between the two planes of a tensor's bf16 pairs: its size rounded up to a multiple of 8.
uint64_t pstride(const fg_exec* e, int node) { return (e->n[node].numel + 7) / 8 * 8; }
float* gptr(fg_exec* e, int node) { return (float*)e->n[node].grad->ptr; }

// Emits the straight-line program that computes `node` from materialised values.
int emit(fg_exec* e, ChainStep& c, int node, int root, int32_t* status) {
    if (*status != FG_OK) return 0;
    const GNode& gn = e->g.nodes[node];
    auto push = [&](int op, int a, int b, float imm) -> int {
        if ((int)c.prog.size() >= FG_EW_MAX_INSTR) { *status = FG_ERR_UNSUPPORTED_FEATURE; return 0; }
        c.prog.push_back(fg_ew_instr{op, a, b, imm});
        return (int)c.prog.size() - 1;
    };
    if (gn.op == FG_EW_CONST) return push(FG_EW_CONST, 0, 0, gn.imm);
    if (node != root && (e->n[node].materialized || gn.op == FG_EW_INPUT)) {
        int slot = -1;
        for (size_t k = 0; k < c.inputs.size(); ++k) if (c.inputs[k] == node) slot = (int)k;
        if (slot < 0) {
            if ((int)c.inputs.size() >= FG_EW_MAX_INPUTS) { *status = FG_ERR_UNSUPPORTED_FEATURE; return 0; }
            c.inputs.push_back(node);
            slot = (int)c.inputs.size() - 1;
        }
        return push(FG_EW_INPUT, slot, 0, 0.0f);
    }
    int va = emit(e, c, gn.a, root, status);
    int vb = is_binary(gn.op) ? emit(e, c, gn.b, root, status) : 0;
    return push(gn.op, va, vb, 0.0f);
}

int32_t alloc_buf(fg_exec* e, uint64_t numel, bool zero, fg_buf** out) {
    return zero ? fg_alloc_zeroed(e->ctx, numel * e->esize, out) : fg_alloc(e->ctx, numel * e->esize, out);
}

int act_of(int op) { return op == FG_EW_TANH ? FG_ACT_TANH : op == FG_EW_RELU ? FG_ACT_RELU : op == FG_EW_GELU ? FG_ACT_GELU : -1; }

// The single consumer of `node`, or -1.
int sole_consumer(const fg_exec* e, int node) {
    if (e->n[node].consumers != 1) return -1;
    for (size_t k = node + 1; k < e->g.nodes.size(); ++k) {
        const GNode& c = e->g.nodes[k];
        if (c.op == FG_EW_INPUT || c.op == FG_EW_CONST) continue;
        if (c.a == node || ((is_binary(c.op) || c.op == OP_MATMUL) && c.b == node)) return (int)k;
    }
    return -1;
}

int32_t lower(fg_exec* e) {
    fg_graph& g = e->g;
    const int N = (int)g.nodes.size();
    e->n.assign(N, ENode());
    e->last = N - 1;
    // ---- storage type: one per graph.  16-bit graphs run their elementwise regions and matmuls in ----
    // ---- that type (f32 accumulation); softmax and the losses are computed in f32 on widened      ----
    // ---- copies and rounded back; AdamW is f32-only.                                              ----
    {
        int dt = -1;
        for (const GNode& gn : g.nodes) {
            if (gn.op != FG_EW_INPUT) continue;
            if (dt >= 0 && gn.dtype != dt) return fail(e, FG_ERR_UNSUPPORTED_FEATURE, "graph: inputs of different storage types");
            dt = gn.dtype;
        }
        e->dtype = dt < 0 ? FG_DTYPE_F32 : dt;
        e->esize = e->dtype == FG_DTYPE_F32 ? 4 : 2;
    }
    // ---- shapes (the reference's validate: backend/mod.rs:854-975) ----
    for (int i = 0; i < N; ++i) {
        const GNode& gn = g.nodes[i];
        ENode& en = e->n[i];
        if (gn.op == FG_EW_INPUT) {
            for (uint32_t f : gn.fields) {
                if (f >= e->meta.size()) return fail(e, FG_ERR_INVALID_ARGUMENT, "graph: shape names a metadata field that is not bound");
                en.dims.push_back(e->meta[f]);
            }
            en.input_slot = (int)e->inputs.size();
            e->inputs.push_back(i);
        } else if (gn.op == FG_EW_CONST) {
            en.dims.clear();
        } else if (gn.op == OP_MATMUL) {
            const auto &da = e->n[gn.a].dims, &db = e->n[gn.b].dims;
            if (da.size() == 2 && db.size() == 2 && da[1] == db[0]) en.dims = {da[0], db[1]};
            else if (da.size() == 3 && db.size() == 3 && da[0] == db[0] && da[2] == db[1]) en.dims = {da[0], da[1], db[2]};
            else if (da.size() == 3 && db.size() == 2 && da[2] == db[0]) en.dims = {da[0], da[1], db[1]};
            else return fail(e, FG_ERR_INVALID_ARGUMENT, "graph: matmul needs [M,K] x [K,N], [T,M,K] x [T,K,N] or [T,M,K] x [K,N]");
        } else if (gn.op == OP_SOFTMAX) {
            en.dims = e->n[gn.a].dims;
            if (en.dims.empty()) return fail(e, FG_ERR_INVALID_ARGUMENT, "graph: softmax of a scalar");
        } else if (is_binary(gn.op)) {
            const auto &da = e->n[gn.a].dims, &db = e->n[gn.b].dims;
            const bool ca = g.nodes[gn.a].op == FG_EW_CONST, cb = g.nodes[gn.b].op == FG_EW_CONST;
            if (ca && cb) return fail(e, FG_ERR_UNSUPPORTED_FEATURE, "graph: operation on two constants");
            if (ca) en.dims = db;
            else if (cb) en.dims = da;
            else if (da == db) en.dims = da;
            else if (gn.op == FG_EW_ADD && da.size() == 2 && g.nodes[gn.b].op == FG_EW_INPUT &&
                     ((db.size() == 1 && db[0] == da[1]) || (db.size() == 2 && db[0] == 1 && db[1] == da[1]))) {
                en.dims = da;
                en.bias_bcast = true;
            } else return fail(e, FG_ERR_INVALID_ARGUMENT, "graph: elementwise operands must have identical shapes");
        } else if (is_ew(gn.op)) {
            if (g.nodes[gn.a].op == FG_EW_CONST) return fail(e, FG_ERR_UNSUPPORTED_FEATURE, "graph: unary op of a constant");
            en.dims = e->n[gn.a].dims;
        } else return fail(e, FG_ERR_INVALID_ARGUMENT, "graph: unknown op");
        en.numel = 1;
        for (uint32_t d : en.dims) en.numel *= d;
        if (gn.op != FG_EW_INPUT && gn.op != FG_EW_CONST) {
            e->n[gn.a].consumers++;
            if (is_binary(gn.op) || gn.op == OP_MATMUL) e->n[gn.b].consumers++;
        }
    }
    if (g.nodes[e->last].op == FG_EW_INPUT || g.nodes[e->last].op == FG_EW_CONST)
        return fail(e, FG_ERR_INVALID_ARGUMENT, "graph: the last node must be an operation");
    e->ce_softmax_tail = g.loss == FG_LOSS_CROSS_ENTROPY && g.nodes[e->last].op == OP_SOFTMAX;

    // ---- fused GEMM patterns ----
    std::vector<int> gemm_of_out(N, -1);
    for (int i = 0; i < N; ++i) {
        if (g.nodes[i].op != OP_MATMUL) continue;
        if (g.nodes[g.nodes[i].a].op == FG_EW_CONST || g.nodes[g.nodes[i].b].op == FG_EW_CONST)
            return fail(e, FG_ERR_UNSUPPORTED_FEATURE, "graph: matmul of a constant");
        GemmStep s{i, g.nodes[i].a, g.nodes[i].b, -1, FG_ACT_NONE, i, nullptr, 1, 0, 0, 0};
        {
            const auto &da = e->n[s.a].dims, &db = e->n[s.b].dims;
            if (da.size() == 2) { s.M = da[0]; s.K = da[1]; s.N = db[1]; }
            else if (db.size() == 3) { s.batch = da[0]; s.M = da[1]; s.K = da[2]; s.N = db[2]; }
            else {
                if ((uint64_t)da[0] * da[1] > 0xffffffffull) return fail(e, FG_ERR_INVALID_ARGUMENT, "graph: matmul has too many rows");
                s.M = da[0] * da[1]; s.K = da[2]; s.N = db[1];
            }
        }
        int c = sole_consumer(e, s.out);
        if (c >= 0 && e->n[c].bias_bcast && g.nodes[c].a == s.out) {
            s.bias = g.nodes[c].b;
            e->n[s.out].absorbed = true;
            s.out = c;
            c = sole_consumer(e, s.out);
        }
        if (c >= 0 && act_of(g.nodes[c].op) >= 0) {
            s.act = act_of(g.nodes[c].op);
            e->n[s.out].absorbed = true;
            s.out = c;
        }
        gemm_of_out[s.out] = (int)e->gemms.size();
        e->n[s.out].produced_by_gemm = (int)e->gemms.size();
        e->gemms.push_back(s);
    }
    e->paired = e->dtype == FG_DTYPE_F32 && e->gemm_mode == FG_GEMM_AUTO;
    for (int i = 0; i < N; ++i)
        if (e->n[i].bias_bcast && !(i > 0 && e->n[g.nodes[i].a].absorbed))
            return fail(e, FG_ERR_UNSUPPORTED_FEATURE, "graph: a broadcast bias is only supported directly after a matmul");

    // ---- materialisation ----
    for (int i = 0; i < N; ++i) {
        const GNode& gn = g.nodes[i];
        ENode& en = e->n[i];
        if (gn.op == FG_EW_INPUT || gn.op == FG_EW_CONST || en.absorbed) continue;
        if (gemm_of_out[i] >= 0 || gn.op == OP_SOFTMAX || i == e->last || en.consumers != 1) { en.materialized = true; continue; }
        const int c = sole_consumer(e, i);
        const int cop = g.nodes[c].op;
        if (cop == OP_MATMUL || cop == OP_SOFTMAX) en.materialized = true;
    }
    // ---- buffers (alloc_tensors) ----
    int32_t s;
    for (int i = 0; i < N; ++i) {
        ENode& en = e->n[i];
        const bool is_input = g.nodes[i].op == FG_EW_INPUT;
        if (en.materialized) {
            if ((s = alloc_buf(e, en.numel, false, &en.value)) != FG_OK) return s;
            en.own_value = true;
            if (i != e->last) e->saved.push_back(i);
        }
        if ((is_input || en.materialized) && i != e->last) {
            // inputs: a view into the gradient arena, made below once the order of the backward pass is known
            if (!is_input && (s = alloc_buf(e, en.numel, true, &en.grad)) != FG_OK) return s;   // zeroed like the reference
            e->grads.push_back(i);
        }
    }
    const uint64_t on = e->n[e->last].numel;
    if ((s = alloc_buf(e, on, true, &e->seed)) != FG_OK) return s;
    if ((s = alloc_buf(e, on, true, &e->loss_t)) != FG_OK) return s;
    if ((s = fg_alloc_zeroed(e->ctx, 256, &e->loss_sum)) != FG_OK) return s;
    uint64_t biggest = 1;
    for (int i = 0; i < N; ++i) biggest = std::max(biggest, e->n[i].numel);
    if ((s = alloc_buf(e, biggest, false, &e->tmp)) != FG_OK) return s;
    if (e->dtype != FG_DTYPE_F32)
        for (fg_buf*& st : e->stage)
            if ((s = fg_alloc(e->ctx, biggest * 4, &st)) != FG_OK) return s;
    for (GemmStep& gs : e->gemms)
        if (gs.act == FG_ACT_GELU && (s = alloc_buf(e, e->n[gs.out].numel, false, &gs.preact)) != FG_OK) return s;
    if (g.optim == FG_OPTIM_ADAMW && (s = fg_alloc_zeroed(e->ctx, 256, &e->step_counter)) != FG_OK) return s;
    // ---- forward step list ----
    for (int i = 0; i < N; ++i) {
        const GNode& gn = g.nodes[i];
        if (!e->n[i].materialized) continue;
        if (gemm_of_out[i] >= 0) { e->fwd.push_back(Step{0, gemm_of_out[i]}); continue; }
        if (gn.op == OP_SOFTMAX) { e->fwd.push_back(Step{2, i}); continue; }
        ChainStep c;
        c.root = i;
        int32_t st = FG_OK;
        emit(e, c, i, i, &st);
        if (st != FG_OK) return fail(e, st, "graph: an elementwise region exceeds the chain limits (24 instructions, 8 inputs)");
        for (int in : c.inputs)
            if (e->n[in].numel != e->n[i].numel) return fail(e, FG_ERR_INVALID_ARGUMENT, "graph: elementwise operands must have identical shapes");
        e->fwd.push_back(Step{1, (int)e->chains.size()});
        e->chains.push_back(c);
    }
    // operands of matmul / softmax must have buffers
    for (const GemmStep& gs : e->gemms)
        if (!(e->n[gs.a].materialized || g.nodes[gs.a].op == FG_EW_INPUT) || !(e->n[gs.b].materialized || g.nodes[gs.b].op == FG_EW_INPUT))
            return fail(e, FG_ERR_INTERNAL, "graph: matmul operand without a buffer");

    // ---- gradient arena: the inputs' gradients in the order in which the backward pass completes them ----
    const int nin = (int)e->inputs.size();
    e->ready_key.assign(nin, INT_MAX);
    auto completes = [&](int node, int key) {
        const int slot = e->n[node].input_slot;
        if (slot < 0) return;
        if (e->ready_key[slot] == INT_MAX || key > e->ready_key[slot]) e->ready_key[slot] = key;
    };
    {
        int bstep = 0;   // index of the step in the backward pass
        for (int k = (int)e->fwd.size() - 1; k >= 0; --k, ++bstep) {
            const Step& st = e->fwd[k];
            if (st.kind == 0) {
                const GemmStep& gs = e->gemms[st.idx];
                completes(gs.b, 2 * bstep);                       // weight gradient: before the exchange point
                if (gs.bias >= 0) completes(gs.bias, 2 * bstep);
                completes(gs.a, 2 * bstep + 1);
            } else if (st.kind == 1) {
                for (int in : e->chains[st.idx].inputs) completes(in, 2 * bstep + 1);
            } else {
                completes(g.nodes[st.idx].a, 2 * bstep + 1);
            }
        }
    }
    e->arena_order.resize(nin);
    for (int k = 0; k < nin; ++k) e->arena_order[k] = k;
    std::stable_sort(e->arena_order.begin(), e->arena_order.end(),
                     [&](int x, int y) { return e->ready_key[x] < e->ready_key[y]; });
    e->arena_off.assign(nin, 0);
    uint64_t off = 0;
    for (int slot : e->arena_order) {
        e->arena_off[slot] = off;
        off += (e->n[e->inputs[slot]].numel + 63) / 64 * 64;       // every tensor 256-byte aligned (f32)
    }
    e->arena_elems = off;
    if ((s = alloc_buf(e, off ? off : 1, true, &e->grad_arena)) != FG_OK) return s;
    const bool adam = g.optim == FG_OPTIM_ADAMW;
    if (adam) {
        if ((s = alloc_buf(e, off ? off : 1, true, &e->m_arena)) != FG_OK) return s;
        if ((s = alloc_buf(e, off ? off : 1, true, &e->v_arena)) != FG_OK) return s;
    }
    auto view = [&](fg_buf* arena, int slot) -> fg_buf* {
        fg_buf* b = new (std::nothrow) fg_buf();
        if (!b) return nullptr;
        b->ptr = (char*)arena->ptr + e->arena_off[slot] * e->esize;
        b->bytes = e->n[e->inputs[slot]].numel * e->esize;
        b->version = 0;
        b->view = true;
        return b;
    };
    for (int slot = 0; slot < nin; ++slot) {
        ENode& en = e->n[e->inputs[slot]];
        if (!(en.grad = view(e->grad_arena, slot))) return fail(e, FG_ERR_OUT_OF_MEMORY, "graph: gradient views");
        if (adam) {
            fg_buf *m = view(e->m_arena, slot), *v = view(e->v_arena, slot);
            if (!m || !v) return fail(e, FG_ERR_OUT_OF_MEMORY, "graph: moment views");
            e->m.push_back(m);
            e->v.push_back(v);
        }
    }
    e->pairs_version.assign(nin, 0);
    e->pairs_fresh.assign(nin, 0);

    // ---- bf16 pairs of everything a matmul reads, and of the dZ a fused backward epilogue hands down ----
    if (e->paired) {
        auto want_pairs = [&](int node) -> int32_t {
            ENode& en = e->n[node];
            return en.pairs ? FG_OK : fg_alloc(e->ctx, pstride(e, node) * 4, &en.pairs);
        };
        for (GemmStep& gs : e->gemms) {
            if (gs.batch != 1) continue;
            if ((s = want_pairs(gs.a)) != FG_OK || (s = want_pairs(gs.b)) != FG_OK) return s;
        }
        for (GemmStep& gs : e->gemms) {
            if (gs.batch != 1) continue;
            const int h = e->n[gs.a].produced_by_gemm;
            if (h >= 0 && e->n[gs.a].consumers == 1 && e->gemms[h].batch == 1 && !e->gemms[h].dz_pairs &&
                (s = fg_alloc(e->ctx, pstride(e, gs.a) * 4, &e->gemms[h].dz_pairs)) != FG_OK)
                return s;
        }
    }
    return FG_OK;
}

// Adds `src` into grad[node] (used when a gradient gets a second contribution from a GEMM).
int32_t accumulate_into(fg_exec* e, int node, const float* src) {
    fg_ew_instr prog[3] = {{FG_EW_INPUT, 0, 0, 0.f}, {FG_EW_INPUT, 1, 0, 0.f}, {FG_EW_ADD, 0, 1, 0.f}};
    const float* in[2] = {gptr(e, node), src};
    return fg_eltwise_chain_fwd_dt(e->ctx, e->dtype, e->n[node].numel, prog, 3, (const void* const*)in, 2, gptr(e, node),
                                   nullptr);
}

void drop_plans(fg_exec* e) {
    for (int k = 0; k < 4; ++k) {
        if (e->plan[k]) fg_plan_destroy(e->plan[k]);
        e->plan[k] = nullptr;
        e->calls[k] = 0;
    }
}

}  // namespace

extern "C" {

int32_t fg_graph_create(int32_t loss, int32_t optim, fg_graph** out) {
    if (!out || loss < FG_LOSS_MSE || loss > FG_LOSS_BINARY_CROSS_ENTROPY || optim < FG_OPTIM_SGD || optim > FG_OPTIM_ADAMW)
        return FG_ERR_INVALID_ARGUMENT;
    fg_graph* g = new (std::nothrow) fg_graph();
    if (!g) return FG_ERR_OUT_OF_MEMORY;
    g->loss = loss;
    g->optim = optim;
    *out = g;
    return FG_OK;
}

int32_t fg_graph_destroy(fg_graph* g) { delete g; return FG_OK; }

int32_t fg_graph_node_count(const fg_graph* g) { return g ? (int32_t)g->nodes.size() : -1; }

int32_t fg_graph_input_dt(fg_graph* g, const uint32_t* shape_fields, uint32_t ndim, int32_t dtype, int32_t* node) {
    if (!g || !shape_fields || !node || ndim < 1 || ndim > 4) return FG_ERR_INVALID_ARGUMENT;
    if (dtype < FG_DTYPE_F32 || dtype > FG_DTYPE_BF16) return FG_ERR_INVALID_ARGUMENT;
    GNode n{FG_EW_INPUT, -1, -1, 0.f, std::vector<uint32_t>(shape_fields, shape_fields + ndim), dtype};
    g->nodes.push_back(n);
    *node = (int32_t)g->nodes.size() - 1;
    return FG_OK;
}

int32_t fg_graph_input(fg_graph* g, const uint32_t* shape_fields, uint32_t ndim, int32_t* node) {
    return fg_graph_input_dt(g, shape_fields, ndim, FG_DTYPE_F32, node);
}

int32_t fg_graph_constant_f32(fg_graph* g, float value, int32_t* node) {
    if (!g || !node) return FG_ERR_INVALID_ARGUMENT;
    g->nodes.push_back(GNode{FG_EW_CONST, -1, -1, value, {}, FG_DTYPE_F32});
    *node = (int32_t)g->nodes.size() - 1;
    return FG_OK;
}

int32_t fg_graph_op(fg_graph* g, int32_t op, int32_t a, int32_t b, int32_t* node) {
    if (!g || !node) return FG_ERR_INVALID_ARGUMENT;
    const int n = (int)g->nodes.size();
    const bool two = is_binary(op) || op == OP_MATMUL;
    if (!(is_ew(op) || op == OP_MATMUL || op == OP_SOFTMAX)) return FG_ERR_INVALID_ARGUMENT;
    if (a < 0 || a >= n || (two && (b < 0 || b >= n))) return FG_ERR_INVALID_ARGUMENT;   // UnresolvedInput
    g->nodes.push_back(GNode{op, a, two ? b : -1, 0.f, {}});
    *node = n;
    return FG_OK;
}

int32_t fg_exec_create(fg_ctx* ctx, const fg_graph* graph, const uint32_t* meta, uint32_t nmeta, int32_t gemm_mode,
                       fg_exec** out) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, graph && meta && out && nmeta >= 1, "fg_exec_create: NULL argument");
    FG_REQUIRE(ctx, !graph->nodes.empty(), "fg_exec_create: the graph is empty");   // ErrorKind::GraphEmpty
    FG_REQUIRE(ctx, gemm_mode >= FG_GEMM_AUTO && gemm_mode <= FG_GEMM_TF32_BF16X2, "fg_exec_create: unknown GEMM mode");
    fg_exec* e = new (std::nothrow) fg_exec();
    if (!e) return fg_fail(ctx, FG_ERR_OUT_OF_MEMORY, "fg_exec_create");
    e->ctx = ctx;
    e->g = *graph;
    e->meta.assign(meta, meta + nmeta);
    e->gemm_mode = gemm_mode;
    int32_t s = lower(e);
    if (s != FG_OK) { fg_exec_destroy(e); return s; }
    *out = e;
    return FG_OK;
}

int32_t fg_exec_destroy(fg_exec* e) {
    if (!e) return FG_OK;
    for (ENode& en : e->n) {
        if (en.own_value && en.value) fg_free(e->ctx, en.value);
        if (en.grad) fg_free(e->ctx, en.grad);
    }
    for (ENode& en : e->n) if (en.pairs) fg_free(e->ctx, en.pairs);
    for (GemmStep& gs : e->gemms) {
        if (gs.preact) fg_free(e->ctx, gs.preact);
        if (gs.dz_pairs) fg_free(e->ctx, gs.dz_pairs);
    }
    for (fg_buf* b : e->m) fg_free(e->ctx, b);       // views
    for (fg_buf* b : e->v) fg_free(e->ctx, b);
    for (fg_buf* b : {e->seed, e->loss_t, e->tmp, e->loss_sum, e->step_counter, e->grad_arena, e->m_arena, e->v_arena})
        if (b) fg_free(e->ctx, b);
    for (fg_buf* b : e->stage) if (b) fg_free(e->ctx, b);
    drop_plans(e);
    delete e;
    return FG_OK;
}

int32_t fg_exec_set_adamw(fg_exec* e, const fg_adamw_hyper* h) {
    if (!e || !h) return FG_ERR_INVALID_ARGUMENT;
    e->hyper = *h;
    return FG_OK;
}

// schedule(): binds the user's tensors to the graph's inputs, in input order.
int32_t fg_exec_bind(fg_exec* e, fg_buf* const* in_tensors, uint32_t count, const uint8_t* trainable) {
    if (!e) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(e->ctx, in_tensors && count == e->inputs.size(), "fg_exec_bind: one tensor per graph input is required");
    for (uint32_t k = 0; k < count; ++k) {
        FG_REQUIRE(e->ctx, in_tensors[k] != nullptr, "fg_exec_bind: NULL tensor");
        FG_REQUIRE(e->ctx, in_tensors[k]->bytes >= e->n[e->inputs[k]].numel * e->esize, "fg_exec_bind: tensor smaller than the input's shape");
        e->n[e->inputs[k]].value = in_tensors[k];
    }
    e->trainable.assign(count, 1);
    if (trainable) e->trainable.assign(trainable, trainable + count);
    e->bound = true;
    std::fill(e->pairs_fresh.begin(), e->pairs_fresh.end(), 0);
    drop_plans(e);        // recorded against the previous tensors
    return FG_OK;
}

// Brings the pairs of the bound input tensors up to date.  A trainable tensor changes only through the optimizer
// (which writes its pairs in the same pass) or through an entry point that bumps the buffer's version; a tensor that is
// only read (the data batch) may be rewritten through its raw pointer at any time, so its pairs are made every pass.
static int32_t refresh_input_pairs(fg_exec* e) {
    for (size_t k = 0; k < e->inputs.size(); ++k) {
        ENode& en = e->n[e->inputs[k]];
        if (!en.pairs) continue;
        if (e->trainable[k] && e->pairs_fresh[k] && e->pairs_version[k] == en.value->version) continue;
        const int32_t s = fg_pairs_from_f32(e->ctx, (const float*)en.value->ptr, en.numel, en.pairs->ptr, pstride(e, e->inputs[k]));
        if (s != FG_OK) return s;
        e->pairs_fresh[k] = 1;
        e->pairs_version[k] = en.value->version;
    }
    return FG_OK;
}

static void* pairs_of(fg_exec* e, int node) { return e->n[node].pairs ? e->n[node].pairs->ptr : nullptr; }

static int32_t forward_eager(fg_exec* e) {
    int32_t s;
    if (e->paired && (s = refresh_input_pairs(e)) != FG_OK) return s;
    for (const Step& st : e->fwd) {
        if (st.kind == 0) {
            const GemmStep& gs = e->gemms[st.idx];
            const size_t sa = (size_t)gs.M * gs.K, sb = (size_t)gs.K * gs.N, sc = (size_t)gs.M * gs.N;
            s = FG_OK;
            if (e->paired && gs.batch == 1) {
                // the tensors themselves are the operands; the epilogue writes the result's pairs for the matmul that reads it
                s = fg_gemm_paired_f32(e->ctx, gs.M, gs.N, gs.K, vptr(e, gs.a), pairs_of(e, gs.a), pstride(e, gs.a), vptr(e, gs.b),
                                       pairs_of(e, gs.b), pstride(e, gs.b), vptr(e, gs.out), gs.bias >= 0 ? vptr(e, gs.bias) : nullptr,
                                       gs.act, gs.preact ? (float*)gs.preact->ptr : nullptr, pairs_of(e, gs.out), pstride(e, gs.out));
                if (s != FG_OK) return s;
                continue;
            }
            if (e->dtype == FG_DTYPE_F32 && gs.batch > 1) {
                // rank-3 product: one launch for small matrices, one pairs pass + one launch per matrix for large ones
                s = fg_gemm_batched_f32(e->ctx, e->gemm_mode, gs.batch, gs.M, gs.N, gs.K, vptr(e, gs.a), sa, vptr(e, gs.b), sb,
                                        vptr(e, gs.out), sc, gs.bias >= 0 ? vptr(e, gs.bias) : nullptr, gs.act,
                                        gs.preact ? (float*)gs.preact->ptr : nullptr);
                if (s != FG_OK) return s;
                continue;
            }
            for (uint32_t t = 0; t < gs.batch && s == FG_OK; ++t) {
                if (e->dtype != FG_DTYPE_F32) {
                    char* const pa = (char*)vptr(e, gs.a) + t * sa * 2;
                    char* const pb = (char*)vptr(e, gs.b) + t * sb * 2;
                    s = fg_gemm_lowp(e->ctx, e->dtype, gs.M, gs.N, gs.K, pa, pb, (char*)vptr(e, gs.out) + t * sc * 2,
                                     gs.bias >= 0 ? vptr(e, gs.bias) : nullptr, gs.act,
                                     gs.preact ? (char*)gs.preact->ptr + t * sc * 2 : nullptr);
                    continue;
                }
                s = fg_gemm_f32(e->ctx, e->gemm_mode, 0, 0, gs.M, gs.N, gs.K, vptr(e, gs.a) + t * sa, vptr(e, gs.b) + t * sb,
                                vptr(e, gs.out) + t * sc, gs.bias >= 0 ? vptr(e, gs.bias) : nullptr, gs.act,
                                gs.preact ? (float*)gs.preact->ptr + t * sc : nullptr);
            }
        } else if (st.kind == 1) {
            const ChainStep& c = e->chains[st.idx];
            const float* in[FG_EW_MAX_INPUTS];
            for (size_t k = 0; k < c.inputs.size(); ++k) in[k] = vptr(e, c.inputs[k]);
            s = fg_eltwise_chain_fwd_dt(e->ctx, e->dtype, e->n[c.root].numel, c.prog.data(), (int)c.prog.size(),
                                        (const void* const*)in, (int)c.inputs.size(), vptr(e, c.root), nullptr);
        } else {
            const auto& d = e->n[st.idx].dims;
            const uint32_t cols = d.back();
            const uint64_t numel = e->n[st.idx].numel;
            if (e->dtype != FG_DTYPE_F32) {
                float *x32 = (float*)e->stage[0]->ptr, *y32 = (float*)e->stage[1]->ptr;
                if ((s = fg_convert(e->ctx, vptr(e, e->g.nodes[st.idx].a), e->dtype, x32, FG_DTYPE_F32, numel)) != FG_OK) return s;
                if ((s = fg_softmax_fwd(e->ctx, (uint32_t)(numel / cols), cols, x32, y32)) != FG_OK) return s;
                s = fg_convert(e->ctx, y32, FG_DTYPE_F32, vptr(e, st.idx), e->dtype, numel);
            } else
            s = fg_softmax_fwd(e->ctx, (uint32_t)(numel / cols), cols, vptr(e, e->g.nodes[st.idx].a), vptr(e, st.idx));
        }
        if (s != FG_OK) return s;
        if (e->paired && st.kind != 0) {
            const int node = st.kind == 1 ? e->chains[st.idx].root : st.idx;
            if (e->n[node].pairs &&
                (s = fg_pairs_from_f32(e->ctx, vptr(e, node), e->n[node].numel, e->n[node].pairs->ptr, pstride(e, node))) != FG_OK)
                return s;
        }
    }
    return FG_OK;
}

static int32_t loss_eager(fg_exec* e, const fg_buf* target) {
    const ENode& o = e->n[e->last];
    if (e->dtype != FG_DTYPE_F32) {
        // widen the prediction (and a dense target) to f32, run the f32 loss kernel, round loss and seed back
        float *p32 = (float*)e->stage[0]->ptr, *t32 = (float*)e->stage[1]->ptr, *l32 = (float*)e->stage[2]->ptr,
              *g32 = (float*)e->stage[3]->ptr;
        int32_t s;
        if ((s = fg_convert(e->ctx, vptr(e, e->last), e->dtype, p32, FG_DTYPE_F32, o.numel)) != FG_OK) return s;
        if (e->g.loss == FG_LOSS_CROSS_ENTROPY) {
            const uint32_t cols = o.dims.back(), rows = (uint32_t)(o.numel / cols);
            FG_REQUIRE(e->ctx, target->bytes >= (uint64_t)rows * 4, "dispatch_loss: one u32 label per row is required");
            s = fg_ce_loss_grad(e->ctx, p32, (const uint32_t*)target->ptr, rows, cols, l32, g32);
        } else {
            FG_REQUIRE(e->ctx, target->bytes >= o.numel * e->esize, "dispatch_loss: target smaller than the output");
            if ((s = fg_convert(e->ctx, target->ptr, e->dtype, t32, FG_DTYPE_F32, o.numel)) != FG_OK) return s;
            s = e->g.loss == FG_LOSS_MSE ? fg_mse_loss_grad(e->ctx, p32, t32, o.numel, 1.0f, l32, nullptr, g32)
                                         : fg_bce_loss_grad(e->ctx, p32, t32, o.numel, 1.0f, l32, nullptr, g32);
        }
        if (s != FG_OK) return s;
        if ((s = fg_convert(e->ctx, l32, FG_DTYPE_F32, e->loss_t->ptr, e->dtype, o.numel)) != FG_OK) return s;
        return fg_convert(e->ctx, g32, FG_DTYPE_F32, e->seed->ptr, e->dtype, o.numel);
    }
    float* const lsum = (float*)e->loss_sum->ptr;
    if (e->g.loss == FG_LOSS_MSE) {
        FG_REQUIRE(e->ctx, target->bytes >= o.numel * 4, "dispatch_loss: target smaller than the output");
        return fg_mse_loss_grad(e->ctx, vptr(e, e->last), (const float*)target->ptr, o.numel, 1.0f, (float*)e->loss_t->ptr,
                                lsum, (float*)e->seed->ptr);
    }
    if (e->g.loss == FG_LOSS_BINARY_CROSS_ENTROPY) {
        FG_REQUIRE(e->ctx, target->bytes >= o.numel * 4, "dispatch_loss: target smaller than the output");
        return fg_bce_loss_grad(e->ctx, vptr(e, e->last), (const float*)target->ptr, o.numel, 1.0f, (float*)e->loss_t->ptr,
                                lsum, (float*)e->seed->ptr);
    }
    const uint32_t cols = o.dims.back();
    const uint32_t rows = (uint32_t)(o.numel / cols);
    FG_REQUIRE(e->ctx, target->bytes >= (uint64_t)rows * 4, "dispatch_loss: one u32 label per row is required");
    const int32_t s = fg_ce_loss_grad(e->ctx, vptr(e, e->last), (const uint32_t*)target->ptr, rows, cols, (float*)e->loss_t->ptr,
                                      (float*)e->seed->ptr);
    return s != FG_OK ? s : fg_sum_f32(e->ctx, (const float*)e->loss_t->ptr, o.numel, lsum);
}

// The backward of one matmul in the graph's storage type.
static int32_t gemm_bwd_any(fg_exec* e, uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, const void* dY, int act,
                            const void* saved, void* dA, void* dB, void* dbias) {
    if (e->dtype == FG_DTYPE_F32)
        return fg_gemm_bwd_f32(e->ctx, e->gemm_mode, M, N, K, (const float*)A, (const float*)B, (const float*)dY, act,
                               (const float*)saved, (float*)dA, (float*)dB, (float*)dbias, nullptr);
    return fg_gemm_bwd_lowp(e->ctx, e->dtype, M, N, K, A, B, dY, act, saved, dA, dB, dbias);
}

// Data-parallel helpers.  Only trainable tensors are exchanged; the arena is ordered by completion, so the
// tensors whose gradients are complete form a prefix.
static bool dp_active(const fg_exec* e) { return e->ctx->comm != nullptr && e->ctx->nranks > 1; }

// End (arena elements) of the trainable tensors whose gradient is complete once the backward step with this key is.
static uint64_t ready_end(const fg_exec* e, int key) {
    uint64_t end = 0;
    for (size_t k = 0; k < e->inputs.size(); ++k)
        if (e->trainable[k] && e->ready_key[k] <= key) end = std::max(end, e->arena_off[k] + e->n[e->inputs[k]].numel);
    return end;
}

static int32_t backward_eager(fg_exec* e) {
    const int N = (int)e->n.size();
    std::vector<uint8_t> written(N, 0);
    for (GemmStep& gs : e->gemms) gs.dz_ready = gs.dbias_done = false;
    e->exchanged_end = 0;
    // an input's gradient is wanted when the input is trainable (every input is, unless fg_exec_bind said otherwise)
    auto wanted = [&](int node) -> bool {
        const int slot = e->n[node].input_slot;
        return slot < 0 || e->trainable[slot] != 0;
    };
    int bstep = -1;
    auto grad_of = [&](int node) -> float* { return node == e->last ? (float*)e->seed->ptr : gptr(e, node); };
    // a tensor's t-th matrix: offsets are in elements of the graph's storage type
    auto off = [&](const void* p, size_t elems) -> float* { return (float*)((char*)p + elems * e->esize); };
    int32_t s;
    for (int k = (int)e->fwd.size() - 1; k >= 0; --k) {
        const Step& st = e->fwd[k];
        ++bstep;
        if (st.kind == 0) {
            GemmStep& gs = e->gemms[st.idx];
            if (gs.out != e->last && !written[gs.out]) continue;   // does not reach the output
            const uint32_t M = gs.M, K = gs.K, Nn = gs.N;
            const size_t sa = (size_t)M * K, sb = (size_t)K * Nn, sc = (size_t)M * Nn;
            // The range of the arena whose gradients are complete once this step's weight (and bias) gradient is:
            // exchanged beside this step's dA product when it is large enough.
            float* exch_buf = nullptr;
            uint64_t exch_count = 0;
            if (dp_active(e)) {
                const uint64_t end0 = ready_end(e, 2 * bstep);
                // a smaller range waits for the next one (launch cost; the GEMMs give up SMs while an exchange runs)
                if (end0 > e->exchanged_end && end0 - e->exchanged_end >= e->ctx->opt_min_exchange) {
                    exch_buf = (float*)e->grad_arena->ptr + e->exchanged_end;
                    exch_count = end0 - e->exchanged_end;
                }
            }
            if (e->paired && gs.batch == 1 && !written[gs.a] && !written[gs.b] && gs.a != gs.b &&
                (gs.act == FG_ACT_NONE || gs.dz_ready) && (gs.bias < 0 || !written[gs.bias] || gs.dbias_done)) {
                // grad(out) is dL/d(pre-activation) already.  When the first operand is the fused result of another
                // matmul that nothing else reads, this call's dA epilogue applies that layer's activation derivative,
                // writes the pairs of the result and sums its columns into that layer's bias gradient.
                const int h = e->n[gs.a].produced_by_gemm;
                GemmStep* below = (h >= 0 && e->n[gs.a].consumers == 1 && e->gemms[h].batch == 1) ? &e->gemms[h] : nullptr;
                const bool want_da = wanted(gs.a), want_db = wanted(gs.b);
                int below_act = FG_ACT_NONE;
                const float* below_saved = nullptr;
                float* below_dbias = nullptr;
                void* da_pairs = nullptr;
                if (below && want_da) {
                    below_act = below->act;
                    if (below_act != FG_ACT_NONE) below_saved = below_act == FG_ACT_GELU ? (const float*)below->preact->ptr : vptr(e, below->out);
                    da_pairs = below->dz_pairs ? below->dz_pairs->ptr : nullptr;
                    if (below->bias >= 0 && !written[below->bias] && wanted(below->bias)) below_dbias = gptr(e, below->bias);
                }
                float* dbias = (gs.bias >= 0 && !gs.dbias_done && wanted(gs.bias)) ? gptr(e, gs.bias) : nullptr;
                s = fg_gemm_bwd_paired_f32(e->ctx, M, Nn, K, vptr(e, gs.a), pairs_of(e, gs.a), pstride(e, gs.a), vptr(e, gs.b),
                                           pairs_of(e, gs.b), pstride(e, gs.b), grad_of(gs.out),
                                           gs.dz_ready && gs.dz_pairs ? gs.dz_pairs->ptr : nullptr, pstride(e, gs.out),
                                           want_db ? gptr(e, gs.b) : nullptr, dbias, want_da ? gptr(e, gs.a) : nullptr, below_act,
                                           below_saved, da_pairs, pstride(e, gs.a), below_dbias, exch_buf, exch_count);
                if (s != FG_OK) return s;
                if (exch_buf) e->exchanged_end += exch_count;
                written[gs.a] = written[gs.b] = 1;
                if (gs.bias >= 0) written[gs.bias] = 1;
                if (below && want_da) {
                    below->dz_ready = true;
                    if (below_dbias) { below->dbias_done = true; written[below->bias] = 1; }
                }
                continue;
            }
            // every other route computes this step's gradients first and exchanges afterwards
            struct ExchangeAfter {
                fg_exec* e; float* buf; uint64_t count;
                ~ExchangeAfter() {
                    if (buf && fg_allreduce_sum_f32(e->ctx, buf, count) == FG_OK) e->exchanged_end += count;
                }
            } exchange_after{e, exch_buf, exch_count};
            if (gs.act != FG_ACT_NONE && gs.dz_ready) return fail(e, FG_ERR_INTERNAL, "graph: fused gradient reached an unfused matmul backward");
            // destinations: the gradient buffer itself for a first contribution, the scratch tensor otherwise
            float* dA = written[gs.a] ? (float*)e->tmp->ptr : gptr(e, gs.a);
            const float* saved = gs.act == FG_ACT_NONE ? nullptr : gs.act == FG_ACT_GELU ? (float*)gs.preact->ptr : vptr(e, gs.out);
            if (gs.batch > 1) {
                // one product per Z index: every operand, gradient and saved tensor is stepped by one matrix
                auto run = [&](float* da_dst, float* db_dst) -> int32_t {
                    if (e->dtype == FG_DTYPE_F32)
                        return fg_gemm_batched_bwd_f32(e->ctx, e->gemm_mode, gs.batch, M, Nn, K, vptr(e, gs.a), sa, vptr(e, gs.b), sb,
                                                       grad_of(gs.out), sc, gs.act, saved, da_dst, db_dst);
                    for (uint32_t t = 0; t < gs.batch; ++t) {
                        int32_t r = gemm_bwd_any(e, M, Nn, K, off(vptr(e, gs.a), t * sa), off(vptr(e, gs.b), t * sb),
                                                 off(grad_of(gs.out), t * sc), gs.act, saved ? off(saved, t * sc) : nullptr,
                                                 da_dst ? off(da_dst, t * sa) : nullptr, db_dst ? off(db_dst, t * sb) : nullptr,
                                                 nullptr);
                        if (r != FG_OK) return r;
                    }
                    return FG_OK;
                };
                if (!written[gs.a] && !written[gs.b] && gs.a != gs.b) {
                    if ((s = run(gptr(e, gs.a), gptr(e, gs.b))) != FG_OK) return s;
                    written[gs.a] = written[gs.b] = 1;
                    continue;
                }
                if ((s = run(dA, nullptr)) != FG_OK) return s;
                if (written[gs.a] && (s = accumulate_into(e, gs.a, dA)) != FG_OK) return s;
                written[gs.a] = 1;
                float* dBt = written[gs.b] ? (float*)e->tmp->ptr : gptr(e, gs.b);
                if ((s = run(nullptr, dBt)) != FG_OK) return s;
                if (written[gs.b] && (s = accumulate_into(e, gs.b, dBt)) != FG_OK) return s;
                written[gs.b] = 1;
                continue;
            }
            float* dbias = nullptr;
            if (gs.bias >= 0) dbias = written[gs.bias] ? nullptr : gptr(e, gs.bias);
            if (gs.bias >= 0 && written[gs.bias]) return fail(e, FG_ERR_UNSUPPORTED_FEATURE, "graph: a bias used by two layers");
            if (!written[gs.a] && !written[gs.b] && gs.a != gs.b) {
                // the common case: one call computes dZ once and both products from it
                s = gemm_bwd_any(e, M, Nn, K, vptr(e, gs.a), vptr(e, gs.b), grad_of(gs.out), gs.act, saved, gptr(e, gs.a),
                                 gptr(e, gs.b), dbias);
                if (s != FG_OK) return s;
                written[gs.a] = written[gs.b] = 1;
                if (gs.bias >= 0) written[gs.bias] = 1;
                continue;
            }
            // dA first (it may need the scratch tensor), then dB
            s = gemm_bwd_any(e, M, Nn, K, vptr(e, gs.a), vptr(e, gs.b), grad_of(gs.out), gs.act, saved, dA, nullptr, dbias);
            if (s != FG_OK) return s;
            if (written[gs.a] && (s = accumulate_into(e, gs.a, dA)) != FG_OK) return s;
            written[gs.a] = 1;
            if (gs.bias >= 0) written[gs.bias] = 1;
            float* dB = written[gs.b] ? (float*)e->tmp->ptr : gptr(e, gs.b);
            s = gemm_bwd_any(e, M, Nn, K, vptr(e, gs.a), vptr(e, gs.b), grad_of(gs.out), gs.act, saved, nullptr, dB, nullptr);
            if (s != FG_OK) return s;
            if (written[gs.b] && (s = accumulate_into(e, gs.b, dB)) != FG_OK) return s;
            written[gs.b] = 1;
        } else if (st.kind == 1) {
            const ChainStep& c = e->chains[st.idx];
            if (c.root != e->last && !written[c.root]) continue;
            const float* in[FG_EW_MAX_INPUTS];
            float* gr[FG_EW_MAX_INPUTS];
            bool any_written = false;
            for (size_t j = 0; j < c.inputs.size(); ++j) any_written |= written[c.inputs[j]] != 0;
            for (size_t j = 0; j < c.inputs.size(); ++j) {
                in[j] = vptr(e, c.inputs[j]);
                gr[j] = gptr(e, c.inputs[j]);
                if (any_written && !written[c.inputs[j]] &&
                    (s = fg_memset_zero(e->ctx, gr[j], e->n[c.inputs[j]].numel * e->esize)) != FG_OK) return s;
            }
            s = fg_eltwise_chain_bwd_dt(e->ctx, e->dtype, e->n[c.root].numel, c.prog.data(), (int)c.prog.size(),
                                        (const void* const*)in, (int)c.inputs.size(), grad_of(c.root), (void* const*)gr,
                                        any_written ? 1 : 0);
            if (s != FG_OK) return s;
            for (int id : c.inputs) written[id] = 1;
        } else {
            const int node = st.idx, src = e->g.nodes[node].a;
            if (node != e->last && !written[node]) continue;
            const auto& d = e->n[node].dims;
            const uint32_t cols = d.back(), rows = (uint32_t)(e->n[node].numel / cols);
            if (node == e->last && e->ce_softmax_tail) {
                // the loss kernel's p - onehot is already dL/dlogits
                if (written[src]) s = accumulate_into(e, src, (const float*)e->seed->ptr);
                else {
                    cudaError_t ce = cudaMemcpyAsync(gptr(e, src), e->seed->ptr, e->n[src].numel * e->esize, cudaMemcpyDeviceToDevice, e->ctx->stream);
                    s = ce == cudaSuccess ? FG_OK : fg_fail_cuda(e->ctx, FG_ERR_FAILED_BUFFER_COPY, "seed copy", ce);
                }
            } else if (e->dtype != FG_DTYPE_F32) {
                const uint64_t numel = e->n[node].numel;
                float *y32 = (float*)e->stage[0]->ptr, *dy32 = (float*)e->stage[1]->ptr, *dx32 = (float*)e->stage[2]->ptr;
                if ((s = fg_convert(e->ctx, vptr(e, node), e->dtype, y32, FG_DTYPE_F32, numel)) != FG_OK) return s;
                if ((s = fg_convert(e->ctx, grad_of(node), e->dtype, dy32, FG_DTYPE_F32, numel)) != FG_OK) return s;
                if ((s = fg_softmax_bwd(e->ctx, rows, cols, y32, dy32, dx32, 0)) != FG_OK) return s;
                if (written[src]) {
                    if ((s = fg_convert(e->ctx, dx32, FG_DTYPE_F32, e->tmp->ptr, e->dtype, numel)) != FG_OK) return s;
                    s = accumulate_into(e, src, (const float*)e->tmp->ptr);
                } else {
                    s = fg_convert(e->ctx, dx32, FG_DTYPE_F32, gptr(e, src), e->dtype, numel);
                }
            } else {
                s = fg_softmax_bwd(e->ctx, rows, cols, vptr(e, node), grad_of(node), gptr(e, src), written[src] ? 1 : 0);
            }
            if (s != FG_OK) return s;
            written[src] = 1;
        }
    }
    // what has been exchanged so far is complete before dispatch_optim reads it; the rest is exchanged there
    e->final_lo = e->exchanged_end;
    if (e->ctx->comm_pending && !e->ctx->capturing) return fg_comm_join(e->ctx);
    return FG_OK;
}

static int32_t optim_one(fg_exec* e, uint32_t slot, fg_buf* weight) {
    const int node = e->inputs[slot];
    float lr;
    memcpy(&lr, &e->meta[0], 4);   // field 0 holds the learning rate's bits (kernel/optim.rs:119-131)
    if (e->dtype != FG_DTYPE_F32) {
        // 16-bit storage: scaled = g*lr; w -= scaled; g = 0 (optim/basic_optim.rs:3-31), each result rounded
        // to the storage type, as a two-input elementwise program written back over w.
        if (e->g.optim != FG_OPTIM_SGD) return fail(e, FG_ERR_UNSUPPORTED_FEATURE, "AdamW needs f32 storage");
        const fg_ew_instr prog[5] = {{FG_EW_INPUT, 0, 0, 0.f}, {FG_EW_INPUT, 1, 0, 0.f}, {FG_EW_CONST, 0, 0, lr},
                                     {FG_EW_MUL, 1, 2, 0.f}, {FG_EW_SUB, 0, 3, 0.f}};
        const void* in[2] = {weight->ptr, gptr(e, node)};
        int32_t s = fg_eltwise_chain_fwd_dt(e->ctx, e->dtype, e->n[node].numel, prog, 5, in, 2, weight->ptr, nullptr);
        if (s != FG_OK) return s;
        return fg_memset_zero(e->ctx, gptr(e, node), e->n[node].numel * e->esize);
    }
    // the updated weights' pairs are written in the same pass when a matmul reads this tensor
    void* wp = (e->n[node].pairs && weight == e->n[node].value) ? e->n[node].pairs->ptr : nullptr;
    int32_t s;
    if (e->g.optim == FG_OPTIM_SGD) {
        s = fg_sgd_step_paired(e->ctx, (float*)weight->ptr, gptr(e, node), e->n[node].numel, lr, 1.0f, 1, wp, pstride(e, node));
    } else {
        fg_adamw_hyper h = e->hyper;
        h.lr = lr;
        s = fg_adamw_step_paired(e->ctx, (float*)weight->ptr, gptr(e, node), (float*)e->m[slot]->ptr, (float*)e->v[slot]->ptr,
                                 e->n[node].numel, &h, 0, (const uint32_t*)e->step_counter->ptr, 1.0f, 1, wp, pstride(e, node));
    }
    if (s == FG_OK && wp) {
        e->pairs_fresh[slot] = 1;
        e->pairs_version[slot] = weight->version;
    }
    return s;
}

// Updates every bound tensor that is marked trainable (the reference updates all of them:
// dispatch/mod.rs:735-748) and zeroes its gradient.
// Updates the given input slots in one launch (f32 graphs), or one by one (16-bit storage).
static int32_t optim_many(fg_exec* e, const std::vector<int>& slots) {
    if (slots.empty()) return FG_OK;
    if (e->dtype != FG_DTYPE_F32) {
        for (int slot : slots) {
            const int32_t s = optim_one(e, (uint32_t)slot, e->n[e->inputs[slot]].value);
            if (s != FG_OK) return s;
        }
        return FG_OK;
    }
    float lr;
    memcpy(&lr, &e->meta[0], 4);
    std::vector<fg_update_tensor> t;
    for (int slot : slots) {
        const int node = e->inputs[slot];
        ENode& en = e->n[node];
        fg_update_tensor u{};
        u.w = (float*)en.value->ptr;
        u.g = gptr(e, node);
        if (e->g.optim == FG_OPTIM_ADAMW) { u.m = (float*)e->m[slot]->ptr; u.v = (float*)e->v[slot]->ptr; }
        u.w_pairs = en.pairs ? en.pairs->ptr : nullptr;      // the updated weights' pairs, same pass
        u.pairs_stride = pstride(e, node);
        u.n = en.numel;
        t.push_back(u);
    }
    int32_t s;
    if (e->g.optim == FG_OPTIM_SGD) s = fg_sgd_step_multi(e->ctx, t.data(), (uint32_t)t.size(), lr, 1.0f, 1);
    else {
        fg_adamw_hyper h = e->hyper;
        h.lr = lr;
        s = fg_adamw_step_multi(e->ctx, t.data(), (uint32_t)t.size(), &h, 0, (const uint32_t*)e->step_counter->ptr, 1.0f, 1);
    }
    if (s != FG_OK) return s;
    for (int slot : slots)
        if (e->n[e->inputs[slot]].pairs) {
            e->pairs_fresh[slot] = 1;
            e->pairs_version[slot] = e->n[e->inputs[slot]].value->version;
        }
    return FG_OK;
}

static int32_t optim_eager(fg_exec* e) {
    int32_t s;
    if (e->g.optim == FG_OPTIM_ADAMW && (s = fg_counter_increment(e->ctx, (uint32_t*)e->step_counter->ptr)) != FG_OK) return s;
    if (dp_active(e)) {
        // Gradients in [0, final_lo) were summed over the ranks during dispatch_backward.  The sum of the rest
        // (the gradients the backward pass finished last) starts now; the tensors of the first range are updated
        // beside it, the others when it has arrived.
        const uint64_t lo = e->optim_lo, hi = ready_end(e, INT_MAX - 1);
        if (hi > lo && (s = fg_allreduce_sum_f32(e->ctx, (float*)e->grad_arena->ptr + lo, hi - lo)) != FG_OK) return s;
        std::vector<int> early, late;
        for (int slot : e->arena_order)
            if (e->trainable[slot]) (e->arena_off[slot] + e->n[e->inputs[slot]].numel <= lo ? early : late).push_back(slot);
        if ((s = optim_many(e, early)) != FG_OK) return s;
        if ((s = fg_comm_join(e->ctx)) != FG_OK) return s;
        return optim_many(e, late);
    }
    std::vector<int> all;
    for (int slot : e->arena_order)
        if (e->trainable[slot]) all.push_back(slot);
    return optim_many(e, all);
}

// Are this graph's dispatches recorded and replayed?  With option exec_plans = auto: when the graph is launch-bound,
// i.e. its estimated device time per launch is under ten microseconds, or under 300 with a communicator (one
// forward + backward pass estimated at
// 300 TFLOP/s for the matmuls and 5 TB/s for every tensor touched three times, over about three launches per step of
// the forward pass).
static bool plans_wanted(const fg_exec* e) {
    if (!e->use_plans || e->ctx->opt_exec_plans == 0) return false;
    if (e->ctx->opt_exec_plans == 1) return true;
    double flop = 0.0, bytes = 0.0;
    for (const GemmStep& gs : e->gemms) flop += 3.0 * 2.0 * gs.batch * (double)gs.M * gs.N * gs.K;
    for (const ENode& en : e->n) bytes += 3.0 * (double)en.numel * (double)e->esize;
    const double est_us = flop / 300e6 + bytes / 5e6;
    const double launches = 3.0 * (double)std::max<size_t>(e->fwd.size(), 1);
    // With a communicator every step also enqueues collectives, whose host-side cost a replayed graph avoids:
    // worth it up to a few hundred microseconds per launch (two GPUs, 784-4096-4096-10, about 125 us per launch:
    // 1.97 ms per step replayed against 2.03 with plain launches; eight 8192-wide layers, about 800 us per
    // launch: 27.0 against 26.5 ms, so those stay with plain launches).
    if (e->ctx->comm != nullptr && e->ctx->nranks > 1) return est_us / launches < 300.0;
    return est_us / launches < 10.0;
}

// Runs one dispatch: eagerly the first time (which also sizes the scratch arena), recorded as a plan the
// second time, replayed afterwards.  A plan is recorded again when its key (the loss target) or the
// scratch arena it was recorded against has changed.  Inside a caller's own recording the work is
// simply enqueued, so that it becomes part of the caller's plan.
static int32_t run_planned(fg_exec* e, int which, const void* key, const std::function<int32_t()>& eager) {
    fg_ctx* ctx = e->ctx;
    if (!plans_wanted(e) || ctx->capturing) return eager();
    if (e->plan[which] && e->plan_key[which] == key && e->plan_ws[which] == (const void*)ctx->ws)
        return fg_plan_launch(ctx, e->plan[which]);
    if (e->calls[which]++ == 0) return eager();
    if (e->plan[which]) { fg_plan_destroy(e->plan[which]); e->plan[which] = nullptr; }
    int32_t s = fg_plan_begin(ctx);
    if (s != FG_OK) return eager();
    s = eager();
    fg_plan* p = nullptr;
    const int32_t s2 = fg_plan_end(ctx, &p);
    if (s != FG_OK || s2 != FG_OK) {
        if (p) fg_plan_destroy(p);
        e->use_plans = false;             // something in this graph cannot be recorded: stay eager
        return s != FG_OK ? s : eager();
    }
    e->plan[which] = p;
    e->plan_key[which] = key;
    e->plan_ws[which] = (const void*)ctx->ws;
    return fg_plan_launch(ctx, p);
}

int32_t fg_exec_dispatch_forward(fg_exec* e) {
    if (!e) return FG_ERR_NOT_INITIALIZED;
    FgRange range("ferrograd dispatch_forward");
    if (!e->bound) return fail(e, FG_ERR_NOT_INITIALIZED, "dispatch_forward: bind the input tensors first");
    if (e->paired) {
        // A recorded forward pass does not contain the pairs of the weights (the optimizer keeps them current).
        // If a weight tensor was rewritten from outside since, its pairs are made now, before the replay.
        for (size_t k = 0; k < e->inputs.size(); ++k) {
            ENode& en = e->n[e->inputs[k]];
            if (!en.pairs || !e->trainable[k] || (e->pairs_fresh[k] && e->pairs_version[k] == en.value->version)) continue;
            const int32_t s = fg_pairs_from_f32(e->ctx, (const float*)en.value->ptr, en.numel, en.pairs->ptr, pstride(e, e->inputs[k]));
            if (s != FG_OK) return s;
            e->pairs_fresh[k] = 1;
            e->pairs_version[k] = en.value->version;
        }
    }
    return run_planned(e, 0, nullptr, [&] { return forward_eager(e); });
}

int32_t fg_exec_dispatch_loss(fg_exec* e, const fg_buf* target) {
    if (!e) return FG_ERR_NOT_INITIALIZED;
    FgRange range("ferrograd dispatch_loss");
    FG_REQUIRE(e->ctx, target != nullptr, "dispatch_loss: target is NULL");
    if (!e->bound) return fail(e, FG_ERR_NOT_INITIALIZED, "dispatch_loss: bind the input tensors first");
    return run_planned(e, 1, target->ptr, [&] { return loss_eager(e, target); });
}

int32_t fg_exec_dispatch_backward(fg_exec* e) {
    if (!e) return FG_ERR_NOT_INITIALIZED;
    FgRange range("ferrograd dispatch_backward");
    if (!e->bound) return fail(e, FG_ERR_NOT_INITIALIZED, "dispatch_backward: bind the input tensors first");
    const int32_t s = run_planned(e, 2, nullptr, [&] { return backward_eager(e); });
    if (s == FG_OK) e->backward_done = true;
    return s;
}

int32_t fg_exec_dispatch_optim(fg_exec* e) {
    if (!e) return FG_ERR_NOT_INITIALIZED;
    FgRange range("ferrograd dispatch_optim");
    if (!e->bound) return fail(e, FG_ERR_NOT_INITIALIZED, "dispatch_optim: bind the input tensors first");
    // With a communicator, the range of the gradient arena that is still to be summed over the ranks depends on
    // whether a backward pass came before (it has exchanged everything below final_lo already); a recorded
    // dispatch is replayed only for the same range.
    e->optim_lo = e->backward_done ? e->final_lo : 0;
    const void* key = dp_active(e) ? (const void*)(uintptr_t)(e->optim_lo + 1) : nullptr;
    const int32_t s = run_planned(e, 3, key, [&] { return optim_eager(e); });
    if (s == FG_OK) e->backward_done = false;
    return s;
}

// dispatch_single_optim (dispatch/mod.rs:790-814): one weight, its gradient chosen by index.
int32_t fg_exec_dispatch_single_optim(fg_exec* e, fg_buf* weight, uint32_t grad_index) {
    if (!e) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(e->ctx, weight != nullptr, "dispatch_single_optim: weight is NULL");
    FG_REQUIRE(e->ctx, grad_index < e->grads.size() && e->n[e->grads[grad_index]].input_slot >= 0,
               "dispatch_single_optim: grad index does not name an input's gradient");
    const uint32_t slot = (uint32_t)e->n[e->grads[grad_index]].input_slot;
    FG_REQUIRE(e->ctx, weight->bytes >= e->n[e->inputs[slot]].numel * e->esize, "dispatch_single_optim: weight smaller than its gradient");
    return optim_one(e, slot, weight);
}

fg_buf* fg_exec_forward_out(fg_exec* e) { return e ? e->n[e->last].value : nullptr; }
fg_buf* fg_exec_seed(fg_exec* e) { return e ? e->seed : nullptr; }
fg_buf* fg_exec_loss_t(fg_exec* e) { return e ? e->loss_t : nullptr; }
fg_buf* fg_exec_loss_sum(fg_exec* e) { return e ? e->loss_sum : nullptr; }
uint32_t fg_exec_num_saved(fg_exec* e) { return e ? (uint32_t)e->saved.size() : 0; }
fg_buf* fg_exec_saved(fg_exec* e, uint32_t i, int32_t* node) {
    if (!e || i >= e->saved.size()) return nullptr;
    if (node) *node = e->saved[i];
    return e->n[e->saved[i]].value;
}
uint32_t fg_exec_num_grads(fg_exec* e) { return e ? (uint32_t)e->grads.size() : 0; }
fg_buf* fg_exec_grad(fg_exec* e, uint32_t i, int32_t* node) {
    if (!e || i >= e->grads.size()) return nullptr;
    if (node) *node = e->grads[i];
    return e->n[e->grads[i]].grad;
}
// Number of kernels the forward pass launches per dispatch (how much was fused).
uint32_t fg_exec_forward_steps(fg_exec* e) { return e ? (uint32_t)e->fwd.size() : 0; }
int32_t fg_exec_plans_active(fg_exec* e) { return e && plans_wanted(e) ? 1 : 0; }

}  // extern "C"
