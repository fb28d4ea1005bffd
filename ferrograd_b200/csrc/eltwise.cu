// Elementwise work: bias + activation, activation backward, MSE loss + gradient, column
// sums (bias gradient) and fused elementwise chains (one forward kernel, one backward
// kernel per chain).
//
// Semantics follow crates/ferrograd-nn/src/op/unary.rs (tanh :270-327, relu :436-490,
// gelu :492-733, elu :328-436, exp :741-756), crates/ferrograd-nn/src/op/binary.rs
// (add :74, mul :236, sub :449, div :644 and their backward forms) and
// MEAN_SQUARED_ERROR (crates/ferrograd-nn/src/loss/basic_loss.rs:3-27).  The reference
// inlines elementwise producers into their consumer kernel
// (crates/fused_gpu/src/dispatch/backend/kernel/forward.rs:298-464); a chain here is the
// same idea with the program interpreted per element: every input is read once, every
// output written once.
#include "fg_internal.cuh"

namespace {

constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

__global__ void __launch_bounds__(256) bias_act_kernel(uint32_t rows, uint32_t cols, const float* __restrict__ z,
                                                       const float* __restrict__ bias, int act, float* __restrict__ y) {
    const uint64_t n = (uint64_t)rows * cols;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        float p = z[i];
        if (bias) p += bias[i % cols];
        y[i] = fg_act_fwd(act, p);
    }
}

__global__ void __launch_bounds__(256) act_bwd_kernel(uint64_t n, int act, const float* __restrict__ dy,
                                                      const float* __restrict__ saved, float* __restrict__ dz) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        dz[i] = act == FG_ACT_NONE ? dy[i] : dy[i] * fg_act_grad(act, saved[i]);
}

// MSE: loss = d*d, grad = 2*d*scale; per-CTA partial sums of the loss go to `partials`.
__global__ void __launch_bounds__(256) mse_kernel(const float* __restrict__ pred, const float* __restrict__ target,
                                                  uint64_t n, float scale, float* __restrict__ loss_elem,
                                                  float* __restrict__ grad, float* __restrict__ partials) {
    __shared__ float red[8];
    float s = 0.0f;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        float d = pred[i] - target[i];
        float l = d * d;
        if (loss_elem) loss_elem[i] = l;
        if (grad) grad[i] = (2.0f * d) * scale;
        s += l;
    }
    if (partials) {
        s = warp_sum(s);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (int w = 0; w < 8; ++w) t += red[w];
            partials[blockIdx.x] = t;
        }
    }
}

// BCE on probabilities: loss = -(t*log(p) + (1-t)*log(1-p)), grad = (p - t)*scale.
__global__ void __launch_bounds__(256) bce_kernel(const float* __restrict__ pred, const float* __restrict__ target,
                                                  uint64_t n, float scale, float* __restrict__ loss_elem,
                                                  float* __restrict__ grad, float* __restrict__ partials) {
    __shared__ float red[8];
    float s = 0.0f;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const float p = pred[i], t = target[i];
        const float l = -(t * logf(p) + (1.0f - t) * logf(1.0f - p));
        if (loss_elem) loss_elem[i] = l;
        if (grad) grad[i] = (p - t) * scale;
        s += l;
    }
    if (partials) {
        s = warp_sum(s);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (int w = 0; w < 8; ++w) t += red[w];
            partials[blockIdx.x] = t;
        }
    }
}

// One CTA folds the partials in a fixed order.
__global__ void __launch_bounds__(256) fold_partials_kernel(const float* __restrict__ partials, int n,
                                                            float* __restrict__ out) {
    __shared__ float red[8];
    float s = 0.0f;
    for (int i = threadIdx.x; i < n; i += 256) s += partials[i];
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < 8; ++w) t += red[w];
        *out = t;
    }
}

// Column sums, stage 1: block (32 x 8) covers 32 columns and `chunk` rows.
__global__ void __launch_bounds__(256) colsum_partial_kernel(uint32_t rows, uint32_t cols, uint32_t chunk,
                                                             const float* __restrict__ x, float* __restrict__ part) {
    __shared__ float red[8][33];
    const uint32_t c = blockIdx.x * 32 + threadIdx.x;
    const uint32_t r0 = blockIdx.y * chunk;
    const uint32_t r1 = min(rows, r0 + chunk);
    float s = 0.0f;
    if (c < cols)
        for (uint32_t r = r0 + threadIdx.y; r < r1; r += 8) s += x[(size_t)r * cols + c];
    red[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < cols) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += red[k][threadIdx.x];
        part[(size_t)blockIdx.y * cols + c] = t;
    }
}
__global__ void __launch_bounds__(256) colsum_fold_kernel(uint32_t cols, uint32_t nchunks,
                                                          const float* __restrict__ part, float* __restrict__ out) {
    uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float s = 0.0f;
    for (uint32_t k = 0; k < nchunks; ++k) s += part[(size_t)k * cols + c];
    out[c] = s;
}

// ---- chains ----
struct ChainArgs {
    fg_ew_instr prog[FG_EW_MAX_INSTR];
    const float* in[FG_EW_MAX_INPUTS];
    float* saved[FG_EW_MAX_INSTR];   // forward: optional stores of intermediates
    float* grads[FG_EW_MAX_INPUTS];  // backward
    const float* seed;
    float* out;
    int ninstr, ninputs, accumulate;
    uint64_t n;
};

__device__ __forceinline__ float ew_eval(const fg_ew_instr& in, const float* v, const ChainArgs& a, uint64_t i) {
    switch (in.op) {
        case FG_EW_INPUT: return a.in[in.a][i];
        case FG_EW_CONST: return in.imm;
        case FG_EW_ADD: return v[in.a] + v[in.b];
        case FG_EW_SUB: return v[in.a] - v[in.b];
        case FG_EW_MUL: return v[in.a] * v[in.b];
        case FG_EW_DIV: return __fdiv_rn(v[in.a], v[in.b]);
        case FG_EW_NEG: return -v[in.a];
        case FG_EW_ABS: return fabsf(v[in.a]);
        case FG_EW_EXP: return expf(v[in.a]);
        case FG_EW_LOG: return logf(v[in.a]);
        case FG_EW_TANH: return tanhf(v[in.a]);
        case FG_EW_RELU: return v[in.a] > 0.0f ? v[in.a] : 0.0f;
        case FG_EW_GELU: return fg_gelu_fwd(v[in.a], nullptr);
        case FG_EW_ELU: return v[in.a] >= 0.0f ? v[in.a] : expf(v[in.a]) - 1.0f;
        default: return 0.0f;
    }
}

__global__ void __launch_bounds__(256) chain_fwd_kernel(const __grid_constant__ ChainArgs a) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (uint64_t)gridDim.x * blockDim.x) {
        float v[FG_EW_MAX_INSTR];
        for (int k = 0; k < a.ninstr; ++k) {
            v[k] = ew_eval(a.prog[k], v, a, i);
            if (a.saved[k]) a.saved[k][i] = v[k];
        }
        a.out[i] = v[a.ninstr - 1];
    }
}

__global__ void __launch_bounds__(256) chain_bwd_kernel(const __grid_constant__ ChainArgs a) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (uint64_t)gridDim.x * blockDim.x) {
        float v[FG_EW_MAX_INSTR], adj[FG_EW_MAX_INSTR], gin[FG_EW_MAX_INPUTS];
        for (int k = 0; k < a.ninstr; ++k) { v[k] = ew_eval(a.prog[k], v, a, i); adj[k] = 0.0f; }
        for (int k = 0; k < a.ninputs; ++k) gin[k] = 0.0f;
        adj[a.ninstr - 1] = a.seed[i];
        for (int k = a.ninstr - 1; k >= 0; --k) {
            const fg_ew_instr& in = a.prog[k];
            const float g = adj[k];
            switch (in.op) {
                case FG_EW_INPUT: gin[in.a] += g; break;
                case FG_EW_ADD: adj[in.a] += g; adj[in.b] += g; break;
                case FG_EW_SUB: adj[in.a] += g; adj[in.b] -= g; break;
                case FG_EW_MUL: { float va = v[in.a], vb = v[in.b]; adj[in.a] += g * vb; adj[in.b] += g * va; break; }
                case FG_EW_DIV: { float va = v[in.a], vb = v[in.b];
                                  adj[in.a] += __fdiv_rn(g, vb);
                                  adj[in.b] -= __fdiv_rn(g * va, vb * vb); break; }
                case FG_EW_NEG: adj[in.a] -= g; break;
                case FG_EW_ABS: adj[in.a] += (v[in.a] >= 0.0f ? g : -g); break;
                case FG_EW_EXP: adj[in.a] += g * v[k]; break;
                case FG_EW_LOG: adj[in.a] += __fdiv_rn(g, v[in.a]); break;
                case FG_EW_TANH: adj[in.a] += g * (1.0f - v[k] * v[k]); break;
                case FG_EW_RELU: adj[in.a] += g * fg_act_grad(FG_ACT_RELU, v[k]); break;
                case FG_EW_GELU: adj[in.a] += g * fg_act_grad(FG_ACT_GELU, v[in.a]); break;
                case FG_EW_ELU: adj[in.a] += (v[k] >= 0.0f ? g : g * (v[k] + 1.0f)); break;
                default: break;
            }
        }
        for (int k = 0; k < a.ninputs; ++k)
            if (a.grads[k]) a.grads[k][i] = a.accumulate ? a.grads[k][i] + gin[k] : gin[k];
    }
}

int32_t check_prog(fg_ctx* ctx, const fg_ew_instr* prog, int32_t ninstr, int32_t ninputs) {
    FG_REQUIRE(ctx, prog != nullptr, "eltwise chain: prog is NULL");
    FG_REQUIRE(ctx, ninstr >= 1 && ninstr <= FG_EW_MAX_INSTR, "eltwise chain: instruction count out of range");
    FG_REQUIRE(ctx, ninputs >= 1 && ninputs <= FG_EW_MAX_INPUTS, "eltwise chain: input count out of range");
    for (int k = 0; k < ninstr; ++k) {
        const fg_ew_instr& in = prog[k];
        FG_REQUIRE(ctx, in.op >= FG_EW_INPUT && in.op <= FG_EW_ELU, "eltwise chain: unknown op code");
        if (in.op == FG_EW_INPUT) {
            FG_REQUIRE(ctx, in.a >= 0 && in.a < ninputs, "eltwise chain: input index out of range");
        } else if (in.op != FG_EW_CONST) {
            FG_REQUIRE(ctx, in.a >= 0 && in.a < k, "eltwise chain: operand a must name an earlier value");
            if (in.op >= FG_EW_ADD && in.op <= FG_EW_DIV)
                FG_REQUIRE(ctx, in.b >= 0 && in.b < k, "eltwise chain: operand b must name an earlier value");
        }
    }
    return FG_OK;
}

}  // namespace

int32_t fg_act_bwd_launch(fg_ctx* ctx, uint64_t n, int act, const float* dy, const float* saved, float* dz) {
    int grid = fg_stream_grid(ctx, n, 256, 8);
    act_bwd_kernel<<<grid, 256, 0, ctx->stream>>>(n, act, dy, saved, dz);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t fg_colsum_fold_launch(fg_ctx* ctx, uint32_t cols, uint32_t nchunks, const float* part, float* out) {
    colsum_fold_kernel<<<(cols + 255) / 256, 256, 0, ctx->stream>>>(cols, nchunks, part, out);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t fg_colsum_launch(fg_ctx* ctx, uint32_t rows, uint32_t cols, const float* x, float* out) {
    const uint32_t chunk = 256;
    const uint32_t nchunks = (rows + chunk - 1) / chunk;
    void* part;
    int32_t s = fg_ws_alloc(ctx, (uint64_t)nchunks * cols * sizeof(float), &part);
    if (s != FG_OK) return s;
    dim3 grid((cols + 31) / 32, nchunks), block(32, 8);
    colsum_partial_kernel<<<grid, block, 0, ctx->stream>>>(rows, cols, chunk, x, (float*)part);
    FG_LAUNCHED(ctx);
    colsum_fold_kernel<<<(cols + 255) / 256, 256, 0, ctx->stream>>>(cols, nchunks, (const float*)part, out);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

extern "C" {

int32_t fg_bias_act_fwd(fg_ctx* ctx, uint32_t rows, uint32_t cols, const float* z, const float* bias, int32_t act,
                        float* y) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, z && y, "fg_bias_act_fwd: NULL pointer");
    FG_REQUIRE(ctx, act >= FG_ACT_NONE && act <= FG_ACT_GELU, "fg_bias_act_fwd: unknown activation");
    if ((uint64_t)rows * cols == 0) return FG_OK;
    int grid = fg_stream_grid(ctx, (uint64_t)rows * cols, 256, 8);
    bias_act_kernel<<<grid, 256, 0, ctx->stream>>>(rows, cols, z, bias, act, y);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t fg_act_bwd(fg_ctx* ctx, uint64_t n, int32_t act, const float* dy, const float* saved, float* dz) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, dy && dz, "fg_act_bwd: NULL pointer");
    FG_REQUIRE(ctx, act >= FG_ACT_NONE && act <= FG_ACT_GELU, "fg_act_bwd: unknown activation");
    FG_REQUIRE(ctx, act == FG_ACT_NONE || saved, "fg_act_bwd: saved tensor required");
    if (n == 0) return FG_OK;
    return fg_act_bwd_launch(ctx, n, act, dy, saved, dz);
}

int32_t fg_mse_loss_grad(fg_ctx* ctx, const float* pred, const float* target, uint64_t n, float grad_scale,
                         float* loss_elem_out, float* loss_sum_out, float* grad_out) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, pred && target, "fg_mse_loss_grad: NULL pointer");
    FG_REQUIRE(ctx, loss_elem_out || loss_sum_out || grad_out, "fg_mse_loss_grad: no output requested");
    if (n == 0) {
        if (loss_sum_out) FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY, cudaMemsetAsync(loss_sum_out, 0, 4, ctx->stream));
        return FG_OK;
    }
    int grid = fg_stream_grid(ctx, n, 256, 8);
    float* partials = nullptr;
    if (loss_sum_out) {
        void* p;
        int32_t s = fg_ws_alloc(ctx, (uint64_t)grid * sizeof(float), &p);
        if (s != FG_OK) return s;
        partials = (float*)p;
    }
    mse_kernel<<<grid, 256, 0, ctx->stream>>>(pred, target, n, grad_scale, loss_elem_out, grad_out, partials);
    FG_LAUNCHED(ctx);
    if (loss_sum_out) {
        fold_partials_kernel<<<1, 256, 0, ctx->stream>>>(partials, grid, loss_sum_out);
        FG_LAUNCHED(ctx);
    }
    return FG_OK;
}

int32_t fg_bce_loss_grad(fg_ctx* ctx, const float* pred, const float* target, uint64_t n, float grad_scale,
                         float* loss_elem_out, float* loss_sum_out, float* grad_out) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, pred && target, "fg_bce_loss_grad: NULL pointer");
    FG_REQUIRE(ctx, loss_elem_out || loss_sum_out || grad_out, "fg_bce_loss_grad: no output requested");
    if (n == 0) {
        if (loss_sum_out) FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY, cudaMemsetAsync(loss_sum_out, 0, 4, ctx->stream));
        return FG_OK;
    }
    int grid = fg_stream_grid(ctx, n, 256, 8);
    float* partials = nullptr;
    if (loss_sum_out) {
        void* p;
        int32_t s = fg_ws_alloc(ctx, (uint64_t)grid * sizeof(float), &p);
        if (s != FG_OK) return s;
        partials = (float*)p;
    }
    bce_kernel<<<grid, 256, 0, ctx->stream>>>(pred, target, n, grad_scale, loss_elem_out, grad_out, partials);
    FG_LAUNCHED(ctx);
    if (loss_sum_out) {
        fold_partials_kernel<<<1, 256, 0, ctx->stream>>>(partials, grid, loss_sum_out);
        FG_LAUNCHED(ctx);
    }
    return FG_OK;
}

int32_t fg_eltwise_chain_fwd(fg_ctx* ctx, uint64_t n, const fg_ew_instr* prog, int32_t ninstr,
                             const float* const* inputs, int32_t ninputs, float* out, float* const* saved_out) {
    FG_ENTER(ctx);
    int32_t s = check_prog(ctx, prog, ninstr, ninputs);
    if (s != FG_OK) return s;
    FG_REQUIRE(ctx, inputs && out, "fg_eltwise_chain_fwd: NULL pointer");
    ChainArgs a;
    memset(&a, 0, sizeof(a));
    for (int k = 0; k < ninstr; ++k) { a.prog[k] = prog[k]; a.saved[k] = saved_out ? saved_out[k] : nullptr; }
    for (int k = 0; k < ninputs; ++k) {
        FG_REQUIRE(ctx, inputs[k] != nullptr, "fg_eltwise_chain_fwd: NULL input");
        a.in[k] = inputs[k];
    }
    a.out = out; a.ninstr = ninstr; a.ninputs = ninputs; a.n = n;
    if (n == 0) return FG_OK;
    int grid = fg_stream_grid(ctx, n, 256, 8);
    chain_fwd_kernel<<<grid, 256, 0, ctx->stream>>>(a);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t fg_eltwise_chain_bwd(fg_ctx* ctx, uint64_t n, const fg_ew_instr* prog, int32_t ninstr,
                             const float* const* inputs, int32_t ninputs, const float* seed, float* const* grads,
                             int32_t accumulate) {
    FG_ENTER(ctx);
    int32_t s = check_prog(ctx, prog, ninstr, ninputs);
    if (s != FG_OK) return s;
    FG_REQUIRE(ctx, inputs && seed && grads, "fg_eltwise_chain_bwd: NULL pointer");
    ChainArgs a;
    memset(&a, 0, sizeof(a));
    for (int k = 0; k < ninstr; ++k) a.prog[k] = prog[k];
    for (int k = 0; k < ninputs; ++k) {
        FG_REQUIRE(ctx, inputs[k] != nullptr, "fg_eltwise_chain_bwd: NULL input");
        a.in[k] = inputs[k];
        a.grads[k] = grads[k];
    }
    a.seed = seed; a.ninstr = ninstr; a.ninputs = ninputs; a.n = n; a.accumulate = accumulate;
    if (n == 0) return FG_OK;
    int grid = fg_stream_grid(ctx, n, 256, 8);
    chain_bwd_kernel<<<grid, 256, 0, ctx->stream>>>(a);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

}  // extern "C"
