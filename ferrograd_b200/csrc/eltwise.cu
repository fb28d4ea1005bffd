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
#include <cuda_bf16.h>
#include <cuda_fp16.h>

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

// Sum of n values, stage 1: one partial per CTA (grid-stride over float4, fixed order inside a CTA).
__global__ void __launch_bounds__(256) sum_partial_kernel(const float* __restrict__ x, uint64_t n, float* __restrict__ partials) {
    __shared__ float red[8];
    float s = 0.0f;
    const uint64_t nv = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) ? n >> 2 : 0, stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(x) + i);
        s += (v.x + v.y) + (v.z + v.w);
    }
    for (uint64_t i = (nv << 2) + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) s += x[i];
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < 8; ++w) t += red[w];
        partials[blockIdx.x] = t;
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
// Storage type of a chain's tensors.  Values are held as float in registers; with 16-bit storage every
// operation's result is rounded to the storage type (round to nearest even), which for + - * / equals
// native half arithmetic (float carries more than twice the bits, so the double rounding is harmless).
template <int DT> struct Stored;
template <> struct Stored<FG_DTYPE_F32> {
    typedef float T;
    static __device__ __forceinline__ float ld(const void* p, uint64_t i) { return static_cast<const float*>(p)[i]; }
    static __device__ __forceinline__ void st(void* p, uint64_t i, float v) { static_cast<float*>(p)[i] = v; }
    static __device__ __forceinline__ float r(float v) { return v; }
};
template <> struct Stored<FG_DTYPE_F16> {
    typedef __half T;
    static __device__ __forceinline__ float ld(const void* p, uint64_t i) { return __half2float(static_cast<const __half*>(p)[i]); }
    static __device__ __forceinline__ void st(void* p, uint64_t i, float v) { static_cast<__half*>(p)[i] = __float2half_rn(v); }
    static __device__ __forceinline__ float r(float v) { return __half2float(__float2half_rn(v)); }
};
template <> struct Stored<FG_DTYPE_BF16> {
    typedef __nv_bfloat16 T;
    static __device__ __forceinline__ float ld(const void* p, uint64_t i) { return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]); }
    static __device__ __forceinline__ void st(void* p, uint64_t i, float v) { static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

struct ChainArgs {
    fg_ew_instr prog[FG_EW_MAX_INSTR];
    const void* in[FG_EW_MAX_INPUTS];
    void* saved[FG_EW_MAX_INSTR];   // forward: optional stores of intermediates
    void* grads[FG_EW_MAX_INPUTS];  // backward
    const void* seed;
    void* out;
    int ninstr, ninputs, accumulate;
    uint64_t n;
};

template <int DT>
__device__ __forceinline__ float ew_eval(const fg_ew_instr& in, const float* v, const ChainArgs& a, uint64_t i) {
    typedef Stored<DT> S;
    switch (in.op) {
        case FG_EW_INPUT: return S::ld(a.in[in.a], i);
        case FG_EW_CONST: return S::r(in.imm);
        case FG_EW_ADD: return S::r(v[in.a] + v[in.b]);
        case FG_EW_SUB: return S::r(v[in.a] - v[in.b]);
        case FG_EW_MUL: return S::r(v[in.a] * v[in.b]);
        case FG_EW_DIV: return S::r(__fdiv_rn(v[in.a], v[in.b]));
        case FG_EW_NEG: return -v[in.a];
        case FG_EW_ABS: return fabsf(v[in.a]);
        case FG_EW_EXP: return S::r(expf(v[in.a]));
        case FG_EW_LOG: return S::r(logf(v[in.a]));
        case FG_EW_TANH: return S::r(tanhf(v[in.a]));
        case FG_EW_RELU: return v[in.a] > 0.0f ? v[in.a] : 0.0f;
        case FG_EW_GELU: return S::r(fg_gelu_fwd(v[in.a], nullptr));
        case FG_EW_ELU: return v[in.a] >= 0.0f ? v[in.a] : S::r(expf(v[in.a]) - 1.0f);
        default: return 0.0f;
    }
}

template <int DT>
__global__ void __launch_bounds__(256) chain_fwd_kernel(const __grid_constant__ ChainArgs a) {
    typedef Stored<DT> S;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (uint64_t)gridDim.x * blockDim.x) {
        float v[FG_EW_MAX_INSTR];
        for (int k = 0; k < a.ninstr; ++k) {
            v[k] = ew_eval<DT>(a.prog[k], v, a, i);
            if (a.saved[k]) S::st(a.saved[k], i, v[k]);
        }
        S::st(a.out, i, v[a.ninstr - 1]);
    }
}

template <int DT>
__global__ void __launch_bounds__(256) chain_bwd_kernel(const __grid_constant__ ChainArgs a) {
    typedef Stored<DT> S;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (uint64_t)gridDim.x * blockDim.x) {
        float v[FG_EW_MAX_INSTR], adj[FG_EW_MAX_INSTR], gin[FG_EW_MAX_INPUTS];
        for (int k = 0; k < a.ninstr; ++k) { v[k] = ew_eval<DT>(a.prog[k], v, a, i); adj[k] = 0.0f; }
        for (int k = 0; k < a.ninputs; ++k) gin[k] = 0.0f;
        adj[a.ninstr - 1] = S::ld(a.seed, i);
        for (int k = a.ninstr - 1; k >= 0; --k) {
            const fg_ew_instr& in = a.prog[k];
            const float g = adj[k];
            switch (in.op) {
                case FG_EW_INPUT: gin[in.a] = S::r(gin[in.a] + g); break;
                case FG_EW_ADD: adj[in.a] = S::r(adj[in.a] + g); adj[in.b] = S::r(adj[in.b] + g); break;
                case FG_EW_SUB: adj[in.a] = S::r(adj[in.a] + g); adj[in.b] = S::r(adj[in.b] - g); break;
                case FG_EW_MUL: { float va = v[in.a], vb = v[in.b];
                                  adj[in.a] = S::r(adj[in.a] + S::r(g * vb));
                                  adj[in.b] = S::r(adj[in.b] + S::r(g * va)); break; }
                case FG_EW_DIV: { float va = v[in.a], vb = v[in.b];
                                  adj[in.a] = S::r(adj[in.a] + S::r(__fdiv_rn(g, vb)));
                                  adj[in.b] = S::r(adj[in.b] - S::r(__fdiv_rn(S::r(g * va), S::r(vb * vb)))); break; }
                case FG_EW_NEG: adj[in.a] = S::r(adj[in.a] - g); break;
                case FG_EW_ABS: adj[in.a] = S::r(adj[in.a] + (v[in.a] >= 0.0f ? g : -g)); break;
                case FG_EW_EXP: adj[in.a] = S::r(adj[in.a] + S::r(g * v[k])); break;
                case FG_EW_LOG: adj[in.a] = S::r(adj[in.a] + S::r(__fdiv_rn(g, v[in.a]))); break;
                case FG_EW_TANH: adj[in.a] = S::r(adj[in.a] + S::r(g * S::r(1.0f - S::r(v[k] * v[k])))); break;
                case FG_EW_RELU: adj[in.a] = S::r(adj[in.a] + g * fg_act_grad(FG_ACT_RELU, v[k])); break;
                case FG_EW_GELU: adj[in.a] = S::r(adj[in.a] + S::r(g * S::r(fg_act_grad(FG_ACT_GELU, v[in.a])))); break;
                case FG_EW_ELU: adj[in.a] = S::r(adj[in.a] + (v[k] >= 0.0f ? g : S::r(g * S::r(v[k] + 1.0f)))); break;
                default: break;
            }
        }
        for (int k = 0; k < a.ninputs; ++k)
            if (a.grads[k]) S::st(a.grads[k], i, a.accumulate ? S::r(S::ld(a.grads[k], i) + gin[k]) : gin[k]);
    }
}

// dst[i] = (type of dst) src[i], round to nearest even
template <int DS, int DD>
__global__ void __launch_bounds__(256) convert_kernel(const void* __restrict__ src, void* __restrict__ dst, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        Stored<DD>::st(dst, i, Stored<DS>::ld(src, i));
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

int32_t fg_sum_f32(fg_ctx* ctx, const float* x, uint64_t n, float* out) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, x && out, "fg_sum_f32: NULL pointer");
    if (n == 0) {
        FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY, cudaMemsetAsync(out, 0, 4, ctx->stream));
        return FG_OK;
    }
    const int grid = fg_stream_grid(ctx, (n + 3) / 4, 256, 4);
    void* p;
    int32_t s = fg_ws_alloc(ctx, (uint64_t)grid * sizeof(float), &p);
    if (s != FG_OK) return s;
    sum_partial_kernel<<<grid, 256, 0, ctx->stream>>>(x, n, (float*)p);
    FG_LAUNCHED(ctx);
    fold_partials_kernel<<<1, 256, 0, ctx->stream>>>((const float*)p, grid, out);
    FG_LAUNCHED(ctx);
    return FG_OK;
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

int32_t fg_eltwise_chain_fwd_dt(fg_ctx* ctx, int32_t dtype, uint64_t n, const fg_ew_instr* prog, int32_t ninstr,
                                const void* const* inputs, int32_t ninputs, void* out, void* const* saved_out) {
    FG_ENTER(ctx);
    int32_t s = check_prog(ctx, prog, ninstr, ninputs);
    if (s != FG_OK) return s;
    FG_REQUIRE(ctx, dtype >= FG_DTYPE_F32 && dtype <= FG_DTYPE_BF16, "fg_eltwise_chain_fwd: unknown dtype");
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
    if (dtype == FG_DTYPE_F32) chain_fwd_kernel<FG_DTYPE_F32><<<grid, 256, 0, ctx->stream>>>(a);
    else if (dtype == FG_DTYPE_F16) chain_fwd_kernel<FG_DTYPE_F16><<<grid, 256, 0, ctx->stream>>>(a);
    else chain_fwd_kernel<FG_DTYPE_BF16><<<grid, 256, 0, ctx->stream>>>(a);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t fg_eltwise_chain_bwd_dt(fg_ctx* ctx, int32_t dtype, uint64_t n, const fg_ew_instr* prog, int32_t ninstr,
                                const void* const* inputs, int32_t ninputs, const void* seed, void* const* grads,
                                int32_t accumulate) {
    FG_ENTER(ctx);
    int32_t s = check_prog(ctx, prog, ninstr, ninputs);
    if (s != FG_OK) return s;
    FG_REQUIRE(ctx, dtype >= FG_DTYPE_F32 && dtype <= FG_DTYPE_BF16, "fg_eltwise_chain_bwd: unknown dtype");
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
    if (dtype == FG_DTYPE_F32) chain_bwd_kernel<FG_DTYPE_F32><<<grid, 256, 0, ctx->stream>>>(a);
    else if (dtype == FG_DTYPE_F16) chain_bwd_kernel<FG_DTYPE_F16><<<grid, 256, 0, ctx->stream>>>(a);
    else chain_bwd_kernel<FG_DTYPE_BF16><<<grid, 256, 0, ctx->stream>>>(a);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t fg_eltwise_chain_fwd(fg_ctx* ctx, uint64_t n, const fg_ew_instr* prog, int32_t ninstr,
                             const float* const* inputs, int32_t ninputs, float* out, float* const* saved_out) {
    return fg_eltwise_chain_fwd_dt(ctx, FG_DTYPE_F32, n, prog, ninstr, reinterpret_cast<const void* const*>(inputs), ninputs,
                                   out, reinterpret_cast<void* const*>(saved_out));
}

int32_t fg_eltwise_chain_bwd(fg_ctx* ctx, uint64_t n, const fg_ew_instr* prog, int32_t ninstr,
                             const float* const* inputs, int32_t ninputs, const float* seed, float* const* grads,
                             int32_t accumulate) {
    return fg_eltwise_chain_bwd_dt(ctx, FG_DTYPE_F32, n, prog, ninstr, reinterpret_cast<const void* const*>(inputs), ninputs,
                                   seed, reinterpret_cast<void* const*>(grads), accumulate);
}

int32_t fg_convert(fg_ctx* ctx, const void* src, int32_t src_dtype, void* dst, int32_t dst_dtype, uint64_t n) {
    FG_ENTER(ctx);
    return fg_convert_launch(ctx, src, src_dtype, dst, dst_dtype, n);
}

}  // extern "C"

int32_t fg_convert_launch(fg_ctx* ctx, const void* src, int src_dtype, void* dst, int dst_dtype, uint64_t n) {
    FG_REQUIRE(ctx, src && dst, "fg_convert: NULL pointer");
    FG_REQUIRE(ctx, src_dtype >= FG_DTYPE_F32 && src_dtype <= FG_DTYPE_BF16 && dst_dtype >= FG_DTYPE_F32 &&
                        dst_dtype <= FG_DTYPE_BF16, "fg_convert: unknown dtype");
    if (n == 0) return FG_OK;
    const int grid = fg_stream_grid(ctx, n, 256, 8);
#define FG_CONV(S, D) if (src_dtype == S && dst_dtype == D) convert_kernel<S, D><<<grid, 256, 0, ctx->stream>>>(src, dst, n)
    FG_CONV(FG_DTYPE_F32, FG_DTYPE_F32); FG_CONV(FG_DTYPE_F32, FG_DTYPE_F16); FG_CONV(FG_DTYPE_F32, FG_DTYPE_BF16);
    FG_CONV(FG_DTYPE_F16, FG_DTYPE_F32); FG_CONV(FG_DTYPE_F16, FG_DTYPE_F16); FG_CONV(FG_DTYPE_F16, FG_DTYPE_BF16);
    FG_CONV(FG_DTYPE_BF16, FG_DTYPE_F32); FG_CONV(FG_DTYPE_BF16, FG_DTYPE_F16); FG_CONV(FG_DTYPE_BF16, FG_DTYPE_BF16);
#undef FG_CONV
    FG_LAUNCHED(ctx);
    return FG_OK;
}
