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

// The streaming kernels below move four consecutive floats per thread and access (128-bit loads and stores) when
// every pointer they are given is 16-byte aligned (VEC), one float otherwise; the last n % 4 elements always go
// singly.  `nv` is the number of whole groups of four.
__device__ __forceinline__ float4 ld4(const float* p, uint64_t i4) { return reinterpret_cast<const float4*>(p)[i4]; }
__device__ __forceinline__ void st4(float* p, uint64_t i4, float4 v) { reinterpret_cast<float4*>(p)[i4] = v; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// y = act(z + bias[col]); with VEC, cols is a multiple of four, so a group of four never straddles a row.
template <bool VEC>
__global__ void __launch_bounds__(256) bias_act_kernel(uint32_t rows, uint32_t cols, const float* __restrict__ z,
                                                       const float* __restrict__ bias, int act, float* __restrict__ y) {
    const uint64_t n = (uint64_t)rows * cols, stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nv = VEC ? n >> 2 : 0;
    const uint32_t cols4 = cols >> 2;
    if constexpr (VEC) for (uint64_t i = g; i < nv; i += stride) {
        float4 p = ld4(z, i);
        if (bias) {
            const float4 b = ld4(bias, i % cols4);
            p.x += b.x; p.y += b.y; p.z += b.z; p.w += b.w;
        }
        st4(y, i, make_float4(fg_act_fwd(act, p.x), fg_act_fwd(act, p.y), fg_act_fwd(act, p.z), fg_act_fwd(act, p.w)));
    }
    for (uint64_t i = (nv << 2) + g; i < n; i += stride) {
        float p = z[i];
        if (bias) p += bias[i % cols];
        y[i] = fg_act_fwd(act, p);
    }
}

template <bool VEC>
__global__ void __launch_bounds__(256) act_bwd_kernel(uint64_t n, int act, const float* __restrict__ dy,
                                                      const float* __restrict__ saved, float* __restrict__ dz) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nv = VEC ? n >> 2 : 0;
    if constexpr (VEC) for (uint64_t i = g; i < nv; i += stride) {
        float4 d = ld4(dy, i);
        if (act != FG_ACT_NONE) {
            const float4 s = ld4(saved, i);
            d.x *= fg_act_grad(act, s.x); d.y *= fg_act_grad(act, s.y);
            d.z *= fg_act_grad(act, s.z); d.w *= fg_act_grad(act, s.w);
        }
        st4(dz, i, d);
    }
    for (uint64_t i = (nv << 2) + g; i < n; i += stride)
        dz[i] = act == FG_ACT_NONE ? dy[i] : dy[i] * fg_act_grad(act, saved[i]);
}

struct MseTerm {   // loss = d*d, grad = 2*d*scale
    static __device__ __forceinline__ float loss(float p, float t) { const float d = p - t; return d * d; }
    static __device__ __forceinline__ float grad(float p, float t, float scale) { return (2.0f * (p - t)) * scale; }
};
struct BceTerm {   // on probabilities: loss = -(t*log(p) + (1-t)*log(1-p)), grad = (p - t)*scale
    static __device__ __forceinline__ float loss(float p, float t) { return -(t * logf(p) + (1.0f - t) * logf(1.0f - p)); }
    static __device__ __forceinline__ float grad(float p, float t, float scale) { return (p - t) * scale; }
};

// Per-element loss and gradient of MSE or BCE; per-CTA partial sums of the loss go to `partials`.
template <class TERM, bool VEC>
__global__ void __launch_bounds__(256) loss_kernel(const float* __restrict__ pred, const float* __restrict__ target,
                                                   uint64_t n, float scale, float* __restrict__ loss_elem,
                                                   float* __restrict__ grad, float* __restrict__ partials) {
    __shared__ float red[8];
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nv = VEC ? n >> 2 : 0;
    float s = 0.0f;
    if constexpr (VEC) for (uint64_t i = g; i < nv; i += stride) {
        const float4 p = ld4(pred, i), t = ld4(target, i);
        const float4 l = make_float4(TERM::loss(p.x, t.x), TERM::loss(p.y, t.y), TERM::loss(p.z, t.z), TERM::loss(p.w, t.w));
        if (loss_elem) st4(loss_elem, i, l);
        if (grad)
            st4(grad, i, make_float4(TERM::grad(p.x, t.x, scale), TERM::grad(p.y, t.y, scale), TERM::grad(p.z, t.z, scale),
                                     TERM::grad(p.w, t.w, scale)));
        s += (l.x + l.y) + (l.z + l.w);
    }
    for (uint64_t i = (nv << 2) + g; i < n; i += stride) {
        const float p = pred[i], t = target[i], l = TERM::loss(p, t);
        if (loss_elem) loss_elem[i] = l;
        if (grad) grad[i] = TERM::grad(p, t, scale);
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
// ldw / stw move W consecutive elements starting at element i (W = 4: one 128-bit access for f32, one 64-bit
// access for the 16-bit types; the caller has checked the alignment).
template <int DT> struct Stored;
template <> struct Stored<FG_DTYPE_F32> {
    typedef float T;
    static __device__ __forceinline__ float ld(const void* p, uint64_t i) { return static_cast<const float*>(p)[i]; }
    static __device__ __forceinline__ void st(void* p, uint64_t i, float v) { static_cast<float*>(p)[i] = v; }
    static __device__ __forceinline__ float r(float v) { return v; }
    static __device__ __forceinline__ void ld4w(const void* p, uint64_t i, float* o) {
        const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + i);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
    static __device__ __forceinline__ void st4w(void* p, uint64_t i, const float* v) {
        *reinterpret_cast<float4*>(static_cast<float*>(p) + i) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Stored<FG_DTYPE_F16> {
    typedef __half T;
    static __device__ __forceinline__ float ld(const void* p, uint64_t i) { return __half2float(static_cast<const __half*>(p)[i]); }
    static __device__ __forceinline__ void st(void* p, uint64_t i, float v) { static_cast<__half*>(p)[i] = __float2half_rn(v); }
    static __device__ __forceinline__ float r(float v) { return __half2float(__float2half_rn(v)); }
    static __device__ __forceinline__ void ld4w(const void* p, uint64_t i, float* o) {
        const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const __half*>(p) + i);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
    }
    static __device__ __forceinline__ void st4w(void* p, uint64_t i, const float* v) {
        const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
        uint2 u;
        u.x = *reinterpret_cast<const uint32_t*>(&a); u.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(static_cast<__half*>(p) + i) = u;
    }
};
template <> struct Stored<FG_DTYPE_BF16> {
    typedef __nv_bfloat16 T;
    static __device__ __forceinline__ float ld(const void* p, uint64_t i) { return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]); }
    static __device__ __forceinline__ void st(void* p, uint64_t i, float v) { static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    static __device__ __forceinline__ void ld4w(const void* p, uint64_t i, float* o) {
        const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p) + i);
        o[0] = __uint_as_float(u.x << 16); o[1] = __uint_as_float(u.x & 0xffff0000u);
        o[2] = __uint_as_float(u.y << 16); o[3] = __uint_as_float(u.y & 0xffff0000u);
    }
    static __device__ __forceinline__ void st4w(void* p, uint64_t i, const float* v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 u;
        u.x = *reinterpret_cast<const uint32_t*>(&a); u.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p) + i) = u;
    }
};
template <int DT, int W> __device__ __forceinline__ void ldw(const void* p, uint64_t i, float* o) {
    if (W == 4) Stored<DT>::ld4w(p, i, o); else o[0] = Stored<DT>::ld(p, i);
}
template <int DT, int W> __device__ __forceinline__ void stw(void* p, uint64_t i, const float* v) {
    if (W == 4) Stored<DT>::st4w(p, i, v); else Stored<DT>::st(p, i, v[0]);
}

struct ChainArgs {
    fg_ew_instr prog[FG_EW_MAX_INSTR];
    const void* in[FG_EW_MAX_INPUTS];
    void* saved[FG_EW_MAX_INSTR];   // forward: optional stores of intermediates
    void* grads[FG_EW_MAX_INPUTS];  // backward
    const void* seed;
    void* out;
    int ninstr, ninputs, accumulate, vec;
    uint64_t n;
};

// One instruction on one element.
template <int DT>
__device__ __forceinline__ float ew_op(int op, float imm, float x, float y) {
    typedef Stored<DT> S;
    switch (op) {
        case FG_EW_CONST: return S::r(imm);
        case FG_EW_ADD: return S::r(x + y);
        case FG_EW_SUB: return S::r(x - y);
        case FG_EW_MUL: return S::r(x * y);
        case FG_EW_DIV: return S::r(__fdiv_rn(x, y));
        case FG_EW_NEG: return -x;
        case FG_EW_ABS: return fabsf(x);
        case FG_EW_EXP: return S::r(expf(x));
        case FG_EW_LOG: return S::r(logf(x));
        case FG_EW_TANH: return S::r(tanhf(x));
        case FG_EW_RELU: return x > 0.0f ? x : 0.0f;
        case FG_EW_GELU: return S::r(fg_gelu_fwd(x, nullptr));
        case FG_EW_ELU: return x >= 0.0f ? x : S::r(expf(x) - 1.0f);
        default: return 0.0f;
    }
}

// The program on W consecutive elements starting at i: the decode of an instruction is shared by the W lanes.
template <int DT, int W>
__device__ __forceinline__ void ew_forward(const ChainArgs& a, uint64_t i, float (*v)[W]) {
    for (int k = 0; k < a.ninstr; ++k) {
        const fg_ew_instr in = a.prog[k];
        if (in.op == FG_EW_INPUT) {
            ldw<DT, W>(a.in[in.a], i, v[k]);
        } else {
            const int ia = in.op == FG_EW_CONST ? 0 : in.a, ib = (in.op >= FG_EW_ADD && in.op <= FG_EW_DIV) ? in.b : ia;
#pragma unroll
            for (int w = 0; w < W; ++w) v[k][w] = ew_op<DT>(in.op, in.imm, v[ia][w], v[ib][w]);
        }
    }
}

template <int DT, int W>
__device__ __forceinline__ void chain_fwd_at(const ChainArgs& a, uint64_t i) {
    float v[FG_EW_MAX_INSTR][W];
    ew_forward<DT, W>(a, i, v);
    for (int k = 0; k < a.ninstr; ++k)
        if (a.saved[k]) stw<DT, W>(a.saved[k], i, v[k]);
    stw<DT, W>(a.out, i, v[a.ninstr - 1]);
}

template <int DT>
__global__ void __launch_bounds__(256) chain_fwd_kernel(const __grid_constant__ ChainArgs a) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nv = a.vec ? a.n >> 2 : 0;
    for (uint64_t i = g; i < nv; i += stride) chain_fwd_at<DT, 4>(a, i << 2);
    for (uint64_t i = (nv << 2) + g; i < a.n; i += stride) chain_fwd_at<DT, 1>(a, i);
}

// Adjoint of one instruction on one element: adds to the adjoints of its operands.
template <int DT>
__device__ __forceinline__ void ew_adjoint(int op, float g, float va, float vb, float vk, float& ga, float& gb) {
    typedef Stored<DT> S;
    switch (op) {
        case FG_EW_ADD: ga = S::r(ga + g); gb = S::r(gb + g); break;
        case FG_EW_SUB: ga = S::r(ga + g); gb = S::r(gb - g); break;
        case FG_EW_MUL: ga = S::r(ga + S::r(g * vb)); gb = S::r(gb + S::r(g * va)); break;
        case FG_EW_DIV: ga = S::r(ga + S::r(__fdiv_rn(g, vb)));
                        gb = S::r(gb - S::r(__fdiv_rn(S::r(g * va), S::r(vb * vb)))); break;
        case FG_EW_NEG: ga = S::r(ga - g); break;
        case FG_EW_ABS: ga = S::r(ga + (va >= 0.0f ? g : -g)); break;
        case FG_EW_EXP: ga = S::r(ga + S::r(g * vk)); break;
        case FG_EW_LOG: ga = S::r(ga + S::r(__fdiv_rn(g, va))); break;
        case FG_EW_TANH: ga = S::r(ga + S::r(g * S::r(1.0f - S::r(vk * vk)))); break;
        case FG_EW_RELU: ga = S::r(ga + g * fg_act_grad(FG_ACT_RELU, vk)); break;
        case FG_EW_GELU: ga = S::r(ga + S::r(g * S::r(fg_act_grad(FG_ACT_GELU, va)))); break;
        case FG_EW_ELU: ga = S::r(ga + (vk >= 0.0f ? g : S::r(g * S::r(vk + 1.0f)))); break;
        default: break;
    }
}

template <int DT, int W>
__device__ __forceinline__ void chain_bwd_at(const ChainArgs& a, uint64_t i) {
    typedef Stored<DT> S;
    float v[FG_EW_MAX_INSTR][W], adj[FG_EW_MAX_INSTR][W], gin[FG_EW_MAX_INPUTS][W];
    ew_forward<DT, W>(a, i, v);
    for (int k = 0; k < a.ninstr; ++k)
#pragma unroll
        for (int w = 0; w < W; ++w) adj[k][w] = 0.0f;
    for (int k = 0; k < a.ninputs; ++k)
#pragma unroll
        for (int w = 0; w < W; ++w) gin[k][w] = 0.0f;
    ldw<DT, W>(a.seed, i, adj[a.ninstr - 1]);
    for (int k = a.ninstr - 1; k >= 0; --k) {
        const fg_ew_instr in = a.prog[k];
        if (in.op == FG_EW_INPUT) {
#pragma unroll
            for (int w = 0; w < W; ++w) gin[in.a][w] = S::r(gin[in.a][w] + adj[k][w]);
        } else if (in.op != FG_EW_CONST) {
            const int ia = in.a, ib = (in.op >= FG_EW_ADD && in.op <= FG_EW_DIV) ? in.b : in.a;
#pragma unroll
            for (int w = 0; w < W; ++w)   // the two adjoint slots may be one and the same (x * x): updated in order
                ew_adjoint<DT>(in.op, adj[k][w], v[ia][w], v[ib][w], v[k][w], adj[ia][w], adj[ib][w]);
        }
    }
    for (int k = 0; k < a.ninputs; ++k) {
        if (!a.grads[k]) continue;
        if (a.accumulate) {
            float old[W];
            ldw<DT, W>(a.grads[k], i, old);
#pragma unroll
            for (int w = 0; w < W; ++w) gin[k][w] = S::r(old[w] + gin[k][w]);
        }
        stw<DT, W>(a.grads[k], i, gin[k]);
    }
}

template <int DT>
__global__ void __launch_bounds__(256) chain_bwd_kernel(const __grid_constant__ ChainArgs a) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nv = a.vec ? a.n >> 2 : 0;
    for (uint64_t i = g; i < nv; i += stride) chain_bwd_at<DT, 4>(a, i << 2);
    for (uint64_t i = (nv << 2) + g; i < a.n; i += stride) chain_bwd_at<DT, 1>(a, i);
}

// dst[i] = (type of dst) src[i], round to nearest even; four elements per access when both ends allow it
template <int DS, int DD>
__global__ void __launch_bounds__(256) convert_kernel(const void* __restrict__ src, void* __restrict__ dst, uint64_t n, int vec) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nv = vec ? n >> 2 : 0;
    for (uint64_t i = g; i < nv; i += stride) {
        float v[4];
        Stored<DS>::ld4w(src, i << 2, v);
        Stored<DD>::st4w(dst, i << 2, v);
    }
    for (uint64_t i = (nv << 2) + g; i < n; i += stride) Stored<DD>::st(dst, i, Stored<DS>::ld(src, i));
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
    const bool vec = aligned16(dy) && aligned16(saved) && aligned16(dz);
    const int grid = fg_stream_grid(ctx, vec ? (n + 3) / 4 : n, 256, 8);
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_ELTWISE, (act == FG_ACT_NONE ? 8.0 : 12.0) * n);
    if (vec) act_bwd_kernel<true><<<grid, 256, 0, ctx->stream>>>(n, act, dy, saved, dz);
    else act_bwd_kernel<false><<<grid, 256, 0, ctx->stream>>>(n, act, dy, saved, dz);
    fg_time_end(ctx, tr);
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
    const uint64_t n = (uint64_t)rows * cols;
    const bool vec = (cols & 3u) == 0 && aligned16(z) && aligned16(bias) && aligned16(y);
    const int grid = fg_stream_grid(ctx, vec ? n / 4 : n, 256, 8);
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_ELTWISE, 8.0 * n);
    if (vec) bias_act_kernel<true><<<grid, 256, 0, ctx->stream>>>(rows, cols, z, bias, act, y);
    else bias_act_kernel<false><<<grid, 256, 0, ctx->stream>>>(rows, cols, z, bias, act, y);
    fg_time_end(ctx, tr);
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
    const bool vec = aligned16(pred) && aligned16(target) && aligned16(loss_elem_out) && aligned16(grad_out);
    const int grid = fg_stream_grid(ctx, vec ? (n + 3) / 4 : n, 256, 8);
    float* partials = nullptr;
    if (loss_sum_out) {
        void* p;
        int32_t s = fg_ws_alloc(ctx, (uint64_t)grid * sizeof(float), &p);
        if (s != FG_OK) return s;
        partials = (float*)p;
    }
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_ELTWISE, (8.0 + (loss_elem_out ? 4.0 : 0.0) + (grad_out ? 4.0 : 0.0)) * n);
    if (vec) loss_kernel<MseTerm, true><<<grid, 256, 0, ctx->stream>>>(pred, target, n, grad_scale, loss_elem_out, grad_out, partials);
    else loss_kernel<MseTerm, false><<<grid, 256, 0, ctx->stream>>>(pred, target, n, grad_scale, loss_elem_out, grad_out, partials);
    fg_time_end(ctx, tr);
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
    const bool vec = aligned16(pred) && aligned16(target) && aligned16(loss_elem_out) && aligned16(grad_out);
    const int grid = fg_stream_grid(ctx, vec ? (n + 3) / 4 : n, 256, 8);
    float* partials = nullptr;
    if (loss_sum_out) {
        void* p;
        int32_t s = fg_ws_alloc(ctx, (uint64_t)grid * sizeof(float), &p);
        if (s != FG_OK) return s;
        partials = (float*)p;
    }
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_ELTWISE, (8.0 + (loss_elem_out ? 4.0 : 0.0) + (grad_out ? 4.0 : 0.0)) * n);
    if (vec) loss_kernel<BceTerm, true><<<grid, 256, 0, ctx->stream>>>(pred, target, n, grad_scale, loss_elem_out, grad_out, partials);
    else loss_kernel<BceTerm, false><<<grid, 256, 0, ctx->stream>>>(pred, target, n, grad_scale, loss_elem_out, grad_out, partials);
    fg_time_end(ctx, tr);
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
    // four elements per access when every tensor starts on a boundary of four elements
    const uintptr_t mask = dtype == FG_DTYPE_F32 ? 15u : 7u;
    uintptr_t bits = reinterpret_cast<uintptr_t>(out);
    for (int k = 0; k < ninputs; ++k) bits |= reinterpret_cast<uintptr_t>(a.in[k]);
    for (int k = 0; k < ninstr; ++k) bits |= reinterpret_cast<uintptr_t>(a.saved[k]);
    a.vec = (bits & mask) == 0;
    int grid = fg_stream_grid(ctx, a.vec ? (n + 3) / 4 : n, 256, 8);
    int tensors = ninputs + 1;
    for (int k = 0; k < ninstr; ++k) tensors += a.saved[k] != nullptr;
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_ELTWISE, (dtype == FG_DTYPE_F32 ? 4.0 : 2.0) * tensors * n);
    if (dtype == FG_DTYPE_F32) chain_fwd_kernel<FG_DTYPE_F32><<<grid, 256, 0, ctx->stream>>>(a);
    else if (dtype == FG_DTYPE_F16) chain_fwd_kernel<FG_DTYPE_F16><<<grid, 256, 0, ctx->stream>>>(a);
    else chain_fwd_kernel<FG_DTYPE_BF16><<<grid, 256, 0, ctx->stream>>>(a);
    fg_time_end(ctx, tr);
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
    const uintptr_t mask = dtype == FG_DTYPE_F32 ? 15u : 7u;
    uintptr_t bits = reinterpret_cast<uintptr_t>(seed);
    for (int k = 0; k < ninputs; ++k) bits |= reinterpret_cast<uintptr_t>(a.in[k]) | reinterpret_cast<uintptr_t>(a.grads[k]);
    a.vec = (bits & mask) == 0;
    int grid = fg_stream_grid(ctx, a.vec ? (n + 3) / 4 : n, 256, 8);
    int tensors = ninputs + 1;
    for (int k = 0; k < ninputs; ++k) tensors += a.grads[k] ? 1 + (accumulate != 0) : 0;
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_ELTWISE, (dtype == FG_DTYPE_F32 ? 4.0 : 2.0) * tensors * n);
    if (dtype == FG_DTYPE_F32) chain_bwd_kernel<FG_DTYPE_F32><<<grid, 256, 0, ctx->stream>>>(a);
    else if (dtype == FG_DTYPE_F16) chain_bwd_kernel<FG_DTYPE_F16><<<grid, 256, 0, ctx->stream>>>(a);
    else chain_bwd_kernel<FG_DTYPE_BF16><<<grid, 256, 0, ctx->stream>>>(a);
    fg_time_end(ctx, tr);
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
    const int vec = (reinterpret_cast<uintptr_t>(src) & (src_dtype == FG_DTYPE_F32 ? 15u : 7u)) == 0 &&
                    (reinterpret_cast<uintptr_t>(dst) & (dst_dtype == FG_DTYPE_F32 ? 15u : 7u)) == 0;
    const int grid = fg_stream_grid(ctx, vec ? (n + 3) / 4 : n, 256, 8);
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_ELTWISE, ((src_dtype == FG_DTYPE_F32 ? 4.0 : 2.0) + (dst_dtype == FG_DTYPE_F32 ? 4.0 : 2.0)) * n);
#define FG_CONV(S, D) if (src_dtype == S && dst_dtype == D) convert_kernel<S, D><<<grid, 256, 0, ctx->stream>>>(src, dst, n, vec)
    FG_CONV(FG_DTYPE_F32, FG_DTYPE_F32); FG_CONV(FG_DTYPE_F32, FG_DTYPE_F16); FG_CONV(FG_DTYPE_F32, FG_DTYPE_BF16);
    FG_CONV(FG_DTYPE_F16, FG_DTYPE_F32); FG_CONV(FG_DTYPE_F16, FG_DTYPE_F16); FG_CONV(FG_DTYPE_F16, FG_DTYPE_BF16);
    FG_CONV(FG_DTYPE_BF16, FG_DTYPE_F32); FG_CONV(FG_DTYPE_BF16, FG_DTYPE_F16); FG_CONV(FG_DTYPE_BF16, FG_DTYPE_BF16);
#undef FG_CONV
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}
