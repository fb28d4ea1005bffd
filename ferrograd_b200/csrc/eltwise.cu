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
#include <atomic>

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
// out[c] = sum over chunks of part[k][c].  A block covers 32 columns; its eight warps each add every eighth chunk
// (so the chain of dependent loads is an eighth as long), then the eight sums are added in order.
__global__ void __launch_bounds__(256) colsum_fold_kernel(uint32_t cols, uint32_t nchunks,
                                                          const float* __restrict__ part, float* __restrict__ out) {
    __shared__ float red[8][33];
    const uint32_t cx = threadIdx.x & 31u, gy = threadIdx.x >> 5;
    const uint32_t c = blockIdx.x * 32 + cx;
    float s = 0.0f;
    if (c < cols)
        for (uint32_t k = gy; k < nchunks; k += 8) s += part[(size_t)k * cols + c];
    red[gy][cx] = s;
    __syncthreads();
    if (gy == 0 && c < cols) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[w][cx];
        out[c] = t;
    }
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
    uint32_t keep;                  // forward: bit k set = value k is read by an instruction other than k + 1
    uint64_t n;
};

// One instruction on W elements: the op-code is decoded once, the lanes loop inside each case.
#define FG_EW_LANES(expr)                      \
    do {                                       \
        _Pragma("unroll") for (int w = 0; w < W; ++w) { const float xx = x[w], yy = y[w]; (void)yy; r[w] = (expr); } \
    } while (0)
template <int DT, int W>
__device__ __forceinline__ void ew_op(int op, float imm, const float* x, const float* y, float* r) {
    typedef Stored<DT> S;
    switch (op) {
        case FG_EW_CONST: FG_EW_LANES(((void)xx, S::r(imm))); break;
        case FG_EW_ADD: FG_EW_LANES(S::r(xx + yy)); break;
        case FG_EW_SUB: FG_EW_LANES(S::r(xx - yy)); break;
        case FG_EW_MUL: FG_EW_LANES(S::r(xx * yy)); break;
        case FG_EW_DIV: FG_EW_LANES(S::r(__fdiv_rn(xx, yy))); break;
        case FG_EW_NEG: FG_EW_LANES(-xx); break;
        case FG_EW_ABS: FG_EW_LANES(fabsf(xx)); break;
        case FG_EW_EXP: FG_EW_LANES(S::r(expf(xx))); break;
        case FG_EW_LOG: FG_EW_LANES(S::r(logf(xx))); break;
        case FG_EW_TANH: FG_EW_LANES(S::r(tanhf(xx))); break;
        case FG_EW_RELU: FG_EW_LANES(xx > 0.0f ? xx : 0.0f); break;
        case FG_EW_GELU: FG_EW_LANES(S::r(fg_gelu_fwd(xx, nullptr))); break;
        case FG_EW_ELU: FG_EW_LANES(xx >= 0.0f ? xx : S::r(expf(xx) - 1.0f)); break;
        default: FG_EW_LANES(((void)xx, 0.0f)); break;
    }
}
#undef FG_EW_LANES

// Where a chain's intermediate values live.  A program is only known at run time, so its values cannot be
// named registers; as a per-thread array they would sit in local memory (with four lanes per thread the arrays
// overflowed the L1 and the backward kernel ran at a tenth of the HBM rate).  They live in shared memory
// instead: slot s, lane w of thread t is word (s * W + w) * 256 + t, so a warp's access to one slot is 32
// consecutive words.  The value of the previous instruction is also kept in registers, which serves the common
// "operand = the instruction just before" without a shared-memory read.
template <int W> struct Slots {
    float* base;   // this thread's word of slot 0, lane 0
    __device__ __forceinline__ void ld(int slot, float* o) const {
#pragma unroll
        for (int w = 0; w < W; ++w) o[w] = base[(slot * W + w) * 256];
    }
    __device__ __forceinline__ void st(int slot, const float* v) const {
#pragma unroll
        for (int w = 0; w < W; ++w) base[(slot * W + w) * 256] = v[w];
    }
};

__device__ __forceinline__ bool ew_two_operands(int op) { return op >= FG_EW_ADD && op <= FG_EW_DIV; }

// The program on W consecutive elements starting at i; the decode of an instruction is shared by the W lanes.
// On return `last` holds the value of the final instruction; values are stored to their slots when store_all is
// set (the backward pass needs them) or when a later instruction other than the next one reads them.
template <int DT, int W>
__device__ __forceinline__ void ew_forward(const ChainArgs& a, uint64_t i, const Slots<W>& v, bool store_all, bool write_saved,
                                           float* last) {
    for (int k = 0; k < a.ninstr; ++k) {
        const fg_ew_instr in = a.prog[k];
        float r[W];
        if (in.op == FG_EW_INPUT) {
            ldw<DT, W>(a.in[in.a], i, r);
        } else {
            float x[W], y[W];
#pragma unroll
            for (int w = 0; w < W; ++w) x[w] = y[w] = 0.0f;
            if (in.op != FG_EW_CONST) {
                if (in.a == k - 1) {
#pragma unroll
                    for (int w = 0; w < W; ++w) x[w] = last[w];
                } else {
                    v.ld(in.a, x);
                }
                if (ew_two_operands(in.op)) {
                    if (in.b == k - 1) {
#pragma unroll
                        for (int w = 0; w < W; ++w) y[w] = last[w];
                    } else if (in.b == in.a) {
#pragma unroll
                        for (int w = 0; w < W; ++w) y[w] = x[w];
                    } else {
                        v.ld(in.b, y);
                    }
                }
            }
            ew_op<DT, W>(in.op, in.imm, x, y, r);
        }
        if (store_all || (a.keep >> k & 1u)) v.st(k, r);
        if (write_saved && a.saved[k]) stw<DT, W>(a.saved[k], i, r);
#pragma unroll
        for (int w = 0; w < W; ++w) last[w] = r[w];
    }
}

template <int DT, int W>
__device__ __forceinline__ void chain_fwd_at(const ChainArgs& a, uint64_t i, float* smem) {
    const Slots<W> v{smem + threadIdx.x};
    float last[W];
    ew_forward<DT, W>(a, i, v, false, true, last);
    stw<DT, W>(a.out, i, last);
}

template <int DT>
__global__ void __launch_bounds__(256) chain_fwd_kernel(const __grid_constant__ ChainArgs a) {
    extern __shared__ float chain_smem[];
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nv = a.vec ? a.n >> 2 : 0;
    for (uint64_t i = g; i < nv; i += stride) chain_fwd_at<DT, 4>(a, i << 2, chain_smem);
    for (uint64_t i = (nv << 2) + g; i < a.n; i += stride) chain_fwd_at<DT, 1>(a, i, chain_smem);
}

// Adjoint of one instruction on W elements: adds to the adjoints of its operands.  ga and gb may be one and the
// same array (x * x): the two updates then apply in order, as they would on one array element.
#define FG_EW_LANES(stmt)                                                                          \
    do {                                                                                           \
        _Pragma("unroll") for (int w = 0; w < W; ++w) {                                            \
            const float g = gk[w], a_ = va[w], b_ = vb[w], k_ = vk[w];                             \
            (void)a_; (void)b_; (void)k_;                                                          \
            stmt;                                                                                  \
        }                                                                                          \
    } while (0)
template <int DT, int W>
__device__ __forceinline__ void ew_adjoint(int op, const float* gk, const float* va, const float* vb, const float* vk,
                                           float* ga, float* gb) {
    typedef Stored<DT> S;
    switch (op) {
        case FG_EW_ADD: FG_EW_LANES(ga[w] = S::r(ga[w] + g); gb[w] = S::r(gb[w] + g)); break;
        case FG_EW_SUB: FG_EW_LANES(ga[w] = S::r(ga[w] + g); gb[w] = S::r(gb[w] - g)); break;
        case FG_EW_MUL: FG_EW_LANES(ga[w] = S::r(ga[w] + S::r(g * b_)); gb[w] = S::r(gb[w] + S::r(g * a_))); break;
        case FG_EW_DIV: FG_EW_LANES(ga[w] = S::r(ga[w] + S::r(__fdiv_rn(g, b_)));
                                    gb[w] = S::r(gb[w] - S::r(__fdiv_rn(S::r(g * a_), S::r(b_ * b_))))); break;
        case FG_EW_NEG: FG_EW_LANES(ga[w] = S::r(ga[w] - g)); break;
        case FG_EW_ABS: FG_EW_LANES(ga[w] = S::r(ga[w] + (a_ >= 0.0f ? g : -g))); break;
        case FG_EW_EXP: FG_EW_LANES(ga[w] = S::r(ga[w] + S::r(g * k_))); break;
        case FG_EW_LOG: FG_EW_LANES(ga[w] = S::r(ga[w] + S::r(__fdiv_rn(g, a_)))); break;
        case FG_EW_TANH: FG_EW_LANES(ga[w] = S::r(ga[w] + S::r(g * S::r(1.0f - S::r(k_ * k_))))); break;
        case FG_EW_RELU: FG_EW_LANES(ga[w] = S::r(ga[w] + g * fg_act_grad(FG_ACT_RELU, k_))); break;
        case FG_EW_GELU: FG_EW_LANES(ga[w] = S::r(ga[w] + S::r(g * S::r(fg_act_grad(FG_ACT_GELU, a_))))); break;
        case FG_EW_ELU: FG_EW_LANES(ga[w] = S::r(ga[w] + (k_ >= 0.0f ? g : S::r(g * S::r(k_ + 1.0f))))); break;
        default: break;
    }
}
#undef FG_EW_LANES

// Forward values in slots [0, ninstr), adjoints in slots [ninstr, 2 ninstr).  An adjoint slot that nothing has
// added to yet counts as zero without being read (`touched`), so no slot is ever cleared.
template <int DT, int W>
__device__ __forceinline__ void chain_bwd_at(const ChainArgs& a, uint64_t i, float* smem) {
    typedef Stored<DT> S;
    const Slots<W> v{smem + threadIdx.x};
    const Slots<W> adj{smem + threadIdx.x + a.ninstr * W * 256};
    float g[W];
    ew_forward<DT, W>(a, i, v, true, false, g);
    ldw<DT, W>(a.seed, i, g);
    adj.st(a.ninstr - 1, g);
    uint32_t touched = 1u << (a.ninstr - 1);
    for (int k = a.ninstr - 1; k >= 0; --k) {
        const fg_ew_instr in = a.prog[k];
        if (in.op == FG_EW_INPUT || in.op == FG_EW_CONST || !(touched >> k & 1u)) continue;   // nothing flows through
        adj.ld(k, g);
        const bool two = ew_two_operands(in.op);
        const int ia = in.a, ib = two ? in.b : in.a;
        const bool need_a = in.op == FG_EW_MUL || in.op == FG_EW_DIV || in.op == FG_EW_ABS || in.op == FG_EW_LOG ||
                            in.op == FG_EW_GELU;
        const bool need_k = in.op == FG_EW_EXP || in.op == FG_EW_TANH || in.op == FG_EW_RELU || in.op == FG_EW_ELU;
        float va[W], vb[W], vk[W], ga[W], gb[W];
#pragma unroll
        for (int w = 0; w < W; ++w) va[w] = vb[w] = vk[w] = ga[w] = gb[w] = 0.0f;
        if (need_a) v.ld(ia, va);
        if (need_a && two) v.ld(ib, vb);
        if (need_k) v.ld(k, vk);
        if (touched >> ia & 1u) adj.ld(ia, ga);
        if (two && ib != ia) {
            if (touched >> ib & 1u) adj.ld(ib, gb);
            ew_adjoint<DT, W>(in.op, g, va, vb, vk, ga, gb);
            adj.st(ib, gb);
        } else if (two) {
            ew_adjoint<DT, W>(in.op, g, va, vb, vk, ga, ga);
        } else {
            ew_adjoint<DT, W>(in.op, g, va, vb, vk, ga, gb);
        }
        adj.st(ia, ga);
        touched |= (1u << ia) | (1u << ib);
    }
    // the gradient of input j: the adjoints of the instructions that read it, from the last one down
    for (int j = 0; j < a.ninputs; ++j) {
        if (!a.grads[j]) continue;
        float gin[W];
#pragma unroll
        for (int w = 0; w < W; ++w) gin[w] = 0.0f;
        for (int k = a.ninstr - 1; k >= 0; --k) {
            if (a.prog[k].op != FG_EW_INPUT || a.prog[k].a != j || !(touched >> k & 1u)) continue;
            adj.ld(k, g);
#pragma unroll
            for (int w = 0; w < W; ++w) gin[w] = S::r(gin[w] + g[w]);
        }
        if (a.accumulate) {
            ldw<DT, W>(a.grads[j], i, g);
#pragma unroll
            for (int w = 0; w < W; ++w) gin[w] = S::r(g[w] + gin[w]);
        }
        stw<DT, W>(a.grads[j], i, gin);
    }
}

template <int DT>
__global__ void __launch_bounds__(256) chain_bwd_kernel(const __grid_constant__ ChainArgs a) {
    extern __shared__ float chain_smem[];
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nv = a.vec ? a.n >> 2 : 0;
    for (uint64_t i = g; i < nv; i += stride) chain_bwd_at<DT, 4>(a, i << 2, chain_smem);
    for (uint64_t i = (nv << 2) + g; i < a.n; i += stride) chain_bwd_at<DT, 1>(a, i, chain_smem);
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

// The chain kernels may need more than the default 48 KB of dynamic shared memory (24 instructions x four lanes:
// 96 KB forward, 192 KB backward): the limit is raised once per device and kernel.
constexpr int kChainSmemMax = 2 * FG_EW_MAX_INSTR * 4 * 256 * 4;
int32_t chain_smem_attr(fg_ctx* ctx, int dtype, bool bwd) {
    static std::atomic<uint64_t> done[6];
    const int which = (bwd ? 3 : 0) + dtype;
    const uint64_t bit = 1ull << (ctx->device & 63);
    if (done[which].load(std::memory_order_acquire) & bit) return FG_OK;
    cudaError_t e;
    if (!bwd) {
        e = dtype == FG_DTYPE_F32 ? cudaFuncSetAttribute(chain_fwd_kernel<FG_DTYPE_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, kChainSmemMax / 2)
          : dtype == FG_DTYPE_F16 ? cudaFuncSetAttribute(chain_fwd_kernel<FG_DTYPE_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kChainSmemMax / 2)
                                  : cudaFuncSetAttribute(chain_fwd_kernel<FG_DTYPE_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kChainSmemMax / 2);
    } else {
        e = dtype == FG_DTYPE_F32 ? cudaFuncSetAttribute(chain_bwd_kernel<FG_DTYPE_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, kChainSmemMax)
          : dtype == FG_DTYPE_F16 ? cudaFuncSetAttribute(chain_bwd_kernel<FG_DTYPE_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kChainSmemMax)
                                  : cudaFuncSetAttribute(chain_bwd_kernel<FG_DTYPE_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kChainSmemMax);
    }
    if (e != cudaSuccess) return fg_fail_cuda(ctx, FG_ERR_INTERNAL, "cudaFuncSetAttribute(chain kernel)", e);
    done[which].fetch_or(bit, std::memory_order_release);
    return FG_OK;
}
// Resident CTAs per SM that the shared memory allows (of at most eight).
int chain_ctas_per_sm(size_t smem) {
    const size_t fit = (220u * 1024u) / (smem + 1024);
    return (int)(fit < 1 ? 1 : fit > 8 ? 8 : fit);
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
    colsum_fold_kernel<<<(cols + 31) / 32, 256, 0, ctx->stream>>>(cols, nchunks, part, out);
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
    colsum_fold_kernel<<<(cols + 31) / 32, 256, 0, ctx->stream>>>(cols, nchunks, (const float*)part, out);
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
    for (int k = 1; k < ninstr; ++k) {
        const fg_ew_instr& in = prog[k];
        if (in.op == FG_EW_INPUT || in.op == FG_EW_CONST) continue;
        if (in.a != k - 1) a.keep |= 1u << in.a;
        if (in.op >= FG_EW_ADD && in.op <= FG_EW_DIV && in.b != k - 1 && in.b != in.a) a.keep |= 1u << in.b;
    }
    const size_t smem = (size_t)ninstr * (a.vec ? 4 : 1) * 256 * sizeof(float);
    int32_t st = chain_smem_attr(ctx, dtype, false);
    if (st != FG_OK) return st;
    int grid = fg_stream_grid(ctx, a.vec ? (n + 3) / 4 : n, 256, chain_ctas_per_sm(smem));
    int tensors = ninputs + 1;
    for (int k = 0; k < ninstr; ++k) tensors += a.saved[k] != nullptr;
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_ELTWISE, (dtype == FG_DTYPE_F32 ? 4.0 : 2.0) * tensors * n);
    if (dtype == FG_DTYPE_F32) chain_fwd_kernel<FG_DTYPE_F32><<<grid, 256, smem, ctx->stream>>>(a);
    else if (dtype == FG_DTYPE_F16) chain_fwd_kernel<FG_DTYPE_F16><<<grid, 256, smem, ctx->stream>>>(a);
    else chain_fwd_kernel<FG_DTYPE_BF16><<<grid, 256, smem, ctx->stream>>>(a);
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
    const size_t smem = (size_t)2 * ninstr * (a.vec ? 4 : 1) * 256 * sizeof(float);
    int32_t st = chain_smem_attr(ctx, dtype, true);
    if (st != FG_OK) return st;
    int grid = fg_stream_grid(ctx, a.vec ? (n + 3) / 4 : n, 256, chain_ctas_per_sm(smem));
    int tensors = ninputs + 1;
    for (int k = 0; k < ninputs; ++k) tensors += a.grads[k] ? 1 + (accumulate != 0) : 0;
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_ELTWISE, (dtype == FG_DTYPE_F32 ? 4.0 : 2.0) * tensors * n);
    if (dtype == FG_DTYPE_F32) chain_bwd_kernel<FG_DTYPE_F32><<<grid, 256, smem, ctx->stream>>>(a);
    else if (dtype == FG_DTYPE_F16) chain_bwd_kernel<FG_DTYPE_F16><<<grid, 256, smem, ctx->stream>>>(a);
    else chain_bwd_kernel<FG_DTYPE_BF16><<<grid, 256, smem, ctx->stream>>>(a);
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
