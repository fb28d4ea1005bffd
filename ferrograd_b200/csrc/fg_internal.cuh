// Internal definitions shared by the translation units of libferrograd_b200.
#pragma once
#include <nvtx3/nvToolsExt.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/ferrograd_b200.h"

// Device error word bits, set by kernels whose bounded waits ran out.
#define FG_DEVERR_TMA_WAIT 1
#define FG_DEVERR_MMA_WAIT 2
#define FG_DEVERR_EPI_WAIT 4

struct fg_buf {
    void* ptr;
    uint64_t bytes;
    uint64_t version;   // bumped by every entry point that writes the buffer through its handle (fg_upload, fg_copy, ...)
    bool view;          // a window into a larger allocation owned by someone else: fg_free releases the handle only
};

struct fg_plan {
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    uint64_t launches;  // kernels recorded in the graph
    uint64_t ws_generation;   // the scratch arena whose addresses the recorded kernels carry
    fg_ctx* ctx;
    bool has_comm;            // the recording contains an exchange: it holds the communicator until it is destroyed
};

// One timed launch: events on the launching stream around a single kernel.
struct fg_time_rec {
    cudaEvent_t a, b;
    int kind;
    double work;   // flop for GEMMs, bytes for bandwidth-bound kernels
};
#define FG_TIME_MAX_RECS 65536

struct fg_ctx {
    int device;
    cudaStream_t stream;
    bool own_stream;
    cudaStream_t comm_stream;
    cudaEvent_t ev_fork, ev_join;
    bool comm_pending;
    cudaEvent_t ev_ckpt[8];             // exchange checkpoints (fg_comm_checkpoint / fg_comm_wait)
    int comm_reserved_sms;              // SMs the persistent GEMM leaves free while an exchange is in flight
    cudaStream_t copy_stream;           // host->device prefetches that overlap compute
    cudaEvent_t ev_copy_done, ev_main_mark;
    bool mark_valid;
    char err[512];
    uint64_t launches;          // kernels launched so far (eager + replayed plans)
    bool capturing;
    uint64_t capture_launches;  // kernels recorded since fg_plan_begin
    // Scratch arena: operand planes of the tensor-core GEMM, reduction partials.
    char* ws;
    uint64_t ws_bytes;
    uint64_t ws_used;           // bump pointer, reset at the start of every entry point
    int* dev_status;            // device error word (see FG_DEVERR_*)
    void* tmap_encode;          // cuTensorMapEncodeTiled, resolved at context creation
    int sm_count;
    // Optional per-kernel timing (eager mode only)
    bool timing_on;
    fg_time_rec* time_recs;
    int time_count;       // records in use
    int time_created;     // records whose events exist
    // NCCL (loaded at run time)
    void* nccl_lib;
    void* comm;
    int nranks, rank;
    // Options (fg_ctx_set_option); the FG_* environment variables give their initial values once, at creation.
    int opt_tile_group;         // pair kernel: tile rows per group of the tile order (0: the default, eight)
    int opt_tile_pair;          // -1: chosen per shape; 1: CTA pairs whenever the shape allows; 0: opt_tile_bn x opt_tile_bk
    int opt_tile_bn, opt_tile_bk;
    bool opt_split_k;           // split-K tail of the pair kernel
    bool opt_pairs;             // multiply f32 tensors as they lie (bf16 pairs) where the shape allows
    int opt_exec_plans;         // the graph engine records each dispatch as a CUDA graph: 1 always, 0 never, -1 when launch-bound
    int opt_comm_max_ctas;      // CTAs the communicator may use (fg_comm_init)
    uint64_t opt_min_exchange;  // elements: the graph engine starts an exchange once this much is complete
    uint64_t ws_generation;     // bumped whenever the scratch arena is reallocated
    bool capture_has_comm;      // an exchange was recorded since fg_plan_begin
    int comm_plans;             // live plans that contain an exchange
};

inline int32_t fg_fail(fg_ctx* ctx, int32_t code, const char* msg) {
    if (ctx) {
        strncpy(ctx->err, msg, sizeof(ctx->err) - 1);
        ctx->err[sizeof(ctx->err) - 1] = 0;
    }
    return code;
}

inline int32_t fg_fail_cuda(fg_ctx* ctx, int32_t code, const char* what, cudaError_t e) {
    if (ctx) snprintf(ctx->err, sizeof(ctx->err), "%s: %s", what, cudaGetErrorString(e));
    return code;
}

#define FG_REQUIRE(ctx, cond, msg) \
    do { if (!(cond)) return fg_fail((ctx), FG_ERR_INVALID_ARGUMENT, msg); } while (0)

#define FG_CUDA(ctx, code, call) \
    do { cudaError_t _e = (call); if (_e != cudaSuccess) return fg_fail_cuda((ctx), (code), #call, _e); } while (0)

// Every compute entry point starts with this: valid context, right device, fresh scratch.
#define FG_ENTER(ctx) \
    do { if (!(ctx)) return FG_ERR_NOT_INITIALIZED; \
         FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice((ctx)->device)); \
         (ctx)->ws_used = 0; } while (0)

// A named range on the calling host thread for timeline tools (NVTX, header-only: without a tool attached a
// range costs one pointer test).  The four dispatches of a training step, plan replays and gradient exchanges
// carry one each.
struct FgRange {
    explicit FgRange(const char* name) { nvtxRangePushA(name); }
    ~FgRange() { nvtxRangePop(); }
    FgRange(const FgRange&) = delete;
    FgRange& operator=(const FgRange&) = delete;
};

// After a kernel launch: count it and surface launch-configuration errors.
#define FG_LAUNCHED(ctx) \
    do { cudaError_t _e = cudaGetLastError(); \
         if (_e != cudaSuccess) return fg_fail_cuda((ctx), FG_ERR_LAUNCH_FAILURE, "kernel launch", _e); \
         if ((ctx)->capturing) (ctx)->capture_launches++; else (ctx)->launches++; } while (0)

// Brackets one kernel launch with events when timing is enabled (never while capturing).
inline fg_time_rec* fg_time_begin(fg_ctx* ctx, int kind, double work) {
    if (!ctx->timing_on || ctx->capturing || !ctx->time_recs || ctx->time_count >= FG_TIME_MAX_RECS) return nullptr;
    fg_time_rec* r = &ctx->time_recs[ctx->time_count];
    if (ctx->time_count >= ctx->time_created) {
        if (cudaEventCreate(&r->a) != cudaSuccess || cudaEventCreate(&r->b) != cudaSuccess) return nullptr;
        ctx->time_created = ctx->time_count + 1;
    }
    r->kind = kind;
    r->work = work;
    cudaEventRecord(r->a, ctx->stream);
    ctx->time_count++;
    return r;
}
inline void fg_time_end(fg_ctx* ctx, fg_time_rec* r) {
    if (r) cudaEventRecord(r->b, ctx->stream);
}

inline bool fg_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Returns a 256-byte aligned slice of the scratch arena, growing it when allowed.
int32_t fg_ws_alloc(fg_ctx* ctx, uint64_t bytes, void** out);
// Room for `bytes` more in the arena (grows it when nothing has been carved yet for this operation).
int32_t fg_ws_ensure(fg_ctx* ctx, uint64_t bytes);

// Grid for a bandwidth-bound grid-stride kernel: a multiple of the SM count.
inline int fg_stream_grid(const fg_ctx* ctx, uint64_t work_items, int threads, int per_sm) {
    uint64_t need = (work_items + threads - 1) / threads;
    uint64_t cap = (uint64_t)ctx->sm_count * per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

// ---- activation maths shared by the GEMM epilogue and the elementwise kernels ----
// Constants of the reference's tanh-approximated GELU (op/unary.rs:493-494).
#define FG_GELU_A 0.044715f
#define FG_GELU_B 0.7978846f

__device__ __forceinline__ float fg_gelu_fwd(float x, float* t_out) {
    float xx = x * x;
    float u = FG_GELU_B * (x + (xx * x) * FG_GELU_A);
    float t = tanhf(u);
    if (t_out) *t_out = t;
    return (0.5f * x) * (1.0f + t);
}

__device__ __forceinline__ float fg_act_fwd(int act, float z) {
    switch (act) {
        case FG_ACT_RELU: return z > 0.0f ? z : 0.0f;
        case FG_ACT_TANH: return tanhf(z);
        case FG_ACT_GELU: return fg_gelu_fwd(z, nullptr);
        default: return z;
    }
}

// d act / d z given the saved value (output y for relu/tanh, pre-activation z for gelu).
__device__ __forceinline__ float fg_act_grad(int act, float saved) {
    switch (act) {
        case FG_ACT_RELU: return saved > 0.0f ? 1.0f : 0.0f;
        case FG_ACT_TANH: return 1.0f - saved * saved;
        case FG_ACT_GELU: {
            float t;
            fg_gelu_fwd(saved, &t);
            float du = FG_GELU_B * (1.0f + (FG_GELU_A * 3.0f) * (saved * saved));
            return 0.5f * ((1.0f + t) + (1.0f - t * t) * (saved * du));
        }
        default: return 1.0f;
    }
}

// ---- the same activations for GEMM epilogues ----
// An epilogue runs while the tensor core is already on the next tile and must be done before the two
// accumulators it can run ahead by are full; eight warps do it, so it is bound by instruction issue and its
// arithmetic is kept short: tanh through one exponential and one reciprocal (both the hardware approximations,
// 1-2 ulp), 0.5*(1 + tanh(u)) = 1 / (1 + exp(-2u)), polynomials as explicit fused multiply-adds.  For GELU this
// form has no cancellation; results agree with the libm forms above to a few 1e-7 of the output's scale.
__device__ __forceinline__ float fg_ex2_fast(float a) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a)); return r; }
__device__ __forceinline__ float fg_rcp_fast(float a) { float r; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a)); return r; }
// 1 / (1 + exp(-a)) with a given pre-multiplied by -log2(e): sigmoid(a) = 1 / (1 + 2^(a * -log2 e)).
__device__ __forceinline__ float fg_sigmoid_l2(float a_neg_l2) { return fg_rcp_fast(1.0f + fg_ex2_fast(a_neg_l2)); }
#define FG_NEG_LOG2E (-1.4426950408889634f)
__device__ __forceinline__ float fg_sigmoid_fast(float a) { return fg_sigmoid_l2(a * FG_NEG_LOG2E); }
// -log2(e) * 2 * FG_GELU_B * (x + FG_GELU_A x^3) = x * (c1 + c3 x^2)
#define FG_GELU_C1 (FG_NEG_LOG2E * 2.0f * FG_GELU_B)
#define FG_GELU_C3 (FG_NEG_LOG2E * 2.0f * FG_GELU_B * FG_GELU_A)

__device__ __forceinline__ float fg_act_fwd_fast(int act, float z) {
    switch (act) {
        case FG_ACT_RELU: return z > 0.0f ? z : 0.0f;
        case FG_ACT_TANH: return __fmaf_rn(2.0f, fg_sigmoid_l2(z * (2.0f * FG_NEG_LOG2E)), -1.0f);
        case FG_ACT_GELU: return z * fg_sigmoid_l2(z * __fmaf_rn(z * z, FG_GELU_C3, FG_GELU_C1));
        default: return z;
    }
}

__device__ __forceinline__ float fg_act_grad_fast(int act, float saved) {
    switch (act) {
        case FG_ACT_RELU: return saved > 0.0f ? 1.0f : 0.0f;
        case FG_ACT_TANH: return __fmaf_rn(-saved, saved, 1.0f);
        case FG_ACT_GELU: {
            // s = 0.5*(1 + tanh(u)); 1 - tanh(u)^2 = 4*s*(1 - s); gelu' = s + 0.5*x*(1 - tanh^2)*du/dx
            const float xx = saved * saved;
            const float s = fg_sigmoid_l2(saved * __fmaf_rn(xx, FG_GELU_C3, FG_GELU_C1));
            const float du = __fmaf_rn(xx, FG_GELU_B * FG_GELU_A * 3.0f, FG_GELU_B);
            return __fmaf_rn((saved + saved) * (s * (1.0f - s)), du, s);
        }
        default: return 1.0f;
    }
}

// Compact forms of the two functions above for code that is unrolled or must stay small: one uniform branch
// separates the activations that need an exponential from those that do not, and selects do the rest (instead
// of a switch whose every case is expanded at every call site).
__device__ __forceinline__ float fg_act_fwd_sel(int act, float z) {
    if (act >= FG_ACT_TANH) {
        const float arg = act == FG_ACT_TANH ? z * (2.0f * FG_NEG_LOG2E) : z * __fmaf_rn(z * z, FG_GELU_C3, FG_GELU_C1);
        const float s = fg_sigmoid_l2(arg);
        return act == FG_ACT_TANH ? __fmaf_rn(2.0f, s, -1.0f) : z * s;
    }
    return act == FG_ACT_RELU ? fmaxf(z, 0.0f) : z;
}
__device__ __forceinline__ float fg_act_grad_sel(int act, float saved) {
    const float xx = saved * saved;
    if (act == FG_ACT_GELU) {
        const float s = fg_sigmoid_l2(saved * __fmaf_rn(xx, FG_GELU_C3, FG_GELU_C1));
        const float du = __fmaf_rn(xx, FG_GELU_B * FG_GELU_A * 3.0f, FG_GELU_B);
        return __fmaf_rn((saved + saved) * (s * (1.0f - s)), du, s);
    }
    const float relu = saved > 0.0f ? 1.0f : 0.0f;
    return act == FG_ACT_TANH ? 1.0f - xx : act == FG_ACT_RELU ? relu : 1.0f;
}

// ---- bf16 pairs of an f32 tensor (operands of the default GEMM mode) ----
// A kind::tf32 MMA that reads an f32 word from shared memory uses sign, exponent and the top 10 mantissa
// bits: it sees trunc(x).  The pairs carry what the split product needs beside that: plane 0 = bf16(x),
// plane 1 = bf16(x - trunc(x)).  Whoever writes a tensor writes its pairs in the same pass.
__device__ __forceinline__ float fg_trunc_tf32(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
__device__ __forceinline__ void fg_store_pairs4(__nv_bfloat16* pairs, uint64_t plane_stride, size_t idx, float4 v) {
    const __nv_bfloat162 h0 = __floats2bfloat162_rn(v.x, v.y), h1 = __floats2bfloat162_rn(v.z, v.w);
    const __nv_bfloat162 l0 = __floats2bfloat162_rn(v.x - fg_trunc_tf32(v.x), v.y - fg_trunc_tf32(v.y));
    const __nv_bfloat162 l1 = __floats2bfloat162_rn(v.z - fg_trunc_tf32(v.z), v.w - fg_trunc_tf32(v.w));
    uint2 h, l;
    h.x = *reinterpret_cast<const uint32_t*>(&h0); h.y = *reinterpret_cast<const uint32_t*>(&h1);
    l.x = *reinterpret_cast<const uint32_t*>(&l0); l.y = *reinterpret_cast<const uint32_t*>(&l1);
    *reinterpret_cast<uint2*>(pairs + idx) = h;
    *reinterpret_cast<uint2*>(pairs + plane_stride + idx) = l;
}
__device__ __forceinline__ void fg_store_pairs1(__nv_bfloat16* pairs, uint64_t plane_stride, size_t idx, float v) {
    pairs[idx] = __float2bfloat16_rn(v);
    pairs[plane_stride + idx] = __float2bfloat16_rn(v - fg_trunc_tf32(v));
}

// ---- internal launchers used across translation units ----
int32_t fg_gemm_simt_launch(fg_ctx* ctx, int transA, int transB, uint32_t M, uint32_t N, uint32_t K,
                            const float* A, const float* B, float* C, const float* bias, int act,
                            float* preact_out);
// The same for `batch` matrices in one launch (grid z = matrix; strides in elements).
int32_t fg_gemm_simt_batched_launch(fg_ctx* ctx, int transA, int transB, uint32_t batch, uint32_t M, uint32_t N, uint32_t K,
                                    const float* A, uint64_t sA, const float* B, uint64_t sB, float* C, uint64_t sC,
                                    const float* bias, int act, float* preact_out);
uint64_t fg_gemm_skinny_scratch_bytes(uint32_t M, uint32_t N, uint32_t K);   // enough for any one skinny launch
int32_t fg_gemm_skinny_n_launch(fg_ctx* ctx, uint32_t M, uint32_t N, uint32_t K, const float* A, const float* B, float* C,
                                const float* bias, int act, float* preact_out);
// Optional extras of the dA kernel: dA = (dZ·Bᵀ) * act'(mul_saved), its bf16 pairs, and partial column sums
// (the partials of the bias gradient of the layer below): room for [ceil(M/32)][K]; the launch reports how many
// rows it wrote.
struct fg_skinny_extras {
    const float* mul_saved;
    int mul_act;
    __nv_bfloat16* pairs;
    uint64_t pairs_stride;
    float* colsum_part;
};
int32_t fg_gemm_skinny_nt_launch(fg_ctx* ctx, uint32_t M, uint32_t K, uint32_t N, const float* dZ, const float* B,
                                 float* dA, const fg_skinny_extras* extras = nullptr, uint32_t* colsum_rows = nullptr);
int32_t fg_gemm_skinny_tn_launch(fg_ctx* ctx, uint32_t M, uint32_t Kd, uint32_t N, const float* A, const float* dZ,
                                 float* dB);
int32_t fg_convert_launch(fg_ctx* ctx, const void* src, int src_dtype, void* dst, int dst_dtype, uint64_t n);
int32_t fg_act_bwd_launch(fg_ctx* ctx, uint64_t n, int act, const float* dy, const float* saved, float* dz);
int32_t fg_colsum_launch(fg_ctx* ctx, uint32_t rows, uint32_t cols, const float* x, float* out);
int32_t fg_colsum_fold_launch(fg_ctx* ctx, uint32_t cols, uint32_t nchunks, const float* part, float* out);
