// Fused parameter updates: one bandwidth-bound pass over a flat parameter range.
//
// SGD restates STOCHASTIC_GRADIENT_DESCENT (crates/ferrograd-nn/src/optim/basic_optim.rs:3-31,
// learning-rate plumbing crates/fused_gpu/src/dispatch/backend/kernel/optim.rs:119-146):
// scaled = g*lr; w -= scaled; g = 0.  AdamW has no counterpart in the reference.
//
// HBM traffic per parameter: SGD 16 B (read w,g; write w,g), AdamW 28 B (read w,g,m,v;
// write w,m,v) or 32 B when it also zeroes g.  128-bit accesses, grid a multiple of the
// SM count, streaming cache hints (nothing is re-read).
#include "fg_internal.cuh"

namespace {

__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }

__device__ __forceinline__ float sgd_one(float w, float g, float lr, float gs) {
    float gi = (gs == 1.0f) ? g : g * gs;
    return w - __fmul_rn(gi, lr);   // keep the product rounded, as the reference's two statements do
}

// pairs (optional): the bf16 pairs of the updated weights, written in the same pass, so the next GEMM that reads
// them needs no pre-pass (fg_store_pairs4).
template <bool ZERO>
__global__ void __launch_bounds__(256) sgd_kernel(float* __restrict__ w, float* __restrict__ g, uint64_t n,
                                                  float lr, float gs, __nv_bfloat16* __restrict__ pairs, uint64_t pairs_stride) {
    const uint64_t nv = n >> 2;
    float4* w4 = reinterpret_cast<float4*>(w);
    float4* g4 = reinterpret_cast<float4*>(g);
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
        float4 a = ld_stream(w4 + i), b = ld_stream(g4 + i);
        a.x = sgd_one(a.x, b.x, lr, gs);
        a.y = sgd_one(a.y, b.y, lr, gs);
        a.z = sgd_one(a.z, b.z, lr, gs);
        a.w = sgd_one(a.w, b.w, lr, gs);
        st_stream(w4 + i, a);
        if (pairs) fg_store_pairs4(pairs, pairs_stride, i * 4, a);
        if (ZERO) st_stream(g4 + i, make_float4(0.f, 0.f, 0.f, 0.f));
    }
    // tail (n not a multiple of 4)
    for (uint64_t i = (nv << 2) + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        w[i] = sgd_one(w[i], g[i], lr, gs);
        if (pairs) fg_store_pairs1(pairs, pairs_stride, i, w[i]);
        if (ZERO) g[i] = 0.0f;
    }
}

struct AdamConsts {
    float lr, b1, b2, eps, wd, gs;
};

__device__ __forceinline__ void adam_one(float& w, float g, float& m, float& v, const AdamConsts& c,
                                         float inv_bc1, float inv_bc2) {
    float gi = g * c.gs;
    float mi = c.b1 * m + (1.0f - c.b1) * gi;
    float vi = c.b2 * v + (1.0f - c.b2) * (gi * gi);
    float mhat = mi * inv_bc1;
    float vhat = vi * inv_bc2;
    float upd = __fdiv_rn(mhat, sqrtf(vhat) + c.eps) + c.wd * w;
    w = w - c.lr * upd;
    m = mi;
    v = vi;
}

template <bool ZERO>
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ w, float* __restrict__ g,
                                                    float* __restrict__ m, float* __restrict__ v, uint64_t n,
                                                    AdamConsts c, uint32_t step, const uint32_t* __restrict__ step_dev,
                                                    __nv_bfloat16* __restrict__ pairs, uint64_t pairs_stride) {
    const uint32_t t = step_dev ? *step_dev : step;
    const float inv_bc1 = 1.0f / (1.0f - powf(c.b1, (float)t));
    const float inv_bc2 = 1.0f / (1.0f - powf(c.b2, (float)t));
    const uint64_t nv = n >> 2;
    float4* w4 = reinterpret_cast<float4*>(w);
    float4* g4 = reinterpret_cast<float4*>(g);
    float4* m4 = reinterpret_cast<float4*>(m);
    float4* v4 = reinterpret_cast<float4*>(v);
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
        float4 a = ld_stream(w4 + i), b = ld_stream(g4 + i), mm = ld_stream(m4 + i), vv = ld_stream(v4 + i);
        adam_one(a.x, b.x, mm.x, vv.x, c, inv_bc1, inv_bc2);
        adam_one(a.y, b.y, mm.y, vv.y, c, inv_bc1, inv_bc2);
        adam_one(a.z, b.z, mm.z, vv.z, c, inv_bc1, inv_bc2);
        adam_one(a.w, b.w, mm.w, vv.w, c, inv_bc1, inv_bc2);
        st_stream(w4 + i, a);
        if (pairs) fg_store_pairs4(pairs, pairs_stride, i * 4, a);
        st_stream(m4 + i, mm);
        st_stream(v4 + i, vv);
        if (ZERO) st_stream(g4 + i, make_float4(0.f, 0.f, 0.f, 0.f));
    }
    for (uint64_t i = (nv << 2) + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float a = w[i], mm = m[i], vv = v[i];
        adam_one(a, g[i], mm, vv, c, inv_bc1, inv_bc2);
        w[i] = a; m[i] = mm; v[i] = vv;
        if (pairs) fg_store_pairs1(pairs, pairs_stride, i, a);
        if (ZERO) g[i] = 0.0f;
    }
}

}  // namespace

extern "C" {

int32_t fg_sgd_step_paired(fg_ctx* ctx, float* w, float* g, uint64_t n, float lr, float grad_scale, int32_t zero_grad,
                           void* w_pairs, uint64_t pairs_stride) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, w && g, "fg_sgd_step: NULL pointer");
    FG_REQUIRE(ctx, fg_aligned16(w) && fg_aligned16(g), "fg_sgd_step: pointers must be 16-byte aligned");
    FG_REQUIRE(ctx, !w_pairs || (fg_aligned16(w_pairs) && pairs_stride % 8 == 0 && pairs_stride >= n),
               "fg_sgd_step_paired: pairs must be 16-byte aligned with a plane stride that is a multiple of 8 and at least n");
    if (n == 0) return FG_OK;
    int grid = fg_stream_grid(ctx, (n + 3) / 4, 256, 8);
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SGD, ((zero_grad ? 16.0 : 12.0) + (w_pairs ? 4.0 : 0.0)) * n);
    if (zero_grad) sgd_kernel<true><<<grid, 256, 0, ctx->stream>>>(w, g, n, lr, grad_scale, (__nv_bfloat16*)w_pairs, pairs_stride);
    else sgd_kernel<false><<<grid, 256, 0, ctx->stream>>>(w, g, n, lr, grad_scale, (__nv_bfloat16*)w_pairs, pairs_stride);
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t fg_sgd_step(fg_ctx* ctx, float* w, float* g, uint64_t n, float lr, float grad_scale, int32_t zero_grad) {
    return fg_sgd_step_paired(ctx, w, g, n, lr, grad_scale, zero_grad, nullptr, 0);
}

int32_t fg_adamw_step_paired(fg_ctx* ctx, float* w, float* g, float* m, float* v, uint64_t n,
                             const fg_adamw_hyper* h, uint32_t step, const uint32_t* step_dev, float grad_scale,
                             int32_t zero_grad, void* w_pairs, uint64_t pairs_stride) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, w && g && m && v && h, "fg_adamw_step: NULL pointer");
    FG_REQUIRE(ctx, fg_aligned16(w) && fg_aligned16(g) && fg_aligned16(m) && fg_aligned16(v),
               "fg_adamw_step: pointers must be 16-byte aligned");
    FG_REQUIRE(ctx, step_dev != nullptr || step >= 1, "fg_adamw_step: step is 1-based");
    FG_REQUIRE(ctx, h->beta1 >= 0.f && h->beta1 < 1.f && h->beta2 >= 0.f && h->beta2 < 1.f,
               "fg_adamw_step: betas must lie in [0,1)");
    FG_REQUIRE(ctx, !w_pairs || (fg_aligned16(w_pairs) && pairs_stride % 8 == 0 && pairs_stride >= n),
               "fg_adamw_step_paired: pairs must be 16-byte aligned with a plane stride that is a multiple of 8 and at least n");
    if (n == 0) return FG_OK;
    AdamConsts c{h->lr, h->beta1, h->beta2, h->eps, h->weight_decay, grad_scale};
    int grid = fg_stream_grid(ctx, (n + 3) / 4, 256, 8);
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_ADAMW, ((zero_grad ? 32.0 : 28.0) + (w_pairs ? 4.0 : 0.0)) * n);
    if (zero_grad) adamw_kernel<true><<<grid, 256, 0, ctx->stream>>>(w, g, m, v, n, c, step, step_dev, (__nv_bfloat16*)w_pairs, pairs_stride);
    else adamw_kernel<false><<<grid, 256, 0, ctx->stream>>>(w, g, m, v, n, c, step, step_dev, (__nv_bfloat16*)w_pairs, pairs_stride);
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t fg_adamw_step(fg_ctx* ctx, float* w, float* g, float* m, float* v, uint64_t n,
                      const fg_adamw_hyper* h, uint32_t step, const uint32_t* step_dev, float grad_scale,
                      int32_t zero_grad) {
    return fg_adamw_step_paired(ctx, w, g, m, v, n, h, step, step_dev, grad_scale, zero_grad, nullptr, 0);
}

}  // extern "C"
