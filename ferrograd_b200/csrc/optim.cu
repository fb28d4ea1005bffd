// Fused parameter updates: one bandwidth-bound pass over a flat parameter range.
//
// SGD restates STOCHASTIC_GRADIENT_DESCENT (crates/ferrograd-nn/src/optim/basic_optim.rs:3-31,
// learning-rate plumbing crates/fused_gpu/src/dispatch/backend/kernel/optim.rs:119-146):
// scaled = g*lr; w -= scaled; g = 0.  AdamW has no counterpart in the reference.
//
// HBM traffic per parameter: SGD 16 B (read w,g; write w,g), AdamW 28 B (read w,g,m,v;
// write w,m,v) or 32 B when it also zeroes g.  128-bit accesses, grid a multiple of the
// SM count, streaming cache hints (nothing is re-read).
#include <algorithm>

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

// ---- several tensors in one launch ----
// A model whose weights are separate tensors (the reference's layout) would otherwise pay one launch per tensor,
// most of them tiny (biases).  The tensors are cut into chunks of kMultiChunk elements; chunk c belongs to the
// tensor t with first_chunk[t] <= c < first_chunk[t + 1]; CTAs stride over the chunks.
constexpr int kMultiMax = 16;
constexpr uint32_t kMultiChunk = 8192;
struct MultiArgs {
    float* w[kMultiMax];
    float* g[kMultiMax];
    float* m[kMultiMax];
    float* v[kMultiMax];
    __nv_bfloat16* pairs[kMultiMax];
    uint64_t pairs_stride[kMultiMax];
    uint64_t n[kMultiMax];
    uint32_t first_chunk[kMultiMax + 1];
    int count;
};

template <bool ADAM, bool ZERO>
__global__ void __launch_bounds__(256) update_multi_kernel(const __grid_constant__ MultiArgs a, AdamConsts c, uint32_t step,
                                                           const uint32_t* __restrict__ step_dev) {
    float inv_bc1 = 1.0f, inv_bc2 = 1.0f;
    if (ADAM) {
        const uint32_t t = step_dev ? *step_dev : step;
        inv_bc1 = 1.0f / (1.0f - powf(c.b1, (float)t));
        inv_bc2 = 1.0f / (1.0f - powf(c.b2, (float)t));
    }
    const uint32_t nchunks = a.first_chunk[a.count];
    for (uint32_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
        int t = 0;
        while (t + 1 < a.count && ch >= a.first_chunk[t + 1]) ++t;
        const uint64_t base = (uint64_t)(ch - a.first_chunk[t]) * kMultiChunk;
        const uint64_t n = a.n[t], end = min(n, base + kMultiChunk);
        float* const w = a.w[t];
        float* const g = a.g[t];
        float* const m = a.m[t];
        float* const v = a.v[t];
        __nv_bfloat16* const pairs = a.pairs[t];
        const uint64_t ps = a.pairs_stride[t];
        const uint64_t vend = base + ((end - base) & ~uint64_t(3));        // base is a multiple of 4
        for (uint64_t i = base + (uint64_t)threadIdx.x * 4; i < vend; i += 1024) {
            float4 ww = ld_stream(reinterpret_cast<const float4*>(w + i)), gg = ld_stream(reinterpret_cast<const float4*>(g + i));
            if (ADAM) {
                float4 mm = ld_stream(reinterpret_cast<const float4*>(m + i)), vv = ld_stream(reinterpret_cast<const float4*>(v + i));
                adam_one(ww.x, gg.x, mm.x, vv.x, c, inv_bc1, inv_bc2);
                adam_one(ww.y, gg.y, mm.y, vv.y, c, inv_bc1, inv_bc2);
                adam_one(ww.z, gg.z, mm.z, vv.z, c, inv_bc1, inv_bc2);
                adam_one(ww.w, gg.w, mm.w, vv.w, c, inv_bc1, inv_bc2);
                st_stream(reinterpret_cast<float4*>(m + i), mm);
                st_stream(reinterpret_cast<float4*>(v + i), vv);
            } else {
                ww.x = sgd_one(ww.x, gg.x, c.lr, c.gs); ww.y = sgd_one(ww.y, gg.y, c.lr, c.gs);
                ww.z = sgd_one(ww.z, gg.z, c.lr, c.gs); ww.w = sgd_one(ww.w, gg.w, c.lr, c.gs);
            }
            st_stream(reinterpret_cast<float4*>(w + i), ww);
            if (pairs) fg_store_pairs4(pairs, ps, i, ww);
            if (ZERO) st_stream(reinterpret_cast<float4*>(g + i), make_float4(0.f, 0.f, 0.f, 0.f));
        }
        for (uint64_t i = vend + threadIdx.x; i < end; i += 256) {
            float ww = w[i];
            if (ADAM) {
                float mm = m[i], vv = v[i];
                adam_one(ww, g[i], mm, vv, c, inv_bc1, inv_bc2);
                m[i] = mm; v[i] = vv;
            } else {
                ww = sgd_one(ww, g[i], c.lr, c.gs);
            }
            w[i] = ww;
            if (pairs) fg_store_pairs1(pairs, ps, i, ww);
            if (ZERO) g[i] = 0.0f;
        }
    }
}

int32_t update_multi(fg_ctx* ctx, bool adam, const fg_update_tensor* t, uint32_t count, AdamConsts c, uint32_t step,
                     const uint32_t* step_dev, int32_t zero_grad, const char* who) {
    for (uint32_t k = 0; k < count; ++k) {
        if (!t[k].w || !t[k].g || (adam && (!t[k].m || !t[k].v))) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, who);
        if (!fg_aligned16(t[k].w) || !fg_aligned16(t[k].g) || (adam && (!fg_aligned16(t[k].m) || !fg_aligned16(t[k].v))) ||
            (t[k].w_pairs && (!fg_aligned16(t[k].w_pairs) || t[k].pairs_stride % 8 != 0 || t[k].pairs_stride < t[k].n)))
            return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, who);
    }
    for (uint32_t k0 = 0; k0 < count; k0 += kMultiMax) {
        MultiArgs a;
        memset(&a, 0, sizeof(a));
        double bytes = 0.0;
        uint64_t chunks = 0;
        int cnt = 0;
        for (uint32_t k = k0; k < count && cnt < kMultiMax; ++k) {
            if (t[k].n == 0) continue;
            a.w[cnt] = t[k].w; a.g[cnt] = t[k].g; a.m[cnt] = t[k].m; a.v[cnt] = t[k].v;
            a.pairs[cnt] = (__nv_bfloat16*)t[k].w_pairs; a.pairs_stride[cnt] = t[k].pairs_stride; a.n[cnt] = t[k].n;
            a.first_chunk[cnt] = (uint32_t)chunks;
            chunks += (t[k].n + kMultiChunk - 1) / kMultiChunk;
            bytes += ((adam ? 28.0 : 12.0) + (zero_grad ? 4.0 : 0.0) + (t[k].w_pairs ? 4.0 : 0.0)) * (double)t[k].n;
            ++cnt;
        }
        if (cnt == 0) continue;
        if (chunks >= (1ull << 32)) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, who);
        a.first_chunk[cnt] = (uint32_t)chunks;
        a.count = cnt;
        const int grid = (int)std::min<uint64_t>(chunks, (uint64_t)ctx->sm_count * 8);
        fg_time_rec* tr = fg_time_begin(ctx, adam ? FG_KERNEL_ADAMW : FG_KERNEL_SGD, bytes);
        if (adam) {
            if (zero_grad) update_multi_kernel<true, true><<<grid, 256, 0, ctx->stream>>>(a, c, step, step_dev);
            else update_multi_kernel<true, false><<<grid, 256, 0, ctx->stream>>>(a, c, step, step_dev);
        } else {
            if (zero_grad) update_multi_kernel<false, true><<<grid, 256, 0, ctx->stream>>>(a, c, step, step_dev);
            else update_multi_kernel<false, false><<<grid, 256, 0, ctx->stream>>>(a, c, step, step_dev);
        }
        fg_time_end(ctx, tr);
        FG_LAUNCHED(ctx);
    }
    return FG_OK;
}

}  // namespace

extern "C" {

int32_t fg_adamw_step_multi(fg_ctx* ctx, const fg_update_tensor* tensors, uint32_t count, const fg_adamw_hyper* h, uint32_t step,
                            const uint32_t* step_dev, float grad_scale, int32_t zero_grad) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, (tensors || count == 0) && h, "fg_adamw_step_multi: NULL pointer");
    FG_REQUIRE(ctx, step_dev != nullptr || step >= 1, "fg_adamw_step_multi: step is 1-based");
    FG_REQUIRE(ctx, h->beta1 >= 0.f && h->beta1 < 1.f && h->beta2 >= 0.f && h->beta2 < 1.f,
               "fg_adamw_step_multi: betas must lie in [0,1)");
    return update_multi(ctx, true, tensors, count, AdamConsts{h->lr, h->beta1, h->beta2, h->eps, h->weight_decay, grad_scale}, step,
                        step_dev, zero_grad, "fg_adamw_step_multi: a tensor is NULL, misaligned, or its pairs do not cover it");
}

int32_t fg_sgd_step_multi(fg_ctx* ctx, const fg_update_tensor* tensors, uint32_t count, float lr, float grad_scale,
                          int32_t zero_grad) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, tensors || count == 0, "fg_sgd_step_multi: NULL pointer");
    return update_multi(ctx, false, tensors, count, AdamConsts{lr, 0.f, 0.f, 0.f, 0.f, grad_scale}, 1, nullptr, zero_grad,
                        "fg_sgd_step_multi: a tensor is NULL, misaligned, or its pairs do not cover it");
}

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
