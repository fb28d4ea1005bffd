// fg_mse_loss_grad_noalloc: the MSE loss + gradient with its reduction scratch in a
// statically allocated device array, for callers that must not trigger device allocations.
//
// fg_mse_loss_grad sums the per-element losses in two stages and keeps the per-CTA partial
// sums in the context's scratch arena, which is created (cudaMalloc) on first use and
// regrown when a later call needs more.  Some hosts cannot live with that: a training
// process that has handed the whole GPU to its own memory pool leaves nothing for the
// driver to give out, so a late cudaMalloc fails; a service with a hard latency bound cannot
// absorb the device-wide synchronisation an allocation implies; and a job that has been
// sized to a fixed memory budget wants no allocation whose failure shows up hours into a
// run.  This variant needs no allocation at any time: the partial sums live in the
// file-scope array below, which every GPU that loads the library holds (16 KiB) until the
// process exits.  There is no counterpart in the reference.
//
// Same arithmetic per element as fg_mse_loss_grad (loss = d*d, grad = 2*d*scale).  The sum
// is formed differently: every CTA owns a fixed run of 65,536 consecutive elements, so the
// summation order depends only on n, not on the GPU's SM count; the result agrees with
// fg_mse_loss_grad to rounding (the tests hold it to 1e-5).
//
// Limits and sharing rules:
//   * n <= FG_MSE_NOALLOC_MAX_N (4096 partial sums x 65,536 elements = 268,435,456);
//     larger inputs are refused with FG_ERR_INVALID_ARGUMENT before anything is launched.
//   * The device address of the array is looked up with cudaGetSymbolAddress once per
//     device, by the first call made with that device's context.  Make that first call
//     outside any stream capture; inside a recording started with fg_plan_begin it is refused
//     (FG_ERR_INCONSISTENT_CAPTURE) rather than attempted.
//   * All calls on one GPU share the array.  Each call overwrites the entries it uses before
//     reading them, so nothing has to be cleared between calls, but two calls that run
//     concurrently on the same GPU (different streams or contexts) race on it.
#include <atomic>

#include "fg_internal.cuh"

#define FG_MSE_NOALLOC_CHUNK 65536u
#define FG_MSE_NOALLOC_MAX_PARTIALS 4096u
static_assert(FG_MSE_NOALLOC_MAX_N == (uint64_t)FG_MSE_NOALLOC_CHUNK * FG_MSE_NOALLOC_MAX_PARTIALS,
              "the limit declared in the header must match the static scratch");

// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to pass on.
static __device__ __align__(256) float g_mse_partials[FG_MSE_NOALLOC_MAX_PARTIALS];

namespace {

constexpr int kMaxDevices = 64;
// Device address of g_mse_partials, per device.  Several host threads (each with its own context) may make the
// first call on one device at the same time; they all look up and store the same value.
std::atomic<float*> s_partials_addr[kMaxDevices];

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(256) mse_chunk_kernel(const float* __restrict__ pred,
                                                        const float* __restrict__ target, uint64_t n, float scale,
                                                        float* __restrict__ loss_elem, float* __restrict__ grad,
                                                        float* __restrict__ partials) {
    __shared__ float red[8];
    const uint64_t base = (uint64_t)blockIdx.x * FG_MSE_NOALLOC_CHUNK;
    const uint64_t end = min(n, base + FG_MSE_NOALLOC_CHUNK);
    float s = 0.0f;
    for (uint64_t i = base + threadIdx.x; i < end; i += 256) {
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
            partials[blockIdx.x] = t;     // every entry that the fold reads is written here first
        }
    }
}

__global__ void __launch_bounds__(256) mse_fold_kernel(const float* __restrict__ partials, uint32_t nparts,
                                                       float* __restrict__ out) {
    __shared__ float red[8];
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < nparts; i += 256) s += partials[i];
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < 8; ++w) t += red[w];
        *out = t;
    }
}

// One-time set-up per device (that device must be current): resolve the array's device address.
int32_t partials_address(fg_ctx* ctx, float** out) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices)
        return fg_fail(ctx, FG_ERR_INVALID_DEVICE, "fg_mse_loss_grad_noalloc: device index out of range");
    float* p = s_partials_addr[ctx->device].load(std::memory_order_acquire);
    if (!p) {
        // The look-up is a runtime call that does not belong inside a stream capture: refuse instead of risking
        // the caller's recording.
        if (ctx->capturing)
            return fg_fail(ctx, FG_ERR_INCONSISTENT_CAPTURE,
                           "fg_mse_loss_grad_noalloc: the first call on a device must be made outside a recording");
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_mse_partials);
        if (e != cudaSuccess || !p)
            return fg_fail_cuda(ctx, FG_ERR_INTERNAL, "cudaGetSymbolAddress(g_mse_partials)", e);
        s_partials_addr[ctx->device].store(p, std::memory_order_release);
    }
    *out = p;
    return FG_OK;
}

}  // namespace

extern "C" int32_t fg_mse_loss_grad_noalloc(fg_ctx* ctx, const float* pred, const float* target, uint64_t n,
                                            float grad_scale, float* loss_elem_out, float* loss_sum_out,
                                            float* grad_out) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, pred && target, "fg_mse_loss_grad_noalloc: NULL pointer");
    FG_REQUIRE(ctx, loss_elem_out || loss_sum_out || grad_out, "fg_mse_loss_grad_noalloc: no output requested");
    FG_REQUIRE(ctx, n <= FG_MSE_NOALLOC_MAX_N,
               "fg_mse_loss_grad_noalloc: n exceeds 268,435,456 elements (the static scratch holds 4096 partial sums "
               "of 65,536 elements each); use fg_mse_loss_grad for larger inputs");
    if (n == 0) {
        if (loss_sum_out) FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY, cudaMemsetAsync(loss_sum_out, 0, 4, ctx->stream));
        return FG_OK;
    }
    float* partials = nullptr;
    if (loss_sum_out) {
        int32_t s = partials_address(ctx, &partials);
        if (s != FG_OK) return s;
    }
    const uint32_t nparts = (uint32_t)((n + FG_MSE_NOALLOC_CHUNK - 1) / FG_MSE_NOALLOC_CHUNK);
    mse_chunk_kernel<<<nparts, 256, 0, ctx->stream>>>(pred, target, n, grad_scale, loss_elem_out, grad_out, partials);
    FG_LAUNCHED(ctx);
    if (loss_sum_out) {
        mse_fold_kernel<<<1, 256, 0, ctx->stream>>>(partials, nparts, loss_sum_out);
        FG_LAUNCHED(ctx);
    }
    return FG_OK;
}
