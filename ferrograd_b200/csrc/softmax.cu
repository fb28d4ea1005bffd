// Row softmax, its backward, and the fused softmax + cross-entropy forward/backward.
//
// Semantics: softmax forward crates/ferrograd-nn/src/op/softmax.rs:112-446 (row max,
// e = exp(x - max), sum, y = e * (1/sum)); backward :448-688 (dx = y * (dy - sum(dy*y)));
// CROSS_ENTROPY crates/ferrograd-nn/src/loss/basic_loss.rs:91-133 (loss = -log p at the
// label column, grad = p - onehot).  The reference runs three kernels with about five
// passes over the matrix; the fused kernel here reads the logits from HBM once and
// writes dlogits once.
//
// Two kernels serve the fused path:
//   * rowreg: one persistent 1024-thread CTA per SM.  The row being worked on lives
//     in registers (8 x float4 per thread, up to 32768 columns) while the NEXT row is
//     already streaming into shared memory with bulk async copies (cp.async.bulk,
//     completion on an mbarrier), so HBM reads never wait for the exp/reduce/store
//     phases.  HBM traffic: rows*cols*4 B read + rows*cols*4 B written.
//   * stream: any shape and alignment; one CTA per row, re-reads the row (L1/L2 hits
//     for the row sizes it is used for).
#include <math_constants.h>

#include <atomic>

#include "fg_internal.cuh"

namespace {

constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

// Block-wide reductions over up to 32 warps; `red` is 32 floats of shared memory.
// Every thread gets the result.  Two barriers per call.
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = lane < nw ? red[lane] : -CUDART_INF_F;
    r = warp_max(r);
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = lane < nw ? red[lane] : 0.0f;
    r = warp_sum(r);
    __syncthreads();
    return r;
}

// (value, index) argmax, first maximum wins.
__device__ __forceinline__ void argmax_merge(float& v, uint32_t& i, float ov, uint32_t oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}
__device__ __forceinline__ uint32_t block_argmax(float v, uint32_t i, float* redv, uint32_t* redi) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(kFull, v, o);
        uint32_t oi = __shfl_xor_sync(kFull, i, o);
        argmax_merge(v, i, ov, oi);
    }
    if (lane == 0) { redv[warp] = v; redi[warp] = i; }
    __syncthreads();
    v = lane < nw ? redv[lane] : -CUDART_INF_F;
    i = lane < nw ? redi[lane] : 0xffffffffu;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(kFull, v, o);
        uint32_t oi = __shfl_xor_sync(kFull, i, o);
        argmax_merge(v, i, ov, oi);
    }
    __syncthreads();
    return i;
}

// ------------------------------------------------------------------------------------
// General kernel: one CTA per row (grid-stride over rows), three reads of the row.
// MODE 0: softmax forward (y).  MODE 1: fused CE.
// ------------------------------------------------------------------------------------
struct CeArgs {
    const float* x;
    const uint32_t* labels;
    uint32_t rows, cols;
    float scale;
    float* loss_row;
    float* dlogits;
    float* probs;
    uint32_t* argmax;
    float* y;   // MODE 0 output
};

template <int MODE, bool VEC>
__global__ void softmax_stream_kernel(CeArgs a) {
    __shared__ float red[32];
    __shared__ uint32_t redi[32];
    const uint32_t cols = a.cols;
    for (uint32_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
        const float* xr = a.x + (size_t)row * cols;
        float mx = -CUDART_INF_F;
        uint32_t mi = 0xffffffffu;
        if (VEC) {
            const float4* x4 = reinterpret_cast<const float4*>(xr);
            for (uint32_t i = threadIdx.x; i < (cols >> 2); i += blockDim.x) {
                float4 v = x4[i];
                if (MODE == 1 && a.argmax) {
                    argmax_merge(mx, mi, v.x, 4 * i);
                    argmax_merge(mx, mi, v.y, 4 * i + 1);
                    argmax_merge(mx, mi, v.z, 4 * i + 2);
                    argmax_merge(mx, mi, v.w, 4 * i + 3);
                } else {
                    mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
                }
            }
        } else {
            for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
                if (MODE == 1 && a.argmax) argmax_merge(mx, mi, xr[c], c);
                else mx = fmaxf(mx, xr[c]);
            }
        }
        if (MODE == 1 && a.argmax) {
            uint32_t am = block_argmax(mx, mi, red, redi);
            if (threadIdx.x == 0) a.argmax[row] = am;
        }
        mx = block_max(mx, red);
        float s = 0.0f;
        if (VEC) {
            const float4* x4 = reinterpret_cast<const float4*>(xr);
            for (uint32_t i = threadIdx.x; i < (cols >> 2); i += blockDim.x) {
                float4 v = x4[i];
                s += (expf(v.x - mx) + expf(v.y - mx)) + (expf(v.z - mx) + expf(v.w - mx));
            }
        } else {
            for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) s += expf(xr[c] - mx);
        }
        s = block_sum(s, red);
        const float inv = 1.0f / s;
        uint32_t lab = 0xffffffffu;
        if (MODE == 1) {
            lab = a.labels[row];
            if (threadIdx.x == 0 && a.loss_row)
                a.loss_row[row] = lab < cols ? (logf(s) + mx) - xr[lab] : 0.0f;
        }
        float* o0 = MODE == 0 ? a.y + (size_t)row * cols : (a.dlogits ? a.dlogits + (size_t)row * cols : nullptr);
        float* o1 = (MODE == 1 && a.probs) ? a.probs + (size_t)row * cols : nullptr;
        if (VEC) {
            const float4* x4 = reinterpret_cast<const float4*>(xr);
            for (uint32_t i = threadIdx.x; i < (cols >> 2); i += blockDim.x) {
                float4 v = x4[i];
                float4 p = make_float4(expf(v.x - mx) * inv, expf(v.y - mx) * inv, expf(v.z - mx) * inv,
                                       expf(v.w - mx) * inv);
                if (MODE == 0) {
                    reinterpret_cast<float4*>(o0)[i] = p;
                } else {
                    if (o1) reinterpret_cast<float4*>(o1)[i] = p;
                    if (o0) {
                        uint32_t c = 4 * i;
                        float4 g = make_float4((p.x - (c == lab ? 1.f : 0.f)) * a.scale,
                                               (p.y - (c + 1 == lab ? 1.f : 0.f)) * a.scale,
                                               (p.z - (c + 2 == lab ? 1.f : 0.f)) * a.scale,
                                               (p.w - (c + 3 == lab ? 1.f : 0.f)) * a.scale);
                        reinterpret_cast<float4*>(o0)[i] = g;
                    }
                }
            }
        } else {
            for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
                float p = expf(xr[c] - mx) * inv;
                if (MODE == 0) o0[c] = p;
                else {
                    if (o1) o1[c] = p;
                    if (o0) o0[c] = (p - (c == lab ? 1.f : 0.f)) * a.scale;
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------
// rowreg kernel: persistent, row in registers, next row prefetched into shared memory.
// Requires cols % 4 == 0, 16-byte aligned base, cols <= 32768.
// ------------------------------------------------------------------------------------
constexpr int kRowT = 1024;   // threads per CTA
constexpr int kRowNV = 8;     // float4 per thread
constexpr long long kWaitCycles = 2000000000LL;  // about one second

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 63u) == 63u && clock64() - t0 > kWaitCycles) return false;
    }
}

// Issue the bulk copies that bring one row (bytes, a multiple of 16) into shared memory.
__device__ __forceinline__ void prefetch_row(uint32_t dst, const float* src, uint32_t bytes, uint32_t bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
    constexpr uint32_t kChunk = 16384;
    for (uint32_t off = 0; off < bytes; off += kChunk) {
        uint32_t n = bytes - off < kChunk ? bytes - off : kChunk;
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
            :: "r"(dst + off), "l"(reinterpret_cast<const char*>(src) + off), "r"(n), "r"(bar) : "memory");
    }
}

template <int MODE>
__global__ void __launch_bounds__(kRowT, 1) softmax_rowreg_kernel(CeArgs a, int* dev_status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* stage = reinterpret_cast<float*>(smem_raw);             // cols floats
    __shared__ float red[32];
    __shared__ uint32_t redi[32];
    __shared__ __align__(8) unsigned long long bar_storage;
    const uint32_t bar = smem_u32(&bar_storage);
    const uint32_t cols = a.cols, ncol4 = cols >> 2, row_bytes = cols * 4u;
    const int tid = threadIdx.x;

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t row = blockIdx.x;
    if (tid == 0 && row < a.rows) prefetch_row(smem_u32(stage), a.x + (size_t)row * cols, row_bytes, bar);
    uint32_t parity = 0;

    for (; row < a.rows; row += gridDim.x) {
        // 1. wait for this row in shared memory, move it to registers
        bool ok = mbar_wait_bounded(bar, parity);
        parity ^= 1u;
        if (__syncthreads_or(!ok)) {
            if (tid == 0) atomicOr(dev_status, FG_DEVERR_TMA_WAIT);
            // give the copies in flight a bounded chance to land before the CTA retires
            if (!ok) mbar_wait_bounded(bar, parity ^ 1u);
            return;
        }
        float4 v[kRowNV];
        const float4* s4 = reinterpret_cast<const float4*>(stage);
#pragma unroll
        for (int j = 0; j < kRowNV; ++j) {
            uint32_t i = tid + j * kRowT;
            v[j] = i < ncol4 ? s4[i] : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
        }
        __syncthreads();   // everyone has read the staging buffer
        // 2. start streaming the next row while this one is processed
        const uint32_t next = row + gridDim.x;
        if (tid == 0 && next < a.rows) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            prefetch_row(smem_u32(stage), a.x + (size_t)next * cols, row_bytes, bar);
        }
        // 3. max (and argmax)
        float mx = -CUDART_INF_F;
        if (MODE == 1 && a.argmax) {
            uint32_t mi = 0xffffffffu;
#pragma unroll
            for (int j = 0; j < kRowNV; ++j) {
                uint32_t c = 4u * (tid + j * kRowT);
                argmax_merge(mx, mi, v[j].x, c);
                argmax_merge(mx, mi, v[j].y, c + 1);
                argmax_merge(mx, mi, v[j].z, c + 2);
                argmax_merge(mx, mi, v[j].w, c + 3);
            }
            uint32_t am = block_argmax(mx, mi, red, redi);
            if (tid == 0) a.argmax[row] = am;
        } else {
#pragma unroll
            for (int j = 0; j < kRowNV; ++j)
                mx = fmaxf(fmaxf(mx, fmaxf(v[j].x, v[j].y)), fmaxf(v[j].z, v[j].w));
        }
        mx = block_max(mx, red);
        // 4. e = exp(x - max), sum
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < kRowNV; ++j) {
            v[j].x = expf(v[j].x - mx);
            v[j].y = expf(v[j].y - mx);
            v[j].z = expf(v[j].z - mx);
            v[j].w = expf(v[j].w - mx);
            s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        }
        s = block_sum(s, red);
        const float inv = 1.0f / s;
        uint32_t lab = 0xffffffffu;
        if (MODE == 1) {
            lab = a.labels[row];
            if (tid == 0 && a.loss_row)
                a.loss_row[row] = lab < cols ? (logf(s) + mx) - a.x[(size_t)row * cols + lab] : 0.0f;
        }
        // 5. write
        float4* o0 = MODE == 0 ? reinterpret_cast<float4*>(a.y + (size_t)row * cols)
                               : (a.dlogits ? reinterpret_cast<float4*>(a.dlogits + (size_t)row * cols) : nullptr);
        float4* o1 = (MODE == 1 && a.probs) ? reinterpret_cast<float4*>(a.probs + (size_t)row * cols) : nullptr;
#pragma unroll
        for (int j = 0; j < kRowNV; ++j) {
            uint32_t i = tid + j * kRowT;
            if (i < ncol4) {
                float4 p = make_float4(v[j].x * inv, v[j].y * inv, v[j].z * inv, v[j].w * inv);
                if (MODE == 0) {
                    __stcs(o0 + i, p);
                } else {
                    if (o1) __stcs(o1 + i, p);
                    if (o0) {
                        uint32_t c = 4u * i;
                        float4 g = make_float4((p.x - (c == lab ? 1.f : 0.f)) * a.scale,
                                               (p.y - (c + 1 == lab ? 1.f : 0.f)) * a.scale,
                                               (p.z - (c + 2 == lab ? 1.f : 0.f)) * a.scale,
                                               (p.w - (c + 3 == lab ? 1.f : 0.f)) * a.scale);
                        __stcs(o0 + i, g);
                    }
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------
// Rows of 512 to 8192 columns (a multiple of four, 16-byte aligned): the row is read ONCE into registers
// (thread t holds the float4s t, t + 256, ...: NV of them), the exponentials are computed once, and the row
// is written once.  The general kernel above reads such a row three times (the second and third time from the
// L1/L2) and evaluates every exponential twice; with its few loads in flight per thread it reached 49 % of the
// DRAM rate on 16384 x 4096.  MODE as above.
// ------------------------------------------------------------------------------------
template <int MODE, int NV>
__global__ void __launch_bounds__(256) softmax_held_kernel(CeArgs a) {
    __shared__ float red[32];
    __shared__ uint32_t redi[32];
    const uint32_t cols = a.cols, n4 = cols >> 2;
    for (uint32_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
        const float* xr = a.x + (size_t)row * cols;
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        float4 v[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const uint32_t i = threadIdx.x + 256u * j;
            v[j] = i < n4 ? __ldcs(x4 + i) : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
        }
        float mx = -CUDART_INF_F;
        uint32_t mi = 0xffffffffu;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const uint32_t i = threadIdx.x + 256u * j;
            if (MODE == 1 && a.argmax) {
                if (i < n4) {
                    argmax_merge(mx, mi, v[j].x, 4 * i);
                    argmax_merge(mx, mi, v[j].y, 4 * i + 1);
                    argmax_merge(mx, mi, v[j].z, 4 * i + 2);
                    argmax_merge(mx, mi, v[j].w, 4 * i + 3);
                }
            } else {
                mx = fmaxf(fmaxf(mx, fmaxf(v[j].x, v[j].y)), fmaxf(v[j].z, v[j].w));
            }
        }
        if (MODE == 1 && a.argmax) {
            uint32_t am = block_argmax(mx, mi, red, redi);
            if (threadIdx.x == 0) a.argmax[row] = am;
        }
        mx = block_max(mx, red);
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {       // padding is -inf: its exponential is zero
            v[j] = make_float4(expf(v[j].x - mx), expf(v[j].y - mx), expf(v[j].z - mx), expf(v[j].w - mx));
            s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        }
        s = block_sum(s, red);
        const float inv = 1.0f / s;
        uint32_t lab = 0xffffffffu;
        if (MODE == 1) {
            lab = a.labels[row];
            if (threadIdx.x == 0 && a.loss_row)
                a.loss_row[row] = lab < cols ? (logf(s) + mx) - xr[lab] : 0.0f;
        }
        float* o0 = MODE == 0 ? a.y + (size_t)row * cols : (a.dlogits ? a.dlogits + (size_t)row * cols : nullptr);
        float* o1 = (MODE == 1 && a.probs) ? a.probs + (size_t)row * cols : nullptr;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const uint32_t i = threadIdx.x + 256u * j;
            if (i >= n4) continue;
            const float4 p = make_float4(v[j].x * inv, v[j].y * inv, v[j].z * inv, v[j].w * inv);
            if (MODE == 0) {
                reinterpret_cast<float4*>(o0)[i] = p;
            } else {
                if (o1) reinterpret_cast<float4*>(o1)[i] = p;
                if (o0) {
                    const uint32_t c = 4 * i;
                    reinterpret_cast<float4*>(o0)[i] = make_float4((p.x - (c == lab ? 1.f : 0.f)) * a.scale,
                                                                   (p.y - (c + 1 == lab ? 1.f : 0.f)) * a.scale,
                                                                   (p.z - (c + 2 == lab ? 1.f : 0.f)) * a.scale,
                                                                   (p.w - (c + 3 == lab ? 1.f : 0.f)) * a.scale);
                }
            }
        }
    }
}

// The same for the backward pass: y and dy of a row are read once.
template <int NV>
__global__ void __launch_bounds__(256) softmax_bwd_held_kernel(uint32_t rows, uint32_t cols, const float* __restrict__ y,
                                                               const float* __restrict__ dy, float* __restrict__ dx,
                                                               int accumulate) {
    __shared__ float red[32];
    const uint32_t n4 = cols >> 2;
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4* y4 = reinterpret_cast<const float4*>(y + (size_t)row * cols);
        const float4* d4 = reinterpret_cast<const float4*>(dy + (size_t)row * cols);
        float4* x4 = reinterpret_cast<float4*>(dx + (size_t)row * cols);
        float4 a[NV], b[NV];
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const uint32_t i = threadIdx.x + 256u * j;
            a[j] = i < n4 ? __ldcs(y4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            b[j] = i < n4 ? __ldcs(d4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) dot += (a[j].x * b[j].x + a[j].y * b[j].y) + (a[j].z * b[j].z + a[j].w * b[j].w);
        dot = block_sum(dot, red);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const uint32_t i = threadIdx.x + 256u * j;
            if (i >= n4) continue;
            float4 g = make_float4(a[j].x * (b[j].x - dot), a[j].y * (b[j].y - dot), a[j].z * (b[j].z - dot), a[j].w * (b[j].w - dot));
            if (accumulate) {
                const float4 o = x4[i];
                g.x += o.x; g.y += o.y; g.z += o.z; g.w += o.w;
            }
            x4[i] = g;
        }
    }
}

// Softmax backward: dx (+)= y * (dy - dot), dot = sum_row(dy * y).
template <bool VEC>
__global__ void softmax_bwd_kernel(uint32_t rows, uint32_t cols, const float* __restrict__ y,
                                   const float* __restrict__ dy, float* __restrict__ dx, int accumulate) {
    __shared__ float red[32];
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* yr = y + (size_t)row * cols;
        const float* dr = dy + (size_t)row * cols;
        float* xr = dx + (size_t)row * cols;
        float dot = 0.0f;
        if (VEC) {
            for (uint32_t i = threadIdx.x; i < (cols >> 2); i += blockDim.x) {
                float4 a = reinterpret_cast<const float4*>(yr)[i], b = reinterpret_cast<const float4*>(dr)[i];
                dot += (a.x * b.x + a.y * b.y) + (a.z * b.z + a.w * b.w);
            }
        } else {
            for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) dot += yr[c] * dr[c];
        }
        dot = block_sum(dot, red);
        if (VEC) {
            for (uint32_t i = threadIdx.x; i < (cols >> 2); i += blockDim.x) {
                float4 a = reinterpret_cast<const float4*>(yr)[i], b = reinterpret_cast<const float4*>(dr)[i];
                float4 g = make_float4(a.x * (b.x - dot), a.y * (b.y - dot), a.z * (b.z - dot), a.w * (b.w - dot));
                if (accumulate) {
                    float4 o = reinterpret_cast<float4*>(xr)[i];
                    g.x += o.x; g.y += o.y; g.z += o.z; g.w += o.w;
                }
                reinterpret_cast<float4*>(xr)[i] = g;
            }
        } else {
            for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
                float g = yr[c] * (dr[c] - dot);
                xr[c] = accumulate ? xr[c] + g : g;
            }
        }
    }
}

// The reference's unfused per-element CE on probabilities.
__global__ void ce_elem_kernel(const float* __restrict__ p, const uint32_t* __restrict__ labels, uint32_t rows,
                               uint32_t cols, float* __restrict__ loss, float* __restrict__ grad) {
    const uint64_t n = (uint64_t)rows * cols;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t r = (uint32_t)(i / cols), c = (uint32_t)(i - (uint64_t)r * cols);
        float pv = p[i];
        bool hit = labels[r] == c;
        loss[i] = hit ? -logf(pv) : 0.0f;
        grad[i] = hit ? pv - 1.0f : pv;
    }
}

// Fixed-order mean of the per-row losses (one CTA).
__global__ void mean_kernel(const float* __restrict__ x, uint32_t n, float* __restrict__ out) {
    __shared__ float red[32];
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
    s = block_sum(s, red);
    if (threadIdx.x == 0) *out = s / (float)n;
}

// Algorithmic HBM bytes of the fused CE kernel: logits in, dlogits (and probs) out.
double ce_bytes(const CeArgs& a) {
    double mat = 4.0 * a.rows * a.cols;
    return mat * (1.0 + (a.dlogits ? 1.0 : 0.0) + (a.probs ? 1.0 : 0.0)) + 8.0 * a.rows;
}

int pick_threads(uint32_t cols) {
    if (cols <= 128) return 32;
    if (cols <= 2048) return 128;
    if (cols <= 8192) return 256;
    return 1024;
}

template <int MODE>
int32_t launch_rows(fg_ctx* ctx, const CeArgs& a) {
    const bool vec = (a.cols % 4 == 0) && fg_aligned16(a.x) &&
                     (MODE == 0 ? fg_aligned16(a.y)
                                : ((!a.dlogits || fg_aligned16(a.dlogits)) && (!a.probs || fg_aligned16(a.probs))));
    const size_t smem = (size_t)a.cols * 4;
    if (vec && a.cols >= 8192 && a.cols <= (uint32_t)(kRowT * kRowNV * 4) && smem <= 200 * 1024) {
        static std::atomic<uint64_t> attr_done{0};   // one bit per device (static per MODE instantiation)
        if (!(attr_done.load(std::memory_order_acquire) >> (ctx->device & 63) & 1ull)) {
            FG_CUDA(ctx, FG_ERR_INTERNAL,
                    cudaFuncSetAttribute(softmax_rowreg_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            attr_done.fetch_or(1ull << (ctx->device & 63), std::memory_order_release);
        }
        int grid = (int)(a.rows < (uint32_t)ctx->sm_count ? a.rows : (uint32_t)ctx->sm_count);
        fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SOFTMAX_CE, MODE == 1 ? ce_bytes(a) : 8.0 * a.rows * a.cols);
        softmax_rowreg_kernel<MODE><<<grid, kRowT, smem, ctx->stream>>>(a, ctx->dev_status);
        fg_time_end(ctx, tr);
        FG_LAUNCHED(ctx);
        return FG_OK;
    }
    if (vec && a.cols >= 512 && a.cols <= 8192) {
        const uint64_t cap = (uint64_t)ctx->sm_count * 8;
        const int grid = (int)(a.rows < cap ? a.rows : cap);
        const uint32_t nv = (a.cols / 4 + 255) / 256;      // float4s per thread: 1 .. 8
        fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SOFTMAX_CE, MODE == 1 ? ce_bytes(a) : 8.0 * a.rows * a.cols);
        if (nv <= 1) softmax_held_kernel<MODE, 1><<<grid, 256, 0, ctx->stream>>>(a);
        else if (nv <= 2) softmax_held_kernel<MODE, 2><<<grid, 256, 0, ctx->stream>>>(a);
        else if (nv <= 4) softmax_held_kernel<MODE, 4><<<grid, 256, 0, ctx->stream>>>(a);
        else softmax_held_kernel<MODE, 8><<<grid, 256, 0, ctx->stream>>>(a);
        fg_time_end(ctx, tr);
        FG_LAUNCHED(ctx);
        return FG_OK;
    }
    int threads = pick_threads(a.cols);
    uint64_t cap = (uint64_t)ctx->sm_count * (2048 / threads);
    int grid = (int)(a.rows < cap ? a.rows : cap);
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SOFTMAX_CE, MODE == 1 ? ce_bytes(a) : 8.0 * a.rows * a.cols);
    if (vec) softmax_stream_kernel<MODE, true><<<grid, threads, 0, ctx->stream>>>(a);
    else softmax_stream_kernel<MODE, false><<<grid, threads, 0, ctx->stream>>>(a);
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

}  // namespace

extern "C" {

int32_t fg_softmax_fwd(fg_ctx* ctx, uint32_t rows, uint32_t cols, const float* x, float* y) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, x && y, "fg_softmax_fwd: NULL pointer");
    FG_REQUIRE(ctx, cols >= 1, "fg_softmax_fwd: cols must be >= 1");
    FG_REQUIRE(ctx, (uint64_t)rows * cols < (1ull << 40), "fg_softmax_fwd: tensor too large");
    if (rows == 0) return FG_OK;
    CeArgs a{};
    a.x = x; a.rows = rows; a.cols = cols; a.y = y;
    return launch_rows<0>(ctx, a);
}

int32_t fg_softmax_bwd(fg_ctx* ctx, uint32_t rows, uint32_t cols, const float* y, const float* dy, float* dx,
                       int32_t accumulate) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, y && dy && dx, "fg_softmax_bwd: NULL pointer");
    FG_REQUIRE(ctx, cols >= 1, "fg_softmax_bwd: cols must be >= 1");
    if (rows == 0) return FG_OK;
    const bool vec = (cols % 4 == 0) && fg_aligned16(y) && fg_aligned16(dy) && fg_aligned16(dx);
    if (vec && cols >= 512 && cols <= 8192) {
        const uint64_t cap8 = (uint64_t)ctx->sm_count * 8;
        const int grid8 = (int)(rows < cap8 ? rows : cap8);
        const uint32_t nv = (cols / 4 + 255) / 256;
        fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SOFTMAX_CE, (accumulate ? 16.0 : 12.0) * rows * cols);
        if (nv <= 1) softmax_bwd_held_kernel<1><<<grid8, 256, 0, ctx->stream>>>(rows, cols, y, dy, dx, accumulate);
        else if (nv <= 2) softmax_bwd_held_kernel<2><<<grid8, 256, 0, ctx->stream>>>(rows, cols, y, dy, dx, accumulate);
        else if (nv <= 4) softmax_bwd_held_kernel<4><<<grid8, 256, 0, ctx->stream>>>(rows, cols, y, dy, dx, accumulate);
        else softmax_bwd_held_kernel<8><<<grid8, 256, 0, ctx->stream>>>(rows, cols, y, dy, dx, accumulate);
        fg_time_end(ctx, tr);
        FG_LAUNCHED(ctx);
        return FG_OK;
    }
    int threads = pick_threads(cols);
    uint64_t cap = (uint64_t)ctx->sm_count * (2048 / threads);
    int grid = (int)(rows < cap ? rows : cap);
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SOFTMAX_CE, (accumulate ? 16.0 : 12.0) * rows * cols);
    if (vec) softmax_bwd_kernel<true><<<grid, threads, 0, ctx->stream>>>(rows, cols, y, dy, dx, accumulate);
    else softmax_bwd_kernel<false><<<grid, threads, 0, ctx->stream>>>(rows, cols, y, dy, dx, accumulate);
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t fg_softmax_ce_fwd_bwd(fg_ctx* ctx, const float* logits, const uint32_t* labels, uint32_t rows,
                              uint32_t cols, float grad_scale, float* loss_row_out, float* loss_mean_out,
                              float* dlogits_out, float* probs_out, uint32_t* argmax_out) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, logits && labels, "fg_softmax_ce_fwd_bwd: logits and labels are required");
    FG_REQUIRE(ctx, cols >= 1, "fg_softmax_ce_fwd_bwd: cols must be >= 1");
    FG_REQUIRE(ctx, !(loss_mean_out && !loss_row_out),
               "fg_softmax_ce_fwd_bwd: loss_mean_out needs loss_row_out (the mean is reduced from it)");
    if (rows == 0) return FG_OK;
    CeArgs a{};
    a.x = logits; a.labels = labels; a.rows = rows; a.cols = cols; a.scale = grad_scale;
    a.loss_row = loss_row_out; a.dlogits = dlogits_out; a.probs = probs_out; a.argmax = argmax_out;
    int32_t s = launch_rows<1>(ctx, a);
    if (s != FG_OK) return s;
    if (loss_mean_out) {
        mean_kernel<<<1, 1024, 0, ctx->stream>>>(loss_row_out, rows, loss_mean_out);
        FG_LAUNCHED(ctx);
    }
    return FG_OK;
}

int32_t fg_ce_loss_grad(fg_ctx* ctx, const float* probs, const uint32_t* labels, uint32_t rows, uint32_t cols,
                        float* loss_out, float* grad_out) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, probs && labels && loss_out && grad_out, "fg_ce_loss_grad: NULL pointer");
    FG_REQUIRE(ctx, cols >= 1, "fg_ce_loss_grad: cols must be >= 1");
    if (rows == 0) return FG_OK;
    int grid = fg_stream_grid(ctx, (uint64_t)rows * cols, 256, 8);
    ce_elem_kernel<<<grid, 256, 0, ctx->stream>>>(probs, labels, rows, cols, loss_out, grad_out);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

}  // extern "C"
