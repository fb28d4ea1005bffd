// SIMT f32 GEMM: the exact-arithmetic path.
//
// Every output element is accumulated as one fmaf per k in increasing k, which is what
// the reference's generated matmul body does (crates/ferrograd-nn/src/op/matmul/generic.rs:98-319:
// out = fmaf(As[ly][i], Bs[i][lx], out) over 16-wide k tiles), so results are bit-identical
// to a sequential-k f32 FMA chain.  Unlike the reference (no bounds checks, shapes must be
// multiples of 16: crates/fused_gpu/src/dispatch/backend/mod.rs:617-619) any M, N, K is
// accepted.  Used for small shapes (the 2->16->2 MLP), as the on-device exact reference
// for the tensor-core path, and when FG_GEMM_SIMT is requested.
//
// 64x64 output tile per CTA, 16x16 threads, 4x4 outputs per thread, k tiles of 16.
#include "fg_internal.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <bool TA, bool TB>
__global__ void __launch_bounds__(256) gemm_simt_kernel(uint32_t M, uint32_t N, uint32_t K,
                                                        const float* __restrict__ A, const float* __restrict__ B,
                                                        float* __restrict__ C, const float* __restrict__ bias, int act,
                                                        float* __restrict__ preact, uint64_t sA, uint64_t sB, uint64_t sC) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];
    // blockIdx.z is the matrix of a batch (the reference puts the batch index in the grid's z too:
    // crates/fused_gpu/src/dispatch/backend/kernel/forward.rs:159-190); the strides are in elements
    A += blockIdx.z * sA;
    B += blockIdx.z * sB;
    C += blockIdx.z * sC;
    if (preact) preact += blockIdx.z * sC;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const uint32_t m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (uint32_t k0 = 0; k0 < K; k0 += TK) {
        // A tile: As[k][m] = opA[m0+m, k0+k]
#pragma unroll
        for (int e = threadIdx.x; e < TM * TK; e += 256) {
            int m, k;
            if (TA) { m = e % TM; k = e / TM; }     // A stored [K, M]: m contiguous
            else    { k = e % TK; m = e / TK; }     // A stored [M, K]: k contiguous
            uint32_t gm = m0 + m, gk = k0 + k;
            float v = 0.0f;
            if (gm < M && gk < K) v = TA ? A[(size_t)gk * M + gm] : A[(size_t)gm * K + gk];
            As[k][m] = v;
        }
        // B tile: Bs[k][n] = opB[k0+k, n0+n]
#pragma unroll
        for (int e = threadIdx.x; e < TN * TK; e += 256) {
            int n, k;
            if (TB) { k = e % TK; n = e / TK; }     // B stored [N, K]: k contiguous
            else    { n = e % TN; k = e / TN; }     // B stored [K, N]: n contiguous
            uint32_t gn = n0 + n, gk = k0 + k;
            float v = 0.0f;
            if (gn < N && gk < K) v = TB ? B[(size_t)gn * K + gk] : B[(size_t)gk * N + gn];
            Bs[k][n] = v;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float z = acc[i][j];
            if (bias) z += bias[gn];
            size_t o = (size_t)gm * N + gn;
            if (preact) preact[o] = z;
            C[o] = fg_act_fwd(act, z);
        }
    }
}

// ---- skinny outputs (N <= 16, e.g. a 10-class output layer) ----
// A 128-row tensor-core tile would leave most SMs idle for such shapes (32 CTAs for M = 4096) and the
// operand pre-pass would cost more than the product.  These kernels are bandwidth-bound on streaming the
// large operand once, and use plain f32 FMAs.  NT is N rounded up to a multiple of four; the small operand
// is zero-padded to NT so that the inner loops carry no predicates.
constexpr int SKN = 16;

// Bt[n][k] = B[k][n], zero for n >= N or k >= K   (Bt is [NT][Kp]).
__global__ void __launch_bounds__(256) skinny_transpose_kernel(uint32_t K, uint32_t N, uint32_t Kp, uint32_t NT,
                                                               const float* __restrict__ B, float* __restrict__ Bt) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i >= NT * Kp) return;
    const uint32_t n = i / Kp, k = i % Kp;
    Bt[i] = (n < N && k < K) ? B[(size_t)k * N + n] : 0.0f;
}

// C[M,N] = act(A[M,K]·B[K,N] + bias) from the transposed copy Bt.  A block of 8 warps owns 8 rows: warp w
// works on rows 4*(w/4) .. +3 and on every fourth 128-wide slice of k (lanes split the slice), so each
// Bt value fetched from L1 feeds four rows, and the four k-quarters of a row meet in shared memory.
template <int NT, bool VEC>
__global__ void __launch_bounds__(256, 2) gemm_skinny_n_kernel(uint32_t M, uint32_t N, uint32_t K, uint32_t Kp,
                                                            const float* __restrict__ A, const float* __restrict__ Bt,
                                                            float* __restrict__ C, const float* __restrict__ bias, int act,
                                                            float* __restrict__ preact) {
    __shared__ float red[8][4][NT];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ks = warp & 3;
    const uint32_t row0 = blockIdx.x * 8 + (warp >> 2) * 4;
    float acc[4][NT];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int n = 0; n < NT; ++n) acc[r][n] = 0.0f;
    const float* a[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) a[r] = A + (size_t)min(row0 + r, M - 1) * K;     // rows past the end are not stored
    if (VEC) {
#pragma unroll 1
        for (uint32_t k = (ks * 32 + lane) * 4; k < K; k += 512) {
            float4 x[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) x[r] = *reinterpret_cast<const float4*>(a[r] + k);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float4 w = *reinterpret_cast<const float4*>(Bt + (size_t)n * Kp + k);
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    acc[r][n] = fmaf(x[r].w, w.w, fmaf(x[r].z, w.z, fmaf(x[r].y, w.y, fmaf(x[r].x, w.x, acc[r][n]))));
            }
        }
    } else {
#pragma unroll 2
        for (uint32_t k = ks * 32 + lane; k < K; k += 128) {
            float x[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) x[r] = a[r][k];
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float w = Bt[(size_t)n * Kp + k];
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[r][n] = fmaf(x[r], w, acc[r][n]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            float v = acc[r][n];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red[warp][r][n] = v;
        }
    __syncthreads();
    // thread t < 8*N: row t / N of the block, column t % N
    const uint32_t t = threadIdx.x;
    if (t < 8 * N) {
        const uint32_t rr = t / N, n = t % N, row = blockIdx.x * 8 + rr;
        if (row < M) {
            const int w0 = (rr >> 2) * 4, r = rr & 3;
            float z = (red[w0][r][n] + red[w0 + 1][r][n]) + (red[w0 + 2][r][n] + red[w0 + 3][r][n]);
            if (bias) z += bias[n];
            const size_t o = (size_t)row * N + n;
            if (preact) preact[o] = z;
            C[o] = fg_act_fwd(act, z);
        }
    }
}

constexpr int TN_ROWS = 64;   // rows of A per partial sum in the dB kernel

// part[chunk][j][n] = sum over the chunk's rows m of A[m][j] * dZ[m][n]   (A is [M, Kd], dZ is [M, N]).
// A thread owns four consecutive j; the chunk's rows of dZ sit in shared memory and are broadcast.
template <int NT, bool VEC>
__global__ void __launch_bounds__(128) gemm_skinny_tn_partial_kernel(uint32_t M, uint32_t Kd, uint32_t N,
                                                                     const float* __restrict__ A,
                                                                     const float* __restrict__ dZ,
                                                                     float* __restrict__ part) {
    __shared__ float zs[TN_ROWS][NT];
    const uint32_t m0 = blockIdx.y * TN_ROWS, rows = min((uint32_t)TN_ROWS, M - m0);
    for (uint32_t e = threadIdx.x; e < TN_ROWS * NT; e += 128) {
        const uint32_t r = e / NT, n = e % NT;
        zs[r][n] = (r < rows && n < N) ? dZ[(size_t)(m0 + r) * N + n] : 0.0f;
    }
    __syncthreads();
    const uint32_t j0 = (blockIdx.x * 128 + threadIdx.x) * 4;
    if (j0 >= Kd) return;
    float acc[4][NT];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int n = 0; n < NT; ++n) acc[q][n] = 0.0f;
    const float* a = A + (size_t)m0 * Kd + j0;
    for (uint32_t r0 = 0; r0 < rows; r0 += 8) {
        float x[8][4];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t r = min(r0 + u, rows - 1);     // rows past the end reload the last one; their dZ is zero
            if (VEC) {
                const float4 t = *reinterpret_cast<const float4*>(a + (size_t)r * Kd);
                x[u][0] = t.x; x[u][1] = t.y; x[u][2] = t.z; x[u][3] = t.w;
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) x[u][q] = (j0 + q < Kd) ? a[(size_t)r * Kd + q] : 0.0f;
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (r0 + u < rows) {
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const float z = zs[r0 + u][n];
#pragma unroll
                    for (int q = 0; q < 4; ++q) acc[q][n] = fmaf(x[u][q], z, acc[q][n]);
                }
            }
        }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (j0 + q < Kd) {
            float* p = part + ((size_t)blockIdx.y * Kd + j0 + q) * N;
#pragma unroll
            for (int n = 0; n < NT; ++n)
                if (n < (int)N) p[n] = acc[q][n];
        }
    }
}

// dA[m][k] = sum_n dZ[m][n] * B[k][n]   (dZ is [M, N], B is [K, N]): bound by writing dA once.
// A thread owns four consecutive k and keeps their rows of B in registers while it walks 32 rows of dZ.
// With extras: the product is multiplied by act'(mul_saved) (the layer below's backward factor), its bf16
// pairs are written beside it, and the thread's own column sums over the 32 rows go to colsum_part.
template <int NT>
__global__ void __launch_bounds__(128) gemm_skinny_nt_kernel(uint32_t M, uint32_t K, uint32_t N,
                                                             const float* __restrict__ dZ, const float* __restrict__ B,
                                                             float* __restrict__ dA, fg_skinny_extras ex) {
    __shared__ float zs[32][NT];
    const uint32_t m0 = blockIdx.y * 32, rows = min(32u, M - m0);
    for (uint32_t e = threadIdx.x; e < 32 * NT; e += 128) {
        const uint32_t r = e / NT, n = e % NT;
        zs[r][n] = (r < rows && n < N) ? dZ[(size_t)(m0 + r) * N + n] : 0.0f;
    }
    __syncthreads();
    const uint32_t k0 = (blockIdx.x * 128 + threadIdx.x) * 4;
    if (k0 >= K) return;
    float b[4][NT];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int n = 0; n < NT; ++n) b[q][n] = (n < (int)N && k0 + q < K) ? B[(size_t)(k0 + q) * N + n] : 0.0f;
    const bool vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(dA) & 15u) == 0) &&
                     (!ex.mul_saved || (reinterpret_cast<uintptr_t>(ex.mul_saved) & 15u) == 0) &&
                     (!ex.pairs || ((reinterpret_cast<uintptr_t>(ex.pairs) & 15u) == 0 && ex.pairs_stride % 4 == 0));
    float cs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
    for (uint32_t r = 0; r < rows; ++r) {
        float o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const float z = zs[r][n];
#pragma unroll
            for (int q = 0; q < 4; ++q) o[q] = fmaf(z, b[q][n], o[q]);
        }
        const size_t off = (size_t)(m0 + r) * K + k0;
        if (vec) {
            if (ex.mul_saved) {
                const float4 sv = __ldcs(reinterpret_cast<const float4*>(ex.mul_saved + off));
                // the short forms the tensor-core epilogues use (one exponential, one reciprocal): the libm tanh of
                // the plain form made this kernel compute-bound
                o[0] *= fg_act_grad_sel(ex.mul_act, sv.x); o[1] *= fg_act_grad_sel(ex.mul_act, sv.y);
                o[2] *= fg_act_grad_sel(ex.mul_act, sv.z); o[3] *= fg_act_grad_sel(ex.mul_act, sv.w);
            }
            const float4 v = make_float4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<float4*>(dA + off) = v;
            if (ex.pairs) fg_store_pairs4(ex.pairs, ex.pairs_stride, off, v);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (k0 + q < K) {
                    if (ex.mul_saved) o[q] *= fg_act_grad_sel(ex.mul_act, ex.mul_saved[off + q]);
                    dA[off + q] = o[q];
                    if (ex.pairs) fg_store_pairs1(ex.pairs, ex.pairs_stride, off + q, o[q]);
                } else o[q] = 0.0f;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) cs[q] += o[q];
    }
    if (ex.colsum_part) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (k0 + q < K) ex.colsum_part[(size_t)blockIdx.y * K + k0 + q] = cs[q];
    }
}

__global__ void __launch_bounds__(256) fold_chunks_kernel(uint64_t n, uint32_t nchunks, const float* __restrict__ part,
                                                          float* __restrict__ out) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        float s = 0.0f;
#pragma unroll 8
        for (uint32_t c = 0; c < nchunks; ++c) s += part[(size_t)c * n + i];
        out[i] = s;
    }
}

// Runs the statement with NT = N rounded up to a multiple of four.
#define FG_SKINNY_DISPATCH(N, ...)                                  \
    do {                                                            \
        if ((N) <= 4) { constexpr int NT = 4; __VA_ARGS__; }        \
        else if ((N) <= 8) { constexpr int NT = 8; __VA_ARGS__; }   \
        else if ((N) <= 12) { constexpr int NT = 12; __VA_ARGS__; } \
        else { constexpr int NT = 16; __VA_ARGS__; }                \
    } while (0)

}  // namespace

uint64_t fg_gemm_skinny_scratch_bytes(uint32_t M, uint32_t N, uint32_t K) {
    const uint64_t kp = (K + 3) / 4 * 4;
    const uint64_t fwd = 16 * kp * 4 + 256;                                              // transposed B
    const uint64_t bwd = (uint64_t)((M + TN_ROWS - 1) / TN_ROWS) * K * N * 4 + 256;      // dB partials
    return fwd > bwd ? fwd : bwd;
}

int32_t fg_gemm_skinny_n_launch(fg_ctx* ctx, uint32_t M, uint32_t N, uint32_t K, const float* A, const float* B, float* C,
                                const float* bias, int act, float* preact_out) {
    if (N > SKN) return fg_fail(ctx, FG_ERR_INTERNAL, "skinny GEMM: N too large");
    const uint32_t Kp = (K + 3) / 4 * 4, NTr = (N + 3) / 4 * 4;
    void* bt;
    int32_t s = fg_ws_alloc(ctx, (uint64_t)NTr * Kp * 4, &bt);
    if (s != FG_OK) return s;
    skinny_transpose_kernel<<<(NTr * Kp + 255) / 256, 256, 0, ctx->stream>>>(K, N, Kp, NTr, B, (float*)bt);
    FG_LAUNCHED(ctx);
    const uint32_t blocks = (M + 7) / 8;
    const bool vec = (K % 4 == 0) && fg_aligned16(A);
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SKINNY, 4.0 * M * K);                 // A read once
    FG_SKINNY_DISPATCH(N, {
        if (vec) gemm_skinny_n_kernel<NT, true><<<blocks, 256, 0, ctx->stream>>>(M, N, K, Kp, A, (const float*)bt, C, bias, act, preact_out);
        else gemm_skinny_n_kernel<NT, false><<<blocks, 256, 0, ctx->stream>>>(M, N, K, Kp, A, (const float*)bt, C, bias, act, preact_out);
    });
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

// dA[M, K] = dZ · B^T with dZ [M, N], B [K, N], N <= 16.
int32_t fg_gemm_skinny_nt_launch(fg_ctx* ctx, uint32_t M, uint32_t K, uint32_t N, const float* dZ, const float* B,
                                 float* dA, const fg_skinny_extras* extras) {
    if (N > SKN) return fg_fail(ctx, FG_ERR_INTERNAL, "skinny GEMM: N too large");
    dim3 grid((K + 511) / 512, (M + 31) / 32);
    if (grid.y > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "skinny GEMM: too many rows");
    const fg_skinny_extras ex = extras ? *extras : fg_skinny_extras{nullptr, 0, nullptr, 0, nullptr};
    // dA written once; with extras also the saved tensor read and the pairs (as many bytes again) written
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SKINNY, 4.0 * M * K * (1.0 + (ex.mul_saved ? 1.0 : 0.0) + (ex.pairs ? 1.0 : 0.0)));
    FG_SKINNY_DISPATCH(N, (gemm_skinny_nt_kernel<NT><<<grid, 128, 0, ctx->stream>>>(M, K, N, dZ, B, dA, ex)));
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

// dB[Kd, N] = A^T · dZ with A [M, Kd], dZ [M, N], N <= 16.  Uses the scratch arena for the per-chunk partials.
int32_t fg_gemm_skinny_tn_launch(fg_ctx* ctx, uint32_t M, uint32_t Kd, uint32_t N, const float* A, const float* dZ,
                                 float* dB) {
    if (N > SKN) return fg_fail(ctx, FG_ERR_INTERNAL, "skinny GEMM: N too large");
    const uint32_t nchunks = (M + TN_ROWS - 1) / TN_ROWS;
    void* part;
    int32_t s = fg_ws_alloc(ctx, (uint64_t)nchunks * Kd * N * 4, &part);
    if (s != FG_OK) return s;
    dim3 grid((Kd + 511) / 512, nchunks);
    if (grid.y > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "skinny GEMM: too many rows");
    const bool vec = (Kd % 4 == 0) && fg_aligned16(A);
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SKINNY, 4.0 * M * Kd);                // A read once
    FG_SKINNY_DISPATCH(N, {
        if (vec) gemm_skinny_tn_partial_kernel<NT, true><<<grid, 128, 0, ctx->stream>>>(M, Kd, N, A, dZ, (float*)part);
        else gemm_skinny_tn_partial_kernel<NT, false><<<grid, 128, 0, ctx->stream>>>(M, Kd, N, A, dZ, (float*)part);
    });
    FG_LAUNCHED(ctx);
    const uint64_t n = (uint64_t)Kd * N;
    fold_chunks_kernel<<<fg_stream_grid(ctx, n, 256, 8), 256, 0, ctx->stream>>>(n, nchunks, (const float*)part, dB);
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t fg_gemm_simt_batched_launch(fg_ctx* ctx, int transA, int transB, uint32_t batch, uint32_t M, uint32_t N, uint32_t K,
                                    const float* A, uint64_t sA, const float* B, uint64_t sB, float* C, uint64_t sC,
                                    const float* bias, int act, float* preact_out) {
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, batch);
    if (grid.y > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "SIMT GEMM: M too large");
    if (batch > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "SIMT GEMM: more than 65535 matrices in a batch");
    if (batch == 0) return FG_OK;
    if (!transA && !transB) gemm_simt_kernel<false, false><<<grid, 256, 0, ctx->stream>>>(M, N, K, A, B, C, bias, act, preact_out, sA, sB, sC);
    else if (transA && !transB) gemm_simt_kernel<true, false><<<grid, 256, 0, ctx->stream>>>(M, N, K, A, B, C, bias, act, preact_out, sA, sB, sC);
    else if (!transA && transB) gemm_simt_kernel<false, true><<<grid, 256, 0, ctx->stream>>>(M, N, K, A, B, C, bias, act, preact_out, sA, sB, sC);
    else gemm_simt_kernel<true, true><<<grid, 256, 0, ctx->stream>>>(M, N, K, A, B, C, bias, act, preact_out, sA, sB, sC);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t fg_gemm_simt_launch(fg_ctx* ctx, int transA, int transB, uint32_t M, uint32_t N, uint32_t K, const float* A,
                            const float* B, float* C, const float* bias, int act, float* preact_out) {
    return fg_gemm_simt_batched_launch(ctx, transA, transB, 1, M, N, K, A, 0, B, 0, C, 0, bias, act, preact_out);
}
