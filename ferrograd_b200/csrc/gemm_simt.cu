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
                                                        float* __restrict__ preact) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];
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

}  // namespace

int32_t fg_gemm_simt_launch(fg_ctx* ctx, int transA, int transB, uint32_t M, uint32_t N, uint32_t K, const float* A,
                            const float* B, float* C, const float* bias, int act, float* preact_out) {
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    if (grid.y > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "SIMT GEMM: M too large");
    if (!transA && !transB) gemm_simt_kernel<false, false><<<grid, 256, 0, ctx->stream>>>(M, N, K, A, B, C, bias, act, preact_out);
    else if (transA && !transB) gemm_simt_kernel<true, false><<<grid, 256, 0, ctx->stream>>>(M, N, K, A, B, C, bias, act, preact_out);
    else if (!transA && transB) gemm_simt_kernel<false, true><<<grid, 256, 0, ctx->stream>>>(M, N, K, A, B, C, bias, act, preact_out);
    else gemm_simt_kernel<true, true><<<grid, 256, 0, ctx->stream>>>(M, N, K, A, B, C, bias, act, preact_out);
    FG_LAUNCHED(ctx);
    return FG_OK;
}
