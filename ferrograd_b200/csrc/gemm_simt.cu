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
#include <atomic>

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
        // The rows of the next k-step are requested before the FMAs of this one, so that two steps' worth of
        // loads (eight 16-byte loads per thread) are in flight: with 128 registers only 16 warps fit an SM, and
        // one step's worth left the memory system half idle (long-scoreboard stalls, 29 % of the DRAM rate).
        uint32_t k = (ks * 32 + lane) * 4;
        float4 x[4], nx[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) x[r] = k < K ? __ldcs(reinterpret_cast<const float4*>(a[r] + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (; k < K; k += 512) {
            const uint32_t kn = k + 512;
#pragma unroll
            for (int r = 0; r < 4; ++r)
                nx[r] = kn < K ? __ldcs(reinterpret_cast<const float4*>(a[r] + kn)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float4 w = *reinterpret_cast<const float4*>(Bt + (size_t)n * Kp + k);
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    acc[r][n] = fmaf(x[r].w, w.w, fmaf(x[r].z, w.z, fmaf(x[r].y, w.y, fmaf(x[r].x, w.x, acc[r][n]))));
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) x[r] = nx[r];
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

// ---- forward, sliced: part[s][m][0..15] = sum over k-slice s of A[m][k] * B[k][n] ----
// The kernel above fetches the transposed small operand through the L1 cache, where the streamed rows of A keep
// evicting it (L1 hit rate 57 %: every miss is an L2 round trip in the middle of the FMA chain, and the kernel ran
// at 29 % of the DRAM rate).  Here a block owns one 512-wide slice of k: the slice of B (NT x 512 floats) sits in
// shared memory, transposed, for the whole block, and the block streams its rows' 2 KB segments of A past it.
// A warp takes four rows at a time, all sixteen 16-byte loads in flight before the first FMA; a lane owns 16 of
// the 512 k-values; the 4 x 16 partial sums meet by a halving exchange (62 shuffles, each lane ends with two sums).
// The slices are added, in order, by skinny_fold_slices_kernel, which also applies bias and activation.
constexpr int SK_SLICE = 512;

template <int NT>
__global__ void __launch_bounds__(256, 2) gemm_skinny_n_slice_kernel(uint32_t M, uint32_t N, uint32_t K, uint32_t rows_per_block,
                                                                     const float* __restrict__ A, const float* __restrict__ B,
                                                                     float* __restrict__ part) {
    __shared__ __align__(16) float bt[NT][SK_SLICE];
    const uint32_t k0 = blockIdx.x * SK_SLICE, kw = min((uint32_t)SK_SLICE, K - k0);
    for (uint32_t e = threadIdx.x; e < NT * SK_SLICE; e += 256) (&bt[0][0])[e] = 0.0f;
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < kw * N; e += 256) bt[e % N][e / N] = B[(size_t)k0 * N + e];   // B as it lies: [k][n]
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t row_end = min(M, (blockIdx.y + 1) * rows_per_block);
    for (uint32_t r0 = blockIdx.y * rows_per_block + warp * 4; r0 < row_end; r0 += 32) {
        float4 x[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float* a = A + (size_t)min(r0 + r, M - 1) * K + k0;      // rows past the end are not stored
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t k = c * 128 + lane * 4;
                x[r][c] = k < kw ? __ldcs(reinterpret_cast<const float4*>(a + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        float v[64];      // [row][16]: columns NT..15 stay zero
#pragma unroll
        for (int i = 0; i < 64; ++i) v[i] = 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float4 w = *reinterpret_cast<const float4*>(&bt[n][c * 128 + lane * 4]);
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    v[r * 16 + n] = fmaf(x[r][c].w, w.w, fmaf(x[r][c].z, w.z, fmaf(x[r][c].y, w.y, fmaf(x[r][c].x, w.x, v[r * 16 + n]))));
            }
        }
        // halving exchange: at each step a lane keeps one half of its values and adds the partner's copy of them
#pragma unroll
        for (int step = 0; step < 5; ++step) {
            const int off = 16 >> step, half = 32 >> step;
            const bool upper = (lane & off) != 0;
#pragma unroll
            for (int i = 0; i < half; ++i) {
                const float send = upper ? v[i] : v[i + half];
                const float keep = upper ? v[i + half] : v[i];
                v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
            }
        }
        // lane bits (16, 8, 4, 2, 1) chose halves of 64, 32, 16, 8, 4: the lane holds values 2*lane' and 2*lane' + 1
        const int idx = ((lane >> 4) & 1) * 32 + ((lane >> 3) & 1) * 16 + ((lane >> 2) & 1) * 8 + ((lane >> 1) & 1) * 4 + (lane & 1) * 2;
        const uint32_t row = r0 + (idx >> 4);
        if (row < row_end)
            *reinterpret_cast<float2*>(part + ((size_t)blockIdx.x * M + row) * 16 + (idx & 15)) = make_float2(v[0], v[1]);
    }
}

// C[m][n] = act(sum over slices of part[s][m][n] + bias[n]); optional copy of the pre-activation.
__global__ void __launch_bounds__(256) skinny_fold_slices_kernel(uint32_t M, uint32_t N, uint32_t nslices,
                                                                 const float* __restrict__ part, const float* __restrict__ bias,
                                                                 int act, float* __restrict__ C, float* __restrict__ preact) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;      // over M x 16
    if (i >= M * 16) return;
    const uint32_t m = i >> 4, n = i & 15;
    if (n >= N) return;
    float z = 0.0f;
    for (uint32_t s = 0; s < nslices; ++s) z += part[(size_t)s * M * 16 + i];
    if (bias) z += bias[n];
    const size_t o = (size_t)m * N + n;
    if (preact) preact[o] = z;
    C[o] = fg_act_fwd(act, z);
}

constexpr int TN_ROWS = 64;   // rows of A per partial sum in the dB kernel

// part[block row][n][j] = sum over the block row's chunks' rows m of A[m][j] * dZ[m][n]   (A is [M, Kd], dZ is [M, N]).
// A thread owns four consecutive j; the chunk's rows of dZ sit in shared memory and are broadcast.
template <int NT, bool VEC>
__global__ void __launch_bounds__(128, 4) gemm_skinny_tn_partial_kernel(uint32_t M, uint32_t Kd, uint32_t N,
                                                                     const float* __restrict__ A,
                                                                     const float* __restrict__ dZ,
                                                                     float* __restrict__ part) {
    __shared__ float zs[TN_ROWS][NT];
    const uint32_t j0 = (blockIdx.x * 128 + threadIdx.x) * 4;
    const bool active = j0 < Kd;
    float acc[4][NT];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int n = 0; n < NT; ++n) acc[q][n] = 0.0f;
    // A block walks the 64-row chunks blockIdx.y, + gridDim.y, ... and keeps its sums in registers across them:
    // the number of partial results is the number of block rows (at most what the SMs hold at once), whatever M is.
    for (uint32_t m0 = blockIdx.y * TN_ROWS; m0 < M; m0 += gridDim.y * TN_ROWS) {
        const uint32_t rows = min((uint32_t)TN_ROWS, M - m0);
        __syncthreads();                                    // the previous chunk's rows of dZ are no longer read
        for (uint32_t e = threadIdx.x; e < TN_ROWS * NT; e += 128) {
            const uint32_t r = e / NT, n = e % NT;
            zs[r][n] = (r < rows && n < N) ? dZ[(size_t)(m0 + r) * N + n] : 0.0f;
        }
        __syncthreads();
        if (!active) continue;
        const float* a = A + (size_t)m0 * Kd + j0;
        // Eight rows are multiplied while the next eight are on their way (16 loads of 16 bytes in flight per
        // thread: with eight, and a grid that fills 70 % of the thread slots, the kernel ran at 23 % of the DRAM rate).
        float x[8][4], nx[8][4];
        auto fetch = [&](uint32_t r0, float (*dst)[4]) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t r = min(r0 + u, rows - 1);     // rows past the end reload the last one; their dZ is zero
                if (VEC) {
                    const float4 t = __ldcs(reinterpret_cast<const float4*>(a + (size_t)r * Kd));
                    dst[u][0] = t.x; dst[u][1] = t.y; dst[u][2] = t.z; dst[u][3] = t.w;
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q) dst[u][q] = (j0 + q < Kd) ? a[(size_t)r * Kd + q] : 0.0f;
                }
            }
        };
        fetch(0, x);
        for (uint32_t r0 = 0; r0 < rows; r0 += 8) {
            if (r0 + 8 < rows) fetch(r0 + 8, nx);
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
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int q = 0; q < 4; ++q) x[u][q] = nx[u][q];
        }
    }
    if (!active) return;
    // part[chunk][n][j]: for one n a thread's four j are one 16-byte store and a warp's are 512 contiguous bytes
    // (as [chunk][j][n] every store instruction touched 32 sectors, and 10 MB of partials cost more L2 write
    // bandwidth than the 67 MB read cost DRAM bandwidth)
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        if (n >= (int)N) break;
        float* p = part + ((size_t)blockIdx.y * N + n) * Kd + j0;
        if (VEC) {
            *reinterpret_cast<float4*>(p) = make_float4(acc[0][n], acc[1][n], acc[2][n], acc[3][n]);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (j0 + q < Kd) p[q] = acc[q][n];
        }
    }
}

// dA[m][k] = sum_n dZ[m][n] * B[k][n]   (dZ is [M, N], B is [K, N]): bound by writing dA once.
// A thread owns four consecutive k and keeps their rows of B in registers; a block walks 8-row chunks of dZ
// (chunk = blockIdx.y, + gridDim.y, ...: the grid is sized to the SMs' thread slots, so every block has the
// same number of chunks to within one).
// With extras: the product is multiplied by act'(mul_saved) (the layer below's backward factor), its bf16
// pairs are written beside it, and the thread's column sums over all of the block's rows go to
// colsum_part[blockIdx.y][k] (the partials of the bias gradient of the layer below).
constexpr int NT_ROWS = 8;

template <int NT>
__global__ void __launch_bounds__(128) gemm_skinny_nt_kernel(uint32_t M, uint32_t K, uint32_t N,
                                                             const float* __restrict__ dZ, const float* __restrict__ B,
                                                             float* __restrict__ dA, fg_skinny_extras ex) {
    __shared__ float zs[NT_ROWS][NT];
    const uint32_t k0 = (blockIdx.x * 128 + threadIdx.x) * 4;
    const bool active = k0 < K;
    float b[4][NT];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int n = 0; n < NT; ++n) b[q][n] = (n < (int)N && k0 + q < K) ? B[(size_t)(k0 + q) * N + n] : 0.0f;
    const bool vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(dA) & 15u) == 0) &&
                     (!ex.mul_saved || (reinterpret_cast<uintptr_t>(ex.mul_saved) & 15u) == 0) &&
                     (!ex.pairs || ((reinterpret_cast<uintptr_t>(ex.pairs) & 15u) == 0 && ex.pairs_stride % 4 == 0));
    const bool vsaved = vec && ex.mul_saved != nullptr;
    float cs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    // Four rows at a time, and the saved tensor's slices of the next four (of this chunk or of the block's next
    // chunk) are requested before these four are stored: inside a one-row loop the compiler may not move those
    // loads above the previous row's stores (the pointers could alias), and every row waited a full memory latency.
    float4 sv[4], nsv[4];
    auto fetch = [&](uint32_t m0, uint32_t r0, float4* dst) {
        const uint32_t last = min((uint32_t)NT_ROWS, M - m0) - 1;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            dst[u] = __ldcs(reinterpret_cast<const float4*>(ex.mul_saved + (size_t)(m0 + min(r0 + u, last)) * K + k0));
    };
    const uint32_t step = gridDim.y * NT_ROWS;
    if (vsaved && active && blockIdx.y * NT_ROWS < M) fetch(blockIdx.y * NT_ROWS, 0, sv);
    for (uint32_t m0 = blockIdx.y * NT_ROWS; m0 < M; m0 += step) {
        const uint32_t rows = min((uint32_t)NT_ROWS, M - m0);
        __syncthreads();                                    // the previous chunk's rows of dZ are no longer read
        for (uint32_t e = threadIdx.x; e < NT_ROWS * NT; e += 128) {
            const uint32_t r = e / NT, n = e % NT;
            zs[r][n] = (r < rows && n < N) ? dZ[(size_t)(m0 + r) * N + n] : 0.0f;
        }
        __syncthreads();
        if (!active) continue;
        for (uint32_t r0 = 0; r0 < rows; r0 += 4) {
            if (vsaved) {
                if (r0 + 4 < rows) fetch(m0, r0 + 4, nsv);
                else if (m0 + step < M) fetch(m0 + step, 0, nsv);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t r = r0 + u;
                if (r >= rows) break;
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
                        // the short forms the tensor-core epilogues use (one exponential, one reciprocal): the libm
                        // tanh of the plain form made this kernel compute-bound
                        o[0] *= fg_act_grad_sel(ex.mul_act, sv[u].x); o[1] *= fg_act_grad_sel(ex.mul_act, sv[u].y);
                        o[2] *= fg_act_grad_sel(ex.mul_act, sv[u].z); o[3] *= fg_act_grad_sel(ex.mul_act, sv[u].w);
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
#pragma unroll
            for (int u = 0; u < 4; ++u) sv[u] = nsv[u];
        }
    }
    if (ex.colsum_part && active) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (k0 + q < K) ex.colsum_part[(size_t)blockIdx.y * K + k0 + q] = cs[q];
    }
}

// dB[j][n] = sum over chunks of part[c][n][j]; output i = n * Kd + j, so the reads are contiguous.  A block covers
// 32 outputs; its eight warps each add every eighth chunk (an eighth of the chain of dependent loads), then the
// eight sums are added in order.
__global__ void __launch_bounds__(256) fold_chunks_kernel(uint32_t Kd, uint32_t N, uint32_t nchunks, const float* __restrict__ part,
                                                          float* __restrict__ out) {
    __shared__ float red[8][33];
    const uint64_t total = (uint64_t)Kd * N;
    const uint32_t cx = threadIdx.x & 31u, gy = threadIdx.x >> 5;
    for (uint64_t i0 = (uint64_t)blockIdx.x * 32; i0 < total; i0 += (uint64_t)gridDim.x * 32) {
        const uint64_t i = i0 + cx;
        float s = 0.0f;
        if (i < total)
            for (uint32_t c = gy; c < nchunks; c += 8) s += part[(size_t)c * total + i];
        __syncthreads();                      // the previous round's sums have been read
        red[gy][cx] = s;
        __syncthreads();
        if (gy == 0 && i < total) {
            float t = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += red[w][cx];
            const uint32_t n = (uint32_t)(i / Kd), j = (uint32_t)(i % Kd);
            out[(size_t)j * N + n] = t;
        }
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
    if (N > SKN) return 0;                                                               // not a narrow layer: these kernels do not run
    const uint64_t kp = (K + 3) / 4 * 4;
    const uint64_t fwd_t = 16 * kp * 4 + 256;                                            // transposed B
    const uint64_t fwd_s = (uint64_t)((K + SK_SLICE - 1) / SK_SLICE) * M * 16 * 4 + 256;  // per-slice partial sums
    const uint64_t fwd = fwd_t > fwd_s ? fwd_t : fwd_s;
    // dB partials: one [N][K] block per block row, and there are at most as many block rows as 64-row chunks or
    // as four blocks per SM allow (fewer than 2048 on any GPU)
    uint64_t rows = (M + TN_ROWS - 1) / TN_ROWS;
    if (rows > 2048) rows = 2048;
    const uint64_t bwd = rows * K * N * 4 + 256;
    return fwd > bwd ? fwd : bwd;
}

int32_t fg_gemm_skinny_n_launch(fg_ctx* ctx, uint32_t M, uint32_t N, uint32_t K, const float* A, const float* B, float* C,
                                const float* bias, int act, float* preact_out) {
    if (N > SKN) return fg_fail(ctx, FG_ERR_INTERNAL, "skinny GEMM: N too large");
    if ((K % 4 == 0) && fg_aligned16(A) && M < (1u << 27)) {
        // sliced: one block per (512-wide k-slice, group of rows); then the slices are folded
        const uint32_t nslices = (K + SK_SLICE - 1) / SK_SLICE;
        void* part;
        int32_t s = fg_ws_alloc(ctx, (uint64_t)nslices * M * 16 * 4, &part);
        if (s != FG_OK) return s;
        // rows per block: 32, 64 or 128, whichever ends soonest on two resident blocks per SM
        const uint64_t slots = 2ull * ctx->sm_count;
        uint32_t rpb = 32;
        uint64_t best = ~0ull;
        for (uint32_t cand = 32; cand <= 128; cand *= 2) {
            const uint64_t blocks = (uint64_t)nslices * ((M + cand - 1) / cand);
            const uint64_t span = ((blocks + slots - 1) / slots) * (cand + 12);     // + the cost of loading the slice of B
            if (span < best) { best = span; rpb = cand; }
        }
        dim3 grid(nslices, (M + rpb - 1) / rpb);
        if (grid.y > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "skinny GEMM: too many rows");
        fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SKINNY, 4.0 * M * K);                 // A read once
        FG_SKINNY_DISPATCH(N, (gemm_skinny_n_slice_kernel<NT><<<grid, 256, 0, ctx->stream>>>(M, N, K, rpb, A, B, (float*)part)));
        FG_LAUNCHED(ctx);
        skinny_fold_slices_kernel<<<(M * 16 + 255) / 256, 256, 0, ctx->stream>>>(M, N, nslices, (const float*)part, bias, act, C, preact_out);
        fg_time_end(ctx, tr);
        FG_LAUNCHED(ctx);
        return FG_OK;
    }
    const uint32_t Kp = (K + 3) / 4 * 4, NTr = (N + 3) / 4 * 4;
    void* bt;
    int32_t s = fg_ws_alloc(ctx, (uint64_t)NTr * Kp * 4, &bt);
    if (s != FG_OK) return s;
    skinny_transpose_kernel<<<(NTr * Kp + 255) / 256, 256, 0, ctx->stream>>>(K, N, Kp, NTr, B, (float*)bt);
    FG_LAUNCHED(ctx);
    const uint32_t blocks = (M + 7) / 8;
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SKINNY, 4.0 * M * K);                 // A read once
    FG_SKINNY_DISPATCH(N, (gemm_skinny_n_kernel<NT, false><<<blocks, 256, 0, ctx->stream>>>(M, N, K, Kp, A, (const float*)bt, C, bias, act, preact_out)));
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

// dA[M, K] = dZ · B^T with dZ [M, N], B [K, N], N <= 16.  With extras->colsum_part, *colsum_rows receives the
// number of partial rows written (at most ceil(M / 32), which is what the caller must have room for).
int32_t fg_gemm_skinny_nt_launch(fg_ctx* ctx, uint32_t M, uint32_t K, uint32_t N, const float* dZ, const float* B,
                                 float* dA, const fg_skinny_extras* extras, uint32_t* colsum_rows) {
    if (N > SKN) return fg_fail(ctx, FG_ERR_INTERNAL, "skinny GEMM: N too large");
    const fg_skinny_extras ex = extras ? *extras : fg_skinny_extras{nullptr, 0, nullptr, 0, nullptr};
    // as many blocks as the SMs hold at once (four or five of 128 threads each, by registers), each walking its
    // share of the 16-row chunks
    const uint32_t gx = (K + 511) / 512, chunks = (M + NT_ROWS - 1) / NT_ROWS;
    // resident blocks per SM, asked of the runtime once per device and kernel variant
    static std::atomic<int> occ[4][64];
    std::atomic<int>& slot = occ[(N <= 4) ? 0 : (N <= 8) ? 1 : (N <= 12) ? 2 : 3][ctx->device & 63];
    int per_sm = slot.load(std::memory_order_acquire);
    if (per_sm == 0) {
        FG_SKINNY_DISPATCH(N, {
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_skinny_nt_kernel<NT>, 128, 0) != cudaSuccess || per_sm < 1) {
                cudaGetLastError();
                per_sm = 4;
            }
        });
        slot.store(per_sm, std::memory_order_release);
    }
    uint32_t gy = (uint32_t)((uint64_t)per_sm * ctx->sm_count / gx);
    if (gy < 1) gy = 1;
    if (gy > chunks) gy = chunks;
    if (gy > (M + 31) / 32) gy = (M + 31) / 32;       // the caller's room for column-sum partials
    if (gy > 65535) gy = 65535;
    if (colsum_rows) *colsum_rows = gy;
    dim3 grid(gx, gy);
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
    // block rows: as many as the SMs hold at once (four blocks of 128 threads per SM), at most one per 64-row chunk
    const uint32_t gx = (Kd + 511) / 512;
    uint32_t nchunks = (uint32_t)(4ull * ctx->sm_count / gx);
    if (nchunks < 1) nchunks = 1;
    if (nchunks > (M + TN_ROWS - 1) / TN_ROWS) nchunks = (M + TN_ROWS - 1) / TN_ROWS;
    void* part;
    int32_t s = fg_ws_alloc(ctx, (uint64_t)nchunks * Kd * N * 4, &part);
    if (s != FG_OK) return s;
    dim3 grid(gx, nchunks);
    const bool vec = (Kd % 4 == 0) && fg_aligned16(A);
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SKINNY, 4.0 * M * Kd);                // A read once
    FG_SKINNY_DISPATCH(N, {
        if (vec) gemm_skinny_tn_partial_kernel<NT, true><<<grid, 128, 0, ctx->stream>>>(M, Kd, N, A, dZ, (float*)part);
        else gemm_skinny_tn_partial_kernel<NT, false><<<grid, 128, 0, ctx->stream>>>(M, Kd, N, A, dZ, (float*)part);
    });
    FG_LAUNCHED(ctx);
    const uint64_t n = (uint64_t)Kd * N;
    fold_chunks_kernel<<<fg_stream_grid(ctx, n * 8, 256, 8), 256, 0, ctx->stream>>>(Kd, N, nchunks, (const float*)part, dB);
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
