// Dense f32 GEMM on the tcgen05 tensor cores with a 3xTF32 split, and the GEMM entry
// points (forward with fused bias + activation epilogue, backward dA / dB / dbias).
//
// What it replaces: the reference's tiled scalar-FMA matmul and its backward edges
// (crates/ferrograd-nn/src/op/matmul/mod.rs:17-188, generic.rs:13-325; dA = dC·Bᵀ via
// transpose_b, dB = Aᵀ·dC via transpose_a, mod.rs:75-101) together with the epilogue
// fusion of trailing elementwise ops (crates/fused_gpu/src/dispatch/backend/kernel/forward.rs:373-457)
// and the activation-derivative factor of the backward chains (op/unary.rs:281-309,
// :453-472, :588-714).
//
// Method.  x = hi + lo with hi = tf32(x), lo = tf32(x - hi); A·B ~= hi·hi + hi·lo + lo·hi,
// accumulated in f32 in tensor memory (the dropped lo·lo term and the rounding of lo are
// both ~2^-23 relative).  A pre-pass writes the hi and lo planes of each operand into the
// scratch arena in K-major form (contraction index contiguous), transposing on the way
// when the operand is stored the other way round; it can also apply dY * act'(saved) so
// the backward GEMMs never see an unfused elementwise pass.  The GEMM kernel is a
// warp-specialised pipeline: one thread issues bulk-tensor loads (no multicast) of the
// four planes of a k-block into 128-byte-swizzled shared memory, one thread issues
// three tcgen05.mma per 8-wide k-step, four warps read the accumulators back with
// tcgen05.ld and apply bias + activation while storing.
//
// Data layout in HBM: planes live in the scratch arena as [2][rows][ld] f32 (plane 0 = hi,
// plane 1 = lo; ld = contraction length rounded up to 4 so row pitches are 16-byte
// multiples).  One 3-D tensor map per operand: dims {contraction, rows, 2},
// box {32, tile rows, 2}, so one load brings the hi and the lo tile of a k-block.
#include "fg_internal.cuh"
#include "ptx_sm100.cuh"

using namespace fgptx;

namespace {

constexpr int BM = 128;         // rows of the output tile = UMMA M
constexpr int BK = 32;          // f32 per k-block: one 128-byte swizzled row
constexpr int UK = 8;           // K of one tcgen05.mma kind::tf32
constexpr long long kWaitCycles = 2000000000LL;   // bound on every device-side wait (about 1 s)

struct Epilogue {
    float* C;
    const float* bias;
    float* preact;
    uint32_t M, N, K;
    int act;
    int* dev_status;
};

template <int BN>
struct TileCfg {
    static constexpr int kABytes = 2 * BM * BK * 4;   // hi + lo tiles of A
    static constexpr int kBBytes = 2 * BN * BK * 4;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = (200 * 1024) / kStageBytes > 6 ? 6 : (200 * 1024) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;   // two accumulators (ping-pong)
    static constexpr int kColsPerThread = BN / 2;                 // each lane quarter is shared by two warps
};

constexpr int kThreads = 320;      // warp 0: loads, warp 1: MMA issue, warps 2..9: accumulate + epilogue
constexpr int kChunkKB = 8;        // k-blocks per accumulation chunk (256 values of k)

// The tensor core adds into its f32 accumulator with truncation, so a long chain of
// tcgen05.mma drifts linearly with K (measured: 1.9e-4 relative at K = 8192).  The K loop is
// therefore cut into chunks of kChunkKB k-blocks.  Each chunk accumulates in one of two
// tensor-memory accumulators, starting from zero; when it completes, the eight epilogue
// warps read it back and add it, rounding to nearest, to running sums held in registers
// while the tensor core is already working on the next chunk in the other accumulator.
template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Epilogue ep) {
    using Cfg = TileCfg<BN>;
    constexpr int S = Cfg::kStages;
    constexpr int CPT = Cfg::kColsPerThread;
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle (descriptor base offset 0).
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - raw);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(base_ptr + S * Cfg::kStageBytes);
    const uint32_t bar0 = base + S * Cfg::kStageBytes;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
    auto acc_full_bar = [&](int b) { return bar0 + 8u * (2 * S + b); };
    auto acc_empty_bar = [&](int b) { return bar0 + 8u * (2 * S + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * S + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const uint32_t nkb = (ep.K + BK - 1) / BK;
    const uint32_t nchunks = (nkb + kChunkKB - 1) / kChunkKB;

    // A wait that expired earlier (this launch or a previous one) makes every CTA leave at once.
    // One thread reads the word so that the whole CTA takes the same branch.
    __shared__ int s_abort;
    if (threadIdx.x == 0) s_abort = *reinterpret_cast<volatile int*>(ep.dev_status);
    __syncthreads();
    if (s_abort != 0) return;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full_bar(b), 1); mbar_init(acc_empty_bar(b), 8); }
        fence_mbar_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: bulk-tensor loads ----
            for (uint32_t kb = 0; kb < nkb; ++kb) {
                const int s = kb % S;
                const uint32_t ph = (kb / S) & 1u;
                if (!mbar_wait_bounded(empty_bar(s), ph ^ 1u, kWaitCycles)) {
                    atomicOr(ep.dev_status, FG_DEVERR_TMA_WAIT);
                    break;
                }
                mbar_expect_tx(full_bar(s), Cfg::kStageBytes);
                const uint32_t sa = base + s * Cfg::kStageBytes;
                tma_load_3d(sa, &tmA, full_bar(s), (int)(kb * BK), (int)m0, 0);
                tma_load_3d(sa + Cfg::kABytes, &tmB, full_bar(s), (int)(kb * BK), (int)n0, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----
            constexpr uint32_t idesc = make_idesc(2u /*tf32*/, BM, BN < 16 ? 16 : BN);
            bool ok = true;
            for (uint32_t c = 0; c < nchunks && ok; ++c) {
                const uint32_t buf = c & 1u;
                // the accumulator must have been drained by the epilogue warps (two chunks ago)
                if (!mbar_wait_bounded(acc_empty_bar(buf), ((c >> 1) & 1u) ^ 1u, kWaitCycles)) {
                    atomicOr(ep.dev_status, FG_DEVERR_MMA_WAIT);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const uint32_t kb_end = min(nkb, (c + 1) * kChunkKB);
                for (uint32_t kb = c * kChunkKB; kb < kb_end; ++kb) {
                    const int s = kb % S;
                    const uint32_t ph = (kb / S) & 1u;
                    if (!mbar_wait_bounded(full_bar(s), ph, kWaitCycles)) {
                        atomicOr(ep.dev_status, FG_DEVERR_MMA_WAIT);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = base + s * Cfg::kStageBytes;
                    const uint64_t a_hi = make_desc_sw128(sa);
                    const uint64_t a_lo = make_desc_sw128(sa + BM * BK * 4);
                    const uint64_t b_hi = make_desc_sw128(sa + Cfg::kABytes);
                    const uint64_t b_lo = make_desc_sw128(sa + Cfg::kABytes + BN * BK * 4);
                    const uint32_t first = (kb == c * kChunkKB) ? 0u : 1u;   // a chunk starts from zero
#pragma unroll
                    for (int kk = 0; kk < BK / UK; ++kk) {
                        // advance along K inside the swizzled row: +32 bytes, i.e. +2 in the address field
                        const uint64_t adv = (uint64_t)(kk * UK * 4 >> 4);
                        mma_tf32(d_tmem, a_lo + adv, b_hi + adv, idesc, first | (uint32_t)kk);
                        mma_tf32(d_tmem, a_hi + adv, b_lo + adv, idesc, 1u);
                        mma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                    }
                    mma_commit(empty_bar(s));   // frees the stage once these MMAs have read it
                }
                if (ok) mma_commit(acc_full_bar(buf));   // this chunk's accumulator is complete
            }
        }
    } else {
        // ---- accumulate + epilogue: warps 2..9.  Warp w may touch TMEM lanes 32*(w%4) .. +31;
        //      warps 2..5 take the first half of the tile's columns, warps 6..9 the second. ----
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        float sum[CPT];
#pragma unroll
        for (int j = 0; j < CPT; ++j) sum[j] = 0.0f;
        bool ok = true;
        for (uint32_t c = 0; c < nchunks; ++c) {
            const uint32_t buf = c & 1u;
            bool got = mbar_wait_bounded(acc_full_bar(buf), (c >> 1) & 1u, kWaitCycles + kWaitCycles / 2);
            got = __all_sync(0xffffffffu, got);
            if (!got) {
                if (lane == 0) atomicOr(ep.dev_status, FG_DEVERR_EPI_WAIT);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + half * CPT;
            if constexpr (CPT >= 32) {
#pragma unroll
                for (int g = 0; g < CPT / 32; ++g) {
                    uint32_t r[32];
                    tmem_ld_32x32(t0 + g * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) sum[g * 32 + j] += __uint_as_float(r[j]);
                }
            } else {
                uint32_t r[16];
                tmem_ld_32x16(t0, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) sum[j] += __uint_as_float(r[j]);
            }
            tc_fence_before();
            if (lane == 0) mbar_arrive(acc_empty_bar(buf));
        }
        if (ok && *reinterpret_cast<volatile int*>(ep.dev_status) == 0) {
            const uint32_t row = m0 + q * 32 + lane;
            const uint32_t cbase = n0 + half * CPT;
            const bool vec_ok = (ep.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(ep.C) & 15u) == 0) &&
                                (!ep.preact || (reinterpret_cast<uintptr_t>(ep.preact) & 15u) == 0);
            if (row < ep.M) {
                float* crow = ep.C + (size_t)row * ep.N;
                float* prow = ep.preact ? ep.preact + (size_t)row * ep.N : nullptr;
#pragma unroll
                for (int j = 0; j < CPT; j += 4) {
                    const uint32_t col = cbase + j;
                    if (col >= ep.N) break;
                    float z[4];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        z[t] = sum[j + t];
                        if (ep.bias && col + t < ep.N) z[t] += ep.bias[col + t];
                    }
                    if (vec_ok && col + 3 < ep.N) {
                        if (prow) *reinterpret_cast<float4*>(prow + col) = make_float4(z[0], z[1], z[2], z[3]);
                        *reinterpret_cast<float4*>(crow + col) =
                            make_float4(fg_act_fwd(ep.act, z[0]), fg_act_fwd(ep.act, z[1]),
                                        fg_act_fwd(ep.act, z[2]), fg_act_fwd(ep.act, z[3]));
                    } else {
#pragma unroll
                        for (int t = 0; t < 4; ++t)
                            if (col + t < ep.N) {
                                if (prow) prow[col + t] = z[t];
                                crow[col + t] = fg_act_fwd(ep.act, z[t]);
                            }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ------------------------------------------------------------------------------------
// Pre-pass: hi/lo planes of X [R, C] (row-major), optionally of dY * act'(saved).
//   planes_n: [2][R][ldn]   (same orientation; contraction index = column)
//   planes_t: [2][C][ldt]   (transposed;       contraction index = row)
// 32x32 tiles, 32x8 threads.
// ------------------------------------------------------------------------------------
struct SplitArgs {
    const float* x;
    const float* saved;    // non-NULL: value = x * act'(saved)
    int act;
    uint32_t R, C;
    float* planes_n; uint32_t ldn;
    float* planes_t; uint32_t ldt;
    float* value_out;      // optional copy of the (fused) value, [R, C]
};

__global__ void __launch_bounds__(256) split_kernel(SplitArgs a) {
    __shared__ float thi[32][33];
    __shared__ float tlo[32][33];
    const uint32_t c = blockIdx.x * 32 + threadIdx.x;
    const uint32_t r0 = blockIdx.y * 32;
    const size_t plane_n = (size_t)a.R * a.ldn, plane_t = (size_t)a.C * a.ldt;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t r = r0 + threadIdx.y + i * 8;
        float hi = 0.0f, lo = 0.0f;
        if (r < a.R && c < a.C) {
            const size_t idx = (size_t)r * a.C + c;
            float v = a.x[idx];
            if (a.saved) v = v * fg_act_grad(a.act, a.saved[idx]);
            if (a.value_out) a.value_out[idx] = v;
            hi = __uint_as_float(cvt_tf32(v));
            lo = __uint_as_float(cvt_tf32(v - hi));
            if (a.planes_n) {
                a.planes_n[(size_t)r * a.ldn + c] = hi;
                a.planes_n[plane_n + (size_t)r * a.ldn + c] = lo;
            }
        }
        thi[threadIdx.y + i * 8][threadIdx.x] = hi;
        tlo[threadIdx.y + i * 8][threadIdx.x] = lo;
    }
    if (!a.planes_t) return;
    __syncthreads();
    const uint32_t tr = r0 + threadIdx.x;          // source row -> destination column
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t tc = blockIdx.x * 32 + threadIdx.y + i * 8;   // source column -> destination row
        if (tc < a.C && tr < a.R) {
            a.planes_t[(size_t)tc * a.ldt + tr] = thi[threadIdx.x][threadIdx.y + i * 8];
            a.planes_t[plane_t + (size_t)tc * a.ldt + tr] = tlo[threadIdx.x][threadIdx.y + i * 8];
        }
    }
}

inline uint32_t round4(uint32_t v) { return (v + 3u) & ~3u; }
inline uint64_t planes_bytes(uint32_t rows, uint32_t contraction) { return 2ull * rows * round4(contraction) * 4ull; }

int32_t launch_split(fg_ctx* ctx, const SplitArgs& a) {
    dim3 grid((a.C + 31) / 32, (a.R + 31) / 32), block(32, 8);
    if (grid.y > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "GEMM operand has too many rows");
    double bytes = 4.0 * a.R * a.C * (1.0 + (a.saved ? 1.0 : 0.0) + (a.value_out ? 1.0 : 0.0) +
                                      (a.planes_n ? 2.0 : 0.0) + (a.planes_t ? 2.0 : 0.0));
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SPLIT, bytes);
    split_kernel<<<grid, block, 0, ctx->stream>>>(a);
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

typedef CUresult (*pfn_encode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map over planes [2][rows][ld] with contraction extent `kdim`; box {32, box_rows, 2}.
int32_t make_tmap(fg_ctx* ctx, CUtensorMap* out, const float* planes, uint32_t rows, uint32_t kdim, uint32_t ld,
                  uint32_t box_rows) {
    if (!ctx->tmap_encode) return fg_fail(ctx, FG_ERR_UNSUPPORTED_FEATURE, "cuTensorMapEncodeTiled unavailable");
    cuuint64_t dims[3] = {kdim, rows, 2};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 4, (cuuint64_t)rows * ld * 4};
    cuuint32_t box[3] = {BK, box_rows, 2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = ((pfn_encode)ctx->tmap_encode)(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)planes, dims, strides,
                                                box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(ctx->err, sizeof(ctx->err), "cuTensorMapEncodeTiled failed with code %d", (int)r);
        return FG_ERR_INTERNAL;
    }
    return FG_OK;
}

template <int BN>
int32_t launch_tc(fg_ctx* ctx, const float* a_planes, uint32_t lda, const float* b_planes, uint32_t ldb,
                  const Epilogue& ep) {
    using Cfg = TileCfg<BN>;
    CUtensorMap tmA, tmB;
    int32_t s = make_tmap(ctx, &tmA, a_planes, ep.M, ep.K, lda, BM);
    if (s != FG_OK) return s;
    s = make_tmap(ctx, &tmB, b_planes, ep.N, ep.K, ldb, BN);
    if (s != FG_OK) return s;
    static uint64_t attr_done = 0;   // one bit per device
    if (!(attr_done >> (ctx->device & 63) & 1ull)) {
        FG_CUDA(ctx, FG_ERR_INTERNAL,
                cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_done |= 1ull << (ctx->device & 63);
    }
    dim3 grid((ep.N + BN - 1) / BN, (ep.M + BM - 1) / BM);
    if (grid.y > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "GEMM: M too large");
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_GEMM_TC, 2.0 * ep.M * ep.N * ep.K);
    gemm_tc_kernel<BN><<<grid, kThreads, Cfg::kSmemBytes, ctx->stream>>>(tmA, tmB, ep);
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

// C[M,N] = act(Aop·Bopᵀ + bias) where Aop planes are [2][M][lda] and Bop planes [2][N][ldb].
int32_t tc_gemm(fg_ctx* ctx, const float* a_planes, uint32_t lda, const float* b_planes, uint32_t ldb, uint32_t M,
                uint32_t N, uint32_t K, float* C, const float* bias, int act, float* preact) {
    Epilogue ep{C, bias, preact, M, N, K, act, ctx->dev_status};
    // Widest tile that still fills the machine; narrow N gets a narrow tile.
    const uint64_t tiles256 = (uint64_t)((M + BM - 1) / BM) * ((N + 255) / 256);
    if (N > 128 && tiles256 >= (uint64_t)ctx->sm_count) return launch_tc<256>(ctx, a_planes, lda, b_planes, ldb, ep);
    if (N > 64) return launch_tc<128>(ctx, a_planes, lda, b_planes, ldb, ep);
    if (N > 32) return launch_tc<64>(ctx, a_planes, lda, b_planes, ldb, ep);
    return launch_tc<32>(ctx, a_planes, lda, b_planes, ldb, ep);
}

bool use_tensor_cores(const fg_ctx* ctx, int mode, uint32_t M, uint32_t N, uint32_t K) {
    if (mode == FG_GEMM_SIMT) return false;
    if (mode == FG_GEMM_3XTF32) return true;
    if (!ctx->tmap_encode) return false;
    return M >= 64 && (uint64_t)M * N * K >= (1ull << 22);
}

}  // namespace

extern "C" {

int32_t fg_gemm_f32(fg_ctx* ctx, int32_t mode, int32_t transA, int32_t transB, uint32_t M, uint32_t N, uint32_t K,
                    const float* A, const float* B, float* C, const float* bias, int32_t act, float* preact_out) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, A && B && C, "fg_gemm_f32: NULL operand");
    FG_REQUIRE(ctx, M >= 1 && N >= 1 && K >= 1, "fg_gemm_f32: dimensions must be >= 1");
    FG_REQUIRE(ctx, mode >= FG_GEMM_AUTO && mode <= FG_GEMM_3XTF32, "fg_gemm_f32: unknown mode");
    FG_REQUIRE(ctx, act >= FG_ACT_NONE && act <= FG_ACT_GELU, "fg_gemm_f32: unknown activation");
    FG_REQUIRE(ctx, (uint64_t)M * N < (1ull << 40) && (uint64_t)M * K < (1ull << 40) && (uint64_t)N * K < (1ull << 40),
               "fg_gemm_f32: operand too large");
    if (!use_tensor_cores(ctx, mode, M, N, K))
        return fg_gemm_simt_launch(ctx, transA, transB, M, N, K, A, B, C, bias, act, preact_out);
    const uint32_t ld = round4(K);
    void *pa, *pb;
    // Size the arena for both operands before carving it.
    if (ctx->ws_bytes < planes_bytes(M, K) + planes_bytes(N, K) + 512) {
        int32_t s0 = fg_ctx_reserve_workspace(ctx, planes_bytes(M, K) + planes_bytes(N, K) + 512);
        if (s0 != FG_OK) return s0;
    }
    int32_t s = fg_ws_alloc(ctx, planes_bytes(M, K), &pa);
    if (s != FG_OK) return s;
    s = fg_ws_alloc(ctx, planes_bytes(N, K), &pb);
    if (s != FG_OK) return s;
    // A operand: [M, K] with K contiguous.
    SplitArgs sa{};
    sa.x = A;
    if (!transA) { sa.R = M; sa.C = K; sa.planes_n = (float*)pa; sa.ldn = ld; }
    else         { sa.R = K; sa.C = M; sa.planes_t = (float*)pa; sa.ldt = ld; }
    s = launch_split(ctx, sa);
    if (s != FG_OK) return s;
    // B operand: [N, K] with K contiguous.
    SplitArgs sb{};
    sb.x = B;
    if (!transB) { sb.R = K; sb.C = N; sb.planes_t = (float*)pb; sb.ldt = ld; }
    else         { sb.R = N; sb.C = K; sb.planes_n = (float*)pb; sb.ldn = ld; }
    s = launch_split(ctx, sb);
    if (s != FG_OK) return s;
    return tc_gemm(ctx, (const float*)pa, ld, (const float*)pb, ld, M, N, K, C, bias, act, preact_out);
}

int32_t fg_gemm_bwd_f32(fg_ctx* ctx, int32_t mode, uint32_t M, uint32_t N, uint32_t K, const float* A, const float* B,
                        const float* dY, int32_t act, const float* saved, float* dA, float* dB, float* dbias,
                        float* dZ_out) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, dY != nullptr, "fg_gemm_bwd_f32: dY is NULL");
    FG_REQUIRE(ctx, M >= 1 && N >= 1 && K >= 1, "fg_gemm_bwd_f32: dimensions must be >= 1");
    FG_REQUIRE(ctx, mode >= FG_GEMM_AUTO && mode <= FG_GEMM_3XTF32, "fg_gemm_bwd_f32: unknown mode");
    FG_REQUIRE(ctx, act >= FG_ACT_NONE && act <= FG_ACT_GELU, "fg_gemm_bwd_f32: unknown activation");
    FG_REQUIRE(ctx, act == FG_ACT_NONE || saved, "fg_gemm_bwd_f32: the activation backward needs the saved tensor");
    FG_REQUIRE(ctx, !dA || B, "fg_gemm_bwd_f32: dA needs B");
    FG_REQUIRE(ctx, !dB || A, "fg_gemm_bwd_f32: dB needs A");
    const bool fuse = act != FG_ACT_NONE;
    const bool tc = use_tensor_cores(ctx, mode, M, N, K);
    const uint64_t mn = (uint64_t)M * N;

    if (!tc) {
        // Exact path: materialise dZ, then two SIMT GEMMs.
        const float* dz = dY;
        {
            uint64_t need = mn * 4 + (uint64_t)((M + 255) / 256) * N * 4 + 1024;
            if (ctx->ws_bytes < need) {
                int32_t s0 = fg_ctx_reserve_workspace(ctx, need);
                if (s0 != FG_OK) return s0;
            }
        }
        if (fuse || dZ_out) {
            float* buf = dZ_out;
            if (!buf) {
                void* p;
                int32_t s = fg_ws_alloc(ctx, mn * 4, &p);
                if (s != FG_OK) return s;
                buf = (float*)p;
            }
            if (fuse) {
                int32_t s = fg_act_bwd_launch(ctx, mn, act, dY, saved, buf);
                if (s != FG_OK) return s;
            } else {
                FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY,
                        cudaMemcpyAsync(buf, dY, mn * 4, cudaMemcpyDeviceToDevice, ctx->stream));
            }
            dz = buf;
        }
        if (dA) { int32_t s = fg_gemm_simt_launch(ctx, 0, 1, M, K, N, dz, B, dA, nullptr, FG_ACT_NONE, nullptr); if (s) return s; }
        if (dB) { int32_t s = fg_gemm_simt_launch(ctx, 1, 0, K, N, M, A, dz, dB, nullptr, FG_ACT_NONE, nullptr); if (s) return s; }
        if (dbias) { int32_t s = fg_colsum_launch(ctx, M, N, dz, dbias); if (s) return s; }
        return FG_OK;
    }

    // Tensor-core path.  Scratch: dZ planes in both orientations, B planes, Aᵀ planes, dZ itself
    // when a bias gradient is wanted, and the column-sum partials.
    const uint32_t ld_n = round4(N), ld_m = round4(M);
    uint64_t need = 1024;
    if (dA) need += planes_bytes(M, N) + planes_bytes(K, N) + 512;
    if (dB) need += planes_bytes(N, M) + planes_bytes(K, M) + 512;
    if (dbias && !dZ_out) need += mn * 4 + 256;
    if (dbias) need += (uint64_t)((M + 255) / 256) * N * 4 + 256;
    if (ctx->ws_bytes < need) {
        int32_t s0 = fg_ctx_reserve_workspace(ctx, need);
        if (s0 != FG_OK) return s0;
    }
    void *dz_n = nullptr, *dz_t = nullptr, *b_n = nullptr, *a_t = nullptr, *dz_val = dZ_out;
    int32_t s;
    if (dA) {
        if ((s = fg_ws_alloc(ctx, planes_bytes(M, N), &dz_n)) != FG_OK) return s;
        if ((s = fg_ws_alloc(ctx, planes_bytes(K, N), &b_n)) != FG_OK) return s;
    }
    if (dB) {
        if ((s = fg_ws_alloc(ctx, planes_bytes(N, M), &dz_t)) != FG_OK) return s;
        if ((s = fg_ws_alloc(ctx, planes_bytes(K, M), &a_t)) != FG_OK) return s;
    }
    if (dbias && !dz_val) {
        if ((s = fg_ws_alloc(ctx, mn * 4, &dz_val)) != FG_OK) return s;
    }
    SplitArgs sz{};
    sz.x = dY; sz.saved = fuse ? saved : nullptr; sz.act = act; sz.R = M; sz.C = N;
    sz.planes_n = (float*)dz_n; sz.ldn = ld_n;
    sz.planes_t = (float*)dz_t; sz.ldt = ld_m;
    sz.value_out = (float*)dz_val;
    if ((s = launch_split(ctx, sz)) != FG_OK) return s;
    if (dA) {
        // dA[M,K] = dZ[M,N] · Bᵀ: contraction over N; B [K,N] is already "rows = K, contraction contiguous".
        SplitArgs sb{};
        sb.x = B; sb.R = K; sb.C = N; sb.planes_n = (float*)b_n; sb.ldn = ld_n;
        if ((s = launch_split(ctx, sb)) != FG_OK) return s;
        if ((s = tc_gemm(ctx, (const float*)dz_n, ld_n, (const float*)b_n, ld_n, M, K, N, dA, nullptr, FG_ACT_NONE, nullptr)) != FG_OK) return s;
    }
    if (dB) {
        // dB[K,N] = Aᵀ · dZ: contraction over M; operands are Aᵀ [K,M] and dZᵀ [N,M].
        SplitArgs sa{};
        sa.x = A; sa.R = M; sa.C = K; sa.planes_t = (float*)a_t; sa.ldt = ld_m;
        if ((s = launch_split(ctx, sa)) != FG_OK) return s;
        if ((s = tc_gemm(ctx, (const float*)a_t, ld_m, (const float*)dz_t, ld_m, K, N, M, dB, nullptr, FG_ACT_NONE, nullptr)) != FG_OK) return s;
    }
    if (dbias) {
        if ((s = fg_colsum_launch(ctx, M, N, (const float*)dz_val, dbias)) != FG_OK) return s;
    }
    return FG_OK;
}

}  // extern "C"
