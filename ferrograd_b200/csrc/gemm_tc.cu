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
#include <atomic>
#include <cuda_bf16.h>
#include <stdlib.h>

#include "fg_internal.cuh"
#include "ptx_sm100.cuh"

using namespace fgptx;

namespace {

constexpr int BM = 128;         // rows of the output tile = UMMA M
// BK (template parameter): f32 per k-block = one swizzled shared-memory row: 32 (128-byte swizzle) or 16 (64-byte).
constexpr int UK = 8;           // K of one tcgen05.mma kind::tf32
constexpr long long kWaitCycles = 2000000000LL;   // bound on every device-side wait (about 1 s)

struct Epilogue {
    float* C;
    const float* bias;
    float* preact;
    uint32_t M, N, K;
    int act;
    int* dev_status;
    // Split-K tail of the pair kernel: tiles [0, t_full) are whole; each later tile is computed as `split`
    // partial sums over equal shares of the K chunks, written raw to `partial` and folded by a second kernel.
    float* partial;
    uint32_t t_full, split;
    int out_dtype;       // storage type of C and preact (fg_dtype); bias and partial are always f32
    // ---- pair kernel on f32 tensors with bf16 pairs (FMT 1) ----
    uint32_t a_mn, b_mn;              // the operand's storage has the non-contraction index contiguous
    __nv_bfloat16* c_pairs;           // optional: bf16 pairs of the stored C (see pairs_kernel)
    uint64_t c_pairs_stride;          // elements between the two planes of c_pairs
    const float* mul_saved;           // optional [M,N]: C = (acc + bias) * act'(mul_saved), act = mul_act
    int mul_act;
    float* colsum_part;               // optional [ceil(M/32)][N]: column sums of the stored C per 32-row block
    uint32_t group;                   // pair kernel: tile rows per group of the tile order (see pair_tile_origin)
#ifdef FG_GEMM_PROFILE
    uint32_t dbg;                     // diagnostic build: bit 0 = leave out the global stores of the epilogue
#endif
};

// Element stores in the output's storage type (idx in elements).
__device__ __forceinline__ void store_out4(void* base, size_t idx, float4 v, int dt) {
    if (dt == FG_DTYPE_F32) {
        *reinterpret_cast<float4*>(static_cast<float*>(base) + idx) = v;
    } else if (dt == FG_DTYPE_F16) {
        const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<const uint32_t*>(&lo);
        u.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(static_cast<__half*>(base) + idx) = u;
    } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<const uint32_t*>(&lo);
        u.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(base) + idx) = u;
    }
}
__device__ __forceinline__ void store_out1(void* base, size_t idx, float v, int dt) {
    if (dt == FG_DTYPE_F32) static_cast<float*>(base)[idx] = v;
    else if (dt == FG_DTYPE_F16) static_cast<__half*>(base)[idx] = __float2half_rn(v);
    else static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
}

// Origin of pair tile `tile`: tiles are numbered so that eight consecutive pair-rows sweep all columns
// before the next eight start.  The pairs working at the same time then cover a squarish block of C and
// re-use both its A rows and its B rows from L2 (with rows-fastest order every wave streamed all of A
// again: 7.7x the operand bytes from DRAM at 8192^3).
__host__ __device__ __forceinline__ void pair_tile_origin(uint32_t tile, uint32_t pairs_m, uint32_t pairs_n,
                                                          uint32_t tile_m, uint32_t tile_n, uint32_t kGroup, uint32_t& m0,
                                                          uint32_t& n0) {
    const uint32_t grp = tile / (kGroup * pairs_n);
    const uint32_t left = pairs_m - grp * kGroup;
    const uint32_t grp_rows = left < kGroup ? left : kGroup;
    const uint32_t rem = tile - grp * kGroup * pairs_n;
    m0 = (grp * kGroup + rem % grp_rows) * tile_m;
    n0 = (rem / grp_rows) * tile_n;
}

// One shared copy of the activation code.  fg_act_fwd inlines tanhf and the GELU polynomial at every call
// site; an epilogue that is unrolled over a thread's 128 accumulators would carry 128 copies and run out
// of instruction cache (measured on the pair kernel: 45,000 cycles for ~1,000 useful instructions).
__device__ __noinline__ float4 act_fwd4(int act, float4 z) {
    return make_float4(fg_act_fwd_fast(act, z.x), fg_act_fwd_fast(act, z.y), fg_act_fwd_fast(act, z.z), fg_act_fwd_fast(act, z.w));
}
// z * act'(saved): the backward factor of the layer below, applied while a dA tile is stored.
__device__ __noinline__ float4 act_mul4(int act, float4 z, float4 sv) {
    return make_float4(z.x * fg_act_grad_fast(act, sv.x), z.y * fg_act_grad_fast(act, sv.y), z.z * fg_act_grad_fast(act, sv.z),
                       z.w * fg_act_grad_fast(act, sv.w));
}

// Four columns of one row, element by element: the ragged right edge of a matrix whose width is not a multiple
// of four, or unaligned pointers.  A cold path, kept out of line so that it does not sit in the unrolled epilogue.
__device__ __noinline__ float4 epi_store_edge(float4 zin, size_t off, uint32_t col, uint32_t col_lim, char* out, char* pre,
                                               __nv_bfloat16* pairs, uint64_t pairs_stride, const float* mul, int mul_act, int act,
                                               int odt) {
    const float z[4] = {zin.x, zin.y, zin.z, zin.w};
    float o4[4] = {0.f, 0.f, 0.f, 0.f};
    for (int t = 0; t < 4; ++t)
        if (col + t < col_lim) {
            const float o = mul ? z[t] * fg_act_grad_fast(mul_act, mul[off + t]) : fg_act_fwd_fast(act, z[t]);
            if (pre) store_out1(pre, off + t, z[t], odt);
            store_out1(out, off + t, o, odt);
            if (pairs) fg_store_pairs1(pairs, pairs_stride, off + t, o);
            o4[t] = o;
        }
    return make_float4(o4[0], o4[1], o4[2], o4[3]);
}

template <int BN, int BK>
struct TileCfg {
    static constexpr int kABytes = 2 * BM * BK * 4;   // hi + lo tiles of A
    static constexpr int kBBytes = 2 * BN * BK * 4;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = (200 * 1024) / kStageBytes > 8 ? 8 : (200 * 1024) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;   // two accumulators (ping-pong)
    static constexpr int kColsPerThread = BN / 2;                 // each lane quarter is shared by two warps
};

#ifdef FG_GEMM_PROFILE
// Diagnostic build only (-DFG_GEMM_PROFILE): cycle counters of the pair kernel's roles, summed over CTAs.
// 0 MMA wait for a drained accumulator, 1 MMA wait for loads, 2 MMA loop total, 3 epilogue (warp 2) wait for a
// finished chunk, 4 epilogue store phase, 5 units, 6 producer wait for a free stage, 7 reporting CTAs.
__device__ unsigned long long g_prof[8];
#define PROF_T0() const long long _pt0 = clock64()
#define PROF_ADD(var) var += clock64() - _pt0
#else
#define PROF_T0()
#define PROF_ADD(var)
#endif

constexpr int kThreads = 320;      // warp 0: loads, warp 1: MMA issue, warps 2..9: accumulate + epilogue
// The pair kernel runs three warpgroups: warps 0..3 (loads, MMA issue, two idle warps) keep kPairRegsLow registers
// per thread, the eight accumulate + epilogue warps 4..11 take kPairRegsHigh.  A thread of those owns 128 running
// sums; with the 168 registers a 384-thread CTA gets by default, the store phase spilled, and with 227 KB of the
// SM's memory configured as shared memory there is next to no L1 behind local memory: every spill access cost an
// L2 round trip (measured: ~50 cycles per instruction in the store phase, 20,000 cycles per tile).
constexpr int kPairThreads = 384;
constexpr int kPairRegsLow = 72, kPairRegsHigh = 216;     // 128 * 72 + 256 * 216 = 64,512 <= 65,536
constexpr int kPairEpiWarp0 = 4;
constexpr int kChunkK = 256;       // values of k per accumulation chunk

// The tensor core adds into its f32 accumulator with truncation, so a long chain of
// tcgen05.mma drifts linearly with K (measured: 1.9e-4 relative at K = 8192).  The K loop is
// therefore cut into chunks of kChunkK values of k.  Each chunk accumulates in one of two
// tensor-memory accumulators, starting from zero; when it completes, the eight epilogue
// warps read it back and add it, rounding to nearest, to running sums held in registers
// while the tensor core is already working on the next chunk in the other accumulator.
//
// FMT selects the operand planes and the MMA sequence per k-block:
//   0  [hi | lo] f32 planes; three kind::tf32 MMAs per 8-wide k-step (lo*hi, hi*lo, hi*hi): "3xTF32".
//   1  hi as f32 (tf32-rounded) plus a bf16 pair [bf16(x) | bf16(x - hi)]; the dominant term hi*hi
//      runs as kind::tf32, the two cross terms as kind::f16 (bf16) MMAs, which take half the time of a
//      tf32 MMA per k: two tf32-units of tensor work per product instead of three.  The cross terms
//      are 2^-12 of the product, so bf16's 2^-9 relative rounding costs ~2^-20 relative per product.
template <int BN, int BK, int FMT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmA16, const __grid_constant__ CUtensorMap tmB16, Epilogue ep) {
    static_assert(FMT == 0 || BK == 32, "the bf16 planes use 64-byte rows: 32 values of k per block");
    using Cfg = TileCfg<BN, BK>;
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
    constexpr uint32_t kChunkKB = kChunkK / BK;   // k-blocks per accumulation chunk
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
        if (FMT == 1) { prefetch_tmap(&tmA16); prefetch_tmap(&tmB16); }
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
                if (FMT == 1) {   // the bf16 pairs follow their operand's f32 tile
                    tma_load_3d(sa + BM * BK * 4, &tmA16, full_bar(s), (int)(kb * BK), (int)m0, 0);
                    tma_load_3d(sa + Cfg::kABytes + BN * BK * 4, &tmB16, full_bar(s), (int)(kb * BK), (int)n0, 0);
                }
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
                    const uint64_t a_hi = make_desc_kmajor<BK * 4>(sa);
                    const uint64_t a_lo = make_desc_kmajor<BK * 4>(sa + BM * BK * 4);
                    const uint64_t b_hi = make_desc_kmajor<BK * 4>(sa + Cfg::kABytes);
                    const uint64_t b_lo = make_desc_kmajor<BK * 4>(sa + Cfg::kABytes + BN * BK * 4);
                    const uint32_t first = (kb == c * kChunkKB) ? 0u : 1u;   // a chunk starts from zero
                    if (FMT == 0) {
#pragma unroll
                        for (int kk = 0; kk < BK / UK; ++kk) {
                            // advance along K inside the swizzled row: +32 bytes, i.e. +2 in the address field
                            const uint64_t adv = (uint64_t)(kk * UK * 4 >> 4);
                            mma_tf32(d_tmem, a_lo + adv, b_hi + adv, idesc, first | (uint32_t)kk);
                            mma_tf32(d_tmem, a_hi + adv, b_lo + adv, idesc, 1u);
                            mma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                        }
                    } else {
                        // bf16 tiles: rows of 64 bytes (32 values of k), two 16-wide k-steps of 32 bytes each
                        constexpr uint32_t idesc16 = make_idesc(1u /*bf16*/, BM, BN < 16 ? 16 : BN);
                        const uint32_t a16 = sa + BM * BK * 4, b16 = sa + Cfg::kABytes + BN * BK * 4;
                        const uint64_t a_h16 = make_desc_kmajor<64>(a16), a_l16 = make_desc_kmajor<64>(a16 + BM * BK * 2);
                        const uint64_t b_h16 = make_desc_kmajor<64>(b16), b_l16 = make_desc_kmajor<64>(b16 + BN * BK * 2);
#pragma unroll
                        for (int kk = 0; kk < BK / 16; ++kk) {
                            const uint64_t adv = (uint64_t)(kk * 16 * 2 >> 4);
                            mma_f16(d_tmem, a_l16 + adv, b_h16 + adv, idesc16, first | (uint32_t)kk);
                            mma_f16(d_tmem, a_h16 + adv, b_l16 + adv, idesc16, 1u);
                        }
#pragma unroll
                        for (int kk = 0; kk < BK / UK; ++kk) {
                            const uint64_t adv = (uint64_t)(kk * UK * 4 >> 4);
                            mma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                        }
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
                    const float4 o = ep.act == FG_ACT_NONE ? make_float4(z[0], z[1], z[2], z[3])
                                                           : act_fwd4(ep.act, make_float4(z[0], z[1], z[2], z[3]));
                    if (vec_ok && col + 3 < ep.N) {
                        if (prow) *reinterpret_cast<float4*>(prow + col) = make_float4(z[0], z[1], z[2], z[3]);
                        *reinterpret_cast<float4*>(crow + col) = o;
                    } else {
                        const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                        for (int t = 0; t < 4; ++t)
                            if (col + t < ep.N) {
                                if (prow) prow[col + t] = z[t];
                                crow[col + t] = ov[t];
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
// CTA-pair kernel (cta_group::2): two CTAs on neighbouring SMs compute one 256 x 256 tile.
// Each CTA loads its own 128 rows of A and HALF of the B tile (128 of its 256 rows); the
// pair's MMA reads both halves, so the bytes each SM pulls from L2 per k-block drop from
// 96 KiB to 64 KiB.  (The single-CTA kernel is limited by exactly that stream: it takes the
// same time with two thirds of the tensor work.)  CTA 0 of the pair issues all MMAs; both
// CTAs keep their 128 rows of the accumulators in their own tensor memory and run their own
// epilogue.  Loads carry no multicast; the only cross-CTA traffic is signalling
// (load-completion bytes counted on the leader's mbarrier, commit arrivals on both CTAs'
// mbarriers, accumulator-drained arrivals on the leader's mbarrier).
// ------------------------------------------------------------------------------------
constexpr long long kPairWaitCycles = 400000000LL;   // about 0.2 s

template <int BK, int FMT>
struct PairCfg {
    static constexpr int kBN = 256;
    static constexpr int kPlanes = FMT >= 2 ? 1 : 2;         // 16-bit operands are loaded as they are: one 128-byte row
    static constexpr int kABytes = kPlanes * BM * BK * 4;          // this CTA's 128 rows of A: hi + lo (or f32 + bf16 pair)
    static constexpr int kBBytes = kPlanes * (kBN / 2) * BK * 4;   // this CTA's half of the B tile
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = (200 * 1024) / kStageBytes > 8 ? 8 : (200 * 1024) / kStageBytes;
    static constexpr int kStoreBytes = 8 * 32 * 32 * 4;       // the epilogue warps' staging blocks (32 x 32 f32 each)
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + kStoreBytes;
    static_assert(kSmemBytes <= 232448, "exceeds the 227 KB a CTA may use");
    static constexpr int kTmemCols = 512;                     // two 256-column accumulators
};

// Persistent: the grid is one CTA pair per SM pair (or fewer); pair p computes tiles p, p + P, p + 2P, ...
// The load ring, the MMA issue and the accumulator ping-pong run straight across tile boundaries, so
// while the epilogue warps apply bias/activation and store tile t from their registers, the loads and
// MMAs of tile t+1 are already under way (per-tile set-up, fill and store cost 20-55 us per wave when
// every tile was its own CTA pair: 17 % of a 4096^3 GEMM, more than half of a K = 784 one).
template <int BK, int FMT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmA16, const __grid_constant__ CUtensorMap tmB16, Epilogue ep) {
    static_assert(FMT == 0 || BK == 32, "the bf16 planes use 64-byte rows: 32 values of k per block");
    // FMT 2 (bf16) and 3 (f16): the operands ARE 16-bit tensors, loaded as they lie (K-major, 64 values of
    // k = one 128-byte row per k-block) and multiplied by one kind::f16 MMA per 16 values of k.
    constexpr bool kDirect16 = FMT >= 2;
    constexpr uint32_t KBE = kDirect16 ? 2 * BK : BK;            // values of k per k-block
    constexpr uint32_t kChunk = kDirect16 ? 1024 : kChunkK;      // 16-bit results tolerate the longer chain
    using Cfg = PairCfg<BK, FMT>;
    constexpr int BN = Cfg::kBN, HB = BN / 2;
    constexpr int S = Cfg::kStages;
    constexpr int CPT = BN / 2;
    extern __shared__ unsigned char smem_raw[];
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
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const uint32_t pairs_m = (ep.M + 2 * BM - 1) / (2 * BM), pairs_n = (ep.N + BN - 1) / BN;
    const uint32_t ntiles = pairs_m * pairs_n;
    const uint32_t npairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
    auto tile_origin = [&](uint32_t tile, uint32_t& m0, uint32_t& n0) {
        pair_tile_origin(tile, pairs_m, pairs_n, 2 * BM, BN, ep.group, m0, n0);
        m0 += rank * BM;                                               // this CTA's rows of A and C
    };
    const uint32_t nkb = (ep.K + KBE - 1) / KBE;
    constexpr uint32_t kChunkKB = kChunk / KBE;
    const uint32_t nchunks = (nkb + kChunkKB - 1) / kChunkKB;
    // Work units: whole tiles first, then the tail tiles in `split` K-shares each (the host sizes the
    // tail so that it fills one last wave instead of leaving most pairs idle for a whole tile time).
    const uint32_t nunits = ep.t_full + (ntiles - ep.t_full) * ep.split;
    auto unit_at = [&](uint32_t u, uint32_t& tile, uint32_t& c0, uint32_t& c1, uint32_t& slot) -> bool {
        if (u < ep.t_full) { tile = u; c0 = 0; c1 = nchunks; slot = 0; return false; }
        const uint32_t v = u - ep.t_full, p = v % ep.split;
        tile = ep.t_full + v / ep.split;
        c0 = p * nchunks / ep.split;
        c1 = (p + 1) * nchunks / ep.split;
        slot = v;
        return true;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full_bar(b), 1); mbar_init(acc_empty_bar(b), 16); }
        fence_mbar_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
        if (FMT >= 1) { prefetch_tmap(&tmA16); prefetch_tmap(&tmB16); }
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();      // the peer's barriers exist before anything is signalled across CTAs
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < kPairEpiWarp0) {
    reg_release<kPairRegsLow>();
    if (warp == 0) {
        if (lane == 0) {
            // ---- producer (both CTAs): own rows of A, own half of B; completion counted on the leader ----
            uint32_t g = 0;      // k-blocks issued so far, across tiles: ring position and phase
            bool ok = true;
            long long prof_a = 0;
            (void)prof_a;
            for (uint32_t u = pair; u < nunits && ok; u += npairs) {
                uint32_t tile, c0, c1, slot, m0, n0;
                unit_at(u, tile, c0, c1, slot);
                tile_origin(tile, m0, n0);
                const uint32_t nb0 = n0 + rank * HB;                    // the rows of B this CTA loads
                const uint32_t kb_last = min(nkb, c1 * kChunkKB);
                for (uint32_t kb = c0 * kChunkKB; kb < kb_last; ++kb, ++g) {
                    const int s = g % S;
                    const uint32_t ph = (g / S) & 1u;
                    {
                        PROF_T0();
                        const bool got = mbar_wait_bounded(empty_bar(s), ph ^ 1u, kPairWaitCycles);
                        PROF_ADD(prof_a);
                        if (!got) {
                            atomicOr(ep.dev_status, FG_DEVERR_TMA_WAIT);
                            ok = false;
                            break;
                        }
                    }
                    const uint32_t lf = map_to_cta(full_bar(s), 0);
                    const uint32_t sa = base + s * Cfg::kStageBytes;
                    if (kDirect16) {
                        if (leader) mbar_expect_tx(full_bar(s), 2 * Cfg::kStageBytes);   // both CTAs' bytes
                        tma_load_3d_pair(sa, &tmA16, lf, (int)(kb * KBE), (int)m0, 0);
                        tma_load_3d_pair(sa + Cfg::kABytes, &tmB16, lf, (int)(kb * KBE), (int)nb0, 0);
                        continue;
                    }
                    if (leader) mbar_expect_tx(full_bar(s), 2 * Cfg::kStageBytes);   // both CTAs' bytes
                    if (FMT == 1) {
                        // One operand tile = 128 rows x 32 values of k as f32 (16 KiB) followed by its two
                        // bf16 planes (2 x 8 KiB).  K-major storage: one box each.  MN-major storage
                        // ([k][rows]): the f32 tile arrives as four boxes of 32 rows x 32 k (each [k][32 rows],
                        // 4 KiB), the bf16 planes as two boxes of 64 rows x 32 k x 2 planes ([plane][k][64 rows]).
                        auto load_tile = [&](uint32_t dst, const CUtensorMap* t32, const CUtensorMap* t16, bool mn, uint32_t r0) {
                            if (!mn) {
                                tma_load_3d_pair(dst, t32, lf, (int)(kb * BK), (int)r0, 0);
                                tma_load_3d_pair(dst + BM * BK * 4, t16, lf, (int)(kb * BK), (int)r0, 0);
                            } else {
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    tma_load_3d_pair(dst + i * 4096, t32, lf, (int)(r0 + 32 * i), (int)(kb * BK), 0);
#pragma unroll
                                for (int i = 0; i < 2; ++i)
                                    tma_load_3d_pair(dst + BM * BK * 4 + i * 8192, t16, lf, (int)(r0 + 64 * i), (int)(kb * BK), 0);
                            }
                        };
                        load_tile(sa, &tmA, &tmA16, ep.a_mn != 0, m0);
                        load_tile(sa + Cfg::kABytes, &tmB, &tmB16, ep.b_mn != 0, nb0);
                    } else {
                        tma_load_3d_pair(sa, &tmA, lf, (int)(kb * BK), (int)m0, 0);
                        tma_load_3d_pair(sa + Cfg::kABytes, &tmB, lf, (int)(kb * BK), (int)nb0, 0);
                    }
                }
            }
#ifdef FG_GEMM_PROFILE
            atomicAdd(&g_prof[6], (unsigned long long)prof_a);
#endif
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // ---- MMA issuer (leader CTA only): M = 256 across the pair, N = 256 ----
            constexpr uint32_t idesc = make_idesc(2u /*tf32*/, 2 * BM, BN);
            bool ok = true;
            uint32_t g = 0, gc = 0;     // k-blocks and chunks consumed so far, across tiles
            long long prof_e = 0, prof_f = 0;
            (void)prof_e; (void)prof_f;
#ifdef FG_GEMM_PROFILE
            const long long prof_start = clock64();
#endif
            for (uint32_t u = pair; u < nunits && ok; u += npairs) {
                uint32_t tile, c0, c1, slot;
                unit_at(u, tile, c0, c1, slot);
                for (uint32_t c = c0; c < c1 && ok; ++c, ++gc) {
                    const uint32_t buf = gc & 1u;
                    // the accumulator must have been drained by both CTAs' epilogue warps (two chunks ago)
                    {
                        PROF_T0();
                        const bool got = mbar_wait_bounded(acc_empty_bar(buf), ((gc >> 1) & 1u) ^ 1u, kPairWaitCycles);
                        PROF_ADD(prof_e);
                        if (!got) {
                            atomicOr(ep.dev_status, FG_DEVERR_MMA_WAIT);
                            ok = false;
                            break;
                        }
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * BN;
                    const uint32_t kb_end = min(nkb, (c + 1) * kChunkKB);
                    for (uint32_t kb = c * kChunkKB; kb < kb_end; ++kb, ++g) {
                        const int s = g % S;
                        const uint32_t ph = (g / S) & 1u;
                        {
                            PROF_T0();
                            const bool got = mbar_wait_bounded(full_bar(s), ph, kPairWaitCycles);
                            PROF_ADD(prof_f);
                            if (!got) {
                                atomicOr(ep.dev_status, FG_DEVERR_MMA_WAIT);
                                ok = false;
                                break;
                            }
                        }
                        tc_fence_after();
                        const uint32_t sa = base + s * Cfg::kStageBytes;
                        const uint64_t a_hi = make_desc_kmajor<BK * 4>(sa);
                        const uint64_t b_hi = make_desc_kmajor<BK * 4>(sa + Cfg::kABytes);
                        const uint32_t first = (kb == c * kChunkKB) ? 0u : 1u;   // a chunk starts from zero
                        if (kDirect16) {
                            constexpr uint32_t idesc16 = make_idesc(FMT == 2 ? 1u /*bf16*/ : 0u /*f16*/, 2 * BM, BN);
#pragma unroll
                            for (int kk = 0; kk < (int)KBE / 16; ++kk) {
                                const uint64_t adv = (uint64_t)(kk * 16 * 2 >> 4);
                                mma_f16_pair(d_tmem, a_hi + adv, b_hi + adv, idesc16, first | (uint32_t)kk);
                            }
                        } else if (FMT == 0) {
                            const uint64_t a_lo = make_desc_kmajor<BK * 4>(sa + BM * BK * 4);
                            const uint64_t b_lo = make_desc_kmajor<BK * 4>(sa + Cfg::kABytes + HB * BK * 4);
#pragma unroll
                            for (int kk = 0; kk < BK / UK; ++kk) {
                                const uint64_t adv = (uint64_t)(kk * UK * 4 >> 4);
                                mma_tf32_pair(d_tmem, a_lo + adv, b_hi + adv, idesc, first | (uint32_t)kk);
                                mma_tf32_pair(d_tmem, a_hi + adv, b_lo + adv, idesc, 1u);
                                mma_tf32_pair(d_tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                            }
                        } else {
                            // Per operand: descriptors of the f32 tile and of its two bf16 planes, and how far
                            // one MMA's worth of k advances them (address field, 16-byte units).  K-major: 32 bytes
                            // inside the swizzled row.  MN-major: eight k-rows = 1024 bytes per tf32 MMA (two 512-byte
                            // atoms of the 32-byte-atomicity swizzle), sixteen k-rows = two 1024-byte atoms per bf16
                            // MMA; column blocks are 4 KiB (f32) / 8 KiB (bf16) apart.
                            const uint32_t idesc_t = idesc | (ep.a_mn ? kIdescAMnMajor : 0u) | (ep.b_mn ? kIdescBMnMajor : 0u);
                            const uint32_t idesc16 = make_idesc(1u /*bf16*/, 2 * BM, BN) | (ep.a_mn ? kIdescAMnMajor : 0u) |
                                                     (ep.b_mn ? kIdescBMnMajor : 0u);
                            const uint32_t a32 = sa, a16 = sa + BM * BK * 4;
                            const uint32_t b32 = sa + Cfg::kABytes, b16 = b32 + HB * BK * 4;
                            uint64_t a_f, a_h16, a_l16, b_f, b_h16, b_l16;
                            uint32_t a_adv32, a_adv16, b_adv32, b_adv16;
                            if (!ep.a_mn) {
                                a_f = make_desc_kmajor<128>(a32);
                                a_h16 = make_desc_kmajor<64>(a16); a_l16 = make_desc_kmajor<64>(a16 + BM * BK * 2);
                                a_adv32 = 2; a_adv16 = 2;
                            } else {
                                a_f = make_desc_mnmajor(a32, 4096, 512, 1);
                                a_h16 = make_desc_mnmajor(a16, 8192, 1024, 2); a_l16 = make_desc_mnmajor(a16 + 4096, 8192, 1024, 2);
                                a_adv32 = 64; a_adv16 = 128;
                            }
                            if (!ep.b_mn) {
                                b_f = make_desc_kmajor<128>(b32);
                                b_h16 = make_desc_kmajor<64>(b16); b_l16 = make_desc_kmajor<64>(b16 + HB * BK * 2);
                                b_adv32 = 2; b_adv16 = 2;
                            } else {
                                b_f = make_desc_mnmajor(b32, 4096, 512, 1);
                                b_h16 = make_desc_mnmajor(b16, 8192, 1024, 2); b_l16 = make_desc_mnmajor(b16 + 4096, 8192, 1024, 2);
                                b_adv32 = 64; b_adv16 = 128;
                            }
#pragma unroll
                            for (int kk = 0; kk < BK / 16; ++kk) {
                                mma_f16_pair(d_tmem, a_l16 + (uint64_t)(kk * a_adv16), b_h16 + (uint64_t)(kk * b_adv16), idesc16,
                                             first | (uint32_t)kk);
                                mma_f16_pair(d_tmem, a_h16 + (uint64_t)(kk * a_adv16), b_l16 + (uint64_t)(kk * b_adv16), idesc16, 1u);
                            }
#pragma unroll
                            for (int kk = 0; kk < BK / UK; ++kk)
                                mma_tf32_pair(d_tmem, a_f + (uint64_t)(kk * a_adv32), b_f + (uint64_t)(kk * b_adv32), idesc_t, 1u);
                        }
                        mma_commit_pair(empty_bar(s), 3);        // frees this stage in both CTAs
                    }
                    if (ok) mma_commit_pair(acc_full_bar(buf), 3);   // both CTAs may drain their half
                }
            }
#ifdef FG_GEMM_PROFILE
            atomicAdd(&g_prof[0], (unsigned long long)prof_e);
            atomicAdd(&g_prof[1], (unsigned long long)prof_f);
            atomicAdd(&g_prof[2], (unsigned long long)(clock64() - prof_start));
            atomicAdd(&g_prof[7], 1ull);
#endif
        }
    }
    } else {
        reg_acquire<kPairRegsHigh>();
        // ---- accumulate + epilogue (both CTAs, own 128 rows); see gemm_tc_kernel ----
        const int q = warp & 3;
        const int half = (warp - kPairEpiWarp0) >> 2;
        const bool vec_ok = (ep.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(ep.C) & 15u) == 0) &&
                            (!ep.preact || (reinterpret_cast<uintptr_t>(ep.preact) & 15u) == 0);
        const uint32_t leader_acc_empty0 = map_to_cta(acc_empty_bar(0), 0);
        float4* tbuf = reinterpret_cast<float4*>(base_ptr + S * Cfg::kStageBytes + 256);   // 8 warps x 32 rows x 8 chunks
        float sum[CPT];
        bool ok = true;
        uint32_t gc = 0;
        long long prof_w = 0, prof_s = 0, prof_n = 0;
        (void)prof_w; (void)prof_s; (void)prof_n;
        for (uint32_t u = pair; u < nunits && ok; u += npairs) {
            uint32_t tile, c0, c1, slot, m0, n0;
            const bool part = unit_at(u, tile, c0, c1, slot);
            tile_origin(tile, m0, n0);
#pragma unroll
            for (int j = 0; j < CPT; ++j) sum[j] = 0.0f;
            // Where this warp's part of the tile goes (a K-share of a tail tile goes out raw into its 256 x 256 slot).
            const uint32_t rsub = lane >> 3, cc = lane & 7;
            const uint32_t out_ld = part ? BN : ep.N, row_lim = part ? 2 * BM : ep.M, col_lim = part ? BN : ep.N;
            const uint32_t row0 = (part ? rank * BM : m0) + q * 32;            // first row of this warp's blocks
            const uint32_t col_base = (part ? 0u : n0) + half * CPT + cc * 4;  // this lane's 4 columns in block 0
            const bool vec = part || vec_ok;
            const float* const mul = part ? nullptr : ep.mul_saved;
            // The saved tensor of the layer below (dA epilogue), rows i*4 + rsub of block `blk`, read a whole block
            // ahead of its use through a rotating set of eight registers per lane: block 0 while the tile's last
            // accumulation chunk is still being computed, block b + 1 while block b is stored.  Read when needed,
            // or only a few rows ahead, each block waited for DRAM two to three times.
            const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
            auto saved_at = [&](int blk, int i) -> float4 {
                const uint32_t row = row0 + i * 4 + rsub, colb = col_base + blk * 32;
                return (mul && vec && blk < CPT / 32 && row < row_lim && colb + 3 < col_lim)
                           ? __ldg(reinterpret_cast<const float4*>(mul + (size_t)row * out_ld + colb)) : zero4;
            };
            float4 s0 = zero4, s1 = zero4, s2 = zero4, s3 = zero4, s4 = zero4, s5 = zero4, s6 = zero4, s7 = zero4;
            for (uint32_t c = c0; c < c1; ++c, ++gc) {
                const uint32_t buf = gc & 1u;
                if (c + 1 == c1 && mul) {
                    s0 = saved_at(0, 0); s1 = saved_at(0, 1); s2 = saved_at(0, 2); s3 = saved_at(0, 3);
                    s4 = saved_at(0, 4); s5 = saved_at(0, 5); s6 = saved_at(0, 6); s7 = saved_at(0, 7);
                }
                PROF_T0();
                bool got = mbar_wait_bounded(acc_full_bar(buf), (gc >> 1) & 1u, kPairWaitCycles + kPairWaitCycles / 2);
                PROF_ADD(prof_w);
                got = __all_sync(0xffffffffu, got);
                if (!got) {
                    if (lane == 0) atomicOr(ep.dev_status, FG_DEVERR_EPI_WAIT);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + half * CPT;
#pragma unroll
                for (int g4 = 0; g4 < CPT / 32; ++g4) {
                    uint32_t r[32];
                    tmem_ld_32x32(t0 + g4 * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) sum[g4 * 32 + j] += __uint_as_float(r[j]);
                }
                tc_fence_before();
                if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + 8u * buf);   // 16 warps report to the leader
            }
            if (!ok) break;
#ifdef FG_GEMM_PROFILE
            const long long prof_st = clock64();
#endif
            // Store this tile from registers; the tensor core is already working on the next one.  A thread
            // owns one row, so storing directly would touch 32 different lines per instruction; instead each
            // warp passes 32x32 blocks through a padded shared-memory buffer and writes 4 rows x 128 bytes
            // per instruction (bias and activation are applied on the way out).
            // A K-share of a tail tile goes out raw (no bias, no activation) into its 256x256 slot.
            // The 32 x 32 staging block of this warp: rows of eight 16-byte chunks, chunk c of row r at position
            // c ^ (r & 7), so that both the row-wise writes (a lane owns a row) and the reads (eight lanes sweep a
            // row) are 128-bit accesses without bank conflicts.  A K-share of a tail tile goes out raw (no bias, no
            // activation, no extras: the fold kernel does those) into its 256 x 256 slot.
            // Nothing below may touch local memory: no calls, no dynamically indexed arrays, no spills.
            float4* tb4 = tbuf + (warp - kPairEpiWarp0) * (32 * 8);
            char* const out = part ? (char*)(ep.partial + (size_t)slot * (2 * BM * BN)) : (char*)ep.C;
            char* const pre = part ? nullptr : (char*)ep.preact;
            const int odt = (part || !kDirect16) ? (int)FG_DTYPE_F32 : ep.out_dtype;   // the f32 kernels store f32 only
            const int act = part ? FG_ACT_NONE : ep.act;
            __nv_bfloat16* const pairs = part ? nullptr : ep.c_pairs;
            float* const csp = part ? nullptr : ep.colsum_part;
#ifdef FG_GEMM_PROFILE
            const bool no_store = (ep.dbg & 1u) != 0;
#else
            constexpr bool no_store = false;
#endif
#pragma unroll
            for (int g4 = 0; g4 < CPT / 32; ++g4) {
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    tb4[lane * 8 + (c ^ (lane & 7))] = make_float4(sum[g4 * 32 + 4 * c], sum[g4 * 32 + 4 * c + 1],
                                                                   sum[g4 * 32 + 4 * c + 2], sum[g4 * 32 + 4 * c + 3]);
                __syncwarp();
                const uint32_t col = col_base + g4 * 32;
                const bool fast = vec && col + 3 < col_lim;                    // the whole float4 is inside the matrix
                float4 bz = make_float4(0.f, 0.f, 0.f, 0.f);
                if (ep.bias && !part) {
                    if (col + 3 < col_lim) bz = __ldg(reinterpret_cast<const float4*>(ep.bias + col));
                    else {
                        if (col < col_lim) bz.x = ep.bias[col];
                        if (col + 1 < col_lim) bz.y = ep.bias[col + 1];
                        if (col + 2 < col_lim) bz.z = ep.bias[col + 2];
                    }
                }
                float4 cs = make_float4(0.f, 0.f, 0.f, 0.f);     // column sums of what this lane stores (rows i*4 + rsub)
                // Rows i*4 + rsub, i = 0..7, one per iteration of a rolled loop (one copy of the activation code per
                // block).  Each iteration takes its row of the saved tensor from the front of the rotating set and
                // refills the back with the same row of the NEXT block.  The staged values come through a rotating
                // set too: the tensor core reads its operands from shared memory at most of the memory's bandwidth,
                // and a shared-memory load issued when its value is needed waits behind that traffic.
                auto staged_row = [&](int i) -> float4 {
                    const uint32_t lr = (uint32_t)(i & 7) * 4 + rsub;
                    return tb4[lr * 8 + (cc ^ (lr & 7))];
                };
                float4 z0 = staged_row(0), z1 = staged_row(1), z2 = staged_row(2), z3 = staged_row(3);
#pragma unroll 1
                for (int i = 0; i < 8; ++i) {
                    const float4 sv = s0;
                    s0 = s1; s1 = s2; s2 = s3; s3 = s4; s4 = s5; s5 = s6; s6 = s7;
                    s7 = saved_at(g4 + 1, i);
                    float4 zin = z0;
                    z0 = z1; z1 = z2; z2 = z3; z3 = staged_row(i + 4);
                    const uint32_t lr = i * 4 + rsub;
                    const uint32_t row = row0 + lr;
                    zin.x += bz.x; zin.y += bz.y; zin.z += bz.z; zin.w += bz.w;
                    if (row < row_lim && col < col_lim) {
                        const size_t off = (size_t)row * out_ld + col;
                        if (fast) {
                            float4 o;
                            if (mul) {
                                o = make_float4(zin.x * fg_act_grad_sel(ep.mul_act, sv.x), zin.y * fg_act_grad_sel(ep.mul_act, sv.y),
                                                zin.z * fg_act_grad_sel(ep.mul_act, sv.z), zin.w * fg_act_grad_sel(ep.mul_act, sv.w));
                            } else if (act != FG_ACT_NONE) {
                                o = make_float4(fg_act_fwd_sel(act, zin.x), fg_act_fwd_sel(act, zin.y), fg_act_fwd_sel(act, zin.z),
                                                fg_act_fwd_sel(act, zin.w));
                            } else o = zin;
                            if (!no_store) {
                                if (pre) store_out4(pre, off, zin, odt);
                                store_out4(out, off, o, odt);
                                if (pairs) fg_store_pairs4(pairs, ep.c_pairs_stride, off, o);
                            }
                            cs.x += o.x; cs.y += o.y; cs.z += o.z; cs.w += o.w;
                        } else {
                            const float4 o = epi_store_edge(zin, off, col, col_lim, out, pre, pairs, ep.c_pairs_stride, mul, ep.mul_act, act, odt);
                            cs.x += o.x; cs.y += o.y; cs.z += o.z; cs.w += o.w;
                        }
                    }
                }
                if (csp) {
                    // the four lanes that share these columns hold rows 0,4,.. / 1,5,.. / 2,6,.. / 3,7,..: add them in a fixed order
                    cs.x += __shfl_xor_sync(0xffffffffu, cs.x, 8); cs.x += __shfl_xor_sync(0xffffffffu, cs.x, 16);
                    cs.y += __shfl_xor_sync(0xffffffffu, cs.y, 8); cs.y += __shfl_xor_sync(0xffffffffu, cs.y, 16);
                    cs.z += __shfl_xor_sync(0xffffffffu, cs.z, 8); cs.z += __shfl_xor_sync(0xffffffffu, cs.z, 16);
                    cs.w += __shfl_xor_sync(0xffffffffu, cs.w, 8); cs.w += __shfl_xor_sync(0xffffffffu, cs.w, 16);
                    if (lane < 8 && row0 < row_lim) {
                        float* d = csp + (size_t)(row0 >> 5) * ep.N + col;
                        if (col < col_lim) d[0] = cs.x;
                        if (col + 1 < col_lim) d[1] = cs.y;
                        if (col + 2 < col_lim) d[2] = cs.z;
                        if (col + 3 < col_lim) d[3] = cs.w;
                    }
                }
                __syncwarp();
            }
#ifdef FG_GEMM_PROFILE
            prof_s += clock64() - prof_st;
            prof_n += 1;
#endif
        }
#ifdef FG_GEMM_PROFILE
        if (warp == kPairEpiWarp0 && lane == 0 && leader) {
            atomicAdd(&g_prof[3], (unsigned long long)prof_w);
            atomicAdd(&g_prof[4], (unsigned long long)prof_s);
            atomicAdd(&g_prof[5], (unsigned long long)prof_n);
        }
#endif
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();      // neither CTA retires while the peer may still read its shared memory
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    }
}

// Folds the K-shares of the pair kernel's tail tiles in a fixed order, then does what the pair kernel's own
// epilogue does for a whole tile: bias, activation (or the act' factor), store, bf16 pairs, column sums.
// 64 blocks of 256 threads per tile, one 32 x 32 sub-block each (so that a block owns whole 32-row column
// sums); thread t handles four consecutive columns of row t / 8.
__global__ void __launch_bounds__(256) gemm_tc_pair_fold_kernel(Epilogue ep) {
    constexpr uint32_t TM = 2 * BM, TN = 256;
    __shared__ float cs_sm[8][32];
    const uint32_t pairs_m = (ep.M + TM - 1) / TM, pairs_n = (ep.N + TN - 1) / TN;
    const uint32_t tail = blockIdx.x >> 6, sub = blockIdx.x & 63u;
    uint32_t m0, n0;
    pair_tile_origin(ep.t_full + tail, pairs_m, pairs_n, TM, TN, ep.group, m0, n0);
    const uint32_t lrow = (sub >> 3) * 32 + (threadIdx.x >> 3), lcol = (sub & 7u) * 32 + (threadIdx.x & 7u) * 4;
    const uint32_t row = m0 + lrow, col = n0 + lcol;
    const bool live = row < ep.M && col < ep.N;
    float ov[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
        const float* p = ep.partial + (size_t)tail * ep.split * (TM * TN) + (size_t)lrow * TN + lcol;
        float4 z = *reinterpret_cast<const float4*>(p);
        for (uint32_t k = 1; k < ep.split; ++k) {
            const float4 t = *reinterpret_cast<const float4*>(p + (size_t)k * (TM * TN));
            z.x += t.x; z.y += t.y; z.z += t.z; z.w += t.w;
        }
        float zz[4] = {z.x, z.y, z.z, z.w};
        if (ep.bias) {
#pragma unroll
            for (int t = 0; t < 4; ++t) if (col + t < ep.N) zz[t] += ep.bias[col + t];
        }
        const size_t off = (size_t)row * ep.N + col;
        const bool vec_ok = (ep.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(ep.C) & 15u) == 0) &&
                            (!ep.preact || (reinterpret_cast<uintptr_t>(ep.preact) & 15u) == 0);
        if (vec_ok && col + 3 < ep.N) {
            const float4 zin = make_float4(zz[0], zz[1], zz[2], zz[3]);
            float4 o;
            if (ep.mul_saved) o = act_mul4(ep.mul_act, zin, __ldg(reinterpret_cast<const float4*>(ep.mul_saved + off)));
            else o = ep.act == FG_ACT_NONE ? zin : act_fwd4(ep.act, zin);
            if (ep.preact) store_out4(ep.preact, off, zin, ep.out_dtype);
            store_out4(ep.C, off, o, ep.out_dtype);
            if (ep.c_pairs) fg_store_pairs4(ep.c_pairs, ep.c_pairs_stride, off, o);
            ov[0] = o.x; ov[1] = o.y; ov[2] = o.z; ov[3] = o.w;
        } else {
#pragma unroll
            for (int t = 0; t < 4; ++t)
                if (col + t < ep.N) {
                    const float o = ep.mul_saved ? zz[t] * fg_act_grad_fast(ep.mul_act, ep.mul_saved[off + t]) : fg_act_fwd_fast(ep.act, zz[t]);
                    if (ep.preact) store_out1(ep.preact, off + t, zz[t], ep.out_dtype);
                    store_out1(ep.C, off + t, o, ep.out_dtype);
                    if (ep.c_pairs) fg_store_pairs1(ep.c_pairs, ep.c_pairs_stride, off + t, o);
                    ov[t] = o;
                }
        }
    }
    if (!ep.colsum_part) return;
    // column sums over this block's 32 rows: four rows inside each warp, then the eight warps in order
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        ov[t] += __shfl_xor_sync(0xffffffffu, ov[t], 8);
        ov[t] += __shfl_xor_sync(0xffffffffu, ov[t], 16);
    }
    if (lane < 8) {
#pragma unroll
        for (int t = 0; t < 4; ++t) cs_sm[warp][lane * 4 + t] = ov[t];
    }
    __syncthreads();
    const uint32_t row0 = m0 + (sub >> 3) * 32, c = n0 + (sub & 7u) * 32 + threadIdx.x;
    if (threadIdx.x < 32 && row0 < ep.M && c < ep.N) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += cs_sm[w][threadIdx.x];
        ep.colsum_part[(size_t)(row0 >> 5) * ep.N + c] = t;
    }
}

// ------------------------------------------------------------------------------------
// Pre-pass: operand planes of X [R, C] (row-major), optionally of dY * act'(saved).
// Orientation n keeps X's layout (contraction index = column): rows R, pitch ld*.
// Orientation t is transposed (contraction index = row): rows C.
// Plane formats (FMT):
//   0  p32 = [2][rows][ld32] f32: hi = tf32(x), lo = tf32(x - hi)
//   1  p32 = [rows][ld32] f32: hi;  p16 = [2][rows][ld16] bf16: bf16(x), bf16(x - hi)
// ------------------------------------------------------------------------------------
struct PlaneSet {
    float* p32;
    __nv_bfloat16* p16;
    uint32_t ld32, ld16;
    uint64_t plane16;      // elements between the two bf16 planes (0: rows * ld16, planes back to back)
    bool mn;               // storage is [contraction][rows] (rows contiguous): the f32 tensor itself with its pairs
};

struct SplitArgs {
    const float* x;
    const float* saved;    // non-NULL: value = x * act'(saved)
    int act;
    uint32_t R, C;
    PlaneSet n, t;         // p32 == NULL: orientation not wanted
    float* value_out;      // optional copy of the (fused) value, [R, C]
    float* colsum_part;    // optional [gridDim.y][C]: column sums of the value over each tile's rows (bias gradient)
};

template <int FMT>
__device__ __forceinline__ void store_planes(const PlaneSet& ps, size_t rows, size_t r, size_t c, float hi, float lo,
                                             float v) {
    ps.p32[r * ps.ld32 + c] = hi;
    if (FMT == 0) {
        ps.p32[rows * ps.ld32 + r * ps.ld32 + c] = lo;
    } else {
        ps.p16[r * ps.ld16 + c] = __float2bfloat16_rn(v);
        ps.p16[rows * ps.ld16 + r * ps.ld16 + c] = __float2bfloat16_rn(lo);
    }
}

// Any shape and alignment: 32x32 tiles, 32x8 threads, scalar accesses.
template <int FMT>
__global__ void __launch_bounds__(256) split_kernel(SplitArgs a) {
    __shared__ float tv[32][33];
    __shared__ float cs[8][33];
    const uint32_t c = blockIdx.x * 32 + threadIdx.x;
    const uint32_t r0 = blockIdx.y * 32;
    float csum = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t r = r0 + threadIdx.y + i * 8;
        float v = 0.0f;
        if (r < a.R && c < a.C) {
            const size_t idx = (size_t)r * a.C + c;
            v = a.x[idx];
            if (a.saved) v = v * fg_act_grad(a.act, a.saved[idx]);
            if (a.value_out) a.value_out[idx] = v;
            if (a.n.p32) {
                const float hi = __uint_as_float(cvt_tf32(v));
                const float lo = v - hi;
                store_planes<FMT>(a.n, a.R, r, c, hi, FMT == 0 ? __uint_as_float(cvt_tf32(lo)) : lo, v);
            }
        }
        tv[threadIdx.y + i * 8][threadIdx.x] = v;
        csum += v;
    }
    if (a.colsum_part) cs[threadIdx.y][threadIdx.x] = csum;
    if (!a.t.p32 && !a.colsum_part) return;
    __syncthreads();
    if (a.colsum_part && threadIdx.y == 0 && c < a.C) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += cs[k][threadIdx.x];
        a.colsum_part[(size_t)blockIdx.y * a.C + c] = t;
    }
    if (!a.t.p32) return;
    const uint32_t tr = r0 + threadIdx.x;          // source row -> destination column
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t tc = blockIdx.x * 32 + threadIdx.y + i * 8;   // source column -> destination row
        if (tc < a.C && tr < a.R) {
            const float v = tv[threadIdx.x][threadIdx.y + i * 8];
            const float hi = __uint_as_float(cvt_tf32(v));
            const float lo = v - hi;
            store_planes<FMT>(a.t, a.C, tc, tr, hi, FMT == 0 ? __uint_as_float(cvt_tf32(lo)) : lo, v);
        }
    }
}

struct Split4 {
    float4 hi, lo;
};
template <int FMT>
__device__ __forceinline__ Split4 split4(float4 v) {
    Split4 o;
    o.hi = make_float4(__uint_as_float(cvt_tf32(v.x)), __uint_as_float(cvt_tf32(v.y)),
                       __uint_as_float(cvt_tf32(v.z)), __uint_as_float(cvt_tf32(v.w)));
    o.lo = make_float4(v.x - o.hi.x, v.y - o.hi.y, v.z - o.hi.z, v.w - o.hi.w);
    if (FMT == 0)
        o.lo = make_float4(__uint_as_float(cvt_tf32(o.lo.x)), __uint_as_float(cvt_tf32(o.lo.y)),
                           __uint_as_float(cvt_tf32(o.lo.z)), __uint_as_float(cvt_tf32(o.lo.w)));
    return o;
}
__device__ __forceinline__ uint2 pack_bf16x4(float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    return u;
}
// Four consecutive elements of one plane row (c a multiple of 4, pitches multiples of 4 / 8).
template <int FMT>
__device__ __forceinline__ void store_planes4(const PlaneSet& ps, size_t rows, size_t r, size_t c, float4 v) {
    const Split4 s = split4<FMT>(v);
    *reinterpret_cast<float4*>(ps.p32 + r * ps.ld32 + c) = s.hi;
    if (FMT == 0) {
        *reinterpret_cast<float4*>(ps.p32 + rows * ps.ld32 + r * ps.ld32 + c) = s.lo;
    } else {
        *reinterpret_cast<uint2*>(ps.p16 + r * ps.ld16 + c) = pack_bf16x4(v);
        *reinterpret_cast<uint2*>(ps.p16 + rows * ps.ld16 + r * ps.ld16 + c) = pack_bf16x4(s.lo);
    }
}

// 128-bit accesses, for R % 4 == 0 and C % 4 == 0 (every group of four is wholly inside or outside)
// and 16-byte aligned pointers.  64x64 tiles, 256 threads: thread t handles column group t%16
// (4 columns) of rows t/16 + 16*i, then writes 4 consecutive source rows of source column t/16 + 16*i.
template <int FMT>
__global__ void __launch_bounds__(256) split_vec_kernel(SplitArgs a) {
    __shared__ float tv[64][65];
    __shared__ float cs[16][64];
    const uint32_t cg = threadIdx.x & 15, rl = threadIdx.x >> 4;
    const uint32_t c = blockIdx.x * 64 + cg * 4;
    const uint32_t r0 = blockIdx.y * 64;
    const bool want_t = a.t.p32 != nullptr;
    float4 csum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lr = rl + 16 * i, r = r0 + lr;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < a.R && c < a.C) {
            const size_t idx = (size_t)r * a.C + c;
            v = __ldcs(reinterpret_cast<const float4*>(a.x + idx));
            if (a.saved) {
                const float4 s = __ldcs(reinterpret_cast<const float4*>(a.saved + idx));
                v.x *= fg_act_grad(a.act, s.x); v.y *= fg_act_grad(a.act, s.y);
                v.z *= fg_act_grad(a.act, s.z); v.w *= fg_act_grad(a.act, s.w);
            }
            if (a.value_out) *reinterpret_cast<float4*>(a.value_out + idx) = v;
            if (a.n.p32) store_planes4<FMT>(a.n, a.R, r, c, v);
        }
        if (want_t) {
            tv[lr][cg * 4 + 0] = v.x; tv[lr][cg * 4 + 1] = v.y; tv[lr][cg * 4 + 2] = v.z; tv[lr][cg * 4 + 3] = v.w;
        }
        csum.x += v.x; csum.y += v.y; csum.z += v.z; csum.w += v.w;
    }
    if (a.colsum_part) {
        cs[rl][cg * 4 + 0] = csum.x; cs[rl][cg * 4 + 1] = csum.y; cs[rl][cg * 4 + 2] = csum.z; cs[rl][cg * 4 + 3] = csum.w;
    }
    if (!want_t && !a.colsum_part) return;
    __syncthreads();
    if (a.colsum_part && threadIdx.x < 64 && blockIdx.x * 64 + threadIdx.x < a.C) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < 16; ++k) t += cs[k][threadIdx.x];
        a.colsum_part[(size_t)blockIdx.y * a.C + blockIdx.x * 64 + threadIdx.x] = t;
    }
    if (!want_t) return;
    const uint32_t tr = r0 + cg * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lc = rl + 16 * i, tc = blockIdx.x * 64 + lc;
        if (tc < a.C && tr < a.R)
            store_planes4<FMT>(a.t, a.C, tc, tr,
                               make_float4(tv[cg * 4 + 0][lc], tv[cg * 4 + 1][lc], tv[cg * 4 + 2][lc], tv[cg * 4 + 3][lc]));
    }
}

inline uint32_t round4(uint32_t v) { return (v + 3u) & ~3u; }
inline uint32_t round8(uint32_t v) { return (v + 7u) & ~7u; }
inline uint64_t align256(uint64_t v) { return (v + 255u) & ~uint64_t(255); }
// Scratch bytes of one operand's planes (rows x contraction k), including internal alignment.
inline uint64_t planes_bytes(int fmt, uint32_t rows, uint32_t k) {
    if (fmt == 0) return 2ull * rows * round4(k) * 4ull + 256;
    return align256((uint64_t)rows * round4(k) * 4ull) + 2ull * rows * round8(k) * 2ull + 512;
}
int32_t alloc_planes(fg_ctx* ctx, int fmt, uint32_t rows, uint32_t k, PlaneSet* out) {
    void* p;
    int32_t s = fg_ws_alloc(ctx, planes_bytes(fmt, rows, k), &p);
    if (s != FG_OK) return s;
    out->p32 = (float*)p;
    out->ld32 = round4(k);
    out->ld16 = round8(k);
    out->p16 = fmt == 0 ? nullptr
                        : (__nv_bfloat16*)((char*)p + align256((uint64_t)rows * round4(k) * 4ull));
    out->plane16 = 0;
    out->mn = false;
    return FG_OK;
}

// `chunks_out` (may be NULL) receives the number of row tiles = rows of a.colsum_part that get written.
int32_t launch_split(fg_ctx* ctx, int fmt, const SplitArgs& a, uint32_t* chunks_out = nullptr) {
    auto ok16 = [](const PlaneSet& ps) { return !ps.p32 || (fg_aligned16(ps.p32) && (!ps.p16 || fg_aligned16(ps.p16))); };
    const bool vec = (a.R % 4 == 0) && (a.C % 4 == 0) && fg_aligned16(a.x) && (!a.saved || fg_aligned16(a.saved)) &&
                     (!a.value_out || fg_aligned16(a.value_out)) && ok16(a.n) && ok16(a.t);
    const uint32_t tile = vec ? 64 : 32;
    dim3 grid((a.C + tile - 1) / tile, (a.R + tile - 1) / tile);
    if (grid.y > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "GEMM operand has too many rows");
    if (chunks_out) *chunks_out = grid.y;
    double bytes = 4.0 * a.R * a.C * (1.0 + (a.saved ? 1.0 : 0.0) + (a.value_out ? 1.0 : 0.0) +
                                      (a.n.p32 ? 2.0 : 0.0) + (a.t.p32 ? 2.0 : 0.0));
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SPLIT, bytes);
    if (fmt == 0) {
        if (vec) split_vec_kernel<0><<<grid, 256, 0, ctx->stream>>>(a);
        else split_kernel<0><<<grid, dim3(32, 8), 0, ctx->stream>>>(a);
    } else {
        if (vec) split_vec_kernel<1><<<grid, 256, 0, ctx->stream>>>(a);
        else split_kernel<1><<<grid, dim3(32, 8), 0, ctx->stream>>>(a);
    }
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

typedef CUresult (*pfn_encode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map over planes [nplanes][rows][ld] with contraction extent `kdim`; box {bk, box_rows, nplanes}.
// The swizzle span equals the box's inner extent in bytes: 128 or 64.
// elem: 0 f32, 1 bf16, 2 f16.
int32_t make_tmap(fg_ctx* ctx, CUtensorMap* out, const void* planes, int elem, uint32_t nplanes, uint32_t rows,
                  uint32_t kdim, uint32_t ld, uint32_t box_rows, uint32_t bk) {
    if (!ctx->tmap_encode) return fg_fail(ctx, FG_ERR_UNSUPPORTED_FEATURE, "cuTensorMapEncodeTiled unavailable");
    const uint32_t esz = elem ? 2 : 4;
    cuuint64_t dims[3] = {kdim, rows, nplanes};
    cuuint64_t strides[2] = {(cuuint64_t)ld * esz, (cuuint64_t)rows * ld * esz};
    cuuint32_t box[3] = {bk, box_rows, nplanes};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapSwizzle swz = bk * esz == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    CUresult r = ((pfn_encode)ctx->tmap_encode)(out, elem == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                     : elem == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                                                3, (void*)planes, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(ctx->err, sizeof(ctx->err), "cuTensorMapEncodeTiled failed with code %d", (int)r);
        return FG_ERR_INTERNAL;
    }
    return FG_OK;
}

// General 3-D tiled map with the 128- or 64-byte swizzle (by the box's inner extent in bytes).
int32_t make_tmap3(fg_ctx* ctx, CUtensorMap* out, const void* base, int elem, uint64_t d0, uint64_t d1, uint64_t d2,
                   uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2, bool atom32 = false) {
    if (!ctx->tmap_encode) return fg_fail(ctx, FG_ERR_UNSUPPORTED_FEATURE, "cuTensorMapEncodeTiled unavailable");
    const uint32_t esz = elem ? 2 : 4;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {b0, b1, b2};
    cuuint32_t estr[3] = {1, 1, 1};
    // atom32: 32-byte chunks permuted within the 128-byte span (what an MN-major tf32 operand needs)
    const CUtensorMapSwizzle swz = atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                   : b0 * esz == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    CUresult r = ((pfn_encode)ctx->tmap_encode)(out, elem == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                     : elem == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                                                3, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(ctx->err, sizeof(ctx->err), "cuTensorMapEncodeTiled failed with code %d", (int)r);
        return FG_ERR_INTERNAL;
    }
    return FG_OK;
}

// The two maps of one operand of the pair kernel in format 1: `rows` x `kdim` values as an f32 tensor
// (hi plane or the tensor itself) plus two bf16 planes, tile_rows rows per tile.
int32_t make_operand_maps(fg_ctx* ctx, const PlaneSet& o, uint32_t rows, uint32_t kdim, uint32_t tile_rows, CUtensorMap* t32,
                          CUtensorMap* t16) {
    const uint64_t plane16 = o.plane16 ? o.plane16 : (uint64_t)rows * o.ld16;
    int32_t s;
    if (!o.mn) {
        if ((s = make_tmap3(ctx, t32, o.p32, 0, kdim, rows, 1, (uint64_t)o.ld32 * 4, (uint64_t)rows * o.ld32 * 4, 32, tile_rows, 1)) != FG_OK) return s;
        return make_tmap3(ctx, t16, o.p16, 1, kdim, rows, 2, (uint64_t)o.ld16 * 2, plane16 * 2, 32, tile_rows, 2);
    }
    // [kdim][rows]: boxes of 128 bytes along rows x 32 values of k
    if ((s = make_tmap3(ctx, t32, o.p32, 0, rows, kdim, 1, (uint64_t)o.ld32 * 4, (uint64_t)kdim * o.ld32 * 4, 32, 32, 1, true)) != FG_OK) return s;
    return make_tmap3(ctx, t16, o.p16, 1, rows, kdim, 2, (uint64_t)o.ld16 * 2, plane16 * 2, 64, 32, 2);
}

template <int BN, int BK, int FMT>
int32_t launch_tc(fg_ctx* ctx, const PlaneSet& a, const PlaneSet& b, const Epilogue& ep) {
    using Cfg = TileCfg<BN, BK>;
    CUtensorMap tmA, tmB, tmA16, tmB16;
    int32_t s;
    if ((s = make_tmap(ctx, &tmA, a.p32, 0, FMT == 0 ? 2 : 1, ep.M, ep.K, a.ld32, BM, BK)) != FG_OK) return s;
    if ((s = make_tmap(ctx, &tmB, b.p32, 0, FMT == 0 ? 2 : 1, ep.N, ep.K, b.ld32, BN, BK)) != FG_OK) return s;
    if (FMT == 1) {
        if ((s = make_tmap(ctx, &tmA16, a.p16, 1, 2, ep.M, ep.K, a.ld16, BM, BK)) != FG_OK) return s;
        if ((s = make_tmap(ctx, &tmB16, b.p16, 1, 2, ep.N, ep.K, b.ld16, BN, BK)) != FG_OK) return s;
    } else {
        tmA16 = tmA;
        tmB16 = tmB;
    }
    // one bit per device; several host threads (one context each) may arrive here together, and setting the
    // attribute twice is harmless
    static std::atomic<uint64_t> attr_done{0};
    if (!(attr_done.load(std::memory_order_acquire) >> (ctx->device & 63) & 1ull)) {
        FG_CUDA(ctx, FG_ERR_INTERNAL,
                cudaFuncSetAttribute(gemm_tc_kernel<BN, BK, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_done.fetch_or(1ull << (ctx->device & 63), std::memory_order_release);
    }
    dim3 grid((ep.N + BN - 1) / BN, (ep.M + BM - 1) / BM);
    if (grid.y > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "GEMM: M too large");
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_GEMM_TC, 2.0 * ep.M * ep.N * ep.K);
    gemm_tc_kernel<BN, BK, FMT><<<grid, kThreads, Cfg::kSmemBytes, ctx->stream>>>(tmA, tmB, tmA16, tmB16, ep);
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

// Scratch the pair kernel's split-K tail may need: at most one 256x256 f32 slot per resident pair.
constexpr uint64_t kPairPartialBytes = 80ull * (2 * BM) * 256 * 4 + 256;

template <int BK, int FMT>
int32_t launch_tc_pair(fg_ctx* ctx, const PlaneSet& a, const PlaneSet& b, const Epilogue& ep_in) {
    Epilogue ep = ep_in;
    using Cfg = PairCfg<BK, FMT>;
    CUtensorMap tmA, tmB, tmA16, tmB16;
    int32_t s;
    constexpr bool kDirect16 = FMT >= 2;
    if (kDirect16) {
        // the operands themselves: one 16-bit "plane", 64 values of k (128 bytes) per row of a k-block
        const int elem = FMT == 2 ? 1 : 2;
        if ((s = make_tmap(ctx, &tmA16, a.p16, elem, 1, ep.M, ep.K, a.ld16, BM, 2 * BK)) != FG_OK) return s;
        if ((s = make_tmap(ctx, &tmB16, b.p16, elem, 1, ep.N, ep.K, b.ld16, Cfg::kBN / 2, 2 * BK)) != FG_OK) return s;
        tmA = tmA16;
        tmB = tmB16;
    } else {
        if (FMT == 1) {
            if ((s = make_operand_maps(ctx, a, ep.M, ep.K, BM, &tmA, &tmA16)) != FG_OK) return s;
            if ((s = make_operand_maps(ctx, b, ep.N, ep.K, Cfg::kBN / 2, &tmB, &tmB16)) != FG_OK) return s;
            ep.a_mn = a.mn ? 1u : 0u;
            ep.b_mn = b.mn ? 1u : 0u;
        } else {
            if ((s = make_tmap(ctx, &tmA, a.p32, 0, 2, ep.M, ep.K, a.ld32, BM, BK)) != FG_OK) return s;
            if ((s = make_tmap(ctx, &tmB, b.p32, 0, 2, ep.N, ep.K, b.ld32, Cfg::kBN / 2, BK)) != FG_OK) return s;
            tmA16 = tmA;
            tmB16 = tmB;
        }
    }
    // one bit per device; several host threads (one context each) may arrive here together, and setting the
    // attribute twice is harmless
    static std::atomic<uint64_t> attr_done{0};
    if (!(attr_done.load(std::memory_order_acquire) >> (ctx->device & 63) & 1ull)) {
        FG_CUDA(ctx, FG_ERR_INTERNAL,
                cudaFuncSetAttribute(gemm_tc_pair_kernel<BK, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_done.fetch_or(1ull << (ctx->device & 63), std::memory_order_release);
    }
    const uint64_t ntiles = (uint64_t)((ep.M + 2 * BM - 1) / (2 * BM)) * ((ep.N + Cfg::kBN - 1) / Cfg::kBN);
    if (ntiles > (1ull << 30)) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "GEMM: too many tiles");
    // Tile rows per group of the tile order: the pairs at work at one time cover `group` tile rows, whose slabs of A
    // (256 x K elements each) should stay in the L2 while the B slabs stream past.  Eight rows for long K; sixteen
    // when the slabs are small (K <= 2048: the dW products of the eight-layer workload ran 5 % faster, its step
    // 23.83 against 23.91 ms; on 784-4096-4096-10, all K = 4096, eight is best: 0.300 ms per launch against
    // 0.302 / 0.305 / 0.307 for 12 / 16 / 4).
    ep.group = ctx->opt_tile_group > 0 ? (uint32_t)ctx->opt_tile_group : (ep.K <= 2048 ? 16u : 8u);
    // persistent: one CTA pair per SM pair, each walking tiles pair, pair + P, ...
    // How many pairs can be resident at once is asked of the runtime (not every SM need be pairable).
    static std::atomic<int> max_clusters[64];       // zero-initialised; the same value whoever computes it
    if (max_clusters[ctx->device & 63].load(std::memory_order_acquire) == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)ctx->sm_count & ~1u);
        cfg.blockDim = dim3(kPairThreads);
        cfg.dynamicSmemBytes = Cfg::kSmemBytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<BK, FMT>, &cfg) != cudaSuccess || n < 1) {
            cudaGetLastError();
            n = ctx->sm_count / 2;
        }
        max_clusters[ctx->device & 63].store(n, std::memory_order_release);
    }
    uint64_t slots = (uint64_t)max_clusters[ctx->device & 63].load(std::memory_order_acquire);
    if (ctx->comm_pending && ctx->comm_reserved_sms > 0) {
        // leave room for the gradient exchange that runs beside this GEMM (see fg_comm_init)
        const uint64_t lim = (uint64_t)(ctx->sm_count - ctx->comm_reserved_sms) / 2;
        if (lim >= 1 && lim < slots) slots = lim;
    }
    // The last wave: `rem` tiles for `slots` pairs.  When at least two pairs are free per tile, each tail
    // tile is cut into K-shares (whole accumulation chunks, at least two per share) so that the wave
    // lasts a fraction of a tile time; the shares are folded by a second, bandwidth-bound kernel.
    const uint32_t chunk_k = kDirect16 ? 1024 : kChunkK;          // as in the kernel
    const uint32_t nchunks = (ep.K + chunk_k - 1) / chunk_k;
    const uint64_t rem = ntiles % slots;
    uint64_t split = rem ? slots / rem : 1;
    if (split > nchunks / 2) split = nchunks / 2;
    if (split > 4) split = 4;
    if (!ctx->opt_split_k) split = 1;
    ep.partial = nullptr;
    ep.t_full = (uint32_t)ntiles;
    ep.split = 1;
    if (split >= 2 && rem * split * (2 * BM) * 256 * 4 + 256 <= kPairPartialBytes) {
        void* part;
        if ((s = fg_ws_alloc(ctx, rem * split * (2 * BM) * 256 * 4, &part)) != FG_OK) return s;
        ep.partial = (float*)part;
        ep.t_full = (uint32_t)(ntiles - rem);
        ep.split = (uint32_t)split;
    }
    const uint64_t nunits = ep.t_full + (ntiles - ep.t_full) * ep.split;
    dim3 grid((unsigned)(2 * (nunits < slots ? nunits : slots)));
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_GEMM_TC, 2.0 * ep.M * ep.N * ep.K);
    gemm_tc_pair_kernel<BK, FMT><<<grid, kPairThreads, Cfg::kSmemBytes, ctx->stream>>>(tmA, tmB, tmA16, tmB16, ep);
    FG_LAUNCHED(ctx);
    if (ep.split > 1) {
        gemm_tc_pair_fold_kernel<<<(unsigned)((ntiles - ep.t_full) * 64), 256, 0, ctx->stream>>>(ep);
        FG_LAUNCHED(ctx);
    }
    fg_time_end(ctx, tr);
    return FG_OK;
}

// C[M,N] = act(Aop·Bopᵀ + bias) where the A operand's planes have M rows and the B operand's N rows.
int32_t tc_gemm(fg_ctx* ctx, int fmt, const PlaneSet& a, const PlaneSet& b, uint32_t M, uint32_t N, uint32_t K, float* C,
                const float* bias, int act, float* preact) {
    Epilogue ep{C, bias, preact, M, N, K, act, ctx->dev_status};
    // Tile choice: one output tile per CTA (or per CTA pair), so the last wave is often part empty.
    // Each candidate is scored by machine fill times its measured relative throughput at 8192^3
    // (hybrid planes: pair 316, 128x256 248, 128x128 ~215 TFLOP/s; hi/lo planes: 262, 260, 217).
    const uint64_t sms = (uint64_t)ctx->sm_count, mt = (M + BM - 1) / BM;
    auto fill = [](uint64_t tiles, uint64_t slots) { return (double)tiles / (double)(((tiles + slots - 1) / slots) * slots); };
    const uint64_t t256 = mt * ((N + 255) / 256), t128 = mt * ((N + 127) / 128);
    const uint64_t tpair = (uint64_t)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
    const double s_pair = (N > 128 && M > BM) ? fill(tpair, sms / 2) * 1.0 : 0.0;
    const double s_256 = N > 128 ? fill(t256, sms) * (fmt == 1 ? 0.78 : 0.98) : 0.0;
    const double s_128 = N > 64 ? fill(t128, sms) * (fmt == 1 ? 0.68 : 0.83) : 0.0;
    int bn = N > 128 ? (s_256 >= s_128 ? 256 : 128) : N > 64 ? 128 : N > 32 ? 64 : 32;
    int bk = (fmt == 0 && bn == 256) ? 16 : 32;
    bool pair = s_pair > 0.0 && s_pair >= s_256 && s_pair >= s_128;
    // Option gemm_tile: "pair" or "<BN>x<BK>" instead of the choice above.
    if (ctx->opt_tile_pair == 1) pair = N > 128;
    else if (ctx->opt_tile_pair == 0 && (ctx->opt_tile_bk == 32 || fmt == 0)) {
        bn = ctx->opt_tile_bn; bk = ctx->opt_tile_bk; pair = false;
    }
    if (pair) return fmt == 1 ? launch_tc_pair<32, 1>(ctx, a, b, ep) : launch_tc_pair<32, 0>(ctx, a, b, ep);
    if (fmt == 1) {
        if (bn == 256) return launch_tc<256, 32, 1>(ctx, a, b, ep);
        if (bn == 128) return launch_tc<128, 32, 1>(ctx, a, b, ep);
        if (bn == 64) return launch_tc<64, 32, 1>(ctx, a, b, ep);
        return launch_tc<32, 32, 1>(ctx, a, b, ep);
    }
    if (bn == 256 && bk == 16) return launch_tc<256, 16, 0>(ctx, a, b, ep);
    if (bn == 128 && bk == 16) return launch_tc<128, 16, 0>(ctx, a, b, ep);
    if (bn == 256) return launch_tc<256, 32, 0>(ctx, a, b, ep);
    if (bn == 128) return launch_tc<128, 32, 0>(ctx, a, b, ep);
    if (bn == 64) return launch_tc<64, 32, 0>(ctx, a, b, ep);
    return launch_tc<32, 32, 0>(ctx, a, b, ep);
}

// ------------------------------------------------------------------------------------
// f32 tensors with bf16 pairs: the pair kernel multiplies the tensors as they lie in HBM.
// The kind::tf32 MMA reads the f32 words themselves (it uses sign, exponent and the top 10
// mantissa bits: hi = trunc(x)); the two cross terms of the split product come from two
// bf16 planes of the same shape and layout, pairs[0] = bf16(x), pairs[1] = bf16(x - trunc(x)).
// An operand whose contraction index is not the contiguous one is read through MN-major
// descriptors, so nothing is ever transposed, and whoever produces a tensor (a GEMM
// epilogue, the optimizer, the kernels below) writes its pairs in the same pass.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) pairs_kernel(const float* __restrict__ x, uint64_t n, __nv_bfloat16* __restrict__ pairs,
                                                    uint64_t plane_stride) {
    const uint64_t nv = n >> 2, stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride)
        fg_store_pairs4(pairs, plane_stride, i * 4, __ldcs(reinterpret_cast<const float4*>(x) + i));
    for (uint64_t i = (nv << 2) + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        fg_store_pairs1(pairs, plane_stride, i, x[i]);
}

// dz = dy * act'(saved) over [R, C] with its pairs and the column sums of each 32-row block (the bias
// gradient's partials), in one pass.  A block covers 32 rows x 512 columns; a thread owns four columns.
// dz may alias dy.  Needs C % 4 == 0 and 16-byte aligned pointers.
__global__ void __launch_bounds__(128) dz_pairs_kernel(uint32_t R, uint32_t C, const float* dy, const float* __restrict__ saved,
                                                       int act, float* dz, __nv_bfloat16* __restrict__ pairs,
                                                       uint64_t plane_stride, float* __restrict__ colsum_part) {
    const uint32_t c = (blockIdx.x * 128 + threadIdx.x) * 4;
    if (c >= C) return;
    const uint32_t r0 = blockIdx.y * 32, r1 = min(R, r0 + 32);
    float4 cs = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (uint32_t r = r0; r < r1; ++r) {
        const size_t off = (size_t)r * C + c;
        float4 v = __ldcs(reinterpret_cast<const float4*>(dy + off));
        if (saved) v = act_mul4(act, v, __ldcs(reinterpret_cast<const float4*>(saved + off)));
        if (dz) *reinterpret_cast<float4*>(dz + off) = v;
        if (pairs) fg_store_pairs4(pairs, plane_stride, off, v);
        cs.x += v.x; cs.y += v.y; cs.z += v.z; cs.w += v.w;
    }
    if (colsum_part) *reinterpret_cast<float4*>(colsum_part + (size_t)blockIdx.y * C + c) = cs;
}

int32_t launch_pairs(fg_ctx* ctx, const float* x, uint64_t n, __nv_bfloat16* pairs, uint64_t plane_stride) {
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SPLIT, 8.0 * (double)n);
    pairs_kernel<<<fg_stream_grid(ctx, (n + 3) / 4, 256, 8), 256, 0, ctx->stream>>>(x, n, pairs, plane_stride);
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

int32_t launch_dz_pairs(fg_ctx* ctx, uint32_t R, uint32_t C, const float* dy, const float* saved, int act, float* dz,
                        __nv_bfloat16* pairs, uint64_t plane_stride, float* colsum_part) {
    dim3 grid((C + 511) / 512, (R + 31) / 32);
    if (grid.y > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "GEMM operand has too many rows");
    fg_time_rec* tr = fg_time_begin(ctx, FG_KERNEL_SPLIT, 4.0 * R * C * (1.0 + (saved ? 1.0 : 0.0) + (dz ? 1.0 : 0.0) + (pairs ? 1.0 : 0.0)));
    dz_pairs_kernel<<<grid, 128, 0, ctx->stream>>>(R, C, dy, saved, act, dz, pairs, plane_stride, colsum_part);
    fg_time_end(ctx, tr);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

// A dense row-major f32 tensor [R, C] and its pairs as an operand of the pair kernel.  `contract_cols`:
// the contraction runs over the columns (K-major), otherwise over the rows (MN-major).
PlaneSet paired_operand(const float* x, const void* pairs, uint64_t plane_stride, uint32_t C, bool contract_cols) {
    PlaneSet o{};
    o.p32 = const_cast<float*>(x);
    o.p16 = (__nv_bfloat16*)pairs;
    o.ld32 = o.ld16 = C;
    o.plane16 = plane_stride;
    o.mn = !contract_cols;
    return o;
}

// Can [M,N] = [M,K] x [K,N] run on the pair kernel straight from f32 tensors and their pairs?  Every
// tensor's row pitch must be a multiple of 16 bytes in both element sizes (columns % 8), and the tile
// shape must suit the pair kernel.
bool paired_shape_ok(const fg_ctx* ctx, uint32_t M, uint32_t N, uint32_t K, uint32_t pitch_a, uint32_t pitch_b) {
    return ctx->opt_pairs && ctx->opt_tile_pair != 0 && ctx->tmap_encode && M > (uint32_t)BM && N > 128 && K >= 32 &&
           pitch_a % 8 == 0 && pitch_b % 8 == 0;
}

struct PairedOut {
    __nv_bfloat16* pairs;     // optional pairs of the result
    uint64_t stride;
    const float* mul_saved;   // optional: result = (acc + bias) * act'(mul_saved)
    int mul_act;
    float* colsum_part;       // optional [ceil(M/32)][N]
};

int32_t paired_gemm(fg_ctx* ctx, const PlaneSet& a, const PlaneSet& b, uint32_t M, uint32_t N, uint32_t K, float* C,
                    const float* bias, int act, float* preact, const PairedOut& o) {
    Epilogue ep{C, bias, preact, M, N, K, act, ctx->dev_status};
#ifdef FG_GEMM_PROFILE
    if (const char* e = getenv("FG_GEMM_DBG")) ep.dbg = (uint32_t)atoi(e);
#endif
    ep.c_pairs = o.pairs;
    ep.c_pairs_stride = o.stride;
    ep.mul_saved = o.mul_saved;
    ep.mul_act = o.mul_act;
    ep.colsum_part = o.colsum_part;
    return launch_tc_pair<32, 1>(ctx, a, b, ep);
}

// Which path a request takes: 0 = SIMT, otherwise the plane format + 1.
int pick_path(const fg_ctx* ctx, int mode, uint32_t M, uint32_t N, uint32_t K) {
    if (mode == FG_GEMM_SIMT) return 0;
    if (mode == FG_GEMM_3XTF32) return 1;
    if (mode == FG_GEMM_TF32_BF16X2) return 2;
    if (!ctx->tmap_encode) return 0;
    if (!(M >= 64 && (uint64_t)M * N * K >= (1ull << 22))) return 0;
    return 2;   // AUTO: tf32 main term + bf16 cross terms (same accuracy class, two thirds of the tensor work)
}

}  // namespace

namespace {

struct PairedArg {
    const float* x;
    const void* pairs;      // NULL: made on the fly in the scratch arena
    uint64_t stride;
};

// Forward product with every way of running it.  c_pairs (optional) receives the pairs of C.
int32_t gemm_fwd_core(fg_ctx* ctx, int32_t mode, int32_t transA, int32_t transB, uint32_t M, uint32_t N, uint32_t K,
                      PairedArg A, PairedArg B, float* C, const float* bias, int32_t act, float* preact_out,
                      __nv_bfloat16* c_pairs, uint64_t c_stride) {
    const uint64_t mn = (uint64_t)M * N;
    const int path = pick_path(ctx, mode, M, N, K);
    // The result's pairs, when no GEMM epilogue wrote them.
    auto pairs_after = [&]() -> int32_t { return c_pairs ? launch_pairs(ctx, C, mn, c_pairs, c_stride) : FG_OK; };
    if (path == 0) {
        int32_t s = fg_gemm_simt_launch(ctx, transA, transB, M, N, K, A.x, B.x, C, bias, act, preact_out);
        return s != FG_OK ? s : pairs_after();
    }
    // A skinny output (say 10 classes) is bandwidth-bound on reading A once: no pre-pass, no tensor cores.
    if (mode == FG_GEMM_AUTO && N <= 16 && !transA && !transB) {
        const uint64_t need = fg_gemm_skinny_scratch_bytes(M, N, K) + 1024;
        { int32_t s0 = fg_ws_ensure(ctx, need); if (s0 != FG_OK) return s0; }
        int32_t s = fg_gemm_skinny_n_launch(ctx, M, N, K, A.x, B.x, C, bias, act, preact_out);
        return s != FG_OK ? s : pairs_after();
    }
    const int fmt = path - 1;
    const uint32_t pitch_a = transA ? M : K, pitch_b = transB ? K : N;
    const bool aligned = fg_aligned16(A.x) && fg_aligned16(B.x) && fg_aligned16(C) && (!preact_out || fg_aligned16(preact_out));
    if (fmt == 1 && aligned && paired_shape_ok(ctx, M, N, K, pitch_a, pitch_b) && N % 4 == 0) {
        // The tensors themselves are the operands; pairs the caller does not keep are made here (8 bytes
        // of traffic per element, no transposition).
        const uint64_t mk = (uint64_t)M * K, kn = (uint64_t)K * N;
        const uint64_t need = (A.pairs ? 0 : mk * 4 + 256) + (B.pairs ? 0 : kn * 4 + 256) + kPairPartialBytes + 1024;
        { int32_t s0 = fg_ws_ensure(ctx, need); if (s0 != FG_OK) return s0; }
        int32_t s;
        void* p;
        if (!A.pairs) {
            if ((s = fg_ws_alloc(ctx, mk * 4, &p)) != FG_OK) return s;
            if ((s = launch_pairs(ctx, A.x, mk, (__nv_bfloat16*)p, mk)) != FG_OK) return s;
            A.pairs = p; A.stride = mk;
        }
        if (!B.pairs) {
            if ((s = fg_ws_alloc(ctx, kn * 4, &p)) != FG_OK) return s;
            if ((s = launch_pairs(ctx, B.x, kn, (__nv_bfloat16*)p, kn)) != FG_OK) return s;
            B.pairs = p; B.stride = kn;
        }
        // A operand: rows = M; stored [M,K] (contraction along columns) or, transposed, [K,M].
        const PlaneSet pa = paired_operand(A.x, A.pairs, A.stride, pitch_a, !transA);
        // B operand: rows = N; stored [K,N] (contraction along rows) or, transposed, [N,K].
        const PlaneSet pb = paired_operand(B.x, B.pairs, B.stride, pitch_b, transB != 0);
        return paired_gemm(ctx, pa, pb, M, N, K, C, bias, act, preact_out, PairedOut{c_pairs, c_stride, nullptr, 0, nullptr});
    }
    // Operand planes written by a pre-pass (any shape and alignment; the strict 3xTF32 mode).
    const uint64_t need = planes_bytes(fmt, M, K) + planes_bytes(fmt, N, K) + kPairPartialBytes + 1024;
    { int32_t s0 = fg_ws_ensure(ctx, need); if (s0 != FG_OK) return s0; }
    PlaneSet pa{}, pb{};
    int32_t s;
    if ((s = alloc_planes(ctx, fmt, M, K, &pa)) != FG_OK) return s;
    if ((s = alloc_planes(ctx, fmt, N, K, &pb)) != FG_OK) return s;
    // A operand: [M, K] with K contiguous.
    SplitArgs sa{};
    sa.x = A.x;
    if (!transA) { sa.R = M; sa.C = K; sa.n = pa; }
    else         { sa.R = K; sa.C = M; sa.t = pa; }
    if ((s = launch_split(ctx, fmt, sa)) != FG_OK) return s;
    // B operand: [N, K] with K contiguous.
    SplitArgs sb{};
    sb.x = B.x;
    if (!transB) { sb.R = K; sb.C = N; sb.t = pb; }
    else         { sb.R = N; sb.C = K; sb.n = pb; }
    if ((s = launch_split(ctx, fmt, sb)) != FG_OK) return s;
    if ((s = tc_gemm(ctx, fmt, pa, pb, M, N, K, C, bias, act, preact_out)) != FG_OK) return s;
    return pairs_after();
}

}  // namespace

extern "C" {

int32_t fg_gemm_f32(fg_ctx* ctx, int32_t mode, int32_t transA, int32_t transB, uint32_t M, uint32_t N, uint32_t K,
                    const float* A, const float* B, float* C, const float* bias, int32_t act, float* preact_out) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, A && B && C, "fg_gemm_f32: NULL operand");
    FG_REQUIRE(ctx, M >= 1 && N >= 1 && K >= 1, "fg_gemm_f32: dimensions must be >= 1");
    FG_REQUIRE(ctx, mode >= FG_GEMM_AUTO && mode <= FG_GEMM_TF32_BF16X2, "fg_gemm_f32: unknown mode");
    FG_REQUIRE(ctx, act >= FG_ACT_NONE && act <= FG_ACT_GELU, "fg_gemm_f32: unknown activation");
    FG_REQUIRE(ctx, (uint64_t)M * N < (1ull << 40) && (uint64_t)M * K < (1ull << 40) && (uint64_t)N * K < (1ull << 40),
               "fg_gemm_f32: operand too large");
    return gemm_fwd_core(ctx, mode, transA, transB, M, N, K, PairedArg{A, nullptr, 0}, PairedArg{B, nullptr, 0}, C, bias, act,
                         preact_out, nullptr, 0);
}

int32_t fg_pairs_from_f32(fg_ctx* ctx, const float* x, uint64_t n, void* pairs, uint64_t plane_stride) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, x && pairs, "fg_pairs_from_f32: NULL pointer");
    FG_REQUIRE(ctx, fg_aligned16(x) && fg_aligned16(pairs) && plane_stride % 8 == 0 && plane_stride >= n,
               "fg_pairs_from_f32: pointers must be 16-byte aligned, the plane stride a multiple of 8 and at least n");
    if (n == 0) return FG_OK;
    return launch_pairs(ctx, x, n, (__nv_bfloat16*)pairs, plane_stride);
}

int32_t fg_gemm_paired_f32(fg_ctx* ctx, uint32_t M, uint32_t N, uint32_t K, const float* A, const void* A_pairs,
                           uint64_t A_stride, const float* B, const void* B_pairs, uint64_t B_stride, float* C,
                           const float* bias, int32_t act, float* preact_out, void* C_pairs_out, uint64_t C_stride) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, A && B && C, "fg_gemm_paired_f32: NULL operand");
    FG_REQUIRE(ctx, M >= 1 && N >= 1 && K >= 1, "fg_gemm_paired_f32: dimensions must be >= 1");
    FG_REQUIRE(ctx, act >= FG_ACT_NONE && act <= FG_ACT_GELU, "fg_gemm_paired_f32: unknown activation");
    FG_REQUIRE(ctx, (uint64_t)M * N < (1ull << 40) && (uint64_t)M * K < (1ull << 40) && (uint64_t)N * K < (1ull << 40),
               "fg_gemm_paired_f32: operand too large");
    FG_REQUIRE(ctx, (!A_pairs || (fg_aligned16(A_pairs) && A_stride % 8 == 0 && A_stride >= (uint64_t)M * K)) &&
                        (!B_pairs || (fg_aligned16(B_pairs) && B_stride % 8 == 0 && B_stride >= (uint64_t)K * N)) &&
                        (!C_pairs_out || (fg_aligned16(C_pairs_out) && C_stride % 8 == 0 && C_stride >= (uint64_t)M * N)),
               "fg_gemm_paired_f32: pairs must be 16-byte aligned with a plane stride that is a multiple of 8 and covers the tensor");
    return gemm_fwd_core(ctx, FG_GEMM_AUTO, 0, 0, M, N, K, PairedArg{A, A_pairs, A_stride}, PairedArg{B, B_pairs, B_stride}, C,
                         bias, act, preact_out, (__nv_bfloat16*)C_pairs_out, C_stride);
}

}  // extern "C"

namespace {

// Backward of one layer through the SIMT kernels, the narrow-layer kernels or operand planes written by a
// pre-pass: any shape and alignment.  With exch_buf set, dB and dbias are finished first, the sum of exch_buf
// over the ranks is started on the exchange stream, and dA is computed while it runs.
int32_t gemm_bwd_planes(fg_ctx* ctx, int32_t mode, uint32_t M, uint32_t N, uint32_t K, const float* A, const float* B,
                        const float* dY, int32_t act, const float* saved, float* dA, float* dB, float* dbias,
                        float* dZ_out, float* exch_buf, uint64_t exch_count) {
    const bool fuse = act != FG_ACT_NONE;
    const int path = pick_path(ctx, mode, M, N, K);
    const uint64_t mn = (uint64_t)M * N;

    if (path == 0) {
        // Exact path: materialise dZ, then two SIMT GEMMs.
        const float* dz = dY;
        {
            uint64_t need = mn * 4 + (uint64_t)((M + 255) / 256) * N * 4 + 1024;
            { int32_t s0 = fg_ws_ensure(ctx, need); if (s0 != FG_OK) return s0; }
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
        if (dB) { int32_t s = fg_gemm_simt_launch(ctx, 1, 0, K, N, M, A, dz, dB, nullptr, FG_ACT_NONE, nullptr); if (s) return s; }
        if (dbias) { int32_t s = fg_colsum_launch(ctx, M, N, dz, dbias); if (s) return s; }
        if (exch_buf) { int32_t s = fg_allreduce_sum_f32(ctx, exch_buf, exch_count); if (s) return s; }
        if (dA) { int32_t s = fg_gemm_simt_launch(ctx, 0, 1, M, K, N, dz, B, dA, nullptr, FG_ACT_NONE, nullptr); if (s) return s; }
        return FG_OK;
    }

    // Tensor-core path.  Scratch: dZ planes in both orientations, B planes, Aᵀ planes, dZ itself
    // when a bias gradient is wanted, and the column-sum partials.
    const int fmt = path - 1;
    // A skinny layer (N <= 16, say 10 classes): dA is bound by writing it once and dB by reading A once, so
    // both run as plain-FMA kernels on dZ itself; the operand pre-passes and a tensor-core GEMM that could
    // only fill M/128 CTAs would cost several times more.
    const bool skinny = mode == FG_GEMM_AUTO && N <= 16;
    const bool tc_da = dA && !skinny, tc_db = dB && !skinny;
    uint64_t need = 2048;
    if (tc_da) need += planes_bytes(fmt, M, N) + planes_bytes(fmt, K, N) + kPairPartialBytes;
    if (tc_db) need += planes_bytes(fmt, N, M) + planes_bytes(fmt, K, M) + kPairPartialBytes;
    if (skinny) need += mn * 4 + 256 + fg_gemm_skinny_scratch_bytes(M, N, K);
    if (dbias) need += (uint64_t)((M + 31) / 32) * N * 4 + 256;   // per-tile column sums from the pre-pass
    { int32_t s0 = fg_ws_ensure(ctx, need); if (s0 != FG_OK) return s0; }
    PlaneSet dz_n{}, dz_t{}, b_n{}, a_t{};
    void* dz_val = dZ_out;
    int32_t s;
    if (tc_da) {
        if ((s = alloc_planes(ctx, fmt, M, N, &dz_n)) != FG_OK) return s;
        if ((s = alloc_planes(ctx, fmt, K, N, &b_n)) != FG_OK) return s;
    }
    if (tc_db) {
        if ((s = alloc_planes(ctx, fmt, N, M, &dz_t)) != FG_OK) return s;
        if ((s = alloc_planes(ctx, fmt, K, M, &a_t)) != FG_OK) return s;
    }
    if (skinny && fuse && !dz_val && (dA || dB)) {      // the skinny kernels read dZ itself
        if ((s = fg_ws_alloc(ctx, mn * 4, &dz_val)) != FG_OK) return s;
    }
    void* cs_part = nullptr;
    if (dbias && (s = fg_ws_alloc(ctx, (uint64_t)((M + 31) / 32) * N * 4, &cs_part)) != FG_OK) return s;
    SplitArgs sz{};
    sz.x = dY; sz.saved = fuse ? saved : nullptr; sz.act = act; sz.R = M; sz.C = N;
    sz.n = dz_n; sz.t = dz_t;
    sz.value_out = (float*)dz_val;
    sz.colsum_part = (float*)cs_part;
    uint32_t cs_chunks = 0;
    if (tc_da || tc_db || dz_val || dbias) {
        if ((s = launch_split(ctx, fmt, sz, &cs_chunks)) != FG_OK) return s;
    }
    const float* dz_src = dz_val ? (const float*)dz_val : dY;   // dZ == dY when there is no activation
    // weight and bias gradients first: with an exchange requested, it starts as soon as they are complete
    if (skinny && dB && (s = fg_gemm_skinny_tn_launch(ctx, M, K, N, A, dz_src, dB)) != FG_OK) return s;
    if (tc_db) {
        // dB[K,N] = Aᵀ · dZ: contraction over M; operands are Aᵀ [K,M] and dZᵀ [N,M].
        SplitArgs sa{};
        sa.x = A; sa.R = M; sa.C = K; sa.t = a_t;
        if ((s = launch_split(ctx, fmt, sa)) != FG_OK) return s;
        if ((s = tc_gemm(ctx, fmt, a_t, dz_t, K, N, M, dB, nullptr, FG_ACT_NONE, nullptr)) != FG_OK) return s;
    }
    if (dbias) {
        // the pre-pass left one row of column sums per row tile: fold them in a fixed order
        if ((s = fg_colsum_fold_launch(ctx, N, cs_chunks, (const float*)cs_part, dbias)) != FG_OK) return s;
    }
    if (exch_buf && (s = fg_allreduce_sum_f32(ctx, exch_buf, exch_count)) != FG_OK) return s;
    if (tc_da) {
        // dA[M,K] = dZ[M,N] · Bᵀ: contraction over N; B [K,N] is already "rows = K, contraction contiguous".
        SplitArgs sb{};
        sb.x = B; sb.R = K; sb.C = N; sb.n = b_n;
        if ((s = launch_split(ctx, fmt, sb)) != FG_OK) return s;
        if ((s = tc_gemm(ctx, fmt, dz_n, b_n, M, K, N, dA, nullptr, FG_ACT_NONE, nullptr)) != FG_OK) return s;
    }
    if (skinny && dA && (s = fg_gemm_skinny_nt_launch(ctx, M, K, N, dz_src, B, dA)) != FG_OK) return s;
    return FG_OK;
}

// Scratch gemm_bwd_planes may carve (an upper bound over its three routes).
uint64_t bwd_planes_need(uint32_t M, uint32_t N, uint32_t K) {
    const uint64_t mn = (uint64_t)M * N;
    uint64_t need = 4096 + mn * 4 + (uint64_t)((M + 31) / 32) * N * 4;
    need += planes_bytes(1, M, N) + planes_bytes(1, K, N) + planes_bytes(1, N, M) + planes_bytes(1, K, M) + 2 * kPairPartialBytes;
    need += fg_gemm_skinny_scratch_bytes(M, N, K);
    return need;
}

// Both products of a backward step straight from the f32 tensors and their pairs?
bool bwd_paired_ok(const fg_ctx* ctx, uint32_t M, uint32_t N, uint32_t K, bool want_dA, bool want_dB) {
    if (N % 8 != 0 || K % 8 != 0) return false;
    if (want_dB && !paired_shape_ok(ctx, K, N, M, K, N)) return false;     // dB [K,N], contraction over M
    if (want_dA && !paired_shape_ok(ctx, M, K, N, N, N)) return false;     // dA [M,K], contraction over N
    return want_dA || want_dB;
}

// Backward of Y = A·B given dZ = dL/dY (already multiplied by this layer's act'), on f32 tensors with pairs:
//   dB [K,N] = Aᵀ·dZ, then the exchange (if asked for), then
//   dA [M,K] = (dZ·Bᵀ) * act'(o.mul_saved) with its pairs (o.pairs) and its column sums (dbias_prev [K]) --
//   i.e. the dZ of the layer below and that layer's bias gradient come out of the dA epilogue.
// Pairs that are not supplied are made in the scratch arena.  The caller has reserved bwd_paired_need().
uint64_t bwd_paired_need(uint32_t M, uint32_t N, uint32_t K) {
    return 4ull * ((uint64_t)M * K + (uint64_t)K * N + (uint64_t)M * N) + (uint64_t)((M + 31) / 32) * K * 4 +
           2 * kPairPartialBytes + 4096 + fg_gemm_skinny_scratch_bytes(M, N, K) + bwd_planes_need(M, N, K);
}

int32_t gemm_bwd_paired_core(fg_ctx* ctx, uint32_t M, uint32_t N, uint32_t K, PairedArg A, PairedArg B, PairedArg dZ, float* dB,
                             float* dA, PairedOut o, float* dbias_prev, float* exch_buf, uint64_t exch_count) {
    int32_t s;
    void* p;
    const uint32_t cs_chunks = (M + 31) / 32;
    float* cs_part = nullptr;
    if (dA && dbias_prev) {
        if ((s = fg_ws_alloc(ctx, (uint64_t)cs_chunks * K * 4, &p)) != FG_OK) return s;
        cs_part = (float*)p;
    }
    if (N <= 16) {
        // narrow layer: plain-FMA streaming kernels on the tensors themselves
        if (dB && (s = fg_gemm_skinny_tn_launch(ctx, M, K, N, A.x, dZ.x, dB)) != FG_OK) return s;
        if (exch_buf && (s = fg_allreduce_sum_f32(ctx, exch_buf, exch_count)) != FG_OK) return s;
        if (dA) {
            const fg_skinny_extras ex{o.mul_saved, o.mul_act, o.pairs, o.stride, cs_part};
            uint32_t cs_rows = 0;
            if ((s = fg_gemm_skinny_nt_launch(ctx, M, K, N, dZ.x, B.x, dA, &ex, &cs_rows)) != FG_OK) return s;
            if (cs_part && (s = fg_colsum_fold_launch(ctx, K, cs_rows, cs_part, dbias_prev)) != FG_OK) return s;
        }
        return FG_OK;
    }
    const bool aligned = (!dB || (fg_aligned16(A.x) && fg_aligned16(dB))) && (!dA || (fg_aligned16(B.x) && fg_aligned16(dA))) &&
                         fg_aligned16(dZ.x) && (!o.mul_saved || fg_aligned16(o.mul_saved));
    if (aligned && bwd_paired_ok(ctx, M, N, K, dA != nullptr, dB != nullptr)) {
        const uint64_t mk = (uint64_t)M * K, kn = (uint64_t)K * N, mn = (uint64_t)M * N;
        if (!dZ.pairs) {
            if ((s = fg_ws_alloc(ctx, mn * 4, &p)) != FG_OK) return s;
            if ((s = launch_pairs(ctx, dZ.x, mn, (__nv_bfloat16*)p, mn)) != FG_OK) return s;
            dZ.pairs = p; dZ.stride = mn;
        }
        if (dB) {
            if (!A.pairs) {
                if ((s = fg_ws_alloc(ctx, mk * 4, &p)) != FG_OK) return s;
                if ((s = launch_pairs(ctx, A.x, mk, (__nv_bfloat16*)p, mk)) != FG_OK) return s;
                A.pairs = p; A.stride = mk;
            }
            // operands Aᵀ (rows = K) and dZᵀ (rows = N), both read from [M, .] storage: contraction over the rows
            const PlaneSet pa = paired_operand(A.x, A.pairs, A.stride, K, false);
            const PlaneSet pz = paired_operand(dZ.x, dZ.pairs, dZ.stride, N, false);
            if ((s = paired_gemm(ctx, pa, pz, K, N, M, dB, nullptr, FG_ACT_NONE, nullptr, PairedOut{nullptr, 0, nullptr, 0, nullptr})) != FG_OK)
                return s;
        }
        if (exch_buf && (s = fg_allreduce_sum_f32(ctx, exch_buf, exch_count)) != FG_OK) return s;
        if (dA) {
            if (!B.pairs) {
                if ((s = fg_ws_alloc(ctx, kn * 4, &p)) != FG_OK) return s;
                if ((s = launch_pairs(ctx, B.x, kn, (__nv_bfloat16*)p, kn)) != FG_OK) return s;
                B.pairs = p; B.stride = kn;
            }
            // operands dZ (rows = M) and B (rows = K), both with the contraction index N contiguous
            const PlaneSet pz = paired_operand(dZ.x, dZ.pairs, dZ.stride, N, true);
            const PlaneSet pb = paired_operand(B.x, B.pairs, B.stride, N, true);
            PairedOut po = o;
            po.colsum_part = cs_part;
            if ((s = paired_gemm(ctx, pz, pb, M, K, N, dA, nullptr, FG_ACT_NONE, nullptr, po)) != FG_OK) return s;
            if (cs_part && (s = fg_colsum_fold_launch(ctx, K, cs_chunks, cs_part, dbias_prev)) != FG_OK) return s;
        }
        return FG_OK;
    }
    // Any other shape: operand planes, then what the dA epilogue would have done as passes of their own.
    if ((s = gemm_bwd_planes(ctx, FG_GEMM_AUTO, M, N, K, A.x, B.x, dZ.x, FG_ACT_NONE, nullptr, dA, dB, nullptr, nullptr, exch_buf,
                             exch_count)) != FG_OK)
        return s;
    if (!dA) return FG_OK;
    const uint64_t mk = (uint64_t)M * K;
    if (K % 4 == 0 && fg_aligned16(dA) && (!o.mul_saved || fg_aligned16(o.mul_saved))) {
        if (o.mul_saved || o.pairs || cs_part) {
            if ((s = launch_dz_pairs(ctx, M, K, dA, o.mul_saved, o.mul_act, o.mul_saved ? dA : nullptr, o.pairs, o.stride, cs_part)) != FG_OK)
                return s;
            if (cs_part && (s = fg_colsum_fold_launch(ctx, K, cs_chunks, cs_part, dbias_prev)) != FG_OK) return s;
        }
        return FG_OK;
    }
    if (o.mul_saved && (s = fg_act_bwd_launch(ctx, mk, o.mul_act, dA, o.mul_saved, dA)) != FG_OK) return s;
    if (o.pairs && (s = launch_pairs(ctx, dA, mk, o.pairs, o.stride)) != FG_OK) return s;
    if (dbias_prev && (s = fg_colsum_launch(ctx, M, K, dA, dbias_prev)) != FG_OK) return s;
    return FG_OK;
}

// Backward of Y = act(A·B + bias) from dY: forms dZ = dY * act'(saved) first.
int32_t gemm_bwd_impl(fg_ctx* ctx, int32_t mode, uint32_t M, uint32_t N, uint32_t K, const float* A, const float* B,
                      const float* dY, int32_t act, const float* saved, float* dA, float* dB, float* dbias,
                      float* dZ_out, float* exch_buf, uint64_t exch_count) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, dY != nullptr, "fg_gemm_bwd_f32: dY is NULL");
    FG_REQUIRE(ctx, M >= 1 && N >= 1 && K >= 1, "fg_gemm_bwd_f32: dimensions must be >= 1");
    FG_REQUIRE(ctx, mode >= FG_GEMM_AUTO && mode <= FG_GEMM_TF32_BF16X2, "fg_gemm_bwd_f32: unknown mode");
    FG_REQUIRE(ctx, act >= FG_ACT_NONE && act <= FG_ACT_GELU, "fg_gemm_bwd_f32: unknown activation");
    FG_REQUIRE(ctx, act == FG_ACT_NONE || saved, "fg_gemm_bwd_f32: the activation backward needs the saved tensor");
    FG_REQUIRE(ctx, !dA || B, "fg_gemm_bwd_f32: dA needs B");
    FG_REQUIRE(ctx, !dB || A, "fg_gemm_bwd_f32: dB needs A");
    const bool fuse = act != FG_ACT_NONE;
    const int path = pick_path(ctx, mode, M, N, K);
    const bool aligned = fg_aligned16(dY) && (!saved || fg_aligned16(saved)) && (!dZ_out || fg_aligned16(dZ_out)) &&
                         (!dA || (fg_aligned16(B) && fg_aligned16(dA))) && (!dB || (fg_aligned16(A) && fg_aligned16(dB)));
    if (path == 2 && N > 16 && aligned && bwd_paired_ok(ctx, M, N, K, dA != nullptr, dB != nullptr)) {
        // dZ with its pairs and the bias gradient's partials in one pass, then both products from the tensors themselves
        const uint64_t mn = (uint64_t)M * N;
        const uint32_t cs_chunks = (M + 31) / 32;
        const uint64_t need = bwd_paired_need(M, N, K) + mn * 4 + (uint64_t)cs_chunks * N * 4 + 1024;
        { int32_t s0 = fg_ws_ensure(ctx, need); if (s0 != FG_OK) return s0; }
        int32_t s;
        void *pz = nullptr, *dzb = dZ_out, *csp = nullptr;
        if ((s = fg_ws_alloc(ctx, mn * 4, &pz)) != FG_OK) return s;
        if (fuse && !dzb && (s = fg_ws_alloc(ctx, mn * 4, &dzb)) != FG_OK) return s;
        if (dbias && (s = fg_ws_alloc(ctx, (uint64_t)cs_chunks * N * 4, &csp)) != FG_OK) return s;
        if ((s = launch_dz_pairs(ctx, M, N, dY, fuse ? saved : nullptr, act, (float*)dzb, (__nv_bfloat16*)pz, mn, (float*)csp)) != FG_OK)
            return s;
        if (dbias && (s = fg_colsum_fold_launch(ctx, N, cs_chunks, (const float*)csp, dbias)) != FG_OK) return s;
        const float* dz_src = dzb ? (const float*)dzb : dY;
        return gemm_bwd_paired_core(ctx, M, N, K, PairedArg{A, nullptr, 0}, PairedArg{B, nullptr, 0}, PairedArg{dz_src, pz, mn}, dB, dA,
                                    PairedOut{nullptr, 0, nullptr, 0, nullptr}, nullptr, exch_buf, exch_count);
    }
    return gemm_bwd_planes(ctx, mode, M, N, K, A, B, dY, act, saved, dA, dB, dbias, dZ_out, exch_buf, exch_count);
}

}  // namespace

extern "C" {

int32_t fg_gemm_bwd_f32(fg_ctx* ctx, int32_t mode, uint32_t M, uint32_t N, uint32_t K, const float* A, const float* B,
                        const float* dY, int32_t act, const float* saved, float* dA, float* dB, float* dbias,
                        float* dZ_out) {
    return gemm_bwd_impl(ctx, mode, M, N, K, A, B, dY, act, saved, dA, dB, dbias, dZ_out, nullptr, 0);
}

int32_t fg_gemm_bwd_exchange_f32(fg_ctx* ctx, int32_t mode, uint32_t M, uint32_t N, uint32_t K, const float* A,
                                 const float* B, const float* dY, int32_t act, const float* saved, float* dA, float* dB,
                                 float* dbias, float* exch_buf, uint64_t exch_count) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, exch_buf != nullptr && exch_count > 0, "fg_gemm_bwd_exchange_f32: nothing to exchange");
    if (!ctx->comm) return fg_fail(ctx, FG_ERR_NOT_INITIALIZED, "fg_gemm_bwd_exchange_f32: call fg_comm_init first");
    return gemm_bwd_impl(ctx, mode, M, N, K, A, B, dY, act, saved, dA, dB, dbias, nullptr, exch_buf, exch_count);
}

int32_t fg_gemm_bwd_paired_f32(fg_ctx* ctx, uint32_t M, uint32_t N, uint32_t K, const float* A, const void* A_pairs,
                               uint64_t A_stride, const float* B, const void* B_pairs, uint64_t B_stride, const float* dZ,
                               const void* dZ_pairs, uint64_t dZ_stride, float* dB, float* dbias, float* dA,
                               int32_t below_act, const float* below_saved, void* dA_pairs_out, uint64_t dA_stride,
                               float* below_dbias, float* exch_buf, uint64_t exch_count) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, dZ != nullptr, "fg_gemm_bwd_paired_f32: dZ is NULL");
    FG_REQUIRE(ctx, M >= 1 && N >= 1 && K >= 1, "fg_gemm_bwd_paired_f32: dimensions must be >= 1");
    FG_REQUIRE(ctx, below_act >= FG_ACT_NONE && below_act <= FG_ACT_GELU, "fg_gemm_bwd_paired_f32: unknown activation");
    FG_REQUIRE(ctx, below_act == FG_ACT_NONE || below_saved, "fg_gemm_bwd_paired_f32: the activation backward needs the saved tensor");
    FG_REQUIRE(ctx, !dA || B, "fg_gemm_bwd_paired_f32: dA needs B");
    FG_REQUIRE(ctx, !dB || A, "fg_gemm_bwd_paired_f32: dB needs A");
    FG_REQUIRE(ctx, dA || (!dA_pairs_out && !below_dbias), "fg_gemm_bwd_paired_f32: pairs and bias gradient of dA need dA");
    auto pairs_ok = [](const void* p, uint64_t stride, uint64_t n) { return !p || (fg_aligned16(p) && stride % 8 == 0 && stride >= n); };
    FG_REQUIRE(ctx, pairs_ok(A_pairs, A_stride, (uint64_t)M * K) && pairs_ok(B_pairs, B_stride, (uint64_t)K * N) &&
                        pairs_ok(dZ_pairs, dZ_stride, (uint64_t)M * N) && pairs_ok(dA_pairs_out, dA_stride, (uint64_t)M * K),
               "fg_gemm_bwd_paired_f32: pairs must be 16-byte aligned with a plane stride that is a multiple of 8 and covers the tensor");
    if (exch_buf && !ctx->comm) return fg_fail(ctx, FG_ERR_NOT_INITIALIZED, "fg_gemm_bwd_paired_f32: call fg_comm_init first");
    FG_REQUIRE(ctx, !exch_buf || exch_count > 0, "fg_gemm_bwd_paired_f32: nothing to exchange");
    { int32_t s0 = fg_ws_ensure(ctx, bwd_paired_need(M, N, K)); if (s0 != FG_OK) return s0; }
    if (dbias) {
        const int32_t s0 = fg_colsum_launch(ctx, M, N, dZ, dbias);
        if (s0 != FG_OK) return s0;
    }
    const bool mul = below_act != FG_ACT_NONE;
    return gemm_bwd_paired_core(ctx, M, N, K, PairedArg{A, A_pairs, A_stride}, PairedArg{B, B_pairs, B_stride},
                                PairedArg{dZ, dZ_pairs, dZ_stride}, dB, dA,
                                PairedOut{(__nv_bfloat16*)dA_pairs_out, dA_stride, mul ? below_saved : nullptr, below_act, nullptr},
                                below_dbias, exch_buf, exch_count);
}

// Batched forms: `batch` independent products, operand t at base + t*stride (strides in elements).
// The reference steps A, B and C by one matrix per Z index of a rank-3 matmul (kernel/forward.rs:159-190).
// Rank-3 products.  Small matrices (the SIMT path's range) run as ONE launch with the matrix index in the grid's
// z, as the reference's generated kernel does (kernel/forward.rs:159-190).  Larger ones use the tensor cores: the
// bf16 pairs of the whole batch are made by one pass per operand, then one GEMM launch per matrix reads its slice
// (batch + 2 launches, and a launch that fills the GPU gains nothing from being merged with its neighbours).
int32_t fg_gemm_batched_f32(fg_ctx* ctx, int32_t mode, uint32_t batch, uint32_t M, uint32_t N, uint32_t K, const float* A,
                            uint64_t strideA, const float* B, uint64_t strideB, float* C, uint64_t strideC,
                            const float* bias, int32_t act, float* preact_out) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, A && B && C, "fg_gemm_batched_f32: NULL pointer");
    FG_REQUIRE(ctx, act >= FG_ACT_NONE && act <= FG_ACT_GELU, "fg_gemm_batched_f32: unknown activation");
    FG_REQUIRE(ctx, strideA >= (uint64_t)M * K && strideB >= (uint64_t)K * N && strideC >= (uint64_t)M * N,
               "fg_gemm_batched_f32: a stride is smaller than its matrix (for one B shared by all products, "
               "call fg_gemm_f32 with batch*M rows)");
    if (batch == 0 || (uint64_t)M * N == 0) return FG_OK;
    if (pick_path(ctx, mode, M, N, K) == 0 && batch <= 65535 && K > 0)
        return fg_gemm_simt_batched_launch(ctx, 0, 0, batch, M, N, K, A, strideA, B, strideB, C, strideC, bias, act, preact_out);
    const bool dense = strideA == (uint64_t)M * K && strideB == (uint64_t)K * N;
    // the condition under which every per-matrix call below takes the path that reads pairs
    const bool shared_pairs = dense && mode == FG_GEMM_AUTO && N > 16 && N % 4 == 0 && strideC % 4 == 0 && fg_aligned16(A) &&
                              fg_aligned16(B) && fg_aligned16(C) && (!preact_out || fg_aligned16(preact_out)) &&
                              paired_shape_ok(ctx, M, N, K, K, N);
    __nv_bfloat16 *pa = nullptr, *pb = nullptr;
    const uint64_t na = (uint64_t)batch * M * K, nb = (uint64_t)batch * K * N;
    if (shared_pairs) {
        void* p;
        int32_t s = fg_ws_ensure(ctx, (na + nb) * 4 + 2 * kPairPartialBytes + 8192);
        if (s != FG_OK) return s;
        if ((s = fg_ws_alloc(ctx, na * 4, &p)) != FG_OK) return s;
        pa = (__nv_bfloat16*)p;
        if ((s = fg_ws_alloc(ctx, nb * 4, &p)) != FG_OK) return s;
        pb = (__nv_bfloat16*)p;
        if ((s = launch_pairs(ctx, A, na, pa, na)) != FG_OK) return s;
        if ((s = launch_pairs(ctx, B, nb, pb, nb)) != FG_OK) return s;
    }
    for (uint32_t t = 0; t < batch; ++t) {
        int32_t s;
        if (shared_pairs) {
            // carve nothing more from the arena: the slices above stay valid for every matrix
            const uint64_t keep = ctx->ws_used;
            s = gemm_fwd_core(ctx, mode, 0, 0, M, N, K, PairedArg{A + t * strideA, pa + t * strideA, na},
                              PairedArg{B + t * strideB, pb + t * strideB, nb}, C + t * strideC, bias, act,
                              preact_out ? preact_out + t * strideC : nullptr, nullptr, 0);
            ctx->ws_used = keep;
        } else {
            s = fg_gemm_f32(ctx, mode, 0, 0, M, N, K, A + t * strideA, B + t * strideB, C + t * strideC, bias, act,
                            preact_out ? preact_out + t * strideC : nullptr);
        }
        if (s != FG_OK) return s;
    }
    return FG_OK;
}

int32_t fg_gemm_batched_bwd_f32(fg_ctx* ctx, int32_t mode, uint32_t batch, uint32_t M, uint32_t N, uint32_t K,
                                const float* A, uint64_t strideA, const float* B, uint64_t strideB, const float* dY,
                                uint64_t strideC, int32_t act, const float* saved, float* dA, float* dB) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, dY != nullptr, "fg_gemm_batched_bwd_f32: dY is NULL");
    FG_REQUIRE(ctx, act >= FG_ACT_NONE && act <= FG_ACT_GELU, "fg_gemm_batched_bwd_f32: unknown activation");
    FG_REQUIRE(ctx, act == FG_ACT_NONE || saved, "fg_gemm_batched_bwd_f32: saved tensor required");
    FG_REQUIRE(ctx, (!dA || B) && (!dB || A), "fg_gemm_batched_bwd_f32: dA needs B, dB needs A");
    FG_REQUIRE(ctx, strideA >= (uint64_t)M * K && strideB >= (uint64_t)K * N && strideC >= (uint64_t)M * N,
               "fg_gemm_batched_bwd_f32: a stride is smaller than its matrix");
    if (batch == 0 || (uint64_t)M * N == 0 || (!dA && !dB)) return FG_OK;
    if (pick_path(ctx, mode, M, N, K) == 0 && batch <= 65535 && strideC == (uint64_t)M * N) {
        // three launches for the whole batch: dZ = dY * act'(saved), dB[t] = A[t]^T dZ[t], dA[t] = dZ[t] B[t]^T
        const float* dz = dY;
        if (act != FG_ACT_NONE) {
            const uint64_t n = (uint64_t)batch * M * N;
            void* p;
            int32_t s = fg_ws_ensure(ctx, n * 4 + 512);
            if (s != FG_OK) return s;
            if ((s = fg_ws_alloc(ctx, n * 4, &p)) != FG_OK) return s;
            if ((s = fg_act_bwd_launch(ctx, n, act, dY, saved, (float*)p)) != FG_OK) return s;
            dz = (const float*)p;
        }
        int32_t s;
        if (dB && (s = fg_gemm_simt_batched_launch(ctx, 1, 0, batch, K, N, M, A, strideA, dz, strideC, dB, strideB, nullptr,
                                                   FG_ACT_NONE, nullptr)) != FG_OK) return s;
        if (dA && (s = fg_gemm_simt_batched_launch(ctx, 0, 1, batch, M, K, N, dz, strideC, B, strideB, dA, strideA, nullptr,
                                                   FG_ACT_NONE, nullptr)) != FG_OK) return s;
        return FG_OK;
    }
    for (uint32_t t = 0; t < batch; ++t) {
        int32_t s = fg_gemm_bwd_f32(ctx, mode, M, N, K, A ? A + t * strideA : nullptr, B ? B + t * strideB : nullptr,
                                    dY + t * strideC, act, saved ? saved + t * strideC : nullptr,
                                    dA ? dA + t * strideA : nullptr, dB ? dB + t * strideB : nullptr, nullptr, nullptr);
        if (s != FG_OK) return s;
    }
    return FG_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------
// 16-bit storage (f16 / bf16 tensors, f32 accumulation).  The operands are multiplied as they
// are: one kind::f16 MMA per 16 values of k, no operand planes.  What the tensor core needs is
// the contraction index contiguous, rows 16-byte aligned; an operand that already lies that way
// is loaded in place, the others go through prep16_kernel (copy with padded pitch and/or
// transpose, optionally fused with dY * act'(saved) and the bias gradient's column sums).
// ------------------------------------------------------------------------------------
namespace {

struct Prep16Args {
    const void* x;        // [R, C] 16-bit
    const void* saved;    // non-NULL: value = x * act'(saved), rounded to the storage type
    int act;
    uint32_t R, C;
    void* n_out;          // [R][ld_n] or NULL
    void* t_out;          // [C][ld_t] or NULL
    uint32_t ld_n, ld_t;
    float* colsum_part;   // [ceil(R/32)][C] f32 or NULL
};

template <typename T> __device__ __forceinline__ float lp_to_float(T v);
template <> __device__ __forceinline__ float lp_to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float lp_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T lp_from_float(float v);
template <> __device__ __forceinline__ __half lp_from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 lp_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) prep16_kernel(const Prep16Args a) {
    __shared__ T tile[32][33];
    __shared__ float cs[8][33];
    const uint32_t c = blockIdx.x * 32 + threadIdx.x;
    const uint32_t r0 = blockIdx.y * 32;
    float colsum = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lr = threadIdx.y + 8 * k, r = r0 + lr;
        T v = lp_from_float<T>(0.0f);
        if (r < a.R && c < a.C) {
            const size_t i = (size_t)r * a.C + c;
            v = static_cast<const T*>(a.x)[i];
            if (a.saved)
                v = lp_from_float<T>(lp_to_float(v) * fg_act_grad(a.act, lp_to_float(static_cast<const T*>(a.saved)[i])));
            if (a.n_out) static_cast<T*>(a.n_out)[(size_t)r * a.ld_n + c] = v;
            colsum += lp_to_float(v);
        }
        tile[lr][threadIdx.x] = v;
    }
    if (a.colsum_part) cs[threadIdx.y][threadIdx.x] = colsum;
    __syncthreads();
    if (a.colsum_part && threadIdx.y == 0 && c < a.C) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += cs[k][threadIdx.x];
        a.colsum_part[(size_t)blockIdx.y * a.C + c] = t;
    }
    if (a.t_out) {
        const uint32_t tr = r0 + threadIdx.x;          // row of x = column of the transposed copy
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t lc = threadIdx.y + 8 * k, tc = blockIdx.x * 32 + lc;
            if (tc < a.C && tr < a.R) static_cast<T*>(a.t_out)[(size_t)tc * a.ld_t + tr] = tile[threadIdx.x][lc];
        }
    }
}

int32_t launch_prep16(fg_ctx* ctx, int dtype, const Prep16Args& a, uint32_t* chunks_out = nullptr) {
    dim3 grid((a.C + 31) / 32, (a.R + 31) / 32), block(32, 8);
    if (grid.y > 65535) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "16-bit GEMM operand has too many rows");
    if (chunks_out) *chunks_out = grid.y;
    if (dtype == FG_DTYPE_F16) prep16_kernel<__half><<<grid, block, 0, ctx->stream>>>(a);
    else prep16_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>(a);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

inline uint32_t pad8(uint32_t x) { return (x + 7u) & ~7u; }
// An operand [rows, kdim] whose contraction index is contiguous can be loaded in place when every row
// starts on a 16-byte boundary.
inline bool in_place16(const void* p, uint32_t kdim) { return fg_aligned16(p) && kdim % 8 == 0; }

int32_t lowp_gemm(fg_ctx* ctx, int dtype, const void* a_rows, uint32_t lda, const void* b_rows, uint32_t ldb, uint32_t M,
                  uint32_t N, uint32_t K, void* C, const float* bias32, int act, void* preact) {
    PlaneSet pa{nullptr, (__nv_bfloat16*)a_rows, 0, lda}, pb{nullptr, (__nv_bfloat16*)b_rows, 0, ldb};
    Epilogue ep{(float*)C, bias32, (float*)preact, M, N, K, act, ctx->dev_status, nullptr, 0, 1, dtype};
    return dtype == FG_DTYPE_BF16 ? launch_tc_pair<32, 2>(ctx, pa, pb, ep) : launch_tc_pair<32, 3>(ctx, pa, pb, ep);
}

}  // namespace

extern "C" {

int32_t fg_gemm_lowp(fg_ctx* ctx, int32_t dtype, uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, void* C,
                     const void* bias, int32_t act, void* preact_out) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, dtype == FG_DTYPE_F16 || dtype == FG_DTYPE_BF16, "fg_gemm_lowp: dtype must be f16 or bf16");
    FG_REQUIRE(ctx, A && B && C, "fg_gemm_lowp: NULL operand");
    FG_REQUIRE(ctx, M >= 1 && N >= 1 && K >= 1, "fg_gemm_lowp: dimensions must be >= 1");
    FG_REQUIRE(ctx, act >= FG_ACT_NONE && act <= FG_ACT_GELU, "fg_gemm_lowp: unknown activation");
    FG_REQUIRE(ctx, fg_aligned16(C) && (!preact_out || fg_aligned16(preact_out)), "fg_gemm_lowp: outputs must be 16-byte aligned");
    if (!ctx->tmap_encode) return fg_fail(ctx, FG_ERR_UNSUPPORTED_FEATURE, "fg_gemm_lowp: tensor maps unavailable");
    const uint32_t ldk = pad8(K);
    const bool a_direct = in_place16(A, K);
    const uint64_t need = (uint64_t)N * ldk * 2 + (a_direct ? 0 : (uint64_t)M * ldk * 2) + (uint64_t)N * 4 + kPairPartialBytes + 2048;
    { int32_t s0 = fg_ws_ensure(ctx, need); if (s0 != FG_OK) return s0; }
    int32_t s;
    void *bt, *ac = nullptr, *bias32 = nullptr;
    if ((s = fg_ws_alloc(ctx, (uint64_t)N * ldk * 2, &bt)) != FG_OK) return s;
    Prep16Args pb{};
    pb.x = B; pb.R = K; pb.C = N; pb.t_out = bt; pb.ld_t = ldk;          // B [K,N] -> [N][K]
    if ((s = launch_prep16(ctx, dtype, pb)) != FG_OK) return s;
    const void* a_rows = A;
    uint32_t lda = K;
    if (!a_direct) {
        if ((s = fg_ws_alloc(ctx, (uint64_t)M * ldk * 2, &ac)) != FG_OK) return s;
        Prep16Args pa{};
        pa.x = A; pa.R = M; pa.C = K; pa.n_out = ac; pa.ld_n = ldk;
        if ((s = launch_prep16(ctx, dtype, pa)) != FG_OK) return s;
        a_rows = ac;
        lda = ldk;
    }
    if (bias) {
        if ((s = fg_ws_alloc(ctx, (uint64_t)N * 4, &bias32)) != FG_OK) return s;
        if ((s = fg_convert_launch(ctx, bias, dtype, bias32, FG_DTYPE_F32, N)) != FG_OK) return s;
    }
    return lowp_gemm(ctx, dtype, a_rows, lda, bt, ldk, M, N, K, C, (const float*)bias32, act, preact_out);
}

int32_t fg_gemm_bwd_lowp(fg_ctx* ctx, int32_t dtype, uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B,
                         const void* dY, int32_t act, const void* saved, void* dA, void* dB, void* dbias) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, dtype == FG_DTYPE_F16 || dtype == FG_DTYPE_BF16, "fg_gemm_bwd_lowp: dtype must be f16 or bf16");
    FG_REQUIRE(ctx, dY != nullptr, "fg_gemm_bwd_lowp: dY is NULL");
    FG_REQUIRE(ctx, M >= 1 && N >= 1 && K >= 1, "fg_gemm_bwd_lowp: dimensions must be >= 1");
    FG_REQUIRE(ctx, act >= FG_ACT_NONE && act <= FG_ACT_GELU, "fg_gemm_bwd_lowp: unknown activation");
    FG_REQUIRE(ctx, act == FG_ACT_NONE || saved, "fg_gemm_bwd_lowp: the activation backward needs the saved tensor");
    FG_REQUIRE(ctx, !dA || B, "fg_gemm_bwd_lowp: dA needs B");
    FG_REQUIRE(ctx, !dB || A, "fg_gemm_bwd_lowp: dB needs A");
    FG_REQUIRE(ctx, (!dA || fg_aligned16(dA)) && (!dB || fg_aligned16(dB)), "fg_gemm_bwd_lowp: outputs must be 16-byte aligned");
    if (!ctx->tmap_encode) return fg_fail(ctx, FG_ERR_UNSUPPORTED_FEATURE, "fg_gemm_bwd_lowp: tensor maps unavailable");
    const bool fuse = act != FG_ACT_NONE;
    const uint32_t ldn = pad8(N), ldm = pad8(M);
    const bool dz_direct = !fuse && in_place16(dY, N);       // dZ == dY, usable as the [M rows, N contiguous] operand
    const bool b_direct = in_place16(B, N);
    const uint32_t nchunk_rows = (M + 31) / 32;
    uint64_t need = 4096 + 2 * kPairPartialBytes;
    if (dA) need += (dz_direct ? 0 : (uint64_t)M * ldn * 2) + (b_direct ? 0 : (uint64_t)K * ldn * 2);
    if (dB) need += (uint64_t)N * ldm * 2 + (uint64_t)K * ldm * 2;
    if (dbias) need += (uint64_t)nchunk_rows * N * 4 + (uint64_t)N * 4 + 512;
    { int32_t s0 = fg_ws_ensure(ctx, need); if (s0 != FG_OK) return s0; }
    int32_t s;
    void *dz_n = nullptr, *dz_t = nullptr, *cs_part = nullptr;
    Prep16Args pz{};
    pz.x = dY; pz.saved = fuse ? saved : nullptr; pz.act = act; pz.R = M; pz.C = N;
    if (dA && !dz_direct) {
        if ((s = fg_ws_alloc(ctx, (uint64_t)M * ldn * 2, &dz_n)) != FG_OK) return s;
        pz.n_out = dz_n; pz.ld_n = ldn;
    }
    if (dB) {
        if ((s = fg_ws_alloc(ctx, (uint64_t)N * ldm * 2, &dz_t)) != FG_OK) return s;
        pz.t_out = dz_t; pz.ld_t = ldm;
    }
    if (dbias) {
        if ((s = fg_ws_alloc(ctx, (uint64_t)nchunk_rows * N * 4, &cs_part)) != FG_OK) return s;
        pz.colsum_part = (float*)cs_part;
    }
    uint32_t cs_chunks = 0;
    if (pz.n_out || pz.t_out || pz.colsum_part) {
        if ((s = launch_prep16(ctx, dtype, pz, &cs_chunks)) != FG_OK) return s;
    }
    if (dB) {
        // dB[K,N] = A^T · dZ: contraction over M; operands A^T [K][M] and dZ^T [N][M]
        void* at;
        if ((s = fg_ws_alloc(ctx, (uint64_t)K * ldm * 2, &at)) != FG_OK) return s;
        Prep16Args pa{};
        pa.x = A; pa.R = M; pa.C = K; pa.t_out = at; pa.ld_t = ldm;
        if ((s = launch_prep16(ctx, dtype, pa)) != FG_OK) return s;
        if ((s = lowp_gemm(ctx, dtype, at, ldm, dz_t, ldm, K, N, M, dB, nullptr, FG_ACT_NONE, nullptr)) != FG_OK) return s;
    }
    if (dbias) {
        void* db32;
        if ((s = fg_ws_alloc(ctx, (uint64_t)N * 4, &db32)) != FG_OK) return s;
        if ((s = fg_colsum_fold_launch(ctx, N, cs_chunks, (const float*)cs_part, (float*)db32)) != FG_OK) return s;
        if ((s = fg_convert_launch(ctx, db32, FG_DTYPE_F32, dbias, dtype, N)) != FG_OK) return s;
    }
    if (dA) {
        // dA[M,K] = dZ · B^T: contraction over N; dZ [M][N] and B [K][N] both have it contiguous already
        const void* b_rows = B;
        uint32_t ldb = N;
        if (!b_direct) {
            void* bc;
            if ((s = fg_ws_alloc(ctx, (uint64_t)K * ldn * 2, &bc)) != FG_OK) return s;
            Prep16Args pb{};
            pb.x = B; pb.R = K; pb.C = N; pb.n_out = bc; pb.ld_n = ldn;
            if ((s = launch_prep16(ctx, dtype, pb)) != FG_OK) return s;
            b_rows = bc;
            ldb = ldn;
        }
        const void* z_rows = dz_direct ? dY : dz_n;
        if ((s = lowp_gemm(ctx, dtype, z_rows, dz_direct ? N : ldn, b_rows, ldb, M, K, N, dA, nullptr, FG_ACT_NONE, nullptr)) != FG_OK)
            return s;
    }
    return FG_OK;
}

}  // extern "C"

// ---- self-test of the bounded waits ----
namespace {
__global__ void bounded_wait_selftest_kernel(int* dev_status, long long max_cycles) {
    __shared__ unsigned long long bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
        // nobody arrives on this barrier: the wait must give up after max_cycles and report it
        if (!mbar_wait_bounded(smem_u32(&bar), 0, max_cycles)) atomicOr(dev_status, FG_DEVERR_EPI_WAIT);
    }
}
}  // namespace

extern "C" int32_t fg_selftest_bounded_wait(fg_ctx* ctx, uint32_t max_cycles) {
    FG_ENTER(ctx);
    const long long limit = max_cycles > 1000000u ? 1000000ll : (long long)max_cycles;
    bounded_wait_selftest_kernel<<<1, 32, 0, ctx->stream>>>(ctx->dev_status, limit);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

#ifdef FG_GEMM_PROFILE
extern "C" int32_t fg_gemm_profile_read(unsigned long long out[8]) {
    unsigned long long zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (cudaDeviceSynchronize() != cudaSuccess) return FG_ERR_SYNC;
    if (cudaMemcpyFromSymbol(out, g_prof, sizeof(zero)) != cudaSuccess) return FG_ERR_INTERNAL;
    if (cudaMemcpyToSymbol(g_prof, zero, sizeof(zero)) != cudaSuccess) return FG_ERR_INTERNAL;
    return FG_OK;
}
#endif
