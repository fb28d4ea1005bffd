/*
 * ferrograd_b200 -- C ABI of the B200 (sm_100a) execution backend for ferrograd.
 *
 * This is the boundary a ferrograd `GpuBackend` implementation binds to
 * (reference trait: crates/fused_gpu/src/dispatch/mod.rs:161-261).  Every entry
 * point is `extern "C"`, takes plain pointers and sizes, returns an `int32_t`
 * status (`FG_OK` == 0) and never throws or aborts.  All compute entry points
 * enqueue work on the context's stream and return immediately, like the
 * reference's `dispatch_*` calls (crates/fused_gpu/src/dispatch/mod.rs:766-814);
 * only `fg_sync`, `fg_download`, `fg_upload` (from pageable memory) block.
 *
 * Conventions
 *   - tensors are dense, row-major, f32 unless stated; labels/indices are u32
 *     (reference: crates/fused_gpu/src/tensor.rs:125-128);
 *   - device pointers handed to compute entry points must be 16-byte aligned
 *     (anything returned by `fg_alloc*` is 256-byte aligned);
 *   - host-side validation failures return FG_ERR_INVALID_ARGUMENT without
 *     launching anything; `fg_last_error` gives the message;
 *   - there is no CPU fallback: every compute entry point runs a CUDA kernel.
 */
#ifndef FERROGRAD_B200_H
#define FERROGRAD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes; one per `ErrorKind` variant a backend can produce
 * (crates/fused_gpu/src/errors.rs:105-140), plus FG_ERR_TIMEOUT for a bounded
 * device-side wait that ran out. */
enum fg_status {
    FG_OK = 0,
    FG_ERR_INVALID_ARGUMENT = 1,    /* ErrorKind::InvalidArgument    */
    FG_ERR_OUT_OF_MEMORY = 2,       /* ErrorKind::OutOfMemory        */
    FG_ERR_INVALID_DEVICE = 3,      /* ErrorKind::InvalidDevice      */
    FG_ERR_LAUNCH_FAILURE = 4,      /* ErrorKind::LaunchFailure      */
    FG_ERR_SYNC = 5,                /* ErrorKind::SyncError          */
    FG_ERR_FAILED_BUFFER_COPY = 6,  /* ErrorKind::FailedBufferCopy   */
    FG_ERR_UNSUPPORTED_FEATURE = 7, /* ErrorKind::UnsupportedFeature */
    FG_ERR_NOT_INITIALIZED = 8,     /* ErrorKind::NotInitialized     */
    FG_ERR_INTERNAL = 9,            /* ErrorKind::InternalError      */
    FG_ERR_PEER_ACCESS = 10,        /* ErrorKind::PeerAccessError    */
    FG_ERR_TIMEOUT = 11,            /* (new) bounded wait expired    */
    FG_ERR_INCONSISTENT_CAPTURE = 12 /* ErrorKind::InconsistentCapture */
};

/* Activations fused into the GEMM epilogue / backward prologue.
 * Reference ops: crates/ferrograd-nn/src/op/unary.rs tanh :270-327,
 * relu :436-490, gelu :492-733 (tanh approximation, constants :493-494). */
enum fg_act { FG_ACT_NONE = 0, FG_ACT_RELU = 1, FG_ACT_TANH = 2, FG_ACT_GELU = 3 };

/* How the f32 GEMM is computed. */
enum fg_gemm_mode {
    FG_GEMM_AUTO = 0,   /* FG_GEMM_TF32_BF16X2 when the shape is large enough; plain-FMA streaming
                           kernels when N <= 16 (a narrow output layer); else SIMT */
    FG_GEMM_SIMT = 1,   /* sequential-k fmaf, bit-identical to the reference kernel body
                           (crates/ferrograd-nn/src/op/matmul/generic.rs:98-319) */
    FG_GEMM_3XTF32 = 2, /* tcgen05 kind::tf32, hi/lo split, three MMAs per k-step */
    FG_GEMM_TF32_BF16X2 = 3 /* the dominant hi*hi term as kind::tf32, the two cross terms
                               (lo*hi, hi*lo: 2^-11 of the product) as bf16 MMAs: two
                               tf32-units of tensor work per product instead of three.
                               Shapes whose dimensions are multiples of 8 are multiplied
                               straight from the f32 tensors (see "f32 tensors with bf16
                               pairs" below); others go through operand planes */
};

typedef struct fg_ctx fg_ctx;   /* one device + one stream (rocm/mod.rs:58-78)   */
typedef struct fg_buf fg_buf;   /* GpuBackend::Buffer                            */
typedef struct fg_plan fg_plan; /* GpuBackend::Schedule: a captured CUDA graph   */

/* ---- context (GpuContext::new, sync, is_ready: dispatch/mod.rs:352-367,:505) ---- */
int32_t fg_ctx_create(int32_t device, fg_ctx** out);
/* Use an existing CUDA stream (e.g. one owned by a host framework); 0 = a new one. */
int32_t fg_ctx_create_on_stream(int32_t device, void* cuda_stream, fg_ctx** out);
int32_t fg_ctx_destroy(fg_ctx* ctx);
int32_t fg_sync(fg_ctx* ctx);                    /* GpuBackend::sync     :253 */
int32_t fg_is_ready(fg_ctx* ctx, int32_t* ready);/* GpuBackend::is_ready :260 */
const char* fg_last_error(fg_ctx* ctx);          /* Error::msg (errors.rs:15-19) */
void* fg_ctx_stream(fg_ctx* ctx);                /* the cudaStream_t, for host plumbing */
int32_t fg_ctx_device(fg_ctx* ctx);
/* Number of kernels this context has launched (eager launches and kernels inside
 * replayed plans); lets a benchmark report its own launch count. */
uint64_t fg_ctx_launch_count(fg_ctx* ctx);
/* Pre-size the scratch arena the tensor-core GEMM uses for its hi/lo operand
 * planes, so that no allocation happens later (required before fg_plan_begin). */
int32_t fg_ctx_reserve_workspace(fg_ctx* ctx, uint64_t bytes);
uint64_t fg_ctx_workspace_bytes(fg_ctx* ctx);
/* Tuning and debugging switches of one context (no counterpart in the reference, whose only switch is
 * CompilationOptions: dispatch/mod.rs:369-455).  Values are strings.
 *   "gemm_tile"     "auto" (default) | "pair" | "256x32" | "256x16" | "128x32" | "128x16": the tensor-core tile
 *   "gemm_split_k"  "1" (default) | "0": cut the tiles of an under-filled last wave into K-shares
 *   "gemm_group"    "0" (default: by shape) | 1..64: tile rows per group of the pair kernel's tile order
 *   "gemm_pairs"    "1" (default) | "0": multiply f32 tensors as they lie, with bf16 pairs, where the shape
 *                   allows; "0" sends every shape through operand planes written by a pre-pass
 *   "exec_plans"    "auto" (default) | "1" | "0": the graph engine records each dispatch as a CUDA graph and
 *                   replays it.  "auto" does so for graphs whose kernels are short (launch-bound: the tiny MLP gains
 *                   several times) and, when the context has a communicator, also for graphs of medium-sized
 *                   kernels (the host-side cost of enqueueing collectives every step is avoided); for large
 *                   layers plain launches keep the GPU fed, and four graph launches per step cost more than
 *                   they save (measured: 1.87 against 1.82 ms per step on 784-4096-4096-10 on one GPU)
 *   "comm_max_ctas" CTAs the communicator may use (default 12; read by fg_comm_init)
 *   "comm_sms"      SMs the persistent GEMM leaves free while an exchange is in flight (default 16; 0 = none)
 *   "comm_min_exchange"  the graph engine starts a gradient exchange during the backward pass once this many
 *                   elements are complete (default 1048576); smaller ranges wait for the next one
 * The environment variables FG_GEMM_TILE, FG_GEMM_NO_SPLITK, FG_GEMM_NO_PAIRS, FG_EXEC_NO_PLANS,
 * FG_GEMM_GROUP, NCCL_MAX_CTAS, FG_COMM_SMS and FG_COMM_MIN_EXCHANGE give the initial values; they are read once, when the
 * context is created. */
int32_t fg_ctx_set_option(fg_ctx* ctx, const char* name, const char* value);
/* Self-test of the bounded device-side waits (no counterpart in the reference).  Launches one tiny kernel that
 * waits, for at most max_cycles SM clock cycles (clamped to 1,000,000), on an mbarrier nobody ever arrives on,
 * with the same wait routine the GEMM kernels use.  The wait runs out, the kernel records it in the device error
 * word and returns: fg_sync then reports FG_ERR_TIMEOUT once and the context stays usable.  Nothing faults or hangs. */
int32_t fg_selftest_bounded_wait(fg_ctx* ctx, uint32_t max_cycles);
/* Reads and clears the device-side error word (bounded waits that expired). */
int32_t fg_ctx_device_status(fg_ctx* ctx, int32_t* status_word);

/* Per-kernel timing for benchmarks (no counterpart in the reference; its examples time
 * whole epochs on the host, examples/matmul_chain3.rs:11-44).  While enabled, each launch
 * of the kernels below is bracketed by CUDA events on the context's stream.  Not
 * available while a plan is being recorded.  fg_ctx_timing_read synchronises, sums the
 * launches of one kind since the last read of that kind and forgets them. */
enum fg_kernel_kind {
    FG_KERNEL_GEMM_TC = 0,    /* work = 2*M*N*K flop                       */
    FG_KERNEL_SOFTMAX_CE = 1, /* fused CE: work = 2*rows*cols*4 bytes (+probs); softmax forward alone the same;
                                 softmax backward 3*rows*cols*4 (4* when it accumulates) */
    FG_KERNEL_ADAMW = 2,      /* work = 28 (or 32 with zero_grad) bytes/param */
    FG_KERNEL_SGD = 3,        /* work = 12 (or 16 with zero_grad) bytes/param */
    FG_KERNEL_SPLIT = 4,      /* work = bytes read + written by the operand pre-pass */
    FG_KERNEL_ELTWISE = 5,    /* bias+activation, activation backward, MSE/BCE, chains, conversions:
                                 work = bytes of the tensors read + written, each once */
    FG_KERNEL_SKINNY = 6      /* GEMMs with N <= 16: work = bytes of the large operand (and of the outputs
                                 that are as large) moved once */
};
int32_t fg_ctx_timing_enable(fg_ctx* ctx, int32_t on);
int32_t fg_ctx_timing_read(fg_ctx* ctx, int32_t kind, uint64_t* launches, double* total_ms,
                           double* total_work);

/* ---- memory (GpuBackend::alloc/alloc_zeroed/alloc_init/upload/copy/download :171-207) ---- */
int32_t fg_alloc(fg_ctx* ctx, uint64_t bytes, fg_buf** out);
int32_t fg_alloc_zeroed(fg_ctx* ctx, uint64_t bytes, fg_buf** out);
int32_t fg_alloc_init(fg_ctx* ctx, const void* data, uint64_t bytes, fg_buf** out);
int32_t fg_free(fg_ctx* ctx, fg_buf* buf);
uint64_t fg_buf_size_bytes(const fg_buf* buf);   /* GpuBufferBackend::size_bytes :150 */
void* fg_buf_device_ptr(const fg_buf* buf);
int32_t fg_upload(fg_ctx* ctx, fg_buf* dst, const void* src, uint64_t bytes, uint64_t dst_off);
int32_t fg_download(fg_ctx* ctx, const fg_buf* src, void* dst, uint64_t bytes, uint64_t src_off);
int32_t fg_copy(fg_ctx* ctx, const fg_buf* src, fg_buf* dst);
/* Tells the library that the buffer's contents were changed through its raw device pointer (by a kernel of
 * the host framework, fg_upload_async, ...).  The graph engine keeps derived data (the bf16 pairs of bound
 * weight tensors) and refreshes it only when a tensor has changed: writes through fg_upload / fg_copy and
 * the engine's own optimizer are seen, writes through the raw pointer need this call. */
int32_t fg_buf_touch(fg_buf* buf);
/* Asynchronous copies from/to PINNED host memory on the context stream. */
int32_t fg_upload_async(fg_ctx* ctx, void* dst_dev, const void* src_pinned, uint64_t bytes);
int32_t fg_download_async(fg_ctx* ctx, void* dst_pinned, const void* src_dev, uint64_t bytes);
/* Input prefetch (no counterpart in the reference, whose uploads are synchronous:
 * rocm/mod.rs:184-205).  fg_upload_prefetch copies from pinned host memory on a side stream, so it
 * overlaps whatever the context's stream is computing; fg_prefetch_wait makes the context's stream
 * wait for the prefetches issued so far; fg_prefetch_mark records that the stream is done reading the
 * prefetch destination, and the next fg_upload_prefetch will not start before that point. */
int32_t fg_upload_prefetch(fg_ctx* ctx, void* dst_dev, const void* src_pinned, uint64_t bytes);
int32_t fg_prefetch_wait(fg_ctx* ctx);
int32_t fg_prefetch_mark(fg_ctx* ctx);
int32_t fg_copy_dev_async(fg_ctx* ctx, void* dst_dev, const void* src_dev, uint64_t bytes);
int32_t fg_host_alloc_pinned(uint64_t bytes, void** out);
int32_t fg_host_free_pinned(void* p);
int32_t fg_memset_zero(fg_ctx* ctx, void* dev, uint64_t bytes);

/* ---- GEMM with fused epilogue (matmul: op/matmul/mod.rs:17-188,:190-296;
 *      epilogue fusion rule: kernel/forward.rs:373-457) ----
 * C[M,N] = act( op(A)·op(B) + bias ), op(X) = X or Xᵀ.  A is [M,K] (or [K,M] when
 * transA), B is [K,N] (or [N,K] when transB).  bias is [N] broadcast over rows or
 * NULL.  preact_out (NULL or [M,N]) receives op(A)·op(B)+bias before the activation
 * (needed by the GELU backward). */
int32_t fg_gemm_f32(fg_ctx* ctx, int32_t mode, int32_t transA, int32_t transB,
                    uint32_t M, uint32_t N, uint32_t K,
                    const float* A, const float* B, float* C,
                    const float* bias, int32_t act, float* preact_out);

/* Backward of Y = act(A·B + bias) for A[M,K], B[K,N]  (matmul backward edges:
 * op/matmul/mod.rs:75-101; activation backward: op/unary.rs:281-309,:453-472,:588-714).
 *   dZ = dY ⊙ act'(saved)        saved = Y for NONE/RELU/TANH, pre-activation Z for GELU
 *   dA = dZ·Bᵀ  [M,K]   (skipped when dA == NULL)
 *   dB = Aᵀ·dZ  [K,N]   (skipped when dB == NULL)
 *   dbias = column sums of dZ [N] (skipped when NULL)
 *   dZ_out (NULL or [M,N]) receives dZ.
 * The ReLU mask is saved > 0 (the standard mask). */
int32_t fg_gemm_bwd_f32(fg_ctx* ctx, int32_t mode, uint32_t M, uint32_t N, uint32_t K,
                        const float* A, const float* B, const float* dY,
                        int32_t act, const float* saved,
                        float* dA, float* dB, float* dbias, float* dZ_out);

/* fg_gemm_bwd_f32 for data-parallel training (no counterpart in the reference, which is single
 * device): dB and dbias are completed first, then the sum over all ranks of exch_buf[0..exch_count)
 * — normally the range of the gradient arena that holds this layer's dB and dbias, plus any later
 * layers not yet exchanged — is started on the exchange stream as by fg_allreduce_sum_f32, and dA is
 * computed while it runs.  dZ is formed once for both products.  Needs fg_comm_init; finish with
 * fg_comm_join before the gradients are used. */
int32_t fg_gemm_bwd_exchange_f32(fg_ctx* ctx, int32_t mode, uint32_t M, uint32_t N, uint32_t K,
                                 const float* A, const float* B, const float* dY,
                                 int32_t act, const float* saved,
                                 float* dA, float* dB, float* dbias,
                                 float* exch_buf, uint64_t exch_count);

/* ---- f32 tensors with bf16 pairs: the default GEMM mode without any operand pre-pass ----
 * (No counterpart in the reference; it serves the same rule as its prologue fusion, kernel/forward.rs:373-457:
 * nothing elementwise runs as a pass of its own between two matmuls.)
 * In the default mode a product a*b is computed as trunc(a)*trunc(b) on kind::tf32 -- the tensor core reads
 * the f32 words themselves and ignores their low 13 mantissa bits -- plus two bf16 cross terms.  The cross
 * terms come from the tensor's PAIRS: two bf16 planes with the tensor's own shape and layout,
 *   pairs[i] = bf16(x[i]),   pairs[plane_stride + i] = bf16(x[i] - trunc(x[i])),
 * `plane_stride` (elements, a multiple of 8, at least the tensor's size) apart; pairs are 16-byte aligned.
 * fg_gemm_f32 / fg_gemm_bwd_f32 make the pairs of their operands on every call (8 bytes of traffic per
 * element).  A caller that keeps each tensor's pairs beside it pays nothing: every entry point that writes
 * a tensor can write its pairs in the same pass (the GEMM epilogues below, fg_adamw_step_paired,
 * fg_sgd_step_paired), and fg_pairs_from_f32 makes them for tensors that arrive from outside.  Operands are
 * never transposed: the product that contracts over a tensor's rows reads it through MN-major descriptors.
 * Shapes the pair kernel cannot take (a dimension that is not a multiple of 8, tiny matrices, N <= 16)
 * are computed as fg_gemm_f32 would, with the same results and outputs. */
int32_t fg_pairs_from_f32(fg_ctx* ctx, const float* x, uint64_t n, void* pairs, uint64_t plane_stride);
/* C[M,N] = act(A[M,K]·B[K,N] + bias), as fg_gemm_f32 in FG_GEMM_AUTO mode.  A_pairs / B_pairs may be NULL
 * (made on the fly).  C_pairs_out (may be NULL) receives the pairs of C. */
int32_t fg_gemm_paired_f32(fg_ctx* ctx, uint32_t M, uint32_t N, uint32_t K,
                           const float* A, const void* A_pairs, uint64_t A_stride,
                           const float* B, const void* B_pairs, uint64_t B_stride,
                           float* C, const float* bias, int32_t act, float* preact_out,
                           void* C_pairs_out, uint64_t C_stride);
/* Backward of Y = A[M,K]·B[K,N] given dZ = dL/dY with this layer's own activation factor already applied
 * (matmul backward edges: op/matmul/mod.rs:75-101):
 *   dB [K,N] = Aᵀ·dZ                                   (skipped when dB == NULL)
 *   dbias [N] = column sums of dZ                      (skipped when NULL; meant for the top layer, whose dZ
 *                                                       comes from the loss and not from a dA epilogue)
 *   then, when exch_buf != NULL, the sum of exch_buf[0..exch_count) over the ranks is started as by
 *   fg_allreduce_sum_f32 (see fg_gemm_bwd_exchange_f32), and beside it
 *   dA [M,K] = (dZ·Bᵀ) ⊙ act'(below_saved)             (skipped when dA == NULL)
 * where below_act / below_saved describe the layer BELOW (the one whose output A is; FG_ACT_NONE: no
 * factor), so dA is that layer's dZ, ready to be passed to its own backward call.  dA_pairs_out (may be
 * NULL) receives dA's pairs and below_dbias (may be NULL, [K]) its column sums, the bias gradient of the
 * layer below -- all from the dA epilogue.  Any of the input pairs may be NULL. */
int32_t fg_gemm_bwd_paired_f32(fg_ctx* ctx, uint32_t M, uint32_t N, uint32_t K,
                               const float* A, const void* A_pairs, uint64_t A_stride,
                               const float* B, const void* B_pairs, uint64_t B_stride,
                               const float* dZ, const void* dZ_pairs, uint64_t dZ_stride,
                               float* dB, float* dbias, float* dA, int32_t below_act, const float* below_saved,
                               void* dA_pairs_out, uint64_t dA_stride, float* below_dbias,
                               float* exch_buf, uint64_t exch_count);

/* Rank-3 matmul: `batch` independent products; product t uses A + t*strideA, B + t*strideB and
 * C (or dY, saved, preact_out) + t*strideC, strides in elements.  The reference steps every operand
 * by one matrix per Z index (kernel/forward.rs:159-190, op/matmul/generic.rs:131,194).  Each stride
 * must be at least its matrix; one B shared by all products is fg_gemm_f32 with batch*M rows. */
int32_t fg_gemm_batched_f32(fg_ctx* ctx, int32_t mode, uint32_t batch, uint32_t M, uint32_t N, uint32_t K,
                            const float* A, uint64_t strideA, const float* B, uint64_t strideB,
                            float* C, uint64_t strideC, const float* bias, int32_t act,
                            float* preact_out);
int32_t fg_gemm_batched_bwd_f32(fg_ctx* ctx, int32_t mode, uint32_t batch, uint32_t M, uint32_t N,
                                uint32_t K, const float* A, uint64_t strideA, const float* B,
                                uint64_t strideB, const float* dY, uint64_t strideC, int32_t act,
                                const float* saved, float* dA, float* dB);

/* ---- activations standalone (op/unary.rs) ---- */
int32_t fg_bias_act_fwd(fg_ctx* ctx, uint32_t rows, uint32_t cols, const float* z,
                        const float* bias, int32_t act, float* y);
int32_t fg_act_bwd(fg_ctx* ctx, uint64_t n, int32_t act, const float* dy,
                   const float* saved, float* dz);

/* ---- softmax (op/softmax.rs:112-446 forward, :448-688 backward) ---- */
int32_t fg_softmax_fwd(fg_ctx* ctx, uint32_t rows, uint32_t cols, const float* x, float* y);
/* dx = y ⊙ (dy − Σ_row dy·y); accumulate != 0 adds into dx like the reference's `+=`. */
int32_t fg_softmax_bwd(fg_ctx* ctx, uint32_t rows, uint32_t cols, const float* y,
                       const float* dy, float* dx, int32_t accumulate);

/* ---- fused softmax + cross-entropy forward and backward
 *      (CROSS_ENTROPY: loss/basic_loss.rs:91-133; loss kernel: kernel/loss.rs:12-165) ----
 * loss_row[r] = −log softmax(logits[r])[labels[r]];  loss_mean = Σ loss_row / rows;
 * dlogits = (softmax − onehot) · grad_scale.  loss_row_out, loss_mean_out, probs_out
 * may be NULL.  argmax_out (NULL or u32[rows]) receives the index of the first
 * maximum of each row. */
int32_t fg_softmax_ce_fwd_bwd(fg_ctx* ctx, const float* logits, const uint32_t* labels,
                              uint32_t rows, uint32_t cols, float grad_scale,
                              float* loss_row_out, float* loss_mean_out,
                              float* dlogits_out, float* probs_out, uint32_t* argmax_out);
/* The reference's unfused per-element CE on probabilities (loss/basic_loss.rs:91-133):
 * loss[r,c] = −log p at c == label[r] else 0; grad[r,c] = p − 1 at the label else p. */
int32_t fg_ce_loss_grad(fg_ctx* ctx, const float* probs, const uint32_t* labels,
                        uint32_t rows, uint32_t cols, float* loss_out, float* grad_out);

/* out[0] = sum of x[0..n), reduced in a fixed order (no counterpart in the reference, whose losses stay
 * unreduced: loss/basic_loss.rs:3-133; used to hand a caller one number per step instead of the loss tensor). */
int32_t fg_sum_f32(fg_ctx* ctx, const float* x, uint64_t n, float* out);

/* ---- MSE (MEAN_SQUARED_ERROR: loss/basic_loss.rs:3-27) ----
 * loss[i] = (p−t)², grad[i] = 2(p−t)·grad_scale.  loss_elem_out and loss_sum_out
 * (one float: Σ loss[i], reduced in a fixed order) may be NULL. */
int32_t fg_mse_loss_grad(fg_ctx* ctx, const float* pred, const float* target, uint64_t n,
                         float grad_scale, float* loss_elem_out, float* loss_sum_out,
                         float* grad_out);

/* ---- BCE (BINARY_CROSS_ENTROPY: loss/basic_loss.rs:29-89), on probabilities p in (0,1) ----
 * loss[i] = −(t·log p + (1−t)·log(1−p)); grad[i] = (p − t)·grad_scale, which is the reference's
 * gradient expression (:81-85: the derivative with respect to the logit of a sigmoid output).
 * The reference's loss expression differs from the definition above in two places (:47-51 takes
 * 1 − target where 1 − pred is meant, and :75-79 subtracts the terms in the opposite order); the
 * standard definition is computed here.  Outputs as for fg_mse_loss_grad. */
int32_t fg_bce_loss_grad(fg_ctx* ctx, const float* pred, const float* target, uint64_t n,
                         float grad_scale, float* loss_elem_out, float* loss_sum_out,
                         float* grad_out);

/* The same loss and gradient for hosts that must never cause a device allocation (a
 * process whose own pool already owns all GPU memory, a latency-bound service, a job run
 * against a fixed memory budget).  It has no counterpart in the reference.  The partial
 * sums of the reduction live in a 16 KiB array built into the library instead of the
 * context's scratch arena, so no cudaMalloc/cudaFree happens on any call.
 *   - n must not exceed FG_MSE_NOALLOC_MAX_N; larger n returns FG_ERR_INVALID_ARGUMENT.
 *   - The first call made on a device looks up the array's address; make it outside any
 *     stream capture (inside a recording started with fg_plan_begin it is refused with
 *     FG_ERR_INCONSISTENT_CAPTURE).
 *   - Calls on the same GPU share the array: do not let two of them run concurrently.
 * loss_sum agrees with fg_mse_loss_grad to rounding (a different, SM-count-independent
 * summation order); loss_elem and grad are identical. */
#define FG_MSE_NOALLOC_MAX_N 268435456ull
int32_t fg_mse_loss_grad_noalloc(fg_ctx* ctx, const float* pred, const float* target, uint64_t n,
                                 float grad_scale, float* loss_elem_out, float* loss_sum_out,
                                 float* grad_out);

/* ---- optimizers ----
 * SGD (STOCHASTIC_GRADIENT_DESCENT: optim/basic_optim.rs:3-31; lr plumbing
 * kernel/optim.rs:119-146): w −= lr·(g·grad_scale); g = 0 when zero_grad != 0
 * (the reference always zeroes). */
int32_t fg_sgd_step(fg_ctx* ctx, float* w, float* g, uint64_t n, float lr,
                    float grad_scale, int32_t zero_grad);

typedef struct fg_adamw_hyper {
    float lr, beta1, beta2, eps, weight_decay;
} fg_adamw_hyper;
/* AdamW (absent from the reference; decoupled weight decay, bias-corrected):
 *   g' = g·grad_scale; m = β1 m + (1−β1) g'; v = β2 v + (1−β2) g'²;
 *   w = w − lr·( (m/(1−β1^t)) / (sqrt(v/(1−β2^t)) + eps) + wd·w ).
 * t = *step_dev when step_dev != NULL (a device counter, so a captured plan can be
 * replayed with a moving step), else `step` (1-based). */
int32_t fg_adamw_step(fg_ctx* ctx, float* w, float* g, float* m, float* v, uint64_t n,
                      const fg_adamw_hyper* hyper, uint32_t step, const uint32_t* step_dev,
                      float grad_scale, int32_t zero_grad);
/* The same updates, also writing the bf16 pairs of the updated weights (see fg_gemm_paired_f32) in the same
 * pass: +4 bytes per parameter.  w_pairs == NULL: exactly fg_sgd_step / fg_adamw_step. */
int32_t fg_sgd_step_paired(fg_ctx* ctx, float* w, float* g, uint64_t n, float lr, float grad_scale,
                           int32_t zero_grad, void* w_pairs, uint64_t pairs_stride);
int32_t fg_adamw_step_paired(fg_ctx* ctx, float* w, float* g, float* m, float* v, uint64_t n,
                             const fg_adamw_hyper* hyper, uint32_t step, const uint32_t* step_dev,
                             float grad_scale, int32_t zero_grad, void* w_pairs, uint64_t pairs_stride);
/* The same updates for several tensors in ONE launch (a model whose weights and biases are separate tensors, as
 * in the reference, otherwise pays one launch per tensor: kernel/optim.rs:12-158 lowers one kernel per weight).
 * m and v are ignored by the SGD form; w_pairs may be NULL. */
typedef struct fg_update_tensor {
    float *w, *g, *m, *v;
    void* w_pairs;
    uint64_t pairs_stride;
    uint64_t n;
} fg_update_tensor;
int32_t fg_adamw_step_multi(fg_ctx* ctx, const fg_update_tensor* tensors, uint32_t count,
                            const fg_adamw_hyper* hyper, uint32_t step, const uint32_t* step_dev,
                            float grad_scale, int32_t zero_grad);
int32_t fg_sgd_step_multi(fg_ctx* ctx, const fg_update_tensor* tensors, uint32_t count, float lr,
                          float grad_scale, int32_t zero_grad);
int32_t fg_counter_increment(fg_ctx* ctx, uint32_t* counter_dev);

/* ---- fused elementwise chains (op/binary.rs add :74, mul :236, sub :449, div :644;
 *      op/unary.rs; inlining rule kernel/forward.rs:298-464) ----
 * A chain is a straight-line program over per-element values.  Instruction i
 * defines value i.  FG_EW_INPUT loads inputs[a][idx]; FG_EW_CONST is `imm`;
 * binary ops read values a and b; unary ops read value a.  The last value is the
 * output.  At most FG_EW_MAX_INSTR instructions and FG_EW_MAX_INPUTS inputs. */
enum fg_ew_op {
    FG_EW_INPUT = 0, FG_EW_CONST = 1, FG_EW_ADD = 2, FG_EW_SUB = 3, FG_EW_MUL = 4,
    FG_EW_DIV = 5, FG_EW_NEG = 6, FG_EW_ABS = 7, FG_EW_EXP = 8, FG_EW_LOG = 9,
    FG_EW_TANH = 10, FG_EW_RELU = 11, FG_EW_GELU = 12, FG_EW_ELU = 13
};
#define FG_EW_MAX_INSTR 24
#define FG_EW_MAX_INPUTS 8
typedef struct fg_ew_instr {
    int32_t op, a, b;
    float imm;
} fg_ew_instr;
/* out[i] = chain(inputs[0][i], ...).  saved_out (NULL or array of ninstr pointers,
 * each NULL or a buffer of n floats) receives intermediate values, the analogue of
 * the reference's forward_saved tensors. */
int32_t fg_eltwise_chain_fwd(fg_ctx* ctx, uint64_t n, const fg_ew_instr* prog, int32_t ninstr,
                             const float* const* inputs, int32_t ninputs, float* out,
                             float* const* saved_out);
/* One kernel recomputes the chain and back-propagates `seed` (dL/dout, [n]) to every
 * input: grads[k][i] (+)= dL/dinputs[k][i]; grads[k] may be NULL. */
int32_t fg_eltwise_chain_bwd(fg_ctx* ctx, uint64_t n, const fg_ew_instr* prog, int32_t ninstr,
                             const float* const* inputs, int32_t ninputs, const float* seed,
                             float* const* grads, int32_t accumulate);

/* ---- 16-bit storage (SimpleDType::{F16,BF16}: crates/fused_gpu/src/dispatch/backend/mod.rs:337-345;
 *      exercised by crates/ferrograd/tests/nonf32.rs:10-99) ----
 * The _dt forms take tensors of one storage type.  With 16-bit storage every operation's result
 * is rounded to that type (round to nearest even), as native half arithmetic does. */
enum fg_dtype { FG_DTYPE_F32 = 0, FG_DTYPE_F16 = 1, FG_DTYPE_BF16 = 2 };
int32_t fg_eltwise_chain_fwd_dt(fg_ctx* ctx, int32_t dtype, uint64_t n, const fg_ew_instr* prog,
                                int32_t ninstr, const void* const* inputs, int32_t ninputs,
                                void* out, void* const* saved_out);
int32_t fg_eltwise_chain_bwd_dt(fg_ctx* ctx, int32_t dtype, uint64_t n, const fg_ew_instr* prog,
                                int32_t ninstr, const void* const* inputs, int32_t ninputs,
                                const void* seed, void* const* grads, int32_t accumulate);
/* GEMM on f16 or bf16 tensors (all of A [M,K], B [K,N], C [M,N], bias [N], preact_out, and in the
 * backward form dY, saved, dA, dB, dbias [N] have the storage type `dtype`): the tensor cores
 * multiply the 16-bit operands directly (kind::f16) and accumulate in f32; bias and activation are
 * applied in f32 and the result is rounded once to the storage type.  Semantics otherwise as
 * fg_gemm_f32 / fg_gemm_bwd_f32; dZ = dY * act'(saved) is rounded to the storage type before the two
 * products.  C, preact_out, dA and dB must be 16-byte aligned. */
int32_t fg_gemm_lowp(fg_ctx* ctx, int32_t dtype, uint32_t M, uint32_t N, uint32_t K,
                     const void* A, const void* B, void* C, const void* bias, int32_t act,
                     void* preact_out);
int32_t fg_gemm_bwd_lowp(fg_ctx* ctx, int32_t dtype, uint32_t M, uint32_t N, uint32_t K,
                         const void* A, const void* B, const void* dY, int32_t act,
                         const void* saved, void* dA, void* dB, void* dbias);
/* dst[i] = src[i] converted between storage types (round to nearest even when narrowing). */
int32_t fg_convert(fg_ctx* ctx, const void* src, int32_t src_dtype, void* dst, int32_t dst_dtype,
                   uint64_t n);

/* ---- graphs: the reference's Graph -> alloc_tensors -> schedule -> dispatch_* flow ----
 * A graph is a list of nodes in definition order (Graph::push_node,
 * crates/fused_gpu/src/dispatch/backend/mod.rs:1224; ops: crates/ferrograd/src/graph.rs:111-158).
 * Elementwise ops use the fg_ew_op codes; matmul and softmax have the two codes below.  An input's
 * shape is a list of metadata FIELD ids (Metadata::new_field, backend/mod.rs:585-596); field 0 is
 * reserved for the learning rate's f32 bits, the bound metadata array gives every field its value. */
enum fg_graph_op { FG_GRAPH_MATMUL = 14, FG_GRAPH_SOFTMAX = 15 };
enum fg_loss { FG_LOSS_MSE = 0, FG_LOSS_CROSS_ENTROPY = 1,     /* loss/basic_loss.rs:3-27, :91-133 */
               FG_LOSS_BINARY_CROSS_ENTROPY = 2 };             /* loss/basic_loss.rs:29-89         */
enum fg_optim { FG_OPTIM_SGD = 0, FG_OPTIM_ADAMW = 1 };        /* optim/basic_optim.rs:3-31; AdamW is new */
typedef struct fg_graph fg_graph;   /* ferrograd::Graph (crates/ferrograd/src/graph.rs:15-98)        */
typedef struct fg_exec fg_exec;     /* AllocTensors + compiled kernels + Schedule of one graph        */

int32_t fg_graph_create(int32_t loss, int32_t optim, fg_graph** out);            /* Graph::new        */
int32_t fg_graph_destroy(fg_graph* g);
int32_t fg_graph_node_count(const fg_graph* g);
int32_t fg_graph_input(fg_graph* g, const uint32_t* shape_fields, uint32_t ndim, int32_t* node); /* DefineOps::input */
/* An input stored as f16 or bf16 (fg_dtype).  All inputs of a graph share one storage type, and every
 * tensor the engine allocates for the graph (results, gradients, seed, loss) has that type.  In a
 * 16-bit graph elementwise regions and SGD compute in the storage type, matmul multiplies the 16-bit
 * operands with f32 accumulation, softmax and the losses are computed in f32 on widened copies and
 * rounded back; a dense loss target has the storage type too (class labels stay u32).  AdamW needs
 * f32 storage. */
int32_t fg_graph_input_dt(fg_graph* g, const uint32_t* shape_fields, uint32_t ndim, int32_t dtype, int32_t* node);
int32_t fg_graph_constant_f32(fg_graph* g, float value, int32_t* node);          /* constant_f32      */
/* op: FG_EW_ADD..FG_EW_ELU, FG_GRAPH_MATMUL, FG_GRAPH_SOFTMAX; b is ignored for unary ops.          */
int32_t fg_graph_op(fg_graph* g, int32_t op, int32_t a, int32_t b, int32_t* node);
/* compute_saved_nodes + validate + alloc_tensors + lower + compile, for one metadata binding
 * (backend/mod.rs:1172-1208; dispatch/mod.rs:369-455, :509-575).  The graph is copied. */
int32_t fg_exec_create(fg_ctx* ctx, const fg_graph* g, const uint32_t* meta, uint32_t nmeta,
                       int32_t gemm_mode, fg_exec** out);
int32_t fg_exec_destroy(fg_exec* e);
int32_t fg_exec_set_adamw(fg_exec* e, const fg_adamw_hyper* hyper);   /* lr is taken from meta[0] */
/* schedule (dispatch/mod.rs:664-764): one tensor per graph input, in input order.  trainable
 * (NULL = all, as in the reference) selects which of them dispatch_optim updates. */
int32_t fg_exec_bind(fg_exec* e, fg_buf* const* in_tensors, uint32_t count, const uint8_t* trainable);
int32_t fg_exec_dispatch_forward(fg_exec* e);                         /* dispatch/mod.rs:766 */
int32_t fg_exec_dispatch_backward(fg_exec* e);                        /* :770                */
int32_t fg_exec_dispatch_loss(fg_exec* e, const fg_buf* target);      /* :774-788            */
int32_t fg_exec_dispatch_optim(fg_exec* e);                           /* :790                */
int32_t fg_exec_dispatch_single_optim(fg_exec* e, fg_buf* weight, uint32_t grad_index); /* :794-814 */
/* AllocTensors (dispatch/mod.rs:835-845).  Saved tensors are the materialised intermediate nodes
 * in node order (a matmul result is always one); gradients exist for every input and every
 * materialised intermediate node, in node order.  `node` (may be NULL) receives the node id.
 * A node that was absorbed into its producer (the add and the activation that follow a matmul run in the GEMM's
 * epilogue; the members of an elementwise region run in one kernel) is not materialised and has no entry, so
 * index i here is NOT index i of the reference's compute_saved_nodes (backend/mod.rs:1189): match the entries
 * by the node id that `node` returns. */
fg_buf* fg_exec_forward_out(fg_exec* e);
fg_buf* fg_exec_seed(fg_exec* e);
fg_buf* fg_exec_loss_t(fg_exec* e);
/* One f32: the sum over loss_t, written by dispatch_loss (f32 graphs; no counterpart in the reference, which
 * leaves the reduction of its unreduced loss tensor to the caller). */
fg_buf* fg_exec_loss_sum(fg_exec* e);
uint32_t fg_exec_num_saved(fg_exec* e);
fg_buf* fg_exec_saved(fg_exec* e, uint32_t i, int32_t* node);
uint32_t fg_exec_num_grads(fg_exec* e);
fg_buf* fg_exec_grad(fg_exec* e, uint32_t i, int32_t* node);
uint32_t fg_exec_forward_steps(fg_exec* e);   /* kernels-level steps of one forward dispatch */
int32_t fg_exec_plans_active(fg_exec* e);     /* 1 when the dispatches of this graph are recorded and replayed */

/* ---- .bpat tensor files (crates/fused_gpu/src/io/headers.rs:16-117; save_tensors / load_tensors:
 *      crates/fused_gpu/src/io/mod.rs:98-159) ----
 * Reading accepts v0, v1, v1m, v2-f32, v2-f16 and v2-bf16 and verifies the CRC-32s of v1/v1m; writing
 * produces v2-f32, v2-f16, v2-bf16 or v1m.  f64 files are narrowed to f32 on load; a 16-bit file loads into
 * 16-bit tensors and is written from 16-bit tensors (fg_bpat_dtype tells which type a file's tensors have). */
enum fg_bpat_format { FG_BPAT_V0 = 0, FG_BPAT_V1 = 1, FG_BPAT_V1_MICRO = 2, FG_BPAT_V2_F32 = 3,
                      FG_BPAT_V2_F16 = 4, FG_BPAT_V2_BF16 = 5 };   /* io/headers.rs:79, :98 */
typedef struct fg_bpat_file fg_bpat_file;
int32_t fg_bpat_save(fg_ctx* ctx, const char* path, int32_t format, uint32_t count, fg_buf* const* tensors,
                     const uint32_t* ndims, const uint32_t* const* shapes);
int32_t fg_bpat_open(const char* path, fg_bpat_file** out);   /* no device needed */
int32_t fg_bpat_close(fg_bpat_file* f);
int32_t fg_bpat_format(const fg_bpat_file* f);
int32_t fg_bpat_dtype(const fg_bpat_file* f);    /* fg_dtype of the tensors fg_bpat_load_tensor returns */
uint32_t fg_bpat_count(const fg_bpat_file* f);
int32_t fg_bpat_shape(const fg_bpat_file* f, uint32_t index, uint32_t* ndim, uint32_t dims_out[8]);
int32_t fg_bpat_load_tensor(fg_ctx* ctx, const fg_bpat_file* f, uint32_t index, fg_buf** out);

/* ---- plans: a captured CUDA graph, the analogue of GpuBackend::schedule /
 *      dispatch_schedule (dispatch/mod.rs:218-250; rocm/mod.rs:324-389 captures a
 *      hipGraph the same way) ----
 * Between fg_plan_begin and fg_plan_end every compute entry point on this context is
 * recorded instead of executed.  No allocation may happen in between: reserve the
 * workspace first (or run the same calls once eagerly).  A plan carries addresses inside the
 * scratch arena as it was when the plan was recorded: if a later eager call needs a larger
 * arena, the arena is reallocated and every older plan becomes stale -- fg_plan_launch then
 * returns FG_ERR_INCONSISTENT_CAPTURE instead of running it, and the plan must be recorded
 * again.  fg_ctx_reserve_workspace with the largest need, before recording, avoids this. */
int32_t fg_plan_begin(fg_ctx* ctx);
int32_t fg_plan_end(fg_ctx* ctx, fg_plan** out);
int32_t fg_plan_launch(fg_ctx* ctx, fg_plan* plan);
int32_t fg_plan_destroy(fg_plan* plan);

/* ---- data-parallel gradient exchange (no counterpart in the reference, which is
 *      single-device: rocm/mod.rs:58-78).  NCCL is loaded at run time. ---- */
#define FG_COMM_ID_BYTES 128
int32_t fg_comm_unique_id(uint8_t id_out[FG_COMM_ID_BYTES]);
int32_t fg_comm_init(fg_ctx* ctx, int32_t nranks, int32_t rank, const uint8_t id[FG_COMM_ID_BYTES]);
/* In-place sum over ranks.  Runs on the context's communication stream: it starts
 * after everything enqueued so far on the compute stream and overlaps with what is
 * enqueued afterwards, until fg_comm_join. */
int32_t fg_allreduce_sum_f32(fg_ctx* ctx, float* buf, uint64_t count);
int32_t fg_comm_join(fg_ctx* ctx);
/* fg_comm_checkpoint(slot) marks the exchanges started so far (slot in [0, 8));
 * fg_comm_wait(slot) makes the compute stream wait for exactly those.  Work that needs only the early
 * exchanges (the update of the last layers) can then run while a later one is still in flight. */
int32_t fg_comm_checkpoint(fg_ctx* ctx, int32_t slot);
int32_t fg_comm_wait(fg_ctx* ctx, int32_t slot);
/* Failure handling (no counterpart in the single-device reference).  fg_comm_sync blocks the host
 * until every exchange started so far is complete, for at most timeout_ms; when the time runs out
 * (a peer died or never joined) the communicator is aborted, FG_ERR_TIMEOUT is returned and the
 * context remains usable for everything except exchanges.  fg_comm_abort ends the communicator
 * without waiting for its peers. */
int32_t fg_comm_sync(fg_ctx* ctx, uint32_t timeout_ms);
int32_t fg_comm_abort(fg_ctx* ctx);
/* Destroy the plans that recorded an exchange (fg_plan_destroy, fg_exec_destroy) before the communicator or the
 * context: a live plan keeps the communicator in use, and tearing it down would wait for the plan for ever.  If
 * such plans are still alive the communicator is not torn down at all (it lasts until the process ends). */
int32_t fg_comm_destroy(fg_ctx* ctx);

/* Library / build information. */
const char* fg_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FERROGRAD_B200_H */
