// Context, memory, plans (CUDA graphs) and the NCCL gradient exchange.
//
// Mirrors the reference backend's responsibilities below the GpuBackend trait
// (crates/fused_gpu/src/dispatch/mod.rs:161-261; ROCm implementation
// crates/fused_gpu/src/dispatch/backend/rocm/mod.rs:58-421): one device, one stream,
// synchronous upload/download, asynchronous dispatch, schedules as captured graphs.
#include <dlfcn.h>
#include <stdlib.h>
#include <time.h>
#include <limits.h>

#include <new>

#include "fg_internal.cuh"

namespace {

// Minimal NCCL surface, resolved with dlsym so the library loads without NCCL.
typedef struct { char internal[FG_COMM_ID_BYTES]; } nccl_uid;
typedef int (*pfn_ncclGetUniqueId)(nccl_uid*);
typedef int (*pfn_ncclCommInitRank)(void**, int, nccl_uid, int);
// ncclCommInitRankConfig with the communicator options as they were laid out in NCCL 2.18; newer
// libraries accept an older, shorter structure (they go by its size and version fields) and default the rest.
struct nccl_config_2_18 {
    size_t size;
    unsigned int magic, version;
    int blocking, cgaClusterSize, minCTAs, maxCTAs;
    const char* netName;
    int splitShare;
};
typedef int (*pfn_ncclCommInitRankConfig)(void**, int, nccl_uid, int, nccl_config_2_18*);
typedef int (*pfn_ncclGetVersion)(int*);
typedef int (*pfn_ncclAllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*pfn_ncclCommDestroy)(void*);
typedef const char* (*pfn_ncclGetErrorString)(int);
constexpr int kNcclFloat32 = 7;  // ncclFloat32
constexpr int kNcclSum = 0;      // ncclSum

void* open_nccl() {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        void* h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) return h;
    }
    return nullptr;
}

__global__ void fg_counter_increment_kernel(uint32_t* c) { *c += 1u; }

}  // namespace

int32_t fg_ws_alloc(fg_ctx* ctx, uint64_t bytes, void** out) {
    uint64_t off = (ctx->ws_used + 255u) & ~uint64_t(255);
    uint64_t need = off + bytes;
    if (need > ctx->ws_bytes) {
        if (ctx->capturing)
            return fg_fail(ctx, FG_ERR_INCONSISTENT_CAPTURE,
                           "scratch arena too small while recording a plan: call fg_ctx_reserve_workspace first");
        if (ctx->ws_used != 0)
            return fg_fail(ctx, FG_ERR_INTERNAL, "scratch arena grown in the middle of an operation");
        // Everything that used the old arena was enqueued on this stream: drain it first.
        FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamSynchronize(ctx->stream));
        if (ctx->ws) cudaFree(ctx->ws);
        ctx->ws = nullptr;
        ctx->ws_bytes = 0;
        ctx->ws_generation++;      // plans recorded against the old arena must not be replayed (fg_plan_launch checks)
        uint64_t want = need + need / 4;
        cudaError_t e = cudaMalloc((void**)&ctx->ws, want);
        if (e != cudaSuccess) return fg_fail_cuda(ctx, FG_ERR_OUT_OF_MEMORY, "scratch arena", e);
        ctx->ws_bytes = want;
    }
    *out = ctx->ws + off;
    ctx->ws_used = need;
    return FG_OK;
}

// Makes sure `bytes` more can be carved from the arena.  Growing is only possible before anything has been
// carved for the current operation, so entry points ask for their whole need up front.
int32_t fg_ws_ensure(fg_ctx* ctx, uint64_t bytes) {
    const uint64_t off = (ctx->ws_used + 255u) & ~uint64_t(255);
    if (off + bytes <= ctx->ws_bytes) return FG_OK;
    if (ctx->ws_used != 0) return fg_fail(ctx, FG_ERR_INTERNAL, "scratch arena grown in the middle of an operation");
    void* p;
    const int32_t s = fg_ws_alloc(ctx, bytes, &p);
    ctx->ws_used = 0;
    return s;
}

static bool create_events(cudaEvent_t* ev, int n) {
    for (int i = 0; i < n; ++i)
        if (cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming) != cudaSuccess) return false;
    return true;
}

extern "C" {

const char* fg_version(void) { return "ferrograd_b200 0.1 (sm_100a)"; }

int32_t fg_ctx_set_option(fg_ctx* ctx, const char* name, const char* value) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, name && value, "fg_ctx_set_option: NULL argument");
    auto truth = [&](bool* dst) -> int32_t {
        if (!strcmp(value, "1") || !strcmp(value, "on")) { *dst = true; return FG_OK; }
        if (!strcmp(value, "0") || !strcmp(value, "off")) { *dst = false; return FG_OK; }
        return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "fg_ctx_set_option: the value must be 0, 1, on or off");
    };
    if (!strcmp(name, "gemm_tile")) {
        int x = 0, y = 0;
        if (!strcmp(value, "auto")) { ctx->opt_tile_pair = -1; return FG_OK; }
        if (!strcmp(value, "pair")) { ctx->opt_tile_pair = 1; return FG_OK; }
        if (sscanf(value, "%dx%d", &x, &y) == 2 && (x == 256 || x == 128) && (y == 32 || y == 16)) {
            ctx->opt_tile_pair = 0; ctx->opt_tile_bn = x; ctx->opt_tile_bk = y;
            return FG_OK;
        }
        return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "fg_ctx_set_option: gemm_tile is auto, pair, 256x32, 256x16, 128x32 or 128x16");
    }
    if (!strcmp(name, "gemm_split_k")) return truth(&ctx->opt_split_k);
    if (!strcmp(name, "gemm_pairs")) return truth(&ctx->opt_pairs);
    if (!strcmp(name, "exec_plans")) {
        if (!strcmp(value, "auto")) { ctx->opt_exec_plans = -1; return FG_OK; }
        bool on = false;
        const int32_t s = truth(&on);
        if (s == FG_OK) ctx->opt_exec_plans = on ? 1 : 0;
        return s;
    }
    if (!strcmp(name, "gemm_group")) {
        const long v = strtol(value, nullptr, 10);
        if (v < 0 || v > 64) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "fg_ctx_set_option: gemm_group must be 0 (default) .. 64");
        ctx->opt_tile_group = (int)v;
        return FG_OK;
    }
    if (!strcmp(name, "comm_min_exchange")) {
        char* end = nullptr;
        const unsigned long long v = strtoull(value, &end, 10);
        if (end == value || *end) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "fg_ctx_set_option: not a count");
        ctx->opt_min_exchange = v;
        return FG_OK;
    }
    if (!strcmp(name, "comm_max_ctas") || !strcmp(name, "comm_sms")) {
        char* end = nullptr;
        const long v = strtol(value, &end, 10);
        if (end == value || *end || v < 0 || v > 1024) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "fg_ctx_set_option: not a count");
        if (!strcmp(name, "comm_max_ctas")) ctx->opt_comm_max_ctas = (int)v;
        else ctx->comm_reserved_sms = (v > ctx->sm_count / 2) ? 0 : (int)v;
        return FG_OK;
    }
    return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "fg_ctx_set_option: unknown option");
}

int32_t fg_ctx_create_on_stream(int32_t device, void* cuda_stream, fg_ctx** out) {
    if (!out) return FG_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count)
        return FG_ERR_INVALID_DEVICE;
    if (cudaSetDevice(device) != cudaSuccess) return FG_ERR_INVALID_DEVICE;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return FG_ERR_INVALID_DEVICE;
    if (prop.major != 10) return FG_ERR_UNSUPPORTED_FEATURE;  // kernels are built for sm_100a only
    fg_ctx* c = new (std::nothrow) fg_ctx();
    if (!c) return FG_ERR_OUT_OF_MEMORY;
    memset(c, 0, sizeof(*c));
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    c->opt_tile_pair = -1;
    c->opt_tile_group = 0;
    c->opt_split_k = true;
    c->opt_pairs = true;
    c->opt_exec_plans = -1;
    c->opt_comm_max_ctas = 12;
    c->opt_min_exchange = 1ull << 20;
    c->comm_reserved_sms = 16;
    // the environment gives initial values, once
    if (const char* e = getenv("FG_GEMM_TILE")) fg_ctx_set_option(c, "gemm_tile", e);
    if (getenv("FG_GEMM_NO_SPLITK")) c->opt_split_k = false;
    if (getenv("FG_GEMM_NO_PAIRS")) c->opt_pairs = false;
    if (getenv("FG_EXEC_NO_PLANS")) c->opt_exec_plans = 0;
    if (const char* e = getenv("NCCL_MAX_CTAS")) fg_ctx_set_option(c, "comm_max_ctas", e);
    if (const char* e = getenv("FG_COMM_SMS")) fg_ctx_set_option(c, "comm_sms", e);
    if (const char* e = getenv("FG_COMM_MIN_EXCHANGE")) fg_ctx_set_option(c, "comm_min_exchange", e);
    if (const char* e = getenv("FG_GEMM_GROUP")) fg_ctx_set_option(c, "gemm_group", e);
    if (cuda_stream) {
        c->stream = (cudaStream_t)cuda_stream;
        c->own_stream = false;
    } else {
        if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) { delete c; return FG_ERR_INTERNAL; }
        c->own_stream = true;
    }
    // The exchange stream has the highest priority, so its CTAs are placed as soon as SMs are free.
    int prio_least = 0, prio_greatest = 0;
    cudaDeviceGetStreamPriorityRange(&prio_least, &prio_greatest);
    if (cudaStreamCreateWithPriority(&c->comm_stream, cudaStreamNonBlocking, prio_greatest) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_copy_done, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_main_mark, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming) != cudaSuccess ||
        !create_events(c->ev_ckpt, 8) ||
        cudaMalloc((void**)&c->dev_status, 256) != cudaSuccess ||
        cudaMemset(c->dev_status, 0, 256) != cudaSuccess) {
        // release whatever was created before the failure (the struct was zeroed: untouched members are NULL)
        if (c->comm_stream) cudaStreamDestroy(c->comm_stream);
        if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
        for (cudaEvent_t ev : {c->ev_copy_done, c->ev_main_mark, c->ev_fork, c->ev_join}) if (ev) cudaEventDestroy(ev);
        for (cudaEvent_t ev : c->ev_ckpt) if (ev) cudaEventDestroy(ev);
        if (c->dev_status) cudaFree(c->dev_status);
        if (c->own_stream && c->stream) cudaStreamDestroy(c->stream);
        delete c;
        return FG_ERR_INTERNAL;
    }
    cudaDriverEntryPointQueryResult qres;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
        c->tmap_encode = fn;
    *out = c;
    return FG_OK;
}

int32_t fg_ctx_create(int32_t device, fg_ctx** out) { return fg_ctx_create_on_stream(device, nullptr, out); }

int32_t fg_ctx_destroy(fg_ctx* ctx) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    cudaStreamSynchronize(ctx->comm_stream);
    fg_comm_destroy(ctx);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->time_recs) {
        for (int i = 0; i < ctx->time_created; ++i) { cudaEventDestroy(ctx->time_recs[i].a); cudaEventDestroy(ctx->time_recs[i].b); }
        delete[] ctx->time_recs;
    }
    cudaEventDestroy(ctx->ev_fork);
    cudaEventDestroy(ctx->ev_join);
    for (cudaEvent_t ev : ctx->ev_ckpt) if (ev) cudaEventDestroy(ev);
    cudaStreamDestroy(ctx->comm_stream);
    cudaStreamSynchronize(ctx->copy_stream);
    cudaStreamDestroy(ctx->copy_stream);
    cudaEventDestroy(ctx->ev_copy_done);
    cudaEventDestroy(ctx->ev_main_mark);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return FG_OK;
}

int32_t fg_sync(fg_ctx* ctx) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamSynchronize(ctx->comm_stream));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamSynchronize(ctx->copy_stream));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamSynchronize(ctx->stream));
    int status = 0;
    FG_CUDA(ctx, FG_ERR_SYNC, cudaMemcpy(&status, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (status != 0) {
        cudaMemset(ctx->dev_status, 0, sizeof(int));
        snprintf(ctx->err, sizeof(ctx->err), "a bounded device-side wait expired (status word 0x%x)", status);
        return FG_ERR_TIMEOUT;
    }
    return FG_OK;
}

int32_t fg_ctx_device_status(fg_ctx* ctx, int32_t* status_word) {
    if (!ctx || !status_word) return FG_ERR_INVALID_ARGUMENT;
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamSynchronize(ctx->stream));
    int status = 0;
    FG_CUDA(ctx, FG_ERR_SYNC, cudaMemcpy(&status, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (status) cudaMemset(ctx->dev_status, 0, sizeof(int));
    *status_word = status;
    return FG_OK;
}

int32_t fg_is_ready(fg_ctx* ctx, int32_t* ready) {
    if (!ctx || !ready) return FG_ERR_INVALID_ARGUMENT;
    cudaError_t e = cudaStreamQuery(ctx->stream);
    if (e == cudaSuccess) e = cudaStreamQuery(ctx->comm_stream);
    if (e == cudaSuccess) { *ready = 1; return FG_OK; }
    if (e == cudaErrorNotReady) { *ready = 0; return FG_OK; }
    return fg_fail_cuda(ctx, FG_ERR_SYNC, "cudaStreamQuery", e);
}

const char* fg_last_error(fg_ctx* ctx) { return ctx ? ctx->err : "no context"; }
void* fg_ctx_stream(fg_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
int32_t fg_ctx_device(fg_ctx* ctx) { return ctx ? ctx->device : -1; }
uint64_t fg_ctx_launch_count(fg_ctx* ctx) { return ctx ? ctx->launches : 0; }
uint64_t fg_ctx_workspace_bytes(fg_ctx* ctx) { return ctx ? ctx->ws_bytes : 0; }

int32_t fg_ctx_timing_enable(fg_ctx* ctx, int32_t on) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    if (ctx->capturing) return fg_fail(ctx, FG_ERR_INCONSISTENT_CAPTURE, "timing cannot change while a plan is recorded");
    if (on && !ctx->time_recs) {
        ctx->time_recs = new (std::nothrow) fg_time_rec[FG_TIME_MAX_RECS];
        if (!ctx->time_recs) return fg_fail(ctx, FG_ERR_OUT_OF_MEMORY, "timing records");
        ctx->time_count = ctx->time_created = 0;
    }
    ctx->timing_on = on != 0;
    return FG_OK;
}

int32_t fg_ctx_timing_read(fg_ctx* ctx, int32_t kind, uint64_t* launches, double* total_ms, double* total_work) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, launches && total_ms && total_work, "fg_ctx_timing_read: NULL output");
    *launches = 0; *total_ms = 0.0; *total_work = 0.0;
    if (!ctx->time_recs) return FG_OK;
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamSynchronize(ctx->stream));
    // Sum and drop the records of this kind; keep the others (and their events) packed at the front.
    int keep = 0;
    for (int i = 0; i < ctx->time_count; ++i) {
        fg_time_rec r = ctx->time_recs[i];
        if (r.kind == kind) {
            float ms = 0.0f;
            if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
                *launches += 1; *total_ms += ms; *total_work += r.work;
            }
            // recycle the events: swap this slot to the end of the used range later
            ctx->time_recs[i].kind = -1;
        }
    }
    // compact: stable partition so used records stay in front; events of dropped records are reused
    for (int i = 0; i < ctx->time_count; ++i) {
        if (ctx->time_recs[i].kind != -1) {
            if (i != keep) { fg_time_rec t = ctx->time_recs[keep]; ctx->time_recs[keep] = ctx->time_recs[i]; ctx->time_recs[i] = t; }
            keep++;
        }
    }
    ctx->time_count = keep;
    return FG_OK;
}

int32_t fg_ctx_reserve_workspace(fg_ctx* ctx, uint64_t bytes) {
    FG_ENTER(ctx);
    if (bytes <= ctx->ws_bytes) return FG_OK;
    return fg_ws_ensure(ctx, bytes);
}

// ---- memory ----
int32_t fg_alloc(fg_ctx* ctx, uint64_t bytes, fg_buf** out) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, out != nullptr, "fg_alloc: out is NULL");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    fg_buf* b = new (std::nothrow) fg_buf();
    if (!b) return fg_fail(ctx, FG_ERR_OUT_OF_MEMORY, "fg_alloc: host allocation failed");
    b->ptr = nullptr;
    b->bytes = bytes;
    b->version = 0;
    b->view = false;
    cudaError_t e = cudaMalloc(&b->ptr, bytes ? bytes : 1);
    if (e != cudaSuccess) { delete b; return fg_fail_cuda(ctx, FG_ERR_OUT_OF_MEMORY, "cudaMalloc", e); }
    *out = b;
    return FG_OK;
}

int32_t fg_alloc_zeroed(fg_ctx* ctx, uint64_t bytes, fg_buf** out) {
    int32_t s = fg_alloc(ctx, bytes, out);
    if (s != FG_OK) return s;
    FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY, cudaMemsetAsync((*out)->ptr, 0, bytes, ctx->stream));
    return FG_OK;
}

int32_t fg_alloc_init(fg_ctx* ctx, const void* data, uint64_t bytes, fg_buf** out) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, data != nullptr || bytes == 0, "fg_alloc_init: data is NULL");
    int32_t s = fg_alloc(ctx, bytes, out);
    if (s != FG_OK) return s;
    return fg_upload(ctx, *out, data, bytes, 0);
}

int32_t fg_free(fg_ctx* ctx, fg_buf* buf) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    if (!buf) return FG_OK;
    cudaSetDevice(ctx->device);
    if (!buf->view) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(buf->ptr);
    }
    delete buf;
    return FG_OK;
}

uint64_t fg_buf_size_bytes(const fg_buf* buf) { return buf ? buf->bytes : 0; }
void* fg_buf_device_ptr(const fg_buf* buf) { return buf ? buf->ptr : nullptr; }

int32_t fg_upload(fg_ctx* ctx, fg_buf* dst, const void* src, uint64_t bytes, uint64_t dst_off) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, dst && (src || bytes == 0), "fg_upload: NULL argument");
    FG_REQUIRE(ctx, dst_off <= dst->bytes && bytes <= dst->bytes - dst_off, "fg_upload: range exceeds the buffer");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    if (bytes == 0) return FG_OK;
    dst->version++;
    FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY,
            cudaMemcpyAsync((char*)dst->ptr + dst_off, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY, cudaStreamSynchronize(ctx->stream));
    return FG_OK;
}

int32_t fg_download(fg_ctx* ctx, const fg_buf* src, void* dst, uint64_t bytes, uint64_t src_off) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, src && (dst || bytes == 0), "fg_download: NULL argument");
    FG_REQUIRE(ctx, src_off <= src->bytes && bytes <= src->bytes - src_off, "fg_download: range exceeds the buffer");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    if (bytes == 0) return FG_OK;
    FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY,
            cudaMemcpyAsync(dst, (const char*)src->ptr + src_off, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY, cudaStreamSynchronize(ctx->stream));
    return FG_OK;
}

int32_t fg_copy(fg_ctx* ctx, const fg_buf* src, fg_buf* dst) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, src && dst, "fg_copy: NULL argument");
    FG_REQUIRE(ctx, src->bytes <= dst->bytes, "fg_copy: destination smaller than source");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    dst->version++;
    FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY,
            cudaMemcpyAsync(dst->ptr, src->ptr, src->bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return FG_OK;
}

int32_t fg_buf_touch(fg_buf* buf) {
    if (!buf) return FG_ERR_INVALID_ARGUMENT;
    buf->version++;
    return FG_OK;
}

int32_t fg_upload_async(fg_ctx* ctx, void* dst_dev, const void* src_pinned, uint64_t bytes) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, dst_dev && src_pinned, "fg_upload_async: NULL argument");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY,
            cudaMemcpyAsync(dst_dev, src_pinned, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return FG_OK;
}

int32_t fg_download_async(fg_ctx* ctx, void* dst_pinned, const void* src_dev, uint64_t bytes) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, dst_pinned && src_dev, "fg_download_async: NULL argument");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY,
            cudaMemcpyAsync(dst_pinned, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return FG_OK;
}

// ---- input prefetch: host->device copies on a side stream, overlapped with compute ----
int32_t fg_upload_prefetch(fg_ctx* ctx, void* dst_dev, const void* src_pinned, uint64_t bytes) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, dst_dev && src_pinned, "fg_upload_prefetch: NULL argument");
    if (ctx->capturing) return fg_fail(ctx, FG_ERR_INCONSISTENT_CAPTURE, "fg_upload_prefetch while recording a plan");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    // do not overwrite the destination before the compute stream has passed the last fg_prefetch_mark
    if (ctx->mark_valid) FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamWaitEvent(ctx->copy_stream, ctx->ev_main_mark, 0));
    FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY,
            cudaMemcpyAsync(dst_dev, src_pinned, bytes, cudaMemcpyHostToDevice, ctx->copy_stream));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaEventRecord(ctx->ev_copy_done, ctx->copy_stream));
    return FG_OK;
}

int32_t fg_prefetch_wait(fg_ctx* ctx) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamWaitEvent(ctx->stream, ctx->ev_copy_done, 0));
    return FG_OK;
}

int32_t fg_prefetch_mark(fg_ctx* ctx) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaEventRecord(ctx->ev_main_mark, ctx->stream));
    ctx->mark_valid = true;
    return FG_OK;
}

int32_t fg_copy_dev_async(fg_ctx* ctx, void* dst_dev, const void* src_dev, uint64_t bytes) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, dst_dev && src_dev, "fg_copy_dev_async: NULL argument");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY,
            cudaMemcpyAsync(dst_dev, src_dev, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return FG_OK;
}

int32_t fg_host_alloc_pinned(uint64_t bytes, void** out) {
    if (!out) return FG_ERR_INVALID_ARGUMENT;
    return cudaMallocHost(out, bytes ? bytes : 1) == cudaSuccess ? FG_OK : FG_ERR_OUT_OF_MEMORY;
}

int32_t fg_host_free_pinned(void* p) { return cudaFreeHost(p) == cudaSuccess ? FG_OK : FG_ERR_INVALID_ARGUMENT; }

int32_t fg_memset_zero(fg_ctx* ctx, void* dev, uint64_t bytes) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, dev != nullptr, "fg_memset_zero: NULL pointer");
    FG_CUDA(ctx, FG_ERR_FAILED_BUFFER_COPY, cudaMemsetAsync(dev, 0, bytes, ctx->stream));
    return FG_OK;
}

int32_t fg_counter_increment(fg_ctx* ctx, uint32_t* counter_dev) {
    FG_ENTER(ctx);
    FG_REQUIRE(ctx, counter_dev != nullptr, "fg_counter_increment: NULL pointer");
    fg_counter_increment_kernel<<<1, 1, 0, ctx->stream>>>(counter_dev);
    FG_LAUNCHED(ctx);
    return FG_OK;
}

// ---- plans ----
int32_t fg_plan_begin(fg_ctx* ctx) {
    FG_ENTER(ctx);
    if (ctx->capturing) return fg_fail(ctx, FG_ERR_INCONSISTENT_CAPTURE, "fg_plan_begin: already recording");
    FG_CUDA(ctx, FG_ERR_INCONSISTENT_CAPTURE, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    ctx->capture_launches = 0;
    ctx->capture_has_comm = false;
    return FG_OK;
}

int32_t fg_plan_end(fg_ctx* ctx, fg_plan** out) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    if (!ctx->capturing) return fg_fail(ctx, FG_ERR_INCONSISTENT_CAPTURE, "fg_plan_end: not recording");
    if (ctx->comm_pending) {
        int32_t s = fg_comm_join(ctx);
        if (s != FG_OK) return s;
    }
    ctx->capturing = false;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    if (e != cudaSuccess || !graph) return fg_fail_cuda(ctx, FG_ERR_INCONSISTENT_CAPTURE, "cudaStreamEndCapture", e);
    if (!out) { cudaGraphDestroy(graph); return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "fg_plan_end: out is NULL"); }
    fg_plan* p = new (std::nothrow) fg_plan();
    if (!p) { cudaGraphDestroy(graph); return fg_fail(ctx, FG_ERR_OUT_OF_MEMORY, "fg_plan_end"); }
    p->graph = graph;
    p->launches = ctx->capture_launches;
    p->ws_generation = ctx->ws_generation;
    p->ctx = ctx;
    p->has_comm = ctx->capture_has_comm;
    if (p->has_comm) ctx->comm_plans++;
    e = cudaGraphInstantiate(&p->exec, graph, 0);
    if (e != cudaSuccess) { cudaGraphDestroy(graph); delete p; return fg_fail_cuda(ctx, FG_ERR_INTERNAL, "cudaGraphInstantiate", e); }
    *out = p;
    return FG_OK;
}

int32_t fg_plan_launch(fg_ctx* ctx, fg_plan* plan) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, plan != nullptr, "fg_plan_launch: plan is NULL");
    if (ctx->capturing) return fg_fail(ctx, FG_ERR_INCONSISTENT_CAPTURE, "fg_plan_launch while recording");
    // The recorded kernels carry addresses inside the scratch arena as it was at recording time.  If an eager
    // call has grown (reallocated) the arena since, replaying would read and write freed memory: refuse.
    if (plan->ws_generation != ctx->ws_generation)
        return fg_fail(ctx, FG_ERR_INCONSISTENT_CAPTURE,
                       "fg_plan_launch: the scratch arena was reallocated after this plan was recorded; record it again "
                       "(fg_ctx_reserve_workspace before recording avoids this)");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_LAUNCH_FAILURE, cudaGraphLaunch(plan->exec, ctx->stream));
    ctx->launches += plan->launches;
    return FG_OK;
}

int32_t fg_plan_destroy(fg_plan* plan) {
    if (!plan) return FG_OK;
    if (plan->has_comm && plan->ctx && plan->ctx->comm_plans > 0) plan->ctx->comm_plans--;
    cudaGraphExecDestroy(plan->exec);
    cudaGraphDestroy(plan->graph);
    delete plan;
    return FG_OK;
}

// ---- NCCL ----
int32_t fg_comm_unique_id(uint8_t id_out[FG_COMM_ID_BYTES]) {
    if (!id_out) return FG_ERR_INVALID_ARGUMENT;
    void* h = open_nccl();
    if (!h) return FG_ERR_UNSUPPORTED_FEATURE;
    auto get = (pfn_ncclGetUniqueId)dlsym(h, "ncclGetUniqueId");
    if (!get) return FG_ERR_UNSUPPORTED_FEATURE;
    nccl_uid uid;
    if (get(&uid) != 0) return FG_ERR_INTERNAL;
    memcpy(id_out, uid.internal, FG_COMM_ID_BYTES);
    return FG_OK;
}

int32_t fg_comm_init(fg_ctx* ctx, int32_t nranks, int32_t rank, const uint8_t id[FG_COMM_ID_BYTES]) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, id != nullptr, "fg_comm_init: id is NULL");
    FG_REQUIRE(ctx, nranks >= 1 && rank >= 0 && rank < nranks, "fg_comm_init: rank outside [0, nranks)");
    if (ctx->comm) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "fg_comm_init: communicator already initialised");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    ctx->nccl_lib = open_nccl();
    if (!ctx->nccl_lib) return fg_fail(ctx, FG_ERR_UNSUPPORTED_FEATURE, "fg_comm_init: libnccl.so.2 not found");
    auto init = (pfn_ncclCommInitRank)dlsym(ctx->nccl_lib, "ncclCommInitRank");
    if (!init) return fg_fail(ctx, FG_ERR_UNSUPPORTED_FEATURE, "fg_comm_init: ncclCommInitRank missing");
    // An exchange CTA and a GEMM CTA cannot share an SM (registers, shared memory), and the pair GEMM is
    // persistent: if it took every SM the exchange would start only when it ended, and if the exchange
    // took some first the GEMM's last CTAs would start late with a full share of tiles.  So the exchange
    // is held to 12 CTAs (unless the caller's environment says otherwise) and the GEMM leaves 16 SMs free
    // while one is in flight (options comm_max_ctas and comm_sms; comm_sms 0 turns the reservation off).  Measured on
    // two GPUs (config-4 step, ms): 12 CTAs / 16 SMs 2.04, 8 / 12 2.03-2.07, 16 / 20 2.12, 4 / 8 2.42
    // (exchange-bound), no reservation 2.15-2.18; one GPU alone 1.96-2.00.
    // The limit is given in the communicator's own options: NCCL reads its environment once per process,
    // so a variable set here would be missed whenever another communicator (the host framework's) came first.
    const int max_ctas = ctx->opt_comm_max_ctas;
    auto init_cfg = (pfn_ncclCommInitRankConfig)dlsym(ctx->nccl_lib, "ncclCommInitRankConfig");
    auto get_ver = (pfn_ncclGetVersion)dlsym(ctx->nccl_lib, "ncclGetVersion");
    int nccl_ver = 0;
    if (get_ver) get_ver(&nccl_ver);
    nccl_uid uid;
    memcpy(uid.internal, id, FG_COMM_ID_BYTES);
    int r = -1;
    if (init_cfg && nccl_ver >= 21800 && max_ctas >= 1) {
        nccl_config_2_18 cfg;
        cfg.size = sizeof(cfg);
        cfg.magic = 0xcafebeef;
        cfg.version = 21800;
        cfg.blocking = 1;
        cfg.cgaClusterSize = INT_MIN;      // INT_MIN / NULL: "not set"
        cfg.minCTAs = INT_MIN;
        cfg.maxCTAs = max_ctas;
        cfg.netName = nullptr;
        cfg.splitShare = INT_MIN;
        r = init_cfg(&ctx->comm, nranks, uid, rank, &cfg);
    } else {
        r = init(&ctx->comm, nranks, uid, rank);
        ctx->comm_reserved_sms = 0;        // the exchange's CTA count is not under control: no reservation
    }
    if (r != 0) {
        auto es = (pfn_ncclGetErrorString)dlsym(ctx->nccl_lib, "ncclGetErrorString");
        snprintf(ctx->err, sizeof(ctx->err), "ncclCommInitRank: %s", es ? es(r) : "error");
        ctx->comm = nullptr;
        return FG_ERR_PEER_ACCESS;
    }
    ctx->nranks = nranks;
    ctx->rank = rank;
    return FG_OK;
}

int32_t fg_allreduce_sum_f32(fg_ctx* ctx, float* buf, uint64_t count) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, buf != nullptr, "fg_allreduce_sum_f32: buf is NULL");
    if (!ctx->comm) return fg_fail(ctx, FG_ERR_NOT_INITIALIZED, "fg_allreduce_sum_f32: call fg_comm_init first");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    if (count == 0) return FG_OK;
    auto ar = (pfn_ncclAllReduce)dlsym(ctx->nccl_lib, "ncclAllReduce");
    if (!ar) return fg_fail(ctx, FG_ERR_UNSUPPORTED_FEATURE, "ncclAllReduce missing");
    // Fork: the exchange starts once everything enqueued so far on the compute stream is done.
    FG_CUDA(ctx, FG_ERR_SYNC, cudaEventRecord(ctx->ev_fork, ctx->stream));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamWaitEvent(ctx->comm_stream, ctx->ev_fork, 0));
    int r = ar(buf, buf, (size_t)count, kNcclFloat32, kNcclSum, ctx->comm, ctx->comm_stream);
    if (r != 0) {
        auto es = (pfn_ncclGetErrorString)dlsym(ctx->nccl_lib, "ncclGetErrorString");
        snprintf(ctx->err, sizeof(ctx->err), "ncclAllReduce: %s", es ? es(r) : "error");
        return FG_ERR_PEER_ACCESS;
    }
    ctx->comm_pending = true;
    if (ctx->capturing) { ctx->capture_launches++; ctx->capture_has_comm = true; } else ctx->launches++;
    return FG_OK;
}

// A checkpoint marks "every exchange started so far"; fg_comm_wait makes the compute stream wait for
// just those, so work that needs only the early exchanges (the update of the last layers) can run while
// a later exchange (the first layer's) is still in flight.
int32_t fg_comm_checkpoint(fg_ctx* ctx, int32_t slot) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, slot >= 0 && slot < 8, "fg_comm_checkpoint: slot outside [0, 8)");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaEventRecord(ctx->ev_ckpt[slot], ctx->comm_stream));
    return FG_OK;
}

int32_t fg_comm_wait(fg_ctx* ctx, int32_t slot) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, slot >= 0 && slot < 8, "fg_comm_wait: slot outside [0, 8)");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamWaitEvent(ctx->stream, ctx->ev_ckpt[slot], 0));
    return FG_OK;
}

int32_t fg_comm_join(fg_ctx* ctx) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    if (!ctx->comm_pending) return FG_OK;
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaEventRecord(ctx->ev_join, ctx->comm_stream));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamWaitEvent(ctx->stream, ctx->ev_join, 0));
    ctx->comm_pending = false;
    return FG_OK;
}

// Tears the communicator down without waiting for its peers: a collective that is still waiting for
// a rank that will never arrive is ended (ncclCommAbort makes its kernel leave).
int32_t fg_comm_abort(fg_ctx* ctx) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    if (ctx->comm && ctx->nccl_lib) {
        auto ab = (pfn_ncclCommDestroy)dlsym(ctx->nccl_lib, "ncclCommAbort");
        if (ab) ab(ctx->comm);
    }
    ctx->comm = nullptr;
    ctx->comm_pending = false;
    return FG_OK;
}

// Host-side wait for every exchange started so far, at most timeout_ms.  On expiry the communicator is
// aborted, the context stays usable for everything but exchanges, and FG_ERR_TIMEOUT is returned.
int32_t fg_comm_sync(fg_ctx* ctx, uint32_t timeout_ms) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    if (ctx->capturing) return fg_fail(ctx, FG_ERR_INCONSISTENT_CAPTURE, "fg_comm_sync while recording a plan");
    FG_CUDA(ctx, FG_ERR_INVALID_DEVICE, cudaSetDevice(ctx->device));
    FG_CUDA(ctx, FG_ERR_SYNC, cudaEventRecord(ctx->ev_join, ctx->comm_stream));
    timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (;;) {
        cudaError_t q = cudaEventQuery(ctx->ev_join);
        if (q == cudaSuccess) break;
        if (q != cudaErrorNotReady) return fg_fail_cuda(ctx, FG_ERR_SYNC, "exchange", q);
        timespec t1;
        clock_gettime(CLOCK_MONOTONIC, &t1);
        const double ms = (t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6;
        if (ms > (double)timeout_ms) {
            fg_comm_abort(ctx);
            cudaStreamSynchronize(ctx->comm_stream);      // the aborted collective's kernel leaves promptly
            return fg_fail(ctx, FG_ERR_TIMEOUT, "fg_comm_sync: the exchange did not complete in time; communicator aborted");
        }
        timespec nap = {0, 200000};
        nanosleep(&nap, nullptr);
    }
    FG_CUDA(ctx, FG_ERR_SYNC, cudaStreamWaitEvent(ctx->stream, ctx->ev_join, 0));
    ctx->comm_pending = false;
    return FG_OK;
}

int32_t fg_comm_destroy(fg_ctx* ctx) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    if (ctx->comm && ctx->nccl_lib) {
        // A recorded plan that contains an exchange keeps the communicator in use: tearing the communicator down
        // waits for the plan to be destroyed, i.e. for ever if the caller destroys things in the other order
        // (seen with ncclCommDestroy and with ncclCommAbort).  With such plans still alive the communicator is
        // left to the end of the process instead.
        if (ctx->comm_plans == 0) {
            auto d = (pfn_ncclCommDestroy)dlsym(ctx->nccl_lib, "ncclCommDestroy");
            if (d) d(ctx->comm);
        }
    }
    ctx->comm = nullptr;
    return FG_OK;
}

}  // extern "C"
