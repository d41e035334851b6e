// extern "C" surface of liblokal_cuda: context, memory, streams, graph capture,
// the op entry points (thin validation + launch) and the host-slice mirrors of
// the reference's CPU signatures. See include/lokal_cuda.h for the contract of
// each function and the reference interface it replaces.
#include <atomic>
#include <cstring>
#include <new>
#include <thread>
#include <vector>

#include "common.cuh"

using lokal::DeviceGuard;

namespace {

constexpr const char* kVersion = "lokal_cuda 0.1 (sm_100a)";

cudaStream_t as_stream(lokal_cuda_stream s) { return static_cast<cudaStream_t>(s); }

// Grow-only device blocks / pinned staging owned by the context.
//
// The table block of lokal_cuda_qk_rope_pos is used in stream order on the callers' streams. Growing it drains the
// device first (work already queued may still read the old block). A block whose address a captured graph holds is
// never freed while the context lives: it is set aside and a new one takes its place, so replays stay valid.
int ensure_scratch(lokal_cuda_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->scratch_bytes) return LOKAL_OK;
    size_t want = ctx->scratch_bytes ? ctx->scratch_bytes : (1u << 20);
    while (want < bytes) want *= 2;
    LOKAL_CUDA_TRY(ctx, cudaDeviceSynchronize());
    if (ctx->scratch) {
        if (ctx->scratch_in_graph) {
            if (ctx->n_retired >= 8)
                return ctx->fail(LOKAL_ERR_UNSUPPORTED, "qk_rope_pos: the table block has been captured into graphs and outgrown eight times; "
                                                         "size it once with the largest call before capturing");
            ctx->retired_scratch[ctx->n_retired++] = ctx->scratch;
        } else {
            LOKAL_CUDA_TRY(ctx, cudaFree(ctx->scratch));
        }
    }
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    ctx->scratch_in_graph = false;
    LOKAL_CUDA_TRY(ctx, cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
    return LOKAL_OK;
}

// The host-slice mirrors have a block of their own: they run on host_stream, one call at a time (ctx->mu), and must
// not touch the table block, which kernels queued on other streams may still be reading.
int ensure_host_scratch(lokal_cuda_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->host_scratch_bytes) return LOKAL_OK;
    size_t want = ctx->host_scratch_bytes ? ctx->host_scratch_bytes : (1u << 20);
    while (want < bytes) want *= 2;
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->host_stream));
    if (ctx->host_scratch) LOKAL_CUDA_TRY(ctx, cudaFree(ctx->host_scratch));
    ctx->host_scratch = nullptr;
    ctx->host_scratch_bytes = 0;
    LOKAL_CUDA_TRY(ctx, cudaMalloc(&ctx->host_scratch, want));
    ctx->host_scratch_bytes = want;
    return LOKAL_OK;
}

int ensure_staging(lokal_cuda_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->staging_bytes) return LOKAL_OK;
    size_t want = ctx->staging_bytes ? ctx->staging_bytes : (1u << 20);
    while (want < bytes) want *= 2;
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->host_stream));
    if (ctx->staging) LOKAL_CUDA_TRY(ctx, cudaFreeHost(ctx->staging));
    ctx->staging = nullptr;
    ctx->staging_bytes = 0;
    LOKAL_CUDA_TRY(ctx, cudaHostAlloc(&ctx->staging, want, cudaHostAllocDefault));
    ctx->staging_bytes = want;
    return LOKAL_OK;
}

// Page-locked host memory that CUDA knows (cudaHostAlloc / cudaHostRegister): a copy engine can reach it directly.
bool is_pinned_host(const void* p) {
    cudaPointerAttributes at{};
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeHost;
}

// Device memory -> ordinary (pageable) host memory, for results too large to bounce through one staging copy and one
// single-threaded memcpy: a few workers, each with its own stream and its own slice of the pinned staging block, pull
// 4 MB chunks in turn, so the DMA of one chunk overlaps the CPU copy (and the page faults of a fresh destination) of
// the others. `s` is the stream the producer kernel ran on.
int d2h_pageable(lokal_cuda_ctx* ctx, cudaStream_t s, const char* dev, char* out, size_t bytes) {
    constexpr size_t kChunk = 4u << 20;
    const size_t chunks = (bytes + kChunk - 1) / kChunk;
    unsigned hw = std::thread::hardware_concurrency();
    unsigned workers = hw >= 16 ? 8 : (hw >= 4 ? hw / 2 : 1);
    if (workers > chunks) workers = static_cast<unsigned>(chunks);
    int rc = ensure_staging(ctx, workers * kChunk);
    if (rc != LOKAL_OK) return rc;
    if (!ctx->copy_ready) LOKAL_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->copy_ready, cudaEventDisableTiming));
    for (unsigned w = 0; w < workers; w++)
        if (!ctx->copy_streams[w]) LOKAL_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->copy_streams[w], cudaStreamNonBlocking));
    LOKAL_CUDA_TRY(ctx, cudaEventRecord(ctx->copy_ready, s));
    std::atomic<size_t> next{0};
    std::atomic<int> first_error{static_cast<int>(cudaSuccess)};
    auto work = [&](unsigned w) {
        cudaError_t e = cudaSetDevice(ctx->device);
        cudaStream_t cs = ctx->copy_streams[w];
        char* slot = static_cast<char*>(ctx->staging) + w * kChunk;
        if (e == cudaSuccess) e = cudaStreamWaitEvent(cs, ctx->copy_ready, 0);
        while (e == cudaSuccess) {
            const size_t c = next.fetch_add(1);
            if (c >= chunks) break;
            const size_t off = c * kChunk, sz = bytes - off < kChunk ? bytes - off : kChunk;
            e = cudaMemcpyAsync(slot, dev + off, sz, cudaMemcpyDeviceToHost, cs);
            if (e == cudaSuccess) e = cudaStreamSynchronize(cs);
            if (e == cudaSuccess) std::memcpy(out + off, slot, sz);
        }
        if (e != cudaSuccess) {
            int want = static_cast<int>(cudaSuccess);
            first_error.compare_exchange_strong(want, static_cast<int>(e));
        }
    };
    std::vector<std::thread> pool;
    for (unsigned w = 1; w < workers; w++) pool.emplace_back(work, w);
    work(0);
    for (std::thread& t : pool) t.join();
    const cudaError_t e = static_cast<cudaError_t>(first_error.load());
    if (e != cudaSuccess) return ctx->fail(LOKAL_ERR_CUDA, "device-to-host copy failed: %s", cudaGetErrorString(e));
    return LOKAL_OK;
}

int read_error_word(lokal_cuda_ctx* ctx, cudaStream_t s) {
    LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->err_word_host, ctx->err_word, sizeof(unsigned), cudaMemcpyDeviceToHost, s));
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(s));
    const unsigned bits = *ctx->err_word_host;
    if (bits == 0) return LOKAL_OK;
    LOKAL_CUDA_TRY(ctx, cudaMemsetAsync(ctx->err_word, 0, sizeof(unsigned), s));
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(s));
    if (bits & lokal::kErrTimeout) return ctx->fail(LOKAL_ERR_TIMEOUT, "a device-side wait on a staged copy gave up");
    if (bits & lokal::kErrPosRange)
        return ctx->fail(LOKAL_ERR_POS_RANGE, "a position was negative or beyond the KV cache (its row was not stored)");
    return ctx->fail(LOKAL_ERR_ID_RANGE, "a token id was out of range for the table (its row was zero-filled)");
}

}  // namespace

#define LOKAL_ENTER(ctx)                                                                 \
    if (!(ctx)) return LOKAL_ERR_BAD_ARG;                                                \
    DeviceGuard guard__((ctx)->device);                                                  \
    if (!guard__.ok) return (ctx)->fail(LOKAL_ERR_CUDA, "cannot select device %d", (ctx)->device)

extern "C" {

const char* lokal_cuda_version(void) { return kVersion; }

int lokal_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int lokal_cuda_create(int device, lokal_cuda_ctx** out) {
    if (!out) return LOKAL_ERR_BAD_ARG;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        return LOKAL_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= n) return LOKAL_ERR_BAD_ARG;
    lokal_cuda_ctx* ctx = new (std::nothrow) lokal_cuda_ctx();
    if (!ctx) return LOKAL_ERR_CUDA;
    ctx->device = device;
    DeviceGuard guard(device);
    cudaDeviceProp prop{};
    bool ok = guard.ok && cudaGetDeviceProperties(&prop, device) == cudaSuccess;
    if (ok && prop.major < 10) {
        // The library holds sm_100a code only; refuse by name rather than fail at the first launch.
        delete ctx;
        return LOKAL_ERR_UNSUPPORTED;
    }
    if (ok) ctx->sm_count = prop.multiProcessorCount;
    ok = ok && cudaMalloc(reinterpret_cast<void**>(&ctx->err_word), sizeof(unsigned)) == cudaSuccess;
    ok = ok && cudaMemset(ctx->err_word, 0, sizeof(unsigned)) == cudaSuccess;
    ok = ok && cudaHostAlloc(reinterpret_cast<void**>(&ctx->err_word_host), sizeof(unsigned), cudaHostAllocDefault) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&ctx->host_stream, cudaStreamNonBlocking) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        lokal_cuda_destroy(ctx);
        return LOKAL_ERR_CUDA;
    }
    *out = ctx;
    return LOKAL_OK;
}

void lokal_cuda_destroy(lokal_cuda_ctx* ctx) {
    if (!ctx) return;
    DeviceGuard guard(ctx->device);
    if (ctx->host_stream) cudaStreamDestroy(ctx->host_stream);
    for (cudaStream_t cs : ctx->copy_streams)
        if (cs) cudaStreamDestroy(cs);
    if (ctx->copy_ready) cudaEventDestroy(ctx->copy_ready);
    if (ctx->scratch_event) cudaEventDestroy(ctx->scratch_event);
    if (ctx->err_word) cudaFree(ctx->err_word);
    if (ctx->err_word_host) cudaFreeHost(ctx->err_word_host);
    if (ctx->scratch) cudaFree(ctx->scratch);
    for (int i = 0; i < ctx->n_retired; i++) cudaFree(ctx->retired_scratch[i]);
    if (ctx->host_scratch) cudaFree(ctx->host_scratch);
    if (ctx->staging) cudaFreeHost(ctx->staging);
    for (void* g : ctx->iq_grids)
        if (g) cudaFree(g);
    delete ctx;
}

const char* lokal_cuda_last_error(const lokal_cuda_ctx* ctx) {
    if (!ctx) return "null context";
    // The string lives in the context and stays valid until the next failing call on it.
    return ctx->last_error.c_str();
}

int lokal_cuda_malloc(lokal_cuda_ctx* ctx, size_t bytes, void** dptr) {
    LOKAL_ENTER(ctx);
    if (!dptr) return ctx->fail(LOKAL_ERR_BAD_ARG, "malloc: output pointer is null");
    *dptr = nullptr;
    if (bytes == 0) return LOKAL_OK;
    LOKAL_CUDA_TRY(ctx, cudaMalloc(dptr, bytes));
    return LOKAL_OK;
}

int lokal_cuda_free(lokal_cuda_ctx* ctx, void* dptr) {
    LOKAL_ENTER(ctx);
    if (dptr) LOKAL_CUDA_TRY(ctx, cudaFree(dptr));
    return LOKAL_OK;
}

int lokal_cuda_host_alloc(lokal_cuda_ctx* ctx, size_t bytes, void** hptr) {
    LOKAL_ENTER(ctx);
    if (!hptr) return ctx->fail(LOKAL_ERR_BAD_ARG, "host_alloc: output pointer is null");
    *hptr = nullptr;
    if (bytes == 0) return LOKAL_OK;
    LOKAL_CUDA_TRY(ctx, cudaHostAlloc(hptr, bytes, cudaHostAllocDefault));
    return LOKAL_OK;
}

int lokal_cuda_host_free(lokal_cuda_ctx* ctx, void* hptr) {
    LOKAL_ENTER(ctx);
    if (hptr) LOKAL_CUDA_TRY(ctx, cudaFreeHost(hptr));
    return LOKAL_OK;
}

int lokal_cuda_memcpy_h2d(lokal_cuda_ctx* ctx, lokal_cuda_stream s, void* dst, const void* src, size_t bytes) {
    LOKAL_ENTER(ctx);
    if (bytes && (!dst || !src)) return ctx->fail(LOKAL_ERR_BAD_ARG, "memcpy_h2d: null pointer");
    if (bytes) LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(s)));
    return LOKAL_OK;
}

int lokal_cuda_memcpy_d2h(lokal_cuda_ctx* ctx, lokal_cuda_stream s, void* dst, const void* src, size_t bytes) {
    LOKAL_ENTER(ctx);
    if (bytes && (!dst || !src)) return ctx->fail(LOKAL_ERR_BAD_ARG, "memcpy_d2h: null pointer");
    if (bytes) LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(s)));
    return LOKAL_OK;
}

int lokal_cuda_stream_create(lokal_cuda_ctx* ctx, lokal_cuda_stream* out) {
    LOKAL_ENTER(ctx);
    if (!out) return ctx->fail(LOKAL_ERR_BAD_ARG, "stream_create: output pointer is null");
    cudaStream_t s = nullptr;
    LOKAL_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *out = s;
    return LOKAL_OK;
}

int lokal_cuda_stream_destroy(lokal_cuda_ctx* ctx, lokal_cuda_stream s) {
    LOKAL_ENTER(ctx);
    if (s) LOKAL_CUDA_TRY(ctx, cudaStreamDestroy(as_stream(s)));
    return LOKAL_OK;
}

int lokal_cuda_stream_sync(lokal_cuda_ctx* ctx, lokal_cuda_stream s) {
    LOKAL_ENTER(ctx);
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(as_stream(s)));
    return read_error_word(ctx, as_stream(s));
}

int lokal_cuda_graph_begin(lokal_cuda_ctx* ctx, lokal_cuda_stream s) {
    LOKAL_ENTER(ctx);
    if (!s) return ctx->fail(LOKAL_ERR_BAD_ARG, "graph_begin: capture needs a stream from lokal_cuda_stream_create");
    LOKAL_CUDA_TRY(ctx, cudaStreamBeginCapture(as_stream(s), cudaStreamCaptureModeThreadLocal));
    return LOKAL_OK;
}

int lokal_cuda_graph_end(lokal_cuda_ctx* ctx, lokal_cuda_stream s, lokal_cuda_graph** out) {
    LOKAL_ENTER(ctx);
    if (!out) return ctx->fail(LOKAL_ERR_BAD_ARG, "graph_end: output pointer is null");
    *out = nullptr;
    cudaGraph_t g = nullptr;
    LOKAL_CUDA_TRY(ctx, cudaStreamEndCapture(as_stream(s), &g));
    cudaGraphExec_t ex = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        return ctx->fail(LOKAL_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    }
    lokal_cuda_graph* h = new (std::nothrow) lokal_cuda_graph();
    if (!h) {
        cudaGraphExecDestroy(ex);
        cudaGraphDestroy(g);
        return ctx->fail(LOKAL_ERR_CUDA, "out of host memory");
    }
    h->graph = g;
    h->exec = ex;
    *out = h;
    return LOKAL_OK;
}

int lokal_cuda_graph_launch(lokal_cuda_ctx* ctx, lokal_cuda_graph* g, lokal_cuda_stream s) {
    LOKAL_ENTER(ctx);
    if (!g || !g->exec) return ctx->fail(LOKAL_ERR_BAD_ARG, "graph_launch: null graph");
    LOKAL_CUDA_TRY(ctx, cudaGraphLaunch(g->exec, as_stream(s)));
    return LOKAL_OK;
}

int lokal_cuda_graph_destroy(lokal_cuda_ctx* ctx, lokal_cuda_graph* g) {
    LOKAL_ENTER(ctx);
    if (!g) return LOKAL_OK;
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    return LOKAL_OK;
}

// ---- block geometry ----

size_t lokal_cuda_blk_elems(int t) {
    switch (t) {
        case LOKAL_F32: case LOKAL_F16: case LOKAL_BF16: return 1;
        case LOKAL_Q4_0: case LOKAL_Q5_0: case LOKAL_Q8_0: case LOKAL_IQ4_NL: return 32;
        case LOKAL_Q2_K: case LOKAL_Q3_K: case LOKAL_Q4_K: case LOKAL_Q5_K: case LOKAL_Q6_K: case LOKAL_IQ4_XS:
        case LOKAL_IQ2_XXS: case LOKAL_IQ2_XS: case LOKAL_IQ2_S: case LOKAL_IQ3_XXS: case LOKAL_IQ3_S: case LOKAL_IQ1_S: case LOKAL_IQ1_M:
            return 256;
        default: return 0;
    }
}

size_t lokal_cuda_blk_bytes(int t) {
    switch (t) {
        case LOKAL_F32: return 4;
        case LOKAL_F16: case LOKAL_BF16: return 2;
        case LOKAL_Q4_0: case LOKAL_IQ4_NL: return 18;
        case LOKAL_Q5_0: return 22;
        case LOKAL_Q8_0: return 34;
        case LOKAL_Q2_K: return 84;
        case LOKAL_Q3_K: return 110;
        case LOKAL_Q4_K: return 144;
        case LOKAL_Q5_K: return 176;
        case LOKAL_Q6_K: return 210;
        case LOKAL_IQ4_XS: return 136;
        case LOKAL_IQ1_S: return 50;
        case LOKAL_IQ1_M: return 56;
        case LOKAL_IQ2_XXS: return 66;
        case LOKAL_IQ2_XS: return 74;
        case LOKAL_IQ2_S: return 82;
        case LOKAL_IQ3_XXS: return 98;
        case LOKAL_IQ3_S: return 110;
        default: return 0;
    }
}

// Codebook entries and entry size of lokal_iq_grid `which`.
static const size_t kIqGridEntries[6] = {256, 512, 1024, 256, 512, 2048};
static const size_t kIqGridEntryBytes[6] = {8, 8, 8, 4, 4, 8};

int lokal_cuda_set_iq_grid(lokal_cuda_ctx* ctx, int which, const void* table, size_t bytes) {
    LOKAL_ENTER(ctx);
    if (which < 0 || which > 5) return ctx->fail(LOKAL_ERR_BAD_ARG, "set_iq_grid: codebook %d does not exist", which);
    const size_t want = kIqGridEntries[which] * kIqGridEntryBytes[which];
    if (!table || bytes != want)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "set_iq_grid: codebook %d holds %zu entries of %zu bytes = %zu bytes, got %zu", which,
                         kIqGridEntries[which], kIqGridEntryBytes[which], want, bytes);
    std::lock_guard<std::mutex> g(ctx->mu);
    if (!ctx->iq_grids[which]) LOKAL_CUDA_TRY(ctx, cudaMalloc(&ctx->iq_grids[which], want));
    LOKAL_CUDA_TRY(ctx, cudaMemcpy(ctx->iq_grids[which], table, want, cudaMemcpyHostToDevice));
    return LOKAL_OK;
}

size_t lokal_cuda_row_bytes(int t, size_t n) {
    const size_t be = lokal_cuda_blk_elems(t);
    return be ? n / be * lokal_cuda_blk_bytes(t) : 0;
}

// ---- ops on device memory ----

int lokal_cuda_rmsnorm(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* x, const void* w, void* y, void* y_h,
                       size_t rows, size_t dim, float eps, int dtype, int w_dtype, int h_dtype) {
    LOKAL_ENTER(ctx);
    return lokal::launch_norm(ctx, as_stream(s), const_cast<void*>(x), nullptr, w, y, y_h, rows, dim, eps, dtype, w_dtype, h_dtype);
}

int lokal_cuda_add_rmsnorm(lokal_cuda_ctx* ctx, lokal_cuda_stream s, void* x_inout, const void* delta, const void* w,
                           void* xn, void* xn_h, size_t rows, size_t dim, float eps, int dtype, int w_dtype, int h_dtype) {
    LOKAL_ENTER(ctx);
    if (!delta) return ctx->fail(LOKAL_ERR_BAD_ARG, "add_rmsnorm: delta is null (use lokal_cuda_rmsnorm for the plain norm)");
    return lokal::launch_norm(ctx, as_stream(s), x_inout, delta, w, xn, xn_h, rows, dim, eps, dtype, w_dtype, h_dtype);
}

int lokal_cuda_rope_table(lokal_cuda_ctx* ctx, lokal_cuda_stream s, float theta, uint32_t rot_dim, const int32_t* positions,
                          int64_t pos0, size_t rows, float* cos_sin) {
    LOKAL_ENTER(ctx);
    return lokal::launch_rope_table(ctx, as_stream(s), theta, rot_dim, positions, pos0, rows, cos_sin);
}

int lokal_cuda_qk_rope(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const lokal_qk_rope_params* p) {
    LOKAL_ENTER(ctx);
    if (!p) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: params are null");
    return lokal::launch_qk_rope(ctx, as_stream(s), *p);
}

int lokal_cuda_qk_rope_pos(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const lokal_qk_rope_params* p, float theta,
                           const int32_t* positions, int64_t pos0) {
    LOKAL_ENTER(ctx);
    if (!p) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope_pos: params are null");
    if (p->rot_dim == 0 || p->rows > (SIZE_MAX / 4) / (p->rot_dim ? p->rot_dim : 1))
        return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope_pos: rot_dim/rows out of range");
    std::lock_guard<std::mutex> g(ctx->mu);
    // The table lives in a block shared by every stream of the context. Sessions on different streams may call
    // this concurrently, so each call first waits (on the device, in its own stream) for the previous call's rope
    // kernel to have consumed the table, and leaves an event behind for the next one. A stream under graph capture
    // cannot take part in that hand-over: a captured call relies on its caller to keep other users of this entry
    // point off the context while the graph runs (lokal_cuda_qk_rope with the caller's own table has no such limit).
    // Nor can a captured call allocate or drain the device: it must find the block large enough already.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    LOKAL_CUDA_TRY(ctx, cudaStreamIsCapturing(as_stream(s), &cap));
    const bool ordered = cap == cudaStreamCaptureStatusNone;
    const size_t table_bytes = static_cast<size_t>(p->rows) * p->rot_dim * sizeof(float);
    if (!ordered) {
        if (table_bytes > ctx->scratch_bytes)
            return ctx->fail(LOKAL_ERR_BAD_ARG,
                             "qk_rope_pos: the stream is being captured and the table block (%zu bytes) is smaller than this call needs "
                             "(%zu): make one uncaptured call of this size first, or pass your own table to lokal_cuda_qk_rope",
                             ctx->scratch_bytes, table_bytes);
        ctx->scratch_in_graph = true;
    }
    int rc = ensure_scratch(ctx, table_bytes);
    if (rc != LOKAL_OK) return rc;
    if (ordered) {
        if (!ctx->scratch_event) LOKAL_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->scratch_event, cudaEventDisableTiming));
        if (ctx->scratch_event_recorded) LOKAL_CUDA_TRY(ctx, cudaStreamWaitEvent(as_stream(s), ctx->scratch_event, 0));
    }
    float* table = static_cast<float*>(ctx->scratch);
    rc = lokal::launch_rope_table(ctx, as_stream(s), theta, p->rot_dim, positions, pos0, p->rows, table);
    if (rc != LOKAL_OK) return rc;
    lokal_qk_rope_params q = *p;
    q.cos_sin = table;
    rc = lokal::launch_qk_rope(ctx, as_stream(s), q);
    if (ordered) {
        LOKAL_CUDA_TRY(ctx, cudaEventRecord(ctx->scratch_event, as_stream(s)));
        ctx->scratch_event_recorded = true;
    }
    return rc;
}

int lokal_cuda_swiglu(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* gate, const void* up, void* out, void* out_h,
                      size_t n, int dtype, int h_dtype) {
    LOKAL_ENTER(ctx);
    return lokal::launch_swiglu(ctx, as_stream(s), gate, up, out, out_h, n, dtype, h_dtype);
}

int lokal_cuda_embed_gather(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* table, int ggml_type, size_t vocab,
                            size_t dim, const uint32_t* ids, size_t n, void* out, int out_dtype) {
    LOKAL_ENTER(ctx);
    if (!ids && n) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather: ids are null");
    return lokal::launch_gather(ctx, as_stream(s), table, ggml_type, vocab, dim, ids, n, out, out_dtype);
}

int lokal_cuda_embed_gather_rmsnorm(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* table, int ggml_type, size_t vocab,
                                    size_t dim, const uint32_t* ids, size_t n, void* x, void* xn, const void* w, float eps,
                                    int out_dtype, int w_dtype) {
    LOKAL_ENTER(ctx);
    if (!ids && n) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather_rmsnorm: ids are null");
    if (!w || !xn) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather_rmsnorm: weights and the normed output must be non-null");
    return lokal::launch_gather_norm(ctx, as_stream(s), table, ggml_type, vocab, dim, ids, n, x, out_dtype, w, w_dtype, xn, eps, nullptr);
}

int lokal_cuda_dequant_rows(lokal_cuda_ctx* ctx, lokal_cuda_stream s, int ggml_type, const void* src, size_t rows,
                            size_t cols, void* out, int out_dtype) {
    LOKAL_ENTER(ctx);
    if (rows == 0) return LOKAL_OK;
    return lokal::launch_gather(ctx, as_stream(s), src, ggml_type, rows, cols, nullptr, rows, out, out_dtype);
}

int lokal_cuda_shard_rows(size_t n_rows, int n_gpus, int rank, size_t* row0, size_t* count) {
    if (!row0 || !count || n_gpus <= 0 || rank < 0 || rank >= n_gpus) return LOKAL_ERR_BAD_ARG;
    const size_t per = (n_rows + static_cast<size_t>(n_gpus) - 1) / static_cast<size_t>(n_gpus);
    size_t r0 = per * static_cast<size_t>(rank);
    if (r0 > n_rows) r0 = n_rows;
    size_t r1 = r0 + per;
    if (r1 > n_rows) r1 = n_rows;
    *row0 = r0;
    *count = r1 - r0;
    return LOKAL_OK;
}

// ---- host-slice mirrors ----
// Layout of one call: inputs are copied into pinned staging, sent to device
// scratch, the op runs, the result comes back through staging. One call at a
// time per context (ctx->mu).

int lokal_cuda_host_rmsnorm(lokal_cuda_ctx* ctx, const float* x, const float* w, float eps, size_t rows, size_t dim, float* y) {
    LOKAL_ENTER(ctx);
    if (!x || !w || !y) return ctx->fail(LOKAL_ERR_BAD_ARG, "host_rmsnorm: null pointer");
    if (rows == 0 || dim == 0) return dim == 0 ? ctx->fail(LOKAL_ERR_BAD_ARG, "host_rmsnorm: dim is zero") : LOKAL_OK;
    std::lock_guard<std::mutex> g(ctx->mu);
    // device scratch: [w | x | y], each part starting on a 256-byte boundary
    const size_t xb = rows * dim * 4, wb = (dim * 4 + 255) & ~size_t(255), xb_al = (xb + 255) & ~size_t(255);
    int rc = ensure_host_scratch(ctx, wb + xb_al + xb);
    if (rc == LOKAL_OK) rc = ensure_staging(ctx, wb + xb);
    if (rc != LOKAL_OK) return rc;
    cudaStream_t s = ctx->host_stream;
    char* st = static_cast<char*>(ctx->staging);
    char* d = static_cast<char*>(ctx->host_scratch);
    std::memcpy(st, w, dim * 4);
    std::memcpy(st + wb, x, xb);
    LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(d, st, wb + xb, cudaMemcpyHostToDevice, s));
    void* dy = d + wb + xb_al;
    rc = lokal::launch_norm(ctx, s, d + wb, nullptr, d, dy, nullptr, rows, dim, eps, LOKAL_F32, LOKAL_F32, 0);
    if (rc != LOKAL_OK) return rc;
    LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(st, dy, xb, cudaMemcpyDeviceToHost, s));
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(s));
    std::memcpy(y, st, xb);
    return LOKAL_OK;
}

int lokal_cuda_host_rope(lokal_cuda_ctx* ctx, float* x, size_t n, size_t pos, size_t head_dim, float theta) {
    LOKAL_ENTER(ctx);
    if (!x) return ctx->fail(LOKAL_ERR_BAD_ARG, "host_rope: null pointer");
    if (head_dim == 0 || (head_dim & 1) || n % head_dim != 0)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "host_rope: %zu elements are not whole heads of even head_dim %zu", n, head_dim);
    if (n == 0) return LOKAL_OK;
    std::lock_guard<std::mutex> g(ctx->mu);
    const size_t xb = (n * 4 + 255) & ~size_t(255), tb = head_dim * 4;
    int rc = ensure_host_scratch(ctx, xb + tb + 256);
    if (rc == LOKAL_OK) rc = ensure_staging(ctx, xb);
    if (rc != LOKAL_OK) return rc;
    cudaStream_t s = ctx->host_stream;
    char* d = static_cast<char*>(ctx->host_scratch);
    std::memcpy(ctx->staging, x, n * 4);
    LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(d, ctx->staging, n * 4, cudaMemcpyHostToDevice, s));
    float* table = reinterpret_cast<float*>(d + xb);
    rc = lokal::launch_rope_table(ctx, s, theta, static_cast<uint32_t>(head_dim), nullptr, static_cast<int64_t>(pos), 1, table);
    if (rc != LOKAL_OK) return rc;
    lokal_qk_rope_params p{};
    p.q = d;
    p.cos_sin = table;
    p.rows = 1;
    p.n_q_heads = static_cast<uint32_t>(n / head_dim);
    p.head_dim = p.rot_dim = static_cast<uint32_t>(head_dim);
    p.q_row_stride = n;
    p.q_dtype = LOKAL_F32;
    rc = lokal::launch_qk_rope(ctx, s, p);
    if (rc != LOKAL_OK) return rc;
    LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->staging, d, n * 4, cudaMemcpyDeviceToHost, s));
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(s));
    std::memcpy(x, ctx->staging, n * 4);
    return LOKAL_OK;
}

int lokal_cuda_host_swiglu(lokal_cuda_ctx* ctx, const float* gate, const float* up, size_t n, float* out) {
    LOKAL_ENTER(ctx);
    if (!gate || !up || !out) return ctx->fail(LOKAL_ERR_BAD_ARG, "host_swiglu: null pointer");
    if (n == 0) return LOKAL_OK;
    std::lock_guard<std::mutex> g(ctx->mu);
    const size_t b = (n * 4 + 255) & ~size_t(255);
    int rc = ensure_host_scratch(ctx, 2 * b);
    if (rc == LOKAL_OK) rc = ensure_staging(ctx, 2 * b);
    if (rc != LOKAL_OK) return rc;
    cudaStream_t s = ctx->host_stream;
    char* st = static_cast<char*>(ctx->staging);
    char* d = static_cast<char*>(ctx->host_scratch);
    std::memcpy(st, gate, n * 4);
    std::memcpy(st + b, up, n * 4);
    LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(d, st, 2 * b, cudaMemcpyHostToDevice, s));
    rc = lokal::launch_swiglu(ctx, s, d, d + b, d, nullptr, n, LOKAL_F32, 0);
    if (rc != LOKAL_OK) return rc;
    LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(st, d, n * 4, cudaMemcpyDeviceToHost, s));
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(s));
    std::memcpy(out, st, n * 4);
    return LOKAL_OK;
}

int lokal_cuda_host_dequant_row(lokal_cuda_ctx* ctx, int ggml_type, const uint8_t* src, size_t src_len, float* out, size_t n) {
    LOKAL_ENTER(ctx);
    if (!src || !out) return ctx->fail(LOKAL_ERR_BAD_ARG, "host_dequant_row: null pointer");
    const size_t be = lokal_cuda_blk_elems(ggml_type);
    if (be == 0) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "host_dequant_row: ggml type %d is not a float type, a Q*_0 / Q*_K block type or an i-quant", ggml_type);
    if (n % be != 0 || src_len != lokal_cuda_row_bytes(ggml_type, n))
        return ctx->fail(LOKAL_ERR_BAD_ARG, "host_dequant_row: src/out size mismatch (%zu bytes for %zu elements of type %d)", src_len, n, ggml_type);
    if (n == 0) return LOKAL_OK;
    std::lock_guard<std::mutex> g(ctx->mu);
    const size_t sb = (src_len + 255) & ~size_t(255);
    int rc = ensure_host_scratch(ctx, sb + n * 4);
    if (rc == LOKAL_OK) rc = ensure_staging(ctx, sb > n * 4 ? sb : n * 4);
    if (rc != LOKAL_OK) return rc;
    cudaStream_t s = ctx->host_stream;
    char* d = static_cast<char*>(ctx->host_scratch);
    std::memcpy(ctx->staging, src, src_len);
    LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(d, ctx->staging, src_len, cudaMemcpyHostToDevice, s));
    rc = lokal::launch_gather(ctx, s, d, ggml_type, 1, n, nullptr, 1, d + sb, LOKAL_F32);
    if (rc != LOKAL_OK) return rc;
    LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->staging, d + sb, n * 4, cudaMemcpyDeviceToHost, s));
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(s));
    std::memcpy(out, ctx->staging, n * 4);
    return LOKAL_OK;
}

int lokal_cuda_host_embed_gather(lokal_cuda_ctx* ctx, const void* table_dev, int ggml_type, size_t vocab, size_t dim,
                                 const uint32_t* ids, size_t n, float* out) {
    LOKAL_ENTER(ctx);
    if (!table_dev || !ids || !out) return ctx->fail(LOKAL_ERR_BAD_ARG, "host_embed_gather: null pointer");
    if (n == 0) return LOKAL_OK;
    std::lock_guard<std::mutex> g(ctx->mu);
    const size_t ib = (n * 4 + 255) & ~size_t(255), ob = n * dim * 4;
    int rc = ensure_host_scratch(ctx, ib + ob);
    if (rc != LOKAL_OK) return rc;
    cudaStream_t s = ctx->host_stream;
    char* d = static_cast<char*>(ctx->host_scratch);
    // Page-locked caller buffers are reached by the copy engines directly; ordinary memory goes through pinned staging.
    if (is_pinned_host(ids)) {
        LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(d, ids, n * 4, cudaMemcpyHostToDevice, s));
    } else {
        rc = ensure_staging(ctx, ib);
        if (rc != LOKAL_OK) return rc;
        std::memcpy(ctx->staging, ids, n * 4);
        LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(d, ctx->staging, n * 4, cudaMemcpyHostToDevice, s));
    }
    rc = lokal::launch_gather(ctx, s, table_dev, ggml_type, vocab, dim, reinterpret_cast<const uint32_t*>(d), n, d + ib, LOKAL_F32);
    if (rc != LOKAL_OK) return rc;
    if (is_pinned_host(out)) {
        LOKAL_CUDA_TRY(ctx, cudaMemcpyAsync(out, d + ib, ob, cudaMemcpyDeviceToHost, s));
    } else {
        LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(s));  // the staged ids have been consumed before staging is reused
        rc = d2h_pageable(ctx, s, d + ib, reinterpret_cast<char*>(out), ob);
        if (rc != LOKAL_OK) return rc;
    }
    LOKAL_CUDA_TRY(ctx, cudaStreamSynchronize(s));
    return read_error_word(ctx, s);
}

}  // extern "C"
