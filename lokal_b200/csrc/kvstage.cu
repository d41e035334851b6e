// K/V staging: where the fresh K and V rows of a step go in the cache, and the narrowing copy that puts them there.
//
// Reference: the windowed store is a sink region (positions 0..sink pinned) followed by a ring
// (WindowCfg, slot_of: src/lowmem/mod.rs:163-193); a chunk of positions is written as at most three spans
// (write_spans: src/lowmem/forward.rs:256-271, src/gpu/metal.rs:673-691); batched decode addresses a row as
// (slot*max_seq + pos)*kv_dim (src/gpu/kernels.metal:3411-3412); values are narrowed with f32_to_f16
// (src/gpu/kernels.metal:2118). Here the cache row of every token row is computed on the device, so one launch
// covers any mix of sink rows, ring rows and wrap-around, and the same index array feeds the rope kernel's k output.
#include "common.cuh"

namespace lokal {
namespace {

__host__ __device__ inline unsigned long long slot_of(const lokal_kv_layout& w, unsigned long long p) {
    return p < w.sink ? p : w.sink_pad + (p - w.sink) % w.ring;
}

struct RowsArgs {
    lokal_kv_layout layout;
    const int32_t* positions;
    long long pos0;
    const uint32_t* slots;
    unsigned slot0;
    unsigned long long rows;
    uint32_t* out;
    unsigned* err_word;
};

// A position the cache cannot hold (negative; at or beyond max_seq in the linear layout, where it would land in the
// next slot's rows; a row index that does not fit 32 bits) gets LOKAL_KV_ROW_NONE, which every consumer of the index
// array skips, and sets an error bit that the next synchronisation reports: one bad position from a scheduler is an
// error code, never a store outside the cache.
__global__ void __launch_bounds__(256) kv_rows_kernel(const RowsArgs a) {
    pdl_sync();
    const unsigned long long r = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r >= a.rows) return;
    const long long spos = a.positions ? static_cast<long long>(a.positions[r]) : a.pos0 + static_cast<long long>(r);
    const unsigned long long pos = static_cast<unsigned long long>(spos);
    const unsigned long long slot = a.slots ? a.slots[r] : a.slot0;
    const unsigned long long row = a.layout.ring ? slot * (a.layout.sink_pad + a.layout.ring) + slot_of(a.layout, pos)
                                                 : slot * a.layout.max_seq + pos;
    const bool bad = spos < 0 || (a.layout.ring == 0 && pos >= a.layout.max_seq) || row >= LOKAL_KV_ROW_NONE;
    if (bad) atomicOr(a.err_word, kErrPosRange);
    a.out[r] = bad ? LOKAL_KV_ROW_NONE : static_cast<uint32_t>(row);
}

struct StageArgs {
    const void* src;
    void* dst;
    const uint32_t* dst_rows;
    unsigned long long rows, src_stride, dst_stride;
    unsigned width;
    int vec_ok;
};

// One warp per row. Each lane converts 8 elements per step (16 bytes of a 16-bit type, 32 of f32).
template <typename S, typename D>
__global__ void __launch_bounds__(256) kv_stage_kernel(const StageArgs a) {
    pdl_sync();
    const unsigned long long r = (static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (r >= a.rows) return;
    const unsigned lane = threadIdx.x & 31u;
    const S* src = reinterpret_cast<const S*>(a.src) + r * a.src_stride;
    const unsigned long long orow = a.dst_rows ? static_cast<unsigned long long>(__ldg(a.dst_rows + r)) : r;
    if (a.dst_rows && orow == LOKAL_KV_ROW_NONE) return;  // a position lokal_cuda_kv_rows refused: nothing is stored
    D* dst = reinterpret_cast<D*>(a.dst) + orow * a.dst_stride;
    if (a.vec_ok) {
        // Up to four steps of a row (1024 elements per warp) are loaded before the first one is converted and stored,
        // so a warp has the whole row of a usual KV width in flight at once.
        constexpr int kSteps = 4;
        constexpr int kVecs = sizeof(S) == 4 ? 2 : 1;  // 16-byte loads per lane step
        for (unsigned e0 = lane * 8; e0 < a.width; e0 += 256 * kSteps) {
            uint4 raw[kSteps][kVecs];
#pragma unroll
            for (int j = 0; j < kSteps; j++) {
                const unsigned e = e0 + j * 256;
                if (e < a.width) {
#pragma unroll
                    for (int v = 0; v < kVecs; v++) raw[j][v] = ld_stream(src + e + v * 4);
                }
            }
#pragma unroll
            for (int j = 0; j < kSteps; j++) {
                const unsigned e = e0 + j * 256;
                if (e >= a.width) break;
                float f[8];
                if constexpr (sizeof(S) == 4) {
                    float t[4];
                    unpack16<float>(raw[j][0], t);
#pragma unroll
                    for (int i = 0; i < 4; i++) f[i] = t[i];
                    unpack16<float>(raw[j][kVecs - 1], t);
#pragma unroll
                    for (int i = 0; i < 4; i++) f[4 + i] = t[i];
                } else {
                    float2 p[4];
                    unpack16p<S>(raw[j][0], p);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        f[2 * i] = p[i].x;
                        f[2 * i + 1] = p[i].y;
                    }
                }
                if constexpr (sizeof(D) == 4) {
                    const float lo[4] = {f[0], f[1], f[2], f[3]}, hi[4] = {f[4], f[5], f[6], f[7]};
                    st_stream(dst + e, pack16<float>(lo));
                    st_stream(dst + e + 4, pack16<float>(hi));
                } else {
                    st_stream(dst + e, pack16<D>(f));
                }
            }
        }
    } else {
        for (unsigned e = lane; e < a.width; e += 32) dst[e] = from_f32<D>(to_f32<S>(src[e]));
    }
}

template <typename S>
int stage_dst(lokal_cuda_ctx* ctx, cudaStream_t s, const StageArgs& a, int dst_dtype, unsigned grid) {
    switch (dst_dtype) {
        case LOKAL_F32: launch_k(kv_stage_kernel<S, float>, grid, 256, 0, s, a); break;
        case LOKAL_F16: launch_k(kv_stage_kernel<S, __half>, grid, 256, 0, s, a); break;
        default: launch_k(kv_stage_kernel<S, __nv_bfloat16>, grid, 256, 0, s, a); break;
    }
    LOKAL_CHECK_LAUNCH(ctx, "kv_stage_kernel");
    return LOKAL_OK;
}

}  // namespace
}  // namespace lokal

extern "C" {

int lokal_cuda_window_cfg(uint64_t window, uint64_t sink, uint64_t prefill_chunk, lokal_kv_layout* out) {
    if (!out || window == 0 || sink > window) return LOKAL_ERR_BAD_ARG;  // the reference's "invalid window config"
    auto up128 = [](uint64_t v) { return (v + 127) / 128 * 128; };
    out->max_seq = 0;
    out->sink = sink;
    out->sink_pad = up128(sink);
    out->ring = up128(window + prefill_chunk);
    return LOKAL_OK;
}

uint64_t lokal_cuda_window_slot_of(const lokal_kv_layout* layout, uint64_t p) {
    if (!layout || layout->ring == 0) return p;
    return lokal::slot_of(*layout, p);
}

int lokal_cuda_window_write_spans(const lokal_kv_layout* w, uint64_t pos0, uint64_t n, uint64_t* spans) {
    if (!w || !spans || w->ring == 0) return -1;
    const uint64_t end = pos0 + n;
    int count = 0;
    if (pos0 < w->sink && n) {
        const uint64_t stop = w->sink < end ? w->sink : end;
        spans[0] = 0;
        spans[1] = pos0;
        spans[2] = stop - pos0;
        count = 1;
    }
    uint64_t p = pos0 > w->sink ? pos0 : w->sink;
    while (p < end && count < 3) {
        const uint64_t rel = (p - w->sink) % w->ring;
        const uint64_t room = w->ring - rel, left = end - p;
        const uint64_t len = room < left ? room : left;
        spans[3 * count + 0] = p - pos0;
        spans[3 * count + 1] = w->sink_pad + rel;
        spans[3 * count + 2] = len;
        count++;
        p += len;
    }
    return p < end ? -1 : count;  // more than one wrap does not fit the reference's three spans (chunk > ring)
}

int lokal_cuda_kv_rows(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const lokal_kv_layout* layout, const int32_t* positions,
                       int64_t pos0, const uint32_t* slots, uint32_t slot0, size_t rows, uint32_t* rows_out) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    lokal::DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!layout || !rows_out) return ctx->fail(LOKAL_ERR_BAD_ARG, "kv_rows: layout and output must be non-null");
    if (layout->ring == 0 && layout->max_seq == 0) return ctx->fail(LOKAL_ERR_BAD_ARG, "kv_rows: linear layout needs max_seq");
    if (layout->ring != 0 && layout->sink_pad < layout->sink) return ctx->fail(LOKAL_ERR_BAD_ARG, "kv_rows: sink_pad is smaller than sink");
    if (!positions && pos0 < 0) return ctx->fail(LOKAL_ERR_BAD_ARG, "kv_rows: pos0 is negative");
    if (!lokal::aligned_to(rows_out, 4) || (positions && !lokal::aligned_to(positions, 4)) || (slots && !lokal::aligned_to(slots, 4)))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "kv_rows: a pointer is not 4-byte aligned");
    if (rows == 0) return LOKAL_OK;
    lokal::RowsArgs a{*layout, positions, pos0, slots, slot0, rows, rows_out, ctx->err_word};
    const unsigned long long blocks = (rows + 255) / 256;
    if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "kv_rows: too many rows for one launch");
    lokal::launch_k(lokal::kv_rows_kernel, static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(s), a);
    LOKAL_CHECK_LAUNCH(ctx, "kv_rows_kernel");
    return LOKAL_OK;
}

int lokal_cuda_kv_stage(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* src, int src_dtype, size_t src_row_stride,
                        void* dst, int dst_dtype, size_t dst_row_stride, const uint32_t* dst_rows, size_t rows, size_t width) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    lokal::DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!src || !dst) return ctx->fail(LOKAL_ERR_BAD_ARG, "kv_stage: src and dst must be non-null");
    if (!lokal::is_act_type(src_dtype) || !lokal::is_act_type(dst_dtype))
        return ctx->fail(LOKAL_ERR_UNSUPPORTED, "kv_stage: types %d -> %d are not F32/F16/BF16", src_dtype, dst_dtype);
    if (width == 0 || width > 0x7fffffffu) return ctx->fail(LOKAL_ERR_BAD_ARG, "kv_stage: width %zu out of range", width);
    if (src_row_stride < width || dst_row_stride < width) return ctx->fail(LOKAL_ERR_BAD_ARG, "kv_stage: a row stride is smaller than the width");
    const size_t ss = lokal::type_size(src_dtype), ds = lokal::type_size(dst_dtype);
    if (!lokal::aligned_to(src, ss) || !lokal::aligned_to(dst, ds) || (dst_rows && !lokal::aligned_to(dst_rows, 4)))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "kv_stage: a pointer is not aligned to its element size");
    if (rows == 0) return LOKAL_OK;
    lokal::StageArgs a{};
    a.src = src;
    a.dst = dst;
    a.dst_rows = dst_rows;
    a.rows = rows;
    a.src_stride = src_row_stride;
    a.dst_stride = dst_row_stride;
    a.width = static_cast<unsigned>(width);
    // 8 elements per lane step: 16-byte accesses on a 16-bit side, two of them on an f32 side
    a.vec_ok = width % 8 == 0 && lokal::aligned_to(src, 16) && lokal::aligned_to(dst, 16) && (src_row_stride * ss) % 16 == 0 &&
               (dst_row_stride * ds) % 16 == 0;
    const unsigned long long blocks = (rows + 7) / 8;
    if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "kv_stage: too many rows for one launch");
    const unsigned grid = static_cast<unsigned>(blocks);
    cudaStream_t st = static_cast<cudaStream_t>(s);
    switch (src_dtype) {
        case LOKAL_F32: return lokal::stage_dst<float>(ctx, st, a, dst_dtype, grid);
        case LOKAL_F16: return lokal::stage_dst<__half>(ctx, st, a, dst_dtype, grid);
        default: return lokal::stage_dst<__nv_bfloat16>(ctx, st, a, dst_dtype, grid);
    }
}

}  // extern "C"
