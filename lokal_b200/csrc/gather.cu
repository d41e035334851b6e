// Token-embedding gather with on-the-fly GGUF row dequantisation.
//
// Reference semantics: LowMemSession::embed_gather (src/lowmem/forward.rs:275-307)
// walks the ids, slices row id out of the table bytes (read_rows,
// src/lowmem/mod.rs:654-668) and expands it with gguf::dequant_row_ref
// (src/gguf/dequant.rs:191-239 F32/F16/Q8_0, :462-483 Q4_K, scale unpack
// :141-150). Results here are bit-identical to that: int -> f32 and f16 -> f32
// conversions are exact, and the Q4_K value d1*q - m1 is computed with
// __fmul_rn / __fsub_rn so the two products and the subtraction are each
// rounded once and never contracted into an FMA.
//
// Kernel shape (quantised tables): one warp per token row, persistent over a
// grid-stride list of rows. Lane 0 stages the raw row into shared memory with
// one bulk asynchronous copy (cp.async.bulk, completion on an mbarrier) while
// the warp decodes the previous row: a two-stage ring per warp. Q8_0 rows are
// a multiple of 34 bytes, so a row start is only 2-byte aligned; the copy
// fetches the enclosing 16-byte-aligned window and the decode indexes from the
// remainder. Each lane then produces 16 bytes of output per step (4 f32 or
// 8 f16/bf16), so every store instruction of a warp writes one 512-byte run.
// HBM traffic per token: row_bytes for the first touch of a row (hot rows hit
// L2) plus dim*sizeof(out) written.
//
// Every wait on an mbarrier is bounded: after the limit the warp records
// kErrTimeout in the context's error word and leaves.
#include "common.cuh"

namespace lokal {
namespace {

struct GatherArgs {
    const unsigned char* table;
    const uint32_t* ids;  // null -> row i
    void* out;
    unsigned long long n;
    unsigned long long vocab;
    unsigned long long table_bytes;
    unsigned dim;
    unsigned row_bytes;
    unsigned stage_bytes;  // per warp per stage, multiple of 16
    unsigned* err_word;
};

// ---- block decoders: EPL consecutive elements starting at element e (e % EPL == 0) ----

// Q8_0 (src/gguf/dequant.rs:231-239): 34-byte block = f16 d, then 32 int8; y = q * d.
template <int EPL>
__device__ __forceinline__ void decode_q8_0(const unsigned char* row, unsigned e, float (&y)[EPL]) {
    const unsigned char* b = row + (e >> 5) * 34;
    const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(b)));
    const unsigned short* q = reinterpret_cast<const unsigned short*>(b + 2 + (e & 31));
#pragma unroll
    for (int j = 0; j < EPL / 2; j++) {
        const unsigned short two = q[j];
        const int q0 = static_cast<int>(static_cast<signed char>(two & 0xFF));
        const int q1 = static_cast<int>(static_cast<signed char>(two >> 8));
        y[2 * j] = __fmul_rn(static_cast<float>(q0), d);
        y[2 * j + 1] = __fmul_rn(static_cast<float>(q1), d);
    }
}

// Q4_K (src/gguf/dequant.rs:462-483): 144-byte super-block = f16 d, f16 dmin,
// 12 bytes of packed 6-bit scales/mins, 128 bytes of nibbles. For group j of
// 32 elements: y = (d * sc_j) * q - (dmin * m_j), products and difference each
// rounded to f32.
template <int EPL>
__device__ __forceinline__ void decode_q4_k(const unsigned char* row, unsigned e, float (&y)[EPL]) {
    const unsigned char* b = row + (e >> 8) * 144;
    const unsigned ib = e & 255;
    const unsigned dd = *reinterpret_cast<const unsigned*>(b);
    const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(dd & 0xFFFF)));
    const float dmin = __half2float(__ushort_as_half(static_cast<unsigned short>(dd >> 16)));
    const unsigned char* sb = b + 4;
    const unsigned j = ib >> 5;
    unsigned sc, mn;
    if (j < 4) {
        sc = sb[j] & 63u;
        mn = sb[j + 4] & 63u;
    } else {
        sc = (sb[j + 4] & 0x0Fu) | ((static_cast<unsigned>(sb[j - 4]) >> 6) << 4);
        mn = (static_cast<unsigned>(sb[j + 4]) >> 4) | ((static_cast<unsigned>(sb[j]) >> 6) << 4);
    }
    const float d1 = __fmul_rn(d, static_cast<float>(sc));
    const float m1 = __fmul_rn(dmin, static_cast<float>(mn));
    const unsigned char* qs = b + 16 + (ib >> 6) * 32 + (ib & 31);
    const unsigned shift = (ib & 32) ? 4u : 0u;
#pragma unroll
    for (int w = 0; w < EPL / 4; w++) {
        const unsigned four = reinterpret_cast<const unsigned*>(qs)[w];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const unsigned q = ((four >> (8 * k)) >> shift) & 0xFu;
            y[4 * w + k] = __fsub_rn(__fmul_rn(d1, static_cast<float>(q)), m1);
        }
    }
}

template <int QT, int EPL>
__device__ __forceinline__ void decode_block(const unsigned char* row, unsigned e, float (&y)[EPL]) {
    if (QT == LOKAL_Q8_0) decode_q8_0<EPL>(row, e, y);
    else decode_q4_k<EPL>(row, e, y);
}

template <typename OutT>
__device__ __forceinline__ void store_out16(OutT* dst, const float (&y)[VecOf<OutT>::N]) {
    st_stream(dst, pack16<OutT>(y));
}

// ---- staged (bulk-copy) kernel for quantised tables ----

template <int QT, typename OutT>
__global__ void __launch_bounds__(256) gather_quant_staged_kernel(const GatherArgs a) {
    pdl_sync();
    constexpr int EPL = VecOf<OutT>::N;
    extern __shared__ __align__(128) unsigned char smem[];
    const unsigned warps_per_cta = blockDim.x >> 5;
    const unsigned warp_in_cta = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem);
    unsigned char* stage0 = smem + ((warps_per_cta * 2 * 8 + 127u) & ~127u) + warp_in_cta * 2 * a.stage_bytes;
    const uint32_t bar0 = smem_addr(&bars[warp_in_cta * 2]);
    if (lane == 0) {
        mbar_init(bar0, 1);
        mbar_init(bar0 + 8, 1);
        mbar_init_fence();
    }
    __syncwarp();

    const unsigned long long total_warps = static_cast<unsigned long long>(gridDim.x) * warps_per_cta;
    const unsigned long long first = static_cast<unsigned long long>(blockIdx.x) * warps_per_cta + warp_in_cta;

    // Ring state of the two stages, kept in one register (uniform across the warp):
    //   bits 2s..2s+1  mode of stage s: 0 = row invalid (zero fill), 1 = bulk copy issued,
    //                  2 = bytes already placed by plain loads
    //   bit  4+s       mbarrier phase parity of stage s
    //   bits 8+4s..    offset of the row start inside the 16-byte-aligned window
    unsigned state = 0;
    auto set_stage = [&](unsigned s, unsigned mode, unsigned off) {
        state = (state & ~((3u << (2 * s)) | (15u << (8 + 4 * s)))) | (mode << (2 * s)) | (off << (8 + 4 * s));
    };
    auto mode_of = [&](unsigned s) { return (state >> (2 * s)) & 3u; };
    auto stage_ptr = [&](unsigned s) { return stage0 + s * a.stage_bytes; };

    auto issue = [&](unsigned long long i, unsigned s) {
        const unsigned long long id = a.ids ? static_cast<unsigned long long>(__ldg(a.ids + i)) : i;
        if (id >= a.vocab) {
            set_stage(s, 0, 0);
            if (lane == 0) atomicOr(a.err_word, kErrIdRange);
            return;
        }
        const unsigned long long start = id * a.row_bytes;
        const unsigned long long w0 = start & ~15ull;
        const unsigned long long w1 = (start + a.row_bytes + 15ull) & ~15ull;
        const unsigned off = static_cast<unsigned>(start - w0);
        if (w1 <= a.table_bytes) {
            set_stage(s, 1, off);
            if (lane == 0) {
                const unsigned bytes = static_cast<unsigned>(w1 - w0);
                mbar_expect_tx(bar0 + 8 * s, bytes);
                bulk_copy_g2s(smem_addr(stage_ptr(s)), a.table + w0, bytes, bar0 + 8 * s);
            }
        } else {
            // The window would run past the end of the table (last row only): plain byte loads.
            set_stage(s, 2, off);
            unsigned char* dst = stage_ptr(s) + off;
            for (unsigned bidx = lane; bidx < a.row_bytes; bidx += 32) dst[bidx] = __ldg(a.table + start + bidx);
        }
    };

    if (first < a.n) issue(first, 0);
    unsigned it = 0;
    for (unsigned long long i = first; i < a.n; i += total_warps, it++) {
        const unsigned s = it & 1u;
        const unsigned long long nxt = i + total_warps;
        if (nxt < a.n) issue(nxt, s ^ 1u);
        else set_stage(s ^ 1u, 0, 0);
        OutT* orow = reinterpret_cast<OutT*>(a.out) + i * a.dim;
        const unsigned mode = mode_of(s);
        if (mode == 1) {
            const unsigned parity = (state >> (4 + s)) & 1u;
            if (!mbar_wait_bounded(bar0 + 8 * s, parity)) {
                if (lane == 0) atomicOr(a.err_word, kErrTimeout);
                // give the copies still in flight one more bounded chance to land before leaving
                mbar_wait_bounded(bar0 + 8 * s, parity);
                if (mode_of(s ^ 1u) == 1) mbar_wait_bounded(bar0 + 8 * (s ^ 1u), (state >> (4 + (s ^ 1u))) & 1u);
                return;
            }
            state ^= 1u << (4 + s);
        } else if (mode == 2) {
            __syncwarp();
        }
        if (mode == 0) {
            float z[EPL];
#pragma unroll
            for (int k = 0; k < EPL; k++) z[k] = 0.0f;
            for (unsigned e = lane * EPL; e < a.dim; e += 32 * EPL) store_out16<OutT>(orow + e, z);
        } else {
            const unsigned char* row = stage_ptr(s) + ((state >> (8 + 4 * s)) & 15u);
            for (unsigned e = lane * EPL; e < a.dim; e += 32 * EPL) {
                float y[EPL];
                decode_block<QT, EPL>(row, e, y);
                store_out16<OutT>(orow + e, y);
            }
        }
        __syncwarp();  // every lane is done with stage s before it is refilled
    }
}

// ---- plain kernel for quantised tables: any alignment, any row size ----
// One warp per row, one element per lane step, byte loads straight from global
// memory (the per-element index form of src/gpu/kernels.metal:77-81, 889-904).
__device__ __forceinline__ float dequant_elem_global(int qt, const unsigned char* row, unsigned col) {
    if (qt == LOKAL_Q8_0) {
        const unsigned char* b = row + (col >> 5) * 34;
        const unsigned short hb = static_cast<unsigned short>(__ldg(b) | (__ldg(b + 1) << 8));
        const float d = __half2float(__ushort_as_half(hb));
        const int q = static_cast<int>(static_cast<signed char>(__ldg(b + 2 + (col & 31))));
        return __fmul_rn(static_cast<float>(q), d);
    }
    const unsigned char* b = row + (col >> 8) * 144;
    const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(__ldg(b) | (__ldg(b + 1) << 8))));
    const float dmin = __half2float(__ushort_as_half(static_cast<unsigned short>(__ldg(b + 2) | (__ldg(b + 3) << 8))));
    const unsigned char* sb = b + 4;
    const unsigned ib = col & 255, j = ib >> 5;
    unsigned sc, mn;
    if (j < 4) {
        sc = __ldg(sb + j) & 63u;
        mn = __ldg(sb + j + 4) & 63u;
    } else {
        sc = (__ldg(sb + j + 4) & 0x0Fu) | ((static_cast<unsigned>(__ldg(sb + j - 4)) >> 6) << 4);
        mn = (static_cast<unsigned>(__ldg(sb + j + 4)) >> 4) | ((static_cast<unsigned>(__ldg(sb + j)) >> 6) << 4);
    }
    const float d1 = __fmul_rn(d, static_cast<float>(sc));
    const float m1 = __fmul_rn(dmin, static_cast<float>(mn));
    const unsigned byte = __ldg(b + 16 + (ib >> 6) * 32 + (ib & 31));
    const unsigned q = (ib & 32) ? (byte >> 4) : (byte & 0xFu);
    return __fsub_rn(__fmul_rn(d1, static_cast<float>(q)), m1);
}

template <typename OutT>
__global__ void __launch_bounds__(256) gather_quant_plain_kernel(const GatherArgs a, int qt) {
    pdl_sync();
    const unsigned long long i = (static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (i >= a.n) return;
    const unsigned lane = threadIdx.x & 31u;
    const unsigned long long id = a.ids ? static_cast<unsigned long long>(__ldg(a.ids + i)) : i;
    OutT* orow = reinterpret_cast<OutT*>(a.out) + i * a.dim;
    if (id >= a.vocab) {
        if (lane == 0) atomicOr(a.err_word, kErrIdRange);
        for (unsigned e = lane; e < a.dim; e += 32) orow[e] = from_f32<OutT>(0.0f);
        return;
    }
    const unsigned char* row = a.table + id * a.row_bytes;
    for (unsigned e = lane; e < a.dim; e += 32) orow[e] = from_f32<OutT>(dequant_elem_global(qt, row, e));
}

// ---- float tables (F32 / F16 / BF16): copy or widen/narrow a row ----
template <typename SrcT, typename OutT>
__global__ void __launch_bounds__(256) gather_float_kernel(const GatherArgs a, int vec_ok) {
    pdl_sync();
    constexpr int N = VecOf<SrcT>::N;  // elements per 16-byte source vector
    const unsigned long long i = (static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (i >= a.n) return;
    const unsigned lane = threadIdx.x & 31u;
    const unsigned long long id = a.ids ? static_cast<unsigned long long>(__ldg(a.ids + i)) : i;
    OutT* orow = reinterpret_cast<OutT*>(a.out) + i * a.dim;
    const bool valid = id < a.vocab;
    if (!valid && lane == 0) atomicOr(a.err_word, kErrIdRange);
    const SrcT* row = reinterpret_cast<const SrcT*>(a.table) + (valid ? id : 0) * a.dim;
    if (vec_ok) {
        for (unsigned e = lane * N; e < a.dim; e += 32 * N) {
            float f[N];
            if (valid) unpack16<SrcT>(ld_keep(row + e), f);
            else {
#pragma unroll
                for (int k = 0; k < N; k++) f[k] = 0.0f;
            }
            constexpr int ON = VecOf<OutT>::N;
            if (ON == N) {
                float g[ON];
#pragma unroll
                for (int k = 0; k < ON; k++) g[k] = f[k % N];
                st_stream(orow + e, pack16<OutT>(g));
            } else if (ON < N) {  // 16-bit source, f32 out: two 16-byte stores
#pragma unroll
                for (int h = 0; h < N / ON; h++) {
                    float g[ON];
#pragma unroll
                    for (int k = 0; k < ON; k++) g[k] = f[(h * ON + k) % N];
                    st_stream(orow + e + h * ON, pack16<OutT>(g));
                }
            } else {  // f32 source, 16-bit out: 4 elements = 8 bytes
#pragma unroll
                for (int k = 0; k < N; k++) orow[e + k] = from_f32<OutT>(f[k]);
            }
        }
    } else {
        for (unsigned e = lane; e < a.dim; e += 32) orow[e] = from_f32<OutT>(valid ? to_f32<SrcT>(row[e]) : 0.0f);
    }
}

template <typename OutT>
int launch_out(lokal_cuda_ctx* ctx, cudaStream_t s, GatherArgs a, int ggml_type, bool aligned) {
    const unsigned long long row_warps_blocks = (a.n + 7) / 8;
    if (row_warps_blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather: too many rows for one launch");
    if (ggml_type == LOKAL_F32 || ggml_type == LOKAL_F16 || ggml_type == LOKAL_BF16) {
        const size_t ses = type_size(ggml_type);
        const int vec_ok = aligned && (static_cast<size_t>(a.dim) * ses) % 16 == 0 &&
                           (static_cast<size_t>(a.dim) * sizeof(OutT)) % 16 == 0;
        const unsigned grid = static_cast<unsigned>(row_warps_blocks);
        if (ggml_type == LOKAL_F32) launch_k(gather_float_kernel<float, OutT>, grid, 256, 0, s, a, vec_ok);
        else if (ggml_type == LOKAL_F16) launch_k(gather_float_kernel<__half, OutT>, grid, 256, 0, s, a, vec_ok);
        else launch_k(gather_float_kernel<__nv_bfloat16, OutT>, grid, 256, 0, s, a, vec_ok);
        LOKAL_CHECK_LAUNCH(ctx, "gather_float_kernel");
        return LOKAL_OK;
    }
    // quantised table
    const unsigned warps = 8;
    a.stage_bytes = ((a.row_bytes + 15u) & ~15u) + 32u;
    const size_t smem = ((warps * 2 * 8 + 127u) & ~127u) + static_cast<size_t>(warps) * 2 * a.stage_bytes;
    const bool staged = aligned && smem <= 200u * 1024u && (a.row_bytes % 2 == 0);
    if (!staged) {
        launch_k(gather_quant_plain_kernel<OutT>, static_cast<unsigned>(row_warps_blocks), 256, 0, s, a, ggml_type);
        LOKAL_CHECK_LAUNCH(ctx, "gather_quant_plain_kernel");
        return LOKAL_OK;
    }
    auto kern = ggml_type == LOKAL_Q8_0 ? gather_quant_staged_kernel<LOKAL_Q8_0, OutT> : gather_quant_staged_kernel<LOKAL_Q4_K, OutT>;
    if (smem > 48u * 1024u) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return ctx->fail(LOKAL_ERR_CUDA, "embed_gather: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    // Persistent grid: as many CTAs as stay resident (8 x 256 threads per SM, or what shared memory allows).
    unsigned per_sm = static_cast<unsigned>((220u * 1024u) / (smem + 1024u));
    if (per_sm > 8) per_sm = 8;
    if (per_sm < 1) per_sm = 1;
    unsigned long long grid = static_cast<unsigned long long>(ctx->sm_count) * per_sm;
    if (grid > row_warps_blocks) grid = row_warps_blocks;
    launch_k(kern, static_cast<unsigned>(grid), warps * 32, smem, s, a);
    LOKAL_CHECK_LAUNCH(ctx, "gather_quant_staged_kernel");
    return LOKAL_OK;
}

}  // namespace

int launch_gather(lokal_cuda_ctx* ctx, cudaStream_t s, const void* table, int ggml_type, size_t vocab, size_t dim,
                  const uint32_t* ids, size_t n, void* out, int out_dtype) {
    if (!table || !out) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather: table and out must be non-null");
    const size_t be = lokal_cuda_blk_elems(ggml_type);
    if (be == 0) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "embed_gather: ggml type %d is not F32/F16/BF16/Q8_0/Q4_K", ggml_type);
    if (!is_act_type(out_dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "embed_gather: output type %d is not F32/F16/BF16", out_dtype);
    if (dim == 0 || dim > 0x7fffffffu) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather: dim %zu out of range", dim);
    if (dim % be != 0)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather: dim %zu is not a whole number of %zu-element blocks", dim, be);
    if (vocab == 0) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather: table has no rows");
    if (ids && !aligned_to(ids, 4)) return ctx->fail(LOKAL_ERR_MISALIGNED, "embed_gather: ids are not 4-byte aligned");
    if (!aligned_to(out, type_size(out_dtype))) return ctx->fail(LOKAL_ERR_MISALIGNED, "embed_gather: out is not aligned to its element size");
    if ((ggml_type == LOKAL_F32 && !aligned_to(table, 4)) || ((ggml_type == LOKAL_F16 || ggml_type == LOKAL_BF16) && !aligned_to(table, 2)))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "embed_gather: table is not aligned to its element size");
    const size_t rb = lokal_cuda_row_bytes(ggml_type, dim);
    if (rb > 0xffffffffu) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather: row of %zu bytes is too large", rb);
    if (n == 0) return LOKAL_OK;
    GatherArgs a{};
    a.table = static_cast<const unsigned char*>(table);
    a.ids = ids;
    a.out = out;
    a.n = n;
    a.vocab = vocab;
    a.table_bytes = static_cast<unsigned long long>(vocab) * rb;
    a.dim = static_cast<unsigned>(dim);
    a.row_bytes = static_cast<unsigned>(rb);
    a.err_word = ctx->err_word;
    const bool aligned = aligned_to(table, 16) && aligned_to(out, 16) && (dim * type_size(out_dtype)) % 16 == 0;
    switch (out_dtype) {
        case LOKAL_F32: return launch_out<float>(ctx, s, a, ggml_type, aligned);
        case LOKAL_F16: return launch_out<__half>(ctx, s, a, ggml_type, aligned);
        default: return launch_out<__nv_bfloat16>(ctx, s, a, ggml_type, aligned);
    }
}

}  // namespace lokal
