/*
 * lokal_cuda.h -- C ABI of the B200 (sm_100a) implementation of lokal's fused
 * per-token layer ops: residual-add + RMSNorm (incl. per-head qk-norm), RoPE of
 * q/k with the bias fold, SiLU(gate)*up, and embedding gather with GGUF row
 * dequantisation (every block type the reference decodes) -- plus the steps
 * either side of that path: K/V staging into the cache, the gated-deltanet
 * per-row ops, and a GGUF container reader.
 *
 * This is the boundary a `-b cuda` backend of the reference binds through FFI:
 * plain pointers and sizes, no C++ or framework types. Each entry point names
 * the reference interface it stands in for (paths are within the reference
 * project).
 *
 * Conventions
 *   - Every function returns a lokal_status (0 = ok). On failure the context
 *     keeps a message readable with lokal_cuda_last_error().
 *   - Ops take DEVICE pointers and are asynchronous on the given stream (NULL =
 *     the legacy default stream), the way the reference encodes a whole step
 *     and waits once (src/gpu/metal.rs:2679-2681). lokal_cuda_stream_sync is
 *     the blocking call. The lokal_cuda_host_* functions take HOST slices,
 *     mirror the CPU signatures in src/math.rs / src/model.rs / src/gguf, and
 *     block until the result is in the caller's buffer.
 *   - Unsupported cases are refused by name with an error code; there is no
 *     CPU fallback anywhere in this library.
 *   - Element types use the on-disk GGUF ids (src/gguf/dequant.rs:21-41), for
 *     activations as well as for tables.
 *   - eps and theta are f32, as in the reference config (src/config.rs:19-21).
 *   - Head geometry is always passed explicitly (n_heads, head_dim, rot_dim),
 *     never derived from the hidden size (src/lowmem/mod.rs:62-101).
 */
#ifndef LOKAL_CUDA_H
#define LOKAL_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define LOKAL_API __attribute__((visibility("default")))
#else
#define LOKAL_API
#endif

typedef enum lokal_status {
    LOKAL_OK = 0,
    LOKAL_ERR_BAD_ARG = 1,     /* null pointer, zero/odd dimension, inconsistent sizes */
    LOKAL_ERR_UNSUPPORTED = 2, /* element type or combination this path does not cover */
    LOKAL_ERR_MISALIGNED = 3,  /* pointer not aligned to its element size */
    LOKAL_ERR_CUDA = 4,        /* a CUDA runtime call failed; message has the detail */
    LOKAL_ERR_ID_RANGE = 5,    /* a token id was >= vocab (row zero-filled on the device) */
    LOKAL_ERR_TIMEOUT = 6,     /* a bounded device-side wait gave up */
    LOKAL_ERR_NO_DEVICE = 7,   /* no usable CUDA device */
    LOKAL_ERR_IO = 8,          /* a file could not be opened or mapped */
    LOKAL_ERR_FORMAT = 9,      /* a GGUF file is malformed, truncated or of an unsupported version */
    LOKAL_ERR_NOT_FOUND = 10,  /* a tensor name or metadata key is not in the file */
    LOKAL_ERR_POS_RANGE = 11   /* a position was negative or beyond the KV cache (its row was not stored) */
} lokal_status;

/* GGUF tensor type ids (src/gguf/dequant.rs:21-41; BF16 = 30 per ggml.h).
 * F32/F16/BF16 are the activation and weight-vector types of every op; all of
 * them are table types of embed_gather / dequant_rows (block sizes
 * src/gguf/dequant.rs:94-114). The codebook types (IQ1_S .. IQ3_S) decode once the
 * caller has handed over their codebooks (lokal_cuda_set_iq_grid). Q4_1, Q5_1 and the
 * activation-only Q8_1/Q8_K are not covered: LOKAL_ERR_UNSUPPORTED, as in the reference. */
typedef enum lokal_type {
    LOKAL_F32 = 0,
    LOKAL_F16 = 1,
    LOKAL_Q4_0 = 2,
    LOKAL_Q5_0 = 6,
    LOKAL_Q8_0 = 8,
    LOKAL_Q2_K = 10,
    LOKAL_Q3_K = 11,
    LOKAL_Q4_K = 12,
    LOKAL_Q5_K = 13,
    LOKAL_Q6_K = 14,
    LOKAL_IQ2_XXS = 16,
    LOKAL_IQ2_XS = 17,
    LOKAL_IQ3_XXS = 18,
    LOKAL_IQ1_S = 19,
    LOKAL_IQ4_NL = 20,
    LOKAL_IQ3_S = 21,
    LOKAL_IQ2_S = 22,
    LOKAL_IQ4_XS = 23,
    LOKAL_IQ1_M = 29,
    LOKAL_BF16 = 30
} lokal_type;

typedef struct lokal_cuda_ctx lokal_cuda_ctx; /* one per device; thread-safe after creation */
typedef void* lokal_cuda_stream;              /* a cudaStream_t */
typedef struct lokal_cuda_graph lokal_cuda_graph;

/* ---- context, memory, streams --------------------------------------------
 * Stand in for engine creation on the backend seam (src/engine.rs:76-111,
 * checklist src/gpu/mod.rs:3-13): weights resident, one submission per step. */
LOKAL_API int lokal_cuda_create(int device, lokal_cuda_ctx** out);
LOKAL_API void lokal_cuda_destroy(lokal_cuda_ctx* ctx);
LOKAL_API const char* lokal_cuda_last_error(const lokal_cuda_ctx* ctx);
LOKAL_API const char* lokal_cuda_version(void);
LOKAL_API int lokal_cuda_device_count(void);

LOKAL_API int lokal_cuda_malloc(lokal_cuda_ctx* ctx, size_t bytes, void** dptr);
LOKAL_API int lokal_cuda_free(lokal_cuda_ctx* ctx, void* dptr);
LOKAL_API int lokal_cuda_host_alloc(lokal_cuda_ctx* ctx, size_t bytes, void** hptr); /* pinned */
LOKAL_API int lokal_cuda_host_free(lokal_cuda_ctx* ctx, void* hptr);
LOKAL_API int lokal_cuda_memcpy_h2d(lokal_cuda_ctx* ctx, lokal_cuda_stream s, void* dst, const void* src, size_t bytes);
LOKAL_API int lokal_cuda_memcpy_d2h(lokal_cuda_ctx* ctx, lokal_cuda_stream s, void* dst, const void* src, size_t bytes);
LOKAL_API int lokal_cuda_stream_create(lokal_cuda_ctx* ctx, lokal_cuda_stream* out);
LOKAL_API int lokal_cuda_stream_destroy(lokal_cuda_ctx* ctx, lokal_cuda_stream s);
/* Blocks until the stream drains, then reports (and clears) any device-side
 * error word: LOKAL_ERR_ID_RANGE / LOKAL_ERR_TIMEOUT (cf. the command-buffer
 * status check of src/lowmem/pool.rs:1291-1320). */
LOKAL_API int lokal_cuda_stream_sync(lokal_cuda_ctx* ctx, lokal_cuda_stream s);

/* Capture every op issued on `s` between begin and end into one replayable
 * submission ("encode everything, submit once", src/gpu/metal.rs:2517, 2679). */
LOKAL_API int lokal_cuda_graph_begin(lokal_cuda_ctx* ctx, lokal_cuda_stream s);
LOKAL_API int lokal_cuda_graph_end(lokal_cuda_ctx* ctx, lokal_cuda_stream s, lokal_cuda_graph** out);
LOKAL_API int lokal_cuda_graph_launch(lokal_cuda_ctx* ctx, lokal_cuda_graph* g, lokal_cuda_stream s);
LOKAL_API int lokal_cuda_graph_destroy(lokal_cuda_ctx* ctx, lokal_cuda_graph* g);

/* ---- GGUF block geometry: GgmlType::{blk_elems, blk_bytes, row_bytes}
 * (src/gguf/dequant.rs:81-119). Return 0 for a type outside this path. */
LOKAL_API size_t lokal_cuda_blk_elems(int ggml_type);
LOKAL_API size_t lokal_cuda_blk_bytes(int ggml_type);
LOKAL_API size_t lokal_cuda_row_bytes(int ggml_type, size_t n);

/* The i-quant codebooks (src/lowmem/iq_grids.rs: iq2xxs_grid ... iq1s_grid of ggml-common.h).
 * They are fitted tables of the file format, not formulas, and this library does not carry
 * them: the host application uploads its own copy once per context. Until then a table of the
 * corresponding type is refused with LOKAL_ERR_UNSUPPORTED. ksigns_iq2xs / kmask_iq2xs are
 * derivable (7 bits + even parity; powers of two) and are computed.
 *   which                entries     used by
 *   LOKAL_GRID_IQ2XXS    256 x u64   IQ2_XXS
 *   LOKAL_GRID_IQ2XS     512 x u64   IQ2_XS
 *   LOKAL_GRID_IQ2S     1024 x u64   IQ2_S
 *   LOKAL_GRID_IQ3XXS    256 x u32   IQ3_XXS
 *   LOKAL_GRID_IQ3S      512 x u32   IQ3_S
 *   LOKAL_GRID_IQ1S     2048 x u64   IQ1_S, IQ1_M
 * `table` is a host pointer, `bytes` must be entries x entry size. Blocking. */
typedef enum lokal_iq_grid {
    LOKAL_GRID_IQ2XXS = 0, LOKAL_GRID_IQ2XS = 1, LOKAL_GRID_IQ2S = 2, LOKAL_GRID_IQ3XXS = 3, LOKAL_GRID_IQ3S = 4, LOKAL_GRID_IQ1S = 5
} lokal_iq_grid;
LOKAL_API int lokal_cuda_set_iq_grid(lokal_cuda_ctx* ctx, int which, const void* table, size_t bytes);

/* ---- RMSNorm --------------------------------------------------------------
 * math::rmsnorm (src/math.rs:45-49) over `rows` rows of `dim`; GPU twins
 * rmsnorm / rmsnorm_hf (src/gpu/kernels.metal:2262, 2341), host encoders
 * enc_rmsnorm / enc_rmsnorm_dim / enc_rmsnorm_hf (src/gpu/metal.rs:1181-1256),
 * NormParams{dim, eps} (src/gpu/metal.rs:90-93).
 *   y[r][i] = (x[r][i] * scale_r) * w[i],  scale_r = 1 / sqrt(mean(x_r^2) + eps)
 * x, y: `dtype` (F32 / F16 / BF16; math in f32, one rounding on store). y may
 * alias x. w: `w_dtype`, `dim` entries. y_h: optional second copy of y in
 * `h_dtype` (F16 or BF16), only with dtype F32; NULL to skip. */
LOKAL_API int lokal_cuda_rmsnorm(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* x, const void* w, void* y,
                                 void* y_h, size_t rows, size_t dim, float eps, int dtype, int w_dtype, int h_dtype);

/* Residual add (src/model.rs:235-237, 253-255; GPU twin add_inplace,
 * src/gpu/kernels.metal:3591) fused with the RMSNorm that follows it:
 *   x[r] += delta[r]   (in place, f32 add, stored in `dtype`)
 *   xn[r] = rmsnorm(x[r] + delta[r], w, eps)   (from the unrounded f32 sum)
 * x_inout is the residual stream, which every add-norm of a step reads and
 * rewrites: when it is at most 32 MB its loads and stores are given the high
 * L2 eviction priority, so that it stays on chip from one call to the next
 * (half the HBM traffic of the call). The lines keep that priority until
 * newer ones of the same priority displace them; an engine that would rather
 * have all of L2 for its other kernels sets LOKAL_CUDA_NORM_L2_KEEP=0 in the
 * environment (read per call). Results do not depend on it. */
LOKAL_API int lokal_cuda_add_rmsnorm(lokal_cuda_ctx* ctx, lokal_cuda_stream s, void* x_inout, const void* delta,
                                     const void* w, void* xn, void* xn_h, size_t rows, size_t dim, float eps,
                                     int dtype, int w_dtype, int h_dtype);

/* ---- RoPE -----------------------------------------------------------------
 * model::rope (src/model.rs:268-279): pair (i, i + rot/2) of every head turned
 * by angle pos * theta^(-(2 i)/rot). GPU twins rope / rope_h / rope_qk_prefill /
 * rope_qk_decode / rope_qk_batch (src/gpu/kernels.metal:2401-2555, 3380);
 * parameter blocks RopeParams, RopeQkParams, RopeQkPrefillParams,
 * RopeQkBatchParams, RowMeta (src/gpu/metal.rs:59-131).
 *
 * The (cos, sin) of a row's angles are the same for every head and every
 * layer of a step, so they are built once into a table:
 *   cos_sin[r][0 .. rot/2) = cos(pos_r * f_i),  cos_sin[r][rot/2 .. rot) = sin(pos_r * f_i)
 * f_i = powf(theta, -(2 i)/rot) is evaluated on the HOST by this call with
 * the C library's powf (the function the reference's CPU path reaches through
 * Rust std), so the angle is one f32 multiply on both sides.
 * positions: device int32[rows] (batched decode, BatchRow.pos of
 * src/engine.rs:30-34) or NULL for pos0 + r (prefill). cos_sin: device f32,
 * rows * rot_dim entries, 16-byte aligned. rot_dim even, <= 1024. */
LOKAL_API int lokal_cuda_rope_table(lokal_cuda_ctx* ctx, lokal_cuda_stream s, float theta, uint32_t rot_dim,
                                    const int32_t* positions, int64_t pos0, size_t rows, float* cos_sin);

/* One launch for q and k of `rows` token rows. Per head, in the reference's
 * order (src/model.rs:208-226): v = raw (+ bias, Linear::forward
 * src/model.rs:27-35; GPU twins bias_add src/gpu/kernels.metal:2131 and the
 * matmul_tb store epilogue :2106-2114) -> per-head rmsnorm with a weight of
 * head_dim entries shared by all heads (src/model.rs:213-221) when a norm
 * weight is given -> rotate the first rot_dim dims; dims rot_dim..head_dim
 * pass through (bit-identical when there is no bias and no norm). */
typedef struct lokal_qk_rope_params {
    void* q;               /* [rows][n_q_heads*head_dim] at q_row_stride; NULL = skip q */
    void* k;               /* [rows][n_kv_heads*head_dim] at k_row_stride; NULL = skip k */
    void* q_out;           /* NULL = in place */
    void* k_out;           /* NULL = in place; rows addressed through k_out_rows if given */
    const void* q_bias;    /* [n_q_heads*head_dim] in w_dtype, or NULL */
    const void* k_bias;    /* [n_kv_heads*head_dim] in w_dtype, or NULL */
    const void* q_norm_w;  /* [head_dim] in w_dtype, or NULL */
    const void* k_norm_w;  /* [head_dim] in w_dtype, or NULL */
    const float* cos_sin;  /* table from lokal_cuda_rope_table, row r for token row r */
    const uint32_t* k_out_rows; /* optional device array: output row index of token row r in k_out
                                   (a KV-cache row, (slot*max_seq+pos) in src/gpu/kernels.metal:3411) */
    uint64_t rows;
    uint32_t n_q_heads, n_kv_heads, head_dim, rot_dim;
    uint64_t q_row_stride, k_row_stride, q_out_row_stride, k_out_row_stride; /* in elements */
    float eps;             /* rms_norm_eps of the layer, used by the per-head norm */
    int32_t q_dtype, k_dtype, w_dtype; /* lokal_type; q F32 with k F16 is the reference GPU layout */
} lokal_qk_rope_params;

LOKAL_API int lokal_cuda_qk_rope(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const lokal_qk_rope_params* p);

/* Same op with the reference's own argument list (pos0 or per-row positions
 * plus theta): the table is built into scratch memory owned by the context
 * (grown on demand with cudaMalloc) and consumed by the same launch sequence.
 * Calls from several streams of one context are safe: each waits, on the
 * device, until the previous call's rope kernel has consumed the shared table
 * (so these short sections run one after another; sessions that want no such
 * coupling build their own table and call lokal_cuda_qk_rope). The block is
 * used by this entry point only (the host-slice mirrors below have their own).
 * A call made while `s` is being captured into a graph cannot take part in that
 * hand-over: keep other callers of this entry point off the context while such
 * a graph runs. Nor can it allocate: if the block is smaller than the call needs
 * it returns LOKAL_ERR_BAD_ARG (make one uncaptured call of that size first). A
 * block whose address a captured graph holds is kept until the context is
 * destroyed, also when a later, larger call replaces it, so replays stay valid. */
LOKAL_API int lokal_cuda_qk_rope_pos(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const lokal_qk_rope_params* p,
                                     float theta, const int32_t* positions, int64_t pos0);

/* lokal_cuda_qk_rope_pos for callers that must not allocate. (No counterpart
 * in the reference: its GPU backends run on unified memory and size every
 * buffer when a session is created.)
 *
 * Who needs it: a serving loop that may not stall -- cudaMalloc and cudaFree
 * synchronise the whole device and take driver-wide locks, so one call from a
 * decode step holds up every request in flight -- and an engine that has
 * handed all remaining HBM to its KV-cache pool at start-up, where a later
 * allocation can simply fail. lokal_cuda_qk_rope_pos grows a scratch block on
 * demand; this variant never calls cudaMalloc, cudaFree or any allocating
 * routine. Its (cos, sin) table lives in a fixed array inside the library
 * image, LOKAL_NOALLOC_TABLE_BYTES per GPU, which every GPU that loads the
 * library carries until the process exits.
 *
 * Limit: p->rows * p->rot_dim * 4 bytes must fit in LOKAL_NOALLOC_TABLE_BYTES
 * (e.g. 2048 rows at rot_dim 128, 4096 rows at 64); anything larger is refused
 * with LOKAL_ERR_BAD_ARG and a message naming the limit. Everything else,
 * inputs, outputs and results, is as in lokal_cuda_qk_rope_pos.
 *
 * The first call on each GPU looks up the array's device address (a one-time
 * host-side query); make that first call outside any stream capture. The
 * array is shared by every call on that GPU and keeps the last call's table:
 * each call first rewrites the rows it is about to read, so nothing has to
 * start at zero, but two calls that overlap on the device (different streams,
 * or different contexts on the same GPU) race on it. Serialise them. */
#define LOKAL_NOALLOC_TABLE_BYTES (1u << 20)
LOKAL_API int lokal_cuda_qk_rope_pos_noalloc(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const lokal_qk_rope_params* p,
                                             float theta, const int32_t* positions, int64_t pos0);

/* ---- SwiGLU ---------------------------------------------------------------
 * inner_i = (g_i / (1 + exp(-g_i))) * u_i (src/math.rs:68-70, src/model.rs:245-248;
 * GPU twins silu_mul / silu_mul_hf src/gpu/kernels.metal:3533, 3548; host
 * enc_elementwise src/gpu/metal.rs:1527; ElemParams{dim} :150-152).
 * out may alias gate (the reference writes in place). out_h: optional second
 * copy in h_dtype (F16/BF16), only with dtype F32. n = total elements. */
LOKAL_API int lokal_cuda_swiglu(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* gate, const void* up, void* out,
                                void* out_h, size_t n, int dtype, int h_dtype);

/* ---- Embedding gather + row dequant -----------------------------------------
 * LowMemSession::embed_gather (src/lowmem/forward.rs:275-307), the quant
 * prefill's Source::Ids arm (src/gpu/metal.rs:3160-3184), the dense lookup
 * (src/model.rs:200-202) and the GPU twin `embed` (src/gpu/kernels.metal:30);
 * row addressing and range check of LowMemSource::read_rows
 * (src/lowmem/mod.rs:654-668); decode = gguf::dequant_row_ref, every arm
 * (src/gguf/dequant.rs:191-535), bit for bit; BF16 tables in addition.
 *   out[i][0..dim) = dequant(table row ids[i])
 * table: device bytes, vocab rows of row_bytes(type, dim), 16-byte aligned.
 * ids: device u32[n]. out: `out_dtype` F32, or F16 / BF16 (the exact f32 value
 * rounded once, nearest-even). An id >= vocab zero-fills its row and raises
 * LOKAL_ERR_ID_RANGE at the next lokal_cuda_stream_sync. dim must be a whole
 * number of blocks (src/gguf/container.rs:220-226). */
LOKAL_API int lokal_cuda_embed_gather(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* table, int ggml_type,
                                      size_t vocab, size_t dim, const uint32_t* ids, size_t n, void* out,
                                      int out_dtype);

/* Embedding gather and the RMSNorm that follows it in a step, as one call: x[i] = dequant(table[ids[i]]) and
 * xn[i] = rmsnorm(x[i], w, eps). The reference's step starts with exactly this pair (Model::forward, src/model.rs:200-209:
 * the row copy, then the first block's input_layernorm; MetalSession::run_from encodes `embed` and `rmsnorm*` back to
 * back, src/gpu/metal.rs:2525, 2552). With a quantised table the norm rides in the gather's launch: the warp that stored
 * a row sums the squares of the values as stored (rounded to out_dtype, what a separate norm launch would read) and
 * writes xn. Float tables and unaligned buffers run the two launches one after the other; the results follow the same
 * definition either way. x and xn are n x dim of out_dtype; w is [dim] of w_dtype. Out-of-range ids as in embed_gather
 * (x and xn rows zero, LOKAL_ERR_ID_RANGE at the next synchronisation). */
LOKAL_API int lokal_cuda_embed_gather_rmsnorm(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* table, int ggml_type,
                                              size_t vocab, size_t dim, const uint32_t* ids, size_t n, void* x, void* xn,
                                              const void* w, float eps, int out_dtype, int w_dtype);

/* Dequantise `rows` consecutive rows: the bit-for-bit gate kernel
 * lm_dequant_oracle (src/gpu/kernels.metal:1417-1428, LmDeqParams :1411). */
LOKAL_API int lokal_cuda_dequant_rows(lokal_cuda_ctx* ctx, lokal_cuda_stream s, int ggml_type, const void* src,
                                      size_t rows, size_t cols, void* out, int out_dtype);

/* ---- K/V staging into the cache -----------------------------------------------------
 * The step right after RoPE: fresh K and V rows are narrowed to the cache type and
 * written to their cache rows. Reference: f32_to_f16 (src/gpu/kernels.metal:2118),
 * batched-decode row addressing (slot*max_seq + pos)*kv_dim (src/gpu/kernels.metal:3310,
 * 3411-3412; RowMeta{pos,slot}, src/gpu/metal.rs:79-82), and the sink + ring store of the
 * windowed backends: WindowCfg / slot_of (src/lowmem/mod.rs:163-193), write_spans
 * (src/lowmem/forward.rs:256-271; src/gpu/metal.rs:673-691).
 *
 * The reference splits a chunk into at most three host-computed spans; here the cache row
 * of every token row is computed on the device into an index array, which both
 * lokal_cuda_kv_stage and lokal_cuda_qk_rope (k_out_rows) consume. */
typedef struct lokal_kv_layout {
    uint64_t max_seq;   /* rows per slot in the linear layout; ignored when windowed */
    uint64_t sink;      /* windowed store: positions 0..sink are pinned ... */
    uint64_t sink_pad;  /* ... in a region padded to this many rows ... */
    uint64_t ring;      /* ... followed by a ring of this many rows; ring == 0 selects the linear layout */
} lokal_kv_layout;

/* WindowCfg::new(w, sink) with the reference's prefill chunk of slack (512 in the reference,
 * src/gpu/metal.rs:30): sink_pad and ring are rounded up to multiples of 128. Host only. */
LOKAL_API int lokal_cuda_window_cfg(uint64_t window, uint64_t sink, uint64_t prefill_chunk, lokal_kv_layout* out);
/* WindowCfg::slot_of: the store row (within one slot) that holds position p. Host only. */
LOKAL_API uint64_t lokal_cuda_window_slot_of(const lokal_kv_layout* layout, uint64_t p);
/* write_spans: destination spans (first chunk row, first store row, length) for positions
 * [pos0, pos0+n); spans[] must hold 3 entries of 3 values. Returns the span count. Host only. */
LOKAL_API int lokal_cuda_window_write_spans(const lokal_kv_layout* layout, uint64_t pos0, uint64_t n, uint64_t* spans);

/* Cache row of every token row, on the device:
 *   linear:   slot_r * max_seq + pos_r            windowed: slot_r * (sink_pad + ring) + slot_of(pos_r)
 * positions / slots: device int32[rows] / uint32[rows], or NULL for pos0 + r / slot0.
 * A position the cache cannot hold (negative; >= max_seq in the linear layout, which would be a row of the next
 * slot; a row index beyond 32 bits) gets LOKAL_KV_ROW_NONE: lokal_cuda_kv_stage and lokal_cuda_qk_rope store nothing
 * for such a row, and the next lokal_cuda_stream_sync returns LOKAL_ERR_POS_RANGE. The slot count is the caller's:
 * a slot beyond the cache is not detectable here. */
#define LOKAL_KV_ROW_NONE 0xFFFFFFFFu
LOKAL_API int lokal_cuda_kv_rows(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const lokal_kv_layout* layout,
                                 const int32_t* positions, int64_t pos0, const uint32_t* slots, uint32_t slot0,
                                 size_t rows, uint32_t* rows_out);
/* dst[dst_rows[r]] = narrow(src[r]) for `rows` rows of `width` elements (strides in elements;
 * dst_rows NULL = row r). Types F32 / F16 / BF16; a narrowing conversion rounds to nearest even. */
LOKAL_API int lokal_cuda_kv_stage(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* src, int src_dtype,
                                  size_t src_row_stride, void* dst, int dst_dtype, size_t dst_row_stride,
                                  const uint32_t* dst_rows, size_t rows, size_t width);

/* ---- Per-row siblings in the gated-deltanet (qwen35) blocks ----------------------
 * The same shape of work as the ops above (one pass over token rows), used by the
 * reference's qwen35 layers. Sums of squares are taken in f64, as the reference's CPU
 * code does (src/deltanet_ref.rs:61-78); its Metal kernels sum in f32 only for want of
 * f64. Rows are F32 / F16 / BF16 with f32 arithmetic and one rounding on store; y may
 * be x (in place, as the reference works). */

/* l2_norm (src/deltanet_ref.rs:61-67; l2norm_rows, src/gpu/kernels.metal:3697-3735):
 *   y = x * (1 / max(sqrt(sum x^2), eps))       -- a zero row stays zero, never NaN.
 * Row r of token t starts at element t*tok_stride + r*dim, the batched kernel's
 * addressing; with n_tokens == 1 tok_stride is ignored. */
LOKAL_API int lokal_cuda_l2norm_rows(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* x, void* y, size_t rows_per_token,
                                     size_t n_tokens, size_t tok_stride, size_t dim, float eps, int dtype);
/* gated_output_norm (src/deltanet_ref.rs:187-198; src/gpu/kernels.metal:3936-3975), per row (V head) of `dim`:
 *   scale = 1 / sqrt(mean(o^2) + eps);   y = ((o * scale) * w) * (z * sigmoid(z))
 * in that association; w[dim] is shared by all rows. */
LOKAL_API int lokal_cuda_gated_output_norm(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* o, const void* w, const void* z,
                                           void* y, size_t rows, size_t dim, float eps, int dtype, int w_dtype);
/* attn_out_gate (src/deltanet_ref.rs:203-207; src/gpu/kernels.metal:3667-3676):
 *   out = attn * (1 / (1 + exp(-gate))), elementwise over n elements; out may be attn. */
LOKAL_API int lokal_cuda_attn_out_gate(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* attn, const void* gate, void* out,
                                       size_t n, int dtype);
/* split_q_gate (src/gpu/kernels.metal:4106-4124): a row of the joint projection is
 * [q(head_dim) | gate(head_dim)] per head; q and gate come out compact,
 * [rows][n_heads][head_dim] each. A pure copy. */
LOKAL_API int lokal_cuda_split_q_gate(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* src, void* q, void* gate, size_t rows,
                                      size_t n_heads, size_t head_dim, int dtype);

/* delta_gates (src/deltanet_ref.rs:48-58, 82-84; src/gpu/kernels.metal:3995-4015), one value per V head and token:
 *   g[t][h]    = a[h] * softplus(alpha[t][h] + dt_bias[h])     softplus(x) = x > 20 ? x : log(1 + exp(x))
 *   beta[t][h] = 1 / (1 + exp(-beta_in[t][h]))
 * All f32, [n_tokens][n_v_heads]; a and dt_bias are [n_v_heads]. g may be alpha and beta may be beta_in. */
LOKAL_API int lokal_cuda_delta_gates(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const float* alpha, const float* beta_in,
                                     const float* a, const float* dt_bias, float* g, float* beta, size_t n_v_heads,
                                     size_t n_tokens);

/* Depthwise causal conv over the token axis, SiLU inside: conv_step (src/deltanet_ref.rs:91-112) applied to
 * n_tokens rows in turn; one launch does what ssm_conv_decode / ssm_conv_prefill + ssm_conv_roll do
 * (src/gpu/kernels.metal:3626-3665, 4039-4093).
 *   acc = sum_{j<k-1} window[j] * w[c][j]  +  x[t][c] * w[c][k-1]      (f32, separate multiply and add, in this order)
 *   out[t][c] = acc * (1 / (1 + exp(-acc)))
 * window = the k-1 inputs before token t: rows of x, or entries of `state` for the first tokens.
 * state: f32 [channels][d_conv-1], oldest first. With roll != 0 it is replaced, after every token has read it, by the
 * window that follows the last token (the decode form always rolls; a prefill chunk rolls once at its end).
 * x, out: [n_tokens][channels] in `dtype` (F32 / F16 / BF16), out must not be x. w: f32 [channels][d_conv].
 * d_conv 1..8 (the reference refuses more taps). */
LOKAL_API int lokal_cuda_ssm_conv(lokal_cuda_ctx* ctx, lokal_cuda_stream s, float* state, const void* x, const float* w,
                                  void* out, size_t channels, size_t d_conv, size_t n_tokens, int dtype, int roll);

/* bf16_to_f16_copy (src/gpu/kernels.metal:3572-3588), the weight-page conversion of the low-memory stage-in:
 * bf16 bits widened exactly to f32, narrowed to f16 with round-to-nearest-even. clip_flag (device u32, may be
 * NULL) is OR-ed with 1 when a finite value leaves the f16 range; the caller clears it. */
LOKAL_API int lokal_cuda_bf16_to_f16_copy(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* src_bf16, void* dst_f16,
                                          size_t n, uint32_t* clip_flag);

/* ---- GGUF container reader -------------------------------------------------------
 * GgufFile (src/gguf/container.rs:152-384): v2/v3, little-endian, mapped read-only.
 * Host only. Enough to find token_embd.weight, norm weights and biases
 * (names: src/gguf/arch.rs:229-263) and feed their bytes to the ops above.
 * open fails with one message that names EVERY tensor type this library does not
 * decode, with counts and an example tensor each (container.rs:190-245). */
typedef struct lokal_gguf lokal_gguf;
typedef struct lokal_gguf_tensor {
    const char* name;      /* owned by the file handle */
    uint32_t n_dims;       /* 1..4 */
    uint64_t dims[4];      /* row-major (the file's ne[] reversed); unused entries are 1 */
    int32_t ggml_type;     /* lokal_type */
    uint64_t file_offset;  /* of the first byte, from the start of the file */
    uint64_t data_offset;  /* the same, from the start of the data section (what the file stores) */
    uint64_t nbytes;       /* row_bytes(type, product of dims) */
    const void* data;      /* into the mapping; valid until lokal_gguf_close */
} lokal_gguf_tensor;

/* GgufFile::open. On failure *out is NULL and `err` (may be NULL) receives the message. */
LOKAL_API int lokal_gguf_open(const char* path, lokal_gguf** out, char* err, size_t err_len);
LOKAL_API void lokal_gguf_close(lokal_gguf* g);
LOKAL_API const char* lokal_gguf_last_error(const lokal_gguf* g);
LOKAL_API uint32_t lokal_gguf_version(const lokal_gguf* g);
LOKAL_API size_t lokal_gguf_n_tensors(const lokal_gguf* g);
LOKAL_API uint64_t lokal_gguf_data_start(const lokal_gguf* g);
/* GgufFile::tensors (by index, file order) and GgufFile::tensor (by name). */
LOKAL_API int lokal_gguf_tensor_at(const lokal_gguf* g, size_t i, lokal_gguf_tensor* out);
LOKAL_API int lokal_gguf_find_tensor(const lokal_gguf* g, const char* name, lokal_gguf_tensor* out);
/* Typed metadata accessors: has_key, get_usize, get_f32, get_str, get_arr_i64, get_arr_str.
 * A missing key is LOKAL_ERR_NOT_FOUND, a value of another kind LOKAL_ERR_BAD_ARG; the
 * message names the key and what was found. Returned pointers are owned by the handle. */
LOKAL_API int lokal_gguf_has_key(const lokal_gguf* g, const char* key);
LOKAL_API int lokal_gguf_get_u64(const lokal_gguf* g, const char* key, uint64_t* out);
LOKAL_API int lokal_gguf_get_f32(const lokal_gguf* g, const char* key, float* out);
LOKAL_API int lokal_gguf_get_str(const lokal_gguf* g, const char* key, const char** out, size_t* len);
LOKAL_API int lokal_gguf_get_arr_i64(const lokal_gguf* g, const char* key, const int64_t** out, size_t* n);
LOKAL_API int lokal_gguf_get_arr_str(const lokal_gguf* g, const char* key, const char* const** out, size_t* n);
/* Copies one tensor's raw bytes into a fresh device allocation (free with lokal_cuda_free);
 * blocks until the copy is done. `info` (may be NULL) receives the tensor's description. */
LOKAL_API int lokal_cuda_gguf_upload(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const lokal_gguf* g, const char* name, void** dptr,
                                     lokal_gguf_tensor* info);

/* ---- Token-row sharding over GPUs ---------------------------------------------
 * Rows are independent, so GPU `rank` of `n_gpus` owns the contiguous block
 * [row0, row0+count); no exchange happens on the path. The reference has no
 * multi-device code; this has no counterpart there. */
LOKAL_API int lokal_cuda_shard_rows(size_t n_rows, int n_gpus, int rank, size_t* row0, size_t* count);

/* ---- Layer pass: the per-token ops of one forward step, layer by layer -----------
 * The place these ops take in the reference's step: MetalSession::run_from
 * (src/gpu/metal.rs:2470-2691), MetalBatcher::decode_step (:3662-3775) and the
 * CPU Model::forward (src/model.rs:196-261), with the projections and attention
 * between them left to the caller. One step over `rows` token rows is
 *   x = embed_gather(ids);  table = rope_table(positions | pos0);  xn = rmsnorm(x, w[0][0])
 *   for each layer l:  qk_rope(q[l], k[l])            (bias -> per-head norm -> rotate, in place)
 *                      x += delta_att[l]; xn = rmsnorm(x, w[l][1])
 *                      inner[l] = silu(gate[l]) * up[l]
 *                      x += delta_mlp[l]; xn = rmsnorm(x, w[l+1][0], or the final norm weight after the last layer)
 * q, k, delta_att, delta_mlp, gate, up are what the out-of-scope projections
 * and attention produce; the caller provides them per layer. The result of a
 * step is the final normed hidden state, rows x hidden. */
typedef struct lokal_pass_config {
    uint64_t max_rows;        /* capacity in token rows of one step on this GPU */
    uint32_t layers, hidden, inter, n_q_heads, n_kv_heads, head_dim, rot_dim;
    float eps, theta;
    int32_t dtype;            /* activation storage type: F32 / F16 / BF16 */
    int32_t w_dtype;          /* type of norm weights and biases */
    int32_t has_qk_bias, has_qk_norm;
    int32_t embed_type;       /* ggml type of the embedding table */
    uint32_t slots;           /* layer slots kept on the device for staged inputs and per-layer outputs:
                                 `layers` keeps every layer's outputs; 2-4 is a ring for lokal_cuda_pass_run_host */
    uint64_t vocab;
} lokal_pass_config;

/* Weights, HOST pointers, copied to the device once (weights resident, src/gpu/mod.rs:3-13). */
typedef struct lokal_pass_weights {
    const void* embed_table;  /* vocab rows of row_bytes(embed_type, hidden) */
    const void* norm_w;       /* [layers][2][hidden]: input norm, post-attention norm */
    const void* final_w;      /* [hidden] */
    const void* q_bias;       /* [layers][n_q_heads*head_dim] or NULL */
    const void* k_bias;       /* [layers][n_kv_heads*head_dim] or NULL */
    const void* q_norm_w;     /* [layers][head_dim] or NULL */
    const void* k_norm_w;     /* [layers][head_dim] or NULL */
} lokal_pass_weights;

/* Inputs of one step. For lokal_cuda_pass_run_host every pointer is HOST memory
 * (pinned memory from lokal_cuda_host_alloc lets copies overlap the kernels); for
 * lokal_cuda_pass_run_device every pointer is DEVICE memory. Per-layer buffers are
 * [layers][rows][width] with the given layer strides (in elements). */
typedef struct lokal_pass_inputs {
    const uint32_t* ids;        /* [rows] */
    const int32_t* positions;   /* [rows] or NULL for pos0 + row */
    int64_t pos0;
    uint64_t rows;
    void* q;                    /* [layers][rows][n_q_heads*head_dim], rotated in place (device runs) */
    void* k;                    /* [layers][rows][n_kv_heads*head_dim] */
    const void* delta_att;      /* [layers][rows][hidden] */
    const void* delta_mlp;      /* [layers][rows][hidden] */
    const void* gate;           /* [layers][rows][inter] */
    const void* up;             /* [layers][rows][inter] */
    uint64_t q_layer_stride, k_layer_stride, delta_layer_stride, mlp_layer_stride;
} lokal_pass_inputs;

typedef struct lokal_cuda_pass lokal_cuda_pass;

LOKAL_API int lokal_cuda_pass_create(lokal_cuda_ctx* ctx, const lokal_pass_config* cfg, const lokal_pass_weights* w,
                                     lokal_cuda_pass** out);
LOKAL_API int lokal_cuda_pass_destroy(lokal_cuda_ctx* ctx, lokal_cuda_pass* pass);
/* One step on device-resident inputs, asynchronous on `s` (capturable between
 * lokal_cuda_graph_begin/end). out_dev: rows x hidden in `dtype`. */
LOKAL_API int lokal_cuda_pass_run_device(lokal_cuda_ctx* ctx, lokal_cuda_pass* pass, lokal_cuda_stream s,
                                         const lokal_pass_inputs* in_dev, void* out_dev);
/* One step on host inputs: layer l+1's inputs are copied while layer l computes
 * (a ring of `slots` layer slots), the result is copied back, and the call
 * returns when out_host is complete. Rotated q/k, xn and inner stay on the device. */
LOKAL_API int lokal_cuda_pass_run_host(lokal_cuda_ctx* ctx, lokal_cuda_pass* pass, const lokal_pass_inputs* in_host,
                                       void* out_host);
/* Device addresses of the per-layer outputs a downstream projection would read
 * (slot = layer % slots): which 0 = xn after the attention residual, 1 = xn after the
 * MLP residual, 2 = inner, 3 = staged/rotated q, 4 = staged/rotated k (3, 4 only after run_host). */
LOKAL_API int lokal_cuda_pass_output(lokal_cuda_ctx* ctx, lokal_cuda_pass* pass, uint32_t layer, int which, void** dptr);
/* Kernels launched by the last run on this pass. */
LOKAL_API uint64_t lokal_cuda_pass_launches(const lokal_cuda_pass* pass);
/* How lokal_cuda_pass_run_device orders the kernels of a step. The reference encodes a step into one command
 * buffer and submits once (src/gpu/metal.rs:2679-2681); its order is the order of Model::forward. Here all inputs
 * of a step are given up front, so the data flow has three independent families: the residual-add + RMSNorm chain
 * (through x), the q/k rotations (q, k and the table), and SwiGLU (gate, up, inner).
 *   SEQUENTIAL  one stream, the order of Model::forward (src/model.rs:207-255)
 *   BRANCHES    the three families on parallel branches forked from and joined into `s` (graph edges under capture),
 *               the norm chain at the highest stream priority; same kernels, same results bit for bit, and the ramp
 *               and drain of one family's kernels is covered by the others
 *   AUTO        the library's choice (the default): BRANCHES, the shorter one at every batch size measured */
#define LOKAL_PASS_SCHEDULE_AUTO 0
#define LOKAL_PASS_SCHEDULE_SEQUENTIAL 1
#define LOKAL_PASS_SCHEDULE_BRANCHES 3
LOKAL_API int lokal_cuda_pass_set_schedule(lokal_cuda_ctx* ctx, lokal_cuda_pass* pass, int schedule);

/* ---- Host-slice mirrors of the reference's CPU signatures ---------------------
 * Inputs and outputs are HOST memory; each call stages through buffers owned
 * by the context, runs the device op and waits for the result. */
/* math::rmsnorm(x, weight, eps) -> y (src/math.rs:45), f32, rows x dim. */
LOKAL_API int lokal_cuda_host_rmsnorm(lokal_cuda_ctx* ctx, const float* x, const float* w, float eps, size_t rows,
                                      size_t dim, float* y);
/* model::rope(x, pos, head_dim, theta) in place on one row of whole heads (src/model.rs:268). */
LOKAL_API int lokal_cuda_host_rope(lokal_cuda_ctx* ctx, float* x, size_t n, size_t pos, size_t head_dim, float theta);
/* the SwiGLU line silu(g) * u (src/model.rs:247-248). */
LOKAL_API int lokal_cuda_host_swiglu(lokal_cuda_ctx* ctx, const float* gate, const float* up, size_t n, float* out);
/* gguf::dequant_row_ref(ty, src, out) (src/gguf/dequant.rs:191); a size
 * mismatch, where the reference panics, returns LOKAL_ERR_BAD_ARG. */
LOKAL_API int lokal_cuda_host_dequant_row(lokal_cuda_ctx* ctx, int ggml_type, const uint8_t* src, size_t src_len,
                                          float* out, size_t n);
/* embed_gather with a DEVICE-resident table and host ids / host f32 output. ids and out may be ordinary memory
 * (copied through pinned staging; a large result is pulled by several worker threads so that DMA and the CPU copy
 * overlap) or page-locked memory from lokal_cuda_host_alloc / cudaHostAlloc, which the copy engines reach directly. */
LOKAL_API int lokal_cuda_host_embed_gather(lokal_cuda_ctx* ctx, const void* table_dev, int ggml_type, size_t vocab,
                                           size_t dim, const uint32_t* ids, size_t n, float* out);

#ifdef __cplusplus
}
#endif
#endif /* LOKAL_CUDA_H */
