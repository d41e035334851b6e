// Token-embedding gather with on-the-fly GGUF row dequantisation.
//
// Reference semantics: LowMemSession::embed_gather (src/lowmem/forward.rs:275-307)
// walks the ids, slices row id out of the table bytes (read_rows,
// src/lowmem/mod.rs:654-668) and expands it with gguf::dequant_row_ref
// (src/gguf/dequant.rs:191-239 F32/F16/Q8_0, :462-483 Q4_K, scale unpack
// :141-150; :204-230 Q4_0/Q5_0, :396-425 IQ4_NL/IQ4_XS, :426-461 Q2_K/Q3_K,
// :484-535 Q5_K/Q6_K, :255-394 the codebook types). Results here are
// bit-identical to that: int -> f32 and f16 -> f32 conversions are exact, and
// every product and difference of the reference's expressions (d1*q - m1,
// (d*sc)*q ...) is computed with __fmul_rn / __fsub_rn or their packed f32x2
// twins, so each is rounded once and never contracted into an FMA. Every block
// type has a vector decoder for the staged kernel (four elements per 32-bit
// word of quants) and an element decoder for the kernel that takes any
// alignment.
//
// Kernel shape (quantised tables): one warp per token row, persistent over a
// grid-stride list of rows. Lane 0 stages the raw row into shared memory with
// one bulk asynchronous copy (cp.async.bulk, completion on an mbarrier) while
// the warp decodes the previous row: a two-stage ring per warp. Q8_0 rows are
// a multiple of 34 bytes, so a row start is only 2-byte aligned; the copy
// fetches the enclosing 16-byte-aligned window and the decode indexes from the
// remainder. Each lane then produces 16 bytes of output per step (4 f32 or
// 8 f16/bf16), so every store instruction of a warp writes one 512-byte run
// (f32 rows of the codebook types: a whole run of 8 values, 32 bytes, per lane).
// 16-bit output rows are decoded two to a warp (gather_quant_pair_kernel), which
// shares the per-row bookkeeping between the two halves of the warp.
// HBM traffic per token: row_bytes for the first touch of a row (hot rows hit
// L2) plus dim*sizeof(out) written.
//
// Every wait on an mbarrier is bounded: after the limit the warp records
// kErrTimeout in the context's error word and leaves.
#include "common.cuh"

#include <type_traits>

namespace lokal {
namespace {

struct GatherArgs {
    const unsigned char* table;
    const uint32_t* ids;  // null -> row i
    void* out;
    unsigned long long n;
    unsigned long long vocab;
    unsigned long long table_bytes;
    // The staged kernel keeps its row bookkeeping in 32 bits (the host hands it at most 2^30 rows per launch):
    unsigned n32;        // rows of this launch
    unsigned max_id;     // min(vocab, 2^32) - 1: an id above it is out of range
    unsigned bulk_ids;   // ids below it have their 16-byte-aligned window inside the table (all but, at most, the last row)
    unsigned out32;      // every output row starts on a 32-byte boundary: a lane may store 32 bytes at once
    unsigned table_keep; // table rows are fetched with the high L2 eviction priority (hot rows outlive the output rows streaming through)
    unsigned dim;
    unsigned row_bytes;
    unsigned stage_bytes;  // per warp per stage, multiple of 16
    const void* grid;      // the codebook of an IQ1 / IQ2 / IQ3 table type (device memory), else null
    unsigned* err_word;
    unsigned wait_limit;   // polls of a staged copy's mbarrier before the kernel gives up (kWaitLimit)
    unsigned extra_tx;     // 0; a test sets it so that a copy never completes its barrier and the bounded wait runs out
    // gather fused with the RMSNorm that follows it in a step (the FUSE variant of the staged kernel)
    const void* norm_w;    // [dim] weights
    void* xn;              // [n][dim] normed rows, of the output type
    float eps, inv_dim;
    int w_dtype, w_vec_ok;
};

// ---- block decoders: EPL consecutive elements starting at element e (e % EPL == 0), as EPL/2 pairs ----

// Exact float of byte k of `word` (0..255) without the conversion pipe: the byte becomes the low mantissa bits of
// 2^23, and subtracting 2^23 (an exact operation) leaves the integer. The caller folds a further integer bias
// (128 for int8 stored as q ^ 0x80) into the subtracted constant; 2^23 + 128 is exact too.
template <int K>
__device__ __forceinline__ float byte_plus_2p23(unsigned word) {
    return __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540u | K));
}

// Four bytes of `w`, each minus `bias`, as two pairs of exact floats. nb = -(2^23 + bias) in both halves.
__device__ __forceinline__ void bytes_to_pairs(unsigned w, float2 nb, float2& a, float2& b) {
    a = add2(make_float2(byte_plus_2p23<0>(w), byte_plus_2p23<1>(w)), nb);
    b = add2(make_float2(byte_plus_2p23<2>(w), byte_plus_2p23<3>(w)), nb);
}
__device__ __forceinline__ float2 both(float v) { return make_float2(v, v); }

// 32 bits from shared memory at a 2-byte-aligned address (rows of 18-, 22-, 34-, 110- and 210-byte blocks).
__device__ __forceinline__ unsigned lds_u32_a2(const unsigned char* p) {
    const unsigned short* h = reinterpret_cast<const unsigned short*>(p);
    return static_cast<unsigned>(h[0]) | (static_cast<unsigned>(h[1]) << 16);
}
__device__ __forceinline__ unsigned lds_u32(const unsigned char* p) { return *reinterpret_cast<const unsigned*>(p); }
__device__ __forceinline__ float lds_f16(const unsigned char* p) {
    return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(p)));
}

// ---- one element of any block type, bytes fetched through rd(offset) ----
// The element-indexed form of the reference's sequential decoders; each arm
// cites the loop it restates. All arithmetic on f32 is one rounded operation
// per reference operation.
struct SharedBytes {
    const unsigned char* p;
    __device__ __forceinline__ unsigned operator()(unsigned i) const { return p[i]; }
};
struct GlobalBytes {
    const unsigned char* p;
    __device__ __forceinline__ unsigned operator()(unsigned i) const { return __ldg(p + i); }
};

template <typename Rd>
__device__ __forceinline__ float rd_f16(const Rd& rd, unsigned off) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(rd(off) | (rd(off + 1) << 8))));
}

// The 16-entry non-linear codebook of IQ4_NL / IQ4_XS (src/gguf/dequant.rs:161-166),
// packed one signed byte per entry so the lookup is a shift, not a divergent memory access.
__device__ __forceinline__ float iq4_value(unsigned q) {
    // -127, -104, -83, -65, -49, -35, -22, -10 | 1, 13, 25, 38, 53, 69, 89, 113
    const unsigned long long lo = 0xF6EADDCFBFAD9881ull, hi = 0x7159453526190D01ull;
    const unsigned long long w = (q & 8u) ? hi : lo;
    return static_cast<float>(static_cast<int>(static_cast<signed char>((w >> (8 * (q & 7u))) & 0xFF)));
}

// get_scale_min_k4 (src/gguf/dequant.rs:141-150): 6-bit scale and min of sub-block j from 12 packed bytes at sb.
template <typename Rd>
__device__ __forceinline__ void scale_min_k4(const Rd& rd, unsigned sb, unsigned j, unsigned& sc, unsigned& mn) {
    if (j < 4) {
        sc = rd(sb + j) & 63u;
        mn = rd(sb + j + 4) & 63u;
    } else {
        sc = (rd(sb + j + 4) & 0x0Fu) | ((rd(sb + j - 4) >> 6) << 4);
        mn = (rd(sb + j + 4) >> 4) | ((rd(sb + j) >> 6) << 4);
    }
}

template <int QT, typename Rd>
__device__ __forceinline__ float dequant_elem(const Rd& rd, unsigned col) {
    if constexpr (QT == LOKAL_Q8_0) {  // src/gguf/dequant.rs:231-239
        const unsigned b = (col >> 5) * 34;
        const int q = static_cast<int>(static_cast<signed char>(rd(b + 2 + (col & 31))));
        return __fmul_rn(static_cast<float>(q), rd_f16(rd, b));
    } else if constexpr (QT == LOKAL_Q4_0 || QT == LOKAL_IQ4_NL) {  // :204-214, :396-406
        const unsigned b = (col >> 5) * 18, j = col & 31;
        const unsigned byte = rd(b + 2 + (j & 15));
        const unsigned q = (j & 16) ? (byte >> 4) : (byte & 15u);
        const float d = rd_f16(rd, b);
        if constexpr (QT == LOKAL_Q4_0) return __fmul_rn(static_cast<float>(static_cast<int>(q) - 8), d);
        else return __fmul_rn(d, iq4_value(q));
    } else if constexpr (QT == LOKAL_Q5_0) {  // :215-230: bit j (low half) or j+16 (high half) of qh is the 5th bit
        const unsigned b = (col >> 5) * 22, j = col & 31;
        const unsigned qh = rd(b + 2) | (rd(b + 3) << 8) | (rd(b + 4) << 16) | (rd(b + 5) << 24);
        const unsigned byte = rd(b + 6 + (j & 15));
        const unsigned nib = (j & 16) ? (byte >> 4) : (byte & 15u);
        const int q = static_cast<int>(nib | (((qh >> j) & 1u) << 4)) - 16;
        return __fmul_rn(static_cast<float>(q), rd_f16(rd, b));
    } else if constexpr (QT == LOKAL_IQ4_XS) {  // :410-425: d, scales_h u16, scales_l[4], qs[128]
        const unsigned b = (col >> 8) * 136, i = col & 255, ib = i >> 5, j = i & 31;
        const unsigned sh = rd(b + 2) | (rd(b + 3) << 8);
        const unsigned ls = ((rd(b + 4 + (ib >> 1)) >> (4 * (ib & 1))) & 15u) | (((sh >> (2 * ib)) & 3u) << 4);
        const float dl = __fmul_rn(rd_f16(rd, b), static_cast<float>(static_cast<int>(ls) - 32));
        const unsigned byte = rd(b + 8 + 16 * ib + (j & 15));
        return __fmul_rn(dl, iq4_value((j & 16) ? (byte >> 4) : (byte & 15u)));
    } else if constexpr (QT == LOKAL_Q2_K) {  // :426-440: scales[16], qs[64], d, dmin
        const unsigned b = (col >> 8) * 84, i = col & 255;
        const unsigned nh = i >> 7, j = (i >> 5) & 3, half = (i >> 4) & 1, l = i & 15;
        const unsigned sc = rd(b + nh * 8 + j * 2 + half);
        const unsigned q = (rd(b + 16 + nh * 32 + half * 16 + l) >> (2 * j)) & 3u;
        const float dl = __fmul_rn(rd_f16(rd, b + 80), static_cast<float>(sc & 15u));
        const float ml = __fmul_rn(rd_f16(rd, b + 82), static_cast<float>(sc >> 4));
        return __fsub_rn(__fmul_rn(dl, static_cast<float>(q)), ml);
    } else if constexpr (QT == LOKAL_Q3_K) {  // :445-461 and q3k_scales :171-189: hmask[32], qs[64], scales[12], d
        const unsigned b = (col >> 8) * 110, i = col & 255;
        const unsigned nh = i >> 7, j = (i >> 5) & 3, half = (i >> 4) & 1, l = i & 15;
        // scale s = aux word a, byte k of the kmask shuffle: low nibble from byte (a&1)*4+k (high nibble of it
        // for a >= 2), two more bits from byte 8+k at bit 2a; stored biased by 32
        const unsigned s = nh * 8 + j * 2 + half, a = s >> 2, k = s & 3;
        const unsigned pb = rd(b + 96 + (a & 1) * 4 + k);
        const unsigned lo = (a < 2) ? (pb & 15u) : (pb >> 4);
        const unsigned hi = (rd(b + 96 + 8 + k) >> (2 * a)) & 3u;
        const float dl = __fmul_rn(rd_f16(rd, b + 108), static_cast<float>(static_cast<int>(lo | (hi << 4)) - 32));
        const unsigned hbit = (rd(b + half * 16 + l) >> (nh * 4 + j)) & 1u;
        const int q = static_cast<int>((rd(b + 32 + nh * 32 + half * 16 + l) >> (2 * j)) & 3u) - (hbit ? 0 : 4);
        return __fmul_rn(dl, static_cast<float>(q));
    } else if constexpr (QT == LOKAL_Q4_K) {  // :462-483
        const unsigned b = (col >> 8) * 144, i = col & 255;
        unsigned sc, mn;
        scale_min_k4(rd, b + 4, i >> 5, sc, mn);
        const float d1 = __fmul_rn(rd_f16(rd, b), static_cast<float>(sc));
        const float m1 = __fmul_rn(rd_f16(rd, b + 2), static_cast<float>(mn));
        const unsigned byte = rd(b + 16 + (i >> 6) * 32 + (i & 31));
        const unsigned q = (i & 32) ? (byte >> 4) : (byte & 0xFu);
        return __fsub_rn(__fmul_rn(d1, static_cast<float>(q)), m1);
    } else if constexpr (QT == LOKAL_Q5_K) {  // :484-511: d, dmin, scales[12], qh[32], qs[128]
        const unsigned b = (col >> 8) * 176, i = col & 255, sub = i >> 5, l = i & 31;
        unsigned sc, mn;
        scale_min_k4(rd, b + 4, sub, sc, mn);
        const float d1 = __fmul_rn(rd_f16(rd, b), static_cast<float>(sc));
        const float m1 = __fmul_rn(rd_f16(rd, b + 2), static_cast<float>(mn));
        const unsigned byte = rd(b + 48 + (i >> 6) * 32 + l);
        const unsigned nib = (i & 32) ? (byte >> 4) : (byte & 0xFu);
        const unsigned q = nib + (((rd(b + 16 + l) >> sub) & 1u) << 4);
        return __fsub_rn(__fmul_rn(d1, static_cast<float>(q)), m1);
    } else {  // LOKAL_Q6_K, :512-535: ql[128], qh[64], int8 scales[16], d
        const unsigned b = (col >> 8) * 210, i = col & 255;
        const unsigned h = i >> 7, k = (i >> 5) & 3, l = i & 31;
        const unsigned qlb = rd(b + h * 64 + (k & 1) * 32 + l);
        const unsigned nib = (k & 2) ? (qlb >> 4) : (qlb & 15u);
        const int q = static_cast<int>(nib | (((rd(b + 128 + h * 32 + l) >> (2 * k)) & 3u) << 4)) - 32;
        const int sc = static_cast<int>(static_cast<signed char>(rd(b + 192 + h * 8 + 2 * k + (l >> 4))));
        return __fmul_rn(__fmul_rn(rd_f16(rd, b + 208), static_cast<float>(sc)), static_cast<float>(q));
    }
}

// ---- codebook types (IQ1_S, IQ1_M, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S) ----
// A 256-element super-block is eight groups of 32; a group is four runs of eight values; a run is one codebook
// entry of eight bytes (IQ1 / IQ2) or two entries of four bytes (IQ3). `grid` is the caller's codebook in device
// memory (lokal_cuda_set_iq_grid); every lookup is a load that L1 serves after the first touch. Element (group ib,
// run l, value j) exactly as src/gguf/dequant.rs:255-394 index it.
template <int QT>
constexpr bool kIsGridType = QT == LOKAL_IQ1_S || QT == LOKAL_IQ1_M || QT == LOKAL_IQ2_XXS || QT == LOKAL_IQ2_XS ||
                             QT == LOKAL_IQ2_S || QT == LOKAL_IQ3_XXS || QT == LOKAL_IQ3_S;

// ksigns_iq2xs[i]: the 7-bit value with bit 7 set so that the byte has even parity (src/lowmem/iq_grids.rs:12-22).
__device__ __forceinline__ unsigned ksigns_iq2xs(unsigned i) { return i | ((__popc(i) & 1u) << 7); }

template <typename Rd>
__device__ __forceinline__ unsigned rd_u16(const Rd& rd, unsigned off) { return rd(off) | (rd(off + 1) << 8); }

template <int QT, typename Rd>
__device__ __forceinline__ float dequant_grid_elem(const Rd& rd, const void* grid, unsigned col) {
    const unsigned i = col & 255, ib = i >> 5, l = (i >> 3) & 3, j = i & 7;
    const unsigned long long* g64 = static_cast<const unsigned long long*>(grid);
    const unsigned* g32 = static_cast<const unsigned*>(grid);
    auto signed_of = [](float t, unsigned signs, unsigned bit) { return ((signs >> bit) & 1u) ? -t : t; };  // t * (+-1.0)
    if constexpr (QT == LOKAL_IQ1_S) {  // :255-270: d | qs[32] | qh[8 x u16]
        const unsigned b = (col >> 8) * 50;
        const unsigned qh = rd_u16(rd, b + 34 + 2 * ib);
        const float dl = __fmul_rn(rd_f16(rd, b), static_cast<float>(2 * ((qh >> 12) & 7u) + 1));
        const float delta = (qh & 0x8000u) ? -0.125f : 0.125f;
        const unsigned gi = rd(b + 2 + 4 * ib + l) | (((qh >> (3 * l)) & 7u) << 8);
        const int g = static_cast<int>(static_cast<signed char>((__ldg(g64 + gi) >> (8 * j)) & 0xFF));
        return __fmul_rn(dl, __fadd_rn(static_cast<float>(g), delta));
    } else if constexpr (QT == LOKAL_IQ1_M) {  // :274-293: qs[32] | qh[16] | scales[4 x u16], the f16 d in their top nibbles
        const unsigned b = (col >> 8) * 56;
        const unsigned s0 = rd_u16(rd, b + 48), s1 = rd_u16(rd, b + 50), s2 = rd_u16(rd, b + 52), s3 = rd_u16(rd, b + 54);
        const unsigned bits = (s0 >> 12) | ((s1 >> 8) & 0x00F0u) | ((s2 >> 4) & 0x0F00u) | (s3 & 0xF000u);
        const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(bits)));
        const unsigned sw = (ib >> 1) == 0 ? s0 : (ib >> 1) == 1 ? s1 : (ib >> 1) == 2 ? s2 : s3;
        const unsigned shift = 6 * (ib & 1) + (l < 2 ? 0 : 3);
        const float dl = __fmul_rn(d, static_cast<float>(2 * ((sw >> shift) & 7u) + 1));
        const unsigned qh = rd(b + 32 + 2 * ib + (l >> 1));
        const bool even = (l & 1) == 0;
        const unsigned gi = rd(b + 4 * ib + l) | ((qh << (even ? 8 : 4)) & 0x700u);
        const float delta = (qh & (even ? 0x08u : 0x80u)) ? -0.125f : 0.125f;
        const int g = static_cast<int>(static_cast<signed char>((__ldg(g64 + gi) >> (8 * j)) & 0xFF));
        return __fmul_rn(dl, __fadd_rn(static_cast<float>(g), delta));
    } else if constexpr (QT == LOKAL_IQ2_XXS) {  // :295-312: d | 8 x (4 grid bytes, u32: 4 x 7 sign bits + 4-bit scale)
        const unsigned b = (col >> 8) * 66 + 2 + 8 * ib;
        const unsigned a1 = rd_u16(rd, b + 4) | (rd_u16(rd, b + 6) << 16);
        const float db = __fmul_rn(__fmul_rn(rd_f16(rd, (col >> 8) * 66), __fadd_rn(0.5f, static_cast<float>(a1 >> 28))), 0.25f);
        const unsigned g = static_cast<unsigned>(__ldg(g64 + rd(b + l)) >> (8 * j)) & 0xFFu;
        return signed_of(__fmul_rn(db, static_cast<float>(g)), ksigns_iq2xs((a1 >> (7 * l)) & 127u), j);
    } else if constexpr (QT == LOKAL_IQ2_XS || QT == LOKAL_IQ2_S) {  // :314-352: 4-bit scales, two runs to a nibble
        constexpr unsigned BB = QT == LOKAL_IQ2_XS ? 74 : 82, SC = QT == LOKAL_IQ2_XS ? 66 : 74;
        const unsigned b = (col >> 8) * BB;
        const unsigned sc = rd(b + SC + ib);
        const float db = __fmul_rn(__fmul_rn(rd_f16(rd, b), __fadd_rn(0.5f, static_cast<float>(l < 2 ? (sc & 15u) : (sc >> 4)))), 0.25f);
        unsigned gi, signs;
        if constexpr (QT == LOKAL_IQ2_XS) {  // qs[32 x u16]: 9-bit grid index, 7-bit sign selector
            const unsigned qv = rd_u16(rd, b + 2 + 2 * (4 * ib + l));
            gi = qv & 511u;
            signs = ksigns_iq2xs(qv >> 9);
        } else {  // qs[32 grid bytes + 32 sign bytes] | qh[8]: two more index bits
            gi = rd(b + 2 + 4 * ib + l) | ((rd(b + 66 + ib) << (8 - 2 * l)) & 0x300u);
            signs = rd(b + 34 + 4 * ib + l);
        }
        const unsigned g = static_cast<unsigned>(__ldg(g64 + gi) >> (8 * j)) & 0xFFu;
        return signed_of(__fmul_rn(db, static_cast<float>(g)), signs, j);
    } else if constexpr (QT == LOKAL_IQ3_XXS) {  // :354-374: d | qs[64 grid bytes] | 8 x u32 (4 x 7 sign bits + 4-bit scale)
        const unsigned b = (col >> 8) * 98;
        const unsigned aux = rd_u16(rd, b + 66 + 4 * ib) | (rd_u16(rd, b + 68 + 4 * ib) << 16);
        const float db = __fmul_rn(__fmul_rn(rd_f16(rd, b), __fadd_rn(0.5f, static_cast<float>(aux >> 28))), 0.5f);
        const unsigned g = (__ldg(g32 + rd(b + 2 + 8 * ib + 2 * l + (j >> 2))) >> (8 * (j & 3))) & 0xFFu;
        return signed_of(__fmul_rn(db, static_cast<float>(g)), ksigns_iq2xs((aux >> (7 * l)) & 127u), j);
    } else {  // LOKAL_IQ3_S, :376-394: d | qs[64] | qh[8] | signs[32] | scales[4]; qh gives a ninth index bit
        const unsigned b = (col >> 8) * 110, hf = j >> 2;
        const unsigned scb = rd(b + 106 + (ib >> 1));
        const float db = __fmul_rn(rd_f16(rd, b), static_cast<float>(1 + 2 * ((ib & 1) ? (scb >> 4) : (scb & 15u))));
        const unsigned gi = rd(b + 2 + 8 * ib + 2 * l + hf) | ((rd(b + 66 + ib) << (8 - 2 * l - hf)) & 256u);
        const unsigned g = (__ldg(g32 + gi) >> (8 * (j & 3))) & 0xFFu;
        return signed_of(__fmul_rn(db, static_cast<float>(g)), rd(b + 74 + 4 * ib + l), j);
    }
}

// Any quantised type: the arms above, chosen at compile time.
template <int QT, typename Rd>
__device__ __forceinline__ float dequant_any_elem(const Rd& rd, const void* grid, unsigned col) {
    if constexpr (kIsGridType<QT>) return dequant_grid_elem<QT>(rd, grid, col);
    else return dequant_elem<QT>(rd, col);
}

// ---- vector decoders for the staged kernel ----
// EPL (4 or 8) consecutive elements starting at e, e % EPL == 0, of the row staged at `row` in shared memory.
// Such a run never crosses a 16-element sub-group, so it has one scale (and one min), its quants sit in EPL
// consecutive bytes of each plane, and the same shift and mask extract all of them: four elements per 32-bit
// word. The values and the order of the rounded f32 operations are those of dequant_elem above, arm by arm;
// integers become floats through byte_plus_2p23, products and sums go through the packed f32x2 instructions.
// `lut` is the IQ4 codebook as 16 floats in shared memory (one bank each, so a warp's lookups never conflict).
// AT_BLOCK (32-element block types only): `row` already points at the block and e < 32 is the offset inside it; the
// kernel then advances the pointer by a constant per step instead of recomputing (e >> 5) * block_bytes.
// Q4_K / Q5_K in two halves, so that a caller can compute the scales once per row instead of once per step.
// k45_scale_min: d1 = d * sc and -(dmin * m) of 32-element sub-block `sub` of the super-block at b (both f32 products
// rounded once, as the reference computes them). k45_quants: EPL elements starting at element i of the super-block.
__device__ __forceinline__ void k45_scale_min(const unsigned char* b, unsigned sub, float& d1, float& nm1) {
    const unsigned dm = lds_u32(b);  // f16 d, f16 dmin
    const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(dm & 0xFFFF)));
    const float dmin = __half2float(__ushort_as_half(static_cast<unsigned short>(dm >> 16)));
    unsigned sc, mn;
    scale_min_k4(SharedBytes{b}, 4, sub, sc, mn);
    d1 = __fmul_rn(d, static_cast<float>(sc));
    nm1 = -__fmul_rn(dmin, static_cast<float>(mn));
}
template <int QT, int EPL>
__device__ __forceinline__ void k45_quants(const unsigned char* b, unsigned i, float2 d1, float2 nm1, float2 (&y)[EPL / 2]) {
    constexpr unsigned QS = QT == LOKAL_Q4_K ? 16 : 48;
    constexpr float k2p23 = 8388608.0f;
    const unsigned sub = i >> 5, l = i & 31, shift = (i & 32) ? 4u : 0u;
#pragma unroll
    for (int w = 0; w < EPL / 4; w++) {
        unsigned four = (lds_u32(b + QS + (i >> 6) * 32 + l + 4 * w) >> shift) & 0x0F0F0F0Fu;
        if constexpr (QT == LOKAL_Q5_K) four |= ((lds_u32(b + 16 + l + 4 * w) >> sub) & 0x01010101u) << 4;
        float2 f0, f1;
        bytes_to_pairs(four, both(-k2p23), f0, f1);
        y[2 * w] = add2(mul2(d1, f0), nm1);
        y[2 * w + 1] = add2(mul2(d1, f1), nm1);
    }
}

template <int QT, int EPL, bool AT_BLOCK = false>
__device__ __forceinline__ void decode_block(const unsigned char* row, unsigned e, const float* lut, float2 (&y)[EPL / 2]) {
    constexpr int W = EPL / 4;
    constexpr float k2p23 = 8388608.0f;
    if constexpr (QT == LOKAL_Q8_0) {
        const unsigned char* b = AT_BLOCK ? row : row + (e >> 5) * 34;
        const float2 dd = both(lds_f16(b)), nb = both(-(k2p23 + 128.0f));
#pragma unroll
        for (int w = 0; w < W; w++) {
            float2 f0, f1;
            bytes_to_pairs(lds_u32_a2(b + 2 + (e & 31) + 4 * w) ^ 0x80808080u, nb, f0, f1);  // int8 -> biased uint8
            y[2 * w] = mul2(f0, dd);
            y[2 * w + 1] = mul2(f1, dd);
        }
    } else if constexpr (QT == LOKAL_Q4_0 || QT == LOKAL_IQ4_NL || QT == LOKAL_Q5_0) {
        constexpr unsigned BB = QT == LOKAL_Q5_0 ? 22 : 18, QS = QT == LOKAL_Q5_0 ? 6 : 2;
        const unsigned char* b = AT_BLOCK ? row : row + (e >> 5) * BB;
        const unsigned j = e & 31, shift = (j & 16) ? 4u : 0u;
        const float2 dd = both(lds_f16(b));
        unsigned qh = 0;
        if constexpr (QT == LOKAL_Q5_0) qh = lds_u32_a2(b + 2) >> j;  // bit k: fifth bit of element e + k
#pragma unroll
        for (int w = 0; w < W; w++) {
            unsigned four = (lds_u32_a2(b + QS + (j & 15) + 4 * w) >> shift) & 0x0F0F0F0Fu;
            if constexpr (QT == LOKAL_IQ4_NL) {
                y[2 * w] = mul2(dd, make_float2(lut[four & 15u], lut[(four >> 8) & 15u]));
                y[2 * w + 1] = mul2(dd, make_float2(lut[(four >> 16) & 15u], lut[four >> 24]));
            } else {
                if constexpr (QT == LOKAL_Q5_0) four |= ((((qh >> (4 * w)) & 15u) * 0x00204081u) & 0x01010101u) << 4;
                float2 f0, f1;
                bytes_to_pairs(four, both(-(k2p23 + (QT == LOKAL_Q5_0 ? 16.0f : 8.0f))), f0, f1);
                y[2 * w] = mul2(f0, dd);
                y[2 * w + 1] = mul2(f1, dd);
            }
        }
    } else if constexpr (QT == LOKAL_IQ4_XS) {
        const unsigned char* b = row + (e >> 8) * 136;
        const unsigned i = e & 255, ib = i >> 5, j = i & 31, shift = (j & 16) ? 4u : 0u;
        const unsigned hdr = lds_u32(b);  // f16 d, u16 scales_h
        const unsigned ls = ((static_cast<unsigned>(b[4 + (ib >> 1)]) >> (4 * (ib & 1))) & 15u) | ((((hdr >> 16) >> (2 * ib)) & 3u) << 4);
        const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(hdr & 0xFFFF)));
        const float2 dl = both(__fmul_rn(d, static_cast<float>(static_cast<int>(ls) - 32)));
#pragma unroll
        for (int w = 0; w < W; w++) {
            const unsigned four = (lds_u32(b + 8 + 16 * ib + (j & 15) + 4 * w) >> shift) & 0x0F0F0F0Fu;
            y[2 * w] = mul2(dl, make_float2(lut[four & 15u], lut[(four >> 8) & 15u]));
            y[2 * w + 1] = mul2(dl, make_float2(lut[(four >> 16) & 15u], lut[four >> 24]));
        }
    } else if constexpr (QT == LOKAL_Q2_K) {
        const unsigned char* b = row + (e >> 8) * 84;
        const unsigned i = e & 255, nh = i >> 7, j = (i >> 5) & 3, half = (i >> 4) & 1, l = i & 15;
        const unsigned sc = b[nh * 8 + j * 2 + half];
        const unsigned dm = lds_u32(b + 80);  // f16 d, f16 dmin
        const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(dm & 0xFFFF)));
        const float dmin = __half2float(__ushort_as_half(static_cast<unsigned short>(dm >> 16)));
        const float2 dl = both(__fmul_rn(d, static_cast<float>(sc & 15u))), nml = both(-__fmul_rn(dmin, static_cast<float>(sc >> 4)));
#pragma unroll
        for (int w = 0; w < W; w++) {
            float2 f0, f1;
            bytes_to_pairs((lds_u32(b + 16 + nh * 32 + half * 16 + l + 4 * w) >> (2 * j)) & 0x03030303u, both(-k2p23), f0, f1);
            y[2 * w] = add2(mul2(dl, f0), nml);
            y[2 * w + 1] = add2(mul2(dl, f1), nml);
        }
    } else if constexpr (QT == LOKAL_Q3_K) {
        const unsigned char* b = row + (e >> 8) * 110;
        const unsigned i = e & 255, nh = i >> 7, j = (i >> 5) & 3, half = (i >> 4) & 1, l = i & 15;
        const unsigned s = nh * 8 + j * 2 + half, a = s >> 2, k = s & 3;
        const unsigned pb = b[96 + (a & 1) * 4 + k];
        const unsigned lo = (a < 2) ? (pb & 15u) : (pb >> 4);
        const unsigned hi = (static_cast<unsigned>(b[104 + k]) >> (2 * a)) & 3u;
        const float2 dl = both(__fmul_rn(lds_f16(b + 108), static_cast<float>(static_cast<int>(lo | (hi << 4)) - 32)));
#pragma unroll
        for (int w = 0; w < W; w++) {
            const unsigned q = (lds_u32_a2(b + 32 + nh * 32 + half * 16 + l + 4 * w) >> (2 * j)) & 0x03030303u;
            const unsigned hb = (lds_u32_a2(b + half * 16 + l + 4 * w) >> (nh * 4 + j)) & 0x01010101u;
            float2 f0, f1;
            bytes_to_pairs(q | (hb << 2), both(-(k2p23 + 4.0f)), f0, f1);  // q - (hbit ? 0 : 4) = (q + 4 hbit) - 4
            y[2 * w] = mul2(dl, f0);
            y[2 * w + 1] = mul2(dl, f1);
        }
    } else if constexpr (QT == LOKAL_Q4_K || QT == LOKAL_Q5_K) {
        constexpr unsigned BB = QT == LOKAL_Q4_K ? 144 : 176;
        const unsigned char* b = row + (e >> 8) * BB;
        float d1, nm1;
        k45_scale_min(b, (e & 255) >> 5, d1, nm1);
        k45_quants<QT, EPL>(b, e & 255, both(d1), both(nm1), y);
    } else {  // LOKAL_Q6_K
        const unsigned char* b = row + (e >> 8) * 210;
        const unsigned i = e & 255, h = i >> 7, k = (i >> 5) & 3, l = i & 31, shift = (k & 2) ? 4u : 0u;
        const int sc = static_cast<int>(static_cast<signed char>(b[192 + h * 8 + 2 * k + (l >> 4)]));
        const float2 dsc = both(__fmul_rn(lds_f16(b + 208), static_cast<float>(sc)));
#pragma unroll
        for (int w = 0; w < W; w++) {
            const unsigned nib = (lds_u32_a2(b + h * 64 + (k & 1) * 32 + l + 4 * w) >> shift) & 0x0F0F0F0Fu;
            const unsigned hb = (lds_u32_a2(b + 128 + h * 32 + l + 4 * w) >> (2 * k)) & 0x03030303u;
            float2 f0, f1;
            bytes_to_pairs(nib | (hb << 4), both(-(k2p23 + 32.0f)), f0, f1);
            y[2 * w] = mul2(dsc, f0);
            y[2 * w + 1] = mul2(dsc, f1);
        }
    }
}

// Eight f16 outputs of a Q8_0 / Q4_0 / Q5_0 block without leaving half precision, bit-identical to rounding the f32
// result. The reference computes f32(q) * f32(d) with q an integer of at most 8 bits and d an f16 (11 significant
// bits): the product has at most 19 significant bits, so the f32 multiply is EXACT, and the f16 row is the
// nearest-even rounding of that exact product. An IEEE f16 multiply of the same two numbers (q is exact in f16) is
// the nearest-even rounding of the same exact product: the same bits, overflow to infinity and gradual underflow
// included. The integer becomes an f16 the way it becomes an f32 elsewhere in this file: its byte is placed in the low
// mantissa bits of 1024.0 (0x6400) and 1024 + bias is subtracted, both exact. 12 instructions per 8 outputs instead
// of 20 plus the packs. `b` points at the block, `in_block` (0, 8, 16 or 24) is the first element.
template <int QT>
__device__ __forceinline__ uint4 decode_small_block_h8(const unsigned char* b, unsigned in_block) {
    static_assert(QT == LOKAL_Q8_0 || QT == LOKAL_Q4_0 || QT == LOKAL_Q5_0, "types whose value is one exact product");
    const unsigned short dbits = *reinterpret_cast<const unsigned short*>(b);
    const __half2 dd = __half2half2(__ushort_as_half(dbits));
    constexpr float kBias = QT == LOKAL_Q8_0 ? 1152.0f : (QT == LOKAL_Q5_0 ? 1040.0f : 1032.0f);  // 1024 + 128 / 16 / 8
    const __half2 bias = __float2half2_rn(kBias);
    unsigned word[2];
    if constexpr (QT == LOKAL_Q8_0) {
        word[0] = lds_u32_a2(b + 2 + in_block) ^ 0x80808080u;  // int8 -> biased uint8
        word[1] = lds_u32_a2(b + 2 + in_block + 4) ^ 0x80808080u;
    } else {
        constexpr unsigned QS = QT == LOKAL_Q5_0 ? 6 : 2;
        const unsigned shift = (in_block & 16) ? 4u : 0u;
        word[0] = (lds_u32_a2(b + QS + (in_block & 15)) >> shift) & 0x0F0F0F0Fu;
        word[1] = (lds_u32_a2(b + QS + (in_block & 15) + 4) >> shift) & 0x0F0F0F0Fu;
        if constexpr (QT == LOKAL_Q5_0) {
            const unsigned qh = lds_u32_a2(b + 2) >> in_block;  // bit k: fifth bit of element in_block + k
            word[0] |= (((qh & 15u) * 0x00204081u) & 0x01010101u) << 4;
            word[1] |= ((((qh >> 4) & 15u) * 0x00204081u) & 0x01010101u) << 4;
        }
    }
    unsigned out[4];
#pragma unroll
    for (int w = 0; w < 2; w++) {
        const unsigned lo = __byte_perm(word[w], 0x64646464u, 0x4140), hi = __byte_perm(word[w], 0x64646464u, 0x4342);
        const __half2 q0 = __hsub2(*reinterpret_cast<const __half2*>(&lo), bias);
        const __half2 q1 = __hsub2(*reinterpret_cast<const __half2*>(&hi), bias);
        const __half2 y0 = __hmul2(q0, dd), y1 = __hmul2(q1, dd);
        out[2 * w] = *reinterpret_cast<const unsigned*>(&y0);
        out[2 * w + 1] = *reinterpret_cast<const unsigned*>(&y1);
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

// 32 bytes to a 32-byte-aligned address in one store: a lane fills a whole sector.
__device__ __forceinline__ void st_stream32(void* p, const uint4& a, const uint4& b) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x),
                 "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}

// Codebook types in the staged kernel. EPL consecutive elements are half a run (EPL = 4) or one run (EPL = 8): one
// scale, one byte of signs (or one delta), and one 8-byte codebook entry (IQ1 / IQ2) or two 4-byte entries (IQ3),
// fetched once. Same values and rounding order as dequant_grid_elem; a sign is applied by flipping the sign bit,
// which is what multiplying by -1.0 does.
template <int QT, int EPL>
__device__ __forceinline__ void decode_grid_block(const unsigned char* row, unsigned e, const void* grid, float2 (&y)[EPL / 2]) {
    constexpr int W = EPL / 4;
    constexpr float k2p23 = 8388608.0f;
    constexpr bool kIq1 = QT == LOKAL_IQ1_S || QT == LOKAL_IQ1_M, kIq3 = QT == LOKAL_IQ3_XXS || QT == LOKAL_IQ3_S;
    const unsigned i = e & 255, ib = i >> 5, l = (i >> 3) & 3, j0 = i & 7;
    const unsigned long long* g64 = static_cast<const unsigned long long*>(grid);
    const unsigned* g32 = static_cast<const unsigned*>(grid);
    auto u16 = [](const unsigned char* p) { return static_cast<unsigned>(*reinterpret_cast<const unsigned short*>(p)); };
    float scale, delta = 0.0f;
    unsigned signs = 0, gi = 0, gi2 = 0;  // gi2: the second entry of a run (IQ3 only)
    if constexpr (QT == LOKAL_IQ1_S) {
        const unsigned char* b = row + (e >> 8) * 50;
        const unsigned qh = u16(b + 34 + 2 * ib);
        scale = __fmul_rn(lds_f16(b), static_cast<float>(2 * ((qh >> 12) & 7u) + 1));
        delta = (qh & 0x8000u) ? -0.125f : 0.125f;
        gi = b[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7u) << 8);
    } else if constexpr (QT == LOKAL_IQ1_M) {
        const unsigned char* b = row + (e >> 8) * 56;
        const unsigned s01 = lds_u32(b + 48), s23 = lds_u32(b + 52);  // 56-byte blocks keep the scale words 4-byte aligned
        const unsigned bits = ((s01 >> 12) & 0xFu) | ((s01 >> 24) & 0x00F0u) | ((s23 >> 4) & 0x0F00u) | ((s23 >> 16) & 0xF000u);
        const unsigned sw = ((ib & 4) ? s23 : s01) >> ((ib & 2) ? 16 : 0);
        scale = __fmul_rn(__half2float(__ushort_as_half(static_cast<unsigned short>(bits))),
                          static_cast<float>(2 * ((sw >> (6 * (ib & 1) + (l < 2 ? 0 : 3))) & 7u) + 1));
        const unsigned qh = b[32 + 2 * ib + (l >> 1)];
        const bool even = (l & 1) == 0;
        gi = b[4 * ib + l] | ((qh << (even ? 8 : 4)) & 0x700u);
        delta = (qh & (even ? 0x08u : 0x80u)) ? -0.125f : 0.125f;
    } else if constexpr (QT == LOKAL_IQ2_XXS) {
        const unsigned char* b = row + (e >> 8) * 66;
        const unsigned a1 = lds_u32_a2(b + 2 + 8 * ib + 4);
        scale = __fmul_rn(__fmul_rn(lds_f16(b), __fadd_rn(0.5f, static_cast<float>(a1 >> 28))), 0.25f);
        signs = ksigns_iq2xs((a1 >> (7 * l)) & 127u);
        gi = b[2 + 8 * ib + l];
    } else if constexpr (QT == LOKAL_IQ2_XS || QT == LOKAL_IQ2_S) {
        constexpr unsigned BB = QT == LOKAL_IQ2_XS ? 74 : 82, SC = QT == LOKAL_IQ2_XS ? 66 : 74;
        const unsigned char* b = row + (e >> 8) * BB;
        const unsigned sc = b[SC + ib];
        scale = __fmul_rn(__fmul_rn(lds_f16(b), __fadd_rn(0.5f, static_cast<float>(l < 2 ? (sc & 15u) : (sc >> 4)))), 0.25f);
        if constexpr (QT == LOKAL_IQ2_XS) {
            const unsigned qv = u16(b + 2 + 2 * (4 * ib + l));
            gi = qv & 511u;
            signs = ksigns_iq2xs(qv >> 9);
        } else {
            gi = b[2 + 4 * ib + l] | ((static_cast<unsigned>(b[66 + ib]) << (8 - 2 * l)) & 0x300u);
            signs = b[34 + 4 * ib + l];
        }
    } else if constexpr (QT == LOKAL_IQ3_XXS) {
        const unsigned char* b = row + (e >> 8) * 98;
        const unsigned aux = lds_u32_a2(b + 66 + 4 * ib);
        scale = __fmul_rn(__fmul_rn(lds_f16(b), __fadd_rn(0.5f, static_cast<float>(aux >> 28))), 0.5f);
        signs = ksigns_iq2xs((aux >> (7 * l)) & 127u);
        gi = b[2 + 8 * ib + 2 * l];
        gi2 = b[2 + 8 * ib + 2 * l + 1];
    } else {  // LOKAL_IQ3_S
        const unsigned char* b = row + (e >> 8) * 110;
        const unsigned scb = b[106 + (ib >> 1)], qh = b[66 + ib];
        scale = __fmul_rn(lds_f16(b), static_cast<float>(1 + 2 * ((ib & 1) ? (scb >> 4) : (scb & 15u))));
        signs = b[74 + 4 * ib + l];
        gi = b[2 + 8 * ib + 2 * l] | ((qh << (8 - 2 * l)) & 256u);
        gi2 = b[2 + 8 * ib + 2 * l + 1] | ((qh << (7 - 2 * l)) & 256u);
    }
    unsigned word[2];  // values 0..3 and 4..7 of the run, one byte each
    if constexpr (kIq3) {
        if (W == 2 || j0 == 0) word[0] = __ldg(g32 + gi);
        if (W == 2 || j0 != 0) word[1] = __ldg(g32 + gi2);
    } else {
        const unsigned long long entry = __ldg(g64 + gi);
        word[0] = static_cast<unsigned>(entry);
        word[1] = static_cast<unsigned>(entry >> 32);
    }
    const float2 sc2 = both(scale);
#pragma unroll
    for (int w = 0; w < W; w++) {
        const unsigned first = W == 2 ? 4u * w : j0;  // index in the run of this word's first value
        const unsigned bytes = (W == 2) ? word[w] : (j0 ? word[1] : word[0]);
        float2 f0, f1;
        if constexpr (kIq1) {  // signed codebook bytes: dl * (g + delta)
            bytes_to_pairs(bytes ^ 0x80808080u, both(-(k2p23 + 128.0f)), f0, f1);
            y[2 * w] = mul2(sc2, add2(f0, both(delta)));
            y[2 * w + 1] = mul2(sc2, add2(f1, both(delta)));
        } else {  // (db * g) * (+-1)
            bytes_to_pairs(bytes, both(-k2p23), f0, f1);
            f0 = mul2(sc2, f0);
            f1 = mul2(sc2, f1);
            const unsigned sg = signs >> first;
            y[2 * w] = make_float2(__uint_as_float(__float_as_uint(f0.x) ^ ((sg & 1u) << 31)), __uint_as_float(__float_as_uint(f0.y) ^ ((sg & 2u) << 30)));
            y[2 * w + 1] = make_float2(__uint_as_float(__float_as_uint(f1.x) ^ ((sg & 4u) << 29)), __uint_as_float(__float_as_uint(f1.y) ^ ((sg & 8u) << 28)));
        }
    }
}

// Calls f(std::integral_constant<int, type>) for a quantised table type.
template <typename F>
void for_quant_type(int t, F&& f) {
    switch (t) {
#define LOKAL_QT_CASE(T) case T: f(std::integral_constant<int, T>{}); break;
        LOKAL_QT_CASE(LOKAL_Q4_0) LOKAL_QT_CASE(LOKAL_Q5_0) LOKAL_QT_CASE(LOKAL_Q8_0) LOKAL_QT_CASE(LOKAL_Q2_K)
        LOKAL_QT_CASE(LOKAL_Q3_K) LOKAL_QT_CASE(LOKAL_Q4_K) LOKAL_QT_CASE(LOKAL_Q5_K) LOKAL_QT_CASE(LOKAL_Q6_K)
        LOKAL_QT_CASE(LOKAL_IQ4_NL) LOKAL_QT_CASE(LOKAL_IQ4_XS) LOKAL_QT_CASE(LOKAL_IQ1_S) LOKAL_QT_CASE(LOKAL_IQ1_M)
        LOKAL_QT_CASE(LOKAL_IQ2_XXS) LOKAL_QT_CASE(LOKAL_IQ2_XS) LOKAL_QT_CASE(LOKAL_IQ2_S) LOKAL_QT_CASE(LOKAL_IQ3_XXS)
        LOKAL_QT_CASE(LOKAL_IQ3_S)
#undef LOKAL_QT_CASE
        default: break;
    }
}

template <typename OutT>
__device__ __forceinline__ void store_out16(OutT* dst, const float2 (&y)[VecOf<OutT>::N / 2]) {
    st_stream(dst, pack16p<OutT>(y));
}

// ---- staged (bulk-copy) kernel for quantised tables ----
// Stages of a warp's ring. Two is the default: a third stage (copies issued two rows ahead) measured no faster on the
// 65,536-id Zipf gather (Q8_0 to f32 45.2 us against 44.0 us, to f16 27.6 us either way) and costs half as much shared
// memory again per CTA, which lowers the resident CTAs for wide rows.
#ifndef LOKAL_GATHER_STAGES
#define LOKAL_GATHER_STAGES 2
#endif
constexpr unsigned kGatherStages = LOKAL_GATHER_STAGES;
static_assert(kGatherStages >= 2 && kGatherStages <= 4, "the row loop is unrolled by the ring length");

// FUSE: the first RMSNorm of a step in the same launch (MetalSession::run_from encodes `embed` and then
// `rmsnorm` over the same rows, src/gpu/metal.rs:2525, 2552). The warp that has just stored a row x accumulates the
// sum of squares of the values AS STORED (rounded to the row type, what a separate norm launch would read), reads its
// own 16-byte vectors back (they are in L2), and writes xn = (x * scale) * w: one launch and one pass over the table
// row instead of two launches.
template <int QT, typename OutT, bool FUSE = false>
__global__ void __launch_bounds__(256) gather_quant_staged_kernel(const GatherArgs a) {
    pdl_launch();  // the wait for the kernel before this one comes after the shared-memory set-up, which touches no global memory
    constexpr int EPL = VecOf<OutT>::N;
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr unsigned NST = kGatherStages;
    const unsigned warps_per_cta = blockDim.x >> 5;
    const unsigned warp_in_cta = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem);
    unsigned char* stage0 = smem + ((warps_per_cta * NST * 8 + 127u) & ~127u) + warp_in_cta * NST * a.stage_bytes;
    const uint32_t bar0 = smem_addr(&bars[warp_in_cta * NST]);
    if (lane == 0) {
#pragma unroll
        for (unsigned st = 0; st < NST; st++) mbar_init(bar0 + 8 * st, 1);
        mbar_init_fence();
    }
    __syncwarp();
    __shared__ float lut[16];  // the IQ4 codebook as floats; unused by the other block types
    if constexpr (QT == LOKAL_IQ4_NL || QT == LOKAL_IQ4_XS) {
        if (threadIdx.x < 16) lut[threadIdx.x] = iq4_value(threadIdx.x);
        __syncthreads();
    }
    pdl_wait();

    // Rows, ids and the look-ahead are 32-bit values here: a row costs this warp a fixed number of instructions before
    // its first element is decoded, and every lane executes them.
    const unsigned total_warps = gridDim.x * warps_per_cta;
    const unsigned first = blockIdx.x * warps_per_cta + warp_in_cta;
    const unsigned n = a.n32;

    // Ring state of the stages (uniform across the warp), one register per stage and field:
    //   mode    0 = row invalid (zero fill), 1 = bulk copy issued, 2 = bytes already placed by plain loads
    //   parity  phase parity of the stage's mbarrier
    //   offs    offset of the row start inside the 16-byte-aligned window
    // Types with small decoders run the row loop unrolled by the ring length, so every stage number is a constant where
    // it is used and the selects below fold away (Q8_0 to f16 rows: 27.6 -> 25.1 us on the 65,536-id gather). For the
    // large decoders the doubled loop body cost more than it saved (Q4_K to f16: 32.5 -> 34.1 us); they keep one body
    // and pick the stage's registers with selects.
    unsigned mode[NST], parity[NST], offs[NST];
#pragma unroll
    for (unsigned st = 0; st < NST; st++) mode[st] = parity[st] = offs[st] = 0;
    auto sel = [&](const unsigned (&arr)[NST], unsigned st) {
        unsigned v = arr[0];
#pragma unroll
        for (unsigned t = 1; t < NST; t++) v = st == t ? arr[t] : v;
        return v;
    };
    auto put = [&](unsigned (&arr)[NST], unsigned st, unsigned v) {
#pragma unroll
        for (unsigned t = 0; t < NST; t++) arr[t] = st == t ? v : arr[t];
    };
    auto sptr = [&](unsigned st) { return stage0 + st * a.stage_bytes; };
    auto bar = [&](unsigned st) { return bar0 + 8 * st; };

    // The id of a row is fetched one iteration before the row's copy is issued, so the copy never waits for it.
    auto id_of = [&](unsigned i) { return a.ids ? __ldg(a.ids + i) : i; };
    auto issue = [&](unsigned id, unsigned st) {
        if (id > a.max_id) {
            put(mode, st, 0u);
            if (lane == 0) atomicOr(a.err_word, kErrIdRange);
            return;
        }
        const unsigned long long start = static_cast<unsigned long long>(id) * a.row_bytes;  // one widening multiply
        const unsigned off = static_cast<unsigned>(start) & 15u;
        put(offs, st, off);
        if (id < a.bulk_ids) {
            put(mode, st, 1u);
            if (lane == 0) {
                const unsigned bytes = (off + a.row_bytes + 15u) & ~15u;
                mbar_expect_tx(bar(st), bytes + a.extra_tx);
                if (a.table_keep) bulk_copy_g2s_l2(smem_addr(sptr(st)), a.table + (start - off), bytes, bar(st), l2_policy_keep());
                else bulk_copy_g2s(smem_addr(sptr(st)), a.table + (start - off), bytes, bar(st));
            }
        } else {
            // The window would run past the end of the table (last row only): plain byte loads.
            put(mode, st, 2u);
            unsigned char* dst = sptr(st) + off;
            for (unsigned bidx = lane; bidx < a.row_bytes; bidx += 32) dst[bidx] = __ldg(a.table + start + bidx);
        }
    };

    // Decodes the row waiting in stage st into output row i; false when the bounded wait on its copy gave up.
    auto consume = [&](unsigned i, unsigned st) -> bool {
        OutT* orow = reinterpret_cast<OutT*>(a.out) + static_cast<unsigned long long>(i) * a.dim;
        float2 ssq = make_float2(0.0f, 0.0f);  // FUSE: this lane's sum of squares of the row as stored
        // one 16-byte vector of the row: stored, and (FUSE) its stored values squared and summed
        auto emit = [&](unsigned e, const uint4& pk) {
            st_stream(orow + e, pk);
            if constexpr (FUSE) {
                float2 r[EPL / 2];
                unpack16p<OutT>(pk, r);
#pragma unroll
                for (int k = 0; k < EPL / 2; k++) {
                    if (sizeof(OutT) == 2) ssq = fma2(r[k], r[k], ssq);
                    else ssq = add2(ssq, mul2(r[k], r[k]));
                }
            }
        };
        const unsigned m = sel(mode, st);
        if (m == 1) {
            const unsigned ph = sel(parity, st);
            // Every lane polls for itself, and every lane whose polls run out reports it (the polls of a warp end
            // together unless completion falls on the very last one; the lanes that leave are exited threads to the
            // warp-wide operations of those that go on, and the error word says the launch's output is not to be used).
            if (!mbar_wait_bounded(bar(st), ph, a.wait_limit)) {
                atomicOr(a.err_word, kErrTimeout);
                // give the copies still in flight one more bounded chance to land before leaving
#pragma unroll
                for (unsigned t = 0; t < NST; t++) {
                    if (mode[t] == 1) mbar_wait_bounded(bar(t), parity[t], a.wait_limit);
                }
                return false;
            }
            put(parity, st, ph ^ 1u);
        } else if (m == 2) {
            __syncwarp();
        }
        if (m == 0) {
            float2 z[EPL / 2];
#pragma unroll
            for (int k = 0; k < EPL / 2; k++) z[k] = make_float2(0.0f, 0.0f);
            for (unsigned e = lane * EPL; e < a.dim; e += 32 * EPL) emit(e, pack16p<OutT>(z));
        } else {
            const unsigned char* row = sptr(st) + sel(offs, st);
            constexpr unsigned kSmallBlock = QT == LOKAL_Q8_0 ? 34u : (QT == LOKAL_Q5_0 ? 22u : ((QT == LOKAL_Q4_0 || QT == LOKAL_IQ4_NL) ? 18u : 0u));
            if constexpr (kSmallBlock != 0) {
                // 32-element blocks: a lane's offset inside its block never changes, and every step moves it EPL blocks on
                const unsigned char* bp = row + ((lane * EPL) >> 5) * kSmallBlock;
                const unsigned in_block = (lane * EPL) & 31u;
                constexpr bool kHalfPath = std::is_same<OutT, __half>::value && (QT == LOKAL_Q8_0 || QT == LOKAL_Q4_0 || QT == LOKAL_Q5_0);
                for (unsigned e = lane * EPL; e < a.dim; e += 32 * EPL, bp += EPL * kSmallBlock) {
                    if constexpr (kHalfPath) {
                        emit(e, decode_small_block_h8<QT>(bp, in_block));
                    } else {
                        float2 y[EPL / 2];
                        decode_block<QT, EPL, true>(bp, in_block, lut, y);
                        emit(e, pack16p<OutT>(y));
                    }
                }
            } else {
                bool done = false;
                if constexpr (QT == LOKAL_Q4_K || QT == LOKAL_Q5_K) {
                    // Rows of at most 32 sub-blocks (1024 elements): lane j works out the scale and min of sub-block j
                    // once, and each step fetches the pair of its own sub-block with two shuffles instead of
                    // recomputing them (the 6-bit unpacking and two products are a third of a step's instructions).
                    // a.dim is a multiple of 256 and a step covers 128 or 256 elements, so all lanes take the same
                    // number of steps and every shuffle is executed by the whole warp.
                    if (a.dim <= 1024u) {
                        constexpr unsigned BB = QT == LOKAL_Q4_K ? 144 : 176;
                        float d1 = 0.0f, nm1 = 0.0f;
                        if (lane * 32u < a.dim) k45_scale_min(row + (lane >> 3) * BB, lane & 7u, d1, nm1);
                        if constexpr (EPL == 8) {
                            // 16-bit rows: a step is one whole super-block, so a lane's place inside the super-block
                            // (lane * 8) never changes: only the block pointer and the shuffle source move
                            const unsigned char* bp = row;
                            unsigned src_lane = lane >> 2;
                            for (unsigned e = lane * EPL; e < a.dim; e += 256, bp += BB, src_lane += 8) {
                                const float d1s = __shfl_sync(0xffffffffu, d1, src_lane), nm1s = __shfl_sync(0xffffffffu, nm1, src_lane);
                                float2 y[EPL / 2];
                                k45_quants<QT, EPL>(bp, lane * 8u, both(d1s), both(nm1s), y);
                                emit(e, pack16p<OutT>(y));
                            }
                        } else {
                            for (unsigned e = lane * EPL; e < a.dim; e += 32 * EPL) {
                                const float d1s = __shfl_sync(0xffffffffu, d1, e >> 5), nm1s = __shfl_sync(0xffffffffu, nm1, e >> 5);
                                float2 y[EPL / 2];
                                k45_quants<QT, EPL>(row + (e >> 8) * BB, e & 255u, both(d1s), both(nm1s), y);
                                emit(e, pack16p<OutT>(y));
                            }
                        }
                        done = true;
                    }
                }
                if constexpr (kIsGridType<QT> && sizeof(OutT) == 4 && !FUSE) {
                    // f32 rows of the codebook types: a lane takes a whole run of eight values (one scale, one byte of
                    // signs or one delta, one codebook entry) instead of half a run, which halves the index and scale
                    // work per value, and stores its 32 bytes as one sector where the rows are 32-byte aligned.
                    // a.dim is a multiple of 256 for these types, so a step of 256 values never overruns the row.
                    for (unsigned e = lane * 8u; e < a.dim; e += 256u) {
                        float2 y[4];
                        decode_grid_block<QT, 8>(row, e, a.grid, y);
                        const uint4 lo = make_uint4(__float_as_uint(y[0].x), __float_as_uint(y[0].y), __float_as_uint(y[1].x), __float_as_uint(y[1].y));
                        const uint4 hi = make_uint4(__float_as_uint(y[2].x), __float_as_uint(y[2].y), __float_as_uint(y[3].x), __float_as_uint(y[3].y));
                        if (a.out32) {
                            st_stream32(orow + e, lo, hi);
                        } else {
                            st_stream(orow + e, lo);
                            st_stream(orow + e + 4, hi);
                        }
                    }
                    done = true;
                }
                if (!done) {
                    for (unsigned e = lane * EPL; e < a.dim; e += 32 * EPL) {
                        float2 y[EPL / 2];
                        if constexpr (kIsGridType<QT>) decode_grid_block<QT, EPL>(row, e, a.grid, y);
                        else decode_block<QT, EPL>(row, e, lut, y);
                        emit(e, pack16p<OutT>(y));
                    }
                }
            }
        }
        __syncwarp();  // every lane is done with the stage before it is refilled
        put(mode, st, 0u);
        if constexpr (FUSE) {
            // xn = (x * scale) * w over the row this warp has just stored; each lane reads back its own vectors
            const float ss = warp_sum(ssq.x + ssq.y);
            const float scale = inv_rms<OutT>(ss, static_cast<float>(a.dim), a.inv_dim, a.eps);
            const float2 s2 = make_float2(scale, scale);
            OutT* nrow = reinterpret_cast<OutT*>(a.xn) + static_cast<unsigned long long>(i) * a.dim;
            for (unsigned e = lane * EPL; e < a.dim; e += 32 * EPL) {
                float2 v[EPL / 2], y[EPL / 2];
                unpack16p<OutT>(*reinterpret_cast<const uint4*>(orow + e), v);
                float wf[EPL];
                load_w<EPL>(a.norm_w, a.w_dtype, e, a.w_vec_ok, wf);
#pragma unroll
                for (int k = 0; k < EPL / 2; k++) y[k] = mul2(mul2(v[k], s2), make_float2(wf[2 * k], wf[2 * k + 1]));
                st_stream(nrow + e, pack16p<OutT>(y));
            }
        }
        return true;
    };

    // Prologue: the copies of this warp's first NST - 1 rows are in flight before the first one is decoded, and the
    // id of the row after them is on its way.
    unsigned id_next = 0;
    {
        unsigned r = first;
#pragma unroll
        for (unsigned st = 0; st + 1 < NST; st++, r += total_warps) {
            if (r < n) issue(id_of(r), st);
        }
        if (r < n) id_next = id_of(r);
    }
    constexpr bool kUnrollRing = QT == LOKAL_Q8_0 || QT == LOKAL_Q5_0 || QT == LOKAL_Q4_0 || QT == LOKAL_IQ4_NL;
    auto step = [&](unsigned i, unsigned st) {  // row i waits in stage st; the copy issued now goes to the stage before it
        const unsigned ahead = i + (NST - 1) * total_warps;  // n <= 2^30 and a grid has fewer than 2^20 warps: no wrap
        if (ahead < n) {
            issue(id_next, (st + NST - 1) % NST);
            if (ahead + total_warps < n) id_next = id_of(ahead + total_warps);
        }
        return consume(i, st);
    };
    unsigned i = first;
    if constexpr (kUnrollRing) {
        while (i < n) {
#pragma unroll
            for (unsigned st = 0; st < NST; st++) {
                if (i >= n) break;
                if (!step(i, st)) return;
                i += total_warps;
            }
        }
    } else {
        for (unsigned st = 0; i < n; i += total_warps, st = (st + 1 == NST) ? 0u : st + 1) {
            if (!step(i, st)) return;
        }
    }
}

// ---- staged kernel, two rows per warp: 16-bit output rows ----
// A row costs its warp a fixed ~120 instructions of bookkeeping (id, window, copy, wait, pointers) whatever its
// length, and a 16-byte store of 16-bit values covers eight elements, so a warp finishes a 1024-element row in four
// steps: for the embedding widths in use the bookkeeping is half of all instructions (measured: 157 / 260 / 392
// instructions per row for Q8_0 rows of 256 / 896 / 2048 elements to f16, whatever the ids; two rows per warp:
// 110 / 201 / 354). Narrow rows and the K-quants gain from sharing it (Q4_K, 1024 wide, to f16: 28.5 -> 27.0 us;
// 256-wide Q8_0 rows 16.3 -> 14.2 us); 896-wide Q8_0 rows, bound by the SM's store path as much as by issue, stay
// where they were. Here each half of the warp owns a row: lanes 0-15 row 2p, lanes 16-31 row 2p + 1. The
// bookkeeping instructions are the same ones, executed once for both rows with per-half values (ids, windows and
// pointers differ by lane); lanes 0 and 16 issue their rows' copies in one instruction each, both against the one
// mbarrier of the stage (two arrivals: a lane whose row needs no copy arrives with zero bytes, so every issued stage
// completes and the wait stays warp-uniform). Same decoders, same values, same stores as the kernel above.
//   mode of a half's row in a stage: 0 = id out of range (zero fill), 1 = bulk copy issued, 2 = bytes placed by plain
//   loads, 3 = no row (the half past the last row of an odd count)
template <int QT, typename OutT>
__global__ void __launch_bounds__(256) gather_quant_pair_kernel(const GatherArgs a) {
    pdl_launch();  // the wait for the kernel before this one comes after the shared-memory set-up
    constexpr int EPL = VecOf<OutT>::N;
    static_assert(EPL == 8, "two rows per warp are for 16-bit output rows");
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr unsigned NST = kGatherStages;
    const unsigned warps_per_cta = blockDim.x >> 5;
    const unsigned warp_in_cta = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const unsigned half = lane >> 4, l16 = lane & 15u;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem);
    // this lane's row buffer of stage 0; stage st lies 2 * st * stage_bytes further on
    unsigned char* stage0 = smem + ((warps_per_cta * NST * 8 + 127u) & ~127u) + (warp_in_cta * NST * 2u + half) * a.stage_bytes;
    const uint32_t bar0 = smem_addr(&bars[warp_in_cta * NST]);
    if (lane == 0) {
#pragma unroll
        for (unsigned st = 0; st < NST; st++) mbar_init(bar0 + 8 * st, 2);
        mbar_init_fence();
    }
    __syncwarp();
    __shared__ float lut[16];  // the IQ4 codebook as floats; unused by the other block types
    if constexpr (QT == LOKAL_IQ4_NL || QT == LOKAL_IQ4_XS) {
        if (threadIdx.x < 16) lut[threadIdx.x] = iq4_value(threadIdx.x);
        __syncthreads();
    }
    pdl_wait();

    const unsigned total_warps = gridDim.x * warps_per_cta;
    const unsigned first = blockIdx.x * warps_per_cta + warp_in_cta;  // pairs are dealt to warps grid-stride
    const unsigned n = a.n32, n_pairs = (n + 1u) >> 1;

    unsigned mode[NST], parity[NST], offs[NST];  // mode and offs differ between the halves, parity does not
#pragma unroll
    for (unsigned st = 0; st < NST; st++) {
        mode[st] = 3u;
        parity[st] = offs[st] = 0;
    }
    auto sel = [&](const unsigned (&arr)[NST], unsigned st) {
        unsigned v = arr[0];
#pragma unroll
        for (unsigned t = 1; t < NST; t++) v = st == t ? arr[t] : v;
        return v;
    };
    auto put = [&](unsigned (&arr)[NST], unsigned st, unsigned v) {
#pragma unroll
        for (unsigned t = 0; t < NST; t++) arr[t] = st == t ? v : arr[t];
    };
    auto sptr = [&](unsigned st) { return stage0 + st * 2u * a.stage_bytes; };
    auto bar = [&](unsigned st) { return bar0 + 8 * st; };

    // id of this half's row of pair p (the value is unused when the row does not exist)
    auto id_of = [&](unsigned p) {
        const unsigned i = 2u * p + half;
        const unsigned ic = i < n ? i : n - 1u;
        return a.ids ? __ldg(a.ids + ic) : ic;
    };
    auto issue = [&](unsigned p, unsigned id, unsigned st) {
        unsigned m = 3u, off = 0, bytes = 0;
        unsigned long long start = 0;
        if (2u * p + half < n) {
            if (id > a.max_id) {
                m = 0u;
                if (l16 == 0) atomicOr(a.err_word, kErrIdRange);
            } else {
                start = static_cast<unsigned long long>(id) * a.row_bytes;
                off = static_cast<unsigned>(start) & 15u;
                m = id < a.bulk_ids ? 1u : 2u;
            }
        }
        put(offs, st, off);
        put(mode, st, m);
        if (l16 == 0) {
            if (m == 1u) bytes = (off + a.row_bytes + 15u) & ~15u;
            mbar_expect_tx(bar(st), m == 1u ? bytes + a.extra_tx : 0u);  // an arrival either way
            if (m == 1u) {
                if (a.table_keep) bulk_copy_g2s_l2(smem_addr(sptr(st)), a.table + (start - off), bytes, bar(st), l2_policy_keep());
                else bulk_copy_g2s(smem_addr(sptr(st)), a.table + (start - off), bytes, bar(st));
            }
        }
        if (m == 2u) {  // the window would run past the end of the table (last row only): plain byte loads
            unsigned char* dst = sptr(st) + off;
            for (unsigned bidx = l16; bidx < a.row_bytes; bidx += 16) dst[bidx] = __ldg(a.table + start + bidx);
        }
    };

    // Decodes the rows waiting in stage st into output rows 2p and 2p + 1; false when the bounded wait gave up.
    auto consume = [&](unsigned p, unsigned st) -> bool {
        const unsigned ph = sel(parity, st);
        // every lane polls for itself, and every lane whose polls run out reports it (see the kernel above)
        if (!mbar_wait_bounded(bar(st), ph, a.wait_limit)) {
            atomicOr(a.err_word, kErrTimeout);
            // give the copies still in flight one more bounded chance to land before leaving
#pragma unroll
            for (unsigned t = 0; t < NST; t++) {
                if (t != st && mode[t] == 1u) mbar_wait_bounded(bar(t), parity[t], a.wait_limit);  // the half whose copy it is waits
            }
            return false;
        }
        put(parity, st, ph ^ 1u);
        __syncwarp();  // bytes placed by plain loads are visible to the half that reads them
        const unsigned m = sel(mode, st);
        OutT* orow = reinterpret_cast<OutT*>(a.out) + static_cast<unsigned long long>(2u * p + half) * a.dim;
        const unsigned char* row = sptr(st) + sel(offs, st);
        auto generic_row = [&]() {
            for (unsigned e = l16 * EPL; e < a.dim; e += 16 * EPL) {
                float2 y[EPL / 2];
                if constexpr (kIsGridType<QT>) decode_grid_block<QT, EPL>(row, e, a.grid, y);
                else decode_block<QT, EPL>(row, e, lut, y);
                st_stream(orow + e, pack16p<OutT>(y));
            }
        };
        if (__all_sync(0xffffffffu, m == 1u || m == 2u)) {  // both rows are there: the usual case, no divergence
            constexpr unsigned kSmallBlock = QT == LOKAL_Q8_0 ? 34u : (QT == LOKAL_Q5_0 ? 22u : ((QT == LOKAL_Q4_0 || QT == LOKAL_IQ4_NL) ? 18u : 0u));
            if constexpr (kSmallBlock != 0) {
                // 32-element blocks: a lane's offset inside its block never changes, and every step moves it four blocks on
                const unsigned char* bp = row + (l16 >> 2) * kSmallBlock;
                const unsigned in_block = (l16 * EPL) & 31u;
                constexpr bool kHalfPath = std::is_same<OutT, __half>::value && (QT == LOKAL_Q8_0 || QT == LOKAL_Q4_0 || QT == LOKAL_Q5_0);
                for (unsigned e = l16 * EPL; e < a.dim; e += 16 * EPL, bp += 4 * kSmallBlock) {
                    if constexpr (kHalfPath) {
                        st_stream(orow + e, decode_small_block_h8<QT>(bp, in_block));
                    } else {
                        float2 y[EPL / 2];
                        decode_block<QT, EPL, true>(bp, in_block, lut, y);
                        st_stream(orow + e, pack16p<OutT>(y));
                    }
                }
            } else if constexpr (QT == LOKAL_Q4_K || QT == LOKAL_Q5_K) {
                if (a.dim <= 1024u) {
                    // Lane l of a half works out the scale and min of sub-blocks l and l + 16 of its row once; a step
                    // (half a super-block per half-warp) fetches the pair of its sub-block with two shuffles. a.dim is a
                    // multiple of 256, so every lane takes the same number of steps and all 32 execute every shuffle.
                    constexpr unsigned BB = QT == LOKAL_Q4_K ? 144 : 176;
                    float d1a = 0.0f, nm1a = 0.0f, d1b = 0.0f, nm1b = 0.0f;
                    if (l16 * 32u < a.dim) k45_scale_min(row + (l16 >> 3) * BB, l16 & 7u, d1a, nm1a);
                    if ((l16 + 16u) * 32u < a.dim) k45_scale_min(row + ((l16 + 16u) >> 3) * BB, l16 & 7u, d1b, nm1b);
                    const unsigned src = (lane & 16u) + (l16 >> 2);
                    const unsigned char* bp = row;
                    for (unsigned k = 0, e = l16 * EPL; e < a.dim; k += 2, e += 256, bp += BB) {
                        const float pd = k >= 4 ? d1b : d1a, pm = k >= 4 ? nm1b : nm1a;  // sub-blocks 16.. live in the second slot
#pragma unroll
                        for (unsigned h = 0; h < 2; h++) {
                            const unsigned from = src + 4u * ((k + h) & 3u);
                            const float ds = __shfl_sync(0xffffffffu, pd, from), ms = __shfl_sync(0xffffffffu, pm, from);
                            float2 y[EPL / 2];
                            k45_quants<QT, EPL>(bp, l16 * EPL + 128u * h, both(ds), both(ms), y);
                            st_stream(orow + e + 128u * h, pack16p<OutT>(y));
                        }
                    }
                } else {
                    generic_row();
                }
            } else {
                generic_row();
            }
        } else if (m == 0u) {
            float2 z[EPL / 2];
#pragma unroll
            for (int k = 0; k < EPL / 2; k++) z[k] = make_float2(0.0f, 0.0f);
            for (unsigned e = l16 * EPL; e < a.dim; e += 16 * EPL) st_stream(orow + e, pack16p<OutT>(z));
        } else if (m != 3u) {
            generic_row();
        }
        __syncwarp();  // every lane is done with the stage before it is refilled
        put(mode, st, 3u);
        return true;
    };

    // Prologue: the copies of this warp's first NST - 1 pairs are in flight before the first one is decoded, and the
    // ids of the pair after them are on their way.
    unsigned id_next = 0;
    {
        unsigned r = first;
#pragma unroll
        for (unsigned st = 0; st + 1 < NST; st++, r += total_warps) {
            if (r < n_pairs) issue(r, id_of(r), st);
        }
        if (r < n_pairs) id_next = id_of(r);
    }
    constexpr bool kUnrollRing = QT == LOKAL_Q8_0 || QT == LOKAL_Q5_0 || QT == LOKAL_Q4_0 || QT == LOKAL_IQ4_NL;
    auto step = [&](unsigned p, unsigned st) {  // pair p waits in stage st; the copies issued now go to the stage before it
        const unsigned ahead = p + (NST - 1) * total_warps;
        if (ahead < n_pairs) {
            issue(ahead, id_next, (st + NST - 1) % NST);
            if (ahead + total_warps < n_pairs) id_next = id_of(ahead + total_warps);
        }
        return consume(p, st);
    };
    unsigned p = first;
    if constexpr (kUnrollRing) {
        while (p < n_pairs) {
#pragma unroll
            for (unsigned st = 0; st < NST; st++) {
                if (p >= n_pairs) break;
                if (!step(p, st)) return;
                p += total_warps;
            }
        }
    } else {
        for (unsigned st = 0; p < n_pairs; p += total_warps, st = (st + 1 == NST) ? 0u : st + 1) {
            if (!step(p, st)) return;
        }
    }
}

// ---- plain kernel for quantised tables: any alignment, any row size ----
// One warp per row, one element per lane step, byte loads straight from global
// memory (the per-element index form of src/gpu/kernels.metal:77-81, 889-904).
template <int QT, typename OutT>
__global__ void __launch_bounds__(256) gather_quant_plain_kernel(const GatherArgs a) {
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
    const GlobalBytes rd{a.table + id * a.row_bytes};
    for (unsigned e = lane; e < a.dim; e += 32) orow[e] = from_f32<OutT>(dequant_any_elem<QT>(rd, a.grid, e));
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
        // Four source vectors per lane are loaded before the first of them is stored, so a row of up to 4 x 512 bytes
        // costs its warp one memory round trip instead of one per vector.
        constexpr unsigned kAhead = 4;
        const unsigned long long pol = a.table_keep ? l2_policy_keep() : 0ull;
        for (unsigned e0 = lane * N; e0 < a.dim; e0 += kAhead * 32 * N) {
            uint4 v[kAhead];
#pragma unroll
            for (unsigned j = 0; j < kAhead; j++) {
                const unsigned e = e0 + j * 32 * N;
                // all-zero bits are 0.0 in every source type; table rows carry the high L2 eviction priority (a.table_keep)
                v[j] = (valid && e < a.dim) ? (a.table_keep ? ld_keep_l2(row + e, pol) : ld_keep(row + e)) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (unsigned j = 0; j < kAhead; j++) {
                const unsigned e = e0 + j * 32 * N;
                if (e >= a.dim) break;
                float f[N];
                unpack16<SrcT>(v[j], f);
                constexpr int ON = VecOf<OutT>::N;
                if (ON == N) {
                    float g[ON];
#pragma unroll
                    for (int k = 0; k < ON; k++) g[k] = f[k % N];
                    st_stream(orow + e, pack16<OutT>(g));
                } else if (ON < N) {  // 16-bit source, f32 out: 32 bytes per lane, one store where the rows are 32-byte aligned
                    float g0[ON], g1[ON];
#pragma unroll
                    for (int k = 0; k < ON; k++) {
                        g0[k] = f[k % N];
                        g1[k] = f[(ON + k) % N];
                    }
                    if (a.out32) {
                        st_stream32(orow + e, pack16<OutT>(g0), pack16<OutT>(g1));
                    } else {
                        st_stream(orow + e, pack16<OutT>(g0));
                        st_stream(orow + e + ON, pack16<OutT>(g1));
                    }
                } else {  // f32 source, 16-bit out: 4 elements = 8 bytes
#pragma unroll
                    for (int k = 0; k < N; k++) orow[e + k] = from_f32<OutT>(f[k]);
                }
            }
        }
    } else {
        for (unsigned e = lane; e < a.dim; e += 32) orow[e] = from_f32<OutT>(valid ? to_f32<SrcT>(row[e]) : 0.0f);
    }
}

// Returns through *fused whether the norm went into the gather launch (quantised table, staged kernel); the caller
// launches the norm itself otherwise.
template <typename OutT>
int launch_out(lokal_cuda_ctx* ctx, cudaStream_t s, GatherArgs a, int ggml_type, bool aligned, bool* fused) {
    if (fused) *fused = false;
    const unsigned long long row_warps_blocks = (a.n + 7) / 8;
    if (row_warps_blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather: too many rows for one launch");
    if (ggml_type == LOKAL_F32 || ggml_type == LOKAL_F16 || ggml_type == LOKAL_BF16) {
        const size_t ses = type_size(ggml_type);
        const int vec_ok = aligned && (static_cast<size_t>(a.dim) * ses) % 16 == 0 &&
                           (static_cast<size_t>(a.dim) * sizeof(OutT)) % 16 == 0;
        const unsigned grid = static_cast<unsigned>(row_warps_blocks);
        a.out32 = (reinterpret_cast<uintptr_t>(a.out) % 32 == 0 && (static_cast<size_t>(a.dim) * sizeof(OutT)) % 32 == 0) ? 1u : 0u;
        if (ggml_type == LOKAL_F32) launch_k(gather_float_kernel<float, OutT>, grid, 256, 0, s, a, vec_ok);
        else if (ggml_type == LOKAL_F16) launch_k(gather_float_kernel<__half, OutT>, grid, 256, 0, s, a, vec_ok);
        else launch_k(gather_float_kernel<__nv_bfloat16, OutT>, grid, 256, 0, s, a, vec_ok);
        LOKAL_CHECK_LAUNCH(ctx, "gather_float_kernel");
        return LOKAL_OK;
    }
    // quantised table
    const unsigned warps = 8;
    a.stage_bytes = ((a.row_bytes + 15u) & ~15u) + 32u;
    const bool fuse = a.norm_w != nullptr;
    // 16-bit rows: two rows per warp (gather_quant_pair_kernel), unless the norm is fused into the launch or the doubled
    // staging area does not fit. LOKAL_CUDA_GATHER_PAIR=0 keeps one row per warp.
    bool pair = sizeof(OutT) == 2 && !fuse && tune_env("LOKAL_CUDA_GATHER_PAIR", 1) != 0;
    auto smem_of = [&](bool two) {
        return ((warps * kGatherStages * 8 + 127u) & ~127u) + static_cast<size_t>(warps) * kGatherStages * (two ? 2u : 1u) * a.stage_bytes;
    };
    if (pair && smem_of(true) > 200u * 1024u) pair = false;
    const size_t smem = smem_of(pair);
    const bool staged = aligned && smem <= 200u * 1024u && (a.row_bytes % 2 == 0);
    if (!staged) {
        for_quant_type(ggml_type, [&](auto qt) {
            launch_k(gather_quant_plain_kernel<decltype(qt)::value, OutT>, static_cast<unsigned>(row_warps_blocks), 256, 0, s, a);
        });
        LOKAL_CHECK_LAUNCH(ctx, "gather_quant_plain_kernel");
        return LOKAL_OK;
    }
    void (*kern)(const GatherArgs) = nullptr;
    if constexpr (sizeof(OutT) == 2) {
        if (pair) for_quant_type(ggml_type, [&](auto qt) { kern = gather_quant_pair_kernel<decltype(qt)::value, OutT>; });
    }
    if (!pair) {
        if (fuse) for_quant_type(ggml_type, [&](auto qt) { kern = gather_quant_staged_kernel<decltype(qt)::value, OutT, true>; });
        else for_quant_type(ggml_type, [&](auto qt) { kern = gather_quant_staged_kernel<decltype(qt)::value, OutT, false>; });
    }
    if (fused) *fused = fuse;
    if (smem > 48u * 1024u) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return ctx->fail(LOKAL_ERR_CUDA, "embed_gather: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    // Grid: 16 CTAs per SM for 16-bit rows, 24 for f32 rows, each warp walking a
    // grid-stride list of rows or row pairs. That is more than are resident at once (a decoder of 40-48 registers holds
    // five or six 256-thread CTAs per SM), and measured better than a grid of exactly the resident CTAs: later CTAs
    // start as earlier ones finish and even out the tail (Q8_0 to f16 rows: 25.4 against 28.0 us). Measured on the
    // 65,536-id gather, CTAs per SM 8 / 12 / 16 / 24: Q8_0 to f16 26.1 / 25.7 / 24.5 / 24.2 us and Q4_K to f16
    // 27.0 / 25.6 / 26.0 / 27.0 us with two rows per warp; Q8_0 / Q4_K / Q6_K to f32 45.7 / 49.5 / 49.4 us at 8 and
    // 41.2 / 45.4 / 46.4 us at 24. LOKAL_CUDA_GATHER_CTAS_PER_SM overrides.
    const unsigned want_per_sm = sizeof(OutT) == 4 ? 24u : 16u;
    unsigned per_sm = want_per_sm;  // CTAs of the grid per SM, not resident ones: wide rows simply run in more waves
    const long forced_ctas = tune_env("LOKAL_CUDA_GATHER_CTAS_PER_SM", 0);
    if (forced_ctas >= 1 && forced_ctas <= 64) per_sm = static_cast<unsigned>(forced_ctas);
    // The kernel counts rows and ids in 32 bits. ids are 32-bit values already; `bulk_ids` says which of them may be
    // fetched as a 16-byte-aligned window without reading past the table (every row but, when the table's size is
    // not a multiple of 16, the last); and a call of more than 2^30 rows goes out as several launches over
    // consecutive slices of ids and output (LOKAL_CUDA_GATHER_CHUNK_ROWS lowers the slice for a test). Without ids
    // (row i of the table to row i of the output) a slice also moves the table pointer, so that ids stay below 2^30.
    a.max_id = static_cast<unsigned>((a.vocab < (1ull << 32) ? a.vocab : (1ull << 32)) - 1ull);
    unsigned long long chunk = 1ull << 30;
    const long forced_chunk = tune_env("LOKAL_CUDA_GATHER_CHUNK_ROWS", 0);
    if (forced_chunk >= 1 && static_cast<unsigned long long>(forced_chunk) < chunk) chunk = static_cast<unsigned long long>(forced_chunk);
    const unsigned long long n_all = a.n;
    for (unsigned long long off = 0; off < n_all; off += chunk) {
        GatherArgs c = a;
        c.n = n_all - off < chunk ? n_all - off : chunk;
        c.n32 = static_cast<unsigned>(c.n);
        c.out = static_cast<OutT*>(a.out) + off * a.dim;
        c.out32 = (reinterpret_cast<uintptr_t>(c.out) % 32 == 0 && (static_cast<size_t>(a.dim) * sizeof(OutT)) % 32 == 0) ? 1u : 0u;
        if (a.xn) c.xn = static_cast<OutT*>(a.xn) + off * a.dim;
        if (a.ids) {
            c.ids = a.ids + off;
        } else {  // row i of the table to row i of the output (n <= vocab, checked by the caller)
            c.table = a.table + off * a.row_bytes;
            c.vocab = a.vocab - off;
            c.table_bytes = a.table_bytes - off * a.row_bytes;
            c.max_id = static_cast<unsigned>((c.vocab < (1ull << 32) ? c.vocab : (1ull << 32)) - 1ull);
        }
        // ids whose window [start & ~15, (start + row_bytes + 15) & ~15) ends inside the table: counted down from the last
        unsigned long long bulk = c.vocab;
        while (bulk > 0 && ((bulk * c.row_bytes + 15ull) & ~15ull) > c.table_bytes) bulk--;
        if ((reinterpret_cast<uintptr_t>(c.table) & 15u) != 0) bulk = 0;  // a moved table pointer off the 16-byte grid: plain loads
        c.bulk_ids = bulk > 0xffffffffull ? 0xffffffffu : static_cast<unsigned>(bulk);
        const unsigned long long blocks = ((pair ? (c.n + 1) / 2 : c.n) + warps - 1) / warps;  // a warp per row, or per pair of rows
        unsigned long long grid = static_cast<unsigned long long>(ctx->sm_count) * per_sm;
        if (grid > blocks) grid = blocks;
        launch_k(kern, static_cast<unsigned>(grid), warps * 32, smem, s, c);
        LOKAL_CHECK_LAUNCH(ctx, "gather_quant_staged_kernel");
    }
    return LOKAL_OK;
}

}  // namespace

int launch_gather(lokal_cuda_ctx* ctx, cudaStream_t s, const void* table, int ggml_type, size_t vocab, size_t dim,
                  const uint32_t* ids, size_t n, void* out, int out_dtype) {
    return launch_gather_norm(ctx, s, table, ggml_type, vocab, dim, ids, n, out, out_dtype, nullptr, 0, nullptr, 0.0f, nullptr);
}

// Gather, and (norm_w != null) the RMSNorm of the gathered rows into xn: in the same launch where the staged kernel
// takes the table, as a second launch otherwise. *launches, when given, receives the number of kernels launched.
int launch_gather_norm(lokal_cuda_ctx* ctx, cudaStream_t s, const void* table, int ggml_type, size_t vocab, size_t dim,
                       const uint32_t* ids, size_t n, void* out, int out_dtype, const void* norm_w, int w_dtype, void* xn,
                       float eps, int* launches) {
    if (launches) *launches = 0;
    if (!table || !out) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather: table and out must be non-null");
    if (norm_w) {
        if (!xn) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather_rmsnorm: the normed output is null");
        if (!is_act_type(w_dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "embed_gather_rmsnorm: weight type %d is not F32/F16/BF16", w_dtype);
        if (!aligned_to(norm_w, type_size(w_dtype)) || (is_act_type(out_dtype) && !aligned_to(xn, type_size(out_dtype))))
            return ctx->fail(LOKAL_ERR_MISALIGNED, "embed_gather_rmsnorm: a pointer is not aligned to its element size");
    }
    const size_t be = lokal_cuda_blk_elems(ggml_type);
    if (be == 0) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "embed_gather: ggml type %d is not a float type, a Q*_0 / Q*_K block type or an i-quant (Q4_1, Q5_1, Q8_1, Q8_K are not covered)", ggml_type);
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
    if (!ids && n > vocab) return ctx->fail(LOKAL_ERR_BAD_ARG, "embed_gather: %zu rows asked of a table of %zu without an id list", n, vocab);
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
    a.wait_limit = static_cast<unsigned>(tune_env("LOKAL_CUDA_WAIT_LIMIT", kWaitLimit));
    a.extra_tx = static_cast<unsigned>(tune_env("LOKAL_CUDA_TEST_EXTRA_TX", 0)) & ~15u;
    // Table rows are fetched with the high L2 eviction priority: the rows of frequent tokens are asked for again and
    // again (within a call and from one call to the next), while the output rows, eight to thirty times the bytes,
    // stream through L2 once. Measured on the 65,536-id Zipf gather run back to back: Q8_0 to f32 42.1 -> 39.2 us,
    // Q4_K to f32 45.4 -> 41.5 us, Q8_0 to f16 24.7 -> 23.5 us. LOKAL_CUDA_GATHER_TABLE_KEEP=0 turns it off.
    a.table_keep = tune_env("LOKAL_CUDA_GATHER_TABLE_KEEP", 1) != 0 ? 1u : 0u;
    static const struct { int type, grid; const char* name; } kGridOf[] = {
        {LOKAL_IQ2_XXS, LOKAL_GRID_IQ2XXS, "iq2xxs"}, {LOKAL_IQ2_XS, LOKAL_GRID_IQ2XS, "iq2xs"}, {LOKAL_IQ2_S, LOKAL_GRID_IQ2S, "iq2s"},
        {LOKAL_IQ3_XXS, LOKAL_GRID_IQ3XXS, "iq3xxs"}, {LOKAL_IQ3_S, LOKAL_GRID_IQ3S, "iq3s"}, {LOKAL_IQ1_S, LOKAL_GRID_IQ1S, "iq1s"},
        {LOKAL_IQ1_M, LOKAL_GRID_IQ1S, "iq1s"}};
    for (const auto& g : kGridOf) {
        if (g.type != ggml_type) continue;
        a.grid = ctx->iq_grids[g.grid];
        if (!a.grid)
            return ctx->fail(LOKAL_ERR_UNSUPPORTED, "embed_gather: ggml type %d needs the %s codebook: hand it over with lokal_cuda_set_iq_grid first",
                             ggml_type, g.name);
    }
    const bool aligned = aligned_to(table, 16) && aligned_to(out, 16) && (dim * type_size(out_dtype)) % 16 == 0;
    if (norm_w && aligned && aligned_to(xn, 16) && tune_env("LOKAL_CUDA_GATHER_FUSE_NORM", 1) != 0) {
        a.norm_w = norm_w;
        a.xn = xn;
        a.eps = eps;
        a.inv_dim = 1.0f / static_cast<float>(dim);
        a.w_dtype = w_dtype;
        a.w_vec_ok = aligned_to(norm_w, 16);
    }
    bool fused = false;
    int rc;
    switch (out_dtype) {
        case LOKAL_F32: rc = launch_out<float>(ctx, s, a, ggml_type, aligned, &fused); break;
        case LOKAL_F16: rc = launch_out<__half>(ctx, s, a, ggml_type, aligned, &fused); break;
        default: rc = launch_out<__nv_bfloat16>(ctx, s, a, ggml_type, aligned, &fused); break;
    }
    if (rc != LOKAL_OK) return rc;
    if (launches) *launches = 1;
    if (norm_w && !fused) {  // float tables, the any-alignment kernel: the norm is its own launch
        rc = launch_norm(ctx, s, out, nullptr, norm_w, xn, nullptr, n, dim, eps, out_dtype, w_dtype, 0);
        if (rc != LOKAL_OK) return rc;
        if (launches) *launches = 2;
    }
    return LOKAL_OK;
}

}  // namespace lokal
