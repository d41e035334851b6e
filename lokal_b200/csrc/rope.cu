// RoPE: the per-step (cos, sin) table and the fused bias + per-head RMSNorm +
// pair rotation of q and k in one HBM pass.
//
// Reference semantics (model::rope, src/model.rs:268-279): within each head,
// element i pairs with i + rot/2; angle = pos * theta^(-(2 i)/rot);
//   out[i]         = a * cos - b * sin
//   out[i + rot/2] = a * sin + b * cos
// with four separately rounded products. Before the rotation, in the order of
// src/model.rs:208-226: bias add (Linear::forward, :27-35), then per-head
// rmsnorm with a head_dim-long weight shared by all heads (:213-221).
//
// The angle's frequency comes from the host's powf (see lokal_cuda_rope_table
// in the header), the angle itself is one f32 multiply on the device, and
// sincosf is the accurate CUDA version (this library is never built with
// fast-math). Because positions are shared by all heads and all layers of a
// step, (cos, sin) live in a small table that stays L2-resident; the q/k
// kernel is then a pure streaming kernel: every q/k element is read once and
// written once.
#include "common.cuh"

#include <cmath>

namespace lokal {
namespace {

constexpr unsigned kMaxRot = 1024;

#ifndef LOKAL_ROPE_IN_FLIGHT
#define LOKAL_ROPE_IN_FLIGHT 3  // head-group passes whose loads are issued together
#endif
constexpr int kRopeInFlight = LOKAL_ROPE_IN_FLIGHT;

#ifndef LOKAL_ROPE_STAGED_UNROLL
#define LOKAL_ROPE_STAGED_UNROLL 1  // head-group passes of the staged kernel interleaved by the compiler (measured at
                                    // 8192 x 24 heads of 128: 18.2 us without interleaving, 18.4 / 18.5 / 19.0 us with 2 / 3 / 6)
#endif
constexpr int kRopeStagedUnroll = LOKAL_ROPE_STAGED_UNROLL;

#ifndef LOKAL_ROPE_MIN_CTAS
#define LOKAL_ROPE_MIN_CTAS 3  // resident 256-thread CTAs per SM the fast kernel is compiled for (caps registers at 80)
#endif

struct TableArgs {
    float inv_freq[kMaxRot / 2];
    const int32_t* positions;
    long long pos0;
    unsigned long long rows;
    unsigned half;
    float* out;
};

__global__ void __launch_bounds__(256) rope_table_kernel(const __grid_constant__ TableArgs a) {
    pdl_sync();
    const unsigned long long gid = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= a.rows * a.half) return;
    const unsigned long long row = gid / a.half;
    const unsigned i = static_cast<unsigned>(gid % a.half);
    const long long pos = a.positions ? static_cast<long long>(a.positions[row]) : a.pos0 + static_cast<long long>(row);
    const float angle = static_cast<float>(pos) * a.inv_freq[i];
    float sn, cs;
    sincosf(angle, &sn, &cs);
    float* o = a.out + row * (2ull * a.half);
    o[i] = cs;
    o[a.half + i] = sn;
}

struct QkArgs {
    const void* q;
    const void* k;
    void* q_out;
    void* k_out;
    const void* q_bias;
    const void* k_bias;
    const void* q_norm_w;
    const void* k_norm_w;
    const float* cos_sin;
    int table_keep;  // keep the cos/sin table in L2 between the launches of a step (see RopeRow::init)
    const uint32_t* k_out_rows;
    unsigned long long rows;
    unsigned n_q, n_kv, head_dim, rot_dim;
    unsigned long long q_stride, k_stride, q_out_stride, k_out_stride;
    float eps;
    int w_dtype;
    int w_vec_ok;      // bias / norm pointers are 16-byte aligned
    unsigned chunks;   // head slots of a row, in groups of (32 / lanes-per-head)
    unsigned cpw;      // chunks handled by one warp
    unsigned wpr;      // warps per row
    unsigned q_row_bytes, k_row_bytes;  // n_q*head_dim*sizeof(T), n_kv*head_dim*sizeof(T) (staged kernel)
    unsigned stage_bytes;               // per-warp staging area, multiple of 128
    int prefetch;                       // ask L2 for the row before waiting for the previous kernel (staged kernel)
    unsigned swpr, swpr_shift;          // warps that share one staged row, a power of two, and its log2 (staged kernel)
    unsigned* err_word;
    unsigned wait_limit;                // polls of the staged row's mbarrier before the kernel gives up (kWaitLimit)
    unsigned extra_tx;                  // 0; a test sets it so that the row's barrier never completes and the wait runs out
};

// ---------------------------------------------------------------------------
// Fast path: head_dim == HD, rot_dim == ROT (ROT == HD, or partial RoPE with
// ROT < HD as qwen35 has it: 64 of 256), 16-byte aligned rows.
//
// Lane mapping: a group of LPH lanes owns one head and each lane holds two
// 16-byte vectors of it. The first ROT/(2N) lanes of the group hold N elements
// of the rotated prefix's first half and their N partners (i, i + ROT/2); the
// remaining lanes hold two consecutive vectors of the unrotated tail, which
// take part in the bias add and the norm and are stored as they come out of
// those (bit-identical to the reference's untouched tail on f32 rows). A
// warp covers HPW heads per pass and the q heads followed by the k heads of a
// row are "head slots" 0 .. n_q+n_kv-1. The row's cos/sin live in registers;
// the per-head norm weights are staged once per CTA in shared memory as f32,
// permuted so that the lanes of a group read consecutive 16-byte words.
// Arithmetic is packed f32x2. For f32 rows every product and sum is rounded
// exactly as the reference's scalar code rounds it, in its order: bias, then
// (v*scale)*w, then the rotation. 16-bit rows are rounded again on store, so
// there the weights and the rotation, which do not depend on the scale, are
// applied while the reduction's shuffles are still in flight, the scale is
// multiplied in last, and one product of each rotated pair rides in an FMA.
// ---------------------------------------------------------------------------
template <typename T, int HD, int ROT, bool NORM, bool BIAS>
struct RopeRow {
    static constexpr int N = VecOf<T>::N;
    static constexpr int P = N / 2;        // f32 pairs per 16-byte vector
    static constexpr int HALF = HD / 2;
    static constexpr int LPH = HALF / N;   // lanes per head
    static constexpr int HPW = 32 / LPH;   // heads per warp pass
    static constexpr int RL = ROT / (2 * N);  // lanes of a group that hold rotated pairs
    static constexpr bool FULL = ROT == HD;
    static_assert(LPH >= 1 && LPH <= 32 && (LPH & (LPH - 1)) == 0, "head must map onto a power-of-two lane group");
    static_assert(ROT <= HD && RL >= 1 && ROT % (2 * N) == 0, "the rotated prefix must be whole lanes");

    float2 cs[P], sn[P], nsn[P];
    T* q_dst;
    T* k_dst;  // pre-shifted by -n_q heads so that both are indexed by the head slot
    const float* w_s;
    unsigned sub, hsel, slots;
    unsigned lo_off, hi_off;  // element offsets inside a head of this lane's two vectors
    bool rot_lane;            // this lane holds a rotated pair (always, when ROT == HD)
    bool k_skip;              // the row's cache row is LOKAL_KV_ROW_NONE: its k heads are not stored

    // The two vectors of lane `s` of a group: a rotated pair, or two consecutive vectors of the tail.
    static __device__ __forceinline__ unsigned lo_of(unsigned s) { return (FULL || s < RL) ? s * N : ROT + (s - RL) * 2 * N; }
    static __device__ __forceinline__ unsigned hi_of(unsigned s) { return (FULL || s < RL) ? ROT / 2 + s * N : ROT + (s - RL) * 2 * N + N; }

    __device__ __forceinline__ void init(const QkArgs& a, unsigned long long row, unsigned lane, const float* w_shared) {
        sub = lane % LPH;
        hsel = lane / LPH;
        slots = a.n_q + a.n_kv;
        w_s = w_shared;
        lo_off = lo_of(sub);
        hi_off = hi_of(sub);
        rot_lane = FULL || sub < RL;
        if (rot_lane) {
            // The table is read again by the rope launch of every layer of a step: its loads carry the high L2
            // eviction priority (a.table_keep: the table is small against L2), so that the q and k rows streaming
            // through between two launches do not push it out to HBM.
            const float* tr = a.cos_sin + row * ROT + sub * N;
            const unsigned long long pol = a.table_keep ? l2_policy_keep() : 0ull;
#pragma unroll
            for (int j = 0; j < N / 4; j++) {
                float2 t[2];
                unpack16p<float>(a.table_keep ? ld_keep_l2(tr + 4 * j, pol) : ld_keep(tr + 4 * j), t);
                cs[2 * j] = t[0];
                cs[2 * j + 1] = t[1];
                unpack16p<float>(a.table_keep ? ld_keep_l2(tr + ROT / 2 + 4 * j, pol) : ld_keep(tr + ROT / 2 + 4 * j), t);
                sn[2 * j] = t[0];
                sn[2 * j + 1] = t[1];
            }
        } else {
#pragma unroll
            for (int i = 0; i < P; i++) cs[i] = sn[i] = make_float2(0.0f, 0.0f);
        }
#pragma unroll
        for (int i = 0; i < P; i++) nsn[i] = make_float2(-sn[i].x, -sn[i].y);
        const long long k_shift = static_cast<long long>(a.n_q) * HD;
        q_dst = reinterpret_cast<T*>(a.q_out) + row * a.q_out_stride + lo_off;
        k_dst = nullptr;
        k_skip = false;
        if (a.n_kv) {
            const unsigned long long orow = a.k_out_rows ? static_cast<unsigned long long>(__ldg(a.k_out_rows + row)) : row;
            k_skip = a.k_out_rows && orow == LOKAL_KV_ROW_NONE;
            k_dst = reinterpret_cast<T*>(a.k_out) + (k_skip ? 0ull : orow) * a.k_out_stride + lo_off - k_shift;
        }
    }

    // Norm weights into shared memory: [q first vectors | q second vectors | k first vectors | k second vectors] of
    // the lanes, each block in (j, lane, e) order; a missing weight vector is staged as ones. Called by every thread
    // of the CTA.
    static __device__ __forceinline__ void stage_weights(const QkArgs& a, float* w_shared) {
        for (unsigned i = threadIdx.x; i < 2u * HD; i += blockDim.x) {
            const unsigned kind = i / HD, which = (i % HD) / HALF, lane_of = (i % HALF) / N, r = i % N;
            const unsigned d = (which ? hi_of(lane_of) : lo_of(lane_of)) + r;  // element of the head this slot holds
            const void* src = kind ? a.k_norm_w : a.q_norm_w;
            w_shared[kind * HD + which * HALF + ((r / 4) * LPH + lane_of) * 4 + r % 4] = src ? load_as_f32(src, a.w_dtype, d) : 1.0f;
        }
    }

    // One pass: the head in slot `slot` (this lane group's head), raw halves in lo / hi. Every lane of the warp
    // must call this together (the reduction shuffles); lanes with live == false contribute zeros and store nothing.
    // wra / wrb, when given, are this lane's norm weights for its two vectors, already in registers (the flat kernel);
    // otherwise they are read from the staged copy in shared memory.
    __device__ __forceinline__ void pass(const QkArgs& a, unsigned slot, bool live, const uint4& lo, const uint4& hi,
                                         const float2* wra = nullptr, const float2* wrb = nullptr) const {
        const bool is_q = slot < a.n_q;
        float2 va[P], vb[P];
        if (live) {
            unpack16p<T>(lo, va);
            unpack16p<T>(hi, vb);
        } else {
#pragma unroll
            for (int i = 0; i < P; i++) va[i] = vb[i] = make_float2(0.0f, 0.0f);
        }
        if (BIAS) {
            const void* bias = is_q ? a.q_bias : a.k_bias;
            if (bias && live) {
                const size_t boff = static_cast<size_t>(is_q ? slot : slot - a.n_q) * HD;
                float ba[N], bb[N];
                load_w<N>(bias, a.w_dtype, boff + lo_off, a.w_vec_ok, ba);
                load_w<N>(bias, a.w_dtype, boff + hi_off, a.w_vec_ok, bb);
#pragma unroll
                for (int i = 0; i < P; i++) {
                    va[i] = add2(va[i], make_float2(ba[2 * i], ba[2 * i + 1]));
                    vb[i] = add2(vb[i], make_float2(bb[2 * i], bb[2 * i + 1]));
                }
            }
        }
        float2 s2 = make_float2(1.0f, 1.0f);
        if (NORM) {
            float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < P; i++) {
                if (sizeof(T) == 2) {
                    acc = fma2(va[i], va[i], acc);
                    acc = fma2(vb[i], vb[i], acc);
                } else {
                    acc = add2(acc, mul2(va[i], va[i]));
                    acc = add2(acc, mul2(vb[i], vb[i]));
                }
            }
            float ss = acc.x + acc.y;
#pragma unroll
            for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const bool has = is_q ? (a.q_norm_w != nullptr) : (a.k_norm_w != nullptr);
            const float scale = has ? inv_rms<T>(ss, static_cast<float>(HD), 1.0f / static_cast<float>(HD), a.eps) : 1.0f;
            s2 = make_float2(scale, scale);
            const float* w = w_s + (is_q ? 0 : HD) + sub * 4;  // ones where a kind has no norm weights
#pragma unroll
            for (int j = 0; j < N / 4; j++) {
                float2 wa0, wa1, wb0, wb1;
                if (wra) {
                    wa0 = wra[2 * j];
                    wa1 = wra[2 * j + 1];
                    wb0 = wrb[2 * j];
                    wb1 = wrb[2 * j + 1];
                } else {
                    const float4 wa = *reinterpret_cast<const float4*>(w + j * LPH * 4);
                    const float4 wb = *reinterpret_cast<const float4*>(w + HALF + j * LPH * 4);
                    wa0 = make_float2(wa.x, wa.y), wa1 = make_float2(wa.z, wa.w);
                    wb0 = make_float2(wb.x, wb.y), wb1 = make_float2(wb.z, wb.w);
                }
                if (sizeof(T) == 2) {  // scale applied after the rotation
                    va[2 * j] = mul2(va[2 * j], wa0);
                    va[2 * j + 1] = mul2(va[2 * j + 1], wa1);
                    vb[2 * j] = mul2(vb[2 * j], wb0);
                    vb[2 * j + 1] = mul2(vb[2 * j + 1], wb1);
                } else {  // the reference's (v * scale) * w
                    va[2 * j] = mul2(mul2(va[2 * j], s2), wa0);
                    va[2 * j + 1] = mul2(mul2(va[2 * j + 1], s2), wa1);
                    vb[2 * j] = mul2(mul2(vb[2 * j], s2), wb0);
                    vb[2 * j + 1] = mul2(mul2(vb[2 * j + 1], s2), wb1);
                }
            }
        }
        if (live && !(k_skip && !is_q)) {
            float2 oa[P], ob[P];
#pragma unroll
            for (int i = 0; i < P; i++) {
                if (!FULL && !rot_lane) {  // the unrotated tail: out of the norm as it is
                    oa[i] = (NORM && sizeof(T) == 2) ? mul2(va[i], s2) : va[i];
                    ob[i] = (NORM && sizeof(T) == 2) ? mul2(vb[i], s2) : vb[i];
                    continue;
                }
                // a*cos - b*sin written as a*cos + b*(-sin): the same bits
                if (sizeof(T) == 2) {
                    oa[i] = fma2(va[i], cs[i], mul2(vb[i], nsn[i]));
                    ob[i] = fma2(va[i], sn[i], mul2(vb[i], cs[i]));
                    if (NORM) {
                        oa[i] = mul2(oa[i], s2);
                        ob[i] = mul2(ob[i], s2);
                    }
                } else {
                    oa[i] = add2(mul2(va[i], cs[i]), mul2(vb[i], nsn[i]));
                    ob[i] = add2(mul2(va[i], sn[i]), mul2(vb[i], cs[i]));
                }
            }
            T* dst = (is_q ? q_dst : k_dst) + static_cast<size_t>(slot) * HD;
            *reinterpret_cast<uint4*>(dst) = pack16p<T>(oa);
            *reinterpret_cast<uint4*>(dst + (hi_off - lo_off)) = pack16p<T>(ob);
        }
    }
};

// Register variant: one warp walks a range of head groups of one row; the loads of kRopeInFlight passes are issued
// before the first is consumed. Used when a row is split over several warps (few rows) or is too large to stage.
template <typename T, int HD, int ROT, bool NORM, bool BIAS>
__global__ void __launch_bounds__(256, LOKAL_ROPE_MIN_CTAS) qk_rope_kernel(const QkArgs a) {
    pdl_sync();
    using R = RopeRow<T, HD, ROT, NORM, BIAS>;
    constexpr int HPW = R::HPW;
    __shared__ __align__(16) float w_s[NORM ? 2 * HD : 4];

    const unsigned long long warp = (static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    // Warps past the last row stay for the staging barrier below but are given an empty chunk range.
    const bool valid = warp / a.wpr < a.rows;
    const unsigned long long row = valid ? warp / a.wpr : a.rows - 1;
    const unsigned first_chunk = static_cast<unsigned>(warp % a.wpr) * a.cpw;
    const unsigned end_chunk = valid ? min(first_chunk + a.cpw, a.chunks) : first_chunk;
    R r;
    r.init(a, row, threadIdx.x & 31u, w_s);
    // slot s of the row is at q_row + s*HD for s < n_q, at k_row + (s - n_q)*HD otherwise (second base pre-shifted)
    const T* q_src = reinterpret_cast<const T*>(a.q) + row * a.q_stride + r.lo_off;
    const T* k_src = reinterpret_cast<const T*>(a.k) + row * a.k_stride + r.lo_off - static_cast<long long>(a.n_q) * HD;
    auto fetch = [&](unsigned c, uint4& lo, uint4& hi) {
        const unsigned slot = c * HPW + r.hsel;
        if (c < end_chunk && slot < r.slots) {
            const T* src = (slot < a.n_q ? q_src : k_src) + static_cast<size_t>(slot) * HD;
            lo = ld_stream(src);
            hi = ld_stream(src + (r.hi_off - r.lo_off));
        }
    };
    unsigned c = first_chunk;
    uint4 lo[kRopeInFlight], hi[kRopeInFlight];
#pragma unroll
    for (int i = 0; i < kRopeInFlight; i++) fetch(c + i, lo[i], hi[i]);  // issued before the staging barrier
    if (NORM) {
        R::stage_weights(a, w_s);
        __syncthreads();
    }
    while (c < end_chunk) {
#pragma unroll
        for (int i = 0; i < kRopeInFlight; i++) {
            const unsigned slot = (c + i) * HPW + r.hsel;
            if (i == 0 || c + i < end_chunk) r.pass(a, slot, c + i < end_chunk && slot < r.slots, lo[i], hi[i]);
        }
        c += kRopeInFlight;
        if (c < end_chunk) {
#pragma unroll
            for (int i = 0; i < kRopeInFlight; i++) fetch(c + i, lo[i], hi[i]);
        }
    }
}

// Flat variant for short launches (few rows per SM): one warp per (row, head group), one pass each, nothing staged and
// no barrier. Every load of the warp (its two data vectors per lane, the row's cos/sin, the norm weights) is issued
// before the first is consumed, and the whole launch is resident at once, so the kernel lasts one memory round trip
// plus the arithmetic of a single pass. Same RopeRow arithmetic and results as the other two.
template <typename T, int HD, int ROT, bool NORM, bool BIAS>
__global__ void __launch_bounds__(256) qk_rope_flat_kernel(const QkArgs a) {
    pdl_launch();
    using R = RopeRow<T, HD, ROT, NORM, BIAS>;
    constexpr int N = R::N, P = R::P;
    const unsigned long long warp = (static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const unsigned long long row = warp / a.chunks;
    if (row >= a.rows) return;  // whole warps leave together; there is no barrier below
    const unsigned c = static_cast<unsigned>(warp % a.chunks);
    const unsigned lane = threadIdx.x & 31u;
    const unsigned sub = lane % R::LPH, slot = c * R::HPW + lane / R::LPH;
    const bool live = slot < a.n_q + a.n_kv, is_q = slot < a.n_q;
    const unsigned lo_off = R::lo_of(sub), hi_off = R::hi_of(sub);
    const T* src = (is_q ? reinterpret_cast<const T*>(a.q) + row * a.q_stride + static_cast<size_t>(slot) * HD
                         : reinterpret_cast<const T*>(a.k) + row * a.k_stride + static_cast<size_t>(slot - a.n_q) * HD) + lo_off;
    if (a.prefetch && live) {  // one request per 128-byte line, while the kernel before this one drains
        if ((reinterpret_cast<uintptr_t>(src) & 127u) == 0) prefetch_l2(src);
        if ((reinterpret_cast<uintptr_t>(src + (hi_off - lo_off)) & 127u) == 0) prefetch_l2(src + (hi_off - lo_off));
    }
    pdl_wait();
    uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
    if (live) {
        lo = ld_stream(src);
        hi = ld_stream(src + (hi_off - lo_off));
    }
    float2 wa[P], wb[P];
    if (NORM) {
        const void* nw = is_q ? a.q_norm_w : a.k_norm_w;
        if (nw && live) {
            float fa[N], fb[N];
            load_w<N>(nw, a.w_dtype, lo_off, a.w_vec_ok, fa);
            load_w<N>(nw, a.w_dtype, hi_off, a.w_vec_ok, fb);
#pragma unroll
            for (int i = 0; i < P; i++) {
                wa[i] = make_float2(fa[2 * i], fa[2 * i + 1]);
                wb[i] = make_float2(fb[2 * i], fb[2 * i + 1]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < P; i++) wa[i] = wb[i] = make_float2(1.0f, 1.0f);
        }
    }
    R r;
    r.init(a, row, lane, nullptr);
    r.pass(a, slot, live, lo, hi, NORM ? wa : nullptr, NORM ? wb : nullptr);
}

// Staged variant: one lane brings the whole row (its q heads, then its k heads) into shared memory with two bulk
// asynchronous copies that complete on an mbarrier, so all of the row's bytes are in flight at once without
// holding registers; the row's warps (one for rows of a few KB, two or four for wider rows, which share the staged
// row and split its head groups) then walk the heads out of shared memory and store results straight to global
// memory. Same lane mapping, arithmetic and results as qk_rope_kernel.
template <typename T, int HD, int ROT, bool NORM, bool BIAS>
__global__ void __launch_bounds__(256, 4) qk_rope_staged_kernel(const QkArgs a) {
    pdl_launch();
    using R = RopeRow<T, HD, ROT, NORM, BIAS>;
    constexpr int HPW = R::HPW;
    extern __shared__ __align__(128) unsigned char dyn_smem[];
    __shared__ __align__(16) float w_s[NORM ? 2 * HD : 4];
    const unsigned warps_per_cta = blockDim.x >> 5, warp_in_cta = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(dyn_smem);
    // a.swpr (1, 2 or 4) warps share a row; the one-warp case keeps constant strides
    const bool shared_row = a.swpr > 1;
    const unsigned row_in_cta = shared_row ? warp_in_cta >> a.swpr_shift : warp_in_cta;
    const unsigned part = shared_row ? warp_in_cta & (a.swpr - 1u) : 0u;
    unsigned char* stage = dyn_smem + 128 + static_cast<size_t>(row_in_cta) * a.stage_bytes;
    const uint32_t bar = smem_addr(&bars[row_in_cta]);
    const unsigned long long grow =
        static_cast<unsigned long long>(blockIdx.x) * (shared_row ? warps_per_cta >> a.swpr_shift : warps_per_cta) + row_in_cta;
    const bool valid = grow < a.rows;
    const unsigned long long row = valid ? grow : a.rows - 1;
    if (a.prefetch && valid && part == 0) {  // the row's lines are asked of L2 while the kernel before this one drains
        const unsigned char* qrow = reinterpret_cast<const unsigned char*>(reinterpret_cast<const T*>(a.q) + row * a.q_stride);
        const unsigned char* krow = reinterpret_cast<const unsigned char*>(reinterpret_cast<const T*>(a.k) + row * a.k_stride);
        for (unsigned off = lane * 128u; off < a.q_row_bytes; off += 32u * 128u) prefetch_l2(qrow + off);
        for (unsigned off = lane * 128u; off < a.k_row_bytes; off += 32u * 128u) prefetch_l2(krow + off);
    }
    if (lane == 0 && part == 0) {  // the barrier is set up while the kernel before this one drains
        mbar_init(bar, 1);
        mbar_init_fence();
    }
    pdl_wait();
    if (lane == 0 && part == 0) {
        if (valid) {
            mbar_expect_tx(bar, a.q_row_bytes + a.k_row_bytes + a.extra_tx);
            if (a.q_row_bytes) bulk_copy_g2s(smem_addr(stage), reinterpret_cast<const T*>(a.q) + row * a.q_stride, a.q_row_bytes, bar);
            if (a.k_row_bytes) bulk_copy_g2s(smem_addr(stage + a.q_row_bytes), reinterpret_cast<const T*>(a.k) + row * a.k_stride, a.k_row_bytes, bar);
        }
    }
    R r;
    r.init(a, row, lane, w_s);
    if (NORM) R::stage_weights(a, w_s);
    __syncthreads();  // norm weights staged; every row's mbarrier initialised before anyone waits on it
    if (!valid) return;
    // Every lane polls for itself, and every lane whose polls run out reports it: the polls of a warp end together
    // unless completion falls on the very last one, and then the lanes that leave are exited threads to the shuffles
    // of those that go on, while the error word says the launch's output is not to be used.
    if (!mbar_wait_bounded(bar, 0, a.wait_limit)) {
        atomicOr(a.err_word, kErrTimeout);
        mbar_wait_bounded(bar, 0, a.wait_limit);  // one more bounded chance for the copies in flight to land before leaving
        return;
    }
    const T* srow = reinterpret_cast<const T*>(stage) + r.lo_off;
    auto one_pass = [&](unsigned c) {
        const unsigned slot = c * HPW + r.hsel;
        const bool live = slot < r.slots;
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
        if (live) {
            lo = *reinterpret_cast<const uint4*>(srow + static_cast<size_t>(slot) * HD);
            hi = *reinterpret_cast<const uint4*>(srow + static_cast<size_t>(slot) * HD + (r.hi_off - r.lo_off));
        }
        r.pass(a, slot, live, lo, hi);
    };
    if (!shared_row) {
#pragma unroll kRopeStagedUnroll
        for (unsigned c = 0; c < a.chunks; c++) one_pass(c);
    } else {
        for (unsigned c = part; c < a.chunks; c += a.swpr) one_pass(c);
    }
}

// Any head_dim, any even rot_dim <= head_dim, any alignment: one warp per
// (row, head). Dims rot_dim..head_dim are not rotated (partial RoPE,
// src/gpu/kernels.metal:2401-2425); they are rewritten only when a bias or a
// norm changed them or the output is a different buffer.
template <typename T>
__global__ void __launch_bounds__(256) qk_rope_generic_kernel(const QkArgs a) {
    pdl_sync();
    const unsigned long long warp = (static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const unsigned slots = a.n_q + a.n_kv;
    const unsigned long long row = warp / slots;
    if (row >= a.rows) return;
    const unsigned slot = static_cast<unsigned>(warp % slots);
    const unsigned lane = threadIdx.x & 31u;
    const bool is_q = slot < a.n_q;
    const unsigned head = is_q ? slot : slot - a.n_q;
    const unsigned hd = a.head_dim, half = a.rot_dim / 2;
    const T* src = (is_q ? reinterpret_cast<const T*>(a.q) + row * a.q_stride
                         : reinterpret_cast<const T*>(a.k) + row * a.k_stride) + static_cast<size_t>(head) * hd;
    T* dst;
    if (is_q) {
        dst = reinterpret_cast<T*>(a.q_out) + row * a.q_out_stride;
    } else {
        const unsigned long long orow = a.k_out_rows ? static_cast<unsigned long long>(a.k_out_rows[row]) : row;
        if (a.k_out_rows && orow == LOKAL_KV_ROW_NONE) return;  // a position lokal_cuda_kv_rows refused (no shuffles follow a return of a whole warp)
        dst = reinterpret_cast<T*>(a.k_out) + orow * a.k_out_stride;
    }
    dst += static_cast<size_t>(head) * hd;
    const void* bias = is_q ? a.q_bias : a.k_bias;
    const void* nw = is_q ? a.q_norm_w : a.k_norm_w;
    const size_t boff = static_cast<size_t>(head) * hd;

    float scale = 1.0f;
    if (nw) {
        float ss = 0.0f;
        for (unsigned i = lane; i < hd; i += 32) {
            float v = to_f32<T>(src[i]);
            if (bias) v = v + load_as_f32(bias, a.w_dtype, boff + i);
            ss += v * v;
        }
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / static_cast<float>(hd) + a.eps);
    }
    auto fetch = [&](unsigned i) {
        float v = to_f32<T>(src[i]);
        if (bias) v = v + load_as_f32(bias, a.w_dtype, boff + i);
        if (nw) v = (v * scale) * load_as_f32(nw, a.w_dtype, i);
        return v;
    };
    const float* tr = a.cos_sin + row * a.rot_dim;
    for (unsigned i = lane; i < half; i += 32) {
        const float va = fetch(i), vb = fetch(i + half);
        const float cs = tr[i], sn = tr[half + i];
        dst[i] = from_f32<T>(va * cs - vb * sn);
        dst[i + half] = from_f32<T>(va * sn + vb * cs);
    }
    const bool rewrite_tail = bias || nw || (static_cast<const void*>(dst) != static_cast<const void*>(src));
    if (rewrite_tail) {
        for (unsigned i = a.rot_dim + lane; i < hd; i += 32) dst[i] = from_f32<T>(fetch(i));
    }
}

template <typename T>
int launch_one(lokal_cuda_ctx* ctx, cudaStream_t s, QkArgs a, bool fast_ok, bool shared_machine) {
    constexpr unsigned N = VecOf<T>::N;
    const unsigned slots = a.n_q + a.n_kv;
    if (slots == 0 || a.rows == 0) return LOKAL_OK;
    // (head_dim, rot_dim) pairs with a lane-mapped kernel: full rotation at 64 / 128 / 256, and the partial rotations
    // 64 of 256 (qwen35) and 64 of 128.
    const unsigned geom = a.head_dim * 1024u + a.rot_dim;
    const bool fast = fast_ok && (geom == 64u * 1024u + 64u || geom == 128u * 1024u + 128u || geom == 256u * 1024u + 256u ||
                                  geom == 256u * 1024u + 64u || geom == 128u * 1024u + 64u);
    if (!fast) {
        const unsigned long long warps = a.rows * slots;
        const unsigned long long blocks = (warps + 7) / 8;
        if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: too many head rows for one launch");
        launch_k(qk_rope_generic_kernel<T>, static_cast<unsigned>(blocks), 256, 0, s, a);
        LOKAL_CHECK_LAUNCH(ctx, "qk_rope_generic_kernel");
        return LOKAL_OK;
    }
    const unsigned lph = (a.head_dim / 2) / N, hpw = 32 / lph;
    a.chunks = (slots + hpw - 1) / hpw;
    // Warps per row: one warp walks all head groups of a row (the row's cos/sin are read once). Measured on B200
    // this beat splitting a row over several warps even for 8192-row batches; few rows spread over more warps.
    // Below about 12 rows per SM a row is split over several warps of the register kernel (measured: at 2048 rows of
    // the 0.5B / 0.6B shapes one staged warp per row is 20-35 % faster, at 1024 rows and fewer the split wins).
    unsigned wpr = 1;
    const unsigned long long want_warps = static_cast<unsigned long long>(ctx->sm_count) * 16;
    // When the caller runs other kernels beside this one, a short launch keeps one warp per row too: alone it is the
    // slower shape, but it occupies a sixth of the thread slots of the flat kernel and leaves the machine to its
    // neighbours (a 1024-row step of the branched layer pass: 0.268 against 0.289 ms).
    // (Below about six rows per SM there are too few warps for that to pay: 512- and 256-row steps measured 3-5 % slower.)
    const bool compact = shared_machine && a.rows >= static_cast<unsigned long long>(ctx->sm_count) * 6;
    if (!compact && a.rows < static_cast<unsigned long long>(ctx->sm_count) * 12) {
        wpr = static_cast<unsigned>((want_warps + a.rows - 1) / a.rows);
        if (wpr > a.chunks) wpr = a.chunks;
    }
    const long forced = tune_env("LOKAL_CUDA_ROPE_WPR", 0);
    if (forced >= 1 && forced <= static_cast<long>(a.chunks)) wpr = static_cast<unsigned>(forced);
    const bool norm = a.q_norm_w || a.k_norm_w, bias = a.q_bias || a.k_bias;
    a.prefetch = prefetch_enabled();
    // Few rows: the flat kernel, a warp per (row, head group). It takes over from the split register kernel wherever
    // that one was used for want of rows (measured at 1024 rows of 24 heads of 128, bf16: see the launch notes in
    // the kernel's header comment); LOKAL_CUDA_ROPE_FLAT=0 / 1 forces the choice.
    const long flat_env = tune_env("LOKAL_CUDA_ROPE_FLAT", -1);
    const bool flat = flat_env >= 0 ? flat_env != 0 : (wpr > 1 && forced == 0);
    if (flat) {
        const unsigned long long fwarps = a.rows * a.chunks;
        const unsigned long long fblocks = (fwarps + 7) / 8;
        if (fblocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: too many rows for one launch");
        const unsigned fgrid = static_cast<unsigned>(fblocks);
#define LOKAL_ROPE_LAUNCH_FLAT(HD_, ROT_)                                                          \
    do {                                                                                           \
        if (norm && bias) launch_k(qk_rope_flat_kernel<T, HD_, ROT_, true, true>, fgrid, 256, 0, s, a);  \
        else if (norm) launch_k(qk_rope_flat_kernel<T, HD_, ROT_, true, false>, fgrid, 256, 0, s, a);    \
        else if (bias) launch_k(qk_rope_flat_kernel<T, HD_, ROT_, false, true>, fgrid, 256, 0, s, a);    \
        else launch_k(qk_rope_flat_kernel<T, HD_, ROT_, false, false>, fgrid, 256, 0, s, a);             \
    } while (0)
        switch (geom) {
            case 64u * 1024u + 64u: LOKAL_ROPE_LAUNCH_FLAT(64, 64); break;
            case 128u * 1024u + 128u: LOKAL_ROPE_LAUNCH_FLAT(128, 128); break;
            case 128u * 1024u + 64u: LOKAL_ROPE_LAUNCH_FLAT(128, 64); break;
            case 256u * 1024u + 64u: LOKAL_ROPE_LAUNCH_FLAT(256, 64); break;
            default: LOKAL_ROPE_LAUNCH_FLAT(256, 256); break;
        }
#undef LOKAL_ROPE_LAUNCH_FLAT
        LOKAL_CHECK_LAUNCH(ctx, "qk_rope_flat_kernel");
        return LOKAL_OK;
    }
    a.cpw = (a.chunks + wpr - 1) / wpr;
    a.wpr = (a.chunks + a.cpw - 1) / a.cpw;
    const unsigned long long warps = a.rows * a.wpr;
    unsigned cta = 256;
    const long forced_cta = tune_env("LOKAL_CUDA_ROPE_CTA", 0);
    if (forced_cta == 32 || forced_cta == 64 || forced_cta == 128) cta = static_cast<unsigned>(forced_cta);
    const unsigned wpc = cta / 32;
    const unsigned long long blocks = (warps + wpc - 1) / wpc;
    if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: too many rows for one launch");
    const unsigned grid = static_cast<unsigned>(blocks);
    a.q_row_bytes = a.n_q * a.head_dim * static_cast<unsigned>(sizeof(T));
    a.k_row_bytes = a.n_kv * a.head_dim * static_cast<unsigned>(sizeof(T));
    a.stage_bytes = (a.q_row_bytes + a.k_row_bytes + 127u) & ~127u;
    a.err_word = ctx->err_word;
    a.wait_limit = static_cast<unsigned>(tune_env("LOKAL_CUDA_WAIT_LIMIT", kWaitLimit));
    a.extra_tx = static_cast<unsigned>(tune_env("LOKAL_CUDA_TEST_EXTRA_TX", 0)) & ~15u;
    // Staged kernel: whole rows through shared memory by bulk copy. Needs one warp per row, row starts that are
    // 16-byte aligned (true on this path) and a row small enough that several warps' stages fit in shared memory.
    // The 48 KB a kernel gets without opting in covers its static shared memory too (the staged norm weights).
    const unsigned static_smem = norm ? 2u * a.head_dim * 4u : 16u;
    const unsigned dyn_budget = 48u * 1024u - static_smem;
    const bool staged_ok = a.wpr == 1 && 128u + a.stage_bytes <= dyn_budget && tune_env("LOKAL_CUDA_ROPE_STAGED", 1) != 0;
    if (staged_ok) {
        // Rows per CTA: as many as fit in 48 KB, at most eight; rows above 12 KB are shared by two warps, above 24 KB
        // by four, so that a CTA still has several warps to work through its few wide rows.
        a.swpr = a.stage_bytes <= 12u * 1024u ? 1u : (a.stage_bytes <= 24u * 1024u ? 2u : 4u);
        while (a.swpr > a.chunks) a.swpr >>= 1;
        a.swpr_shift = a.swpr == 4 ? 2u : (a.swpr == 2 ? 1u : 0u);
        unsigned rpc = 8 / a.swpr;
        while (rpc > 1 && 128u + rpc * a.stage_bytes > dyn_budget) rpc -= (rpc > 4 ? 4 : (rpc > 2 ? 2 : 1));
        const unsigned swpc = rpc * a.swpr;  // warps per CTA
        const unsigned sgrid = static_cast<unsigned>((a.rows + rpc - 1) / rpc);
        const size_t smem = 128u + static_cast<size_t>(rpc) * a.stage_bytes;
#define LOKAL_ROPE_LAUNCH_STAGED(HD_, ROT_)                                                                      \
    do {                                                                                                         \
        if (norm && bias) launch_k(qk_rope_staged_kernel<T, HD_, ROT_, true, true>, sgrid, swpc * 32, smem, s, a);   \
        else if (norm) launch_k(qk_rope_staged_kernel<T, HD_, ROT_, true, false>, sgrid, swpc * 32, smem, s, a);     \
        else if (bias) launch_k(qk_rope_staged_kernel<T, HD_, ROT_, false, true>, sgrid, swpc * 32, smem, s, a);     \
        else launch_k(qk_rope_staged_kernel<T, HD_, ROT_, false, false>, sgrid, swpc * 32, smem, s, a);              \
    } while (0)
        switch (geom) {
            case 64u * 1024u + 64u: LOKAL_ROPE_LAUNCH_STAGED(64, 64); break;
            case 128u * 1024u + 128u: LOKAL_ROPE_LAUNCH_STAGED(128, 128); break;
            case 128u * 1024u + 64u: LOKAL_ROPE_LAUNCH_STAGED(128, 64); break;
            case 256u * 1024u + 64u: LOKAL_ROPE_LAUNCH_STAGED(256, 64); break;
            default: LOKAL_ROPE_LAUNCH_STAGED(256, 256); break;
        }
#undef LOKAL_ROPE_LAUNCH_STAGED
        LOKAL_CHECK_LAUNCH(ctx, "qk_rope_staged_kernel");
        return LOKAL_OK;
    }
#define LOKAL_ROPE_LAUNCH(HD_, ROT_)                                                               \
    do {                                                                                           \
        if (norm && bias) launch_k(qk_rope_kernel<T, HD_, ROT_, true, true>, grid, cta, 0, s, a);        \
        else if (norm) launch_k(qk_rope_kernel<T, HD_, ROT_, true, false>, grid, cta, 0, s, a);          \
        else if (bias) launch_k(qk_rope_kernel<T, HD_, ROT_, false, true>, grid, cta, 0, s, a);          \
        else launch_k(qk_rope_kernel<T, HD_, ROT_, false, false>, grid, cta, 0, s, a);                   \
    } while (0)
    switch (geom) {
        case 64u * 1024u + 64u: LOKAL_ROPE_LAUNCH(64, 64); break;
        case 128u * 1024u + 128u: LOKAL_ROPE_LAUNCH(128, 128); break;
        case 128u * 1024u + 64u: LOKAL_ROPE_LAUNCH(128, 64); break;
        case 256u * 1024u + 64u: LOKAL_ROPE_LAUNCH(256, 64); break;
        default: LOKAL_ROPE_LAUNCH(256, 256); break;
    }
#undef LOKAL_ROPE_LAUNCH
    LOKAL_CHECK_LAUNCH(ctx, "qk_rope_kernel");
    return LOKAL_OK;
}

int launch_by_type(lokal_cuda_ctx* ctx, cudaStream_t s, const QkArgs& a, int dtype, bool fast_ok, bool shared_machine) {
    switch (dtype) {
        case LOKAL_F32: return launch_one<float>(ctx, s, a, fast_ok, shared_machine);
        case LOKAL_F16: return launch_one<__half>(ctx, s, a, fast_ok, shared_machine);
        default: return launch_one<__nv_bfloat16>(ctx, s, a, fast_ok, shared_machine);
    }
}

}  // namespace

int launch_rope_table(lokal_cuda_ctx* ctx, cudaStream_t s, float theta, uint32_t rot_dim, const int32_t* positions,
                      int64_t pos0, size_t rows, float* cos_sin) {
    if (!cos_sin) return ctx->fail(LOKAL_ERR_BAD_ARG, "rope_table: output is null");
    if (rot_dim == 0 || (rot_dim & 1u) || rot_dim > kMaxRot)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "rope_table: rot_dim %u must be even and <= %u", rot_dim, kMaxRot);
    if (!aligned_to(cos_sin, 16) || (positions && !aligned_to(positions, 4)))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "rope_table: table must be 16-byte aligned, positions 4-byte aligned");
    if (!positions && pos0 < 0) return ctx->fail(LOKAL_ERR_BAD_ARG, "rope_table: pos0 is negative");
    if (rows == 0) return LOKAL_OK;
    TableArgs a;
    const unsigned half = rot_dim / 2;
    // theta.powf(-(2 i) / rot) in f32, as src/model.rs:272 evaluates it, through the host C library.
    for (unsigned i = 0; i < half; i++) a.inv_freq[i] = powf(theta, -(2.0f * static_cast<float>(i)) / static_cast<float>(rot_dim));
    for (unsigned i = half; i < kMaxRot / 2; i++) a.inv_freq[i] = 0.0f;
    a.positions = positions;
    a.pos0 = pos0;
    a.rows = rows;
    a.half = half;
    a.out = cos_sin;
    const unsigned long long total = static_cast<unsigned long long>(rows) * half;
    const unsigned long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "rope_table: too many rows for one launch");
    launch_k(rope_table_kernel, static_cast<unsigned>(blocks), 256, 0, s, a);
    LOKAL_CHECK_LAUNCH(ctx, "rope_table_kernel");
    return LOKAL_OK;
}

int launch_qk_rope(lokal_cuda_ctx* ctx, cudaStream_t s, const lokal_qk_rope_params& p, bool shared_machine) {
    if (!p.cos_sin) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: cos_sin table is null");
    if (!p.q && !p.k) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: both q and k are null");
    if (p.head_dim == 0 || (p.head_dim & 1u)) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: head_dim %u must be even and non-zero", p.head_dim);
    if (p.rot_dim == 0 || (p.rot_dim & 1u) || p.rot_dim > p.head_dim || p.rot_dim > kMaxRot)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: rot_dim %u must be even, non-zero and <= head_dim %u", p.rot_dim, p.head_dim);
    if (p.q && p.n_q_heads == 0) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: q given with zero heads");
    if (p.k && p.n_kv_heads == 0) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: k given with zero heads");
    if (p.q && !is_act_type(p.q_dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "qk_rope: q type %d is not F32/F16/BF16", p.q_dtype);
    if (p.k && !is_act_type(p.k_dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "qk_rope: k type %d is not F32/F16/BF16", p.k_dtype);
    const bool has_w = p.q_bias || p.k_bias || p.q_norm_w || p.k_norm_w;
    if (has_w && !is_act_type(p.w_dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "qk_rope: weight type %d is not F32/F16/BF16", p.w_dtype);
    const unsigned long long q_w = static_cast<unsigned long long>(p.n_q_heads) * p.head_dim;
    const unsigned long long k_w = static_cast<unsigned long long>(p.n_kv_heads) * p.head_dim;
    if (p.q && p.q_row_stride < q_w) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: q_row_stride %llu < n_q_heads*head_dim %llu", (unsigned long long)p.q_row_stride, q_w);
    if (p.k && p.k_row_stride < k_w) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: k_row_stride %llu < n_kv_heads*head_dim %llu", (unsigned long long)p.k_row_stride, k_w);
    if (p.q && p.q_out && p.q_out_row_stride < q_w) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: q_out_row_stride too small");
    if (p.k && p.k_out && p.k_out_row_stride < k_w) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: k_out_row_stride too small");
    if (p.k_out_rows && !p.k_out) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope: k_out_rows needs k_out");
    const size_t wes = has_w ? type_size(p.w_dtype) : 1;
    const void* wptrs[4] = {p.q_bias, p.k_bias, p.q_norm_w, p.k_norm_w};
    bool w_vec = true;
    for (const void* wp : wptrs) {
        if (wp && !aligned_to(wp, wes)) return ctx->fail(LOKAL_ERR_MISALIGNED, "qk_rope: a weight pointer is not aligned to its element size");
        if (wp && !aligned_to(wp, 16)) w_vec = false;
    }
    if (!aligned_to(p.cos_sin, 4) || (p.k_out_rows && !aligned_to(p.k_out_rows, 4)))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "qk_rope: table or row-index pointer is not 4-byte aligned");

    QkArgs a{};
    a.q_bias = p.q_bias;
    a.k_bias = p.k_bias;
    a.q_norm_w = p.q_norm_w;
    a.k_norm_w = p.k_norm_w;
    a.cos_sin = p.cos_sin;
    a.table_keep = (static_cast<size_t>(p.rows) * p.rot_dim * 4 <= (32u << 20) && tune_env("LOKAL_CUDA_ROPE_TABLE_KEEP", 1) != 0) ? 1 : 0;
    a.k_out_rows = p.k_out_rows;
    a.rows = p.rows;
    a.head_dim = p.head_dim;
    a.rot_dim = p.rot_dim;
    a.eps = p.eps;
    a.w_dtype = p.w_dtype;
    a.w_vec_ok = w_vec;
    a.q_stride = p.q_row_stride;
    a.k_stride = p.k_row_stride;
    a.q_out = p.q_out ? p.q_out : p.q;
    a.k_out = p.k_out ? p.k_out : p.k;
    a.q_out_stride = p.q_out ? p.q_out_row_stride : p.q_row_stride;
    a.k_out_stride = p.k_out ? p.k_out_row_stride : p.k_row_stride;

    auto tensor_fast = [&](const void* in, const void* out, unsigned long long in_stride, unsigned long long out_stride, int dtype) {
        const size_t es = type_size(dtype);
        return aligned_to(in, 16) && aligned_to(out, 16) && (in_stride * es) % 16 == 0 && (out_stride * es) % 16 == 0 &&
               (static_cast<size_t>(p.head_dim) * es) % 32 == 0;
    };
    if (p.q && (!aligned_to(p.q, type_size(p.q_dtype)) || !aligned_to(a.q_out, type_size(p.q_dtype))))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "qk_rope: q is not aligned to its element size");
    if (p.k && (!aligned_to(p.k, type_size(p.k_dtype)) || !aligned_to(a.k_out, type_size(p.k_dtype))))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "qk_rope: k is not aligned to its element size");
    const bool table_fast = aligned_to(p.cos_sin, 16) && (static_cast<size_t>(p.rot_dim) * 4) % 32 == 0;

    if (p.q && p.k && p.q_dtype == p.k_dtype) {
        a.q = p.q;
        a.k = p.k;
        a.n_q = p.n_q_heads;
        a.n_kv = p.n_kv_heads;
        const bool fast = table_fast && tensor_fast(p.q, a.q_out, a.q_stride, a.q_out_stride, p.q_dtype) &&
                          tensor_fast(p.k, a.k_out, a.k_stride, a.k_out_stride, p.k_dtype);
        return launch_by_type(ctx, s, a, p.q_dtype, fast, shared_machine);
    }
    // q and k of different types (the reference GPU layout: f32 q, f16 k in the cache): one launch each.
    if (p.q) {
        QkArgs aq = a;
        aq.q = p.q;
        aq.k = nullptr;
        aq.n_q = p.n_q_heads;
        aq.n_kv = 0;
        const bool fast = table_fast && tensor_fast(p.q, a.q_out, a.q_stride, a.q_out_stride, p.q_dtype);
        int rc = launch_by_type(ctx, s, aq, p.q_dtype, fast, shared_machine);
        if (rc != LOKAL_OK) return rc;
    }
    if (p.k) {
        QkArgs ak = a;
        ak.q = nullptr;
        ak.k = p.k;
        ak.n_q = 0;
        ak.n_kv = p.n_kv_heads;
        const bool fast = table_fast && tensor_fast(p.k, a.k_out, a.k_stride, a.k_out_stride, p.k_dtype);
        return launch_by_type(ctx, s, ak, p.k_dtype, fast, shared_machine);
    }
    return LOKAL_OK;
}

}  // namespace lokal

// ---------------------------------------------------------------------------
// qk_rope with positions, for callers that must not allocate
// ---------------------------------------------------------------------------
//
// Some callers cannot afford a cudaMalloc on this path: a decode loop that
// must not stall (an allocation synchronises the whole device and takes
// driver-wide locks), or an engine that gave the rest of HBM to its KV-cache
// pool at start-up, where a later allocation may fail. For them the cos/sin
// table lives here, in a fixed array that is part of the library image: every
// GPU that loads the library carries these LOKAL_NOALLOC_TABLE_BYTES until the
// process exits, and nothing is ever allocated or freed by the entry point
// below.
//
// In host code the array's name is only a stand-in; the address a kernel can
// use comes from cudaGetSymbolAddress, looked up once per GPU with that GPU
// current and kept in g_noalloc_table_addr.
//
// The array is shared by every call on a GPU and keeps whatever the last call
// left in it. A call first rewrites the rows it is going to read, so no part
// of it has to start at zero; calls that overlap on the device race on it.

static __device__ __align__(256) float g_noalloc_rope_table[LOKAL_NOALLOC_TABLE_BYTES / sizeof(float)];

namespace {
constexpr int kNoallocMaxDevices = 64;
std::mutex g_noalloc_mu;
float* g_noalloc_table_addr[kNoallocMaxDevices] = {};
}  // namespace

extern "C" int lokal_cuda_qk_rope_pos_noalloc(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const lokal_qk_rope_params* p,
                                              float theta, const int32_t* positions, int64_t pos0) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    lokal::DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!p) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope_pos_noalloc: params are null");
    if (p->rot_dim == 0) return ctx->fail(LOKAL_ERR_BAD_ARG, "qk_rope_pos_noalloc: rot_dim is zero");
    const unsigned long long limit_floats = LOKAL_NOALLOC_TABLE_BYTES / sizeof(float);
    if (p->rows > limit_floats / p->rot_dim)
        return ctx->fail(LOKAL_ERR_BAD_ARG,
                         "qk_rope_pos_noalloc: %llu rows x rot_dim %u needs %llu bytes of table, the built-in table holds %u "
                         "(use lokal_cuda_qk_rope_pos, or fewer rows per call)",
                         (unsigned long long)p->rows, p->rot_dim, (unsigned long long)p->rows * p->rot_dim * 4ull,
                         (unsigned)LOKAL_NOALLOC_TABLE_BYTES);
    if (ctx->device < 0 || ctx->device >= kNoallocMaxDevices)
        return ctx->fail(LOKAL_ERR_UNSUPPORTED, "qk_rope_pos_noalloc: device index %d is beyond %d", ctx->device, kNoallocMaxDevices);
    float* table = nullptr;
    {
        // one-time set-up per GPU, with that GPU current (the guard above): the device address of the array
        std::lock_guard<std::mutex> g(g_noalloc_mu);
        table = g_noalloc_table_addr[ctx->device];
        if (!table) {
            void* addr = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&addr, g_noalloc_rope_table);
            if (e != cudaSuccess || !addr)
                return ctx->fail(LOKAL_ERR_CUDA, "qk_rope_pos_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            table = static_cast<float*>(addr);
            g_noalloc_table_addr[ctx->device] = table;
        }
    }
    cudaStream_t stream = static_cast<cudaStream_t>(s);
    int rc = lokal::launch_rope_table(ctx, stream, theta, p->rot_dim, positions, pos0, p->rows, table);
    if (rc != LOKAL_OK) return rc;
    lokal_qk_rope_params q = *p;
    q.cos_sin = table;
    return lokal::launch_qk_rope(ctx, stream, q);
}
