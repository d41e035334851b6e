// Per-token ops of the gated-deltanet (qwen35) blocks that sit beside the per-row norms: the gate scalars, the
// depthwise causal conv over the token axis with its rolling window, and the bf16 -> f16 page conversion of the
// weight stage-in. All are one pass over their inputs (HBM-bound), f32 arithmetic with the reference's operation
// order: separate multiply and add per tap, SiLU as x * (1 / (1 + exp(-x))), softplus with the x > 20 shortcut.
//
// Reference: delta_gates (src/gpu/kernels.metal:3995-4015; src/deltanet_ref.rs:48-58, 82-84), ssm_conv_decode /
// ssm_conv_prefill / ssm_conv_roll (src/gpu/kernels.metal:3626-3665, 4039-4093; conv_step src/deltanet_ref.rs:91-112),
// bf16_to_f16_copy (src/gpu/kernels.metal:3572-3588).
#include "common.cuh"

#include <type_traits>

namespace lokal {
namespace {

constexpr unsigned kMaxTaps = 8;  // the reference refuses a checkpoint with more filter taps
#ifndef LOKAL_CONV_THREADS
#define LOKAL_CONV_THREADS 128
#endif
#ifndef LOKAL_CONV_BATCH
#define LOKAL_CONV_BATCH 4
#endif
#ifndef LOKAL_CONV_TOKENS
#define LOKAL_CONV_TOKENS 32
#endif
constexpr unsigned kConvThreads = LOKAL_CONV_THREADS;  // the 16-bit variants hold many registers: small CTAs keep several resident

__device__ __forceinline__ float sigmoid_rcp(float x) { return __frcp_rn(__fadd_rn(1.0f, expf(-x))); }

// ---- gate scalars ----
struct GatesArgs {
    const float* alpha;
    const float* beta_in;
    const float* a;
    const float* dt_bias;
    float* g;
    float* beta;
    unsigned n_v_heads;
    unsigned long long total;
};

__global__ void __launch_bounds__(256) delta_gates_kernel(const GatesArgs p) {
    pdl_sync();
    const unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= p.total) return;
    const unsigned h = static_cast<unsigned>(i % p.n_v_heads);
    const float x = __fadd_rn(p.alpha[i], __ldg(p.dt_bias + h));
    const float sp = x > 20.0f ? x : logf(__fadd_rn(1.0f, expf(x)));
    p.g[i] = __fmul_rn(__ldg(p.a + h), sp);
    p.beta[i] = sigmoid_rcp(p.beta_in[i]);
}

// ---- depthwise causal conv over tokens ----
struct ConvArgs {
    float* state;      // [channels][k-1], oldest first
    const void* x;     // [n][channels]
    const float* w;    // [channels][k]
    void* out;         // [n][channels]
    unsigned channels, d_conv, n_tokens, tokens_per_thread;
    int write_state;   // only with a single token chunk per channel: the thread that read the window writes it back
};

// A thread owns N (four, or one) neighbouring channels and a run of tokens, and slides the window of the last k-1 inputs through
// registers, so every input is read once (plus k-1 rows of overlap per run). The window is kept right-aligned in
// KMAX-1 slots so that a tap count known only at run time still indexes registers statically. Channels are held in
// pairs and the taps use the packed f32x2 multiply and add (each lane rounds as the scalar instruction does, and a
// multiply is never fused with the add that follows it).
template <typename T, int N, int KT>
__global__ void __launch_bounds__(kConvThreads) ssm_conv_kernel(const ConvArgs a) {
    pdl_sync();
    constexpr int KMAX = KT ? KT : static_cast<int>(kMaxTaps);
    constexpr int P = N >= 2 ? N / 2 : 1;  // channel pairs (a single channel rides in .x)
    const int k = KT ? KT : static_cast<int>(a.d_conv);
    const int lead = KMAX - k;  // unused leading slots
    const unsigned cv = blockIdx.x * blockDim.x + threadIdx.x;
    if (cv >= a.channels / N) return;
    const unsigned c0 = cv * N;
    const unsigned C = a.channels;
    const unsigned t0 = blockIdx.y * a.tokens_per_thread;
    const unsigned t1 = min(t0 + a.tokens_per_thread, a.n_tokens);
    const T* __restrict__ x = reinterpret_cast<const T*>(a.x);
    T* __restrict__ out = reinterpret_cast<T*>(a.out);

    // a row's slice as loaded, before widening: one element, or four channels (16 bytes of f32, 8 bytes of a 16-bit type)
    using Raw = typename std::conditional<N == 1, T, typename std::conditional<sizeof(T) == 4, uint4, uint2>::type>::type;
    auto load_raw = [&](unsigned t) -> Raw {
        const T* p = x + static_cast<unsigned long long>(t) * C + c0;
        if constexpr (N == 1) return *p;
        else if constexpr (sizeof(T) == 4) return ld_stream(p);
        else return *reinterpret_cast<const uint2*>(p);
    };
    auto widen = [](const Raw& r, float2 (&v)[P]) {
        if constexpr (N == 1) {
            v[0] = make_float2(to_f32<T>(r), 0.0f);
        } else if constexpr (sizeof(T) == 4) {
            unpack16p<T>(r, v);
        } else {
            float2 four[4];
            unpack16p<T>(make_uint4(r.x, r.y, 0u, 0u), four);
            v[0] = four[0];
            v[1] = four[1];
        }
    };
    auto load_row = [&](unsigned t, float2 (&v)[P]) { widen(load_raw(t), v); };
    auto chan = [&](const float* base, unsigned stride, int pair, unsigned idx) {  // the two channels of a pair at base[c*stride + idx]
        const unsigned long long c = c0 + 2 * pair;
        return make_float2(base[c * stride + idx], N == 1 ? 0.0f : base[(c + (N == 1 ? 0 : 1)) * stride + idx]);
    };

    float2 wt[KMAX][P];       // wt[s][p]: tap s - lead of channel pair p
    float2 win[KMAX - 1][P];  // win[s][p]: input of channel pair p at token t - (KMAX-1) + s
#pragma unroll
    for (int s = 0; s < KMAX; s++) {
#pragma unroll
        for (int p = 0; p < P; p++) wt[s][p] = s >= lead ? chan(a.w, k, p, s - lead) : make_float2(0.0f, 0.0f);
    }
#pragma unroll
    for (int s = 0; s < KMAX - 1; s++) {
#pragma unroll
        for (int p = 0; p < P; p++) win[s][p] = make_float2(0.0f, 0.0f);
        if (s >= lead) {
            const long long u = static_cast<long long>(t0) - (KMAX - 1) + s;  // token this slot holds
            if (u >= 0) {
                load_row(static_cast<unsigned>(u), win[s]);
            } else {
#pragma unroll
                for (int p = 0; p < P; p++) win[s][p] = chan(a.state, k - 1, p, static_cast<unsigned>(k - 1 + u));
            }
        }
    }

    auto silu = [](float acc) {
        // 16-bit rows: the store rounds to 8 or 11 bits, so the fast exponential and division are used (as in the
        // SwiGLU kernel); f32 rows keep the accurate exponential and the exact reciprocal of the reference's form.
        if constexpr (sizeof(T) == 2) return acc * __fdividef(1.0f, 1.0f + __expf(-acc));
        else return __fmul_rn(acc, sigmoid_rcp(acc));
    };
    auto one_token = [&](unsigned t, const float2 (&xr)[P]) {
        float2 o[P];
#pragma unroll
        for (int p = 0; p < P; p++) {
            float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int s = 0; s < KMAX - 1; s++) {
                if (s >= lead) acc = add2(acc, mul2(win[s][p], wt[s][p]));
            }
            acc = add2(acc, mul2(xr[p], wt[KMAX - 1][p]));
            o[p].x = silu(acc.x);
            o[p].y = N == 1 ? 0.0f : silu(acc.y);
        }
        T* q = out + static_cast<unsigned long long>(t) * C + c0;
        if constexpr (N == 1) {
            *q = from_f32<T>(o[0].x);
        } else if constexpr (sizeof(T) == 4) {
            st_stream(q, pack16p<T>(o));
        } else {
            const float2 four[4] = {o[0], o[1], make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
            const uint4 w = pack16p<T>(four);
            *reinterpret_cast<uint2*>(q) = make_uint2(w.x, w.y);
        }
#pragma unroll
        for (int s = 0; s + 1 < KMAX - 1; s++) {
#pragma unroll
            for (int p = 0; p < P; p++) win[s][p] = win[s + 1][p];
        }
        if constexpr (KMAX >= 2) {
#pragma unroll
            for (int p = 0; p < P; p++) win[KMAX - 2][p] = xr[p];
        }
    };

    // Whole batches of kBatch tokens run without a branch, and the loads of the next batch are issued (and held as
    // loaded, not widened) before the current one is worked on, so a warp always has loads in flight while it
    // computes. The last tokens of a run go one at a time.
    constexpr int kBatch = KT == 0 ? 2 : (sizeof(T) == 2 ? 2 * LOKAL_CONV_BATCH : LOKAL_CONV_BATCH);  // run-time tap counts hold 8 slots: short batches
    unsigned tb = t0;
    if (tb + kBatch <= t1) {
        Raw cur[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; b++) cur[b] = load_raw(tb + b);
        for (;;) {
            const bool more = tb + 2 * kBatch <= t1;
            Raw nxt[kBatch];
            if (more) {
#pragma unroll
                for (int b = 0; b < kBatch; b++) nxt[b] = load_raw(tb + kBatch + b);
            }
#pragma unroll
            for (int b = 0; b < kBatch; b++) {
                float2 xr[P];
                widen(cur[b], xr);
                one_token(tb + b, xr);
            }
            tb += kBatch;
            if (!more) break;
#pragma unroll
            for (int b = 0; b < kBatch; b++) cur[b] = nxt[b];
        }
    }
    for (; tb < t1; tb++) {
        float2 xr[P];
        load_row(tb, xr);
        one_token(tb, xr);
    }

    if (a.write_state) {
#pragma unroll
        for (int s = 0; s < KMAX - 1; s++) {
            if (s >= lead) {
#pragma unroll
                for (int p = 0; p < P; p++) {
                    const unsigned long long c = c0 + 2 * p;
                    a.state[c * (k - 1) + (s - lead)] = win[s][p].x;
                    if constexpr (N > 1) a.state[(c + 1) * (k - 1) + (s - lead)] = win[s][p].y;
                }
            }
        }
    }
}

// The window as it stands after the whole chunk: the last k-1 inputs, or entries of the old window where the chunk
// is shorter than that. Staged through registers because old entries move while new ones arrive.
template <typename T>
__global__ void __launch_bounds__(256) ssm_conv_roll_kernel(const ConvArgs a) {
    pdl_sync();
    const unsigned c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.channels) return;
    const int k = static_cast<int>(a.d_conv);
    const T* x = reinterpret_cast<const T*>(a.x);
    float* st = a.state + static_cast<unsigned long long>(c) * (k - 1);
    float tmp[kMaxTaps - 1];
#pragma unroll
    for (int m = 0; m < static_cast<int>(kMaxTaps) - 1; m++) {
        tmp[m] = 0.0f;
        if (m < k - 1) {
            const long long u = static_cast<long long>(a.n_tokens) - (k - 1) + m;
            tmp[m] = u < 0 ? st[k - 1 + u] : to_f32<T>(x[static_cast<unsigned long long>(u) * a.channels + c]);
        }
    }
#pragma unroll
    for (int m = 0; m < static_cast<int>(kMaxTaps) - 1; m++) {
        if (m < k - 1) st[m] = tmp[m];
    }
}

// CTAs of `kernel` that fit on one SM (asked once per kernel).
inline unsigned resident_ctas(void (*kernel)(const ConvArgs)) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, static_cast<int>(kConvThreads), 0) != cudaSuccess || n < 1) n = 1;
    return static_cast<unsigned>(n);
}

// Tokens per thread. Long runs amortise the k-1 rows of overlap that every run re-reads; the grid should fill a whole
// number of waves (a last wave that is a third full costs as much as a full one); short chunks should still fill the
// GPU. The cost of a candidate is its number of waves times the rows a thread touches.
inline unsigned pick_tokens_per_thread(unsigned n_tokens, unsigned ctas_x, unsigned slots, unsigned d_conv) {
    const unsigned hi = LOKAL_CONV_TOKENS * 2, lo = 4;
    if (n_tokens <= lo) return n_tokens;
    unsigned best = lo;
    double best_cost = 1e300;
    for (unsigned tpt = lo; tpt <= hi && tpt <= n_tokens + 3; tpt++) {
        const unsigned long long ctas = static_cast<unsigned long long>(ctas_x) * ((n_tokens + tpt - 1) / tpt);
        const unsigned long long waves = (ctas + slots - 1) / slots;
        // a wave that is not full still runs at the speed its CTAs can pull from memory: count at least half a wave
        const double fill = static_cast<double>(ctas) / static_cast<double>(slots);
        const double eff_waves = waves > 1 ? static_cast<double>(waves) : (fill < 0.5 ? 0.5 : 1.0);
        const double cost = eff_waves * (tpt + 0.5 * (d_conv - 1));
        if (cost < best_cost * 0.999) {
            best_cost = cost;
            best = tpt;
        }
    }
    return best;
}

template <typename T>
int launch_conv(lokal_cuda_ctx* ctx, cudaStream_t s, ConvArgs a, bool vec_ok, int roll) {
    constexpr int N = 4;  // channels per thread on the vector path: 16 bytes of f32, 8 bytes of a 16-bit type
    void (*kern)(const ConvArgs) = vec_ok ? (a.d_conv == 4 ? ssm_conv_kernel<T, N, 4> : ssm_conv_kernel<T, N, 0>)
                                          : (a.d_conv == 4 ? ssm_conv_kernel<T, 1, 4> : ssm_conv_kernel<T, 1, 0>);
    static unsigned per_sm[4] = {0, 0, 0, 0};  // per instantiation of this template, per variant
    const int variant = (vec_ok ? 0 : 2) + (a.d_conv == 4 ? 0 : 1);
    if (per_sm[variant] == 0) per_sm[variant] = resident_ctas(kern);
    const unsigned per_thread = vec_ok ? N : 1;
    const unsigned threads = a.channels / per_thread;
    const unsigned ctas_x = (threads + kConvThreads - 1) / kConvThreads;
    const unsigned tpt = pick_tokens_per_thread(a.n_tokens, ctas_x, per_sm[variant] * static_cast<unsigned>(ctx->sm_count), a.d_conv);
    const unsigned chunks = (a.n_tokens + tpt - 1) / tpt;
    if (chunks > 65535u) return ctx->fail(LOKAL_ERR_BAD_ARG, "ssm_conv: %u tokens are too many for one launch", a.n_tokens);
    a.tokens_per_thread = tpt;
    a.write_state = (roll && chunks == 1) ? 1 : 0;
    launch_k(kern, dim3(ctas_x, chunks), kConvThreads, 0, s, a);
    LOKAL_CHECK_LAUNCH(ctx, "ssm_conv_kernel");
    if (roll && chunks > 1 && a.d_conv > 1) {
        // every run of tokens has read the old window by the time this launch starts (stream order)
        launch_k(ssm_conv_roll_kernel<T>, (a.channels + 255) / 256, 256, 0, s, a);
        LOKAL_CHECK_LAUNCH(ctx, "ssm_conv_roll_kernel");
    }
    return LOKAL_OK;
}

// ---- bf16 -> f16 page conversion ----
struct PageArgs {
    const unsigned short* src;
    __half* dst;
    unsigned long long n;
    unsigned* clip;
};

__device__ __forceinline__ bool narrow_bf16(unsigned short bits, __half& h) {
    const float v = __uint_as_float(static_cast<unsigned>(bits) << 16);
    h = __float2half_rn(v);
    return __hisinf(h) && !isinf(v);
}

__global__ void __launch_bounds__(256) bf16_to_f16_kernel(const PageArgs a, int vec_ok) {
    pdl_sync();
    const unsigned long long e = (static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8ull;
    if (e >= a.n) return;
    bool clipped = false;
    if (vec_ok && e + 8 <= a.n) {
        const uint4 v = ld_stream(a.src + e);
        const unsigned wv[4] = {v.x, v.y, v.z, v.w};
        unsigned ov[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            __half lo, hi;
            clipped |= narrow_bf16(static_cast<unsigned short>(wv[j] & 0xffffu), lo);
            clipped |= narrow_bf16(static_cast<unsigned short>(wv[j] >> 16), hi);
            ov[j] = static_cast<unsigned>(__half_as_ushort(lo)) | (static_cast<unsigned>(__half_as_ushort(hi)) << 16);
        }
        st_stream(a.dst + e, make_uint4(ov[0], ov[1], ov[2], ov[3]));
    } else {
        for (unsigned long long i = e; i < e + 8 && i < a.n; i++) {
            __half h;
            clipped |= narrow_bf16(a.src[i], h);
            a.dst[i] = h;
        }
    }
    if (clipped && a.clip) atomicOr(a.clip, 1u);
}

}  // namespace
}  // namespace lokal

extern "C" {

int lokal_cuda_delta_gates(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const float* alpha, const float* beta_in, const float* a,
                           const float* dt_bias, float* g, float* beta, size_t n_v_heads, size_t n_tokens) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    lokal::DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!alpha || !beta_in || !a || !dt_bias || !g || !beta) return ctx->fail(LOKAL_ERR_BAD_ARG, "delta_gates: every pointer must be non-null");
    if (n_v_heads == 0 || n_v_heads > 0xffffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "delta_gates: n_v_heads %zu out of range", n_v_heads);
    const void* ptrs[6] = {alpha, beta_in, a, dt_bias, g, beta};
    for (const void* p : ptrs)
        if (!lokal::aligned_to(p, 4)) return ctx->fail(LOKAL_ERR_MISALIGNED, "delta_gates: a pointer is not 4-byte aligned");
    if (n_tokens == 0) return LOKAL_OK;
    lokal::GatesArgs p{alpha, beta_in, a, dt_bias, g, beta, static_cast<unsigned>(n_v_heads),
                       static_cast<unsigned long long>(n_v_heads) * n_tokens};
    const unsigned long long blocks = (p.total + 255) / 256;
    if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "delta_gates: too many elements for one launch");
    lokal::launch_k(lokal::delta_gates_kernel, static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(s), p);
    LOKAL_CHECK_LAUNCH(ctx, "delta_gates_kernel");
    return LOKAL_OK;
}

int lokal_cuda_ssm_conv(lokal_cuda_ctx* ctx, lokal_cuda_stream s, float* state, const void* x, const float* w, void* out,
                        size_t channels, size_t d_conv, size_t n_tokens, int dtype, int roll) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    lokal::DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!x || !w || !out) return ctx->fail(LOKAL_ERR_BAD_ARG, "ssm_conv: x, w and out must be non-null");
    if (d_conv == 0 || d_conv > lokal::kMaxTaps) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "ssm_conv: d_conv %zu is outside 1..%u", d_conv, lokal::kMaxTaps);
    if (d_conv > 1 && !state) return ctx->fail(LOKAL_ERR_BAD_ARG, "ssm_conv: state must be non-null when d_conv > 1");
    if (x == out) return ctx->fail(LOKAL_ERR_BAD_ARG, "ssm_conv: out must not be x (later tokens read earlier inputs)");
    if (!lokal::is_act_type(dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "ssm_conv: row type %d is not F32/F16/BF16", dtype);
    if (channels == 0 || channels > 0x7fffffffu) return ctx->fail(LOKAL_ERR_BAD_ARG, "ssm_conv: channels %zu out of range", channels);
    if (n_tokens > 0x7fffffffu) return ctx->fail(LOKAL_ERR_BAD_ARG, "ssm_conv: n_tokens %zu out of range", n_tokens);
    const size_t es = lokal::type_size(dtype);
    if (!lokal::aligned_to(x, es) || !lokal::aligned_to(out, es) || !lokal::aligned_to(w, 4) || !lokal::aligned_to(state, 4))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "ssm_conv: a pointer is not aligned to its element size");
    if (n_tokens == 0) return LOKAL_OK;
    lokal::ConvArgs a{};
    a.state = state;
    a.x = x;
    a.w = w;
    a.out = out;
    a.channels = static_cast<unsigned>(channels);
    a.d_conv = static_cast<unsigned>(d_conv);
    a.n_tokens = static_cast<unsigned>(n_tokens);
    const size_t vb = 4 * es;  // a thread's four channels
    const bool vec_ok = lokal::aligned_to(x, vb) && lokal::aligned_to(out, vb) && (channels * es) % vb == 0;
    cudaStream_t st = static_cast<cudaStream_t>(s);
    switch (dtype) {
        case LOKAL_F32: return lokal::launch_conv<float>(ctx, st, a, vec_ok, roll);
        case LOKAL_F16: return lokal::launch_conv<__half>(ctx, st, a, vec_ok, roll);
        default: return lokal::launch_conv<__nv_bfloat16>(ctx, st, a, vec_ok, roll);
    }
}

int lokal_cuda_bf16_to_f16_copy(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* src_bf16, void* dst_f16, size_t n,
                                uint32_t* clip_flag) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    lokal::DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!src_bf16 || !dst_f16) return ctx->fail(LOKAL_ERR_BAD_ARG, "bf16_to_f16_copy: src and dst must be non-null");
    if (!lokal::aligned_to(src_bf16, 2) || !lokal::aligned_to(dst_f16, 2) || !lokal::aligned_to(clip_flag, 4))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "bf16_to_f16_copy: a pointer is not aligned to its element size");
    if (n == 0) return LOKAL_OK;
    const unsigned long long blocks = ((n + 7) / 8 + 255) / 256;
    if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "bf16_to_f16_copy: too many elements for one launch");
    lokal::PageArgs a{static_cast<const unsigned short*>(src_bf16), static_cast<__half*>(dst_f16), n, clip_flag};
    const int vec_ok = lokal::aligned_to(src_bf16, 16) && lokal::aligned_to(dst_f16, 16);
    lokal::launch_k(lokal::bf16_to_f16_kernel, static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(s), a, vec_ok);
    LOKAL_CHECK_LAUNCH(ctx, "bf16_to_f16_kernel");
    return LOKAL_OK;
}

}  // extern "C"
