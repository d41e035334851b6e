// SwiGLU activation: inner_i = (g_i / (1 + exp(-g_i))) * u_i
// (math::silu, src/math.rs:68-70, and the SwiGLU line src/model.rs:245-248 of
// the reference; note the expression shape is g / (1 + exp(-g)), not
// g * sigmoid(g), which rounds differently).
//
// Pure streaming kernel: two 16-byte loads and one 16-byte store per thread
// per step, 3 * sizeof(T) bytes of HBM traffic per element. f32 rows use the
// accurate expf and IEEE division (the result has to hold to about one ulp);
// 16-bit rows are rounded to 11 or 8 significant bits on store, so they use
// the hardware exp2 / reciprocal approximations (relative error ~1e-6), which
// keeps the kernel memory-bound instead of issue-bound.
#include "common.cuh"

namespace lokal {
namespace {

template <typename T>
__device__ __forceinline__ float silu_mul(float g, float u) {
    if (sizeof(T) == 4) {
        return (g / (1.0f + expf(-g))) * u;
    } else {
        const float e = __expf(-g);
        return __fdividef(g, 1.0f + e) * u;
    }
}

struct SwigluArgs {
    const void* gate;
    const void* up;
    void* out;
    void* out_h;
    unsigned long long nvec;  // whole 16-byte vectors
    unsigned long long n;     // elements
    int h_dtype;
    int prefetch;  // ask L2 for the tile before waiting for the previous kernel
};

constexpr int kSwigluMaxUnroll = 4;

template <typename T>
__device__ __forceinline__ void swiglu_store(const SwigluArgs& a, uint4* o, unsigned long long v, const uint4& gv, const uint4& uv) {
    constexpr int N = VecOf<T>::N;
    float gf[N], uf[N], y[N];
    unpack16<T>(gv, gf);
    unpack16<T>(uv, uf);
#pragma unroll
    for (int e = 0; e < N; e++) y[e] = silu_mul<T>(gf[e], uf[e]);
    *o = pack16<T>(y);
    if (sizeof(T) == 4 && a.out_h) {
        unsigned w[2];
        if (a.h_dtype == LOKAL_F16) {
            __half2 h0 = __floats2half2_rn(y[0], y[1]), h1 = __floats2half2_rn(y[2], y[3]);
            w[0] = *reinterpret_cast<unsigned*>(&h0);
            w[1] = *reinterpret_cast<unsigned*>(&h1);
        } else {
            __nv_bfloat162 h0 = __floats2bfloat162_rn(y[0], y[1]), h1 = __floats2bfloat162_rn(y[2], y[3]);
            w[0] = *reinterpret_cast<unsigned*>(&h0);
            w[1] = *reinterpret_cast<unsigned*>(&h1);
        }
        *reinterpret_cast<uint2*>(reinterpret_cast<unsigned short*>(a.out_h) + v * N) = make_uint2(w[0], w[1]);
    }
}

template <typename T, int kSwigluUnroll>
__global__ void __launch_bounds__(256) swiglu_kernel(const SwigluArgs a) {
    pdl_launch();
    // Each CTA owns a contiguous tile of kSwigluUnroll * 256 vectors (16 KB per stream at four vectors per thread);
    // a thread's vectors are 256 apart, so every load instruction of a warp is one 512-byte run. Many small CTAs:
    // the machine drains evenly at the end of the kernel. All 64-bit address arithmetic is done once per CTA.
    constexpr unsigned kTile = 256u * kSwigluUnroll;
    const unsigned long long tile0 = static_cast<unsigned long long>(blockIdx.x) * kTile;
    const uint4* g = reinterpret_cast<const uint4*>(a.gate) + tile0 + threadIdx.x;
    const uint4* u = reinterpret_cast<const uint4*>(a.up) + tile0 + threadIdx.x;
    uint4* o = reinterpret_cast<uint4*>(a.out) + tile0 + threadIdx.x;
    const unsigned long long left = a.nvec - tile0;
    if (a.prefetch && (threadIdx.x & 7u) == 0) {  // one request per 128-byte line of the tile, before the wait
#pragma unroll
        for (int j = 0; j < kSwigluUnroll; j++) {
            if (threadIdx.x + j * 256 < left) {
                prefetch_l2(g + j * 256);
                prefetch_l2(u + j * 256);
            }
        }
    }
    pdl_wait();
    uint4 gv[kSwigluUnroll], uv[kSwigluUnroll];
    if (left >= kTile) {
#pragma unroll
        for (int j = 0; j < kSwigluUnroll; j++) {
            gv[j] = ld_stream(g + j * 256);
            uv[j] = ld_stream(u + j * 256);
        }
#pragma unroll
        for (int j = 0; j < kSwigluUnroll; j++) swiglu_store<T>(a, o + j * 256, tile0 + threadIdx.x + j * 256, gv[j], uv[j]);
    } else {
        const unsigned n = static_cast<unsigned>(left);
#pragma unroll
        for (int j = 0; j < kSwigluUnroll; j++) {
            if (threadIdx.x + j * 256 < n) {
                gv[j] = ld_stream(g + j * 256);
                uv[j] = ld_stream(u + j * 256);
            }
        }
#pragma unroll
        for (int j = 0; j < kSwigluUnroll; j++) {
            if (threadIdx.x + j * 256 < n) swiglu_store<T>(a, o + j * 256, tile0 + threadIdx.x + j * 256, gv[j], uv[j]);
        }
    }
}

// Elements [first, n): the ragged tail, or everything when pointers are not 16-byte aligned.
template <typename T>
__global__ void __launch_bounds__(256) swiglu_scalar_kernel(const SwigluArgs a, unsigned long long first) {
    pdl_sync();
    const unsigned long long i = first + static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= a.n) return;
    const float g = to_f32<T>(reinterpret_cast<const T*>(a.gate)[i]);
    const float u = to_f32<T>(reinterpret_cast<const T*>(a.up)[i]);
    const float y = silu_mul<T>(g, u);
    reinterpret_cast<T*>(a.out)[i] = from_f32<T>(y);
    if (a.out_h) {
        reinterpret_cast<unsigned short*>(a.out_h)[i] =
            a.h_dtype == LOKAL_F16 ? __half_as_ushort(__float2half_rn(y)) : __bfloat16_as_ushort(__float2bfloat16_rn(y));
    }
}

template <typename T>
int launch_typed(lokal_cuda_ctx* ctx, cudaStream_t s, SwigluArgs a, bool aligned) {
    constexpr unsigned N = VecOf<T>::N;
    a.nvec = aligned ? a.n / N : 0;
    if (a.nvec) {
        // Vectors per thread: four while that still gives every SM eight CTAs (a long launch: fewer, fatter CTAs cost
        // fewer instructions per byte); a short launch takes two or one, so that all of its loads are in flight at
        // once across the whole machine instead of queueing behind a few CTAs per SM.
        int unroll = kSwigluMaxUnroll;
        const unsigned long long want_ctas = static_cast<unsigned long long>(ctx->sm_count) * 8ull;
        while (unroll > 1 && (a.nvec + 256ull * unroll - 1) / (256ull * unroll) < want_ctas) unroll >>= 1;
        const long forced = tune_env("LOKAL_CUDA_SWIGLU_UNROLL", 0);
        if (forced == 1 || forced == 2 || forced == 4) unroll = static_cast<int>(forced);
        const unsigned long long per_cta = 256ull * unroll;
        const unsigned long long blocks = (a.nvec + per_cta - 1) / per_cta;
        if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "swiglu: too many elements for one launch");
        if (unroll == 4) launch_k(swiglu_kernel<T, 4>, static_cast<unsigned>(blocks), 256, 0, s, a);
        else if (unroll == 2) launch_k(swiglu_kernel<T, 2>, static_cast<unsigned>(blocks), 256, 0, s, a);
        else launch_k(swiglu_kernel<T, 1>, static_cast<unsigned>(blocks), 256, 0, s, a);
        LOKAL_CHECK_LAUNCH(ctx, "swiglu_kernel");
    }
    const unsigned long long first = a.nvec * N;
    if (first < a.n) {
        const unsigned long long blocks = (a.n - first + 255) / 256;
        if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "swiglu: too many elements for one launch");
        launch_k(swiglu_scalar_kernel<T>, static_cast<unsigned>(blocks), 256, 0, s, a, first);
        LOKAL_CHECK_LAUNCH(ctx, "swiglu_scalar_kernel");
    }
    return LOKAL_OK;
}

}  // namespace

int launch_swiglu(lokal_cuda_ctx* ctx, cudaStream_t s, const void* gate, const void* up, void* out, void* out_h,
                  size_t n, int dtype, int h_dtype) {
    if (!gate || !up || !out) return ctx->fail(LOKAL_ERR_BAD_ARG, "swiglu: gate, up and out must be non-null");
    if (!is_act_type(dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "swiglu: element type %d is not F32/F16/BF16", dtype);
    if (out_h) {
        if (dtype != LOKAL_F32) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "swiglu: the half copy needs F32 elements");
        if (h_dtype != LOKAL_F16 && h_dtype != LOKAL_BF16)
            return ctx->fail(LOKAL_ERR_UNSUPPORTED, "swiglu: half-copy type %d is not F16/BF16", h_dtype);
        if (!aligned_to(out_h, 2)) return ctx->fail(LOKAL_ERR_MISALIGNED, "swiglu: half copy is not 2-byte aligned");
    }
    const size_t es = type_size(dtype);
    if (!aligned_to(gate, es) || !aligned_to(up, es) || !aligned_to(out, es))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "swiglu: a pointer is not aligned to its element size");
    if (n == 0) return LOKAL_OK;
    SwigluArgs a{};
    a.gate = gate;
    a.up = up;
    a.out = out;
    a.out_h = out_h;
    a.n = n;
    a.h_dtype = h_dtype;
    a.prefetch = prefetch_enabled();
    const bool aligned = aligned_to(gate, 16) && aligned_to(up, 16) && aligned_to(out, 16) && (!out_h || aligned_to(out_h, 8));
    switch (dtype) {
        case LOKAL_F32: return launch_typed<float>(ctx, s, a, aligned);
        case LOKAL_F16: return launch_typed<__half>(ctx, s, a, aligned);
        default: return launch_typed<__nv_bfloat16>(ctx, s, a, aligned);
    }
}

}  // namespace lokal
