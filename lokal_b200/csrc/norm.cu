// RMSNorm and fused residual-add + RMSNorm over token rows.
//
// Semantics follow math::rmsnorm (src/math.rs:45-49 of the reference):
//   mean_sq = sum(x_i^2) / n;  scale = 1 / sqrt(mean_sq + eps);  y_i = (x_i * scale) * w_i
// preceded, when a delta is given, by the residual add x_i += delta_i
// (src/model.rs:235-237, 253-255). The sum of squares is reduced in parallel
// (lane partials, warp shuffle, then shared memory across warps), so it differs
// from the reference's 8-lane order in the last bits of the scale only.
//
// Kernel shape: one warp per row (rows kept in registers, no barrier) while
// there are enough rows to fill the machine, otherwise one CTA per row. Each
// thread owns up to VPT 16-byte vectors of the row; x and delta are read once,
// x' and xn written once: 4*dim*sizeof(T) bytes of HBM traffic per row.
#include "common.cuh"

#include <type_traits>

namespace lokal {
namespace {

struct NormArgs {
    const void* x;
    const void* delta;  // may be null
    const void* w;
    void* x_out;  // where x + delta goes (null when no delta)
    void* xn;
    void* xn_h;  // may be null
    size_t rows;
    unsigned dim;
    unsigned nvec;
    float eps;
    float inv_dim;
    int w_dtype;
    int h_dtype;
    int w_vec_ok;
    int prefetch;  // ask L2 for the row before waiting for the previous kernel
    int l2_keep;   // x is read and rewritten by a chain of launches: give it the high L2 priority, the rest the low one
};

template <typename T, int N>
__device__ __forceinline__ void store_h_copy(void* base, int h_dtype, size_t elem, const float (&y)[N]) {
    // second copy of the row in f16 / bf16 (only used with f32 rows: N == 4 -> 8 bytes)
    unsigned w[N / 2];
#pragma unroll
    for (int i = 0; i < N / 2; i++) {
        if (h_dtype == LOKAL_F16) {
            __half2 h = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
            w[i] = *reinterpret_cast<unsigned*>(&h);
        } else {
            __nv_bfloat162 h = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
            w[i] = *reinterpret_cast<unsigned*>(&h);
        }
    }
    unsigned short* p = reinterpret_cast<unsigned short*>(base) + elem;
    if (N == 4) *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
    else {
#pragma unroll
        for (int i = 0; i < N / 2; i++) reinterpret_cast<unsigned*>(p)[i] = w[i];
    }
}

// WSAME: the weight vector has the rows' element type and is 16-byte aligned, so it is read like a row (the
// usual case); otherwise through the type-switching loader. Arithmetic is packed f32x2 throughout: the same bits
// as scalar round-to-nearest operations at half the instruction count (the kernel is as much issue-bound as
// memory-bound: two loads and two stores per thread against some hundred instructions).
#ifndef LOKAL_NORM_WARP_MIN_CTAS
#define LOKAL_NORM_WARP_MIN_CTAS 1  // resident 256-thread CTAs per SM the warp-per-row shape is compiled for
#endif
template <typename T, int VPT, bool CTA_MODE, bool WSAME>
__global__ void __launch_bounds__(CTA_MODE ? 1024 : 256, CTA_MODE ? 1 : LOKAL_NORM_WARP_MIN_CTAS) norm_rows_kernel(const NormArgs a) {
    pdl_launch();
    constexpr int N = VecOf<T>::N, P = N / 2;
    const unsigned tpr = CTA_MODE ? blockDim.x : 32u;
    const unsigned t = CTA_MODE ? threadIdx.x : (threadIdx.x & 31u);
    const size_t row = CTA_MODE ? static_cast<size_t>(blockIdx.x)
                                : static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (!CTA_MODE && row >= a.rows) return;  // whole warps leave together

    const size_t row_off = row * a.dim;
    const T* xr = reinterpret_cast<const T*>(a.x) + row_off;
    const T* dr = a.delta ? reinterpret_cast<const T*>(a.delta) + row_off : nullptr;
    if (a.prefetch) {  // one request per 128-byte line of the row, while the kernel before this one drains
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            const unsigned idx = t + j * tpr;
            if (idx < a.nvec && (idx & 7u) == 0) {
                prefetch_l2(xr + idx * N);
                if (dr) prefetch_l2(dr + idx * N);
            }
        }
    }
    pdl_wait();

    // All loads of the row are issued before any is consumed; in the CTA-per-row shape so are the loads of the weights
    // (of the rows' own type, the usual case), which do not depend on the reduction: left after it they would start
    // only behind the barrier, a cache round trip on the critical path of a short launch. (The warp-per-row shape has
    // no barrier, and four more vectors in registers would cost it a resident CTA per SM.)
    constexpr bool kEarlyW = WSAME && CTA_MODE;
    // The residual stream x is read and rewritten in place by every add-norm of a step (two per layer), with a few
    // hundred megabytes of other rows streaming through L2 between two of them. Its loads and stores carry the high L2
    // eviction priority, so that it stays on chip from one launch to the next: at 8192 rows of 2 KB the DRAM traffic of
    // a launch falls from 57.6 to 36.0 MB (ncu, steady state: what is left is delta in and xn out) and the 28-layer
    // step from 1.59-1.60 to 1.50-1.51 ms. delta and xn keep the default priority: the next consumer of xn is a
    // projection that should find it in L2.
    const bool keep = a.l2_keep != 0;
    const unsigned long long pol_keep = keep ? l2_policy_keep() : 0ull;
    uint4 xv[VPT], dv[VPT], wv4[kEarlyW ? VPT : 1];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        const unsigned idx = t + j * tpr;
        if (idx < a.nvec) {
            xv[j] = keep ? ld_stream_l2(xr + idx * N, pol_keep) : ld_stream(xr + idx * N);
            if (dr) dv[j] = ld_stream(dr + idx * N);
            if (kEarlyW) wv4[j] = ld_keep(reinterpret_cast<const T*>(a.w) + idx * N);
        }
    }

    float2 v[VPT][P];
    float2 acc2 = make_float2(0.0f, 0.0f);
    T* xo = reinterpret_cast<T*>(a.x_out) + row_off;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        const unsigned idx = t + j * tpr;
        if (idx < a.nvec) {
            unpack16p<T>(xv[j], v[j]);
            if (dr) {
                float2 d[P];
                unpack16p<T>(dv[j], d);
#pragma unroll
                for (int e = 0; e < P; e++) v[j][e] = add2(v[j][e], d[e]);
                if (keep) st_stream_l2(xo + idx * N, pack16p<T>(v[j]), pol_keep);
                else *reinterpret_cast<uint4*>(xo + idx * N) = pack16p<T>(v[j]);
            }
#pragma unroll
            for (int e = 0; e < P; e++) {
                if (sizeof(T) == 2) acc2 = fma2(v[j][e], v[j][e], acc2);
                else acc2 = add2(acc2, mul2(v[j][e], v[j][e]));  // separately rounded product and sum, as the reference
            }
        }
    }

    float acc = warp_sum(acc2.x + acc2.y);
    if (CTA_MODE) {
        __shared__ __align__(16) float partial[32];
        const unsigned warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
        if ((threadIdx.x & 31u) == 0) partial[warp] = acc;
        __syncthreads();
        float total;
        if (nwarps == 4) {  // the usual shape (rows of 2 KB): one 16-byte read, the same left-to-right sum
            const float4 p4 = *reinterpret_cast<const float4*>(partial);
            total = ((p4.x + p4.y) + p4.z) + p4.w;
        } else {
            total = 0.0f;
            for (unsigned wv = 0; wv < nwarps; wv++) total += partial[wv];
        }
        acc = total;
    }
    const float scale = inv_rms<T>(acc, static_cast<float>(a.dim), a.inv_dim, a.eps);
    const float2 s2 = make_float2(scale, scale);

    T* yr = reinterpret_cast<T*>(a.xn) + row_off;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        const unsigned idx = t + j * tpr;
        if (idx < a.nvec) {
            float2 w[P];
            if (kEarlyW) {
                unpack16p<T>(wv4[j], w);
            } else if (WSAME) {
                unpack16p<T>(ld_keep(reinterpret_cast<const T*>(a.w) + idx * N), w);
            } else {
                float wv[N];
                load_w<N>(a.w, a.w_dtype, static_cast<size_t>(idx) * N, a.w_vec_ok, wv);
#pragma unroll
                for (int e = 0; e < P; e++) w[e] = make_float2(wv[2 * e], wv[2 * e + 1]);
            }
            float2 y[P];
#pragma unroll
            for (int e = 0; e < P; e++) y[e] = mul2(mul2(v[j][e], s2), w[e]);  // (x * scale) * w
            *reinterpret_cast<uint4*>(yr + idx * N) = pack16p<T>(y);
            if (sizeof(T) == 4 && a.xn_h) {
                float yf[N];
#pragma unroll
                for (int e = 0; e < P; e++) {
                    yf[2 * e] = y[e].x;
                    yf[2 * e + 1] = y[e].y;
                }
                store_h_copy<T, N>(a.xn_h, a.h_dtype, row_off + static_cast<size_t>(idx) * N, yf);
            }
        }
    }
}

// Any dim, any alignment: one CTA per row, scalar accesses, the row is read
// twice (the second read hits L1/L2).
template <typename T>
__global__ void __launch_bounds__(256) norm_rows_generic_kernel(const NormArgs a) {
    pdl_sync();
    const size_t row = blockIdx.x;
    const T* xr = reinterpret_cast<const T*>(a.x) + row * a.dim;
    const T* dr = a.delta ? reinterpret_cast<const T*>(a.delta) + row * a.dim : nullptr;
    float acc = 0.0f;
    for (unsigned i = threadIdx.x; i < a.dim; i += blockDim.x) {
        float v = to_f32<T>(xr[i]);
        if (dr) v = v + to_f32<T>(dr[i]);
        acc += v * v;
    }
    acc = warp_sum(acc);
    __shared__ float partial[32];
    const unsigned warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    if ((threadIdx.x & 31u) == 0) partial[warp] = acc;
    __syncthreads();
    float total = 0.0f;
    for (unsigned wv = 0; wv < nwarps; wv++) total += partial[wv];
    const float mean_sq = total / static_cast<float>(a.dim);
    const float scale = 1.0f / sqrtf(mean_sq + a.eps);
    T* yr = reinterpret_cast<T*>(a.xn) + row * a.dim;
    T* xo = dr ? reinterpret_cast<T*>(a.x_out) + row * a.dim : nullptr;
    for (unsigned i = threadIdx.x; i < a.dim; i += blockDim.x) {
        float v = to_f32<T>(xr[i]);
        if (dr) {
            v = v + to_f32<T>(dr[i]);
            xo[i] = from_f32<T>(v);
        }
        const float y = (v * scale) * load_as_f32(a.w, a.w_dtype, i);
        yr[i] = from_f32<T>(y);
        if (a.xn_h) {
            unsigned short* hp = reinterpret_cast<unsigned short*>(a.xn_h) + row * a.dim + i;
            *hp = a.h_dtype == LOKAL_F16 ? __half_as_ushort(__float2half_rn(y))
                                         : __bfloat16_as_ushort(__float2bfloat16_rn(y));
        }
    }
}

template <typename T, bool CTA_MODE, bool WSAME>
cudaError_t launch_vec(const NormArgs& a, unsigned tpr, unsigned vpt, cudaStream_t s) {
    dim3 grid, block;
    if (CTA_MODE) {
        grid = dim3(static_cast<unsigned>(a.rows));
        block = dim3(tpr);
    } else {
        long wpc = tune_env("LOKAL_CUDA_NORM_WARPS", 8);  // rows (warps) per CTA in warp mode
        if (wpc != 1 && wpc != 2 && wpc != 4 && wpc != 8) wpc = 8;
        block = dim3(static_cast<unsigned>(wpc) * 32u);
        grid = dim3(ceil_div(a.rows, static_cast<size_t>(wpc)));
    }
    switch (vpt) {
        case 1: launch_k(norm_rows_kernel<T, 1, CTA_MODE, WSAME>, grid, block, 0, s, a); break;
        case 2: launch_k(norm_rows_kernel<T, 2, CTA_MODE, WSAME>, grid, block, 0, s, a); break;
        case 3: launch_k(norm_rows_kernel<T, 3, CTA_MODE, WSAME>, grid, block, 0, s, a); break;
        case 4: launch_k(norm_rows_kernel<T, 4, CTA_MODE, WSAME>, grid, block, 0, s, a); break;
        case 5: launch_k(norm_rows_kernel<T, 5, CTA_MODE, WSAME>, grid, block, 0, s, a); break;
        case 6: launch_k(norm_rows_kernel<T, 6, CTA_MODE, WSAME>, grid, block, 0, s, a); break;
        default: launch_k(norm_rows_kernel<T, 8, CTA_MODE, WSAME>, grid, block, 0, s, a); break;
    }
    return cudaGetLastError();
}

template <typename T>
int launch_typed(lokal_cuda_ctx* ctx, cudaStream_t s, NormArgs a, bool ptrs_aligned) {
    constexpr unsigned N = VecOf<T>::N;
    const bool vec = ptrs_aligned && a.dim % N == 0 && a.dim / N <= 1024u * 8u;
    if (!vec) {
        launch_k(norm_rows_generic_kernel<T>, static_cast<unsigned>(a.rows), 256, 0, s, a);
        LOKAL_CHECK_LAUNCH(ctx, "norm_rows_generic_kernel");
        return LOKAL_OK;
    }
    a.nvec = a.dim / N;
    // Threads per row. One 16-byte vector per thread (a CTA per row, shared-memory combine) keeps every CTA small and
    // short-lived, so the machine drains evenly at the end of the kernel; rows wider than 1024 vectors give each
    // thread several vectors, and rows of at most 32 vectors take one warp each, eight rows to a CTA. With enough
    // rows to give every SM 32 of them, rows of up to 128 vectors also take one warp each (four vectors per lane, no
    // barrier): measured at 8192 x 2 KB rows 12.0 against 12.3 us alone and 1.84 against 1.86 ms for the step;
    // at 2048 rows and fewer the one-vector shape wins.
    unsigned tpr = ((a.nvec + 31u) / 32u) * 32u;
    if (tpr > 1024) tpr = 1024;
    if (a.nvec <= 128 && a.rows >= static_cast<size_t>(ctx->sm_count) * 32u) tpr = 32;
    const long forced = tune_env("LOKAL_CUDA_NORM_TPR", 0);
    if (forced >= 32 && forced <= 1024 && forced % 32 == 0) tpr = static_cast<unsigned>(forced);
    while (tpr < 1024 && (a.nvec + tpr - 1) / tpr > 8) tpr *= 2;
    unsigned vpt = (a.nvec + tpr - 1) / tpr;
    if (vpt == 7) vpt = 8;
    // weights of the rows' own type, 16-byte aligned: read like a row
    const int own_type = sizeof(T) == 4 ? LOKAL_F32 : (std::is_same<T, __half>::value ? LOKAL_F16 : LOKAL_BF16);
    const bool wsame = a.w_dtype == own_type && a.w_vec_ok;
    cudaError_t e;
    if (tpr == 32) e = wsame ? launch_vec<T, false, true>(a, tpr, vpt, s) : launch_vec<T, false, false>(a, tpr, vpt, s);
    else e = wsame ? launch_vec<T, true, true>(a, tpr, vpt, s) : launch_vec<T, true, false>(a, tpr, vpt, s);
    if (e != cudaSuccess) return ctx->fail(LOKAL_ERR_CUDA, "launch of norm_rows_kernel failed: %s", cudaGetErrorString(e));
    return LOKAL_OK;
}

}  // namespace

int launch_norm(lokal_cuda_ctx* ctx, cudaStream_t s, void* x, const void* delta, const void* w, void* xn, void* xn_h,
                size_t rows, size_t dim, float eps, int dtype, int w_dtype, int h_dtype) {
    if (!x || !w || !xn) return ctx->fail(LOKAL_ERR_BAD_ARG, "rmsnorm: x, w and the output must be non-null");
    if (dim == 0 || dim > 0x7fffffffu) return ctx->fail(LOKAL_ERR_BAD_ARG, "rmsnorm: dim %zu out of range", dim);
    if (rows > 0x7fffffffu) return ctx->fail(LOKAL_ERR_BAD_ARG, "rmsnorm: rows %zu out of range", rows);
    if (!is_act_type(dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "rmsnorm: row type %d is not F32/F16/BF16", dtype);
    if (!is_act_type(w_dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "rmsnorm: weight type %d is not F32/F16/BF16", w_dtype);
    if (xn_h) {
        if (dtype != LOKAL_F32) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "rmsnorm: the half copy needs F32 rows");
        if (h_dtype != LOKAL_F16 && h_dtype != LOKAL_BF16)
            return ctx->fail(LOKAL_ERR_UNSUPPORTED, "rmsnorm: half-copy type %d is not F16/BF16", h_dtype);
        if (!aligned_to(xn_h, 2)) return ctx->fail(LOKAL_ERR_MISALIGNED, "rmsnorm: half copy is not 2-byte aligned");
    }
    const size_t es = type_size(dtype);
    if (!aligned_to(x, es) || !aligned_to(xn, es) || (delta && !aligned_to(delta, es)) ||
        !aligned_to(w, type_size(w_dtype)))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "rmsnorm: a pointer is not aligned to its element size");
    if (rows == 0) return LOKAL_OK;

    NormArgs a{};
    a.x = x;
    a.delta = delta;
    a.w = w;
    a.x_out = delta ? x : nullptr;
    a.xn = xn;
    a.xn_h = xn_h;
    a.rows = rows;
    a.dim = static_cast<unsigned>(dim);
    a.eps = eps;
    a.inv_dim = 1.0f / static_cast<float>(dim);
    a.w_dtype = w_dtype;
    a.h_dtype = h_dtype;
    a.w_vec_ok = aligned_to(w, 16);
    a.prefetch = prefetch_enabled();
    // x of an add-norm is a residual stream (see the kernel): kept in L2 when it is small against the 126 MB there.
    // LOKAL_CUDA_NORM_L2_KEEP=0 turns the priority off.
    a.l2_keep = (delta != nullptr && rows * dim * es <= (32u << 20) && tune_env("LOKAL_CUDA_NORM_L2_KEEP", 1) != 0) ? 1 : 0;
    const bool aligned = aligned_to(x, 16) && aligned_to(xn, 16) && (!delta || aligned_to(delta, 16)) &&
                         (!xn_h || aligned_to(xn_h, 8)) && (dim * es) % 16 == 0;
    switch (dtype) {
        case LOKAL_F32: return launch_typed<float>(ctx, s, a, aligned);
        case LOKAL_F16: return launch_typed<__half>(ctx, s, a, aligned);
        default: return launch_typed<__nv_bfloat16>(ctx, s, a, aligned);
    }
}

}  // namespace lokal
