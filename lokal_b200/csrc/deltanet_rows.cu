// Per-row siblings of the layer path inside the gated-deltanet (qwen35) blocks:
//   l2norm_rows        x / max(sqrt(sum x^2), eps)                 src/deltanet_ref.rs:61-67,  src/gpu/kernels.metal:3697-3735
//   gated_output_norm  ((o * scale) * w) * silu(z), per head       src/deltanet_ref.rs:187-198, src/gpu/kernels.metal:3936-3975
//   attn_out_gate      attn * sigmoid(gate)                        src/deltanet_ref.rs:203-207, src/gpu/kernels.metal:3667-3676
//   split_q_gate       [q | gate] per head -> compact q, gate      src/gpu/kernels.metal:4106-4124
//
// The reference's CPU code sums squares in f64 (ggml_float); its Metal kernels sum in f32 only because Metal has
// no f64, and its tests bound that gap. This device has f64, so the sums here are f64 like the CPU reference:
// every square of an f32 is exact in f64, the sum's rounding error sits 29 bits below an f32 ulp, and the value
// narrowed to f32 is the reference's except where the f64 sum lands within that margin of an f32 rounding
// boundary. sqrt, the reciprocal and the divisions are IEEE; exp is the library's expf (1 ulp), the one place the
// result may differ from the reference's by more than the order of a sum.
//
// All four are HBM-bound streams: one warp per row with the row in registers (one 16-byte vector per lane for the
// 128-wide rows of the model), 16 bytes per lane for the elementwise ones. Rows of f16 / bf16 are widened on
// load and rounded once on store.
#include "common.cuh"

#include <type_traits>

namespace lokal {
namespace {

struct RowNormArgs {
    const void* x;
    void* y;
    const void* w;  // gated_output_norm only
    const void* z;  // gated_output_norm only
    unsigned long long rows, tok_stride;  // row g = (t, r): element offset t*tok_stride + r*dim; tok_stride 0 = contiguous rows
    unsigned rows_per_token;
    double inv_dim;  // 1 / dim when dim is a power of two (the product is then the quotient, exactly), else 0
    unsigned dim;
    float eps;
    int w_dtype;
    int w_vec_ok;
};

// Element offset of row g. Contiguous rows (one token, or tokens packed back to back) need one multiply; the strided
// form divides in 32 bits (the host refuses more than 2^32 - 1 rows): a 64-bit division costs more than the rest of
// the kernel.
__device__ __forceinline__ unsigned long long row_offset(const RowNormArgs& a, unsigned long long g) {
    if (a.tok_stride == 0) return g * a.dim;
    const unsigned g32 = static_cast<unsigned>(g), t = g32 / a.rows_per_token;
    return static_cast<unsigned long long>(t) * a.tok_stride + static_cast<unsigned long long>(g32 - t * a.rows_per_token) * a.dim;
}

// mean of squares as the reference takes it: the f64 sum divided by n, narrowed to f32
__device__ __forceinline__ float mean_f32(const RowNormArgs& a, double sum) {
    return static_cast<float>(a.inv_dim != 0.0 ? sum * a.inv_dim : sum / static_cast<double>(a.dim));
}

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 1 / (1 + exp(-x)); the correctly rounded reciprocal is the same f32 as the IEEE division 1.0f / y, without the
// division's slow path.
__device__ __forceinline__ float sigmoid_f32(float x) { return __frcp_rn(1.0f + expf(-x)); }

// MODE 0: l2norm. MODE 1: gated output norm. A warp owns kRowsPerWarp consecutive rows of up to VPT 16-byte vectors
// per lane and issues every load of all of them before the first reduction. Measured at 128-wide f32 rows: four
// rows per warp are slower than one (l2norm 52 vs 50 us, gated norm 168 vs 115 us for 8192 x 48 rows): the
// registers they hold halve the resident warps and the f64 reductions of a warp's rows run one after another.
#ifndef LOKAL_DELTANET_ROWS_PER_WARP
#define LOKAL_DELTANET_ROWS_PER_WARP 1
#endif
constexpr int kRowsPerWarp = LOKAL_DELTANET_ROWS_PER_WARP;

template <typename T, int VPT, int MODE>
__global__ void __launch_bounds__(256) deltanet_rows_kernel(const RowNormArgs a) {
    pdl_sync();
    constexpr int N = VecOf<T>::N;
    constexpr int RPW = kRowsPerWarp;
    const unsigned long long g0 = ((static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * RPW;
    if (g0 >= a.rows) return;
    const unsigned lane = threadIdx.x & 31u;
    unsigned long long off[RPW];
    uint4 v[RPW][VPT], zv[RPW][VPT];
#pragma unroll
    for (int r = 0; r < RPW; r++) {
        const unsigned long long g = g0 + r;
        off[r] = row_offset(a, g);
        if (g < a.rows) {
#pragma unroll
            for (int j = 0; j < VPT; j++) {
                const unsigned e = (j * 32 + lane) * N;
                if (e < a.dim) {
                    v[r][j] = ld_stream(reinterpret_cast<const T*>(a.x) + off[r] + e);
                    if (MODE == 1) zv[r][j] = ld_stream(reinterpret_cast<const T*>(a.z) + off[r] + e);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RPW; r++) {
        if (g0 + r >= a.rows) break;  // uniform across the warp
        double acc = 0.0;
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            if ((j * 32 + lane) * N < a.dim) {
                float f[N];
                unpack16<T>(v[r][j], f);
#pragma unroll
                for (int k = 0; k < N; k++) acc += static_cast<double>(f[k]) * static_cast<double>(f[k]);
            }
        }
        acc = warp_sum_f64(acc);
        float scale;
        if (MODE == 0) scale = 1.0f / fmaxf(static_cast<float>(sqrt(acc)), a.eps);
        else scale = 1.0f / sqrtf(mean_f32(a, acc) + a.eps);
        T* dst = reinterpret_cast<T*>(a.y) + off[r];
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            const unsigned e = (j * 32 + lane) * N;
            if (e < a.dim) {
                float f[N];
                unpack16<T>(v[r][j], f);
                if (MODE == 0) {
#pragma unroll
                    for (int k = 0; k < N; k++) f[k] = f[k] * scale;
                } else {
                    float w[N], z[N];
                    load_w<N>(a.w, a.w_dtype, e, a.w_vec_ok, w);
                    unpack16<T>(zv[r][j], z);
#pragma unroll
                    for (int k = 0; k < N; k++) f[k] = ((f[k] * scale) * w[k]) * (z[k] * sigmoid_f32(z[k]));
                }
                st_stream(dst + e, pack16<T>(f));
            }
        }
    }
}

// Any dim, any alignment: one CTA of 256 threads per row, the row read twice (the second read hits L1/L2).
template <typename T, int MODE>
__global__ void __launch_bounds__(256) deltanet_rows_generic_kernel(const RowNormArgs a) {
    pdl_sync();
    __shared__ double part[8];
    const unsigned long long g = blockIdx.x;
    const unsigned long long off = row_offset(a, g);
    const T* src = reinterpret_cast<const T*>(a.x) + off;
    T* dst = reinterpret_cast<T*>(a.y) + off;
    double acc = 0.0;
    for (unsigned i = threadIdx.x; i < a.dim; i += 256) {
        const double f = static_cast<double>(to_f32<T>(src[i]));
        acc += f * f;
    }
    acc = warp_sum_f64(acc);
    if ((threadIdx.x & 31u) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    double total = 0.0;
#pragma unroll
    for (int j = 0; j < 8; j++) total += part[j];
    float scale;
    if (MODE == 0) scale = 1.0f / fmaxf(static_cast<float>(sqrt(total)), a.eps);
    else scale = 1.0f / sqrtf(mean_f32(a, total) + a.eps);
    for (unsigned i = threadIdx.x; i < a.dim; i += 256) {
        float f = to_f32<T>(src[i]);
        if (MODE == 0) {
            f = f * scale;
        } else {
            const float z = to_f32<T>(reinterpret_cast<const T*>(a.z)[off + i]);
            f = ((f * scale) * load_as_f32(a.w, a.w_dtype, i)) * (z * sigmoid_f32(z));
        }
        dst[i] = from_f32<T>(f);
    }
}

struct GateArgs {
    const void* attn;
    const void* gate;
    void* out;
    unsigned long long n;
};

template <typename T>
__global__ void __launch_bounds__(256) attn_out_gate_kernel(const GateArgs a, int vec_ok) {
    pdl_sync();
    constexpr int N = VecOf<T>::N;
    const unsigned long long t = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const T* at = reinterpret_cast<const T*>(a.attn);
    const T* gt = reinterpret_cast<const T*>(a.gate);
    T* out = reinterpret_cast<T*>(a.out);
    const unsigned long long e = t * N;
    if (e >= a.n) return;
    if (vec_ok && e + N <= a.n) {
        float x[N], g[N];
        unpack16<T>(ld_stream(at + e), x);
        unpack16<T>(ld_stream(gt + e), g);
#pragma unroll
        for (int k = 0; k < N; k++) x[k] = x[k] * sigmoid_f32(g[k]);
        st_stream(out + e, pack16<T>(x));
    } else {
        for (unsigned long long i = e; i < e + N && i < a.n; i++) out[i] = from_f32<T>(to_f32<T>(at[i]) * sigmoid_f32(to_f32<T>(gt[i])));
    }
}

struct SplitArgs {
    const void* src;
    void* q;
    void* gate;
    unsigned long long heads_total;  // rows * n_heads
    unsigned head_dim;
};

// One 16-byte vector of the source per thread (or one element when the shapes are not vectorisable): consecutive
// threads read consecutive vectors; vector v of a head's 2*hd elements goes to q for v < hd/N, to gate otherwise.
template <int BYTES>
__global__ void __launch_bounds__(256) split_q_gate_kernel(const SplitArgs a) {
    pdl_sync();
    using V = typename std::conditional<BYTES == 16, uint4, typename std::conditional<BYTES == 4, unsigned, unsigned short>::type>::type;
    const unsigned per_half = a.head_dim;  // in units of V
    const unsigned long long t = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const unsigned long long head = t / (2ull * per_half);
    if (head >= a.heads_total) return;
    const unsigned within = static_cast<unsigned>(t % (2ull * per_half));
    const V v = reinterpret_cast<const V*>(a.src)[t];
    if (within < per_half) reinterpret_cast<V*>(a.q)[head * per_half + within] = v;
    else reinterpret_cast<V*>(a.gate)[head * per_half + (within - per_half)] = v;
}

template <typename T, int MODE>
int launch_rows_t(lokal_cuda_ctx* ctx, cudaStream_t s, const RowNormArgs& a, bool vec_ok) {
    constexpr int N = VecOf<T>::N;
    const unsigned nvec = (a.dim + N - 1) / N;
    const char* what = MODE == 0 ? "l2norm_rows" : "gated_output_norm";
    if (vec_ok && nvec <= 128) {
        const unsigned rpw = kRowsPerWarp;
        const unsigned long long blocks = (a.rows + 8ull * rpw - 1) / (8ull * rpw);
        if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "%s: too many rows for one launch", what);
        const unsigned grid = static_cast<unsigned>(blocks);
        if (nvec <= 32) launch_k(deltanet_rows_kernel<T, 1, MODE>, grid, 256, 0, s, a);
        else if (nvec <= 64) launch_k(deltanet_rows_kernel<T, 2, MODE>, grid, 256, 0, s, a);
        else launch_k(deltanet_rows_kernel<T, 4, MODE>, grid, 256, 0, s, a);
    } else {
        if (a.rows > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "%s: too many rows for one launch", what);
        launch_k(deltanet_rows_generic_kernel<T, MODE>, static_cast<unsigned>(a.rows), 256, 0, s, a);
    }
    LOKAL_CHECK_LAUNCH(ctx, what);
    return LOKAL_OK;
}

template <int MODE>
int launch_rows(lokal_cuda_ctx* ctx, cudaStream_t s, const RowNormArgs& a, int dtype, bool vec_ok) {
    switch (dtype) {
        case LOKAL_F32: return launch_rows_t<float, MODE>(ctx, s, a, vec_ok);
        case LOKAL_F16: return launch_rows_t<__half, MODE>(ctx, s, a, vec_ok);
        default: return launch_rows_t<__nv_bfloat16, MODE>(ctx, s, a, vec_ok);
    }
}

}  // namespace
}  // namespace lokal

extern "C" {

int lokal_cuda_l2norm_rows(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* x, void* y, size_t rows_per_token, size_t n_tokens,
                           size_t tok_stride, size_t dim, float eps, int dtype) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    lokal::DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!x || !y) return ctx->fail(LOKAL_ERR_BAD_ARG, "l2norm_rows: x and y must be non-null");
    if (!lokal::is_act_type(dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "l2norm_rows: row type %d is not F32/F16/BF16", dtype);
    if (dim == 0 || dim > 0x7fffffffu) return ctx->fail(LOKAL_ERR_BAD_ARG, "l2norm_rows: dim %zu out of range", dim);
    if (n_tokens > 1 && tok_stride < rows_per_token * dim)
        return ctx->fail(LOKAL_ERR_BAD_ARG, "l2norm_rows: tok_stride %zu is smaller than a token's %zu rows of %zu", tok_stride, rows_per_token, dim);
    const size_t es = lokal::type_size(dtype);
    if (!lokal::aligned_to(x, es) || !lokal::aligned_to(y, es)) return ctx->fail(LOKAL_ERR_MISALIGNED, "l2norm_rows: a pointer is not aligned to its element size");
    if (rows_per_token == 0 || n_tokens == 0) return LOKAL_OK;
    lokal::RowNormArgs a{};
    a.x = x;
    a.y = y;
    a.rows = static_cast<unsigned long long>(rows_per_token) * n_tokens;
    if (a.rows > 0xffffffffull || rows_per_token > 0xffffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "l2norm_rows: too many rows for one launch");
    a.rows_per_token = static_cast<unsigned>(rows_per_token);
    a.tok_stride = (n_tokens > 1 && tok_stride != rows_per_token * dim) ? tok_stride : 0;  // 0: rows back to back
    a.dim = static_cast<unsigned>(dim);
    a.eps = eps;
    const bool vec_ok = lokal::aligned_to(x, 16) && lokal::aligned_to(y, 16) && (dim * es) % 16 == 0 && (a.tok_stride * es) % 16 == 0;
    return lokal::launch_rows<0>(ctx, static_cast<cudaStream_t>(s), a, dtype, vec_ok);
}

int lokal_cuda_gated_output_norm(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* o, const void* w, const void* z, void* y,
                                 size_t rows, size_t dim, float eps, int dtype, int w_dtype) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    lokal::DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!o || !w || !z || !y) return ctx->fail(LOKAL_ERR_BAD_ARG, "gated_output_norm: o, w, z and y must be non-null");
    if (!lokal::is_act_type(dtype) || !lokal::is_act_type(w_dtype))
        return ctx->fail(LOKAL_ERR_UNSUPPORTED, "gated_output_norm: types %d / %d are not F32/F16/BF16", dtype, w_dtype);
    if (dim == 0 || dim > 0x7fffffffu) return ctx->fail(LOKAL_ERR_BAD_ARG, "gated_output_norm: dim %zu out of range", dim);
    const size_t es = lokal::type_size(dtype);
    if (!lokal::aligned_to(o, es) || !lokal::aligned_to(z, es) || !lokal::aligned_to(y, es) || !lokal::aligned_to(w, lokal::type_size(w_dtype)))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "gated_output_norm: a pointer is not aligned to its element size");
    if (rows == 0) return LOKAL_OK;
    lokal::RowNormArgs a{};
    a.x = o;
    a.y = y;
    a.w = w;
    a.z = z;
    a.rows = rows;
    if (rows > 0xffffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "gated_output_norm: too many rows for one launch");
    a.rows_per_token = static_cast<unsigned>(rows);
    a.tok_stride = 0;
    a.inv_dim = (dim & (dim - 1)) == 0 ? 1.0 / static_cast<double>(dim) : 0.0;
    a.dim = static_cast<unsigned>(dim);
    a.eps = eps;
    a.w_dtype = w_dtype;
    a.w_vec_ok = lokal::aligned_to(w, 16) && (dim * lokal::type_size(w_dtype)) % 16 == 0;
    const bool vec_ok = lokal::aligned_to(o, 16) && lokal::aligned_to(z, 16) && lokal::aligned_to(y, 16) && (dim * es) % 16 == 0;
    return lokal::launch_rows<1>(ctx, static_cast<cudaStream_t>(s), a, dtype, vec_ok);
}

int lokal_cuda_attn_out_gate(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* attn, const void* gate, void* out, size_t n, int dtype) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    lokal::DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!attn || !gate || !out) return ctx->fail(LOKAL_ERR_BAD_ARG, "attn_out_gate: attn, gate and out must be non-null");
    if (!lokal::is_act_type(dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "attn_out_gate: element type %d is not F32/F16/BF16", dtype);
    const size_t es = lokal::type_size(dtype);
    if (!lokal::aligned_to(attn, es) || !lokal::aligned_to(gate, es) || !lokal::aligned_to(out, es))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "attn_out_gate: a pointer is not aligned to its element size");
    if (n == 0) return LOKAL_OK;
    const size_t per = 16 / es;
    const unsigned long long blocks = ((n + per - 1) / per + 255) / 256;
    if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "attn_out_gate: too many elements for one launch");
    const int vec_ok = lokal::aligned_to(attn, 16) && lokal::aligned_to(gate, 16) && lokal::aligned_to(out, 16);
    lokal::GateArgs a{attn, gate, out, n};
    cudaStream_t st = static_cast<cudaStream_t>(s);
    const unsigned grid = static_cast<unsigned>(blocks);
    if (dtype == LOKAL_F32) lokal::launch_k(lokal::attn_out_gate_kernel<float>, grid, 256, 0, st, a, vec_ok);
    else if (dtype == LOKAL_F16) lokal::launch_k(lokal::attn_out_gate_kernel<__half>, grid, 256, 0, st, a, vec_ok);
    else lokal::launch_k(lokal::attn_out_gate_kernel<__nv_bfloat16>, grid, 256, 0, st, a, vec_ok);
    LOKAL_CHECK_LAUNCH(ctx, "attn_out_gate_kernel");
    return LOKAL_OK;
}

int lokal_cuda_split_q_gate(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const void* src, void* q, void* gate, size_t rows, size_t n_heads,
                            size_t head_dim, int dtype) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    lokal::DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!src || !q || !gate) return ctx->fail(LOKAL_ERR_BAD_ARG, "split_q_gate: src, q and gate must be non-null");
    if (!lokal::is_act_type(dtype)) return ctx->fail(LOKAL_ERR_UNSUPPORTED, "split_q_gate: element type %d is not F32/F16/BF16", dtype);
    if (n_heads == 0 || head_dim == 0 || head_dim > 0x3fffffffu) return ctx->fail(LOKAL_ERR_BAD_ARG, "split_q_gate: n_heads and head_dim must be non-zero");
    const size_t es = lokal::type_size(dtype);
    if (!lokal::aligned_to(src, es) || !lokal::aligned_to(q, es) || !lokal::aligned_to(gate, es))
        return ctx->fail(LOKAL_ERR_MISALIGNED, "split_q_gate: a pointer is not aligned to its element size");
    if (src == q || src == gate || q == gate) return ctx->fail(LOKAL_ERR_BAD_ARG, "split_q_gate: src, q and gate must be distinct buffers");
    if (rows == 0) return LOKAL_OK;
    const bool vec = lokal::aligned_to(src, 16) && lokal::aligned_to(q, 16) && lokal::aligned_to(gate, 16) && (head_dim * es) % 16 == 0;
    lokal::SplitArgs a{src, q, gate, static_cast<unsigned long long>(rows) * n_heads, static_cast<unsigned>(vec ? head_dim * es / 16 : head_dim)};
    const unsigned long long threads = a.heads_total * 2ull * a.head_dim;
    const unsigned long long blocks = (threads + 255) / 256;
    if (blocks > 0x7fffffffull) return ctx->fail(LOKAL_ERR_BAD_ARG, "split_q_gate: too many elements for one launch");
    cudaStream_t st = static_cast<cudaStream_t>(s);
    const unsigned grid = static_cast<unsigned>(blocks);
    if (vec) lokal::launch_k(lokal::split_q_gate_kernel<16>, grid, 256, 0, st, a);
    else if (es == 4) lokal::launch_k(lokal::split_q_gate_kernel<4>, grid, 256, 0, st, a);
    else lokal::launch_k(lokal::split_q_gate_kernel<2>, grid, 256, 0, st, a);
    LOKAL_CHECK_LAUNCH(ctx, "split_q_gate_kernel");
    return LOKAL_OK;
}

}  // extern "C"
