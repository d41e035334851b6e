// Shared device helpers and the context object of liblokal_cuda.
//
// All kernels here are HBM-bound streaming kernels for sm_100a: 128-bit
// coalesced accesses, rows kept in registers between the reduction and the
// scaled store (one pass over HBM), streaming cache hints on data touched
// once. f32 arithmetic follows the reference's expression shapes; the library
// is compiled with -fmad=false so multiplies and adds are rounded separately,
// as in the reference's Rust code, and sqrt/div are the IEEE versions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <set>
#include <vector>
#include <utility>
#include <string>

#include "../../include/lokal_cuda.h"

namespace lokal {

constexpr int kSmCountB200 = 148;

// Device-side error word bits (read back by lokal_cuda_stream_sync).
enum : unsigned { kErrIdRange = 1u, kErrTimeout = 2u, kErrPosRange = 4u };

}  // namespace lokal

struct lokal_cuda_ctx {
    int device = 0;
    int sm_count = lokal::kSmCountB200;
    unsigned* err_word = nullptr;      // device, 4 bytes
    unsigned* err_word_host = nullptr; // pinned, 4 bytes
    // cos/sin table of lokal_cuda_qk_rope_pos, used in stream order on the caller's streams
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    bool scratch_in_graph = false;         // a captured graph holds the block's address: it is retired, not freed, on growth
    void* retired_scratch[8] = {};         // such blocks, freed with the context
    int n_retired = 0;
    // device block of the host-slice mirrors (lokal_cuda_host_*), used on host_stream only, under `mu`
    void* host_scratch = nullptr;
    size_t host_scratch_bytes = 0;
    void* staging = nullptr;  // pinned host
    size_t staging_bytes = 0;
    cudaStream_t host_stream = nullptr;
    cudaStream_t copy_streams[8] = {};  // device-to-host workers of the host-slice gather, created on first use
    cudaEvent_t copy_ready = nullptr;
    cudaEvent_t scratch_event = nullptr;  // recorded after the last stream-ordered use of `scratch` (qk_rope_pos)
    bool scratch_event_recorded = false;
    void* iq_grids[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // device copies of the caller's i-quant codebooks
    std::mutex mu;  // guards scratch growth and the host-slice calls
    mutable std::mutex err_mu;
    std::string last_error;

    int fail(int code, const char* fmt, ...) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        std::lock_guard<std::mutex> g(err_mu);
        last_error = buf;
        return code;
    }
};

struct lokal_cuda_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

#define LOKAL_CUDA_TRY(ctx, expr)                                                                  \
    do {                                                                                           \
        cudaError_t e__ = (expr);                                                                  \
        if (e__ != cudaSuccess)                                                                    \
            return (ctx)->fail(LOKAL_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));   \
    } while (0)

#define LOKAL_CHECK_LAUNCH(ctx, what)                                                              \
    do {                                                                                           \
        cudaError_t e__ = cudaGetLastError();                                                      \
        if (e__ != cudaSuccess)                                                                    \
            return (ctx)->fail(LOKAL_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e__)); \
    } while (0)

namespace lokal {

// RAII device selection for every entry point.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

inline bool is_act_type(int t) { return t == LOKAL_F32 || t == LOKAL_F16 || t == LOKAL_BF16; }
inline size_t type_size(int t) { return t == LOKAL_F32 ? 4 : 2; }
inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---------------------------------------------------------------------------
// 16-byte vector access
// ---------------------------------------------------------------------------

template <typename T>
struct VecOf;  // elements per 16-byte vector
template <>
struct VecOf<float> {
    static constexpr int N = 4;
};
template <>
struct VecOf<__half> {
    static constexpr int N = 8;
};
template <>
struct VecOf<__nv_bfloat16> {
    static constexpr int N = 8;
};

// Loads/stores of the activation streams (touched once per kernel): 16-byte loads that do not allocate in L1 (each
// byte is consumed once, by the thread that loaded it) and plain 16-byte stores. Chosen by measurement on B200 over
// the default-policy and the evict-first (.cs) forms, on the time of a whole step.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }
// The same accesses with an L2 eviction priority (createpolicy): `keep` for the few megabytes a chain of launches
// reads and rewrites again and again (the residual stream), so that they survive what streams through L2 between
// two of those launches.
__device__ __forceinline__ unsigned long long l2_policy_keep() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint4 ld_stream_l2(const void* p, unsigned long long pol) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.b32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ uint4 ld_keep_l2(const void* p, unsigned long long pol) {  // read-only data, cached in L1 too
    uint4 v;
    asm volatile("ld.global.nc.L2::cache_hint.v4.b32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ void st_stream_l2(void* p, uint4 v, unsigned long long pol) {
    asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(pol)
                 : "memory");
}
__device__ __forceinline__ uint4 ld_keep(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& v, float (&f)[VecOf<T>::N]);

template <>
__device__ __forceinline__ void unpack16<float>(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void unpack16<__half>(const uint4& v, float (&f)[8]) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        float2 t = __half22float2(h);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
template <>
__device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}

template <typename T>
__device__ __forceinline__ uint4 pack16(const float (&f)[VecOf<T>::N]);

template <>
__device__ __forceinline__ uint4 pack16<float>(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
template <>
__device__ __forceinline__ uint4 pack16<__half>(const float (&f)[8]) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *reinterpret_cast<unsigned*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float (&f)[8]) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *reinterpret_cast<unsigned*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Scalar element access by runtime type (weights, biases: small, cache-resident).
__device__ __forceinline__ float load_as_f32(const void* p, int type, size_t i) {
    if (type == LOKAL_F32) return __ldg(reinterpret_cast<const float*>(p) + i);
    unsigned short b = __ldg(reinterpret_cast<const unsigned short*>(p) + i);
    if (type == LOKAL_F16) return __half2float(__ushort_as_half(b));
    return __uint_as_float(static_cast<unsigned>(b) << 16);
}

// N consecutive elements starting at element index i (i % N == 0 and the base
// 16-byte aligned when vec_ok; otherwise scalar loads).
template <int N>
__device__ __forceinline__ void load_w(const void* p, int type, size_t i, bool vec_ok, float (&f)[N]) {
    if (vec_ok) {
        if (type == LOKAL_F32) {
#pragma unroll
            for (int j = 0; j < N / 4; j++) {
                float t[4];
                unpack16<float>(ld_keep(reinterpret_cast<const float*>(p) + i + 4 * j), t);
#pragma unroll
                for (int k = 0; k < 4; k++) f[4 * j + k] = t[k];
            }
        } else if constexpr (N >= 8) {
#pragma unroll
            for (int j = 0; j < N / 8; j++) {
                float t[8];
                uint4 v = ld_keep(reinterpret_cast<const unsigned short*>(p) + i + 8 * j);
                if (type == LOKAL_F16) unpack16<__half>(v, t);
                else unpack16<__nv_bfloat16>(v, t);
#pragma unroll
                for (int k = 0; k < 8; k++) f[8 * j + k] = t[k];
            }
        } else {  // N == 4 halves: one 8-byte load
            uint2 v = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned short*>(p) + i));
            const unsigned w[2] = {v.x, v.y};
#pragma unroll
            for (int k = 0; k < 2; k++) {
                if (type == LOKAL_F16) {
                    float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
                    f[2 * k] = t.x;
                    f[2 * k + 1] = t.y;
                } else {
                    f[2 * k] = __uint_as_float(w[k] << 16);
                    f[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
                }
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < N; j++) f[j] = load_as_f32(p, type, i + j);
    }
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

inline unsigned ceil_div(size_t a, size_t b) { return static_cast<unsigned>((a + b - 1) / b); }

// Diagnostic launch-shape overrides (LOKAL_CUDA_* environment variables, read per call; unset = the built-in
// heuristic). They change how work is split over threads, never the results.
inline long tune_env(const char* name, long fallback) {
    const char* v = getenv(name);
    if (!v || !*v) return fallback;
    char* end = nullptr;
    const long x = strtol(v, &end, 10);
    return end && *end == '\0' ? x : fallback;
}

// Reduction arithmetic for 16-bit rows. A result that is rounded to 8 or 11 significant bits on store does not
// depend on whether the f32 sum of squares used fused multiply-adds or whether the scale came from the hardware
// reciprocal square root (both within a few f32 ulps of the exact value), so 16-bit rows take the shorter
// instruction sequences; f32 rows keep the reference's separately rounded multiply/add and IEEE 1/sqrt.
template <typename T>
__device__ __forceinline__ float sq_acc(float acc, float v) {
    if (sizeof(T) == 2) return fmaf(v, v, acc);
    return acc + v * v;
}
template <typename T>
__device__ __forceinline__ float inv_rms(float sum_sq, float n, float inv_n, float eps) {
    if (sizeof(T) == 2) return rsqrtf(fmaf(sum_sq, inv_n, eps));
    return 1.0f / sqrtf(sum_sq / n + eps);
}

// ---------------------------------------------------------------------------
// Packed f32 arithmetic (Blackwell: two IEEE round-to-nearest f32 operations per
// lane in one instruction). mul2 / add2 give exactly the bits of two scalar
// multiplies / adds, so the reference's separately rounded products and sums
// are kept while the kernels issue half as many floating-point instructions.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
          "l"(*reinterpret_cast<unsigned long long*>(&c)));
    return *reinterpret_cast<float2*>(&d);
}

// 16 bytes <-> N/2 pairs of f32
template <typename T>
__device__ __forceinline__ void unpack16p(const uint4& v, float2 (&p)[VecOf<T>::N / 2]);
template <>
__device__ __forceinline__ void unpack16p<float>(const uint4& v, float2 (&p)[2]) {
    p[0] = make_float2(__uint_as_float(v.x), __uint_as_float(v.y));
    p[1] = make_float2(__uint_as_float(v.z), __uint_as_float(v.w));
}
template <>
__device__ __forceinline__ void unpack16p<__half>(const uint4& v, float2 (&p)[4]) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) p[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
}
template <>
__device__ __forceinline__ void unpack16p<__nv_bfloat16>(const uint4& v, float2 (&p)[4]) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) p[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u));
}
template <typename T>
__device__ __forceinline__ uint4 pack16p(const float2 (&p)[VecOf<T>::N / 2]);
template <>
__device__ __forceinline__ uint4 pack16p<float>(const float2 (&p)[2]) {
    return make_uint4(__float_as_uint(p[0].x), __float_as_uint(p[0].y), __float_as_uint(p[1].x), __float_as_uint(p[1].y));
}
template <>
__device__ __forceinline__ uint4 pack16p<__half>(const float2 (&p)[4]) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __half2 h = __floats2half2_rn(p[i].x, p[i].y);
        w[i] = *reinterpret_cast<unsigned*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ uint4 pack16p<__nv_bfloat16>(const float2 (&p)[4]) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __nv_bfloat162 h = __floats2bfloat162_rn(p[i].x, p[i].y);
        w[i] = *reinterpret_cast<unsigned*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---------------------------------------------------------------------------
// Bulk asynchronous copies (TMA, untiled form) completing on an mbarrier. No cluster multicast is used anywhere:
// the .shared::cluster qualifier below is only the address-space spelling of this CTA's own shared memory.
// Every wait is bounded; a caller that sees `false` records kErrTimeout in the context's error word and leaves.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t mbar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
// Bulk copy global -> this CTA's shared memory; src, dst and bytes are multiples of 16.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, unsigned bytes, uint32_t mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(mbar)
                 : "memory");
}
// The same copy with an L2 eviction priority for the lines it reads (createpolicy).
__device__ __forceinline__ void bulk_copy_g2s_l2(uint32_t dst, const void* src, unsigned bytes, uint32_t mbar, unsigned long long pol) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(mbar), "l"(pol)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t mbar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(mbar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Polls before a wait gives up. LOKAL_CUDA_WAIT_LIMIT (read per launch) lowers it and LOKAL_CUDA_TEST_EXTRA_TX makes a
// staged copy announce more bytes than it delivers, so that a test can watch a wait run out and come back as
// LOKAL_ERR_TIMEOUT; nothing else uses them.
constexpr unsigned kWaitLimit = 1u << 20;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, unsigned parity, unsigned limit = kWaitLimit) {
    for (unsigned spin = 0; spin < limit; spin++) {
        if (mbar_try_wait(mbar, parity)) return true;
    }
    return false;
}

// ---------------------------------------------------------------------------
// Kernel launch with programmatic dependent launch (PDL). Each kernel of this library begins with pdl_sync():
// it lets the next kernel in the stream start its launch and block scheduling while this one drains, and it
// waits until the kernel before it has completed (and its writes are visible) before touching global memory.
// Stream order semantics are unchanged; what is hidden is launch latency between the short kernels of a step.
// LOKAL_CUDA_PDL=0 turns the launch attribute off (the device-side calls then return at once).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_sync() {
    pdl_launch();
    pdl_wait();
}

// A kernel's CTAs become resident while the kernel before it drains, and then sit in pdl_wait(). Before they
// wait they may ask L2 for the lines they are about to load: a prefetch reads nothing into the SM, and L2 is the
// point every write of the earlier kernel passes through, so a line fetched early is still the current one when
// the load comes. What is gained is the HBM latency of a kernel's first wave of loads, which otherwise starts
// only after the previous kernel has finished; for kernels of 10-25 us that ramp is a tenth of the run time.
// Only addresses the thread will load are prefetched. LOKAL_CUDA_PREFETCH=0 turns it off (read per call).
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
inline int prefetch_enabled() { return tune_env("LOKAL_CUDA_PREFETCH", 1) != 0; }

inline bool pdl_enabled() {
    static const bool on = tune_env("LOKAL_CUDA_PDL", 1) != 0;
    return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    // Every kernel of the library asks for the same L1/shared-memory split. Two of them stage rows in shared memory,
    // the others use next to none; left to the driver each would get its own split, and an SM has to drain before
    // its split can change (measured: several microseconds between consecutive kernels of a step). 60 % shared
    // memory gave the shortest step on B200; LOKAL_CUDA_CARVEOUT=<percent> overrides it, -1 leaves it to the driver.
    {
        static const long carve = tune_env("LOKAL_CUDA_CARVEOUT", 60);
        if (carve >= 0 && carve <= 100) {
            static std::mutex mu;
            static std::set<std::pair<int, const void*>> done;
            int dev = 0;
            cudaGetDevice(&dev);
            const std::pair<int, const void*> key(dev, reinterpret_cast<const void*>(kernel));
            std::lock_guard<std::mutex> g(mu);
            if (done.find(key) == done.end()) {
                cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, static_cast<int>(carve));
                done.insert(key);
            }
        }
    }
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace lokal

// Launchers implemented in the per-op translation units.
namespace lokal {
int launch_norm(lokal_cuda_ctx* ctx, cudaStream_t s, void* x, const void* delta, const void* w, void* xn, void* xn_h,
                size_t rows, size_t dim, float eps, int dtype, int w_dtype, int h_dtype);
int launch_rope_table(lokal_cuda_ctx* ctx, cudaStream_t s, float theta, uint32_t rot_dim, const int32_t* positions,
                      int64_t pos0, size_t rows, float* cos_sin);
// `shared_machine`: the caller runs other kernels beside this one (the branched schedule of the layer pass); a short
// launch then takes its compact shape (one warp per row) instead of the one that is fastest alone.
int launch_qk_rope(lokal_cuda_ctx* ctx, cudaStream_t s, const lokal_qk_rope_params& p, bool shared_machine = false);
int launch_swiglu(lokal_cuda_ctx* ctx, cudaStream_t s, const void* gate, const void* up, void* out, void* out_h,
                  size_t n, int dtype, int h_dtype);
int launch_gather(lokal_cuda_ctx* ctx, cudaStream_t s, const void* table, int ggml_type, size_t vocab, size_t dim,
                  const uint32_t* ids, size_t n, void* out, int out_dtype);
int launch_gather_norm(lokal_cuda_ctx* ctx, cudaStream_t s, const void* table, int ggml_type, size_t vocab, size_t dim,
                       const uint32_t* ids, size_t n, void* out, int out_dtype, const void* norm_w, int w_dtype, void* xn,
                       float eps, int* launches);
}  // namespace lokal
