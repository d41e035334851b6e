// CPU oracle for lokal's fused per-token layer ops.
//
// TEST INFRASTRUCTURE ONLY. This file is a plain C++ restatement of the
// reference's CPU algorithm for the hot path; it is the checker the CUDA
// library is compared against and the timed CPU baseline. Nothing in the
// shipped package may call it: only the test suite, the smoke check and the
// benchmark's CPU-baseline leg load this library.
//
// Parity status:
//   * GGUF dequant, block-size table, embedding gather: Q8_0, Q4_K, Q4_0, Q5_0,
//     Q2_K, Q3_K, Q5_K, Q6_K PINNED by the reference's own known-answer vectors
//     (src/gguf/dequant.rs:567-577, 579-766, 768-780); Q8_0 / Q4_K also by a
//     second, independently written per-element decoder in this file (the index
//     form of src/gpu/kernels.metal:77-81, 108-116, 889-904). IQ4_NL, IQ4_XS and
//     the seven codebook types have no hand vector in the reference: they are
//     pinned by agreeing bit for bit with independent numpy decoders (tests/).
//   * deltanet siblings (l2_norm, f64-mean rmsnorm, gated_output_norm,
//     attn_out_gate): pinned by src/deltanet_ref.rs:226-235, 306-329; sigmoid
//     shares the libm caveat below.
//   * deltanet per-token ops: softplus and the gate scalars pinned by
//     src/deltanet_ref.rs:225-236 (the > 20 shortcut exactly, ln 2 at zero);
//     conv_step by the hand vector and the rolled window of
//     src/deltanet_ref.rs:289-303, and by agreeing bit for bit with a second,
//     whole-chunk reading of the conv (tests/); the bf16 -> f16 page
//     conversion by numpy's float16 over all 65,536 patterns. exp / log inside
//     them share the libm caveat below.
//   * rmsnorm / dot: pinned by src/math.rs:86-108 (dot tail vector, all-3s row).
//   * RoPE and SiLU: PARITY UNPINNED at the libm boundary. The reference calls
//     the platform libm (powf, sinf, cosf, expf) through Rust std and holds no
//     test that fixes those bits; on Linux that libm is glibc, the same one
//     this file links, so the restated results are what the Rust code would
//     produce on this machine.
//
// Arithmetic rules that make this a faithful restatement (the file must be
// built with -ffp-contract=off and without -ffast-math): every f32 multiply,
// add, subtract, divide and sqrt is separately rounded (Rust never contracts
// to FMA), association follows the reference expression by expression.
//
// Third-party arithmetic restated here: the `half` crate, version 2.7.1
// (Cargo.lock:966-968) -- f16/bf16 <-> f32 conversions, done below as bit
// manipulation with round-to-nearest-even, gradual underflow and overflow to
// infinity, which is that crate's published behaviour.

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define ORACLE_API extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------
// half / bf16 conversions (crate `half` 2.7.1 semantics)
// ---------------------------------------------------------------------------

static inline float bits_to_f32(uint32_t u) {
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

static inline uint32_t f32_to_bits(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}

// f16 bits -> f32, exact (src/gguf/dequant.rs:135-137 uses f16::to_f32).
static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_to_f32(sign);
        // subnormal: value = man * 2^-24, exactly representable in f32
        float v = (float)man * 5.9604644775390625e-08f;  // 2^-24
        return sign ? -v : v;
    }
    if (exp == 31) return bits_to_f32(sign | 0x7F800000u | (man << 13));
    return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

// f32 -> f16 bits, round to nearest even, overflow to infinity, gradual
// underflow (src/gpu/metal.rs:723 uses f16::from_f32).
static inline uint16_t f32_to_f16(float f) {
    uint32_t x = f32_to_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 255) {  // inf / nan (keep a quiet nan payload bit)
        return (uint16_t)(sign | 0x7C00u | (man ? (0x200u | (man >> 13)) : 0u));
    }
    int32_t e = (int32_t)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;  // rounds to zero
        man |= 0x800000u;                    // implicit leading one
        uint32_t shift = (uint32_t)(14 - e); // 14..24
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half_bits = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half_bits & 1u))) half_bits++;  // may carry into exp/inf
    return (uint16_t)(sign | half_bits);
}

// bf16 bits -> f32 is an exact shift (src/weights.rs:57-60).
static inline float bf16_to_f32(uint16_t b) { return bits_to_f32((uint32_t)b << 16); }

// f32 -> bf16 bits, round to nearest even.
static inline uint16_t f32_to_bf16(float f) {
    uint32_t x = f32_to_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u);  // nan stays nan
    uint32_t round_bit = 0x8000u;
    if ((x & round_bit) != 0 && (x & (3u * round_bit - 1u)) != 0) return (uint16_t)((x >> 16) + 1u);
    return (uint16_t)(x >> 16);
}

ORACLE_API float lokal_ref_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
ORACLE_API uint16_t lokal_ref_f32_to_f16(float f) { return f32_to_f16(f); }
ORACLE_API float lokal_ref_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
ORACLE_API uint16_t lokal_ref_f32_to_bf16(float f) { return f32_to_bf16(f); }

ORACLE_API void lokal_ref_f32_to_f16_array(const float* x, size_t n, uint16_t* out) {
    for (size_t i = 0; i < n; i++) out[i] = f32_to_f16(x[i]);
}
ORACLE_API void lokal_ref_f32_to_bf16_array(const float* x, size_t n, uint16_t* out) {
    for (size_t i = 0; i < n; i++) out[i] = f32_to_bf16(x[i]);
}
ORACLE_API void lokal_ref_f16_to_f32_array(const uint16_t* x, size_t n, float* out) {
    for (size_t i = 0; i < n; i++) out[i] = f16_to_f32(x[i]);
}
ORACLE_API void lokal_ref_bf16_to_f32_array(const uint16_t* x, size_t n, float* out) {
    for (size_t i = 0; i < n; i++) out[i] = bf16_to_f32(x[i]);
}

// ---------------------------------------------------------------------------
// math.rs leaf ops
// ---------------------------------------------------------------------------

// src/math.rs:25-38 -- eight independent lane accumulators over chunks of 8,
// lanes summed in index order, then the tail added sequentially.
static float ref_dot(const float* a, const float* b, size_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t chunks = n / 8;
    for (size_t c = 0; c < chunks; c++) {
        for (size_t i = 0; i < 8; i++) {
            float p = a[c * 8 + i] * b[c * 8 + i];
            acc[i] = acc[i] + p;
        }
    }
    float sum = 0.0f;
    for (size_t i = 0; i < 8; i++) sum = sum + acc[i];
    for (size_t i = chunks * 8; i < n; i++) {
        float p = a[i] * b[i];
        sum = sum + p;
    }
    return sum;
}

// src/math.rs:45-49 -- y_i = (x_i * scale) * w_i with scale = 1/sqrt(mean+eps).
static void ref_rmsnorm(const float* x, const float* w, float eps, size_t n, float* y) {
    float mean_sq = ref_dot(x, x, n) / (float)n;
    float scale = 1.0f / std::sqrt(mean_sq + eps);
    for (size_t i = 0; i < n; i++) {
        float t = x[i] * scale;
        y[i] = t * w[i];
    }
}

// src/math.rs:68-70 -- x / (1 + exp(-x)).
static inline float ref_silu(float x) { return x / (1.0f + std::exp(-x)); }

// src/model.rs:268-279, with the rotated prefix `rot_dim` of the GPU twin
// (src/gpu/kernels.metal:2401-2425). rot_dim == head_dim is the CPU function
// itself: pairs (i, i + rot/2), freq = theta^(-(2 i)/rot), angle = pos * freq.
// powf and sincos are recomputed for every head, as the reference does.
static void ref_rope(float* x, size_t n, size_t pos, size_t head_dim, size_t rot_dim, float theta) {
    size_t half = rot_dim / 2;
    for (size_t h0 = 0; h0 + head_dim <= n; h0 += head_dim) {
        float* head = x + h0;
        for (size_t i = 0; i < half; i++) {
            float freq = std::pow(theta, -(2.0f * (float)i) / (float)rot_dim);
            float angle = (float)pos * freq;
            float s = std::sin(angle), c = std::cos(angle);
            float a = head[i], b = head[i + half];
            float ac = a * c, bs = b * s, as = a * s, bc = b * c;
            head[i] = ac - bs;
            head[i + half] = as + bc;
        }
    }
}

ORACLE_API float lokal_ref_dot(const float* a, const float* b, size_t n) { return ref_dot(a, b, n); }
ORACLE_API void lokal_ref_rmsnorm(const float* x, const float* w, float eps, size_t n, float* y) {
    ref_rmsnorm(x, w, eps, n, y);
}
ORACLE_API float lokal_ref_silu(float x) { return ref_silu(x); }
ORACLE_API void lokal_ref_rope(float* x, size_t n, size_t pos, size_t head_dim, float theta) {
    ref_rope(x, n, pos, head_dim, head_dim, theta);
}
ORACLE_API void lokal_ref_rope_partial(float* x, size_t n, size_t pos, size_t head_dim, size_t rot_dim,
                                       float theta) {
    ref_rope(x, n, pos, head_dim, rot_dim, theta);
}

// inv-freq vector theta^(-(2 i)/rot) exactly as ref_rope evaluates it.
ORACLE_API void lokal_ref_inv_freq(float theta, size_t rot_dim, float* out) {
    for (size_t i = 0; i < rot_dim / 2; i++) out[i] = std::pow(theta, -(2.0f * (float)i) / (float)rot_dim);
}

// (cos, sin) rows for given positions: out[row][0..half) = cos, [half..rot) = sin.
ORACLE_API void lokal_ref_rope_table(float theta, size_t rot_dim, const int32_t* positions, int64_t pos0,
                                     size_t rows, float* out) {
    size_t half = rot_dim / 2;
    for (size_t r = 0; r < rows; r++) {
        size_t pos = positions ? (size_t)positions[r] : (size_t)(pos0 + (int64_t)r);
        for (size_t i = 0; i < half; i++) {
            float freq = std::pow(theta, -(2.0f * (float)i) / (float)rot_dim);
            float angle = (float)pos * freq;
            out[r * rot_dim + i] = std::cos(angle);
            out[r * rot_dim + half + i] = std::sin(angle);
        }
    }
}

// Self-check hook: do sincosf and the sinf/cosf pair agree bit for bit on x?
ORACLE_API int lokal_ref_sincos_spellings_agree(float x) {
    float s, c;
    sincosf(x, &s, &c);
    float s2 = std::sin(x), c2 = std::cos(x);
    return f32_to_bits(s) == f32_to_bits(s2) && f32_to_bits(c) == f32_to_bits(c2);
}

// ---------------------------------------------------------------------------
// Row-batched composites (definition = the reference's steps in model.rs order)
// ---------------------------------------------------------------------------

template <typename F>
static void parallel_rows(size_t rows, int threads, F fn) {
    if (threads <= 1 || rows < 2) {
        fn((size_t)0, rows);
        return;
    }
    size_t nt = (size_t)threads < rows ? (size_t)threads : rows;
    std::vector<std::thread> pool;
    size_t per = (rows + nt - 1) / nt;
    for (size_t t = 0; t < nt; t++) {
        size_t r0 = t * per, r1 = r0 + per < rows ? r0 + per : rows;
        if (r0 >= r1) break;
        pool.emplace_back([=] { fn(r0, r1); });
    }
    for (auto& th : pool) th.join();
}

// x' = x + delta (src/model.rs:235-237, 253-255); xn = rmsnorm(x', w, eps)
// (src/math.rs:45-49). delta may be null (plain rmsnorm, x untouched).
ORACLE_API void lokal_ref_add_rmsnorm_rows(float* x, const float* delta, const float* w, float* xn, size_t rows,
                                           size_t dim, float eps, int threads) {
    parallel_rows(rows, threads, [=](size_t r0, size_t r1) {
        for (size_t r = r0; r < r1; r++) {
            float* xr = x + r * dim;
            if (delta) {
                const float* dr = delta + r * dim;
                for (size_t i = 0; i < dim; i++) xr[i] = xr[i] + dr[i];
            }
            ref_rmsnorm(xr, w, eps, dim, xn + r * dim);
        }
    });
}

// One q or k row: bias add (src/model.rs:29-33), per-head rmsnorm with a
// weight of head_dim entries shared by all heads (src/model.rs:213-221), then
// rope (src/model.rs:225-226). bias / norm_w may be null.
static void ref_qk_row(float* v, size_t n_heads, size_t head_dim, size_t rot_dim, const float* bias,
                       const float* norm_w, float eps, size_t pos, float theta, std::vector<float>& tmp) {
    size_t n = n_heads * head_dim;
    if (bias) {
        for (size_t i = 0; i < n; i++) v[i] = v[i] + bias[i];
    }
    if (norm_w) {
        tmp.resize(head_dim);
        for (size_t h = 0; h < n_heads; h++) {
            ref_rmsnorm(v + h * head_dim, norm_w, eps, head_dim, tmp.data());
            std::memcpy(v + h * head_dim, tmp.data(), head_dim * sizeof(float));
        }
    }
    ref_rope(v, n, pos, head_dim, rot_dim, theta);
}

ORACLE_API void lokal_ref_qk_rope_rows(float* q, float* k, const float* q_bias, const float* k_bias,
                                       const float* q_norm_w, const float* k_norm_w, const int32_t* positions,
                                       int64_t pos0, size_t rows, size_t n_q_heads, size_t n_kv_heads,
                                       size_t head_dim, size_t rot_dim, float eps, float theta, int threads) {
    parallel_rows(rows, threads, [=](size_t r0, size_t r1) {
        std::vector<float> tmp;
        for (size_t r = r0; r < r1; r++) {
            size_t pos = positions ? (size_t)positions[r] : (size_t)(pos0 + (int64_t)r);
            if (q) ref_qk_row(q + r * n_q_heads * head_dim, n_q_heads, head_dim, rot_dim, q_bias, q_norm_w, eps, pos,
                              theta, tmp);
            if (k) ref_qk_row(k + r * n_kv_heads * head_dim, n_kv_heads, head_dim, rot_dim, k_bias, k_norm_w, eps,
                              pos, theta, tmp);
        }
    });
}

// inner_i = silu(gate_i) * up_i (src/model.rs:245-248).
ORACLE_API void lokal_ref_swiglu(const float* gate, const float* up, size_t n, float* out, int threads) {
    parallel_rows(n, threads, [=](size_t i0, size_t i1) {
        for (size_t i = i0; i < i1; i++) out[i] = ref_silu(gate[i]) * up[i];
    });
}

// ---------------------------------------------------------------------------
// Per-row siblings of the path in the gated-deltanet (qwen35) blocks
// (src/deltanet_ref.rs). They accumulate in f64 where the ops above use f32.
// ---------------------------------------------------------------------------

// src/deltanet_ref.rs:51-57
static inline float ref_sigmoid(float x) { return 1.0f / (1.0f + std::exp(-x)); }
static inline float ref_silu_deltanet(float x) { return x * ref_sigmoid(x); }
ORACLE_API float lokal_ref_sigmoid(float x) { return ref_sigmoid(x); }

// l2_norm (src/deltanet_ref.rs:61-67): x / max(sqrt(sum x^2), eps), sum in f64, in order; the root is taken in f64
// and narrowed to f32 before the clamp. Rows are addressed as the batched kernel addresses them
// (src/gpu/kernels.metal:3708-3720): row r of token t starts at t*tok_stride + r*dim.
ORACLE_API void lokal_ref_l2norm_rows(float* x, size_t rows_per_token, size_t n_tokens, size_t tok_stride, size_t dim, float eps) {
    for (size_t t = 0; t < n_tokens; t++)
        for (size_t r = 0; r < rows_per_token; r++) {
            float* v = x + t * tok_stride + r * dim;
            double sum = 0.0;
            for (size_t i = 0; i < dim; i++) sum += (double)v[i] * (double)v[i];
            const float scale = 1.0f / std::max((float)std::sqrt(sum), eps);
            for (size_t i = 0; i < dim; i++) v[i] *= scale;
        }
}

// rmsnorm with ggml's accumulation (src/deltanet_ref.rs:71-78): mean of squares in f64 narrowed to f32, then
// (x * scale) * w with scale = 1 / sqrt(mean + eps).
static void ref_rmsnorm_f64(float* x, const float* w, size_t n, float eps) {
    double sum = 0.0;
    for (size_t i = 0; i < n; i++) sum += (double)x[i] * (double)x[i];
    const float mean = (float)(sum / (double)n);
    const float scale = 1.0f / std::sqrt(mean + eps);
    for (size_t i = 0; i < n; i++) x[i] = x[i] * scale * w[i];
}

// gated_output_norm (src/deltanet_ref.rs:187-198): per head, rmsnorm(o; w) then o *= silu(z); w is shared by heads.
ORACLE_API void lokal_ref_gated_output_norm(float* o, const float* w, const float* z, size_t heads, size_t dim, float eps) {
    for (size_t h = 0; h < heads; h++) {
        float* oh = o + h * dim;
        ref_rmsnorm_f64(oh, w, dim, eps);
        for (size_t i = 0; i < dim; i++) oh[i] *= ref_silu_deltanet(z[h * dim + i]);
    }
}

// attn_out_gate (src/deltanet_ref.rs:203-207): attn *= sigmoid(gate), elementwise.
ORACLE_API void lokal_ref_attn_out_gate(float* attn, const float* gate, size_t n) {
    for (size_t i = 0; i < n; i++) attn[i] *= ref_sigmoid(gate[i]);
}

// split_q_gate (src/gpu/kernels.metal:4106-4124): a row of the joint projection is [q(hd) | gate(hd)] per head;
// q and gate come out compact, [rows][heads][hd] each.
ORACLE_API void lokal_ref_split_q_gate(const float* src, float* q, float* gate, size_t rows, size_t heads, size_t hd) {
    for (size_t r = 0; r < rows; r++)
        for (size_t h = 0; h < heads; h++) {
            const float* s = src + (r * heads + h) * 2 * hd;
            std::memcpy(q + (r * heads + h) * hd, s, hd * sizeof(float));
            std::memcpy(gate + (r * heads + h) * hd, s + hd, hd * sizeof(float));
        }
}

// softplus with ggml's shortcut (src/deltanet_ref.rs:48-50): x > 20 returns x unchanged.
static inline float ref_softplus(float x) { return x > 20.0f ? x : std::log(1.0f + std::exp(x)); }
ORACLE_API float lokal_ref_softplus(float x) { return ref_softplus(x); }

// delta_gates (src/deltanet_ref.rs:82-84 per scalar; the batched addressing of src/gpu/kernels.metal:3995-4015):
//   g[t][h] = a[h] * softplus(alpha[t][h] + dt_bias[h]);   beta[t][h] = sigmoid(beta_in[t][h])
ORACLE_API void lokal_ref_delta_gates(const float* alpha, const float* beta_in, const float* a, const float* dt_bias, float* g,
                                      float* beta, size_t n_v_heads, size_t n_tokens) {
    for (size_t t = 0; t < n_tokens; t++)
        for (size_t h = 0; h < n_v_heads; h++) {
            const size_t i = t * n_v_heads + h;
            g[i] = a[h] * ref_softplus(alpha[i] + dt_bias[h]);
            beta[i] = ref_sigmoid(beta_in[i]);
        }
}

// conv_step (src/deltanet_ref.rs:91-112) applied to n tokens in turn: depthwise causal conv over the rolling window
// [state.., x] with separate multiply and add per tap, SiLU inside as x * sigmoid(x), the window rolled after the dot.
// state: [channels][d_conv-1] oldest first (updated); x, out: [n][channels]; kernel: [channels][d_conv].
ORACLE_API void lokal_ref_ssm_conv(float* state, const float* x, const float* kernel, float* out, size_t channels, size_t d_conv,
                                   size_t n_tokens) {
    const size_t k = d_conv;
    for (size_t t = 0; t < n_tokens; t++)
        for (size_t c = 0; c < channels; c++) {
            float* st = state + c * (k - 1);
            float acc = 0.0f;
            for (size_t j = 0; j + 1 < k; j++) acc += st[j] * kernel[c * k + j];
            const float xv = x[t * channels + c];
            acc += xv * kernel[c * k + (k - 1)];
            out[t * channels + c] = ref_silu_deltanet(acc);
            if (k >= 2) {
                for (size_t j = 0; j + 2 < k; j++) st[j] = st[j + 1];
                st[k - 2] = xv;
            }
        }
}

// bf16_to_f16_copy (src/gpu/kernels.metal:3572-3588): bf16 bits widened exactly, narrowed to f16 nearest-even; the flag
// is raised when a finite value leaves the f16 range.
ORACLE_API void lokal_ref_bf16_to_f16(const uint16_t* src, size_t n, uint16_t* dst, uint32_t* clip) {
    for (size_t i = 0; i < n; i++) {
        const float v = bf16_to_f32(src[i]);
        const uint16_t h = f32_to_f16(v);
        if ((h & 0x7fffu) == 0x7c00u && !std::isinf(v)) *clip = 1u;
        dst[i] = h;
    }
}

// ---------------------------------------------------------------------------
// GGUF block formats (src/gguf/dequant.rs:21-41, 81-119)
// ---------------------------------------------------------------------------

enum : uint32_t {
    GGML_F32 = 0, GGML_F16 = 1, GGML_Q4_0 = 2, GGML_Q5_0 = 6, GGML_Q8_0 = 8, GGML_Q2_K = 10, GGML_Q3_K = 11,
    GGML_Q4_K = 12, GGML_Q5_K = 13, GGML_Q6_K = 14, GGML_IQ2_XXS = 16, GGML_IQ2_XS = 17, GGML_IQ3_XXS = 18,
    GGML_IQ1_S = 19, GGML_IQ4_NL = 20, GGML_IQ3_S = 21, GGML_IQ2_S = 22, GGML_IQ4_XS = 23, GGML_IQ1_M = 29, GGML_BF16 = 30
};

ORACLE_API size_t lokal_ref_blk_elems(uint32_t ty) {
    switch (ty) {
        case GGML_F32: case GGML_F16: case GGML_BF16: return 1;
        case GGML_Q4_0: case GGML_Q5_0: case GGML_Q8_0: case GGML_IQ4_NL: return 32;
        case GGML_Q2_K: case GGML_Q3_K: case GGML_Q4_K: case GGML_Q5_K: case GGML_Q6_K: case GGML_IQ4_XS:
        case GGML_IQ2_XXS: case GGML_IQ2_XS: case GGML_IQ2_S: case GGML_IQ3_XXS: case GGML_IQ3_S: case GGML_IQ1_S: case GGML_IQ1_M:
            return 256;
        default: return 0;
    }
}

// The i-quant codebooks (src/lowmem/iq_grids.rs: fitted tables, not formulas). They are handed in by the caller,
// never written out here: 0 iq2xxs u64[256], 1 iq2xs u64[512], 2 iq2s u64[1024], 3 iq3xxs u32[256], 4 iq3s u32[512],
// 5 iq1s u64[2048]. A row of a codebook type decodes only after its table has been set.
static std::vector<uint64_t> g_grid64[6];
static const size_t kGridLen[6] = {256, 512, 1024, 256, 512, 2048};
ORACLE_API int lokal_ref_set_iq_grid(int which, const void* table, size_t entries) {
    if (which < 0 || which > 5 || !table || entries != kGridLen[which]) return -1;
    g_grid64[which].resize(entries);
    const bool wide = which != 3 && which != 4;
    for (size_t i = 0; i < entries; i++)
        g_grid64[which][i] = wide ? static_cast<const uint64_t*>(table)[i] : static_cast<const uint32_t*>(table)[i];
    return 0;
}
static inline const uint64_t* iq_grid(int which) { return g_grid64[which].empty() ? nullptr : g_grid64[which].data(); }
// ksigns_iq2xs[i]: i with bit 7 set so that the byte has even parity (src/lowmem/iq_grids.rs:12-22 holds the
// same 128 values as data; this is the rule they follow).
static inline uint8_t ksigns_iq2xs(unsigned i) { return (uint8_t)(i | ((__builtin_popcount(i) & 1u) << 7)); }

// sizeof(block_*) of ggml, as src/gguf/dequant.rs:94-114 lists them.
ORACLE_API size_t lokal_ref_blk_bytes(uint32_t ty) {
    switch (ty) {
        case GGML_F32: return 4;
        case GGML_F16: case GGML_BF16: return 2;
        case GGML_Q4_0: return 2 + 16;
        case GGML_Q5_0: return 2 + 4 + 16;
        case GGML_Q8_0: return 2 + 32;
        case GGML_IQ4_NL: return 2 + 16;
        case GGML_IQ4_XS: return 2 + 2 + 4 + 128;
        case GGML_Q2_K: return 16 + 64 + 2 + 2;
        case GGML_Q3_K: return 32 + 64 + 12 + 2;
        case GGML_Q4_K: return 2 + 2 + 12 + 128;
        case GGML_Q5_K: return 2 + 2 + 12 + 32 + 128;
        case GGML_Q6_K: return 128 + 64 + 16 + 2;
        case GGML_IQ1_S: return 2 + 32 + 16;
        case GGML_IQ1_M: return 32 + 16 + 8;
        case GGML_IQ2_XXS: return 2 + 64;
        case GGML_IQ2_XS: return 2 + 64 + 8;
        case GGML_IQ2_S: return 2 + 64 + 8 + 8;
        case GGML_IQ3_XXS: return 2 + 64 + 32;
        case GGML_IQ3_S: return 2 + 64 + 8 + 32 + 4;
        default: return 0;
    }
}

// The 16-entry codebook of the IQ4 types (kvalues_iq4nl of ggml; src/gguf/dequant.rs:165-166). Format data.
static const int8_t kIq4nlValues[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// n / blk_elems * blk_bytes with integer division (src/gguf/dequant.rs:117-119).
ORACLE_API size_t lokal_ref_row_bytes(uint32_t ty, size_t n) {
    size_t be = lokal_ref_blk_elems(ty);
    return be ? n / be * lokal_ref_blk_bytes(ty) : 0;
}

static inline float f16_bits_at(const uint8_t* src, size_t off) {
    return f16_to_f32((uint16_t)(src[off] | (src[off + 1] << 8)));
}

// src/gguf/dequant.rs:141-150.
static inline void scale_min_k4(size_t j, const uint8_t* q, uint8_t* sc, uint8_t* mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

// Sequential row decode (src/gguf/dequant.rs:191-239, 462-483). Returns 0, or
// -1 where the reference would panic on a src/out size mismatch (:192), or -2
// for a type outside this path.
ORACLE_API int lokal_ref_dequant_row(uint32_t ty, const uint8_t* src, size_t src_len, float* out, size_t n) {
    if (lokal_ref_blk_elems(ty) == 0) return -2;
    if (src_len != lokal_ref_row_bytes(ty, n)) return -1;
    switch (ty) {
        case GGML_F32:
            for (size_t i = 0; i < n; i++) {
                uint32_t u = (uint32_t)src[4 * i] | ((uint32_t)src[4 * i + 1] << 8) | ((uint32_t)src[4 * i + 2] << 16) |
                             ((uint32_t)src[4 * i + 3] << 24);
                out[i] = bits_to_f32(u);
            }
            return 0;
        case GGML_F16:
            for (size_t i = 0; i < n; i++) out[i] = f16_bits_at(src, 2 * i);
            return 0;
        case GGML_BF16:
            for (size_t i = 0; i < n; i++) out[i] = bf16_to_f32((uint16_t)(src[2 * i] | (src[2 * i + 1] << 8)));
            return 0;
        case GGML_Q8_0:
            for (size_t b = 0; b < n / 32; b++) {
                const uint8_t* blk = src + b * 34;
                float d = f16_bits_at(blk, 0);
                float* y = out + b * 32;
                for (size_t j = 0; j < 32; j++) y[j] = (float)(int8_t)blk[2 + j] * d;
            }
            return 0;
        case GGML_Q4_K:
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 144;
                float d = f16_bits_at(blk, 0);
                float dmin = f16_bits_at(blk, 2);
                const uint8_t* scales = blk + 4;
                const uint8_t* qs = blk + 16;
                float* y = out + b * 256;
                size_t is = 0;
                for (size_t j = 0; j < 256; j += 64) {
                    const uint8_t* q = qs + j / 2;
                    uint8_t sc, m;
                    scale_min_k4(is, scales, &sc, &m);
                    float d1 = d * (float)sc, m1 = dmin * (float)m;
                    scale_min_k4(is + 1, scales, &sc, &m);
                    float d2 = d * (float)sc, m2 = dmin * (float)m;
                    for (size_t l = 0; l < 32; l++) {
                        float lo = d1 * (float)(q[l] & 0x0F);
                        float hi = d2 * (float)(q[l] >> 4);
                        y[j + l] = lo - m1;
                        y[j + 32 + l] = hi - m2;
                    }
                    is += 2;
                }
            }
            return 0;
        case GGML_Q4_0:  // src/gguf/dequant.rs:204-214: f16 d, 16 bytes of nibbles; (nibble - 8) * d
            for (size_t b = 0; b < n / 32; b++) {
                const uint8_t* blk = src + b * 18;
                float d = f16_bits_at(blk, 0);
                float* y = out + b * 32;
                for (size_t j = 0; j < 16; j++) {
                    uint8_t q = blk[2 + j];
                    y[j] = (float)((int)(q & 0x0F) - 8) * d;
                    y[j + 16] = (float)((int)(q >> 4) - 8) * d;
                }
            }
            return 0;
        case GGML_Q5_0:  // src/gguf/dequant.rs:215-230: Q4_0 plus a fifth bit per element in a u32; (value - 16) * d
            for (size_t b = 0; b < n / 32; b++) {
                const uint8_t* blk = src + b * 22;
                float d = f16_bits_at(blk, 0);
                uint32_t qh = (uint32_t)blk[2] | ((uint32_t)blk[3] << 8) | ((uint32_t)blk[4] << 16) | ((uint32_t)blk[5] << 24);
                float* y = out + b * 32;
                for (size_t j = 0; j < 16; j++) {
                    uint8_t hi0 = (uint8_t)(((qh >> j) << 4) & 0x10);
                    uint8_t hi1 = (uint8_t)((qh >> (j + 12)) & 0x10);
                    uint8_t q = blk[6 + j];
                    y[j] = (float)((int)((q & 0x0F) | hi0) - 16) * d;
                    y[j + 16] = (float)((int)((q >> 4) | hi1) - 16) * d;
                }
            }
            return 0;
        // ---- codebook types: 256-element super-blocks of eight 32-element groups; a group is four runs of eight
        // values, each run one codebook entry (IQ1 / IQ2: eight bytes of a u64) or two (IQ3: four bytes of a u32).
        case GGML_IQ1_S: {  // src/gguf/dequant.rs:255-270: d | qs[32] | qh[8 x u16]; value = dl * (grid + delta)
            const uint64_t* grid = iq_grid(5);
            if (!grid) return -3;
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 50;
                const float d = f16_bits_at(blk, 0);
                float* y = out + b * 256;
                for (size_t ib = 0; ib < 8; ib++) {
                    const unsigned qh = (unsigned)blk[34 + 2 * ib] | ((unsigned)blk[35 + 2 * ib] << 8);
                    const float dl = d * (float)(2 * ((qh >> 12) & 7) + 1);
                    const float delta = (qh & 0x8000) ? -0.125f : 0.125f;
                    for (size_t l = 0; l < 4; l++) {
                        const uint64_t g8 = grid[blk[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7) << 8)];
                        for (size_t j = 0; j < 8; j++) y[32 * ib + 8 * l + j] = dl * ((float)(int8_t)(g8 >> (8 * j)) + delta);
                    }
                }
            }
            return 0;
        }
        case GGML_IQ1_M: {  // src/gguf/dequant.rs:274-293: qs[32] | qh[16] | scales[4 x u16]; the f16 d is spread over the scales' top nibbles
            const uint64_t* grid = iq_grid(5);
            if (!grid) return -3;
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 56;
                unsigned sc[4];
                for (size_t k = 0; k < 4; k++) sc[k] = (unsigned)blk[48 + 2 * k] | ((unsigned)blk[49 + 2 * k] << 8);
                const float d = f16_to_f32((uint16_t)((sc[0] >> 12) | ((sc[1] >> 8) & 0x00f0) | ((sc[2] >> 4) & 0x0f00) | (sc[3] & 0xf000)));
                float* y = out + b * 256;
                for (size_t ib = 0; ib < 8; ib++) {
                    for (size_t l = 0; l < 4; l++) {
                        const unsigned shift = 6 * (ib % 2) + (l < 2 ? 0 : 3);
                        const float dl = d * (float)(2 * ((sc[ib / 2] >> shift) & 7) + 1);
                        const unsigned qh = blk[32 + 2 * ib + (l >> 1)];
                        const bool even = (l % 2) == 0;
                        const uint64_t g8 = grid[blk[4 * ib + l] | ((qh << (even ? 8 : 4)) & 0x700)];
                        const float delta = (qh & (even ? 0x08u : 0x80u)) ? -0.125f : 0.125f;
                        for (size_t j = 0; j < 8; j++) y[32 * ib + 8 * l + j] = dl * ((float)(int8_t)(g8 >> (8 * j)) + delta);
                    }
                }
            }
            return 0;
        }
        case GGML_IQ2_XXS: {  // src/gguf/dequant.rs:295-312: d | 8 x (4 grid bytes, u32 of 4 x 7 sign bits + 4-bit scale)
            const uint64_t* grid = iq_grid(0);
            if (!grid) return -3;
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 66;
                const float d = f16_bits_at(blk, 0);
                float* y = out + b * 256;
                for (size_t ib = 0; ib < 8; ib++) {
                    const uint8_t* q = blk + 2 + 8 * ib;
                    const uint32_t a1 = (uint32_t)q[4] | ((uint32_t)q[5] << 8) | ((uint32_t)q[6] << 16) | ((uint32_t)q[7] << 24);
                    const float db = d * (0.5f + (float)(a1 >> 28)) * 0.25f;
                    for (size_t l = 0; l < 4; l++) {
                        const uint8_t signs = ksigns_iq2xs((a1 >> (7 * l)) & 127);
                        const uint64_t g8 = grid[q[l]];
                        for (size_t j = 0; j < 8; j++)
                            y[32 * ib + 8 * l + j] = db * (float)((g8 >> (8 * j)) & 0xFF) * ((signs >> j) & 1 ? -1.0f : 1.0f);
                    }
                }
            }
            return 0;
        }
        case GGML_IQ2_XS: {  // src/gguf/dequant.rs:314-334: d | qs[32 x u16: 9-bit grid index, 7-bit sign selector] | scales[8]
            const uint64_t* grid = iq_grid(1);
            if (!grid) return -3;
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 74;
                const float d = f16_bits_at(blk, 0);
                float* y = out + b * 256;
                for (size_t ib = 0; ib < 8; ib++) {
                    const uint8_t sc = blk[66 + ib];
                    for (size_t l = 0; l < 4; l++) {
                        const float db = d * (0.5f + (float)(l < 2 ? (sc & 0xF) : (sc >> 4))) * 0.25f;
                        const unsigned qv = (unsigned)blk[2 + 2 * (4 * ib + l)] | ((unsigned)blk[3 + 2 * (4 * ib + l)] << 8);
                        const uint8_t signs = ksigns_iq2xs(qv >> 9);
                        const uint64_t g8 = grid[qv & 511];
                        for (size_t j = 0; j < 8; j++)
                            y[32 * ib + 8 * l + j] = db * (float)((g8 >> (8 * j)) & 0xFF) * ((signs >> j) & 1 ? -1.0f : 1.0f);
                    }
                }
            }
            return 0;
        }
        case GGML_IQ2_S: {  // src/gguf/dequant.rs:336-352: d | qs[32 grid bytes + 32 sign bytes] | qh[8] | scales[8]
            const uint64_t* grid = iq_grid(2);
            if (!grid) return -3;
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 82;
                const float d = f16_bits_at(blk, 0);
                float* y = out + b * 256;
                for (size_t ib = 0; ib < 8; ib++) {
                    const uint8_t sc = blk[74 + ib];
                    const unsigned qh = blk[66 + ib];
                    for (size_t l = 0; l < 4; l++) {
                        const float db = d * (0.5f + (float)(l < 2 ? (sc & 0xF) : (sc >> 4))) * 0.25f;
                        const uint64_t g8 = grid[blk[2 + 4 * ib + l] | ((qh << (8 - 2 * l)) & 0x300)];
                        const uint8_t signs = blk[2 + 32 + 4 * ib + l];
                        for (size_t j = 0; j < 8; j++)
                            y[32 * ib + 8 * l + j] = db * (float)((g8 >> (8 * j)) & 0xFF) * ((signs >> j) & 1 ? -1.0f : 1.0f);
                    }
                }
            }
            return 0;
        }
        case GGML_IQ3_XXS: {  // src/gguf/dequant.rs:354-374: d | qs[64 grid bytes] | 8 x u32 (4 x 7 sign bits + 4-bit scale)
            const uint64_t* grid = iq_grid(3);
            if (!grid) return -3;
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 98;
                const float d = f16_bits_at(blk, 0);
                float* y = out + b * 256;
                for (size_t ib = 0; ib < 8; ib++) {
                    const uint8_t* s = blk + 66 + 4 * ib;
                    const uint32_t aux = (uint32_t)s[0] | ((uint32_t)s[1] << 8) | ((uint32_t)s[2] << 16) | ((uint32_t)s[3] << 24);
                    const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
                    for (size_t l = 0; l < 4; l++) {
                        const uint8_t signs = ksigns_iq2xs((aux >> (7 * l)) & 127);
                        for (size_t hf = 0; hf < 2; hf++) {
                            const uint64_t g4 = grid[blk[2 + 8 * ib + 2 * l + hf]];
                            for (size_t j = 0; j < 4; j++)
                                y[32 * ib + 8 * l + 4 * hf + j] = db * (float)((g4 >> (8 * j)) & 0xFF) * ((signs >> (4 * hf + j)) & 1 ? -1.0f : 1.0f);
                        }
                    }
                }
            }
            return 0;
        }
        case GGML_IQ3_S: {  // src/gguf/dequant.rs:376-394: d | qs[64] | qh[8] | signs[32] | scales[4]; qh gives a ninth index bit
            const uint64_t* grid = iq_grid(4);
            if (!grid) return -3;
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 110;
                const float d = f16_bits_at(blk, 0);
                float* y = out + b * 256;
                for (size_t g = 0; g < 8; g++) {
                    const uint8_t scb = blk[106 + g / 2];
                    const float db = d * (float)(1 + 2 * (unsigned)(g % 2 == 0 ? (scb & 0xF) : (scb >> 4)));
                    const unsigned qh = blk[66 + g];
                    for (size_t l = 0; l < 4; l++) {
                        const uint8_t signs = blk[74 + 4 * g + l];
                        for (size_t hf = 0; hf < 2; hf++) {
                            const uint64_t g4 = grid[blk[2 + 8 * g + 2 * l + hf] | ((qh << (8 - 2 * l - hf)) & 256)];
                            for (size_t j = 0; j < 4; j++)
                                y[32 * g + 8 * l + 4 * hf + j] = db * (float)((g4 >> (8 * j)) & 0xFF) * ((signs >> (4 * hf + j)) & 1 ? -1.0f : 1.0f);
                        }
                    }
                }
            }
            return 0;
        }
        case GGML_IQ4_NL:  // src/gguf/dequant.rs:396-409: f16 d, nibbles index the 16-entry codebook
            for (size_t b = 0; b < n / 32; b++) {
                const uint8_t* blk = src + b * 18;
                float d = f16_bits_at(blk, 0);
                float* y = out + b * 32;
                for (size_t j = 0; j < 16; j++) {
                    uint8_t q = blk[2 + j];
                    y[j] = d * (float)kIq4nlValues[q & 0x0F];
                    y[j + 16] = d * (float)kIq4nlValues[q >> 4];
                }
            }
            return 0;
        case GGML_IQ4_XS:  // src/gguf/dequant.rs:410-425: d | scales_h u16 | scales_l[4] | qs[128]; 6-bit scales biased by -32
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 136;
                float d = f16_bits_at(blk, 0);
                unsigned scales_h = (unsigned)blk[2] | ((unsigned)blk[3] << 8);
                float* y = out + b * 256;
                for (size_t ib = 0; ib < 8; ib++) {  // eight sub-blocks of 32
                    int ls = (int)((blk[4 + ib / 2] >> (4 * (ib % 2))) & 0xF) | (int)(((scales_h >> (2 * ib)) & 3) << 4);
                    float dl = d * (float)(ls - 32);
                    const uint8_t* q = blk + 8 + ib * 16;
                    for (size_t j = 0; j < 16; j++) {
                        y[ib * 32 + j] = dl * (float)kIq4nlValues[q[j] & 0x0F];
                        y[ib * 32 + 16 + j] = dl * (float)kIq4nlValues[q[j] >> 4];
                    }
                }
            }
            return 0;
        case GGML_Q2_K:  // src/gguf/dequant.rs:426-440: scales[16] | qs[64] | d | dmin; (d*sc)*q - dmin*min
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 84;
                float d = f16_bits_at(blk, 80), dmin = f16_bits_at(blk, 82);
                float* y = out + b * 256;
                for (size_t nh = 0; nh < 2; nh++) {          // halves of 128 elements share a 32-byte run of quants
                    for (size_t j = 0; j < 4; j++) {         // 2-bit field j of each quant byte
                        for (size_t half = 0; half < 2; half++) {
                            uint8_t sc = blk[nh * 8 + j * 2 + half];
                            float dl = d * (float)(sc & 0xF), ml = dmin * (float)(sc >> 4);
                            const uint8_t* q = blk + 16 + nh * 32 + half * 16;
                            for (size_t l = 0; l < 16; l++) {
                                float t = dl * (float)((q[l] >> (2 * j)) & 3);
                                y[nh * 128 + j * 32 + half * 16 + l] = t - ml;
                            }
                        }
                    }
                }
            }
            return 0;
        case GGML_Q3_K:  // src/gguf/dequant.rs:441-461 (scale shuffle :171-189): hmask[32] | qs[64] | scales[12] | d; a CLEAR hmask bit subtracts 4
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 110;
                float d_all = f16_bits_at(blk, 108);
                const uint8_t* p = blk + 96;
                int scales[16];
                for (size_t s = 0; s < 16; s++) {
                    // six-bit scale s: low nibble from bytes 0..7 (low nibbles first, then high nibbles), top two bits
                    // from the 2-bit fields of bytes 8..11 -- ggml's aux shuffle written out per scale
                    size_t byte = s % 4, grp = s / 4;
                    unsigned lo = grp < 2 ? (unsigned)(p[(grp & 1) * 4 + byte] & 0xF) : (unsigned)(p[(grp & 1) * 4 + byte] >> 4);
                    unsigned hi = ((unsigned)p[8 + byte] >> (2 * grp)) & 3u;
                    scales[s] = (int)(lo | (hi << 4)) - 32;
                }
                float* y = out + b * 256;
                for (size_t nh = 0; nh < 2; nh++) {
                    for (size_t j = 0; j < 4; j++) {
                        uint8_t mbit = (uint8_t)(1u << (nh * 4 + j));
                        for (size_t half = 0; half < 2; half++) {
                            float dl = d_all * (float)scales[nh * 8 + j * 2 + half];
                            const uint8_t* q = blk + 32 + nh * 32 + half * 16;
                            const uint8_t* hm = blk + half * 16;
                            for (size_t l = 0; l < 16; l++) {
                                int v = (int)((q[l] >> (2 * j)) & 3) - ((hm[l] & mbit) ? 0 : 4);
                                y[nh * 128 + j * 32 + half * 16 + l] = dl * (float)v;
                            }
                        }
                    }
                }
            }
            return 0;
        case GGML_Q5_K:  // src/gguf/dequant.rs:484-510: Q4_K plus one high bit per element in qh[32]
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 176;
                float d = f16_bits_at(blk, 0), dmin = f16_bits_at(blk, 2);
                const uint8_t* scales = blk + 4;
                const uint8_t* qh = blk + 16;
                const uint8_t* qs = blk + 48;
                float* y = out + b * 256;
                for (size_t g = 0; g < 4; g++) {  // groups of 64 elements
                    const uint8_t* ql = qs + g * 32;
                    uint8_t sc, m;
                    scale_min_k4(2 * g, scales, &sc, &m);
                    float d1 = d * (float)sc, m1 = dmin * (float)m;
                    scale_min_k4(2 * g + 1, scales, &sc, &m);
                    float d2 = d * (float)sc, m2 = dmin * (float)m;
                    uint8_t u1 = (uint8_t)(1u << (2 * g)), u2 = (uint8_t)(2u << (2 * g));
                    for (size_t l = 0; l < 32; l++) {
                        int lo = (int)(ql[l] & 0x0F) + ((qh[l] & u1) ? 16 : 0);
                        int hi = (int)(ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0);
                        float a = d1 * (float)lo, c = d2 * (float)hi;
                        y[g * 64 + l] = a - m1;
                        y[g * 64 + 32 + l] = c - m2;
                    }
                }
            }
            return 0;
        case GGML_Q6_K:  // src/gguf/dequant.rs:511-533: ql[128] | qh[64] | int8 scales[16] | d; (d*sc)*(q - 32)
            for (size_t b = 0; b < n / 256; b++) {
                const uint8_t* blk = src + b * 210;
                float d = f16_bits_at(blk, 208);
                float* y = out + b * 256;
                for (size_t h = 0; h < 2; h++) {  // halves of 128 elements
                    const uint8_t* ql = blk + h * 64;
                    const uint8_t* qh = blk + 128 + h * 32;
                    const int8_t* sc = (const int8_t*)(blk + 192 + h * 8);
                    for (size_t l = 0; l < 32; l++) {
                        size_t is = l / 16;
                        int q1 = (int)(int8_t)((ql[l] & 0x0F) | (((qh[l] >> 0) & 3) << 4)) - 32;
                        int q2 = (int)(int8_t)((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
                        int q3 = (int)(int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                        int q4 = (int)(int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                        float s1 = d * (float)sc[is], s2 = d * (float)sc[is + 2], s3 = d * (float)sc[is + 4], s4 = d * (float)sc[is + 6];
                        y[h * 128 + l] = s1 * (float)q1;
                        y[h * 128 + l + 32] = s2 * (float)q2;
                        y[h * 128 + l + 64] = s3 * (float)q3;
                        y[h * 128 + l + 96] = s4 * (float)q4;
                    }
                }
            }
            return 0;
    }
    return -2;
}

// Second, independently written decoder: random access to one element, the
// index form of src/gpu/kernels.metal:77-81 (Q8_0) and :889-904 (Q4_K) with
// its own scale unpack (:108-116). Used to cross-check the sequential decode.
ORACLE_API float lokal_ref_dequant_elem(uint32_t ty, const uint8_t* row, size_t col) {
    if (ty == GGML_Q8_0) {
        const uint8_t* b = row + (col >> 5) * 34;
        uint16_t hb = (uint16_t)(b[0] | (b[1] << 8));
        float d = f16_to_f32(hb);
        int q = (int)b[2 + (col & 31)];
        if (q > 127) q -= 256;
        return (float)q * d;
    }
    if (ty == GGML_Q4_K) {
        const uint8_t* b = row + (col >> 8) * 144;
        float d = f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        float dmin = f16_to_f32((uint16_t)(b[2] | (b[3] << 8)));
        const uint8_t* s = b + 4;
        size_t ib = col & 255;
        size_t j = ib >> 5;
        unsigned sc, mn;
        if (j < 4) {
            sc = s[j] & 63u;
            mn = s[j + 4] & 63u;
        } else {
            sc = (s[j + 4] & 0xFu) | ((unsigned)(s[j - 4] >> 6) << 4);
            mn = ((unsigned)s[j + 4] >> 4) | ((unsigned)(s[j] >> 6) << 4);
        }
        float d1 = d * (float)sc;
        float m1 = dmin * (float)mn;
        uint8_t byte = b[16 + (ib >> 6) * 32 + (ib & 31)];
        unsigned q = (ib & 32) ? (unsigned)(byte >> 4) : (unsigned)(byte & 0xF);
        float p = d1 * (float)q;
        return p - m1;
    }
    if (ty == GGML_F16) return f16_to_f32((uint16_t)(row[2 * col] | (row[2 * col + 1] << 8)));
    if (ty == GGML_BF16) return bf16_to_f32((uint16_t)(row[2 * col] | (row[2 * col + 1] << 8)));
    if (ty == GGML_F32) {
        uint32_t u;
        std::memcpy(&u, row + 4 * col, 4);
        return bits_to_f32(u);
    }
    return std::nanf("");
}

// Embedding gather with per-row dequant (src/lowmem/forward.rs:275-307; row
// lookup and range check src/lowmem/mod.rs:654-668). Returns 0, or 1 + the
// index of the first id that is out of range (the reference returns Err).
ORACLE_API int64_t lokal_ref_embed_gather(const uint8_t* table, uint32_t ty, size_t vocab, size_t dim,
                                          const uint32_t* ids, size_t n, float* out, int threads) {
    size_t rb = lokal_ref_row_bytes(ty, dim);
    if (rb == 0) return -1;
    for (size_t i = 0; i < n; i++) {
        if ((size_t)ids[i] + 1 > vocab) return (int64_t)i + 1;
    }
    parallel_rows(n, threads, [=](size_t i0, size_t i1) {
        for (size_t i = i0; i < i1; i++) {
            lokal_ref_dequant_row(ty, table + (size_t)ids[i] * rb, rb, out + i * dim, dim);
        }
    });
    return 0;
}

// Adversarial block generator of the reference's bit-for-bit dequant gate
// (src/lowmem/pool.rs:1079-1195), Q8_0 and Q4_K arms: block variant
// (row*n_blocks+blk)%4 in {all zero, LCG bytes + smallest subnormal scale,
// LCG bytes + negative subnormal scale, LCG bytes + max f16 scale with
// max-magnitude quants}. `out` holds n_rows*n_blocks*blk_bytes bytes.
ORACLE_API int lokal_ref_adversarial_rows(uint32_t ty, size_t n_blocks, size_t n_rows, uint8_t* out) {
    size_t bb = lokal_ref_blk_bytes(ty);
    if (lokal_ref_blk_elems(ty) < 32) return -2;
    // where the f16 scale d sits in a block, and dmin for the types that have one (-1 = none)
    int d_off = 0, dmin_off = -1;
    switch (ty) {
        case GGML_Q4_K: case GGML_Q5_K: dmin_off = 2; break;
        case GGML_Q2_K: d_off = 80; dmin_off = 82; break;   // at the END of the block
        case GGML_Q3_K: d_off = 108; break;
        case GGML_Q6_K: d_off = 208; break;
        default: break;
    }
    uint32_t lcg = 0x2545F491u;
    const uint8_t scale_bytes[4][2] = {{0x00, 0x00}, {0x01, 0x00}, {0xFF, 0x83}, {0xFF, 0x7B}};
    for (size_t row = 0; row < n_rows; row++) {
        for (size_t blk = 0; blk < n_blocks; blk++) {
            size_t variant = (row * n_blocks + blk) % 4;
            uint8_t* b = out + (row * n_blocks + blk) * bb;
            std::memset(b, 0, bb);
            if (variant == 0) continue;
            for (size_t i = 0; i < bb; i++) {
                lcg = lcg * 1664525u + 1013904223u;
                b[i] = (uint8_t)(lcg >> 16);
            }
            if (ty == GGML_IQ1_M) {  // no d field: the f16 goes in through the top nibbles of the four scale u16s
                const unsigned bits = (unsigned)scale_bytes[variant][0] | ((unsigned)scale_bytes[variant][1] << 8);
                for (int k = 0; k < 4; k++) b[49 + 2 * k] = (uint8_t)((b[49 + 2 * k] & 0x0F) | (((bits >> (4 * k)) & 0x0F) << 4));
            } else {
                b[d_off] = scale_bytes[variant][0];
                b[d_off + 1] = scale_bytes[variant][1];
            }
            if (dmin_off >= 0) {
                b[dmin_off] = scale_bytes[3 - variant + 1][0];
                b[dmin_off + 1] = scale_bytes[3 - variant + 1][1];
            }
            if (variant != 3) continue;
            switch (ty) {  // max-magnitude quants under the max scale (src/lowmem/pool.rs:1131-1189)
                case GGML_Q8_0: std::memset(b + 2, 0x80, 32); break;
                case GGML_Q4_0: std::memset(b + 2, 0x0F, 16); break;
                case GGML_Q5_0: std::memset(b + 2, 0xFF, 20); break;          // qh and nibbles all set
                case GGML_Q4_K: std::memset(b + 4, 0xFF, 140); break;         // all scale/min bits, all nibbles
                case GGML_Q5_K: std::memset(b + 4, 0xFF, 172); break;         // scales, high bits, nibbles
                case GGML_IQ4_NL: std::memset(b + 2, 0xFF, 16); break;        // codebook index 15 everywhere
                case GGML_IQ4_XS: std::memset(b + 2, 0xFF, 134); break;       // ls = 63, every nibble 15
                case GGML_Q2_K: std::memset(b, 0xFF, 80); break;              // every scale and min maxed, quants 3
                case GGML_Q3_K:
                    std::memset(b, 0x00, 32);        // hmask clear: the -4 path everywhere
                    std::memset(b + 32, 0xFF, 64);   // quants all 3
                    std::memset(b + 96, 0xFF, 12);   // scales all 63
                    break;
                case GGML_Q6_K:
                    std::memset(b, 0xFF, 192);
                    std::memset(b + 192, 0x80, 16);  // scales = -128
                    break;
                // codebook types: grid indices stay random, the max case drives scales and signs
                case GGML_IQ3_XXS: std::memset(b + 66, 0xFF, 32); break;
                case GGML_IQ2_XXS:
                    for (int g = 0; g < 8; g++) b[2 + 8 * g + 7] = 0xFF;  // top nibble of each group's second u32 is the scale
                    break;
                case GGML_IQ2_XS: std::memset(b + 66, 0xFF, 8); break;
                case GGML_IQ1_S: std::memset(b + 34, 0xFF, 16); break;  // qh: max scale, negative delta
                case GGML_IQ1_M: std::memset(b + 32, 0xFF, 16); break;  // qh only; the scales carry the f16
                case GGML_IQ2_S: std::memset(b + 34, 0xFF, 48); break;  // sign half of qs, qh, scales
                case GGML_IQ3_S: std::memset(b + 66, 0xFF, 44); break;  // qh, signs, scales
                default: break;
            }
        }
    }
    return 0;
}

// ---------------------------------------------------------------------------
// Timed CPU baseline: the per-token layer ops of one forward pass, in the
// order src/model.rs:205-256 runs them, with the projections and attention
// (out of scope) replaced by caller-provided buffers. Each worker walks its
// tokens one at a time through all layers, allocating a fresh vector per op
// as the reference does (src/math.rs:48, src/model.rs:247).
// ---------------------------------------------------------------------------

struct LayerPassArgs {
    uint64_t rows, layers, hidden, inter, n_q_heads, n_kv_heads, head_dim;
    float eps, theta;
    int32_t has_bias, has_qk_norm;
    const int32_t* positions;  // null -> pos0 + row
    int64_t pos0;
    // tables / weights
    const uint8_t* embed_table;  // may be null (x starts from x0)
    uint32_t embed_type;
    uint64_t vocab;
    const uint32_t* ids;
    const float* norm_w;     // [layers][2][hidden]
    const float* final_w;    // [hidden]
    const float* q_bias;     // [layers][nq*hd] or null
    const float* k_bias;     // [layers][nkv*hd] or null
    const float* q_norm_w;   // [layers][hd] or null
    const float* k_norm_w;   // [layers][hd] or null
    // per-layer activations produced by the out-of-scope projections,
    // indexed [layer][row][...]; layer stride given in elements
    const float* delta_att;  // [layers][rows][hidden]
    const float* delta_mlp;  // [layers][rows][hidden]
    const float* q;          // [layers][rows][nq*hd]
    const float* k;          // [layers][rows][nkv*hd]
    const float* gate;       // [layers][rows][inter]
    const float* up;         // [layers][rows][inter]
    uint64_t layer_period;   // layers of distinct data; layer l uses l % layer_period
    float* out;              // [rows][hidden] final normed hidden
    float* sink;             // [threads] checksum so nothing is optimised away
};

ORACLE_API void lokal_ref_layer_pass(const LayerPassArgs* ap, int threads) {
    const LayerPassArgs a = *ap;
    size_t H = a.hidden, I = a.inter, QD = a.n_q_heads * a.head_dim, KD = a.n_kv_heads * a.head_dim;
    std::vector<float> sinks((size_t)(threads > 0 ? threads : 1), 0.0f);
    size_t nt = threads > 1 ? (size_t)threads : 1;
    size_t per = (a.rows + nt - 1) / nt;
    auto work = [&](size_t tix, size_t r0, size_t r1) {
        float sink = 0.0f;
        size_t rb = a.embed_table ? lokal_ref_row_bytes(a.embed_type, H) : 0;
        for (size_t r = r0; r < r1; r++) {
            size_t pos = a.positions ? (size_t)a.positions[r] : (size_t)(a.pos0 + (int64_t)r);
            std::vector<float> x(H, 0.0f);
            if (a.embed_table) lokal_ref_dequant_row(a.embed_type, a.embed_table + (size_t)a.ids[r] * rb, rb, x.data(), H);
            for (size_t l = 0; l < a.layers; l++) {
                size_t ld = l % a.layer_period;
                // input norm (the residual from the previous MLP was added below)
                std::vector<float> xn(H);
                ref_rmsnorm(x.data(), a.norm_w + (l * 2 + 0) * H, a.eps, H, xn.data());
                sink += xn[0];
                // q / k: bias, per-head norm, rope
                std::vector<float> q(a.q + (ld * a.rows + r) * QD, a.q + (ld * a.rows + r) * QD + QD);
                std::vector<float> k(a.k + (ld * a.rows + r) * KD, a.k + (ld * a.rows + r) * KD + KD);
                if (a.has_bias) {
                    const float* qb = a.q_bias + l * QD;
                    const float* kb = a.k_bias + l * KD;
                    for (size_t i = 0; i < QD; i++) q[i] += qb[i];
                    for (size_t i = 0; i < KD; i++) k[i] += kb[i];
                }
                if (a.has_qk_norm) {
                    for (size_t h = 0; h < a.n_q_heads; h++) {
                        std::vector<float> normed(a.head_dim);
                        ref_rmsnorm(q.data() + h * a.head_dim, a.q_norm_w + l * a.head_dim, a.eps, a.head_dim, normed.data());
                        std::memcpy(q.data() + h * a.head_dim, normed.data(), a.head_dim * 4);
                    }
                    for (size_t h = 0; h < a.n_kv_heads; h++) {
                        std::vector<float> normed(a.head_dim);
                        ref_rmsnorm(k.data() + h * a.head_dim, a.k_norm_w + l * a.head_dim, a.eps, a.head_dim, normed.data());
                        std::memcpy(k.data() + h * a.head_dim, normed.data(), a.head_dim * 4);
                    }
                }
                ref_rope(q.data(), QD, pos, a.head_dim, a.head_dim, a.theta);
                ref_rope(k.data(), KD, pos, a.head_dim, a.head_dim, a.theta);
                sink += q[0] + k[0];
                // attention residual
                const float* da = a.delta_att + (ld * a.rows + r) * H;
                for (size_t i = 0; i < H; i++) x[i] += da[i];
                // post-attention norm
                std::vector<float> xn2(H);
                ref_rmsnorm(x.data(), a.norm_w + (l * 2 + 1) * H, a.eps, H, xn2.data());
                sink += xn2[0];
                // SwiGLU
                const float* g = a.gate + (ld * a.rows + r) * I;
                const float* u = a.up + (ld * a.rows + r) * I;
                std::vector<float> inner(I);
                for (size_t i = 0; i < I; i++) inner[i] = ref_silu(g[i]) * u[i];
                sink += inner[0];
                // MLP residual
                const float* dm = a.delta_mlp + (ld * a.rows + r) * H;
                for (size_t i = 0; i < H; i++) x[i] += dm[i];
            }
            ref_rmsnorm(x.data(), a.final_w, a.eps, H, a.out + r * H);
        }
        sinks[tix] = sink;
    };
    if (nt == 1) {
        work(0, 0, a.rows);
    } else {
        std::vector<std::thread> pool;
        for (size_t t = 0; t < nt; t++) {
            size_t r0 = t * per, r1 = r0 + per < a.rows ? r0 + per : a.rows;
            if (r0 >= r1) break;
            pool.emplace_back(work, t, r0, r1);
        }
        for (auto& th : pool) th.join();
    }
    if (a.sink) {
        float s = 0;
        for (float v : sinks) s += v;
        *a.sink = s;
    }
}

ORACLE_API unsigned lokal_ref_hardware_threads(void) { return std::thread::hardware_concurrency(); }
