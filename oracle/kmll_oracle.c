/*
 * kmll_oracle.c — CPU restatement of kmll's own CPU code for the quantized decode path.
 * TEST INFRASTRUCTURE ONLY (see kmll_oracle.h).  Compile with
 *   gcc -O3 -march=x86-64-v3 -ffp-contract=off -fopenmp -shared -fPIC
 * -ffp-contract=off is required: the reference (Rust) never fuses a*b+c.
 */
#include "kmll_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int kmll_oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void kmll_oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

static inline uint32_t f32_bits(float v) {
    uint32_t b;
    memcpy(&b, &v, 4);
    return b;
}
static inline float f32_from_bits(uint32_t b) {
    float v;
    memcpy(&v, &b, 4);
    return v;
}

/* crates/inference/src/dtypes.rs:148-150: widen = bits << 16 */
float kmll_oracle_bf16_to_f32(uint16_t bits) { return f32_from_bits((uint32_t)bits << 16); }

/* crates/inference/src/dtypes.rs:153-157: bias trick, wrapping u32 add, no NaN special case */
uint16_t kmll_oracle_bf16_from_f32(float value) {
    uint32_t bits = f32_bits(value);
    uint32_t rounding_bias = ((bits >> 16) & 1u) + 0x7fffu;
    return (uint16_t)((bits + rounding_bias) >> 16);
}

void kmll_oracle_bf16_from_f32_array(const float* src, size_t n, uint16_t* dst) {
    for (size_t i = 0; i < n; ++i) dst[i] = kmll_oracle_bf16_from_f32(src[i]);
}
void kmll_oracle_bf16_to_f32_array(const uint16_t* src, size_t n, float* dst) {
    for (size_t i = 0; i < n; ++i) dst[i] = kmll_oracle_bf16_to_f32(src[i]);
}

/* IEEE binary16 <-> binary32, round to nearest even, written out by hand so the result does
 * not depend on compiler support for _Float16. */
uint16_t kmll_oracle_f16_from_f32(float value) {
    uint32_t x = f32_bits(value);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mag = x & 0x7fffffffu;
    if (mag >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((mag > 0x7f800000u) ? 0x0200u : 0u));
    }
    if (mag >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (mag < 0x33000001u) { /* <= 2^-25 -> +-0 (exactly 2^-25 ties to even = 0) */
        return (uint16_t)sign;
    }
    int exp = (int)(mag >> 23) - 127;
    uint32_t man = (mag & 0x7fffffu) | 0x800000u; /* 24-bit significand */
    int shift;
    uint32_t base;
    if (exp < -14) { /* subnormal half */
        shift = 13 + (-14 - exp);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(exp + 15) << 10;
        man &= 0x7fffffu;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q += 1; /* carry propagates into exponent */
    return (uint16_t)(sign | (base + q));
}

float kmll_oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return f32_from_bits(sign);
        float v = (float)man * 5.9604644775390625e-08f; /* 2^-24, exact */
        return sign ? -v : v;
    }
    if (exp == 31) return f32_from_bits(sign | 0x7f800000u | (man << 13));
    return f32_from_bits(sign | ((exp + 112u) << 23) | (man << 13));
}

/* src/main.rs:4763-4769 */
float kmll_oracle_lcg_next(uint64_t* seed) {
    *seed = (*seed) * 6364136223846793005ull + 1442695040888963407ull;
    float bucket = (float)((*seed >> 32) & 0xffffull) / 65535.0f;
    return bucket * 2.0f - 1.0f;
}
/* src/main.rs:4508-4512 (fill_stress_slice); scale 1.0 gives fill_matrix over a packed layout */
void kmll_oracle_lcg_fill_f32(float* dst, size_t n, uint64_t* seed, float scale) {
    for (size_t i = 0; i < n; ++i) dst[i] = kmll_oracle_lcg_next(seed) * scale;
}
/* src/main.rs:4514-4527 (fill_bf16_matrix over a packed row-major layout) */
void kmll_oracle_lcg_fill_bf16(uint16_t* dst, size_t n, uint64_t* seed) {
    for (size_t i = 0; i < n; ++i) dst[i] = kmll_oracle_bf16_from_f32(kmll_oracle_lcg_next(seed));
}

/* Rust f32::max: returns the other operand when one is NaN. */
static inline float rust_f32_max(float a, float b) {
    if (a != a) return b;
    if (b != b) return a;
    return a > b ? a : b;
}

/* Rust `f as i8`: saturating, NaN -> 0. The value is already clamped to [-127,127]. */
static inline int8_t rust_f32_as_i8(float v) {
    if (v != v) return 0;
    if (v <= -128.0f) return -128;
    if (v >= 127.0f) return 127;
    return (int8_t)v;
}

/* Rust f32::clamp(min,max): NaN stays NaN. */
static inline float rust_clamp(float v, float lo, float hi) {
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

/* crates/inference/src/rowwise_scaled.rs:21-51 */
void kmll_oracle_rs_i8_quantize(const uint16_t* weight, size_t rows, size_t cols, int8_t* values,
                                float* scales) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r) {
        const uint16_t* row = weight + (size_t)r * cols;
        float max_abs = 0.0f;
        for (size_t c = 0; c < cols; ++c)
            max_abs = rust_f32_max(max_abs, fabsf(kmll_oracle_bf16_to_f32(row[c])));
        float scale = (max_abs == 0.0f) ? 1.0f : max_abs / 127.0f;
        scales[r] = scale;
        for (size_t c = 0; c < cols; ++c) {
            float scaled = rust_clamp(roundf(kmll_oracle_bf16_to_f32(row[c]) / scale), -127.0f, 127.0f);
            values[(size_t)r * cols + c] = rust_f32_as_i8(scaled);
        }
    }
}

/* crates/inference/src/rowwise_scaled.rs:53-63 */
void kmll_oracle_rs_i8_dequant(const int8_t* values, const float* scales, size_t rows, size_t cols,
                               float* out) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r)
        for (size_t c = 0; c < cols; ++c)
            out[(size_t)r * cols + c] = (float)values[(size_t)r * cols + c] * scales[r];
}

/* crates/inference/src/rowwise_scaled.rs:108-126: acc += (w as f32 * scale) * x, left to right */
void kmll_oracle_rs_i8_matvec(const int8_t* values, const float* scales, size_t rows, size_t cols,
                              const float* x, float* y) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r) {
        const int8_t* row = values + (size_t)r * cols;
        float scale = scales[r];
        float acc = 0.0f;
        for (size_t c = 0; c < cols; ++c) acc += (float)row[c] * scale * x[c];
        y[r] = acc;
    }
}

/* src/main.rs:4617-4637: acc += input * scaled_value(col, kk) */
void kmll_oracle_rs_i8_linear_batched(const float* x, size_t batch, const int8_t* values,
                                      const float* scales, size_t out_dim, size_t in_dim,
                                      float* y) {
#pragma omp parallel for schedule(static)
    for (long col = 0; col < (long)out_dim; ++col) {
        const int8_t* wrow = values + (size_t)col * in_dim;
        float scale = scales[col];
        for (size_t row = 0; row < batch; ++row) {
            const float* xr = x + row * in_dim;
            float acc = 0.0f;
            for (size_t kk = 0; kk < in_dim; ++kk) acc += xr[kk] * ((float)wrow[kk] * scale);
            y[row * out_dim + (size_t)col] = acc;
        }
    }
}

/* W4-G128: the rule of rowwise_scaled.rs:21-51 applied per 128-column group with
 * max level 7 and the scale rounded to binary16 BEFORE it is used to quantize.
 * Nibble = q + 8 (1..15), low nibble = even column. */
#define KMLL_W4_GROUP 128

void kmll_oracle_w4_quantize(const float* weight, size_t rows, size_t cols, uint8_t* packed,
                             uint16_t* gscales) {
    size_t groups = cols / KMLL_W4_GROUP;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r) {
        const float* row = weight + (size_t)r * cols;
        for (size_t g = 0; g < groups; ++g) {
            const float* grp = row + g * KMLL_W4_GROUP;
            float max_abs = 0.0f;
            for (size_t c = 0; c < KMLL_W4_GROUP; ++c) max_abs = rust_f32_max(max_abs, fabsf(grp[c]));
            float scale_f32 = (max_abs == 0.0f) ? 1.0f : max_abs / 7.0f;
            uint16_t scale_h = kmll_oracle_f16_from_f32(scale_f32);
            if ((scale_h & 0x7fffu) == 0) scale_h = 0x0001u; /* never divide by a zero scale */
            gscales[(size_t)r * groups + g] = scale_h;
            float scale = kmll_oracle_f16_to_f32(scale_h);
            uint8_t* dst = packed + ((size_t)r * cols + g * KMLL_W4_GROUP) / 2;
            for (size_t c = 0; c < KMLL_W4_GROUP; c += 2) {
                float q0 = rust_clamp(roundf(grp[c] / scale), -7.0f, 7.0f);
                float q1 = rust_clamp(roundf(grp[c + 1] / scale), -7.0f, 7.0f);
                int n0 = (int)rust_f32_as_i8(q0) + 8;
                int n1 = (int)rust_f32_as_i8(q1) + 8;
                dst[c / 2] = (uint8_t)(n0 | (n1 << 4));
            }
        }
    }
}

static inline float w4_value(const uint8_t* packed, const uint16_t* gscales, size_t groups,
                             size_t cols, size_t r, size_t c) {
    uint8_t byte = packed[(r * cols + c) / 2];
    int nib = (c & 1) ? (byte >> 4) : (byte & 0xf);
    float scale = kmll_oracle_f16_to_f32(gscales[r * groups + c / KMLL_W4_GROUP]);
    return (float)(nib - 8) * scale;
}

void kmll_oracle_w4_dequant(const uint8_t* packed, const uint16_t* gscales, size_t rows,
                            size_t cols, float* out) {
    size_t groups = cols / KMLL_W4_GROUP;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r)
        for (size_t c = 0; c < cols; ++c)
            out[(size_t)r * cols + c] = w4_value(packed, gscales, groups, cols, (size_t)r, c);
}

/* matvec_cpu (rowwise_scaled.rs:108-126) with the W4 dequantized value in place of w*scale */
void kmll_oracle_w4_matvec(const uint8_t* packed, const uint16_t* gscales, size_t rows, size_t cols,
                           const float* x, float* y) {
    size_t groups = cols / KMLL_W4_GROUP;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r) {
        const uint8_t* prow = packed + (size_t)r * cols / 2;
        float acc = 0.0f;
        for (size_t g = 0; g < groups; ++g) {
            float scale = kmll_oracle_f16_to_f32(gscales[(size_t)r * groups + g]);
            const uint8_t* pg = prow + g * (KMLL_W4_GROUP / 2);
            const float* xg = x + g * KMLL_W4_GROUP;
            for (size_t b = 0; b < KMLL_W4_GROUP / 2; ++b) {
                uint8_t byte = pg[b];
                acc += (float)((int)(byte & 0xf) - 8) * scale * xg[2 * b];
                acc += (float)((int)(byte >> 4) - 8) * scale * xg[2 * b + 1];
            }
        }
        y[r] = acc;
    }
}

void kmll_oracle_w4_linear_batched(const float* x, size_t batch, const uint8_t* packed,
                                   const uint16_t* gscales, size_t out_dim, size_t in_dim,
                                   float* y) {
    size_t groups = in_dim / KMLL_W4_GROUP;
#pragma omp parallel for schedule(static)
    for (long col = 0; col < (long)out_dim; ++col) {
        const uint8_t* prow = packed + (size_t)col * in_dim / 2;
        for (size_t row = 0; row < batch; ++row) {
            const float* xr = x + row * in_dim;
            float acc = 0.0f;
            for (size_t g = 0; g < groups; ++g) {
                float scale = kmll_oracle_f16_to_f32(gscales[(size_t)col * groups + g]);
                const uint8_t* pg = prow + g * (KMLL_W4_GROUP / 2);
                const float* xg = xr + g * KMLL_W4_GROUP;
                for (size_t b = 0; b < KMLL_W4_GROUP / 2; ++b) {
                    uint8_t byte = pg[b];
                    acc += xg[2 * b] * ((float)((int)(byte & 0xf) - 8) * scale);
                    acc += xg[2 * b + 1] * ((float)((int)(byte >> 4) - 8) * scale);
                }
            }
            y[row * out_dim + (size_t)col] = acc;
        }
    }
}

/* crates/inference/src/model.rs:11524-11535 */
void kmll_oracle_matvec_bf16(const float* x, const uint16_t* weight, size_t out_dim, size_t in_dim,
                             float* y) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)out_dim; ++r) {
        const uint16_t* row = weight + (size_t)r * in_dim;
        float acc = 0.0f;
        for (size_t c = 0; c < in_dim; ++c) acc += kmll_oracle_bf16_to_f32(row[c]) * x[c];
        y[r] = acc;
    }
}

/* crates/inference/src/model.rs:11514-11522 */
void kmll_oracle_rmsnorm(const float* x, const uint16_t* weight, size_t n, float eps, float* y) {
    float sum_sq = 0.0f;
    for (size_t i = 0; i < n; ++i) sum_sq += x[i] * x[i];
    float inv_scale = 1.0f / sqrtf(sum_sq / (float)n + eps);
    for (size_t i = 0; i < n; ++i) y[i] = x[i] * inv_scale * kmll_oracle_bf16_to_f32(weight[i]);
}

void kmll_oracle_rmsnorm_batched(const float* x, const uint16_t* weight, size_t batch, size_t dim,
                                 float eps, float* y) {
#pragma omp parallel for schedule(static)
    for (long b = 0; b < (long)batch; ++b)
        kmll_oracle_rmsnorm(x + (size_t)b * dim, weight, dim, eps, y + (size_t)b * dim);
}

/* crates/inference/src/model.rs:11651-11656 */
void kmll_oracle_add(const float* a, const float* b, size_t n, float* out) {
    for (size_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

/* crates/inference/src/model.rs:11662-11666: (gate / (1 + exp(-gate))) * up */
void kmll_oracle_silu_mul(const float* gate, const float* up, size_t n, float* out) {
    for (size_t i = 0; i < n; ++i) out[i] = (gate[i] / (1.0f + expf(-gate[i]))) * up[i];
}

/* crates/inference/src/model.rs:9240-9249 */
void kmll_oracle_rope_frequencies(float theta, size_t rotary_dim, float* freqs) {
    size_t half = rotary_dim / 2;
    for (size_t i = 0; i < half; ++i)
        freqs[i] = 1.0f / powf(theta, (float)(2 * i) / (float)rotary_dim);
}

/* crates/inference/src/model.rs:9285-9296 */
static float yarn_correction_dim(float num_rotations, size_t dim, float base, size_t max_pos) {
    return ((float)dim * logf((float)max_pos / (num_rotations * 2.0f * 3.14159265358979323846f))) /
           (2.0f * logf(base));
}
/* crates/inference/src/model.rs:9298-9303 */
static float yarn_linear_ramp(float low, float high, float dim) {
    if (fabsf(low - high) < 1.1920929e-07f) high += 0.001f;
    return rust_clamp((dim - low) / (high - low), 0.0f, 1.0f);
}
/* crates/inference/src/model.rs:9257-9283 */
void kmll_oracle_rope_frequencies_yarn(float theta, size_t rotary_dim, float factor, float beta_fast,
                                       float beta_slow, size_t original_max_position, float* freqs) {
    size_t half = rotary_dim / 2;
    kmll_oracle_rope_frequencies(theta, rotary_dim, freqs);
    float low = rust_f32_max(floorf(yarn_correction_dim(beta_fast, rotary_dim, theta, original_max_position)), 0.0f);
    float high = ceilf(yarn_correction_dim(beta_slow, rotary_dim, theta, original_max_position));
    float cap = (float)(rotary_dim - 1);
    if (high > cap) high = cap;
    for (size_t i = 0; i < half; ++i) {
        float extrapolated = freqs[i];
        float interpolation = extrapolated / factor;
        float w = 1.0f - yarn_linear_ramp(low, high, (float)i);
        freqs[i] = interpolation * (1.0f - w) + extrapolated * w;
    }
}

/* crates/inference/src/model.rs:11554-11579 */
void kmll_oracle_apply_rope(const float* x, size_t len, const float* freqs, size_t n_freqs,
                            size_t position, size_t head_dim, float* out) {
    size_t half = n_freqs;
    size_t rotary_dim = half * 2;
    for (size_t i = 0; i < len; ++i) {
        size_t head = i / head_dim;
        size_t dim = i - head * head_dim;
        if (dim >= rotary_dim) {
            out[i] = x[i];
            continue;
        }
        size_t pair_dim = dim < half ? dim : dim - half;
        size_t base = head * head_dim;
        float first = x[base + pair_dim];
        float second = x[base + pair_dim + half];
        float angle = (float)position * freqs[pair_dim];
        float s = sinf(angle);
        float c = cosf(angle);
        out[i] = dim < half ? first * c - second * s : second * c + first * s;
    }
}

/* crates/inference/src/model.rs:11581-11608 */
void kmll_oracle_attention_scores(const float* query, const float* key_cache, size_t seq_len,
                                  size_t max_seq_len, size_t n_heads, size_t n_kv_heads,
                                  size_t head_dim, float* scores) {
    size_t heads_per_kv = n_heads / n_kv_heads;
    float scale = 1.0f / sqrtf((float)head_dim);
    memset(scores, 0, sizeof(float) * n_heads * max_seq_len);
#pragma omp parallel for schedule(static)
    for (long head = 0; head < (long)n_heads; ++head) {
        size_t kv_head = (size_t)head / heads_per_kv;
        size_t q_offset = (size_t)head * head_dim;
        for (size_t pos = 0; pos < seq_len; ++pos) {
            size_t k_offset = pos * n_kv_heads * head_dim + kv_head * head_dim;
            float dot = 0.0f;
            for (size_t d = 0; d < head_dim; ++d) dot += query[q_offset + d] * key_cache[k_offset + d];
            scores[(size_t)head * max_seq_len + pos] = dot * scale;
        }
    }
}

/* crates/inference/src/model.rs:11610-11649 */
void kmll_oracle_softmax_value(const float* scores, const float* value_cache, size_t seq_len,
                               size_t max_seq_len, size_t n_heads, size_t n_kv_heads,
                               size_t head_dim, float* out) {
    size_t heads_per_kv = n_heads / n_kv_heads;
#pragma omp parallel for schedule(static)
    for (long head = 0; head < (long)n_heads; ++head) {
        size_t score_base = (size_t)head * max_seq_len;
        float max_score = scores[score_base];
        for (size_t pos = 1; pos < seq_len; ++pos) max_score = rust_f32_max(max_score, scores[score_base + pos]);
        size_t kv_head = (size_t)head / heads_per_kv;
        float denom = 0.0f;
        float* weights = (float*)malloc(sizeof(float) * (seq_len ? seq_len : 1));
        for (size_t pos = 0; pos < seq_len; ++pos) {
            float w = expf(scores[score_base + pos] - max_score);
            denom += w;
            weights[pos] = w;
        }
        for (size_t d = 0; d < head_dim; ++d) {
            float acc = 0.0f;
            for (size_t pos = 0; pos < seq_len; ++pos)
                acc += weights[pos] * value_cache[pos * n_kv_heads * head_dim + kv_head * head_dim + d];
            out[(size_t)head * head_dim + d] = acc / denom;
        }
        free(weights);
    }
}

void kmll_oracle_single_query_attention(const float* query, const float* key_cache,
                                        const float* value_cache, size_t seq_len, size_t n_heads,
                                        size_t n_kv_heads, size_t head_dim, float* out) {
    float* scores = (float*)malloc(sizeof(float) * n_heads * (seq_len ? seq_len : 1));
    kmll_oracle_attention_scores(query, key_cache, seq_len, seq_len, n_heads, n_kv_heads, head_dim, scores);
    kmll_oracle_softmax_value(scores, value_cache, seq_len, seq_len, n_heads, n_kv_heads, head_dim, out);
    free(scores);
}

void kmll_oracle_prefill_causal_attention(const float* query_batch, const float* key_cache,
                                          const float* value_cache, size_t prompt_len,
                                          size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                          float* out) {
    size_t q_len = n_heads * head_dim;
    for (size_t row = 0; row < prompt_len; ++row)
        kmll_oracle_single_query_attention(query_batch + row * q_len, key_cache, value_cache, row + 1,
                                           n_heads, n_kv_heads, head_dim, out + row * q_len);
}

/* crates/inference/src/kernels/inference.rs:1343-1398: max, sum exp(x-max), exp(x-max)/sum */
void kmll_oracle_softmax_rows(const float* x, size_t rows, size_t cols, float* out) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r) {
        const float* xr = x + (size_t)r * cols;
        float* yr = out + (size_t)r * cols;
        float m = xr[0];
        for (size_t c = 1; c < cols; ++c) m = rust_f32_max(m, xr[c]);
        float denom = 0.0f;
        for (size_t c = 0; c < cols; ++c) denom += expf(xr[c] - m);
        for (size_t c = 0; c < cols; ++c) yr[c] = expf(xr[c] - m) / denom;
    }
}

/* src/main.rs:4187-4201 */
uint64_t kmll_oracle_top1_packed(const float* logits, size_t n) {
    uint32_t best_token = 0;
    float best_logit = 0.0f;
    int have = 0;
    for (size_t i = 0; i < n; ++i) {
        float logit = logits[i];
        uint32_t token = (uint32_t)i;
        if (!have || logit > best_logit || (logit == best_logit && token < best_token)) {
            best_token = token;
            best_logit = logit;
            have = 1;
        }
    }
    return ((uint64_t)f32_bits(best_logit) << 32) | (uint64_t)best_token;
}

/* f32::total_cmp key: sign-magnitude bits -> monotone signed integer */
static inline int32_t total_order_key(float v) {
    int32_t b = (int32_t)f32_bits(v);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}

/* crates/inference/src/model.rs:11796-11806: stable descending sort by total_cmp, truncate to k */
void kmll_oracle_top_k(const float* logits, size_t n, size_t k, uint32_t* tokens, float* values) {
    if (k > n) k = n;
    for (size_t j = 0; j < k; ++j) {
        size_t best = (size_t)-1;
        int32_t best_key = 0;
        for (size_t i = 0; i < n; ++i) {
            int taken = 0;
            for (size_t p = 0; p < j; ++p)
                if (tokens[p] == (uint32_t)i) { taken = 1; break; }
            if (taken) continue;
            int32_t key = total_order_key(logits[i]);
            if (best == (size_t)-1 || key > best_key) {
                best = i;
                best_key = key;
            }
        }
        tokens[j] = (uint32_t)best;
        values[j] = logits[best];
    }
}

/* crates/inference/src/kernels/inference.rs:21-34 */
void kmll_oracle_embedding(const uint16_t* table, size_t dim, uint32_t token, float* out) {
    for (size_t i = 0; i < dim; ++i) out[i] = kmll_oracle_bf16_to_f32(table[(size_t)token * dim + i]);
}
