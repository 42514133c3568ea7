/*
 * kmll_oracle.h — CPU restatement of kmll's (nn-rust) own CPU code for the quantized
 * decode path.  TEST INFRASTRUCTURE ONLY: this library is the checker that the CUDA
 * kernels are compared against and the timed CPU baseline; nothing in the shipped
 * package may call it.
 *
 * Every function cites the reference file:line (paths inside the kmll repository)
 * whose arithmetic it follows.  All float arithmetic is plain IEEE binary32 evaluated in
 * the reference's order; the library must be compiled with -ffp-contract=off and without
 * -ffast-math so no FMA contraction or re-association happens (Rust does neither).
 *
 * Row loops are OpenMP-parallel; each row is still evaluated sequentially by one thread
 * in the reference's left-to-right order, so results are bit-identical for any thread
 * count.  kmll_oracle_set_threads(1) gives the single-thread run.
 *
 * Parity status: the RS-I8 path, RMSNorm, RoPE, attention, SwiGLU, add, argmax and the
 * bf16 conversions restate reference code and are pinned by the reference's own
 * known-answer tests (tests/golden).  The W4-G128 format does not exist in the reference:
 * its functions follow the same per-row rule applied per 128-column group and are
 * PARITY UNPINNED with respect to the reference.
 */
#ifndef KMLL_ORACLE_H
#define KMLL_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int kmll_oracle_max_threads(void);
void kmll_oracle_set_threads(int n);

/* crates/inference/src/dtypes.rs:148-157 */
float kmll_oracle_bf16_to_f32(uint16_t bits);
uint16_t kmll_oracle_bf16_from_f32(float value);
void kmll_oracle_bf16_from_f32_array(const float* src, size_t n, uint16_t* dst);
void kmll_oracle_bf16_to_f32_array(const uint16_t* src, size_t n, float* dst);

/* IEEE binary16 conversions (round to nearest even) used by the W4-G128 group scales. */
uint16_t kmll_oracle_f16_from_f32(float value);
float kmll_oracle_f16_to_f32(uint16_t bits);

/* src/main.rs:4763-4769 (next_stress_value) and :4494-4527 (fill helpers) */
float kmll_oracle_lcg_next(uint64_t* seed);
void kmll_oracle_lcg_fill_f32(float* dst, size_t n, uint64_t* seed, float scale);
void kmll_oracle_lcg_fill_bf16(uint16_t* dst, size_t n, uint64_t* seed);

/* RS-I8: crates/inference/src/rowwise_scaled.rs:21-51, :53-63, :108-126 */
void kmll_oracle_rs_i8_quantize(const uint16_t* weight_bf16, size_t rows, size_t cols,
                                int8_t* values, float* scales);
void kmll_oracle_rs_i8_dequant(const int8_t* values, const float* scales, size_t rows,
                               size_t cols, float* out);
void kmll_oracle_rs_i8_matvec(const int8_t* values, const float* scales, size_t rows,
                              size_t cols, const float* x, float* y);
/* src/main.rs:4617-4637 (cpu_batched_linear_i8_scaled_reference) */
void kmll_oracle_rs_i8_linear_batched(const float* x, size_t batch, const int8_t* values,
                                      const float* scales, size_t out_dim, size_t in_dim,
                                      float* y);

/* W4-G128 (new format, same rule per 128-column group; see header comment). */
void kmll_oracle_w4_quantize(const float* weight, size_t rows, size_t cols, uint8_t* packed,
                             uint16_t* gscales_f16);
void kmll_oracle_w4_dequant(const uint8_t* packed, const uint16_t* gscales_f16, size_t rows,
                            size_t cols, float* out);
void kmll_oracle_w4_matvec(const uint8_t* packed, const uint16_t* gscales_f16, size_t rows,
                           size_t cols, const float* x, float* y);
void kmll_oracle_w4_linear_batched(const float* x, size_t batch, const uint8_t* packed,
                                   const uint16_t* gscales_f16, size_t out_dim, size_t in_dim,
                                   float* y);

/* crates/inference/src/model.rs:11524-11535 (cpu_matvec_bf16) */
void kmll_oracle_matvec_bf16(const float* x, const uint16_t* weight_bf16, size_t out_dim,
                             size_t in_dim, float* y);

/* crates/inference/src/model.rs:11514-11522 (cpu_rmsnorm_bf16); batched form applies it per
 * row as rmsnorm_batched_bf16_kernel does (crates/inference/src/kernels/inference.rs:117-177). */
void kmll_oracle_rmsnorm(const float* x, const uint16_t* weight_bf16, size_t n, float eps,
                         float* y);
void kmll_oracle_rmsnorm_batched(const float* x, const uint16_t* weight_bf16, size_t batch,
                                 size_t dim, float eps, float* y);

/* crates/inference/src/model.rs:11651-11656 (cpu_add), :11662-11666 (SiLU·up) */
void kmll_oracle_add(const float* a, const float* b, size_t n, float* out);
void kmll_oracle_silu_mul(const float* gate, const float* up, size_t n, float* out);

/* crates/inference/src/model.rs:9240-9255 (rope_frequencies, no YaRN) and :9257-9306 (YaRN) */
void kmll_oracle_rope_frequencies(float theta, size_t rotary_dim, float* freqs);
void kmll_oracle_rope_frequencies_yarn(float theta, size_t rotary_dim, float factor,
                                       float beta_fast, float beta_slow,
                                       size_t original_max_position, float* freqs);
/* crates/inference/src/model.rs:11554-11579 (cpu_apply_rope) */
void kmll_oracle_apply_rope(const float* x, size_t len, const float* freqs, size_t n_freqs,
                            size_t position, size_t head_dim, float* out);

/* crates/inference/src/model.rs:11581-11608 and :11610-11649 */
void kmll_oracle_attention_scores(const float* query, const float* key_cache, size_t seq_len,
                                  size_t max_seq_len, size_t n_heads, size_t n_kv_heads,
                                  size_t head_dim, float* scores);
void kmll_oracle_softmax_value(const float* scores, const float* value_cache, size_t seq_len,
                               size_t max_seq_len, size_t n_heads, size_t n_kv_heads,
                               size_t head_dim, float* out);
/* scores + softmax·V for one query; the fused kernel's contract
 * (crates/inference/src/kernels/inference.rs:1420-1550). */
void kmll_oracle_single_query_attention(const float* query, const float* key_cache,
                                        const float* value_cache, size_t seq_len,
                                        size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                        float* out);
/* Row r attends to cache positions 0..=r (crates/inference/src/kernels/inference.rs:1553-1686). */
void kmll_oracle_prefill_causal_attention(const float* query_batch, const float* key_cache,
                                          const float* value_cache, size_t prompt_len,
                                          size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                          float* out);

/* Row softmax with the three-pass math of crates/inference/src/kernels/inference.rs:1343-1398:
 * max, sum of exp(x-max), exp(x-max)/sum. */
void kmll_oracle_softmax_rows(const float* x, size_t rows, size_t cols, float* out);

/* src/main.rs:4187-4201 (top1_from_logits): strictly greater wins, ties -> lower index.
 * Returns (f32 bits << 32) | token, crates/inference/src/kernels/inference.rs:1803-1807. */
uint64_t kmll_oracle_top1_packed(const float* logits, size_t n);
/* crates/inference/src/model.rs:11796-11806 (top_k_logits): stable sort by total order, descending. */
void kmll_oracle_top_k(const float* logits, size_t n, size_t k, uint32_t* tokens, float* values);

/* crates/inference/src/kernels/inference.rs:21-34 (bf16 row -> f32) */
void kmll_oracle_embedding(const uint16_t* table_bf16, size_t dim, uint32_t token, float* out);

#ifdef __cplusplus
}
#endif
#endif
