/*
 * kmll_b200.h — C ABI of the B200 (sm_100a) implementation of kmll's quantized decode path.
 *
 * One entry point per operator of kmll's `crates/inference/src/ops` module, so that the Rust
 * host can bind them with a plain `extern "C"` block in place of its `cuda_launch!` wrappers.
 * Conventions shared by every function:
 *   - `stream` is a CUDA stream handle (cudaStream_t / CUstream); ops only enqueue work on it
 *     and never synchronise (kmll ops have the same contract, crates/inference/src/ops/inference.rs).
 *   - every pointer is a DEVICE pointer owned by the caller; nothing is allocated or freed by an
 *     operator call (buffers: crates/inference/src/model.rs:9339-9498 allocates scratch once); operators that
 *     need scratch take a caller-owned workspace and say how large it must be.
 *   - the return value is 0 on success or a negative KMLL_ERR_* code.  Where kmll panics on a
 *     shape mismatch (`assert!`, `LayoutError`, crates/inference/src/layout.rs:569-666) the C ABI
 *     returns KMLL_ERR_SHAPE / KMLL_ERR_NULL instead; kmll_last_error() gives the message of the
 *     last failure on the calling thread.
 *   - activations, KV caches, scores and logits are f32, norm weights and embeddings bf16 bit
 *     patterns (uint16_t), exactly as in kmll (crates/inference/src/model.rs:5040-5099).
 *   - calls are thread-safe as long as each thread uses its own stream
 *     (kmll's worker contract, src/cuda_worker.rs:220-226).
 *
 * Weight formats:
 *   RS-I8   kmll's row-symmetric int8: int8 values[rows*cols] row-major + float scales[rows]
 *           (crates/inference/src/rowwise_scaled.rs:12-51); dequant = (float)v * scale[row].
 *   W4-G128 4-bit group-128 symmetric: uint8 packed[rows*cols/2] (low nibble = even column,
 *           nibble = q + 8, q in [-7,7]) + binary16 gscales[rows*cols/128]; dequant =
 *           (float)(nibble - 8) * (float)gscale.  Not present in kmll; follows the RS-I8 rule per
 *           128-column group.  cols must be a multiple of 128.
 */
#ifndef KMLL_B200_H
#define KMLL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* kmll_stream_t; /* cudaStream_t */

enum {
    KMLL_OK = 0,
    KMLL_ERR_NULL = -1,        /* a required pointer is null */
    KMLL_ERR_SHAPE = -2,       /* shape / length mismatch (kmll: assert!/LayoutError) */
    KMLL_ERR_UNSUPPORTED = -3, /* valid request outside what the kernels implement */
    KMLL_ERR_CUDA = -4,        /* a CUDA runtime call failed; see kmll_last_error() */
    KMLL_ERR_CAPACITY = -5,    /* size beyond a fixed capacity of the entry point */
    KMLL_ERR_STATE = -6        /* runtime object used in the wrong state */
};

/* Message of the last failing call on this thread ("" if none). */
const char* kmll_last_error(void);
/* Library version and the SM architecture the kernels were compiled for (100 = sm_100a). */
int kmll_version(void);
/* Device-side status word of the current device: 0 = ok, 1 = a bounded wait inside a kernel timed
 * out (the kernel returned early; its output is invalid), 2 = a tensor-parallel peer did not deliver
 * its part of an exchange within the wait limit.  Synchronises the device. */
int kmll_device_status(int* status_out);
int kmll_compiled_arch(void);

/* Kernel timeline (diagnostics; no counterpart in kmll).  While a device buffer is attached, every
 * launch of the batch<=4 linear kernel and of the decode attention kernel takes the next slot of
 * blocks*6 64-bit words in it, and thread 0 of each block writes the device clock (%globaltimer, ns)
 * at six points: 0 entry, 1 dependency wait passed, 2 inputs staged, 3 main loop done, 4 block done,
 * 5 unused.  Launches recorded into a CUDA graph keep their slots across replays.  Attach a null
 * buffer to stop.  The decoders of kmll_b200_runtime.h capture their per-token graph again after every
 * attach or detach, so their replays never write to a detached buffer; a graph the CALLER captured while a
 * buffer was attached keeps writing to it, so that buffer must outlive the graph.
 * kernel_id: 100 + 10*format + epilogue for the linear kernel, 200 for attention. */
int kmll_trace_attach(void* device_buffer, size_t bytes);
int kmll_trace_launches(int* kernel_ids, int* blocks, size_t* offset_words, int max_launches, int* count_out);

/* ------------------------------------------------------------------------------------------
 * Quantization (device-side restatement of the host quantizer; bit-exact with it)
 * ---------------------------------------------------------------------------------------- */
/* RowwiseScaledI8Matrix::from_bf16_rows_symmetric, crates/inference/src/rowwise_scaled.rs:21-51 */
int kmll_quantize_rs_i8(kmll_stream_t stream, const uint16_t* weight_bf16, int rows, int cols,
                        int8_t* values, float* scales);
/* RowwiseScaledI8Matrix::scaled_value for every element, crates/inference/src/rowwise_scaled.rs:53-63 */
int kmll_dequant_rs_i8(kmll_stream_t stream, const int8_t* values, const float* scales, int rows,
                       int cols, float* out);
/* W4-G128 counterparts (no kmll counterpart; same rule per 128-column group, f32 source). */
int kmll_quantize_w4g128(kmll_stream_t stream, const float* weight, int rows, int cols,
                         uint8_t* packed, uint16_t* gscales_f16);
int kmll_dequant_w4g128(kmll_stream_t stream, const uint8_t* packed, const uint16_t* gscales_f16,
                        int rows, int cols, float* out);
/* f32 -> bf16 bits with kmll's rounding (Bf16::from_f32, crates/inference/src/dtypes.rs:153-157). */
int kmll_f32_to_bf16(kmll_stream_t stream, const float* src, size_t n, uint16_t* dst);
/* Seeded synthetic weights: N(0, std) f32 from a counter-based generator (test/bench helper). */
int kmll_fill_normal_f32(kmll_stream_t stream, float* dst, size_t n, uint64_t seed, float std);

/* ------------------------------------------------------------------------------------------
 * Linear: y = dequant(W) . x        (W is [rows, cols] = [out_features, in_features])
 * ---------------------------------------------------------------------------------------- */
/* CudaLinearWeight::launch_linear for DeviceRowwiseScaledI8Matrix,
 * crates/inference/src/ops/inference.rs:205-252 (matvec_i8_scaled_kernel). */
int kmll_linear_i8(kmll_stream_t stream, const float* x, const int8_t* w, const float* scales,
                   int rows, int cols, float* y);
/* Third implementation of the same trait for the W4-G128 format. */
int kmll_linear_w4g128(kmll_stream_t stream, const float* x, const uint8_t* packed,
                       const uint16_t* gscales_f16, int rows, int cols, float* y);

/* out = residual + W.x — linear_residual_bf16, crates/inference/src/ops/inference.rs:872-921,
 * offered here for the quantized formats. */
int kmll_linear_residual_i8(kmll_stream_t stream, const float* x, const int8_t* w,
                            const float* scales, const float* residual, int rows, int cols,
                            float* out);
int kmll_linear_residual_w4g128(kmll_stream_t stream, const float* x, const uint8_t* packed,
                                const uint16_t* gscales_f16, const float* residual, int rows,
                                int cols, float* out);

/* q,k,v = Wq.x, Wk.x, Wv.x in one launch — linear_triple_bf16,
 * crates/inference/src/ops/inference.rs:924-990 (ragged row counts, shared input). */
int kmll_linear_triple_i8(kmll_stream_t stream, const float* x, const int8_t* wq,
                          const float* sq, const int8_t* wk, const float* sk, const int8_t* wv,
                          const float* sv, int q_rows, int kv_rows, int cols, float* q, float* k,
                          float* v);
int kmll_linear_triple_w4g128(kmll_stream_t stream, const float* x, const uint8_t* wq,
                              const uint16_t* sq, const uint8_t* wk, const uint16_t* sk,
                              const uint8_t* wv, const uint16_t* sv, int q_rows, int kv_rows,
                              int cols, float* q, float* k, float* v);

/* a, b = Wa.x, Wb.x in one launch, two matrices of the same shape — linear_pair_bf16,
 * crates/inference/src/ops/inference.rs:712-775 (kernel matvec_pair, crates/inference/src/kernels/inference.rs:458-532). */
int kmll_linear_pair_i8(kmll_stream_t stream, const float* x, const int8_t* wa, const float* sa, const int8_t* wb,
                        const float* sb, int rows, int cols, float* out_a, float* out_b);
int kmll_linear_pair_w4g128(kmll_stream_t stream, const float* x, const uint8_t* wa, const uint16_t* sa,
                            const uint8_t* wb, const uint16_t* sb, int rows, int cols, float* out_a,
                            float* out_b);

/* out = silu(Wgate.x) * (Wup.x) — silu_gate_up_bf16, crates/inference/src/ops/inference.rs:777-869. */
int kmll_silu_gate_up_i8(kmll_stream_t stream, const float* x, const int8_t* w_gate,
                         const float* s_gate, const int8_t* w_up, const float* s_up, int rows,
                         int cols, float* out);
int kmll_silu_gate_up_w4g128(kmll_stream_t stream, const float* x, const uint8_t* w_gate,
                             const uint16_t* s_gate, const uint8_t* w_up, const uint16_t* s_up,
                             int rows, int cols, float* out);

/* Fused RMSNorm prologue variants (no kmll counterpart as one op; equal to kmll_rmsnorm followed by
 * the op above on the normalised vector): x is normalised with norm_weight_bf16/eps inside the
 * kernel that streams the weights. */
int kmll_rmsnorm_linear_triple_w4g128(kmll_stream_t stream, const float* x,
                                      const uint16_t* norm_weight_bf16, float eps,
                                      const uint8_t* wq, const uint16_t* sq, const uint8_t* wk,
                                      const uint16_t* sk, const uint8_t* wv, const uint16_t* sv,
                                      int q_rows, int kv_rows, int cols, float* q, float* k,
                                      float* v);
int kmll_rmsnorm_linear_triple_i8(kmll_stream_t stream, const float* x,
                                  const uint16_t* norm_weight_bf16, float eps, const int8_t* wq,
                                  const float* sq, const int8_t* wk, const float* sk,
                                  const int8_t* wv, const float* sv, int q_rows, int kv_rows,
                                  int cols, float* q, float* k, float* v);
int kmll_rmsnorm_silu_gate_up_w4g128(kmll_stream_t stream, const float* x,
                                     const uint16_t* norm_weight_bf16, float eps,
                                     const uint8_t* w_gate, const uint16_t* s_gate,
                                     const uint8_t* w_up, const uint16_t* s_up, int rows, int cols,
                                     float* out);
int kmll_rmsnorm_silu_gate_up_i8(kmll_stream_t stream, const float* x,
                                 const uint16_t* norm_weight_bf16, float eps, const int8_t* w_gate,
                                 const float* s_gate, const int8_t* w_up, const float* s_up,
                                 int rows, int cols, float* out);

/* lm_head matvec fused with arg-max — linear_top1_i8_scaled,
 * crates/inference/src/ops/inference.rs:454-560.  packed_out[0] = (f32 bits << 32) | token,
 * ties -> lower token (crates/inference/src/kernels/inference.rs:402-404, :1803-1807).
 * partial_* hold kmll_linear_top1_partial_count(rows) entries
 * (linear_top1_i8_scaled_partial_count, crates/inference/src/ops/inference.rs:258-260). */
int kmll_linear_top1_partial_count(int rows);
int kmll_linear_top1_i8(kmll_stream_t stream, const float* x, const int8_t* w, const float* scales,
                        int rows, int cols, uint32_t* partial_tokens, float* partial_logits,
                        uint64_t* packed_out);
int kmll_linear_top1_w4g128(kmll_stream_t stream, const float* x, const uint8_t* packed,
                            const uint16_t* gscales_f16, int rows, int cols,
                            uint32_t* partial_tokens, float* partial_logits, uint64_t* packed_out);
/* Same with the final RMSNorm folded in (output_top1_from_hidden_i8_into,
 * crates/inference/src/model.rs:10619-10657 runs rmsnorm then linear_top1). */
int kmll_rmsnorm_linear_top1_w4g128(kmll_stream_t stream, const float* x,
                                    const uint16_t* norm_weight_bf16, float eps,
                                    const uint8_t* packed, const uint16_t* gscales_f16, int rows,
                                    int cols, uint32_t* partial_tokens, float* partial_logits,
                                    uint64_t* packed_out);
int kmll_rmsnorm_linear_top1_i8(kmll_stream_t stream, const float* x,
                                const uint16_t* norm_weight_bf16, float eps, const int8_t* w,
                                const float* scales, int rows, int cols, uint32_t* partial_tokens,
                                float* partial_logits, uint64_t* packed_out);

/* ------------------------------------------------------------------------------------------
 * W4-G128 in the PREPARED layout (load-time re-ordering of the same 4-bit values and binary16 scales; no
 * counterpart in kmll, whose int8 weights are used as stored).  The prepared bytes are what the batch-1 kernels
 * stream: records of 32 rows x one 128-column group, 2112 bytes each (2048 bytes of nibbles in tensor-core
 * fragment order + 32 scales), two row blocks sharing every byte so that one logic operation per register
 * separates them.  The canonical arrays stay the interchange format and the dequantization contract
 * (kmll_dequant_w4g128); a prepared buffer is derived from them and holds exactly the same values.
 *   kmll_w4g128_prepare        rows r of a matrix: record u holds rows 32u..32u+15 and 32u+16..32u+31
 *   kmll_w4g128_prepare_pair   gate and up matrices of a gated MLP: record u holds gate rows 16u..16u+15 and the
 *                              same rows of up, so SiLU(gate) * up meets inside one thread
 * The operators below equal their canonical-layout namesakes (same arithmetic contract: exact integer products,
 * activations rounded to 2^-29 of the largest element, f32 accumulation over the 128-column groups);
 * norm_weight_bf16 may be null (no RMSNorm prologue), residual may be null.  Batch 1.
 * ---------------------------------------------------------------------------------------- */
size_t kmll_w4g128_prepared_bytes(int rows, int cols);
size_t kmll_w4g128_prepared_pair_bytes(int rows, int cols);
int kmll_w4g128_prepare(kmll_stream_t stream, const uint8_t* packed, const uint16_t* gscales_f16, int rows, int cols,
                        uint8_t* prepared);
int kmll_w4g128_prepare_pair(kmll_stream_t stream, const uint8_t* gate_packed, const uint16_t* gate_gscales_f16,
                             const uint8_t* up_packed, const uint16_t* up_gscales_f16, int rows, int cols,
                             uint8_t* prepared);
/* y = [residual +] dequant(W) . [rmsnorm](x) — CudaLinearWeight::launch_linear, crates/inference/src/ops/inference.rs:205-252 */
int kmll_linear_w4p(kmll_stream_t stream, const float* x, const uint16_t* norm_weight_bf16, float eps,
                    const uint8_t* prepared, const float* residual, int rows, int cols, float* y);
/* Q, K, V in one launch — matvec_triple, crates/inference/src/kernels/inference.rs:629-739 */
int kmll_linear_triple_w4p(kmll_stream_t stream, const float* x, const uint16_t* norm_weight_bf16, float eps,
                           const uint8_t* prepared_q, const uint8_t* prepared_k, const uint8_t* prepared_v, int q_rows,
                           int kv_rows, int cols, float* q, float* k, float* v);
/* silu(gate . x) * (up . x) — matvec_silu_gate_up, crates/inference/src/kernels/inference.rs:535-626 */
int kmll_silu_gate_up_w4p(kmll_stream_t stream, const float* x, const uint16_t* norm_weight_bf16, float eps,
                          const uint8_t* prepared_pair, int rows, int cols, float* out);
/* lm_head + arg-max — linear_top1_i8_scaled, crates/inference/src/ops/inference.rs:454-560.  Calls of this entry
 * point that overlap on one GPU share an arrival counter and must not run concurrently. */
int kmll_linear_top1_w4p(kmll_stream_t stream, const float* x, const uint16_t* norm_weight_bf16, float eps,
                         const uint8_t* prepared, int rows, int cols, uint32_t* partial_tokens, float* partial_logits,
                         uint64_t* packed_out);

/* y[batch, out] = x[batch, in] . dequant(W)^T — linear_batched_i8_scaled,
 * crates/inference/src/ops/matmul.rs:423-463 (gemm_f32_i8_scaled_tiled_kernel).  x and y are
 * row-major prefixes of possibly larger buffers, as in kmll.
 * `workspace` is caller-owned scratch of kmll_linear_batched_workspace_bytes(batch, in_dim) bytes (16-byte aligned),
 * as kmll's runtime owns every scratch buffer (crates/inference/src/model.rs:9339-9498); with it, 5 or more rows
 * run on the tensor cores (tcgen05, up to 256 rows of x per pass over the weights, exact f16 operand splitting: the
 * result carries f32 accuracy).  It may be null: the call then streams the weights once per 4 rows of x.  Calls
 * that share a workspace must not overlap. */
size_t kmll_linear_batched_workspace_bytes(int batch, int in_dim);
int kmll_linear_batched_i8(kmll_stream_t stream, const float* x, const int8_t* w,
                           const float* scales, int batch, int in_dim, int out_dim, void* workspace, float* y);
int kmll_linear_batched_w4g128(kmll_stream_t stream, const float* x, const uint8_t* packed,
                               const uint16_t* gscales_f16, int batch, int in_dim, int out_dim,
                               void* workspace, float* y);
/* linear_qkv_batched_i8_scaled, crates/inference/src/ops/matmul.rs:465-510 */
int kmll_linear_qkv_batched_i8(kmll_stream_t stream, const float* x, const int8_t* wq,
                               const float* sq, const int8_t* wk, const float* sk,
                               const int8_t* wv, const float* sv, int batch, int in_dim,
                               int q_dim, int kv_dim, void* workspace, float* q, float* k, float* v);
int kmll_linear_qkv_batched_w4g128(kmll_stream_t stream, const float* x, const uint8_t* wq,
                                   const uint16_t* sq, const uint8_t* wk, const uint16_t* sk,
                                   const uint8_t* wv, const uint16_t* sv, int batch, int in_dim,
                                   int q_dim, int kv_dim, void* workspace, float* q, float* k, float* v);

/* ------------------------------------------------------------------------------------------
 * Row reductions and elementwise ops
 * ---------------------------------------------------------------------------------------- */
/* rmsnorm, crates/inference/src/ops/inference.rs:631-653: y = x * (1/sqrt(mean(x^2)+eps)) * w */
int kmll_rmsnorm(kmll_stream_t stream, const float* x, const uint16_t* weight_bf16, int n,
                 float eps, float* y);
/* rmsnorm_batched_bf16, crates/inference/src/ops/inference.rs:655-700 (also per-head q/k norm) */
int kmll_rmsnorm_batched(kmll_stream_t stream, const float* x, const uint16_t* weight_bf16,
                         int batch, int dim, float eps, float* y);
/* add / add_prefix, crates/inference/src/ops/inference.rs:1129-1172 */
int kmll_add(kmll_stream_t stream, const float* a, const float* b, size_t n, float* out);
int kmll_add_prefix(kmll_stream_t stream, const float* a, const float* b, size_t count, float* out);
/* silu_mul / silu_mul_prefix, crates/inference/src/ops/inference.rs:1061-1127: (g/(1+exp(-g)))*u */
int kmll_silu_mul(kmll_stream_t stream, const float* gate, const float* up, size_t n, float* out);
int kmll_silu_mul_prefix(kmll_stream_t stream, const float* gate, const float* up, size_t count,
                         float* out);
/* Row softmax (the three-pass math fused inside softmax_value,
 * crates/inference/src/kernels/inference.rs:1343-1398) as a standalone op. */
int kmll_softmax_rows(kmll_stream_t stream, const float* x, int rows, int cols, float* out);

/* bf16 I/O forms of the micro-suite ops: load bf16 -> f32, same arithmetic, store with
 * Bf16::from_f32 rounding.  positions[b] is the RoPE position of batch row b. */
int kmll_rmsnorm_batched_bf16io(kmll_stream_t stream, const uint16_t* x, const uint16_t* weight_bf16,
                                int batch, int dim, float eps, uint16_t* y);
int kmll_silu_mul_bf16io(kmll_stream_t stream, const uint16_t* gate, const uint16_t* up, size_t n,
                         uint16_t* out);
int kmll_apply_rope_batched_bf16io(kmll_stream_t stream, const uint16_t* x, const float* freqs,
                                   int n_freqs, const int32_t* positions, int batch, int n_heads,
                                   int head_dim, uint16_t* out);
int kmll_softmax_rows_bf16io(kmll_stream_t stream, const uint16_t* x, int rows, int cols,
                             uint16_t* out);

/* apply_rope, crates/inference/src/ops/inference.rs:1400-1421: half-split rotation, dims beyond
 * 2*n_freqs pass through; angle = (float)position * freqs[d]. */
int kmll_apply_rope(kmll_stream_t stream, const float* x, const float* freqs, int n_freqs,
                    int position, int head_dim, size_t len, float* out);
/* write_kv_cache / apply_rope_write_kv_cache, crates/inference/src/ops/inference.rs:1423-1489;
 * cache layout [max_seq_len, n_kv_heads, head_dim] f32. */
int kmll_write_kv_cache(kmll_stream_t stream, const float* x, int position, int max_seq_len,
                        int n_kv_heads, int head_dim, float* cache);
int kmll_apply_rope_write_kv_cache(kmll_stream_t stream, const float* x, const float* freqs,
                                   int n_freqs, int position, int max_seq_len, int n_kv_heads,
                                   int head_dim, float* cache);
/* prepare_incremental_attention, crates/inference/src/ops/inference.rs:1291-1362 */
int kmll_prepare_incremental_attention(kmll_stream_t stream, const float* query, const float* key,
                                       const float* value, const float* freqs, int n_freqs,
                                       int position, int max_seq_len, int n_heads, int n_kv_heads,
                                       int head_dim, float* query_rot, float* key_cache,
                                       float* value_cache);
/* prepare_prefill_attention_batch, crates/inference/src/ops/inference.rs:1220-1288; row i of the
 * batch is position i. */
int kmll_prepare_prefill_attention_batch(kmll_stream_t stream, const float* query_batch,
                                         const float* key_batch, const float* value_batch,
                                         const float* freqs, int n_freqs, int prompt_len,
                                         int q_len, int kv_len, int head_dim,
                                         float* query_rot_batch, float* key_cache,
                                         float* value_cache);

/* ------------------------------------------------------------------------------------------
 * Attention
 * ---------------------------------------------------------------------------------------- */
/* attention_scores / softmax_value, crates/inference/src/ops/inference.rs:1492-1544, :1606-1654 */
int kmll_attention_scores(kmll_stream_t stream, const float* query, const float* key_cache,
                          int seq_len, int max_seq_len, int n_heads, int n_kv_heads, int head_dim,
                          float* scores);
int kmll_softmax_value(kmll_stream_t stream, const float* scores, const float* value_cache,
                       int seq_len, int max_seq_len, int n_heads, int n_kv_heads, int head_dim,
                       float* out);
/* single_query_attention, crates/inference/src/ops/inference.rs:1657-1710.  kmll's kernel caps
 * seq_len at 4096; this one splits the sequence across thread blocks and has no cap.
 * `workspace` holds kmll_single_query_attention_workspace_floats(...) floats of scratch and a
 * trailing counter area that must be zero before the first call (the kernel leaves it zero). */
size_t kmll_single_query_attention_workspace_floats(int n_heads, int head_dim, int max_seq_len);
int kmll_single_query_attention(kmll_stream_t stream, const float* query, const float* key_cache,
                                const float* value_cache, int seq_len, int max_seq_len,
                                int n_heads, int n_kv_heads, int head_dim, float* workspace,
                                float* out);
/* Same operator for hosts that cannot hand over a workspace because they cannot allocate device memory at
 * all: a thread that was given a stream and the operator bindings but no allocator, or a latency-bound loop
 * where a cudaMalloc would stall the whole device.  It has no counterpart in the reference.  The scratch is a
 * fixed 2.08 MiB array inside the library image (every GPU that loads the library holds it until the
 * process exits), so the geometry is limited: kmll_single_query_attention_workspace_floats(n_heads, head_dim,
 * max_seq_len) must not exceed 544768, otherwise KMLL_ERR_CAPACITY is returned and nothing runs.  The entry
 * point calls no allocating routine.  The first call on a device looks up the device address of the array;
 * make that first call outside any stream capture.  All calls on a device share the one array: two calls
 * that overlap on the GPU (different streams) race on it and must be serialised by the caller. */
int kmll_single_query_attention_noalloc(kmll_stream_t stream, const float* query,
                                        const float* key_cache, const float* value_cache,
                                        int seq_len, int max_seq_len, int n_heads, int n_kv_heads,
                                        int head_dim, float* out);
/* prefill_causal_attention, crates/inference/src/ops/inference.rs:1713-1771: row r attends to
 * cache positions 0..=r. */
int kmll_prefill_causal_attention(kmll_stream_t stream, const float* query_batch,
                                  const float* key_cache, const float* value_cache, int prompt_len,
                                  int max_seq_len, int n_heads, int n_kv_heads, int head_dim,
                                  float* out);

/* ------------------------------------------------------------------------------------------
 * Embedding and logit selection
 * ---------------------------------------------------------------------------------------- */
/* embedding / embedding_tokens_bf16, crates/inference/src/ops/inference.rs:562-628 */
int kmll_embedding(kmll_stream_t stream, const uint16_t* table_bf16, int vocab, int dim,
                   uint32_t token, float* out);
int kmll_embedding_tokens(kmll_stream_t stream, const uint16_t* table_bf16, int vocab, int dim,
                          const uint32_t* tokens, int token_count, float* out);
/* argmax_f32_packed, crates/inference/src/ops/inference.rs:1858-1882 */
int kmll_argmax_f32_packed(kmll_stream_t stream, const float* logits, size_t n,
                           uint64_t* packed_out);
/* top_k_f32 (k <= 16), crates/inference/src/ops/inference.rs:1884-1916 */
int kmll_top_k_f32(kmll_stream_t stream, const float* logits, size_t n, int k, uint32_t* tokens,
                   float* values);

#ifdef __cplusplus
}
#endif
#endif /* KMLL_B200_H */
