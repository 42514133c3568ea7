/*
 * kmll_b200_runtime.h — C ABI of the decode runtime built on the operators of kmll_b200.h.
 *
 * The runtime is the counterpart of kmll's quantized-weights runtime
 * (MinistralAllLinearInt8Runtime / RuntimeCore, crates/inference/src/model.rs:5151-5166,
 * :6327-6384): resident quantized weights, per-layer f32 KV caches [max_seq, n_kv, head_dim]
 * (crates/inference/src/model.rs:9308-9324), scratch allocated once, `prefill` then greedy
 * generation (generate_greedy_until_i8_top1_from_next, crates/inference/src/model.rs:6021-6106).
 * Differences: the per-token work is captured once in a CUDA graph and replayed; the next token
 * stays on the device between steps (kmll reads it back every token,
 * crates/inference/src/model.rs:10655); tensor parallelism over several GPUs is supported.
 *
 * All functions return 0 or a KMLL_ERR_* code (kmll_b200.h); kmll_last_error() has the message.
 * A decoder belongs to the CUDA device that was current when it was created and must be used
 * from one thread at a time.
 */
#ifndef KMLL_B200_RUNTIME_H
#define KMLL_B200_RUNTIME_H

#include <stddef.h>
#include <stdint.h>

#include "kmll_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void* kmll_decoder_t;

enum { KMLL_FORMAT_RS_I8 = 0, KMLL_FORMAT_W4G128 = 1 };

/* Tensor ids for kmll_decoder_*_tensor.  Linear weights are [out_features, in_features]
 * (crates/inference/src/model.rs:8711-8760); names follow kmll's layer fields. */
enum {
    KMLL_T_ATTENTION_NORM = 0, /* bf16 [dim] */
    KMLL_T_WQ = 1,             /* [n_heads*head_dim, dim] */
    KMLL_T_WK = 2,             /* [n_kv_heads*head_dim, dim] */
    KMLL_T_WV = 3,
    KMLL_T_WO = 4,             /* [dim, n_heads*head_dim] */
    KMLL_T_FFN_NORM = 5,       /* bf16 [dim] */
    KMLL_T_W1 = 6,             /* gate [hidden_dim, dim] */
    KMLL_T_W3 = 7,             /* up   [hidden_dim, dim] */
    KMLL_T_W2 = 8,             /* down [dim, hidden_dim] */
    KMLL_T_FINAL_NORM = 9,     /* bf16 [dim]            (layer = -1) */
    KMLL_T_EMBEDDING = 10,     /* bf16 [vocab, dim]     (layer = -1) */
    KMLL_T_OUTPUT = 11,        /* lm_head [vocab, dim]  (layer = -1) */
    KMLL_T_Q_NORM = 12,        /* optional, bf16 [head_dim]: per-head RMSNorm of the query rows before RoPE (model.rs:10165-10194); */
    KMLL_T_K_NORM = 13         /* same for the key rows.  Set them before the first decode step; a model without them sets neither. */
};

/* TextConfig of kmll (crates/inference/src/model.rs:271-366) reduced to what the decoder path uses. */
typedef struct {
    int n_layers;
    int dim;
    int n_heads;
    int n_kv_heads;
    int head_dim;
    int hidden_dim;
    int vocab_size;
    int rotary_dim; /* <= head_dim, even */
    float rope_theta;
    float norm_eps;
    int max_seq_len;
    int format;   /* KMLL_FORMAT_* */
    int fused;    /* 1: fused kernels (RMSNorm+QKV, gate*up, +residual, lm_head arg-max); 0: one
                     launch per kmll operator, in kmll's order (crates/inference/src/model.rs:10102-10300) */
    int tp_rank;  /* tensor parallel rank / size; 0 / 1 for a single GPU */
    int tp_size;
    int kv_bf16;  /* 1: the KV cache holds bf16 (rounded to nearest-even when a row is written) instead of kmll's f32 rows
                     (crates/inference/src/model.rs:10160-10186 writes f32): half the cache bytes and half the attention
                     traffic, results no longer bit-equal to kmll's. */
    int sliding_window;  /* > 0: every position attends only the last `sliding_window` positions (itself included), the
                            mask of Mistral-style checkpoints; 0: full causal attention, which is all kmll implements
                            (crates/inference/src/kernels/inference.rs:1420-1686).  The cache still keeps every row. */
} kmll_decoder_config;

/* sizeof(kmll_decoder_config) as this library was compiled: a binding checks its own mirror of the struct against it
   (fields are only ever appended) */
size_t kmll_decoder_config_bytes(void);
int kmll_decoder_create(const kmll_decoder_config* config, kmll_decoder_t* out);
int kmll_decoder_destroy(kmll_decoder_t dec);

/* Random-init weights, generated and quantized on the device: linear weights ~ N(0, std) (rounded to
 * bf16 first for RS-I8, as kmll quantizes bf16 checkpoints), embeddings ~ N(0, std) bf16, norm
 * weights 1.  With tie_embeddings != 0 the output matrix is the quantized embedding table.  Under
 * tensor parallelism every rank generates the full tensor with the same seed and keeps its shard,
 * so shards are slices of the single-GPU tensors. */
int kmll_decoder_init_random(kmll_decoder_t dec, uint64_t seed, float std, int tie_embeddings);

/* Upload one tensor from host memory: bf16 bits for norms/embedding; for linear weights the
 * already quantized parts (RS-I8: int8 values + float scales; W4-G128: packed bytes + binary16
 * group scales).  Full (unsharded) tensors; the decoder keeps its tensor-parallel shard. */
int kmll_decoder_set_tensor(kmll_decoder_t dec, int layer, int tensor, const void* values,
                            const void* scales);
/* Download this rank's shard of a tensor to host memory (sizes as uploaded; tp_size == 1 gives the
 * full tensor).  Either pointer may be null. */
int kmll_decoder_get_tensor(kmll_decoder_t dec, int layer, int tensor, void* values, void* scales);

/* Tensor parallelism over NCCL.  Rank 0 obtains an id, the caller distributes the 128 bytes to all
 * ranks (any transport), then every rank calls kmll_decoder_tp_init with the same id. */
int kmll_tp_unique_id(unsigned char id_out[128]);
int kmll_decoder_tp_init(kmll_decoder_t dec, const unsigned char id[128]);

/* prefill (crates/inference/src/model.rs:5945-5968): runs the prompt through the batched path,
 * fills the KV caches and leaves the arg-max of the last position ready.  Resets the sequence. */
int kmll_decoder_prefill(kmll_decoder_t dec, kmll_stream_t stream, const uint32_t* tokens_host,
                         int n_tokens);
/* Same result through the per-token decode path (prefill_token_loop_reference,
 * crates/inference/src/model.rs:6393-6395). */
int kmll_decoder_prefill_token_loop(kmll_decoder_t dec, kmll_stream_t stream,
                                    const uint32_t* tokens_host, int n_tokens);

/* Greedy generation: n_steps tokens, each step = forward of the pending token + lm_head arg-max.
 * The whole step is one CUDA graph; tokens never leave the device during the loop.  On return
 * tokens_out[i] / logits_out[i] hold token and logit of step i (GreedyGenerationStep,
 * crates/inference/src/model.rs:6072-6077).  Synchronises the stream at the end. */
int kmll_decoder_generate_greedy(kmll_decoder_t dec, kmll_stream_t stream, int n_steps,
                                 uint32_t* tokens_out, float* logits_out);
/* The same steps without waiting and without reading anything back (timing loops). */
int kmll_decoder_enqueue_steps(kmll_decoder_t dec, kmll_stream_t stream, int n_steps);
/* The device keeps the packed (logit, token) of every step since the last prefill / rewind / generate_greedy:
 * packed_out[i] = entry first + i (the token step first + i consumed).  Lets a timing loop built on
 * kmll_decoder_enqueue_steps check afterwards what it generated.  Synchronises the stream. */
int kmll_decoder_history(kmll_decoder_t dec, kmll_stream_t stream, int first, int count, uint64_t* packed_out);
/* One step the way kmll's host loop does it: the token comes from host memory, the packed
 * (logit, token) result is copied back and the stream is synchronised
 * (crates/inference/src/model.rs:10655).  *packed_out = (f32 bits << 32) | next token. */
int kmll_decoder_step_host(kmll_decoder_t dec, kmll_stream_t stream, uint32_t token,
                           uint64_t* packed_out);

/* Pending next token (arg-max of the last logits) as packed (f32 bits << 32) | token; synchronises. */
int kmll_decoder_next_top(kmll_decoder_t dec, kmll_stream_t stream, uint64_t* packed_out);
/* Truncate the sequence to `position` tokens (<= current position); the pending token is kept.  Used to
 * replay the same positions again (timing legs, speculative roll-back). */
int kmll_decoder_rewind(kmll_decoder_t dec, kmll_stream_t stream, int position);
/* Replace the pending token (packed (f32 bits << 32) | token) that the next step will consume; with kmll_decoder_rewind
 * this replays a recorded continuation from an earlier position. */
int kmll_decoder_set_pending(kmll_decoder_t dec, kmll_stream_t stream, uint64_t packed);
/* Number of tokens in the sequence (= next position). */
int kmll_decoder_position(kmll_decoder_t dec);
/* Final hidden state of the last forward [dim] to host (parity checks); synchronises. */
int kmll_decoder_last_hidden(kmll_decoder_t dec, kmll_stream_t stream, float* hidden_out);
/* Replace the RoPE frequency table (rotary_dim / 2 host values), e.g. with YaRN-scaled frequencies
 * (yarn_rope_frequencies, crates/inference/src/model.rs:9257-9306).  Synchronises the device. */
int kmll_decoder_set_rope_freqs(kmll_decoder_t dec, const float* freqs_host, int count);
/* Next-token logits [vocab_size] of the sequence as it stands (final RMSNorm + lm_head over the last hidden state) into a
 * DEVICE buffer of the caller; enqueues only.  Replaces what next_logits_to_host / next_top_logits start from
 * (crates/inference/src/model.rs:5319-5352).  One GPU only (a tensor-parallel rank holds a slice of the vocabulary). */
int kmll_decoder_next_logits(kmll_decoder_t dec, kmll_stream_t stream, float* logits_device);
/* Kernel launches per decode step; bytes of weights / KV cache resident on this rank; bytes of every device allocation of
 * the decoder (weights + KV cache + scratch: RuntimeMemoryStats, crates/inference/src/model.rs:803-808,5368-5391). */
int kmll_decoder_launches_per_step(kmll_decoder_t dec);
size_t kmll_decoder_weight_bytes(kmll_decoder_t dec);
size_t kmll_decoder_kv_bytes(kmll_decoder_t dec);
size_t kmll_decoder_resident_bytes(kmll_decoder_t dec);

/* ---- on-disk archive of the quantized linear weights ---------------------------------------------------------
 * The directory layout of kmll's quantization export, so an archive written by either side loads on the other:
 *   manifest.json with "quantization": "row-symmetric-int8-with-f32-row-scales" (crates/inference/src/model.rs:9047-9053),
 *   NNNN_<name>.i8 (raw int8, row-major) and NNNN_<name>.scales.f32 (little-endian f32) per tensor, where <name> has
 *   every non-alphanumeric character replaced by '_' (crates/inference/src/rowwise_scaled.rs:141-157) and NNNN is the
 *   tensor index: 0 = output.weight, 1 + layer * 7 + offset for wq, wk, wv, wo, w1, w3, w2
 *   (crates/inference/src/model.rs:9082-9140, :9185-9187).
 * W4-G128 archives (no counterpart in kmll) use the manifest value "group128-symmetric-int4-with-f16-group-scales" and
 * the suffixes .w4 (packed nibbles) / .gscales.f16.  Host functions; `values` / `scales` are HOST pointers.
 * Norm weights and embeddings are not part of kmll's archive (they stay in the checkpoint). */
int kmll_archive_tensor_index(int layer, int offset); /* layer < 0: 0 (output.weight); exported_int8_layer_tensor_index */
int kmll_archive_file_paths(const char* dir, int index, const char* name, int format, char* values_path, char* scales_path,
                            size_t capacity);
int kmll_archive_write_tensor(const char* dir, int index, const char* name, int format, int rows, int cols,
                              const void* values, const void* scales);
/* RowwiseScaledI8Matrix::read_exported (rowwise_scaled.rs:94-106): fails unless both files have exactly the bytes of
 * a rows x cols tensor. */
int kmll_archive_read_tensor(const char* dir, int index, const char* name, int format, int rows, int cols, void* values,
                             void* scales);
int kmll_archive_write_manifest(const char* dir, const kmll_decoder_config* config, const char* weights_path);
/* validate_all_linear_int8_export_archive (crates/inference/src/model.rs:8984-9035): directory, manifest key, byte
 * length of every expected file; with expected_weights_path also the manifest's weights_path. */
int kmll_archive_validate(const char* dir, const kmll_decoder_config* config, const char* expected_weights_path);
/* Write every linear tensor of a single-GPU decoder + the manifest / validate an archive and upload it (new_from_export,
 * crates/inference/src/model.rs:6327-6384); `config` is the configuration the decoder was created with. */
int kmll_decoder_export_archive(kmll_decoder_t dec, const kmll_decoder_config* config, const char* dir, const char* weights_path);
int kmll_decoder_load_archive(kmll_decoder_t dec, const kmll_decoder_config* config, const char* dir,
                              const char* expected_weights_path);

/* ---- lockstep batch of sequences (new; kmll decodes one sequence at a time) -------------------------
 * Up to 16 independent sequences at the same position are decoded together so that every weight is read
 * once per step for all of them.  The batch shares the decoder's weights and owns its KV caches
 * ([batch] x the decoder's cache size).  Each sequence is prefilled with the ordinary decoder and then
 * adopted into a slot (its KV rows and pending token are copied); all sequences must be at the same
 * position.  Single GPU, rotary_dim == head_dim.  The per-sequence results equal those of the
 * single-sequence decoder up to the rounding of the batched linear kernel. */
typedef void* kmll_batch_t;
int kmll_batch_create(kmll_decoder_t dec, int batch, kmll_batch_t* out);
int kmll_batch_destroy(kmll_batch_t batch);
int kmll_batch_adopt(kmll_batch_t batch, kmll_stream_t stream, int slot);
/* n_steps greedy tokens for every sequence: tokens_out / logits_out are [batch][n_steps]. */
int kmll_batch_generate_greedy(kmll_batch_t batch, kmll_stream_t stream, int n_steps, uint32_t* tokens_out,
                               float* logits_out);
int kmll_batch_enqueue_steps(kmll_batch_t batch, kmll_stream_t stream, int n_steps);
int kmll_batch_position(kmll_batch_t batch);
int kmll_batch_launches_per_step(kmll_batch_t batch);

#ifdef __cplusplus
}
#endif
#endif /* KMLL_B200_RUNTIME_H */
