// Functions shared between translation units of libkmll_b200 that are not part of the C ABI:
// operator variants whose position / token operand lives in device memory, so that one captured
// CUDA graph stays valid while the sequence grows.
#pragma once

#include "common.cuh"

namespace kmll {

// Device-resident state of a decode loop.
struct DecodeState {
    int position;        // number of tokens in the KV caches = position of the token being processed
    int seq_len;         // position + 1 while a step runs (attention length)
    int step;            // steps generated so far (index into history)
    int pad;
    uint64_t next_top;   // packed (f32 bits << 32) | token of the pending token
};

// attention.cu
int decode_attention_launch(cudaStream_t stream, const float* q, const float* k_cache, const float* v_cache,
                            const int* seq_len_ptr, int seq_len, int seq_cap, int n_heads, int n_kv_heads,
                            int head_dim, float* workspace, float* out, const float* k_new = nullptr,
                            const float* v_new = nullptr, const float* freqs = nullptr, float* k_cache_w = nullptr,
                            float* v_cache_w = nullptr);
size_t decode_attention_workspace_floats(int n_heads, int head_dim, int seq_cap);

// elementwise.cu
int prepare_incremental_dyn(cudaStream_t stream, const float* q, const float* k, const float* v, const float* freqs,
                            int n_freqs, const DecodeState* state, int max_seq_len, int n_heads, int n_kv_heads,
                            int head_dim, float* q_rot, float* k_cache, float* v_cache);
int prepare_prefill_offset(cudaStream_t stream, const float* q, const float* k, const float* v, const float* freqs,
                           int n_freqs, int rows, int q_len, int kv_len, int head_dim, int position0, float* q_rot,
                           float* k_cache, float* v_cache);
// hidden = embedding[state->next_top.token]; also records next_top into history[state->step] and
// sets seq_len = position + 1.
int decode_begin(cudaStream_t stream, const uint16_t* table, int vocab, int dim, DecodeState* state, uint64_t* history,
                 int history_cap, float* hidden);
// state->next_top = *packed; position += 1; step += 1.
int decode_end(cudaStream_t stream, const uint64_t* packed, DecodeState* state);

// quantize.cu: bf16 bits -> f32 (exact)
int widen_bf16(cudaStream_t stream, const uint16_t* src, size_t n, float* dst);

// linear.cu: lm_head arg-max whose token ids are offset (vocabulary shards of tensor parallelism)
int linear_top1_offset(cudaStream_t stream, int fmt, const float* x, const uint16_t* norm_w, float eps, const void* w,
                       const void* scales, int rows, int cols, uint32_t token_offset, uint32_t* partial_tokens,
                       float* partial_logits, uint64_t* packed_out);
// Deterministic merge of per-rank packed results: higher logit wins, ties -> lower token.
int merge_packed_top1(cudaStream_t stream, const uint64_t* packed_all, int n, uint64_t* packed_out);

}  // namespace kmll
