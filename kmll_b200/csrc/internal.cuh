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

// ---- tensor-parallel exchange over peer memory ------------------------------------------------------
// Replaces the all-reduce after the row-parallel projections (wo, w2) inside the decode step.  The producing
// kernel PUSHES its partial output vector into slot [parity][own rank] of every rank's inbox with plain 8-byte
// stores over NVLink; each store carries one value AND the number of the exchange, so data and "ready" arrive
// in one indivisible word and no fence, flag or completion counter is needed.  The consuming kernel (the next
// RMSNorm + projection, which reads the vector anyway) polls the words of all ranks until they carry the
// expected number - a bounded wait - and adds the partial vectors in rank order, so the sum is deterministic
// and no separate reduction kernel or library collective runs.  The number of exchange i of decode step n is
// n * 128 + i + 1 (monotonic), its parity selects one of two inbox halves.  Two halves suffice: a rank can
// push exchange k+2 only after it consumed k+1, which every rank pushed after consuming k.
constexpr int kMaxTp = 8;
struct TpExchange {  // lives in device memory; entry d of each table is rank d's buffer as mapped into this process
    int tp, rank, dim;
    int mult;                  // exchange numbers are step * mult + index + 1 (index < mult)
    int top_index;             // index of the arg-max hand-over within a step (mult - 1)
    int local_dim;
    int push_mode;             // how the chained kernel publishes words to the ranks: 1 = max-reduction, 2 = plain store
    uint2* inbox[kMaxTp];      // [2][tp][dim] words (value bits, exchange number)
    uint2* top_inbox[kMaxTp];  // [2][tp][2] words (logit bits, number), (token, number): each rank's arg-max
    uint2* local_box;          // [local_dim] words: a vector handed from one phase of the chained kernel to the next on this GPU
    unsigned int* ready[kMaxTp];  // [mult] arrival hints of the inbox exchanges (chained kernel), one table per rank
    unsigned int* ready_local;    // [mult] arrival hints of the local vector
    unsigned int* epoch;       // local: decode steps started (decode_begin increments it)
};
// An exchange word is ONE 64-bit scalar: low half = value bits, high half = exchange number.  It is written with a
// single 64-bit store and read as 64-bit elements, and a naturally aligned 64-bit scalar access is single-copy
// atomic, so a reader can never see the number of one store with the value of another.  (A 2 x 32-bit vector
// access would be two scalar accesses to the memory model, with no such promise.)
__device__ inline void st_exchange_word(uint2* slot, uint32_t value_bits, uint32_t number) {
    const unsigned long long w = ((unsigned long long)number << 32) | (unsigned long long)value_bits;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(slot), "l"(w) : "memory");
}
// The chained kernel publishes its words with a 64-bit MAX reduction instead of a store.  Exchange numbers only grow,
// so the new word (number in the high half) is larger than whatever the slot held and the maximum IS the new word;
// but a reduction is carried out at the L2 cache (or at the peer over NVLink) right away, whereas a relaxed store may
// linger in the multiprocessor's write path for microseconds before anybody can see it (measured: ~3.5 us behind a
// reduction issued after it).  Device scope for words that never leave this GPU.
__device__ inline void push_exchange_word(uint2* slot, uint32_t value_bits, uint32_t number, int mode) {
    const unsigned long long w = ((unsigned long long)number << 32) | (unsigned long long)value_bits;
    if (mode == 1) asm volatile("red.relaxed.sys.global.max.u64 [%0], %1;" ::"l"(slot), "l"(w) : "memory");
    else if (mode == 0) asm volatile("red.relaxed.gpu.global.max.u64 [%0], %1;" ::"l"(slot), "l"(w) : "memory");
    else asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(slot), "l"(w) : "memory");
}
// Polling loads of the chained kernel: plain loads that bypass L1 (.cg), not strong ones.  The words live in this GPU's
// memory, whose point of coherence is the L2 cache, so an L1-bypassing load returns what L2 holds; the number inside
// the word says whether it is the awaited one, and a stale word is simply read again.  Strong loads (relaxed / volatile)
// were measured to complete one after the other within a thread (eight of them: 3.5-4.4 us), plain ones overlap.
__device__ inline uint4 ld_exchange_pair_gpu(const uint4* p) {
    unsigned long long a, b;
    asm volatile("ld.global.cg.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    return make_uint4((uint32_t)a, (uint32_t)(a >> 32), (uint32_t)b, (uint32_t)(b >> 32));
}
// two neighbouring exchange words with one 16-byte request; each 64-bit element is atomic on its own
__device__ inline uint4 ld_exchange_pair(const uint4* p) {
    unsigned long long a, b;
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    return make_uint4((uint32_t)a, (uint32_t)(a >> 32), (uint32_t)b, (uint32_t)(b >> 32));
}
// Deadline clock of the bounded waits: the multiprocessor's own cycle counter.  (The nanosecond %globaltimer is a
// system-wide register whose read takes a good fraction of a microsecond - measured: a wait that read it once before
// polling cost 0.4 us even when the awaited event was already there - so it is kept out of every wait.)
__device__ inline unsigned long long wait_clock_ticks() { return (unsigned long long)clock64(); }
constexpr unsigned long long kPeerWaitLimitTicks = 4000000000ull;  // a peer that is this late (2 to 4 s by the clock rate) is given up on
// ---- chained streaming kernel over prepared W4-G128 records (linear_chain.cuh) -----------------------------
enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SILU = 2, EPI_TOP1 = 3 };
constexpr int kCRecBytes = 2112;   // one prepared record: 32 rows x 128 columns of nibbles + 32 binary16 scales
constexpr int kCRows = 32;         // weight rows per unit
constexpr int kCDepth = 4;         // records in flight per warp (8 KB; 128 KB per block)
constexpr int kCRedBufs = 8;       // units whose partial sums may be pending at once
constexpr int kCMaxPhases = 4;

enum { CHAIN_IN_PLAIN = 0, CHAIN_IN_INBOX = 1, CHAIN_IN_LOCAL = 2 };
enum { CHAIN_OUT_PLAIN = 0, CHAIN_OUT_INBOX = 1, CHAIN_OUT_LOCAL = 2 };

struct ChainPhase {
    const uint8_t* w[3];      // prepared records of up to three matrices; the units of a matrix are consecutive
    float* out[3];            // plain outputs (unused when the output is pushed)
    int out_rows[3];          // valid output rows per matrix (gate/up: rows of the gate matrix)
    int unit_start[4];        // first unit of each matrix; [3] = total
    int total_units;
    int K, ngroups;
    int epi;                  // EPI_STORE / EPI_RESIDUAL / EPI_SILU / EPI_TOP1
    int in_kind, in_index;    // CHAIN_IN_*: plain pointer, rank-ordered sum of inbox exchange in_index, local buffer
    int in_units;             // gathered input produced by an earlier phase of the SAME launch: its units per rank (arrival hint); else 0
    int out_kind, out_index;  // CHAIN_OUT_*
    int residual_index;       // EPI_RESIDUAL: >= 0 takes the residual from the rank-ordered sum of that inbox exchange
    int add_residual;         // 0 on tensor-parallel ranks above 0 (rank 0's partial vector carries the residual)
    const float* x;           // plain input
    float* x_out;             // gathered input: block 0 also stores the summed vector here (may be null)
    const uint16_t* norm_w;   // fused RMSNorm weight or null
    float eps;
    const float* residual;    // plain residual
};

struct ChainParams {
    ChainPhase phase[kCMaxPhases];
    int n_phases;
    int off_corr, off_red, off_bars, off_misc, off_ring, off_sring;  // shared-memory offsets in bytes
    int xs_pitch;             // bytes per digit row (>= max K + 16)
    const TpExchange* xc;     // exchange tables (also on one GPU, where tp == 1 and the inbox is local) or null
    TpExchange xcv;           // their contents, by value (launch_chain copies them): the kernel chases no pointer to find them
    // lm_head arg-max (EPI_TOP1): per-block partials, merged by the block that finishes last
    uint32_t* partial_tokens;
    float* partial_logits;
    uint64_t* packed_out;
    unsigned int* top1_counter;  // zero between launches
    uint32_t token_offset;
    DecodeState* state;       // not null: the merging block also advances the decode state (single GPU)
    int push_top;             // 1: the merging block hands this rank's arg-max to every rank (tensor parallel)
    unsigned long long* trace;
};

// Plans the shared memory of a chain and launches it (every phase: K % 128 == 0, K <= 24576, 16-byte aligned inputs).
int launch_chain(cudaStream_t stream, ChainParams& cp);
size_t w4_prepared_bytes(int rows, int cols, int pair);
int w4_prepare(cudaStream_t stream, const uint8_t* pa, const uint16_t* sa, const uint8_t* pb, const uint16_t* sb, int rows, int cols,
               uint8_t* out);

// Arguments for the NEXT linear launch of this thread (consumed and cleared by it): push the output as exchange
// `push_index` instead of storing it, and / or take the input vector from exchange `gather_index` (writing the
// summed vector to x_out as well).  -1 = off.
void set_exchange_args(const TpExchange* xc, int push_index, int gather_index, float* x_out);
// Publishes this rank's packed arg-max to every rank (top1_reduce does it when xc is given), then
// decode_end_gather waits for all ranks, merges (higher logit, then lower token) and advances the state.
int decode_end_gather(cudaStream_t stream, const TpExchange* xc, DecodeState* state, uint64_t* packed_final);

// attention.cu
int decode_attention_launch(cudaStream_t stream, const float* q, const float* k_cache, const float* v_cache,
                            const int* seq_len_ptr, int seq_len, int seq_cap, int n_heads, int n_kv_heads,
                            int head_dim, float* workspace, float* out, const float* k_new = nullptr,
                            const float* v_new = nullptr, const float* freqs = nullptr, float* k_cache_w = nullptr,
                            float* v_cache_w = nullptr, int batch = 1, size_t cache_stride = 0, int kv_bf16 = 0,
                            int window = 0);
size_t decode_attention_workspace_floats(int n_heads, int head_dim, int seq_cap);

// elementwise.cu
int prepare_incremental_dyn(cudaStream_t stream, const float* q, const float* k, const float* v, const float* freqs,
                            int n_freqs, const DecodeState* state, int max_seq_len, int n_heads, int n_kv_heads,
                            int head_dim, float* q_rot, float* k_cache, float* v_cache, int kv_bf16 = 0);
int qk_head_rmsnorm(cudaStream_t stream, float* q, float* k, const uint16_t* q_w, const uint16_t* k_w, int rows, int n_heads, int n_kv_heads,
                    int head_dim, float eps, size_t q_stride, size_t k_stride);
int prepare_prefill_offset(cudaStream_t stream, const float* q, const float* k, const float* v, const float* freqs,
                           int n_freqs, int rows, int q_len, int kv_len, int head_dim, int position0, float* q_rot,
                           float* k_cache, float* v_cache, int kv_bf16 = 0);
// one row of the KV cache at `position` (f32, or rounded to bf16 when the decoder keeps its cache in bf16)
int write_kv_row(cudaStream_t stream, const float* x, int position, int token_len, int head_dim, float* cache, int kv_bf16);
int prefill_attention_launch(cudaStream_t stream, const float* q_batch, const float* k_cache, const float* v_cache, int prompt_len,
                             int n_heads, int n_kv_heads, int head_dim, float* out, int kv_bf16, int window, int tensor_cores);
// hidden = embedding[state->next_top.token]; also records next_top into history[state->step] and
// sets seq_len = position + 1.
int decode_begin(cudaStream_t stream, const uint16_t* table, int vocab, int dim, DecodeState* state, uint64_t* history,
                 int history_cap, float* hidden, unsigned int* exchange_epoch = nullptr);
// state->next_top = *packed; position += 1; step += 1.
int decode_end(cudaStream_t stream, const uint64_t* packed, DecodeState* state);

// Lockstep batch of sequences: shared position, one pending token per sequence.
constexpr int kMaxBatch = 16;
struct BatchState {
    int position, seq_len, step, pad;
    uint64_t next_top[kMaxBatch];
};
// hidden[b] = embedding[next_top[b].token]; records the tokens into history[b][step]; seq_len = position + 1.
int batch_begin(cudaStream_t stream, const uint16_t* table, int vocab, int dim, int batch, BatchState* state, uint64_t* history,
                int history_cap, float* hidden);
// packed[b] = arg-max of logits[b] (ties -> lower token); next_top[b] = packed[b]; position += 1; step += 1.
int batch_end(cudaStream_t stream, const float* logits, int vocab, int batch, BatchState* state);

// quantize.cu: bf16 bits -> f32 (exact)
int widen_bf16(cudaStream_t stream, const uint16_t* src, size_t n, float* dst);

// linear.cu: lm_head arg-max whose token ids are offset (vocabulary shards of tensor parallelism)
int linear_top1_offset(cudaStream_t stream, int fmt, const float* x, const uint16_t* norm_w, float eps, const void* w,
                       const void* scales, int rows, int cols, uint32_t token_offset, uint32_t* partial_tokens,
                       float* partial_logits, uint64_t* packed_out, const TpExchange* xc = nullptr);
// Batched fused linear forms for rows of x that are independent sequences (batch <= 16 per pass):
// form 0 = RMSNorm + QKV (3 matrices, rows[0..2]), 1 = RMSNorm + gate/up + SiLU*up (2 matrices of rows[0]),
// 2 = projection + residual, 3 = (RMSNorm +) projection.  Outputs are [batch, rows] row-major.
// `workspace` (linear_batched_workspace_bytes(batch, cols) bytes) enables the tensor-core path for 5 or more rows; form 1
// then also needs two [batch, rows] scratch matrices for the gate and up projections.
int linear_batched_form(int form, cudaStream_t stream, int fmt, const float* x, int batch, const uint16_t* norm_w, float eps,
                        const void* const* w, const void* const* scales, const int* rows, int cols, float* const* outs,
                        const float* residual, void* workspace = nullptr, float* gate_tmp = nullptr, float* up_tmp = nullptr);
size_t linear_batched_workspace_bytes(int batch, int in_dim);
// Deterministic merge of per-rank packed results: higher logit wins, ties -> lower token.
int merge_packed_top1(cudaStream_t stream, const uint64_t* packed_all, int n, uint64_t* packed_out);

}  // namespace kmll
