// Decode runtime: resident quantized weights, f32 KV caches, scratch, batched prefill, and a greedy
// decode loop whose per-token work is one CUDA graph with the next token kept on the device.
// Counterpart of kmll's RuntimeCore / MinistralAllLinearInt8Runtime
// (crates/inference/src/model.rs:5151-5166, :6327-6384) built on this library's own C ABI operators:
// every launch below goes through the same entry points an external host would bind.
#include <dlfcn.h>
#include <nccl.h>

#include <cmath>
#include <cstring>
#include <vector>

#include "../../include/kmll_b200_runtime.h"
#include "internal.cuh"

namespace kmll {

#define KMLL_TRY(expr)                 \
    do {                               \
        int rc__ = (expr);             \
        if (rc__ != KMLL_OK) return rc__; \
    } while (0)

#define KMLL_CUDA(expr)                                                                        \
    do {                                                                                       \
        cudaError_t e__ = (expr);                                                              \
        if (e__ != cudaSuccess) return fail(KMLL_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

// ---- NCCL, loaded on first use (single-GPU users need no NCCL at all) ------------------------------
struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

static NcclApi* nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (api.handle != nullptr) {
            api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(api.handle, "ncclGetUniqueId"));
            api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(api.handle, "ncclCommInitRank"));
            api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(api.handle, "ncclCommDestroy"));
            api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(api.handle, "ncclAllReduce"));
            api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(api.handle, "ncclAllGather"));
            api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(api.handle, "ncclGetErrorString"));
        }
    }
    if (api.handle == nullptr || api.GetUniqueId == nullptr || api.CommInitRank == nullptr || api.AllReduce == nullptr ||
        api.AllGather == nullptr)
        return nullptr;
    return &api;
}

struct QWeight {
    void* w = nullptr;       // int8 values or packed nibbles
    void* scales = nullptr;  // float[rows] or half[rows, cols/128]
    int rows = 0, cols = 0;  // local (sharded) shape
    uint8_t* prep = nullptr;  // W4-G128: the same values in the prepared layout the batch-1 kernels stream
};

struct Layer {
    uint16_t* attention_norm = nullptr;
    uint16_t* q_norm = nullptr;  // optional per-head RMSNorm weights [head_dim] of the query / key rows (null: the model has none)
    uint16_t* k_norm = nullptr;
    uint16_t* ffn_norm = nullptr;
    QWeight wq, wk, wv, wo, w1, w3, w2;
    uint8_t* w13_prep = nullptr;  // W4-G128: gate (w1) and up (w3) interleaved in the prepared layout
    float* key_cache = nullptr;
    float* value_cache = nullptr;
};

enum ShardKind { SHARD_NONE, SHARD_ROWS, SHARD_COLS };

struct Decoder {
    kmll_decoder_config cfg;
    int device = 0;
    int n_heads_l = 0, n_kv_l = 0, hidden_l = 0, vocab_l = 0;  // per-rank sizes
    std::vector<Layer> layers;
    uint16_t* final_norm = nullptr;
    uint16_t* embedding = nullptr;
    QWeight output;
    float* freqs = nullptr;
    // per-token scratch (crates/inference/src/model.rs:9339-9498 allocates the same set once)
    float *hidden_a = nullptr, *hidden_b = nullptr, *hidden_mid = nullptr;
    float *normed = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *q_rot = nullptr, *k_rot = nullptr;
    float *attn = nullptr, *delta = nullptr, *gate = nullptr, *up = nullptr, *act = nullptr;
    float* attn_ws = nullptr;
    uint32_t* part_tok = nullptr;
    float* part_logit = nullptr;
    uint64_t* packed = nullptr;      // this rank's arg-max
    uint64_t* packed_all = nullptr;  // [tp_size]
    uint64_t* packed_final = nullptr;
    DecodeState* state = nullptr;
    uint64_t* history = nullptr;
    int history_cap = 0;
    uint64_t* pinned = nullptr;  // host, pinned
    int host_position = 0;
    bool have_next = false;
    bool warmed = false;
    cudaGraphExec_t graph = nullptr;
    unsigned long long graph_trace_generation = 0;  // trace_generation() when `graph` was captured
    cudaStream_t capture_stream = nullptr;  // the caller's stream may be the legacy default stream, which cannot capture
    ncclComm_t comm = nullptr;
    // peer-memory exchange (tensor parallel decode step); null = NCCL collectives
    TpExchange* xc = nullptr;          // device copy of the tables
    TpExchange xc_host;                // the same tables on the host (the chained kernel takes them by value)
    void* xc_local = nullptr;          // this rank's exchange buffer (shared with the peers through CUDA IPC)
    unsigned int* xc_epoch = nullptr;  // inside xc_local
    void* xc_peer_base[kMaxTp] = {};   // peers' buffers as mapped here (null for the own rank)
    std::vector<void*> allocs;
    size_t weight_bytes = 0, kv_bytes = 0, resident_bytes = 0;  // resident = every device allocation of this decoder
    int launches_per_step = 0;
    bool weights_set = false;
    // chained decode step (W4-G128, fused): prepared weights, exchange words also on a single GPU
    bool chain = false;            // the decode step runs linear_chain_kernel
    bool chain_split = true;       // ... one launch per projection (default) instead of one launch per layer (KMLL_CHAIN=layer)
    bool chain_words = false;      // one GPU, one launch per projection: still hand the vectors over as exchange words (KMLL_CHAIN=words)
    bool prepared_valid = false;   // the prepared buffers match the canonical tensors
    unsigned int* top1_counter = nullptr;
};

template <typename T>
static int dalloc(Decoder* d, T** out, size_t count) {
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, count * sizeof(T) + 16);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "cudaMalloc(%zu bytes): %s", count * sizeof(T), cudaGetErrorString(e));
    d->allocs.push_back(p);
    d->resident_bytes += count * sizeof(T);
    *out = static_cast<T*>(p);
    return KMLL_OK;
}

static size_t qweight_bytes(int fmt, int rows, int cols, size_t* scale_bytes) {
    if (fmt == KMLL_FORMAT_W4G128) {
        *scale_bytes = (size_t)rows * (cols / 128) * 2;
        return (size_t)rows * cols / 2;
    }
    *scale_bytes = (size_t)rows * 4;
    return (size_t)rows * cols;
}

static int alloc_qweight(Decoder* d, QWeight* w, int rows, int cols) {
    size_t sb = 0;
    const size_t wb = qweight_bytes(d->cfg.format, rows, cols, &sb);
    uint8_t* pw = nullptr;
    uint8_t* ps = nullptr;
    KMLL_TRY(dalloc(d, &pw, wb));
    KMLL_TRY(dalloc(d, &ps, sb));
    w->w = pw;
    w->scales = ps;
    w->rows = rows;
    w->cols = cols;
    d->weight_bytes += wb + sb;
    return KMLL_OK;
}

static int validate_config(const kmll_decoder_config& c) {
    if (c.n_layers <= 0 || c.dim <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.head_dim <= 0 || c.hidden_dim <= 0 ||
        c.vocab_size <= 0 || c.max_seq_len <= 0)
        return fail(KMLL_ERR_SHAPE, "decoder config: every size must be positive");
    if (c.n_heads % c.n_kv_heads != 0) return fail(KMLL_ERR_SHAPE, "decoder config: n_heads must be divisible by n_kv_heads");
    if (c.head_dim != 64 && c.head_dim != 128) return fail(KMLL_ERR_UNSUPPORTED, "decoder config: head_dim must be 64 or 128");
    if (c.n_heads / c.n_kv_heads > 8) return fail(KMLL_ERR_UNSUPPORTED, "decoder config: at most 8 query heads per KV head");
    if (c.rotary_dim <= 0 || c.rotary_dim > c.head_dim || (c.rotary_dim & 1))
        return fail(KMLL_ERR_SHAPE, "decoder config: rotary_dim must be even and within head_dim");
    if (c.format != KMLL_FORMAT_RS_I8 && c.format != KMLL_FORMAT_W4G128) return fail(KMLL_ERR_SHAPE, "decoder config: unknown format");
    const int unit = c.format == KMLL_FORMAT_W4G128 ? 128 : 64;
    if (c.tp_size < 1 || c.tp_rank < 0 || c.tp_rank >= c.tp_size) return fail(KMLL_ERR_SHAPE, "decoder config: bad tensor-parallel rank/size");
    if (c.n_kv_heads % c.tp_size != 0 || c.hidden_dim % c.tp_size != 0 || c.vocab_size % c.tp_size != 0)
        return fail(KMLL_ERR_SHAPE, "decoder config: n_kv_heads, hidden_dim and vocab_size must be divisible by tp_size");
    if (c.dim % unit != 0 || ((c.n_heads / c.tp_size) * c.head_dim) % unit != 0 || (c.hidden_dim / c.tp_size) % unit != 0)
        return fail(KMLL_ERR_SHAPE, "decoder config: every (sharded) input dimension must be a multiple of %d", unit);
    if (c.kv_bf16 != 0 && c.kv_bf16 != 1) return fail(KMLL_ERR_SHAPE, "decoder config: kv_bf16 must be 0 or 1");
    if (c.sliding_window < 0) return fail(KMLL_ERR_SHAPE, "decoder config: sliding_window must be 0 (off) or a positive number of positions");
    return KMLL_OK;
}

static int tp_allreduce(Decoder* d, cudaStream_t s, float* buf, size_t count) {
    if (d->cfg.tp_size == 1) return KMLL_OK;
    NcclApi* api = nccl_api();
    if (api == nullptr || d->comm == nullptr) return fail(KMLL_ERR_STATE, "tensor parallel decoder used before kmll_decoder_tp_init");
    ncclResult_t r = api->AllReduce(buf, buf, count, ncclFloat, ncclSum, d->comm, s);
    if (r != ncclSuccess) return fail(KMLL_ERR_CUDA, "ncclAllReduce: %s", api->GetErrorString ? api->GetErrorString(r) : "error");
    return KMLL_OK;
}

// ---- linear dispatch on the decoder's format ------------------------------------------------------
static int op_linear(Decoder* d, cudaStream_t s, const float* x, const QWeight& w, float* y) {
    if (d->cfg.format == KMLL_FORMAT_W4G128)
        return kmll_linear_w4g128(s, x, (const uint8_t*)w.w, (const uint16_t*)w.scales, w.rows, w.cols, y);
    return kmll_linear_i8(s, x, (const int8_t*)w.w, (const float*)w.scales, w.rows, w.cols, y);
}
static int op_linear_residual(Decoder* d, cudaStream_t s, const float* x, const QWeight& w, const float* res, float* y) {
    if (d->cfg.format == KMLL_FORMAT_W4G128)
        return kmll_linear_residual_w4g128(s, x, (const uint8_t*)w.w, (const uint16_t*)w.scales, res, w.rows, w.cols, y);
    return kmll_linear_residual_i8(s, x, (const int8_t*)w.w, (const float*)w.scales, res, w.rows, w.cols, y);
}
static int op_linear_batched(Decoder* d, cudaStream_t s, const float* x, const QWeight& w, int batch, void* workspace, float* y) {
    if (d->cfg.format == KMLL_FORMAT_W4G128)
        return kmll_linear_batched_w4g128(s, x, (const uint8_t*)w.w, (const uint16_t*)w.scales, batch, w.cols, w.rows, workspace, y);
    return kmll_linear_batched_i8(s, x, (const int8_t*)w.w, (const float*)w.scales, batch, w.cols, w.rows, workspace, y);
}

// Per-head q/k RMSNorm between the projections and RoPE (crates/inference/src/model.rs:10165-10194); nothing is launched for
// a model without these weights.
static int apply_qk_norm(Decoder* d, cudaStream_t s, const Layer& L, float* q, float* k, int rows) {
    const kmll_decoder_config& c = d->cfg;
    return qk_head_rmsnorm(s, q, k, L.q_norm, L.k_norm, rows, d->n_heads_l, d->n_kv_l, c.head_dim, c.norm_eps, (size_t)d->n_heads_l * c.head_dim,
                           (size_t)d->n_kv_l * c.head_dim);
}

// Row-parallel projection followed by the residual add; under tensor parallelism rank 0 adds the
// residual in its epilogue and the partial sums meet in an all-reduce.
// With push_index >= 0 the partial vector goes to every rank's inbox instead (peer-memory exchange) and the kernel
// that consumes it does the sum.
static int row_parallel_residual(Decoder* d, cudaStream_t s, const float* x, const QWeight& w, const float* residual, float* out,
                                 int push_index = -1) {
    if (push_index >= 0) set_exchange_args(d->xc, push_index, -1, nullptr);
    if (d->cfg.tp_size == 1 || d->cfg.tp_rank == 0) {
        KMLL_TRY(op_linear_residual(d, s, x, w, residual, out));
    } else {
        KMLL_TRY(op_linear(d, s, x, w, out));
    }
    if (push_index >= 0) return KMLL_OK;
    return tp_allreduce(d, s, out, (size_t)w.rows);
}

// lm_head arg-max of `hidden` into d->packed_final (and the decode state is NOT touched).
// With gather_index >= 0 (peer-memory exchange) the hidden state is first summed from the ranks' partial vectors
// (and written to `hidden_out`), and this rank's result is pushed to every rank for decode_end_gather.
static int output_top1(Decoder* d, cudaStream_t s, const float* hidden, int gather_index = -1, float* hidden_out = nullptr) {
    const kmll_decoder_config& c = d->cfg;
    const uint32_t offset = (uint32_t)(c.tp_rank * d->vocab_l);
    uint64_t* dst = c.tp_size == 1 ? d->packed_final : d->packed;
    if (gather_index >= 0) {
        set_exchange_args(d->xc, -1, gather_index, hidden_out);
        return linear_top1_offset(s, c.format, hidden, d->final_norm, c.norm_eps, d->output.w, d->output.scales, d->vocab_l, c.dim,
                                  offset, d->part_tok, d->part_logit, dst, d->xc);
    }
    if (c.fused) {
        KMLL_TRY(linear_top1_offset(s, c.format, hidden, d->final_norm, c.norm_eps, d->output.w, d->output.scales, d->vocab_l, c.dim,
                                    offset, d->part_tok, d->part_logit, dst));
    } else {
        KMLL_TRY(kmll_rmsnorm(s, hidden, d->final_norm, c.dim, c.norm_eps, d->normed));
        KMLL_TRY(linear_top1_offset(s, c.format, d->normed, nullptr, 0.0f, d->output.w, d->output.scales, d->vocab_l, c.dim, offset,
                                    d->part_tok, d->part_logit, dst));
    }
    if (c.tp_size > 1) {
        NcclApi* api = nccl_api();
        if (api == nullptr || d->comm == nullptr) return fail(KMLL_ERR_STATE, "tensor parallel decoder used before kmll_decoder_tp_init");
        ncclResult_t r = api->AllGather(d->packed, d->packed_all, 1, ncclUint64, d->comm, s);
        if (r != ncclSuccess) return fail(KMLL_ERR_CUDA, "ncclAllGather failed");
        KMLL_TRY(merge_packed_top1(s, d->packed_all, c.tp_size, d->packed_final));
    }
    return KMLL_OK;
}

// One decode step with every position-dependent operand read from the device state (graph-safe).
static int enqueue_step_fused(Decoder* d, cudaStream_t s, int* launches) {
    const kmll_decoder_config& c = d->cfg;
    const int q_len = d->n_heads_l * c.head_dim, kv_len = d->n_kv_l * c.head_dim;
    const bool peer = d->xc != nullptr;  // tensor parallel with the peer-memory exchange (no library collective in the step)
    int n = 0;
    KMLL_TRY(decode_begin(s, d->embedding, c.vocab_size, c.dim, d->state, d->history, d->history_cap, d->hidden_a,
                          peer ? d->xc_epoch : nullptr));
    ++n;
    float* hidden = d->hidden_a;
    float* other = d->hidden_b;
    const bool w4 = c.format == KMLL_FORMAT_W4G128;
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = d->layers[l];
        // peer exchange: the hidden state of layers > 0 is still spread over the ranks' inboxes (exchange 2l-1);
        // the QKV kernel sums it while staging and writes it to `hidden`
        if (peer && l > 0) set_exchange_args(d->xc, -1, 2 * l - 1, hidden);
        if (w4) {
            KMLL_TRY(kmll_rmsnorm_linear_triple_w4g128(s, hidden, L.attention_norm, c.norm_eps, (const uint8_t*)L.wq.w,
                                                       (const uint16_t*)L.wq.scales, (const uint8_t*)L.wk.w, (const uint16_t*)L.wk.scales,
                                                       (const uint8_t*)L.wv.w, (const uint16_t*)L.wv.scales, q_len, kv_len, c.dim, d->q,
                                                       d->k, d->v));
        } else {
            KMLL_TRY(kmll_rmsnorm_linear_triple_i8(s, hidden, L.attention_norm, c.norm_eps, (const int8_t*)L.wq.w, (const float*)L.wq.scales,
                                                   (const int8_t*)L.wk.w, (const float*)L.wk.scales, (const int8_t*)L.wv.w,
                                                   (const float*)L.wv.scales, q_len, kv_len, c.dim, d->q, d->k, d->v));
        }
        ++n;
        if (L.q_norm != nullptr || L.k_norm != nullptr) { KMLL_TRY(apply_qk_norm(d, s, L, d->q, d->k, 1)); ++n; }
        if (c.rotary_dim == c.head_dim) {
            // RoPE of q and of the new K row and the KV-cache write happen inside the attention kernel
            KMLL_TRY(decode_attention_launch(s, d->q, L.key_cache, L.value_cache, &d->state->seq_len, 0, c.max_seq_len, d->n_heads_l,
                                             d->n_kv_l, c.head_dim, d->attn_ws, d->attn, d->k, d->v, d->freqs, L.key_cache, L.value_cache, 1, 0, c.kv_bf16,
                                             c.sliding_window));
            ++n;
        } else {
            KMLL_TRY(prepare_incremental_dyn(s, d->q, d->k, d->v, d->freqs, c.rotary_dim / 2, d->state, c.max_seq_len, d->n_heads_l,
                                             d->n_kv_l, c.head_dim, d->q_rot, L.key_cache, L.value_cache, c.kv_bf16));
            KMLL_TRY(decode_attention_launch(s, d->q_rot, L.key_cache, L.value_cache, &d->state->seq_len, 0, c.max_seq_len, d->n_heads_l,
                                             d->n_kv_l, c.head_dim, d->attn_ws, d->attn, nullptr, nullptr, nullptr, nullptr, nullptr, 1, 0,
                                             c.kv_bf16, c.sliding_window));
            n += 2;
        }
        KMLL_TRY(row_parallel_residual(d, s, d->attn, L.wo, hidden, d->hidden_mid, peer ? 2 * l : -1));
        if (peer) set_exchange_args(d->xc, -1, 2 * l, d->hidden_mid);
        if (w4) {
            KMLL_TRY(kmll_rmsnorm_silu_gate_up_w4g128(s, d->hidden_mid, L.ffn_norm, c.norm_eps, (const uint8_t*)L.w1.w,
                                                      (const uint16_t*)L.w1.scales, (const uint8_t*)L.w3.w, (const uint16_t*)L.w3.scales,
                                                      d->hidden_l, c.dim, d->act));
        } else {
            KMLL_TRY(kmll_rmsnorm_silu_gate_up_i8(s, d->hidden_mid, L.ffn_norm, c.norm_eps, (const int8_t*)L.w1.w, (const float*)L.w1.scales,
                                                  (const int8_t*)L.w3.w, (const float*)L.w3.scales, d->hidden_l, c.dim, d->act));
        }
        KMLL_TRY(row_parallel_residual(d, s, d->act, L.w2, d->hidden_mid, other, peer ? 2 * l + 1 : -1));
        n += 3 + ((c.tp_size > 1 && !peer) ? 2 : 0);
        float* t = hidden;
        hidden = other;
        other = t;
    }
    if (peer) {
        KMLL_TRY(output_top1(d, s, hidden, 2 * c.n_layers - 1, hidden));
        KMLL_TRY(decode_end_gather(s, d->xc, d->state, d->packed_final));
        n += 3;
    } else {
        KMLL_TRY(output_top1(d, s, hidden));
        n += 2 + (c.tp_size > 1 ? 2 : 0);
        KMLL_TRY(decode_end(s, d->packed_final, d->state));
        ++n;
    }
    // keep the final hidden state where kmll_decoder_last_hidden finds it
    if (hidden != d->hidden_a) {
        KMLL_CUDA(cudaMemcpyAsync(d->hidden_a, hidden, sizeof(float) * c.dim, cudaMemcpyDeviceToDevice, s));
        ++n;
    }
    if (launches) *launches = n;
    return KMLL_OK;
}


// ---- chained decode step (W4-G128) ---------------------------------------------------------------------
// Per layer two launches: the attention kernel, then ONE chained kernel that runs the output projection + residual,
// RMSNorm + gate/up + SiLU, the down projection + residual and RMSNorm + the NEXT layer's Q/K/V (after the last
// layer: the final RMSNorm + lm_head arg-max and the end of the step).  Inside the chain the vectors travel as
// exchange words (internal.cuh); under tensor parallelism the row-parallel projections push theirs to every rank.
static bool chain_supported(const Decoder* d) {
    const kmll_decoder_config& c = d->cfg;
    if (c.format != KMLL_FORMAT_W4G128 || !c.fused) return false;
    if (2 * c.n_layers + 1 > 250) return false;
    const char* v = std::getenv("KMLL_CHAIN");
    if (v != nullptr && v[0] == '0') return false;
    // Under tensor parallelism the kernels over the canonical layout are faster today (measured at 2 GPUs: 736 against
    // 671 tokens/s): the prepared-layout kernel pays more per exchange than it gains in its main loop.  KMLL_CHAIN=tp
    // selects it anyway.
    if (c.tp_size > 1 && !(v != nullptr && strcmp(v, "tp") == 0)) return false;
    return true;
}

static int ensure_prepared(Decoder* d) {
    if (!d->chain || d->prepared_valid) return KMLL_OK;
    const kmll_decoder_config& c = d->cfg;
    auto one = [&](QWeight& w) -> int {
        if (w.prep == nullptr) KMLL_TRY(dalloc(d, &w.prep, w4_prepared_bytes(w.rows, w.cols, 0)));
        return w4_prepare(nullptr, (const uint8_t*)w.w, (const uint16_t*)w.scales, nullptr, nullptr, w.rows, w.cols, w.prep);
    };
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = d->layers[l];
        KMLL_TRY(one(L.wq));
        KMLL_TRY(one(L.wk));
        KMLL_TRY(one(L.wv));
        KMLL_TRY(one(L.wo));
        KMLL_TRY(one(L.w2));
        if (L.w13_prep == nullptr) KMLL_TRY(dalloc(d, &L.w13_prep, w4_prepared_bytes(L.w1.rows, L.w1.cols, 1)));
        KMLL_TRY(w4_prepare(nullptr, (const uint8_t*)L.w1.w, (const uint16_t*)L.w1.scales, (const uint8_t*)L.w3.w, (const uint16_t*)L.w3.scales,
                            L.w1.rows, L.w1.cols, L.w13_prep));
    }
    KMLL_TRY(one(d->output));
    KMLL_CUDA(cudaDeviceSynchronize());
    d->prepared_valid = true;
    return KMLL_OK;
}

static void chain_phase_common(ChainPhase& ph, int epi, int K) {
    memset(&ph, 0, sizeof(ph));
    ph.epi = epi;
    ph.K = K;
    ph.residual_index = -1;
}
static void chain_phase_mats(ChainPhase& ph, const uint8_t* const* w, const int* rows, float* const* outs, int nmat) {
    int units = 0;
    for (int m = 0; m < 3; ++m) {
        ph.unit_start[m] = units;
        if (m < nmat) {
            ph.w[m] = w[m];
            ph.out[m] = outs ? outs[m] : nullptr;
            ph.out_rows[m] = rows[m];
            units += ph.epi == EPI_SILU ? (rows[m] + 15) / 16 : (rows[m] + 31) / 32;
        }
    }
    ph.unit_start[3] = units;
    ph.total_units = units;
}

static int enqueue_step_chain(Decoder* d, cudaStream_t s, int* launches) {
    const kmll_decoder_config& c = d->cfg;
    const int q_len = d->n_heads_l * c.head_dim, kv_len = d->n_kv_l * c.head_dim;
    const unsigned long long before = launch_counter();
    const bool tp = c.tp_size > 1;
    KMLL_TRY(decode_begin(s, d->embedding, c.vocab_size, c.dim, d->state, d->history, d->history_cap, d->hidden_a, d->xc_epoch));
    // Q/K/V of layer `l` from the vector `in` (plain pointer or exchange 2l - 1)
    auto qkv_phase = [&](ChainPhase& ph, int l) {
        Layer& L = d->layers[l];
        chain_phase_common(ph, EPI_STORE, c.dim);
        const uint8_t* w[3] = {L.wq.prep, L.wk.prep, L.wv.prep};
        const int rows[3] = {q_len, kv_len, kv_len};
        float* outs[3] = {d->q, d->k, d->v};
        chain_phase_mats(ph, w, rows, outs, 3);
        ph.norm_w = L.attention_norm;
        ph.eps = c.norm_eps;
        if (l == 0) {
            ph.in_kind = CHAIN_IN_PLAIN;
            ph.x = d->hidden_a;
        } else {
            ph.in_kind = CHAIN_IN_INBOX;
            ph.in_index = 2 * l - 1;
        }
    };
    {
        ChainParams cp;
        memset(&cp, 0, sizeof(cp));
        cp.n_phases = 1;
        cp.xc = d->xc;
        if (d->xc != nullptr) cp.xcv = d->xc_host;
        qkv_phase(cp.phase[0], 0);
        KMLL_TRY(launch_chain(s, cp));
    }
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = d->layers[l];
        KMLL_TRY(apply_qk_norm(d, s, L, d->q, d->k, 1));
        if (c.rotary_dim == c.head_dim) {
            KMLL_TRY(decode_attention_launch(s, d->q, L.key_cache, L.value_cache, &d->state->seq_len, 0, c.max_seq_len, d->n_heads_l,
                                             d->n_kv_l, c.head_dim, d->attn_ws, d->attn, d->k, d->v, d->freqs, L.key_cache, L.value_cache, 1, 0, c.kv_bf16,
                                             c.sliding_window));
        } else {
            KMLL_TRY(prepare_incremental_dyn(s, d->q, d->k, d->v, d->freqs, c.rotary_dim / 2, d->state, c.max_seq_len, d->n_heads_l,
                                             d->n_kv_l, c.head_dim, d->q_rot, L.key_cache, L.value_cache, c.kv_bf16));
            KMLL_TRY(decode_attention_launch(s, d->q_rot, L.key_cache, L.value_cache, &d->state->seq_len, 0, c.max_seq_len, d->n_heads_l,
                                             d->n_kv_l, c.head_dim, d->attn_ws, d->attn, nullptr, nullptr, nullptr, nullptr, nullptr, 1, 0,
                                             c.kv_bf16, c.sliding_window));
        }
        ChainParams cp;
        memset(&cp, 0, sizeof(cp));
        cp.n_phases = 4;
        cp.xc = d->xc;
        if (d->xc != nullptr) cp.xcv = d->xc_host;
        {   // output projection + residual -> exchange 2l
            ChainPhase& ph = cp.phase[0];
            chain_phase_common(ph, EPI_RESIDUAL, q_len);
            const uint8_t* w[1] = {L.wo.prep};
            const int rows[1] = {c.dim};
            chain_phase_mats(ph, w, rows, nullptr, 1);
            ph.in_kind = CHAIN_IN_PLAIN;
            ph.x = d->attn;
            ph.add_residual = c.tp_rank == 0;
            if (l == 0) ph.residual = d->hidden_a;
            else ph.residual_index = 2 * l - 1;
            ph.out_kind = CHAIN_OUT_INBOX;
            ph.out_index = 2 * l;
        }
        {   // RMSNorm + gate/up + SiLU -> local exchange l
            ChainPhase& ph = cp.phase[1];
            chain_phase_common(ph, EPI_SILU, c.dim);
            const uint8_t* w[1] = {L.w13_prep};
            const int rows[1] = {d->hidden_l};
            chain_phase_mats(ph, w, rows, nullptr, 1);
            ph.norm_w = L.ffn_norm;
            ph.eps = c.norm_eps;
            ph.in_kind = CHAIN_IN_INBOX;
            ph.in_index = 2 * l;
            ph.in_units = cp.phase[0].total_units;
            ph.out_kind = CHAIN_OUT_LOCAL;
            ph.out_index = l;
        }
        {   // down projection + residual -> exchange 2l + 1
            ChainPhase& ph = cp.phase[2];
            chain_phase_common(ph, EPI_RESIDUAL, d->hidden_l);
            const uint8_t* w[1] = {L.w2.prep};
            const int rows[1] = {c.dim};
            chain_phase_mats(ph, w, rows, nullptr, 1);
            ph.in_kind = CHAIN_IN_LOCAL;
            ph.in_index = l;
            ph.in_units = cp.phase[1].total_units;
            ph.add_residual = c.tp_rank == 0;
            ph.residual_index = 2 * l;
            ph.out_kind = CHAIN_OUT_INBOX;
            ph.out_index = 2 * l + 1;
        }
        if (l + 1 < c.n_layers) {
            qkv_phase(cp.phase[3], l + 1);
        } else {  // final RMSNorm + lm_head arg-max; the block that finishes last ends the step
            ChainPhase& ph = cp.phase[3];
            chain_phase_common(ph, EPI_TOP1, c.dim);
            const uint8_t* w[1] = {d->output.prep};
            const int rows[1] = {d->vocab_l};
            chain_phase_mats(ph, w, rows, nullptr, 1);
            ph.norm_w = d->final_norm;
            ph.eps = c.norm_eps;
            ph.in_kind = CHAIN_IN_INBOX;
            ph.in_index = 2 * l + 1;
            ph.x_out = d->hidden_a;  // where kmll_decoder_last_hidden finds the final hidden state
            cp.partial_tokens = d->part_tok;
            cp.partial_logits = d->part_logit;
            cp.packed_out = tp ? d->packed : d->packed_final;
            cp.top1_counter = d->top1_counter;
            cp.token_offset = (uint32_t)(c.tp_rank * d->vocab_l);
            cp.state = tp ? nullptr : d->state;
            cp.push_top = tp ? 1 : 0;
        }
        cp.phase[3].in_units = cp.phase[2].total_units;  // its input comes from the down projection of this launch
        if (d->chain_split && !tp && !d->chain_words) {
            // one GPU, one launch per projection: the vectors go through plain buffers (the grid dependency of consecutive
            // launches orders them), exactly like kmll's own operator sequence
            float* hidden = (l & 1) ? d->hidden_b : d->hidden_a;   // input of this layer
            float* other = (l & 1) ? d->hidden_a : d->hidden_b;    // its output
            ChainPhase& wo = cp.phase[0];
            wo.residual = hidden; wo.residual_index = -1; wo.out_kind = CHAIN_OUT_PLAIN; wo.out[0] = d->hidden_mid;
            ChainPhase& gu = cp.phase[1];
            gu.in_kind = CHAIN_IN_PLAIN; gu.x = d->hidden_mid; gu.out_kind = CHAIN_OUT_PLAIN; gu.out[0] = d->act;
            ChainPhase& w2 = cp.phase[2];
            w2.in_kind = CHAIN_IN_PLAIN; w2.x = d->act; w2.residual = d->hidden_mid; w2.residual_index = -1;
            w2.out_kind = CHAIN_OUT_PLAIN; w2.out[0] = other;
            ChainPhase& nx = cp.phase[3];
            nx.in_kind = CHAIN_IN_PLAIN; nx.x = other; nx.x_out = nullptr;
        }
        if (d->chain_split) {
            // one launch per phase: the grid dependency of consecutive launches hands the vectors over (the words are
            // complete when a launch starts, so no arrival hint is needed); same kernel, same arithmetic
            for (int i = 0; i < 4; ++i) {
                ChainParams one = cp;
                one.n_phases = 1;
                one.phase[0] = cp.phase[i];
                one.phase[0].in_units = 0;
                if (i != 3) {
                    one.partial_tokens = nullptr;
                    one.state = nullptr;
                    one.push_top = 0;
                }
                KMLL_TRY(launch_chain(s, one));
            }
        } else {
            KMLL_TRY(launch_chain(s, cp));
        }
    }
    if (tp) KMLL_TRY(decode_end_gather(s, d->xc, d->state, d->packed_final));
    if (launches) *launches = (int)(launch_counter() - before);
    if (d->chain_split && !tp && !d->chain_words && (c.n_layers & 1)) {  // keep the final hidden state where kmll_decoder_last_hidden finds it
        KMLL_CUDA(cudaMemcpyAsync(d->hidden_a, d->hidden_b, sizeof(float) * c.dim, cudaMemcpyDeviceToDevice, s));
        if (launches) *launches += 1;
    }
    return KMLL_OK;
}

static int enqueue_step(Decoder* d, cudaStream_t s, int* launches) {
    return d->chain ? enqueue_step_chain(d, s, launches) : enqueue_step_fused(d, s, launches);
}

// One decode step launched operator by operator with the position known on the host, in kmll's own
// order (run_incremental_layer_token_into, crates/inference/src/model.rs:10102-10300).
static int enqueue_step_unfused(Decoder* d, cudaStream_t s, uint32_t token, int position) {
    const kmll_decoder_config& c = d->cfg;
    const int q_len = d->n_heads_l * c.head_dim, kv_len = d->n_kv_l * c.head_dim;
    const int nf = c.rotary_dim / 2;
    KMLL_TRY(kmll_embedding(s, d->embedding, c.vocab_size, c.dim, token, d->hidden_a));
    float* hidden = d->hidden_a;
    float* other = d->hidden_b;
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = d->layers[l];
        KMLL_TRY(kmll_rmsnorm(s, hidden, L.attention_norm, c.dim, c.norm_eps, d->normed));
        KMLL_TRY(op_linear(d, s, d->normed, L.wq, d->q));
        KMLL_TRY(op_linear(d, s, d->normed, L.wk, d->k));
        KMLL_TRY(op_linear(d, s, d->normed, L.wv, d->v));
        KMLL_TRY(apply_qk_norm(d, s, L, d->q, d->k, 1));
        KMLL_TRY(kmll_apply_rope(s, d->q, d->freqs, nf, position, c.head_dim, (size_t)q_len, d->q_rot));
        KMLL_TRY(kmll_apply_rope(s, d->k, d->freqs, nf, position, c.head_dim, (size_t)kv_len, d->k_rot));
        if (c.kv_bf16 || c.sliding_window > 0) {  // the same three operators with the options kmll's forms do not have
            KMLL_TRY(write_kv_row(s, d->k_rot, position, kv_len, c.head_dim, L.key_cache, c.kv_bf16));
            KMLL_TRY(write_kv_row(s, d->v, position, kv_len, c.head_dim, L.value_cache, c.kv_bf16));
            KMLL_TRY(decode_attention_launch(s, d->q_rot, L.key_cache, L.value_cache, nullptr, position + 1, c.max_seq_len, d->n_heads_l,
                                             d->n_kv_l, c.head_dim, d->attn_ws, d->attn, nullptr, nullptr, nullptr, nullptr, nullptr, 1, 0,
                                             c.kv_bf16, c.sliding_window));
        } else {
            KMLL_TRY(kmll_write_kv_cache(s, d->k_rot, position, c.max_seq_len, d->n_kv_l, c.head_dim, L.key_cache));
            KMLL_TRY(kmll_write_kv_cache(s, d->v, position, c.max_seq_len, d->n_kv_l, c.head_dim, L.value_cache));
            KMLL_TRY(kmll_single_query_attention(s, d->q_rot, L.key_cache, L.value_cache, position + 1, c.max_seq_len, d->n_heads_l, d->n_kv_l,
                                                 c.head_dim, d->attn_ws, d->attn));
        }
        KMLL_TRY(op_linear(d, s, d->attn, L.wo, d->delta));
        KMLL_TRY(tp_allreduce(d, s, d->delta, (size_t)c.dim));
        KMLL_TRY(kmll_add(s, hidden, d->delta, (size_t)c.dim, d->hidden_mid));
        // run_ffn_from_hidden_into, crates/inference/src/model.rs:11463-11508
        KMLL_TRY(kmll_rmsnorm(s, d->hidden_mid, L.ffn_norm, c.dim, c.norm_eps, d->normed));
        KMLL_TRY(op_linear(d, s, d->normed, L.w1, d->gate));
        KMLL_TRY(op_linear(d, s, d->normed, L.w3, d->up));
        KMLL_TRY(kmll_silu_mul(s, d->gate, d->up, (size_t)d->hidden_l, d->act));
        KMLL_TRY(op_linear(d, s, d->act, L.w2, d->delta));
        KMLL_TRY(tp_allreduce(d, s, d->delta, (size_t)c.dim));
        KMLL_TRY(kmll_add(s, d->hidden_mid, d->delta, (size_t)c.dim, other));
        float* t = hidden;
        hidden = other;
        other = t;
    }
    KMLL_TRY(output_top1(d, s, hidden));
    if (hidden != d->hidden_a) KMLL_CUDA(cudaMemcpyAsync(d->hidden_a, hidden, sizeof(float) * c.dim, cudaMemcpyDeviceToDevice, s));
    return KMLL_OK;
}

static int write_state(Decoder* d, cudaStream_t s, int position, int step, uint64_t next_top) {
    DecodeState st;
    st.position = position;
    st.seq_len = position + 1;
    st.step = step;
    st.pad = 0;
    st.next_top = next_top;
    memcpy(d->pinned + 8, &st, sizeof(st));
    KMLL_CUDA(cudaMemcpyAsync(d->state, d->pinned + 8, sizeof(st), cudaMemcpyHostToDevice, s));
    return KMLL_OK;
}

static int ensure_graph(Decoder* d, cudaStream_t s) {
    // a timeline buffer was attached or detached since the capture: the graph holds stale slot pointers
    if (d->graph != nullptr && d->graph_trace_generation != trace_generation()) {
        KMLL_CUDA(cudaStreamSynchronize(s));
        cudaGraphExecDestroy(d->graph);
        d->graph = nullptr;
    }
    KMLL_TRY(ensure_prepared(d));  // (never inside a capture: the capture below happens after this returned)
    if (d->graph != nullptr) return KMLL_OK;
    d->graph_trace_generation = trace_generation();
    if (!d->warmed) {
        // one eager step so that every kernel has its attributes set before capture; the state is
        // restored afterwards and the KV row it wrote is rewritten by the real step at this position
        DecodeState saved;
        KMLL_CUDA(cudaStreamSynchronize(s));
        KMLL_CUDA(cudaMemcpy(&saved, d->state, sizeof(saved), cudaMemcpyDeviceToHost));
        if (d->host_position >= d->cfg.max_seq_len) return fail(KMLL_ERR_CAPACITY, "sequence is full");
        KMLL_TRY(enqueue_step(d, s, &d->launches_per_step));
        KMLL_CUDA(cudaStreamSynchronize(s));
        KMLL_CUDA(cudaMemcpy(d->state, &saved, sizeof(saved), cudaMemcpyHostToDevice));
        d->warmed = true;
    }
    cudaGraph_t g = nullptr;
    if (d->capture_stream == nullptr) KMLL_CUDA(cudaStreamCreateWithFlags(&d->capture_stream, cudaStreamNonBlocking));
    KMLL_CUDA(cudaStreamBeginCapture(d->capture_stream, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_step(d, d->capture_stream, &d->launches_per_step);
    cudaError_t e = cudaStreamEndCapture(d->capture_stream, &g);
    if (rc != KMLL_OK) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&d->graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

static uint64_t tensor_seed(uint64_t seed, int layer, int tensor) {
    return seed * 0x9e3779b97f4a7c15ull + (uint64_t)(layer + 2) * 1000003ull + (uint64_t)tensor * 7919ull;
}

// Copies this rank's shard of a full quantized tensor (device -> device).
static int copy_shard(Decoder* d, const QWeight& dst, const void* full_w, const void* full_s, int full_rows, int full_cols,
                      ShardKind kind) {
    const int fmt = d->cfg.format;
    const int r = d->cfg.tp_rank;
    const size_t wrow_full = fmt == KMLL_FORMAT_W4G128 ? (size_t)full_cols / 2 : (size_t)full_cols;
    const size_t wrow_dst = fmt == KMLL_FORMAT_W4G128 ? (size_t)dst.cols / 2 : (size_t)dst.cols;
    const size_t srow_full = fmt == KMLL_FORMAT_W4G128 ? (size_t)(full_cols / 128) * 2 : 4;
    const size_t srow_dst = fmt == KMLL_FORMAT_W4G128 ? (size_t)(dst.cols / 128) * 2 : 4;
    size_t row0 = 0, wcol0 = 0, scol0 = 0;
    if (kind == SHARD_ROWS) row0 = (size_t)r * dst.rows;
    if (kind == SHARD_COLS) {
        wcol0 = (size_t)r * wrow_dst;
        scol0 = fmt == KMLL_FORMAT_W4G128 ? (size_t)r * srow_dst : 0;  // RS-I8 row scales are replicated
    }
    (void)full_rows;
    KMLL_CUDA(cudaMemcpy2D(dst.w, wrow_dst, (const uint8_t*)full_w + row0 * wrow_full + wcol0, wrow_full, wrow_dst, dst.rows,
                           cudaMemcpyDeviceToDevice));
    KMLL_CUDA(cudaMemcpy2D(dst.scales, srow_dst, (const uint8_t*)full_s + row0 * srow_full + scol0, srow_full, srow_dst, dst.rows,
                           cudaMemcpyDeviceToDevice));
    return KMLL_OK;
}

struct TensorRef {
    QWeight* q = nullptr;
    uint16_t** bf16 = nullptr;
    int full_rows = 0, full_cols = 0;
    ShardKind kind = SHARD_NONE;
    size_t bf16_count = 0;
};

static int tensor_ref(Decoder* d, int layer, int tensor, TensorRef* out) {
    const kmll_decoder_config& c = d->cfg;
    TensorRef t;
    const int q_full = c.n_heads * c.head_dim, kv_full = c.n_kv_heads * c.head_dim;
    if (tensor >= KMLL_T_FINAL_NORM && tensor <= KMLL_T_OUTPUT) {
        if (layer != -1) return fail(KMLL_ERR_SHAPE, "tensor %d is not a per-layer tensor (use layer = -1)", tensor);
        if (tensor == KMLL_T_FINAL_NORM) { t.bf16 = &d->final_norm; t.bf16_count = c.dim; }
        else if (tensor == KMLL_T_EMBEDDING) { t.bf16 = &d->embedding; t.bf16_count = (size_t)c.vocab_size * c.dim; }
        else if (tensor == KMLL_T_OUTPUT) { t.q = &d->output; t.full_rows = c.vocab_size; t.full_cols = c.dim; t.kind = SHARD_ROWS; }
        else return fail(KMLL_ERR_SHAPE, "unknown tensor id %d", tensor);
    } else {
        if (layer < 0 || layer >= c.n_layers) return fail(KMLL_ERR_SHAPE, "layer %d out of range", layer);
        Layer& L = d->layers[layer];
        switch (tensor) {
            case KMLL_T_ATTENTION_NORM: t.bf16 = &L.attention_norm; t.bf16_count = c.dim; break;
            case KMLL_T_FFN_NORM: t.bf16 = &L.ffn_norm; t.bf16_count = c.dim; break;
            case KMLL_T_Q_NORM: t.bf16 = &L.q_norm; t.bf16_count = c.head_dim; break;
            case KMLL_T_K_NORM: t.bf16 = &L.k_norm; t.bf16_count = c.head_dim; break;
            case KMLL_T_WQ: t.q = &L.wq; t.full_rows = q_full; t.full_cols = c.dim; t.kind = SHARD_ROWS; break;
            case KMLL_T_WK: t.q = &L.wk; t.full_rows = kv_full; t.full_cols = c.dim; t.kind = SHARD_ROWS; break;
            case KMLL_T_WV: t.q = &L.wv; t.full_rows = kv_full; t.full_cols = c.dim; t.kind = SHARD_ROWS; break;
            case KMLL_T_WO: t.q = &L.wo; t.full_rows = c.dim; t.full_cols = q_full; t.kind = SHARD_COLS; break;
            case KMLL_T_W1: t.q = &L.w1; t.full_rows = c.hidden_dim; t.full_cols = c.dim; t.kind = SHARD_ROWS; break;
            case KMLL_T_W3: t.q = &L.w3; t.full_rows = c.hidden_dim; t.full_cols = c.dim; t.kind = SHARD_ROWS; break;
            case KMLL_T_W2: t.q = &L.w2; t.full_rows = c.dim; t.full_cols = c.hidden_dim; t.kind = SHARD_COLS; break;
            default: return fail(KMLL_ERR_SHAPE, "unknown tensor id %d", tensor);
        }
    }
    if (c.tp_size == 1) t.kind = SHARD_NONE;
    *out = t;
    return KMLL_OK;
}

}  // namespace kmll

using namespace kmll;

// ---- lockstep batch of sequences ---------------------------------------------------------------------
// Several independent sequences at the same position share every weight read: the activations of a step are
// [batch, dim] rows through the batched linear kernel, attention runs per sequence (grid z) on per-sequence
// KV caches.  kmll has no batched decode; the per-sequence math is that of the single-sequence step.
struct BatchDecoder {
    Decoder* d = nullptr;  // weights and configuration (not owned)
    int batch = 0;
    size_t cache_stride = 0;  // floats between two sequences' caches
    std::vector<float*> key_cache, value_cache;  // per layer: [batch][max_seq * kv_len]
    float *hidden_a = nullptr, *hidden_b = nullptr, *hidden_mid = nullptr, *q = nullptr, *k = nullptr, *v = nullptr;
    float *attn = nullptr, *act = nullptr, *logits = nullptr, *attn_ws = nullptr;
    float *gate = nullptr, *up = nullptr;  // [batch, hidden] scratch of the tensor-core gate/up path
    void* linear_ws = nullptr;             // scratch of the batched linears (f16 planes of the activations)
    BatchState* state = nullptr;
    uint64_t* history = nullptr;  // [batch][history_cap]
    int history_cap = 0;
    int host_position = -1;
    unsigned filled = 0;  // bit b: slot b holds a sequence
    cudaGraphExec_t graph = nullptr;
    unsigned long long graph_trace_generation = 0;
    cudaStream_t capture_stream = nullptr;
    bool warmed = false;
    int launches_per_step = 0;
    std::vector<void*> allocs;
};

template <typename T>
static int balloc(BatchDecoder* b, T** out, size_t count) {
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, count * sizeof(T) + 16);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "cudaMalloc(%zu bytes): %s", count * sizeof(T), cudaGetErrorString(e));
    b->allocs.push_back(p);
    *out = static_cast<T*>(p);
    return KMLL_OK;
}

static int enqueue_batch_step(BatchDecoder* b, cudaStream_t s, int* launches) {
    Decoder* d = b->d;
    const kmll_decoder_config& c = d->cfg;
    const int B = b->batch;
    const int q_len = c.n_heads * c.head_dim, kv_len = c.n_kv_heads * c.head_dim;
    const unsigned long long launches_before = launch_counter();  // the batched linear forms issue several kernels each
    KMLL_TRY(batch_begin(s, d->embedding, c.vocab_size, c.dim, B, b->state, b->history, b->history_cap, b->hidden_a));
    float* hidden = b->hidden_a;
    float* other = b->hidden_b;
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = d->layers[l];
        {
            const void* w[3] = {L.wq.w, L.wk.w, L.wv.w};
            const void* sc[3] = {L.wq.scales, L.wk.scales, L.wv.scales};
            const int rows[3] = {q_len, kv_len, kv_len};
            float* outs[3] = {b->q, b->k, b->v};
            KMLL_TRY(linear_batched_form(0, s, c.format, hidden, B, L.attention_norm, c.norm_eps, w, sc, rows, c.dim, outs, nullptr, b->linear_ws));
        }
        KMLL_TRY(apply_qk_norm(d, s, L, b->q, b->k, B));
        KMLL_TRY(decode_attention_launch(s, b->q, b->key_cache[l], b->value_cache[l], &b->state->seq_len, 0, c.max_seq_len, c.n_heads,
                                         c.n_kv_heads, c.head_dim, b->attn_ws, b->attn, b->k, b->v, d->freqs, b->key_cache[l],
                                         b->value_cache[l], B, b->cache_stride, c.kv_bf16, c.sliding_window));
        {
            const void* w[1] = {L.wo.w};
            const void* sc[1] = {L.wo.scales};
            const int rows[1] = {c.dim};
            float* outs[1] = {b->hidden_mid};
            KMLL_TRY(linear_batched_form(2, s, c.format, b->attn, B, nullptr, 0.f, w, sc, rows, q_len, outs, hidden, b->linear_ws));
        }
        {
            const void* w[2] = {L.w1.w, L.w3.w};
            const void* sc[2] = {L.w1.scales, L.w3.scales};
            const int rows[1] = {c.hidden_dim};
            float* outs[1] = {b->act};
            KMLL_TRY(linear_batched_form(1, s, c.format, b->hidden_mid, B, L.ffn_norm, c.norm_eps, w, sc, rows, c.dim, outs, nullptr, b->linear_ws, b->gate,
                                         b->up));
        }
        {
            const void* w[1] = {L.w2.w};
            const void* sc[1] = {L.w2.scales};
            const int rows[1] = {c.dim};
            float* outs[1] = {other};
            KMLL_TRY(linear_batched_form(2, s, c.format, b->act, B, nullptr, 0.f, w, sc, rows, c.hidden_dim, outs, b->hidden_mid, b->linear_ws));
        }
        float* t = hidden;
        hidden = other;
        other = t;
    }
    {
        const void* w[1] = {d->output.w};
        const void* sc[1] = {d->output.scales};
        const int rows[1] = {c.vocab_size};
        float* outs[1] = {b->logits};
        KMLL_TRY(linear_batched_form(3, s, c.format, hidden, B, d->final_norm, c.norm_eps, w, sc, rows, c.dim, outs, nullptr, b->linear_ws));
    }
    KMLL_TRY(batch_end(s, b->logits, c.vocab_size, B, b->state));
    if (launches) *launches = (int)(launch_counter() - launches_before);
    return KMLL_OK;
}

static int ensure_batch_graph(BatchDecoder* b, cudaStream_t s) {
    if (b->graph != nullptr && b->graph_trace_generation != trace_generation()) {
        KMLL_CUDA(cudaStreamSynchronize(s));
        cudaGraphExecDestroy(b->graph);
        b->graph = nullptr;
    }
    if (b->graph != nullptr) return KMLL_OK;
    b->graph_trace_generation = trace_generation();
    if (!b->warmed) {
        // one eager step (kernel attributes get set outside capture); the state is restored afterwards and the KV
        // rows it wrote are rewritten by the real step at this position
        BatchState saved;
        KMLL_CUDA(cudaStreamSynchronize(s));
        KMLL_CUDA(cudaMemcpy(&saved, b->state, sizeof(saved), cudaMemcpyDeviceToHost));
        KMLL_TRY(enqueue_batch_step(b, s, &b->launches_per_step));
        KMLL_CUDA(cudaStreamSynchronize(s));
        KMLL_CUDA(cudaMemcpy(b->state, &saved, sizeof(saved), cudaMemcpyHostToDevice));
        b->warmed = true;
    }
    cudaGraph_t g = nullptr;
    if (b->capture_stream == nullptr) KMLL_CUDA(cudaStreamCreateWithFlags(&b->capture_stream, cudaStreamNonBlocking));
    KMLL_CUDA(cudaStreamBeginCapture(b->capture_stream, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_batch_step(b, b->capture_stream, &b->launches_per_step);
    cudaError_t e = cudaStreamEndCapture(b->capture_stream, &g);
    if (rc != KMLL_OK) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&b->graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    return KMLL_OK;
}


// Exchange buffer of a decoder: inboxes [2][tp][dim], arg-max slots [2][tp][2], the local vector of the chained step
// [hidden_l] and the step counter.  On one GPU it is plain device memory.  Under tensor parallelism every rank
// allocates one, the ranks swap CUDA IPC handles through an NCCL all-gather and map each other's buffers; the
// unchained path needs batch-1 stream kernels for every exchanged vector and at most 63 layers (its exchange numbers
// stay below 127), the chained path at most 124 layers.
static int setup_exchange(Decoder* d) {
    const kmll_decoder_config& c = d->cfg;
    const int tp = c.tp_size;
    if (tp > kMaxTp || !c.fused) return KMLL_OK;  // stay on NCCL
    if (!d->chain && 2 * c.n_layers > 126) return KMLL_OK;
    NcclApi* api = tp > 1 ? nccl_api() : nullptr;
    const size_t inbox_bytes = (size_t)2 * tp * c.dim * sizeof(uint2);
    const size_t off_top = (inbox_bytes + 127) & ~(size_t)127;
    const size_t top_bytes = ((size_t)2 * tp * 2 * sizeof(uint2) + 127) & ~(size_t)127;
    const size_t off_box = off_top + top_bytes;
    const size_t box_bytes = ((size_t)d->hidden_l * sizeof(uint2) + 127) & ~(size_t)127;
    const size_t off_ready = off_box + box_bytes;  // arrival hints: inbox exchanges, then the local vector (256 each)
    const size_t off_local = off_ready + 2 * 256 * sizeof(unsigned int);  // epoch
    const size_t total = off_local + 256;
    KMLL_CUDA(cudaMalloc(&d->xc_local, total));
    KMLL_CUDA(cudaMemset(d->xc_local, 0, total));
    std::vector<cudaIpcMemHandle_t> handles(tp);
    if (tp > 1) {
        cudaIpcMemHandle_t mine;
        KMLL_CUDA(cudaIpcGetMemHandle(&mine, d->xc_local));
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handles are 64 bytes");
        unsigned char* handles_dev = nullptr;
        KMLL_CUDA(cudaMalloc(&handles_dev, (size_t)tp * 64));
        KMLL_CUDA(cudaMemcpy(handles_dev + (size_t)c.tp_rank * 64, &mine, 64, cudaMemcpyHostToDevice));
        // (in-place all-gather: the send buffer is this rank's slot of the receive buffer; it also orders every
        // rank's memset above before anybody's first push)
        ncclResult_t r = api->AllGather(handles_dev + (size_t)c.tp_rank * 64, handles_dev, 64, ncclChar, d->comm, nullptr);
        if (r != ncclSuccess) { cudaFree(handles_dev); return fail(KMLL_ERR_CUDA, "ncclAllGather (IPC handles) failed"); }
        KMLL_CUDA(cudaStreamSynchronize(nullptr));
        KMLL_CUDA(cudaMemcpy(handles.data(), handles_dev, (size_t)tp * 64, cudaMemcpyDeviceToHost));
        cudaFree(handles_dev);
    }
    TpExchange h;
    memset(&h, 0, sizeof(h));
    h.tp = tp; h.rank = c.tp_rank; h.dim = c.dim;
    h.mult = d->chain ? 256 : 128;
    h.top_index = h.mult - 1;
    h.local_dim = d->hidden_l;
    {
        const char* v = std::getenv("KMLL_PUSH");
        h.push_mode = (v != nullptr && strcmp(v, "st") == 0) ? 2 : 1;
    }
    for (int rnk = 0; rnk < tp; ++rnk) {
        void* base = d->xc_local;
        if (rnk != c.tp_rank) {
            cudaError_t e = cudaIpcOpenMemHandle(&base, handles[rnk], cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "cudaIpcOpenMemHandle (rank %d): %s", rnk, cudaGetErrorString(e));
            d->xc_peer_base[rnk] = base;
        }
        unsigned char* b = static_cast<unsigned char*>(base);
        h.inbox[rnk] = reinterpret_cast<uint2*>(b);
        h.top_inbox[rnk] = reinterpret_cast<uint2*>(b + off_top);
        h.ready[rnk] = reinterpret_cast<unsigned int*>(b + off_ready);
    }
    unsigned char* lb = static_cast<unsigned char*>(d->xc_local);
    h.local_box = reinterpret_cast<uint2*>(lb + off_box);
    h.ready_local = reinterpret_cast<unsigned int*>(lb + off_ready) + 256;
    h.epoch = reinterpret_cast<unsigned int*>(lb + off_local);
    d->xc_epoch = h.epoch;
    KMLL_TRY(dalloc(d, &d->xc, 1));
    KMLL_CUDA(cudaMemcpy(d->xc, &h, sizeof(h), cudaMemcpyHostToDevice));
    d->xc_host = h;
    return KMLL_OK;
}

extern "C" {

size_t kmll_decoder_config_bytes(void) { return sizeof(kmll_decoder_config); }

int kmll_decoder_create(const kmll_decoder_config* config, kmll_decoder_t* out) {
    KMLL_REQUIRE_PTR(config);
    KMLL_REQUIRE_PTR(out);
    KMLL_TRY(validate_config(*config));
    Decoder* d = new Decoder();
    d->cfg = *config;
    const kmll_decoder_config& c = d->cfg;
    int rc = KMLL_OK;
    auto body = [&]() -> int {
        KMLL_CUDA(cudaGetDevice(&d->device));
        d->n_heads_l = c.n_heads / c.tp_size;
        d->n_kv_l = c.n_kv_heads / c.tp_size;
        d->hidden_l = c.hidden_dim / c.tp_size;
        d->vocab_l = c.vocab_size / c.tp_size;
        const int q_len = d->n_heads_l * c.head_dim, kv_len = d->n_kv_l * c.head_dim;
        d->layers.resize(c.n_layers);
        for (int l = 0; l < c.n_layers; ++l) {
            Layer& L = d->layers[l];
            KMLL_TRY(dalloc(d, &L.attention_norm, (size_t)c.dim));
            KMLL_TRY(dalloc(d, &L.ffn_norm, (size_t)c.dim));
            KMLL_TRY(alloc_qweight(d, &L.wq, q_len, c.dim));
            KMLL_TRY(alloc_qweight(d, &L.wk, kv_len, c.dim));
            KMLL_TRY(alloc_qweight(d, &L.wv, kv_len, c.dim));
            KMLL_TRY(alloc_qweight(d, &L.wo, c.dim, q_len));
            KMLL_TRY(alloc_qweight(d, &L.w1, d->hidden_l, c.dim));
            KMLL_TRY(alloc_qweight(d, &L.w3, d->hidden_l, c.dim));
            KMLL_TRY(alloc_qweight(d, &L.w2, c.dim, d->hidden_l));
            // f32 elements, or bf16 bit patterns in the same [max_seq, n_kv, head_dim] layout (kv_len is even)
            const size_t cache = (size_t)c.max_seq_len * kv_len / (c.kv_bf16 ? 2 : 1);
            KMLL_TRY(dalloc(d, &L.key_cache, cache));
            KMLL_TRY(dalloc(d, &L.value_cache, cache));
            KMLL_CUDA(cudaMemset(L.key_cache, 0, cache * sizeof(float)));
            KMLL_CUDA(cudaMemset(L.value_cache, 0, cache * sizeof(float)));
            d->kv_bytes += 2 * cache * sizeof(float);
        }
        KMLL_TRY(dalloc(d, &d->final_norm, (size_t)c.dim));
        KMLL_TRY(dalloc(d, &d->embedding, (size_t)c.vocab_size * c.dim));
        d->weight_bytes += (size_t)c.vocab_size * c.dim * 2;
        KMLL_TRY(alloc_qweight(d, &d->output, d->vocab_l, c.dim));
        // RoPE frequencies, rope_frequencies of crates/inference/src/model.rs:9240-9249 (f32 powf on the host)
        std::vector<float> freqs(c.rotary_dim / 2);
        for (int i = 0; i < c.rotary_dim / 2; ++i) freqs[i] = 1.0f / powf(c.rope_theta, (float)(2 * i) / (float)c.rotary_dim);
        KMLL_TRY(dalloc(d, &d->freqs, freqs.size()));
        KMLL_CUDA(cudaMemcpy(d->freqs, freqs.data(), freqs.size() * sizeof(float), cudaMemcpyHostToDevice));
        KMLL_TRY(dalloc(d, &d->hidden_a, (size_t)c.dim));
        KMLL_TRY(dalloc(d, &d->hidden_b, (size_t)c.dim));
        KMLL_TRY(dalloc(d, &d->hidden_mid, (size_t)c.dim));
        KMLL_TRY(dalloc(d, &d->normed, (size_t)c.dim));
        KMLL_TRY(dalloc(d, &d->delta, (size_t)c.dim));
        KMLL_TRY(dalloc(d, &d->q, (size_t)q_len));
        KMLL_TRY(dalloc(d, &d->q_rot, (size_t)q_len));
        KMLL_TRY(dalloc(d, &d->attn, (size_t)q_len));
        KMLL_TRY(dalloc(d, &d->k, (size_t)kv_len));
        KMLL_TRY(dalloc(d, &d->k_rot, (size_t)kv_len));
        KMLL_TRY(dalloc(d, &d->v, (size_t)kv_len));
        KMLL_TRY(dalloc(d, &d->gate, (size_t)d->hidden_l));
        KMLL_TRY(dalloc(d, &d->up, (size_t)d->hidden_l));
        KMLL_TRY(dalloc(d, &d->act, (size_t)d->hidden_l));
        const size_t ws = decode_attention_workspace_floats(d->n_heads_l, c.head_dim, c.max_seq_len);
        KMLL_TRY(dalloc(d, &d->attn_ws, ws));
        KMLL_CUDA(cudaMemset(d->attn_ws, 0, ws * sizeof(float)));
        // (the chained kernel writes one partial per block of its grid, which another phase may have sized)
        const int parts = kmll_linear_top1_partial_count(d->vocab_l) + 1024;
        KMLL_TRY(dalloc(d, &d->part_tok, (size_t)parts));
        KMLL_TRY(dalloc(d, &d->part_logit, (size_t)parts));
        KMLL_TRY(dalloc(d, &d->packed, (size_t)2));
        KMLL_TRY(dalloc(d, &d->packed_all, (size_t)c.tp_size + 1));
        KMLL_TRY(dalloc(d, &d->packed_final, (size_t)2));
        KMLL_TRY(dalloc(d, &d->state, (size_t)1));
        d->history_cap = c.max_seq_len;
        KMLL_TRY(dalloc(d, &d->history, (size_t)d->history_cap));
        KMLL_CUDA(cudaMemset(d->state, 0, sizeof(DecodeState)));
        KMLL_CUDA(cudaMallocHost((void**)&d->pinned, 64 * sizeof(uint64_t)));
        d->chain = chain_supported(d);
        {
            const char* v = std::getenv("KMLL_CHAIN");
            d->chain_split = !(v != nullptr && strcmp(v, "layer") == 0);
            d->chain_words = v != nullptr && strcmp(v, "words") == 0;
        }
        if (d->chain) {
            KMLL_TRY(dalloc(d, &d->top1_counter, (size_t)4));
            KMLL_CUDA(cudaMemset(d->top1_counter, 0, 16));
            if (c.tp_size == 1) KMLL_TRY(setup_exchange(d));
        }
        return KMLL_OK;
    };
    rc = body();
    if (rc != KMLL_OK) {
        kmll_decoder_destroy(d);
        return rc;
    }
    *out = d;
    return KMLL_OK;
}

int kmll_decoder_destroy(kmll_decoder_t dec) {
    if (dec == nullptr) return KMLL_OK;
    Decoder* d = static_cast<Decoder*>(dec);
    if (d->graph) cudaGraphExecDestroy(d->graph);
    if (d->capture_stream) cudaStreamDestroy(d->capture_stream);
    if (d->comm) {
        NcclApi* api = nccl_api();
        if (api && api->CommDestroy) api->CommDestroy(d->comm);
    }
    for (int r = 0; r < kMaxTp; ++r)
        if (d->xc_peer_base[r]) cudaIpcCloseMemHandle(d->xc_peer_base[r]);
    if (d->xc_local) cudaFree(d->xc_local);
    for (void* p : d->allocs) cudaFree(p);
    if (d->pinned) cudaFreeHost(d->pinned);
    delete d;
    return KMLL_OK;
}

int kmll_decoder_init_random(kmll_decoder_t dec, uint64_t seed, float std, int tie_embeddings) {
    KMLL_REQUIRE_PTR(dec);
    Decoder* d = static_cast<Decoder*>(dec);
    const kmll_decoder_config& c = d->cfg;
    const int q_full = c.n_heads * c.head_dim;
    size_t max_elems = (size_t)c.vocab_size * c.dim;
    const size_t e2 = (size_t)c.hidden_dim * c.dim, e3 = (size_t)q_full * c.dim;
    if (e2 > max_elems) max_elems = e2;
    if (e3 > max_elems) max_elems = e3;
    float* tmp = nullptr;
    uint16_t* tmp_bf16 = nullptr;
    uint8_t* full_w = nullptr;
    uint8_t* full_s = nullptr;
    auto cleanup = [&]() {
        cudaFree(tmp); cudaFree(tmp_bf16); cudaFree(full_w); cudaFree(full_s);
    };
    auto body = [&]() -> int {
        KMLL_CUDA(cudaMalloc((void**)&tmp, max_elems * sizeof(float)));
        KMLL_CUDA(cudaMalloc((void**)&tmp_bf16, max_elems * sizeof(uint16_t)));
        KMLL_CUDA(cudaMalloc((void**)&full_w, max_elems));
        KMLL_CUDA(cudaMalloc((void**)&full_s, max_elems / 16 + 16 + (size_t)c.vocab_size * 4));
        std::vector<uint16_t> ones(c.dim, 0x3f80);  // bf16 1.0
        auto fill_quant = [&](int layer, int tensor, const uint16_t* bf16_source) -> int {
            TensorRef t;
            KMLL_TRY(tensor_ref(d, layer, tensor, &t));
            const size_t n = (size_t)t.full_rows * t.full_cols;
            if (c.format == KMLL_FORMAT_W4G128) {
                if (bf16_source != nullptr) return fail(KMLL_ERR_UNSUPPORTED, "internal: W4 quantizes from f32");
                KMLL_TRY(kmll_fill_normal_f32(nullptr, tmp, n, tensor_seed(seed, layer, tensor), std));
                KMLL_TRY(kmll_quantize_w4g128(nullptr, tmp, t.full_rows, t.full_cols, full_w, (uint16_t*)full_s));
            } else {
                const uint16_t* src = bf16_source;
                if (src == nullptr) {
                    KMLL_TRY(kmll_fill_normal_f32(nullptr, tmp, n, tensor_seed(seed, layer, tensor), std));
                    KMLL_TRY(kmll_f32_to_bf16(nullptr, tmp, n, tmp_bf16));
                    src = tmp_bf16;
                }
                KMLL_TRY(kmll_quantize_rs_i8(nullptr, src, t.full_rows, t.full_cols, (int8_t*)full_w, (float*)full_s));
            }
            KMLL_CUDA(cudaDeviceSynchronize());
            return copy_shard(d, *t.q, full_w, full_s, t.full_rows, t.full_cols, t.kind);
        };
        for (int l = 0; l < c.n_layers; ++l) {
            KMLL_CUDA(cudaMemcpy(d->layers[l].attention_norm, ones.data(), c.dim * 2, cudaMemcpyHostToDevice));
            KMLL_CUDA(cudaMemcpy(d->layers[l].ffn_norm, ones.data(), c.dim * 2, cudaMemcpyHostToDevice));
            const int ids[7] = {KMLL_T_WQ, KMLL_T_WK, KMLL_T_WV, KMLL_T_WO, KMLL_T_W1, KMLL_T_W3, KMLL_T_W2};
            for (int i = 0; i < 7; ++i) KMLL_TRY(fill_quant(l, ids[i], nullptr));
        }
        KMLL_CUDA(cudaMemcpy(d->final_norm, ones.data(), c.dim * 2, cudaMemcpyHostToDevice));
        const size_t ne = (size_t)c.vocab_size * c.dim;
        KMLL_TRY(kmll_fill_normal_f32(nullptr, tmp, ne, tensor_seed(seed, -1, KMLL_T_EMBEDDING), std));
        KMLL_TRY(kmll_f32_to_bf16(nullptr, tmp, ne, d->embedding));
        if (tie_embeddings) {
            if (c.format == KMLL_FORMAT_W4G128) {
                // the output matrix is the bf16 embedding table itself: widen it (exact) and quantize
                KMLL_TRY(widen_bf16(nullptr, d->embedding, ne, tmp));
                KMLL_TRY(kmll_quantize_w4g128(nullptr, tmp, c.vocab_size, c.dim, full_w, (uint16_t*)full_s));
                KMLL_CUDA(cudaDeviceSynchronize());
                KMLL_TRY(copy_shard(d, d->output, full_w, full_s, c.vocab_size, c.dim, c.tp_size == 1 ? SHARD_NONE : SHARD_ROWS));
            } else {
                KMLL_TRY(fill_quant(-1, KMLL_T_OUTPUT, d->embedding));
            }
        } else {
            KMLL_TRY(fill_quant(-1, KMLL_T_OUTPUT, nullptr));
        }
        KMLL_CUDA(cudaDeviceSynchronize());
        return KMLL_OK;
    };
    const int rc = body();
    cleanup();
    if (rc == KMLL_OK) d->weights_set = true;
    d->prepared_valid = false;
    return rc;
}

int kmll_decoder_set_tensor(kmll_decoder_t dec, int layer, int tensor, const void* values, const void* scales) {
    KMLL_REQUIRE_PTR(dec);
    KMLL_REQUIRE_PTR(values);
    Decoder* d = static_cast<Decoder*>(dec);
    TensorRef t;
    KMLL_TRY(tensor_ref(d, layer, tensor, &t));
    if (t.bf16 != nullptr) {
        if (*t.bf16 == nullptr) {  // an optional tensor (q / k norm) seen for the first time: the step gains a launch
            if (d->graph != nullptr) return fail(KMLL_ERR_STATE, "set_tensor: optional tensors must be set before the first decode step");
            KMLL_TRY(dalloc(d, t.bf16, t.bf16_count));
        }
        KMLL_CUDA(cudaMemcpy(*t.bf16, values, t.bf16_count * 2, cudaMemcpyHostToDevice));
        d->weights_set = true;
        return KMLL_OK;
    }
    KMLL_REQUIRE_PTR(scales);
    size_t sb = 0;
    const size_t wb = qweight_bytes(d->cfg.format, t.full_rows, t.full_cols, &sb);
    uint8_t *fw = nullptr, *fs = nullptr;
    KMLL_CUDA(cudaMalloc((void**)&fw, wb));
    cudaError_t e = cudaMalloc((void**)&fs, sb);
    if (e != cudaSuccess) { cudaFree(fw); return fail(KMLL_ERR_CUDA, "cudaMalloc: %s", cudaGetErrorString(e)); }
    int rc = KMLL_OK;
    if (cudaMemcpy(fw, values, wb, cudaMemcpyHostToDevice) != cudaSuccess || cudaMemcpy(fs, scales, sb, cudaMemcpyHostToDevice) != cudaSuccess)
        rc = fail(KMLL_ERR_CUDA, "tensor upload failed");
    if (rc == KMLL_OK) rc = copy_shard(d, *t.q, fw, fs, t.full_rows, t.full_cols, t.kind);
    cudaFree(fw);
    cudaFree(fs);
    if (rc == KMLL_OK) d->weights_set = true;
    d->prepared_valid = false;
    return rc;
}

int kmll_decoder_get_tensor(kmll_decoder_t dec, int layer, int tensor, void* values, void* scales) {
    KMLL_REQUIRE_PTR(dec);
    Decoder* d = static_cast<Decoder*>(dec);
    TensorRef t;
    KMLL_TRY(tensor_ref(d, layer, tensor, &t));
    KMLL_CUDA(cudaDeviceSynchronize());
    if (t.bf16 != nullptr) {
        if (*t.bf16 == nullptr) return fail(KMLL_ERR_STATE, "get_tensor: the model has no tensor %d in layer %d", tensor, layer);
        if (values) KMLL_CUDA(cudaMemcpy(values, *t.bf16, t.bf16_count * 2, cudaMemcpyDeviceToHost));
        return KMLL_OK;
    }
    size_t sb = 0;
    const size_t wb = qweight_bytes(d->cfg.format, t.q->rows, t.q->cols, &sb);
    if (values) KMLL_CUDA(cudaMemcpy(values, t.q->w, wb, cudaMemcpyDeviceToHost));
    if (scales) KMLL_CUDA(cudaMemcpy(scales, t.q->scales, sb, cudaMemcpyDeviceToHost));
    return KMLL_OK;
}

int kmll_tp_unique_id(unsigned char id_out[128]) {
    KMLL_REQUIRE_PTR(id_out);
    NcclApi* api = nccl_api();
    if (api == nullptr) return fail(KMLL_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded");
    ncclUniqueId id;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    if (api->GetUniqueId(&id) != ncclSuccess) return fail(KMLL_ERR_CUDA, "ncclGetUniqueId failed");
    memcpy(id_out, &id, 128);
    return KMLL_OK;
}

int kmll_decoder_tp_init(kmll_decoder_t dec, const unsigned char id[128]) {
    KMLL_REQUIRE_PTR(dec);
    KMLL_REQUIRE_PTR(id);
    Decoder* d = static_cast<Decoder*>(dec);
    if (d->cfg.tp_size == 1) return KMLL_OK;
    NcclApi* api = nccl_api();
    if (api == nullptr) return fail(KMLL_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded");
    ncclUniqueId nid;
    memcpy(&nid, id, 128);
    ncclResult_t r = api->CommInitRank(&d->comm, d->cfg.tp_size, nid, d->cfg.tp_rank);
    if (r != ncclSuccess) return fail(KMLL_ERR_CUDA, "ncclCommInitRank: %s", api->GetErrorString ? api->GetErrorString(r) : "error");
    const char* mode = std::getenv("KMLL_TP_EXCHANGE");  // "nccl" keeps the library collectives inside the decode step
    if (mode != nullptr && strcmp(mode, "nccl") == 0) {
        d->chain = false;  // the chained step hands its vectors over through exchange words only
        return KMLL_OK;
    }
    return setup_exchange(d);
}

int kmll_decoder_prefill_token_loop(kmll_decoder_t dec, kmll_stream_t stream, const uint32_t* tokens, int n_tokens) {
    KMLL_REQUIRE_PTR(dec);
    KMLL_REQUIRE_PTR(tokens);
    Decoder* d = static_cast<Decoder*>(dec);
    cudaStream_t s = as_stream(stream);
    KMLL_REQUIRE(n_tokens > 0 && n_tokens <= d->cfg.max_seq_len, "prefill: prompt length %d outside 1..max_seq_len %d", n_tokens, d->cfg.max_seq_len);
    if (!d->weights_set) return fail(KMLL_ERR_STATE, "decoder has no weights");
    for (int i = 0; i < n_tokens; ++i)
        KMLL_REQUIRE(tokens[i] < (uint32_t)d->cfg.vocab_size, "prefill: token %u out of range", tokens[i]);
    d->host_position = 0;
    d->have_next = false;
    for (int i = 0; i < n_tokens; ++i) {
        KMLL_TRY(enqueue_step_unfused(d, s, tokens[i], i));
        d->host_position = i + 1;
    }
    KMLL_CUDA(cudaMemcpyAsync(d->pinned, d->packed_final, 8, cudaMemcpyDeviceToHost, s));
    KMLL_CUDA(cudaStreamSynchronize(s));
    KMLL_TRY(write_state(d, s, n_tokens, 0, d->pinned[0]));
    KMLL_CUDA(cudaStreamSynchronize(s));
    d->have_next = true;
    return KMLL_OK;
}

int kmll_decoder_prefill(kmll_decoder_t dec, kmll_stream_t stream, const uint32_t* tokens, int n) {
    KMLL_REQUIRE_PTR(dec);
    KMLL_REQUIRE_PTR(tokens);
    Decoder* d = static_cast<Decoder*>(dec);
    const kmll_decoder_config& c = d->cfg;
    cudaStream_t s = as_stream(stream);
    KMLL_REQUIRE(n > 0 && n <= c.max_seq_len, "prefill: prompt length %d outside 1..max_seq_len %d", n, c.max_seq_len);
    if (!d->weights_set) return fail(KMLL_ERR_STATE, "decoder has no weights");
    for (int i = 0; i < n; ++i) KMLL_REQUIRE(tokens[i] < (uint32_t)c.vocab_size, "prefill: token %u out of range", tokens[i]);
    const int q_len = d->n_heads_l * c.head_dim, kv_len = d->n_kv_l * c.head_dim;
    d->host_position = 0;
    d->have_next = false;
    // batched scratch (prefill_batched_i8_hidden, crates/inference/src/model.rs:5849-5943)
    std::vector<void*> tmp;
    auto talloc = [&](float** p, size_t count) -> int {
        void* q = nullptr;
        cudaError_t e = cudaMalloc(&q, count * sizeof(float));
        if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "prefill scratch: %s", cudaGetErrorString(e));
        tmp.push_back(q);
        *p = (float*)q;
        return KMLL_OK;
    };
    float *xb = nullptr, *x2b = nullptr, *nb = nullptr, *ob = nullptr, *qb = nullptr, *kb = nullptr, *vb = nullptr, *qrb = nullptr,
          *ab = nullptr, *gb = nullptr, *ub = nullptr, *actb = nullptr;
    uint32_t* dtok = nullptr;
    auto body = [&]() -> int {
        KMLL_TRY(talloc(&xb, (size_t)n * c.dim));
        KMLL_TRY(talloc(&x2b, (size_t)n * c.dim));
        KMLL_TRY(talloc(&nb, (size_t)n * c.dim));
        KMLL_TRY(talloc(&ob, (size_t)n * c.dim));
        KMLL_TRY(talloc(&qb, (size_t)n * q_len));
        KMLL_TRY(talloc(&qrb, (size_t)n * q_len));
        KMLL_TRY(talloc(&ab, (size_t)n * q_len));
        KMLL_TRY(talloc(&kb, (size_t)n * kv_len));
        KMLL_TRY(talloc(&vb, (size_t)n * kv_len));
        KMLL_TRY(talloc(&gb, (size_t)n * d->hidden_l));
        KMLL_TRY(talloc(&ub, (size_t)n * d->hidden_l));
        KMLL_TRY(talloc(&actb, (size_t)n * d->hidden_l));
        float* tokf = nullptr;
        KMLL_TRY(talloc(&tokf, (size_t)n));
        dtok = (uint32_t*)tokf;
        // scratch of the batched linears (f16 planes of the activations), sized for the widest input
        float* wsf = nullptr;
        const int widest = d->hidden_l > c.dim ? (d->hidden_l > q_len ? d->hidden_l : q_len) : (c.dim > q_len ? c.dim : q_len);
        const size_t ws_bytes = kmll_linear_batched_workspace_bytes(n, widest);
        if (ws_bytes > 0) KMLL_TRY(talloc(&wsf, ws_bytes / sizeof(float) + 64));
        void* ws = wsf;
        KMLL_CUDA(cudaMemcpyAsync(dtok, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, s));
        KMLL_TRY(kmll_embedding_tokens(s, d->embedding, c.vocab_size, c.dim, dtok, n, xb));
        const bool w4 = c.format == KMLL_FORMAT_W4G128;
        for (int l = 0; l < c.n_layers; ++l) {
            Layer& L = d->layers[l];
            // run_prefill_rowwise_scaled_layer_device_with_cache, crates/inference/src/model.rs:9803-10017
            KMLL_TRY(kmll_rmsnorm_batched(s, xb, L.attention_norm, n, c.dim, c.norm_eps, nb));
            if (w4) {
                KMLL_TRY(kmll_linear_qkv_batched_w4g128(s, nb, (const uint8_t*)L.wq.w, (const uint16_t*)L.wq.scales, (const uint8_t*)L.wk.w,
                                                        (const uint16_t*)L.wk.scales, (const uint8_t*)L.wv.w, (const uint16_t*)L.wv.scales, n,
                                                        c.dim, q_len, kv_len, ws, qb, kb, vb));
            } else {
                KMLL_TRY(kmll_linear_qkv_batched_i8(s, nb, (const int8_t*)L.wq.w, (const float*)L.wq.scales, (const int8_t*)L.wk.w,
                                                    (const float*)L.wk.scales, (const int8_t*)L.wv.w, (const float*)L.wv.scales, n, c.dim,
                                                    q_len, kv_len, ws, qb, kb, vb));
            }
            KMLL_TRY(apply_qk_norm(d, s, L, qb, kb, n));
            KMLL_TRY(prepare_prefill_offset(s, qb, kb, vb, d->freqs, c.rotary_dim / 2, n, q_len, kv_len, c.head_dim, 0, qrb, L.key_cache,
                                            L.value_cache, c.kv_bf16));
            KMLL_TRY(prefill_attention_launch(s, qrb, L.key_cache, L.value_cache, n, d->n_heads_l, d->n_kv_l, c.head_dim, ab, c.kv_bf16,
                                              c.sliding_window, c.fused ? 1 : 0));  // fused = 0: kmll's f32 operator arithmetic throughout
            KMLL_TRY(op_linear_batched(d, s, ab, L.wo, n, ws, ob));
            KMLL_TRY(tp_allreduce(d, s, ob, (size_t)n * c.dim));
            KMLL_TRY(kmll_add_prefix(s, xb, ob, (size_t)n * c.dim, x2b));
            // run_ffn_batched_i8_from_hidden_into, crates/inference/src/model.rs:11326-11421
            KMLL_TRY(kmll_rmsnorm_batched(s, x2b, L.ffn_norm, n, c.dim, c.norm_eps, nb));
            KMLL_TRY(op_linear_batched(d, s, nb, L.w1, n, ws, gb));
            KMLL_TRY(op_linear_batched(d, s, nb, L.w3, n, ws, ub));
            KMLL_TRY(kmll_silu_mul_prefix(s, gb, ub, (size_t)n * d->hidden_l, actb));
            KMLL_TRY(op_linear_batched(d, s, actb, L.w2, n, ws, ob));
            KMLL_TRY(tp_allreduce(d, s, ob, (size_t)n * c.dim));
            KMLL_TRY(kmll_add_prefix(s, x2b, ob, (size_t)n * c.dim, xb));
        }
        KMLL_CUDA(cudaMemcpyAsync(d->hidden_a, xb + (size_t)(n - 1) * c.dim, sizeof(float) * c.dim, cudaMemcpyDeviceToDevice, s));
        KMLL_TRY(output_top1(d, s, d->hidden_a));
        KMLL_CUDA(cudaMemcpyAsync(d->pinned, d->packed_final, 8, cudaMemcpyDeviceToHost, s));
        KMLL_CUDA(cudaStreamSynchronize(s));
        KMLL_TRY(write_state(d, s, n, 0, d->pinned[0]));
        KMLL_CUDA(cudaStreamSynchronize(s));
        return KMLL_OK;
    };
    const int rc = body();
    cudaStreamSynchronize(s);
    for (void* p : tmp) cudaFree(p);
    if (rc != KMLL_OK) return rc;
    d->host_position = n;
    d->have_next = true;
    return KMLL_OK;
}

int kmll_decoder_enqueue_steps(kmll_decoder_t dec, kmll_stream_t stream, int n_steps) {
    KMLL_REQUIRE_PTR(dec);
    Decoder* d = static_cast<Decoder*>(dec);
    cudaStream_t s = as_stream(stream);
    if (!d->have_next) return fail(KMLL_ERR_STATE, "runtime must be prefilled before generation");
    KMLL_REQUIRE(n_steps >= 0, "generate: negative step count");
    if (d->host_position + n_steps > d->cfg.max_seq_len)
        return fail(KMLL_ERR_CAPACITY, "position %d exceeds max sequence length %d", d->host_position + n_steps, d->cfg.max_seq_len);
    if (!d->cfg.fused) return fail(KMLL_ERR_STATE, "enqueue_steps needs the fused (graph) path; use kmll_decoder_step_host");
    KMLL_TRY(ensure_graph(d, s));
    for (int i = 0; i < n_steps; ++i) {
        KMLL_CUDA(cudaGraphLaunch(d->graph, s));
        d->host_position += 1;
    }
    return KMLL_OK;
}

int kmll_decoder_generate_greedy(kmll_decoder_t dec, kmll_stream_t stream, int n_steps, uint32_t* tokens_out, float* logits_out) {
    KMLL_REQUIRE_PTR(dec);
    Decoder* d = static_cast<Decoder*>(dec);
    cudaStream_t s = as_stream(stream);
    if (!d->have_next) return fail(KMLL_ERR_STATE, "runtime must be prefilled before generation");
    KMLL_REQUIRE(n_steps >= 0 && n_steps <= d->history_cap, "generate: step count %d outside 0..%d", n_steps, d->history_cap);
    if (n_steps == 0) return KMLL_OK;
    std::vector<uint64_t> hist(n_steps);
    if (d->cfg.fused) {
        // restart the history index, keep position and pending token
        KMLL_CUDA(cudaStreamSynchronize(s));
        DecodeState st;
        KMLL_CUDA(cudaMemcpy(&st, d->state, sizeof(st), cudaMemcpyDeviceToHost));
        st.step = 0;
        KMLL_CUDA(cudaMemcpy(d->state, &st, sizeof(st), cudaMemcpyHostToDevice));
        KMLL_TRY(kmll_decoder_enqueue_steps(dec, stream, n_steps));
        KMLL_CUDA(cudaMemcpyAsync(hist.data(), d->history, sizeof(uint64_t) * n_steps, cudaMemcpyDeviceToHost, s));
        KMLL_CUDA(cudaStreamSynchronize(s));
    } else {
        uint64_t packed = 0;
        KMLL_TRY(kmll_decoder_next_top(dec, stream, &packed));
        for (int i = 0; i < n_steps; ++i) {
            hist[i] = packed;
            KMLL_TRY(kmll_decoder_step_host(dec, stream, (uint32_t)(packed & 0xffffffffull), &packed));
        }
    }
    for (int i = 0; i < n_steps; ++i) {
        if (tokens_out) tokens_out[i] = (uint32_t)(hist[i] & 0xffffffffull);
        if (logits_out) {
            const uint32_t bits = (uint32_t)(hist[i] >> 32);
            memcpy(&logits_out[i], &bits, 4);
        }
    }
    return KMLL_OK;
}

int kmll_decoder_history(kmll_decoder_t dec, kmll_stream_t stream, int first, int count, uint64_t* packed_out) {
    KMLL_REQUIRE_PTR(dec);
    KMLL_REQUIRE_PTR(packed_out);
    Decoder* d = static_cast<Decoder*>(dec);
    cudaStream_t s = as_stream(stream);
    KMLL_REQUIRE(first >= 0 && count >= 0 && first + count <= d->history_cap, "history: entries %d..%d outside 0..%d", first, first + count,
                 d->history_cap);
    if (count == 0) return KMLL_OK;
    KMLL_CUDA(cudaMemcpyAsync(packed_out, d->history + first, sizeof(uint64_t) * (size_t)count, cudaMemcpyDeviceToHost, s));
    KMLL_CUDA(cudaStreamSynchronize(s));
    return KMLL_OK;
}

int kmll_decoder_step_host(kmll_decoder_t dec, kmll_stream_t stream, uint32_t token, uint64_t* packed_out) {
    KMLL_REQUIRE_PTR(dec);
    KMLL_REQUIRE_PTR(packed_out);
    Decoder* d = static_cast<Decoder*>(dec);
    cudaStream_t s = as_stream(stream);
    if (!d->weights_set) return fail(KMLL_ERR_STATE, "decoder has no weights");
    KMLL_REQUIRE(token < (uint32_t)d->cfg.vocab_size, "step: token %u out of range", token);
    if (d->host_position >= d->cfg.max_seq_len)
        return fail(KMLL_ERR_CAPACITY, "position %d exceeds max sequence length %d", d->host_position, d->cfg.max_seq_len);
    if (d->cfg.fused) {
        KMLL_TRY(ensure_graph(d, s));
        // the token travels host -> device, the packed result device -> host, then the stream is
        // synchronised: the per-token traffic of kmll's own loop (crates/inference/src/model.rs:10655)
        d->pinned[0] = (uint64_t)token;
        KMLL_CUDA(cudaMemcpyAsync(&d->state->next_top, d->pinned, 8, cudaMemcpyHostToDevice, s));
        KMLL_CUDA(cudaGraphLaunch(d->graph, s));
        KMLL_CUDA(cudaMemcpyAsync(d->pinned + 1, &d->state->next_top, 8, cudaMemcpyDeviceToHost, s));
        KMLL_CUDA(cudaStreamSynchronize(s));
        *packed_out = d->pinned[1];
    } else {
        KMLL_TRY(enqueue_step_unfused(d, s, token, d->host_position));
        KMLL_CUDA(cudaMemcpyAsync(d->pinned + 1, d->packed_final, 8, cudaMemcpyDeviceToHost, s));
        KMLL_CUDA(cudaStreamSynchronize(s));
        *packed_out = d->pinned[1];
        KMLL_TRY(write_state(d, s, d->host_position + 1, 0, *packed_out));
    }
    d->host_position += 1;
    d->have_next = true;
    return KMLL_OK;
}

int kmll_decoder_next_top(kmll_decoder_t dec, kmll_stream_t stream, uint64_t* packed_out) {
    KMLL_REQUIRE_PTR(dec);
    KMLL_REQUIRE_PTR(packed_out);
    Decoder* d = static_cast<Decoder*>(dec);
    cudaStream_t s = as_stream(stream);
    if (!d->have_next) return fail(KMLL_ERR_STATE, "runtime must be prefilled before generation");
    KMLL_CUDA(cudaMemcpyAsync(d->pinned + 2, &d->state->next_top, 8, cudaMemcpyDeviceToHost, s));
    KMLL_CUDA(cudaStreamSynchronize(s));
    *packed_out = d->pinned[2];
    return KMLL_OK;
}

int kmll_decoder_rewind(kmll_decoder_t dec, kmll_stream_t stream, int position) {
    KMLL_REQUIRE_PTR(dec);
    Decoder* d = static_cast<Decoder*>(dec);
    cudaStream_t s = as_stream(stream);
    KMLL_REQUIRE(position >= 1 && position <= d->host_position, "rewind: position %d outside 1..%d", position, d->host_position);
    uint64_t packed = 0;
    KMLL_TRY(kmll_decoder_next_top(dec, stream, &packed));
    KMLL_TRY(write_state(d, s, position, 0, packed));
    KMLL_CUDA(cudaStreamSynchronize(s));
    d->host_position = position;
    return KMLL_OK;
}

int kmll_decoder_set_pending(kmll_decoder_t dec, kmll_stream_t stream, uint64_t packed) {
    KMLL_REQUIRE_PTR(dec);
    Decoder* d = static_cast<Decoder*>(dec);
    cudaStream_t s = as_stream(stream);
    if (!d->have_next) return fail(KMLL_ERR_STATE, "runtime must be prefilled before a pending token can be set");
    KMLL_REQUIRE((uint32_t)(packed & 0xffffffffull) < (uint32_t)d->cfg.vocab_size, "set_pending: token %u out of range",
                 (uint32_t)(packed & 0xffffffffull));
    KMLL_CUDA(cudaStreamSynchronize(s));
    KMLL_TRY(write_state(d, s, d->host_position, 0, packed));
    KMLL_CUDA(cudaStreamSynchronize(s));
    return KMLL_OK;
}

int kmll_decoder_position(kmll_decoder_t dec) { return dec ? static_cast<Decoder*>(dec)->host_position : 0; }

int kmll_decoder_last_hidden(kmll_decoder_t dec, kmll_stream_t stream, float* hidden_out) {
    KMLL_REQUIRE_PTR(dec);
    KMLL_REQUIRE_PTR(hidden_out);
    Decoder* d = static_cast<Decoder*>(dec);
    cudaStream_t s = as_stream(stream);
    KMLL_CUDA(cudaMemcpyAsync(hidden_out, d->hidden_a, sizeof(float) * d->cfg.dim, cudaMemcpyDeviceToHost, s));
    KMLL_CUDA(cudaStreamSynchronize(s));
    return KMLL_OK;
}

// Next-token logits of the sequence as it stands (final RMSNorm + lm_head over the last hidden state), into a device
// buffer of the caller: what kmll's next_logits_to_host / next_top_logits start from (crates/inference/src/model.rs:5319-5352).
int kmll_decoder_next_logits(kmll_decoder_t dec, kmll_stream_t stream, float* logits_device) {
    KMLL_REQUIRE_PTR(dec);
    KMLL_REQUIRE_PTR(logits_device);
    Decoder* d = static_cast<Decoder*>(dec);
    const kmll_decoder_config& c = d->cfg;
    if (c.tp_size > 1) return fail(KMLL_ERR_UNSUPPORTED, "next_logits: a tensor-parallel decoder holds a slice of the vocabulary per rank");
    cudaStream_t s = as_stream(stream);
    KMLL_TRY(kmll_rmsnorm(s, d->hidden_a, d->final_norm, c.dim, c.norm_eps, d->normed));
    if (c.format == KMLL_FORMAT_W4G128)
        return kmll_linear_w4g128(s, d->normed, static_cast<const uint8_t*>(d->output.w), static_cast<const uint16_t*>(d->output.scales), c.vocab_size,
                                  c.dim, logits_device);
    return kmll_linear_i8(s, d->normed, static_cast<const int8_t*>(d->output.w), static_cast<const float*>(d->output.scales), c.vocab_size, c.dim,
                          logits_device);
}

// Replace the rotation frequencies (rotary_dim / 2 values; e.g. a YaRN-scaled table, crates/inference/src/model.rs:9257-9306).
// They are read by kernels on every step, so the call synchronises the device first.
int kmll_decoder_set_rope_freqs(kmll_decoder_t dec, const float* freqs_host, int count) {
    KMLL_REQUIRE_PTR(dec);
    KMLL_REQUIRE_PTR(freqs_host);
    Decoder* d = static_cast<Decoder*>(dec);
    KMLL_REQUIRE(count == d->cfg.rotary_dim / 2, "set_rope_freqs: %d values given, rotary_dim / 2 = %d expected", count, d->cfg.rotary_dim / 2);
    for (int i = 0; i < count; ++i)
        if (!std::isfinite(freqs_host[i])) return fail(KMLL_ERR_SHAPE, "set_rope_freqs: value %d is not finite", i);
    KMLL_CUDA(cudaDeviceSynchronize());
    KMLL_CUDA(cudaMemcpy(d->freqs, freqs_host, sizeof(float) * count, cudaMemcpyHostToDevice));
    return KMLL_OK;
}

size_t kmll_decoder_resident_bytes(kmll_decoder_t dec) { return dec ? static_cast<Decoder*>(dec)->resident_bytes : 0; }
int kmll_decoder_launches_per_step(kmll_decoder_t dec) { return dec ? static_cast<Decoder*>(dec)->launches_per_step : 0; }
size_t kmll_decoder_weight_bytes(kmll_decoder_t dec) { return dec ? static_cast<Decoder*>(dec)->weight_bytes : 0; }
size_t kmll_decoder_kv_bytes(kmll_decoder_t dec) { return dec ? static_cast<Decoder*>(dec)->kv_bytes : 0; }

int kmll_batch_destroy(kmll_batch_t batch) {
    if (batch == nullptr) return KMLL_OK;
    BatchDecoder* b = static_cast<BatchDecoder*>(batch);
    if (b->graph) cudaGraphExecDestroy(b->graph);
    if (b->capture_stream) cudaStreamDestroy(b->capture_stream);
    for (void* p : b->allocs) cudaFree(p);
    delete b;
    return KMLL_OK;
}

int kmll_batch_create(kmll_decoder_t dec, int batch, kmll_batch_t* out) {
    KMLL_REQUIRE_PTR(dec);
    KMLL_REQUIRE_PTR(out);
    Decoder* d = static_cast<Decoder*>(dec);
    const kmll_decoder_config& c = d->cfg;
    KMLL_REQUIRE(batch >= 1 && batch <= kMaxBatch, "batch %d outside 1..%d", batch, kMaxBatch);
    if (c.tp_size != 1) return fail(KMLL_ERR_UNSUPPORTED, "batched decode is single-GPU");
    if (c.rotary_dim != c.head_dim) return fail(KMLL_ERR_UNSUPPORTED, "batched decode needs rotary_dim == head_dim");
    if ((c.head_dim != 64 && c.head_dim != 128) || c.n_heads / c.n_kv_heads > 8)
        return fail(KMLL_ERR_UNSUPPORTED, "batched decode needs head_dim 64 or 128 and at most 8 query heads per KV head");
    BatchDecoder* b = new BatchDecoder();
    b->d = d;
    b->batch = batch;
    auto body = [&]() -> int {
        const int q_len = c.n_heads * c.head_dim, kv_len = c.n_kv_heads * c.head_dim;
        b->cache_stride = (size_t)c.max_seq_len * kv_len;  // elements (f32, or bf16 with kv_bf16) between two sequences
        const size_t cache_floats = b->cache_stride * batch / (c.kv_bf16 ? 2 : 1);
        b->key_cache.resize(c.n_layers);
        b->value_cache.resize(c.n_layers);
        for (int l = 0; l < c.n_layers; ++l) {
            KMLL_TRY(balloc(b, &b->key_cache[l], cache_floats));
            KMLL_TRY(balloc(b, &b->value_cache[l], cache_floats));
            KMLL_CUDA(cudaMemset(b->key_cache[l], 0, cache_floats * sizeof(float)));
            KMLL_CUDA(cudaMemset(b->value_cache[l], 0, cache_floats * sizeof(float)));
        }
        KMLL_TRY(balloc(b, &b->hidden_a, (size_t)batch * c.dim));
        KMLL_TRY(balloc(b, &b->hidden_b, (size_t)batch * c.dim));
        KMLL_TRY(balloc(b, &b->hidden_mid, (size_t)batch * c.dim));
        KMLL_TRY(balloc(b, &b->q, (size_t)batch * q_len));
        KMLL_TRY(balloc(b, &b->attn, (size_t)batch * q_len));
        KMLL_TRY(balloc(b, &b->k, (size_t)batch * kv_len));
        KMLL_TRY(balloc(b, &b->v, (size_t)batch * kv_len));
        KMLL_TRY(balloc(b, &b->act, (size_t)batch * c.hidden_dim));
        KMLL_TRY(balloc(b, &b->gate, (size_t)batch * c.hidden_dim));
        KMLL_TRY(balloc(b, &b->up, (size_t)batch * c.hidden_dim));
        {
            const int widest = c.hidden_dim > c.dim ? (c.hidden_dim > q_len ? c.hidden_dim : q_len) : (c.dim > q_len ? c.dim : q_len);
            const size_t ws_bytes = linear_batched_workspace_bytes(batch, widest);
            if (ws_bytes > 0) {
                unsigned char* p = nullptr;
                KMLL_TRY(balloc(b, &p, ws_bytes));
                b->linear_ws = p;
            }
        }
        KMLL_TRY(balloc(b, &b->logits, (size_t)batch * c.vocab_size));
        const size_t ws = (decode_attention_workspace_floats(c.n_heads, c.head_dim, c.max_seq_len) + 3) & ~(size_t)3;
        KMLL_TRY(balloc(b, &b->attn_ws, ws * batch));
        KMLL_CUDA(cudaMemset(b->attn_ws, 0, ws * batch * sizeof(float)));
        KMLL_TRY(balloc(b, &b->state, (size_t)1));
        KMLL_CUDA(cudaMemset(b->state, 0, sizeof(BatchState)));
        b->history_cap = c.max_seq_len;
        KMLL_TRY(balloc(b, &b->history, (size_t)batch * b->history_cap));
        return KMLL_OK;
    };
    const int rc = body();
    if (rc != KMLL_OK) {
        kmll_batch_destroy(b);
        return rc;
    }
    *out = b;
    return KMLL_OK;
}

int kmll_batch_adopt(kmll_batch_t batch, kmll_stream_t stream, int slot) {
    KMLL_REQUIRE_PTR(batch);
    BatchDecoder* b = static_cast<BatchDecoder*>(batch);
    Decoder* d = b->d;
    cudaStream_t s = as_stream(stream);
    KMLL_REQUIRE(slot >= 0 && slot < b->batch, "slot %d outside 0..%d", slot, b->batch - 1);
    if (!d->have_next) return fail(KMLL_ERR_STATE, "the decoder must be prefilled before its sequence can be adopted");
    if (b->filled != 0 && d->host_position != b->host_position)
        return fail(KMLL_ERR_STATE, "sequences of a batch advance in lockstep: slot at position %d, batch at %d", d->host_position,
                    b->host_position);
    const kmll_decoder_config& c = d->cfg;
    const size_t kv_len = (size_t)c.n_kv_heads * c.head_dim;
    const size_t esz = c.kv_bf16 ? 2 : sizeof(float);
    const size_t bytes = (size_t)d->host_position * kv_len * esz, slot_at = (size_t)slot * b->cache_stride * esz;
    for (int l = 0; l < c.n_layers; ++l) {
        KMLL_CUDA(cudaMemcpyAsync(reinterpret_cast<char*>(b->key_cache[l]) + slot_at, d->layers[l].key_cache, bytes, cudaMemcpyDeviceToDevice, s));
        KMLL_CUDA(cudaMemcpyAsync(reinterpret_cast<char*>(b->value_cache[l]) + slot_at, d->layers[l].value_cache, bytes, cudaMemcpyDeviceToDevice, s));
    }
    KMLL_CUDA(cudaMemcpyAsync(&b->state->next_top[slot], &d->state->next_top, sizeof(uint64_t), cudaMemcpyDeviceToDevice, s));
    if (b->filled == 0) {
        int head[4] = {d->host_position, d->host_position + 1, 0, 0};
        KMLL_CUDA(cudaMemcpyAsync(b->state, head, sizeof(head), cudaMemcpyHostToDevice, s));
        KMLL_CUDA(cudaStreamSynchronize(s));  // `head` lives on this stack frame
        b->host_position = d->host_position;
    }
    b->filled |= 1u << slot;
    return KMLL_OK;
}

int kmll_batch_enqueue_steps(kmll_batch_t batch, kmll_stream_t stream, int n_steps) {
    KMLL_REQUIRE_PTR(batch);
    BatchDecoder* b = static_cast<BatchDecoder*>(batch);
    cudaStream_t s = as_stream(stream);
    if (b->filled != (b->batch >= 32 ? 0xffffffffu : ((1u << b->batch) - 1u)))
        return fail(KMLL_ERR_STATE, "every slot of the batch must hold a sequence (kmll_batch_adopt)");
    KMLL_REQUIRE(n_steps >= 0, "generate: negative step count");
    if (b->host_position + n_steps > b->d->cfg.max_seq_len)
        return fail(KMLL_ERR_CAPACITY, "position %d exceeds max sequence length %d", b->host_position + n_steps, b->d->cfg.max_seq_len);
    KMLL_TRY(ensure_batch_graph(b, s));
    for (int i = 0; i < n_steps; ++i) {
        KMLL_CUDA(cudaGraphLaunch(b->graph, s));
        b->host_position += 1;
    }
    return KMLL_OK;
}

int kmll_batch_generate_greedy(kmll_batch_t batch, kmll_stream_t stream, int n_steps, uint32_t* tokens_out, float* logits_out) {
    KMLL_REQUIRE_PTR(batch);
    BatchDecoder* b = static_cast<BatchDecoder*>(batch);
    cudaStream_t s = as_stream(stream);
    KMLL_REQUIRE(n_steps >= 0 && n_steps <= b->history_cap, "generate: step count %d outside 0..%d", n_steps, b->history_cap);
    if (n_steps == 0) return KMLL_OK;
    // restart the history index, keep position and pending tokens
    KMLL_CUDA(cudaStreamSynchronize(s));
    int head[4];
    KMLL_CUDA(cudaMemcpy(head, b->state, sizeof(head), cudaMemcpyDeviceToHost));
    head[2] = 0;
    KMLL_CUDA(cudaMemcpy(b->state, head, sizeof(head), cudaMemcpyHostToDevice));
    KMLL_TRY(kmll_batch_enqueue_steps(batch, stream, n_steps));
    std::vector<uint64_t> hist((size_t)b->batch * b->history_cap);
    KMLL_CUDA(cudaMemcpyAsync(hist.data(), b->history, hist.size() * sizeof(uint64_t), cudaMemcpyDeviceToHost, s));
    KMLL_CUDA(cudaStreamSynchronize(s));
    for (int q = 0; q < b->batch; ++q)
        for (int i = 0; i < n_steps; ++i) {
            const uint64_t h = hist[(size_t)q * b->history_cap + i];
            if (tokens_out) tokens_out[(size_t)q * n_steps + i] = (uint32_t)(h & 0xffffffffull);
            if (logits_out) {
                const uint32_t bits = (uint32_t)(h >> 32);
                memcpy(&logits_out[(size_t)q * n_steps + i], &bits, 4);
            }
        }
    return KMLL_OK;
}

int kmll_batch_position(kmll_batch_t batch) {
    if (batch == nullptr) return -1;
    return static_cast<BatchDecoder*>(batch)->host_position;
}
int kmll_batch_launches_per_step(kmll_batch_t batch) {
    if (batch == nullptr) return 0;
    return static_cast<BatchDecoder*>(batch)->launches_per_step;
}

}  // extern "C"
