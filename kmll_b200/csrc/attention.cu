// Attention operators of the decode path.
//   * attention_scores / softmax_value: the two-kernel split form of kmll
//     (crates/inference/src/kernels/inference.rs:1165-1222, :1311-1417), any head_dim.
//   * single_query_attention: decode attention, split along the sequence so that the whole GPU
//     streams the f32 KV cache ("flash-decoding"); the query heads that share a KV head are
//     processed together so K and V are read from HBM exactly once.  The last block to finish a
//     KV head merges the per-split partial results.
//   * prefill_causal_attention: tiled causal attention with an online softmax.
// Math contract (all f32): score = dot * (1/sqrt(head_dim)); weights exp(s - max); out = sum(w*v)/sum(w)
// (crates/inference/src/model.rs:11581-11649).  KV cache layout [max_seq, n_kv_heads, head_dim].
#include <mutex>

#include "internal.cuh"

namespace kmll {

// ---- split form -------------------------------------------------------------------------------
__global__ void attention_scores_kernel(const float* __restrict__ q, const float* __restrict__ k_cache, int seq_len,
                                        int max_seq_len, int n_heads, int n_kv_heads, int head_dim,
                                        float* __restrict__ scores) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= n_heads * seq_len) return;
    const int head = item / seq_len;
    const int pos = item - head * seq_len;
    const int kv_head = head / (n_heads / n_kv_heads);
    const float* qh = q + (size_t)head * head_dim;
    const float* kr = k_cache + ((size_t)pos * n_kv_heads + kv_head) * head_dim;
    float dot = 0.0f;
    for (int d = lane; d < head_dim; d += 32) dot += qh[d] * kr[d];
    dot = warp_sum(dot);
    if (lane == 0) scores[(size_t)head * max_seq_len + pos] = dot * (1.0f / sqrtf((float)head_dim));
}

__global__ void __launch_bounds__(256) softmax_value_kernel(const float* __restrict__ scores,
                                                            const float* __restrict__ v_cache, int seq_len,
                                                            int max_seq_len, int n_heads, int n_kv_heads, int head_dim,
                                                            float* __restrict__ out) {
    __shared__ float scratch[40];
    pdl_wait();
    const int head = blockIdx.x;
    const int kv_head = head / (n_heads / n_kv_heads);
    const float* sc = scores + (size_t)head * max_seq_len;
    float m = -INFINITY;
    for (int p = threadIdx.x; p < seq_len; p += blockDim.x) m = fmaxf(m, sc[p]);
    m = block_max(m, scratch);
    float denom = 0.0f;
    for (int p = threadIdx.x; p < seq_len; p += blockDim.x) denom += expf(sc[p] - m);
    denom = block_sum(denom, scratch);
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float acc = 0.0f;
        for (int p = 0; p < seq_len; ++p)
            acc += expf(sc[p] - m) * v_cache[((size_t)p * n_kv_heads + kv_head) * head_dim + d];
        out[(size_t)head * head_dim + d] = acc / denom;
    }
}

// ---- decode attention, split along the sequence ---------------------------------------------------
constexpr int kAttnWarps = 8;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kAttnTile = 64;  // positions staged in shared memory at a time
constexpr int kMaxGq = 8;      // query heads per KV head handled by the fused kernel

struct DecodeAttnParams {
    const float* q;        // [n_heads, head_dim]
    const float* k_cache;  // [max_seq, n_kv, head_dim]
    const float* v_cache;
    const int* seq_len_ptr;  // device-side sequence length (CUDA-graph replays), or null
    int seq_len;             // used when seq_len_ptr is null
    int n_heads, n_kv_heads, gq;
    int chunk;    // positions per block
    int nsplit;   // gridDim.y
    int window;   // sliding window: only the last `window` positions are attended (0: all of them)
    float* part_acc;  // [n_heads, nsplit, HD]
    float* part_ml;   // [n_heads, nsplit, 2]
    unsigned int* counters;  // [n_kv_heads], zero on entry, zero on exit
    float* out;       // [n_heads, head_dim]
    // fused form (prepare_incremental_attention folded in): q is NOT yet rotated; the new K / V rows of
    // position seq_len-1 are rotated / copied into the caches by the block whose slice holds that position
    const float* k_new;   // [n_kv, head_dim] or null
    const float* v_new;
    const float* freqs;   // [head_dim / 2]
    float* k_cache_w;
    float* v_cache_w;
    unsigned long long* trace;  // timeline slot of this launch, or null
    // batch of independent sequences in lockstep (blockIdx.z = sequence): element strides between sequences
    size_t q_stride, new_stride, cache_stride, ws_stride, out_stride;
};

// Half-split RoPE of a head slice held 4 (or 2) consecutive dims per lane: the partner dim d +- HD/2 lives
// in lane ^ 16 (crates/inference/src/kernels/inference.rs:1078-1098 with rotary_dim == head_dim).
// `cs_sn` holds (cos, sin) of position * freqs[pair] for the HD/2 pairs, computed once per block.
template <int EPL>
__device__ inline void rope_lane_slice(float (&x)[EPL], const float2* cs_sn, int lane) {
    constexpr int HALF_LANES = 16;
    const bool upper = lane >= HALF_LANES;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, x[e], HALF_LANES);
        const float2 t = cs_sn[(lane & (HALF_LANES - 1)) * EPL + e];
        x[e] = upper ? x[e] * t.x + other * t.y : x[e] * t.x - other * t.y;
    }
}

template <int EPL>
__device__ inline void load_lane_slice(const float* src, float (&dst)[EPL]);
template <>
__device__ inline void load_lane_slice<4>(const float* src, float (&dst)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(src);
    dst[0] = t.x; dst[1] = t.y; dst[2] = t.z; dst[3] = t.w;
}
template <>
__device__ inline void load_lane_slice<2>(const float* src, float (&dst)[2]) {
    const float2 t = *reinterpret_cast<const float2*>(src);
    dst[0] = t.x; dst[1] = t.y;
}

__device__ inline void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src)
                 : "memory");
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ inline void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// End of a block of the decode attention kernels.  On entry `red` holds NW planes [gq][HD] of un-normalised
// accumulators (summed here) and hstat[h * 4], hstat[h * 4 + 1] the block's running max and sum per head, all
// visible to the block.  Writes the result (one split) or this split's partial; the last block of each KV head to
// arrive merges the partials.  `scratch` is shared memory of at least 3 * GQM * 64 + GQM floats that is free.
template <int HD, int GQM, int NW>
__device__ __forceinline__ void finish_split(const DecodeAttnParams& p, int kv_head, int split, int nactive, float* red,
                                             float* hstat, float* scratch, bool* is_last) {
    constexpr int EPL = HD / 32;
    const int gq = p.gq;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* const Ks = scratch;
    float acc[GQM][EPL];
    pdl_launch_dependents();

    // write this split's partial (or the final result when there is a single split)
#pragma unroll 1
    for (int idx = tid; idx < gq * HD; idx += kAttnThreads) {
        const int h = idx / HD, d = idx - h * HD;
        const int head = kv_head * gq + h;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; ++w) v += red[(w * gq + h) * HD + d];
        if (p.nsplit == 1) {
            p.out[(size_t)head * HD + d] = v / hstat[h * 4 + 1];
        } else {
            p.part_acc[((size_t)head * p.nsplit + split) * HD + d] = v;
            if (d == 0) {
                p.part_ml[((size_t)head * p.nsplit + split) * 2] = hstat[h * 4];
                p.part_ml[((size_t)head * p.nsplit + split) * 2 + 1] = hstat[h * 4 + 1];
            }
        }
    }
    trace_stamp(p.trace, 3);
    if (p.nsplit == 1) return;

    // last block of this KV head merges the splits
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int prev = atomicAdd(&p.counters[kv_head], 1u);
        *is_last = (prev == (unsigned int)nactive - 1);
    }
    __syncthreads();
    if (!*is_last) return;
    __threadfence();
    // merge: bring every split's (max, sum) into shared memory, derive the weights exp(m_s - m) once per head,
    // then combine the partial accumulators - warp w takes splits w, w+8, ... for all heads, so every load of a
    // round is independent of the others and a handful of L2 round trips cover the whole merge
    float* ml_s = Ks;                       // [gq][nsplit][2]
    float* f_s = Ks + 2 * GQM * 64;      // [gq][nsplit] weights, then [gq] denominators after them
    float* l_s = f_s + GQM * 64;
    const int ns = nactive;  // only these splits wrote partials
    // the first round of partial accumulators (splits w, w+8, w+16, w+24) is requested before the statistics are even
    // loaded, so that both L2 round trips overlap (only where the registers allow it: 4 heads x 4 floats per lane)
    constexpr bool kHoist = (GQM == 4 && EPL == 4);
    float4 early[kHoist ? 4 : 1][kHoist ? GQM : 1];
    if (kHoist) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int sp = warp + kAttnWarps * i;
#pragma unroll
            for (int h = 0; h < GQM; ++h) {
                early[kHoist ? i : 0][kHoist ? h : 0] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (h < gq && sp < ns)
                    early[kHoist ? i : 0][kHoist ? h : 0] = __ldcg(reinterpret_cast<const float4*>(
                        p.part_acc + ((size_t)(kv_head * gq + h) * p.nsplit + sp) * HD + lane * EPL));
            }
        }
    }
#pragma unroll 1
    for (int idx = tid; idx < gq * ns * 2; idx += kAttnThreads) {
        const int h = idx / (ns * 2), r = idx - h * ns * 2;
        ml_s[idx] = __ldcg(p.part_ml + (size_t)(kv_head * gq + h) * p.nsplit * 2 + r);
    }
    __syncthreads();
    if (warp < gq) {
        const int h = warp;
        const float m_a = lane < ns ? ml_s[(h * ns + lane) * 2] : -INFINITY;
        const float m_b = lane + 32 < ns ? ml_s[(h * ns + lane + 32) * 2] : -INFINITY;
        const float m = warp_max(fmaxf(m_a, m_b));
        const float f_a = m_a == -INFINITY ? 0.0f : expf(m_a - m), f_b = m_b == -INFINITY ? 0.0f : expf(m_b - m);
        float l = 0.0f;
        if (lane < ns) { f_s[h * ns + lane] = f_a; l += ml_s[(h * ns + lane) * 2 + 1] * f_a; }
        if (lane + 32 < ns) { f_s[h * ns + lane + 32] = f_b; l += ml_s[(h * ns + lane + 32) * 2 + 1] * f_b; }
        l = warp_sum(l);
        if (lane == 0) l_s[h] = l;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < GQM; ++h)
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[h][e] = 0.0f;
    if (kHoist) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int sp = warp + kAttnWarps * i;
#pragma unroll
            for (int h = 0; h < GQM; ++h)
                if (h < gq && sp < ns) {
                    const float4 t4 = early[kHoist ? i : 0][kHoist ? h : 0];
                    const float f = f_s[h * ns + sp];
                    acc[h][0] = fmaf(t4.x, f, acc[h][0]);
                    acc[h][1] = fmaf(t4.y, f, acc[h][1]);
                    acc[h][EPL - 2] = fmaf(t4.z, f, acc[h][EPL - 2]);
                    acc[h][EPL - 1] = fmaf(t4.w, f, acc[h][EPL - 1]);
                }
        }
    }
#pragma unroll(GQM == 4 ? 4 : 2)
    for (int s = warp + (kHoist ? 4 * kAttnWarps : 0); s < ns; s += kAttnWarps) {
#pragma unroll
        for (int h = 0; h < GQM; ++h)
            if (h < gq) {
                float pv[EPL];
                const float* src = p.part_acc + ((size_t)(kv_head * gq + h) * p.nsplit + s) * HD + lane * EPL;
                if (EPL == 4) {
                    const float4 t4 = __ldcg(reinterpret_cast<const float4*>(src));
                    pv[0] = t4.x; pv[1] = t4.y; pv[EPL - 2] = t4.z; pv[EPL - 1] = t4.w;
                } else {
                    const float2 t2 = __ldcg(reinterpret_cast<const float2*>(src));
                    pv[0] = t2.x; pv[1] = t2.y;
                }
                const float f = f_s[h * ns + s];
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[h][e] = fmaf(pv[e], f, acc[h][e]);
            }
    }
#pragma unroll
    for (int h = 0; h < GQM; ++h)
        if (h < gq)
#pragma unroll
            for (int e = 0; e < EPL; ++e) red[(warp * gq + h) * HD + lane * EPL + e] = acc[h][e];
    __syncthreads();
#pragma unroll 1
    for (int idx = tid; idx < gq * HD; idx += kAttnThreads) {
        const int h = idx / HD, d = idx - h * HD;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) v += red[(w * gq + h) * HD + d];
        p.out[(size_t)(kv_head * gq + h) * HD + d] = v / l_s[h];
    }
    if (tid == 0) p.counters[kv_head] = 0;  // leave the counter area zero for the next call
    trace_stamp(p.trace, 4);
}

// One block = one KV head x one slice of the sequence.  The K and V rows of up to 64 positions are
// brought into shared memory with 16-byte asynchronous copies that are all issued up front
// (64 KB in flight per block, two blocks per SM), so the f32 KV cache streams at HBM rate; the
// query heads sharing the KV head are processed together, so K and V are read once.
// In the fused form the copies are issued BEFORE the wait on the previous kernel: rows below
// seq_len - 1 were written by earlier steps, and the sequence length by a kernel at least two launches back.
// GQM bounds the query heads per KV head at compile time (4 or 8): the per-head register arrays and unrolled
// loops are sized by it.
template <int HD, int GQM>
__global__ void __launch_bounds__(kAttnThreads, 2) decode_attention_kernel(const DecodeAttnParams p_in) {
    DecodeAttnParams p = p_in;
    constexpr size_t ESZ = 4;  // bytes per cache element (the bf16 cache has a kernel of its own)
    if (gridDim.z > 1) {  // sequence blockIdx.z of a batch: shift every per-sequence operand
        const size_t b = blockIdx.z;
        const size_t cache_shift = b * p.cache_stride * ESZ;
        p.q += b * p.q_stride;
        p.out += b * p.out_stride;
        p.k_cache = reinterpret_cast<const float*>(reinterpret_cast<const char*>(p.k_cache) + cache_shift);
        p.v_cache = reinterpret_cast<const float*>(reinterpret_cast<const char*>(p.v_cache) + cache_shift);
        if (p.k_new != nullptr) {
            p.k_new += b * p.new_stride;
            p.v_new += b * p.new_stride;
            p.k_cache_w = reinterpret_cast<float*>(reinterpret_cast<char*>(p.k_cache_w) + cache_shift);
            p.v_cache_w = reinterpret_cast<float*>(reinterpret_cast<char*>(p.v_cache_w) + cache_shift);
        }
        p.part_acc += b * p.ws_stride;
        p.part_ml += b * p.ws_stride;
        p.counters += b * p.ws_stride;
    }
    constexpr int EPL = HD / 32;        // elements per lane
    constexpr int V16 = HD * (int)ESZ / 16;  // 16-byte pieces per row
    constexpr int KP = HD + 16;         // padded K row (elements): the score pass reads its pieces at stride KP conflict-free
    constexpr int KROWB = KP * (int)ESZ, VROWB = HD * (int)ESZ;  // bytes per staged K / V row
    extern __shared__ __align__(16) float smem[];
    float* Ks = smem;                         // [kAttnTile][KP]   
    float* Vs = Ks + kAttnTile * KP;          // [kAttnTile][HD]
    char* const Kb = reinterpret_cast<char*>(Ks);
    char* const Vb = reinterpret_cast<char*>(Vs);
    float* sc = Vs + kAttnTile * HD;          // [GQM][kAttnTile] scores, then weights
    float* hstat = sc + GQM * kAttnTile;   // [GQM][4]: running max, running sum, correction
    float* qs = hstat + GQM * 4;           // [GQM][HD] rotated query heads
    float* red = Vs;                          // [kAttnWarps][gq][HD] (reuses the V tile at the end)
    __shared__ bool is_last;
    __shared__ float2 cs_sn[HD / 2];  // fused form: (cos, sin) of the rotation angles of this position

    trace_stamp(p.trace, 0);
    const int kv_head = blockIdx.x, gq = p.gq;
    int split = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t kv_stride = (size_t)p.n_kv_heads * HD;
    const bool fused = p.k_new != nullptr;
    // this block's positions: its slice of the sequence, cut to [first attended position, seq_len)
    int s0 = split * p.chunk;
    int seq_len = 0, n = 0, first_split = 0;
    auto set_range = [&]() {
        seq_len = p.seq_len_ptr ? *p.seq_len_ptr : p.seq_len;
        const int lo = (p.window > 0 && seq_len > p.window) ? seq_len - p.window : 0;
        first_split = lo / p.chunk;  // splits before it hold no attended position and leave at once
        const int slice_end = min(s0 + p.chunk, seq_len);
        s0 = max(s0, lo);
        n = slice_end - s0;
    };
    // one commit group per K tile and per V tile (also when the tile does not exist, so the group count is uniform)
    auto issue_k = [&](int t0) {
        const int nt = min(kAttnTile, n - t0);
        const char* kg = reinterpret_cast<const char*>(p.k_cache) + ((size_t)(s0 + t0) * kv_stride + (size_t)kv_head * HD) * ESZ;
#pragma unroll 2
        for (int i = tid; i < nt * V16; i += kAttnThreads) {
            const int r = i / V16, cidx = i - r * V16;
            cp_async16(Kb + r * KROWB + cidx * 16, kg + (size_t)r * kv_stride * ESZ + cidx * 16);
        }
        cp_async_commit();
    };
    auto issue_v = [&](int t0) {
        const int nt = min(kAttnTile, n - t0);
        const char* vg = reinterpret_cast<const char*>(p.v_cache) + ((size_t)(s0 + t0) * kv_stride + (size_t)kv_head * HD) * ESZ;
#pragma unroll 2
        for (int i = tid; i < nt * V16; i += kAttnThreads) {
            const int r = i / V16, cidx = i - r * V16;
            cp_async16(Vb + r * VROWB + cidx * 16, vg + (size_t)r * kv_stride * ESZ + cidx * 16);
        }
        cp_async_commit();
    };
    if (fused) {
        set_range();
        if (n > 0) {
            issue_k(0);
            issue_v(0);
            // rotation angles depend on the position only: one sine / cosine evaluation per pair and block, done
            // while the copies are in flight and before the query exists (the accurate sincosf is long code)
            if (tid < HD / 2) {
                float sn, cs;
                sincosf((float)(seq_len - 1) * p.freqs[tid], &sn, &cs);
                cs_sn[tid] = make_float2(cs, sn);
            }
        }
    }
    if (tid < GQM) { hstat[tid * 4] = -INFINITY; hstat[tid * 4 + 1] = 0.0f; hstat[tid * 4 + 2] = 1.0f; }
    pdl_wait();
    trace_stamp(p.trace, 1);
    if (!fused) set_range();
    const int nactive = (seq_len + p.chunk - 1) / p.chunk - first_split;  // splits that hold attended positions
    if (n <= 0) return;
    split -= first_split;  // index of this block's partial among the active splits
    const float scale = 1.0f / sqrtf((float)HD);

    // Everything this block needs from the previous kernel is requested at once: the query heads (warp h loads
    // head h) and, in the block whose slice holds the position being written, the new K and V rows (warps 6 and 7).
    const int newpos = seq_len - 1 - s0;  // position being written, relative to this block's slice
    const bool owns_new = fused && newpos >= 0 && newpos < n;
    float qh[EPL], kvn[EPL];
    if (warp < gq) load_lane_slice<EPL>(p.q + (size_t)(kv_head * gq + warp) * HD + lane * EPL, qh);
    if (owns_new && warp == kAttnWarps - 2) load_lane_slice<EPL>(p.k_new + (size_t)kv_head * HD + lane * EPL, kvn);
    if (owns_new && warp == kAttnWarps - 1) load_lane_slice<EPL>(p.v_new + (size_t)kv_head * HD + lane * EPL, kvn);
    if (fused) __syncthreads();  // cs_sn is visible
    if (warp < gq) {
        if (fused) rope_lane_slice<EPL>(qh, cs_sn, lane);
#pragma unroll
        for (int e = 0; e < EPL; ++e) qs[warp * HD + lane * EPL + e] = qh[e];
    }
    if (owns_new && warp == kAttnWarps - 2) rope_lane_slice<EPL>(kvn, cs_sn, lane);

    float acc[GQM][EPL];
#pragma unroll
    for (int h = 0; h < GQM; ++h)
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[h][e] = 0.0f;

#pragma unroll 1
    for (int t0 = 0; t0 < n; t0 += kAttnTile) {
        const int nt = min(kAttnTile, n - t0);
        __syncthreads();  // the previous V tile has been consumed (first tile: qs / hstat are written)
        // Copies run one phase ahead of their use: the V tile of this iteration is requested as soon as the previous
        // one has been consumed, the next K tile as soon as the scores below are done.  The first tile of the fused
        // form was requested before the dependency wait.
        if (t0 == 0) {
            if (!fused) { issue_k(0); issue_v(0); }
        } else {
            issue_v(t0);
        }
        cp_async_wait<1>();  // K has landed (at most the V tile is still in flight)
        __syncthreads();
        const int newrow = newpos - t0;  // row of this tile that is the position being written
        const bool has_new = owns_new && newrow >= 0 && newrow < nt;
        if (has_new && warp == kAttnWarps - 2) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                const size_t at = (size_t)(seq_len - 1) * kv_stride + (size_t)kv_head * HD + lane * EPL + e;
                Ks[newrow * KP + lane * EPL + e] = kvn[e];
                p.k_cache_w[at] = kvn[e];
            }
        }
        if (has_new) __syncthreads();
        // scores: four lanes per position, each over an interleaved quarter of the head dimension
        {
            const int pl = tid >> 2, c = tid & 3;
            float4 kk[HD / 16];
            const float* kr = Ks + (pl < nt ? pl : 0) * KP + c * 4;
#pragma unroll
            for (int i = 0; i < HD / 16; ++i) kk[i] = *reinterpret_cast<const float4*>(kr + i * 16);
#pragma unroll 1
            for (int h = 0; h < gq; ++h) {
                const float* qr = qs + h * HD + c * 4;
                // two packed accumulators (even / odd dims of each 16-byte piece): half the multiply-add instructions
                float2 v2 = make_float2(0.0f, 0.0f), w2 = make_float2(0.0f, 0.0f);
#pragma unroll
                for (int i = 0; i < HD / 16; ++i) {
                    const float4 qq = *reinterpret_cast<const float4*>(qr + i * 16);
                    v2 = __ffma2_rn(make_float2(kk[i].x, kk[i].y), make_float2(qq.x, qq.y), v2);
                    w2 = __ffma2_rn(make_float2(kk[i].z, kk[i].w), make_float2(qq.z, qq.w), w2);
                }
                float v = (v2.x + w2.x) + (v2.y + w2.y);
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                if (c == 0 && pl < nt) sc[h * kAttnTile + pl] = v * scale;
            }
        }
        __syncthreads();
        issue_k(t0 + kAttnTile);  // the K tile is free: request the next one (an empty group after the last tile)
        // running softmax statistics: one warp per query head
        if (warp < gq) {
            const int h = warp;
            const float m_old = hstat[h * 4], l_old = hstat[h * 4 + 1];
            const float s_a = lane < nt ? sc[h * kAttnTile + lane] : -INFINITY;
            const float s_b = lane + 32 < nt ? sc[h * kAttnTile + lane + 32] : -INFINITY;
            const float m = warp_max(fmaxf(m_old, fmaxf(s_a, s_b)));
            const float e_a = lane < nt ? expf(s_a - m) : 0.0f, e_b = lane + 32 < nt ? expf(s_b - m) : 0.0f;
            if (lane < nt) sc[h * kAttnTile + lane] = e_a;
            if (lane + 32 < nt) sc[h * kAttnTile + lane + 32] = e_b;
            const float l = warp_sum(e_a + e_b);
            const float corr = expf(m_old - m);  // exp(-inf) = 0 on the first tile
            if (lane == 0) { hstat[h * 4] = m; hstat[h * 4 + 1] = l_old * corr + l; hstat[h * 4 + 2] = corr; }
        }
        cp_async_wait<1>();  // V has landed (at most the next K tile is still in flight)
        __syncthreads();
        if (has_new) {
            if (warp == kAttnWarps - 1) {
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    const size_t at = (size_t)(seq_len - 1) * kv_stride + (size_t)kv_head * HD + lane * EPL + e;
                    Vs[newrow * HD + lane * EPL + e] = kvn[e];
                    p.v_cache_w[at] = kvn[e];
                }
            }
            __syncthreads();
        }
        // weighted sum of V: one warp per position
#pragma unroll
        for (int h = 0; h < GQM; ++h)
            if (h < gq) {
                const float corr = hstat[h * 4 + 2];
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[h][e] *= corr;
            }
#pragma unroll 2
        for (int i = warp; i < nt; i += kAttnWarps) {
            float vv[EPL];
            load_lane_slice<EPL>(Vs + i * HD + lane * EPL, vv);
#pragma unroll
            for (int h = 0; h < GQM; ++h) {
                if (h < gq) {
                    const float w = sc[h * kAttnTile + i];
#pragma unroll
                    for (int e = 0; e < EPL; e += 2) {
                        const float2 r2 = __ffma2_rn(make_float2(w, w), make_float2(vv[e], vv[e + 1]), make_float2(acc[h][e], acc[h][e + 1]));
                        acc[h][e] = r2.x;
                        acc[h][e + 1] = r2.y;
                    }
                }
            }
        }
    }
    trace_stamp(p.trace, 2);
    __syncthreads();  // the V tile is free: reuse it for the cross-warp reduction
#pragma unroll
    for (int h = 0; h < GQM; ++h)
        if (h < gq)
#pragma unroll
            for (int e = 0; e < EPL; ++e) red[(warp * gq + h) * HD + lane * EPL + e] = acc[h][e];
    __syncthreads();
    finish_split<HD, GQM, kAttnWarps>(p, kv_head, split, nactive, red, hstat, Ks, &is_last);
}

// ---- decode attention over a bf16 KV cache: tensor-core form ------------------------------------------
// The f32 kernel above spends its time issuing multiply-adds (about 950 instructions per thread and 64-position tile);
// with bf16 rows the two contractions fit the tensor cores without touching the cache values: K and V are MMA operands
// exactly as stored, and the f32 side of each product (the query, the softmax weights) is split into a bf16 head and a
// bf16 remainder, two MMAs with f32 accumulation (16 mantissa bits of the f32 operand, products exact).
// Every warp is a pipeline of its own over stages of 16 positions (stage j = rows 16j.., warp w takes w, w + 8, ...):
//   S^T[pos][head] = K[pos] . q[head]:  A = the warp's K stage as it lies in shared memory ([pos][dim], ldmatrix),
//                                       B = the query heads (fragments built once per block)
//   running softmax per head in registers (a lane holds two heads of two positions; quad-of-lanes shuffles)
//   O^T[dim][head] += V^T[dim][pos] P^T[pos][head]:  A = the warp's V stage (ldmatrix.trans), B = the weights, moved from
//                                       the accumulator layout of S^T to an operand layout by movmatrix
// The warp copies its own rows (16-byte asynchronous copies; rows a stage does not have are zero-filled), requests its
// next K stage as soon as the scores are done and its next V stage after the weighted sum: warp-level synchronisation
// only.  Rows are padded by 16 bytes so that the 8 row addresses of an ldmatrix fall in distinct banks.  The warps'
// states are combined once at the end.  Range, split plan, fused RoPE + row write and the split merge are those of the
// f32 kernel; in the fused form the row being written is attended from shared memory (f32 arithmetic, one row).
// F32KV: the same pipelines over an f32 cache (used for batches of sequences, where the f32 kernel above is bound by
// instruction issue): the K and V fragments are read from the staged f32 rows in place and split into a bf16 head and
// remainder like the other operand; three of the four partial products are accumulated, so both operands count with 16
// mantissa bits (a relative 2^-17 per product, far inside the tolerance of the parity tests, but not the f32 products
// of the kernel above).  One block per multiprocessor (137 KB of stages).
// the same copies with the destination given as a shared-space address; the second form writes zeros when src_bytes is 0
__device__ inline void cp_async16_to(uint32_t smem_addr, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gmem_src) : "memory");
}
__device__ inline void cp_async16_zfill_to(uint32_t smem_addr, const void* gmem_src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gmem_src), "r"(src_bytes) : "memory");
}
__device__ inline float ex2_approx(float x) {  // 2^x, about 2 ulp; ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ inline void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(smem_row))
                 : "memory");
}
__device__ inline void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(smem_row))
                 : "memory");
}
// 8x8 transpose of 16-bit elements across the warp: lane T holds row T/4, columns 2(T%4), 2(T%4)+1 before and after
__device__ inline uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
// D += A * B, m16n8k16, bf16 operands, f32 accumulate
__device__ inline void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (x0, x1) -> bf16 pair of the values rounded to nearest-even (x0 in the low half) and bf16 pair of the remainders
__device__ inline void split_bf16x2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(x1), "f"(x0));
    const float r0 = x0 - __uint_as_float(hi << 16), r1 = x1 - __uint_as_float(hi & 0xffff0000u);
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(r1), "f"(r0));
}

template <int HD, int GQM, bool F32KV>
__global__ void __launch_bounds__(kAttnThreads, F32KV ? 1 : 2) decode_attention_mma_kernel(const DecodeAttnParams p_in) {
    DecodeAttnParams p = p_in;
    if (gridDim.z > 1) {  // sequence blockIdx.z of a batch: shift every per-sequence operand
        const size_t b = blockIdx.z;
        const size_t cache_shift = b * p.cache_stride * (F32KV ? 4 : 2);
        p.q += b * p.q_stride;
        p.out += b * p.out_stride;
        p.k_cache = reinterpret_cast<const float*>(reinterpret_cast<const char*>(p.k_cache) + cache_shift);
        p.v_cache = reinterpret_cast<const float*>(reinterpret_cast<const char*>(p.v_cache) + cache_shift);
        if (p.k_new != nullptr) {
            p.k_new += b * p.new_stride;
            p.v_new += b * p.new_stride;
            p.k_cache_w = reinterpret_cast<float*>(reinterpret_cast<char*>(p.k_cache_w) + cache_shift);
            p.v_cache_w = reinterpret_cast<float*>(reinterpret_cast<char*>(p.v_cache_w) + cache_shift);
        }
        p.part_acc += b * p.ws_stride;
        p.part_ml += b * p.ws_stride;
        p.counters += b * p.ws_stride;
    }
    constexpr int EPL = HD / 32;          // elements per lane where a warp holds one row (query, new K / V row)
    constexpr int ESZ = F32KV ? 4 : 2;    // bytes per cache element
    // padded rows (elements): 8 row addresses of an ldmatrix fall in distinct banks (bf16); f32 rows are read as
    // fragments directly, K two dims per lane (stride = 8 mod 32 words), V one dim of two rows (2 x stride = 8 mod 32)
    constexpr int KRP = HD + 8, VRP = F32KV ? HD + 4 : HD + 8;
    constexpr int KROWB = KRP * ESZ, VROWB = VRP * ESZ;  // bytes per staged row
    constexpr int V16 = HD * ESZ / 16;    // 16-byte pieces per row
    constexpr int R = 16;                 // positions per stage
    constexpr int KSTAGEB = R * KROWB, VSTAGEB = R * VROWB;
    constexpr int KSTEPS = HD / 16;       // MMA k-steps over the head dimension (scores)
    constexpr int DBLOCKS = HD / 16;      // 16-dim output blocks (weighted sum)
    constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
    extern __shared__ __align__(16) float smem[];
    char* const stages = reinterpret_cast<char*>(smem);                          // [kAttnWarps][K stage, V stage]
    float* wstat = reinterpret_cast<float*>(stages + kAttnWarps * (KSTAGEB + VSTAGEB));   // [kAttnWarps][8][2]: every warp's (max, sum)
    float* hstat = wstat + kAttnWarps * 8 * 2;                                   // [GQM][4]: block max, block sum
    float* qs = hstat + GQM * 4;                                                 // [GQM][HD] rotated query heads
    float* red = reinterpret_cast<float*>(stages) + 2048;                        // after the loop: [kAttnWarps][gq][HD]
    __shared__ bool is_last;
    __shared__ float2 cs_sn[HD / 2];
    __shared__ __align__(16) float newrow[2][HD];  // fused form: the K and V rows of the position being written, as stored

    trace_stamp(p.trace, 0);
    const int kv_head = blockIdx.x, gq = p.gq;
    int split = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t kv_stride = (size_t)p.n_kv_heads * HD;
    const bool fused = p.k_new != nullptr;
    int s0 = split * p.chunk;
    int seq_len = 0, n = 0, first_split = 0, n_stream = 0;
    bool owns_new = false;
    auto set_range = [&]() {
        seq_len = p.seq_len_ptr ? *p.seq_len_ptr : p.seq_len;
        const int lo = (p.window > 0 && seq_len > p.window) ? seq_len - p.window : 0;
        first_split = lo / p.chunk;
        const int slice_end = min(s0 + p.chunk, seq_len);
        s0 = max(s0, lo);
        n = slice_end - s0;
        owns_new = fused && n > 0 && slice_end == seq_len;  // the row being written is the last of the sequence
        n_stream = n - (owns_new ? 1 : 0);                   // ... and is not read from the cache
    };
    char* const kw = stages + warp * (KSTAGEB + VSTAGEB);
    char* const vw = kw + KSTAGEB;
    // Stage copies: one warp-wide copy instruction moves RSTEP rows (a lane always copies piece `cidx` of rows r0,
    // r0 + RSTEP, ...), so everything but the stage's first row is a per-lane constant.
    constexpr int RSTEP = 32 / V16;
    const int r0 = lane / V16, cidx = lane - r0 * V16;
    const size_t lane_goff = ((size_t)r0 * kv_stride + (size_t)kv_head * HD) * ESZ + cidx * 16;
    const size_t gstep = (size_t)RSTEP * kv_stride * ESZ;
    const uint32_t kw_addr = (uint32_t)__cvta_generic_to_shared(kw) + (uint32_t)(r0 * KROWB + cidx * 16);
    const uint32_t vw_addr = (uint32_t)__cvta_generic_to_shared(vw) + (uint32_t)(r0 * VROWB + cidx * 16);
    // rows 16j .. 16j+15 of the streamed rows into this warp's stage; one commit group (also when the stage does not exist)
    auto issue_stage = [&](const float* cache, uint32_t dst, int ROWB, int j) {
        const int rows = n_stream - j * R;
        if (rows > 0) {
            const char* gsrc = reinterpret_cast<const char*>(cache) + (size_t)(s0 + j * R) * kv_stride * ESZ + lane_goff;
            if (rows >= R) {
#pragma unroll
                for (int it = 0; it < R / RSTEP; ++it) cp_async16_to(dst + it * RSTEP * ROWB, gsrc + it * gstep);
            } else {  // the last stage of the slice: rows it does not have are zero-filled (the source is then not read)
#pragma unroll
                for (int it = 0; it < R / RSTEP; ++it) {
                    const bool have = r0 + it * RSTEP < rows;
                    cp_async16_zfill_to(dst + it * RSTEP * ROWB, have ? gsrc + it * gstep : reinterpret_cast<const char*>(cache), have ? 16u : 0u);
                }
            }
        }
        cp_async_commit();
    };
    if (fused) {
        set_range();
        if (n > 0) {
            issue_stage(p.k_cache, kw_addr, KROWB, warp);  // rows below seq_len - 1 were written by earlier steps
            issue_stage(p.v_cache, vw_addr, VROWB, warp);
            if (tid < HD / 2) {
                float sn, cs;
                sincosf((float)(seq_len - 1) * p.freqs[tid], &sn, &cs);
                cs_sn[tid] = make_float2(cs, sn);
            }
        }
    }
    pdl_wait();
    trace_stamp(p.trace, 1);
    if (!fused) set_range();
    const int nactive = (seq_len + p.chunk - 1) / p.chunk - first_split;
    if (n <= 0) return;
    split -= first_split;
    if (!fused) {
        issue_stage(p.k_cache, kw_addr, KROWB, warp);
        issue_stage(p.v_cache, vw_addr, VROWB, warp);
    }

    float qh[EPL], kvn[EPL];
    if (warp < gq) load_lane_slice<EPL>(p.q + (size_t)(kv_head * gq + warp) * HD + lane * EPL, qh);
    if (owns_new && warp == kAttnWarps - 2) load_lane_slice<EPL>(p.k_new + (size_t)kv_head * HD + lane * EPL, kvn);
    if (owns_new && warp == kAttnWarps - 1) load_lane_slice<EPL>(p.v_new + (size_t)kv_head * HD + lane * EPL, kvn);
    if (fused) __syncthreads();  // cs_sn is visible
    if (warp < gq) {
        if (fused) rope_lane_slice<EPL>(qh, cs_sn, lane);
#pragma unroll
        for (int e = 0; e < EPL; ++e) qs[warp * HD + lane * EPL + e] = qh[e];
    }
    if (owns_new && warp == kAttnWarps - 2) rope_lane_slice<EPL>(kvn, cs_sn, lane);
    if (owns_new && warp >= kAttnWarps - 2) {
        float* const cache_w = warp == kAttnWarps - 2 ? p.k_cache_w : p.v_cache_w;
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            const size_t at = (size_t)(seq_len - 1) * kv_stride + (size_t)kv_head * HD + lane * EPL + e;
            if (F32KV) {
                cache_w[at] = kvn[e];
                newrow[warp - (kAttnWarps - 2)][lane * EPL + e] = kvn[e];
            } else {
                const uint16_t bits = f32_to_bf16_bits(kvn[e]);  // rounded once; the stored value is what this step attends
                reinterpret_cast<uint16_t*>(cache_w)[at] = bits;
                newrow[warp - (kAttnWarps - 2)][lane * EPL + e] = bf16_bits_to_f32(bits);
            }
        }
    }
    __syncthreads();  // qs and newrow are visible

    // B fragments of the query heads: column g = head, this lane's dim pairs of every k-step, head and remainder
    const int g = lane >> 2, tq = lane & 3;
    uint32_t qhi[KSTEPS][2], qlo[KSTEPS][2];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float2 x = make_float2(0.0f, 0.0f);
            if (g < gq) x = *reinterpret_cast<const float2*>(qs + g * HD + ks * 16 + half * 8 + tq * 2);
            split_bf16x2(x.x, x.y, qhi[ks][half], qlo[ks][half]);
        }
    // this lane's two heads (2 tq, 2 tq + 1): running max in log2 units, running sum; accumulators of dims g, g + 8 of
    // every 16-dim block for those two heads
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[DBLOCKS][4];
#pragma unroll
    for (int db = 0; db < DBLOCKS; ++db)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[db][e] = 0.0f;
    const float scale2 = kLog2e / sqrtf((float)HD);  // scores in log2 units: the weights are exp2(s - m)

    const int nstages = (n_stream + R - 1) / R;
#pragma unroll 1
    for (int j = warp; j < nstages; j += kAttnWarps) {
        const int rows = min(R, n_stream - j * R);
        cp_async_wait<1>();  // this lane's K copies have landed (at most the V stage is still in flight)
        __syncwarp();        // ... and every other lane's
        float sh[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sl[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t a[4];  // 16 positions x 16 dims
            if (F32KV) {
                // f32 rows: the fragment is read in place (positions g, g + 8; dims 2tq.. and 8 + 2tq..) and split into a
                // bf16 head and remainder like the query: three of the four partial products (the last is below 2^-16)
                const float* kf = reinterpret_cast<const float*>(kw) + g * KRP + ks * 16 + 2 * tq;
                uint32_t al[4];
                const float2 x0 = *reinterpret_cast<const float2*>(kf), x1 = *reinterpret_cast<const float2*>(kf + 8 * KRP);
                const float2 x2 = *reinterpret_cast<const float2*>(kf + 8), x3 = *reinterpret_cast<const float2*>(kf + 8 * KRP + 8);
                split_bf16x2(x0.x, x0.y, a[0], al[0]);
                split_bf16x2(x1.x, x1.y, a[1], al[1]);
                split_bf16x2(x2.x, x2.y, a[2], al[2]);
                split_bf16x2(x3.x, x3.y, a[3], al[3]);
                mma_bf16(sl, al, qhi[ks][0], qhi[ks][1]);
            } else {
                ldmatrix_x4(a, kw + ((lane & 7) + ((lane >> 3) & 1) * 8) * KROWB + (ks * 16 + (lane >> 4) * 8) * 2);
            }
            mma_bf16(sh, a, qhi[ks][0], qhi[ks][1]);
            mma_bf16(sl, a, qlo[ks][0], qlo[ks][1]);
        }
        __syncwarp();  // every lane has read the K stage: it is free
        issue_stage(p.k_cache, kw_addr, KROWB, j + kAttnWarps);
        // s[0], s[1]: position g, heads 2tq, 2tq+1;  s[2], s[3]: position g + 8
        float s[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) s[e] = (sh[e] + sl[e]) * scale2;
        if (g >= rows) s[0] = s[1] = -INFINITY;
        if (g + 8 >= rows) s[2] = s[3] = -INFINITY;
        float corr[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float mx = fmaxf(s[hh], s[hh + 2]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m_run[hh], mx);  // finite: row 0 of a stage always exists
            s[hh] = ex2_approx(s[hh] - m_new);              // exp2(-inf) = 0 for rows the stage does not have
            s[hh + 2] = ex2_approx(s[hh + 2] - m_new);
            corr[hh] = ex2_approx(m_run[hh] - m_new);       // 0 on the first stage
            float ps = s[hh] + s[hh + 2];
            ps += __shfl_xor_sync(0xffffffffu, ps, 4);
            ps += __shfl_xor_sync(0xffffffffu, ps, 8);
            ps += __shfl_xor_sync(0xffffffffu, ps, 16);
            l_run[hh] = l_run[hh] * corr[hh] + ps;
            m_run[hh] = m_new;
        }
        if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
            for (int db = 0; db < DBLOCKS; ++db) { o[db][0] *= corr[0]; o[db][1] *= corr[1]; o[db][2] *= corr[0]; o[db][3] *= corr[1]; }
        }
        // weights as B fragments: (position g; heads 2tq, 2tq+1) -> (head g; positions 2tq, 2tq+1), head and remainder
        uint32_t ph0, pl0, ph1, pl1;
        split_bf16x2(s[0], s[1], ph0, pl0);
        split_bf16x2(s[2], s[3], ph1, pl1);
        ph0 = movmatrix_trans(ph0); pl0 = movmatrix_trans(pl0);
        ph1 = movmatrix_trans(ph1); pl1 = movmatrix_trans(pl1);
        cp_async_wait<1>();  // V has landed (at most the next K stage is still in flight)
        __syncwarp();
#pragma unroll
        for (int db = 0; db < DBLOCKS; ++db) {
            uint32_t a[4];  // V^T: 16 dims x 16 positions
            if (F32KV) {
                // dims g, g + 8 of positions 2tq, 2tq+1 and 8 + 2tq, 9 + 2tq
                const float* vf = reinterpret_cast<const float*>(vw) + (2 * tq) * VRP + db * 16 + g;
                uint32_t al[4];
                split_bf16x2(vf[0], vf[VRP], a[0], al[0]);
                split_bf16x2(vf[8], vf[VRP + 8], a[1], al[1]);
                split_bf16x2(vf[8 * VRP], vf[9 * VRP], a[2], al[2]);
                split_bf16x2(vf[8 * VRP + 8], vf[9 * VRP + 8], a[3], al[3]);
                mma_bf16(o[db], al, ph0, ph1);
            } else {
                ldmatrix_x4_trans(a, vw + ((lane & 7) + (lane >> 4) * 8) * VROWB + (db * 16 + ((lane >> 3) & 1) * 8) * 2);
            }
            mma_bf16(o[db], a, ph0, ph1);
            mma_bf16(o[db], a, pl0, pl1);
        }
        __syncwarp();  // every lane has read the V stage: it is free
        issue_stage(p.v_cache, vw_addr, VROWB, j + kAttnWarps);
    }
    // the position being written: one more row, attended from shared memory by warp 0 (plain f32 arithmetic)
    if (owns_new && warp == 0) {
        float snew[2] = {0.0f, 0.0f};
#pragma unroll
        for (int h = 0; h < GQM; ++h) {
            if (h < gq) {
                float v = 0.0f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) v = fmaf(qs[h * HD + lane * EPL + e], newrow[0][lane * EPL + e], v);
                v = warp_sum(v) * scale2;
                if (h == 2 * tq) snew[0] = v;
                if (h == 2 * tq + 1) snew[1] = v;
            }
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            if (2 * tq + hh < gq) {
                const float m_new = fmaxf(m_run[hh], snew[hh]);
                const float pw = ex2_approx(snew[hh] - m_new), c = ex2_approx(m_run[hh] - m_new);
                l_run[hh] = l_run[hh] * c + pw;
                m_run[hh] = m_new;
#pragma unroll
                for (int db = 0; db < DBLOCKS; ++db) {
                    o[db][hh] = fmaf(pw, newrow[1][db * 16 + g], o[db][hh] * c);
                    o[db][hh + 2] = fmaf(pw, newrow[1][db * 16 + g + 8], o[db][hh + 2] * c);
                }
            }
        }
    }
    trace_stamp(p.trace, 2);
    // combine the warps: block max per head, every warp's accumulators rescaled to it, summed by the common end
    if (g == 0) {
        wstat[(warp * 8 + 2 * tq) * 2] = m_run[0];
        wstat[(warp * 8 + 2 * tq) * 2 + 1] = l_run[0];
        wstat[(warp * 8 + 2 * tq + 1) * 2] = m_run[1];
        wstat[(warp * 8 + 2 * tq + 1) * 2 + 1] = l_run[1];
    }
    __syncthreads();  // every warp is done with its stages: their memory is free for the cross-warp reduction
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int h = 2 * tq + hh;
        if (h < gq) {
            float mb = -INFINITY;
#pragma unroll
            for (int w = 0; w < kAttnWarps; ++w) mb = fmaxf(mb, wstat[(w * 8 + h) * 2]);
            const float f = m_run[hh] == -INFINITY ? 0.0f : ex2_approx(m_run[hh] - mb);  // a warp without rows contributes nothing
#pragma unroll
            for (int db = 0; db < DBLOCKS; ++db) {
                red[(warp * gq + h) * HD + db * 16 + g] = o[db][hh] * f;
                red[(warp * gq + h) * HD + db * 16 + g + 8] = o[db][hh + 2] * f;
            }
            if (warp == 0 && g == 0) {
                float lb = 0.0f;
#pragma unroll
                for (int w = 0; w < kAttnWarps; ++w) {
                    const float mw = wstat[(w * 8 + h) * 2];
                    lb += mw == -INFINITY ? 0.0f : wstat[(w * 8 + h) * 2 + 1] * ex2_approx(mw - mb);
                }
                hstat[h * 4] = mb * kLn2;  // natural-log units, as the merge of the splits expects
                hstat[h * 4 + 1] = lb;
            }
        }
    }
    __syncthreads();
    finish_split<HD, GQM, kAttnWarps>(p, kv_head, split, nactive, red, hstat, reinterpret_cast<float*>(stages), &is_last);
}

// ---- prefill: tiled causal attention ---------------------------------------------------------------
constexpr int kPfBQ = 16;  // query rows per block
constexpr int kPfBK = 32;  // key positions per tile

template <int HD>
__global__ void __launch_bounds__(128) prefill_attention_kernel(const float* __restrict__ q_batch,
                                                                const float* __restrict__ k_cache,
                                                                const float* __restrict__ v_cache, int prompt_len,
                                                                int n_heads, int n_kv_heads, float* __restrict__ out,
                                                                int kv_bf16, int window) {
    constexpr int EPL = HD / 32;
    constexpr int KP = HD + 4;  // padded K row: 16-byte lane accesses hit disjoint banks
    __shared__ __align__(16) float Qs[kPfBQ][HD];
    __shared__ __align__(16) float Ks[kPfBK][KP];
    __shared__ __align__(16) float Vs[kPfBK][HD];
    pdl_wait();
    const int head = blockIdx.x;
    const int r0 = blockIdx.y * kPfBQ;
    const int kv_head = head / (n_heads / n_kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t q_len = (size_t)n_heads * HD;
    const size_t kv_stride = (size_t)n_kv_heads * HD;
    const float scale = 1.0f / sqrtf((float)HD);

    for (int idx = threadIdx.x; idx < kPfBQ * HD; idx += blockDim.x) {
        const int r = idx / HD, d = idx - r * HD;
        Qs[r][d] = (r0 + r) < prompt_len ? q_batch[(size_t)(r0 + r) * q_len + (size_t)head * HD + d] : 0.0f;
    }
    constexpr int QPW = kPfBQ / 4;  // queries per warp
    float m[QPW], l[QPW], acc[QPW][EPL];
#pragma unroll
    for (int j = 0; j < QPW; ++j) {
        m[j] = -INFINITY;
        l[j] = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[j][e] = 0.0f;
    }
    const int last_row = min(r0 + kPfBQ, prompt_len) - 1;
    // sliding window: row r attends keys r - window + 1 .. r; tiles wholly before the first row's window are skipped
    const int first_key = window > 0 ? max(0, r0 - window + 1) : 0;
    for (int t0 = first_key / kPfBK * kPfBK; t0 <= last_row; t0 += kPfBK) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < kPfBK * HD; idx += blockDim.x) {
            const int kk = idx / HD, d = idx - kk * HD;
            const int pos = t0 + kk;
            const bool ok = pos <= last_row;
            const size_t at = (size_t)pos * kv_stride + (size_t)kv_head * HD + d;
            if (kv_bf16) {
                Ks[kk][d] = ok ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(k_cache)[at]) : 0.0f;
                Vs[kk][d] = ok ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(v_cache)[at]) : 0.0f;
            } else {
                Ks[kk][d] = ok ? k_cache[at] : 0.0f;
                Vs[kk][d] = ok ? v_cache[at] : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < QPW; ++j) {
            const int r = warp * QPW + j;
            const int row = r0 + r;
            if (row >= prompt_len || t0 > row) continue;  // warp-uniform
            const int row_lo = window > 0 ? row - window + 1 : 0;  // first key this row attends
            if (t0 + kPfBK - 1 < row_lo) continue;  // the tile lies before this row's window (warp-uniform)
            // lane = key index inside the tile
            float s = 0.0f;
#pragma unroll 8
            for (int d = 0; d < HD; d += 4) {
                const float4 kq = *reinterpret_cast<const float4*>(&Ks[lane][d]);
                const float4 qq = *reinterpret_cast<const float4*>(&Qs[r][d]);
                s += qq.x * kq.x;
                s += qq.y * kq.y;
                s += qq.z * kq.z;
                s += qq.w * kq.w;
            }
            s = ((t0 + lane) <= row && (t0 + lane) >= row_lo) ? s * scale : -INFINITY;
            const float m_new = fmaxf(m[j], warp_max(s));
            const float pexp = expf(s - m_new);  // exp(-inf) = 0 for masked keys
            const float corr = expf(m[j] - m_new);
            l[j] = l[j] * corr + warp_sum(pexp);
            m[j] = m_new;
#pragma unroll
            for (int e = 0; e < EPL; ++e) acc[j][e] *= corr;
            for (int kk = 0; kk < kPfBK; ++kk) {
                const float w = __shfl_sync(0xffffffffu, pexp, kk);
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[j][e] = fmaf(w, Vs[kk][lane * EPL + e], acc[j][e]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < QPW; ++j) {
        const int row = r0 + warp * QPW + j;
        if (row < prompt_len) {
#pragma unroll
            for (int e = 0; e < EPL; ++e)
                out[(size_t)row * q_len + (size_t)head * HD + lane * EPL + e] = acc[j][e] / l[j];
        }
    }
}

// ---- prefill on the tensor cores --------------------------------------------------------------------------
// The same causal attention as prefill_attention_kernel for the decoder's batched prefill, where it was more than half of
// the time (2048-token prompt, Mistral-7B shape: 114 of 204 ms on CUDA cores).  One block = one query head x 64 query rows,
// four warps of 16 rows each; key tiles of 64 positions.  Both contractions run as bf16 MMAs with f32 accumulation, every
// f32 operand split into a bf16 head and remainder and three of the four partial products kept (16 mantissa bits per
// operand, a relative 2^-17 per product); with a bf16 cache K and V are exact and two products remain.
//   load: the tile's K and V rows go from the cache through registers into shared memory as bf16 head / remainder tiles
//         (rows padded by 16 bytes for ldmatrix); rows beyond the causal range are zeros
//   S = Q K^T: A = this warp's 16 query rows (fragments built once, in registers), B = K tile (ldmatrix)
//   online softmax in registers (rows g and g + 8 of the warp; quad shuffles), weights in log2 units
//   O += P V: A = the weights, re-used from the accumulator layout of S, B = V tile (ldmatrix.trans)
// Query tiles are issued last-first (the longest rows start first).  The plain operator form
// (kmll_prefill_causal_attention) keeps the f32 kernel above.
template <int HD, bool KVB>
__global__ void __launch_bounds__(128, 2) prefill_attention_mma_kernel(const float* __restrict__ q_batch, const float* __restrict__ k_cache,
                                                                       const float* __restrict__ v_cache, int prompt_len, int n_heads,
                                                                       int n_kv_heads, float* __restrict__ out, int window) {
    constexpr int BQ = 64, BK = 64;
    constexpr int RP = HD + 8;        // padded tile row, elements
    constexpr int ROWB = RP * 2;
    constexpr int TILEB = BK * ROWB;
    constexpr int KSTEPS = HD / 16, NBO = HD / 8;
    constexpr float kLog2e = 1.4426950408889634f;
    extern __shared__ __align__(16) float smem[];
    char* const k_hi = reinterpret_cast<char*>(smem);
    char* const v_hi = k_hi + TILEB;
    char* const k_lo = v_hi + TILEB;  // f32 cache only
    char* const v_lo = k_lo + TILEB;
    pdl_wait();
    const int head = blockIdx.x;
    const int r0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * BQ;
    const int kv_head = head / (n_heads / n_kv_heads);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const size_t q_len = (size_t)n_heads * HD, kv_stride = (size_t)n_kv_heads * HD;
    const float scale2 = kLog2e / sqrtf((float)HD);
    const int row_a = r0 + warp * 16 + g, row_b = row_a + 8;  // this lane's two query rows

    // A fragments of the warp's 16 query rows, head and remainder
    uint32_t qh[KSTEPS][4], ql[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int f = 0; f < 4; ++f) {
            const int row = (f & 1) ? row_b : row_a;
            float2 x = make_float2(0.0f, 0.0f);
            if (row < prompt_len) x = *reinterpret_cast<const float2*>(q_batch + (size_t)row * q_len + (size_t)head * HD + ks * 16 + (f >> 1) * 8 + 2 * tq);
            split_bf16x2(x.x, x.y, qh[ks][f], ql[ks][f]);
        }
    }
    float o[NBO][4];
#pragma unroll
    for (int nb = 0; nb < NBO; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[nb][e] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    const int last_row = min(r0 + BQ, prompt_len) - 1;
    const int first_key = window > 0 ? max(0, r0 - window + 1) : 0;  // tiles wholly before the first row's window are skipped
    const int lo_a = window > 0 ? row_a - window + 1 : 0, lo_b = window > 0 ? row_b - window + 1 : 0;
    const int warp_last = r0 + warp * 16 + 15;                        // last query row of this warp
    const int warp_lo = window > 0 ? r0 + warp * 16 - window + 1 : 0; // first key any row of this warp attends
#pragma unroll 1
    for (int t0 = first_key / BK * BK; t0 <= last_row; t0 += BK) {
        __syncthreads();  // the previous tile has been consumed
        // ---- K and V rows of the tile -> bf16 tiles (head, remainder)
        constexpr int C4 = HD / 4;  // four-element pieces per row
#pragma unroll 4
        for (int i = tid; i < BK * C4; i += 128) {
            const int key = i / C4, c4 = i - key * C4;
            const int pos = t0 + key;
            const size_t at = (size_t)pos * kv_stride + (size_t)kv_head * HD + c4 * 4;
            const int so = key * ROWB + c4 * 8;
            if (KVB) {
                uint2 kb = make_uint2(0u, 0u), vb = make_uint2(0u, 0u);
                if (pos <= last_row) {
                    kb = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(k_cache) + at);
                    vb = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(v_cache) + at);
                }
                *reinterpret_cast<uint2*>(k_hi + so) = kb;
                *reinterpret_cast<uint2*>(v_hi + so) = vb;
            } else {
                float4 kf = make_float4(0.0f, 0.0f, 0.0f, 0.0f), vf = kf;
                if (pos <= last_row) {
                    kf = *reinterpret_cast<const float4*>(k_cache + at);
                    vf = *reinterpret_cast<const float4*>(v_cache + at);
                }
                uint2 h, l;
                split_bf16x2(kf.x, kf.y, h.x, l.x);
                split_bf16x2(kf.z, kf.w, h.y, l.y);
                *reinterpret_cast<uint2*>(k_hi + so) = h;
                *reinterpret_cast<uint2*>(k_lo + so) = l;
                split_bf16x2(vf.x, vf.y, h.x, l.x);
                split_bf16x2(vf.z, vf.w, h.y, l.y);
                *reinterpret_cast<uint2*>(v_hi + so) = h;
                *reinterpret_cast<uint2*>(v_lo + so) = l;
            }
        }
        __syncthreads();
        if (t0 > warp_last || t0 + BK - 1 < warp_lo) continue;  // nothing of this tile is attended by this warp's rows (warp-uniform)
        // ---- S = Q K^T for 16 rows x 64 keys
        float sacc[BK / 8][4];
#pragma unroll
        for (int nb = 0; nb < BK / 8; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[nb][e] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int n2 = 0; n2 < BK / 16; ++n2) {
                const int off = (n2 * 16 + (lane >> 4) * 8 + (lane & 7)) * ROWB + (ks * 16 + ((lane >> 3) & 1) * 8) * 2;
                uint32_t b[4];
                ldmatrix_x4(b, k_hi + off);
                mma_bf16(sacc[2 * n2], qh[ks], b[0], b[1]);
                mma_bf16(sacc[2 * n2 + 1], qh[ks], b[2], b[3]);
                mma_bf16(sacc[2 * n2], ql[ks], b[0], b[1]);
                mma_bf16(sacc[2 * n2 + 1], ql[ks], b[2], b[3]);
                if (!KVB) {
                    ldmatrix_x4(b, k_lo + off);
                    mma_bf16(sacc[2 * n2], qh[ks], b[0], b[1]);
                    mma_bf16(sacc[2 * n2 + 1], qh[ks], b[2], b[3]);
                }
            }
        }
        // ---- scale, causal / window mask, running softmax (rows a = g, b = g + 8)
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < BK / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = t0 + nb * 8 + 2 * tq + e;
                sacc[nb][e] = (key <= row_a && key >= lo_a) ? sacc[nb][e] * scale2 : -INFINITY;
                sacc[nb][2 + e] = (key <= row_b && key >= lo_b) ? sacc[nb][2 + e] * scale2 : -INFINITY;
                mx_a = fmaxf(mx_a, sacc[nb][e]);
                mx_b = fmaxf(mx_b, sacc[nb][2 + e]);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        // a row with nothing attended so far keeps its maximum at -inf; the subtraction then uses 0 so that no NaN appears
        const float mn_a = fmaxf(m_run[0], mx_a), mn_b = fmaxf(m_run[1], mx_b);
        const float ma = mn_a == -INFINITY ? 0.0f : mn_a, mb = mn_b == -INFINITY ? 0.0f : mn_b;
        const float corr_a = ex2_approx(m_run[0] - ma), corr_b = ex2_approx(m_run[1] - mb);
        float ps_a = 0.0f, ps_b = 0.0f;
#pragma unroll
        for (int nb = 0; nb < BK / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                sacc[nb][e] = ex2_approx(sacc[nb][e] - ma);
                sacc[nb][2 + e] = ex2_approx(sacc[nb][2 + e] - mb);
                ps_a += sacc[nb][e];
                ps_b += sacc[nb][2 + e];
            }
        }
        ps_a += __shfl_xor_sync(0xffffffffu, ps_a, 1);
        ps_a += __shfl_xor_sync(0xffffffffu, ps_a, 2);
        ps_b += __shfl_xor_sync(0xffffffffu, ps_b, 1);
        ps_b += __shfl_xor_sync(0xffffffffu, ps_b, 2);
        l_run[0] = l_run[0] * corr_a + ps_a;
        l_run[1] = l_run[1] * corr_b + ps_b;
        m_run[0] = mn_a;
        m_run[1] = mn_b;
        if (__any_sync(0xffffffffu, corr_a != 1.0f || corr_b != 1.0f)) {
#pragma unroll
            for (int nb = 0; nb < NBO; ++nb) { o[nb][0] *= corr_a; o[nb][1] *= corr_a; o[nb][2] *= corr_b; o[nb][3] *= corr_b; }
        }
        // ---- O += P V: the weights of keys 16j .. 16j+15 are the A fragment of k-step j
#pragma unroll
        for (int j = 0; j < BK / 16; ++j) {
            uint32_t ph[4], pl[4];
            split_bf16x2(sacc[2 * j][0], sacc[2 * j][1], ph[0], pl[0]);
            split_bf16x2(sacc[2 * j][2], sacc[2 * j][3], ph[1], pl[1]);
            split_bf16x2(sacc[2 * j + 1][0], sacc[2 * j + 1][1], ph[2], pl[2]);
            split_bf16x2(sacc[2 * j + 1][2], sacc[2 * j + 1][3], ph[3], pl[3]);
#pragma unroll
            for (int d2 = 0; d2 < HD / 16; ++d2) {
                const int off = (j * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * ROWB + (d2 * 16 + (lane >> 4) * 8) * 2;
                uint32_t b[4];
                ldmatrix_x4_trans(b, v_hi + off);
                mma_bf16(o[2 * d2], ph, b[0], b[1]);
                mma_bf16(o[2 * d2 + 1], ph, b[2], b[3]);
                mma_bf16(o[2 * d2], pl, b[0], b[1]);
                mma_bf16(o[2 * d2 + 1], pl, b[2], b[3]);
                if (!KVB) {
                    ldmatrix_x4_trans(b, v_lo + off);
                    mma_bf16(o[2 * d2], ph, b[0], b[1]);
                    mma_bf16(o[2 * d2 + 1], ph, b[2], b[3]);
                }
            }
        }
    }
    const float inv_a = 1.0f / l_run[0], inv_b = 1.0f / l_run[1];
#pragma unroll
    for (int nb = 0; nb < NBO; ++nb) {
        if (row_a < prompt_len)
            *reinterpret_cast<float2*>(out + (size_t)row_a * q_len + (size_t)head * HD + nb * 8 + 2 * tq) = make_float2(o[nb][0] * inv_a, o[nb][1] * inv_a);
        if (row_b < prompt_len)
            *reinterpret_cast<float2*>(out + (size_t)row_b * q_len + (size_t)head * HD + nb * 8 + 2 * tq) = make_float2(o[nb][2] * inv_b, o[nb][3] * inv_b);
    }
}

struct AttnPlan {
    int chunk;
    int nsplit;
};

// Split plan: a pure function of the sequence capacity, so a CUDA graph captured for a given
// max_seq_len stays valid while the device-side sequence length grows.
static AttnPlan plan_decode_attention(int seq_cap, int kv_heads_times_batch = 0, int resident_blocks = 296) {
    AttnPlan pl;
    int nsplit = (seq_cap + 63) / 64;
    if (nsplit > 64) nsplit = 64;
    // A batch of sequences already fills the GPU along the batch axis: aim at one wave of blocks (`resident_blocks`: 296
    // at two per SM, 148 for the kernel that runs one per SM) with longer slices per block.  Measured at 16 sequences x 8 KV heads x 2051 positions: 256 blocks of 17
    // tiles beat 512 blocks of 9 (a second, partly filled wave) and every finer split (each block pays its own latency
    // chain: query load, RoPE table, partial results, merge).
    if (kv_heads_times_batch > 0) {
        int cap = resident_blocks / kv_heads_times_batch;
        if (cap < 1) cap = 1;
        if (nsplit > cap) nsplit = cap;
    }
    if (nsplit < 1) nsplit = 1;
    int chunk = (seq_cap + nsplit - 1) / nsplit;
    chunk = kv_heads_times_batch > 0 ? ((chunk + 63) & ~63) : ((chunk + 3) & ~3);
    pl.chunk = chunk;
    pl.nsplit = (seq_cap + chunk - 1) / chunk;
    if (pl.nsplit < 1) pl.nsplit = 1;
    return pl;
}

int decode_attention_launch(cudaStream_t stream, const float* q, const float* k_cache, const float* v_cache,
                            const int* seq_len_ptr, int seq_len, int seq_cap, int n_heads, int n_kv_heads,
                            int head_dim, float* workspace, float* out, const float* k_new, const float* v_new,
                            const float* freqs, float* k_cache_w, float* v_cache_w, int batch, size_t cache_stride,
                            int kv_bf16, int window) {
    const int gq = n_heads / n_kv_heads;
    // f32 cache inside the decoder (batches of sequences, fused step): the tensor-core kernel, one block per SM;
    // KMLL_ATTN_MMA_F32=0 keeps the f32 kernel
    static const bool mma_f32_allowed = [] { const char* e = getenv("KMLL_ATTN_MMA_F32"); return !(e != nullptr && e[0] == '0'); }();
    // (also the decoder's fused batch-1 form: 136 blocks of one stage per warp instead of 264, half as many partials to
    // merge - 673 against 661 tokens/s on the Mistral-7B shape; the plain operator form keeps the f32 kernel)
    bool mma_f32 = !kv_bf16 && (batch > 1 || k_new != nullptr) && mma_f32_allowed;
    AttnPlan pl = plan_decode_attention(seq_cap, batch > 1 ? n_kv_heads * batch : (mma_f32 ? n_kv_heads : 0), mma_f32 ? 148 : 296);
    if (mma_f32 && batch == 1 && pl.chunk < 128) {
        // few KV heads (a tensor-parallel shard of 1 or 2) or a short cache: slices under 8 stages would leave warps of
        // the tensor-core kernel idle; the f32 kernel's 64-position blocks are faster there (TP4: 857 against 840 tokens/s)
        mma_f32 = false;
        pl = plan_decode_attention(seq_cap, 0, 296);
    }
    if (kv_bf16 && batch == 1) {
        // bf16 cache, one sequence: slices of 8 stages (one per warp) where the KV heads allow it, like the f32 form
        const AttnPlan wide = plan_decode_attention(seq_cap, n_kv_heads, 148);
        if (wide.chunk >= 128) pl = wide;
    }
    DecodeAttnParams p;
    p.q = q; p.k_cache = k_cache; p.v_cache = v_cache;
    p.seq_len_ptr = seq_len_ptr; p.seq_len = seq_len;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.gq = gq;
    p.chunk = pl.chunk; p.nsplit = pl.nsplit;
    p.window = window > 0 ? window : 0;
    p.part_acc = workspace;
    p.part_ml = workspace + (size_t)n_heads * pl.nsplit * head_dim;
    p.counters = reinterpret_cast<unsigned int*>(p.part_ml + (size_t)n_heads * pl.nsplit * 2);
    p.out = out;
    p.k_new = k_new; p.v_new = v_new; p.freqs = freqs; p.k_cache_w = k_cache_w; p.v_cache_w = v_cache_w;
    p.trace = batch > 1 ? nullptr : trace_next_slot(200, n_kv_heads * pl.nsplit);
    // batch: q / out rows of n_heads*head_dim, new K/V rows of n_kv_heads*head_dim, one workspace per sequence
    p.q_stride = p.out_stride = (size_t)n_heads * head_dim;
    p.new_stride = (size_t)n_kv_heads * head_dim;
    p.cache_stride = cache_stride;
    p.ws_stride = (decode_attention_workspace_floats(n_heads, head_dim, seq_cap) + 3) & ~(size_t)3;  // keeps 16-byte alignment
    // K tile (padded rows), V tile, scores, statistics, query heads; the cross-warp reduction reuses the V tile
    // (kAttnWarps * gq <= kAttnTile rows because gq <= kMaxGq)
    const size_t smem = ((size_t)kAttnTile * (head_dim + 16) + (size_t)kAttnTile * head_dim + (size_t)kMaxGq * kAttnTile +
                         (size_t)kMaxGq * 4 + (size_t)kMaxGq * head_dim) * sizeof(float);
    cudaError_t e;
    auto go = [&](auto kern) {
        // (the attribute is per kernel and per device; setting it again is cheap and keeps this re-entrant)
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        return launch(kern, dim3(n_kv_heads, pl.nsplit, batch > 1 ? batch : 1), dim3(kAttnThreads), smem, stream, true, p);
    };
    if (kv_bf16 || mma_f32) {
        // per warp a K stage and a V stage of 16 padded rows; the warps' statistics, the block's, the query heads
        const size_t gqm = gq <= 4 ? 4 : kMaxGq;
        const size_t stage_bytes = kv_bf16 ? (size_t)2 * 16 * (head_dim + 8) * 2 : (size_t)16 * ((head_dim + 8) + (head_dim + 4)) * 4;
        const size_t smem16 = (size_t)kAttnWarps * stage_bytes + ((size_t)kAttnWarps * 16 + gqm * 4 + gqm * head_dim) * sizeof(float);
        auto go16 = [&](auto kern) {
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            return launch(kern, dim3(n_kv_heads, pl.nsplit, batch > 1 ? batch : 1), dim3(kAttnThreads), smem16, stream, true, p);
        };
        if (kv_bf16) {
            if (head_dim == 128) e = gq <= 4 ? go16(decode_attention_mma_kernel<128, 4, false>) : go16(decode_attention_mma_kernel<128, 8, false>);
            else e = gq <= 4 ? go16(decode_attention_mma_kernel<64, 4, false>) : go16(decode_attention_mma_kernel<64, 8, false>);
        } else {
            if (head_dim == 128) e = gq <= 4 ? go16(decode_attention_mma_kernel<128, 4, true>) : go16(decode_attention_mma_kernel<128, 8, true>);
            else e = gq <= 4 ? go16(decode_attention_mma_kernel<64, 4, true>) : go16(decode_attention_mma_kernel<64, 8, true>);
        }
    } else {
        if (head_dim == 128) e = gq <= 4 ? go(decode_attention_kernel<128, 4>) : go(decode_attention_kernel<128, 8>);
        else e = gq <= 4 ? go(decode_attention_kernel<64, 4>) : go(decode_attention_kernel<64, 8>);
    }
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "single_query_attention: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

int prefill_attention_launch(cudaStream_t stream, const float* q_batch, const float* k_cache, const float* v_cache, int prompt_len,
                             int n_heads, int n_kv_heads, int head_dim, float* out, int kv_bf16, int window, int tensor_cores) {
    cudaError_t e;
    static const bool mma_allowed = [] { const char* v = getenv("KMLL_PREFILL_MMA"); return !(v != nullptr && v[0] == '0'); }();
    if (tensor_cores && mma_allowed && (head_dim == 64 || head_dim == 128)) {
        const dim3 grid_mma(n_heads, (prompt_len + 63) / 64);
        const size_t smem = (size_t)(kv_bf16 ? 2 : 4) * 64 * (head_dim + 8) * 2;
        auto go = [&](auto kern) {
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            return launch(kern, grid_mma, dim3(128), smem, stream, true, q_batch, k_cache, v_cache, prompt_len, n_heads, n_kv_heads, out, window);
        };
        if (head_dim == 128) e = kv_bf16 ? go(prefill_attention_mma_kernel<128, true>) : go(prefill_attention_mma_kernel<128, false>);
        else e = kv_bf16 ? go(prefill_attention_mma_kernel<64, true>) : go(prefill_attention_mma_kernel<64, false>);
        if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "prefill attention (tensor cores): %s", cudaGetErrorString(e));
        return KMLL_OK;
    }
    const dim3 grid(n_heads, (prompt_len + kPfBQ - 1) / kPfBQ);
    if (head_dim == 128) {
        e = launch(prefill_attention_kernel<128>, grid, dim3(128), 0, stream, true, q_batch, k_cache, v_cache, prompt_len, n_heads, n_kv_heads, out, kv_bf16, window);
    } else if (head_dim == 64) {
        e = launch(prefill_attention_kernel<64>, grid, dim3(128), 0, stream, true, q_batch, k_cache, v_cache, prompt_len, n_heads, n_kv_heads, out, kv_bf16, window);
    } else {
        return fail(KMLL_ERR_UNSUPPORTED, "prefill_causal_attention: head_dim must be 64 or 128, got %d", head_dim);
    }
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "prefill_causal_attention: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

size_t decode_attention_workspace_floats(int n_heads, int head_dim, int seq_cap) {
    AttnPlan pl = plan_decode_attention(seq_cap);
    return (size_t)n_heads * pl.nsplit * (head_dim + 2) + (size_t)n_heads + 16;  // counters <= n_kv_heads <= n_heads
}

static int check_geometry(const char* name, int seq_len, int max_seq_len, int n_heads, int n_kv_heads, int head_dim) {
    if (n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || max_seq_len <= 0)
        return fail(KMLL_ERR_SHAPE, "%s: attention geometry must be positive", name);
    if (n_heads % n_kv_heads != 0) return fail(KMLL_ERR_SHAPE, "%s: n_heads must be divisible by n_kv_heads", name);
    if (seq_len <= 0 || seq_len > max_seq_len)
        return fail(KMLL_ERR_SHAPE, "%s: seq_len %d outside 1..max_seq_len %d", name, seq_len, max_seq_len);
    return KMLL_OK;
}

}  // namespace kmll

using namespace kmll;

extern "C" {

int kmll_attention_scores(kmll_stream_t s, const float* q, const float* k_cache, int seq_len, int max_seq_len, int n_heads,
                          int n_kv_heads, int head_dim, float* scores) {
    KMLL_REQUIRE_PTR(q); KMLL_REQUIRE_PTR(k_cache); KMLL_REQUIRE_PTR(scores);
    int rc = check_geometry("attention_scores", seq_len, max_seq_len, n_heads, n_kv_heads, head_dim);
    if (rc) return rc;
    const int items = n_heads * seq_len;
    cudaError_t e = launch(attention_scores_kernel, dim3((items + 3) / 4), dim3(128), 0, as_stream(s), true, q, k_cache, seq_len,
                           max_seq_len, n_heads, n_kv_heads, head_dim, scores);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "attention_scores: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

int kmll_softmax_value(kmll_stream_t s, const float* scores, const float* v_cache, int seq_len, int max_seq_len, int n_heads,
                       int n_kv_heads, int head_dim, float* out) {
    KMLL_REQUIRE_PTR(scores); KMLL_REQUIRE_PTR(v_cache); KMLL_REQUIRE_PTR(out);
    int rc = check_geometry("softmax_value", seq_len, max_seq_len, n_heads, n_kv_heads, head_dim);
    if (rc) return rc;
    cudaError_t e = launch(softmax_value_kernel, dim3(n_heads), dim3(256), 0, as_stream(s), true, scores, v_cache, seq_len,
                           max_seq_len, n_heads, n_kv_heads, head_dim, out);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "softmax_value: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

size_t kmll_single_query_attention_workspace_floats(int n_heads, int head_dim, int max_seq_len) {
    if (n_heads <= 0 || head_dim <= 0 || max_seq_len <= 0) return 0;
    return decode_attention_workspace_floats(n_heads, head_dim, max_seq_len);
}

int kmll_single_query_attention(kmll_stream_t s, const float* q, const float* k_cache, const float* v_cache, int seq_len,
                                int max_seq_len, int n_heads, int n_kv_heads, int head_dim, float* workspace, float* out) {
    KMLL_REQUIRE_PTR(q); KMLL_REQUIRE_PTR(k_cache); KMLL_REQUIRE_PTR(v_cache); KMLL_REQUIRE_PTR(out); KMLL_REQUIRE_PTR(workspace);
    int rc = check_geometry("single_query_attention", seq_len, max_seq_len, n_heads, n_kv_heads, head_dim);
    if (rc) return rc;
    if ((head_dim != 64 && head_dim != 128) || n_heads / n_kv_heads > kMaxGq)
        return fail(KMLL_ERR_UNSUPPORTED, "single_query_attention: head_dim must be 64 or 128 and n_heads/n_kv_heads <= %d; use attention_scores + softmax_value", kMaxGq);
    if (max_seq_len > 131072) return fail(KMLL_ERR_CAPACITY, "single_query_attention: max_seq_len %d beyond 131072", max_seq_len);
    return decode_attention_launch(as_stream(s), q, k_cache, v_cache, nullptr, seq_len, max_seq_len, n_heads, n_kv_heads, head_dim,
                                   workspace, out, nullptr, nullptr, nullptr, nullptr, nullptr);
}

// ---- decode attention for callers that cannot allocate device memory -----------------------------
// The split-sequence kernel needs scratch for the per-split partial results.  Hosts that bind only the
// operator layer (a worker thread that owns a stream and nothing else, or a serving loop in which a
// cudaMalloc would stall every stream of the device) have no way to provide it, so this entry point keeps
// its scratch in a fixed array that lives inside the loaded library image on every GPU that loads it.
constexpr size_t kNoAllocScratchFloats = 544768;  // 2.08 MiB: e.g. 64 heads x 64 splits x (128 + 2) floats + counters
static __device__ __align__(256) float g_attention_scratch[kNoAllocScratchFloats];

// Device address of the scratch array, looked up once per device while that device is current.  In host code
// the array's name is only a handle for the runtime; a kernel needs the address cudaGetSymbolAddress returns.
static int attention_scratch_address(float** out) {
    constexpr int kMaxDevices = 64;
    static std::mutex lock;
    static float* cached[kMaxDevices] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "single_query_attention_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(KMLL_ERR_CAPACITY, "single_query_attention_noalloc: device index %d beyond %d", dev, kMaxDevices);
    std::lock_guard<std::mutex> guard(lock);
    if (cached[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_attention_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return fail(KMLL_ERR_CUDA, "single_query_attention_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        cached[dev] = static_cast<float*>(ptr);
    }
    *out = cached[dev];
    return KMLL_OK;
}

int kmll_single_query_attention_noalloc(kmll_stream_t s, const float* q, const float* k_cache, const float* v_cache, int seq_len,
                                        int max_seq_len, int n_heads, int n_kv_heads, int head_dim, float* out) {
    KMLL_REQUIRE_PTR(q); KMLL_REQUIRE_PTR(k_cache); KMLL_REQUIRE_PTR(v_cache); KMLL_REQUIRE_PTR(out);
    int rc = check_geometry("single_query_attention_noalloc", seq_len, max_seq_len, n_heads, n_kv_heads, head_dim);
    if (rc) return rc;
    if ((head_dim != 64 && head_dim != 128) || n_heads / n_kv_heads > kMaxGq)
        return fail(KMLL_ERR_UNSUPPORTED, "single_query_attention_noalloc: head_dim must be 64 or 128 and n_heads/n_kv_heads <= %d", kMaxGq);
    if (max_seq_len > 131072) return fail(KMLL_ERR_CAPACITY, "single_query_attention_noalloc: max_seq_len %d beyond 131072", max_seq_len);
    const size_t need = decode_attention_workspace_floats(n_heads, head_dim, max_seq_len);
    if (need > kNoAllocScratchFloats)
        return fail(KMLL_ERR_CAPACITY,
                    "single_query_attention_noalloc: this geometry needs %zu floats of scratch, the built-in array holds %zu; "
                    "use kmll_single_query_attention with a caller-owned workspace",
                    need, (size_t)kNoAllocScratchFloats);
    float* scratch = nullptr;
    rc = attention_scratch_address(&scratch);
    if (rc) return rc;
    // The array keeps whatever the previous call left.  Only the per-KV-head arrival counters have to start at
    // zero; they sit behind the partial results (same layout as the caller-owned workspace).
    AttnPlan pl = plan_decode_attention(max_seq_len);
    float* counters = scratch + (size_t)n_heads * pl.nsplit * (head_dim + 2);
    cudaError_t e = cudaMemsetAsync(counters, 0, sizeof(unsigned int) * (size_t)n_kv_heads, as_stream(s));
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "single_query_attention_noalloc: cudaMemsetAsync: %s", cudaGetErrorString(e));
    return decode_attention_launch(as_stream(s), q, k_cache, v_cache, nullptr, seq_len, max_seq_len, n_heads, n_kv_heads, head_dim,
                                   scratch, out, nullptr, nullptr, nullptr, nullptr, nullptr);
}

int kmll_prefill_causal_attention(kmll_stream_t s, const float* q_batch, const float* k_cache, const float* v_cache, int prompt_len,
                                  int max_seq_len, int n_heads, int n_kv_heads, int head_dim, float* out) {
    KMLL_REQUIRE_PTR(q_batch); KMLL_REQUIRE_PTR(k_cache); KMLL_REQUIRE_PTR(v_cache); KMLL_REQUIRE_PTR(out);
    int rc = check_geometry("prefill_causal_attention", prompt_len, max_seq_len, n_heads, n_kv_heads, head_dim);
    if (rc) return rc;
    return prefill_attention_launch(as_stream(s), q_batch, k_cache, v_cache, prompt_len, n_heads, n_kv_heads, head_dim, out, 0, 0, 0);
}

}  // extern "C"
