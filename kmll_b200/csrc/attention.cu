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

// bf16 KV cache (kernel template flag KVB): the caches hold bf16 bit patterns (2 bytes per element, same
// [max_seq, n_kv, head_dim] layout); rows are staged raw and widened to f32 where they are used, the new K / V rows
// are rounded to nearest-even once, and that rounded value is both what is stored and what this step attends over.
__device__ inline float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ inline float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

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
template <int HD, int GQM, bool KVB>
__global__ void __launch_bounds__(kAttnThreads, 2) decode_attention_kernel(const DecodeAttnParams p_in) {
    DecodeAttnParams p = p_in;
    constexpr size_t ESZ = KVB ? 2 : 4;  // bytes per cache element
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
    float* Ks = smem;                         // [kAttnTile][KP]   (bf16 cache: the same areas, half used)
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
    if (KVB && owns_new && warp >= kAttnWarps - 2) {
#pragma unroll
        for (int e = 0; e < EPL; ++e) kvn[e] = bf16_bits_to_f32(f32_to_bf16_bits(kvn[e]));
    }

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
                if (KVB) {
                    const uint16_t bits = (uint16_t)(__float_as_uint(kvn[e]) >> 16);
                    reinterpret_cast<uint16_t*>(Ks)[newrow * KP + lane * EPL + e] = bits;
                    reinterpret_cast<uint16_t*>(p.k_cache_w)[at] = bits;
                } else {
                    Ks[newrow * KP + lane * EPL + e] = kvn[e];
                    p.k_cache_w[at] = kvn[e];
                }
            }
        }
        if (has_new) __syncthreads();
        // scores: four lanes per position, each over an interleaved quarter of the head dimension
        {
            const int pl = tid >> 2, c = tid & 3;
            float4 kk[HD / 16];
            if (KVB) {
                const uint16_t* kr = reinterpret_cast<const uint16_t*>(Ks) + (pl < nt ? pl : 0) * KP + c * 4;
#pragma unroll
                for (int i = 0; i < HD / 16; ++i) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(kr + i * 16);
                    kk[i] = make_float4(bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y));
                }
            } else {
                const float* kr = Ks + (pl < nt ? pl : 0) * KP + c * 4;
#pragma unroll
                for (int i = 0; i < HD / 16; ++i) kk[i] = *reinterpret_cast<const float4*>(kr + i * 16);
            }
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
                    if (KVB) {
                        const uint16_t bits = (uint16_t)(__float_as_uint(kvn[e]) >> 16);
                        reinterpret_cast<uint16_t*>(Vs)[newrow * HD + lane * EPL + e] = bits;
                        reinterpret_cast<uint16_t*>(p.v_cache_w)[at] = bits;
                    } else {
                        Vs[newrow * HD + lane * EPL + e] = kvn[e];
                        p.v_cache_w[at] = kvn[e];
                    }
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
            if (KVB) {
                const uint16_t* vr = reinterpret_cast<const uint16_t*>(Vs) + i * HD + lane * EPL;
                if (EPL == 4) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(vr);
                    vv[0] = bf16_lo(raw.x); vv[1] = bf16_hi(raw.x); vv[EPL - 2] = bf16_lo(raw.y); vv[EPL - 1] = bf16_hi(raw.y);
                } else {
                    const uint32_t raw = *reinterpret_cast<const uint32_t*>(vr);
                    vv[0] = bf16_lo(raw); vv[1] = bf16_hi(raw);
                }
            } else {
                load_lane_slice<EPL>(Vs + i * HD + lane * EPL, vv);
            }
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
//   S[h][pos] = q[h] . K[pos]:  A = query heads (rows 0..gq-1 of a 16-row fragment, built once per block),
//                               B = K tile as it lies in shared memory ([pos][dim], ldmatrix); warp w owns positions 8w..8w+7
//   O[h][dim] += P[h][pos] V[pos][dim]:  A = softmax weights of the tile, B = V tile ([pos][dim], ldmatrix.trans);
//                               warp w owns dims w*HD/8 .. of every head, so no cross-warp reduction at the end
// Tiles of 64 positions in a two-stage ring: the K and V rows of tile t+1 are requested before tile t is touched.
// Rows are padded by 16 bytes so that the 8 row addresses of an ldmatrix fall in distinct banks; rows a tile does not
// have are zero-filled by the copy.  Range, split plan, fused RoPE + row write and the split merge are those of the
// f32 kernel.
__device__ inline void cp_async16_zfill(void* smem_dst, const void* gmem_src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src),
                 "r"(src_bytes)
                 : "memory");
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
__device__ inline void ldmatrix_x2_trans(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1])
                 : "r"((uint32_t)__cvta_generic_to_shared(smem_row))
                 : "memory");
}
// D += A * B, m16n8k16, bf16 operands, f32 accumulate; only rows 0..7 of A are populated (a1 = a3 = 0)
__device__ inline void mma_bf16_rows8(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
// (x0, x1) -> bf16 pair of the values rounded to nearest-even (x0 in the low half) and bf16 pair of the remainders
__device__ inline void split_bf16x2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(x1), "f"(x0));
    const float r0 = x0 - __uint_as_float(hi << 16), r1 = x1 - __uint_as_float(hi & 0xffff0000u);
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(r1), "f"(r0));
}

template <int HD, int GQM>
__global__ void __launch_bounds__(kAttnThreads, 2) decode_attention_bf16_kernel(const DecodeAttnParams p_in) {
    DecodeAttnParams p = p_in;
    if (gridDim.z > 1) {  // sequence blockIdx.z of a batch: shift every per-sequence operand
        const size_t b = blockIdx.z;
        const size_t cache_shift = b * p.cache_stride * 2;
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
    constexpr int RP = HD + 8;            // padded row, elements
    constexpr int ROWB = RP * 2;          // bytes per staged row
    constexpr int V16 = HD / 8;           // 16-byte pieces per row
    constexpr int TILEB = kAttnTile * ROWB;
    constexpr int KSTEPS = HD / 16;       // MMA k-steps over the head dimension
    constexpr int NBW = HD / 64;          // 8-dim output blocks per warp (8 warps cover the head dimension)
    constexpr int SCP = kAttnTile + 8;    // padded score row: the fragment accesses of four heads fall in distinct banks
    extern __shared__ __align__(16) float smem[];
    char* const tiles = reinterpret_cast<char*>(smem);                // [2 stages][K tile, V tile]
    float* sc = reinterpret_cast<float*>(tiles + 4 * TILEB);          // [GQM][SCP] scores, then weights
    float* hstat = sc + GQM * SCP;                              // [GQM][4]: running max, running sum, correction
    float* qs = hstat + GQM * 4;                                      // [GQM][HD] rotated query heads
    float* red = reinterpret_cast<float*>(tiles + 2 * TILEB);         // after the loop: [kAttnWarps][gq][HD]
    __shared__ bool is_last;
    __shared__ float2 cs_sn[HD / 2];

    trace_stamp(p.trace, 0);
    const int kv_head = blockIdx.x, gq = p.gq;
    int split = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t kv_stride = (size_t)p.n_kv_heads * HD;
    const bool fused = p.k_new != nullptr;
    int s0 = split * p.chunk;
    int seq_len = 0, n = 0, first_split = 0;
    auto set_range = [&]() {
        seq_len = p.seq_len_ptr ? *p.seq_len_ptr : p.seq_len;
        const int lo = (p.window > 0 && seq_len > p.window) ? seq_len - p.window : 0;
        first_split = lo / p.chunk;
        const int slice_end = min(s0 + p.chunk, seq_len);
        s0 = max(s0, lo);
        n = slice_end - s0;
    };
    // K and V rows of tile t into stage t & 1, one commit group (also when the tile does not exist)
    auto issue_tile = [&](int t) {
        const int t0 = t * kAttnTile;
        const int nt = n - t0;
        if (nt > 0) {
            char* ks = tiles + (t & 1) * 2 * TILEB;
            char* vs = ks + TILEB;
            const size_t g0 = ((size_t)(s0 + t0) * kv_stride + (size_t)kv_head * HD) * 2;
#pragma unroll
            for (int i = tid; i < kAttnTile * V16; i += kAttnThreads) {
                const int r = i / V16, cidx = i - r * V16;
                const bool have = r < nt;
                const size_t off = g0 + (have ? (size_t)r * kv_stride * 2 : 0) + cidx * 16;
                cp_async16_zfill(ks + r * ROWB + cidx * 16, reinterpret_cast<const char*>(p.k_cache) + off, have ? 16u : 0u);
                cp_async16_zfill(vs + r * ROWB + cidx * 16, reinterpret_cast<const char*>(p.v_cache) + off, have ? 16u : 0u);
            }
        }
        cp_async_commit();
    };
    if (fused) {
        set_range();
        if (n > 0) {
            issue_tile(0);  // rows below seq_len - 1 were written by earlier steps
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
    const int nactive = (seq_len + p.chunk - 1) / p.chunk - first_split;
    if (n <= 0) return;
    split -= first_split;
    if (!fused) issue_tile(0);
    const float scale = 1.0f / sqrtf((float)HD);

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
    __syncthreads();  // qs is visible

    // A fragments of the query heads: row g = head, this lane's column pairs of every k-step, head and remainder
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
    float o[NBW][4];
#pragma unroll
    for (int nb = 0; nb < NBW; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[nb][e] = 0.0f;

    const int ntiles = (n + kAttnTile - 1) / kAttnTile;
#pragma unroll 1
    for (int t = 0; t < ntiles; ++t) {
        cp_async_wait<0>();  // tile t has landed (this thread's copies; the barrier covers everybody's)
        __syncthreads();     // ... and every warp is done with tile t - 1: its stage and the weights are free
        issue_tile(t + 1);
        char* const ks_t = tiles + (t & 1) * 2 * TILEB;
        char* const vs_t = ks_t + TILEB;
        const int nt = min(kAttnTile, n - t * kAttnTile);
        const int newrow = newpos - t * kAttnTile;
        if (owns_new && newrow >= 0 && newrow < nt) {  // block-uniform
            if (warp >= kAttnWarps - 2) {
                char* const tile = warp == kAttnWarps - 2 ? ks_t : vs_t;
                uint16_t* const cache_w = reinterpret_cast<uint16_t*>(warp == kAttnWarps - 2 ? p.k_cache_w : p.v_cache_w);
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    const uint16_t bits = f32_to_bf16_bits(kvn[e]);
                    reinterpret_cast<uint16_t*>(tile + newrow * ROWB)[lane * EPL + e] = bits;
                    cache_w[(size_t)(seq_len - 1) * kv_stride + (size_t)kv_head * HD + lane * EPL + e] = bits;
                }
            }
            __syncthreads();
        }
        // scores of positions 8 * warp .. + 7 for every head
        {
            float ch[4] = {0.0f, 0.0f, 0.0f, 0.0f}, cl[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int k2 = 0; k2 < KSTEPS / 2; ++k2) {
                uint32_t b[4];  // 8 positions x 32 dims: B fragments of two k-steps
                ldmatrix_x4(b, ks_t + (warp * 8 + (lane & 7)) * ROWB + (k2 * 32 + (lane >> 3) * 8) * 2);
                mma_bf16_rows8(ch, qhi[2 * k2][0], qhi[2 * k2][1], b[0], b[1]);
                mma_bf16_rows8(cl, qlo[2 * k2][0], qlo[2 * k2][1], b[0], b[1]);
                mma_bf16_rows8(ch, qhi[2 * k2 + 1][0], qhi[2 * k2 + 1][1], b[2], b[3]);
                mma_bf16_rows8(cl, qlo[2 * k2 + 1][0], qlo[2 * k2 + 1][1], b[2], b[3]);
            }
            if (g < gq)
                *reinterpret_cast<float2*>(sc + g * SCP + warp * 8 + tq * 2) = make_float2((ch[0] + cl[0]) * scale, (ch[1] + cl[1]) * scale);
        }
        __syncthreads();
        // running softmax statistics: one warp per query head (rows the tile does not have get weight 0)
        if (warp < gq) {
            const int h = warp;
            const float m_old = hstat[h * 4], l_old = hstat[h * 4 + 1];
            const float s_a = lane < nt ? sc[h * SCP + lane] : -INFINITY;
            const float s_b = lane + 32 < nt ? sc[h * SCP + lane + 32] : -INFINITY;
            const float m = warp_max(fmaxf(m_old, fmaxf(s_a, s_b)));
            const float e_a = lane < nt ? expf(s_a - m) : 0.0f, e_b = lane + 32 < nt ? expf(s_b - m) : 0.0f;
            sc[h * SCP + lane] = e_a;
            sc[h * SCP + lane + 32] = e_b;
            const float l = warp_sum(e_a + e_b);
            const float corr = expf(m_old - m);  // exp(-inf) = 0 on the first tile
            if (lane == 0) { hstat[h * 4] = m; hstat[h * 4 + 1] = l_old * corr + l; hstat[h * 4 + 2] = corr; }
        }
        __syncthreads();
        // weighted sum of V: dims warp * HD/8 .. of every head
        {
            const float corr = g < gq ? hstat[g * 4 + 2] : 0.0f;
#pragma unroll
            for (int nb = 0; nb < NBW; ++nb) { o[nb][0] *= corr; o[nb][1] *= corr; }
            float ol[NBW][4];
#pragma unroll
            for (int nb = 0; nb < NBW; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) ol[nb][e] = 0.0f;
#pragma unroll
            for (int k4 = 0; k4 < kAttnTile / 16; ++k4) {
                float2 pa = make_float2(0.0f, 0.0f), pb = make_float2(0.0f, 0.0f);
                if (g < gq) {
                    pa = *reinterpret_cast<const float2*>(sc + g * SCP + k4 * 16 + tq * 2);
                    pb = *reinterpret_cast<const float2*>(sc + g * SCP + k4 * 16 + 8 + tq * 2);
                }
                uint32_t ah0, al0, ah2, al2;
                split_bf16x2(pa.x, pa.y, ah0, al0);
                split_bf16x2(pb.x, pb.y, ah2, al2);
                uint32_t b[4];  // 16 positions x (8 * NBW) dims, transposed on the way in
                const char* row = vs_t + (k4 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * ROWB + (warp * (HD / 8)) * 2;
                if (NBW == 2) ldmatrix_x4_trans(b, row + (lane >> 4) * 16);
                else ldmatrix_x2_trans(b, row);
                mma_bf16_rows8(o[0], ah0, ah2, b[0], b[1]);
                mma_bf16_rows8(ol[0], al0, al2, b[0], b[1]);
                if (NBW == 2) {
                    mma_bf16_rows8(o[NBW - 1], ah0, ah2, b[2], b[3]);
                    mma_bf16_rows8(ol[NBW - 1], al0, al2, b[2], b[3]);
                }
            }
#pragma unroll
            for (int nb = 0; nb < NBW; ++nb) { o[nb][0] += ol[nb][0]; o[nb][1] += ol[nb][1]; }
        }
    }
    trace_stamp(p.trace, 2);
    __syncthreads();  // every warp is done with the last tile: the stages are free
    // every (head, dim) is complete in one lane: one plane for the common end
    if (g < gq) {
#pragma unroll
        for (int nb = 0; nb < NBW; ++nb)
            *reinterpret_cast<float2*>(red + g * HD + warp * (HD / 8) + nb * 8 + tq * 2) = make_float2(o[nb][0], o[nb][1]);
    }
    __syncthreads();
    finish_split<HD, GQM, 1>(p, kv_head, split, nactive, red, hstat, reinterpret_cast<float*>(tiles), &is_last);
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

struct AttnPlan {
    int chunk;
    int nsplit;
};

// Split plan: a pure function of the sequence capacity, so a CUDA graph captured for a given
// max_seq_len stays valid while the device-side sequence length grows.
static AttnPlan plan_decode_attention(int seq_cap, int kv_heads_times_batch = 0) {
    AttnPlan pl;
    int nsplit = (seq_cap + 63) / 64;
    if (nsplit > 64) nsplit = 64;
    // A batch of sequences already fills the GPU along the batch axis: aim at one wave of blocks (296 are resident at
    // two per SM) with longer slices per block.  Measured at 16 sequences x 8 KV heads x 2051 positions: 256 blocks of 17
    // tiles beat 512 blocks of 9 (a second, partly filled wave) and every finer split (each block pays its own latency
    // chain: query load, RoPE table, partial results, merge).
    if (kv_heads_times_batch > 0) {
        int cap = 296 / kv_heads_times_batch;
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
    AttnPlan pl = plan_decode_attention(seq_cap, batch > 1 ? n_kv_heads * batch : 0);
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
    if (kv_bf16) {
        // two stages of (K tile, V tile) with padded bf16 rows, scores, statistics, query heads
        const size_t gqm = gq <= 4 ? 4 : kMaxGq;
        const size_t smem16 = (size_t)4 * kAttnTile * (head_dim + 8) * 2 + (gqm * (kAttnTile + 8) + gqm * 4 + gqm * head_dim) * sizeof(float);
        auto go16 = [&](auto kern) {
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            return launch(kern, dim3(n_kv_heads, pl.nsplit, batch > 1 ? batch : 1), dim3(kAttnThreads), smem16, stream, true, p);
        };
        if (head_dim == 128) e = gq <= 4 ? go16(decode_attention_bf16_kernel<128, 4>) : go16(decode_attention_bf16_kernel<128, 8>);
        else e = gq <= 4 ? go16(decode_attention_bf16_kernel<64, 4>) : go16(decode_attention_bf16_kernel<64, 8>);
    } else {
        if (head_dim == 128) e = gq <= 4 ? go(decode_attention_kernel<128, 4, false>) : go(decode_attention_kernel<128, 8, false>);
        else e = gq <= 4 ? go(decode_attention_kernel<64, 4, false>) : go(decode_attention_kernel<64, 8, false>);
    }
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "single_query_attention: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

int prefill_attention_launch(cudaStream_t stream, const float* q_batch, const float* k_cache, const float* v_cache, int prompt_len,
                             int n_heads, int n_kv_heads, int head_dim, float* out, int kv_bf16, int window) {
    const dim3 grid(n_heads, (prompt_len + kPfBQ - 1) / kPfBQ);
    cudaError_t e;
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
    return prefill_attention_launch(as_stream(s), q_batch, k_cache, v_cache, prompt_len, n_heads, n_kv_heads, head_dim, out, 0, 0);
}

}  // extern "C"
