// Row-reduction and elementwise operators of the decode path: RMSNorm, add, SiLU*up, RoPE,
// KV-cache writes, row softmax, embedding lookup, arg-max / top-k.  Each makes one pass over
// HBM with 128-bit accesses where alignment allows; all arithmetic is f32 in kmll's order.
#include "internal.cuh"

namespace kmll {

// ---- RMSNorm --------------------------------------------------------------------------------
// y = x * (1/sqrt(sum(x^2)/n + eps)) * w, evaluated left to right
// (crates/inference/src/kernels/inference.rs:60-114; 1.0/sqrt, not rsqrt.approx, crates/inference/src/math.rs:73-78).
// One block per row; the row is read once into registers (up to 8 values per thread per pass).
template <typename TIn, typename TOut>
__device__ inline float load_as_f32(const TIn* p, size_t i);
template <>
__device__ inline float load_as_f32<float, float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ inline float load_as_f32<uint16_t, uint16_t>(const uint16_t* p, size_t i) { return bf16_bits_to_f32(p[i]); }
__device__ inline void store_from_f32(float* p, size_t i, float v) { p[i] = v; }
__device__ inline void store_from_f32(uint16_t* p, size_t i, float v) { p[i] = f32_to_bf16_bits(v); }

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const T* __restrict__ x, const uint16_t* __restrict__ w, int dim,
                                                      float eps, T* __restrict__ y) {
    __shared__ float scratch[40];
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * dim;
    constexpr int kMaxPerThread = 16;  // rows up to 4096 stay in registers; longer rows are re-read
    float v[kMaxPerThread];
    float ss = 0.0f;
    const bool in_regs = dim <= kMaxPerThread * 256;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kMaxPerThread; ++j) {
            const int i = threadIdx.x + j * 256;
            v[j] = i < dim ? load_as_f32<T, T>(x, base + i) : 0.0f;
            ss += v[j] * v[j];
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += 256) {
            const float t = load_as_f32<T, T>(x, base + i);
            ss += t * t;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    pdl_launch_dependents();
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kMaxPerThread; ++j) {
            const int i = threadIdx.x + j * 256;
            if (i < dim) store_from_f32(y, base + i, v[j] * inv * bf16_bits_to_f32(w[i]));
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += 256)
            store_from_f32(y, base + i, load_as_f32<T, T>(x, base + i) * inv * bf16_bits_to_f32(w[i]));
    }
}

// ---- add / silu*up ----------------------------------------------------------------------------
__device__ inline float silu_mul_f32(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

template <int OP>  // 0 add, 1 silu_mul
__global__ void binary_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, size_t n,
                                  float* __restrict__ out, int vec_ok) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec_ok) {
        const size_t n4 = n >> 2;
        if (i < n4) {
            const float4 va = reinterpret_cast<const float4*>(a)[i];
            const float4 vb = reinterpret_cast<const float4*>(b)[i];
            float4 r;
            if (OP == 0) {
                r = make_float4(va.x + vb.x, va.y + vb.y, va.z + vb.z, va.w + vb.w);
            } else {
                r = make_float4(silu_mul_f32(va.x, vb.x), silu_mul_f32(va.y, vb.y), silu_mul_f32(va.z, vb.z),
                                silu_mul_f32(va.w, vb.w));
            }
            reinterpret_cast<float4*>(out)[i] = r;
        }
        const size_t tail = (n4 << 2) + i;
        if (i < (n & 3)) out[tail] = OP == 0 ? a[tail] + b[tail] : silu_mul_f32(a[tail], b[tail]);
    } else if (i < n) {
        out[i] = OP == 0 ? a[i] + b[i] : silu_mul_f32(a[i], b[i]);
    }
}

__global__ void silu_mul_bf16_kernel(const uint16_t* __restrict__ g, const uint16_t* __restrict__ u, size_t n,
                                     uint16_t* __restrict__ out, int vec_ok) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec_ok) {
        const size_t n8 = n >> 3;
        if (i < n8) {
            const uint4 vg = reinterpret_cast<const uint4*>(g)[i];
            const uint4 vu = reinterpret_cast<const uint4*>(u)[i];
            const uint32_t gw[4] = {vg.x, vg.y, vg.z, vg.w};
            const uint32_t uw[4] = {vu.x, vu.y, vu.z, vu.w};
            uint32_t r[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float g0 = bf16_bits_to_f32((uint16_t)(gw[j] & 0xffff)), g1 = bf16_bits_to_f32((uint16_t)(gw[j] >> 16));
                const float u0 = bf16_bits_to_f32((uint16_t)(uw[j] & 0xffff)), u1 = bf16_bits_to_f32((uint16_t)(uw[j] >> 16));
                r[j] = (uint32_t)f32_to_bf16_bits(silu_mul_f32(g0, u0)) | ((uint32_t)f32_to_bf16_bits(silu_mul_f32(g1, u1)) << 16);
            }
            reinterpret_cast<uint4*>(out)[i] = make_uint4(r[0], r[1], r[2], r[3]);
        }
        const size_t tail = (n8 << 3) + i;
        if (i < (n & 7)) out[tail] = f32_to_bf16_bits(silu_mul_f32(bf16_bits_to_f32(g[tail]), bf16_bits_to_f32(u[tail])));
    } else if (i < n) {
        out[i] = f32_to_bf16_bits(silu_mul_f32(bf16_bits_to_f32(g[i]), bf16_bits_to_f32(u[i])));
    }
}

// ---- RoPE -------------------------------------------------------------------------------------
// Half-split rotation of kmll (crates/inference/src/kernels/inference.rs:1066-1100):
// dims >= 2*n_freqs pass through; angle = (float)position * freqs[pair]; sinf/cosf in f32.
__device__ inline float rope_value(const float* x, size_t base, int dim, const float* freqs, int half, float position) {
    if (dim >= 2 * half) return x[base + dim];
    const int pair = dim < half ? dim : dim - half;
    const float first = x[base + pair];
    const float second = x[base + pair + half];
    const float angle = position * freqs[pair];
    const float s = sinf(angle), c = cosf(angle);
    return dim < half ? first * c - second * s : second * c + first * s;
}

__global__ void rope_kernel(const float* __restrict__ x, const float* __restrict__ freqs, int half, int position,
                            int head_dim, size_t len, float* __restrict__ out) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= len) return;
    const size_t head = i / head_dim;
    const int dim = (int)(i - head * head_dim);
    out[i] = rope_value(x, head * head_dim, dim, freqs, half, (float)position);
}

// One thread per rotated pair (or pass-through element): bf16 I/O, per-row positions.
__global__ void rope_batched_bf16_kernel(const uint16_t* __restrict__ x, const float* __restrict__ freqs, int half,
                                         const int32_t* __restrict__ positions, int batch, int n_heads, int head_dim,
                                         uint16_t* __restrict__ out) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)batch * n_heads * head_dim;
    if (i >= total) return;
    const size_t head = i / head_dim;
    const int dim = (int)(i - head * head_dim);
    const int b = (int)(head / n_heads);
    const size_t base = head * head_dim;
    if (dim >= 2 * half) {
        out[i] = x[i];
        return;
    }
    const int pair = dim < half ? dim : dim - half;
    const float first = bf16_bits_to_f32(x[base + pair]);
    const float second = bf16_bits_to_f32(x[base + pair + half]);
    const float angle = (float)positions[b] * freqs[pair];
    const float s = sinf(angle), c = cosf(angle);
    out[i] = f32_to_bf16_bits(dim < half ? first * c - second * s : second * c + first * s);
}

// write_kv_cache / apply_rope_write_kv_cache (crates/inference/src/kernels/inference.rs:1103-1162)
template <int ROPE>
__global__ void kv_write_kernel(const float* __restrict__ x, const float* __restrict__ freqs, int half, int position,
                                int head_dim, int token_len, float* __restrict__ cache, int kv_bf16) {
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= token_len) return;
    float v;
    if (ROPE) {
        const int head = i / head_dim;
        v = rope_value(x, (size_t)head * head_dim, i - head * head_dim, freqs, half, (float)position);
    } else {
        v = x[i];
    }
    if (kv_bf16) reinterpret_cast<uint16_t*>(cache)[(size_t)position * token_len + i] = f32_to_bf16_bits(v);
    else cache[(size_t)position * token_len + i] = v;
}

// prepare_incremental_attention (crates/inference/src/kernels/inference.rs:952-987)
__global__ void prepare_incremental_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                           const float* __restrict__ v, const float* __restrict__ freqs, int half,
                                           int position, int q_len, int kv_len, int head_dim, float* __restrict__ q_rot,
                                           float* __restrict__ k_cache, float* __restrict__ v_cache) {
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < q_len) {
        const int head = i / head_dim;
        q_rot[i] = rope_value(q, (size_t)head * head_dim, i - head * head_dim, freqs, half, (float)position);
    }
    if (i < kv_len) {
        const int head = i / head_dim;
        const size_t off = (size_t)position * kv_len + i;
        k_cache[off] = rope_value(k, (size_t)head * head_dim, i - head * head_dim, freqs, half, (float)position);
        v_cache[off] = v[i];
    }
}

// Per-head RMSNorm of query and key rows in place (rmsnorm_batched_bf16 over [n_heads, head_dim] with one [head_dim]
// weight, before RoPE: crates/inference/src/model.rs:10165-10194).  One warp per (row, head); q heads first, then k heads.
__global__ void __launch_bounds__(256) qk_head_rmsnorm_kernel(float* q, float* k, const uint16_t* __restrict__ q_w, const uint16_t* __restrict__ k_w,
                                                              int rows, int n_heads, int n_kv_heads, int head_dim, float eps, size_t q_stride,
                                                              size_t k_stride) {
    pdl_wait();
    pdl_launch_dependents();
    const int per_row = n_heads + n_kv_heads;
    const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= (long long)rows * per_row) return;
    const int row = (int)(item / per_row), hh = (int)(item - (long long)row * per_row);
    const bool is_q = hh < n_heads;
    const uint16_t* w = is_q ? q_w : k_w;
    if (w == nullptr) return;
    float* x = is_q ? q + (size_t)row * q_stride + (size_t)hh * head_dim : k + (size_t)row * k_stride + (size_t)(hh - n_heads) * head_dim;
    const int lane = threadIdx.x & 31;
    float v[8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = lane + 32 * j;
        v[j] = i < head_dim ? x[i] : 0.0f;
        ss += v[j] * v[j];
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)head_dim + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = lane + 32 * j;
        if (i < head_dim) x[i] = v[j] * inv * __uint_as_float((uint32_t)w[i] << 16);
    }
}

// prepare_prefill_attention_batch (crates/inference/src/kernels/inference.rs:896-949): row = position
__global__ void prepare_prefill_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                       const float* __restrict__ v, const float* __restrict__ freqs, int half,
                                       int prompt_len, int q_len, int kv_len, int head_dim, int position0,
                                       float* __restrict__ q_rot, float* __restrict__ k_cache,
                                       float* __restrict__ v_cache, int kv_bf16) {
    pdl_wait();
    const int width = q_len > kv_len ? q_len : kv_len;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)prompt_len * width) return;
    const int row = (int)(i / width);
    const int col = (int)(i - (size_t)row * width);
    const float position = (float)(position0 + row);
    if (col < q_len) {
        const int head = col / head_dim;
        const size_t base = (size_t)row * q_len + (size_t)head * head_dim;
        q_rot[(size_t)row * q_len + col] = rope_value(q, base, col - head * head_dim, freqs, half, position);
    }
    if (col < kv_len) {
        const int head = col / head_dim;
        const size_t base = (size_t)row * kv_len + (size_t)head * head_dim;
        const size_t off = (size_t)(position0 + row) * kv_len + col;
        const float kr = rope_value(k, base, col - head * head_dim, freqs, half, position);
        const float vr = v[(size_t)row * kv_len + col];
        if (kv_bf16) {  // bf16 cache: the same layout in 2-byte elements, rounded to nearest-even
            reinterpret_cast<uint16_t*>(k_cache)[off] = f32_to_bf16_bits(kr);
            reinterpret_cast<uint16_t*>(v_cache)[off] = f32_to_bf16_bits(vr);
        } else {
            k_cache[off] = kr;
            v_cache[off] = vr;
        }
    }
}

// ---- row softmax --------------------------------------------------------------------------------
// max, sum of exp(x-max), exp(x-max)/sum (crates/inference/src/kernels/inference.rs:1343-1398).
// The row is held in registers between the passes when it fits, so HBM sees one read + one write.
template <typename T>
__global__ void __launch_bounds__(256) softmax_rows_kernel(const T* __restrict__ x, int cols, T* __restrict__ out) {
    __shared__ float scratch[40];
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * cols;
    constexpr int kMaxPerThread = 16;
    float v[kMaxPerThread];
    const bool in_regs = cols <= kMaxPerThread * 256;
    float m = -INFINITY;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kMaxPerThread; ++j) {
            const int i = threadIdx.x + j * 256;
            v[j] = i < cols ? load_as_f32<T, T>(x, base + i) : -INFINITY;
            m = fmaxf(m, v[j]);
        }
    } else {
        for (int i = threadIdx.x; i < cols; i += 256) m = fmaxf(m, load_as_f32<T, T>(x, base + i));
    }
    m = block_max(m, scratch);
    float s = 0.0f;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kMaxPerThread; ++j) {
            const int i = threadIdx.x + j * 256;
            if (i < cols) {
                v[j] = expf(v[j] - m);
                s += v[j];
            }
        }
    } else {
        for (int i = threadIdx.x; i < cols; i += 256) s += expf(load_as_f32<T, T>(x, base + i) - m);
    }
    s = block_sum(s, scratch);
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kMaxPerThread; ++j) {
            const int i = threadIdx.x + j * 256;
            if (i < cols) store_from_f32(out, base + i, v[j] / s);
        }
    } else {
        for (int i = threadIdx.x; i < cols; i += 256)
            store_from_f32(out, base + i, expf(load_as_f32<T, T>(x, base + i) - m) / s);
    }
}

// ---- embedding ------------------------------------------------------------------------------------
// bf16 row -> f32 (crates/inference/src/kernels/inference.rs:21-57)
__global__ void embedding_kernel(const uint16_t* __restrict__ table, int dim, const uint32_t* __restrict__ tokens,
                                 uint32_t single_token, int token_count, int vocab, float* __restrict__ out) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)token_count * dim) return;
    const int row = (int)(i / dim);
    const int col = (int)(i - (size_t)row * dim);
    uint32_t token = tokens != nullptr ? tokens[row] : single_token;
    if (token >= (uint32_t)vocab) token = (uint32_t)vocab - 1;  // callers validate; never read out of bounds
    out[i] = bf16_bits_to_f32(table[(size_t)token * dim + col]);
}

// ---- arg-max / top-k --------------------------------------------------------------------------------
// Stage 1: per-block arg-max of a slice; stage 2 (one block) merges.  Tie -> lower index
// (crates/inference/src/kernels/inference.rs:1712,1731-1732).
__device__ inline void block_top1(float& best, uint32_t& tok) {
    __shared__ float s_logit[32];
    __shared__ uint32_t s_tok[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, off);
        const uint32_t ot = __shfl_xor_sync(0xffffffffu, tok, off);
        if (top1_better(ov, ot, best, tok)) { best = ov; tok = ot; }
    }
    if (lane == 0) { s_logit[warp] = best; s_tok[warp] = tok; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? s_logit[lane] : -INFINITY;
        tok = lane < nw ? s_tok[lane] : 0xffffffffu;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const uint32_t ot = __shfl_xor_sync(0xffffffffu, tok, off);
            if (top1_better(ov, ot, best, tok)) { best = ov; tok = ot; }
        }
    }
}

// Single-block arg-max (logit vectors are at most a few hundred KB; one block of 1024 threads
// with 128-bit loads reads them in a few microseconds and needs no scratch buffer).
__global__ void __launch_bounds__(1024) argmax_packed_kernel(const float* __restrict__ logits, size_t n,
                                                             uint64_t* __restrict__ packed_out) {
    pdl_wait();
    float best = -INFINITY;
    uint32_t tok = 0xffffffffu;
    bool have = false;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = logits[i];
        if (!have || top1_better(v, (uint32_t)i, best, tok)) { best = v; tok = (uint32_t)i; have = true; }
    }
    // a NaN-free -inf vector still needs a valid token: seed lanes without data as "no candidate"
    block_top1(best, tok);
    if (threadIdx.x == 0) packed_out[0] = pack_top1(best, tok);
}

// top-k for k <= 16: k rounds of block arg-max over the total order of f32 (f32::total_cmp,
// crates/inference/src/model.rs:11796-11806), earlier winners masked out; ties -> lower index.
__device__ inline int32_t total_order_key(float v) {
    const int32_t b = __float_as_int(v);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}
__global__ void __launch_bounds__(1024) top_k_kernel(const float* __restrict__ logits, size_t n, int k,
                                                     uint32_t* __restrict__ tokens, float* __restrict__ values) {
    __shared__ uint32_t chosen[16];
    __shared__ long long s_key[32];
    __shared__ uint32_t s_idx[32];
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int round = 0; round < k; ++round) {
        long long best = LLONG_MIN;  // key in the high bits, inverted index in the low bits
        for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
            bool taken = false;
            for (int j = 0; j < round; ++j) taken |= (chosen[j] == (uint32_t)i);
            if (taken) continue;
            const long long key = (long long)(((unsigned long long)(uint32_t)total_order_key(logits[i]) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i));
            best = key > best ? key : best;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const long long o = __shfl_xor_sync(0xffffffffu, best, off);
            best = o > best ? o : best;
        }
        if (lane == 0) s_key[warp] = best;
        __syncthreads();
        if (warp == 0) {
            best = lane < (int)(blockDim.x >> 5) ? s_key[lane] : LLONG_MIN;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const long long o = __shfl_xor_sync(0xffffffffu, best, off);
                best = o > best ? o : best;
            }
            if (lane == 0) {
                const uint32_t idx = 0xffffffffu - (uint32_t)(best & 0xffffffffll);
                chosen[round] = idx;
                tokens[round] = idx;
                values[round] = logits[idx];
            }
        }
        __syncthreads();
    }
    (void)s_idx;
}

// ---- decode-loop glue: operands that live in device memory --------------------------------------
__global__ void prepare_incremental_dyn_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                               const float* __restrict__ v, const float* __restrict__ freqs, int half,
                                               const DecodeState* __restrict__ state, int q_len, int kv_len, int head_dim,
                                               float* __restrict__ q_rot, float* __restrict__ k_cache,
                                               float* __restrict__ v_cache, int kv_bf16) {
    pdl_wait();
    const int position = state->position;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < q_len) {
        const int head = i / head_dim;
        q_rot[i] = rope_value(q, (size_t)head * head_dim, i - head * head_dim, freqs, half, (float)position);
    }
    if (i < kv_len) {
        const int head = i / head_dim;
        const size_t off = (size_t)position * kv_len + i;
        const float kr = rope_value(k, (size_t)head * head_dim, i - head * head_dim, freqs, half, (float)position);
        if (kv_bf16) {
            reinterpret_cast<uint16_t*>(k_cache)[off] = f32_to_bf16_bits(kr);
            reinterpret_cast<uint16_t*>(v_cache)[off] = f32_to_bf16_bits(v[i]);
        } else {
            k_cache[off] = kr;
            v_cache[off] = v[i];
        }
    }
}

__global__ void decode_begin_kernel(const uint16_t* __restrict__ table, int vocab, int dim, DecodeState* state,
                                    uint64_t* __restrict__ history, int history_cap, float* __restrict__ hidden,
                                    unsigned int* exchange_epoch) {
    pdl_wait();
    const uint64_t packed = state->next_top;
    uint32_t token = (uint32_t)(packed & 0xffffffffull);
    if (token >= (uint32_t)vocab) token = (uint32_t)vocab - 1;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < dim) hidden[i] = bf16_bits_to_f32(table[(size_t)token * dim + i]);
    if (i == 0) {
        const int step = state->step;
        if (step < history_cap) history[step] = packed;
        state->seq_len = state->position + 1;
        if (exchange_epoch != nullptr) *exchange_epoch += 1u;  // numbers the peer-memory exchanges of this step
    }
}

__global__ void decode_end_kernel(const uint64_t* __restrict__ packed, DecodeState* state) {
    pdl_wait();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        state->next_top = packed[0];
        state->position += 1;
        state->step += 1;
    }
}

int prepare_incremental_dyn(cudaStream_t stream, const float* q, const float* k, const float* v, const float* freqs,
                            int n_freqs, const DecodeState* state, int max_seq_len, int n_heads, int n_kv_heads,
                            int head_dim, float* q_rot, float* k_cache, float* v_cache, int kv_bf16) {
    (void)max_seq_len;
    const int q_len = n_heads * head_dim, kv_len = n_kv_heads * head_dim;
    const int width = q_len > kv_len ? q_len : kv_len;
    cudaError_t e = launch(prepare_incremental_dyn_kernel, dim3((width + 255) / 256), dim3(256), 0, stream, true, q, k, v,
                           freqs, n_freqs, state, q_len, kv_len, head_dim, q_rot, k_cache, v_cache, kv_bf16);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "prepare_incremental_dyn: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

int qk_head_rmsnorm(cudaStream_t stream, float* q, float* k, const uint16_t* q_w, const uint16_t* k_w, int rows, int n_heads, int n_kv_heads,
                    int head_dim, float eps, size_t q_stride, size_t k_stride) {
    if (q_w == nullptr && k_w == nullptr) return KMLL_OK;
    if (head_dim > 256) return fail(KMLL_ERR_UNSUPPORTED, "q/k RMSNorm: head_dim %d above 256", head_dim);
    const long long items = (long long)rows * (n_heads + n_kv_heads);
    cudaError_t e = launch(qk_head_rmsnorm_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, stream, true, q, k, q_w, k_w, rows, n_heads,
                           n_kv_heads, head_dim, eps, q_stride, k_stride);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "qk_head_rmsnorm: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

int prepare_prefill_offset(cudaStream_t stream, const float* q, const float* k, const float* v, const float* freqs,
                           int n_freqs, int rows, int q_len, int kv_len, int head_dim, int position0, float* q_rot,
                           float* k_cache, float* v_cache, int kv_bf16) {
    const int width = q_len > kv_len ? q_len : kv_len;
    const size_t total = (size_t)rows * width;
    cudaError_t e = launch(prepare_prefill_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, true, q, k, v,
                           freqs, n_freqs, rows, q_len, kv_len, head_dim, position0, q_rot, k_cache, v_cache, kv_bf16);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "prepare_prefill: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

int write_kv_row(cudaStream_t stream, const float* x, int position, int token_len, int head_dim, float* cache, int kv_bf16) {
    cudaError_t e = launch(kv_write_kernel<0>, dim3((token_len + 255) / 256), dim3(256), 0, stream, true, x, (const float*)nullptr, 0,
                           position, head_dim, token_len, cache, kv_bf16);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "write_kv_cache: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

int decode_begin(cudaStream_t stream, const uint16_t* table, int vocab, int dim, DecodeState* state, uint64_t* history,
                 int history_cap, float* hidden, unsigned int* exchange_epoch) {
    cudaError_t e = launch(decode_begin_kernel, dim3((dim + 255) / 256), dim3(256), 0, stream, true, table, vocab, dim, state,
                           history, history_cap, hidden, exchange_epoch);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "decode_begin: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

__global__ void batch_begin_kernel(const uint16_t* __restrict__ table, int vocab, int dim, BatchState* state,
                                   uint64_t* __restrict__ history, int history_cap, float* __restrict__ hidden) {
    pdl_wait();
    const int b = blockIdx.y;
    const uint64_t packed = state->next_top[b];
    uint32_t token = (uint32_t)(packed & 0xffffffffull);
    if (token >= (uint32_t)vocab) token = (uint32_t)vocab - 1;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < dim) hidden[(size_t)b * dim + i] = bf16_bits_to_f32(table[(size_t)token * dim + i]);
    if (i == 0) {
        const int step = state->step;
        if (step < history_cap) history[(size_t)b * history_cap + step] = packed;
        if (b == 0) state->seq_len = state->position + 1;
    }
}

// one block per sequence: arg-max over its logits row with the tie rule of the packed arg-max (lower token wins)
__global__ void batch_end_kernel(const float* __restrict__ logits, int vocab, BatchState* state) {
    pdl_wait();
    __shared__ float s_logit[32];
    __shared__ uint32_t s_tok[32];
    const int b = blockIdx.x;
    const float* row = logits + (size_t)b * vocab;
    float best = -INFINITY;
    uint32_t tok = 0xffffffffu;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (tok == 0xffffffffu || top1_better(v, (uint32_t)i, best, tok)) { best = v; tok = (uint32_t)i; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, off);
        const uint32_t ot = __shfl_xor_sync(0xffffffffu, tok, off);
        if (ot != 0xffffffffu && (tok == 0xffffffffu || top1_better(ov, ot, best, tok))) { best = ov; tok = ot; }
    }
    if (lane == 0) { s_logit[warp] = best; s_tok[warp] = tok; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? s_logit[lane] : -INFINITY;
        tok = lane < nw ? s_tok[lane] : 0xffffffffu;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const uint32_t ot = __shfl_xor_sync(0xffffffffu, tok, off);
            if (ot != 0xffffffffu && (tok == 0xffffffffu || top1_better(ov, ot, best, tok))) { best = ov; tok = ot; }
        }
        if (lane == 0) {
            state->next_top[b] = pack_top1(best, tok);
            if (b == 0) {
                state->position += 1;
                state->step += 1;
            }
        }
    }
}

int batch_begin(cudaStream_t stream, const uint16_t* table, int vocab, int dim, int batch, BatchState* state, uint64_t* history,
                int history_cap, float* hidden) {
    cudaError_t e = launch(batch_begin_kernel, dim3((dim + 255) / 256, batch), dim3(256), 0, stream, true, table, vocab, dim, state,
                           history, history_cap, hidden);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "batch_begin: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

int batch_end(cudaStream_t stream, const float* logits, int vocab, int batch, BatchState* state) {
    cudaError_t e = launch(batch_end_kernel, dim3(batch), dim3(1024), 0, stream, true, logits, vocab, state);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "batch_end: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

int decode_end(cudaStream_t stream, const uint64_t* packed, DecodeState* state) {
    cudaError_t e = launch(decode_end_kernel, dim3(1), dim3(32), 0, stream, true, packed, state);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "decode_end: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace kmll

using namespace kmll;

#define KMLL_LAUNCH_CHECK(expr, what)                                                         \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess) return fail(KMLL_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e__)); \
    } while (0)

extern "C" {

int kmll_rmsnorm(kmll_stream_t s, const float* x, const uint16_t* w, int n, float eps, float* y) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(w); KMLL_REQUIRE_PTR(y);
    KMLL_REQUIRE(n > 0, "rmsnorm: length must be positive, got %d", n);
    KMLL_LAUNCH_CHECK(launch(rmsnorm_kernel<float>, dim3(1), dim3(256), 0, as_stream(s), true, x, w, n, eps, y), "rmsnorm");
    return KMLL_OK;
}
int kmll_rmsnorm_batched(kmll_stream_t s, const float* x, const uint16_t* w, int batch, int dim, float eps, float* y) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(w); KMLL_REQUIRE_PTR(y);
    KMLL_REQUIRE(batch >= 0 && dim > 0, "rmsnorm_batched: bad shape batch=%d dim=%d", batch, dim);
    if (batch == 0) return KMLL_OK;
    KMLL_LAUNCH_CHECK(launch(rmsnorm_kernel<float>, dim3(batch), dim3(256), 0, as_stream(s), true, x, w, dim, eps, y), "rmsnorm_batched");
    return KMLL_OK;
}
int kmll_rmsnorm_batched_bf16io(kmll_stream_t s, const uint16_t* x, const uint16_t* w, int batch, int dim, float eps, uint16_t* y) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(w); KMLL_REQUIRE_PTR(y);
    KMLL_REQUIRE(batch >= 0 && dim > 0, "rmsnorm_batched_bf16io: bad shape batch=%d dim=%d", batch, dim);
    if (batch == 0) return KMLL_OK;
    KMLL_LAUNCH_CHECK(launch(rmsnorm_kernel<uint16_t>, dim3(batch), dim3(256), 0, as_stream(s), true, x, w, dim, eps, y), "rmsnorm_batched_bf16io");
    return KMLL_OK;
}

static int binary_f32(const char* name, int op, kmll_stream_t s, const float* a, const float* b, size_t n, float* out) {
    if (a == nullptr || b == nullptr || out == nullptr) return fail(KMLL_ERR_NULL, "%s: null pointer", name);
    if (n == 0) return KMLL_OK;
    const int vec = al16(a) && al16(b) && al16(out);
    const size_t work = vec ? (n + 3) / 4 : n;
    const unsigned grid = (unsigned)((work + 255) / 256);
    cudaError_t e = op == 0 ? launch(binary_f32_kernel<0>, dim3(grid), dim3(256), 0, as_stream(s), true, a, b, n, out, vec)
                            : launch(binary_f32_kernel<1>, dim3(grid), dim3(256), 0, as_stream(s), true, a, b, n, out, vec);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e));
    return KMLL_OK;
}
int kmll_add(kmll_stream_t s, const float* a, const float* b, size_t n, float* out) { return binary_f32("add", 0, s, a, b, n, out); }
int kmll_add_prefix(kmll_stream_t s, const float* a, const float* b, size_t count, float* out) { return binary_f32("add_prefix", 0, s, a, b, count, out); }
int kmll_silu_mul(kmll_stream_t s, const float* g, const float* u, size_t n, float* out) { return binary_f32("silu_mul", 1, s, g, u, n, out); }
int kmll_silu_mul_prefix(kmll_stream_t s, const float* g, const float* u, size_t count, float* out) { return binary_f32("silu_mul_prefix", 1, s, g, u, count, out); }

int kmll_silu_mul_bf16io(kmll_stream_t s, const uint16_t* g, const uint16_t* u, size_t n, uint16_t* out) {
    KMLL_REQUIRE_PTR(g); KMLL_REQUIRE_PTR(u); KMLL_REQUIRE_PTR(out);
    if (n == 0) return KMLL_OK;
    const int vec = al16(g) && al16(u) && al16(out);
    const size_t work = vec ? (n + 7) / 8 : n;
    KMLL_LAUNCH_CHECK(launch(silu_mul_bf16_kernel, dim3((unsigned)((work + 255) / 256)), dim3(256), 0, as_stream(s), true, g, u, n, out, vec), "silu_mul_bf16io");
    return KMLL_OK;
}

int kmll_softmax_rows(kmll_stream_t s, const float* x, int rows, int cols, float* out) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(out);
    KMLL_REQUIRE(rows >= 0 && cols > 0, "softmax_rows: bad shape rows=%d cols=%d", rows, cols);
    if (rows == 0) return KMLL_OK;
    KMLL_LAUNCH_CHECK(launch(softmax_rows_kernel<float>, dim3(rows), dim3(256), 0, as_stream(s), true, x, cols, out), "softmax_rows");
    return KMLL_OK;
}
int kmll_softmax_rows_bf16io(kmll_stream_t s, const uint16_t* x, int rows, int cols, uint16_t* out) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(out);
    KMLL_REQUIRE(rows >= 0 && cols > 0, "softmax_rows_bf16io: bad shape rows=%d cols=%d", rows, cols);
    if (rows == 0) return KMLL_OK;
    KMLL_LAUNCH_CHECK(launch(softmax_rows_kernel<uint16_t>, dim3(rows), dim3(256), 0, as_stream(s), true, x, cols, out), "softmax_rows_bf16io");
    return KMLL_OK;
}

static int check_rope(const char* name, int n_freqs, int head_dim) {
    if (head_dim <= 0 || (head_dim & 1)) return fail(KMLL_ERR_SHAPE, "%s: RoPE head_dim must be even and nonzero, got %d", name, head_dim);
    if (n_freqs < 0 || n_freqs > head_dim / 2)
        return fail(KMLL_ERR_SHAPE, "%s: RoPE frequency length mismatch: got %d, expected at most %d", name, n_freqs, head_dim / 2);
    return KMLL_OK;
}

int kmll_apply_rope(kmll_stream_t s, const float* x, const float* freqs, int n_freqs, int position, int head_dim, size_t len, float* out) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(freqs); KMLL_REQUIRE_PTR(out);
    int rc = check_rope("apply_rope", n_freqs, head_dim);
    if (rc) return rc;
    KMLL_REQUIRE(position >= 0, "apply_rope: negative position");
    KMLL_REQUIRE(len % (size_t)head_dim == 0, "apply_rope: input shape mismatch: len %zu not a multiple of head_dim %d", len, head_dim);
    if (len == 0) return KMLL_OK;
    KMLL_LAUNCH_CHECK(launch(rope_kernel, dim3((unsigned)((len + 255) / 256)), dim3(256), 0, as_stream(s), true, x, freqs, n_freqs, position, head_dim, len, out), "apply_rope");
    return KMLL_OK;
}

int kmll_apply_rope_batched_bf16io(kmll_stream_t s, const uint16_t* x, const float* freqs, int n_freqs, const int32_t* positions,
                                   int batch, int n_heads, int head_dim, uint16_t* out) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(freqs); KMLL_REQUIRE_PTR(positions); KMLL_REQUIRE_PTR(out);
    int rc = check_rope("apply_rope_batched_bf16io", n_freqs, head_dim);
    if (rc) return rc;
    KMLL_REQUIRE(batch >= 0 && n_heads > 0, "apply_rope_batched_bf16io: bad shape");
    const size_t total = (size_t)batch * n_heads * head_dim;
    if (total == 0) return KMLL_OK;
    KMLL_LAUNCH_CHECK(launch(rope_batched_bf16_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, as_stream(s), true, x, freqs, n_freqs, positions, batch, n_heads, head_dim, out), "apply_rope_batched_bf16io");
    return KMLL_OK;
}

static int check_cache(const char* name, int position, int max_seq_len, int n_kv_heads, int head_dim) {
    if (max_seq_len <= 0 || n_kv_heads <= 0 || head_dim <= 0) return fail(KMLL_ERR_SHAPE, "%s: KV cache geometry must be positive", name);
    if (position < 0 || position >= max_seq_len)
        return fail(KMLL_ERR_SHAPE, "%s: position %d exceeds max_seq_len %d", name, position, max_seq_len);
    return KMLL_OK;
}

int kmll_write_kv_cache(kmll_stream_t s, const float* x, int position, int max_seq_len, int n_kv_heads, int head_dim, float* cache) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(cache);
    int rc = check_cache("write_kv_cache", position, max_seq_len, n_kv_heads, head_dim);
    if (rc) return rc;
    const int token_len = n_kv_heads * head_dim;
    KMLL_LAUNCH_CHECK(launch(kv_write_kernel<0>, dim3((token_len + 255) / 256), dim3(256), 0, as_stream(s), true, x, (const float*)nullptr, 0, position, head_dim, token_len, cache, 0), "write_kv_cache");
    return KMLL_OK;
}
int kmll_apply_rope_write_kv_cache(kmll_stream_t s, const float* x, const float* freqs, int n_freqs, int position, int max_seq_len,
                                   int n_kv_heads, int head_dim, float* cache) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(freqs); KMLL_REQUIRE_PTR(cache);
    int rc = check_cache("apply_rope_write_kv_cache", position, max_seq_len, n_kv_heads, head_dim);
    if (rc) return rc;
    rc = check_rope("apply_rope_write_kv_cache", n_freqs, head_dim);
    if (rc) return rc;
    const int token_len = n_kv_heads * head_dim;
    KMLL_LAUNCH_CHECK(launch(kv_write_kernel<1>, dim3((token_len + 255) / 256), dim3(256), 0, as_stream(s), true, x, freqs, n_freqs, position, head_dim, token_len, cache, 0), "apply_rope_write_kv_cache");
    return KMLL_OK;
}

int kmll_prepare_incremental_attention(kmll_stream_t s, const float* q, const float* k, const float* v, const float* freqs, int n_freqs,
                                       int position, int max_seq_len, int n_heads, int n_kv_heads, int head_dim, float* q_rot,
                                       float* k_cache, float* v_cache) {
    KMLL_REQUIRE_PTR(q); KMLL_REQUIRE_PTR(k); KMLL_REQUIRE_PTR(v); KMLL_REQUIRE_PTR(freqs);
    KMLL_REQUIRE_PTR(q_rot); KMLL_REQUIRE_PTR(k_cache); KMLL_REQUIRE_PTR(v_cache);
    int rc = check_rope("prepare_incremental_attention", n_freqs, head_dim);
    if (rc) return rc;
    KMLL_REQUIRE(n_kv_heads > 0 && n_heads > 0 && n_heads % n_kv_heads == 0, "prepare_incremental_attention: n_heads must be divisible by n_kv_heads");
    rc = check_cache("prepare_incremental_attention", position, max_seq_len, n_kv_heads, head_dim);
    if (rc) return rc;
    const int q_len = n_heads * head_dim, kv_len = n_kv_heads * head_dim;
    const int width = q_len > kv_len ? q_len : kv_len;
    KMLL_LAUNCH_CHECK(launch(prepare_incremental_kernel, dim3((width + 255) / 256), dim3(256), 0, as_stream(s), true, q, k, v, freqs, n_freqs, position, q_len, kv_len, head_dim, q_rot, k_cache, v_cache), "prepare_incremental_attention");
    return KMLL_OK;
}

int kmll_prepare_prefill_attention_batch(kmll_stream_t s, const float* q, const float* k, const float* v, const float* freqs, int n_freqs,
                                         int prompt_len, int q_len, int kv_len, int head_dim, float* q_rot, float* k_cache, float* v_cache) {
    KMLL_REQUIRE_PTR(q); KMLL_REQUIRE_PTR(k); KMLL_REQUIRE_PTR(v); KMLL_REQUIRE_PTR(freqs);
    KMLL_REQUIRE_PTR(q_rot); KMLL_REQUIRE_PTR(k_cache); KMLL_REQUIRE_PTR(v_cache);
    KMLL_REQUIRE(prompt_len > 0, "prepare_prefill_attention_batch: prompt length must be nonzero");
    int rc = check_rope("prepare_prefill_attention_batch", n_freqs, head_dim);
    if (rc) return rc;
    KMLL_REQUIRE(q_len > 0 && q_len % head_dim == 0, "prepare_prefill_attention_batch: query row shape mismatch");
    KMLL_REQUIRE(kv_len > 0 && kv_len % head_dim == 0, "prepare_prefill_attention_batch: KV row shape mismatch");
    const int width = q_len > kv_len ? q_len : kv_len;
    const size_t total = (size_t)prompt_len * width;
    KMLL_LAUNCH_CHECK(launch(prepare_prefill_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, as_stream(s), true, q, k, v, freqs, n_freqs, prompt_len, q_len, kv_len, head_dim, 0, q_rot, k_cache, v_cache, 0), "prepare_prefill_attention_batch");
    return KMLL_OK;
}

int kmll_embedding(kmll_stream_t s, const uint16_t* table, int vocab, int dim, uint32_t token, float* out) {
    KMLL_REQUIRE_PTR(table); KMLL_REQUIRE_PTR(out);
    KMLL_REQUIRE(vocab > 0 && dim > 0, "embedding: table shape mismatch");
    KMLL_REQUIRE(token < (uint32_t)vocab, "embedding: token %u out of range for vocab %d", token, vocab);
    KMLL_LAUNCH_CHECK(launch(embedding_kernel, dim3((dim + 255) / 256), dim3(256), 0, as_stream(s), true, table, dim, (const uint32_t*)nullptr, token, 1, vocab, out), "embedding");
    return KMLL_OK;
}
int kmll_embedding_tokens(kmll_stream_t s, const uint16_t* table, int vocab, int dim, const uint32_t* tokens, int token_count, float* out) {
    KMLL_REQUIRE_PTR(table); KMLL_REQUIRE_PTR(out); KMLL_REQUIRE_PTR(tokens);
    KMLL_REQUIRE(vocab > 0 && dim > 0 && token_count >= 0, "embedding_tokens: shape mismatch");
    if (token_count == 0) return KMLL_OK;
    const size_t total = (size_t)token_count * dim;
    KMLL_LAUNCH_CHECK(launch(embedding_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, as_stream(s), true, table, dim, tokens, 0u, token_count, vocab, out), "embedding_tokens");
    return KMLL_OK;
}

int kmll_argmax_f32_packed(kmll_stream_t s, const float* logits, size_t n, uint64_t* packed_out) {
    KMLL_REQUIRE_PTR(logits); KMLL_REQUIRE_PTR(packed_out);
    KMLL_REQUIRE(n > 0 && n <= 0xffffffffull, "argmax_f32_packed: logits must be nonempty");
    KMLL_LAUNCH_CHECK(launch(argmax_packed_kernel, dim3(1), dim3(1024), 0, as_stream(s), true, logits, n, packed_out), "argmax_f32_packed");
    return KMLL_OK;
}
int kmll_top_k_f32(kmll_stream_t s, const float* logits, size_t n, int k, uint32_t* tokens, float* values) {
    KMLL_REQUIRE_PTR(logits); KMLL_REQUIRE_PTR(tokens); KMLL_REQUIRE_PTR(values);
    KMLL_REQUIRE(n > 0 && n <= 0xffffffffull, "top_k_f32: logits must be nonempty");
    KMLL_REQUIRE(k > 0 && k <= 16 && (size_t)k <= n, "top_k_f32: k=%d must be in 1..min(16, n)", k);
    KMLL_LAUNCH_CHECK(launch(top_k_kernel, dim3(1), dim3(1024), 0, as_stream(s), true, logits, n, k, tokens, values), "top_k_f32");
    return KMLL_OK;
}

}  // extern "C"
