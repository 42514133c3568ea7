// Batched quantized linear (prefill, batches of sequences, GEMM shapes) on the 5th-generation tensor cores, included
// by linear.cu.  Serves kmll's batched i8 linear (gemm_f32_i8_scaled_tiled_kernel,
// crates/inference/src/kernels/matmul.rs:116-214; linear_batched_i8_scaled, crates/inference/src/ops/matmul.rs:423-463)
// for RS-I8 and for W4-G128 weights, 5 or more rows of activations.
//
// y[m, r] = sum_k dequant(W)[r, k] * x[m, k] as a tcgen05.mma.kind::f16 contraction with f32 accumulators in tensor
// memory.  Operands are swapped relative to the usual GEMM: the 128 weight rows of a block are the M side of the MMA
// (tensor-memory lanes), up to 256 rows of x are the N side (tensor-memory columns), so one pass over a weight tile
// serves 256 rows of x.
//
// Exactness.  f16 carries 11 significant bits, f32 activations 24 and a dequantized W4 weight q * scale up to 14, so
// both operands are split and the cross terms are kept:
//   x = 2^-sh (x_hi + x_lo)            x_hi = f16(x 2^sh), x_lo = f16(x 2^sh - x_hi); 2^sh puts the row maximum near 2^14
//   w = w_hi + 2^-11 w_lo              w_hi = f16(q s), w_lo = f16((q s - w_hi) 2^11)   (exact: q s has 14 bits)
//   D1 += w_hi x_hi + w_hi x_lo        D2 += w_lo x_hi        y = (D1 + 2^-11 D2) 2^-sh
// The dropped term w_lo x_lo is below 2^-22 of the product, like the rounding of x_lo.  RS-I8 weights are exact in f16
// as they are (one operand plane, row scale applied in the epilogue).  All products are exact in the f32 accumulators.
//
// Data path per 64-column k-tile and pipeline stage:
//   * TMA (cp.async.bulk.tensor.2d, tensor maps over this GPU's memory only, no multicast): the raw weight tile
//     (128 rows x 32 bytes of nibbles, or x 64 int8) and the x_hi / x_lo tiles (N rows x 128 bytes) with the 128-byte
//     swizzle the MMA descriptors expect.  The f16 planes of x are written once per call by split_rows_kernel.
//   * eight warps expand the raw weights into the w_hi / w_lo tiles (same swizzled K-major layout), fence the async
//     proxy and report on an mbarrier;
//   * one thread issues the MMAs (three per 16-column k-step for W4, two for RS-I8) and commits them to the stage's
//     `empty` barrier; accumulators stay in tensor memory for the whole K loop;
//   * epilogue: the eight warps read the accumulators (tcgen05.ld), apply 2^-sh (and the RS-I8 row scale), add the
//     residual and store; with split-K the partial tiles meet in the caller's workspace and the block that arrives
//     last adds them in split order (deterministic).
// Every mbarrier wait is bounded; on time-out the block raises the device status word, frees its tensor memory and
// returns.
#pragma once

#include <cuda.h>

namespace kmll {

constexpr int kGRows = 128;        // weight rows per block = MMA M
constexpr int kGMaxN = 256;        // rows of x per block = MMA N (multiple of 16)
constexpr int kGKT = 64;           // columns per k-tile (one 128-byte swizzle atom of f16)
constexpr int kGDequantWarps = 8;
constexpr int kGThreads = (3 + kGDequantWarps) * 32;  // warp 0: TMA of x, warp 1: MMA, warps 2..9: dequantize + epilogue, warp 10: TMA of the weights
constexpr int kGMaxSplit = 8;

struct GemmParams {
    int fmt;                   // FMT_I8 / FMT_W4
    int rows, K, M;            // weight rows, columns, rows of x
    int n_block;               // rows of x per block (multiple of 16, <= 256)
    int stages;
    const void* scales;        // RS-I8: float[rows]; W4: binary16 [rows, K / 128]
    const float* inv_xscale;   // [M] 2^-sh per row of x
    float* out;                // [M, ldo]
    const float* residual;     // [M, ldo] or null
    int ldo;
    float* partial;            // split-K: [row tiles][x blocks][splits][n_block][128] partial sums
    unsigned int* counters;    // split-K: [row tiles * x blocks] arrivals, zero between launches
};

// ---- activations -> f16 planes ----------------------------------------------------------------------------------
// One block per row of x: optional RMSNorm (kmll's order x * inv * w), power-of-two scale, hi / lo split.  Block 0
// also clears the split-K counters.
__global__ void __launch_bounds__(512) split_rows_kernel(const float* __restrict__ x, int ldx, int K, const uint16_t* __restrict__ norm_w,
                                                         float eps, __half* __restrict__ x_hi, __half* __restrict__ x_lo,
                                                         float* __restrict__ inv_xscale, unsigned int* counters, int n_counters, int permute) {
    __shared__ float scratch[40];
    pdl_wait();
    const int m = blockIdx.x;
    if (m == 0)
        for (int i = threadIdx.x; i < n_counters; i += blockDim.x) counters[i] = 0u;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)m * ldx);
    const uint2* nw = reinterpret_cast<const uint2*>(norm_w);
    float ss = 0.0f, mx = 0.0f;
    for (int k4 = threadIdx.x; k4 < K / 4; k4 += blockDim.x) {
        const float4 v = xr[k4];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        if (norm_w) {
            const uint2 w = nw[k4];
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x * __uint_as_float(w.x << 16)), fabsf(v.y * __uint_as_float(w.x & 0xffff0000u))),
                                 fmaxf(fabsf(v.z * __uint_as_float(w.y << 16)), fabsf(v.w * __uint_as_float(w.y & 0xffff0000u)))));
        } else {
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    }
    ss = block_sum(ss, scratch);
    mx = block_max(mx, scratch);
    const float inv = norm_w ? 1.0f / sqrtf(ss / (float)K + eps) : 1.0f;
    const float amax = mx * inv * 1.00001f;
    float xscale = 0.0f, inv_scale = 1.0f;
    if (amax > 0.0f && amax < INFINITY) {
        const int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127;
        int sh = 13 - e;  // the row maximum lands in [2^13, 2^14): far from the binary16 overflow
        sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
        xscale = __uint_as_float((uint32_t)(sh + 127) << 23);
        inv_scale = __uint_as_float((uint32_t)(127 - sh) << 23);
    }
    // eight columns per thread and step.  permute != 0 (W4-G128): inside every group of eight columns the planes hold the
    // columns in the order 0 4 1 5 2 6 3 7 - the order in which the weight expansion of linear_gemm_kernel produces the
    // nibbles of a word; a contraction does not care in which order its terms are summed as long as both operands agree
    uint4* hi = reinterpret_cast<uint4*>(x_hi + (size_t)m * K);
    uint4* lo = reinterpret_cast<uint4*>(x_lo + (size_t)m * K);
    const uint4* nw8 = reinterpret_cast<const uint4*>(norm_w);
    for (int k8 = threadIdx.x; k8 < K / 8; k8 += blockDim.x) {
        const float4 a = xr[2 * k8], b = xr[2 * k8 + 1];
        float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        if (norm_w) {
            const uint4 w = nw8[k8];
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                v[2 * q] = v[2 * q] * inv * __uint_as_float(ww[q] << 16);
                v[2 * q + 1] = v[2 * q + 1] * inv * __uint_as_float(ww[q] & 0xffff0000u);
            }
        }
        uint32_t h[4], l[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int i0 = permute ? q : 2 * q, i1 = permute ? q + 4 : 2 * q + 1;
            const float v0 = v[i0] * xscale, v1 = v[i1] * xscale;
            const __half2 hh = __floats2half2_rn(v0, v1);
            const float2 hf = __half22float2(hh);
            const __half2 ll = __floats2half2_rn(v0 - hf.x, v1 - hf.y);
            h[q] = *reinterpret_cast<const uint32_t*>(&hh);
            l[q] = *reinterpret_cast<const uint32_t*>(&ll);
        }
        hi[k8] = make_uint4(h[0], h[1], h[2], h[3]);
        lo[k8] = make_uint4(l[0], l[1], l[2], l[3]);
    }
    if (threadIdx.x == 0) inv_xscale[m] = inv_scale;
}

// ---- tcgen05 / TMA helpers ------------------------------------------------------------------------------------------
__device__ inline void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ inline void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// shared-memory matrix descriptor: K-major operand tile with 128-byte rows in the 128-byte swizzle (what TMA writes with
// CU_TENSOR_MAP_SWIZZLE_128B): groups of 8 rows are 1024 bytes apart; version 1 (sm_100); layout type 2 = SWIZZLE_128B
__device__ inline uint64_t gemm_smem_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor of kind::f16: D = f32, A = B = binary16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
__host__ __device__ constexpr uint32_t gemm_idesc_f16(int m, int n) {
    return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ inline void gemm_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ inline void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// 2-D tiled TMA load into this block's shared memory (no multicast), completion on an mbarrier
__device__ inline void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_dst), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

// 3-D tiled TMA load (inner, row, plane)
__device__ inline void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
                 : "memory");
}

template <int FMT>
__global__ void __launch_bounds__(kGThreads, 1) linear_gemm_kernel(const GemmParams p, const __grid_constant__ CUtensorMap map_w,
                                                                  const __grid_constant__ CUtensorMap map_x) {
    constexpr bool W4 = FMT == FMT_W4;
    constexpr int kRawBytes = W4 ? kGRows * 32 : kGRows * 64;  // raw weight tile
    constexpr int kABytes = kGRows * 128;                      // one f16 operand plane of the weights
    extern __shared__ unsigned char gsmem_raw[];
    // the swizzled tiles must start on 1024-byte boundaries; the launch reserves the slack
    unsigned char* gsmem = gsmem_raw + ((1024u - (smem_u32(gsmem_raw) & 1023u)) & 1023u);
    const int n_block = p.n_block;
    const int b_bytes = n_block * 128;  // one f16 plane of the activations
    // stage layout: [A hi | A lo (W4) | B hi | B lo | raw]; every tile start is a multiple of 1024 bytes
    const int stage_bytes = (W4 ? 2 : 1) * kABytes + 2 * b_bytes + ((kRawBytes + 1023) & ~1023);
    const int stages = p.stages;
    uint64_t* full = reinterpret_cast<uint64_t*>(gsmem + (size_t)stages * stage_bytes);  // TMA bytes of a stage have landed
    uint64_t* a_ready = full + stages;   // the weight planes of a stage have been written
    uint64_t* empty = a_ready + stages;  // the MMAs that read a stage have completed
    uint64_t* all_done = empty + stages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(all_done + 1);
    __shared__ bool s_is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = blockIdx.x * kGRows;
    const int m0 = blockIdx.y * n_block;
    const int kt_all = p.K / kGKT;
    const int kt_per = (kt_all + (int)gridDim.z - 1) / (int)gridDim.z;
    const int kt0 = (int)blockIdx.z * kt_per;
    const int KT = max(0, min(kt_per, kt_all - kt0));
    constexpr uint32_t kTmemCols = W4 ? 512u : 256u;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 2); mbar_init(&a_ready[s], kGDequantWarps); mbar_init(&empty[s], 1); }
        mbar_init(all_done, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t smem_base = smem_u32(gsmem);
    const uint32_t idesc = gemm_idesc_f16(kGRows, n_block);
    // Up to 128 rows of x per block: the x_hi and x_lo tiles lie back to back in shared memory, so ONE MMA with N = 2 n_block
    // multiplies the weight plane by both (columns [0, n) and [n, 2 n) of the accumulator, added in the epilogue).  An MMA
    // costs about the same for N = 16 as for N = 64, so fewer, wider MMAs is what small batches need.
    const bool fused_n = 2 * n_block <= kGMaxN;
    const uint32_t idesc2 = gemm_idesc_f16(kGRows, 2 * n_block);

    pdl_wait();  // the f16 planes of x come from the previous kernel
    bool ok = true;
    if (warp == 0 || warp == 10) {
        // ---- TMA producers: issuing a tensor copy occupies the issuing thread for a good fraction of a microsecond, so the
        // two copies of a k-tile come from two warps: warp 0 brings both f16 planes of x with one 3-D box, warp 10 the raw
        // weight tile.  Each registers its bytes on the stage's barrier (two arrivals).
        if (lane == 0) {
#pragma unroll 1
            for (int kt = 0; kt < KT; ++kt) {
                const int stage = kt % stages, use = kt / stages;
                if (use > 0 && !mbar_wait<false>(&empty[stage], (uint32_t)(use - 1) & 1u)) { ok = false; break; }
                const uint32_t st = smem_base + (uint32_t)stage * stage_bytes;
                const uint32_t b_hi = st + (W4 ? 2 : 1) * kABytes, raw = b_hi + 2 * b_bytes;
                const int k = (kt0 + kt) * kGKT;
                if (warp == 0) {
                    mbar_arrive_expect_tx(&full[stage], (uint32_t)(2 * b_bytes));
                    tma_load_3d(b_hi, &map_x, k, m0, 0, &full[stage]);
                } else {
                    mbar_arrive_expect_tx(&full[stage], (uint32_t)kRawBytes);
                    tma_load_2d(raw, &map_w, W4 ? k / 2 : k, row0, &full[stage]);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: one thread; three (RS-I8: two) MMAs per 16-column k-step
        if (lane == 0) {
#pragma unroll 1
            for (int kt = 0; kt < KT; ++kt) {
                const int stage = kt % stages, use = kt / stages;
                if (!mbar_wait<false>(&a_ready[stage], (uint32_t)use & 1u)) { ok = false; break; }  // (implies `full`: the expanding warps waited for it)
                tcgen05_fence_after();
                const uint32_t st = smem_base + (uint32_t)stage * stage_bytes;
                const uint32_t a_hi = st, a_lo = st + kABytes;
                const uint32_t b_hi = st + (W4 ? 2 : 1) * kABytes, b_lo = b_hi + b_bytes;
#pragma unroll
                for (int ks = 0; ks < kGKT / 16; ++ks) {
                    const uint32_t first = (kt > 0 || ks > 0) ? 1u : 0u;
                    const uint64_t da = gemm_smem_desc(a_hi + ks * 32), dbh = gemm_smem_desc(b_hi + ks * 32), dbl = gemm_smem_desc(b_lo + ks * 32);
                    if (fused_n) {
                        gemm_mma_f16(tmem_base, da, dbh, idesc2, first);
                    } else {
                        gemm_mma_f16(tmem_base, da, dbh, idesc, first);
                        gemm_mma_f16(tmem_base, da, dbl, idesc, 1u);
                    }
                    if (W4) gemm_mma_f16(tmem_base + 256u, gemm_smem_desc(a_lo + ks * 32), dbh, idesc, first);
                }
                umma_commit(&empty[stage]);
            }
            if (ok) umma_commit(all_done);
        }
    } else if (warp < 2 + kGDequantWarps) {
        // ---- weight expansion: thread pair (row, half) turns 32 columns of one raw row into f16 in the swizzled tile
        const int dt = tid - 64;               // 0..255
        const int r = dt >> 1, h = dt & 1;     // tile row, which half of the 64 columns
        const int grow = min(row0 + r, p.rows - 1);
        // W4 group scales of this row, four groups (eight k-tiles) per 64-bit word: the word in use and the one after it are
        // held in registers and the next is requested when a word is first used, so the load latency (most of a microsecond,
        // as much as the whole expansion of several tiles) never sits between a tile landing and its planes being ready.
        const int n_groups = p.K >> 7;
        const unsigned short* srow = W4 ? reinterpret_cast<const unsigned short*>(p.scales) + (size_t)grow * n_groups : nullptr;
        auto load_scales4 = [&](int word) -> uint2 {
            uint32_t v[4] = {0u, 0u, 0u, 0u};
            if (W4) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (4 * word + j < n_groups) v[j] = __ldg(srow + 4 * word + j);
            }
            return make_uint2(v[0] | (v[1] << 16), v[2] | (v[3] << 16));
        };
        int word_cur = (kt0 * kGKT) >> 9;
        uint2 sc_cur = load_scales4(word_cur), sc_next = load_scales4(word_cur + 1);
#pragma unroll 1
        for (int kt = 0; kt < KT; ++kt) {
            const int stage = kt % stages, use = kt / stages;
            if (W4 && (((kt0 + kt) * kGKT) >> 9) != word_cur) {
                ++word_cur;
                sc_cur = sc_next;
                sc_next = load_scales4(word_cur + 1);
            }
            if (!mbar_wait<false>(&full[stage], (uint32_t)use & 1u)) { ok = false; break; }
            unsigned char* st = gsmem + (size_t)stage * stage_bytes;
            unsigned char* a_hi = st;
            unsigned char* a_lo = st + kABytes;
            const unsigned char* raw = st + (W4 ? 2 : 1) * kABytes + 2 * b_bytes;
            if (W4) {
                const int grp = ((kt0 + kt) * kGKT) >> 7;
                const __half sh = __ushort_as_half((unsigned short)(((grp & 2) ? sc_cur.y : sc_cur.x) >> ((grp & 1) * 16)));
                const uint4 w = *reinterpret_cast<const uint4*>(raw + r * 32 + h * 16);  // 32 nibbles = columns 32 h .. 32 h + 31
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
                const __half2 s2 = __half2half2(sh);
#pragma unroll
                for (int c = 0; c < 4; ++c) {  // one word = 8 columns -> one 16-byte chunk of each plane, columns in the order 0 4 1 5 2 6 3 7
                    // nibbles -> exact binary16 values q = n - 8 without a conversion instruction: 0x6400 | n is 1024 + n,
                    // 0x6400 | (n << 4) is 1024 + 16 n
                    const uint32_t kMagic = 0x64006400u, kSubLo = 0x64086408u /* 1032 */, kMulHi = 0x2c002c00u /* 1/16 */, kAddHi = 0xd480d480u /* -72 */;
                    const uint32_t w0 = ww[c], w8 = ww[c] >> 8;
                    uint32_t qa = lop3_and_or(w0, 0x000f000fu, kMagic), qb = lop3_and_or(w0, 0x00f000f0u, kMagic);
                    uint32_t qc = lop3_and_or(w8, 0x000f000fu, kMagic), qd = lop3_and_or(w8, 0x00f000f0u, kMagic);
                    __half2 q2[4];
                    q2[0] = __hsub2(*reinterpret_cast<__half2*>(&qa), *reinterpret_cast<const __half2*>(&kSubLo));                                            // (n0, n4)
                    q2[1] = __hfma2(*reinterpret_cast<__half2*>(&qb), *reinterpret_cast<const __half2*>(&kMulHi), *reinterpret_cast<const __half2*>(&kAddHi));  // (n1, n5)
                    q2[2] = __hsub2(*reinterpret_cast<__half2*>(&qc), *reinterpret_cast<const __half2*>(&kSubLo));                                            // (n2, n6)
                    q2[3] = __hfma2(*reinterpret_cast<__half2*>(&qd), *reinterpret_cast<const __half2*>(&kMulHi), *reinterpret_cast<const __half2*>(&kAddHi));  // (n3, n7)
                    uint32_t hi2[4], lo2[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __half2 hh = __hmul2(q2[e], s2);                          // w_hi = f16(q s)
                        const __half2 rr = __hfma2(q2[e], s2, __hneg2(hh));             // q s - w_hi, exact (a multiple of 2^-24 below half an ulp of w_hi)
                        const __half2 ll = __hmul2(rr, __float2half2_rn(2048.0f));      // w_lo = (q s - w_hi) 2^11
                        hi2[e] = *reinterpret_cast<const uint32_t*>(&hh);
                        lo2[e] = *reinterpret_cast<const uint32_t*>(&ll);
                    }
                    const int chunk = (4 * h + c) ^ (r & 7);
                    *reinterpret_cast<uint4*>(a_hi + r * 128 + chunk * 16) = make_uint4(hi2[0], hi2[1], hi2[2], hi2[3]);
                    *reinterpret_cast<uint4*>(a_lo + r * 128 + chunk * 16) = make_uint4(lo2[0], lo2[1], lo2[2], lo2[3]);
                }
            } else {
                const uint4 w0 = *reinterpret_cast<const uint4*>(raw + r * 64 + h * 32);
                const uint4 w1 = *reinterpret_cast<const uint4*>(raw + r * 64 + h * 32 + 16);
                const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t h2[4];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {  // 4 signed bytes -> 2 half2, exact (bias to unsigned, 1024 + u as a half, minus 1152)
                        const uint32_t u = ww[2 * c + e] ^ 0x80808080u;
                        uint32_t lo = __byte_perm(u, 0x64646464u, 0x4140), hi = __byte_perm(u, 0x64646464u, 0x4342);
                        const uint32_t kSub = 0x64806480u;
                        const __half2 r0 = __hsub2(*reinterpret_cast<__half2*>(&lo), *reinterpret_cast<const __half2*>(&kSub));
                        const __half2 r1 = __hsub2(*reinterpret_cast<__half2*>(&hi), *reinterpret_cast<const __half2*>(&kSub));
                        h2[2 * e] = *reinterpret_cast<const uint32_t*>(&r0);
                        h2[2 * e + 1] = *reinterpret_cast<const uint32_t*>(&r1);
                    }
                    const int chunk = (4 * h + c) ^ (r & 7);
                    *reinterpret_cast<uint4*>(a_hi + r * 128 + chunk * 16) = make_uint4(h2[0], h2[1], h2[2], h2[3]);
                }
            }
            fence_proxy_async_smem();  // the tensor core reads these tiles through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_ready[stage]);  // one arrival per warp
        }
    }

    // ---- epilogue: warps 2..9; warp w reads tensor-memory lanes 32 (w % 4) .., warps w and w + 4 share the columns
    const bool split = gridDim.z > 1;
    if (warp >= 2 && warp < 2 + kGDequantWarps) {
        ok = __all_sync(0xffffffffu, ok);
        if (ok && KT > 0 && !mbar_wait<true>(all_done, 0u)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        tcgen05_fence_after();
        if (ok) {
            const int q = warp & 3;                  // lane quarter this warp may read
            const int half = (warp - 2) >> 2;        // which half of the columns
            const int rl = q * 32 + lane;            // row inside the tile
            const int row = row0 + rl;
            const float rscale = (!W4 && row < p.rows) ? reinterpret_cast<const float*>(p.scales)[row] : 1.0f;
            const int ncols = n_block / 2;           // columns per half (multiple of 8)
            float* part = split ? p.partial + (((size_t)blockIdx.x * gridDim.y + blockIdx.y) * gridDim.z + blockIdx.z) * (size_t)n_block * kGRows : nullptr;
#pragma unroll 1
            for (int c0 = half * ncols; c0 < (half + 1) * ncols; c0 += 8) {
                uint32_t d1[8], d2[8], d3[8];
                if (KT > 0) {
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                 : "=r"(d1[0]), "=r"(d1[1]), "=r"(d1[2]), "=r"(d1[3]), "=r"(d1[4]), "=r"(d1[5]), "=r"(d1[6]), "=r"(d1[7])
                                 : "r"(taddr)
                                 : "memory");
                    if (W4)
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                     : "=r"(d2[0]), "=r"(d2[1]), "=r"(d2[2]), "=r"(d2[3]), "=r"(d2[4]), "=r"(d2[5]), "=r"(d2[6]), "=r"(d2[7])
                                     : "r"(taddr + 256u)
                                     : "memory");
                    if (fused_n)  // the x_lo half of the wide accumulator
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                     : "=r"(d3[0]), "=r"(d3[1]), "=r"(d3[2]), "=r"(d3[3]), "=r"(d3[4]), "=r"(d3[5]), "=r"(d3[6]), "=r"(d3[7])
                                     : "r"(taddr + (uint32_t)n_block)
                                     : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) d1[j] = d2[j] = d3[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int n = c0 + j, m = m0 + n;
                    float v = __uint_as_float(d1[j]);
                    if (fused_n) v += __uint_as_float(d3[j]);
                    if (W4) v = fmaf(__uint_as_float(d2[j]), 1.0f / 2048.0f, v);
                    if (split) {
                        part[(size_t)n * kGRows + rl] = v;  // scales and residual are applied after the merge
                    } else if (m < p.M && row < p.rows) {
                        v = v * p.inv_xscale[m] * rscale;
                        const size_t o = (size_t)m * p.ldo + row;
                        if (p.residual != nullptr) v = p.residual[o] + v;
                        p.out[o] = v;
                    }
                }
            }
        }
    }
    if (split) {
        // the block that delivers last adds the partial tiles in split order and finishes the rows
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned int prev = atomicAdd(&p.counters[blockIdx.x * gridDim.y + blockIdx.y], 1u);
            s_is_last = prev == gridDim.z - 1;
        }
        __syncthreads();
        if (s_is_last) {
            __threadfence();
            const float* base = p.partial + ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * gridDim.z * (size_t)n_block * kGRows;
            for (int idx = tid; idx < n_block * kGRows; idx += kGThreads) {
                const int n = idx / kGRows, rl = idx - n * kGRows;
                const int row = row0 + rl, m = m0 + n;
                if (row < p.rows && m < p.M) {
                    float acc = 0.0f;
                    for (int z = 0; z < (int)gridDim.z; ++z) acc += __ldcg(base + ((size_t)z * n_block + n) * kGRows + rl);
                    float v = acc * p.inv_xscale[m];
                    if (!W4) v *= reinterpret_cast<const float*>(p.scales)[row];
                    const size_t o = (size_t)m * p.ldo + row;
                    if (p.residual != nullptr) v = p.residual[o] + v;
                    p.out[o] = v;
                }
            }
            if (tid == 0) p.counters[blockIdx.x * gridDim.y + blockIdx.y] = 0u;
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    if (!ok) atomicCAS(&g_device_status, 0, 1);
}

}  // namespace kmll
