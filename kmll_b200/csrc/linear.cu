// Quantized linear layers (matvec and small-batch) for sm_100a.
//
// One kernel template serves RS-I8 and W4-G128 weights and every fused form (plain, +residual,
// Q/K/V triple, SiLU gate*up, lm_head arg-max, optional RMSNorm prologue).
//
// How one thread block works
//   * It owns RB = 16*MT output rows and ALL of K.  Its warps split K into contiguous runs of
//     "units" (W4: one 128-column quantization group = 64 B per row; I8: 64 columns = 64 B per
//     row).  Per unit each lane issues one 16-byte streaming load per row it holds, so a warp
//     request covers 8 rows x 64 B, fully using every 32 B sector.
//   * The integer weights are widened to exact binary16 values in registers (magic-number
//     lop3/prmt tricks, no int->float conversion instructions) and multiplied on the tensor
//     cores with mma.sync m16n8k16 (f32 accumulate): weights are the 16-row A operand, the
//     activations the 8-column B operand.  Each batch row occupies TWO columns: x scaled by a
//     power of two and split as hi = f16(x*s), lo = f16(x*s - hi), which carries ~22 bits of x,
//     so the products are exact and the result is an f32-accurate dot product.  The tensor pipe
//     does the multiply-adds; the CUDA cores only unpack, which keeps the kernel HBM-bound
//     (a plain f32 FMA loop would need ~4 instructions per 4-bit weight and be issue-bound).
//   * The k order inside an MMA is free as long as A and B agree, so activations are staged in
//     shared memory in the order the unpack produces; no shuffles are needed.
//   * W4 group scales multiply the per-group accumulator (exact dequantised value * x summed in
//     f32); the RS-I8 row scale multiplies the row total once.  kmll multiplies scale per
//     element ((w*scale)*x, crates/inference/src/kernels/inference.rs:778-781); the difference is
//     a re-association of f32 roundings, far inside kmll's own 1e-4*sqrt(K) tolerance.
//   * Warps combine their K-partials through shared memory in a fixed order, so results are
//     deterministic run to run.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "internal.cuh"

namespace kmll {
// 0 = ok; first failure wins: 1 = a wait inside the linear kernel timed out, 2 = a tensor-parallel peer did not
// deliver its part of an exchange in time
__device__ int g_device_status = 0;
}  // namespace kmll

namespace kmll {

enum { FMT_I8 = 0, FMT_W4 = 1 };

struct LinearMat {
    const uint8_t* w;       // int8 values [rows, K] or packed nibbles [rows, K/2]
    const void* scales;     // float[rows] (I8) or half[rows, K/128] (W4)
    float* out;             // [M, ldo]
    const float* residual;  // [M, ldo] or null
    int rows;
    int ldo;
};

struct LinearParams {
    const float* x;  // [M, ldx]
    int M;
    int K;
    int ldx;
    int kc;                  // K chunk staged in shared memory at a time (multiple of the unit)
    const uint16_t* norm_w;  // optional fused RMSNorm weight (bf16 bits), null = none
    float eps;
    LinearMat mat[3];
    int nmat;
    int block_start[4];  // first blockIdx.x of each matrix; [nmat] = grid size
    uint32_t* partial_tokens;
    float* partial_logits;
    const TpExchange* xc;  // tensor-parallel exchange of the next launch (set_exchange_args), or null
    int push_index, gather_index;
    float* x_out;
    int ldw, lds;  // weight row stride in bytes / W4 scales per row when K is a column slice; 0 = the K of this call
};

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

template <int FMT>
struct Fmt;
template <>
struct Fmt<FMT_W4> {
    static constexpr int kUnit = 128;       // columns per unit
    static constexpr int kRowPad = 32;      // halves: row stride = kc + 32 (64 B) -> g=0/1 rows hit disjoint banks
};
template <>
struct Fmt<FMT_I8> {
    static constexpr int kUnit = 64;
    static constexpr int kRowPad = 8;       // halves: 16 B
};

// Position of column k inside the staged activation row.
template <int FMT>
__device__ inline int stage_index(int k) {
    if (FMT == FMT_W4) {
        // k = unit*128 + t*32 + i*8 + p  ->  unit*128 + i*32 + t*8 + perm(p), perm = [0,4,1,5,2,6,3,7]^-1
        const int unit = k >> 7, t = (k >> 5) & 3, i = (k >> 3) & 3, p = k & 7;
        const int pp = ((p & 3) << 1) | (p >> 2);
        return (unit << 7) | (i << 5) | (t << 3) | pp;
    }
    return k;
}

__device__ inline void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ inline uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & b) | c
    return r;
}

// 8 nibbles of one 32-bit word -> 4 half2 registers holding (q0,q4) (q1,q5) (q2,q6) (q3,q7),
// q = nibble - 8, exact.
__device__ inline void unpack_w4(uint32_t w, uint32_t (&h)[4]) {
    const uint32_t kMagic = 0x64006400u;          // half2(1024, 1024)
    const uint32_t kSubLo = 0x64086408u;          // half2(1032, 1032)
    const uint32_t kMulHi = 0x2c002c00u;          // half2(1/16, 1/16)
    const uint32_t kAddHi = 0xd480d480u;          // half2(-72, -72)
    uint32_t lo0 = lop3_and_or(w, 0x000f000fu, kMagic);
    uint32_t hi0 = lop3_and_or(w, 0x00f000f0u, kMagic);
    uint32_t w8 = w >> 8;
    uint32_t lo1 = lop3_and_or(w8, 0x000f000fu, kMagic);
    uint32_t hi1 = lop3_and_or(w8, 0x00f000f0u, kMagic);
    __half2 r0 = __hsub2(*reinterpret_cast<__half2*>(&lo0), *reinterpret_cast<const __half2*>(&kSubLo));
    __half2 r1 = __hfma2(*reinterpret_cast<__half2*>(&hi0), *reinterpret_cast<const __half2*>(&kMulHi),
                         *reinterpret_cast<const __half2*>(&kAddHi));
    __half2 r2 = __hsub2(*reinterpret_cast<__half2*>(&lo1), *reinterpret_cast<const __half2*>(&kSubLo));
    __half2 r3 = __hfma2(*reinterpret_cast<__half2*>(&hi1), *reinterpret_cast<const __half2*>(&kMulHi),
                         *reinterpret_cast<const __half2*>(&kAddHi));
    h[0] = *reinterpret_cast<uint32_t*>(&r0);
    h[1] = *reinterpret_cast<uint32_t*>(&r1);
    h[2] = *reinterpret_cast<uint32_t*>(&r2);
    h[3] = *reinterpret_cast<uint32_t*>(&r3);
}

// 4 signed bytes -> 2 half2 registers (b0,b1) (b2,b3), exact.
__device__ inline void unpack_i8(uint32_t w, uint32_t (&h)[2]) {
    const uint32_t kSub = 0x64806480u;  // half2(1152, 1152) = 1024 + 128
    uint32_t u = w ^ 0x80808080u;       // bias to unsigned
    uint32_t lo = __byte_perm(u, 0x64646464u, 0x4140);
    uint32_t hi = __byte_perm(u, 0x64646464u, 0x4342);
    __half2 r0 = __hsub2(*reinterpret_cast<__half2*>(&lo), *reinterpret_cast<const __half2*>(&kSub));
    __half2 r1 = __hsub2(*reinterpret_cast<__half2*>(&hi), *reinterpret_cast<const __half2*>(&kSub));
    h[0] = *reinterpret_cast<uint32_t*>(&r0);
    h[1] = *reinterpret_cast<uint32_t*>(&r1);
}

template <int FMT, int MT, int NT, int EPI, int DEPTH>
__global__ void __launch_bounds__(kThreads, (MT * NT <= 2) ? 2 : 1) linear_mma_kernel(const LinearParams p) {
    using F = Fmt<FMT>;
    constexpr int UNIT = F::kUnit;
    constexpr int RB = 16 * MT;  // tile rows held by a block (for EPI_SILU: 16 gate + 16 up)
    extern __shared__ __align__(16) unsigned char smem_raw[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int M = p.M;
    const int K = p.K;
    const int kc = p.kc;
    const int row_stride = kc + F::kRowPad;  // halves

    // shared memory carve-up
    __half* xs = reinterpret_cast<__half*>(smem_raw);                    // [2*M][row_stride]
    float* red = reinterpret_cast<float*>(xs + (size_t)2 * M * row_stride + 8);  // [kWarps][RB][NT*4]
    float* misc = red + kWarps * RB * NT * 4;                            // [64]: reductions, inv, scale

    // which matrix / row block
    int mi = 0;
#pragma unroll
    for (int i = 1; i < 3; ++i)
        if (i < p.nmat && (int)blockIdx.x >= p.block_start[i]) mi = i;
    const int rb = blockIdx.x - p.block_start[mi];
    const int row0 = (EPI == EPI_SILU) ? rb * 16 : rb * RB;

    // per-thread row pointers (clamped for loads)
    const uint8_t* wrow[MT][2];
    const void* srow_base[MT];
    int rows_mt[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const LinearMat& m = (EPI == EPI_SILU) ? p.mat[mt] : p.mat[mi];
        const int base = (EPI == EPI_SILU) ? row0 : row0 + mt * 16;
        rows_mt[mt] = m.rows;
        const size_t row_bytes = (FMT == FMT_W4) ? (size_t)K / 2 : (size_t)K;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int r = base + g + h * 8;
            r = r < m.rows ? r : m.rows - 1;
            wrow[mt][h] = m.w + (size_t)r * row_bytes + t * 16;
        }
        srow_base[mt] = m.scales;
    }

    float acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[mt][nt][j] = 0.0f;

    bool bvalid[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) bvalid[nt] = (nt * 8 + g) < 2 * M;

    uint4 wreg[DEPTH][MT][2];

    // The weights do not depend on the previous kernel; the activations do.
    // (first batch of weight loads is issued before waiting on the producer of x)
    const int nchunks = (K + kc - 1) / kc;
    bool waited = false;

    for (int chunk = 0; chunk < nchunks; ++chunk) {
        const int k0 = chunk * kc;
        const int klen = min(kc, K - k0);
        const int nunits = klen / UNIT;
        const int per = (nunits + kWarps - 1) / kWarps;
        const int u_begin = min(warp * per, nunits);
        const int u_end = min(u_begin + per, nunits);

        auto load_batch = [&](int ub) {
#pragma unroll
            for (int d = 0; d < DEPTH; ++d) {
                const int u = ub + d;
                if (u < u_end) {
                    const size_t off = (FMT == FMT_W4) ? ((size_t)(k0 + u * UNIT) >> 1) : (size_t)(k0 + u * UNIT);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        wreg[d][mt][0] = ld_stream_u4(wrow[mt][0] + off);
                        wreg[d][mt][1] = ld_stream_u4(wrow[mt][1] + off);
                    }
                }
            }
        };
        load_batch(u_begin);

        if (!waited) {
            pdl_wait();
            waited = true;
        }
        __syncthreads();  // previous chunk fully consumed before xs is overwritten

        // ---- stage activations: (optional RMSNorm) -> scale by 2^e -> hi/lo binary16 ----------
        // pass A: sum of squares over the whole row (first chunk only) and max |v| of this chunk
        if (p.norm_w != nullptr && chunk == 0) {
            for (int m = 0; m < M; ++m) {
                float ss = 0.0f;
                for (int k = tid; k < K; k += kThreads) {
                    const float v = p.x[(size_t)m * p.ldx + k];
                    ss += v * v;
                }
                ss = block_sum(ss, misc);
                if (tid == 0) misc[40 + m] = 1.0f / sqrtf(ss / (float)K + p.eps);
            }
            __syncthreads();
        }
        float amax = 0.0f;
        for (int idx = tid; idx < M * klen; idx += kThreads) {
            const int m = idx / klen;
            const int kk = idx - m * klen;
            float v = p.x[(size_t)m * p.ldx + k0 + kk];
            if (p.norm_w != nullptr) v = v * misc[40 + m] * bf16_bits_to_f32(p.norm_w[k0 + kk]);
            amax = fmaxf(amax, fabsf(v));
        }
        amax = block_max(amax, misc);
        // power-of-two scale that puts the chunk maximum in [2^13, 2^14)
        float xscale = 1.0f, inv_xscale = 1.0f;
        if (amax > 0.0f && amax < INFINITY) {
            const int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127;  // floor(log2(amax)) for normals
            int sh = 13 - e;
            sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
            xscale = __uint_as_float((uint32_t)(sh + 127) << 23);
            inv_xscale = __uint_as_float((uint32_t)(127 - sh) << 23);
        }
        for (int idx = tid; idx < M * klen; idx += kThreads) {
            const int m = idx / klen;
            const int kk = idx - m * klen;
            float v = p.x[(size_t)m * p.ldx + k0 + kk];
            if (p.norm_w != nullptr) v = v * misc[40 + m] * bf16_bits_to_f32(p.norm_w[k0 + kk]);
            v *= xscale;
            const __half hi = __float2half_rn(v);
            const __half lo = __float2half_rn(v - __half2float(hi));
            const int si = stage_index<FMT>(kk);
            xs[(size_t)(2 * m) * row_stride + si] = hi;
            xs[(size_t)(2 * m + 1) * row_stride + si] = lo;
        }
        __syncthreads();

        // ---- stream this warp's units ----------------------------------------------------------
        float c[MT][NT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) c[mt][nt][j] = 0.0f;

        for (int ub = u_begin; ub < u_end; ub += DEPTH) {
            if (ub != u_begin) load_batch(ub);
#pragma unroll
            for (int d = 0; d < DEPTH; ++d) {
                const int u = ub + d;
                if (u >= u_end) break;
                if (FMT == FMT_W4) {
                    // B fragments: for word i the lane reads 8 halves (16 B) of its column
                    uint4 bq[NT][4];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (bvalid[nt]) {
                                bq[nt][i] = *reinterpret_cast<const uint4*>(
                                    xs + (size_t)(nt * 8 + g) * row_stride + u * 128 + i * 32 + t * 8);
                            } else {
                                bq[nt][i] = make_uint4(0, 0, 0, 0);
                            }
                        }
                    }
                    // group scales of the rows this lane holds
                    float gs[MT][2];
                    const int gidx = (k0 >> 7) + u;
                    const int gpr = K >> 7;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const int base = (EPI == EPI_SILU) ? row0 : row0 + mt * 16;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            int r = base + g + h * 8;
                            r = r < rows_mt[mt] ? r : rows_mt[mt] - 1;
                            const __half s = __ldg(reinterpret_cast<const __half*>(srow_base[mt]) + (size_t)r * gpr + gidx);
                            gs[mt][h] = __half2float(s) * inv_xscale;
                        }
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint32_t wlo[4] = {wreg[d][mt][0].x, wreg[d][mt][0].y, wreg[d][mt][0].z, wreg[d][mt][0].w};
                        const uint32_t whi[4] = {wreg[d][mt][1].x, wreg[d][mt][1].y, wreg[d][mt][1].z, wreg[d][mt][1].w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t al[4], ah[4];
                            unpack_w4(wlo[i], al);
                            unpack_w4(whi[i], ah);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                mma_f16(c[mt][nt], al[0], ah[0], al[1], ah[1], bq[nt][i].x, bq[nt][i].y);
                                mma_f16(c[mt][nt], al[2], ah[2], al[3], ah[3], bq[nt][i].z, bq[nt][i].w);
                            }
                        }
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            acc[mt][nt][0] = fmaf(c[mt][nt][0], gs[mt][0], acc[mt][nt][0]);
                            acc[mt][nt][1] = fmaf(c[mt][nt][1], gs[mt][0], acc[mt][nt][1]);
                            acc[mt][nt][2] = fmaf(c[mt][nt][2], gs[mt][1], acc[mt][nt][2]);
                            acc[mt][nt][3] = fmaf(c[mt][nt][3], gs[mt][1], acc[mt][nt][3]);
                            c[mt][nt][0] = c[mt][nt][1] = c[mt][nt][2] = c[mt][nt][3] = 0.0f;
                        }
                    }
                } else {
                    // I8: 16 columns per lane, natural order: two 16 B reads of the lane's column
                    uint4 bq[NT][2];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            if (bvalid[nt]) {
                                bq[nt][i] = *reinterpret_cast<const uint4*>(
                                    xs + (size_t)(nt * 8 + g) * row_stride + u * 64 + t * 16 + i * 8);
                            } else {
                                bq[nt][i] = make_uint4(0, 0, 0, 0);
                            }
                        }
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint32_t wlo[4] = {wreg[d][mt][0].x, wreg[d][mt][0].y, wreg[d][mt][0].z, wreg[d][mt][0].w};
                        const uint32_t whi[4] = {wreg[d][mt][1].x, wreg[d][mt][1].y, wreg[d][mt][1].z, wreg[d][mt][1].w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t al[2], ah[2];
                            unpack_i8(wlo[i], al);
                            unpack_i8(whi[i], ah);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                const uint4 b = bq[nt][i >> 1];
                                const uint32_t b0 = (i & 1) ? b.z : b.x;
                                const uint32_t b1 = (i & 1) ? b.w : b.y;
                                mma_f16(c[mt][nt], al[0], ah[0], al[1], ah[1], b0, b1);
                            }
                        }
                    }
                }
            }
        }
        if (FMT == FMT_I8) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[mt][nt][j] = fmaf(c[mt][nt][j], inv_xscale, acc[mt][nt][j]);
        }
    }
    pdl_launch_dependents();

    // ---- combine the warps' K-partials (fixed order) -------------------------------------------
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int m = nt * 4 + t;
            red[((size_t)warp * RB + mt * 16 + g) * (NT * 4) + m] = acc[mt][nt][0] + acc[mt][nt][1];
            red[((size_t)warp * RB + mt * 16 + g + 8) * (NT * 4) + m] = acc[mt][nt][2] + acc[mt][nt][3];
        }
    __syncthreads();

    constexpr int RO = (EPI == EPI_SILU) ? 16 : RB;  // output rows per block
    const LinearMat& om = p.mat[(EPI == EPI_SILU) ? 0 : mi];
    for (int idx = tid; idx < RO * M; idx += kThreads) {
        const int r = idx % RO;
        const int m = idx / RO;
        const int row = row0 + r;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) v += red[((size_t)w * RB + r) * (NT * 4) + m];
        if (FMT == FMT_I8 && row < om.rows) v *= reinterpret_cast<const float*>(om.scales)[row];
        if (EPI == EPI_SILU) {
            float u = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) u += red[((size_t)w * RB + 16 + r) * (NT * 4) + m];
            if (FMT == FMT_I8 && row < om.rows) u *= reinterpret_cast<const float*>(p.mat[1].scales)[row];
            v = (v / (1.0f + expf(-v))) * u;  // silu(gate) * up, crates/inference/src/kernels/inference.rs:995
        }
        if (EPI == EPI_TOP1) {
            misc[idx] = row < om.rows ? v : -INFINITY;  // M == 1, idx == r
        } else if (row < om.rows) {
            const size_t o = (size_t)m * om.ldo + row;
            if (EPI == EPI_RESIDUAL) v = om.residual[o] + v;
            om.out[o] = v;
        }
    }
    if (EPI == EPI_TOP1) {
        __syncthreads();
        if (warp == 0) {
            float best = -INFINITY;
            uint32_t tok = 0xffffffffu;
            for (int r = lane; r < RB; r += 32) {
                const float v = misc[r];
                const uint32_t tk = (row0 + r) < om.rows ? (uint32_t)(row0 + r) : 0xffffffffu;
                if (top1_better(v, tk, best, tok)) { best = v; tok = tk; }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, off);
                const uint32_t ot = __shfl_xor_sync(0xffffffffu, tok, off);
                if (top1_better(ov, ot, best, tok)) { best = ov; tok = ot; }
            }
            if (lane == 0) {
                p.partial_tokens[blockIdx.x] = tok;
                p.partial_logits[blockIdx.x] = best;
            }
        }
    }
}

// Reference-order fallback for shapes the tensor-core kernel does not take (K not a multiple of
// the unit): one warp per row, lane-strided columns, (w*scale)*x per element and the
// shuffle-down tree of kmll's matvec_i8_scaled_kernel
// (crates/inference/src/kernels/inference.rs:742-800, :180-187).
template <int EPI>
__global__ void linear_i8_rowwarp_kernel(const float* __restrict__ x, int M, int ldx, const int8_t* __restrict__ w,
                                         const float* __restrict__ scales, int rows, int K,
                                         const float* __restrict__ residual, float* __restrict__ out, int ldo) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float scale = scales[row];
    const int8_t* wr = w + (size_t)row * K;
    for (int m = 0; m < M; ++m) {
        const float* xr = x + (size_t)m * ldx;
        float acc = 0.0f;
        for (int col = lane; col < K; col += 32) acc = __fadd_rn(acc, __fmul_rn(__fmul_rn((float)wr[col], scale), xr[col]));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
        if (lane == 0) {
            const size_t o = (size_t)m * ldo + row;
            out[o] = (EPI == EPI_RESIDUAL) ? residual[o] + acc : acc;
        }
    }
}

// Reference-order lm_head + arg-max for shapes the tensor-core kernel does not take: 32 warps per
// block, one row per warp, block arg-max -> one partial per 32 rows
// (matvec_top1_i8_scaled_stage_kernel, crates/inference/src/kernels/inference.rs:331-417).
__global__ void __launch_bounds__(1024) linear_i8_rowwarp_top1_kernel(const float* __restrict__ x, const int8_t* __restrict__ w,
                                                                      const float* __restrict__ scales, int rows, int K,
                                                                      uint32_t* __restrict__ partial_tokens,
                                                                      float* __restrict__ partial_logits) {
    __shared__ float s_logit[32];
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * 32 + warp;
    float acc = -INFINITY;
    if (row < rows) {
        const float scale = scales[row];
        const int8_t* wr = w + (size_t)row * K;
        float part = 0.0f;
        for (int col = lane; col < K; col += 32) part = __fadd_rn(part, __fmul_rn(__fmul_rn((float)wr[col], scale), x[col]));
        acc = part;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
    if (lane == 0) s_logit[warp] = acc;
    __syncthreads();
    if (warp == 0) {
        const int r = blockIdx.x * 32 + lane;
        float best = r < rows ? s_logit[lane] : -INFINITY;
        uint32_t tok = r < rows ? (uint32_t)r : 0xffffffffu;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const uint32_t ot = __shfl_xor_sync(0xffffffffu, tok, off);
            if (top1_better(ov, ot, best, tok)) { best = ov; tok = ot; }
        }
        if (lane == 0) {
            partial_tokens[blockIdx.x] = tok;
            partial_logits[blockIdx.x] = best;
        }
    }
}

// Second stage of the fused arg-max: one block reduces the per-block partials
// (argmax_pairs_f32_packed_kernel, crates/inference/src/kernels/inference.rs:1812-1878).
__global__ void top1_reduce_kernel(const uint32_t* __restrict__ tokens, const float* __restrict__ logits, int count,
                                   uint32_t token_offset, uint64_t* __restrict__ packed_out, const TpExchange* xcp) {
    pdl_wait();
    __shared__ float s_logit[32];
    __shared__ uint32_t s_tok[32];
    float best = -INFINITY;
    uint32_t tok = 0xffffffffu;
    bool have = false;
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
        const float v = logits[i];
        const uint32_t tk = tokens[i];
        if (!have || top1_better(v, tk, best, tok)) { best = v; tok = tk; have = true; }
    }
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
        if (lane == 0) {
            const uint64_t packed = pack_top1(best, tok == 0xffffffffu ? tok : tok + token_offset);
            packed_out[0] = packed;
            if (xcp != nullptr) {  // tensor parallel: hand this rank's result to every rank (two 8-byte words)
                const TpExchange& xc = *xcp;
                const unsigned int epoch = *xc.epoch * (unsigned int)xc.mult + (unsigned int)xc.top_index + 1u;
                const size_t slot = ((size_t)(epoch & 1u) * xc.tp + xc.rank) * 2;
                for (int dst = 0; dst < xc.tp; ++dst) {
                    st_exchange_word(xc.top_inbox[dst] + slot, (uint32_t)(packed >> 32), epoch);
                    st_exchange_word(xc.top_inbox[dst] + slot + 1, (uint32_t)(packed & 0xffffffffull), epoch);
                }
            }
        }
    }
}

// Tensor-parallel end of a decode step: wait (bounded) for the packed arg-max of every rank, merge in rank order
// (higher logit, then lower token) and advance the decode state.
__global__ void decode_end_gather_kernel(const TpExchange* xcp, DecodeState* state, uint64_t* __restrict__ packed_final) {
    pdl_wait();
    if (threadIdx.x != 0) return;
    const TpExchange& xc = *xcp;
    const unsigned int epoch = *xc.epoch * (unsigned int)xc.mult + (unsigned int)xc.top_index + 1u;
    const uint4* box = reinterpret_cast<const uint4*>(xc.top_inbox[xc.rank]) + (size_t)(epoch & 1u) * xc.tp;
    const unsigned long long t0 = wait_clock_ticks();
    float best = -INFINITY;
    uint32_t tok = 0xffffffffu;
    for (int r = 0; r < xc.tp; ++r) {
        uint4 q;
        for (;;) {
            q = ld_exchange_pair(box + r);
            if (q.y == epoch && q.w == epoch) break;
            if (wait_clock_ticks() - t0 > kPeerWaitLimitTicks) { atomicCAS(&g_device_status, 0, 2); break; }
        }
        const float v = __uint_as_float(q.x);
        if (r == 0 || top1_better(v, q.z, best, tok)) { best = v; tok = q.z; }
    }
    const uint64_t merged = pack_top1(best, tok);
    packed_final[0] = merged;
    state->next_top = merged;
    state->position += 1;
    state->step += 1;
}

}  // namespace kmll

#include "linear_stream.cuh"
#include "linear_chain.cuh"
#include "linear_gemm.cuh"
#include "linear_gemm_small.cuh"

namespace kmll {

// ---- host side --------------------------------------------------------------------------------

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int num_sms() {
    static const int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 148;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
        return v;
    }();
    return n;
}

static bool stream_kernel_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("KMLL_LINEAR");
        return !(v != nullptr && std::strcmp(v, "legacy") == 0);
    }();
    return on;
}

// Plans and launches the persistent streaming kernel.  *launched stays false when the shape does
// not fit its shared-memory plan (the caller then uses the tiled kernel).
template <int FMT, int MT, int NT, int EPI>
static int launch_stream_variant(cudaStream_t stream, const LinearParams& lp, bool* launched, int* top1_count) {
    constexpr int ROWS = 16 * MT;
    constexpr int RU = (EPI == EPI_SILU) ? 16 : ROWS;
    StreamParams sp;
    memset(&sp, 0, sizeof(sp));
    sp.x = lp.x; sp.M = lp.M; sp.K = lp.K; sp.ldx = lp.ldx;
    sp.norm_w = lp.norm_w; sp.eps = lp.eps;
    for (int i = 0; i < 3; ++i) sp.mat[i] = lp.mat[i];
    sp.partial_tokens = lp.partial_tokens;
    sp.partial_logits = lp.partial_logits;
    sp.xc = lp.xc; sp.push_index = lp.push_index; sp.gather_index = lp.gather_index; sp.x_out = lp.x_out;
    sp.ldw = lp.ldw > 0 ? lp.ldw : (FMT == FMT_W4 ? lp.K / 2 : lp.K);
    sp.lds = lp.lds > 0 ? lp.lds : lp.K / 128;
    const int K = lp.K, M = lp.M;
    // digit rows: 16-byte reads of two rows (lanes g, g+1) must fall into different banks
    sp.xs_pitch = K + (FMT == FMT_W4 ? 16 : 64);
    auto up128 = [](size_t v) { return (v + 127) & ~(size_t)127; };
    const size_t xs_bytes = up128((size_t)4 * M * sp.xs_pitch + 16);  // digit rows + 16 zero bytes (absent MMA columns)
    const size_t red_bytes = up128((size_t)red_bufs(NT) * (kSWarps + 2) * ROWS * M * sizeof(float));  // partials + epilogue operands
    const size_t bars_bytes = 128;
    const size_t misc_bytes = 1024;
    const size_t ring_bytes = (size_t)ring_halves(NT) * 2 * kSThreads * 16;  // tile halves in flight per lane (128 KB for batch 1)
    const size_t sring_bytes = FMT == FMT_W4 ? (size_t)ring_halves(NT) * 2 * kSWarps * 32 : 0;  // scale words of the tiles in flight
    const size_t smem = xs_bytes + red_bytes + bars_bytes + misc_bytes + ring_bytes + sring_bytes;
    if (smem > 226 * 1024) return KMLL_OK;  // *launched stays false
    // the activation staging keeps x in registers (M*K <= 24576) and reads it with 16-byte loads
    if ((size_t)M * K > (size_t)kStageBlocks * 8 * kSThreads || (lp.ldx & 3) != 0 ||
        (reinterpret_cast<uintptr_t>(lp.x) & 15) != 0 || (lp.norm_w != nullptr && (reinterpret_cast<uintptr_t>(lp.norm_w) & 15) != 0))
        return KMLL_OK;
    sp.off_red = (int)xs_bytes;
    sp.off_bars = sp.off_red + (int)red_bytes;
    sp.off_misc = sp.off_bars + (int)bars_bytes;
    sp.off_ring = sp.off_misc + (int)misc_bytes;
    sp.off_sring = sp.off_ring + (int)ring_bytes;

    int units = 0;
    if (EPI == EPI_SILU) {
        sp.nmat = 1;
        sp.unit_start[0] = 0;
        units = (lp.mat[0].rows + 15) / 16;
        sp.unit_start[1] = sp.unit_start[2] = sp.unit_start[3] = units;
    } else {
        sp.nmat = lp.nmat;
        for (int i = 0; i < lp.nmat; ++i) {
            sp.unit_start[i] = units;
            units += (lp.mat[i].rows + RU - 1) / RU;
        }
        for (int i = lp.nmat; i < 4; ++i) sp.unit_start[i] = units;
    }
    sp.total_units = units;
    int grid = units < num_sms() ? units : num_sms();
    if (top1_count) *top1_count = grid;
    sp.trace = trace_next_slot(100 + FMT * 10 + EPI, grid);

    auto kern = linear_stream_kernel<FMT, MT, NT, EPI>;
    // (the attribute is per kernel and per DEVICE: a thread that moves to another GPU must set it there too, so it is
    // set on every launch; the call is cheap and not a stream operation)
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024));
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    e = launch(kern, dim3(grid), dim3(kSBlock), smem, stream, true, sp);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "linear stream launch: %s", cudaGetErrorString(e));
    *launched = true;
    return KMLL_OK;
}


static size_t linear_smem_bytes(int fmt, int M, int kc, int MT, int NT) {
    const int pad = fmt == FMT_W4 ? Fmt<FMT_W4>::kRowPad : Fmt<FMT_I8>::kRowPad;
    size_t xs = (size_t)2 * M * (kc + pad) * sizeof(__half) + 16;
    size_t red = (size_t)kWarps * 16 * MT * NT * 4 * sizeof(float);
    return xs + red + 64 * sizeof(float);
}

template <int FMT, int MT, int NT, int EPI, int DEPTH>
static int launch_variant(cudaStream_t stream, LinearParams& p, int grid) {
    auto kern = linear_mma_kernel<FMT, MT, NT, EPI, DEPTH>;
    // choose the K chunk so that the staged activations stay within ~96 KB
    const int unit = Fmt<FMT>::kUnit;
    int kc_max = (96 * 1024) / (2 * p.M * (int)sizeof(__half));
    kc_max = (kc_max / unit) * unit;
    if (kc_max < unit) kc_max = unit;
    p.kc = p.K < kc_max ? p.K : kc_max;
    const size_t smem = linear_smem_bytes(FMT, p.M, p.kc, MT, NT);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024));  // per device: every launch
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    e = launch(kern, dim3(grid), dim3(kThreads), smem, stream, true, p);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "linear launch: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

template <int FMT, int EPI>
static int launch_linear(cudaStream_t stream, LinearParams& p, int* top1_count) {
    if (p.M <= 4 && stream_kernel_enabled()) {
        bool launched = false;
        constexpr int MT = (EPI == EPI_SILU || EPI == EPI_TOP1 || EPI == EPI_RESIDUAL) ? 2 : 1;
        const int rc = p.M == 1 ? launch_stream_variant<FMT, MT, 1, EPI>(stream, p, &launched, top1_count)
                                : launch_stream_variant<FMT, MT, 2, EPI>(stream, p, &launched, top1_count);
        if (rc != KMLL_OK || launched) return rc;
    }
    if (p.xc != nullptr) return fail(KMLL_ERR_UNSUPPORTED, "linear: this shape cannot use the peer-memory exchange");
    if (top1_count) {
        int n = 0;
        for (int i = 0; i < p.nmat; ++i) n += (p.mat[i].rows + 31) / 32;
        *top1_count = n;
    }
    // rows per block: 32 when that still gives every SM a few blocks, else 16
    int total32 = 0, total16 = 0;
    for (int i = 0; i < p.nmat; ++i) {
        total32 += (p.mat[i].rows + 31) / 32;
        total16 += (p.mat[i].rows + 15) / 16;
    }
    const bool silu = (EPI == EPI_SILU);
    (void)total16;
    // the arg-max form always uses 32-row blocks so its partial count depends on rows only
    const bool mt2 = silu || EPI == EPI_TOP1 || total32 >= 2 * 148;
    int grid = 0;
    if (silu) {
        p.block_start[0] = 0;
        grid = (p.mat[0].rows + 15) / 16;
        p.block_start[1] = p.block_start[2] = p.block_start[3] = grid;
        p.nmat = 1;  // block lookup uses matrix 0 only; gate/up are mat[0], mat[1]
    } else {
        const int rb = mt2 ? 32 : 16;
        for (int i = 0; i < p.nmat; ++i) {
            p.block_start[i] = grid;
            grid += (p.mat[i].rows + rb - 1) / rb;
        }
        for (int i = p.nmat; i < 4; ++i) p.block_start[i] = grid;
    }
    const int M = p.M;
    if (EPI == EPI_TOP1 || EPI == EPI_SILU) {
        // rows-per-block fixed at 32 tile rows so the partial count is a pure function of rows
        if (M <= 4) return launch_variant<FMT, 2, 1, EPI, 4>(stream, p, grid);
        if constexpr (EPI == EPI_SILU) {
            if (M <= 8) return launch_variant<FMT, 2, 2, EPI, 2>(stream, p, grid);
            return launch_variant<FMT, 2, 4, EPI, 1>(stream, p, grid);
        }
        return fail(KMLL_ERR_UNSUPPORTED, "the arg-max epilogue supports batch <= 4 per call");
    }
    if (M <= 4) {
        if (mt2) return launch_variant<FMT, 2, 1, EPI, 4>(stream, p, grid);
        return launch_variant<FMT, 1, 1, EPI, 4>(stream, p, grid);
    }
    if (M <= 8) {
        if (mt2) return launch_variant<FMT, 2, 2, EPI, 2>(stream, p, grid);
        return launch_variant<FMT, 1, 2, EPI, 2>(stream, p, grid);
    }
    if (mt2) return launch_variant<FMT, 2, 4, EPI, 1>(stream, p, grid);
    return launch_variant<FMT, 1, 4, EPI, 2>(stream, p, grid);
}

// ---- chained kernel over prepared W4-G128 records ---------------------------------------------------------------
__device__ unsigned int g_chain_top1_counter = 0;  // arrival counter of operator-level arg-max calls (left at zero by every launch)

size_t w4_prepared_bytes(int rows, int cols, int pair) {
    if (rows <= 0 || cols <= 0 || cols % 128 != 0) return 0;
    const size_t units = pair ? ((size_t)rows + 15) / 16 : ((size_t)rows + 31) / 32;
    return units * (size_t)(cols / 128) * kCRecBytes;
}

int w4_prepare(cudaStream_t stream, const uint8_t* pa, const uint16_t* sa, const uint8_t* pb, const uint16_t* sb, int rows, int cols,
               uint8_t* out) {
    const int pair = pb != nullptr;
    const size_t words = w4_prepared_bytes(rows, cols, pair) / 4;
    if (words == 0) return fail(KMLL_ERR_SHAPE, "w4g128_prepare: rows=%d cols=%d (cols must be a positive multiple of 128)", rows, cols);
    if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return fail(KMLL_ERR_UNSUPPORTED, "w4g128_prepare: the output must be 16-byte aligned");
    const size_t blocks = (words + 255) / 256;
    if (blocks > 0x7fffffffull) return fail(KMLL_ERR_CAPACITY, "w4g128_prepare: matrix too large");
    w4_prepare_kernel<<<(unsigned)blocks, 256, 0, stream>>>(pa, sa, pb, sb, rows, cols, pair, words, reinterpret_cast<uint32_t*>(out));
    return check_launch("w4g128_prepare");
}

// Opt a kernel in to all the dynamic shared memory a block can have (227 KB less the kernel's static part).  Set to the same
// value at every launch, on whatever device is current: a CUDA graph replays its kernel nodes against the attribute the
// function has at that time, so a value that followed the needs of the last captured launch would be too small for an
// earlier node that needs more.
template <typename K>
static cudaError_t allow_all_dynamic_smem(K kernel) {
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, kernel);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - (int)fa.sharedSizeBytes);
}

int launch_chain(cudaStream_t stream, ChainParams& cp) {
    if (cp.n_phases < 1 || cp.n_phases > kCMaxPhases) return fail(KMLL_ERR_SHAPE, "chain: %d phases", cp.n_phases);
    int kmax = 0, units_max = 0;
    for (int i = 0; i < cp.n_phases; ++i) {
        ChainPhase& ph = cp.phase[i];
        if (ph.K <= 0 || ph.K % 128 != 0) return fail(KMLL_ERR_SHAPE, "chain: in_dim %d must be a positive multiple of 128", ph.K);
        if ((size_t)ph.K > (size_t)kCStageBlocks * 8 * kSThreads) return fail(KMLL_ERR_CAPACITY, "chain: in_dim %d beyond %d", ph.K, kCStageBlocks * 8 * kSThreads);
        if (ph.in_kind == CHAIN_IN_PLAIN && (ph.x == nullptr || (reinterpret_cast<uintptr_t>(ph.x) & 15u) != 0))
            return fail(KMLL_ERR_UNSUPPORTED, "chain: the input vector must be 16-byte aligned");
        if (ph.norm_w != nullptr && (reinterpret_cast<uintptr_t>(ph.norm_w) & 15u) != 0)
            return fail(KMLL_ERR_UNSUPPORTED, "chain: the norm weight must be 16-byte aligned");
        if ((ph.in_kind != CHAIN_IN_PLAIN || ph.out_kind != CHAIN_OUT_PLAIN || ph.residual_index >= 0) && cp.xc == nullptr)
            return fail(KMLL_ERR_STATE, "chain: a phase uses exchange words but no exchange tables were given");
        ph.ngroups = ph.K / 128;
        if (ph.total_units <= 0) return fail(KMLL_ERR_SHAPE, "chain: a phase has no rows");
        for (int m = 0; m < 3; ++m)
            if (ph.unit_start[m] < ph.total_units && (ph.w[m] == nullptr || (reinterpret_cast<uintptr_t>(ph.w[m]) & 15u) != 0))
                return fail(KMLL_ERR_UNSUPPORTED, "chain: prepared weights must be 16-byte aligned");
        if (ph.K > kmax) kmax = ph.K;
        if (ph.total_units > units_max) units_max = ph.total_units;
    }
    if (cp.xc != nullptr) {
        // the tables live in device memory (they are also what the other kernels of a tensor-parallel step read); the chain
        // gets a copy by value.  (host copy kept by the caller: see ChainParams::xcv)
        if (cp.xcv.epoch == nullptr) return fail(KMLL_ERR_STATE, "chain: the exchange tables were not copied into the launch parameters");
    }
    auto up128 = [](size_t v) { return (v + 127) & ~(size_t)127; };
    cp.xs_pitch = kmax + 16;
    const size_t xs_bytes = up128((size_t)4 * cp.xs_pitch + 32);
    const size_t corr_bytes = up128((size_t)(kmax / 128) * 16);
    const size_t red_bytes = up128((size_t)kCRedBufs * (kSWarps + 2) * kCRows * sizeof(float));
    const size_t bars_bytes = 128, misc_bytes = 1024;
    const size_t ring_bytes = (size_t)kCDepth * 4 * kCPlane;
    const size_t sring_bytes = (size_t)kSWarps * kCDepth * 64;
    cp.off_corr = (int)xs_bytes;
    cp.off_red = cp.off_corr + (int)corr_bytes;
    cp.off_bars = cp.off_red + (int)red_bytes;
    cp.off_misc = cp.off_bars + (int)bars_bytes;
    cp.off_ring = cp.off_misc + (int)misc_bytes;
    cp.off_sring = cp.off_ring + (int)ring_bytes;
    const size_t smem = (size_t)cp.off_sring + sring_bytes;
    if (smem > 224 * 1024) return fail(KMLL_ERR_CAPACITY, "chain: in_dim %d needs %zu bytes of shared memory", kmax, smem);
    // every block must be resident at once (blocks of one launch wait for each other's words): one block per
    // multiprocessor at most
    const int grid = units_max < num_sms() ? units_max : num_sms();
    cp.trace = trace_next_slot(400, 4 * grid);  // 24 stamps per block
    cudaError_t e = allow_all_dynamic_smem(linear_chain_kernel);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "cudaFuncSetAttribute (chain, %zu bytes wanted): %s", smem, cudaGetErrorString(e));
    e = launch(linear_chain_kernel, dim3(grid), dim3(kSBlock), smem, stream, true, cp);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "linear chain launch: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

// one phase over up to three prepared matrices with plain input and output
static void chain_plain_phase(ChainPhase& ph, int epi, const float* x, const uint16_t* norm_w, float eps, int K, const uint8_t* const* w,
                              const int* rows, float* const* outs, int nmat, const float* residual) {
    memset(&ph, 0, sizeof(ph));
    ph.epi = epi;
    ph.K = K;
    ph.x = x;
    ph.norm_w = norm_w;
    ph.eps = eps;
    ph.in_kind = CHAIN_IN_PLAIN;
    ph.out_kind = CHAIN_OUT_PLAIN;
    ph.residual = residual;
    ph.residual_index = -1;
    ph.add_residual = residual != nullptr;
    int units = 0;
    for (int m = 0; m < 3; ++m) {
        ph.unit_start[m] = units;
        if (m < nmat) {
            ph.w[m] = w[m];
            ph.out[m] = outs ? outs[m] : nullptr;
            ph.out_rows[m] = rows[m];
            units += epi == EPI_SILU ? (rows[m] + 15) / 16 : (rows[m] + 31) / 32;
        }
    }
    ph.unit_start[3] = units;
    ph.total_units = units;
}

// ---- tcgen05 GEMM path (linear_gemm.cuh) ------------------------------------------------------------------------
struct GemmPlan {
    int n_block, x_blocks, row_tiles, ksplit, stages;
    size_t smem;
    size_t off_lo, off_inv, off_partial, off_counters, total;  // workspace layout in bytes
};
static bool gemm_plan(int fmt, int M, int K, int rows, GemmPlan* out) {
    if (M < 5 || K % kGKT != 0 || (fmt == FMT_W4 && K % 128 != 0) || rows <= 0) return false;
    GemmPlan pl;
    pl.x_blocks = (M + kGMaxN - 1) / kGMaxN;
    pl.n_block = (((M + pl.x_blocks - 1) / pl.x_blocks) + 15) & ~15;
    pl.row_tiles = (rows + kGRows - 1) / kGRows;
    const int tiles = pl.row_tiles * pl.x_blocks, kt_all = K / kGKT;
    pl.ksplit = 1;
    if (tiles < 148) {  // few tiles (a narrow matrix, or few rows of x): split K so that every multiprocessor has work
        pl.ksplit = 148 / tiles;
        if (pl.ksplit > kGMaxSplit) pl.ksplit = kGMaxSplit;
        // a split must bring more than its merge costs (the last block of a tile reads every partial back): at least 8 k-tiles
        // per split for narrow blocks of x, 32 for wide ones (measured: 3584 x 3584 at 256 rows loses with 5 splits of 11
        // k-tiles, 3584 x 18944 doubles its rate with 5 splits of 59)
        const int min_kt = pl.n_block <= 64 ? 8 : 32;
        if (pl.ksplit > kt_all / min_kt) pl.ksplit = kt_all / min_kt;
        if (pl.ksplit < 1) pl.ksplit = 1;
    }
    // (raw weight tiles with 128-byte rows in a ring of their own - 4 k-tiles of W4, 2 of RS-I8 per TMA box - were measured
    // and brought nothing: the small-batch shapes are bound by the per-k-tile hand-offs, not by the row pieces TMA moves)
    const size_t raw = fmt == FMT_W4 ? 4096 : 8192;
    const size_t stage = (size_t)(fmt == FMT_W4 ? 2 : 1) * kGRows * 128 + (size_t)2 * pl.n_block * 128 + raw;
    pl.stages = (int)((220 * 1024 - 2048) / stage);
    if (pl.stages > 8) pl.stages = 8;
    if (pl.stages < 2) return false;
    pl.smem = (size_t)pl.stages * stage + (3 * pl.stages + 1) * 8 + 16 + 1024;  // + slack for the 1024-byte alignment
    auto up256 = [](size_t v) { return (v + 255) & ~(size_t)255; };
    pl.off_lo = (size_t)M * K * 2;  // the two f16 planes of x are contiguous: one 3-D tensor [2, M, K]
    pl.off_inv = up256(pl.off_lo * 2);
    pl.off_partial = pl.off_inv + up256((size_t)M * 4);
    // the layout depends on (M, K) only, so one workspace serves matrices of any height: split-K keeps tiles * splits
    // at or below 148 partial tiles; 16384 arrival counters
    if (tiles > 16384) return false;
    size_t partial_bytes = (size_t)148 * pl.n_block * kGRows * 4;
    if (M <= 32) {  // the small-batch kernel (linear_gemm_small.cuh) keeps up to kSMaxUnits partial tiles
        const size_t small = (size_t)kBtMaxUnits * (M <= 16 ? 16 : 32) * 128 * 4;
        partial_bytes = small > partial_bytes ? small : partial_bytes;
    }
    pl.off_counters = pl.off_partial + up256(partial_bytes);
    pl.total = pl.off_counters + 16384 * 4;
    *out = pl;
    return true;
}

typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                     CUtensorMapFloatOOBfill);
static TensorMapEncodeFn tensor_map_encoder() {
    static TensorMapEncodeFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess)
            return (TensorMapEncodeFn) nullptr;
        return reinterpret_cast<TensorMapEncodeFn>(sym);
    }();
    return fn;
}
// 2-D row-major tensor [rows, inner] of `elem` bytes, box = [box_rows, box_inner]
static int make_map_2d(CUtensorMap* map, CUtensorMapDataType type, int elem, const void* base, uint64_t inner, uint64_t rows, uint64_t pitch_bytes,
                       uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swizzle,
                       CUtensorMapL2promotion promotion = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (enc == nullptr) return fail(KMLL_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    (void)elem;
    const CUresult r = enc(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                           promotion, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(KMLL_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return KMLL_OK;
}

static bool gemm_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("KMLL_GEMM");
        return !(v != nullptr && v[0] == '0');
    }();
    return on;
}

static bool gemm_small_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("KMLL_GEMM_SMALL");
        return !(v != nullptr && v[0] == '0');
    }();
    return on;
}

// Small batches of W4-G128 (linear_gemm_small.cuh): byte digits of x, then ONE persistent launch over the row tiles of
// all matrices.
static int run_gemm_small(int fmt, cudaStream_t stream, const float* x, int M, int K, int ldx, const uint16_t* norm_w, float eps, const void* const* w,
                          const void* const* scales, const int* rows, float* const* outs, const float* const* residuals, const int* ldos,
                          int nmat, void* workspace, const GemmPlan& big) {
    const bool w4 = fmt == FMT_W4;
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    int8_t* digits = reinterpret_cast<int8_t*>(ws);
    float* inv = reinterpret_cast<float*>(ws + big.off_inv);
    float* partial = reinterpret_cast<float*>(ws + big.off_partial);
    unsigned int* counters = reinterpret_cast<unsigned int*>(ws + big.off_counters);
    const int permute = w4 ? 1 : 0;
    cudaError_t e = K <= 16384 ? launch(digit_rows_kernel<true>, dim3(M), dim3(512), 0, stream, true, x, ldx, K, M, norm_w, eps, digits, inv, counters, 16384, permute)
                               : launch(digit_rows_kernel<false>, dim3(M), dim3(512), 0, stream, true, x, ldx, K, M, norm_w, eps, digits, inv, counters, 16384, permute);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "digit_rows: %s", cudaGetErrorString(e));
    const int nb = M <= 16 ? 16 : 32;
    const int gp = (w4 && nb == 16 && K >= 256) ? 2 : 1;  // groups per pipeline item (SmallShape)
    const size_t smem = w4 ? (nb == 32 ? SmallShape<32, 1>::kSmemBytes : gp == 2 ? SmallShape<16, 2>::kSmemBytes : SmallShape<16, 1>::kSmemBytes)
                           : (nb == 16 ? SmallShapeI8<16>::kSmemBytes : SmallShapeI8<32>::kSmemBytes);
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (enc == nullptr) return fail(KMLL_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap map_x, map_w[kBtMaxMats];
    {   // digit planes as one 3-D tensor [4, M, K] of bytes; box = [4, nb, 128 columns], 128-byte swizzle
        const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)M, 4};
        const cuuint64_t strides[2] = {(cuuint64_t)K, (cuuint64_t)M * K};
        const cuuint32_t box[3] = {128, (cuuint32_t)nb, 4};
        const cuuint32_t estr[3] = {1, 1, 1};
        const CUresult r = enc(&map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, digits, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(KMLL_ERR_CUDA, "cuTensorMapEncodeTiled (digits) failed (%d)", (int)r);
    }
    const int G = (K + 127) / 128;
    SmallParams sp;
    memset(&sp, 0, sizeof(sp));
    sp.K = K; sp.M = M; sp.nmat = nmat;
    int tiles = 0;
    for (int i = 0; i < kBtMaxMats; ++i) {
        const int src = i < nmat ? i : 0;  // unused tensor-map slots repeat the first matrix
        if (w4)  // nibbles of one group per row and box, or of two groups in the 128-byte swizzle
            KMLL_TRY_RC(make_map_2d(&map_w[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w[src], (uint64_t)K / 2, (uint64_t)rows[src], (uint64_t)K / 2, 64 * gp, 128,
                                    gp == 2 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE));
        else  // int8 rows as they lie: 128 rows x 128 bytes, 128-byte swizzle - the MMA reads the tile TMA wrote
            KMLL_TRY_RC(make_map_2d(&map_w[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w[src], (uint64_t)K, (uint64_t)rows[src], (uint64_t)K, 128, 128,
                                    CU_TENSOR_MAP_SWIZZLE_128B));
        if (i >= nmat) continue;
        sp.mat[i].scales = w4 ? static_cast<const uint16_t*>(scales[i]) : nullptr;
        sp.mat[i].row_scales = w4 ? nullptr : static_cast<const float*>(scales[i]);
        sp.mat[i].out = outs[i];
        sp.mat[i].residual = residuals[i];
        sp.mat[i].rows = rows[i];
        sp.mat[i].ldo = ldos[i];
        sp.mat[i].tile_start = tiles;
        tiles += (rows[i] + 127) / 128;
    }
    if (tiles > 16384) return fail(KMLL_ERR_UNSUPPORTED, "linear_batched: too many row tiles for the split-K counters");
    // k-split by a cost model fitted to measurements of both small-batch kernels: a block walks `rounds` units in sequence;
    // a unit costs 0.45 us per 128-column group plus its hand-over - about 1 us when it stores its rows itself, about 4 us
    // when its partial sums go through the workspace (fence, arrival counter, the last arrival reads every partial back)
    int best = 1;
    double best_cost = 1e30;
    for (int ks = 1; ks <= kGMaxSplit; ++ks) {
        if (ks > 1 && (G / ks < 4 || tiles * ks > kBtMaxUnits)) break;
        const int units = tiles * ks, rounds = (units + 147) / 148;
        const double cost = rounds * (((G + ks - 1) / ks) * 0.45 + (ks > 1 ? 4.0 : 1.0));
        if (cost < best_cost - 1e-9) { best_cost = cost; best = ks; }
    }
    sp.tiles = tiles;
    sp.ksplit = best;
    sp.units = tiles * best;
    sp.inv_xscale = inv;
    sp.partial = partial;
    sp.counters = counters;
#ifdef KMLL_ROLE_PROFILE
    { const char* pv = std::getenv("KMLL_ROLE_PROF"); sp.prof = pv ? reinterpret_cast<unsigned long long*>(strtoull(pv, nullptr, 0)) : nullptr; }
#endif
    const int grid = sp.units < 148 ? sp.units : 148;
    if (!w4) {
        if (nb == 16) {
            auto kern = linear_gemm_small_i8_kernel<16>;
            e = allow_all_dynamic_smem(kern);
            if (e == cudaSuccess) e = launch(kern, dim3(grid), dim3(512), smem, stream, true, sp, map_w[0], map_w[1], map_w[2], map_x);
        } else {
            auto kern = linear_gemm_small_i8_kernel<32>;
            e = allow_all_dynamic_smem(kern);
            if (e == cudaSuccess) e = launch(kern, dim3(grid), dim3(512), smem, stream, true, sp, map_w[0], map_w[1], map_w[2], map_x);
        }
    } else if (nb == 32) {
        auto kern = linear_gemm_small_kernel<32, 1>;
        e = allow_all_dynamic_smem(kern);
        if (e == cudaSuccess) e = launch(kern, dim3(grid), dim3(kBtThreads), smem, stream, true, sp, map_w[0], map_w[1], map_w[2], map_x);
    } else if (gp == 2) {
        auto kern = linear_gemm_small_kernel<16, 2>;
        e = allow_all_dynamic_smem(kern);
        if (e == cudaSuccess) e = launch(kern, dim3(grid), dim3(kBtThreads), smem, stream, true, sp, map_w[0], map_w[1], map_w[2], map_x);
    } else {
        auto kern = linear_gemm_small_kernel<16, 1>;
        e = allow_all_dynamic_smem(kern);
        if (e == cudaSuccess) e = launch(kern, dim3(grid), dim3(kBtThreads), smem, stream, true, sp, map_w[0], map_w[1], map_w[2], map_x);
    }
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "linear_gemm_small (%zu bytes of shared memory): %s", smem, cudaGetErrorString(e));
    return KMLL_OK;
}

// y[m, :] (+= residual) = dequant(W_i) x[m, :] for every matrix i; x is split into f16 planes once for all of them
template <int FMT>
static int run_gemm(cudaStream_t stream, const float* x, int M, int K, int ldx, const uint16_t* norm_w, float eps, const void* const* w,
                    const void* const* scales, const int* rows, float* const* outs, const float* const* residuals, const int* ldos, int nmat,
                    void* workspace) {
    int max_rows = 0;
    for (int i = 0; i < nmat; ++i) max_rows = rows[i] > max_rows ? rows[i] : max_rows;
    GemmPlan big;
    if (!gemm_plan(FMT, M, K, max_rows, &big)) return fail(KMLL_ERR_UNSUPPORTED, "linear_batched: shape not supported by the tensor-core path");
    // 5 to 32 rows of x: the persistent kind::i8 kernels (RS-I8 needs at least two 128-column groups and K <= 131072 for its
    // s32 accumulators)
    if (M <= 32 && gemm_small_enabled() && (FMT == FMT_W4 || (K >= 256 && K <= 131072)))
        return run_gemm_small(FMT, stream, x, M, K, ldx, norm_w, eps, w, scales, rows, outs, residuals, ldos, nmat, workspace, big);
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    __half* x_hi = reinterpret_cast<__half*>(ws);
    __half* x_lo = reinterpret_cast<__half*>(ws + big.off_lo);
    float* inv = reinterpret_cast<float*>(ws + big.off_inv);
    float* partial = reinterpret_cast<float*>(ws + big.off_partial);
    unsigned int* counters = reinterpret_cast<unsigned int*>(ws + big.off_counters);
    const int n_counters = 16384;
    cudaError_t e = launch(split_rows_kernel, dim3(M), dim3(512), 0, stream, true, x, ldx, K, norm_w, eps, x_hi, x_lo, inv, counters, n_counters,
                           FMT == FMT_W4 ? 1 : 0);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "split_rows: %s", cudaGetErrorString(e));
    auto kern = linear_gemm_kernel<FMT>;
    for (int i = 0; i < nmat; ++i) {
        GemmPlan pl;
        if (!gemm_plan(FMT, M, K, rows[i], &pl)) return fail(KMLL_ERR_UNSUPPORTED, "linear_batched: shape not supported by the tensor-core path");
        CUtensorMap map_w, map_x;
        if (FMT == FMT_W4) KMLL_TRY_RC(make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w[i], (uint64_t)K / 2, (uint64_t)rows[i], (uint64_t)K / 2, 32, kGRows, CU_TENSOR_MAP_SWIZZLE_NONE));
        else KMLL_TRY_RC(make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w[i], (uint64_t)K, (uint64_t)rows[i], (uint64_t)K, 64, kGRows, CU_TENSOR_MAP_SWIZZLE_NONE));
        {   // both f16 planes of x as one 3-D tensor [2, M, K]; box = [2, n_block, 64 columns], 128-byte swizzle
            TensorMapEncodeFn enc = tensor_map_encoder();
            if (enc == nullptr) return fail(KMLL_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
            const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)M, 2};
            const cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)M * K * 2};
            const cuuint32_t box[3] = {kGKT, (cuuint32_t)pl.n_block, 2};
            const cuuint32_t estr[3] = {1, 1, 1};
            const CUresult r = enc(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, x_hi, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(KMLL_ERR_CUDA, "cuTensorMapEncodeTiled (activations) failed (%d)", (int)r);
        }
        GemmParams gp;
        memset(&gp, 0, sizeof(gp));
        gp.fmt = FMT; gp.rows = rows[i]; gp.K = K; gp.M = M;
        gp.n_block = pl.n_block; gp.stages = pl.stages;
        gp.scales = scales[i];
        gp.inv_xscale = inv;
        gp.out = outs[i];
        gp.residual = residuals[i];
        gp.ldo = ldos[i];
        gp.partial = partial;
        gp.counters = counters;
        e = allow_all_dynamic_smem(kern);
        if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "cudaFuncSetAttribute(%zu): %s", pl.smem, cudaGetErrorString(e));
        e = launch(kern, dim3(pl.row_tiles, pl.x_blocks, pl.ksplit), dim3(kGThreads), pl.smem, stream, true, gp, map_w, map_x);
        if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "linear_gemm: %s", cudaGetErrorString(e));
    }
    return KMLL_OK;
}

static bool fast_shape(int fmt, int K) { return fmt == FMT_W4 ? (K % 128 == 0) : (K % 64 == 0); }


// Exchange arguments for the next linear launch of this thread (internal.cuh).
struct ExchangeArgs {
    const TpExchange* xc = nullptr;
    int push_index = -1, gather_index = -1;
    float* x_out = nullptr;
};
static thread_local ExchangeArgs g_exchange_args;
void set_exchange_args(const TpExchange* xc, int push_index, int gather_index, float* x_out) {
    g_exchange_args.xc = xc;
    g_exchange_args.push_index = push_index;
    g_exchange_args.gather_index = gather_index;
    g_exchange_args.x_out = x_out;
}

struct MatArg {
    const void* w;
    const void* scales;
    int rows;
    float* out;
    const float* residual;
};

// Common entry: validates, then dispatches batch chunks of up to 16 rows.
template <int FMT, int EPI>
static int run_linear(const char* name, cudaStream_t stream, const float* x, int M, int K, int ldx,
                      const uint16_t* norm_w, float eps, const MatArg* mats, int nmat, int ldo_override,
                      uint32_t* partial_tokens, float* partial_logits, int* top1_count = nullptr, int ldw = 0, int lds = 0,
                      void* workspace = nullptr) {
    const ExchangeArgs xa = g_exchange_args;
    g_exchange_args = ExchangeArgs();
    if (xa.xc != nullptr && M != 1) return fail(KMLL_ERR_UNSUPPORTED, "%s: the peer-memory exchange needs batch 1", name);
    if (x == nullptr) return fail(KMLL_ERR_NULL, "%s: null input", name);
    if (M <= 0 || K <= 0) return fail(KMLL_ERR_SHAPE, "%s: batch=%d in_dim=%d must be positive", name, M, K);
    for (int i = 0; i < nmat; ++i) {
        if (mats[i].w == nullptr || mats[i].scales == nullptr) return fail(KMLL_ERR_NULL, "%s: null weight", name);
        if (EPI != EPI_TOP1 && mats[i].out == nullptr && !(EPI == EPI_SILU && i == 1))
            return fail(KMLL_ERR_NULL, "%s: null output", name);
        if (mats[i].rows <= 0) return fail(KMLL_ERR_SHAPE, "%s: weight must have rows", name);
        if (EPI == EPI_RESIDUAL && mats[i].residual == nullptr) return fail(KMLL_ERR_NULL, "%s: null residual", name);
    }
    if (FMT == FMT_W4 && K % 128 != 0)
        return fail(KMLL_ERR_SHAPE, "%s: W4-G128 needs in_dim %% 128 == 0, got %d", name, K);
    for (int i = 0; i < nmat; ++i)
        if ((reinterpret_cast<uintptr_t>(mats[i].scales) & 3u) != 0)
            return fail(KMLL_ERR_UNSUPPORTED, "%s: scales must be 4-byte aligned", name);
    const bool fast = fast_shape(FMT, K) && aligned16(mats[0].w) && (nmat < 2 || aligned16(mats[1].w)) &&
                      (nmat < 3 || aligned16(mats[2].w));
    if (!fast && xa.xc != nullptr) return fail(KMLL_ERR_UNSUPPORTED, "%s: this shape cannot use the peer-memory exchange", name);
    if (!fast) {
        if constexpr (FMT == FMT_I8 && (EPI == EPI_STORE || EPI == EPI_RESIDUAL || EPI == EPI_TOP1)) {
            if (norm_w != nullptr)
                return fail(KMLL_ERR_UNSUPPORTED, "%s: fused RMSNorm needs in_dim %% 64 == 0, got %d", name, K);
            if constexpr (EPI == EPI_TOP1) {
                const int grid = (mats[0].rows + 31) / 32;
                cudaError_t e = launch(linear_i8_rowwarp_top1_kernel, dim3(grid), dim3(1024), 0, stream, true, x,
                                       reinterpret_cast<const int8_t*>(mats[0].w), reinterpret_cast<const float*>(mats[0].scales),
                                       mats[0].rows, K, partial_tokens, partial_logits);
                if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e));
                if (top1_count) *top1_count = grid;
                return KMLL_OK;
            } else {
                for (int i = 0; i < nmat; ++i) {
                    const int ldo = ldo_override > 0 ? ldo_override : mats[i].rows;
                    const int wpb = 4;
                    cudaError_t e = launch(linear_i8_rowwarp_kernel<EPI>, dim3((mats[i].rows + wpb - 1) / wpb), dim3(wpb * 32), 0,
                                           stream, true, x, M, ldx, reinterpret_cast<const int8_t*>(mats[i].w),
                                           reinterpret_cast<const float*>(mats[i].scales), mats[i].rows, K, mats[i].residual,
                                           mats[i].out, ldo);
                    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e));
                }
                return KMLL_OK;
            }
        } else {
            return fail(KMLL_ERR_UNSUPPORTED, "%s: in_dim=%d needs a multiple of %d and 16-byte aligned weights", name, K,
                        FMT == FMT_W4 ? 128 : 64);
        }
    }
    // 5 or more rows of x and a caller-owned workspace: the tcgen05 kernel (linear_gemm.cuh), up to 256 rows of x per pass
    // over the weights
    if constexpr (EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
        GemmPlan pl;
        bool ok = workspace != nullptr && gemm_enabled() && ldw == 0 && (ldx & 3) == 0 && aligned16(x) && aligned16(workspace) &&
                  (norm_w == nullptr || (reinterpret_cast<uintptr_t>(norm_w) & 7u) == 0);
        for (int i = 0; i < nmat && ok; ++i) ok = aligned16(mats[i].w) && gemm_plan(FMT, M, K, mats[i].rows, &pl);
        if (ok) {
            const void* w_[3];
            const void* s_[3];
            int rows_[3], ldos_[3];
            float* outs_[3];
            const float* res_[3];
            for (int i = 0; i < nmat; ++i) {
                w_[i] = mats[i].w; s_[i] = mats[i].scales; rows_[i] = mats[i].rows; outs_[i] = mats[i].out;
                res_[i] = EPI == EPI_RESIDUAL ? mats[i].residual : nullptr;
                ldos_[i] = ldo_override > 0 ? ldo_override : mats[i].rows;
            }
            return run_gemm<FMT>(stream, x, M, K, ldx, norm_w, eps, w_, s_, rows_, outs_, res_, ldos_, nmat, workspace);
        }
    }
    // Batches above one row: the streaming kernel takes up to 4 rows of x per pass when its shared-memory plan fits
    // (digit rows of 4 rows of x + partial sums + the weight ring: in_dim <= 5376); a single projection without
    // RMSNorm prologue whose in_dim is larger is cut into column slices of 5376 whose results accumulate through
    // the +residual epilogue (out = out + W[:, slice] x[slice]).  Everything else goes to the tiled kernel, 16 rows
    // per pass.
    constexpr int kStreamBatchRows = 4, kStreamBatchMaxK = 5376, kSlice = 5376;
    int mstep = 16, kslice = K;
    if (M > 1 && EPI != EPI_TOP1 && stream_kernel_enabled()) {
        if (K <= kStreamBatchMaxK) {
            mstep = kStreamBatchRows;
        } else if (nmat == 1 && norm_w == nullptr && (EPI == EPI_STORE || EPI == EPI_RESIDUAL)) {
            mstep = kStreamBatchRows;
            kslice = kSlice;
        }
    }
    for (int m0 = 0; m0 < M; m0 += mstep) {
        for (int k0 = 0; k0 < K; k0 += kslice) {
            LinearParams p;
            memset(&p, 0, sizeof(p));
            p.x = x + (size_t)m0 * ldx + k0;
            p.M = (M - m0) < mstep ? (M - m0) : mstep;
            p.K = (K - k0) < kslice ? (K - k0) : kslice;
            p.ldx = ldx;
            p.norm_w = norm_w;
            p.eps = eps;
            p.nmat = nmat;
            p.ldw = ldw > 0 ? ldw : (FMT == FMT_W4 ? K / 2 : K);
            p.lds = lds > 0 ? lds : K / 128;
            for (int i = 0; i < nmat; ++i) {
                const int ldo = ldo_override > 0 ? ldo_override : mats[i].rows;
                p.mat[i].w = reinterpret_cast<const uint8_t*>(mats[i].w) + (FMT == FMT_W4 ? k0 / 2 : k0);
                p.mat[i].scales = FMT == FMT_W4 ? static_cast<const void*>(reinterpret_cast<const uint16_t*>(mats[i].scales) + k0 / 128)
                                                : mats[i].scales;
                p.mat[i].rows = mats[i].rows;
                p.mat[i].ldo = ldo;
                p.mat[i].out = mats[i].out ? mats[i].out + (size_t)m0 * ldo : nullptr;
                p.mat[i].residual = mats[i].residual ? mats[i].residual + (size_t)m0 * ldo : nullptr;
                if (k0 > 0) p.mat[i].residual = p.mat[i].out;  // later slices accumulate onto the first one's result
            }
            p.partial_tokens = partial_tokens;
            p.partial_logits = partial_logits;
            p.xc = xa.xc;
            p.push_index = xa.xc ? xa.push_index : -1;
            p.gather_index = xa.xc ? xa.gather_index : -1;
            p.x_out = xa.x_out;
            int rc;
            if constexpr (EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
                rc = k0 == 0 ? launch_linear<FMT, EPI>(stream, p, top1_count) : launch_linear<FMT, EPI_RESIDUAL>(stream, p, top1_count);
            } else {
                rc = launch_linear<FMT, EPI>(stream, p, top1_count);
            }
            if (rc != KMLL_OK) return rc;
        }
    }
    return KMLL_OK;
}

template <int FMT>
static int run_top1(const char* name, cudaStream_t stream, const float* x, const uint16_t* norm_w, float eps,
                    const void* w, const void* scales, int rows, int cols, uint32_t* partial_tokens,
                    float* partial_logits, uint64_t* packed_out, uint32_t token_offset = 0, const TpExchange* xc = nullptr) {
    if (partial_tokens == nullptr || partial_logits == nullptr || packed_out == nullptr) {
        set_exchange_args(nullptr, -1, -1, nullptr);
        return fail(KMLL_ERR_NULL, "%s: null partial/packed buffer", name);
    }
    MatArg m = {w, scales, rows, nullptr, nullptr};
    int count = 0;
    int rc = run_linear<FMT, EPI_TOP1>(name, stream, x, 1, cols, cols, norm_w, eps, &m, 1, 0, partial_tokens, partial_logits, &count);
    if (rc != KMLL_OK) return rc;
    cudaError_t e = launch(top1_reduce_kernel, dim3(1), dim3(256), 0, stream, true, (const uint32_t*)partial_tokens,
                           (const float*)partial_logits, count, token_offset, packed_out, xc);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e));
    return KMLL_OK;
}

// Merge of per-rank packed arg-max results (tensor parallel lm_head): higher logit, then lower token.
__global__ void merge_packed_kernel(const uint64_t* __restrict__ packed_all, int n, uint64_t* __restrict__ packed_out) {
    pdl_wait();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    float best = -INFINITY;
    uint32_t tok = 0xffffffffu;
    for (int i = 0; i < n; ++i) {
        const uint64_t p = packed_all[i];
        const float v = __uint_as_float((uint32_t)(p >> 32));
        const uint32_t tk = (uint32_t)(p & 0xffffffffull);
        if (i == 0 || top1_better(v, tk, best, tok)) { best = v; tok = tk; }
    }
    packed_out[0] = pack_top1(best, tok);
}

int linear_top1_offset(cudaStream_t stream, int fmt, const float* x, const uint16_t* norm_w, float eps, const void* w,
                       const void* scales, int rows, int cols, uint32_t token_offset, uint32_t* partial_tokens,
                       float* partial_logits, uint64_t* packed_out, const TpExchange* xc) {
    if (fmt == FMT_W4)
        return run_top1<FMT_W4>("linear_top1", stream, x, norm_w, eps, w, scales, rows, cols, partial_tokens, partial_logits,
                                packed_out, token_offset, xc);
    return run_top1<FMT_I8>("linear_top1", stream, x, norm_w, eps, w, scales, rows, cols, partial_tokens, partial_logits,
                            packed_out, token_offset, xc);
}

int decode_end_gather(cudaStream_t stream, const TpExchange* xc, DecodeState* state, uint64_t* packed_final) {
    cudaError_t e = launch(decode_end_gather_kernel, dim3(1), dim3(32), 0, stream, true, xc, state, packed_final);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "decode_end_gather: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

// ---- batched fused forms (rows of x = independent sequences), used by the lockstep batch decoder ------------
template <int FMT>
static int batched_forms(int form, cudaStream_t stream, const float* x, int batch, const uint16_t* norm_w, float eps,
                         const void* const* w, const void* const* scales, const int* rows, int cols, float* const* outs,
                         const float* residual, void* workspace, float* gate_tmp, float* up_tmp) {
    switch (form) {
        case 0: {  // RMSNorm + QKV
            MatArg m[3] = {{w[0], scales[0], rows[0], outs[0], nullptr}, {w[1], scales[1], rows[1], outs[1], nullptr},
                           {w[2], scales[2], rows[2], outs[2], nullptr}};
            return run_linear<FMT, EPI_STORE>("linear_qkv_batched_norm", stream, x, batch, cols, cols, norm_w, eps, m, 3, 0, nullptr, nullptr,
                                              nullptr, 0, 0, workspace);
        }
        case 1: {  // RMSNorm + gate/up + SiLU*up
            GemmPlan pl;
            if (workspace != nullptr && gate_tmp != nullptr && up_tmp != nullptr && gemm_enabled() && gemm_plan(FMT, batch, cols, rows[0], &pl)) {
                // tensor-core path: gate and up as two plain projections over the same f16 planes of x, then SiLU(gate) * up
                MatArg m[2] = {{w[0], scales[0], rows[0], gate_tmp, nullptr}, {w[1], scales[1], rows[0], up_tmp, nullptr}};
                const int rc = run_linear<FMT, EPI_STORE>("silu_gate_up_batched_norm", stream, x, batch, cols, cols, norm_w, eps, m, 2, 0, nullptr,
                                                          nullptr, nullptr, 0, 0, workspace);
                if (rc != KMLL_OK) return rc;
                return kmll_silu_mul_prefix(stream, gate_tmp, up_tmp, (size_t)batch * rows[0], outs[0]);
            }
            MatArg m[2] = {{w[0], scales[0], rows[0], outs[0], nullptr}, {w[1], scales[1], rows[0], nullptr, nullptr}};
            return run_linear<FMT, EPI_SILU>("silu_gate_up_batched_norm", stream, x, batch, cols, cols, norm_w, eps, m, 2, 0, nullptr, nullptr);
        }
        case 2: {  // projection + residual
            MatArg m = {w[0], scales[0], rows[0], outs[0], residual};
            return run_linear<FMT, EPI_RESIDUAL>("linear_residual_batched", stream, x, batch, cols, cols, nullptr, 0.f, &m, 1, 0, nullptr, nullptr,
                                                 nullptr, 0, 0, workspace);
        }
        default: {  // (RMSNorm +) projection
            MatArg m = {w[0], scales[0], rows[0], outs[0], nullptr};
            return run_linear<FMT, EPI_STORE>("linear_batched_norm", stream, x, batch, cols, cols, norm_w, eps, &m, 1, 0, nullptr, nullptr,
                                              nullptr, 0, 0, workspace);
        }
    }
}
int linear_batched_form(int form, cudaStream_t stream, int fmt, const float* x, int batch, const uint16_t* norm_w, float eps,
                        const void* const* w, const void* const* scales, const int* rows, int cols, float* const* outs,
                        const float* residual, void* workspace, float* gate_tmp, float* up_tmp) {
    if (fmt == FMT_W4)
        return batched_forms<FMT_W4>(form, stream, x, batch, norm_w, eps, w, scales, rows, cols, outs, residual, workspace, gate_tmp, up_tmp);
    return batched_forms<FMT_I8>(form, stream, x, batch, norm_w, eps, w, scales, rows, cols, outs, residual, workspace, gate_tmp, up_tmp);
}
size_t linear_batched_workspace_bytes(int batch, int in_dim) {
    GemmPlan pl;
    if (!gemm_plan(FMT_W4, batch, in_dim - in_dim % 128, 128, &pl) || in_dim % 64 != 0) {
        if (!gemm_plan(FMT_I8, batch, in_dim, 128, &pl)) return 0;
    }
    return pl.total;
}

int merge_packed_top1(cudaStream_t stream, const uint64_t* packed_all, int n, uint64_t* packed_out) {
    cudaError_t e = launch(merge_packed_kernel, dim3(1), dim3(32), 0, stream, true, packed_all, n, packed_out);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "merge_packed_top1: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

}  // namespace kmll

using namespace kmll;

// An entry point that returns before run_linear has consumed the exchange arguments must not leave them armed
// for an unrelated later call of the same thread.
#define KMLL_REQUIRE_PTR_DISARM(p)                                                          \
    do {                                                                                    \
        if ((p) == nullptr) {                                                               \
            set_exchange_args(nullptr, -1, -1, nullptr);                                    \
            return ::kmll::fail(KMLL_ERR_NULL, "%s: null pointer %s", __func__, #p);        \
        }                                                                                   \
    } while (0)

extern "C" {

// Upper bound of the partial (token, logit) pairs a fused lm_head arg-max writes for `rows` vocabulary rows: one per
// 32-row block.  The streaming kernel writes one per thread block (at most the number of multiprocessors), never
// more than this bound.  kmll's own plan has one partial per 4 rows (ops/inference.rs:254-260); callers size
// their buffers through this function on both sides, so only the bound is part of the contract.
int kmll_linear_top1_partial_count(int rows) { return rows <= 0 ? 0 : (rows + 31) / 32; }

int kmll_device_status(int* status_out) {
    KMLL_REQUIRE_PTR(status_out);
    cudaError_t e = cudaMemcpyFromSymbol(status_out, g_device_status, sizeof(int));
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
    return KMLL_OK;
}

int kmll_linear_i8(kmll_stream_t s, const float* x, const int8_t* w, const float* scales, int rows, int cols, float* y) {
    MatArg m = {w, scales, rows, y, nullptr};
    return run_linear<FMT_I8, EPI_STORE>(__func__, as_stream(s), x, 1, cols, cols, nullptr, 0.f, &m, 1, 0, nullptr, nullptr);
}
int kmll_linear_w4g128(kmll_stream_t s, const float* x, const uint8_t* packed, const uint16_t* gs, int rows, int cols, float* y) {
    MatArg m = {packed, gs, rows, y, nullptr};
    return run_linear<FMT_W4, EPI_STORE>(__func__, as_stream(s), x, 1, cols, cols, nullptr, 0.f, &m, 1, 0, nullptr, nullptr);
}
int kmll_linear_residual_i8(kmll_stream_t s, const float* x, const int8_t* w, const float* scales, const float* residual,
                            int rows, int cols, float* out) {
    MatArg m = {w, scales, rows, out, residual};
    return run_linear<FMT_I8, EPI_RESIDUAL>(__func__, as_stream(s), x, 1, cols, cols, nullptr, 0.f, &m, 1, 0, nullptr, nullptr);
}
int kmll_linear_residual_w4g128(kmll_stream_t s, const float* x, const uint8_t* packed, const uint16_t* gs,
                                const float* residual, int rows, int cols, float* out) {
    MatArg m = {packed, gs, rows, out, residual};
    return run_linear<FMT_W4, EPI_RESIDUAL>(__func__, as_stream(s), x, 1, cols, cols, nullptr, 0.f, &m, 1, 0, nullptr, nullptr);
}

int kmll_linear_triple_i8(kmll_stream_t s, const float* x, const int8_t* wq, const float* sq, const int8_t* wk,
                          const float* sk, const int8_t* wv, const float* sv, int q_rows, int kv_rows, int cols,
                          float* q, float* k, float* v) {
    MatArg m[3] = {{wq, sq, q_rows, q, nullptr}, {wk, sk, kv_rows, k, nullptr}, {wv, sv, kv_rows, v, nullptr}};
    return run_linear<FMT_I8, EPI_STORE>(__func__, as_stream(s), x, 1, cols, cols, nullptr, 0.f, m, 3, 0, nullptr, nullptr);
}
int kmll_linear_triple_w4g128(kmll_stream_t s, const float* x, const uint8_t* wq, const uint16_t* sq, const uint8_t* wk,
                              const uint16_t* sk, const uint8_t* wv, const uint16_t* sv, int q_rows, int kv_rows, int cols,
                              float* q, float* k, float* v) {
    MatArg m[3] = {{wq, sq, q_rows, q, nullptr}, {wk, sk, kv_rows, k, nullptr}, {wv, sv, kv_rows, v, nullptr}};
    return run_linear<FMT_W4, EPI_STORE>(__func__, as_stream(s), x, 1, cols, cols, nullptr, 0.f, m, 3, 0, nullptr, nullptr);
}
int kmll_linear_pair_i8(kmll_stream_t s, const float* x, const int8_t* wa, const float* sa, const int8_t* wb, const float* sb, int rows,
                        int cols, float* out_a, float* out_b) {
    MatArg m[2] = {{wa, sa, rows, out_a, nullptr}, {wb, sb, rows, out_b, nullptr}};
    return run_linear<FMT_I8, EPI_STORE>(__func__, as_stream(s), x, 1, cols, cols, nullptr, 0.f, m, 2, 0, nullptr, nullptr);
}
int kmll_linear_pair_w4g128(kmll_stream_t s, const float* x, const uint8_t* wa, const uint16_t* sa, const uint8_t* wb, const uint16_t* sb,
                            int rows, int cols, float* out_a, float* out_b) {
    MatArg m[2] = {{wa, sa, rows, out_a, nullptr}, {wb, sb, rows, out_b, nullptr}};
    return run_linear<FMT_W4, EPI_STORE>(__func__, as_stream(s), x, 1, cols, cols, nullptr, 0.f, m, 2, 0, nullptr, nullptr);
}
int kmll_rmsnorm_linear_triple_i8(kmll_stream_t s, const float* x, const uint16_t* nw, float eps, const int8_t* wq,
                                  const float* sq, const int8_t* wk, const float* sk, const int8_t* wv, const float* sv,
                                  int q_rows, int kv_rows, int cols, float* q, float* k, float* v) {
    KMLL_REQUIRE_PTR_DISARM(nw);
    MatArg m[3] = {{wq, sq, q_rows, q, nullptr}, {wk, sk, kv_rows, k, nullptr}, {wv, sv, kv_rows, v, nullptr}};
    return run_linear<FMT_I8, EPI_STORE>(__func__, as_stream(s), x, 1, cols, cols, nw, eps, m, 3, 0, nullptr, nullptr);
}
int kmll_rmsnorm_linear_triple_w4g128(kmll_stream_t s, const float* x, const uint16_t* nw, float eps, const uint8_t* wq,
                                      const uint16_t* sq, const uint8_t* wk, const uint16_t* sk, const uint8_t* wv,
                                      const uint16_t* sv, int q_rows, int kv_rows, int cols, float* q, float* k, float* v) {
    KMLL_REQUIRE_PTR_DISARM(nw);
    MatArg m[3] = {{wq, sq, q_rows, q, nullptr}, {wk, sk, kv_rows, k, nullptr}, {wv, sv, kv_rows, v, nullptr}};
    return run_linear<FMT_W4, EPI_STORE>(__func__, as_stream(s), x, 1, cols, cols, nw, eps, m, 3, 0, nullptr, nullptr);
}

int kmll_silu_gate_up_i8(kmll_stream_t s, const float* x, const int8_t* wg, const float* sg, const int8_t* wu,
                         const float* su, int rows, int cols, float* out) {
    MatArg m[2] = {{wg, sg, rows, out, nullptr}, {wu, su, rows, nullptr, nullptr}};
    return run_linear<FMT_I8, EPI_SILU>(__func__, as_stream(s), x, 1, cols, cols, nullptr, 0.f, m, 2, 0, nullptr, nullptr);
}
int kmll_silu_gate_up_w4g128(kmll_stream_t s, const float* x, const uint8_t* wg, const uint16_t* sg, const uint8_t* wu,
                             const uint16_t* su, int rows, int cols, float* out) {
    MatArg m[2] = {{wg, sg, rows, out, nullptr}, {wu, su, rows, nullptr, nullptr}};
    return run_linear<FMT_W4, EPI_SILU>(__func__, as_stream(s), x, 1, cols, cols, nullptr, 0.f, m, 2, 0, nullptr, nullptr);
}
int kmll_rmsnorm_silu_gate_up_i8(kmll_stream_t s, const float* x, const uint16_t* nw, float eps, const int8_t* wg,
                                 const float* sg, const int8_t* wu, const float* su, int rows, int cols, float* out) {
    KMLL_REQUIRE_PTR_DISARM(nw);
    MatArg m[2] = {{wg, sg, rows, out, nullptr}, {wu, su, rows, nullptr, nullptr}};
    return run_linear<FMT_I8, EPI_SILU>(__func__, as_stream(s), x, 1, cols, cols, nw, eps, m, 2, 0, nullptr, nullptr);
}
int kmll_rmsnorm_silu_gate_up_w4g128(kmll_stream_t s, const float* x, const uint16_t* nw, float eps, const uint8_t* wg,
                                     const uint16_t* sg, const uint8_t* wu, const uint16_t* su, int rows, int cols,
                                     float* out) {
    KMLL_REQUIRE_PTR_DISARM(nw);
    MatArg m[2] = {{wg, sg, rows, out, nullptr}, {wu, su, rows, nullptr, nullptr}};
    return run_linear<FMT_W4, EPI_SILU>(__func__, as_stream(s), x, 1, cols, cols, nw, eps, m, 2, 0, nullptr, nullptr);
}

int kmll_linear_top1_i8(kmll_stream_t s, const float* x, const int8_t* w, const float* scales, int rows, int cols,
                        uint32_t* pt, float* pl, uint64_t* packed_out) {
    return run_top1<FMT_I8>(__func__, as_stream(s), x, nullptr, 0.f, w, scales, rows, cols, pt, pl, packed_out);
}
int kmll_linear_top1_w4g128(kmll_stream_t s, const float* x, const uint8_t* packed, const uint16_t* gs, int rows, int cols,
                            uint32_t* pt, float* pl, uint64_t* packed_out) {
    return run_top1<FMT_W4>(__func__, as_stream(s), x, nullptr, 0.f, packed, gs, rows, cols, pt, pl, packed_out);
}
int kmll_rmsnorm_linear_top1_i8(kmll_stream_t s, const float* x, const uint16_t* nw, float eps, const int8_t* w,
                                const float* scales, int rows, int cols, uint32_t* pt, float* pl, uint64_t* packed_out) {
    KMLL_REQUIRE_PTR_DISARM(nw);
    return run_top1<FMT_I8>(__func__, as_stream(s), x, nw, eps, w, scales, rows, cols, pt, pl, packed_out);
}
int kmll_rmsnorm_linear_top1_w4g128(kmll_stream_t s, const float* x, const uint16_t* nw, float eps, const uint8_t* packed,
                                    const uint16_t* gs, int rows, int cols, uint32_t* pt, float* pl, uint64_t* packed_out) {
    KMLL_REQUIRE_PTR_DISARM(nw);
    return run_top1<FMT_W4>(__func__, as_stream(s), x, nw, eps, packed, gs, rows, cols, pt, pl, packed_out);
}

size_t kmll_w4g128_prepared_bytes(int rows, int cols) { return w4_prepared_bytes(rows, cols, 0); }
size_t kmll_w4g128_prepared_pair_bytes(int rows, int cols) { return w4_prepared_bytes(rows, cols, 1); }
int kmll_w4g128_prepare(kmll_stream_t s, const uint8_t* packed, const uint16_t* gscales, int rows, int cols, uint8_t* prepared) {
    KMLL_REQUIRE_PTR(packed); KMLL_REQUIRE_PTR(gscales); KMLL_REQUIRE_PTR(prepared);
    return w4_prepare(as_stream(s), packed, gscales, nullptr, nullptr, rows, cols, prepared);
}
int kmll_w4g128_prepare_pair(kmll_stream_t s, const uint8_t* gate_packed, const uint16_t* gate_gscales, const uint8_t* up_packed,
                             const uint16_t* up_gscales, int rows, int cols, uint8_t* prepared) {
    KMLL_REQUIRE_PTR(gate_packed); KMLL_REQUIRE_PTR(gate_gscales); KMLL_REQUIRE_PTR(up_packed); KMLL_REQUIRE_PTR(up_gscales);
    KMLL_REQUIRE_PTR(prepared);
    return w4_prepare(as_stream(s), gate_packed, gate_gscales, up_packed, up_gscales, rows, cols, prepared);
}
int kmll_linear_w4p(kmll_stream_t s, const float* x, const uint16_t* norm_w, float eps, const uint8_t* prepared, const float* residual,
                    int rows, int cols, float* y) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(prepared); KMLL_REQUIRE_PTR(y);
    KMLL_REQUIRE(rows > 0 && cols > 0, "%s: rows=%d cols=%d must be positive", __func__, rows, cols);
    ChainParams cp;
    memset(&cp, 0, sizeof(cp));
    cp.n_phases = 1;
    chain_plain_phase(cp.phase[0], residual ? EPI_RESIDUAL : EPI_STORE, x, norm_w, eps, cols, &prepared, &rows, &y, 1, residual);
    return launch_chain(as_stream(s), cp);
}
int kmll_linear_triple_w4p(kmll_stream_t s, const float* x, const uint16_t* norm_w, float eps, const uint8_t* pq, const uint8_t* pk,
                           const uint8_t* pv, int q_rows, int kv_rows, int cols, float* q, float* k, float* v) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(pq); KMLL_REQUIRE_PTR(pk); KMLL_REQUIRE_PTR(pv); KMLL_REQUIRE_PTR(q); KMLL_REQUIRE_PTR(k);
    KMLL_REQUIRE_PTR(v);
    KMLL_REQUIRE(q_rows > 0 && kv_rows > 0 && cols > 0, "%s: sizes must be positive", __func__);
    const uint8_t* w[3] = {pq, pk, pv};
    const int rows[3] = {q_rows, kv_rows, kv_rows};
    float* outs[3] = {q, k, v};
    ChainParams cp;
    memset(&cp, 0, sizeof(cp));
    cp.n_phases = 1;
    chain_plain_phase(cp.phase[0], EPI_STORE, x, norm_w, eps, cols, w, rows, outs, 3, nullptr);
    return launch_chain(as_stream(s), cp);
}
int kmll_silu_gate_up_w4p(kmll_stream_t s, const float* x, const uint16_t* norm_w, float eps, const uint8_t* prepared_pair, int rows,
                          int cols, float* out) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(prepared_pair); KMLL_REQUIRE_PTR(out);
    KMLL_REQUIRE(rows > 0 && cols > 0, "%s: rows=%d cols=%d must be positive", __func__, rows, cols);
    ChainParams cp;
    memset(&cp, 0, sizeof(cp));
    cp.n_phases = 1;
    chain_plain_phase(cp.phase[0], EPI_SILU, x, norm_w, eps, cols, &prepared_pair, &rows, &out, 1, nullptr);
    return launch_chain(as_stream(s), cp);
}
int kmll_linear_top1_w4p(kmll_stream_t s, const float* x, const uint16_t* norm_w, float eps, const uint8_t* prepared, int rows, int cols,
                         uint32_t* pt, float* pl, uint64_t* packed_out) {
    KMLL_REQUIRE_PTR(x); KMLL_REQUIRE_PTR(prepared); KMLL_REQUIRE_PTR(pt); KMLL_REQUIRE_PTR(pl); KMLL_REQUIRE_PTR(packed_out);
    KMLL_REQUIRE(rows > 0 && cols > 0, "%s: rows=%d cols=%d must be positive", __func__, rows, cols);
    ChainParams cp;
    memset(&cp, 0, sizeof(cp));
    cp.n_phases = 1;
    chain_plain_phase(cp.phase[0], EPI_TOP1, x, norm_w, eps, cols, &prepared, &rows, nullptr, 1, nullptr);
    cp.partial_tokens = pt;
    cp.partial_logits = pl;
    cp.packed_out = packed_out;
    void* counter = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&counter, g_chain_top1_counter);
    if (e != cudaSuccess) return fail(KMLL_ERR_CUDA, "%s: cudaGetSymbolAddress: %s", __func__, cudaGetErrorString(e));
    cp.top1_counter = static_cast<unsigned int*>(counter);
    return launch_chain(as_stream(s), cp);
}

size_t kmll_linear_batched_workspace_bytes(int batch, int in_dim) {
    if (batch <= 0 || in_dim <= 0) return 0;
    return linear_batched_workspace_bytes(batch, in_dim);
}
int kmll_linear_batched_i8(kmll_stream_t s, const float* x, const int8_t* w, const float* scales, int batch, int in_dim,
                           int out_dim, void* workspace, float* y) {
    MatArg m = {w, scales, out_dim, y, nullptr};
    return run_linear<FMT_I8, EPI_STORE>(__func__, as_stream(s), x, batch, in_dim, in_dim, nullptr, 0.f, &m, 1, 0, nullptr, nullptr, nullptr, 0,
                                         0, workspace);
}
int kmll_linear_batched_w4g128(kmll_stream_t s, const float* x, const uint8_t* packed, const uint16_t* gs, int batch,
                               int in_dim, int out_dim, void* workspace, float* y) {
    MatArg m = {packed, gs, out_dim, y, nullptr};
    return run_linear<FMT_W4, EPI_STORE>(__func__, as_stream(s), x, batch, in_dim, in_dim, nullptr, 0.f, &m, 1, 0, nullptr, nullptr, nullptr, 0,
                                         0, workspace);
}
int kmll_linear_qkv_batched_i8(kmll_stream_t s, const float* x, const int8_t* wq, const float* sq, const int8_t* wk,
                               const float* sk, const int8_t* wv, const float* sv, int batch, int in_dim, int q_dim,
                               int kv_dim, void* workspace, float* q, float* k, float* v) {
    MatArg m[3] = {{wq, sq, q_dim, q, nullptr}, {wk, sk, kv_dim, k, nullptr}, {wv, sv, kv_dim, v, nullptr}};
    return run_linear<FMT_I8, EPI_STORE>(__func__, as_stream(s), x, batch, in_dim, in_dim, nullptr, 0.f, m, 3, 0, nullptr, nullptr, nullptr, 0, 0,
                                         workspace);
}
int kmll_linear_qkv_batched_w4g128(kmll_stream_t s, const float* x, const uint8_t* wq, const uint16_t* sq, const uint8_t* wk,
                                   const uint16_t* sk, const uint8_t* wv, const uint16_t* sv, int batch, int in_dim,
                                   int q_dim, int kv_dim, void* workspace, float* q, float* k, float* v) {
    MatArg m[3] = {{wq, sq, q_dim, q, nullptr}, {wk, sk, kv_dim, k, nullptr}, {wv, sv, kv_dim, v, nullptr}};
    return run_linear<FMT_W4, EPI_STORE>(__func__, as_stream(s), x, batch, in_dim, in_dim, nullptr, 0.f, m, 3, 0, nullptr, nullptr, nullptr, 0, 0,
                                         workspace);
}

}  // extern "C"
