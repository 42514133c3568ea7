// Persistent streaming form of the quantized linear kernel (batch <= 4), included by linear.cu.
//
// One thread block (16 warps) per SM stays resident and walks over "units" of 16 (or 32) weight rows.
// The activations are staged in shared memory ONCE per block as byte digits (see stage_activations).
// The weights stream from HBM into a shared-memory ring with 16-byte asynchronous copies; the ring is
// private to each lane (a lane reads back exactly the bytes its own copies wrote), so
// cp.async.wait_group is the only synchronisation, accesses are bank-conflict free and no registers
// hold data in flight.  Eight tiles per lane are in flight: 128 KB per SM.  A warp request covers
// 8 rows x 64 B.  The 16 warps split the columns of a unit; their partial sums meet in shared memory
// once per unit and the warp that delivers last adds them in fixed warp order and runs the epilogue,
// so warps drift freely, loads never drain and nobody spin-waits.
// Bulk-copy (TMA) staging of the weights was measured and rejected for this kernel: issuing a bulk
// copy blocks the issuing lane for hundreds of cycles.
//
// Arithmetic: the integer tensor-core MMA (mma.sync m16n8k32, s8 weights x u8 activation bytes -> s32).
// x * 2^sh is rounded to an integer X below 2^22 in magnitude whose bytes (u0, u1, 64 + (X >> 16)) are
// three of the eight MMA columns; a fourth column of ones yields the row sum of the weights, which
// removes the offset of the top byte.  One MMA multiplies 16 weight rows by all bytes at once,
// exactly (int32 accumulation cannot round).  RS-I8 weights are the A operand as they lie in memory -
// no unpack instruction at all; a W4 nibble n = q + 8 becomes the int8 value 16*q with three logic
// operations per eight weights.  The only roundings are x -> 23-bit fixed point relative to max|x|
// and the final few f32 operations per output row.
// The single wait on an mbarrier (reuse of a partial-sum buffer) is bounded: on time-out a warp raises
// the device status word, stops and lets the others run out as well.
#pragma once

namespace kmll {

constexpr int kSWarps = 16;
constexpr int kSThreads = kSWarps * 32;
constexpr unsigned long long kWaitLimitTicks = 4000000000ull;  // every mbarrier wait gives up after this many cycles (2 to 4 s)


struct StreamParams {
    const float* x;
    int M, K, ldx;
    const uint16_t* norm_w;
    float eps;
    LinearMat mat[3];
    int nmat;
    int unit_start[4];
    int total_units;
    int xs_pitch;   // bytes per staged digit row of the activations
    int ldw, lds;   // bytes per weight row and (W4) scales per weight row: larger than K implies when K is a column slice
    int off_red, off_bars, off_misc, off_ring, off_sring;  // shared-memory offsets in bytes
    uint32_t* partial_tokens;
    float* partial_logits;
    unsigned long long* trace;  // timeline slot of this launch, or null
    // tensor-parallel exchange over peer memory (internal.cuh); indices < 0 = off
    const TpExchange* xc;
    int push_index;    // >= 0: the output vector goes to every rank's inbox instead of mat[0].out
    int gather_index;  // >= 0: x is the rank-ordered sum of the inbox vectors of this exchange
    float* x_out;      // gather: block 0 also writes the summed vector here (the residual stream)
};

__device__ inline uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ inline void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ inline void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ inline unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait; false = timed out (the caller raises the status word and unwinds).  There is no
// blocking hardware barrier anywhere in the kernel, so a time-out in one warp can never leave
// another warp waiting forever.
template <bool BACKOFF = true>
__device__ inline bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();  // (not %globaltimer: reading that register costs a good fraction of a microsecond)
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
            if (BACKOFF) __nanosleep(64);  // leave the issue slots to the warps that share the scheduler
        }
        if ((unsigned long long)(clock64() - t0) > kWaitLimitTicks) return false;
    }
}
// 16-byte asynchronous global->shared copy that bypasses L1 (weights are read once).
__device__ inline void cp_async_stream16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ inline void cp_async_stream16_to(uint32_t smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ inline void cp_async_word_to(uint32_t smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ inline void cp_async_word(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}

constexpr int kSBlock = kSThreads;
// units whose partial sums may be pending at once, and weight tile halves in flight per lane: the batch-1 form
// takes 8 and 8 (128 KB of weights in flight per SM); the batched form (NT = 2, up to 4 rows of x, whose digit rows
// and partial sums need more shared memory) takes 4 and 6
__host__ __device__ constexpr int red_bufs(int nt) { return nt == 1 ? 8 : 4; }
__host__ __device__ constexpr int ring_halves(int nt) { return nt == 1 ? 8 : 6; }

__device__ inline void consumer_bar_sync() { __syncthreads(); }

__device__ inline void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// first MMA of a group: the accumulator input is the zero register, so nothing has to be cleared
__device__ inline void mma_s8_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Stages x (M <= 4 rows of K) into shared memory as four byte rows per batch row: row 4*m + j holds the
// MMA B column j of batch row m (u0, u1, top, ones - see below).
// W4 order inside each 8-column block: even columns first ([0,2,4,6,1,3,5,7]), because the low nibbles
// of a weight word (the even columns) become one MMA operand register and the high nibbles another;
// I8: natural order.
// Returns 2^-sh.  One pass: each thread keeps its (at most kStageBlocks) 8-column blocks of x in
// registers between the block-wide reduction and the conversion.  SINGLE fixes M = 1 at compile time.
//
// Digits: X = round(x * 2^sh) with |X| < 2^22, obtained with ONE fused multiply-add: x * 2^sh + 1.5 * 2^23
// is a float in [2^23, 2^24) whose 23 mantissa bits hold 2^22 + X.  Its bytes are the digits as they lie:
// byte 0 = u0, byte 1 = u1 (unsigned base-256 digits), byte 2 = 64 + (X >> 16) ("top"), so
//   X = u0 + 256 * u1 + 65536 * (top - 64).
// The MMA takes the bytes as UNSIGNED operands; a fourth column of ones yields sum(w) per weight row, which
// removes the offset of the top digit: sum(w * X) = c0 + 256 * c1 + 65536 * (c2 - 64 * c_ones), all integers.
constexpr int kStageBlocks = 6;  // M*K <= 6*8*512 = 24576
constexpr float kDigitMagic = 12582912.0f;  // 1.5 * 2^23
// rows[r] = byte r of (a, b, c, d), r = 0..2
__device__ inline void transpose_bytes3(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&rows)[3]) {
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);
    const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);
    rows[0] = __byte_perm(t0, t1, 0x5410);
    rows[1] = __byte_perm(t0, t1, 0x7632);
    rows[2] = __byte_perm(t2, t3, 0x5410);
}
// Tensor-parallel exchange, consuming side: waits (bounded) until every rank's partial vector of exchange
// `gather_index` has arrived in this rank's inbox, adds the vectors in rank order and leaves the sum as K floats at
// `xf` (block 0 also writes it to x_out).  Kept out of line: single-GPU launches never execute it and the decode
// kernels are sensitive to the size of their instruction stream.
// (scalar arguments only: a reference to the kernel parameters would force them onto the stack)
__device__ __noinline__ void gather_exchange(const TpExchange* xcp, int gather_index, int K, float* x_out, float2* xf) {
    const int tid = threadIdx.x;
    const TpExchange& xc = *xcp;
    const unsigned int epoch = *xc.epoch * (unsigned int)xc.mult + (unsigned int)gather_index + 1u;
    const int tp = xc.tp, npair = K >> 1;  // a 16-byte load = two (value, number) words
    const uint4* gb = reinterpret_cast<const uint4*>(xc.inbox[xc.rank]) + (size_t)(epoch & 1u) * tp * npair;
    const unsigned long long t0 = wait_clock_ticks();
    bool good = true;
#pragma unroll 1
    for (int i0 = tid; i0 < npair; i0 += 4 * kSThreads) {
        float2 sum[4];
#pragma unroll 1
        for (int r = 0; r < tp; ++r) {
            uint4 q[4];
            // poll until all four words of this rank carry the number of this exchange (bounded)
            for (;;) {
                bool all = true;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + u * kSThreads;
                    q[u] = ld_exchange_pair(gb + (size_t)r * npair + (i < npair ? i : i0));
                    all = all && q[u].y == epoch && q[u].w == epoch;
                }
                if (all) break;
                if (wait_clock_ticks() - t0 > kPeerWaitLimitTicks) { good = false; break; }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float2 pv = make_float2(__uint_as_float(q[u].x), __uint_as_float(q[u].z));
                sum[u] = (r == 0) ? pv : make_float2(sum[u].x + pv.x, sum[u].y + pv.y);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * kSThreads;
            if (i < npair) {
                xf[i] = sum[u];
                if (blockIdx.x == 0 && x_out != nullptr) reinterpret_cast<float2*>(x_out)[i] = sum[u];
            }
        }
    }
    if (!good) atomicCAS(&g_device_status, 0, 2);
}

// `after_loads` runs once the loads of x have been issued and before anything waits for them (the caller
// issues the second half of its first weight copies there, so they queue behind x instead of ahead of it).
template <int FMT, bool SINGLE, typename AfterLoads>
__device__ inline float stage_activations(const StreamParams& p, int8_t* xs, float* misc, AfterLoads after_loads) {
    constexpr int NM = SINGLE ? 1 : 4;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int M = SINGLE ? 1 : p.M, K = p.K;
    const int nblk = (M * K) >> 3;  // 8-element blocks; a multiple of 8 (W4: of 16)
    const bool norm = p.norm_w != nullptr;
    float v[kStageBlocks][8];
    uint4 nw[kStageBlocks];  // bf16 RMSNorm weights of the block
    // x comes from p.x, or (tensor-parallel exchange) is the rank-ordered sum of the tp partial vectors in this
    // rank's inbox.  The sum is formed first, as floats in the (not yet used) digit area, and read from there.
    const float* src_base = p.x;
    if (SINGLE && p.gather_index >= 0) {
        gather_exchange(p.xc, p.gather_index, K, p.x_out, reinterpret_cast<float2*>(xs));
        consumer_bar_sync();
        src_base = reinterpret_cast<const float*>(xs);
    }
#pragma unroll
    for (int j = 0; j < kStageBlocks; ++j) {  // every load is issued before anything is consumed
        if (j * kSThreads + warp * 32 < nblk) {  // warp-uniform; lanes past the end re-read block 0 and are masked later
            const int blk = j * kSThreads + tid;
            const int e = (blk < nblk ? blk : 0) << 3;
            const int m = SINGLE ? 0 : e / K;
            const int k = e - m * K;
            const float4* src = reinterpret_cast<const float4*>(src_base + (size_t)m * p.ldx + k);
            const float4 a = src[0], b = src[1];
            if (norm) nw[j] = *reinterpret_cast<const uint4*>(p.norm_w + k);
            v[j][0] = a.x; v[j][1] = a.y; v[j][2] = a.z; v[j][3] = a.w;
            v[j][4] = b.x; v[j][5] = b.y; v[j][6] = b.z; v[j][7] = b.w;
        }
    }
    after_loads();
    float ss[NM], mx[NM];
#pragma unroll
    for (int mm = 0; mm < NM; ++mm) ss[mm] = mx[mm] = 0.0f;
#pragma unroll
    for (int j = 0; j < kStageBlocks; ++j) {
        if (j * kSThreads + warp * 32 < nblk) {  // warp-uniform: blocks that do not exist cost nothing
            const int blk = j * kSThreads + tid;
            const bool active = blk < nblk;
            const int m = SINGLE ? 0 : ((active ? blk : 0) << 3) / K;
            float s_ = 0.0f, m_ = 0.0f;
            if (norm) {
                const uint32_t ww[4] = {nw[j].x, nw[j].y, nw[j].z, nw[j].w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    s_ += v[j][2 * q] * v[j][2 * q] + v[j][2 * q + 1] * v[j][2 * q + 1];
                    m_ = fmaxf(m_, fmaxf(fabsf(v[j][2 * q] * __uint_as_float(ww[q] << 16)),
                                         fabsf(v[j][2 * q + 1] * __uint_as_float(ww[q] & 0xffff0000u))));
                }
            } else {
#pragma unroll
                for (int q = 0; q < 8; ++q) m_ = fmaxf(m_, fabsf(v[j][q]));
            }
            if (!active) s_ = m_ = 0.0f;
#pragma unroll
            for (int mm = 0; mm < NM; ++mm)
                if (SINGLE || m == mm) { ss[mm] += s_; mx[mm] = fmaxf(mx[mm], m_); }
        }
    }
#pragma unroll
    for (int mm = 0; mm < NM; ++mm) {
        ss[mm] = warp_sum(ss[mm]);
        mx[mm] = warp_max(mx[mm]);
    }
    if (lane == 0) {
#pragma unroll
        for (int mm = 0; mm < NM; ++mm) { misc[warp * 8 + mm] = ss[mm]; misc[warp * 8 + 4 + mm] = mx[mm]; }
    }
    consumer_bar_sync();
    // second level: lanes 0..15 fold the 16 warps' sums, lanes 16..31 their maxima (a butterfly over 16 lanes)
    float inv[NM];
    float amax = 0.0f;
    {
        const bool upper = lane >= 16;
        float r[NM];
#pragma unroll
        for (int mm = 0; mm < NM; ++mm) r[mm] = misc[(lane & 15) * 8 + (upper ? 4 : 0) + mm];
#pragma unroll
        for (int off = 1; off < 16; off <<= 1)
#pragma unroll
            for (int mm = 0; mm < NM; ++mm) {
                const float o = __shfl_xor_sync(0xffffffffu, r[mm], off);
                r[mm] = upper ? fmaxf(r[mm], o) : r[mm] + o;
            }
#pragma unroll
        for (int mm = 0; mm < NM; ++mm) {
            const float s_ = __shfl_sync(0xffffffffu, r[mm], 0), m_ = __shfl_sync(0xffffffffu, r[mm], 16);
            inv[mm] = norm ? 1.0f / sqrtf(s_ / (float)K + p.eps) : 1.0f;
            amax = fmaxf(amax, m_ * inv[mm]);
        }
    }
    // power-of-two scale: |x * 2^sh| < 2^22 for every element (the margin covers the few ulps by which the
    // product recomputed below may exceed the maximum found above).  A non-finite maximum gives all-zero digits.
    float xscale = 0.0f, inv_xscale = 1.0f;
    amax *= 1.00001f;
    if (amax > 0.0f && amax < INFINITY) {
        const int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127;  // floor(log2(amax)) (denormals: -127)
        int sh = 21 - e;
        sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
        xscale = __uint_as_float((uint32_t)(sh + 127) << 23);
        inv_xscale = __uint_as_float((uint32_t)(127 - sh) << 23);
    }
    // The conversion is a ROLLED loop: block j is always taken from v[0] and the remaining blocks move down one
    // place, so the conversion sequence exists once in the instruction stream (code that runs once per launch
    // costs instruction fetches, not issue slots).
#pragma unroll 1
    for (int j = 0; j < kStageBlocks; ++j) {
        const int wbase = j * kSThreads + warp * 32;
        if (wbase >= nblk) break;  // warp-uniform
        const int blk = wbase + lane;
        const bool active = blk < nblk;
        const int e = (active ? blk : wbase) << 3;
        const int m = SINGLE ? 0 : e / K;
        const int k = e - m * K;
        float u[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) u[q] = v[0][q];
        const uint32_t ww[4] = {nw[0].x, nw[0].y, nw[0].z, nw[0].w};
#pragma unroll
        for (int jj = 0; jj + 1 < kStageBlocks; ++jj) {
#pragma unroll
            for (int q = 0; q < 8; ++q) v[jj][q] = v[jj + 1][q];
            nw[jj] = nw[jj + 1];
        }
        if (norm) {
            float im = inv[0];
#pragma unroll
            for (int mm = 1; mm < NM; ++mm) im = (m == mm) ? inv[mm] : im;
#pragma unroll
            for (int q = 0; q < 4; ++q) {  // kmll's order: x * inv * w
                u[2 * q] = u[2 * q] * im * __uint_as_float(ww[q] << 16);
                u[2 * q + 1] = u[2 * q + 1] * im * __uint_as_float(ww[q] & 0xffff0000u);
            }
        }
        uint32_t d[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) d[q] = __float_as_uint(fmaf(u[q], xscale, kDigitMagic));
        uint32_t r0[3], r1[3];  // byte j of the block's first / second word of four elements
        if (FMT == FMT_W4) {
            transpose_bytes3(d[0], d[2], d[4], d[6], r0);
            transpose_bytes3(d[1], d[3], d[5], d[7], r1);
        } else {
            transpose_bytes3(d[0], d[1], d[2], d[3], r0);
            transpose_bytes3(d[4], d[5], d[6], d[7], r1);
        }
        if (active) {
#pragma unroll
            for (int r = 0; r < 3; ++r)
                *reinterpret_cast<uint2*>(xs + (size_t)(4 * m + r) * p.xs_pitch + k) = make_uint2(r0[r], r1[r]);
            *reinterpret_cast<uint2*>(xs + (size_t)(4 * m + 3) * p.xs_pitch + k) = make_uint2(0x01010101u, 0x01010101u);
        }
    }
    if (tid < 4) reinterpret_cast<uint32_t*>(xs + (size_t)4 * M * p.xs_pitch)[tid] = 0u;  // what absent MMA columns read
    consumer_bar_sync();
    return inv_xscale;
}


template <int FMT, int MT, int NT, int EPI>
__global__ void __launch_bounds__(kSBlock, 1) linear_stream_kernel(const StreamParams p) {
    constexpr int ROWS = 16 * MT;                       // weight rows per unit tile
    constexpr int RU = (EPI == EPI_SILU) ? 16 : ROWS;   // output rows per unit
    constexpr int kDepth = ring_halves(NT) / MT;  // weight tiles in flight per lane
    constexpr int kRedBufs = red_bufs(NT);
    extern __shared__ __align__(128) unsigned char smem[];

    trace_stamp(p.trace, 0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    constexpr bool kSingle = (NT == 1);  // one batch row, known at compile time (the decode path)
    const int M = kSingle ? 1 : p.M, K = p.K;
    const int rowbytes = (FMT == FMT_W4) ? (K >> 1) : K;
    const int nseg = rowbytes >> 6;  // 64-byte segments per row (W4: quantization groups)
    const int j0 = (warp * nseg) / kSWarps, j1 = ((warp + 1) * nseg) / kSWarps;  // this warp's K slice
    const int spu = j1 - j0;         // tiles per unit for this warp
    const int xs_pitch = p.xs_pitch;
    const int ngr = p.lds;  // W4: binary16 scales per weight row (= groups of the whole row; K may be a column slice)
    const int ldw = p.ldw;  // bytes per weight row

    int8_t* xs = reinterpret_cast<int8_t*>(smem);                       // [4*M][xs_pitch] digit rows
    float* red = reinterpret_cast<float*>(smem + p.off_red);            // [kRedBufs][kSWarps + 2][ROWS][M]
    uint64_t* done = reinterpret_cast<uint64_t*>(smem + p.off_bars);    // [kRedBufs] the finishing warp consumed the partials
    unsigned int* cnt = reinterpret_cast<unsigned int*>(done + kRedBufs);  // [kRedBufs] warps that delivered their partials
    float* misc = reinterpret_cast<float*>(smem + p.off_misc);

    if (tid == 0) {
        for (int b = 0; b < kRedBufs; ++b) { mbar_init(&done[b], 1); cnt[b] = 0u; }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    auto unit_rows = [&](int unit, int& mi, int& row0) {
        mi = 0;
#pragma unroll
        for (int i = 1; i < 3; ++i)
            if (i < p.nmat && unit >= p.unit_start[i]) mi = i;
        row0 = (unit - p.unit_start[mi]) * RU;
    };

    // ---- weight stream: a ring of kDepth tiles per lane, filled with 16-byte asynchronous copies ----
    // A tile is 16*MT rows x 64 bytes; this lane owns 16 bytes of rows g and g+8 of each 16-row block.  The
    // ring lives in shared memory but is PRIVATE to each lane: a lane reads back exactly the bytes its own
    // cp.async wrote (slot plane + tid*16, conflict-free both ways), so cp.async.wait_group is the only
    // synchronisation and no registers are spent on data in flight.
    unsigned char* ring = smem + p.off_ring + (size_t)tid * 16;  // plane stride = kSThreads * 16 bytes
    constexpr int kPlane = kSThreads * 16;
    // W4 group scales ride in a second, tiny ring: per (slot, 16-row block, row half) one 4-byte word per row
    // (the aligned word that contains the binary16 scale).  Lane (g, t) copies the word of row g of block t >> 1,
    // half t & 1: one copy and one pointer per lane and tile.
    unsigned char* sring = smem + p.off_sring + warp * 32 + g * 4;
    constexpr int kSPlane = kSWarps * 32;
    const bool scale_lane = FMT == FMT_W4 && t < 2 * MT;
    const uint32_t ring_dst = smem_u32(ring);
    const uint32_t sring_dst = smem_u32(sring) + (uint32_t)t * kSPlane;  // plane (t >> 1) * 2 + (t & 1) = t
    int l_unit = blockIdx.x, l_seg = j0;  // load cursor
    const unsigned char* lw[MT][2];   // this lane's 16 bytes of the cursor's segment, rows g and g+8
    const unsigned short* ls_mine = nullptr;  // W4: the group scale this lane copies
    auto enter_unit = [&]() {         // row pointers of the cursor's unit (rows past the end re-read the last row)
        if (l_unit >= p.total_units || spu <= 0) return;
        int mi, row0;
        unit_rows(l_unit, mi, row0);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const LinearMat& m = (EPI == EPI_SILU) ? p.mat[mt] : p.mat[mi];
            const int base = (EPI == EPI_SILU) ? row0 : row0 + mt * 16;
            const int r0 = min(base + g, m.rows - 1), r1 = min(base + g + 8, m.rows - 1);
            lw[mt][0] = m.w + (size_t)r0 * ldw + (size_t)j0 * 64 + t * 16;
            lw[mt][1] = m.w + (size_t)r1 * ldw + (size_t)j0 * 64 + t * 16;
            if (FMT == FMT_W4 && (t >> 1) == mt)
                ls_mine = reinterpret_cast<const unsigned short*>(m.scales) + (size_t)((t & 1) ? r1 : r0) * ngr + j0;
        }
    };
    enter_unit();
    auto load_tile = [&](int slot) {
        if (l_unit < p.total_units && spu > 0) {
            const uint32_t dst = ring_dst + (uint32_t)slot * (MT * 2 * kPlane);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                cp_async_stream16_to(dst + (mt * 2) * kPlane, lw[mt][0]);
                cp_async_stream16_to(dst + (mt * 2 + 1) * kPlane, lw[mt][1]);
                lw[mt][0] += 64;
                lw[mt][1] += 64;
            }
            if (scale_lane) {
                cp_async_word_to(sring_dst + (uint32_t)slot * (MT * 2 * kSPlane),
                                 reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(ls_mine) & ~(uintptr_t)3));
                ls_mine += 1;
            }
            if (++l_seg == j1) {
                l_seg = j0;
                l_unit += gridDim.x;
                enter_unit();
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per tile, also when nothing was left to copy
    };
    // weights do not depend on the previous kernel: half of the ring is requested before the dependency wait, the
    // other half right behind the loads of x (so x is not queued behind 128 KB of weights)
    constexpr int kEarly = (kDepth + 1) / 2;
#pragma unroll 1
    for (int d = 0; d < kEarly; ++d) load_tile(d);

    // ---- stage the activations once -----------------------------------------------------------------
    pdl_wait();
    trace_stamp(p.trace, 1);
    const float inv_xscale = stage_activations<FMT, kSingle>(p, xs, misc, [&]() {
#pragma unroll 1
        for (int d = kEarly; d < kDepth; ++d) load_tile(d);
    });
    trace_stamp(p.trace, 2);

    // this lane's B columns: column g of each n-tile; a batch row owns 4 consecutive columns.  A lane whose
    // column does not exist reads the 16 zero bytes behind the digit rows with stride 0 (no select in the loop).
    const int8_t* xcol[NT];
    int bstride[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const bool bvalid = (nt * 8 + g) < 4 * M;
        xcol[nt] = bvalid ? xs + (size_t)(nt * 8 + g) * xs_pitch : xs + (size_t)4 * M * xs_pitch;
        bstride[nt] = bvalid ? 1 : 0;
    }
    // this lane's C columns 2t, 2t+1 of each n-tile: (u0, u1) of a batch row for even t, (top, ones) for odd t.
    // Either pair is combined as c[2t] + pair_mul * c[2t+1] (256 resp. -64) and weighted by 1 resp. 65536.
    const int pair_mul = (t & 1) ? -64 : 256;
    const float w_pair = ((t & 1) ? 65536.0f : 1.0f) * inv_xscale * (FMT == FMT_W4 ? 0.0625f : 1.0f);

    float best_logit = -INFINITY;  // EPI_TOP1 running best (warp 0)
    uint32_t best_token = 0xffffffffu;
    bool ok = true;

    float acc[MT][NT][2];  // W4: group-scaled sums of this lane's digit pair, rows g and g+8
    int c[MT][NT][4];      // exact integer dot products
    auto reset_acc = [&]() {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                acc[mt][nt][0] = acc[mt][nt][1] = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j) c[mt][nt][j] = 0;
            }
    };
    reset_acc();

    int c_par = 0;  // W4: parity of row*ngr for the rows this lane holds in the current unit (bit 2*mt + half)
    // multiply one tile (segment sg of the current unit) from the lane's ring slot
    auto compute_tile = [&](int slot, int sg) {
        uint4 w[MT][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            w[mt][0] = *reinterpret_cast<const uint4*>(ring + (size_t)((slot * MT + mt) * 2) * kPlane);
            w[mt][1] = *reinterpret_cast<const uint4*>(ring + (size_t)((slot * MT + mt) * 2 + 1) * kPlane);
        }
        if (FMT == FMT_W4) {
            uint4 bq[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int8_t* bp = xcol[nt] + (sg * 128 + t * 32) * bstride[nt];
                bq[nt][0] = *reinterpret_cast<const uint4*>(bp);
                bq[nt][1] = *reinterpret_cast<const uint4*>(bp + 16 * bstride[nt]);
            }
            const int spar = (sg & 1) * 2;  // byte offset of this group's binary16 scale inside the copied word
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const uint32_t wlo[4] = {w[mt][0].x, w[mt][0].y, w[mt][0].z, w[mt][0].w};
                const uint32_t whi[4] = {w[mt][1].x, w[mt][1].y, w[mt][1].z, w[mt][1].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    // a stored nibble n = q + 8 moved to the top of a byte and its top bit flipped is the int8
                    // value 16*q: word i gives the even columns (a0/a1) from the low nibbles and the odd columns
                    // (a2/a3) from the high nibbles; the factor 16 leaves with the final scale
                    const uint32_t a0 = ((wlo[i] << 4) & 0xf0f0f0f0u) ^ 0x80808080u, a2 = (wlo[i] & 0xf0f0f0f0u) ^ 0x80808080u;
                    const uint32_t a1 = ((whi[i] << 4) & 0xf0f0f0f0u) ^ 0x80808080u, a3 = (whi[i] & 0xf0f0f0f0u) ^ 0x80808080u;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const uint4 b = bq[nt][i >> 1];
                        if (i == 0) mma_s8_first(c[mt][nt], a0, a1, a2, a3, b.x, b.y);
                        else mma_s8(c[mt][nt], a0, a1, a2, a3, (i & 1) ? b.z : b.x, (i & 1) ? b.w : b.y);
                    }
                }
                // the copied word holds the scales of groups (2i, 2i+1) of the row: pick by the parity of row*ngr + sg
                const int o0 = (ngr & 1) ? ((((c_par >> (mt * 2)) ^ sg) & 1) * 2) : spar;
                const int o1 = (ngr & 1) ? ((((c_par >> (mt * 2 + 1)) ^ sg) & 1) * 2) : spar;
                const float gs0 = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(sring + (size_t)((slot * MT + mt) * 2) * kSPlane + o0)));
                const float gs1 = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(sring + (size_t)((slot * MT + mt) * 2 + 1) * kSPlane + o1)));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    // combined column pair (an integer below 2^30), then the group scale
                    acc[mt][nt][0] = fmaf((float)(c[mt][nt][0] + pair_mul * c[mt][nt][1]), gs0, acc[mt][nt][0]);
                    acc[mt][nt][1] = fmaf((float)(c[mt][nt][2] + pair_mul * c[mt][nt][3]), gs1, acc[mt][nt][1]);
                }
            }
        } else {
            uint4 bq[NT];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                bq[nt] = *reinterpret_cast<const uint4*>(xcol[nt] + (sg * 64 + t * 16) * bstride[nt]);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma_s8(c[mt][nt], w[mt][0].x, w[mt][1].x, w[mt][0].y, w[mt][1].y, bq[nt].x, bq[nt].y);
                    mma_s8(c[mt][nt], w[mt][0].z, w[mt][1].z, w[mt][0].w, w[mt][1].w, bq[nt].z, bq[nt].w);
                }
            }
        }
    };

    // End of a unit: the partial sums of the 16 warps meet in shared memory and ONE warp finishes the
    // rows (sum in fixed warp order, scale, epilogue).  The finishing duty rotates over the warps
    // (unit it -> warp it % 16) and kRedBufs units may be pending, so no warp is a serial bottleneck;
    // the finisher fetches what its epilogue needs from global memory (residual, RS-I8 row scales)
    // when the unit starts, long before it is used.
    float pre_res[(RU + 31) / 32 * 4];  // prefetched residual values of the unit this warp will finish
    float pre_s0[(RU + 31) / 32], pre_s1[(RU + 31) / 32];
    auto prefetch_epilogue = [&](int it, int unit) {
        if ((it % kSWarps) != warp) return;
        int mi, row0;
        unit_rows(unit, mi, row0);
        const LinearMat& om = p.mat[(EPI == EPI_SILU) ? 0 : mi];
#pragma unroll
        for (int q = 0; q < (RU + 31) / 32; ++q) {
            const int r = lane + q * 32;
            const int row = row0 + r;
            const bool okrow = r < RU && row < om.rows;
            if (FMT == FMT_I8) {
                pre_s0[q] = okrow ? reinterpret_cast<const float*>(om.scales)[row] : 0.0f;
                if (EPI == EPI_SILU) pre_s1[q] = okrow ? reinterpret_cast<const float*>(p.mat[1].scales)[row] : 0.0f;
            }
            if (EPI == EPI_RESIDUAL) {
#pragma unroll
                for (int m = 0; m < 4; ++m) pre_res[q * 4 + m] = (okrow && m < M) ? om.residual[(size_t)m * om.ldo + row] : 0.0f;
            }
        }
    };
    auto finish_unit = [&](int it, int unit) {
        const int buf = it % kRedBufs;
        const uint32_t bpar = (uint32_t)(it / kRedBufs) & 1u;
        // this buffer was last used kRedBufs units ago: wait until that unit has been finished
        if (it >= kRedBufs && !mbar_wait(&done[buf], bpar ^ 1u)) { ok = false; return; }
        float* ub = red + (size_t)buf * (kSWarps + 2) * ROWS * M;  // 16 partial blocks, then the epilogue operands
        float* rp = ub + (size_t)warp * ROWS * M;
        float* ex = ub + (size_t)kSWarps * ROWS * M;  // [RU][M] residual, then (RS-I8) [RU] row scales (x2 for gate/up)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float v0, v1;  // rows g and g+8: this lane's digit pair, weighted
                if (FMT == FMT_W4) {
                    v0 = acc[mt][nt][0] * w_pair;
                    v1 = acc[mt][nt][1] * w_pair;
                } else {
                    v0 = ((float)c[mt][nt][0] + (float)pair_mul * (float)c[mt][nt][1]) * w_pair;
                    v1 = ((float)c[mt][nt][2] + (float)pair_mul * (float)c[mt][nt][3]) * w_pair;
                }
                v0 += __shfl_xor_sync(0xffffffffu, v0, 1);  // low pair + top pair
                v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
                const int b = nt * 2 + (t >> 1);  // batch row
                if ((t & 1) == 0 && b < M) {
                    rp[(mt * 16 + g) * M + b] = v0;
                    rp[(mt * 16 + g + 8) * M + b] = v1;
                }
            }
        if ((it % kSWarps) == warp) {  // this warp fetched the epilogue operands when the unit started
#pragma unroll
            for (int q = 0; q < (RU + 31) / 32; ++q) {
                const int r = lane + q * 32;
                if (r < RU) {
                    if (EPI == EPI_RESIDUAL) {
#pragma unroll
                        for (int m = 0; m < 4; ++m)
                            if (m < M) ex[r * M + m] = pre_res[q * 4 + m];
                    }
                    if (FMT == FMT_I8) {
                        ex[ROWS * M + r] = pre_s0[q];
                        if (EPI == EPI_SILU) ex[ROWS * M + RU + r] = pre_s1[q];
                    }
                }
            }
        }
        reset_acc();
        // The warp that delivers LAST finishes the unit: nobody waits (a spinning warp would take issue slots from
        // the three warps that share its scheduler); the sum runs over the warps in index order whoever does it.
        __syncwarp();
        unsigned int prev = 0;
        if (lane == 0) {
            __threadfence_block();
            prev = atomicAdd(&cnt[buf], 1u);
        }
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev != kSWarps - 1) return;
        __threadfence_block();
        if (lane == 0) cnt[buf] = 0u;  // the buffer is handed out again only after `done` below
        int mi, row0;
        unit_rows(unit, mi, row0);
        const LinearMat& om = p.mat[(EPI == EPI_SILU) ? 0 : mi];
        float cand = -INFINITY;
        uint32_t cand_tok = 0xffffffffu;
#pragma unroll
        for (int q = 0; q < (RU + 31) / 32; ++q) {
            const int r = lane + q * 32;
            const int row = row0 + r;
            if (r < RU) {
                for (int m = 0; m < M; ++m) {
                    float v = 0.0f;
#pragma unroll
                    for (int w = 0; w < kSWarps; ++w) v += ub[((size_t)w * ROWS + r) * M + m];
                    if (FMT == FMT_I8) v *= ex[ROWS * M + r];
                    if (EPI == EPI_SILU) {
                        float u = 0.0f;
#pragma unroll
                        for (int w = 0; w < kSWarps; ++w) u += ub[((size_t)w * ROWS + 16 + r) * M + m];
                        if (FMT == FMT_I8) u *= ex[ROWS * M + RU + r];
                        v = (v / (1.0f + expf(-v))) * u;
                    }
                    if (EPI == EPI_TOP1) {
                        if (row < om.rows) { cand = v; cand_tok = (uint32_t)row; }  // M == 1: one row per lane
                    } else if (row < om.rows) {
                        if (EPI == EPI_RESIDUAL) v = ex[r * M + m] + v;
                        if (kSingle && p.push_index >= 0) {
                            // tensor-parallel exchange: (value, exchange number) goes to every rank's inbox in one
                            // 8-byte peer store
                            const TpExchange& xc = *p.xc;
                            const unsigned int epoch = *xc.epoch * (unsigned int)xc.mult + (unsigned int)p.push_index + 1u;
                            const size_t slot = ((size_t)(epoch & 1u) * xc.tp + xc.rank) * xc.dim + row;
                            for (int dst = 0; dst < xc.tp; ++dst) st_exchange_word(xc.inbox[dst] + slot, __float_as_uint(v), epoch);
                        } else {
                            om.out[(size_t)m * om.ldo + row] = v;
                        }
                    }
                }
            }
        }
        if (EPI == EPI_TOP1) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, cand, off);
                const uint32_t ot = __shfl_xor_sync(0xffffffffu, cand_tok, off);
                if (top1_better(ov, ot, cand, cand_tok)) { cand = ov; cand_tok = ot; }
            }
            if (top1_better(cand, cand_tok, best_logit, best_token)) { best_logit = cand; best_token = cand_tok; }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&done[buf]);
    };

    // ---- main loop: consume a tile, refill its register slot with the tile kDepth ahead ------------
    int c_unit = blockIdx.x, c_seg = j0, it = 0;
    auto enter_unit_consumer = [&]() {
        if (c_unit >= p.total_units) return;
        prefetch_epilogue(it, c_unit);
        if (FMT == FMT_W4 && (ngr & 1)) {  // odd group count (e.g. K = 896): the word parity depends on the row
            int mi, row0;
            unit_rows(c_unit, mi, row0);
            c_par = 0;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const LinearMat& m = (EPI == EPI_SILU) ? p.mat[mt] : p.mat[mi];
                const int base = (EPI == EPI_SILU) ? row0 : row0 + mt * 16;
                const int r0 = min(base + g, m.rows - 1), r1 = min(base + g + 8, m.rows - 1);
                c_par |= ((r0 & 1) << (mt * 2)) | ((r1 & 1) << (mt * 2 + 1));
            }
        }
    };
    enter_unit_consumer();
    // one loop for both kinds of warp: a warp with no columns (fewer segments than warps) still takes part in
    // the unit hand-shake
    int slot = 0;
    while (c_unit < p.total_units && ok) {
        if (spu > 0) {
            asm volatile("cp.async.wait_group %0;" ::"n"(kDepth - 1) : "memory");  // this lane's oldest tile has landed
            if (FMT == FMT_W4) __syncwarp();  // scale words were copied by the t == 0 lanes
            compute_tile(slot, c_seg);
            if (FMT == FMT_W4) __syncwarp();  // every lane has read the slot's scale words before they are replaced
            load_tile(slot);
            if (++slot == kDepth) slot = 0;
            if (++c_seg != j1) continue;
            c_seg = j0;
        }
        finish_unit(it, c_unit);
        ++it;
        c_unit += gridDim.x;
        enter_unit_consumer();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    trace_stamp(p.trace, 3);
    if (EPI == EPI_TOP1) {
        // every warp finished some units: merge the 16 running bests (fixed order) into one partial per block
        __syncthreads();
        if (lane == 0) { misc[warp * 2] = best_logit; misc[warp * 2 + 1] = __uint_as_float(best_token); }
        __syncthreads();
        if (tid == 0) {
            float bl = -INFINITY;
            uint32_t bt = 0xffffffffu;
            for (int w = 0; w < kSWarps; ++w) {
                const float l = misc[w * 2];
                const uint32_t tk = __float_as_uint(misc[w * 2 + 1]);
                if (top1_better(l, tk, bl, bt)) { bl = l; bt = tk; }
            }
            p.partial_tokens[blockIdx.x] = bt;
            p.partial_logits[blockIdx.x] = bl;
        }
    }
    if (lane == 0) trace_stamp_latest(p.trace, 4);
    if (!ok) atomicCAS(&g_device_status, 0, 1);
}

}  // namespace kmll
