// W4-G128 linear for small batches (5 to 32 rows of activations: batches of sequences decoding in lockstep), included
// by linear.cu after linear_gemm.cuh.  Serves the same kmll operator as linear_gemm.cuh (linear_batched_i8_scaled,
// crates/inference/src/ops/matmul.rs:423-463, over W4-G128 weights) where the work is a stream of weights, not a
// contraction: the point is to keep every multiprocessor's share of the HBM stream in flight.
//
// Arithmetic.  Each row of x becomes a 30-bit fixed-point integer X = rint(x 2^sh) (2^sh puts the row maximum in
// [2^28, 2^29)), written as four balanced base-256 digits d0..d3 in [-128, 127] (digit_rows_kernel).  The 4-bit weights
// are used as the signed bytes q = nibble - 8.  For one group of 128 columns
//   D_i[r, m] = sum_k q[r, k] d_i[m, k]          tcgen05.mma.kind::i8, s8 x s8 -> s32, exact
//   y[m, r]  += scale[r, group] * sum_i 256^i D_i[r, m]
// so the group scale is applied to an exact integer dot product after the MMA, in f32, as kmll's own kernel applies it
// per group.  No second weight plane and no cross terms are needed.
//
// Pipeline.  One persistent block per multiprocessor walks its (row tile, k-split) units group by group; up to three
// matrices that share x (q / k / v, gate / up) are one launch, their row tiles numbered through.  Measured on B200: every
// mbarrier, TMA or tcgen05 instruction costs the thread that issues it 100 to 250 cycles, so ONE pass of any role over a
// group takes 1100 to 1300 cycles however little it computes - several times the HBM share of a group (8 KB at 44 GB/s
// per multiprocessor = 360 cycles).  Two things follow.  Each buffer has a ring of its own, sized by how long its contents
// live; and the roles that do work per group exist twice and take the groups alternately:
//   * raw weight tiles (128 rows x 64 bytes of nibbles, TMA by warp 8): 12 slots (7 with 32 rows of x) - they wait out the HBM latency;
//   * digit planes of the same 128 columns (one 3-D TMA box, 128-byte swizzle, warp 4): 5 or 6 slots - L2 latency;
//   * signed-byte weight tiles in the swizzled K-major layout the MMA reads: 4 slots, written by two sets of four
//     expanding warps (seven integer instructions per word; the even and odd columns of a word come out as two runs, the
//     digit planes are stored in that column order);
//   * accumulators in tensor memory: 8 (16 rows of x) or 4 (32 rows) buffers of 4 n_block columns.
//   One thread of each of warps 0 and 11 waits for a group's `a_ready` barrier, its digit planes and its accumulator
//   buffer, issues the four MMAs (M = 128 weight rows, N = 4 n_block digit columns, K = 32 bytes each) and one commit on a
//   ring of 16 `done` barriers; the producers, the expanding warps and the draining warps all derive what they wait for
//   from that ring (the slot they want to refill was last used by the group `ring size` back).  Two sets of four warps
//   drain: tcgen05.ld of the buffer, release it, integer -> f32 without conversion instructions (the sums are below 2^22:
//   add them to the bits of 1.5 * 2^23 and subtract that constant), combine the digits, one FMA with the group scale into
//   f32 accumulators in registers.  After the last group of a unit the second set hands its sums to the first through
//   shared memory, and the first stores the rows (or the split-K partial; the unit that arrives last adds the partials in
//   split order, so results are bit-identical from call to call).
// Because an accumulator lives for one group only, the pipeline runs on across unit boundaries without draining.
// Tensor maps cover this GPU's memory only; no multicast.  Every wait is bounded (mbar_wait); a time-out raises the device
// status word, and the block frees its tensor memory and returns.  There is no blocking hardware barrier inside the loops.
// Compiled with -DKMLL_ROLE_PROFILE, block 0 records per role the cycles spent waiting and in all (the figures above).
#pragma once

namespace kmll {

constexpr int kBtSetWarps = 4;     // warps per expanding set and per draining set; two sets of each take the groups alternately
constexpr int kBtThreads = 20 * 32;  // roles by warp: see linear_gemm_small_kernel
constexpr int kBtABytes = 128 * 128;  // expanded weight tile: 128 rows x 128 signed bytes
constexpr int kBtRawBytes = 128 * 64;
constexpr int kBtASlots = 4;   // expanded-tile slots with one group per item
constexpr int kBtDoneRing = 16;    // `done` barriers; a power of two above every ring size
constexpr int kBtMaxUnits = 592;   // split-K partial tiles the workspace holds (four per multiprocessor)
constexpr int kBtMaxMats = 3;

struct SmallMat {
    const uint16_t* scales;    // W4-G128: binary16 [rows, K / 128]
    const float* row_scales;   // RS-I8: float [rows]
    float* out;                // [M, ldo]
    const float* residual;     // [M, ldo] or null
    int rows, ldo;
    int tile_start;            // first row tile of this matrix in the launch's numbering
};

struct SmallParams {
    int K, M;
    int nmat, tiles, ksplit, units;  // tiles = row tiles of all matrices; units = tiles * ksplit
    SmallMat mat[kBtMaxMats];
    const float* inv_xscale;   // [M] 2^-sh per row of x
    float* partial;            // split-K: [tile][split][n_block][128]
    unsigned int* counters;    // split-K: [tiles] arrivals, zero between launches
#ifdef KMLL_ROLE_PROFILE
    unsigned long long* prof;  // per role of block 0: cycles spent waiting, cycles in all
#endif
};

// One block per row of x: optional RMSNorm (kmll's order x * inv * w), power-of-two scale, four balanced byte digits.
// digits = [4][M][K] signed bytes; with `permute` (W4-G128) position p of every run of eight columns holds column
// {0,2,4,6,1,3,5,7}[p], the order in which the weight expansion lays out the nibbles of a 32-bit word; RS-I8 weights are
// used as they lie, so their digits keep the natural order.  Block 0 also clears the split-K counters.
// RESIDENT (K <= 16384): the row is read once and stays in registers between the statistics and the digits.
__device__ inline void digits_of_eight(const float (&v)[8], float xscale, int permute, uint32_t (&d)[4][2]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i][0] = d[i][1] = 0u;
#pragma unroll
    for (int pos = 0; pos < 8; ++pos) {
        const int col = !permute ? pos : pos < 4 ? 2 * pos : 2 * (pos - 4) + 1;
        int X = __float2int_rn(v[col] * xscale);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int di = i < 3 ? ((X + 128) & 255) - 128 : X;  // balanced digit; the top one is what is left (|.| <= 33)
            X = (X - di) >> 8;
            d[i][pos >> 2] |= (uint32_t)(di & 255) << (8 * (pos & 3));
        }
    }
}
template <bool RESIDENT>
__global__ void __launch_bounds__(512) digit_rows_kernel(const float* __restrict__ x, int ldx, int K, int M, const uint16_t* __restrict__ norm_w,
                                                         float eps, int8_t* __restrict__ digits, float* __restrict__ inv_xscale,
                                                         unsigned int* counters, int n_counters, int permute) {
    __shared__ float scratch[40];
    pdl_wait();
    pdl_launch_dependents();  // the kernel that follows starts bringing in its weights; it waits for this grid before it reads the digits
    const int m = blockIdx.x;
    if (m == 0)
        for (int i = threadIdx.x; i < n_counters; i += blockDim.x) counters[i] = 0u;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)m * ldx);
    const uint4* nw8 = reinterpret_cast<const uint4*>(norm_w);
    constexpr int kPer = 4;  // runs of eight columns per thread when the row is resident: 512 * 4 * 8 = 16384 columns
    float v[RESIDENT ? kPer : 1][8];
    float ss = 0.0f, mx = 0.0f;
    auto load8 = [&](int k8, float (&o)[8], float& ss_, float& mx_) {
        const float4 a = xr[2 * k8], b = xr[2 * k8 + 1];
        o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
#pragma unroll
        for (int q = 0; q < 8; ++q) ss_ = fmaf(o[q], o[q], ss_);
        if (norm_w) {  // largest |x w|; the factor 1 / rms follows once it is known (the margin below covers the rounding)
            const uint4 w = nw8[k8];
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int q = 0; q < 4; ++q)
                mx_ = fmaxf(mx_, fmaxf(fabsf(o[2 * q] * __uint_as_float(ww[q] << 16)), fabsf(o[2 * q + 1] * __uint_as_float(ww[q] & 0xffff0000u))));
        } else {
#pragma unroll
            for (int q = 0; q < 8; ++q) mx_ = fmaxf(mx_, fabsf(o[q]));
        }
    };
    if (RESIDENT) {
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int k8 = threadIdx.x + i * 512;
            if (k8 < K / 8) load8(k8, v[RESIDENT ? i : 0], ss, mx);
        }
    } else {
        for (int k8 = threadIdx.x; k8 < K / 8; k8 += 512) {
            float t[8];
            load8(k8, t, ss, mx);
        }
    }
    ss = block_sum(ss, scratch);
    mx = block_max(mx, scratch);
    const float inv = norm_w ? 1.0f / sqrtf(ss / (float)K + eps) : 1.0f;
    const float amax = mx * inv * 1.00001f;
    float xscale = 0.0f, inv_scale = 1.0f;
    if (amax > 0.0f && amax < INFINITY) {
        const int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127;
        int sh = 28 - e;  // the row maximum lands in [2^28, 2^29)
        sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
        xscale = __uint_as_float((uint32_t)(sh + 127) << 23);
        inv_scale = __uint_as_float((uint32_t)(127 - sh) << 23);
    }
    const size_t plane = (size_t)M * K;
    int8_t* drow = digits + (size_t)m * K;
    auto store8 = [&](int k8, const float (&o)[8]) {
        float t[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) t[q] = o[q];
        if (norm_w) {  // kmll's order: x * inv * w
            const uint4 w = nw8[k8];
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                t[2 * q] = t[2 * q] * inv * __uint_as_float(ww[q] << 16);
                t[2 * q + 1] = t[2 * q + 1] * inv * __uint_as_float(ww[q] & 0xffff0000u);
            }
        }
        uint32_t d[4][2];
        digits_of_eight(t, xscale, permute, d);
#pragma unroll
        for (int i = 0; i < 4; ++i) reinterpret_cast<uint2*>(drow + (size_t)i * plane)[k8] = make_uint2(d[i][0], d[i][1]);
    };
    if (RESIDENT) {
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int k8 = threadIdx.x + i * 512;
            if (k8 < K / 8) store8(k8, v[RESIDENT ? i : 0]);
        }
    } else {
        for (int k8 = threadIdx.x; k8 < K / 8; k8 += 512) {
            float t[8], s2 = 0.0f, m2 = 0.0f;
            load8(k8, t, s2, m2);
            store8(k8, t);
        }
    }
    if (threadIdx.x == 0) inv_xscale[m] = inv_scale;
}

// instruction descriptor of kind::i8: D = s32, A and B signed bytes, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
__host__ __device__ constexpr uint32_t gemm_idesc_s8s8(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ inline void gemm_mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// four unsigned nibble bytes (0..15 each) -> four signed bytes nibble - 8, without a carry between the bytes
__device__ inline uint32_t nibble_bytes_to_s8(uint32_t w, uint32_t shift) {
    const uint32_t t = lop3_and_or(w >> shift, 0x0f0f0f0fu, 0x80808080u);
    return (t - 0x08080808u) ^ 0x80808080u;
}
__device__ inline void tmem_ld8(uint32_t taddr, uint32_t (&d)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7])
                 : "r"(taddr)
                 : "memory");
}

// Ring position with its phase bit, advanced without divisions.
template <int N>
struct RingPos {
    int idx = 0;
    uint32_t phase = 0;
    bool wrapped = false;  // the ring has been used once: there is an earlier use to wait for
    __device__ inline void next() {
        if (++idx == N) { idx = 0; phase ^= 1u; wrapped = true; }
    }
};

// Ring sizes and the shared-memory plan: [raw slots | digit slots | expanded slots | hand-over | barriers].  An *item* - what
// moves through the rings and what every role handles per pass - is GP consecutive 128-column groups: 2 with 16 rows of x
// (every role's pass costs about the same however much it carries, so two groups per pass halve the cost per byte), 1 with
// 32 rows (tensor memory holds 512 columns: four buffers of 4 x 32).
template <int NB, int GP>
struct SmallShape {
    static constexpr int kBBytes = GP * 4 * NB * 128;      // the four digit planes of the item's groups
    static constexpr int kABytes = GP * kBtABytes;         // expanded tiles of the item
    static constexpr int kRawBytes = GP * kBtRawBytes;     // 128 rows x 64 GP bytes of nibbles
    static constexpr int kASlots = GP == 2 ? 3 : kBtASlots;
    static constexpr int kXSlots = GP == 2 ? 3 : (NB == 16 ? 6 : 5);
    static constexpr int kBufs = 512 / (GP * 4 * NB);      // accumulator buffers of GP x 4 NB columns
    static constexpr int kXchgBytes = NB * 128 * 4;        // partial rows handed from the second drain set to the first
    static constexpr int kRawSlots = (224 * 1024 - 2048 - kASlots * kABytes - kXSlots * kBBytes - kXchgBytes) / kRawBytes;
    static constexpr int kOffX = kRawSlots * kRawBytes;
    static constexpr int kOffA = kOffX + kXSlots * kBBytes;
    static constexpr int kOffXchg = kOffA + kASlots * kABytes;
    static constexpr int kOffBars = kOffXchg + kXchgBytes;
    static constexpr int kNumBars = 2 * kRawSlots + kXSlots + kASlots + kBtDoneRing + kBufs + 3;
    static constexpr int kSmemBytes = kOffBars + kNumBars * 8 + 16 + 1024;  // + slack for the 1024-byte alignment
    static_assert(kRawSlots >= 4 && kRawSlots < kBtDoneRing && kXSlots < kBtDoneRing && kBufs < kBtDoneRing && kBufs >= 2, "ring sizes");
    static_assert(kOffX % 1024 == 0 && kOffA % 1024 == 0 && kSmemBytes <= 227 * 1024, "swizzled tiles start on 1024-byte boundaries");
};

// The unit sequence of one block: units u = blockIdx.x, + gridDim.x, ...; unit = (row tile over all matrices, split);
// every role walks it with its own copy of this cursor.
struct UnitCursor {
    int u, tile, z, g, g1;
    __device__ inline bool start(const SmallParams& p, int first, int G) {
        u = first;
        return load(p, G);
    }
    __device__ inline bool load(const SmallParams& p, int G) {
        if (u >= p.units) return false;
        tile = u / p.ksplit;
        z = u - tile * p.ksplit;
        g = (int)(((long long)z * G) / p.ksplit);
        g1 = (int)(((long long)(z + 1) * G) / p.ksplit);
        return true;
    }
    // next item (`step` groups on); false when the block's work is over
    __device__ inline bool advance(const SmallParams& p, int G, int step = 1) {
        g += step;
        if (g < g1) return true;
        u += gridDim.x;
        return load(p, G);
    }
};

#ifdef KMLL_ROLE_PROFILE
#define PROF_DECL long long prof_wait = 0, prof_t0 = clock64(), prof_w0 = 0
#define PROF_W0 prof_w0 = clock64()
#define PROF_W1 prof_wait += clock64() - prof_w0
#define PROF_END(role) do { if (p.prof && blockIdx.x == 0) { p.prof[2 * (role)] = (unsigned long long)prof_wait; p.prof[2 * (role) + 1] = (unsigned long long)(clock64() - prof_t0); } } while (0)
#else
#define PROF_DECL
#define PROF_W0
#define PROF_W1
#define PROF_END(role)
#endif
// NB = rows of x per block (16 or 32): N = 4 NB digit columns per MMA; GP = groups per item (SmallShape).
// Warp roles are placed by scheduler (warp % 4): an MMA warp shares its scheduler with the two TMA warps, which sleep on
// barriers most of the time, and drain warps; the expanding warps, which spin and compute, sit on the other three.
//   warps 0, 11: MMA     warp 4: TMA digits     warp 8: TMA weights     warps 1 2 3 5 | 6 7 9 10: the two expanding sets
//   warps 12..15 | 16..19: the two draining sets (tensor-memory lanes 32 (w % 4) ..)
template <int NB, int GP>
__global__ void __launch_bounds__(kBtThreads, 1) linear_gemm_small_kernel(const SmallParams p, const __grid_constant__ CUtensorMap map_w0,
                                                                        const __grid_constant__ CUtensorMap map_w1,
                                                                        const __grid_constant__ CUtensorMap map_w2,
                                                                        const __grid_constant__ CUtensorMap map_x) {
    using S = SmallShape<NB, GP>;
    constexpr int kGroupB = 4 * NB * 128;  // digit planes of one group
    constexpr int kN = 4 * NB;
    constexpr uint32_t kTmemCols = 512;
    extern __shared__ unsigned char ssmem_raw[];
    unsigned char* ssmem = ssmem_raw + ((1024u - (smem_u32(ssmem_raw) & 1023u)) & 1023u);
    uint64_t* raw_full = reinterpret_cast<uint64_t*>(ssmem + S::kOffBars);  // [kRawSlots] the raw weight tile has landed
    uint64_t* raw_free = raw_full + S::kRawSlots;   // [kRawSlots] the expanding warps have read it
    uint64_t* x_full = raw_free + S::kRawSlots;     // [kXSlots] the digit planes have landed
    uint64_t* a_ready = x_full + S::kXSlots;        // [kASlots] the signed-byte tiles of an item are written
    uint64_t* done = a_ready + S::kASlots;          // [kBtDoneRing] the MMAs of item number n (n % 16 here) have completed
    uint64_t* tmem_free = done + kBtDoneRing;       // [kBufs] the drain warps have read the buffer
    uint64_t* drain_bar = tmem_free + S::kBufs;     // meeting point of the first drain set (split-K hand-off)
    uint64_t* xchg_full = drain_bar + 1;            // the second drain set has written its partial rows of a unit
    uint64_t* xchg_free = xchg_full + 1;            // the first set has taken them
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xchg_free + 1);
    uint32_t* last_flag = tmem_slot + 1;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = p.K >> 7;  // 128-column groups

    if (tid == 0) {
        for (int s = 0; s < S::kRawSlots; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_free[s], kBtSetWarps); }
        for (int s = 0; s < S::kXSlots; ++s) mbar_init(&x_full[s], 1);
        for (int s = 0; s < S::kASlots; ++s) mbar_init(&a_ready[s], kBtSetWarps);
        for (int s = 0; s < kBtDoneRing; ++s) mbar_init(&done[s], 1);
        for (int b = 0; b < S::kBufs; ++b) mbar_init(&tmem_free[b], kBtSetWarps);
        mbar_init(drain_bar, kBtSetWarps);
        mbar_init(xchg_full, kBtSetWarps);
        mbar_init(xchg_free, kBtSetWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t smem_base = smem_u32(ssmem);
    bool ok = true;
    // the `done` barrier and parity that report the completion of item number n of this block
    auto done_wait = [&](int n) { return mbar_wait<false>(&done[n & (kBtDoneRing - 1)], (uint32_t)(n >> 4) & 1u); };
    static_assert(kBtDoneRing == 16, "done_wait shifts by 4");
    const bool expander = warp < 11 && (warp & 3) != 0;  // warps 1 2 3 5 6 7 9 10
    UnitCursor cur;

    if (warp == 8) {
        // ---- TMA of the raw weight tiles.  The weights never change, so these copies start at once, whatever the previous
        // kernel is still doing.  With two groups per item the box is 128 bytes wide (128-byte swizzle, which the expanding
        // warps undo when they read); a box that reaches past the unit or past K brings bytes nobody uses, or zeros.
        if (lane == 0 && cur.start(p, blockIdx.x, G)) {
            RingPos<S::kRawSlots> rp;
            PROF_DECL;
            do {
                PROF_W0;
                if (rp.wrapped && !mbar_wait<false>(&raw_free[rp.idx], rp.phase ^ 1u)) { ok = false; break; }
                PROF_W1;
                const int mi = (p.nmat > 2 && cur.tile >= p.mat[2].tile_start) ? 2 : (p.nmat > 1 && cur.tile >= p.mat[1].tile_start) ? 1 : 0;
                const CUtensorMap* map = mi == 0 ? &map_w0 : mi == 1 ? &map_w1 : &map_w2;
                mbar_arrive_expect_tx(&raw_full[rp.idx], (uint32_t)S::kRawBytes);
                tma_load_2d(smem_base + (uint32_t)rp.idx * S::kRawBytes, map, cur.g * 64, (cur.tile - p.mat[mi].tile_start) * 128, &raw_full[rp.idx]);
                rp.next();
            } while (cur.advance(p, G, GP));
            PROF_END(0);
        }
    } else if (warp == 4) {
        // ---- TMA of the digit planes: they come from the previous kernel; a slot is free when the item that used it
        // last (kXSlots back) has been multiplied
        pdl_wait();
        if (lane == 0 && cur.start(p, blockIdx.x, G)) {
            RingPos<S::kXSlots> xp;
            int it = 0;
            PROF_DECL;
            do {
                PROF_W0;
                if (it >= S::kXSlots && !done_wait(it - S::kXSlots)) { ok = false; break; }
                PROF_W1;
                mbar_arrive_expect_tx(&x_full[xp.idx], (uint32_t)S::kBBytes);
#pragma unroll
                for (int j = 0; j < GP; ++j)
                    tma_load_3d(smem_base + S::kOffX + (uint32_t)xp.idx * S::kBBytes + j * kGroupB, &map_x, (cur.g + j) * 128, 0, 0, &x_full[xp.idx]);
                xp.next();
                ++it;
            } while (cur.advance(p, G, GP));
            PROF_END(1);
        }
    } else if (warp == 0 || warp == 11) {
        // ---- MMA issuers: one thread of each of two warps, alternate items (their accumulators are different buffers, so
        // no order is needed between them).  Per item: the tiles are expanded, the digit planes have landed, the accumulator
        // buffer has been read out; four MMAs per group; one commit.
        const int set = warp == 0 ? 0 : 1;
        if (lane == 0 && cur.start(p, blockIdx.x, G)) {
            constexpr uint32_t idesc = gemm_idesc_s8s8(128, kN);
            const uint64_t desc_a0 = gemm_smem_desc(smem_base + S::kOffA), desc_b0 = gemm_smem_desc(smem_base + S::kOffX);
            RingPos<S::kASlots> ap;
            RingPos<S::kXSlots> xp;
            RingPos<S::kBufs> bp;
            int it = 0;
            PROF_DECL;
            do {
                if ((it & 1) == set) {
                    PROF_W0;
                    if (!mbar_wait<false>(&a_ready[ap.idx], ap.phase) || !mbar_wait<false>(&x_full[xp.idx], xp.phase) ||
                        (bp.wrapped && !mbar_wait<false>(&tmem_free[bp.idx], bp.phase ^ 1u))) {
                        ok = false;
                        break;
                    }
                    PROF_W1;
                    tcgen05_fence_after();
                    const int ng = min(GP, cur.g1 - cur.g);
#pragma unroll
                    for (int j = 0; j < GP; ++j) {
                        if (j < ng) {
                            const uint64_t da = desc_a0 + (uint64_t)((uint32_t)ap.idx * (S::kABytes >> 4) + j * (kBtABytes >> 4));
                            const uint64_t db = desc_b0 + (uint64_t)((uint32_t)xp.idx * (S::kBBytes >> 4) + j * (kGroupB >> 4));
                            const uint32_t d = tmem_base + (uint32_t)(bp.idx * GP * kN + j * kN);
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) gemm_mma_i8(d, da + 2 * ks, db + 2 * ks, idesc, ks > 0 ? 1u : 0u);
                        }
                    }
                    umma_commit(&done[it & (kBtDoneRing - 1)]);
                }
                ap.next(); xp.next(); bp.next();
                ++it;
            } while (cur.advance(p, G, GP));
            PROF_END(2 + set);
        }
    } else if (expander) {
        // ---- weight expansion, two sets of four warps that take the items alternately.  A thread turns four 16-byte pieces
        // of raw nibbles per group (32 columns each) into signed bytes.  One group per item: piece id = 128 i + (thread of
        // the set) is (row id / 4, quarter id % 4) of the 64-byte rows - a warp reads 512 contiguous bytes.  Two groups per
        // item: the raw rows are 128 bytes in the 128-byte swizzle, and the eight lanes of a quarter warp take eight
        // consecutive rows at the same quarter, so that their reads and their writes fall on distinct banks.
        const int e = warp - 1 - (warp > 4 ? 1 : 0) - (warp > 8 ? 1 : 0);  // 0..7
        const int set = e >> 2;
        const int wv = e & 3;
        const int dt = wv * 32 + lane;  // thread of the set, 0..127
        if (cur.start(p, blockIdx.x, G)) {
            RingPos<S::kRawSlots> rp;
            RingPos<S::kASlots> ap;
            int it = 0;
            PROF_DECL;
            do {
                if ((it & 1) == set) {
                    // the raw tile has landed; the expanded slot is free (its last user, kASlots items back, has been multiplied)
                    PROF_W0;
                    if (!mbar_wait<false>(&raw_full[rp.idx], rp.phase) || (it >= S::kASlots && !done_wait(it - S::kASlots))) { ok = false; break; }
                    PROF_W1;
                    const unsigned char* raw = ssmem + (size_t)rp.idx * S::kRawBytes;
                    const int ng = min(GP, cur.g1 - cur.g);
#pragma unroll
                    for (int j = 0; j < GP; ++j) {
                        if (j < ng) {
                            unsigned char* a = ssmem + S::kOffA + (size_t)ap.idx * S::kABytes + (size_t)j * kBtABytes;
                            uint4 w[4];
                            int row[4], qt[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                if (GP == 1) {
                                    const int id = i * 128 + dt;
                                    row[i] = id >> 2;
                                    qt[i] = id & 3;
                                    w[i] = *reinterpret_cast<const uint4*>(raw + (size_t)id * 16);
                                } else {
                                    row[i] = i * 32 + wv * 8 + (lane & 7);
                                    qt[i] = lane >> 3;
                                    w[i] = *reinterpret_cast<const uint4*>(raw + row[i] * 128 + (((4 * j + qt[i]) ^ (row[i] & 7)) << 4));
                                }
                            }
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int r = row[i];
                                const uint4 lo = make_uint4(nibble_bytes_to_s8(w[i].x, 0), nibble_bytes_to_s8(w[i].x, 4), nibble_bytes_to_s8(w[i].y, 0),
                                                            nibble_bytes_to_s8(w[i].y, 4));
                                const uint4 hi = make_uint4(nibble_bytes_to_s8(w[i].z, 0), nibble_bytes_to_s8(w[i].z, 4), nibble_bytes_to_s8(w[i].w, 0),
                                                            nibble_bytes_to_s8(w[i].w, 4));
                                *reinterpret_cast<uint4*>(a + r * 128 + (((2 * qt[i]) ^ (r & 7)) << 4)) = lo;
                                *reinterpret_cast<uint4*>(a + r * 128 + (((2 * qt[i] + 1) ^ (r & 7)) << 4)) = hi;
                            }
                        }
                    }
                    fence_proxy_async_smem();  // the tensor core reads the tiles through the async proxy
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&raw_free[rp.idx]);
                        mbar_arrive(&a_ready[ap.idx]);
                    }
                }
                rp.next(); ap.next();
                ++it;
            } while (cur.advance(p, G, GP));
            if (dt == 0) PROF_END(4 + set);
        }
    } else if (warp >= 12) {
        // ---- drain, two sets of four warps that take the items alternately: warp w may read tensor-memory lanes
        // 32 (w % 4) ..; lane = weight row inside the tile; each thread accumulates its row for all rows of x.  At the end of
        // a unit the second set hands its sums to the first through shared memory; the first set finishes the rows.
        const int q = warp & 3;
        const int rl = q * 32 + lane;
        const int set = warp >= 16 ? 1 : 0;
        float* xchg = reinterpret_cast<float*>(ssmem + S::kOffXchg);  // [NB][128]
        uint32_t drain_phase = 0, xchg_phase = 0;
        pdl_wait();  // inv_xscale, the residual and the cleared counters come from earlier kernels
        if (cur.start(p, blockIdx.x, G)) {
            RingPos<S::kBufs> bp;
            int it = 0;
            bool more = true;
            PROF_DECL;
            while (more && ok) {
                const int tile = cur.tile, z = cur.z;
                const int mi = (p.nmat > 2 && tile >= p.mat[2].tile_start) ? 2 : (p.nmat > 1 && tile >= p.mat[1].tile_start) ? 1 : 0;
                const SmallMat& mt = p.mat[mi];
                const int row = (tile - mt.tile_start) * 128 + rl;
                const uint16_t* srow = mt.scales + (size_t)min(row, mt.rows - 1) * G;
                float acc[NB];
#pragma unroll
                for (int m = 0; m < NB; ++m) acc[m] = 0.0f;
                // group scales of this row for this set's next item, requested one of its items ahead
                uint32_t s_next[GP];
                {
                    const int g_mine = cur.g + (((it & 1) == set) ? 0 : GP);
#pragma unroll
                    for (int j = 0; j < GP; ++j) s_next[j] = g_mine + j < cur.g1 ? __ldg(srow + g_mine + j) : 0u;
                }
                bool same_unit = true;
                while (same_unit) {
                    if ((it & 1) == set) {
                        float sc[GP];
#pragma unroll
                        for (int j = 0; j < GP; ++j) {
                            sc[j] = __half2float(__ushort_as_half((unsigned short)s_next[j]));
                            s_next[j] = cur.g + 2 * GP + j < cur.g1 ? __ldg(srow + cur.g + 2 * GP + j) : 0u;
                        }
                        PROF_W0;
                        if (!done_wait(it)) { ok = false; break; }
                        PROF_W1;
                        tcgen05_fence_after();
                        const int ng = min(GP, cur.g1 - cur.g);
                        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(bp.idx * GP * kN);
#pragma unroll
                        for (int j = 0; j < GP; ++j) {
#pragma unroll
                            for (int m0 = 0; m0 < NB; m0 += 8) {
                                uint32_t d0[8], d1[8], d2[8], d3[8];
                                if (j < ng) {
                                    tmem_ld8(taddr + j * kN + m0, d0);
                                    tmem_ld8(taddr + j * kN + NB + m0, d1);
                                    tmem_ld8(taddr + j * kN + 2 * NB + m0, d2);
                                    tmem_ld8(taddr + j * kN + 3 * NB + m0, d3);
                                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                                }
                                if (j == GP - 1 && m0 + 8 >= NB) {  // everything of this buffer is in registers: hand it back
                                    tcgen05_fence_before();
                                    __syncwarp();
                                    if (lane == 0) mbar_arrive(&tmem_free[bp.idx]);
                                }
                                if (j < ng) {
                                    // |D_i| <= 128 * 8 * 128 = 2^17: the integer added to the bits of 1.5 * 2^23 is that float plus the integer
                                    const float kMagic = 12582912.0f;
#pragma unroll
                                    for (int t8 = 0; t8 < 8; ++t8) {
                                        const float f0 = __uint_as_float(0x4b400000u + d0[t8]) - kMagic, f1 = __uint_as_float(0x4b400000u + d1[t8]) - kMagic;
                                        const float f2 = __uint_as_float(0x4b400000u + d2[t8]) - kMagic, f3 = __uint_as_float(0x4b400000u + d3[t8]) - kMagic;
                                        const float t = fmaf(fmaf(fmaf(f3, 256.0f, f2), 256.0f, f1), 256.0f, f0);
                                        acc[m0 + t8] = fmaf(t, sc[j], acc[m0 + t8]);
                                    }
                                }
                            }
                        }
                    }
                    bp.next();
                    ++it;
                    const int u_before = cur.u;
                    more = cur.advance(p, G, GP);
                    same_unit = more && cur.u == u_before;
                }
                if (!ok) break;
                // ---- the unit's groups are done: the second set hands over, the first finishes the rows
                if (set == 1) {
                    if (xchg_phase > 0 && !mbar_wait<false>(xchg_free, (xchg_phase - 1) & 1u)) { ok = false; break; }
#pragma unroll
                    for (int m = 0; m < NB; ++m) xchg[m * 128 + rl] = acc[m];
                    __syncwarp();
                    if (lane == 0) mbar_arrive(xchg_full);
                    ++xchg_phase;
                    continue;
                }
                if (!mbar_wait<false>(xchg_full, xchg_phase & 1u)) { ok = false; break; }
                ++xchg_phase;
#pragma unroll
                for (int m = 0; m < NB; ++m) acc[m] += xchg[m * 128 + rl];
                __syncwarp();
                if (lane == 0) mbar_arrive(xchg_free);
                if (p.ksplit == 1) {
                    if (row < mt.rows) {
#pragma unroll
                        for (int m = 0; m < NB; ++m)
                            if (m < p.M) {
                                float v = acc[m] * p.inv_xscale[m];
                                const size_t o = (size_t)m * mt.ldo + row;
                                if (mt.residual != nullptr) v = mt.residual[o] + v;
                                mt.out[o] = v;
                            }
                    }
                } else {
                    float* part = p.partial + ((size_t)tile * p.ksplit + z) * (size_t)(NB * 128);
#pragma unroll
                    for (int m = 0; m < NB; ++m) part[m * 128 + rl] = acc[m];
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(drain_bar);
                    if (!mbar_wait<false>(drain_bar, drain_phase & 1u)) { ok = false; break; }
                    ++drain_phase;
                    if (warp == 12 && lane == 0) {
                        const unsigned int prev = atomicAdd(&p.counters[tile], 1u);
                        *last_flag = prev == (unsigned int)p.ksplit - 1u ? 1u : 0u;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(drain_bar);
                    if (!mbar_wait<false>(drain_bar, drain_phase & 1u)) { ok = false; break; }
                    ++drain_phase;
                    if (*reinterpret_cast<volatile uint32_t*>(last_flag) != 0u) {
                        // the last arrival of a tile adds the partials in split order; all loads of a split are issued together
                        __threadfence();
                        const float* base = p.partial + (size_t)tile * p.ksplit * (size_t)(NB * 128) + rl;
#pragma unroll
                        for (int m = 0; m < NB; ++m) acc[m] = 0.0f;
#pragma unroll 1
                        for (int zz = 0; zz < p.ksplit; ++zz) {
                            float t[NB];
#pragma unroll
                            for (int m = 0; m < NB; ++m) t[m] = __ldcg(base + (size_t)zz * (NB * 128) + m * 128);
#pragma unroll
                            for (int m = 0; m < NB; ++m) acc[m] += t[m];
                        }
                        if (row < mt.rows) {
#pragma unroll
                            for (int m = 0; m < NB; ++m)
                                if (m < p.M) {
                                    float v = acc[m] * p.inv_xscale[m];
                                    const size_t o = (size_t)m * mt.ldo + row;
                                    if (mt.residual != nullptr) v = mt.residual[o] + v;
                                    mt.out[o] = v;
                                }
                        }
                        if (warp == 12 && lane == 0) p.counters[tile] = 0u;
                    }
                }
            }
            if (q == 0 && lane == 0) PROF_END(6 + set);
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    if (!ok) atomicCAS(&g_device_status, 0, 1);
}

// ---- RS-I8 form ---------------------------------------------------------------------------------------------------------
// The int8 weights are MMA operands exactly as they lie in memory: TMA writes 128 rows x 128 bytes with the 128-byte
// swizzle and the tensor core reads them; no thread touches a weight.  One row scale per output, so the s32 accumulators
// run over the whole K range of a unit (|sum| <= 127 * 128 * K < 2^31 for K <= 131072) and are read once per unit.
// Two MMA-issuing threads take the groups alternately; each keeps its OWN accumulator (the first MMA of a unit overwrites,
// and nothing orders the two threads), the drain adds the two.  Buffers alternate with the unit's parity, so the MMAs of
// the next unit run while the previous one is read out.
//   warps 0, 11: MMA     warp 4: TMA digit planes     warp 8: TMA weights     warps 12..15: drain     others: idle
template <int NB>
struct SmallShapeI8 {
    static constexpr int kWBytes = 128 * 128;
    static constexpr int kBBytes = 4 * NB * 128;
    static constexpr int kStageBytes = kWBytes + kBBytes;
    static constexpr int kStages = NB == 16 ? 9 : 6;
    static constexpr int kOffBars = kStages * kStageBytes;
    static constexpr int kNumBars = kStages + kBtDoneRing + 2 + 2 + 1;
    static constexpr int kSmemBytes = kOffBars + kNumBars * 8 + 16 + 1024;
    static_assert(kStages < kBtDoneRing && kSmemBytes <= 227 * 1024, "ring");
};

template <int NB>
__global__ void __launch_bounds__(512, 1) linear_gemm_small_i8_kernel(const SmallParams p, const __grid_constant__ CUtensorMap map_w0,
                                                                       const __grid_constant__ CUtensorMap map_w1,
                                                                       const __grid_constant__ CUtensorMap map_w2,
                                                                       const __grid_constant__ CUtensorMap map_x) {
    using S = SmallShapeI8<NB>;
    constexpr int kN = 4 * NB;
    constexpr uint32_t kTmemCols = 4 * kN;  // [unit parity][MMA thread]: 256 or 512 columns
    extern __shared__ unsigned char ssmem_raw[];
    unsigned char* ssmem = ssmem_raw + ((1024u - (smem_u32(ssmem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(ssmem + S::kOffBars);  // [kStages] weights and digit planes have landed (two arrivals)
    uint64_t* done = full + S::kStages;                                 // [kBtDoneRing] the MMAs of group number n have completed
    uint64_t* tmem_free = done + kBtDoneRing;                           // [2] the drain warps have read the buffers of that unit parity
    uint64_t* unit_done = tmem_free + 2;                                // [2] both issuing threads' MMAs of a unit of that parity have completed
    uint64_t* drain_bar = unit_done + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
    uint32_t* last_flag = tmem_slot + 1;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = (p.K + 127) >> 7;  // 128-column groups (the last may be partial: TMA fills with zeros)
    if (tid == 0) {
        for (int s = 0; s < S::kStages; ++s) mbar_init(&full[s], 2);
        for (int s = 0; s < kBtDoneRing; ++s) mbar_init(&done[s], 1);
        mbar_init(&tmem_free[0], kBtSetWarps);
        mbar_init(&tmem_free[1], kBtSetWarps);
        mbar_init(&unit_done[0], 2);
        mbar_init(&unit_done[1], 2);
        mbar_init(drain_bar, kBtSetWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t smem_base = smem_u32(ssmem);
    bool ok = true;
    auto done_wait = [&](int n) { return mbar_wait<false>(&done[n & (kBtDoneRing - 1)], (uint32_t)(n >> 4) & 1u); };
    UnitCursor cur;

    if (warp == 4 || warp == 8) {
        // ---- TMA producers: a stage is free when the group that used it last (kStages back) has been multiplied.
        // (Two alternating threads per stream were tried: no faster, and one run of a 250-tile matrix ended in a launch
        // failure whose cause was not found by reading; the single-thread form below is the one that has run every shape.)
        const bool digits = warp == 4;
        if (digits) pdl_wait();  // the digit planes come from the previous kernel; the weights never change
        if (lane == 0 && cur.start(p, blockIdx.x, G)) {
            RingPos<S::kStages> sp;
            int it = 0;
            do {
                if (it >= S::kStages && !done_wait(it - S::kStages)) { ok = false; break; }
                const uint32_t st = smem_base + (uint32_t)sp.idx * S::kStageBytes;
                if (digits) {
                    mbar_arrive_expect_tx(&full[sp.idx], (uint32_t)S::kBBytes);
                    tma_load_3d(st + S::kWBytes, &map_x, cur.g * 128, 0, 0, &full[sp.idx]);
                } else {
                    const int mi = (p.nmat > 2 && cur.tile >= p.mat[2].tile_start) ? 2 : (p.nmat > 1 && cur.tile >= p.mat[1].tile_start) ? 1 : 0;
                    const CUtensorMap* map = mi == 0 ? &map_w0 : mi == 1 ? &map_w1 : &map_w2;
                    mbar_arrive_expect_tx(&full[sp.idx], (uint32_t)S::kWBytes);
                    tma_load_2d(st, map, cur.g * 128, (cur.tile - p.mat[mi].tile_start) * 128, &full[sp.idx]);
                }
                sp.next();
                ++it;
            } while (cur.advance(p, G));
        }
    } else if (warp == 0 || warp == 11) {
        const int set = warp == 0 ? 0 : 1;
        if (lane == 0 && cur.start(p, blockIdx.x, G)) {
            constexpr uint32_t idesc = gemm_idesc_s8s8(128, kN);
            const uint64_t desc_a0 = gemm_smem_desc(smem_base), desc_b0 = gemm_smem_desc(smem_base + S::kWBytes);
            RingPos<S::kStages> sp;
            int it = 0, unit_no = 0;
            bool more = true;
            while (more && ok) {
                // accumulators of this unit: parity of the unit, then this thread's half
                const int par = unit_no & 1;
                if (unit_no >= 2 && !mbar_wait<false>(&tmem_free[par], (uint32_t)((unit_no >> 1) - 1) & 1u)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t d = tmem_base + (uint32_t)((par * 2 + set) * kN);
                bool first = true, same_unit = true;
                while (same_unit) {
                    if ((it & 1) == set) {
                        if (!mbar_wait<false>(&full[sp.idx], sp.phase)) { ok = false; break; }
                        tcgen05_fence_after();
                        const uint64_t soff = (uint64_t)((uint32_t)sp.idx * (S::kStageBytes >> 4));
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) gemm_mma_i8(d, desc_a0 + soff + 2 * ks, desc_b0 + soff + 2 * ks, idesc, (first && ks == 0) ? 0u : 1u);
                        first = false;
                        umma_commit(&done[it & (kBtDoneRing - 1)]);
                    }
                    sp.next();
                    ++it;
                    const int u_before = cur.u;
                    more = cur.advance(p, G);
                    same_unit = more && cur.u == u_before;
                }
                if (!ok) break;
                umma_commit(&unit_done[par]);  // everything this thread issued for the unit (a unit has at least two groups)
                ++unit_no;
            }
        }
    } else if (warp >= 12) {
        // ---- drain: lane = weight row inside the tile; once per unit
        const int q = warp & 3;
        const int rl = q * 32 + lane;
        uint32_t drain_phase = 0;
        pdl_wait();
        if (cur.start(p, blockIdx.x, G)) {
            int it = 0, unit_no = 0;
            bool more = true;
            while (more && ok) {
                const int tile = cur.tile, z = cur.z;
                const int n_items = cur.g1 - cur.g;
                const int mi = (p.nmat > 2 && tile >= p.mat[2].tile_start) ? 2 : (p.nmat > 1 && tile >= p.mat[1].tile_start) ? 1 : 0;
                const SmallMat& mt = p.mat[mi];
                const int row = (tile - mt.tile_start) * 128 + rl;
                const int it_first = it;
                it += n_items;
                for (int k = 0; k < n_items && more; ++k) more = cur.advance(p, G);
                const int par = unit_no & 1;
                if (!mbar_wait<false>(&unit_done[par], (uint32_t)(unit_no >> 1) & 1u)) { ok = false; break; }
                tcgen05_fence_after();
                // which thread took the first group of the unit decides nothing here: both accumulators are simply added
                const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((par * 2 + 0) * kN);
                const uint32_t tb = ta + (uint32_t)kN;
                float acc[NB];
#pragma unroll
                for (int m0 = 0; m0 < NB; m0 += 8) {
                    long long v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = 0;
#pragma unroll
                    for (int dgt = 3; dgt >= 0; --dgt) {
                        uint32_t a[8], b[8];
                        tmem_ld8(ta + dgt * NB + m0, a);
                        tmem_ld8(tb + dgt * NB + m0, b);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] = v[j] * 256 + (long long)((int)a[j] + (int)b[j]);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[m0 + j] = (float)v[j];
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_free[par]);
                (void)it_first;
                const float rscale = row < mt.rows ? mt.row_scales[row] : 0.0f;
                if (p.ksplit == 1) {
                    if (row < mt.rows) {
#pragma unroll
                        for (int m = 0; m < NB; ++m)
                            if (m < p.M) {
                                float y = acc[m] * p.inv_xscale[m] * rscale;
                                const size_t o = (size_t)m * mt.ldo + row;
                                if (mt.residual != nullptr) y = mt.residual[o] + y;
                                mt.out[o] = y;
                            }
                    }
                } else {
                    float* part = p.partial + ((size_t)tile * p.ksplit + z) * (size_t)(NB * 128);
#pragma unroll
                    for (int m = 0; m < NB; ++m) part[m * 128 + rl] = acc[m];
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(drain_bar);
                    if (!mbar_wait<false>(drain_bar, drain_phase & 1u)) { ok = false; break; }
                    ++drain_phase;
                    if (warp == 12 && lane == 0) {
                        const unsigned int prev = atomicAdd(&p.counters[tile], 1u);
                        *last_flag = prev == (unsigned int)p.ksplit - 1u ? 1u : 0u;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(drain_bar);
                    if (!mbar_wait<false>(drain_bar, drain_phase & 1u)) { ok = false; break; }
                    ++drain_phase;
                    if (*reinterpret_cast<volatile uint32_t*>(last_flag) != 0u) {
                        __threadfence();
                        const float* base = p.partial + (size_t)tile * p.ksplit * (size_t)(NB * 128) + rl;
#pragma unroll
                        for (int m = 0; m < NB; ++m) acc[m] = 0.0f;
                        // (two splits per round trip where the registers allow it - this kernel has 128 per thread; the order of the additions stays)
                        constexpr int kPerTrip = NB <= 16 ? 2 : 1;
#pragma unroll 1
                        for (int zz = 0; zz < p.ksplit; zz += kPerTrip) {
                            float t[kPerTrip][NB];
#pragma unroll
                            for (int q2 = 0; q2 < kPerTrip; ++q2)
                                if (zz + q2 < p.ksplit) {
#pragma unroll
                                    for (int m = 0; m < NB; ++m) t[q2][m] = __ldcg(base + (size_t)(zz + q2) * (NB * 128) + m * 128);
                                }
#pragma unroll
                            for (int q2 = 0; q2 < kPerTrip; ++q2)
                                if (zz + q2 < p.ksplit) {
#pragma unroll
                                    for (int m = 0; m < NB; ++m) acc[m] += t[q2][m];
                                }
                        }
                        if (row < mt.rows) {
#pragma unroll
                            for (int m = 0; m < NB; ++m)
                                if (m < p.M) {
                                    float y = acc[m] * p.inv_xscale[m] * rscale;
                                    const size_t o = (size_t)m * mt.ldo + row;
                                    if (mt.residual != nullptr) y = mt.residual[o] + y;
                                    mt.out[o] = y;
                                }
                        }
                        if (warp == 12 && lane == 0) p.counters[tile] = 0u;
                    }
                }
                ++unit_no;
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    if (!ok) atomicCAS(&g_device_status, 0, 1);
}

}  // namespace kmll
