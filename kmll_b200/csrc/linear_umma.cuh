// Batched RS-I8 linear on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory),
// included by linear.cu.  Serves kmll's batched i8 linear (gemm_f32_i8_scaled_tiled_kernel,
// crates/inference/src/kernels/matmul.rs:116-214) for 5 or more rows of activations: prefill and
// batches of sequences.
//
// Operands are swapped relative to the usual GEMM: the 128 weight rows of a block are the M side of the
// MMA, the activations are the N side.  The activations arrive as byte digits (digitize_rows_kernel:
// x * 2^sh = u0 + 256 * u1 + 65536 * (top - 64), plus a column of ones that yields the row sum of the
// weights; the same scheme as the batch-1 stream kernel), four columns per row of x, so 16 rows of x are
// N = 64 columns and one tcgen05.mma.kind::i8 (s8 x u8 -> s32, M = 128, N = 64, K = 32) multiplies 128 x 32
// weights by all of them.  The int8 weights are used exactly as they lie in memory: 16-byte asynchronous
// copies place them in shared memory in the canonical K-major no-swizzle layout (core matrix = 8 rows x 16
// bytes), a matrix descriptor points at them, no thread ever touches a weight.  The int32 accumulators of
// the whole K loop live in 64 columns of tensor memory and are read once (tcgen05.ld) by the four warps
// for the epilogue: combine the digit columns, row scale, 2^-sh, optional residual.
//
// Pipeline: kUmmaStages stages of one k-tile each (128 weight rows x 256 bytes + 64 digit rows x 256 bytes; core
// matrices 144 bytes apart so that a warp's 16-byte copies spread over all shared-memory banks).  Eight warps copy;
// a copied k-tile is reported on the stage's `full` mbarrier kUmmaLag tiles later (cp.async.wait_group, then a plain
// arrive).  One thread of a ninth warp waits for `full`, issues the proxy fence and the eight MMAs of the stage and
// commits them to the stage's `empty` mbarrier, which releases the stage for refilling; no block-wide barrier inside
// the loop.  Measured and rejected: an arrive-on-completion copy barrier (cp.async.mbarrier.arrive) and a proxy fence
// in every copying thread - both serialise a thread's copies tile by tile.  Every mbarrier wait is bounded
// (mbar_wait); on time-out the block raises the device status word and leaves after freeing its tensor memory.
#pragma once

namespace kmll {

constexpr int kUmmaRows = 128;    // weight rows per block = MMA M
constexpr int kUmmaBatch = 16;    // rows of x per pass
constexpr int kUmmaN = 4 * kUmmaBatch;  // digit columns = MMA N
constexpr int kUmmaKT = 256;      // bytes of K per stage (8 MMAs of K = 32)
constexpr int kUmmaStages = 4;
constexpr int kUmmaLag = 2;       // a copied k-tile is reported to the MMA thread this many k-tiles later
constexpr int kUmmaABytes = (kUmmaRows / 8) * (kUmmaKT / 16) * (128 + 16);  // weight tile incl. padding
constexpr int kUmmaBBytes = (kUmmaN / 8) * (kUmmaKT / 16) * (128 + 16);     // digit tile incl. padding
constexpr int kUmmaLoaders = 256;  // copying threads (8 warps)
constexpr int kUmmaLbo = 128 + 16;  // bytes between core matrices that are neighbours along K: 16 bytes of padding
                                    // spread a warp's 16-byte copies over all shared-memory banks (with 128 the 16
                                    // chunks of a row would all fall on the same four banks)
constexpr int kUmmaSbo = (kUmmaKT / 16) * kUmmaLbo;  // bytes between groups of 8 rows
constexpr int kUmmaThreads = kUmmaLoaders + 32;  // + the warp whose lane 0 issues the MMAs

struct UmmaParams {
    const int8_t* w;          // [rows, ldw] int8 weights
    const float* row_scales;  // [rows]
    int rows, K, ldw;
    const uint8_t* digits;    // [4 * kUmmaBatch, K]: rows 4b..4b+3 = u0, u1, top, ones of batch row b
    const float* inv_xscale;  // [kUmmaBatch] 2^-sh per batch row
    int batch;                // valid batch rows (<= kUmmaBatch)
    float* out;               // [batch, ldo]
    const float* residual;    // [batch, ldo] or null
    int ldo;
    float* partial;           // split-K: [row tiles][gridDim.y][kUmmaBatch][kUmmaRows] digit-combined partial sums
    unsigned int* counters;   // split-K: [row tiles] arrivals, zero between launches
    unsigned long long* trace;  // timeline slot of this launch, or null (stamps: 0 entry, 1 tensor memory ready,
                                // 2 first k-tile landed, 3 last MMA issued, 4 block done, 5 copies issued)
};

// ---- activations -> byte digits (optionally RMSNorm first), one block per row of x -------------------
__global__ void __launch_bounds__(1024) digitize_rows_kernel(const float* __restrict__ x, int ldx, int K,
                                                             const uint16_t* __restrict__ norm_w, float eps,
                                                             uint8_t* __restrict__ digits, float* __restrict__ inv_xscale) {
    __shared__ float scratch[40];
    pdl_wait();
    const int b = blockIdx.x;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)b * ldx);  // K % 128 == 0, rows 16-byte aligned
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
    float amax = mx * inv * 1.00001f;
    float xscale = 0.0f, inv_scale = 1.0f;
    if (amax > 0.0f && amax < INFINITY) {
        const int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127;
        int sh = 21 - e;
        sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
        xscale = __uint_as_float((uint32_t)(sh + 127) << 23);
        inv_scale = __uint_as_float((uint32_t)(127 - sh) << 23);
    }
    uint32_t* d0 = reinterpret_cast<uint32_t*>(digits + (size_t)(4 * b) * K);
    const int kw = K / 4;  // words per digit row
    for (int k4 = threadIdx.x; k4 < kw; k4 += blockDim.x) {
        float4 v = xr[k4];
        if (norm_w) {  // kmll's order: x * inv * w
            const uint2 w = nw[k4];
            v.x = v.x * inv * __uint_as_float(w.x << 16);
            v.y = v.y * inv * __uint_as_float(w.x & 0xffff0000u);
            v.z = v.z * inv * __uint_as_float(w.y << 16);
            v.w = v.w * inv * __uint_as_float(w.y & 0xffff0000u);
        }
        // mantissa = 2^22 + round(v * 2^sh); its bytes are the digits
        const uint32_t b0 = __float_as_uint(fmaf(v.x, xscale, 12582912.0f)), b1 = __float_as_uint(fmaf(v.y, xscale, 12582912.0f));
        const uint32_t b2 = __float_as_uint(fmaf(v.z, xscale, 12582912.0f)), b3 = __float_as_uint(fmaf(v.w, xscale, 12582912.0f));
        const uint32_t t0 = __byte_perm(b0, b1, 0x5140), t1 = __byte_perm(b2, b3, 0x5140);
        const uint32_t t2 = __byte_perm(b0, b1, 0x7362), t3 = __byte_perm(b2, b3, 0x7362);
        d0[k4] = __byte_perm(t0, t1, 0x5410);
        d0[kw + k4] = __byte_perm(t0, t1, 0x7632);
        d0[2 * kw + k4] = __byte_perm(t2, t3, 0x5410);
        d0[3 * kw + k4] = 0x01010101u;
    }
    if (threadIdx.x == 0) inv_xscale[b] = inv_scale;
}

// ---- tcgen05 helpers -----------------------------------------------------------------------------------
// shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes; `lbo` = bytes between
// the two 16-byte K chunks of one MMA, `sbo` = bytes between groups of 8 rows; version 1 (sm_100)
__device__ inline uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}
// instruction descriptor of kind::i8: D = s32, A = signed 8 bit, B = unsigned 8 bit, both K-major, N >> 3, M >> 4
__host__ __device__ constexpr uint32_t umma_idesc_s8u8(int m, int n) {
    return (2u << 4) | (1u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ inline void umma_mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ inline void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ inline void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ inline void cp_async16_ca(uint32_t smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns of tensor memory -> 16 registers per thread
__device__ inline void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__global__ void __launch_bounds__(kUmmaThreads, 1) linear_umma_i8_kernel(const UmmaParams p) {
    extern __shared__ __align__(1024) unsigned char usmem[];
    // [stage][A 16 KB | B 8 KB], then the mbarriers and the tensor-memory base address
    uint64_t* full = reinterpret_cast<uint64_t*>(usmem + (size_t)kUmmaStages * (kUmmaABytes + kUmmaBBytes));  // copies of a stage landed
    uint64_t* empty = full + kUmmaStages;                                                                    // its MMAs completed
    uint64_t* all_done = empty + kUmmaStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(all_done + 1);
    trace_stamp(p.trace, 0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = blockIdx.x * kUmmaRows;
    // split-K: blockIdx.y takes k-tiles [kt0, kt0 + KT) of the row; the blocks of a row tile meet in the epilogue
    const int kt_all = p.K / kUmmaKT;
    const int kt_per = (kt_all + (int)gridDim.y - 1) / (int)gridDim.y;
    const int kt0 = (int)blockIdx.y * kt_per;
    const int KT = max(0, min(kt_per, kt_all - kt0));

    if (tid == 0) {
        for (int s = 0; s < kUmmaStages; ++s) { mbar_init(&full[s], kUmmaLoaders); mbar_init(&empty[s], 1); }
        mbar_init(all_done, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kUmmaN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t smem_base = smem_u32(usmem);
    trace_stamp(p.trace, 1);
    constexpr uint32_t kIdesc = umma_idesc_s8u8(kUmmaRows, kUmmaN);

    pdl_wait();  // the digits come from the previous kernel
    bool ok = true;
    if (warp < kUmmaLoaders / 32) {
        // ---- loader warps: thread t moves 16-byte chunk t % kChunks of rows t / kChunks + kPass * i of every k-tile.  Destination:
        // core matrix (row / 8, chunk) at (row / 8) * kUmmaSbo + chunk * kUmmaLbo, row (row % 8) of it at + (row % 8) * 16.
        constexpr int kChunks = kUmmaKT / 16, kPass = kUmmaLoaders / kChunks;  // 16-byte chunks per row, rows per pass
        const int chunk = tid % kChunks, rsub = tid / kChunks;
#pragma unroll 1
        for (int kt = 0; kt < KT; ++kt) {
            const int stage = kt % kUmmaStages, use = kt / kUmmaStages;
            if (use > 0 && !mbar_wait<false>(&empty[stage], (uint32_t)(use - 1) & 1u)) { ok = false; break; }
            const uint32_t a_dst = smem_base + (uint32_t)stage * (kUmmaABytes + kUmmaBBytes);
            const uint32_t b_dst = a_dst + kUmmaABytes;
            // Blocks walk K from staggered starting points (integer accumulation does not depend on the order): with
            // every block on the same k-tile at the same time, all rows' addresses would agree modulo the row pitch
            // and crowd onto a few memory channels.
            const int kt_eff = kt0 + (kt + (int)blockIdx.x * 5) % KT;
            const size_t koff = (size_t)kt_eff * kUmmaKT + (size_t)chunk * 16;
#pragma unroll
            for (int i = 0; i < kUmmaRows / kPass; ++i) {
                const int r = rsub + kPass * i;
                const int row = min(row0 + r, p.rows - 1);
                cp_async16_ca(a_dst + (uint32_t)((r >> 3) * kUmmaSbo + chunk * kUmmaLbo + (r & 7) * 16), p.w + (size_t)row * p.ldw + koff);
            }
#pragma unroll
            for (int i = 0; i < (kUmmaN + kPass - 1) / kPass; ++i) {
                const int r = rsub + kPass * i;
                if (r >= kUmmaN) break;
                const int drow = min(r, 4 * p.batch - 1);  // columns of absent batch rows repeat a valid one and are ignored
                cp_async16_ca(b_dst + (uint32_t)((r >> 3) * kUmmaSbo + chunk * kUmmaLbo + (r & 7) * 16), p.digits + (size_t)drow * p.K + koff);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            // k-tile kt - kUmmaLag has landed (for this thread): report it.  A proxy fence here, in every copying thread, was
            // measured to wait for ALL of the thread's copies in flight and so to serialise the tiles.
            // (An arrive-on-completion copy barrier was measured to serialise a warp's copies tile by tile.)
            if (kt >= kUmmaLag) {
                asm volatile("cp.async.wait_group %0;" ::"n"(kUmmaLag) : "memory");
                mbar_arrive(&full[(kt - kUmmaLag) % kUmmaStages]);  // (the MMA thread issues the proxy fence)
            }
        }
        trace_stamp(p.trace, 5);
        // drain: the last kUmmaLag k-tiles
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (ok)
            for (int kt = (KT > kUmmaLag ? KT - kUmmaLag : 0); kt < KT; ++kt) mbar_arrive(&full[kt % kUmmaStages]);
    } else if (lane == 0) {
        // ---- MMA issuer: one thread; the tensor core reads the operands through the descriptors
#pragma unroll 1
        for (int kt = 0; kt < KT; ++kt) {
            const int stage = kt % kUmmaStages, use = kt / kUmmaStages;
            if (!mbar_wait<false>(&full[stage], (uint32_t)use & 1u)) { ok = false; break; }
            if (kt == 0 && p.trace != nullptr) trace_stamp_latest(p.trace, 2);
            fence_proxy_async_smem();  // the copies went through the generic proxy; the tensor core reads through the async proxy
            tcgen05_fence_after();
            const uint32_t a_addr = smem_base + (uint32_t)stage * (kUmmaABytes + kUmmaBBytes);
            const uint32_t b_addr = a_addr + kUmmaABytes;
#pragma unroll
            for (int ks = 0; ks < kUmmaKT / 32; ++ks) {
                const uint64_t da = umma_smem_desc(a_addr + ks * 2 * kUmmaLbo, kUmmaLbo, kUmmaSbo);
                const uint64_t db = umma_smem_desc(b_addr + ks * 2 * kUmmaLbo, kUmmaLbo, kUmmaSbo);
                umma_mma_i8(tmem_base, da, db, kIdesc, (kt > 0 || ks > 0) ? 1u : 0u);
            }
            umma_commit(&empty[stage]);  // arrives when the MMAs issued so far have completed: the stage may be refilled
        }
        if (ok) umma_commit(all_done);
        if (p.trace != nullptr) trace_stamp_latest(p.trace, 3);
    }
    // ---- epilogue (warps 0..3; warp w reads tensor-memory lanes 32 w .. 32 w + 31)
    __shared__ bool is_last;
    const bool split = gridDim.y > 1;
    if (warp < 4) {
        if (ok && KT > 0 && !mbar_wait<false>(all_done, 0u)) ok = false;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        tcgen05_fence_after();
        ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below are warp-collective: all lanes or none
        if (ok) {
            const int rl = warp * 32 + lane;  // row inside the tile
            const int row = row0 + rl;
            const float rs = row < p.rows ? p.row_scales[row] : 0.0f;
            float* part = split ? p.partial + ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * kUmmaBatch * kUmmaRows : nullptr;
#pragma unroll
            for (int c0 = 0; c0 < kUmmaN; c0 += 16) {
                uint32_t r[16];
                if (KT > 0) {
                    tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int q = 0; q < 16; ++q) r[q] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int b = c0 / 4 + j;
                    const int u0 = (int)r[4 * j], u1 = (int)r[4 * j + 1], top = (int)r[4 * j + 2], ones = (int)r[4 * j + 3];
                    const float comb = (float)u0 + 256.0f * (float)u1 + 65536.0f * (float)(top - 64 * ones);
                    if (split) {
                        part[b * kUmmaRows + rl] = comb;  // scales and residual are applied after the merge
                    } else if (b < p.batch && row < p.rows) {
                        float v = comb * p.inv_xscale[b] * rs;
                        const size_t o = (size_t)b * p.ldo + row;
                        if (p.residual != nullptr) v = p.residual[o] + v;
                        p.out[o] = v;
                    }
                }
            }
        }
    }
    if (split) {
        // the block that delivers last adds the partial sums of the row tile in blockIdx.y order and finishes the rows
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned int prev = atomicAdd(&p.counters[blockIdx.x], 1u);
            is_last = prev == gridDim.y - 1;
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            const float* base = p.partial + (size_t)blockIdx.x * gridDim.y * kUmmaBatch * kUmmaRows;
            for (int idx = tid; idx < p.batch * kUmmaRows; idx += kUmmaThreads) {
                const int b = idx / kUmmaRows, rl = idx - b * kUmmaRows;
                const int row = row0 + rl;
                if (row < p.rows) {
                    float acc = 0.0f;
                    for (int z = 0; z < (int)gridDim.y; ++z) acc += __ldcg(base + ((size_t)z * kUmmaBatch + b) * kUmmaRows + rl);
                    float v = acc * p.inv_xscale[b] * p.row_scales[row];
                    const size_t o = (size_t)b * p.ldo + row;
                    if (p.residual != nullptr) v = p.residual[o] + v;
                    p.out[o] = v;
                }
            }
            if (tid == 0) p.counters[blockIdx.x] = 0u;  // ready for the next launch
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    trace_stamp(p.trace, 4);
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kUmmaN) : "memory");
    if (!ok) atomicCAS(&g_device_status, 0, 1);
}

}  // namespace kmll
