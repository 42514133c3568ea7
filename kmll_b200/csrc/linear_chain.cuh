// Chained streaming linear kernel for W4-G128 weights in the PREPARED layout (batch 1), included by linear.cu.
//
// One launch runs up to four projections of a decoder layer back to back ("phases": output projection + residual,
// RMSNorm + gate/up + SiLU, down projection + residual, RMSNorm + next layer's Q/K/V or the lm_head arg-max) on one
// resident 512-thread block per multiprocessor.  The weight ring of a block never drains at a projection boundary:
// its load cursor runs ahead into the next phase's weights while the block still multiplies, waits for its input
// or converts it, so HBM stays busy across the boundary.  The vector that one phase produces for the next travels
// through device memory as 64-bit words (value, exchange number): the consumer polls the words until they carry the
// number it expects, so a word is its own "ready" flag and neither a fence nor a grid-wide barrier is needed.  Under
// tensor parallelism the same words are pushed into every rank's inbox over NVLink and the consumer adds the ranks'
// partial vectors in rank order.  All blocks of the grid are resident at once (grid <= multiprocessors, one block
// each), so a polled producer is always running; every poll is bounded in time and raises the device status word.
//
// Prepared layout (kmll_w4g128_prepare): the matrix is cut into records of 32 weight rows x one 128-column
// quantization group.  A record is 2112 bytes: 2048 bytes of weights + 32 binary16 group scales.  The weight
// bytes are stored in the order the tensor-core fragments want them: bytes [512 i + 16 l, +16) are the four A
// registers of lane l for the i-th m16n8k32 MMA of the group.  Every byte holds TWO weights of the same column:
// the high nibble is the two's-complement value q of a row of the first 16-row block ("A rows"), the low nibble is
// q + 8 of the same row of the second block ("B rows").  Read as a signed byte this is 16 q_A + (q_B + 8), so
//     MMA(raw bytes)            = 16 dot_A + dot_B + 8 sum(x)
//     MMA(bytes & 0x0f)         =            dot_B + 8 sum(x)
// and one logic operation per register (instead of three) separates the two row blocks exactly, in integers.
// For the gate/up pair the A rows are gate rows and the B rows the matching up rows, so SiLU(gate) * up meets in one
// lane.  Column order inside a group: MMA i, register half h, lane quad position t, byte e  <->  column
// 32 t + 8 i + 4 h + e, which lets a lane read its B operands of a whole group as 32 consecutive activation bytes.
//
// Activations: x * 2^sh is rounded to an integer X with |X| < 2^29; X + 2^30 is split into four unsigned bytes
// d0..d3, which are four of the eight MMA columns; a column of ones gives the row sum of the weights, which removes
// the offset: sum(w X) = c0 + 256 c1 + 65536 c2 + 2^24 (c3 - 64 c_ones).  All integer, exact.  The only roundings
// are x -> a multiple of 2^-29 max|x| (f32 itself resolves 2^-24 of each element) and a few f32 operations per
// group and row, so the result is at least as accurate as an f32 dot product in any order.
#pragma once

namespace kmll {

constexpr int kCPlane = kSThreads * 16;
constexpr int kCEarly = 0;  // records of a later phase a warp may have in flight before that phase's input has been requested

// one exchange word; waits (bounded) until it carries `number`
__device__ inline bool ld_exchange_value(const uint2* slot, uint32_t number, unsigned long long t0, float* value) {
    for (;;) {
        unsigned long long w;
        asm volatile("ld.global.cg.u64 %0, [%1];" : "=l"(w) : "l"(slot) : "memory");
        if ((uint32_t)(w >> 32) == number) {
            *value = __uint_as_float((uint32_t)w);
            return true;
        }
        if (wait_clock_ticks() - t0 > kPeerWaitLimitTicks) {
            *value = 0.0f;
            return false;
        }
    }
}

__device__ inline uint32_t chain_epoch(const TpExchange& xc, uint32_t step, int index) { return step * (uint32_t)xc.mult + (uint32_t)index + 1u; }

// Arrival hint of an exchange: every finished unit adds one to a counter next to the consumer (a remote reduction for
// the inbox of a tensor-parallel peer).  Counters only grow: after `step` decode steps an exchange fed by n units per
// rank stands at step * tp * n.  The hint carries no data and orders nothing - the words themselves say whether they
// are valid - it only keeps 148 blocks x 512 threads from hammering L2 with polls while the producers still work.
__device__ inline void chain_signal(const TpExchange& xc, int kind, int index) {
    if (kind == CHAIN_OUT_INBOX) {
        for (int dst = 0; dst < xc.tp; ++dst)
            asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(xc.ready[dst] + index) : "memory");
    } else {
        asm volatile("red.relaxed.gpu.global.add.u32 [%0], 1;" ::"l"(xc.ready_local + index) : "memory");
    }
}

// timeline of the chained kernel: 24 stamps per block (four ordinary slots): 0 entry, 1 dependency wait passed,
// phase i at 2 + 5 i: arrival hint seen, input words loaded, statistics reduced, digits staged, units done (as seen by
// thread 0); 22 end
constexpr int kChainStamps = 4 * kTraceStamps;
__device__ inline void chain_stamp(unsigned long long* base, int stamp) {
    if (base != nullptr && threadIdx.x == 0) base[(size_t)blockIdx.x * kChainStamps + stamp] = global_timer_ns();
}

// rows[r] = byte r of (a, b, c, d), r = 0..3
__device__ inline void transpose_bytes4(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&rows)[4]) {
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);
    const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);
    rows[0] = __byte_perm(t0, t1, 0x5410);
    rows[1] = __byte_perm(t0, t1, 0x7632);
    rows[2] = __byte_perm(t2, t3, 0x5410);
    rows[3] = __byte_perm(t2, t3, 0x7632);
}

// Stages the K activations of a phase as four digit rows d0..d3 of (x * 2^sh + 2^30) in natural column order, plus
// the per-group correction words of the low-nibble rows (see the file comment): corr[4 g + t] for lane position t.
// The input comes from a plain vector or straight out of exchange words (rank-ordered sum of the inbox slots, or the
// local vector): thread 0 first sleeps on the arrival hint, then every thread loads the words of its own blocks
// into registers and checks their numbers (bounded retries), so the vector never takes a detour through shared
// memory.  Block 0 also stores a gathered vector to x_out.  Returns 2^-sh.
constexpr int kCStageBlocks = 4;  // 8-element blocks of the input a thread holds in registers while it is staged: K <= 16384
template <typename AfterLoads>
__device__ __forceinline__ float chain_stage(const ChainPhase& ph, const TpExchange& xc, uint32_t step, int xs_pitch, int8_t* xs, int* corr,
                                             float* misc, unsigned long long* dbg, AfterLoads after_loads) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = ph.K;
    const int nblk = K >> 3;
    const bool norm = ph.norm_w != nullptr;
    float v[kCStageBlocks][8];
    if (ph.in_kind == CHAIN_IN_PLAIN) {
#pragma unroll
        for (int j = 0; j < kCStageBlocks; ++j) {
            if (j * kSThreads + warp * 32 < nblk) {
                const int blk = j * kSThreads + tid;
                const float4* src = reinterpret_cast<const float4*>(ph.x + ((blk < nblk ? blk : 0) << 3));
                const float4 a = src[0], b = src[1];
                v[j][0] = a.x; v[j][1] = a.y; v[j][2] = a.z; v[j][3] = a.w;
                v[j][4] = b.x; v[j][5] = b.y; v[j][6] = b.z; v[j][7] = b.w;
            }
        }
    } else {
        const bool inbox = ph.in_kind == CHAIN_IN_INBOX;
        const uint32_t epoch = chain_epoch(xc, step, ph.in_index);
        const int tp = inbox ? xc.tp : 1;
        const uint4* gb = inbox ? reinterpret_cast<const uint4*>(xc.inbox[xc.rank]) + (size_t)(ph.in_index & 1) * tp * (xc.dim >> 1)
                                : reinterpret_cast<const uint4*>(xc.local_box);
        const int stride = inbox ? (xc.dim >> 1) : 0;
        const unsigned long long t0 = wait_clock_ticks();
        bool good = true;
        bool topped = false;
        // the last pair of blocks this warp loads: the held-back weight copies are requested right behind its loads
        int last_half = 0;
#pragma unroll
        for (int half = 1; half < kCStageBlocks / 2; ++half)
            if ((2 * half) * kSThreads + warp * 32 < nblk) last_half = half;
        if (ph.in_units > 0) {
            if (tid == 0) {
                const unsigned int* hint = (inbox ? xc.ready[xc.rank] : xc.ready_local) + ph.in_index;
                const unsigned int target = step * (unsigned int)(tp * ph.in_units);
                for (;;) {
                    unsigned int c;
                    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(c) : "l"(hint) : "memory");
                    if ((int)(c - target) >= 0) break;
                    if (wait_clock_ticks() - t0 > kPeerWaitLimitTicks) break;  // the word loads below report the failure
                    __nanosleep(64);
                }
            }
            __syncthreads();
        }
        chain_stamp(dbg, 0);
        // two blocks (eight 16-byte loads) of a rank at a time
#pragma unroll
        for (int half = 0; half < kCStageBlocks / 2; ++half) {
            if ((2 * half) * kSThreads + warp * 32 < nblk) {
#pragma unroll 1
                for (int r = 0; r < tp; ++r) {
                    const uint4* src = gb + (size_t)r * stride;
                    uint4 q[2][4];
                    for (;;) {
                        bool all = true;
#pragma unroll
                        for (int jj = 0; jj < 2; ++jj) {
                            const int blk = (2 * half + jj) * kSThreads + tid;
                            const uint4* bp = src + (size_t)(blk < nblk ? blk : 0) * 4;
#pragma unroll
                            for (int m = 0; m < 4; ++m) q[jj][m] = ld_exchange_pair_gpu(bp + m);
                        }
                        if (!topped && half == last_half && r == tp - 1) {
                            after_loads();
                            topped = true;
                        }
#pragma unroll
                        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                            for (int m = 0; m < 4; ++m) all = all && q[jj][m].y == epoch && q[jj][m].w == epoch;
                        if (all) break;
                        if (wait_clock_ticks() - t0 > kPeerWaitLimitTicks) { good = false; break; }
                        __nanosleep(32);
                    }
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                        for (int m = 0; m < 4; ++m) {
                            const float a = __uint_as_float(q[jj][m].x), b = __uint_as_float(q[jj][m].z);
                            v[2 * half + jj][2 * m] = r == 0 ? a : v[2 * half + jj][2 * m] + a;
                            v[2 * half + jj][2 * m + 1] = r == 0 ? b : v[2 * half + jj][2 * m + 1] + b;
                        }
                }
            }
        }
        if (!good) atomicCAS(&g_device_status, 0, 2);
        if (!topped) after_loads();
        if (blockIdx.x == 0 && ph.x_out != nullptr) {
#pragma unroll
            for (int j = 0; j < kCStageBlocks; ++j) {
                const int blk = j * kSThreads + tid;
                if (blk < nblk) {
                    float4* dst = reinterpret_cast<float4*>(ph.x_out + (blk << 3));
                    dst[0] = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
                    dst[1] = make_float4(v[j][4], v[j][5], v[j][6], v[j][7]);
                }
            }
        }
    }
    if (ph.in_kind == CHAIN_IN_PLAIN) after_loads();  // the input has been requested: weight copies held back for it may go now
    chain_stamp(dbg, 1);
    float ss = 0.0f, mx = 0.0f;
#pragma unroll
    for (int j = 0; j < kCStageBlocks; ++j) {
        if (j * kSThreads + warp * 32 < nblk) {
            const bool active = j * kSThreads + tid < nblk;
            float s_ = 0.0f, m_ = 0.0f;
            if (norm) {
                const uint4 nwj = *reinterpret_cast<const uint4*>(ph.norm_w + (active ? (j * kSThreads + tid) << 3 : 0));
                const uint32_t ww[4] = {nwj.x, nwj.y, nwj.z, nwj.w};
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
            if (active) { ss += s_; mx = fmaxf(mx, m_); }
        }
    }
    ss = warp_sum(ss);
    mx = warp_max(mx);
    if (lane == 0) { misc[warp * 2] = ss; misc[warp * 2 + 1] = mx; }
    __syncthreads();  // (also: every warp is past the previous phase's records, so the digit rows may be replaced)
    float inv, amax;
    {
        float s_ = misc[(lane & 15) * 2], m_ = misc[(lane & 15) * 2 + 1];
#pragma unroll
        for (int off = 1; off < 16; off <<= 1) {
            s_ += __shfl_xor_sync(0xffffffffu, s_, off);
            m_ = fmaxf(m_, __shfl_xor_sync(0xffffffffu, m_, off));
        }
        inv = norm ? 1.0f / sqrtf(s_ / (float)K + ph.eps) : 1.0f;
        amax = m_ * inv;
    }
    chain_stamp(dbg, 2);
    // power-of-two scale: |x * 2^sh| < 2^29 for every element (margin for the few ulps by which the product
    // recomputed below may exceed the maximum found above).  A non-finite maximum gives all-zero digits.
    float xscale = 0.0f, inv_xscale = 1.0f;
    amax *= 1.00001f;
    if (amax > 0.0f && amax < INFINITY) {
        const int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127;
        int sh = 28 - e;
        sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
        xscale = __uint_as_float((uint32_t)(sh + 127) << 23);
        inv_xscale = __uint_as_float((uint32_t)(127 - sh) << 23);
    }
#pragma unroll
    for (int j = 0; j < kCStageBlocks; ++j) {
        const int wbase = j * kSThreads + warp * 32;
        if (wbase < nblk) {  // warp-uniform
            const int blk = wbase + lane;
            const bool active = blk < nblk;
            const int k = (active ? blk : wbase) << 3;
            float u[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) u[q] = v[j][q];
            if (norm) {
                const uint4 nwj = *reinterpret_cast<const uint4*>(ph.norm_w + k);  // (read before: a cache hit)
                const uint32_t ww[4] = {nwj.x, nwj.y, nwj.z, nwj.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {  // kmll's order: x * inv * w
                    u[2 * q] = u[2 * q] * inv * __uint_as_float(ww[q] << 16);
                    u[2 * q + 1] = u[2 * q + 1] * inv * __uint_as_float(ww[q] & 0xffff0000u);
                }
            }
            uint32_t d[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) d[q] = (uint32_t)(__float2int_rn(u[q] * xscale) + 0x40000000);
            uint32_t r0[4], r1[4];
            transpose_bytes4(d[0], d[1], d[2], d[3], r0);
            transpose_bytes4(d[4], d[5], d[6], d[7], r1);
            if (active) {
#pragma unroll
                for (int r = 0; r < 4; ++r) *reinterpret_cast<uint2*>(xs + (size_t)r * xs_pitch + k) = make_uint2(r0[r], r1[r]);
            }
            // per-group sums of the digit bytes -> correction words of the low-nibble rows: a group is the 16 blocks of
            // a half warp; the four sums travel as two packed pairs (each sum < 2^16)
            uint32_t s01 = 0u, s23 = 0u;
            if (active) {
                s01 = __dp4a(r0[0], 0x01010101u, __dp4a(r1[0], 0x01010101u, 0u)) | (__dp4a(r0[1], 0x01010101u, __dp4a(r1[1], 0x01010101u, 0u)) << 16);
                s23 = __dp4a(r0[2], 0x01010101u, __dp4a(r1[2], 0x01010101u, 0u)) | (__dp4a(r0[3], 0x01010101u, __dp4a(r1[3], 0x01010101u, 0u)) << 16);
            }
#pragma unroll
            for (int off = 1; off < 16; off <<= 1) {
                s01 += __shfl_xor_sync(0xffffffffu, s01, off);
                s23 += __shfl_xor_sync(0xffffffffu, s23, off);
            }
            if ((lane & 15) == 0 && active) {
                const int s0 = (int)(s01 & 0xffffu), s1 = (int)(s01 >> 16), s2 = (int)(s23 & 0xffffu), s3 = (int)(s23 >> 16);
                *reinterpret_cast<int4*>(corr + 4 * (k >> 7)) = make_int4(8 * (s0 + 256 * s1), 8 * s2, 8 * (s3 - 64 * 128), 0);
            }
        }
    }
    // constants behind the digit rows: 16 bytes of ones, then 16 bytes of zeros (absent MMA columns); in this order the
    // broadcast reads of either fall on banks the digit row read by the same quarter warp does not use
    if (tid < 4) reinterpret_cast<uint32_t*>(xs + (size_t)4 * xs_pitch)[tid] = 0x01010101u;
    else if (tid < 8) reinterpret_cast<uint32_t*>(xs + (size_t)4 * xs_pitch)[tid] = 0u;
    __syncthreads();
    chain_stamp(dbg, 3);
    return inv_xscale;
}

__global__ void __launch_bounds__(kSBlock, 1) linear_chain_kernel(const __grid_constant__ ChainParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    chain_stamp(p.trace, 0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    int8_t* xs = reinterpret_cast<int8_t*>(smem);
    int* corr = reinterpret_cast<int*>(smem + p.off_corr);
    float* red = reinterpret_cast<float*>(smem + p.off_red);            // [kCRedBufs][kSWarps + 2][32]
    uint64_t* done = reinterpret_cast<uint64_t*>(smem + p.off_bars);    // [kCRedBufs]
    unsigned int* cnt = reinterpret_cast<unsigned int*>(done + kCRedBufs);
    float* misc = reinterpret_cast<float*>(smem + p.off_misc);
    __shared__ bool s_last_block;

    if (tid == 0) {
        for (int b = 0; b < kCRedBufs; ++b) { mbar_init(&done[b], 1); cnt[b] = 0u; }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    // ---- weight stream: lane-private ring, one record (4 x 16 bytes per lane + 64 bytes of scales per warp) per slot
    const uint32_t ring_dst = smem_u32(smem + p.off_ring + (size_t)tid * 16);
    const unsigned char* ring = smem + p.off_ring + (size_t)tid * 16;
    const unsigned char* sring = smem + p.off_sring + (size_t)warp * (kCDepth * 64);
    const uint32_t sring_dst = smem_u32(sring) + (uint32_t)lane * 16;  // lanes 0..3 copy the 64 bytes of scales

    auto warp_slice = [&](int ngroups, int& j0, int& j1) {
        j0 = (warp * ngroups) / kSWarps;
        j1 = ((warp + 1) * ngroups) / kSWarps;
    };
    auto record_ptr = [&](const ChainPhase& ph, int unit, int seg) -> const unsigned char* {
        int mi = 0;
#pragma unroll
        for (int i = 1; i < 3; ++i)
            if (unit >= ph.unit_start[i]) mi = i;
        return ph.w[mi] + ((size_t)(unit - ph.unit_start[mi]) * ph.ngroups + seg) * kCRecBytes;
    };

    // load cursor: (phase, unit, records left in the unit, next record)
    int l_phase = 0, l_unit = 0, l_left = 0;
    const unsigned char* l_src = nullptr;
    auto l_enter = [&]() {  // positions the cursor on the next record this warp has to load, or past the last phase
        for (; l_phase < p.n_phases; ++l_phase, l_unit = blockIdx.x) {
            const ChainPhase& ph = p.phase[l_phase];
            int j0, j1;
            warp_slice(ph.ngroups, j0, j1);
            if (j1 > j0 && l_unit < ph.total_units) {
                l_left = j1 - j0;
                l_src = record_ptr(ph, l_unit, j0) + lane * 16;
                return;
            }
        }
    };
    l_unit = blockIdx.x;
    l_enter();
    // Records of a LATER phase than the one being consumed are held back (beyond kCEarly per warp): a multiprocessor
    // gets its load responses back in request order, so the loads of the next phase's input vector - the critical
    // path of a phase change - would wait behind every weight read from HBM that was requested before them (measured:
    // 3.5 us with the ring full, against 1 us for the same loads alone).  The slots held back are requested right
    // behind those loads (top_up).
    int c_phase_now = 0, ahead = 0, held = 0;
    bool hold_all = false;
    auto issue_record = [&](int slot) {
        const uint32_t dst = ring_dst + (uint32_t)slot * (4 * kCPlane);
#pragma unroll
        for (int i = 0; i < 4; ++i) cp_async_stream16_to(dst + i * kCPlane, l_src + i * 512);
        if (lane < 4) cp_async_stream16_to(sring_dst + (uint32_t)slot * 64, l_src + 2048);
        if (l_phase != c_phase_now) ++ahead;
        l_src += kCRecBytes;
        if (--l_left == 0) {
            l_unit += gridDim.x;
            l_enter();
        }
    };
    auto load_record = [&](int slot) {
        if (l_phase < p.n_phases) {
            if (hold_all || (l_phase != c_phase_now && ahead >= kCEarly)) ++held;  // its slot stays empty until top_up
            else issue_record(slot);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per slot, also when nothing was copied
    };
    // weights do not depend on the previous kernel: half of the ring is requested before the dependency wait, the other
    // half right behind the loads of the first phase's input (so that those do not wait behind 128 KB of weights)
#pragma unroll 1
    for (int d = 0; d < kCDepth; ++d) {
        hold_all = d >= kCDepth / 2;
        load_record(d);
    }
    hold_all = false;

    pdl_wait();
    chain_stamp(p.trace, 1);
    // number of the running decode step (written by the kernel that began the step, at least one launch ago)
    const uint32_t step = p.xc != nullptr ? *p.xcv.epoch : 0u;

    // this lane's B column g: digit rows d0, d1, d2, -, d3, ones, -, -; absent columns read 16 zero bytes with stride 0
    const int8_t* ones = xs + (size_t)4 * p.xs_pitch;
    const int8_t* xcol;
    int bstride = 0;
    if (g < 3) { xcol = xs + (size_t)g * p.xs_pitch + t * 32; bstride = 1; }
    else if (g == 4) { xcol = xs + (size_t)3 * p.xs_pitch + t * 32; bstride = 1; }
    else if (g == 5) xcol = ones;
    else xcol = ones + 16;
    // this lane's C columns 2t, 2t+1: (d0, d1), (d2, -), (d3, ones), (-, -)
    const int pair_mul = t == 0 ? 256 : (t == 2 ? -64 : 0);
    const float w_lane = t == 0 ? 1.0f : (t == 1 ? 65536.0f : (t == 2 ? 16777216.0f : 0.0f));

    float best_logit = -INFINITY;
    uint32_t best_token = 0xffffffffu;
    bool ok = true;
    int it = 0, slot = 0;
    auto top_up = [&]() {  // the `held` most recently consumed slots are empty: fill them, oldest first
        while (held > 0) {
            int sl = slot - held;
            if (sl < 0) sl += kCDepth;
            if (l_phase < p.n_phases) issue_record(sl);
            asm volatile("cp.async.commit_group;" ::: "memory");
            --held;
        }
    };

#pragma unroll 1
    for (int c_phase = 0; c_phase < p.n_phases; ++c_phase) {
        const ChainPhase& ph = p.phase[c_phase];
        int j0, j1;
        warp_slice(ph.ngroups, j0, j1);
        const int spu = j1 - j0;
        if ((int)blockIdx.x >= ph.total_units) continue;  // no unit of this phase for this block
        c_phase_now = c_phase;
        ahead = 0;
        const float inv_xscale = chain_stage(ph, p.xcv, step, p.xs_pitch, xs, corr, misc, p.trace != nullptr ? p.trace + 2 + 5 * c_phase : nullptr, top_up);
        const float wA = w_lane * inv_xscale * 0.0625f, wB = w_lane * inv_xscale;
        const int epi = ph.epi;

#pragma unroll 1
        for (int c_unit = blockIdx.x; c_unit < ph.total_units && ok; c_unit += gridDim.x, ++it) {
            int mi = 0;
#pragma unroll
            for (int i = 1; i < 3; ++i)
                if (c_unit >= ph.unit_start[i]) mi = i;
            const int unit_in_mat = c_unit - ph.unit_start[mi];
            const int row0 = unit_in_mat * (epi == EPI_SILU ? 16 : kCRows);
            // the warp that owns the epilogue fetch of this unit asks for the residual long before it is used
            float pre_res = 0.0f;
            bool res_ok = true;
            if (epi == EPI_RESIDUAL && ph.add_residual && (it % kSWarps) == warp) {
                const int row = row0 + lane;
                if (row < ph.out_rows[mi]) {
                    if (ph.residual_index >= 0) {
                        const TpExchange& xc = p.xcv;
                        const uint32_t epoch = chain_epoch(xc, step, ph.residual_index);
                        const uint2* box = xc.inbox[xc.rank] + (size_t)(ph.residual_index & 1) * xc.tp * xc.dim + row;
                        const unsigned long long t0 = wait_clock_ticks();
                        for (int r = 0; r < xc.tp; ++r) {
                            float pv;
                            res_ok = ld_exchange_value(box + (size_t)r * xc.dim, epoch, t0, &pv) && res_ok;
                            pre_res = r == 0 ? pv : pre_res + pv;
                        }
                    } else {
                        pre_res = ph.residual[row];
                    }
                }
            }
            float accA0 = 0.0f, accA1 = 0.0f, accB0 = 0.0f, accB1 = 0.0f;
#pragma unroll 1
            for (int sg = j0; sg < j1; ++sg) {
                asm volatile("cp.async.wait_group %0;" ::"n"(kCDepth - 1) : "memory");  // this lane's oldest record has landed
                __syncwarp();  // the scales were copied by lanes 0..3
                const unsigned char* rs = ring + (size_t)slot * (4 * kCPlane);
                const uint4 xb0 = *reinterpret_cast<const uint4*>(xcol + (size_t)(sg * 128) * bstride);
                const uint4 xb1 = *reinterpret_cast<const uint4*>(xcol + (size_t)(sg * 128 + 16) * bstride);
                const uint2 sc = *reinterpret_cast<const uint2*>(sring + slot * 64 + g * 8);
                const int cw = corr[4 * sg + t];
                const uint32_t bx[8] = {xb0.x, xb0.y, xb0.z, xb0.w, xb1.x, xb1.y, xb1.z, xb1.w};
                int c2[4], c1[4];  // raw bytes (16 q_A + q_B + 8) and low nibbles (q_B + 8)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint4 w = *reinterpret_cast<const uint4*>(rs + (size_t)i * kCPlane);
                    const uint32_t m0 = w.x & 0x0f0f0f0fu, m1 = w.y & 0x0f0f0f0fu, m2 = w.z & 0x0f0f0f0fu, m3 = w.w & 0x0f0f0f0fu;
                    if (i == 0) {
                        mma_s8_first(c2, w.x, w.y, w.z, w.w, bx[0], bx[1]);
                        mma_s8_first(c1, m0, m1, m2, m3, bx[0], bx[1]);
                    } else {
                        mma_s8(c2, w.x, w.y, w.z, w.w, bx[2 * i], bx[2 * i + 1]);
                        mma_s8(c1, m0, m1, m2, m3, bx[2 * i], bx[2 * i + 1]);
                    }
                }
                __syncwarp();  // every lane has read the slot's scales before they are replaced
                load_record(slot);
                if (++slot == kCDepth) slot = 0;
                // rows g (c[0], c[1]) and g + 8 (c[2], c[3]); the lane's column pair is combined in integers
                const int p2a = c2[0] + pair_mul * c2[1], p1a = c1[0] + pair_mul * c1[1];
                const int p2b = c2[2] + pair_mul * c2[3], p1b = c1[2] + pair_mul * c1[3];
                const float sA0 = __half2float(__ushort_as_half((unsigned short)(sc.x & 0xffffu)));
                const float sA1 = __half2float(__ushort_as_half((unsigned short)(sc.x >> 16)));
                const float sB0 = __half2float(__ushort_as_half((unsigned short)(sc.y & 0xffffu)));
                const float sB1 = __half2float(__ushort_as_half((unsigned short)(sc.y >> 16)));
                accA0 = fmaf((float)(p2a - p1a), sA0, accA0);
                accA1 = fmaf((float)(p2b - p1b), sA1, accA1);
                accB0 = fmaf((float)(p1a - cw), sB0, accB0);
                accB1 = fmaf((float)(p1b - cw), sB1, accB1);
            }
            // ---- end of the unit: the warps' partial sums meet in shared memory; the warp that delivers last finishes
            const int buf = it % kCRedBufs;
            const uint32_t bpar = (uint32_t)(it / kCRedBufs) & 1u;
            if (it >= kCRedBufs && !mbar_wait(&done[buf], bpar ^ 1u)) { ok = false; break; }
            float* ub = red + (size_t)buf * (kSWarps + 2) * kCRows;
            {
                float vA0 = accA0 * wA, vA1 = accA1 * wA, vB0 = accB0 * wB, vB1 = accB1 * wB;
                vA0 += __shfl_xor_sync(0xffffffffu, vA0, 1); vA0 += __shfl_xor_sync(0xffffffffu, vA0, 2);
                vA1 += __shfl_xor_sync(0xffffffffu, vA1, 1); vA1 += __shfl_xor_sync(0xffffffffu, vA1, 2);
                vB0 += __shfl_xor_sync(0xffffffffu, vB0, 1); vB0 += __shfl_xor_sync(0xffffffffu, vB0, 2);
                vB1 += __shfl_xor_sync(0xffffffffu, vB1, 1); vB1 += __shfl_xor_sync(0xffffffffu, vB1, 2);
                if (t == 0) {
                    float* rp = ub + warp * kCRows;
                    rp[g] = vA0; rp[g + 8] = vA1; rp[16 + g] = vB0; rp[24 + g] = vB1;
                }
            }
            if (epi == EPI_RESIDUAL && (it % kSWarps) == warp) ub[kSWarps * kCRows + lane] = pre_res;
            if (!res_ok) { ok = false; atomicCAS(&g_device_status, 0, 2); }
            __syncwarp();
            unsigned int prev = 0;
            if (lane == 0) {
                __threadfence_block();
                prev = atomicAdd(&cnt[buf], 1u);
            }
            prev = __shfl_sync(0xffffffffu, prev, 0);
            if (prev != kSWarps - 1) continue;
            __threadfence_block();
            if (lane == 0) cnt[buf] = 0u;
            {
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < kSWarps; ++w) v += ub[w * kCRows + lane];
                int row = row0 + lane;
                bool valid = row < ph.out_rows[mi];
                if (epi == EPI_SILU) {
                    // lanes 0..15 hold the gate rows, lanes 16..31 the matching up rows
                    const float u = __shfl_down_sync(0xffffffffu, v, 16);
                    v = (v / (1.0f + expf(-v))) * u;
                    valid = valid && lane < 16;
                }
                if (epi == EPI_TOP1) {
                    float cand = valid ? v : -INFINITY;
                    uint32_t cand_tok = valid ? (uint32_t)row : 0xffffffffu;
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, cand, off);
                        const uint32_t ot = __shfl_xor_sync(0xffffffffu, cand_tok, off);
                        if (top1_better(ov, ot, cand, cand_tok)) { cand = ov; cand_tok = ot; }
                    }
                    if (top1_better(cand, cand_tok, best_logit, best_token)) { best_logit = cand; best_token = cand_tok; }
                } else if (valid) {
                    if (epi == EPI_RESIDUAL && ph.add_residual) v = ub[kSWarps * kCRows + lane] + v;
                    if (ph.out_kind == CHAIN_OUT_PLAIN) {
                        ph.out[mi][row] = v;
                    } else {
                        const TpExchange& xc = p.xcv;
                        const uint32_t epoch = chain_epoch(xc, step, ph.out_index);
                        if (ph.out_kind == CHAIN_OUT_INBOX) {
                            const size_t s = ((size_t)(ph.out_index & 1) * xc.tp + xc.rank) * xc.dim + row;
                            for (int dst = 0; dst < xc.tp; ++dst) push_exchange_word(xc.inbox[dst] + s, __float_as_uint(v), epoch, xc.tp > 1 ? xc.push_mode : 0);
                        } else {
                            push_exchange_word(xc.local_box + row, __float_as_uint(v), epoch, 0);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) {
                if (ph.out_kind != CHAIN_OUT_PLAIN) chain_signal(p.xcv, ph.out_kind, ph.out_index);
                mbar_arrive(&done[buf]);
            }
        }
        chain_stamp(p.trace, 2 + 5 * c_phase + 4);
        if (!ok) break;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (p.partial_tokens != nullptr) {
        // every warp finished some units: merge the 16 running bests (fixed order) into one partial per block; the
        // block that arrives last merges the blocks' partials (arg-max of kmll: higher logit, then lower token)
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
            __threadfence();
            const unsigned int prev = atomicAdd(p.top1_counter, 1u);
            s_last_block = prev == gridDim.x - 1;
        }
        __syncthreads();
        if (s_last_block && warp == 0) {
            __threadfence();
            float bl = -INFINITY;
            uint32_t bt = 0xffffffffu;
            for (int i = lane; i < (int)gridDim.x; i += 32) {
                const float l = __ldcg(p.partial_logits + i);
                const uint32_t tk = __ldcg(p.partial_tokens + i);
                if (top1_better(l, tk, bl, bt)) { bl = l; bt = tk; }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bl, off);
                const uint32_t ot = __shfl_xor_sync(0xffffffffu, bt, off);
                if (top1_better(ov, ot, bl, bt)) { bl = ov; bt = ot; }
            }
            if (lane == 0) {
                const uint64_t packed = pack_top1(bl, bt == 0xffffffffu ? bt : bt + p.token_offset);
                p.packed_out[0] = packed;
                *p.top1_counter = 0u;  // ready for the next launch
                if (p.state != nullptr) {  // single GPU: this is the end of the decode step
                    p.state->next_top = packed;
                    p.state->position += 1;
                    p.state->step += 1;
                }
                if (p.push_top) {  // tensor parallel: hand this rank's result to every rank (two exchange words)
                    const TpExchange& xc = p.xcv;
                    const uint32_t epoch = step * (uint32_t)xc.mult + (uint32_t)xc.top_index + 1u;
                    const size_t s = ((size_t)(epoch & 1u) * xc.tp + xc.rank) * 2;
                    for (int dst = 0; dst < xc.tp; ++dst) {
                        st_exchange_word(xc.top_inbox[dst] + s, (uint32_t)(packed >> 32), epoch);
                        st_exchange_word(xc.top_inbox[dst] + s + 1, (uint32_t)(packed & 0xffffffffull), epoch);
                    }
                }
            }
        }
    }
    chain_stamp(p.trace, 22);
    if (!ok) atomicCAS(&g_device_status, 0, 1);
}

// ---- canonical W4-G128 -> prepared records --------------------------------------------------------------------
// One thread per 32-bit word of the output.  pair != 0: the A rows of unit u are rows 16u.. of matrix a (gate) and
// the B rows the same rows of matrix b (up); else A rows = 32u.., B rows = 32u + 16.. of matrix a.
__global__ void w4_prepare_kernel(const uint8_t* __restrict__ pa, const uint16_t* __restrict__ sa, const uint8_t* __restrict__ pb,
                                  const uint16_t* __restrict__ sb, int rows, int cols, int pair, size_t total_words,
                                  uint32_t* __restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total_words) return;
    constexpr int kWords = kCRecBytes / 4;  // 528
    const int ngroups = cols >> 7;
    const size_t rec = idx / kWords;
    const int wi = (int)(idx - rec * kWords);
    const int unit = (int)(rec / ngroups), grp = (int)(rec - (size_t)unit * ngroups);
    const int rowA0 = pair ? unit * 16 : unit * 32, rowB0 = pair ? unit * 16 : unit * 32 + 16;
    const uint8_t* pB = pair ? pb : pa;
    const uint16_t* sB = pair ? sb : sa;
    const size_t rowbytes = (size_t)cols >> 1;
    uint32_t word = 0;
    if (wi < 512) {
        const int i = wi >> 7, l = (wi >> 2) & 31, a = wi & 3;
        const int gq = l >> 2, tq = l & 3;
        const int rp = gq + 8 * (a & 1), h = a >> 1;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int col = grp * 128 + tq * 32 + i * 8 + h * 4 + e;
            const int ra = rowA0 + rp, rb = rowB0 + rp;
            uint32_t na = 8u, nb = 8u;  // rows past the end: q = 0
            if (ra < rows) { const uint8_t b = pa[(size_t)ra * rowbytes + (col >> 1)]; na = (col & 1) ? (b >> 4) : (b & 15u); }
            if (rb < rows) { const uint8_t b = pB[(size_t)rb * rowbytes + (col >> 1)]; nb = (col & 1) ? (b >> 4) : (b & 15u); }
            const uint32_t byte = (((na - 8u) & 15u) << 4) | nb;  // high nibble: two's complement q_A; low nibble: q_B + 8
            word |= byte << (8 * e);
        }
    } else {
        const int si = wi - 512;  // (g, which): g = si / 2; which = 0: A rows g, g + 8; 1: B rows g, g + 8
        const int gq = si >> 1;
        const int r0 = (si & 1) ? rowB0 + gq : rowA0 + gq, r1 = r0 + 8;
        const uint16_t* s = (si & 1) ? sB : sa;
        const uint32_t lo = r0 < rows ? s[(size_t)r0 * ngroups + grp] : 0u;
        const uint32_t hi = r1 < rows ? s[(size_t)r1 * ngroups + grp] : 0u;
        word = lo | (hi << 16);
    }
    out[idx] = word;
}

}  // namespace kmll
