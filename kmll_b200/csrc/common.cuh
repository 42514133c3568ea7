// Shared helpers for the kmll_b200 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/kmll_b200.h"

namespace kmll {

// ---- error reporting ----------------------------------------------------------------------
char* last_error_buffer();
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);

#define KMLL_REQUIRE_PTR(p)                                                   \
    do {                                                                      \
        if ((p) == nullptr) return ::kmll::fail(KMLL_ERR_NULL, "%s: null pointer %s", __func__, #p); \
    } while (0)

#define KMLL_REQUIRE(cond, ...)                                               \
    do {                                                                      \
        if (!(cond)) return ::kmll::fail(KMLL_ERR_SHAPE, __VA_ARGS__);        \
    } while (0)

#define KMLL_TRY_RC(expr)                 \
    do {                                  \
        const int rc__ = (expr);          \
        if (rc__ != KMLL_OK) return rc__; \
    } while (0)

// ---- bf16 bit patterns (kmll stores norm weights / embeddings as raw bf16 bits) ------------
__host__ __device__ inline float bf16_bits_to_f32(uint16_t bits) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(static_cast<uint32_t>(bits) << 16);
#else
    union { uint32_t u; float f; } v;
    v.u = static_cast<uint32_t>(bits) << 16;
    return v.f;
#endif
}

// Bf16::from_f32 of kmll: add 0x7fff + lsb, take the top half (round to nearest even, no NaN
// special case).
__device__ inline uint16_t f32_to_bf16_bits(float value) {
    uint32_t bits = __float_as_uint(value);
    uint32_t rounding_bias = ((bits >> 16) & 1u) + 0x7fffu;
    return static_cast<uint16_t>((bits + rounding_bias) >> 16);
}

// ---- warp / block reductions ---------------------------------------------------------------
__device__ inline float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
__device__ inline float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

// Block-wide sum; every thread gets the result.  `scratch` holds >= 33 floats.
__device__ inline float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ inline float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// arg-max combine rule of kmll: strictly greater wins, equal logits -> lower token id
// (crates/inference/src/kernels/inference.rs:402-404).
__device__ inline bool top1_better(float cand_logit, uint32_t cand_token, float best_logit,
                                   uint32_t best_token) {
    return cand_logit > best_logit || (cand_logit == best_logit && cand_token < best_token);
}
__device__ inline uint64_t pack_top1(float logit, uint32_t token) {
    return (static_cast<uint64_t>(__float_as_uint(logit)) << 32) | static_cast<uint64_t>(token);
}

// 128-bit streaming load that does not allocate in L1 (weights are read exactly once).
__device__ inline uint4 ld_stream_u4(const void* ptr) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr));
    return v;
}

// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialisation
// attribute may start before its predecessor has finished; everything that reads the
// predecessor's output must come after pdl_wait().  Both are no-ops for a normal launch.
//
// pdl_wait() also releases this kernel's own dependents at once: they are scheduled as soon as
// multiprocessors become free (while this grid is still in its tail), run the part of their code
// that needs no input - above all the first weight loads - and then block in their own wait until
// this grid has completed.  Because every kernel releases its dependents only AFTER its own wait has
// returned, a kernel can only start once everything up to its predecessor's predecessor has
// completed; code placed before pdl_wait() may therefore read constants and data written two or more
// launches earlier, nothing else.
__device__ inline void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ inline void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    pdl_launch_dependents();
}

// ---- kernel timeline (diagnostics) -------------------------------------------------------------------
// While a trace buffer is attached (kmll_trace_attach), every launch of the linear stream kernel and of the
// decode attention kernel is given a slot in it and thread 0 of each block stamps %globaltimer at fixed
// points.  Slots are assigned on the host at launch time, so the launches baked into a CUDA graph keep theirs
// and every replay overwrites the same words.  With no buffer attached the kernels get a null pointer.
constexpr int kTraceStamps = 6;
unsigned long long* trace_next_slot(int kernel_id, int blocks);  // host side; null when tracing is off
// Bumped by every kmll_trace_attach.  A CUDA graph bakes the slot pointers of the launches it captured, so whoever
// caches a graph records the generation at capture and captures again when it has changed (otherwise replays would
// keep stamping a buffer the caller has detached, and possibly freed).
unsigned long long trace_generation();
__device__ inline void trace_stamp(unsigned long long* base, int stamp) {
    if (base != nullptr && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        base[(size_t)(blockIdx.y * gridDim.x + blockIdx.x) * kTraceStamps + stamp] = t;
    }
}

// latest time over all callers (one lane per warp calls it); the buffer must be zero before the launch
__device__ inline void trace_stamp_latest(unsigned long long* base, int stamp) {
    if (base != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        atomicMax(base + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * kTraceStamps + stamp, t);
    }
}

inline cudaStream_t as_stream(kmll_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Launch helper: optional programmatic dependent launch attribute.  Every launch through it is counted per host
// thread, so a caller can report how many kernels an operator sequence really issued.
bool pdl_enabled();
unsigned long long& launch_counter();
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, bool pdl, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl && pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    ++launch_counter();
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace kmll
