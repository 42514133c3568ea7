// Device-side quantizers and dequantizers.  They restate kmll's host quantizer
// (RowwiseScaledI8Matrix::from_bf16_rows_symmetric, crates/inference/src/rowwise_scaled.rs:21-51)
// with IEEE f32 division and round-half-away-from-zero, so the produced bytes are identical to
// the host result; max() is order-independent, hence the parallel reduction is exact.
#include "internal.cuh"

namespace kmll {

__device__ inline float clamp_f32(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

__global__ void __launch_bounds__(256) quantize_rs_i8_kernel(const uint16_t* __restrict__ w, int cols,
                                                             int8_t* __restrict__ values, float* __restrict__ scales) {
    __shared__ float scratch[40];
    const size_t base = (size_t)blockIdx.x * cols;
    float mx = 0.0f;
    for (int c = threadIdx.x; c < cols; c += 256) mx = fmaxf(mx, fabsf(bf16_bits_to_f32(w[base + c])));
    mx = block_max(mx, scratch);
    const float scale = (mx == 0.0f) ? 1.0f : mx / 127.0f;
    if (threadIdx.x == 0) scales[blockIdx.x] = scale;
    for (int c = threadIdx.x; c < cols; c += 256) {
        const float q = clamp_f32(roundf(bf16_bits_to_f32(w[base + c]) / scale), -127.0f, 127.0f);
        values[base + c] = (int8_t)(int)q;
    }
}

__global__ void dequant_rs_i8_kernel(const int8_t* __restrict__ values, const float* __restrict__ scales, int rows,
                                     int cols, float* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * cols) return;
    out[i] = (float)values[i] * scales[i / cols];
}

// One warp per 128-column group; each lane owns 4 consecutive columns (2 packed bytes).
__global__ void __launch_bounds__(256) quantize_w4_kernel(const float* __restrict__ w, size_t n_groups,
                                                          uint8_t* __restrict__ packed, uint16_t* __restrict__ gscales) {
    const int lane = threadIdx.x & 31;
    const size_t grp = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (grp >= n_groups) return;
    const float4 v = reinterpret_cast<const float4*>(w + grp * 128)[lane];
    float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    mx = warp_max(mx);
    const float scale_f32 = (mx == 0.0f) ? 1.0f : mx / 7.0f;
    __half sh = __float2half_rn(scale_f32);
    uint16_t sbits = __half_as_ushort(sh);
    if ((sbits & 0x7fffu) == 0) {
        sbits = 0x0001u;  // never divide by a zero scale
        sh = __ushort_as_half(sbits);
    }
    if (lane == 0) gscales[grp] = sbits;
    const float scale = __half2float(sh);
    const int q0 = (int)clamp_f32(roundf(v.x / scale), -7.0f, 7.0f) + 8;
    const int q1 = (int)clamp_f32(roundf(v.y / scale), -7.0f, 7.0f) + 8;
    const int q2 = (int)clamp_f32(roundf(v.z / scale), -7.0f, 7.0f) + 8;
    const int q3 = (int)clamp_f32(roundf(v.w / scale), -7.0f, 7.0f) + 8;
    const uint16_t two = (uint16_t)((q0 | (q1 << 4)) | ((q2 | (q3 << 4)) << 8));
    reinterpret_cast<uint16_t*>(packed + grp * 64)[lane] = two;
}

__global__ void dequant_w4_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ gscales, size_t n,
                                  float* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint8_t byte = packed[i >> 1];
    const int nib = (i & 1) ? (byte >> 4) : (byte & 0xf);
    out[i] = (float)(nib - 8) * __half2float(__ushort_as_half(gscales[i >> 7]));
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ src, size_t n, uint16_t* __restrict__ dst) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = f32_to_bf16_bits(src[i]);
}

__global__ void widen_bf16_kernel(const uint16_t* __restrict__ src, size_t n, float* __restrict__ dst) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = bf16_bits_to_f32(src[i]);
}

__device__ inline uint64_t splitmix64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}

// Counter-based N(0, std): element i depends only on (seed, i).
__global__ void fill_normal_kernel(float* __restrict__ dst, size_t n, uint64_t seed, float stddev) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t r = splitmix64(seed * 0xd1342543de82ef95ull + i);
    const float u1 = ((float)((r >> 40) & 0xffffffull) + 1.0f) * (1.0f / 16777216.0f);  // (0,1]
    const float u2 = (float)((r >> 16) & 0xffffffull) * (1.0f / 16777216.0f);           // [0,1)
    dst[i] = stddev * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

int widen_bf16(cudaStream_t stream, const uint16_t* src, size_t n, float* dst) {
    if (n == 0) return KMLL_OK;
    widen_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(src, n, dst);
    return check_launch("widen_bf16");
}

}  // namespace kmll

using namespace kmll;

extern "C" {

int kmll_quantize_rs_i8(kmll_stream_t s, const uint16_t* w, int rows, int cols, int8_t* values, float* scales) {
    KMLL_REQUIRE_PTR(w); KMLL_REQUIRE_PTR(values); KMLL_REQUIRE_PTR(scales);
    KMLL_REQUIRE(rows > 0 && cols > 0, "quantize_rs_i8: shape [%d, %d] must be positive", rows, cols);
    quantize_rs_i8_kernel<<<rows, 256, 0, as_stream(s)>>>(w, cols, values, scales);
    return check_launch("quantize_rs_i8");
}
int kmll_dequant_rs_i8(kmll_stream_t s, const int8_t* values, const float* scales, int rows, int cols, float* out) {
    KMLL_REQUIRE_PTR(values); KMLL_REQUIRE_PTR(scales); KMLL_REQUIRE_PTR(out);
    KMLL_REQUIRE(rows > 0 && cols > 0, "dequant_rs_i8: shape [%d, %d] must be positive", rows, cols);
    const size_t n = (size_t)rows * cols;
    dequant_rs_i8_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(s)>>>(values, scales, rows, cols, out);
    return check_launch("dequant_rs_i8");
}
int kmll_quantize_w4g128(kmll_stream_t s, const float* w, int rows, int cols, uint8_t* packed, uint16_t* gscales) {
    KMLL_REQUIRE_PTR(w); KMLL_REQUIRE_PTR(packed); KMLL_REQUIRE_PTR(gscales);
    KMLL_REQUIRE(rows > 0 && cols > 0 && cols % 128 == 0, "quantize_w4g128: cols %d must be a positive multiple of 128", cols);
    KMLL_REQUIRE((reinterpret_cast<uintptr_t>(w) & 15u) == 0, "quantize_w4g128: source must be 16-byte aligned");
    const size_t n_groups = (size_t)rows * (cols / 128);
    quantize_w4_kernel<<<(unsigned)((n_groups + 7) / 8), 256, 0, as_stream(s)>>>(w, n_groups, packed, gscales);
    return check_launch("quantize_w4g128");
}
int kmll_dequant_w4g128(kmll_stream_t s, const uint8_t* packed, const uint16_t* gscales, int rows, int cols, float* out) {
    KMLL_REQUIRE_PTR(packed); KMLL_REQUIRE_PTR(gscales); KMLL_REQUIRE_PTR(out);
    KMLL_REQUIRE(rows > 0 && cols > 0 && cols % 128 == 0, "dequant_w4g128: cols %d must be a positive multiple of 128", cols);
    const size_t n = (size_t)rows * cols;
    dequant_w4_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(s)>>>(packed, gscales, n, out);
    return check_launch("dequant_w4g128");
}
int kmll_f32_to_bf16(kmll_stream_t s, const float* src, size_t n, uint16_t* dst) {
    KMLL_REQUIRE_PTR(src); KMLL_REQUIRE_PTR(dst);
    if (n == 0) return KMLL_OK;
    f32_to_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(s)>>>(src, n, dst);
    return check_launch("f32_to_bf16");
}
int kmll_fill_normal_f32(kmll_stream_t s, float* dst, size_t n, uint64_t seed, float stddev) {
    KMLL_REQUIRE_PTR(dst);
    if (n == 0) return KMLL_OK;
    fill_normal_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(s)>>>(dst, n, seed, stddev);
    return check_launch("fill_normal_f32");
}

}  // extern "C"
