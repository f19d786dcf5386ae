// Weight preparation and the small element-wise kernels around the GEMMs: the group quantiser (bit for bit the reference's),
// the scale preparation of the int8 tensor-core multiply, the gate/up row interleave and the 16-bit conversions.
#include "gemm.hpp"

#include <cstdint>
#include <stdexcept>
#include <string>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace sepal::b200 {

void count_launch();

namespace {

// The group quantiser as a streaming pass sized for the memory system rather than for the arithmetic: a persistent grid walks the
// (row, group) items; sixteen lanes share an item, each holding eight of its 128 values (two 16-byte loads, one 8-byte store),
// so a warp has two items in flight and every load instruction of the warp covers whole 128-byte lines. What must match the
// reference's kernel bit for bit (runner/cuda/src/gemm_simt_kernels.cu:267-286) is the arithmetic, not the thread layout: the group's
// largest magnitude (a maximum is the same in any order), scale = max / 127 and q = rint(w / scale) clamped to [-127, 127], both
// divisions IEEE round-to-nearest, and an all-zero group giving scale 0 and zeros.
__device__ __forceinline__ unsigned quantized_byte(float w, float scale) {
    const float r = fminf(fmaxf(rintf(__fdiv_rn(w, scale)), -127.0f), 127.0f);
    return static_cast<unsigned>(static_cast<int>(r)) & 0xFFu;
}

__global__ void __launch_bounds__(256) quantize_group_s8_kernel(const float* src, std::size_t ld_src, std::int8_t* q, std::size_t ld_q, float* s,
                                                                std::size_t ld_s, std::size_t rows, std::size_t groups) {
    const unsigned part = threadIdx.x % 16;                      // which eight values of the item
    const std::size_t half_warps = static_cast<std::size_t>(gridDim.x) * (blockDim.x / 16);
    const std::size_t items = rows * groups;
    // every lane of a warp runs the same number of rounds (the shuffles below need all 32 lanes); lanes without an item idle through them
    const std::size_t first = (static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x) / 16;
    const std::size_t rounds = (items + half_warps - 1) / half_warps;
    for (std::size_t r = 0; r < rounds; ++r) {
        const std::size_t item = first + r * half_warps;
        const bool live = item < items;
        const std::size_t row = live ? item / groups : 0, g = live ? item % groups : 0;
        float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        if (live) {
            const float4* from = reinterpret_cast<const float4*>(src + row * ld_src + g * kGroup + part * 8);
            const float4 lo = from[0], hi = from[1];
            v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w, v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
        }
        float top = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) top = fmaxf(top, fabsf(v[i]));
        for (int o = 8; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));  // over the item's sixteen lanes
        if (!live) continue;
        const float scale = __fdiv_rn(top, 127.0f);
        uint2 bytes = make_uint2(0u, 0u);
        if (scale > 0.0f) {
            bytes.x = quantized_byte(v[0], scale) | (quantized_byte(v[1], scale) << 8) | (quantized_byte(v[2], scale) << 16) | (quantized_byte(v[3], scale) << 24);
            bytes.y = quantized_byte(v[4], scale) | (quantized_byte(v[5], scale) << 8) | (quantized_byte(v[6], scale) << 16) | (quantized_byte(v[7], scale) << 24);
        }
        *reinterpret_cast<uint2*>(q + row * ld_q + g * kGroup + part * 8) = bytes;
        if (part == 0) s[row * ld_s + g] = scale;
    }
}

// One block per row of a binary16 weight matrix: the row's largest magnitude (a maximum does not depend on the order it is taken in),
// then every element on its own. Same arithmetic as the reference (runner/cuda/src/gemm_s8_kernels.cu:28-31,83-118): inv = 127 / max
// (IEEE division), q = round-to-nearest-even of w * inv clamped to [-127, 127], scale = max / 127.
__global__ void quantize_rows_s8_kernel(const __half* w, std::size_t ld_w, std::int8_t* q, std::size_t ld_q, float* scales, std::size_t k,
                                        const float* col_scale) {
    __shared__ float warp_max[8];
    const std::size_t row = blockIdx.x;
    const __half* wr = w + row * ld_w;
    const auto value = [&](std::size_t c) {
        const float v = __half2float(wr[c]);
        return col_scale != nullptr ? __fmul_rn(v, col_scale[c]) : v;
    };
    float amax = 0.0f;
    for (std::size_t c = threadIdx.x; c < k; c += blockDim.x) amax = fmaxf(amax, fabsf(value(c)));
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if (threadIdx.x % 32 == 0) warp_max[threadIdx.x / 32] = amax;
    __syncthreads();
    amax = warp_max[0];
    for (unsigned i = 1; i < blockDim.x / 32; ++i) amax = fmaxf(amax, warp_max[i]);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    if (threadIdx.x == 0) scales[row] = __fdiv_rn(amax, 127.0f);
    for (std::size_t c = threadIdx.x; c < k; c += blockDim.x) {
        const int r = __float2int_rn(__fmul_rn(value(c), inv));
        q[row * ld_q + c] = static_cast<std::int8_t>(min(127, max(-127, r)));
    }
}

// Largest scale of the matrix, as the bit pattern of a non-negative float (which orders like an unsigned integer).
__global__ void scale_max_kernel(const float* s, std::size_t ld_s, std::size_t n, std::size_t groups, unsigned* max_bits) {
    const std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    float v = 0.0f;
    if (i < n * groups) v = fabsf(s[(i / groups) * ld_s + i % groups]);
    if (!(v == v) || v > 3.0e38f) v = 0.0f;  // a NaN or infinite scale does not choose the exponent
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    if (threadIdx.x % 32 == 0 && v > 0.0f) atomicMax(max_bits, __float_as_uint(v));
}

// scales_t[g][n] = binary16(s[n][g] * 2^e) with 2^e bringing the largest scale into [128, 256); *descale = 2^-e.
__global__ void prepare_scales_kernel(const float* s, std::size_t ld_s, std::size_t n, std::size_t groups, __half* scales_t, std::size_t ld_st,
                                      float* descale, const unsigned* max_bits) {
    const float largest = __uint_as_float(*max_bits);
    int e = 0;
    if (largest > 0.0f) {
        int ex = 0;
        (void)frexpf(largest, &ex);  // largest = m * 2^ex, m in [0.5, 1)
        e = 8 - ex;
        e = max(-120, min(120, e));
    }
    const std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i == 0) *descale = ldexpf(1.0f, -e);
    if (i >= n * groups) return;
    const std::size_t g = i / n, col = i % n;  // consecutive threads write consecutive columns of one group
    scales_t[g * ld_st + col] = __float2half_rn(ldexpf(s[col * ld_s + g], e));
}

__global__ void pack_gate_up_kernel(const uint4* src, std::size_t src_stride, uint4* dst, std::size_t dst_stride, std::size_t inter, std::size_t row_vecs) {
    const std::size_t p = blockIdx.x;  // packed row
    const std::size_t b = p / 128, r = p % 128;  // pack_gate_up_source, spelled out for the device
    const std::size_t from = r < 64 ? 64 * b + r : inter + 64 * b + (r - 64);
    for (std::size_t v = threadIdx.x; v < row_vecs; v += blockDim.x) dst[p * dst_stride + v] = src[from * src_stride + v];
}

__global__ void float_to_half_kernel(const float* src, __half* dst, std::size_t count) {
    const std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) dst[i] = __float2half_rn(src[i]);
}
__global__ void half_to_float_kernel(const __half* src, float* dst, std::size_t count) {
    const std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) dst[i] = __half2float(src[i]);
}

unsigned blocks_for(std::size_t threads, unsigned per_block) {
    const std::size_t b = (threads + per_block - 1) / per_block;
    if (b > 0x7FFFFFFFu) throw std::invalid_argument("sepal_b200: too many elements for one launch");
    return static_cast<unsigned>(b);
}

}  // namespace

void launch_quantize_group_s8(const float* src, std::size_t ld_src, std::int8_t* q, std::size_t ld_q, float* s, std::size_t ld_s, std::size_t rows,
                              std::size_t k, cudaStream_t stream) {
    if (k % kGroup != 0 || ld_src % 4 != 0 || ld_q % 8 != 0 || ld_src < k || ld_q < k || ld_s < k / kGroup)
        throw std::invalid_argument("launch_quantize_group_s8: K must be a multiple of 128, the stride of the source a multiple of 4 and of q a multiple of 8, and the strides must hold a row");
    const std::size_t groups = k / kGroup;
    if (rows * groups == 0) return;
    if (src == nullptr || q == nullptr || s == nullptr) throw std::invalid_argument("launch_quantize_group_s8: null pointer");
    if (reinterpret_cast<std::uintptr_t>(src) % 16 != 0 || reinterpret_cast<std::uintptr_t>(q) % 8 != 0)
        throw std::invalid_argument("launch_quantize_group_s8: the source must be 16-byte aligned and q 8-byte aligned");
    // a persistent grid: enough 256-thread blocks to fill the SMs a few times over, never more than there are items
    const std::size_t want = (rows * groups + 15) / 16;
    const unsigned blocks = static_cast<unsigned>(want < 148 * 8 ? want : 148 * 8);
    quantize_group_s8_kernel<<<blocks, 256, 0, stream>>>(src, ld_src, q, ld_q, s, ld_s, rows, groups);
    check(cudaGetLastError(), "quantize_group_s8_kernel launch");
    count_launch();
}

void launch_quantize_rows_s8(const void* w, std::size_t ld_w, std::int8_t* q, std::size_t ld_q, float* scales, std::size_t n, std::size_t k,
                             const float* col_scale, cudaStream_t stream) {
    if (k % 16 != 0 || ld_w % 16 != 0 || ld_q % 16 != 0 || ld_w < k || ld_q < k)
        throw std::invalid_argument("launch_quantize_rows_s8: K and the strides must be multiples of 16, and the strides must hold a row");
    if (n * k == 0) return;
    if (w == nullptr || q == nullptr || scales == nullptr) throw std::invalid_argument("launch_quantize_rows_s8: null pointer");
    if (n > 0x7FFFFFFFu) throw std::invalid_argument("launch_quantize_rows_s8: too many rows for one launch");
    quantize_rows_s8_kernel<<<static_cast<unsigned>(n), 256, 0, stream>>>(static_cast<const __half*>(w), ld_w, q, ld_q, scales, k, col_scale);
    check(cudaGetLastError(), "quantize_rows_s8_kernel launch");
    count_launch();
}

void launch_prepare_w8g_scales(const float* s, std::size_t ld_s, std::size_t n, std::size_t groups, void* scales_t, std::size_t ld_st, float* descale,
                               unsigned* max_bits, cudaStream_t stream) {
    if (ld_s < groups || ld_st < n) throw std::invalid_argument("launch_prepare_w8g_scales: a stride is shorter than its row");
    if (n * groups == 0) return;
    if (s == nullptr || scales_t == nullptr || descale == nullptr || max_bits == nullptr) throw std::invalid_argument("launch_prepare_w8g_scales: null pointer");
    check(cudaMemsetAsync(max_bits, 0, sizeof(unsigned), stream), "cudaMemsetAsync");
    scale_max_kernel<<<blocks_for(n * groups, 256), 256, 0, stream>>>(s, ld_s, n, groups, max_bits);
    check(cudaGetLastError(), "scale_max_kernel launch");
    count_launch();
    prepare_scales_kernel<<<blocks_for(n * groups, 256), 256, 0, stream>>>(s, ld_s, n, groups, static_cast<__half*>(scales_t), ld_st, descale, max_bits);
    check(cudaGetLastError(), "prepare_scales_kernel launch");
    count_launch();
}

void launch_pack_gate_up(const void* src, std::size_t src_stride_bytes, void* dst, std::size_t dst_stride_bytes, std::size_t inter, std::size_t row_bytes,
                         cudaStream_t stream) {
    if (inter % 64 != 0 || row_bytes % 16 != 0 || src_stride_bytes % 16 != 0 || dst_stride_bytes % 16 != 0 || src_stride_bytes < row_bytes ||
        dst_stride_bytes < row_bytes)
        throw std::invalid_argument("launch_pack_gate_up: the intermediate size must be a multiple of 64 and rows and strides multiples of 16 bytes");
    if (inter == 0 || row_bytes == 0) return;
    if (reinterpret_cast<std::uintptr_t>(src) % 16 != 0 || reinterpret_cast<std::uintptr_t>(dst) % 16 != 0)
        throw std::invalid_argument("launch_pack_gate_up: pointers must be 16-byte aligned");
    pack_gate_up_kernel<<<static_cast<unsigned>(2 * inter), 256, 0, stream>>>(static_cast<const uint4*>(src), src_stride_bytes / 16, static_cast<uint4*>(dst),
                                                                               dst_stride_bytes / 16, inter, row_bytes / 16);
    check(cudaGetLastError(), "pack_gate_up_kernel launch");
    count_launch();
}

void launch_float_to_half(const float* src, void* dst, std::size_t count, cudaStream_t stream) {
    if (count == 0) return;
    float_to_half_kernel<<<blocks_for(count, 256), 256, 0, stream>>>(src, static_cast<__half*>(dst), count);
    check(cudaGetLastError(), "float_to_half_kernel launch");
    count_launch();
}
void launch_half_to_float(const void* src, float* dst, std::size_t count, cudaStream_t stream) {
    if (count == 0) return;
    half_to_float_kernel<<<blocks_for(count, 256), 256, 0, stream>>>(static_cast<const __half*>(src), dst, count);
    check(cudaGetLastError(), "half_to_float_kernel launch");
    count_launch();
}

}  // namespace sepal::b200
