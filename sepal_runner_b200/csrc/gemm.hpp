// Launchers of the trunk projection GEMMs for sm_100a, with the conventions of the reference's own launchers
// (runner/cuda/src/device.hpp:26-29): a launcher enqueues on the stream it is given and returns without waiting, throws
// std::invalid_argument for a violated requirement and std::runtime_error when the launch fails. There is no CPU or library
// fallback: a device that is not sm_100 is refused when the Context is created.
//
//   Y[t, n] = epilogue( sum over k of X[t, k] * W[n, k] )        X [T, K], W [N, K], both K-contiguous ("NT")
//
// launch_gemm_f16 stands where the reference calls launch_gemm_nt (runner/cuda/src/gemm_kernels.hpp:22-31) or cublasGemmEx
// (runner/cuda/src/cuda_engine.cpp:1138-1150); launch_gemm_w8g stands where it calls launch_gemm_simt with SimtWeight::Int8Group
// (runner/cuda/src/gemm_simt_kernels.hpp:42-56), with binary16 activations instead of float32 ones. The epilogues are the
// reference's SimtEpilogue (runner/cuda/src/gemm_simt_kernels.hpp:19-25).
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_runtime.h>

#include "context.hpp"

namespace sepal::b200 {

/// What happens to the finished sums (same numbering as the reference's SimtEpilogue).
enum class Epilogue : int {
    Store = 0,   // Y[t, n] = acc
    Add = 1,     // Y[t, n] = Y[t, n] + acc: the residual stream updated in place, one addition in float32
    SwiGLU = 2,  // W rows are gate and up interleaved in blocks of 64 (pack_gate_up_source); N is the packed width 2 I and Y has
                 // I columns: Y[t, 64 b + r] = silu(acc[128 b + r]) * acc[128 b + 64 + r]
};

inline constexpr std::size_t kGroup = 128;  // values of k per int8 scale (the reference's kSimtGroup)

/// Schedules, for tests and benchmarks (`config`). Every schedule gives results within float32 rounding of one another; bits are
/// fixed for a given shape, schedule and SM count.
///   -1  picks the tile width from the shape so that the tiles fill whole waves of the SMs; whole tiles dealt round-robin; CTA pairs
///       (tcgen05.mma.cta_group::2: 256 x w tiles, each CTA loads its 128 rows of X and half of the W tile) for more than 128 rows
///   0   128 x 256 tiles, whole tiles dealt round-robin to the persistent CTAs
///   1   128 x 256 tiles, all k iterations of all tiles split evenly over the CTAs (partial tiles summed in k order by the last arriver)
///   2   128 x 128 tiles, whole tiles
///   3   128 x 128 tiles, even split
///   w, w + 1 (w a multiple of 16 in [16, 256]): 128 x w tiles, whole tiles / even split. SwiGLU and int8 weights take w = 128 or 256.
///   w + 2, w + 3, w + 6: 256 x w tiles on CTA pairs: whole tiles / even split / whole tiles first and the last waves split.
///   512 + w (int8 weights, w a multiple of 32 in [64, 192], or 256 or 320): the swapped kernel. The weights are the tensor cores' first
///       operand, widened and scaled into tensor memory, the tokens the second, w of them to a tile of 256 weight rows (256 and 320: two
///       blocks of 128 and 160 that share the converted weights); whole tiles. -1 picks it, and w, by an estimate of both families
///       (pick_w8t_tokens in gemm_tc.cu).
inline constexpr int kConfigs = 4;

/// Row of the stacked [gate; up] matrix that packed row p holds (the reference's pack_gate_up_source,
/// runner/cuda/src/gemm_simt_kernels.hpp:72-77).
constexpr std::size_t pack_gate_up_source(std::size_t p, std::size_t inter) noexcept {
    const std::size_t b = p / 128, r = p % 128;
    return r < 64 ? 64 * b + r : inter + 64 * b + (r - 64);
}

/// Whether launch_gemm_f16 takes these dimensions and strides (pointer alignment, 16 bytes, is the caller's): K and the strides of X
/// and W multiples of 8 (the reference's gemm_nt_supports), N and the stride of Y even; SwiGLU needs N a multiple of 128.
constexpr bool gemm_f16_supports(std::size_t n, std::size_t k, std::size_t ld_x, std::size_t ld_w, std::size_t ld_y, Epilogue e) noexcept {
    if (k == 0 || n == 0 || k % 8 != 0 || ld_x % 8 != 0 || ld_w % 8 != 0 || ld_x < k || ld_w < k || n % 2 != 0 || ld_y % 2 != 0) return false;
    if (e == Epilogue::SwiGLU) return n % 128 == 0 && ld_y >= n / 2;
    return ld_y >= n;
}

/// Whether launch_gemm_w8g takes these: K a multiple of 128 (one scale per group), ld_x a multiple of 8, ld_q a multiple of 16 bytes.
constexpr bool gemm_w8g_supports(std::size_t n, std::size_t k, std::size_t ld_x, std::size_t ld_q, std::size_t ld_s, std::size_t ld_y,
                                 Epilogue e) noexcept {
    if (k == 0 || n == 0 || k % kGroup != 0 || ld_x % 8 != 0 || ld_q % 16 != 0 || ld_x < k || ld_q < k || ld_s < k / kGroup || n % 2 != 0 ||
        ld_y % 2 != 0)
        return false;
    if (e == Epilogue::SwiGLU) return n % 128 == 0 && ld_y >= n / 2;
    return ld_y >= n;
}

/// X [T, K] and W [N, K] binary16 (row strides ld_x, ld_w, 16-byte aligned), float32 accumulation on the tensor cores (tcgen05.mma),
/// Y row-major with stride ld_y, binary16 when y_half and float32 otherwise.
void launch_gemm_f16(Context& ctx, const void* x, std::size_t ld_x, const void* w, std::size_t ld_w, void* y, std::size_t ld_y, bool y_half,
                     std::size_t t, std::size_t n, std::size_t k, Epilogue epilogue, int config, cudaStream_t stream);

/// launch_gemm_f16 for callers that may not allocate device memory (see include/sepal_b200.h, sepal_b200_gemm_f16_noalloc): no
/// Context; the split-k scratch is a fixed array inside the library. Runs on the current device. With `status_out` the call waits for
/// the stream and stores the kernel status word there (0 = fine).
void launch_gemm_f16_noalloc(const void* x, std::size_t ld_x, const void* w, std::size_t ld_w, void* y, std::size_t ld_y, bool y_half, std::size_t t,
                             std::size_t n, std::size_t k, Epilogue epilogue, cudaStream_t stream, int* status_out);

/// An int8 weight matrix as the tensor-core multiply reads it (the counterpart of the reference's SimtMatrix with
/// SimtWeight::Int8Group, runner/cuda/src/gemm_simt_kernels.hpp:42-51). q is the reference's layout unchanged. The scales are
/// "prepared" once at weight placement by launch_prepare_w8g_scales: transposed to group-major order, multiplied by a power of two
/// that brings the largest one into [128, 256) and rounded to binary16, so that float32(q) * s fits binary16 whatever the
/// magnitude of the weights; `descale` is the device scalar (the inverse power of two) the finished sums are multiplied by.
struct W8gMatrix {
    const std::int8_t* q = nullptr;  // [N, ld_q] bytes
    std::size_t ld_q = 0;
    const void* scales_t = nullptr;  // binary16 [K / 128, ld_st], 16-byte aligned, ld_st >= N rounded up to 256 (padding zero)
    std::size_t ld_st = 0;
    const float* descale = nullptr;  // device pointer to one float
    const float* col_scale = nullptr;  // float32 [N] multiplying the finished sums column by column (null: none); see launch_gemm_w8r
};

/// X [T, K] binary16; W int8 with one scale per row and group of 128 values of k. Each group is dequantised (q widened exactly to
/// binary16, one binary16 multiplication by the prepared scale) in shared memory on its way to the tensor cores; float32 accumulation.
void launch_gemm_w8g(Context& ctx, const void* x, std::size_t ld_x, const W8gMatrix& w, void* y, std::size_t ld_y, bool y_half, std::size_t t,
                     std::size_t n, std::size_t k, Epilogue epilogue, int config, cudaStream_t stream);

/// Which kernel the automatic schedule (`config` -1) of launch_gemm_w8g gives a [t x k] by [n x k] multiply on a device of `sm_count`
/// SMs: the tokens to a tile of the swapped kernel (96 to 192: one block; 256 or 320: two blocks of half as many), or 0 for the
/// unswapped kernels. `staged`: the result leaves through shared memory and the TMA (16-byte aligned rows; every result but a float32
/// SwiGLU and a binary16 residual update); `epilogue`: the SwiGLU's epilogue costs more, and a staged residual update with CTA pairs to
/// spare has them share the tiles. Host arithmetic only.
unsigned w8g_swapped_tokens(unsigned sm_count, std::size_t t, std::size_t n, std::size_t k, bool staged, Epilogue epilogue);

/// s [N, K / 128] float32 (row stride ld_s: the quantiser's and the reference's layout) -> scales_t binary16 [K / 128, ld_st] and
/// *descale, as W8gMatrix describes. `max_bits` is a device word of scratch (4 bytes). Enqueued on `stream`; no host synchronisation.
/// X [T, K] binary16; W int8 with ONE float32 scale per output row (the counterpart of the reference's launch_gemm_w8a16,
/// runner/cuda/src/gemm_s8_kernels.hpp:51-57, with the bytes in plain row-major order): Y[t, n] = sw[n] * sum_k x[t, k] * q[n, k]. The
/// bytes are widened exactly to binary16 on their way to the tensor cores, the sums are float32, and the scale multiplies the finished
/// sum in float32, as in the reference. K must be a multiple of 128 here and N at most 65536. The epilogues are those of launch_gemm_w8g.
void launch_gemm_w8r(Context& ctx, const void* x, std::size_t ld_x, const std::int8_t* q, std::size_t ld_q, const float* sw, void* y, std::size_t ld_y,
                     bool y_half, std::size_t t, std::size_t n, std::size_t k, Epilogue epilogue, int config, cudaStream_t stream);

/// Per-output-row symmetric int8 quantisation of a binary16 weight matrix, bit for bit the reference's launch_quantize_weights_s8 with
/// the Plain layout (runner/cuda/src/gemm_s8_kernels.cu:83-118): scales[r] = max|w[r, :]| / 127, q[r, c] = rint(w[r, c] * (127 / max))
/// clamped to [-127, 127]; a zero row gets scale 0 and zeros. `col_scale` (null or K floats): w[r, c] is multiplied by col_scale[c] in
/// float32 first. K a multiple of 16 and the strides multiples of 16 that hold a row.
void launch_quantize_rows_s8(const void* w, std::size_t ld_w, std::int8_t* q, std::size_t ld_q, float* scales, std::size_t n, std::size_t k,
                             const float* col_scale, cudaStream_t stream);

void launch_prepare_w8g_scales(const float* s, std::size_t ld_s, std::size_t n, std::size_t groups, void* scales_t, std::size_t ld_st,
                               float* descale, unsigned* max_bits, cudaStream_t stream);

/// The group quantiser, bit for bit the reference's (runner/cuda/src/gemm_simt_kernels.cu:267-286): s = max|w| / 127 per row and group of
/// 128, q = rint(w / s) clamped to [-127, 127]; an all-zero group gets s = 0, q = 0. src float32 [rows, K] (stride ld_src).
void launch_quantize_group_s8(const float* src, std::size_t ld_src, std::int8_t* q, std::size_t ld_q, float* s, std::size_t ld_s,
                              std::size_t rows, std::size_t k, cudaStream_t stream);

/// dst[p, :] = src[pack_gate_up_source(p, inter), :] for the 2 * inter rows of a stacked [gate; up] matrix: the row order the fused
/// SwiGLU multiply wants. Rows are `row_bytes` long (16-byte multiples), strides in bytes.
void launch_pack_gate_up(const void* src, std::size_t src_stride_bytes, void* dst, std::size_t dst_stride_bytes, std::size_t inter,
                         std::size_t row_bytes, cudaStream_t stream);

/// float32 -> binary16, round to nearest even (weights are rounded once at load, runner/include/sepal/trained_model.hpp:8-9).
void launch_float_to_half(const float* src, void* dst, std::size_t count, cudaStream_t stream);
void launch_half_to_float(const void* src, float* dst, std::size_t count, cudaStream_t stream);

/// How many kernels of this library the calling thread has launched since the last call (benchmarks report it).
std::uint64_t take_launch_count();

}  // namespace sepal::b200
