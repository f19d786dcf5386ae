// TEST INFRASTRUCTURE, not product code.
//
// A thin extern "C" face over the reference's own GPU multiplies, so that the GPU parity tests can use them as a second
// oracle ("the reference's own implementation of the same GEMMs on identical seeded inputs") and the benchmark can time
// them on the same box as the kernels of this repository. This file holds no arithmetic of its own: oracle/Makefile
// compiles the reference's kernel sources where they lie (runner/cuda/src/gemm_kernels.cu, gemm_s8_kernels.cu,
// gemm_simt_kernels.cu) for sm_100 into oracle/_ref/libsepal_ref_gpu.so together with this file; the cuBLAS call below
// is written as the reference writes its own (runner/cuda/src/cuda_gemm.cpp:212-233, runner/cuda/src/cuda_engine.cpp:1138-1150).
// Nothing of the reference is copied into this repository, and the product library never links or loads this one.
//
// Reference interfaces bound here:
//   launch_gemm_nt                 runner/cuda/src/gemm_kernels.hpp:22-31
//   launch_gemm_w8a16              runner/cuda/src/gemm_s8_kernels.hpp:51-57
//   launch_quantize_weights_s8     runner/cuda/src/gemm_s8_kernels.hpp:29-34
//   launch_gemm_simt               runner/cuda/src/gemm_simt_kernels.hpp:55-56
//   launch_quantize_group_s8       runner/cuda/src/gemm_simt_kernels.hpp:63-64
//   cublasGemmEx (COMPUTE_32F / COMPUTE_16F), as the engine's default multiply calls it
//
// Every pointer is a DEVICE pointer; `stream` is a cudaStream_t. A call returns 0, or non-zero with the message in
// ref_gpu_last_error().
#include <cstddef>
#include <cstdint>
#include <exception>
#include <stdexcept>
#include <string>

#include <cublas_v2.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "gemm_kernels.hpp"
#include "gemm_s8_kernels.hpp"
#include "gemm_simt_kernels.hpp"

namespace {

thread_local std::string g_error;

template <class F>
int guarded(F&& f) {
    try {
        f();
        g_error.clear();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
    } catch (...) {
        g_error = "unknown exception";
    }
    return 1;
}

cublasHandle_t g_blas = nullptr;  // one per process; the tests and the benchmark use one device

void need(cublasStatus_t s, const char* call) {
    if (s != CUBLAS_STATUS_SUCCESS) throw std::runtime_error(std::string(call) + " failed with cuBLAS status " + std::to_string(static_cast<int>(s)));
}

}  // namespace

extern "C" {

__attribute__((visibility("default"))) const char* ref_gpu_last_error() { return g_error.c_str(); }

/// launch_gemm_nt: accumulate 0 = Float32, 1 = Float16Flush with `flush_k`.
__attribute__((visibility("default"))) int ref_gpu_gemm_nt(const void* x, size_t ld_x, const void* w, size_t ld_w, void* y, size_t ld_y, int y_half,
                                                            size_t t, size_t n, size_t k, int accumulate, unsigned flush_k, int config, void* stream) {
    return guarded([&] {
        sepal::cuda::launch_gemm_nt(x, ld_x, w, ld_w, y, ld_y, y_half != 0, t, n, k,
                                    accumulate == 0 ? sepal::cuda::GemmAccumulate::Float32 : sepal::cuda::GemmAccumulate::Float16Flush, flush_k, config,
                                    static_cast<cudaStream_t>(stream));
    });
}

/// launch_quantize_weights_s8: layout 0 = Plain, 1 = Fp16Pairs.
__attribute__((visibility("default"))) int ref_gpu_quantize_weights_s8(const void* w, size_t ld_w, void* wq, float* scales, size_t n, size_t k, int layout,
                                                                       void* stream) {
    return guarded([&] {
        sepal::cuda::launch_quantize_weights_s8(w, ld_w, wq, scales, n, k,
                                                layout == 0 ? sepal::cuda::S8WeightLayout::Plain : sepal::cuda::S8WeightLayout::Fp16Pairs,
                                                static_cast<cudaStream_t>(stream), nullptr);
    });
}

/// launch_gemm_w8a16 (wq in the Fp16Pairs layout, as launch_quantize_weights_s8 leaves it).
__attribute__((visibility("default"))) int ref_gpu_gemm_w8a16(const void* x, size_t ld_x, const void* wq, size_t ld_w, const float* sw, void* y, size_t ld_y,
                                                              int y_half, size_t t, size_t n, size_t k, int config, void* stream) {
    return guarded([&] { sepal::cuda::launch_gemm_w8a16(x, ld_x, wq, ld_w, sw, y, ld_y, y_half != 0, t, n, k, config, static_cast<cudaStream_t>(stream)); });
}

/// launch_gemm_simt: type 0 = F32, 1 = BF16, 2 = Int8Group; epilogue 0 = Store, 1 = Add, 2 = SwiGLU. X and Y are float32.
__attribute__((visibility("default"))) int ref_gpu_gemm_simt(const float* x, size_t ld_x, const void* w, size_t ld_w, const float* scales, size_t ld_s, int type,
                                                             float* y, size_t ld_y, size_t t, size_t n, size_t k, int epilogue, int config, void* stream) {
    return guarded([&] {
        sepal::cuda::SimtMatrix m;
        m.w = w;
        m.ld_w = ld_w;
        m.scales = scales;
        m.ld_s = ld_s;
        m.type = static_cast<sepal::cuda::SimtWeight>(type);
        sepal::cuda::launch_gemm_simt(x, ld_x, m, y, ld_y, t, n, k, static_cast<sepal::cuda::SimtEpilogue>(epilogue), config, static_cast<cudaStream_t>(stream));
    });
}

__attribute__((visibility("default"))) int ref_gpu_quantize_group_s8(const float* src, size_t ld_src, int8_t* q, size_t ld_q, float* s, size_t ld_s, size_t rows,
                                                                     size_t k, void* stream) {
    return guarded([&] { sepal::cuda::launch_quantize_group_s8(src, ld_src, q, ld_q, s, ld_s, rows, k, static_cast<cudaStream_t>(stream)); });
}

/// Y [t, n] (row stride ld_y; binary16 when y_half, else float32) = X [t, k] (binary16, stride ld_x) W [n, k]^T (binary16, dense) through
/// cublasGemmEx as the reference's engine calls it: Y^T (n x t) = op_T(W) X^T, CUBLAS_COMPUTE_32F, or CUBLAS_COMPUTE_16F with a
/// binary16 result when compute16 (then y_half must be set, as the engine's half_acc path writes binary16).
__attribute__((visibility("default"))) int ref_gpu_cublas_gemm(const void* x, size_t ld_x, const void* w, void* y, size_t ld_y, int y_half, size_t t, size_t n,
                                                               size_t k, int compute16, void* stream) {
    return guarded([&] {
        if (g_blas == nullptr) need(cublasCreate(&g_blas), "cublasCreate");
        need(cublasSetStream(g_blas, static_cast<cudaStream_t>(stream)), "cublasSetStream");
        const int m_ = static_cast<int>(n), t_ = static_cast<int>(t), k_ = static_cast<int>(k);
        if (compute16 != 0) {
            if (y_half == 0) throw std::invalid_argument("ref_gpu_cublas_gemm: COMPUTE_16F writes binary16");
            const __half alpha = __float2half(1.0f), beta = __float2half(0.0f);
            need(cublasGemmEx(g_blas, CUBLAS_OP_T, CUBLAS_OP_N, m_, t_, k_, &alpha, w, CUDA_R_16F, k_, x, CUDA_R_16F, static_cast<int>(ld_x), &beta, y,
                              CUDA_R_16F, static_cast<int>(ld_y), CUBLAS_COMPUTE_16F, CUBLAS_GEMM_DEFAULT),
                 "cublasGemmEx");
        } else {
            const float alpha = 1.0f, beta = 0.0f;
            need(cublasGemmEx(g_blas, CUBLAS_OP_T, CUBLAS_OP_N, m_, t_, k_, &alpha, w, CUDA_R_16F, k_, x, CUDA_R_16F, static_cast<int>(ld_x), &beta, y,
                              y_half != 0 ? CUDA_R_16F : CUDA_R_32F, static_cast<int>(ld_y), CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT),
                 "cublasGemmEx");
        }
    });
}

}  // extern "C"
