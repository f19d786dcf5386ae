// The host-pointer face of the GEMMs: weights uploaded once, then Y = beta Y + X W^T with X uploaded and Y downloaded inside the
// call. It mirrors the reference's cuBLAS provider sepal::cuda::CudaGemm (runner/cuda/include/sepal/cuda/cuda_gemm.hpp:112-160):
// one device allocation made at creation, weights carved from its bottom, per-call temporaries from the rest, a stream of its own.
#pragma once

#include <cstddef>
#include <cstdint>
#include <mutex>
#include <vector>

#include <cuda_runtime.h>

#include "gemm.hpp"

namespace sepal::b200 {

enum class HostType : int { F32 = 0, F16 = 1 };

struct WeightId {
    std::uint32_t index = 0xFFFFFFFFu;
    constexpr bool valid() const noexcept { return index != 0xFFFFFFFFu; }
};

class B200Gemm {
public:
    B200Gemm(int device, std::size_t arena_bytes);
    ~B200Gemm();
    B200Gemm(const B200Gemm&) = delete;
    B200Gemm& operator=(const B200Gemm&) = delete;

    /// W [N, K] on the host -> binary16 on the device, kept for the provider's life.
    WeightId upload_weights(const void* w, HostType type, std::size_t n, std::size_t k);
    /// W float32 [N, K] on the host -> int8 groups + prepared scales on the device (K a multiple of 128).
    WeightId upload_weights_w8g(const float* w, std::size_t n, std::size_t k);
    /// Y [T, N] float32 (host) = beta Y + X [T, K] (host) W^T. Returns when Y is complete. Throws std::runtime_error when a kernel
    /// reported a wait that ran out. Calls of 512 rows and more are cut into up to four pieces of rows whose upload, multiply and
    /// download overlap (a piece is a product of its own, so a row's float32 sum may be rounded differently than in the uncut product).
    void gemm_f(const void* x, HostType type, std::size_t t, WeightId w, float* y, float beta);

    Context& context() { return ctx_; }
    cudaStream_t stream() const { return stream_; }

private:
    struct Weight {
        std::size_t n = 0, k = 0;
        bool w8g = false;
        void* data = nullptr;       // binary16 [N, K] or int8 [N, K]
        void* scales_t = nullptr;   // w8g: binary16 [K / 128, N]
        float* descale = nullptr;   // w8g
    };
    void* carve(std::size_t bytes);            // from the bottom: stays
    void* scratch(std::size_t bytes, std::size_t& top);  // from the top: the caller resets `top` when done

    Context ctx_;
    cudaStream_t stream_ = nullptr;                          // the multiplies (and the weight uploads)
    cudaStream_t stream_in_ = nullptr, stream_out_ = nullptr;  // a call's uploads and downloads, overlapped with its multiplies
    cudaEvent_t uploaded_[4] = {}, multiplied_[4] = {};        // one pair per piece of a call
    unsigned char* arena_ = nullptr;
    std::size_t arena_bytes_ = 0, resident_ = 0;
    std::vector<Weight> weights_;
    std::mutex mutex_;
};

}  // namespace sepal::b200
