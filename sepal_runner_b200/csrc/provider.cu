#include "provider.hpp"

#include <initializer_list>
#include <stdexcept>
#include <string>

#include <cuda_fp16.h>

namespace sepal::b200 {

void count_launch();

namespace {

constexpr std::size_t kAlign = 1024;
std::size_t round_up(std::size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

__global__ void scale_rows_kernel(float* y, std::size_t count, float beta) {
    const std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) y[i] = __fmul_rn(beta, y[i]);
}

}  // namespace

B200Gemm::B200Gemm(int device, std::size_t arena_bytes) : ctx_(device, 0) {
    ctx_.static_weights = true;  // upload_weights returns only after its stream has finished: no multiply follows a kernel that writes its weights
    arena_bytes_ = arena_bytes != 0 ? arena_bytes : (std::size_t{1} << 30);
    check(cudaSetDevice(device), "cudaSetDevice");
    check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
    check(cudaStreamCreateWithFlags(&stream_in_, cudaStreamNonBlocking), "cudaStreamCreate");
    check(cudaStreamCreateWithFlags(&stream_out_, cudaStreamNonBlocking), "cudaStreamCreate");
    for (cudaEvent_t& e : uploaded_) check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
    for (cudaEvent_t& e : multiplied_) check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
    check(cudaMalloc(reinterpret_cast<void**>(&arena_), arena_bytes_), "cudaMalloc(arena)");
}

B200Gemm::~B200Gemm() {
    (void)cudaSetDevice(ctx_.device);
    for (cudaStream_t s : {stream_in_, stream_, stream_out_}) {
        if (s != nullptr) {
            (void)cudaStreamSynchronize(s);
            (void)cudaStreamDestroy(s);
        }
    }
    for (cudaEvent_t e : uploaded_)
        if (e != nullptr) (void)cudaEventDestroy(e);
    for (cudaEvent_t e : multiplied_)
        if (e != nullptr) (void)cudaEventDestroy(e);
    if (arena_ != nullptr) (void)cudaFree(arena_);
}

void* B200Gemm::carve(std::size_t bytes) {
    const std::size_t need = round_up(bytes);
    if (resident_ + need > arena_bytes_)
        throw std::runtime_error("sepal_b200 provider: the arena is too small by " + std::to_string(resident_ + need - arena_bytes_) + " bytes");
    void* p = arena_ + resident_;
    resident_ += need;
    return p;
}

void* B200Gemm::scratch(std::size_t bytes, std::size_t& top) {
    const std::size_t need = round_up(bytes);
    if (top < resident_ + need)
        throw std::runtime_error("sepal_b200 provider: the arena is too small for this call by " + std::to_string(resident_ + need - top) + " bytes");
    top -= need;
    return arena_ + top;
}

WeightId B200Gemm::upload_weights(const void* w, HostType type, std::size_t n, std::size_t k) {
    if (w == nullptr || n == 0 || k == 0) throw std::invalid_argument("upload_weights: empty matrix");
    if (!gemm_f16_supports(n, k, k, k, n, Epilogue::Store)) throw std::invalid_argument("upload_weights: K must be a multiple of 8 and N even");
    std::lock_guard<std::mutex> lock(mutex_);
    check(cudaSetDevice(ctx_.device), "cudaSetDevice");
    Weight wt;
    wt.n = n;
    wt.k = k;
    const std::size_t before = resident_;
    try {
        wt.data = carve(n * k * 2);
        if (type == HostType::F16) {
            check(cudaMemcpyAsync(wt.data, w, n * k * 2, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync(W)");
        } else {
            std::size_t top = arena_bytes_;
            float* tmp = static_cast<float*>(scratch(n * k * 4, top));
            check(cudaMemcpyAsync(tmp, w, n * k * 4, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync(W)");
            launch_float_to_half(tmp, wt.data, n * k, stream_);
        }
        check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    } catch (...) {
        resident_ = before;
        throw;
    }
    weights_.push_back(wt);
    return WeightId{static_cast<std::uint32_t>(weights_.size() - 1)};
}

WeightId B200Gemm::upload_weights_w8g(const float* w, std::size_t n, std::size_t k) {
    if (w == nullptr || n == 0 || k == 0) throw std::invalid_argument("upload_weights_w8g: empty matrix");
    if (k % kGroup != 0 || n % 2 != 0) throw std::invalid_argument("upload_weights_w8g: K must be a multiple of 128 and N even");
    std::lock_guard<std::mutex> lock(mutex_);
    check(cudaSetDevice(ctx_.device), "cudaSetDevice");
    Weight wt;
    wt.n = n;
    wt.k = k;
    wt.w8g = true;
    const std::size_t groups = k / kGroup;
    const std::size_t before = resident_;
    try {
        wt.data = carve(n * k);
        const std::size_t ld_st = (n + 255) / 256 * 256;
        wt.scales_t = carve(groups * ld_st * 2);
        check(cudaMemsetAsync(wt.scales_t, 0, groups * ld_st * 2, stream_), "cudaMemsetAsync(scales)");
        wt.descale = static_cast<float*>(carve(sizeof(float) + sizeof(unsigned)));
        std::size_t top = arena_bytes_;
        float* tmp = static_cast<float*>(scratch(n * k * 4, top));
        float* s = static_cast<float*>(scratch(n * groups * 4, top));
        check(cudaMemcpyAsync(tmp, w, n * k * 4, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync(W)");
        launch_quantize_group_s8(tmp, k, static_cast<std::int8_t*>(wt.data), k, s, groups, n, k, stream_);
        launch_prepare_w8g_scales(s, groups, n, groups, wt.scales_t, ld_st, wt.descale, reinterpret_cast<unsigned*>(wt.descale + 1), stream_);
        check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    } catch (...) {
        resident_ = before;
        throw;
    }
    weights_.push_back(wt);
    return WeightId{static_cast<std::uint32_t>(weights_.size() - 1)};
}

void B200Gemm::gemm_f(const void* x, HostType type, std::size_t t, WeightId id, float* y, float beta) {
    if (t == 0) {
        std::lock_guard<std::mutex> lock(mutex_);
        if (!id.valid() || id.index >= weights_.size()) throw std::invalid_argument("gemm_f: unknown weight id");
        return;
    }
    if (x == nullptr || y == nullptr) throw std::invalid_argument("gemm_f: null data pointer");
    std::lock_guard<std::mutex> lock(mutex_);
    if (!id.valid() || id.index >= weights_.size()) throw std::invalid_argument("gemm_f: unknown weight id");
    check(cudaSetDevice(ctx_.device), "cudaSetDevice");
    const Weight& w = weights_[id.index];
    std::size_t top = arena_bytes_;
    char* dx = static_cast<char*>(scratch(t * w.k * 2, top));
    float* dy = static_cast<float*>(scratch(t * w.n * 4, top));
    float* tmp = type == HostType::F16 ? nullptr : static_cast<float*>(scratch(t * w.k * 4, top));
    // The rows of a large call go through in up to kChunks pieces on three streams, so that the upload of piece i + 1, the multiply of
    // piece i and the download of piece i - 1 run at the same time (the bus carries both directions at once). The multiplies of all
    // pieces run on one stream, one after another: they share the context's split-k scratch.
    constexpr std::size_t kChunks = 4, kMinChunk = 256;
    std::size_t pieces = t / kMinChunk;
    pieces = pieces < 1 ? 1 : (pieces > kChunks ? kChunks : pieces);
    const std::size_t rows_per = ((t + pieces - 1) / pieces + 127) / 128 * 128;
    const std::size_t x_elem = type == HostType::F16 ? 2 : 4;
    std::size_t piece = 0;
    for (std::size_t r0 = 0; r0 < t; r0 += rows_per, ++piece) {
        const std::size_t rows = t - r0 < rows_per ? t - r0 : rows_per;
        const char* hx = static_cast<const char*>(x) + r0 * w.k * x_elem;
        char* dxp = dx + r0 * w.k * 2;
        float* dyp = dy + r0 * w.n;
        float* hy = y + r0 * w.n;
        if (type == HostType::F16)
            check(cudaMemcpyAsync(dxp, hx, rows * w.k * 2, cudaMemcpyHostToDevice, stream_in_), "cudaMemcpyAsync(X)");
        else
            check(cudaMemcpyAsync(tmp + r0 * w.k, hx, rows * w.k * 4, cudaMemcpyHostToDevice, stream_in_), "cudaMemcpyAsync(X)");
        if (beta != 0.0f) check(cudaMemcpyAsync(dyp, hy, rows * w.n * 4, cudaMemcpyHostToDevice, stream_in_), "cudaMemcpyAsync(Y)");
        check(cudaEventRecord(uploaded_[piece], stream_in_), "cudaEventRecord");
        check(cudaStreamWaitEvent(stream_, uploaded_[piece], 0), "cudaStreamWaitEvent");
        if (type != HostType::F16) launch_float_to_half(tmp + r0 * w.k, dxp, rows * w.k, stream_);
        Epilogue ep = Epilogue::Store;
        if (beta != 0.0f) {
            if (beta != 1.0f) {
                const std::size_t count = rows * w.n;
                scale_rows_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, stream_>>>(dyp, count, beta);
                check(cudaGetLastError(), "scale_rows_kernel launch");
                count_launch();
            }
            ep = Epilogue::Add;
        }
        if (w.w8g) {
            W8gMatrix m;
            m.q = static_cast<const std::int8_t*>(w.data);
            m.ld_q = w.k;
            m.scales_t = w.scales_t;
            m.ld_st = (w.n + 255) / 256 * 256;
            m.descale = w.descale;
            launch_gemm_w8g(ctx_, dxp, w.k, m, dyp, w.n, false, rows, w.n, w.k, ep, -1, stream_);
        } else {
            launch_gemm_f16(ctx_, dxp, w.k, w.data, w.k, dyp, w.n, false, rows, w.n, w.k, ep, -1, stream_);
        }
        check(cudaEventRecord(multiplied_[piece], stream_), "cudaEventRecord");
        check(cudaStreamWaitEvent(stream_out_, multiplied_[piece], 0), "cudaStreamWaitEvent");
        check(cudaMemcpyAsync(hy, dyp, rows * w.n * 4, cudaMemcpyDeviceToHost, stream_out_), "cudaMemcpyAsync(Y)");
    }
    // One wait for everything: the download stream is behind every multiply (it waited for each piece's event), so the status word is
    // read behind the last download.
    const int status = ctx_.read_status(stream_out_);
    if (status != 0) throw std::runtime_error("sepal_b200 provider: a kernel gave up waiting (status " + std::to_string(status) + ")");
}

}  // namespace sepal::b200
