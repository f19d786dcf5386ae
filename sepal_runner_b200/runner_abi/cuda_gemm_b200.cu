// The reference's CUDA provider class, sepal::cuda::CudaGemm, implemented over this library's kernels.
//
// The class and everything it promises are DECLARED by the reference (runner/cuda/include/sepal/cuda/cuda_gemm.hpp:112-160: one
// device allocation made at creation, weights and device matrices carved from its bottom, a call's temporaries from the rest,
// a stream of its own, CudaError naming the failing call; sepal::GemmProvider in runner/include/sepal/gemm.hpp:44-60). The
// reference defines it in runner/cuda/src/cuda_gemm.cpp on cuBLAS; this file defines the same member functions on
// sepal_b200_gemm_f16 (include/sepal_b200.h), so that code written against the reference's header -- its own conformance suite
// runner/cuda/tests/test_cuda_gemm.cpp, its reference executor, its engines -- links against this object file instead and runs
// its float16 products on the tcgen05 kernels. It is compiled only where the reference tree is present (Makefile beside it);
// nothing of the reference is copied here.
//
// Precision::F16 is the path of this library: operands are binary16 on the device (float32 and bfloat16 inputs rounded to
// nearest), float32 accumulation, float32 output. Shapes the kernels do not take directly (K not a multiple of 8, odd N) are
// zero-padded on the device. Precision::F32 is not a path of this library; so that code which also creates a float32 provider
// still runs, it is served by a plain float32 SIMT kernel below (no tensor cores, one fused multiply-add chain per output in k
// order).
#include "sepal/cuda/cuda_gemm.hpp"

#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "sepal_b200.h"

namespace sepal::cuda {

CudaError::CudaError(std::string call, long long code, const std::string& reason, const std::string& context)
    : std::runtime_error(call + " failed: " + reason + " (code " + std::to_string(code) + ")" + (context.empty() ? "" : ": " + context)),
      call_(std::move(call)), code_(code) {}

namespace {

void need(cudaError_t status, const char* call, const std::string& context = {}) {
    if (status == cudaSuccess) return;
    (void)cudaGetLastError();
    throw CudaError(call, static_cast<long long>(status), cudaGetErrorString(status), context);
}

void need_b200(int32_t rc, const char* call) {
    if (rc != 0) throw CudaError(call, rc, sepal_b200_last_error());
}

constexpr std::size_t kAlign = 256;
constexpr std::size_t round_up(std::size_t v, std::size_t to) { return (v + to - 1) / to * to; }

// dst [rows, ld_dst] (To) = src [rows, cols] (From, dense), columns cols .. ld_dst - 1 and rows rows .. rows_dst - 1 zero.
template <class From, class To>
__global__ void convert_pad_kernel(const From* src, std::size_t rows, std::size_t cols, To* dst, std::size_t rows_dst, std::size_t ld_dst) {
    const std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows_dst * ld_dst) return;
    const std::size_t r = i / ld_dst, c = i % ld_dst;
    float v = 0.0f;
    if (r < rows && c < cols) v = static_cast<float>(src[r * cols + c]);
    dst[i] = static_cast<To>(v);
}

__global__ void scale_kernel(float* y, std::size_t count, float beta) {
    const std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) y[i] = __fmul_rn(beta, y[i]);
}

// dst [rows, cols] dense = src [rows, ld_src] (the padded product without its padding).
__global__ void unpad_kernel(const float* src, std::size_t ld_src, float* dst, std::size_t rows, std::size_t cols) {
    const std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < rows * cols) dst[i] = src[(i / cols) * ld_src + i % cols];
}

// The float32 product of Precision::F32 (see the head of the file): Y[t, n] = beta Y[t, n] + sum_k X[t, k] W[n, k], one thread per output.
__global__ void product_f32_kernel(const float* x, const float* w, float* y, std::size_t t, std::size_t n, std::size_t k, float beta) {
    __shared__ float xs[16][17], ws[16][17];
    const std::size_t row = static_cast<std::size_t>(blockIdx.y) * 16 + threadIdx.y, col = static_cast<std::size_t>(blockIdx.x) * 16 + threadIdx.x;
    const std::size_t w_row = static_cast<std::size_t>(blockIdx.x) * 16 + threadIdx.y;
    float acc = 0.0f;
    for (std::size_t k0 = 0; k0 < k; k0 += 16) {
        xs[threadIdx.y][threadIdx.x] = (row < t && k0 + threadIdx.x < k) ? x[row * k + k0 + threadIdx.x] : 0.0f;
        ws[threadIdx.y][threadIdx.x] = (w_row < n && k0 + threadIdx.x < k) ? w[w_row * k + k0 + threadIdx.x] : 0.0f;
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc = __fmaf_rn(xs[threadIdx.y][j], ws[threadIdx.x][j], acc);
        __syncthreads();
    }
    if (row < t && col < n) y[row * n + col] = beta != 0.0f ? __fmaf_rn(beta, y[row * n + col], acc) : acc;
}

unsigned blocks(std::size_t count) { return static_cast<unsigned>((count + 255) / 256); }

std::string shape_text(std::size_t r, std::size_t c) { return "[" + std::to_string(r) + ", " + std::to_string(c) + "]"; }

void require_float(MatRef m, const char* what) {
    if (m.dtype == DType::I8)
        throw std::invalid_argument(std::string("gemm_f: ") + what + " has element type i8, which is not a float type");
}

void check_shapes(MatRef x, std::size_t w_rows, std::size_t w_cols, const void* w_data, MatView y) {
    if (x.cols != w_cols)
        throw std::invalid_argument("gemm_f: X " + shape_text(x.rows, x.cols) + " and W " + shape_text(w_rows, w_cols) + " disagree on K");
    if (y.rows != x.rows || y.cols != w_rows)
        throw std::invalid_argument("gemm_f: Y " + shape_text(y.rows, y.cols) + " must be " + shape_text(x.rows, w_rows));
    if ((x.data == nullptr && x.rows * x.cols != 0) || (w_data == nullptr && w_rows * w_cols != 0) || (y.data == nullptr && y.rows * y.cols != 0))
        throw std::invalid_argument("gemm_f: null data pointer");
}

}  // namespace

DeviceMemory query_device_memory(int device) {
    need(cudaSetDevice(device), "cudaSetDevice");
    DeviceMemory m;
    need(cudaMemGetInfo(&m.free_bytes, &m.total_bytes), "cudaMemGetInfo");
    return m;
}

struct CudaGemm::Impl {
    struct Weight {
        std::size_t rows = 0, cols = 0;      // N, K as the caller sees them
        std::size_t ld = 0, rows_padded = 0;  // F16: K rounded up to 8, N rounded up to 2 (zero padding); F32: cols, rows
        void* data = nullptr;
    };
    struct Registered {
        const void* host = nullptr;
        DType dtype = DType::F32;
        std::size_t rows = 0, cols = 0;
        std::uint32_t index = 0;
    };

    CudaGemmOptions options;
    DType compute = DType::F16;
    cudaStream_t stream = nullptr;
    sepal_b200_ctx* ctx = nullptr;
    char* arena = nullptr;
    std::size_t arena_bytes = 0, resident = 0, scratch = 0, scratch_peak = 0, arena_peak = 0;
    std::size_t free_at_start = 0, free_min = 0, total = 0;
    std::vector<Weight> weights;
    std::vector<Registered> registered;
    mutable std::mutex mutex;

    ~Impl() {
        if (stream == nullptr && ctx == nullptr && arena == nullptr) return;  // nothing was created (the device did not exist)
        (void)cudaSetDevice(options.device);
        if (stream != nullptr) {
            (void)cudaStreamSynchronize(stream);
            (void)cudaStreamDestroy(stream);
        }
        if (ctx != nullptr) sepal_b200_close(ctx);
        if (arena != nullptr) (void)cudaFree(arena);
        (void)cudaGetLastError();  // nothing a destructor met may surface in a later call's check
    }

    [[noreturn]] void arena_full(const char* what, std::size_t bytes) const {
        throw CudaError("arena", 0, "out of arena memory",
                        std::string(what) + " needs " + std::to_string(bytes) + " bytes, " + std::to_string(arena_bytes - resident - scratch) + " of " +
                            std::to_string(arena_bytes) + " are free (" + std::to_string(resident) +
                            " resident); raise CudaGemmOptions::arena_bytes or send fewer rows per call");
    }
    void* keep(std::size_t bytes, const char* what) {  // from the bottom: stays for the provider's life
        const std::size_t n = round_up(bytes, kAlign);
        if (scratch != 0) throw std::logic_error("CudaGemm: resident memory asked for while a call holds temporaries");
        if (n > arena_bytes - resident) arena_full(what, n);
        void* p = arena + resident;
        resident += n;
        arena_peak = std::max(arena_peak, resident);
        return p;
    }
    void* borrow(std::size_t bytes, const char* what) {  // above the resident part: released when the call returns
        const std::size_t n = round_up(bytes, kAlign);
        if (n > arena_bytes - resident - scratch) arena_full(what, n);
        void* p = arena + resident + scratch;
        scratch += n;
        scratch_peak = std::max(scratch_peak, scratch);
        arena_peak = std::max(arena_peak, resident + scratch);
        return p;
    }
    struct Borrowing {  // releases a call's temporaries on every way out
        Impl& s;
        ~Borrowing() { s.scratch = 0; }
    };

    // Host matrix -> the provider's element type on the device, [rows_dst, ld_dst] with zero padding.
    void upload_converted(MatRef m, void* dst, std::size_t rows_dst, std::size_t ld_dst, const char* what) {
        const std::size_t count = m.rows * m.cols;
        if (count == 0) {
            need(cudaMemsetAsync(dst, 0, rows_dst * ld_dst * bytes_of(compute), stream), "cudaMemsetAsync", what);
            return;
        }
        if (m.dtype == compute && ld_dst == m.cols && rows_dst == m.rows) {
            need(cudaMemcpyAsync(dst, m.data, count * bytes_of(compute), cudaMemcpyHostToDevice, stream), "cudaMemcpyAsync", what);
            return;
        }
        void* raw = borrow(count * bytes_of(m.dtype), what);
        need(cudaMemcpyAsync(raw, m.data, count * bytes_of(m.dtype), cudaMemcpyHostToDevice, stream), "cudaMemcpyAsync", what);
        const unsigned grid = blocks(rows_dst * ld_dst);
        const auto launch = [&](auto* from, auto* to) { convert_pad_kernel<<<grid, 256, 0, stream>>>(from, m.rows, m.cols, to, rows_dst, ld_dst); };
        if (compute == DType::F16) {
            auto* to = static_cast<__half*>(dst);
            if (m.dtype == DType::F32) launch(static_cast<const float*>(raw), to);
            else if (m.dtype == DType::F16) launch(static_cast<const __half*>(raw), to);
            else launch(static_cast<const __nv_bfloat16*>(raw), to);
        } else {
            auto* to = static_cast<float*>(dst);
            if (m.dtype == DType::F32) launch(static_cast<const float*>(raw), to);
            else if (m.dtype == DType::F16) launch(static_cast<const __half*>(raw), to);
            else launch(static_cast<const __nv_bfloat16*>(raw), to);
        }
        need(cudaGetLastError(), "convert_pad_kernel", what);
    }

    std::size_t k_padded(std::size_t k) const { return compute == DType::F16 ? round_up(k, 8) : k; }
    std::size_t n_padded(std::size_t n) const { return compute == DType::F16 ? round_up(n, 2) : n; }

    Weight place_weight(MatRef w, bool resident_copy) {
        Weight e;
        e.rows = w.rows;
        e.cols = w.cols;
        e.ld = k_padded(w.cols);
        e.rows_padded = n_padded(w.rows);
        const std::size_t bytes = std::max<std::size_t>(e.rows_padded * e.ld * bytes_of(compute), 1);
        e.data = resident_copy ? keep(bytes, "W") : borrow(bytes, "W");
        upload_converted(w, e.data, e.rows_padded, e.ld, "W");
        return e;
    }

    // Yd [t, n_pad] float32 = beta Yd + Xd [t, ld_x] Wd^T on the device; Xd and Wd in the provider's type, padded as place_weight pads.
    void multiply(const void* xd, std::size_t ld_x, const Weight& w, float* yd, std::size_t t, float beta) {
        if (t == 0 || w.rows == 0) return;
        if (compute == DType::F32) {
            const dim3 grid(static_cast<unsigned>((w.rows + 15) / 16), static_cast<unsigned>((t + 15) / 16));
            product_f32_kernel<<<grid, dim3(16, 16), 0, stream>>>(static_cast<const float*>(xd), static_cast<const float*>(w.data), yd, t, w.rows, w.cols, beta);
            need(cudaGetLastError(), "product_f32_kernel");
            return;
        }
        const std::size_t ld_y = w.rows_padded;
        if (w.cols == 0) {  // an empty sum: Y = beta Y
            if (beta == 0.0f) need(cudaMemsetAsync(yd, 0, t * ld_y * 4, stream), "cudaMemsetAsync");
            else if (beta != 1.0f) scale_kernel<<<blocks(t * ld_y), 256, 0, stream>>>(yd, t * ld_y, beta);
            return;
        }
        int32_t epilogue = SEPAL_B200_STORE;
        if (beta != 0.0f) {
            if (beta != 1.0f) {
                scale_kernel<<<blocks(t * ld_y), 256, 0, stream>>>(yd, t * ld_y, beta);
                need(cudaGetLastError(), "scale_kernel");
            }
            epilogue = SEPAL_B200_ADD;
        }
        need_b200(sepal_b200_gemm_f16(ctx, xd, ld_x, w.data, w.ld, yd, ld_y, /*y_half=*/0, t, w.rows_padded, w.ld, epilogue, /*config=*/-1, stream),
                  "sepal_b200_gemm_f16");
    }

    void finish_call() {
        int32_t status = 0;
        need_b200(sepal_b200_status(ctx, stream, &status), "sepal_b200_status");  // waits for the stream
        if (status != 0) throw CudaError("sepal_b200_gemm_f16", status, "a kernel gave up waiting");
    }

    void run(MatRef x, const Weight& w, MatView y, float beta) {
        const std::size_t t = x.rows, ld_x = k_padded(x.cols), ld_y = w.rows_padded;
        if (t == 0 || w.rows == 0) return;
        void* xd = borrow(std::max<std::size_t>(t * ld_x * bytes_of(compute), 1), "X");
        upload_converted(x, xd, t, ld_x, "X");
        float* yd = static_cast<float*>(borrow(t * ld_y * 4, "Y"));
        const bool padded = ld_y != w.rows;
        if (beta != 0.0f) {
            if (padded) {
                need(cudaMemsetAsync(yd, 0, t * ld_y * 4, stream), "cudaMemsetAsync", "Y");
                need(cudaMemcpy2DAsync(yd, ld_y * 4, y.data, w.rows * 4, w.rows * 4, t, cudaMemcpyHostToDevice, stream), "cudaMemcpy2DAsync", "Y");
            } else {
                need(cudaMemcpyAsync(yd, y.data, t * ld_y * 4, cudaMemcpyHostToDevice, stream), "cudaMemcpyAsync", "Y");
            }
        }
        multiply(xd, ld_x, w, yd, t, beta);
        if (padded)
            need(cudaMemcpy2DAsync(y.data, w.rows * 4, yd, ld_y * 4, w.rows * 4, t, cudaMemcpyDeviceToHost, stream), "cudaMemcpy2DAsync", "Y");
        else
            need(cudaMemcpyAsync(y.data, yd, t * ld_y * 4, cudaMemcpyDeviceToHost, stream), "cudaMemcpyAsync", "Y");
        finish_call();
    }
};

CudaGemm::CudaGemm(const CudaGemmOptions& options) : impl_(std::make_unique<Impl>()) {
    Impl& s = *impl_;
    s.options = options;
    s.compute = dtype_of(options.precision);
    need(cudaSetDevice(options.device), "cudaSetDevice", "device " + std::to_string(options.device));
    need(cudaFree(nullptr), "cudaFree");  // creates the context
    need(cudaMemGetInfo(&s.free_at_start, &s.total), "cudaMemGetInfo");
    s.free_min = s.free_at_start;
    need(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
    need_b200(sepal_b200_open(options.device, 0, &s.ctx), "sepal_b200_open");
    std::size_t bytes = options.arena_bytes != 0 ? options.arena_bytes : s.free_at_start / 10 * 8;
    void* base = nullptr;
    need(cudaMalloc(&base, bytes), "cudaMalloc",
         "the arena of " + std::to_string(bytes) + " bytes, with " + std::to_string(s.free_at_start) + " free on the device");
    s.arena = static_cast<char*>(base);
    s.arena_bytes = bytes;
}

CudaGemm::~CudaGemm() = default;

GemmCaps CudaGemm::caps() const {
    GemmCaps c;
    c.name = "sepal_b200";
    c.version = std::to_string(sepal_b200_api_version());
    c.isa = "sm_100a tcgen05";
    c.float_dtypes = {DType::F32, DType::F16, DType::BF16};
    c.integer_exact = false;
    c.fixed_summation_order = true;  // a row's sum runs over k in an order fixed by the shape and the schedule, never by timing
    return c;
}

void CudaGemm::gemm_f(MatRef x, MatRef w, MatView y, float beta) const {
    check_shapes(x, w.rows, w.cols, w.data, y);
    require_float(x, "X");
    require_float(w, "W");
    Impl& s = *impl_;
    std::lock_guard<std::mutex> lock(s.mutex);
    for (const Impl::Registered& r : s.registered) {
        if (r.host == w.data && r.dtype == w.dtype && r.rows == w.rows && r.cols == w.cols) {
            need(cudaSetDevice(s.options.device), "cudaSetDevice");
            Impl::Borrowing release{s};
            s.run(x, s.weights[r.index], y, beta);
            return;
        }
    }
    need(cudaSetDevice(s.options.device), "cudaSetDevice");
    Impl::Borrowing release{s};
    const Impl::Weight travelling = s.place_weight(w, /*resident_copy=*/false);
    s.run(x, travelling, y, beta);
}

void CudaGemm::gemm_f(MatRef x, WeightId w, MatView y, float beta) const {
    Impl& s = *impl_;
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!w.valid() || w.index >= s.weights.size()) throw std::invalid_argument("gemm_f: unknown weight id");
    const Impl::Weight& e = s.weights[w.index];
    check_shapes(x, e.rows, e.cols, e.data, y);
    require_float(x, "X");
    need(cudaSetDevice(s.options.device), "cudaSetDevice");
    Impl::Borrowing release{s};
    s.run(x, e, y, beta);
}

void CudaGemm::gemm_f64(ConstMatViewD x, ConstMatViewD w, MatViewD y, double beta) const { make_reference_gemm()->gemm_f64(x, w, y, beta); }

WeightId CudaGemm::upload_weights(MatRef w) {
    require_float(w, "W");
    if (w.data == nullptr && w.rows * w.cols != 0) throw std::invalid_argument("upload_weights: null data pointer");
    Impl& s = *impl_;
    std::lock_guard<std::mutex> lock(s.mutex);
    need(cudaSetDevice(s.options.device), "cudaSetDevice");
    const std::size_t before = s.resident;
    Impl::Borrowing release{s};
    try {
        // the resident copy first (temporaries of the conversion sit above it and go when this call returns)
        Impl::Weight e = s.place_weight(w, /*resident_copy=*/true);
        need(cudaStreamSynchronize(s.stream), "cudaStreamSynchronize");
        s.weights.push_back(e);
    } catch (...) {
        s.resident = before;
        throw;
    }
    return WeightId{static_cast<std::uint32_t>(s.weights.size() - 1)};
}

WeightId CudaGemm::register_weights(MatRef w) {
    {
        std::lock_guard<std::mutex> lock(impl_->mutex);
        for (const Impl::Registered& r : impl_->registered)
            if (r.host == w.data && r.dtype == w.dtype && r.rows == w.rows && r.cols == w.cols) return WeightId{r.index};
    }
    const WeightId id = upload_weights(w);
    std::lock_guard<std::mutex> lock(impl_->mutex);
    impl_->registered.push_back({w.data, w.dtype, w.rows, w.cols, id.index});
    return id;
}

DeviceMatrix CudaGemm::upload_matrix(MatRef x) {
    require_float(x, "X");
    if (x.data == nullptr && x.rows * x.cols != 0) throw std::invalid_argument("upload_matrix: null data pointer");
    Impl& s = *impl_;
    std::lock_guard<std::mutex> lock(s.mutex);
    need(cudaSetDevice(s.options.device), "cudaSetDevice");
    Impl::Borrowing release{s};
    void* dst = s.keep(std::max<std::size_t>(x.rows * x.cols * bytes_of(s.compute), 1), "X");
    s.upload_converted(x, dst, x.rows, x.cols, "X");
    need(cudaStreamSynchronize(s.stream), "cudaStreamSynchronize");
    return DeviceMatrix{dst, s.compute, x.rows, x.cols};
}

DeviceMatrix CudaGemm::alloc_output(std::size_t rows, std::size_t cols) {
    Impl& s = *impl_;
    std::lock_guard<std::mutex> lock(s.mutex);
    return DeviceMatrix{s.keep(std::max<std::size_t>(rows * cols * 4, 1), "Y"), DType::F32, rows, cols};
}

void CudaGemm::gemm_device(const DeviceMatrix& x, WeightId w, const DeviceMatrix& y, float beta) const {
    Impl& s = *impl_;
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!w.valid() || w.index >= s.weights.size()) throw std::invalid_argument("gemm_device: unknown weight id");
    const Impl::Weight& e = s.weights[w.index];
    if (x.dtype != s.compute || y.dtype != DType::F32) throw std::invalid_argument("gemm_device: X must have the provider's element type and Y must be float32");
    if (x.cols != e.cols || y.rows != x.rows || y.cols != e.rows) throw std::invalid_argument("gemm_device: shapes disagree");
    need(cudaSetDevice(s.options.device), "cudaSetDevice");
    if (x.rows == 0 || e.rows == 0) return;
    const std::size_t ld_x = s.k_padded(x.cols);
    if (ld_x == x.cols && e.rows_padded == e.rows) {
        s.multiply(x.data, ld_x, e, static_cast<float*>(y.data), x.rows, beta);
        return;
    }
    // a shape the kernels take only padded: pad X and Y into temporaries, multiply, copy the product back without its padding.
    // (The temporaries stay borrowed until synchronize(): this call returns without waiting.)
    void* xd = s.borrow(x.rows * ld_x * 2, "X");
    convert_pad_kernel<<<blocks(x.rows * ld_x), 256, 0, s.stream>>>(static_cast<const __half*>(x.data), x.rows, x.cols, static_cast<__half*>(xd), x.rows, ld_x);
    float* yd = static_cast<float*>(s.borrow(x.rows * e.rows_padded * 4, "Y"));
    if (beta != 0.0f)
        convert_pad_kernel<<<blocks(x.rows * e.rows_padded), 256, 0, s.stream>>>(static_cast<const float*>(y.data), y.rows, y.cols, yd, y.rows, e.rows_padded);
    s.multiply(xd, ld_x, e, yd, x.rows, beta);
    unpad_kernel<<<blocks(y.rows * y.cols), 256, 0, s.stream>>>(yd, e.rows_padded, static_cast<float*>(y.data), y.rows, y.cols);
    need(cudaGetLastError(), "unpad_kernel");
}

void CudaGemm::synchronize() const {
    Impl& s = *impl_;
    std::lock_guard<std::mutex> lock(s.mutex);
    need(cudaSetDevice(s.options.device), "cudaSetDevice");
    Impl::Borrowing release{s};
    s.finish_call();
}

void CudaGemm::download(const DeviceMatrix& m, MatView out) const {
    if (m.dtype != DType::F32 || out.rows != m.rows || out.cols != m.cols) throw std::invalid_argument("download: a float32 matrix of the same shape is needed");
    Impl& s = *impl_;
    std::lock_guard<std::mutex> lock(s.mutex);
    need(cudaSetDevice(s.options.device), "cudaSetDevice");
    Impl::Borrowing release{s};
    need(cudaMemcpyAsync(out.data, m.data, m.rows * m.cols * 4, cudaMemcpyDeviceToHost, s.stream), "cudaMemcpyAsync");
    s.finish_call();
}

Precision CudaGemm::precision() const noexcept { return impl_->options.precision; }

DeviceInfo CudaGemm::device_info() const {
    DeviceInfo d;
    d.device = impl_->options.device;
    cudaDeviceProp p{};
    need(cudaGetDeviceProperties(&p, d.device), "cudaGetDeviceProperties");
    d.name = p.name;
    d.compute_major = p.major;
    d.compute_minor = p.minor;
    d.total_bytes = p.totalGlobalMem;
    need(cudaRuntimeGetVersion(&d.runtime_version), "cudaRuntimeGetVersion");
    need(cudaDriverGetVersion(&d.driver_version), "cudaDriverGetVersion");
    d.cublas_version = 0;  // no cuBLAS behind this provider
    return d;
}

MemoryStats CudaGemm::memory() const {
    Impl& s = *impl_;
    std::lock_guard<std::mutex> lock(s.mutex);
    need(cudaSetDevice(s.options.device), "cudaSetDevice");
    std::size_t free_now = 0, total = 0;
    need(cudaMemGetInfo(&free_now, &total), "cudaMemGetInfo");
    s.free_min = std::min(s.free_min, free_now);
    MemoryStats m;
    m.device_total = s.total;
    m.device_free_at_start = s.free_at_start;
    m.device_free_min = s.free_min;
    m.arena_bytes = s.arena_bytes;
    m.resident_bytes = s.resident;
    m.scratch_peak_bytes = s.scratch_peak;
    m.arena_peak_bytes = s.arena_peak;
    return m;
}

std::unique_ptr<GemmProvider> make_cuda_gemm(const CudaGemmOptions& options) { return std::make_unique<CudaGemm>(options); }

}  // namespace sepal::cuda
