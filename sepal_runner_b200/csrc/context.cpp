#include "context.hpp"

#include <atomic>
#include <cstring>
#include <vector>

namespace sepal::b200 {

namespace {
std::atomic<bool> g_launch_overlap{true};
}
bool launch_overlap() { return g_launch_overlap.load(std::memory_order_relaxed); }
void set_launch_overlap(bool on) { g_launch_overlap.store(on, std::memory_order_relaxed); }

std::size_t default_workspace_bytes(int sm_count) {
    return static_cast<std::size_t>(sm_count) * 2u * (128u * 256u * sizeof(float));
}

Context::Context(int device_, std::size_t workspace_bytes) : device(device_) {
    int count = 0;
    check(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
    if (device < 0 || device >= count)
        throw std::invalid_argument("sepal_b200: device " + std::to_string(device) + " does not exist (" + std::to_string(count) + " visible)");
    check(cudaSetDevice(device), "cudaSetDevice");
    check(cudaDeviceGetAttribute(&compute_major, cudaDevAttrComputeCapabilityMajor, device), "cudaDeviceGetAttribute");
    check(cudaDeviceGetAttribute(&compute_minor, cudaDevAttrComputeCapabilityMinor, device), "cudaDeviceGetAttribute");
    check(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device), "cudaDeviceGetAttribute");
    int optin = 0;
    check(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device), "cudaDeviceGetAttribute");
    smem_optin = static_cast<std::size_t>(optin);
    if (compute_major != 10)
        throw std::runtime_error("sepal_b200: the kernels are built for sm_100a only; device " + std::to_string(device) + " is sm_" +
                                 std::to_string(compute_major) + std::to_string(compute_minor) + " (there is no fallback path)");

    // cuTensorMapEncodeTiled comes from the driver; fetching it through the runtime keeps the library free of a link to libcuda.
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult query{};
    check(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query), "cudaGetDriverEntryPoint");
    if (fn == nullptr || query != cudaDriverEntryPointSuccess) throw std::runtime_error("sepal_b200: the driver has no cuTensorMapEncodeTiled");
    encode = reinterpret_cast<TensorMapEncodeFn>(fn);

    if (workspace_bytes == 0) workspace_bytes = default_workspace_bytes(sm_count);
    scratch.partial_bytes = workspace_bytes;
    check(cudaMalloc(reinterpret_cast<void**>(&scratch.partials), scratch.partial_bytes), "cudaMalloc(scratch)");
    scratch.counter_count = 1u << 16;
    check(cudaMalloc(reinterpret_cast<void**>(&scratch.tile_counters), scratch.counter_count * sizeof(unsigned)), "cudaMalloc(counters)");
    check(cudaMemset(scratch.tile_counters, 0, scratch.counter_count * sizeof(unsigned)), "cudaMemset(counters)");
    check(cudaMalloc(reinterpret_cast<void**>(&status), sizeof(int)), "cudaMalloc(status)");
    check(cudaMemset(status, 0, sizeof(int)), "cudaMemset(status)");
    check(cudaMallocHost(reinterpret_cast<void**>(&status_host), sizeof(int)), "cudaMallocHost(status)");
    {
        check(cudaMalloc(&unit_scales, kUnitScales * 2), "cudaMalloc(unit scales)");
        check(cudaMalloc(reinterpret_cast<void**>(&unit), sizeof(float)), "cudaMalloc(unit)");
        const std::vector<std::uint16_t> ones(kUnitScales, 0x3C00u);  // binary16 1.0
        const float one = 1.0f;
        check(cudaMemcpy(unit_scales, ones.data(), kUnitScales * 2, cudaMemcpyHostToDevice), "cudaMemcpy(unit scales)");
        check(cudaMemcpy(unit, &one, sizeof one, cudaMemcpyHostToDevice), "cudaMemcpy(unit)");
        table_bytes = std::size_t{4} << 20;
        check(cudaMalloc(&table, table_bytes), "cudaMalloc(table)");
    }
    check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
}

Context::Context(Borrowed, int device_, float* partials, std::size_t partial_bytes, unsigned* counters, std::size_t counter_count, int* status_word)
    : device(device_) {
    check(cudaDeviceGetAttribute(&compute_major, cudaDevAttrComputeCapabilityMajor, device), "cudaDeviceGetAttribute");
    check(cudaDeviceGetAttribute(&compute_minor, cudaDevAttrComputeCapabilityMinor, device), "cudaDeviceGetAttribute");
    check(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device), "cudaDeviceGetAttribute");
    int optin = 0;
    check(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device), "cudaDeviceGetAttribute");
    smem_optin = static_cast<std::size_t>(optin);
    if (compute_major != 10)
        throw std::runtime_error("sepal_b200: the kernels are built for sm_100a only; device " + std::to_string(device) + " is sm_" +
                                 std::to_string(compute_major) + std::to_string(compute_minor) + " (there is no fallback path)");
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult query{};
    check(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query), "cudaGetDriverEntryPoint");
    if (fn == nullptr || query != cudaDriverEntryPointSuccess) throw std::runtime_error("sepal_b200: the driver has no cuTensorMapEncodeTiled");
    encode = reinterpret_cast<TensorMapEncodeFn>(fn);
    scratch.partials = partials;
    scratch.partial_bytes = partial_bytes;
    scratch.tile_counters = counters;
    scratch.counter_count = counter_count;
    status = status_word;
}

Context::~Context() {
    (void)cudaSetDevice(device);
    if (scratch.partials != nullptr) cudaFree(scratch.partials);
    if (scratch.tile_counters != nullptr) cudaFree(scratch.tile_counters);
    if (status != nullptr) cudaFree(status);
    if (unit_scales != nullptr) cudaFree(unit_scales);
    if (unit != nullptr) cudaFree(unit);
    if (table != nullptr) cudaFree(table);
    if (status_host != nullptr) cudaFreeHost(status_host);
}

int Context::read_status(cudaStream_t stream) {
    check(cudaMemcpyAsync(status_host, status, sizeof(int), cudaMemcpyDeviceToHost, stream), "cudaMemcpyAsync(status)");
    check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    const int value = *status_host;
    if (value != 0) {
        check(cudaMemsetAsync(status, 0, sizeof(int), stream), "cudaMemsetAsync(status)");
        // A kernel that gave up may have left tile counters behind: clear them so the next launch starts clean.
        check(cudaMemsetAsync(scratch.tile_counters, 0, scratch.counter_count * sizeof(unsigned), stream), "cudaMemsetAsync(counters)");
        check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    }
    return value;
}

CUtensorMap make_tensor_map_2d(const Context& ctx, const void* base, CUtensorMapDataType type, std::size_t elem_bytes, std::size_t rows,
                               std::size_t cols, std::size_t ld, unsigned box_rows, unsigned box_cols, bool swizzle128) {
    CUtensorMap map;
    std::memset(&map, 0, sizeof map);
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld * elem_bytes)};  // bytes between rows; the innermost stride is implied
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult rc = ctx.encode(&map, type, 2, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS)
        throw std::invalid_argument("sepal_b200: cuTensorMapEncodeTiled rejected a [" + std::to_string(rows) + " x " + std::to_string(cols) +
                                    "] matrix with row stride " + std::to_string(ld) + " (driver code " + std::to_string(static_cast<int>(rc)) +
                                    "): the base must be 16-byte aligned and the row stride a multiple of 16 bytes");
    return map;
}

}  // namespace sepal::b200
