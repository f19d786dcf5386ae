// TEST INFRASTRUCTURE, not product code.
//
// A thin extern "C" face over the reference's own CPU GEMM so that Python tests and the benchmark's CPU-baseline leg
// can call it through ctypes. This file holds no arithmetic of its own: every product is computed by the reference's
// sources, which oracle/Makefile compiles where they lie (runner/src/cpu/{gemm,gemm_kernels_*,thread_pool,isa,
// elementwise}.cpp and runner/src/provider/gemm_ref.cpp) into oracle/_ref/libsepal_ref.so. Nothing of the reference
// is copied into this repository.
//
// Reference interfaces bound here:
//   pack_weight / pack_weight_swiglu / pack_acts / gemm_packed   runner/include/sepal/cpu/gemm.hpp:86-108
//   make_reference_gemm()->gemm_f (float64 accumulation)        runner/include/sepal/gemm.hpp:44-73
//   rmsnorm_rows                                                 runner/include/sepal/cpu/elementwise.hpp:13-16
//   float_to_bf16                                                runner/include/sepal/cpu/gemm.hpp:49
#include <chrono>
#include <cstdint>
#include <cstring>
#include <exception>
#include <memory>
#include <string>

#include "sepal/cpu/elementwise.hpp"
#include "sepal/cpu/gemm.hpp"
#include "sepal/cpu/isa.hpp"
#include "sepal/cpu/thread_pool.hpp"
#include "sepal/gemm.hpp"

using namespace sepal;
using namespace sepal::cpu;

namespace {

thread_local std::string g_error;

struct Pool {
    std::unique_ptr<ThreadPool> pool;
    unsigned threads = 0;
};
Pool& pool_for(unsigned threads) {
    static Pool p;
    if (!p.pool || p.threads != threads) {
        p.pool = std::make_unique<ThreadPool>(threads);
        p.threads = threads;
    }
    return p;
}

WeightKind kind_of(int kind) { return kind == 0 ? WeightKind::F32 : kind == 1 ? WeightKind::BF16 : WeightKind::I8; }

Isa isa_of(const char* name) { return (name == nullptr || name[0] == '\0') ? best_isa() : parse_isa(name); }

struct Packed {
    PackedWeight w;
    PackedActs x;
    Isa isa;
};

template <class F>
int guarded(F&& f) {
    try {
        f();
        g_error.clear();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}

double now_s() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

} // namespace

extern "C" {

const char* ref_last_error() { return g_error.c_str(); }

/// Threads the reference's pool runs with when asked for `threads` (0 = its own default: physical cores within the cgroup quota).
unsigned ref_pool_threads(unsigned threads) { return pool_for(threads).pool->size(); }

/// The kernel variant the reference picks for (kind, isa) on this host, e.g. "bf16/avx512-bf16".
const char* ref_variant_name(int kind, const char* isa) {
    static thread_local std::string s;
    try {
        s = name_of(pick_variant(kind_of(kind), isa_of(isa)));
    } catch (const std::exception& e) {
        s = std::string("error: ") + e.what();
    }
    return s.c_str();
}

const char* ref_cpu_brand() { return features().brand.c_str(); }

std::uint16_t ref_float_to_bf16(float x) { return float_to_bf16(x); }

/// y [rows, n] (stride ldy) = (accumulate ? y : 0) + x [rows, k] w[n, k]^T through pack_weight -> pack_acts -> gemm_packed.
int ref_cpu_gemm(int kind, const char* isa, unsigned threads, const float* x, std::size_t ldx, std::size_t rows, std::size_t k, const float* w,
                 std::size_t ldw, std::size_t n, float* y, std::size_t ldy, int accumulate) {
    return guarded([&] {
        ThreadPool& pool = *pool_for(threads).pool;
        const Isa i = isa_of(isa);
        const PackedWeight pw = pack_weight(w, ldw, n, k, kind_of(kind), i, pool);
        PackedActs pa;
        pack_acts(pa, x, ldx, rows, k, pw.variant(), pool);
        gemm_packed(pw, pa, y, ldy, accumulate != 0, pool);
    });
}

/// y [rows, n] = silu(x gate^T) * (x up^T) through pack_weight_swiglu (gate, up: [n, k], n = the intermediate size).
int ref_cpu_gemm_swiglu(int kind, const char* isa, unsigned threads, const float* x, std::size_t ldx, std::size_t rows, std::size_t k,
                        const float* gate, const float* up, std::size_t ldw, std::size_t n, float* y, std::size_t ldy) {
    return guarded([&] {
        ThreadPool& pool = *pool_for(threads).pool;
        const Isa i = isa_of(isa);
        const PackedWeight pw = pack_weight_swiglu(gate, up, ldw, n, k, kind_of(kind), i, pool);
        PackedActs pa;
        pack_acts(pa, x, ldx, rows, k, pw.variant(), pool);
        gemm_packed(pw, pa, y, ldy, false, pool);
    });
}

/// Packs `w` once; the handle is timed with ref_packed_time and freed with ref_packed_free.
void* ref_pack(int kind, const char* isa, unsigned threads, const float* w, std::size_t ldw, std::size_t n, std::size_t k) {
    void* out = nullptr;
    guarded([&] {
        ThreadPool& pool = *pool_for(threads).pool;
        const Isa i = isa_of(isa);
        auto p = std::make_unique<Packed>(Packed{pack_weight(w, ldw, n, k, kind_of(kind), i, pool), PackedActs{}, i});
        out = p.release();
    });
    return out;
}
void ref_packed_free(void* handle) { delete static_cast<Packed*>(handle); }

/// One product with the packed weights, timed the way the reference's own bench does (runner/tools/sepal_cpu_gemm_bench.cpp:153-201):
/// seconds_out[0] = packing of the activations, seconds_out[1] = gemm_packed alone.
int ref_packed_run(void* handle, unsigned threads, const float* x, std::size_t ldx, std::size_t rows, float* y, std::size_t ldy, int accumulate,
                   double* seconds_out) {
    return guarded([&] {
        Packed& p = *static_cast<Packed*>(handle);
        ThreadPool& pool = *pool_for(threads).pool;
        const double t0 = now_s();
        pack_acts(p.x, x, ldx, rows, p.w.k(), p.w.variant(), pool);
        const double t1 = now_s();
        gemm_packed(p.w, p.x, y, ldy, accumulate != 0, pool);
        const double t2 = now_s();
        if (seconds_out != nullptr) {
            seconds_out[0] = t1 - t0;
            seconds_out[1] = t2 - t1;
        }
    });
}

/// The reference provider: y = beta y + x w^T, float64 accumulation in increasing k, rounded to float32 once.
/// dtype codes: 0 float32, 1 binary16, 2 bfloat16 (DType of runner/include/sepal/dtype.hpp).
int ref_gemm_f64acc(const void* x, int x_dtype, const void* w, int w_dtype, std::size_t rows, std::size_t n, std::size_t k, float* y, float beta) {
    return guarded([&] {
        const auto dt = [](int c) { return c == 0 ? DType::F32 : c == 1 ? DType::F16 : DType::BF16; };
        const auto provider = make_reference_gemm();
        provider->gemm_f(MatRef(x, dt(x_dtype), rows, k), MatRef(w, dt(w_dtype), n, k), MatView(y, rows, n), beta);
    });
}

/// y = x / sqrt(mean(x^2) + eps) * w1 per row (w1 = 1 + stored weight), as the CPU trunk applies it before a projection.
int ref_rmsnorm_rows(unsigned threads, const float* x, std::size_t ldx, float* y, std::size_t ldy, std::size_t rows, std::size_t cols, const float* w1,
                     double eps) {
    return guarded([&] { rmsnorm_rows(x, ldx, y, ldy, rows, cols, w1, eps, *pool_for(threads).pool); });
}

} // extern "C"
