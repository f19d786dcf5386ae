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
//   the attention mixer between its projections                  runner/include/sepal/ref/attention.hpp:33-231 (unpack_query_and_gate,
//       rope_angles, apply_rope, grouped_query_attention; rms_norm and sigmoid of ref/primitives.hpp), composed below in the order of
//       attention_mixer (:176-231) with the four projections left out
//   the Gated DeltaNet mixer between its projections             runner/include/sepal/ref/deltanet.hpp:41-330 (causal_conv, split_heads,
//       l2_normalise, share_key_heads, decay_gate, delta_rule_scan, gated_rms_norm), composed in the order of deltanet_mixer (:246-279)
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
#include "sepal/ref/attention.hpp"
#include "sepal/ref/deltanet.hpp"

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


/// The full-attention mixer between q/k/v_proj and o_proj in float64, by the reference's own template functions. q_gate [T, 2 heads hd]
/// (per head: query, then gate), k and v [T, kv_heads hd], positions [T]; ctx_keys / ctx_values [context, kv_heads, hd]: the keys
/// (already normed and rotated) and values of the tokens before this run (context may be 0). Writes the gated output [T, heads hd] and
/// this run's own keys and values [T, kv_heads, hd] (what a cache would append).
int ref_attention_core(const double* q_gate, const double* k, const double* v, const double* q_norm, const double* k_norm, const double* positions,
                       std::size_t tokens, const double* ctx_keys, const double* ctx_values, std::size_t context, unsigned heads, unsigned kv_heads,
                       unsigned head_dim, unsigned rotary_dims, double theta, double eps, double* out, double* keys_out, double* values_out) {
    return guarded([&] {
        ModelConfig cfg;
        cfg.attn_heads = heads;
        cfg.attn_kv_heads = kv_heads;
        cfg.attn_head_dim = head_dim;
        cfg.rope_theta = theta;
        cfg.partial_rotary_factor = static_cast<double>(rotary_dims) / static_cast<double>(head_dim);
        cfg.rms_norm_eps = eps;
        if (cfg.attn_rotary_dims() != rotary_dims) throw std::invalid_argument("ref_attention_core: the rotary dims do not survive the config's rounding");
        const auto provider = make_reference_gemm();
        const std::size_t kv_width = static_cast<std::size_t>(kv_heads) * head_dim;
        const std::vector<std::size_t> kv_shape = {tokens, kv_heads, head_dim};
        const ref::QueryAndGate<double> unpacked = ref::unpack_query_and_gate<double>(ConstMatViewD(q_gate, tokens, 2 * static_cast<std::size_t>(heads) * head_dim), cfg);
        const TensorD angles = ref::rope_angles(std::span<const double>(positions, tokens), cfg);
        TensorD q = ref::rms_norm<double>(unpacked.query.as_mat(head_dim), std::span<const double>(q_norm, head_dim), eps);
        q.reshape({tokens, heads, head_dim});
        ref::apply_rope(q, angles);
        TensorD k_flat({tokens, kv_width});
        std::copy(k, k + tokens * kv_width, k_flat.data());
        TensorD kk = ref::rms_norm<double>(k_flat.as_mat(head_dim), std::span<const double>(k_norm, head_dim), eps);
        kk.reshape(kv_shape);
        ref::apply_rope(kk, angles);
        TensorD vv(kv_shape);
        std::copy(v, v + tokens * kv_width, vv.data());
        std::copy(kk.data(), kk.data() + kk.size(), keys_out);
        std::copy(vv.data(), vv.data() + vv.size(), values_out);
        auto parent = std::make_shared<ref::AttentionState<double>>();
        if (context != 0) {
            parent->keys = TensorD({context, kv_heads, head_dim});
            parent->values = TensorD({context, kv_heads, head_dim});
            std::copy(ctx_keys, ctx_keys + context * kv_width, parent->keys.data());
            std::copy(ctx_values, ctx_values + context * kv_width, parent->values.data());
            parent->tokens = context;
        }
        ref::AttentionState<double> state;
        if (context != 0) state.parent = parent;
        state.keys = std::move(kk);
        state.values = std::move(vv);
        state.tokens = context + tokens;
        TensorD attended = ref::grouped_query_attention(*provider, q, state, context, ref::attention_scale(cfg));
        for (std::size_t i = 0; i < attended.size(); ++i) out[i] = attended[i] * ref::sigmoid(unpacked.gate[i]);
    });
}

/// The Gated DeltaNet mixer between its in- and out-projections in float64, by the reference's own template functions. mixed [T, conv_dim]
/// ([q; k] of the key heads, then v), z [T, value_dim], b and a [T, value_heads]; conv [conv_dim, taps]; state [value_heads, dk, dv] and
/// tail [taps - 1, conv_dim] are read and the state after the run is written to state_out / tail_out. out [T, value_dim].
int ref_deltanet_core(const double* mixed, const double* z, const double* b, const double* a, const double* conv, const double* a_log,
                      const double* dt_bias, const double* norm, const double* state_in, const double* tail_in, std::size_t tokens, unsigned key_heads,
                      unsigned value_heads, unsigned dk, unsigned dv, unsigned taps, double eps, double* out, double* state_out, double* tail_out) {
    return guarded([&] {
        ModelConfig cfg;
        cfg.dn_key_heads = key_heads;
        cfg.dn_value_heads = value_heads;
        cfg.dn_key_head_dim = dk;
        cfg.dn_value_head_dim = dv;
        cfg.conv_kernel = taps;
        cfg.rms_norm_eps = eps;
        const std::size_t conv_dim = 2 * static_cast<std::size_t>(key_heads) * dk + static_cast<std::size_t>(value_heads) * dv;
        const std::size_t value_dim = static_cast<std::size_t>(value_heads) * dv;
        TensorD tail({static_cast<std::size_t>(taps) - 1, conv_dim});
        std::copy(tail_in, tail_in + tail.size(), tail.data());
        ref::ConvResult<double> c = ref::causal_conv<double>(ConstMatViewD(mixed, tokens, conv_dim), ConstMatViewD(conv, conv_dim, taps), tail.mat());
        for (double& value : c.outputs.span()) value = ref::silu(value);
        ref::SplitHeads<double> split = ref::split_heads<double>(c.outputs.mat(), cfg);
        ref::l2_normalise(split.q.as_mat(dk));
        ref::l2_normalise(split.k.as_mat(dk));
        const TensorD q = ref::share_key_heads(split.q, cfg);
        const TensorD kk = ref::share_key_heads(split.k, cfg);
        const TensorD decay = ref::decay_gate<double>(ConstMatViewD(a, tokens, value_heads), std::span<const double>(a_log, value_heads),
                                                      std::span<const double>(dt_bias, value_heads));
        TensorD beta({tokens, value_heads});
        for (std::size_t i = 0; i < beta.size(); ++i) beta[i] = ref::sigmoid(b[i]);
        TensorD state({value_heads, dk, dv});
        std::copy(state_in, state_in + state.size(), state.data());
        ref::ScanResult<double> scan = ref::delta_rule_scan(q, kk, split.v, decay, beta, std::move(state), ref::delta_rule_output_scale(cfg));
        const TensorD normed = ref::gated_rms_norm<double>(scan.reads.as_mat(dv), ConstMatViewD(z, tokens * value_heads, dv), std::span<const double>(norm, dv), eps);
        std::copy(normed.data(), normed.data() + tokens * value_dim, out);
        std::copy(scan.state.data(), scan.state.data() + scan.state.size(), state_out);
        std::copy(c.tail.data(), c.tail.data() + c.tail.size(), tail_out);
    });
}

} // extern "C"
