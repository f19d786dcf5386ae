// The C ABI (include/sepal_b200.h): argument checks, exception -> error string, nothing else. Modelled on the engine's own
// boundary file (runner/src/capi/c_api.cpp:28-43: thread-local message, every entry point wrapped).
#include "../../include/sepal_b200.h"

#include <cstring>
#include <exception>
#include <new>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "attention.hpp"
#include "checkpoint.hpp"
#include "deltanet.hpp"
#include "gemm.hpp"
#include "model.hpp"
#include "provider.hpp"
#include "trunk.hpp"

using namespace sepal::b200;

struct sepal_b200_ctx {
    Context ctx;
    sepal_b200_ctx(int device, std::size_t bytes) : ctx(device, bytes) {}
};
struct sepal_b200_provider {
    B200Gemm gemm;
    sepal_b200_provider(int device, std::size_t bytes) : gemm(device, bytes) {}
};

struct sepal_b200_trunk {
    Trunk trunk;
    sepal_b200_trunk(int device, const TrunkConfig& c, const Checkpoint* checkpoint) : trunk(device, c, checkpoint) {}
};

namespace {

thread_local std::string g_error;

template <class F>
int32_t guarded(F&& f) noexcept {
    try {
        f();
        g_error.clear();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
    } catch (...) {
        g_error = "unknown error";
    }
    return 1;
}

Epilogue epilogue_of(int32_t e) {
    if (e < 0 || e > 2) throw std::invalid_argument("epilogue must be 0 (store), 1 (add) or 2 (swiglu)");
    return static_cast<Epilogue>(e);
}
HostType host_type_of(int32_t t) {
    if (t != SEPAL_B200_F32 && t != SEPAL_B200_F16) throw std::invalid_argument("element type must be 0 (float32) or 1 (binary16)");
    return static_cast<HostType>(t);
}
void require(const void* p, const char* what) {
    if (p == nullptr) throw std::invalid_argument(std::string(what) + " is null");
}

}  // namespace

extern "C" {

int32_t sepal_b200_api_version(void) { return 1; }

const char* sepal_b200_last_error(void) { return g_error.c_str(); }

int32_t sepal_b200_open(int32_t device, uint64_t workspace_bytes, sepal_b200_ctx** out) {
    if (out != nullptr) *out = nullptr;
    return guarded([&] {
        require(out, "out");
        *out = new sepal_b200_ctx(device, static_cast<std::size_t>(workspace_bytes));
    });
}

void sepal_b200_close(sepal_b200_ctx* ctx) { delete ctx; }

int32_t sepal_b200_info(sepal_b200_ctx* ctx, char* buffer, uint64_t capacity, uint64_t* needed) {
    return guarded([&] {
        require(ctx, "ctx");
        const Context& c = ctx->ctx;
        const std::string json = std::string("{\"library\":\"sepal_b200\",\"api_version\":1,\"device\":") + std::to_string(c.device) +
                                 ",\"compute_capability\":\"" + std::to_string(c.compute_major) + "." + std::to_string(c.compute_minor) +
                                 "\",\"sm_count\":" + std::to_string(c.sm_count) + ",\"workspace_bytes\":" + std::to_string(c.scratch.partial_bytes) +
                                 ",\"kernels\":[\"gemm_tc_kernel<W8> (tcgen05.mma kind::f16, TMA, TMEM)\",\"gemm_pair_kernel\",\"gemm_w8_pair_kernel\",\"gemm_w8t_pair_kernel\","
                                 "\"gemm_f16t_pair_kernel\",\"quantize_group_s8_kernel\","
                                 "\"prepare_scales_kernel\",\"pack_gate_up_kernel\"],\"fallback\":\"none\"}";
        if (needed != nullptr) *needed = json.size() + 1;
        if (buffer == nullptr || capacity < json.size() + 1) throw std::length_error("buffer too small: " + std::to_string(json.size() + 1) + " bytes needed");
        std::memcpy(buffer, json.c_str(), json.size() + 1);
    });
}

int32_t sepal_b200_status(sepal_b200_ctx* ctx, void* stream, int32_t* status_out) {
    return guarded([&] {
        require(ctx, "ctx");
        require(status_out, "status_out");
        check(cudaSetDevice(ctx->ctx.device), "cudaSetDevice");
        *status_out = ctx->ctx.read_status(static_cast<cudaStream_t>(stream));
    });
}

int32_t sepal_b200_debug_leave_status(sepal_b200_ctx* ctx, void* stream, int32_t code, uint32_t stale_counters) {
    return guarded([&] {
        require(ctx, "ctx");
        Context& c = ctx->ctx;
        check(cudaSetDevice(c.device), "cudaSetDevice");
        if (stale_counters > c.scratch.counter_count) throw std::invalid_argument("sepal_b200_debug_leave_status: more counters than the context has");
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        check(cudaMemcpyAsync(c.status, &code, sizeof code, cudaMemcpyHostToDevice, s), "cudaMemcpyAsync(status)");
        if (stale_counters != 0) check(cudaMemsetAsync(c.scratch.tile_counters, 1, stale_counters * sizeof(unsigned), s), "cudaMemsetAsync(counters)");
        check(cudaStreamSynchronize(s), "cudaStreamSynchronize");  // `code` lives on this call's stack
    });
}

uint64_t sepal_b200_take_launch_count(void) { return take_launch_count(); }

int32_t sepal_b200_w8g_schedule(uint32_t sm_count, uint64_t t, uint64_t n, uint64_t k, int32_t epilogue, int32_t staged) {
    return static_cast<int32_t>(w8g_swapped_tokens(sm_count, t, n, k, staged != 0, epilogue_of(epilogue)));
}

void sepal_b200_set_launch_overlap(int32_t on) { set_launch_overlap(on != 0); }

int32_t sepal_b200_set_static_weights(sepal_b200_ctx* ctx, int32_t on) {
    return guarded([&] {
        require(ctx, "ctx");
        ctx->ctx.static_weights = on != 0;
    });
}

int32_t sepal_b200_gemm_f16(sepal_b200_ctx* ctx, const void* x, uint64_t ld_x, const void* w, uint64_t ld_w, void* y, uint64_t ld_y, int32_t y_half,
                            uint64_t t, uint64_t n, uint64_t k, int32_t epilogue, int32_t config, void* stream) {
    return guarded([&] {
        require(ctx, "ctx");
        launch_gemm_f16(ctx->ctx, x, ld_x, w, ld_w, y, ld_y, y_half != 0, t, n, k, epilogue_of(epilogue), config, static_cast<cudaStream_t>(stream));
    });
}

int32_t sepal_b200_gemm_f16_noalloc(const void* x, uint64_t ld_x, const void* w, uint64_t ld_w, void* y, uint64_t ld_y, int32_t y_half, uint64_t t,
                                    uint64_t n, uint64_t k, int32_t epilogue, void* stream, int32_t* status_out) {
    return guarded([&] {
        int status = 0;
        launch_gemm_f16_noalloc(x, ld_x, w, ld_w, y, ld_y, y_half != 0, t, n, k, epilogue_of(epilogue), static_cast<cudaStream_t>(stream),
                                status_out != nullptr ? &status : nullptr);
        if (status_out != nullptr) *status_out = status;
    });
}

int32_t sepal_b200_gemm_w8g(sepal_b200_ctx* ctx, const void* x, uint64_t ld_x, const int8_t* q, uint64_t ld_q, const void* scales_t, uint64_t ld_st,
                            const float* descale, void* y, uint64_t ld_y, int32_t y_half, uint64_t t, uint64_t n, uint64_t k, int32_t epilogue,
                            int32_t config, void* stream) {
    return guarded([&] {
        require(ctx, "ctx");
        W8gMatrix m;
        m.q = q;
        m.ld_q = ld_q;
        m.scales_t = scales_t;
        m.ld_st = ld_st;
        m.descale = descale;
        launch_gemm_w8g(ctx->ctx, x, ld_x, m, y, ld_y, y_half != 0, t, n, k, epilogue_of(epilogue), config, static_cast<cudaStream_t>(stream));
    });
}

int32_t sepal_b200_gemm_w8r(sepal_b200_ctx* ctx, const void* x, uint64_t ld_x, const int8_t* q, uint64_t ld_q, const float* sw, void* y, uint64_t ld_y,
                            int32_t y_half, uint64_t t, uint64_t n, uint64_t k, int32_t epilogue, int32_t config, void* stream) {
    return guarded([&] {
        require(ctx, "ctx");
        launch_gemm_w8r(ctx->ctx, x, ld_x, q, ld_q, sw, y, ld_y, y_half != 0, t, n, k, epilogue_of(epilogue), config, static_cast<cudaStream_t>(stream));
    });
}

int32_t sepal_b200_quantize_rows_s8(const void* w, uint64_t ld_w, int8_t* q, uint64_t ld_q, float* scales, uint64_t n, uint64_t k, const float* col_scale,
                                    void* stream) {
    return guarded([&] { launch_quantize_rows_s8(w, ld_w, q, ld_q, scales, n, k, col_scale, static_cast<cudaStream_t>(stream)); });
}

int32_t sepal_b200_quantize_group_s8(const float* src, uint64_t ld_src, int8_t* q, uint64_t ld_q, float* s, uint64_t ld_s, uint64_t rows, uint64_t k,
                                     void* stream) {
    return guarded([&] { launch_quantize_group_s8(src, ld_src, q, ld_q, s, ld_s, rows, k, static_cast<cudaStream_t>(stream)); });
}

int32_t sepal_b200_prepare_w8g_scales(const float* s, uint64_t ld_s, uint64_t n, uint64_t groups, void* scales_t, uint64_t ld_st, float* descale,
                                      uint32_t* max_bits, void* stream) {
    return guarded([&] { launch_prepare_w8g_scales(s, ld_s, n, groups, scales_t, ld_st, descale, max_bits, static_cast<cudaStream_t>(stream)); });
}

int32_t sepal_b200_pack_gate_up(const void* src, uint64_t src_stride_bytes, void* dst, uint64_t dst_stride_bytes, uint64_t inter, uint64_t row_bytes,
                                void* stream) {
    return guarded([&] { launch_pack_gate_up(src, src_stride_bytes, dst, dst_stride_bytes, inter, row_bytes, static_cast<cudaStream_t>(stream)); });
}

int32_t sepal_b200_float_to_half(const float* src, void* dst, uint64_t count, void* stream) {
    return guarded([&] {
        if (count != 0) {
            require(src, "src");
            require(dst, "dst");
        }
        launch_float_to_half(src, dst, count, static_cast<cudaStream_t>(stream));
    });
}
int32_t sepal_b200_half_to_float(const void* src, float* dst, uint64_t count, void* stream) {
    return guarded([&] {
        if (count != 0) {
            require(src, "src");
            require(dst, "dst");
        }
        launch_half_to_float(src, dst, count, static_cast<cudaStream_t>(stream));
    });
}

int32_t sepal_b200_embed(const void* table_half, const uint32_t* tokens, float* x, uint64_t rows, uint64_t hidden, uint64_t vocab, void* stream) {
    return guarded([&] {
        if (rows != 0) {
            require(table_half, "table");
            require(tokens, "tokens");
            require(x, "x");
        }
        launch_embed(table_half, tokens, x, rows, hidden, vocab, static_cast<cudaStream_t>(stream));
    });
}
int32_t sepal_b200_embed_rms_norm_half(const void* table_half, const uint32_t* tokens, float* x, const float* w, void* y_half, uint64_t ld_y, uint64_t rows,
                                       uint64_t hidden, uint64_t vocab, float eps, void* stream) {
    return guarded([&] {
        if (rows != 0) {
            require(table_half, "table");
            require(tokens, "tokens");
            require(x, "x");
            require(w, "w");
            require(y_half, "y");
        }
        launch_embed_rms_norm_half(table_half, tokens, x, w, y_half, ld_y, rows, hidden, vocab, eps, static_cast<cudaStream_t>(stream));
    });
}
int32_t sepal_b200_rms_norm_half(const float* x, uint64_t ld_x, const float* w, void* y_half, uint64_t ld_y, uint64_t rows, uint64_t cols, float eps,
                                 void* stream) {
    return guarded([&] {
        if (rows != 0) {
            require(x, "x");
            require(w, "w");
            require(y_half, "y");
        }
        launch_rms_norm_half(x, ld_x, w, y_half, ld_y, rows, cols, eps, static_cast<cudaStream_t>(stream));
    });
}

namespace {
TrunkConfig trunk_config_of(const sepal_b200_trunk_config& config) {
    TrunkConfig c;
    c.layers = config.layers;
    c.hidden = config.hidden;
    c.intermediate = config.intermediate;
    c.vocab = config.vocab;
    c.attn_q = config.attn_q;
    c.attn_kv = config.attn_kv;
    c.dn_in = config.dn_in;
    c.dn_v_offset = config.dn_v_offset;
    c.dn_v = config.dn_v;
    c.max_call_tokens = config.max_call_tokens;
    c.mlp_int8 = config.mlp_int8;
    c.eps = config.eps;
    c.seed = config.seed;
    c.attn_o = config.attn_o;
    c.attn_heads = config.attn_heads;
    c.attn_kv_heads = config.attn_kv_heads;
    c.attn_head_dim = config.attn_head_dim;
    c.attn_rotary_dims = config.attn_rotary_dims;
    if (config.rope_theta > 0.0) c.rope_theta = config.rope_theta;
    c.dn_key_heads = config.dn_key_heads;
    c.dn_value_heads = config.dn_value_heads;
    if (config.dn_conv_kernel != 0) c.dn_conv_kernel = config.dn_conv_kernel;
    return c;
}
}  // namespace

struct sepal_b200_checkpoint {
    std::shared_ptr<const Checkpoint> checkpoint;
    std::vector<std::string> names;  // engine names, sorted
};

namespace {
AttentionShape attention_shape_of(const sepal_b200_attention_shape& s) {
    AttentionShape a;
    a.heads = s.heads;
    a.kv_heads = s.kv_heads;
    a.head_dim = s.head_dim;
    a.rotary_dims = s.rotary_dims;
    a.rope_theta = s.rope_theta;
    a.eps = s.eps;
    return a;
}
static_assert(sizeof(sepal_b200_attention_row) == sizeof(AttentionRow), "the row tables must have one layout");
}  // namespace

int32_t sepal_b200_attention_prepare(sepal_b200_ctx* ctx, const sepal_b200_attention_shape* shape, const sepal_b200_attention_row* rows, uint64_t n_rows,
                                     const void* q_gate, uint64_t q_gate_stride, int32_t q_gate_half, const void* k, uint64_t k_stride, int32_t k_half,
                                     const void* v, uint64_t v_stride, int32_t v_half, const float* q_norm, const float* k_norm, void* q_out,
                                     uint64_t q_stride, void* k_arena, void* v_arena, uint64_t arena_tokens, void* stream) {
    return guarded([&] {
        require(ctx, "ctx");
        require(shape, "shape");
        launch_attention_prepare(ctx->ctx, attention_shape_of(*shape), reinterpret_cast<const AttentionRow*>(rows), n_rows, Band{q_gate, q_gate_stride, q_gate_half != 0},
                                 Band{k, k_stride, k_half != 0}, Band{v, v_stride, v_half != 0}, q_norm, k_norm, q_out, q_stride, k_arena, v_arena, arena_tokens,
                                 static_cast<cudaStream_t>(stream));
    });
}
int32_t sepal_b200_attention(sepal_b200_ctx* ctx, const sepal_b200_attention_shape* shape, const sepal_b200_attention_row* rows, uint64_t n_rows,
                             uint64_t n_tokens, const void* q, uint64_t q_stride, const void* k_arena, const void* v_arena, uint64_t arena_tokens,
                             const void* gate, uint64_t gate_stride, int32_t gate_half, void* out, uint64_t out_stride, void* stream) {
    return guarded([&] {
        require(ctx, "ctx");
        require(shape, "shape");
        launch_attention(ctx->ctx, attention_shape_of(*shape), reinterpret_cast<const AttentionRow*>(rows), n_rows, n_tokens, q, q_stride, k_arena, v_arena,
                         arena_tokens, Band{gate, gate_stride, gate_half != 0}, out, out_stride, static_cast<cudaStream_t>(stream));
    });
}

static_assert(sizeof(sepal_b200_deltanet_row) == sizeof(DeltaNetRow), "the row tables must have one layout");

int32_t sepal_b200_deltanet(sepal_b200_ctx* ctx, const sepal_b200_deltanet_shape* shape, const sepal_b200_deltanet_row* rows, uint64_t n_rows,
                            const void* mixed, uint64_t mixed_stride, const void* z, uint64_t z_stride, const void* b, uint64_t b_stride, const void* a,
                            uint64_t a_stride, int32_t bands_half, const float* conv, const float* a_log, const float* dt_bias, const float* norm,
                            float* scratch, float* states, float* tails, uint64_t slots, void* out, uint64_t out_stride, void* stream) {
    return guarded([&] {
        require(ctx, "ctx");
        require(shape, "shape");
        DeltaNetShape s;
        s.key_heads = shape->key_heads;
        s.value_heads = shape->value_heads;
        s.head_dim = shape->head_dim;
        s.conv_kernel = shape->conv_kernel;
        s.eps = shape->eps;
        if (n_rows != 0) {
            require(rows, "rows");
            require(scratch, "scratch");
        }
        std::size_t tokens = 0;
        if (n_rows != 0) tokens = static_cast<std::size_t>(rows[n_rows - 1].q_begin) + rows[n_rows - 1].length;
        const DeltaNetScratch sc = deltanet_scratch(scratch, s, tokens);
        const bool half = bands_half != 0;
        launch_deltanet(ctx->ctx, s, reinterpret_cast<const DeltaNetRow*>(rows), n_rows, Band{mixed, mixed_stride, half}, Band{z, z_stride, half},
                        Band{b, b_stride, half}, Band{a, a_stride, half}, DeltaNetWeights{conv, a_log, dt_bias, norm}, sc, states, tails, slots, out,
                        out_stride, static_cast<cudaStream_t>(stream));
    });
}

int32_t sepal_b200_trunk_open(int32_t device, const sepal_b200_trunk_config* config, sepal_b200_trunk** out) {
    if (out != nullptr) *out = nullptr;
    return guarded([&] {
        require(out, "out");
        require(config, "config");
        *out = new sepal_b200_trunk(device, trunk_config_of(*config), nullptr);
    });
}
int32_t sepal_b200_trunk_open_checkpoint(int32_t device, const sepal_b200_trunk_config* config, const sepal_b200_checkpoint* checkpoint,
                                         sepal_b200_trunk** out) {
    if (out != nullptr) *out = nullptr;
    return guarded([&] {
        require(out, "out");
        require(config, "config");
        require(checkpoint, "checkpoint");
        *out = new sepal_b200_trunk(device, trunk_config_of(*config), checkpoint->checkpoint.get());
    });
}
int32_t sepal_b200_trunk_save(sepal_b200_trunk* trunk, const char* path) {
    return guarded([&] {
        require(trunk, "trunk");
        require(path, "path");
        trunk->trunk.save(path);
    });
}

int32_t sepal_b200_checkpoint_open(const char* path, sepal_b200_checkpoint** out) {
    if (out != nullptr) *out = nullptr;
    return guarded([&] {
        require(out, "out");
        require(path, "path");
        auto handle = std::make_unique<sepal_b200_checkpoint>();
        handle->checkpoint = Checkpoint::open(path);
        handle->names = handle->checkpoint->names();
        *out = handle.release();
    });
}
void sepal_b200_checkpoint_close(sepal_b200_checkpoint* checkpoint) { delete checkpoint; }
int32_t sepal_b200_checkpoint_count(const sepal_b200_checkpoint* checkpoint, uint64_t* count) {
    return guarded([&] {
        require(checkpoint, "checkpoint");
        require(count, "count");
        *count = checkpoint->names.size();
    });
}
int32_t sepal_b200_checkpoint_tensor(const sepal_b200_checkpoint* checkpoint, uint64_t index, const char* name, sepal_b200_tensor_info* info) {
    return guarded([&] {
        require(checkpoint, "checkpoint");
        require(info, "info");
        const TensorView* t = nullptr;
        if (name != nullptr) {
            t = &checkpoint->checkpoint->at(name);
        } else {
            if (index >= checkpoint->names.size()) throw std::out_of_range("the checkpoint has " + std::to_string(checkpoint->names.size()) + " tensors");
            t = &checkpoint->checkpoint->at(checkpoint->names[index]);
        }
        if (t->shape.size() > 8) throw std::length_error("tensor '" + t->name + "' has more than 8 dimensions");
        std::memset(info, 0, sizeof *info);
        const std::string& prefix = checkpoint->checkpoint->prefix();
        const std::string engine_name = t->name.compare(0, prefix.size(), prefix) == 0 ? t->name.substr(prefix.size()) : t->name;
        std::strncpy(info->name, engine_name.c_str(), sizeof info->name - 1);
        info->dtype = static_cast<int32_t>(t->type);
        info->rank = static_cast<uint32_t>(t->shape.size());
        for (std::size_t d = 0; d < t->shape.size(); ++d) info->shape[d] = t->shape[d];
        info->data = t->data;
        info->bytes = t->bytes;
    });
}
int32_t sepal_b200_checkpoint_metadata(const sepal_b200_checkpoint* checkpoint, const char* key, char* buffer, uint64_t capacity, uint64_t* needed) {
    return guarded([&] {
        require(checkpoint, "checkpoint");
        require(key, "key");
        const std::string value = std::string(key) == "__prefix__" ? checkpoint->checkpoint->prefix() : checkpoint->checkpoint->metadata(key);
        if (needed != nullptr) *needed = value.size() + 1;
        if (buffer != nullptr) {
            if (capacity < value.size() + 1) throw std::length_error("buffer too small: " + std::to_string(value.size() + 1) + " bytes needed");
            std::memcpy(buffer, value.c_str(), value.size() + 1);
        }
    });
}
int32_t sepal_b200_tensor_file_write(const char* path, uint64_t n, const sepal_b200_tensor_info* tensors, uint64_t n_metadata, const char* const* keys,
                                     const char* const* values) {
    return guarded([&] {
        require(path, "path");
        if (n != 0) require(tensors, "tensors");
        std::vector<TensorToWrite> out;
        for (uint64_t i = 0; i < n; ++i) {
            const sepal_b200_tensor_info& t = tensors[i];
            if (t.rank > 8 || t.dtype < 0 || t.dtype > 12) throw std::invalid_argument("tensor " + std::to_string(i) + ": bad rank or element type");
            out.push_back(TensorToWrite{std::string(t.name), static_cast<ElementType>(t.dtype), std::vector<std::uint64_t>(t.shape, t.shape + t.rank), t.data});
        }
        std::map<std::string, std::string> meta;
        for (uint64_t i = 0; i < n_metadata; ++i) meta[keys[i]] = values[i];
        write_tensor_file(path, out, meta);
    });
}

int32_t sepal_b200_model_preset(const char* name, sepal_b200_model* out) {
    return guarded([&] {
        require(name, "name");
        require(out, "out");
        const std::optional<ModelGeometry> g = find_model(name);
        if (!g) throw std::invalid_argument(std::string("no model preset '") + name + "' (0.8b, 2b, 4b, 9b)");
        out->layers = g->layers;
        out->hidden = g->hidden;
        out->intermediate = g->intermediate;
        out->vocab = g->vocab;
        out->attn_heads = g->attn_heads;
        out->attn_kv_heads = g->attn_kv_heads;
        out->attn_head_dim = g->attn_head_dim;
        out->dn_key_heads = g->dn_key_heads;
        out->dn_value_heads = g->dn_value_heads;
        out->dn_key_head_dim = g->dn_key_head_dim;
        out->dn_value_head_dim = g->dn_value_head_dim;
        out->conv_kernel = g->conv_kernel;
        out->attention_interval = g->attention_interval;
    });
}
int32_t sepal_b200_plan_weight_bytes(const sepal_b200_model* model, const char* profile, uint64_t* bytes) {
    return guarded([&] {
        require(model, "model");
        require(profile, "profile");
        require(bytes, "bytes");
        const std::optional<StorageProfile> p = find_profile(profile);
        if (!p) throw std::invalid_argument(std::string("no storage profile '") + profile + "' (w16, w8, gpu-f16, gpu-q8w, cpu-q8, gpu-bf16, gpu-w8g)");
        ModelGeometry g;
        g.layers = model->layers;
        g.hidden = model->hidden;
        g.intermediate = model->intermediate;
        g.vocab = model->vocab;
        g.attn_heads = model->attn_heads;
        g.attn_kv_heads = model->attn_kv_heads;
        g.attn_head_dim = model->attn_head_dim;
        g.dn_key_heads = model->dn_key_heads;
        g.dn_value_heads = model->dn_value_heads;
        g.dn_key_head_dim = model->dn_key_head_dim;
        g.dn_value_head_dim = model->dn_value_head_dim;
        g.conv_kernel = model->conv_kernel;
        g.attention_interval = model->attention_interval;
        *bytes = trunk_weight_bytes(g, *p);
    });
}

void sepal_b200_trunk_close(sepal_b200_trunk* trunk) { delete trunk; }
int32_t sepal_b200_trunk_run(sepal_b200_trunk* trunk, const uint32_t* tokens, uint64_t n, float* last_hidden, float* all_hidden, double* times_ms) {
    return guarded([&] {
        require(trunk, "trunk");
        trunk->trunk.run(tokens, n, last_hidden, all_hidden, times_ms);
    });
}
int32_t sepal_b200_trunk_score(sepal_b200_trunk* trunk, uint64_t n_requests, const uint32_t* tokens, const uint64_t* offsets, float* last_hidden,
                               double* times_s) {
    return guarded([&] {
        require(trunk, "trunk");
        trunk->trunk.score(n_requests, tokens, offsets, last_hidden, times_s);
    });
}
int32_t sepal_b200_trunk_weight(sepal_b200_trunk* trunk, uint32_t layer, int32_t which, void* host_out, uint64_t capacity, uint64_t* needed) {
    return guarded([&] {
        require(trunk, "trunk");
        if (which < 0 || which > 14) throw std::invalid_argument("which must be 0 .. 14");
        const std::size_t bytes = trunk->trunk.weight(layer, static_cast<TrunkWeight>(which), host_out, capacity);
        if (needed != nullptr) *needed = bytes;
    });
}
int32_t sepal_b200_trunk_info(sepal_b200_trunk* trunk, uint64_t* gemm_flops_per_token, uint64_t* weight_bytes) {
    return guarded([&] {
        require(trunk, "trunk");
        if (gemm_flops_per_token != nullptr) *gemm_flops_per_token = trunk->trunk.gemm_flops_per_token();
        if (weight_bytes != nullptr) *weight_bytes = trunk->trunk.weight_bytes();
    });
}

int32_t sepal_b200_provider_open(int32_t device, uint64_t arena_bytes, sepal_b200_provider** out) {
    if (out != nullptr) *out = nullptr;
    return guarded([&] {
        require(out, "out");
        *out = new sepal_b200_provider(device, static_cast<std::size_t>(arena_bytes));
    });
}
void sepal_b200_provider_close(sepal_b200_provider* provider) { delete provider; }

int32_t sepal_b200_provider_upload_weights(sepal_b200_provider* provider, const void* w, int32_t dtype, uint64_t n, uint64_t k, uint32_t* id_out) {
    return guarded([&] {
        require(provider, "provider");
        require(id_out, "id_out");
        *id_out = provider->gemm.upload_weights(w, host_type_of(dtype), n, k).index;
    });
}
int32_t sepal_b200_provider_upload_weights_w8g(sepal_b200_provider* provider, const float* w, uint64_t n, uint64_t k, uint32_t* id_out) {
    return guarded([&] {
        require(provider, "provider");
        require(id_out, "id_out");
        *id_out = provider->gemm.upload_weights_w8g(w, n, k).index;
    });
}
int32_t sepal_b200_provider_gemm_f(sepal_b200_provider* provider, const void* x, int32_t x_dtype, uint64_t t, uint32_t weight_id, float* y, float beta) {
    return guarded([&] {
        require(provider, "provider");
        provider->gemm.gemm_f(x, host_type_of(x_dtype), t, WeightId{weight_id}, y, beta);
    });
}

int32_t sepal_b200_host_alloc(uint64_t bytes, void** out) {
    if (out != nullptr) *out = nullptr;
    return guarded([&] {
        require(out, "out");
        check(cudaMallocHost(out, bytes), "cudaMallocHost");
    });
}
void sepal_b200_host_free(void* ptr) {
    if (ptr != nullptr) (void)cudaFreeHost(ptr);
}

}  // extern "C"
