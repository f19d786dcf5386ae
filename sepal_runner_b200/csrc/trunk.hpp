// A synthetic hybrid trunk made of the projection GEMMs only: the caller of the hot path, laid out as the reference's layer loop
// (runner/cuda/src/cuda_engine.cpp:1724-1952) with the mixer cores (attention, gated delta rule) replaced by a fixed wiring, so
// that a whole forward pass is the chain of GEMMs and the small element-wise kernels between them:
//
//   x (float32 residual) = embedding[token]
//   per layer:  a1 = rmsnorm(x) (binary16)
//               attention layer:  p = a1 [q; k; v]^T (binary16);  x += p[:, 0:q] o^T                 (the o projection reads the q band)
//               DeltaNet layer:   p = a1 in^T (binary16);         x += p[:, v0:v0+vk] out^T          (the out projection reads the v band)
//               a1 = rmsnorm(x);  a3 = silu(gate) * up of a1 [gate; up]^T (fused epilogue, binary16);  x += a3 down^T (fused residual)
//
// Every fourth layer (layer % 4 == 3) is an attention layer, the others DeltaNet layers (the 3 : 1 pattern of the reference's presets,
// runner/src/core/config.cpp:119). Weights are random N(0, 0.02), rounded to bfloat16 and stored as binary16; the MLP weights can be
// stored as int8 groups instead. Tokens of a request are processed in calls of at most `max_call_tokens` rows, as the reference cuts a
// long request into segments (runner/cuda/src/gpu_decision_engine.cpp:233-245); with the mixer cores wired out the calls are independent.
// Nothing is allocated after construction.
#pragma once

#include <cstddef>
#include <cstdint>
#include <vector>

#include <cuda_runtime.h>

#include "attention.hpp"
#include "checkpoint.hpp"
#include "deltanet.hpp"

#include "gemm.hpp"

namespace sepal::b200 {

struct TrunkConfig {
    std::uint32_t layers = 36, hidden = 2560, intermediate = 9728, vocab = 151936;
    std::uint32_t attn_q = 4096, attn_kv = 1024;           // q width; k and v width each
    std::uint32_t dn_in = 8192, dn_v_offset = 4096, dn_v = 2048;  // fused in-projection width; the band the out-projection reads
    std::uint32_t max_call_tokens = 4096;
    std::uint32_t mlp_int8 = 0;                             // 1: gate_up and down stored as int8 groups
    float eps = 1e-6f;
    std::uint64_t seed = 1;
    std::uint32_t attn_o = 0;                               // width the attention out-projection reads (0: attn_q); q_proj may carry a gate
    // attn_heads > 0: the attention layers run the real core between their projections (norm, RoPE, cache, causal grouped-query
    // attention, output gate) instead of the fixed wiring; then attn_q = 2 * heads * head_dim (query and gate), attn_kv = kv_heads *
    // head_dim, attn_o = heads * head_dim.
    std::uint32_t attn_heads = 0, attn_kv_heads = 0, attn_head_dim = 0, attn_rotary_dims = 0;
    // dn_value_heads > 0: the DeltaNet layers run the real core (convolution, gated delta rule, gated norm) instead of the fixed wiring;
    // then dn_in = 2 key_dim + 2 value_dim + 2 value_heads ([qkv; z; b; a]) and dn_v = value_dim, with heads of 128.
    std::uint32_t dn_key_heads = 0, dn_value_heads = 0, dn_conv_kernel = 4;
    double rope_theta = 1.0e7;
};

/// The value of the "format" metadata key of a file written by Trunk::save.
extern const char* const kSavedFormat;

enum class TrunkWeight : int { Embedding = 0, NormIn = 1, MixIn = 2, MixOut = 3, NormPost = 4, GateUp = 5, Down = 6, QNorm = 7, KNorm = 8, DnConv = 9, DnALog = 10, DnDtBias = 11, DnNorm = 12,
                               GateUpScales = 13, DownScales = 14 };  // mlp_int8: the quantiser's float32 scales, [rows, k / 128]

class Trunk {
public:
    /// Random weights (N(0, 0.02) on the bfloat16 grid, from config.seed), or, with a checkpoint, the weights it holds: either the
    /// reference's tensor names (embed_tokens.weight, layers.N.input_layernorm.weight, ...self_attn.{q,k,v,o}_proj.weight,
    /// ...linear_attn.{in_proj_qkv,in_proj_z,in_proj_b,in_proj_a,out_proj}.weight, ...mlp.{gate,up,down}_proj.weight), stacked, converted,
    /// interleaved and quantised as the reference's placement does (runner/cuda/src/cuda_engine.cpp:525-711), or a file written by save().
    Trunk(int device, const TrunkConfig& config, const Checkpoint* checkpoint = nullptr);
    ~Trunk();
    Trunk(const Trunk&) = delete;
    Trunk& operator=(const Trunk&) = delete;

    /// One request: `n` token ids on the host. Writes the final hidden state of the last token to last_hidden (hidden floats, host)
    /// and, when all_hidden is not null, of every token ([n, hidden], host). Returns when the results are on the host.
    /// times_ms (optional, 2 doubles): device time of the whole request and of its GEMM launches (CUDA events).
    void run(const std::uint32_t* tokens, std::size_t n, float* last_hidden, float* all_hidden, double* times_ms);

    /// Many requests in one go, packed into calls the way the reference's engine packs them (runner/cuda/src/gpu_decision_engine.cpp:
    /// 233-266): a request longer than max_call_tokens is cut into segments of that many tokens, and the segments, in the order of the
    /// requests, fill a call until the next one does not fit (or the call has kMaxCallRows of them). tokens holds all requests end to end,
    /// offsets[r] .. offsets[r + 1] being request r (the flat arrays of sepal_score, runner/include/sepal/c_api.h:46-60). Writes the final
    /// hidden state of each request's last token to last_hidden [n_requests, hidden] (host) and, when times_s is not null, the seconds
    /// from the start of the call until each request's result was complete on the device. The projections see the rows of a call as one
    /// matrix, so short requests share the large-M efficiency of a full call.
    static constexpr std::size_t kMaxCallRows = 64;
    void score(std::size_t n_requests, const std::uint32_t* tokens, const std::uint64_t* offsets, float* last_hidden, double* times_s);

    /// Writes the weights as they are placed on the device (stacked, interleaved, quantised) to one file in the checkpoint format, so
    /// that the next start copies them to the device as they are. Tensors start on 256-byte boundaries of the file.
    void save(const std::string& path);

    /// A weight as stored (binary16, or float32 for the norms), copied to the host: for parity checks. Returns the byte size.
    std::size_t weight(std::uint32_t layer, TrunkWeight which, void* host_out, std::size_t capacity);

    const TrunkConfig& config() const { return cfg_; }
    std::uint64_t gemm_flops_per_token() const;
    std::size_t weight_bytes() const { return weight_bytes_; }

private:
    struct Layer {
        bool attention = false;
        float* norm_in = nullptr;
        float* norm_post = nullptr;
        void* mix_in = nullptr;   // binary16 [mix_in_n, hidden]
        void* mix_out = nullptr;  // binary16 [hidden, mix_out_k]
        std::uint32_t mix_in_n = 0, mix_out_k = 0, band = 0;
        void* gate_up = nullptr;  // binary16 packed [2 I, hidden] (mlp_int8: int8)
        void* down = nullptr;     // binary16 [hidden, I] (mlp_int8: int8)
        W8gMatrix gate_up_q, down_q;
        float* q_norm = nullptr;  // attention layers with the real core: per-head norm weights [head_dim]
        float* k_norm = nullptr;
        float* dn_conv = nullptr;     // DeltaNet layers with the real core: [conv_dim, taps], [value heads], [value heads], [128]
        float* dn_a_log = nullptr;
        float* dn_dt_bias = nullptr;
        float* dn_norm = nullptr;
        float* dn_states = nullptr;   // [slots, value heads, 128, 128]: the requests being served
        float* dn_tails = nullptr;    // [slots, taps - 1, conv_dim]
        void* k_cache = nullptr;  // binary16 [arena tokens, kv width]: the keys (normed, rotated) and values of the requests being served
        void* v_cache = nullptr;
        float* gate_up_scales = nullptr;  // mlp_int8: the quantiser's float32 scales [2 I, hidden / 128] and [hidden, I / 128]
        float* down_scales = nullptr;
    };
    void* alloc(std::size_t bytes);
    void place_random();
    void place_checkpoint(const Checkpoint& checkpoint);
    void place_saved(const Checkpoint& checkpoint);
    void shape_layer(std::uint32_t l);
    void prepare_mlp_scales(Layer& L);
    void forward_call(const std::uint32_t* tokens_dev, std::size_t rows, const std::vector<AttentionRow>& runs, const std::vector<DeltaNetRow>& dn_runs);
    void reserve_cache(std::size_t tokens);
    void reserve_states(std::size_t slots);
    bool real_attention() const { return cfg_.attn_heads != 0; }
    bool real_deltanet() const { return cfg_.dn_value_heads != 0; }
    DeltaNetShape deltanet_shape() const;

    TrunkConfig cfg_;
    Context ctx_;
    cudaStream_t stream_ = nullptr;
    cudaEvent_t ev_[4] = {};
    std::vector<void*> allocations_;
    std::vector<Layer> layers_;
    void* embedding_ = nullptr;  // binary16 [vocab, hidden]
    float* x_ = nullptr;         // [max_call_tokens, hidden]
    void* a1_ = nullptr;         // binary16 [max_call_tokens, hidden]
    void* p_ = nullptr;          // binary16 [max_call_tokens, p_width]
    void* a3_ = nullptr;         // binary16 [max_call_tokens, intermediate]
    void* q_ = nullptr;          // binary16 [max_call_tokens, attn_o]: normed, rotated queries
    void* a2_ = nullptr;         // binary16 [max_call_tokens, attn_o]: the attention output, o_proj's operand
    std::size_t cache_tokens_ = 0;
    std::size_t state_slots_ = 0;
    float* dn_scratch_ = nullptr;  // q, k, v, decay, beta of one call
    std::uint32_t* tokens_dev_ = nullptr;     // two buffers of max_call_tokens: a call's ids are copied while the call before it runs
    std::uint32_t* tokens_pinned_ = nullptr;  // likewise
    float* out_pinned_ = nullptr;             // kMaxCallRows rows of hidden floats, twice
    cudaEvent_t call_done_[2] = {};
    std::uint32_t p_width_ = 0;
    std::size_t weight_bytes_ = 0;
    double gemm_ms_ = 0.0;
};

/// Element-wise kernels of the trunk (also used by tests): token embedding gather and the zero-centred RMSNorm of the reference
/// (y = x / sqrt(mean(x^2) + eps) * (1 + w), runner/cuda/src/kernels_elementwise.hpp:41-46), float32 in, binary16 out.
void launch_embed(const void* table_half, const std::uint32_t* tokens, float* x, std::size_t rows, std::size_t hidden, std::size_t vocab, cudaStream_t stream);
/// Both at once for the first layer: x[t, :] = table[tokens[t], :] widened, y = norm(x) with the weight w, one pass over the row.
void launch_embed_rms_norm_half(const void* table_half, const std::uint32_t* tokens, float* x, const float* w, void* y_half, std::size_t ld_y, std::size_t rows,
                                std::size_t hidden, std::size_t vocab, float eps, cudaStream_t stream);
void launch_rms_norm_half(const float* x, std::size_t ld_x, const float* w, void* y_half, std::size_t ld_y, std::size_t rows, std::size_t cols, float eps,
                          cudaStream_t stream);
/// Normal(0, stddev) values from a counter-based generator (seed, element index), rounded to bfloat16 and stored as binary16 / float32.
void launch_fill_normal_half(void* dst_half, std::size_t count, std::uint64_t seed, float stddev, cudaStream_t stream);
void launch_fill_normal_float(float* dst, std::size_t count, std::uint64_t seed, float stddev, cudaStream_t stream);

}  // namespace sepal::b200
