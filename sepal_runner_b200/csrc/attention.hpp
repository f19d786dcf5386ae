// The core of the full-attention mixer between its projections: per-head RMSNorm of q and k, partial RoPE, the keys and values of the
// run appended to the request's cache, causal grouped-query attention over the request's earlier tokens and the run itself, and the
// output gate. The arithmetic is the reference's (runner/include/sepal/ref/attention.hpp:33-235; device contract
// runner/cuda/src/kernels_attention.hpp:1-206): q_proj's output holds, per head, the query then its gate; the norm is
// x / sqrt(mean(x^2) + eps) * (1 + w) over the head; the first rotary_dims of a head rotate, dimension i paired with i + rotary_dims / 2,
// by position * theta^(-2 i / rotary_dims) (angles in float64); query head h reads key/value head h / (heads / kv_heads); scores are
// scaled by 1 / sqrt(head_dim); the attended vector is multiplied by sigmoid(gate) and handed to o_proj as binary16.
//
// Layout. A call holds runs ("rows") of consecutive tokens of different requests in one flat token list. Keys and values live in one
// arena per layer, [arena tokens, kv_heads * head_dim] binary16 each; a request owns a contiguous range of it, so a run's keys are its
// request's range up to the run's last token (the reference chains segments instead, kernels_attention.hpp:17-33; a contiguous range
// is what a chain of calls over one request amounts to). The arena must hold finite numbers everywhere (zero it once): a masked
// probability is exactly 0, and 0 times a NaN would not be.
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_runtime.h>

#include "context.hpp"

namespace sepal::b200 {

struct AttentionShape {
    std::uint32_t heads = 0, kv_heads = 0, head_dim = 0;  // head_dim 128 or 256; heads a multiple of kv_heads
    std::uint32_t rotary_dims = 0;                          // even, at most head_dim
    double rope_theta = 1.0e7;
    float eps = 1.0e-6f;
};

struct AttentionRow {
    std::uint32_t q_begin;   // the run's first token in the flat list of the call
    std::uint32_t length;    // its tokens
    std::uint32_t kv_begin;  // where its request's keys and values start in the arena (a token index)
    std::uint32_t context;   // tokens of the request that precede the run (already in the arena); the position of the run's first token
};

/// A matrix of the call: element (token, c) at data[token * stride + c]; binary16 when `half`, else float32.
struct Band {
    const void* data = nullptr;
    std::size_t stride = 0;
    bool half = true;
};

/// Norm and RoPE of q and k, and the run's keys and values stored at arena rows kv_begin + context + t.
///   q_gate [N, 2 * heads * head_dim]; k, v [N, kv_heads * head_dim]; q_norm, k_norm float32 [head_dim] (device);
///   q_out binary16 [N, heads * head_dim] with row stride q_stride; k_arena, v_arena binary16 [arena tokens, kv_heads * head_dim].
/// `rows` is a HOST array (sorted by q_begin, runs adjacent); it is copied to the context's table on the stream.
void launch_attention_prepare(Context& ctx, const AttentionShape& shape, const AttentionRow* rows, std::size_t n_rows, Band q_gate, Band k, Band v,
                              const float* q_norm, const float* k_norm, void* q_out, std::size_t q_stride, void* k_arena, void* v_arena,
                              std::size_t arena_tokens, cudaStream_t stream);

/// out[token, h * head_dim + d] = sigmoid(gate) * sum_j softmax_j(q . k_j / sqrt(head_dim)) v_j over the visible keys of the token:
/// its request's arena rows kv_begin .. kv_begin + context + t. q binary16 [N, heads * head_dim] (what the prepare launch wrote);
/// gate: the q_gate band of the prepare launch (read at column h * 2 * head_dim + head_dim + d); out binary16 [N, heads * head_dim].
/// Flash attention on the tensor cores (tcgen05.mma for Q K^T and P V, the accumulators in tensor memory, float32 online softmax):
/// one CTA per 128 queries of a run and query head, keys walked in blocks counted from the request's first token, so a token's result
/// depends on its own request alone.
void launch_attention(Context& ctx, const AttentionShape& shape, const AttentionRow* rows, std::size_t n_rows, std::size_t n_tokens, const void* q,
                      std::size_t q_stride, const void* k_arena, const void* v_arena, std::size_t arena_tokens, Band gate, void* out,
                      std::size_t out_stride, cudaStream_t stream);

bool attention_supports(const AttentionShape& shape);

}  // namespace sepal::b200
