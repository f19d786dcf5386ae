/* sepal_b200: the trunk projection GEMMs of Sepal-Runner's GPU engine, written for NVIDIA B200 (sm_100a).
 *
 * This is the whole boundary of the library: a C ABI with plain pointers and sizes. It follows the conventions of the engine's own
 * C ABI (runner/include/sepal/c_api.h:1-9,29-60): every function returns 0 on success and non-zero on failure, the message of the
 * last failure on the calling thread is at sepal_b200_last_error() (cleared by the next successful call), no exception crosses
 * the boundary, and the caller owns every buffer it passes.
 *
 * Two layers:
 *   - launchers on DEVICE pointers, one for each kernel launcher of the reference's engine that this library replaces. They enqueue
 *     on the given CUDA stream (a cudaStream_t passed as void*, NULL = the default stream) and return without waiting.
 *   - a provider on HOST pointers, the face the reference gives its cuBLAS provider (sepal::cuda::CudaGemm,
 *     runner/cuda/include/sepal/cuda/cuda_gemm.hpp:112-160): weights uploaded once, then Y = beta Y + X W^T with X uploaded and Y
 *     downloaded inside the call.
 *
 * Matrices are row-major; a matrix argument is a pointer and a row stride in elements (runner/cuda/src/device.hpp:14-16).
 *   Y[t, n] = epilogue( sum over k of X[t, k] * W[n, k] ),   X [T, K], W [N, K] (one output feature per row, K contiguous).
 *
 * There is no CPU path and no library GEMM behind these functions: on a device that is not sm_100 sepal_b200_open fails.
 */
#ifndef SEPAL_B200_H
#define SEPAL_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define SEPAL_B200_API __declspec(dllexport)
#else
#define SEPAL_B200_API __attribute__((visibility("default")))
#endif

typedef struct sepal_b200_ctx sepal_b200_ctx;
typedef struct sepal_b200_provider sepal_b200_provider;

/* Epilogues: the reference's SimtEpilogue (runner/cuda/src/gemm_simt_kernels.hpp:19-25). */
#define SEPAL_B200_STORE 0  /* Y = acc */
#define SEPAL_B200_ADD 1    /* Y = Y + acc (the residual stream updated in place; one float32 addition) */
#define SEPAL_B200_SWIGLU 2 /* W rows are [gate; up] interleaved in blocks of 64; N is the packed width 2 I, Y has I columns */

/* Element types of host matrices given to the provider (the codes of sepal::DType's float types). */
#define SEPAL_B200_F32 0
#define SEPAL_B200_F16 1

/* ---- library ------------------------------------------------------------------------------------------------------------ */

/* Version of this ABI (1). Counterpart of sepal_api_version, runner/include/sepal/c_api.h:31. */
SEPAL_B200_API int32_t sepal_b200_api_version(void);

/* Message of the calling thread's last failed call, "" after a successful one. Counterpart of sepal_last_error, c_api.h:34. */
SEPAL_B200_API const char* sepal_b200_last_error(void);

/* Creates the per-device state every launcher needs: device properties, the scratch memory of the split-k schedule
 * (`workspace_bytes`, 0 = two 128 x 256 float32 tiles per SM, about 39 MB on a B200) and the device status word. All device
 * memory the launchers ever use is allocated here, as the engine allocates its call buffers once (runner/cuda/src/cuda_engine.cpp:714-743).
 * One context serves one stream at a time: launches that overlap on the device must use different contexts.
 * On failure *out is NULL. Counterpart of the engine creation behind sepal_open, c_api.h:39. */
SEPAL_B200_API int32_t sepal_b200_open(int32_t device, uint64_t workspace_bytes, sepal_b200_ctx** out);

/* Frees a context (NULL is allowed). Counterpart of sepal_close, c_api.h:41. */
SEPAL_B200_API void sepal_b200_close(sepal_b200_ctx* ctx);

/* A JSON description of the context (device, SM count, scratch bytes, kernel names). Size-query protocol of sepal_info,
 * c_api.h:43-46: with capacity too small nothing is written, *needed gets the size including the terminator, the call fails. */
SEPAL_B200_API int32_t sepal_b200_info(sepal_b200_ctx* ctx, char* buffer, uint64_t capacity, uint64_t* needed);

/* Waits for `stream`, then reads and clears the device status word: *status_out = 0 when no kernel reported a problem, otherwise
 * the code of the first bounded wait that ran out (low byte: which wait, 1 .. 8 in the GEMM kernels, 16 .. 23 in the attention
 * kernels, 24 in the DeltaNet scan; higher bits: the CTA). A non-zero status means the
 * outputs of the launches since the last call are not to be trusted. The reference reports device faults through
 * cudaStreamSynchronize in CudaEngine::run (runner/cuda/src/cuda_engine.cpp:1969); this is the same place in the flow. */
SEPAL_B200_API int32_t sepal_b200_status(sepal_b200_ctx* ctx, void* stream, int32_t* status_out);

/* For tests of the recovery path, which no healthy launch takes: leaves the context as a kernel that gave up waiting would leave it,
 * the status word set to `code` and the first `stale_counters` tile counters non-zero (enqueued on `stream`). The next
 * sepal_b200_status then reports `code` and clears both, as after a real give-up. No counterpart in the reference. */
SEPAL_B200_API int32_t sepal_b200_debug_leave_status(sepal_b200_ctx* ctx, void* stream, int32_t code, uint32_t stale_counters);

/* Kernels of this library the calling thread has launched since the previous call of this function. */
SEPAL_B200_API uint64_t sepal_b200_take_launch_count(void);

/* Process-wide switch, on by default: the GEMM kernels (and the trunk's embedding and norm kernels) are launched as programmatic
 * dependents of the kernel before them in the stream, so a kernel's set-up overlaps the end of the one before it; each of them waits for
 * that kernel to complete before it touches global memory, so results do not change. No counterpart in the reference (whose engine
 * launches its kernels one after the other, runner/cuda/src/cuda_engine.cpp:1724-1952); off = plain stream order, for comparisons. */
SEPAL_B200_API void sepal_b200_set_launch_overlap(int32_t on);

/* The caller's promise for the multiplies it launches through `ctx` from now on (on != 0), or its withdrawal (0, the default): the
 * weight matrix of a multiply (w, or q with its scales) is not written by the kernel that runs directly before the multiply in its
 * stream. An inference engine's weights are uploaded once, so every multiply of the reference's engine qualifies
 * (CudaEngine::Impl::gemm, runner/cuda/src/cuda_engine.cpp:1093-1154, reads device copies written at load time, as
 * CudaGemm::upload_weights writes a provider's, runner/cuda/src/cuda_gemm.cpp:389-394). With the promise a kernel launched as a programmatic dependent (see above)
 * requests its first weight tiles while the kernel before it is still finishing, and waits for that kernel only before it touches the
 * activations and the result: a launch starts about a microsecond earlier. The provider and the trunk of this library, whose weights
 * are uploaded through a synchronising call, set it for their own contexts. Results do not change. */
SEPAL_B200_API int32_t sepal_b200_set_static_weights(sepal_b200_ctx* ctx, int32_t on);

/* ---- launchers on device pointers ------------------------------------------------------------------------------------------ */

/* binary16 x binary16 -> float32 accumulation on the tensor cores (tcgen05.mma), result binary16 (y_half != 0) or float32.
 * Replaces launch_gemm_nt (runner/cuda/src/gemm_kernels.hpp:22-31) and the cublasGemmEx call of CudaEngine::Impl::gemm
 * (runner/cuda/src/cuda_engine.cpp:1093-1154); the epilogues replace launch_swiglu / launch_add after it (cuda_engine.cpp:1919-1945).
 * Requires K, ld_x, ld_w multiples of 8, N and ld_y even, x and w 16-byte aligned (gemm_nt_supports, gemm_kernels.hpp:34-36);
 * SWIGLU needs N a multiple of 128. config: -1 picks the tile width and schedule from the shape; other values force one (tests and
 * tuning: 0..3, or a tile width that is a multiple of 16 up to 256, plus 1 for the even split of k, 2 for CTA pairs, 3 for both,
 * 6 for pairs that run whole tiles first and split only the last waves, and, for a float32 residual update (ADD, y_half == 0, 16-byte
 * aligned rows) only, 7 for pairs that share every tile when there are fewer tiles than pairs, or 5 for pairs that share the tiles
 * of the last, partial wave: the parts of a shared tile are added to Y one after the other in the order of their ranges of k, two
 * or three float32 additions in a fixed order instead of one; -1 takes these forms where they are the faster ones); or 512 + w (w =
 * 64, 96, ..., 192, 256 or 320) for the kernel that takes the weights as the tensor cores' first operand with w tokens to a tile,
 * which -1 takes where its tiles make one well-filled wave. t == 0 is a no-op. */
SEPAL_B200_API int32_t sepal_b200_gemm_f16(sepal_b200_ctx* ctx, const void* x, uint64_t ld_x, const void* w, uint64_t ld_w, void* y, uint64_t ld_y,
                                           int32_t y_half, uint64_t t, uint64_t n, uint64_t k, int32_t epilogue, int32_t config, void* stream);

/* The same product for callers that cannot allocate device memory. This function has NO counterpart in the reference: its engine
 * allocates its buffers itself at creation. It exists for hosts that may not call cudaMalloc once they are running - a process
 * that gave all device memory to its own pool at start-up, a plug-in whose host forbids allocation after initialisation, code
 * that runs while another component holds the allocator. It takes no context: the scratch of the split-k schedule (partial tiles,
 * tile counters, the status word) is a fixed array of 20 MiB + 17 KiB inside the library, held by every GPU that loads the library
 * until the process exits. It calls no cudaMalloc, cudaFree or allocating library routine, on any call.
 *   - Runs on the CURRENT device, with 128 x 128 tiles and the even split of all k iterations (the schedule that uses the scratch).
 *   - Limit: ceil(T / 128) * ceil(N / 128) <= 4096 output tiles (for example T = 4096 with N = 16384); a larger product fails with a
 *     message and nothing is launched. Otherwise the requirements of sepal_b200_gemm_f16.
 *   - The first call on a device resolves the array's device address and reads the device's properties; make that call before
 *     any stream capture begins.
 *   - All calls share the one array. Each call first clears the counters and the status word on `stream` (the array keeps what the
 *     previous call left); two calls that overlap on the device (different streams, different threads) race on it and give
 *     wrong results: keep every call of this function on one stream, or order them yourself.
 *   - status_out == NULL: enqueue and return; a status such a call leaves is lost, because the next call clears the word before it
 *     launches: pass status_out on the call whose result you are about to trust. Otherwise the call waits for `stream` and stores
 *     the kernel status word (0 = every wait completed; see sepal_b200_status).
 *   - One CTA per SM runs (each leaves at most two partial tiles of 128 x 128 floats in the array, which holds 160 CTAs' worth). */
SEPAL_B200_API int32_t sepal_b200_gemm_f16_noalloc(const void* x, uint64_t ld_x, const void* w, uint64_t ld_w, void* y, uint64_t ld_y,
                                                   int32_t y_half, uint64_t t, uint64_t n, uint64_t k, int32_t epilogue, void* stream,
                                                   int32_t* status_out);

/* binary16 activations x int8 weights with one scale per output row and group of 128 values of k (the gpu-w8g layout). Replaces
 * launch_gemm_simt with SimtWeight::Int8Group (runner/cuda/src/gemm_simt_kernels.hpp:42-56). q is int8 [N, ld_q]; scales_t / descale come from sepal_b200_prepare_w8g_scales.
 * Requires K a multiple of 128, ld_x a multiple of 8, ld_q a multiple of 16, scales_t 16-byte aligned with ld_st >= N rounded up to
 * 256 (the padding zero). config as sepal_b200_gemm_f16, and 512 + w (w = 64, 96, ..., 192, 256 or 320) forces the kernel that takes the
 * weights as the tensor cores' first operand with w tokens to a tile, which -1 picks where it is the faster one; 512 + w + 1 (a
 * float32 result, stored or added, in 16-byte aligned rows; a last wave of fewer tiles than CTA pairs) forces its shared form, in which
 * the CTA pairs that would idle in that wave take the first scale groups of each of its tiles: Y becomes (Y + the first groups' product) + the other groups' product
 * (without the Y for a stored result), float32 additions in a fixed order (-1 takes this form where it is the faster one). */
SEPAL_B200_API int32_t sepal_b200_gemm_w8g(sepal_b200_ctx* ctx, const void* x, uint64_t ld_x, const int8_t* q, uint64_t ld_q, const void* scales_t,
                                           uint64_t ld_st, const float* descale, void* y, uint64_t ld_y, int32_t y_half, uint64_t t, uint64_t n,
                                           uint64_t k, int32_t epilogue, int32_t config, void* stream);

/* Which kernel the automatic schedule (config -1) of sepal_b200_gemm_w8g gives a [t x k] by [n x k] multiply on a GPU of `sm_count` SMs:
 * the tokens to a tile of the swapped kernel (96, 128, 160 or 192: one block; 256 or 320: two blocks of half as many that share the
 * converted weights; sepal_b200_gemm_w8g's config 512 + w forces it), or 0 for the unswapped kernels. `epilogue` as in the multiply;
 * `staged` != 0: the result goes into 16-byte aligned rows and is neither a float32 SwiGLU nor a binary16 residual update (it then
 * leaves through shared memory and the TMA, which the estimate counts). Host arithmetic only: needs no GPU and no context. No counterpart in the reference. */
SEPAL_B200_API int32_t sepal_b200_w8g_schedule(uint32_t sm_count, uint64_t t, uint64_t n, uint64_t k, int32_t epilogue, int32_t staged);

/* binary16 activations x int8 weights with ONE float32 scale per output row (the gpu-q8w layout): Y[t, n] = sw[n] * sum_k x[t, k] q[n, k].
 * Replaces launch_gemm_w8a16 (runner/cuda/src/gemm_s8_kernels.hpp:51-57; its engine use cuda_engine.cpp:1118-1129). The bytes are
 * widened exactly to binary16 on their way to the tensor cores, summed in float32, and the finished sum is multiplied by sw[n] in
 * float32, as the reference does. q is int8 [N, ld_q] in plain row-major order (the reference's S8WeightLayout::Plain; its Fp16Pairs
 * byte permutation serves its own mma.sync fragments and has no use here). Requires K a multiple of 128, ld_x a multiple of 8, ld_q a
 * multiple of 16, N at most 65536. Epilogues and `config` as sepal_b200_gemm_w8g. */
SEPAL_B200_API int32_t sepal_b200_gemm_w8r(sepal_b200_ctx* ctx, const void* x, uint64_t ld_x, const int8_t* q, uint64_t ld_q, const float* sw, void* y,
                                           uint64_t ld_y, int32_t y_half, uint64_t t, uint64_t n, uint64_t k, int32_t epilogue, int32_t config,
                                           void* stream);

/* Per-output-row int8 quantisation of a binary16 weight matrix w [N, ld_w], bit for bit launch_quantize_weights_s8 with the Plain layout
 * (runner/cuda/src/gemm_s8_kernels.hpp:36-41, gemm_s8_kernels.cu:28-31,83-118): scales[r] = max|w[r, :]| / 127, q[r, c] = round to
 * nearest even of w[r, c] * (127 / max), clamped to [-127, 127]; a zero row gets scale 0 and zeros. col_scale: NULL, or K floats by
 * which the columns are multiplied in float32 first (the smoothing factors). K, ld_w and ld_q multiples of 16. */
SEPAL_B200_API int32_t sepal_b200_quantize_rows_s8(const void* w, uint64_t ld_w, int8_t* q, uint64_t ld_q, float* scales, uint64_t n, uint64_t k,
                                                   const float* col_scale, void* stream);

/* The group quantiser, bit for bit launch_quantize_group_s8 (runner/cuda/src/gemm_simt_kernels.hpp:64-65): src float32 [rows, K],
 * q int8 [rows, ld_q], s float32 [rows, ld_s] with one scale per group of 128. */
SEPAL_B200_API int32_t sepal_b200_quantize_group_s8(const float* src, uint64_t ld_src, int8_t* q, uint64_t ld_q, float* s, uint64_t ld_s,
                                                    uint64_t rows, uint64_t k, void* stream);

/* s float32 [N, ld_s] (the quantiser's layout) -> scales_t binary16 [groups, ld_st] and *descale (device float), the form the
 * tensor-core multiply reads: group-major (give it rows of ld_st >= N rounded up to 256 binary16 values, zeroed beforehand), times
 * the power of two that puts the largest scale in [128, 256). max_bits: 4 bytes of
 * device scratch. Part of weight placement, where the reference's put_simt quantises (runner/cuda/src/cuda_engine.cpp:580-627). */
SEPAL_B200_API int32_t sepal_b200_prepare_w8g_scales(const float* s, uint64_t ld_s, uint64_t n, uint64_t groups, void* scales_t, uint64_t ld_st,
                                                     float* descale, uint32_t* max_bits, void* stream);

/* dst row p = src row pack_gate_up_source(p, inter) for the 2 * inter rows of a stacked [gate; up] matrix
 * (runner/cuda/src/gemm_simt_kernels.hpp:72-77; the engine's interleave at cuda_engine.cpp:597-611). Strides and row length in bytes. */
SEPAL_B200_API int32_t sepal_b200_pack_gate_up(const void* src, uint64_t src_stride_bytes, void* dst, uint64_t dst_stride_bytes, uint64_t inter,
                                               uint64_t row_bytes, void* stream);

/* float32 <-> binary16 on the device, round to nearest even (runner/cuda/src/convert_kernels.hpp). */
SEPAL_B200_API int32_t sepal_b200_float_to_half(const float* src, void* dst, uint64_t count, void* stream);
SEPAL_B200_API int32_t sepal_b200_half_to_float(const void* src, float* dst, uint64_t count, void* stream);

/* Token embedding gather and the zero-centred RMSNorm that produce a multiply's binary16 operand from the float32 residual stream
 * (launch_embed / launch_rms_norm of runner/cuda/src/kernels_elementwise.hpp:41-46,85-95): x[t, :] = table[tokens[t], :] widened;
 * y = (x / sqrt(sum(x^2) / cols + eps)) * (1 + w), float32 in, binary16 out, with the reference's float32 arithmetic and its fixed order
 * of summation (runner/cuda/src/kernels_elementwise.cu:6-11,114-141), so a row's bits are the reference kernel's. hidden a multiple of
 * 8; cols, ld_x, ld_y multiples of 4. sepal_b200_embed_rms_norm_half does both for the first layer in one pass over the row (the
 * engine's back-to-back launches at runner/cuda/src/cuda_engine.cpp:1676-1692). */
SEPAL_B200_API int32_t sepal_b200_embed(const void* table_half, const uint32_t* tokens, float* x, uint64_t rows, uint64_t hidden, uint64_t vocab,
                                        void* stream);
SEPAL_B200_API int32_t sepal_b200_embed_rms_norm_half(const void* table_half, const uint32_t* tokens, float* x, const float* w, void* y_half,
                                                      uint64_t ld_y, uint64_t rows, uint64_t hidden, uint64_t vocab, float eps, void* stream);
SEPAL_B200_API int32_t sepal_b200_rms_norm_half(const float* x, uint64_t ld_x, const float* w, void* y_half, uint64_t ld_y, uint64_t rows,
                                                uint64_t cols, float eps, void* stream);

/* ---- a synthetic trunk made of the projection GEMMs ---------------------------------------------------------------------------- */

/* The caller of the hot path for whole-pass measurements: the reference's layer loop (runner/cuda/src/cuda_engine.cpp:1724-1952) with
 * random N(0, 0.02) weights and the mixer cores wired out (the o projection reads the q band of the fused [q; k; v] product, the
 * DeltaNet out projection the v band of the fused in-projection), so that a pass is embedding, RMSNorms and the GEMMs with their fused
 * SwiGLU and residual epilogues. Layer l is an attention layer when l % 4 == 3. Counterpart of creating a CudaEngine from a config and
 * random weights (runner/cuda/include/sepal/cuda/cuda_engine.hpp:395-403) and of CudaEngine::run. */
typedef struct sepal_b200_trunk sepal_b200_trunk;
typedef struct sepal_b200_trunk_config {
    uint32_t layers, hidden, intermediate, vocab;
    uint32_t attn_q, attn_kv;             /* q width; k and v width each (one fused [q; k; v] multiply) */
    uint32_t dn_in, dn_v_offset, dn_v;    /* fused DeltaNet in-projection width; the band its out-projection reads */
    uint32_t max_call_tokens;             /* rows per call; a longer request is cut into calls (gpu_decision_engine.cpp:233-245) */
    uint32_t mlp_int8;                    /* 1: gate_up and down stored as int8 groups */
    float eps;
    uint64_t seed;
    uint32_t attn_o;                      /* width the attention out-projection reads; 0: attn_q (a real q_proj also carries the output gate) */
    /* attn_heads > 0: the attention layers run the real core between their projections (sepal_b200_attention_prepare / _attention on
     * the in-projection's bands, key/value caches per layer) instead of the fixed wiring. Then attn_q = 2 * heads * head_dim,
     * attn_kv = kv_heads * head_dim, attn_o = heads * head_dim, head_dim 128 or 256. */
    uint32_t attn_heads, attn_kv_heads, attn_head_dim, attn_rotary_dims;
    /* dn_value_heads > 0: the DeltaNet layers run the real core (sepal_b200_deltanet on the in-projection's [qkv; z; b; a] bands, a
     * recurrent state and a convolution tail per request and layer). Then dn_v = 128 * dn_value_heads and dn_in = 256 * dn_key_heads +
     * 256 * dn_value_heads + 2 * dn_value_heads. dn_conv_kernel: 0 = 4 taps. */
    uint32_t dn_key_heads, dn_value_heads, dn_conv_kernel;
    double rope_theta;                    /* 0: 1e7 */
} sepal_b200_trunk_config;
SEPAL_B200_API int32_t sepal_b200_trunk_open(int32_t device, const sepal_b200_trunk_config* config, sepal_b200_trunk** out);
SEPAL_B200_API void sepal_b200_trunk_close(sepal_b200_trunk* trunk);

/* ---- the full-attention core between its projections ---------------------------------------------------------------------------------
 *
 * Replaces launch_attention_prepare and launch_attention (runner/cuda/src/kernels_attention.hpp:154-183) for requests whose keys and
 * values are contiguous: per-head RMSNorm of q and k ("1 + weight" form), partial RoPE (the first rotary_dims of a head, dimension i
 * paired with i + rotary_dims / 2, angles position * theta^(-2 i / rotary_dims) in float64), keys and values appended to the request's
 * range of the arena, causal grouped-query attention scaled by 1 / sqrt(head_dim), times sigmoid(gate)
 * (runner/include/sepal/ref/attention.hpp:33-235). q_proj's output holds, per head, the query then its gate. A call's tokens form runs
 * ("rows") of consecutive tokens of different requests; a row names where its request's keys start in the arena (kv_begin) and how many
 * of the request's tokens are there already (context = the position of the row's first token). The arenas are binary16 [arena_tokens,
 * kv_heads * head_dim] and must hold finite numbers everywhere (zero them once). head_dim 128 or 256. `rows` is a host array, sorted by
 * q_begin. *_half: 1 = the band is binary16, 0 = float32. Both calls enqueue on `stream` and return. */
typedef struct sepal_b200_attention_shape {
    uint32_t heads, kv_heads, head_dim, rotary_dims;
    double rope_theta;
    float eps;
    uint32_t reserved;
} sepal_b200_attention_shape;
typedef struct sepal_b200_attention_row {
    uint32_t q_begin, length, kv_begin, context;
} sepal_b200_attention_row;
/* q_gate [N, 2 * heads * head_dim], k and v [N, kv_heads * head_dim]; q_norm, k_norm float32 [head_dim]; q_out binary16 [N, heads * head_dim]. */
SEPAL_B200_API int32_t sepal_b200_attention_prepare(sepal_b200_ctx* ctx, const sepal_b200_attention_shape* shape, const sepal_b200_attention_row* rows,
                                                    uint64_t n_rows, const void* q_gate, uint64_t q_gate_stride, int32_t q_gate_half, const void* k,
                                                    uint64_t k_stride, int32_t k_half, const void* v, uint64_t v_stride, int32_t v_half,
                                                    const float* q_norm, const float* k_norm, void* q_out, uint64_t q_stride, void* k_arena,
                                                    void* v_arena, uint64_t arena_tokens, void* stream);
/* q: what the prepare call wrote; gate: the q_gate band again (read at column head * 2 * head_dim + head_dim + d); out binary16
 * [N, heads * head_dim], the operand of o_proj. Flash attention on tcgen05 (Q K^T and P V on the tensor cores, accumulators in tensor
 * memory, float32 online softmax), one CTA per 128 queries of a row and head, keys in blocks counted from the request's first token. */
SEPAL_B200_API int32_t sepal_b200_attention(sepal_b200_ctx* ctx, const sepal_b200_attention_shape* shape, const sepal_b200_attention_row* rows,
                                            uint64_t n_rows, uint64_t n_tokens, const void* q, uint64_t q_stride, const void* k_arena,
                                            const void* v_arena, uint64_t arena_tokens, const void* gate, uint64_t gate_stride, int32_t gate_half,
                                            void* out, uint64_t out_stride, void* stream);

/* ---- the Gated DeltaNet core between its projections ---------------------------------------------------------------------------------
 *
 * Replaces the DeltaNet launches of the reference's layer loop (runner/cuda/src/cuda_engine.cpp:1827-1857; contract
 * runner/cuda/src/kernels_deltanet.hpp; math runner/include/sepal/ref/deltanet.hpp:33-330): causal depthwise convolution over `mixed`
 * (K taps, the last on the current token, continued from the request's previous K - 1 rows), SiLU, q / k / v split, q and k L2-normalised
 * per head, value head h on key head h / (value_heads / key_heads), the gated delta rule on a float32 state per value head
 * (S <- decay S; S <- S + k (x) beta (v - k . S); read = S^T q / sqrt(dk); decay = exp(-exp(A_log) softplus(a + dt_bias)), beta =
 * sigmoid(b)), the head-wise RMSNorm of the read with the norm weight itself and the silu(z) gate, binary16 out for out_proj.
 * mixed [N, 2 key_dim + value_dim], z [N, value_dim], b and a [N, value_heads] are bands of the in-projection (all binary16 or all
 * float32); conv float32 [conv_dim, K], a_log and dt_bias [value_heads], norm [head_dim]; scratch: N * (264 key_heads + 2 value_dim + 58
 * value_heads) floats, 16-byte aligned; states float32 [slots, value_heads, 128, 128] and tails float32 [slots, K - 1, conv_dim] persist between calls
 * (a row with fresh = 1 starts from zero whatever its slot holds); a row is {first token, length, slot, fresh}; rows: host array sorted
 * by first token, one row per slot in a call. head_dim 128. The scan takes a row in chunks of sixteen tokens (eight warps per row and value head; float32 state, TF32 operands in the
 * chunk's matrix products). */
typedef struct sepal_b200_deltanet_shape {
    uint32_t key_heads, value_heads, head_dim, conv_kernel;
    float eps;
    uint32_t reserved;
} sepal_b200_deltanet_shape;
typedef struct sepal_b200_deltanet_row {
    uint32_t q_begin, length, slot, fresh;
} sepal_b200_deltanet_row;
SEPAL_B200_API int32_t sepal_b200_deltanet(sepal_b200_ctx* ctx, const sepal_b200_deltanet_shape* shape, const sepal_b200_deltanet_row* rows,
                                           uint64_t n_rows, const void* mixed, uint64_t mixed_stride, const void* z, uint64_t z_stride, const void* b,
                                           uint64_t b_stride, const void* a, uint64_t a_stride, int32_t bands_half, const float* conv,
                                           const float* a_log, const float* dt_bias, const float* norm, float* scratch, float* states, float* tails,
                                           uint64_t slots, void* out, uint64_t out_stride, void* stream);

/* ---- checkpoints and weight placement (the data format on the input side of the path) ----------------------------------------------
 *
 * The reader of the safetensors format (runner/include/sepal/safetensors.hpp:1-154) and of checkpoint directories with their name
 * prefixes (runner/include/sepal/loader.hpp:5-8): a file is mapped read-only and checked once (every tensor inside the file, of the size
 * its shape and type imply, aligned, overlapping no other); `path` is one file or a directory with model.safetensors or the shards
 * model-0000i-of-0000N.safetensors. Tensors are addressed by their engine names (the prefix dropped), in sorted order by index. */
typedef struct sepal_b200_checkpoint sepal_b200_checkpoint;
typedef struct sepal_b200_tensor_info {
    char name[256];
    int32_t dtype;      /* 0 F32, 1 F16, 2 BF16, 3 I8, 4 U8, 5 I32, 6 I64, 7 F64, 8 BOOL, 9 I16, 10 U16, 11 U32, 12 U64 */
    uint32_t rank;
    uint64_t shape[8];
    const void* data;   /* host; valid while the checkpoint is open (for sepal_b200_tensor_file_write: the values to write) */
    uint64_t bytes;
} sepal_b200_tensor_info;
SEPAL_B200_API int32_t sepal_b200_checkpoint_open(const char* path, sepal_b200_checkpoint** out);
SEPAL_B200_API void sepal_b200_checkpoint_close(sepal_b200_checkpoint* checkpoint);
SEPAL_B200_API int32_t sepal_b200_checkpoint_count(const sepal_b200_checkpoint* checkpoint, uint64_t* count);
/* By name when name is not NULL, else by index. */
SEPAL_B200_API int32_t sepal_b200_checkpoint_tensor(const sepal_b200_checkpoint* checkpoint, uint64_t index, const char* name, sepal_b200_tensor_info* info);
/* A "__metadata__" value ("" when absent; the key "__prefix__" yields the name prefix that was dropped); size-query protocol. */
SEPAL_B200_API int32_t sepal_b200_checkpoint_metadata(const sepal_b200_checkpoint* checkpoint, const char* key, char* buffer, uint64_t capacity,
                                                      uint64_t* needed);
/* Writes a file of the same format (name, dtype, rank, shape, data of each tensor are read; tensors are stored in the order given, the
 * first on a 256-byte boundary of the file). */
SEPAL_B200_API int32_t sepal_b200_tensor_file_write(const char* path, uint64_t n, const sepal_b200_tensor_info* tensors, uint64_t n_metadata,
                                                    const char* const* keys, const char* const* values);

/* The trunk with the weights of a checkpoint instead of random ones: the reference's placement (runner/cuda/src/cuda_engine.cpp:525-711)
 * for the projections this path has: [q; k; v] and [qkv; z; b; a] stacked, everything converted to binary16 (norms float32), [gate; up]
 * interleaved in blocks of 64 rows, the MLP quantised per group of 128 from a float32 copy when mlp_int8 is set. The configuration must
 * agree with the tensors' shapes (attn_q = rows of q_proj, attn_o = columns of o_proj, dn_in = rows of the four in-projections together).
 * A file written by sepal_b200_trunk_save (metadata format = "sepal_b200.placed.1") is copied to the device as it is. */
SEPAL_B200_API int32_t sepal_b200_trunk_open_checkpoint(int32_t device, const sepal_b200_trunk_config* config, const sepal_b200_checkpoint* checkpoint,
                                                        sepal_b200_trunk** out);
/* Writes the placed weights (stacked, interleaved, quantised: int8 values and their float32 group scales) to one file. */
SEPAL_B200_API int32_t sepal_b200_trunk_save(sepal_b200_trunk* trunk, const char* path);

/* The planner's byte accounting of the trunk weights (runner/src/plan/planner.cpp:45-130, runner/src/core/config.cpp:156-188): the bytes
 * every parameter but the embedding table and the head takes under a storage profile ("w16", "w8", "gpu-f16", "gpu-q8w", "cpu-q8",
 * "gpu-bf16", "gpu-w8g"); per-group scales are counted, per-row scales are not. Presets: "0.8b", "2b", "4b", "9b". Host arithmetic only. */
typedef struct sepal_b200_model {
    uint64_t layers, hidden, intermediate, vocab;
    uint64_t attn_heads, attn_kv_heads, attn_head_dim;
    uint64_t dn_key_heads, dn_value_heads, dn_key_head_dim, dn_value_head_dim, conv_kernel;
    uint64_t attention_interval;
} sepal_b200_model;
SEPAL_B200_API int32_t sepal_b200_model_preset(const char* name, sepal_b200_model* out);
SEPAL_B200_API int32_t sepal_b200_plan_weight_bytes(const sepal_b200_model* model, const char* profile, uint64_t* bytes);
/* One request of n host token ids. last_hidden: `hidden` floats (host) for the last token's final hidden state; all_hidden: NULL or
 * [n, hidden] floats (host). times_ms: NULL or 2 doubles (device time of the request by CUDA events; reserved). Returns when done. */
SEPAL_B200_API int32_t sepal_b200_trunk_run(sepal_b200_trunk* trunk, const uint32_t* tokens, uint64_t n, float* last_hidden, float* all_hidden,
                                            double* times_ms);
/* Many requests at once, with the flat arrays of sepal_score (runner/include/sepal/c_api.h:46-60): tokens holds the requests end to end,
 * request r being tokens[offsets[r] .. offsets[r + 1]). They are packed into calls as the reference's engine packs them
 * (runner/cuda/src/gpu_decision_engine.cpp:233-266: segments of at most max_call_tokens in request order, a new call when the next
 * segment does not fit, at most 64 segments a call), so short requests share a call and its large-M GEMMs. last_hidden: [n_requests,
 * hidden] floats (host); times_s: NULL or n_requests doubles, the seconds from the start of this function's device work until the
 * request's result was complete (CUDA events). Returns when everything is on the host. */
SEPAL_B200_API int32_t sepal_b200_trunk_score(sepal_b200_trunk* trunk, uint64_t n_requests, const uint32_t* tokens, const uint64_t* offsets,
                                              float* last_hidden, double* times_s);
/* Copies a stored weight to the host (size-query protocol: host_out NULL only reports *needed). which: 0 embedding, 1 input norm,
 * 2 mixer in-projection, 3 mixer out-projection, 4 post norm, 5 packed [gate; up], 6 down, 7 / 8 the attention core's q / k head norms,
 * 9 .. 12 the DeltaNet core's convolution, A_log, dt_bias and norm weight, 13 / 14 (int8 MLP only) the group quantiser's float32 scales of
 * [gate; up] and down, [rows, k / 128]. */
SEPAL_B200_API int32_t sepal_b200_trunk_weight(sepal_b200_trunk* trunk, uint32_t layer, int32_t which, void* host_out, uint64_t capacity,
                                               uint64_t* needed);
SEPAL_B200_API int32_t sepal_b200_trunk_info(sepal_b200_trunk* trunk, uint64_t* gemm_flops_per_token, uint64_t* weight_bytes);

/* ---- provider on host pointers ------------------------------------------------------------------------------------------------ */

/* A provider owns a context, a stream and one device allocation (`arena_bytes`, 0 = 1 GiB) from which weights (bottom, for the
 * provider's life) and per-call temporaries (top, released when the call returns) are carved; nothing else is allocated afterwards.
 * Counterpart of CudaGemm's constructor (cuda_gemm.hpp:112-115, memory model :7-10). */
SEPAL_B200_API int32_t sepal_b200_provider_open(int32_t device, uint64_t arena_bytes, sepal_b200_provider** out);
SEPAL_B200_API void sepal_b200_provider_close(sepal_b200_provider* provider);

/* Copies W [N, K] (host, SEPAL_B200_F32 or _F16) to the device once, rounded to binary16, and returns its id.
 * Counterpart of CudaGemm::upload_weights (cuda_gemm.hpp:128-129). */
SEPAL_B200_API int32_t sepal_b200_provider_upload_weights(sepal_b200_provider* provider, const void* w, int32_t dtype, uint64_t n, uint64_t k,
                                                          uint32_t* id_out);

/* The same for int8-group storage: W float32 [N, K] (host) is quantised on the device (K a multiple of 128) and kept as int8 +
 * prepared scales, as the gpu-w8g profile stores its matrices (runner/cuda/src/cuda_engine.cpp:580-627). */
SEPAL_B200_API int32_t sepal_b200_provider_upload_weights_w8g(sepal_b200_provider* provider, const float* w, uint64_t n, uint64_t k, uint32_t* id_out);

/* Y[t, n] = beta Y[t, n] + sum_k X[t, k] W[n, k]: X [T, K] host (F32 or F16; rounded to binary16 on the device), Y [T, N] host
 * float32. X is uploaded, Y downloaded, and the call returns when Y is complete. With beta == 0 Y is written without being read.
 * Counterpart of CudaGemm::gemm_f(MatRef, WeightId, MatView, float) (cuda_gemm.hpp:136-137). Pinned host buffers
 * (sepal_b200_host_alloc) make the copies asynchronous and fast; pageable ones work too. */
SEPAL_B200_API int32_t sepal_b200_provider_gemm_f(sepal_b200_provider* provider, const void* x, int32_t x_dtype, uint64_t t, uint32_t weight_id,
                                                  float* y, float beta);

/* Pinned host memory for the provider's callers. */
SEPAL_B200_API int32_t sepal_b200_host_alloc(uint64_t bytes, void** out);
SEPAL_B200_API void sepal_b200_host_free(void* ptr);

#ifdef __cplusplus
}
#endif

#endif /* SEPAL_B200_H */
