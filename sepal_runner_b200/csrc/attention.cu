#include "attention.hpp"

#include <algorithm>
#include <cmath>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_fp16.h>

#include "ptx.cuh"

namespace sepal::b200 {

void count_launch();

namespace {

constexpr int kQueries = 128;                   // queries of one CTA = lanes of tensor memory
constexpr long long kWaitLimit = 1ll << 30;     // clock cycles before a wait gives up
constexpr int kStatusAttention = 16;            // status codes 16 .. 23: a wait of the attention kernel ran out

__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity, volatile unsigned* abort_flag, int* status, int code) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    unsigned spins = 0;
    for (;;) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((++spins & 31u) == 0) {
            if (*abort_flag != 0) return false;
            if (clock64() - t0 > kWaitLimit) {
                *abort_flag = 1;
                atomicCAS(status, 0, code | (static_cast<int>(blockIdx.x) << 8));
                return false;
            }
        }
    }
}

// ---- prepare --------------------------------------------------------------------------------------------------------------------

struct PrepareParams {
    const AttentionRow* rows;
    unsigned n_rows;
    unsigned heads, kv_heads, head_dim, rotary_dims;
    float eps;
    const double* inv_freq;  // theta^(-2 i / rotary_dims), i < rotary_dims / 2
    const void* q_gate;
    const void* k;
    const void* v;
    unsigned long long q_gate_stride, k_stride, v_stride;
    unsigned q_gate_half, k_half, v_half;
    const float* q_norm;
    const float* k_norm;
    __half* q_out;
    unsigned long long q_stride;
    __half* k_arena;
    __half* v_arena;
};

__device__ __forceinline__ float band_value(const void* base, unsigned long long index, unsigned half) {
    return half != 0 ? __half2float(static_cast<const __half*>(base)[index]) : static_cast<const float*>(base)[index];
}

// One block per token; a warp takes heads in turn (query heads, then key heads, then the value heads' copy). Lane l holds dimensions
// l, l + 32, ... of the head. Sum of squares: each lane in that order, then a butterfly: fixed, a function of the head alone. The
// normed head goes through shared memory so that a rotated dimension can read its partner (i with i + rotary_dims / 2) from any lane.
__global__ void __launch_bounds__(256) attention_prepare_kernel(const PrepareParams p) {
    __shared__ float cs[256];          // cos then sin of the token's rotary_dims / 2 angles
    __shared__ float normed[8][256];   // one head per warp
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const unsigned token = blockIdx.x;
    // the run this token belongs to: the last row whose q_begin is at or before it
    unsigned lo = 0, hi = p.n_rows;
    while (hi - lo > 1) {
        const unsigned mid = (lo + hi) / 2;
        if (p.rows[mid].q_begin <= token) lo = mid; else hi = mid;
    }
    const AttentionRow row = p.rows[lo];
    if (token < row.q_begin || token >= row.q_begin + row.length) return;  // a token outside every run (gaps are allowed)
    const unsigned t = token - row.q_begin;
    const double position = static_cast<double>(row.context + t);
    const unsigned half_rot = p.rotary_dims / 2;
    for (unsigned i = threadIdx.x; i < half_rot; i += blockDim.x) {
        const double angle = position * p.inv_freq[i];  // float64: a position is a large whole number
        cs[i] = static_cast<float>(cos(angle));
        cs[128 + i] = static_cast<float>(sin(angle));
    }
    __syncthreads();
    const unsigned warp = threadIdx.x / 32, lane = threadIdx.x % 32, warps = blockDim.x / 32;
    const unsigned hd = p.head_dim, per_lane = hd / 32;  // 4 or 8
    const size_t arena_row = static_cast<size_t>(row.kv_begin) + row.context + t;
    for (unsigned job = warp; job < p.heads + 2 * p.kv_heads; job += warps) {
        if (job >= p.heads + p.kv_heads) {  // a value head: stored as it is
            const unsigned h = job - p.heads - p.kv_heads;
            for (unsigned e = 0; e < per_lane; ++e) {
                const unsigned d = lane + 32 * e;
                p.v_arena[arena_row * (p.kv_heads * hd) + h * hd + d] = __float2half_rn(band_value(p.v, token * p.v_stride + h * hd + d, p.v_half));
            }
            continue;
        }
        const bool is_q = job < p.heads;
        const unsigned h = is_q ? job : job - p.heads;
        const float* w = is_q ? p.q_norm : p.k_norm;
        float x[8];
        float ss = 0.0f;
        for (unsigned e = 0; e < per_lane; ++e) {
            const unsigned d = lane + 32 * e;
            x[e] = is_q ? band_value(p.q_gate, token * p.q_gate_stride + static_cast<size_t>(h) * 2 * hd + d, p.q_gate_half)
                        : band_value(p.k, token * p.k_stride + h * hd + d, p.k_half);
            ss = __fmaf_rn(x[e], x[e], ss);
        }
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        const float rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(hd)), p.eps));
        __syncwarp();  // the previous head's readers are done with the buffer
        for (unsigned e = 0; e < per_lane; ++e) normed[warp][lane + 32 * e] = __fmul_rn(__fdiv_rn(x[e], rms), __fadd_rn(1.0f, w[lane + 32 * e]));
        __syncwarp();
        __half* dst = is_q ? p.q_out + token * p.q_stride + static_cast<size_t>(h) * hd : p.k_arena + arena_row * (p.kv_heads * hd) + h * hd;
        for (unsigned e = 0; e < per_lane; ++e) {
            const unsigned d = lane + 32 * e;
            float y = normed[warp][d];
            if (d < half_rot) {  // (a, b) -> (a cos - b sin, b cos + a sin) for a = dimension i, b = dimension i + rotary_dims / 2
                y = __fsub_rn(__fmul_rn(y, cs[d]), __fmul_rn(normed[warp][d + half_rot], cs[128 + d]));
            } else if (d < 2 * half_rot) {
                const unsigned i = d - half_rot;
                y = __fadd_rn(__fmul_rn(y, cs[i]), __fmul_rn(normed[warp][i], cs[128 + i]));
            }
            dst[d] = __float2half_rn(y);
        }
    }
}

// ---- attention -------------------------------------------------------------------------------------------------------------------

// 2^x by the special-function unit (two units in the last place; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct AttentionParams {
    const AttentionRow* rows;
    const unsigned* blocks;  // (row, query block) pairs, heaviest first
    unsigned heads, group;   // query heads; heads / kv_heads
    float scale_log2;        // log2(e) / sqrt(head_dim)
    const void* gate;
    unsigned long long gate_stride;
    unsigned gate_half;
    __half* out;
    unsigned long long out_stride;
    int* status;
};

template <int D>
struct AttentionTile {
    static constexpr int kKeys = D == 128 ? 128 : 64;         // keys per block
    static constexpr int kBoxes = D / 64;                      // 64-column boxes of a Q, K or V tile
    static constexpr int kQBytes = kQueries * D * 2;
    static constexpr int kKvBytes = kKeys * D * 2;             // one K tile or one V tile
    static constexpr int kPBytes = kQueries * kKeys * 2;
    static constexpr int kStages = 2;
    static constexpr int kSmem = 1024 + kQBytes + kStages * 2 * kKvBytes + 2 * kPBytes + 256 + 1024;  // two P buffers; barriers; the halves' exchange
    static constexpr int kSCols = kKeys;                       // tensor-memory columns of one score buffer
    static constexpr int kOCol = 2 * kKeys;                    // where the output accumulator starts
};

// Warp 0: TMA (Q once, then K and V blocks into a ring of two). Warp 1: MMA issuer: S_j = Q K_j^T into one of two score buffers (S_{j+1}
// is issued before P_j V_j, so the tensor core has work while the softmax of block j runs), then O += P_j V_j. Warps 2-9: one query per
// thread pair: scores from tensor memory, masked, running maximum and sum in the base-2 domain, P_j as binary16 into shared memory in the
// layout the MMA reads, O rescaled in tensor memory when the maximum moved; at the end O / l * sigmoid(gate).
template <int D>
__global__ void __launch_bounds__(320, 1)
attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                 const AttentionParams p) {
    using T = AttentionTile<D>;
    constexpr int kKeys = T::kKeys;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_addr(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* const smem = smem_raw + (base - raw_addr);
    const uint32_t q_addr = base;
    const uint32_t kv_addr = base + T::kQBytes;  // stage s: K at kv_addr + s * 2 * kKvBytes, V right after it
    const uint32_t p_addr = kv_addr + T::kStages * 2 * T::kKvBytes;
    uint8_t* const p_smem = smem + (p_addr - base);
    uint8_t* const tail = smem + (p_addr - base) + 2 * T::kPBytes;
    const uint32_t bars = ptx::smem_addr(tail);
    const uint32_t q_full = bars;
    const auto p_full = [&](int b) { return bars + 8u + 8u * b; };    // P_j is written (j & 1 picks the buffer)
    const auto kv_full = [&](int s) { return bars + 24u + 8u * s; };
    const auto kv_empty = [&](int s) { return bars + 40u + 8u * s; };
    const auto s_full = [&](int b) { return bars + 56u + 8u * b; };
    const auto s_free = [&](int b) { return bars + 72u + 8u * b; };
    const auto p_free = [&](int b) { return bars + 88u + 8u * b; };   // P_j V_j has finished: buffer j & 1 is free, and O holds blocks 0 .. j
    unsigned* const words = reinterpret_cast<unsigned*>(tail + 112);
    unsigned* const tmem_slot = words;
    volatile unsigned* const abort_flag = words + 1;
    float* const exchange = reinterpret_cast<float*>(tail + 256);  // 2 x 128 floats: what the two halves of a query tell each other

    const unsigned warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const unsigned head = blockIdx.y, kv_head = head / p.group;
    const AttentionRow row = p.rows[p.blocks[2 * blockIdx.x]];
    const unsigned qb = p.blocks[2 * blockIdx.x + 1];
    const unsigned q0 = qb * kQueries;                                  // first query of the block inside the run
    const unsigned valid = min(static_cast<unsigned>(kQueries), row.length - q0);
    // keys the block's last valid query sees, and the blocks that hold them
    const unsigned n_keys = row.context + q0 + valid;
    const unsigned n_blocks = (n_keys + kKeys - 1) / kKeys;

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(p_full(s), 256);
            ptx::mbar_init(p_free(s), 1);
            ptx::mbar_init(kv_full(s), 1);
            ptx::mbar_init(kv_empty(s), 1);
            ptx::mbar_init(s_full(s), 1);
            ptx::mbar_init(s_free(s), 256);
        }
        words[1] = 0;
        ptx::fence_barrier_init();
        ptx::tma_prefetch_descriptor(&map_q);
        ptx::tma_prefetch_descriptor(&map_k);
        ptx::tma_prefetch_descriptor(&map_v);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(tmem_slot), 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();

    if (warp == 0) {
        if (lane == 0) {
            ptx::mbar_arrive_expect_tx(q_full, T::kQBytes);
            for (int b = 0; b < T::kBoxes; ++b)
                ptx::tma_load_2d(q_addr + b * (kQueries * 128), &map_q, q_full, static_cast<int>(head * D + 64 * b), static_cast<int>(row.q_begin + q0));
            for (unsigned j = 0; j < n_blocks; ++j) {
                const int s = static_cast<int>(j & 1u);
                if (j >= 2 && !wait_barrier(kv_empty(s), ((j >> 1) - 1) & 1u, abort_flag, p.status, kStatusAttention + 0)) break;
                const uint32_t k_dst = kv_addr + s * 2 * T::kKvBytes, v_dst = k_dst + T::kKvBytes;
                const int key_row = static_cast<int>(row.kv_begin + j * kKeys);
                ptx::mbar_arrive_expect_tx(kv_full(s), 2 * T::kKvBytes);
                for (int b = 0; b < T::kBoxes; ++b) {
                    ptx::tma_load_2d(k_dst + b * (kKeys * 128), &map_k, kv_full(s), static_cast<int>(kv_head * D + 64 * b), key_row);
                    ptx::tma_load_2d(v_dst + b * (kKeys * 128), &map_v, kv_full(s), static_cast<int>(kv_head * D + 64 * b), key_row);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_s = ptx::instr_desc_f16_f32acc(kQueries, kKeys);
            const uint32_t idesc_o = ptx::instr_desc_f16_f32acc_b_mn(kQueries, D);
            const uint32_t o_tmem = tmem_base + T::kOCol;
            const auto issue_scores = [&](unsigned j) {  // S_j = Q K_j^T into score buffer j & 1
                const int s = static_cast<int>(j & 1u);
                const uint32_t k_tile = kv_addr + s * 2 * T::kKvBytes;
#pragma unroll
                for (int b = 0; b < T::kBoxes; ++b) {
                    const uint64_t dq = ptx::smem_desc_k_major_sw128(q_addr + b * (kQueries * 128));
                    const uint64_t dk = ptx::smem_desc_k_major_sw128(k_tile + b * (kKeys * 128));
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) ptx::mma_f16_ss(tmem_base + s * T::kSCols, dq + 2u * kk, dk + 2u * kk, idesc_s, (b | kk) != 0 ? 1u : 0u);
                }
                ptx::mma_commit(s_full(s));
            };
            bool ok = wait_barrier(q_full, 0, abort_flag, p.status, kStatusAttention + 1) && wait_barrier(kv_full(0), 0, abort_flag, p.status, kStatusAttention + 1);
            if (ok) {
                ptx::tc_fence_after_sync();
                issue_scores(0);
            }
            for (unsigned j = 0; ok && j < n_blocks; ++j) {
                const int s = static_cast<int>(j & 1u);
                if (j + 1 < n_blocks) {
                    const unsigned n = j + 1;
                    ok = wait_barrier(kv_full(n & 1u), (n >> 1) & 1u, abort_flag, p.status, kStatusAttention + 2);
                    if (ok && n >= 2) ok = wait_barrier(s_free(n & 1u), ((n >> 1) - 1) & 1u, abort_flag, p.status, kStatusAttention + 3);
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    issue_scores(n);
                }
                ok = wait_barrier(p_full(s), (j >> 1) & 1u, abort_flag, p.status, kStatusAttention + 4);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t v_tile = kv_addr + s * 2 * T::kKvBytes + T::kKvBytes;
#pragma unroll
                for (int kb = 0; kb < kKeys / 16; ++kb) {
                    const uint64_t dp = ptx::smem_desc_k_major_sw128(p_addr + s * T::kPBytes + (kb / 4) * (kQueries * 128)) + 2u * (kb % 4);
                    const uint64_t dv = ptx::smem_desc_mn_major_sw128(v_tile + kb * 2048, kKeys * 128);
                    ptx::mma_f16_ss(o_tmem, dp, dv, idesc_o, (j > 0 || kb > 0) ? 1u : 0u);
                }
                ptx::mma_commit(kv_empty(s));
                ptx::mma_commit(p_free(s));
            }
        }
        __syncwarp();
    } else {
        // Eight warps: warps w and w + 4 share the 32 queries of tensor-memory lanes 32 (w % 4) ..., each taking half of a block's keys
        // (and later half of the head's dimensions), so that two warps per scheduler hide each other's latencies.
        constexpr int kW = kKeys / 2;                 // keys of a block per thread
        constexpr int kDh = D / 2;                    // output dimensions per thread
        const unsigned quarter = warp % 4;
        const unsigned side = (warp - 2) / 4;         // which half
        const unsigned r = quarter * 32 + lane;       // this thread's query inside the block
        const uint32_t lane_base = tmem_base + ((quarter * 32u) << 16);
        const unsigned q_index = row.context + q0 + r;  // the last key this query sees
        const auto pair_sync = [&] { asm volatile("bar.sync %0, 64;" ::"r"(2u + quarter) : "memory"); };
        // Running state in the base-2 domain: the reference maximum m (the row's probabilities are exp2(t - m)) and the sum l of this
        // thread's half of them. m follows the true maximum lazily: it moves only when the maximum has grown by more than 8, so a
        // probability is at most 2^8 (binary16 holds it with its full relative precision) and O is rescaled only then. O / l does not care.
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        for (unsigned j = 0; j < n_blocks; ++j) {
            const int s = static_cast<int>(j & 1u);
            ok = wait_barrier(s_full(s), (j >> 1) & 1u, abort_flag, p.status, kStatusAttention + 5);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const unsigned key0 = j * kKeys + side * kW;  // this thread's first key of the block
            const bool diagonal = j * kKeys + kKeys - 1 > row.context + q0;  // some key of the block is hidden from some query
            float t[kW];
#pragma unroll
            for (int c = 0; c < kW; c += 32) {
                uint32_t v[32];
                ptx::tmem_ld_32x32(lane_base + s * T::kSCols + side * kW + c, v);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) t[c + i] = __uint_as_float(v[i]);
            }
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(s_free(s));  // the scores are in registers: the buffer may be overwritten
            if (diagonal) {
#pragma unroll
                for (int i = 0; i < kW; ++i)
                    if (key0 + i > q_index) t[i] = -INFINITY;
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < kW; ++i) mx[i & 3] = fmaxf(mx[i & 3], t[i]);
            const float mine = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            exchange[side * 128 + r] = mine;
            pair_sync();
            const float block_max = fmaxf(mine, exchange[(side ^ 1u) * 128 + r]) * p.scale_log2;
            pair_sync();  // both have read: the next block may overwrite
            float alpha = 1.0f;
            if (block_max > m + 8.0f) {  // also the first block (m = -inf), where alpha is 0 and O is not touched
                alpha = fast_exp2(m - block_max);
                m = block_max;
            }
            // P buffer j & 1 was last read by P_{j-2} V_{j-2}
            if (j >= 2) {
                ok = wait_barrier(p_free(s), ((j >> 1) - 1) & 1u, abort_flag, p.status, kStatusAttention + 6);
                if (!ok) break;
            }
            // probabilities (a hidden key: exp2(-inf) = 0), their sum, P as binary16 in the swizzled K-major layout
            float sum[2] = {0.0f, 0.0f};
            uint8_t* const p_row = p_smem + s * T::kPBytes + r * 128;
#pragma unroll
            for (int c = 0; c < kW; c += 8) {
                unsigned packed[4];
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const float e0 = fast_exp2(__fmaf_rn(t[c + i], p.scale_log2, -m));
                    const float e1 = fast_exp2(__fmaf_rn(t[c + i + 1], p.scale_log2, -m));
                    sum[0] += e0;
                    sum[1] += e1;
                    const __half2 h = __floats2half2_rn(e0, e1);
                    packed[i / 2] = *reinterpret_cast<const unsigned*>(&h);
                }
                const unsigned col = side * kW + c;  // column of the block: box col / 64, 16-byte chunk (col % 64) / 8
                *reinterpret_cast<uint4*>(p_row + (col / 64) * (kQueries * 128) + ((((col % 64) / 8) ^ (r & 7u)) * 16)) =
                    make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            // rescale this thread's half of O where the reference maximum moved (a warp's loads and stores of tensor memory are
            // collective: all lanes go together); O must hold P_{j-1} V_{j-1} first
            if (j > 0 && __any_sync(0xFFFFFFFFu, alpha != 1.0f)) {
                ok = wait_barrier(p_free(s ^ 1), ((j - 1) >> 1) & 1u, abort_flag, p.status, kStatusAttention + 6);
                if (!ok) break;
                ptx::tc_fence_after_sync();
#pragma unroll 1
                for (int c = 0; c < kDh; c += 32) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(lane_base + T::kOCol + side * kDh + c, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    ptx::tmem_st_32x32(lane_base + T::kOCol + side * kDh + c, v);
                }
                ptx::tmem_st_wait();
            }
            l = l * alpha + (sum[0] + sum[1]);
            ptx::fence_proxy_async_smem();  // P was written with ordinary stores; the MMA reads it through the async proxy
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(p_full(s));
        }
        if (ok && n_blocks > 0) ok = wait_barrier(p_free((n_blocks - 1) & 1u), ((n_blocks - 1) >> 1) & 1u, abort_flag, p.status, kStatusAttention + 7);
        // the row's sum: the first half's plus the second half's
        exchange[side * 128 + r] = l;
        pair_sync();
        const float total = exchange[r] + exchange[128 + r];
        // every lane takes part in the loads; only valid queries store
        if (ok) {
            ptx::tc_fence_after_sync();
            const float inv_l = 1.0f / total;
            const size_t token = static_cast<size_t>(row.q_begin) + q0 + r;
            __half* dst = p.out + token * p.out_stride + static_cast<size_t>(head) * D + side * kDh;
            const size_t gate0 = token * p.gate_stride + static_cast<size_t>(head) * 2 * D + D + side * kDh;
#pragma unroll 1
            for (int c = 0; c < kDh; c += 32) {
                uint32_t v[32];
                ptx::tmem_ld_32x32(lane_base + T::kOCol + side * kDh + c, v);
                ptx::tmem_ld_wait();
                if (r < valid) {
                    unsigned packed[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float g0 = band_value(p.gate, gate0 + c + i, p.gate_half), g1 = band_value(p.gate, gate0 + c + i + 1, p.gate_half);
                        const float o0 = __uint_as_float(v[i]) * inv_l * (1.0f / (1.0f + expf(-g0)));
                        const float o1 = __uint_as_float(v[i + 1]) * inv_l * (1.0f / (1.0f + expf(-g1)));
                        const __half2 h = __floats2half2_rn(o0, o1);
                        packed[i / 2] = *reinterpret_cast<const unsigned*>(&h);
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        *reinterpret_cast<uint4*>(dst + c + 8 * q) = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
            }
        }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, 512);
    }
}

// ---- the same on CTA pairs ---------------------------------------------------------------------------------------------------------
//
// One CTA keeps two key/value blocks in flight and needs a new one every thousand cycles of tensor work: the loads do not arrive in
// time. A pair of CTAs (tcgen05.mma.cta_group::2) takes 256 queries of one head against each block of 128 keys: every CTA holds its own
// 128 queries, scores and output rows, and loads HALF of the block: 64 of the 128 keys for S = Q K^T (the B operand is split along its
// rows) and half of the head's dimensions of all 128 values for O += P V (split along the output columns). Twice the work per loaded
// byte and per stage. Two threads of the first CTA issue the pair's MMAs, one the score products and one O += P V (a thread that has
// issued a tcgen05.commit cannot issue again until the MMAs before it have drained; the other thread's MMAs fill the gap); their
// commits reach both CTAs; arrivals of the second CTA's warps go to the first CTA's barriers. P_j never touches shared memory: the softmax threads store it as binary16 over the scores in tensor memory
// and O += P_j V_j takes its A operand from there, which leaves the whole of shared memory to Q and the key/value ring.
constexpr int kAttentionPairThreads = 608;            // TMA warp, score-MMA warp, sixteen softmax warps, value-MMA warp
constexpr unsigned kAttentionPairValueIssuer = 18;    // the warp whose first thread issues O += P V

template <int D>
struct AttentionPairTile {
    static constexpr int kKeys = 128;
    static constexpr int kStages = D == 128 ? 5 : 2;
    static constexpr int kQBytes = kQueries * D * 2;
    static constexpr int kHalfBytes = 128 * D;                 // 64 keys x D, and 128 values x D / 2, in binary16
    static constexpr int kStageBytes = 2 * kHalfBytes;
    static constexpr int kSmem = 1024 + kQBytes + kStages * kStageBytes + 256 + 2048;  // barriers; 4 x 128 floats the warps of a query exchange
    static constexpr int kOCol = 256;
};

template <int D>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kAttentionPairThreads, 1)
attention_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const AttentionParams p) {
    using T = AttentionPairTile<D>;
    constexpr int kKeys = T::kKeys, kStages = T::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_addr(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* const smem = smem_raw + (base - raw_addr);
    const uint32_t q_addr = base;
    const uint32_t kv_addr = base + T::kQBytes;  // stage s: this CTA's 64 keys at kv_addr + s * kStageBytes, its half of the values after them
    uint8_t* const tail = smem + T::kQBytes + kStages * T::kStageBytes;
    const uint32_t bars = ptx::smem_addr(tail);
    const uint32_t q_full = bars;
    const auto kv_full = [&](int s) { return bars + 8u + 8u * s; };
    const auto kv_empty = [&](int s) { return bars + 72u + 8u * s; };
    const auto s_full = [&](int b) { return bars + 136u + 8u * b; };   // S_j is in score buffer j & 1
    const auto p_full = [&](int b) { return bars + 152u + 8u * b; };   // P_j has replaced S_j there
    const auto p_free = [&](int b) { return bars + 168u + 8u * b; };   // P_j V_j has finished: O holds blocks 0 .. j
    unsigned* const words = reinterpret_cast<unsigned*>(tail + 184);
    unsigned* const tmem_slot = words;
    volatile unsigned* const abort_flag = words + 1;
    float* const exchange = reinterpret_cast<float*>(tail + 256);

    const unsigned warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const unsigned rank = ptx::cluster_ctarank();
    const unsigned head = blockIdx.y, kv_head = head / p.group;
    const unsigned block = blockIdx.x / 2;
    const AttentionRow row = p.rows[p.blocks[2 * block]];
    const unsigned qb = p.blocks[2 * block + 1];
    const unsigned pair_q0 = qb * 2 * kQueries;                         // first query of the pair inside the run
    const unsigned q0 = pair_q0 + rank * kQueries;                      // and of this CTA
    const unsigned pair_valid = min(2u * kQueries, row.length - pair_q0);
    const unsigned valid = pair_valid > rank * kQueries ? min(static_cast<unsigned>(kQueries), pair_valid - rank * kQueries) : 0u;
    const unsigned n_keys = row.context + pair_q0 + pair_valid;         // keys the pair's last valid query sees
    const unsigned n_blocks = (n_keys + kKeys - 1) / kKeys;

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(kv_full(s), 1);
            ptx::mbar_init(kv_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(s_full(b), 1);
            ptx::mbar_init(p_full(b), 32);  // one arrival from each softmax warp of both CTAs (used in the first CTA only)
            ptx::mbar_init(p_free(b), 1);
        }
        words[1] = 0;
        ptx::fence_barrier_init();
        ptx::tma_prefetch_descriptor(&map_q);
        ptx::tma_prefetch_descriptor(&map_k);
        ptx::tma_prefetch_descriptor(&map_v);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_addr(tmem_slot), 512);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();  // the partner's barriers exist before anything signals them
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t q_first = ptx::map_to_cta(q_full, 0);
            if (rank == 0) ptx::mbar_arrive_expect_tx(q_full, 2 * T::kQBytes);
            for (int b = 0; b < D / 64; ++b)
                ptx::tma_load_2d_pair(q_addr + b * (kQueries * 128), &map_q, q_first, static_cast<int>(head * D + 64 * b), static_cast<int>(row.q_begin + q0));
            for (unsigned j = 0; j < n_blocks; ++j) {
                const int s = static_cast<int>(j % kStages);
                if (j >= static_cast<unsigned>(kStages) && !wait_barrier(kv_empty(s), ((j / kStages) - 1) & 1u, abort_flag, p.status, kStatusAttention + 0)) break;
                const uint32_t k_dst = kv_addr + s * T::kStageBytes, v_dst = k_dst + T::kHalfBytes;
                const uint32_t full_first = ptx::map_to_cta(kv_full(s), 0);
                if (rank == 0) ptx::mbar_arrive_expect_tx(kv_full(s), 2 * T::kStageBytes);
                const int key_row = static_cast<int>(row.kv_begin + j * kKeys);
                for (int b = 0; b < D / 64; ++b)  // this CTA's 64 keys: boxes of [64 keys x 64 dimensions]
                    ptx::tma_load_2d_pair(k_dst + b * (64 * 128), &map_k, full_first, static_cast<int>(kv_head * D + 64 * b), key_row + static_cast<int>(rank * 64));
                for (int b = 0; b < D / 128; ++b)  // this CTA's half of the dimensions of all 128 values: boxes of [128 values x 64 dimensions]
                    ptx::tma_load_2d_pair(v_dst + b * (kKeys * 128), &map_v, full_first, static_cast<int>(kv_head * D + rank * (D / 2) + 64 * b), key_row);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc_s = ptx::instr_desc_f16_f32acc(2 * kQueries, kKeys);
            // The descriptors are made once: an MMA of 256 x 128 x 16 is 64 cycles of tensor work, and building two descriptors for each
            // would take the issuing thread about as long.
            uint64_t dq[D / 16];
#pragma unroll
            for (int i = 0; i < D / 16; ++i) dq[i] = ptx::smem_desc_k_major_sw128(q_addr + (i / 4) * (kQueries * 128)) + 2u * (i % 4);
            const uint64_t dk_base = ptx::smem_desc_k_major_sw128(kv_addr);
            const auto issue_scores = [&](unsigned j) {
                const int s = static_cast<int>(j % kStages), sb = static_cast<int>(j & 1u);
                const uint64_t dk = dk_base + static_cast<uint64_t>((s * T::kStageBytes) >> 4);
#pragma unroll
                for (int i = 0; i < D / 16; ++i)  // box i / 4 of 64 dimensions (8 KB of this CTA's 64 keys), 16 dimensions i % 4 inside it
                    ptx::mma_f16_ss_pair(tmem_base + sb * kKeys, dq[i], dk + static_cast<uint64_t>((i / 4) * 512 + (i % 4) * 2), idesc_s, i != 0 ? 1u : 0u);
                ptx::mma_commit_pair(s_full(sb), 3);
            };
            // This thread issues the score products only; O += P V has a thread of its own (below). A thread that has issued a
            // tcgen05.commit cannot issue MMAs again until the MMAs before the commit have drained (about 500 clocks), so one thread
            // issuing both took about 128 clocks an MMA whatever its width (3,072 a block of keys for 2,048 clocks of tensor work);
            // with two, one thread's drain is the other's turn. The two write different accumulators, so the order in which the
            // tensor core takes their MMAs does not matter; what does is kept by barriers: S_n goes into the buffer of P_{n-2} and is
            // issued only when P_{n-2} V_{n-2} has finished (p_free).
            bool ok = wait_barrier(q_full, 0, abort_flag, p.status, kStatusAttention + 1);
            for (unsigned n = 0; ok && n < n_blocks; ++n) {
                ok = wait_barrier(kv_full(n % kStages), (n / kStages) & 1u, abort_flag, p.status, kStatusAttention + 2);
                if (ok && n >= 2) ok = wait_barrier(p_free(n & 1u), ((n - 2) >> 1) & 1u, abort_flag, p.status, kStatusAttention + 3);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                issue_scores(n);
            }
        }
        __syncwarp();
    } else if (warp == kAttentionPairValueIssuer) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc_o = ptx::instr_desc_f16_f32acc_b_mn(2 * kQueries, D);
            const uint32_t o_tmem = tmem_base + T::kOCol;
            const uint64_t dv_base = ptx::smem_desc_mn_major_sw128(kv_addr + T::kHalfBytes, kKeys * 128);
            bool ok = true;
            for (unsigned j = 0; ok && j < n_blocks; ++j) {
                const int s = static_cast<int>(j % kStages), sb = static_cast<int>(j & 1u);
                // the values of block j have landed (the score thread waited for the same barrier), and P_j is in tensor memory
                ok = wait_barrier(kv_full(s), (j / kStages) & 1u, abort_flag, p.status, kStatusAttention + 2) &&
                     wait_barrier(p_full(sb), (j >> 1) & 1u, abort_flag, p.status, kStatusAttention + 4);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint64_t dv = dv_base + static_cast<uint64_t>((s * T::kStageBytes) >> 4);
#pragma unroll
                for (int kb = 0; kb < kKeys / 16; ++kb)  // P_j from tensor memory: 16 keys are 8 columns; 16 values are 2048 bytes further
                    ptx::mma_f16_ts_pair(o_tmem, tmem_base + sb * kKeys + kb * 8, dv + static_cast<uint64_t>(kb * 128), idesc_o, (j > 0 || kb > 0) ? 1u : 0u);
                // S_j was consumed before P_j existed, so the stage's keys are done with too when these MMAs are
                ptx::mma_commit_pair(kv_empty(s), 3);
                ptx::mma_commit_pair(p_free(sb), 3);
            }
        }
        __syncwarp();
    } else {
        // Sixteen warps: the four warps w, w + 4, w + 8, w + 12 share the 32 queries of tensor-memory lanes 32 (w % 4) ..., each taking a
        // quarter of a block's keys (and later of the head's dimensions): four warps per scheduler hide each other's latencies (with two,
        // the schedulers issued one cycle in three).
        constexpr int kSplit = 4;
        constexpr int kW = kKeys / kSplit;            // keys of a block per thread: 32
        constexpr int kDq = D / kSplit;               // output dimensions per thread: 32 or 64
        const unsigned quarter = warp % 4;
        const unsigned side = (warp - 2) / 4;         // which quarter of the keys
        const unsigned r = quarter * 32 + lane;
        const uint32_t lane_base = tmem_base + ((quarter * 32u) << 16);
        const unsigned q_index = row.context + q0 + r;
        const auto row_sync = [&] { asm volatile("bar.sync %0, 128;" ::"r"(2u + quarter) : "memory"); };  // the four warps of these rows
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        for (unsigned j = 0; j < n_blocks; ++j) {
            const int sb = static_cast<int>(j & 1u);
            // (once a wait has given up, the waits return at once and the loop runs on over garbage: the warps of a quarter must keep
            // meeting at their named barrier, which has no time limit)
            if (ok) ok = wait_barrier(s_full(sb), (j >> 1) & 1u, abort_flag, p.status, kStatusAttention + 5);
            ptx::tc_fence_after_sync();
            const unsigned key0 = j * kKeys + side * kW;
            const bool diagonal = j * kKeys + kKeys - 1 > row.context + q0;
            float t[kW];
            {
                uint32_t v[32];
                ptx::tmem_ld_32x32(lane_base + sb * kKeys + side * kW, v);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) t[i] = __uint_as_float(v[i]);
            }
            if (diagonal) {
#pragma unroll
                for (int i = 0; i < kW; ++i)
                    if (key0 + i > q_index) t[i] = -INFINITY;
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < kW; ++i) mx[i & 3] = fmaxf(mx[i & 3], t[i]);
            exchange[side * 128 + r] = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            row_sync();
            const float block_max = fmaxf(fmaxf(exchange[r], exchange[128 + r]), fmaxf(exchange[256 + r], exchange[384 + r])) * p.scale_log2;
            row_sync();  // all four have read: the next block may overwrite
            float alpha = 1.0f;
            if (block_max > m + 8.0f) {  // also the first block (m = -inf), where alpha is 0 and O is not touched
                alpha = fast_exp2(m - block_max);
                m = block_max;
            }
            // Probabilities as binary16, two keys to a 32-bit column, over the scores they came from: all four parts of the query have
            // their scores in registers (the exchange above saw to that), and the next S into this buffer is issued after P_j V_j.
            float sum[2] = {0.0f, 0.0f};
            uint32_t packed[kW / 2];
#pragma unroll
            for (int i = 0; i < kW; i += 2) {
                const float e0 = fast_exp2(__fmaf_rn(t[i], p.scale_log2, -m));
                const float e1 = fast_exp2(__fmaf_rn(t[i + 1], p.scale_log2, -m));
                sum[0] += e0;
                sum[1] += e1;
                const __half2 h = __floats2half2_rn(e0, e1);
                packed[i / 2] = *reinterpret_cast<const unsigned*>(&h);
            }
            ptx::tmem_st_32x16(lane_base + sb * kKeys + side * (kW / 2), packed);
            if (j > 0 && __any_sync(0xFFFFFFFFu, alpha != 1.0f)) {  // O must hold P V of block j - 1 first
                const unsigned before = j - 1;
                if (ok) ok = wait_barrier(p_free(before & 1u), (before >> 1) & 1u, abort_flag, p.status, kStatusAttention + 6);
                ptx::tc_fence_after_sync();
#pragma unroll 1
                for (int c = 0; c < kDq; c += 32) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(lane_base + T::kOCol + side * kDq + c, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    ptx::tmem_st_32x32(lane_base + T::kOCol + side * kDq + c, v);
                }
            }
            ptx::tmem_st_wait();
            l = l * alpha + (sum[0] + sum[1]);
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(p_full(sb), 0));  // one arrival for the warp
        }
        if (ok && n_blocks > 0) {
            const unsigned last = n_blocks - 1;
            ok = wait_barrier(p_free(last & 1u), (last >> 1) & 1u, abort_flag, p.status, kStatusAttention + 7);
        }
        exchange[side * 128 + r] = l;
        row_sync();
        const float total = (exchange[r] + exchange[128 + r]) + (exchange[256 + r] + exchange[384 + r]);
        if (ok) {
            ptx::tc_fence_after_sync();
            const float inv_l = 1.0f / total;
            const size_t token = static_cast<size_t>(row.q_begin) + q0 + r;
            __half* dst = p.out + token * p.out_stride + static_cast<size_t>(head) * D + side * kDq;
            const size_t gate0 = token * p.gate_stride + static_cast<size_t>(head) * 2 * D + D + side * kDq;
#pragma unroll 1
            for (int c = 0; c < kDq; c += 32) {
                uint32_t v[32];
                ptx::tmem_ld_32x32(lane_base + T::kOCol + side * kDq + c, v);
                ptx::tmem_ld_wait();
                if (r < valid) {
                    unsigned packed[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float g0 = band_value(p.gate, gate0 + c + i, p.gate_half), g1 = band_value(p.gate, gate0 + c + i + 1, p.gate_half);
                        const float o0 = __uint_as_float(v[i]) * inv_l * (1.0f / (1.0f + expf(-g0)));
                        const float o1 = __uint_as_float(v[i + 1]) * inv_l * (1.0f / (1.0f + expf(-g1)));
                        const __half2 h = __floats2half2_rn(o0, o1);
                        packed[i / 2] = *reinterpret_cast<const unsigned*>(&h);
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        *reinterpret_cast<uint4*>(dst + c + 8 * q) = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
            }
        }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();  // neither CTA leaves while the other may still signal its barriers or read its shared memory
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, 512);
    }
}

void check_shape(const AttentionShape& s) {
    if (!attention_supports(s))
        throw std::invalid_argument("sepal_b200 attention: head_dim must be 128 or 256, heads a multiple of kv_heads, rotary_dims even and at most head_dim");
}

// The rows and, after them, what else a launch needs, copied to the context's table. Returns the device address of the rows.
const AttentionRow* upload_rows(Context& ctx, const AttentionRow* rows, std::size_t n_rows, const void* extra, std::size_t extra_bytes, const void** extra_dev,
                                cudaStream_t stream) {
    if (ctx.table == nullptr) throw std::invalid_argument("sepal_b200 attention: this context has no table memory");
    const std::size_t row_bytes = n_rows * sizeof(AttentionRow);
    const std::size_t need = (row_bytes + 15) / 16 * 16 + extra_bytes;
    if (need > ctx.table_bytes / 2) throw std::invalid_argument("sepal_b200 attention: " + std::to_string(n_rows) + " rows are more than the context's table holds");
    // two halves used in turn, so that the table of the launch before this one is not overwritten while it may still run
    char* base = static_cast<char*>(ctx.table) + (ctx.table_turn++ & 1u) * (ctx.table_bytes / 2);
    check(cudaMemcpyAsync(base, rows, row_bytes, cudaMemcpyHostToDevice, stream), "cudaMemcpyAsync(rows)");
    if (extra_bytes != 0) {
        check(cudaMemcpyAsync(base + (row_bytes + 15) / 16 * 16, extra, extra_bytes, cudaMemcpyHostToDevice, stream), "cudaMemcpyAsync(table)");
        *extra_dev = base + (row_bytes + 15) / 16 * 16;
    }
    return reinterpret_cast<const AttentionRow*>(base);
}

void check_rows(const AttentionRow* rows, std::size_t n_rows, std::size_t n_tokens, std::size_t arena_tokens) {
    for (std::size_t i = 0; i < n_rows; ++i) {
        const AttentionRow& r = rows[i];
        if (r.length == 0) throw std::invalid_argument("sepal_b200 attention: row " + std::to_string(i) + " is empty");
        if (i > 0 && r.q_begin < rows[i - 1].q_begin + rows[i - 1].length) throw std::invalid_argument("sepal_b200 attention: rows must be sorted by their first token and must not overlap");
        if (n_tokens != 0 && static_cast<std::size_t>(r.q_begin) + r.length > n_tokens) throw std::invalid_argument("sepal_b200 attention: row " + std::to_string(i) + " ends past the call's tokens");
        if (static_cast<std::size_t>(r.kv_begin) + r.context + r.length > arena_tokens)
            throw std::invalid_argument("sepal_b200 attention: row " + std::to_string(i) + " ends past the key/value arena");
    }
}

}  // namespace

bool attention_supports(const AttentionShape& s) {
    return (s.head_dim == 128 || s.head_dim == 256) && s.kv_heads != 0 && s.heads != 0 && s.heads % s.kv_heads == 0 && s.rotary_dims % 2 == 0 &&
           s.rotary_dims <= s.head_dim;
}

void launch_attention_prepare(Context& ctx, const AttentionShape& shape, const AttentionRow* rows, std::size_t n_rows, Band q_gate, Band k, Band v,
                              const float* q_norm, const float* k_norm, void* q_out, std::size_t q_stride, void* k_arena, void* v_arena,
                              std::size_t arena_tokens, cudaStream_t stream) {
    check_shape(shape);
    if (n_rows == 0) return;
    if (rows == nullptr || q_gate.data == nullptr || k.data == nullptr || v.data == nullptr || q_norm == nullptr || k_norm == nullptr || q_out == nullptr ||
        k_arena == nullptr || v_arena == nullptr)
        throw std::invalid_argument("sepal_b200 attention: null pointer");
    check_rows(rows, n_rows, 0, arena_tokens);
    check(cudaSetDevice(ctx.device), "cudaSetDevice");
    std::vector<double> inv_freq(shape.rotary_dims / 2);
    for (std::size_t i = 0; i < inv_freq.size(); ++i) inv_freq[i] = std::pow(shape.rope_theta, -static_cast<double>(2 * i) / static_cast<double>(shape.rotary_dims));
    const void* inv_dev = nullptr;
    PrepareParams p{};
    p.rows = upload_rows(ctx, rows, n_rows, inv_freq.data(), inv_freq.size() * sizeof(double), &inv_dev, stream);
    p.n_rows = static_cast<unsigned>(n_rows);
    p.heads = shape.heads;
    p.kv_heads = shape.kv_heads;
    p.head_dim = shape.head_dim;
    p.rotary_dims = shape.rotary_dims;
    p.eps = shape.eps;
    p.inv_freq = static_cast<const double*>(inv_dev);
    p.q_gate = q_gate.data;
    p.k = k.data;
    p.v = v.data;
    p.q_gate_stride = q_gate.stride;
    p.k_stride = k.stride;
    p.v_stride = v.stride;
    p.q_gate_half = q_gate.half ? 1u : 0u;
    p.k_half = k.half ? 1u : 0u;
    p.v_half = v.half ? 1u : 0u;
    p.q_norm = q_norm;
    p.k_norm = k_norm;
    p.q_out = static_cast<__half*>(q_out);
    p.q_stride = q_stride;
    p.k_arena = static_cast<__half*>(k_arena);
    p.v_arena = static_cast<__half*>(v_arena);
    const unsigned first = rows[0].q_begin, last = rows[n_rows - 1].q_begin + rows[n_rows - 1].length;
    (void)first;
    launch_kernel(attention_prepare_kernel, dim3(last), dim3(256), 0, stream, "attention_prepare_kernel launch", p);
    count_launch();
}

void launch_attention(Context& ctx, const AttentionShape& shape, const AttentionRow* rows, std::size_t n_rows, std::size_t n_tokens, const void* q,
                      std::size_t q_stride, const void* k_arena, const void* v_arena, std::size_t arena_tokens, Band gate, void* out,
                      std::size_t out_stride, cudaStream_t stream) {
    check_shape(shape);
    if (n_rows == 0) return;
    if (rows == nullptr || q == nullptr || k_arena == nullptr || v_arena == nullptr || gate.data == nullptr || out == nullptr)
        throw std::invalid_argument("sepal_b200 attention: null pointer");
    if (q_stride % 8 != 0 || out_stride % 8 != 0 || reinterpret_cast<std::uintptr_t>(q) % 16 != 0 || reinterpret_cast<std::uintptr_t>(out) % 16 != 0 ||
        reinterpret_cast<std::uintptr_t>(k_arena) % 16 != 0 || reinterpret_cast<std::uintptr_t>(v_arena) % 16 != 0)
        throw std::invalid_argument("sepal_b200 attention: q, out and the arenas must be 16-byte aligned with row strides that are multiples of 8");
    check_rows(rows, n_rows, n_tokens, arena_tokens);
    check(cudaSetDevice(ctx.device), "cudaSetDevice");
    const unsigned D = shape.head_dim;
    unsigned longest = 0;
    for (std::size_t i = 0; i < n_rows; ++i) longest = std::max(longest, rows[i].length);
    const bool pair = longest > static_cast<unsigned>(kQueries);  // CTA pairs take 256 queries at a time
    const unsigned per_block = pair ? 2u * kQueries : static_cast<unsigned>(kQueries);
    const unsigned keys = pair ? 128u : (D == 128 ? 128u : 64u);
    // (row, query block) pairs, the ones with the most keys first: they take longest
    struct Block {
        unsigned row, qb, work;
    };
    std::vector<Block> blocks;
    for (std::size_t i = 0; i < n_rows; ++i)
        for (unsigned qb = 0; qb * per_block < rows[i].length; ++qb) blocks.push_back({static_cast<unsigned>(i), qb, rows[i].context + (qb + 1) * per_block});
    std::stable_sort(blocks.begin(), blocks.end(), [](const Block& a, const Block& b) { return a.work > b.work; });
    std::vector<unsigned> table(2 * blocks.size());
    for (std::size_t i = 0; i < blocks.size(); ++i) {
        table[2 * i] = blocks[i].row;
        table[2 * i + 1] = blocks[i].qb;
    }
    const void* table_dev = nullptr;
    AttentionParams p{};
    p.rows = upload_rows(ctx, rows, n_rows, table.data(), table.size() * sizeof(unsigned), &table_dev, stream);
    p.blocks = static_cast<const unsigned*>(table_dev);
    p.heads = shape.heads;
    p.group = shape.heads / shape.kv_heads;
    p.scale_log2 = static_cast<float>(1.4426950408889634 / std::sqrt(static_cast<double>(D)));
    p.gate = gate.data;
    p.gate_stride = gate.stride;
    p.gate_half = gate.half ? 1u : 0u;
    p.out = static_cast<__half*>(out);
    p.out_stride = out_stride;
    p.status = ctx.status;
    const std::size_t kv_cols = static_cast<std::size_t>(shape.kv_heads) * D;
    const CUtensorMap map_q = make_tensor_map_2d(ctx, q, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, n_tokens, static_cast<std::size_t>(shape.heads) * D, q_stride, kQueries, 64, true);
    // a CTA of a pair loads 64 of a block's 128 keys, and all 128 values (half of their dimensions)
    const CUtensorMap map_k = make_tensor_map_2d(ctx, k_arena, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, arena_tokens, kv_cols, kv_cols, pair ? 64u : keys, 64, true);
    const CUtensorMap map_v = make_tensor_map_2d(ctx, v_arena, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, arena_tokens, kv_cols, kv_cols, keys, 64, true);
    const auto launch = [&](auto kernel, int smem, unsigned ctas_per_block, const char* what) {
        static bool configured[4][64] = {};
        const int which = (pair ? 2 : 0) + (D == 256 ? 1 : 0);
        if (ctx.device >= 64 || !configured[which][ctx.device]) {
            check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute");
            if (ctx.device < 64) configured[which][ctx.device] = true;
        }
        launch_kernel(kernel, dim3(static_cast<unsigned>(blocks.size()) * ctas_per_block, shape.heads), dim3(pair ? kAttentionPairThreads : 320), static_cast<std::size_t>(smem), stream,
                      what, map_q, map_k, map_v, p);
    };
    if (pair && D == 128) launch(attention_pair_kernel<128>, AttentionPairTile<128>::kSmem, 2, "attention_pair_kernel launch");
    else if (pair) launch(attention_pair_kernel<256>, AttentionPairTile<256>::kSmem, 2, "attention_pair_kernel launch");
    else if (D == 128) launch(attention_kernel<128>, AttentionTile<128>::kSmem, 1, "attention_kernel launch");
    else launch(attention_kernel<256>, AttentionTile<256>::kSmem, 1, "attention_kernel launch");
    count_launch();
}

}  // namespace sepal::b200
