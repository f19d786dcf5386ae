#include "deltanet.hpp"

#include <algorithm>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_fp16.h>

#include "ptx.cuh"

namespace sepal::b200 {

void count_launch();

namespace {

constexpr int kDim = 128;  // dk = dv

// Sixteen (at the end of a run: fewer) consecutive tokens of a run, counted from the run's first token.
struct DeltaChunk {
    unsigned token0, count, row, unused;
};

struct DeltaParams {
    const DeltaNetRow* rows;
    unsigned n_rows;
    unsigned key_heads, value_heads, taps;
    unsigned key_dim, value_dim, conv_dim;
    float eps;
    const void* mixed;
    const void* z;
    const void* b;
    const void* a;
    unsigned long long mixed_stride, z_stride, b_stride, a_stride;
    unsigned mixed_half, z_half, b_half, a_half;
    const float* conv;
    const float* a_log;
    const float* dt_bias;
    const float* norm;
    float* q;
    float* k;
    float* v;
    float* decay;
    float* beta;
    float* reads;  // [N, value_dim]: the scan's output before the gated norm
    float* coef;   // [N, value_heads, 36]: the chunk coefficients of every token
    const DeltaChunk* chunks;
    float* states;
    float* tails;  // [slots, taps - 1, conv_dim]
    __half* out;
    unsigned long long out_stride;
};

__device__ __forceinline__ float value_of(const void* base, unsigned long long index, unsigned half) {
    return half != 0 ? __half2float(static_cast<const __half*>(base)[index]) : static_cast<const float*>(base)[index];
}
// softplus in the reference's form (runner/include/sepal/ref/primitives.hpp:25-40); sigmoid as 1 / (1 + e^-x), which the reference
// writes as exp(-softplus(-x)): the same function, an ulp or two apart in float32, and a third of the instructions (it runs once per
// element of the convolution's output).
__device__ __forceinline__ float softplus(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoid(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float silu(float x) { return __fmul_rn(x, sigmoid(x)); }

__device__ __forceinline__ unsigned row_of(const DeltaNetRow* rows, unsigned n_rows, unsigned token) {
    unsigned lo = 0, hi = n_rows;
    while (hi - lo > 1) {
        const unsigned mid = (lo + hi) / 2;
        if (rows[mid].q_begin <= token) lo = mid; else hi = mid;
    }
    return lo;
}

// One block per token: the convolution (taps in ascending order, the last on the token itself; inputs before the run come from the
// slot's tail, zeros for a fresh request), SiLU, q and k normalised per head, v as it is; the token's decay and beta per value head.
__global__ void __launch_bounds__(256) deltanet_prepare_kernel(const DeltaParams p) {
    extern __shared__ float activated[];  // [conv_dim]
    __shared__ float head_sums[64];
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const unsigned token = blockIdx.x;
    const DeltaNetRow row = p.rows[row_of(p.rows, p.n_rows, token)];
    if (token < row.q_begin || token >= row.q_begin + row.length) return;
    const unsigned t = token - row.q_begin;
    const unsigned history = p.taps - 1;
    const float* tail = p.tails + static_cast<size_t>(row.slot) * history * p.conv_dim;
    if (p.mixed_half != 0 && p.taps == 4 && t >= history && p.mixed_stride % 2 == 0 && p.conv_dim % 2 == 0 &&
        reinterpret_cast<unsigned long long>(p.mixed) % 4 == 0 && reinterpret_cast<unsigned long long>(p.conv) % 16 == 0) {
        // the common case: every tap reads the call's own rows; two channels a thread (one 4-byte load a tap, the taps of a channel as
        // one 16-byte load), the same sums in the same order as the general loop below
        const __half2* in = reinterpret_cast<const __half2*>(static_cast<const __half*>(p.mixed) + (static_cast<size_t>(token) - history) * p.mixed_stride);
        const unsigned pitch = static_cast<unsigned>(p.mixed_stride / 2);
        const float4* taps = reinterpret_cast<const float4*>(p.conv);
        for (unsigned c2 = threadIdx.x; c2 < p.conv_dim / 2; c2 += blockDim.x) {
            const float2 x0 = __half22float2(in[c2]), x1 = __half22float2(in[c2 + pitch]), x2 = __half22float2(in[c2 + 2 * pitch]),
                         x3 = __half22float2(in[c2 + 3 * pitch]);
            const float4 w0 = taps[2 * c2], w1 = taps[2 * c2 + 1];
            float lo = __fadd_rn(0.0f, __fmul_rn(w0.x, x0.x)), hi = __fadd_rn(0.0f, __fmul_rn(w1.x, x0.y));
            lo = __fadd_rn(lo, __fmul_rn(w0.y, x1.x)), hi = __fadd_rn(hi, __fmul_rn(w1.y, x1.y));
            lo = __fadd_rn(lo, __fmul_rn(w0.z, x2.x)), hi = __fadd_rn(hi, __fmul_rn(w1.z, x2.y));
            lo = __fadd_rn(lo, __fmul_rn(w0.w, x3.x)), hi = __fadd_rn(hi, __fmul_rn(w1.w, x3.y));
            *reinterpret_cast<float2*>(&activated[2 * c2]) = make_float2(silu(lo), silu(hi));
        }
    } else {
        for (unsigned c = threadIdx.x; c < p.conv_dim; c += blockDim.x) {
            float acc = 0.0f;
            for (unsigned j = 0; j < p.taps; ++j) {
                // window index t + j over (tail, then the run's inputs): the input of token t + j - history, or tail row t + j
                float x;
                if (t + j >= history) x = value_of(p.mixed, (static_cast<size_t>(token) + j - history) * p.mixed_stride + c, p.mixed_half);
                else x = row.fresh != 0 ? 0.0f : tail[static_cast<size_t>(t + j) * p.conv_dim + c];
                acc = __fadd_rn(acc, __fmul_rn(p.conv[static_cast<size_t>(c) * p.taps + j], x));
            }
            activated[c] = silu(acc);
        }
    }
    __syncthreads();
    // q and k heads: 2 * key_heads vectors of 128; one warp per head in turn
    const unsigned warp = threadIdx.x / 32, lane = threadIdx.x % 32, warps = blockDim.x / 32;
    for (unsigned h = warp; h < 2 * p.key_heads; h += warps) {
        const float* x = activated + h * kDim;
        float ss = 0.0f;
        for (int e = 0; e < 4; ++e) ss = __fmaf_rn(x[lane + 32 * e], x[lane + 32 * e], ss);
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        if (lane == 0) head_sums[h] = ss;
    }
    __syncthreads();
    for (unsigned c = threadIdx.x; c < p.conv_dim; c += blockDim.x) {
        if (c < 2 * p.key_dim) {
            const float value = __fdiv_rn(activated[c], __fsqrt_rn(__fadd_rn(head_sums[c / kDim], 1.0e-6f)));
            if (c < p.key_dim) p.q[static_cast<size_t>(token) * p.key_dim + c] = value;
            else p.k[static_cast<size_t>(token) * p.key_dim + (c - p.key_dim)] = value;
        } else {
            p.v[static_cast<size_t>(token) * p.value_dim + (c - 2 * p.key_dim)] = activated[c];
        }
    }
    for (unsigned h = threadIdx.x; h < p.value_heads; h += blockDim.x) {
        const float a = value_of(p.a, static_cast<size_t>(token) * p.a_stride + h, p.a_half);
        const float b = value_of(p.b, static_cast<size_t>(token) * p.b_stride + h, p.b_half);
        p.decay[static_cast<size_t>(token) * p.value_heads + h] = expf(-expf(p.a_log[h]) * softplus(a + p.dt_bias[h]));
        p.beta[static_cast<size_t>(token) * p.value_heads + h] = sigmoid(b);
    }
}

// After the prepare launch: the slot's tail becomes the last K - 1 rows of (old tail, then the run's inputs). One thread per run and
// channel.
__global__ void deltanet_tail_kernel(const DeltaParams p) {
    const DeltaNetRow row = p.rows[blockIdx.x];
    const unsigned history = p.taps - 1;
    float* tail = p.tails + static_cast<size_t>(row.slot) * history * p.conv_dim;
    const unsigned c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c < p.conv_dim) {
        for (unsigned i = 0; i < history; ++i) {  // ascending: row length + i of the window is read before row i is written (length >= 1)
            const unsigned w = row.length + i;
            float x;
            if (w >= history) x = value_of(p.mixed, (static_cast<size_t>(row.q_begin) + w - history) * p.mixed_stride + c, p.mixed_half);
            else x = row.fresh != 0 ? 0.0f : tail[static_cast<size_t>(w) * p.conv_dim + c];
            tail[static_cast<size_t>(i) * p.conv_dim + c] = x;
        }
    }
}

// The delta rule in chunks of sixteen tokens. With d_t the decay of token t, c_t its correction beta_t (v_t - k_t . d_t S_{t-1}) and
// S_t = d_t S_{t-1} + k_t (x) c_t, unrolling from the state S_0 before the chunk gives, with P(s, t) = d_{s+1} ... d_t and
// gamma_t = d_0 ... d_t (tokens numbered from 0 inside the chunk):
//     c_t    = beta_t (v_t - gamma_t k_t . S_0 - sum_{s<t} P(s, t) (k_t . k_s) c_s)
//     read_t = (gamma_t q_t . S_0 + sum_{s<=t} P(s, t) (q_t . k_s) c_s) / sqrt(dk)
//     S_end  = gamma_last S_0 + sum_s P(s, last) k_s (x) c_s
// so the products with S_0 of all sixteen tokens are independent (their cross-lane sums go out together: one shuffle latency a chunk
// instead of one a token), and what is left of the chain is a few multiply-adds per token on coefficients that do not involve the
// state. Those coefficients, per token s and value head, are formed by deltanet_gram_kernel: col_a[t] = P(s, t) (k_t . k_s) for t > s,
// col_b[t] = P(s, t) (q_t . k_s) for t >= s, gamma_s and the carry P(s, last). The same sums as the token-by-token rule in another
// order: float32 results agree to rounding.
constexpr int kChunk = 16;
constexpr int kCoef = 36;  // floats per (token, value head): col_a[16], col_b[16], gamma, carry, two of padding (rows of 144 bytes)
constexpr int kCols = 16;  // columns of the state per CTA: four warps of four columns
constexpr int kScanThreads = 8 * kCols;  // eight row groups of 16 rows a column

// One block per chunk and key head, 256 threads: thread (s, t) forms k_t . k_s and q_t . k_s once and, for every value head of the
// key head, scales them by that head's P(s, t).
__global__ void __launch_bounds__(256) deltanet_gram_kernel(const DeltaParams p) {
    __shared__ float k_sh[kChunk][kDim + 1], q_sh[kChunk][kDim + 1];
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const DeltaChunk chunk = p.chunks[blockIdx.x];
    const unsigned key_head = blockIdx.y;
    for (unsigned e = threadIdx.x; e < kChunk * kDim; e += 256) {
        const unsigned t = e / kDim, d = e % kDim;
        const bool live = t < chunk.count;
        k_sh[t][d] = live ? p.k[(static_cast<size_t>(chunk.token0) + t) * p.key_dim + key_head * kDim + d] : 0.0f;
        q_sh[t][d] = live ? p.q[(static_cast<size_t>(chunk.token0) + t) * p.key_dim + key_head * kDim + d] : 0.0f;
    }
    __syncthreads();
    const unsigned s = threadIdx.x / kChunk, t = threadIdx.x % kChunk;
    if (s >= chunk.count) return;
    float kk = 0.0f, qk = 0.0f;
    for (int d = 0; d < kDim; ++d) {
        kk = __fmaf_rn(k_sh[t][d], k_sh[s][d], kk);
        qk = __fmaf_rn(q_sh[t][d], k_sh[s][d], qk);
    }
    const unsigned group = p.value_heads / p.key_heads;
    for (unsigned h = key_head * group; h < (key_head + 1) * group; ++h) {
        const float* decay = p.decay + static_cast<size_t>(chunk.token0) * p.value_heads + h;  // token r of the chunk at decay[r * value_heads]
        float product = 1.0f;  // P(s, t), 0 where t < s or the token does not exist
        for (unsigned r = s + 1; r <= t && r < chunk.count; ++r) product = __fmul_rn(product, decay[static_cast<size_t>(r) * p.value_heads]);
        float* row = p.coef + ((static_cast<size_t>(chunk.token0) + s) * p.value_heads + h) * kCoef;
        const bool live = t < chunk.count;
        row[t] = live && t > s ? __fmul_rn(product, kk) : 0.0f;
        row[kChunk + t] = live && t >= s ? __fmul_rn(product, qk) : 0.0f;
        if (t == 0) {
            float gamma = 1.0f, carry = 1.0f;
            for (unsigned r = 0; r <= s; ++r) gamma = __fmul_rn(gamma, decay[static_cast<size_t>(r) * p.value_heads]);
            for (unsigned r = s + 1; r < chunk.count; ++r) carry = __fmul_rn(carry, decay[static_cast<size_t>(r) * p.value_heads]);
            row[2 * kChunk] = gamma;
            row[2 * kChunk + 1] = carry;
            row[2 * kChunk + 2] = 0.0f;
            row[2 * kChunk + 3] = 0.0f;
        }
    }
}

// What the sixteen tokens of a chunk need from global memory, fetched by asynchronous copies into one of two buffers while the chunk
// before it is being worked on.
struct ScanStage {
    float k[kChunk][kDim], q[kChunk][kDim];
    float coef[kChunk][kCoef];
    float v[kChunk][kCols];
    float beta[kChunk];
};

__device__ __forceinline__ void scan_prefetch(const DeltaParams& p, ScanStage& st, const DeltaNetRow& row, unsigned t0, unsigned head,
                                              unsigned key_head, unsigned first_col) {
    if (t0 >= row.length) return;
    const unsigned count = min(static_cast<unsigned>(kChunk), row.length - t0);
    const size_t token0 = static_cast<size_t>(row.q_begin) + t0;
    for (unsigned e = threadIdx.x; e < 2 * kChunk * kDim / 4; e += kScanThreads) {  // 16 bytes a copy
        const unsigned which = e / (kChunk * kDim / 4), tt = (e / (kDim / 4)) % kChunk, d = 4 * (e % (kDim / 4));
        if (tt < count)
            ptx::cp_async_16(which == 0 ? &st.k[tt][d] : &st.q[tt][d],
                             (which == 0 ? p.k : p.q) + (token0 + tt) * p.key_dim + key_head * kDim + d);
    }
    for (unsigned e = threadIdx.x; e < kChunk * kCoef / 4; e += kScanThreads) {
        const unsigned tt = e / (kCoef / 4), d = 4 * (e % (kCoef / 4));
        if (tt < count) ptx::cp_async_16(&st.coef[tt][d], p.coef + ((token0 + tt) * p.value_heads + head) * kCoef + d);
    }
    for (unsigned e = threadIdx.x; e < kChunk * kCols / 4; e += kScanThreads) {
        const unsigned tt = e / (kCols / 4), d = 4 * (e % (kCols / 4));
        if (tt < count) ptx::cp_async_16(&st.v[tt][d], p.v + (token0 + tt) * p.value_dim + head * kDim + first_col + d);
    }
    if (threadIdx.x < kChunk && threadIdx.x < count) ptx::cp_async_4(&st.beta[threadIdx.x], p.beta + (token0 + threadIdx.x) * p.value_heads + head);
}

// The columns of a head's state S [dk, dv] evolve independently of one another, so a head is spread over eight CTAs of 16 columns:
// 128 threads, each holding 16 rows (one of eight row groups) of one column in registers; a warp owns four columns, lane = 4 g + c
// holding row group g of column c of them, so the eight partial sums of a column meet by three shuffles inside the warp, and the
// eight lanes of a quarter warp read two 16-byte pieces of k or q (no bank conflict). The reads go to global memory in float32; the
// gated norm over a head's 128 reads is the next launch.
__global__ void __launch_bounds__(kScanThreads) deltanet_scan_kernel(const DeltaParams p) {
    extern __shared__ __align__(16) unsigned char scan_smem[];
    ScanStage* stages = reinterpret_cast<ScanStage*>(scan_smem);
    ptx::grid_dependency_wait();
    const DeltaNetRow row = p.rows[blockIdx.x];
    const unsigned head = blockIdx.y, key_head = head / (p.value_heads / p.key_heads);
    const unsigned warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const unsigned g = lane / 4, jl = 4 * warp + lane % 4;
    const unsigned j = blockIdx.z * kCols + jl;  // this thread's column of the head
    scan_prefetch(p, stages[0], row, 0, head, key_head, blockIdx.z * kCols);
    float s[16];
    float* state = p.states + (static_cast<size_t>(row.slot) * p.value_heads + head) * kDim * kDim;
#pragma unroll
    for (int i = 0; i < 16; ++i) s[i] = row.fresh != 0 ? 0.0f : state[static_cast<size_t>(16 * g + i) * kDim + j];
    const float scale = rsqrtf(static_cast<float>(kDim));
    for (unsigned t0 = 0, turn = 0; t0 < row.length; t0 += kChunk, turn ^= 1u) {
        const int count = static_cast<int>(min(static_cast<unsigned>(kChunk), row.length - t0));
        const size_t token0 = static_cast<size_t>(row.q_begin) + t0;
        const ScanStage& st = stages[turn];
        ptx::cp_async_wait_all();
        __syncthreads();  // this chunk's values are in place; the chunk before it is done with the other buffer
        scan_prefetch(p, stages[turn ^ 1u], row, t0 + kChunk, head, key_head, blockIdx.z * kCols);
        // x[t] = k_t . S_0[:, j] and o[t] = q_t . S_0[:, j] over this thread's rows, then over the eight row groups
        float x[kChunk], o[kChunk];
#pragma unroll
        for (int t = 0; t < kChunk; ++t) {
            x[t] = 0.0f;
            o[t] = 0.0f;
            if (t < count) {
                const float4* k4 = reinterpret_cast<const float4*>(&st.k[t][16 * g]);
                const float4* q4 = reinterpret_cast<const float4*>(&st.q[t][16 * g]);
                float rec[4] = {0.0f, 0.0f, 0.0f, 0.0f}, rd[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float4 kk = k4[c], qq = q4[c];
                    rec[0] = __fmaf_rn(kk.x, s[4 * c], rec[0]);
                    rec[1] = __fmaf_rn(kk.y, s[4 * c + 1], rec[1]);
                    rec[2] = __fmaf_rn(kk.z, s[4 * c + 2], rec[2]);
                    rec[3] = __fmaf_rn(kk.w, s[4 * c + 3], rec[3]);
                    rd[0] = __fmaf_rn(qq.x, s[4 * c], rd[0]);
                    rd[1] = __fmaf_rn(qq.y, s[4 * c + 1], rd[1]);
                    rd[2] = __fmaf_rn(qq.z, s[4 * c + 2], rd[2]);
                    rd[3] = __fmaf_rn(qq.w, s[4 * c + 3], rd[3]);
                }
                x[t] = (rec[0] + rec[1]) + (rec[2] + rec[3]);
                o[t] = (rd[0] + rd[1]) + (rd[2] + rd[3]);
            }
        }
#pragma unroll
        for (int t = 0; t < kChunk; ++t) {
            if (t < count) {
#pragma unroll
                for (int w = 4; w < 32; w <<= 1) {  // every lane ends with the same sums
                    x[t] += __shfl_xor_sync(0xFFFFFFFFu, x[t], w);
                    o[t] += __shfl_xor_sync(0xFFFFFFFFu, o[t], w);
                }
                const float gamma = st.coef[t][2 * kChunk];
                x[t] = __fsub_rn(st.v[t][jl], __fmul_rn(gamma, x[t]));
                o[t] = __fmul_rn(gamma, o[t]);
            }
        }
        const float gamma_last = st.coef[count - 1][2 * kChunk];
#pragma unroll
        for (int i = 0; i < 16; ++i) s[i] = __fmul_rn(s[i], gamma_last);
        // the corrections in turn: each enters the later tokens' x and o through its coefficients, and the state through its carry
#pragma unroll
        for (int u = 0; u < kChunk; ++u) {
            if (u >= count) break;
            const float correction = __fmul_rn(st.beta[u], x[u]);
            float col[2 * kChunk];
#pragma unroll
            for (int c = u / 4; c < 4; ++c) {
                const float4 a4 = reinterpret_cast<const float4*>(&st.coef[u][0])[c], b4 = reinterpret_cast<const float4*>(&st.coef[u][kChunk])[c];
                col[4 * c] = a4.x, col[4 * c + 1] = a4.y, col[4 * c + 2] = a4.z, col[4 * c + 3] = a4.w;
                col[kChunk + 4 * c] = b4.x, col[kChunk + 4 * c + 1] = b4.y, col[kChunk + 4 * c + 2] = b4.z, col[kChunk + 4 * c + 3] = b4.w;
            }
#pragma unroll
            for (int t = u + 1; t < kChunk; ++t) x[t] = __fmaf_rn(-col[t], correction, x[t]);
#pragma unroll
            for (int t = u; t < kChunk; ++t) o[t] = __fmaf_rn(col[kChunk + t], correction, o[t]);
            const float carried = __fmul_rn(correction, st.coef[u][2 * kChunk + 1]);
            const float4* k4 = reinterpret_cast<const float4*>(&st.k[u][16 * g]);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float4 kk = k4[c];
                s[4 * c] = __fmaf_rn(kk.x, carried, s[4 * c]);
                s[4 * c + 1] = __fmaf_rn(kk.y, carried, s[4 * c + 1]);
                s[4 * c + 2] = __fmaf_rn(kk.z, carried, s[4 * c + 2]);
                s[4 * c + 3] = __fmaf_rn(kk.w, carried, s[4 * c + 3]);
            }
        }
        if (g == 0) {
#pragma unroll
            for (int t = 0; t < kChunk; ++t)
                if (t < count) p.reads[(token0 + t) * p.value_dim + head * kDim + j] = __fmul_rn(o[t], scale);
        }
    }
    ptx::grid_launch_dependents();
#pragma unroll
    for (int i = 0; i < 16; ++i) state[static_cast<size_t>(16 * g + i) * kDim + j] = s[i];
}

// The gated norm of every token's and value head's 128 reads: x / sqrt(mean(x^2) + eps) * weight * silu(z) (the weight itself, not
// 1 + weight). One warp per (token, head): lane l holds reads l, l + 32, ...; squares by fused multiply-add in that order, a butterfly.
__global__ void __launch_bounds__(256) deltanet_norm_kernel(const DeltaParams p, unsigned tokens) {
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const size_t unit = static_cast<size_t>(blockIdx.x) * 8 + threadIdx.x / 32;  // (token, head)
    if (unit >= static_cast<size_t>(tokens) * p.value_heads) return;
    const size_t token = unit / p.value_heads;
    const unsigned head = static_cast<unsigned>(unit % p.value_heads), lane = threadIdx.x % 32;
    const DeltaNetRow row = p.rows[row_of(p.rows, p.n_rows, static_cast<unsigned>(token))];
    if (token < row.q_begin || token >= static_cast<size_t>(row.q_begin) + row.length) return;
    const float* x = p.reads + token * p.value_dim + head * kDim;
    float v[4], ss = 0.0f;
    for (int e = 0; e < 4; ++e) {
        v[e] = x[lane + 32 * e];
        ss = __fmaf_rn(v[e], v[e], ss);
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    const float rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(kDim)), p.eps));
    __half* dst = p.out + token * p.out_stride + head * kDim;
    for (int e = 0; e < 4; ++e) {
        const unsigned d = lane + 32 * e;
        const float z = value_of(p.z, token * p.z_stride + head * kDim + d, p.z_half);
        dst[d] = __float2half_rn(__fmul_rn(__fmul_rn(__fdiv_rn(v[e], rms), p.norm[d]), silu(z)));
    }
}

}  // namespace

bool deltanet_supports(const DeltaNetShape& s) {
    return s.head_dim == 128 && s.key_heads != 0 && s.value_heads != 0 && s.value_heads % s.key_heads == 0 && s.key_heads <= 32 && s.conv_kernel >= 1 &&
           s.conv_kernel <= 8;
}

void launch_deltanet(Context& ctx, const DeltaNetShape& shape, const DeltaNetRow* rows, std::size_t n_rows, Band mixed, Band z, Band b, Band a,
                     const DeltaNetWeights& weights, const DeltaNetScratch& scratch, float* states, float* tails, std::size_t slots,
                     void* out, std::size_t out_stride, cudaStream_t stream) {
    if (!deltanet_supports(shape))
        throw std::invalid_argument("sepal_b200 deltanet: head_dim must be 128, value_heads a multiple of key_heads (at most 32 key heads), 1 to 8 conv taps");
    if (n_rows == 0) return;
    if (rows == nullptr || mixed.data == nullptr || z.data == nullptr || b.data == nullptr || a.data == nullptr || weights.conv == nullptr ||
        weights.a_log == nullptr || weights.dt_bias == nullptr || weights.norm == nullptr || scratch.q == nullptr || scratch.k == nullptr ||
        scratch.v == nullptr || scratch.decay == nullptr || scratch.beta == nullptr || scratch.reads == nullptr || scratch.coef == nullptr || states == nullptr || tails == nullptr || out == nullptr)
        throw std::invalid_argument("sepal_b200 deltanet: null pointer");
    for (std::size_t i = 0; i < n_rows; ++i) {
        if (rows[i].length == 0) throw std::invalid_argument("sepal_b200 deltanet: row " + std::to_string(i) + " is empty");
        if (i > 0 && rows[i].q_begin < rows[i - 1].q_begin + rows[i - 1].length) throw std::invalid_argument("sepal_b200 deltanet: rows must be sorted by their first token and must not overlap");
        if (rows[i].slot >= slots) throw std::invalid_argument("sepal_b200 deltanet: row " + std::to_string(i) + " names a state slot that does not exist");
        for (std::size_t o = 0; o < i; ++o)
            if (rows[o].slot == rows[i].slot) throw std::invalid_argument("sepal_b200 deltanet: two rows of one call share a state slot");
    }
    check(cudaSetDevice(ctx.device), "cudaSetDevice");
    // the table of the call: the runs, then their chunks of sixteen tokens
    std::vector<DeltaChunk> chunks;
    for (std::size_t i = 0; i < n_rows; ++i)
        for (std::uint32_t t0 = 0; t0 < rows[i].length; t0 += kChunk)
            chunks.push_back(DeltaChunk{rows[i].q_begin + t0, std::min<std::uint32_t>(kChunk, rows[i].length - t0), static_cast<unsigned>(i), 0u});
    const std::size_t rows_bytes = n_rows * sizeof(DeltaNetRow), table_bytes = rows_bytes + chunks.size() * sizeof(DeltaChunk);
    if (ctx.table == nullptr || table_bytes > ctx.table_bytes / 2) throw std::invalid_argument("sepal_b200 deltanet: too many rows for the context's table");
    std::vector<char> host(table_bytes);
    std::memcpy(host.data(), rows, rows_bytes);
    std::memcpy(host.data() + rows_bytes, chunks.data(), chunks.size() * sizeof(DeltaChunk));
    char* table = static_cast<char*>(ctx.table) + (ctx.table_turn++ & 1u) * (ctx.table_bytes / 2);
    check(cudaMemcpyAsync(table, host.data(), table_bytes, cudaMemcpyHostToDevice, stream), "cudaMemcpyAsync(rows)");
    DeltaParams p{};
    p.rows = reinterpret_cast<const DeltaNetRow*>(table);
    p.chunks = reinterpret_cast<const DeltaChunk*>(table + rows_bytes);
    p.n_rows = static_cast<unsigned>(n_rows);
    p.key_heads = shape.key_heads;
    p.value_heads = shape.value_heads;
    p.taps = shape.conv_kernel;
    p.key_dim = shape.key_dim();
    p.value_dim = shape.value_dim();
    p.conv_dim = shape.conv_dim();
    p.eps = shape.eps;
    p.mixed = mixed.data;
    p.z = z.data;
    p.b = b.data;
    p.a = a.data;
    p.mixed_stride = mixed.stride;
    p.z_stride = z.stride;
    p.b_stride = b.stride;
    p.a_stride = a.stride;
    p.mixed_half = mixed.half ? 1u : 0u;
    p.z_half = z.half ? 1u : 0u;
    p.b_half = b.half ? 1u : 0u;
    p.a_half = a.half ? 1u : 0u;
    p.conv = weights.conv;
    p.a_log = weights.a_log;
    p.dt_bias = weights.dt_bias;
    p.norm = weights.norm;
    p.q = scratch.q;
    p.k = scratch.k;
    p.v = scratch.v;
    p.decay = scratch.decay;
    p.beta = scratch.beta;
    p.reads = scratch.reads;
    p.coef = scratch.coef;
    p.states = states;
    p.tails = tails;
    p.out = static_cast<__half*>(out);
    p.out_stride = out_stride;
    const unsigned last = rows[n_rows - 1].q_begin + rows[n_rows - 1].length;
    const std::size_t prepare_smem = static_cast<std::size_t>(p.conv_dim) * sizeof(float);
    if (prepare_smem > 160 * 1024) throw std::invalid_argument("sepal_b200 deltanet: the convolution is wider than the prepare kernel's shared memory");
    static bool configured[64] = {};
    if (ctx.device >= 64 || !configured[ctx.device]) {
        check(cudaFuncSetAttribute(deltanet_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024), "cudaFuncSetAttribute");
        if (ctx.device < 64) configured[ctx.device] = true;
    }
    launch_kernel(deltanet_prepare_kernel, dim3(last), dim3(256), prepare_smem, stream, "deltanet_prepare_kernel launch", p);
    count_launch();
    if (shape.conv_kernel > 1) {
        deltanet_tail_kernel<<<dim3(static_cast<unsigned>(n_rows), (p.conv_dim + 255) / 256), 256, 0, stream>>>(p);
        check(cudaGetLastError(), "deltanet_tail_kernel launch");
        count_launch();
    }
    launch_kernel(deltanet_gram_kernel, dim3(static_cast<unsigned>(chunks.size()), shape.key_heads), dim3(256), 0, stream, "deltanet_gram_kernel launch", p);
    count_launch();
    // An ordinary launch, not an overlapped one: blocks of the scan that arrive while the launch before it still fills the SMs settle
    // wherever room appears first, several to an SM with other SMs left empty, and a run's eight blocks per head then take twice as long.
    deltanet_scan_kernel<<<dim3(static_cast<unsigned>(n_rows), shape.value_heads, kDim / kCols), dim3(kScanThreads), 2 * sizeof(ScanStage), stream>>>(p);
    check(cudaGetLastError(), "deltanet_scan_kernel launch");
    count_launch();
    const std::size_t units = static_cast<std::size_t>(last) * shape.value_heads;
    launch_kernel(deltanet_norm_kernel, dim3(static_cast<unsigned>((units + 7) / 8)), dim3(256), 0, stream, "deltanet_norm_kernel launch", p, last);
    count_launch();
}

}  // namespace sepal::b200
