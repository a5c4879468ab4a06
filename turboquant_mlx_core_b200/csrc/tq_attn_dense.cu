// The fp16 decode window (include/turboquant/decode_buffer.h:11-47, src/decode_buffer.cpp) on the
// device, and attention over it (the short-context branch of hybrid_attention,
// src/attention_dispatch.cpp:37-56: plain scaled-dot-product attention over the window's keys and
// values, fp16 operands, no mask, scale 1/sqrt(head_dim)).
//
// The window is a ring of `window` token slots, [slot][head][dim] fp16 per tensor; the slot of a
// token is its absolute index modulo the window size.  The reference keeps fp32 copies on the host
// and rounds to fp16 when a range is read; rounding once when a token is written gives the same
// fp16 values and halves the bytes the attention reads.
//
// Attention: one query position, GQA.  A CTA is (context split, KV head, group of up to 8 query
// heads); each of its four warps walks tiles of 32 tokens.  Scores: lane = token (the key row is
// read with 16-byte loads, the query sits in shared memory as fp32 and is read by broadcast); values: lane = a group of head_dim / 32 dims (rows read coalesced), probabilities
// passed through shared memory.  fp32 accumulation, online softmax per tile, partial
// (max, sum, accumulator) triples merged by dense_combine_kernel.  HBM-bound by design: 4 * head_dim
// bytes per (token, KV head).
#include <algorithm>
#include <cmath>
#include <cstdint>

#include "tq_attn.cuh"
#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

template <typename InT>
__global__ void __launch_bounds__(256) ring_write_kernel(const InT* __restrict__ src_k, const InT* __restrict__ src_v, long n_tokens,
                                                         long src_token0, int row, int window, long slot0, __half* __restrict__ ring_k,
                                                         __half* __restrict__ ring_v) {
    // token t of the source (counted from src_token0) goes to slot (slot0 + t) % window; `row` = heads * dim
    const long total = n_tokens * row;
    for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<long>(gridDim.x) * blockDim.x) {
        const long t = i / row, e = i - t * row;
        const long slot = (slot0 + t) % window;
        const size_t s = static_cast<size_t>(src_token0 + t) * row + e;
        ring_k[slot * row + e] = __float2half_rn(static_cast<float>(src_k[s]));
        ring_v[slot * row + e] = __float2half_rn(static_cast<float>(src_v[s]));
    }
}

__global__ void __launch_bounds__(256) ring_read_kernel(const __half* __restrict__ ring, long n_tokens, int row, int window, long start,
                                                        __half* __restrict__ out) {
    const long total = n_tokens * row;
    for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<long>(gridDim.x) * blockDim.x) {
        const long t = i / row, e = i - t * row;
        out[i] = ring[((start + t) % window) * row + e];
    }
}

constexpr int kDenseG = 8;

template <int E, typename QT>
__global__ void __launch_bounds__(128) dense_attn_partial_kernel(const __half* __restrict__ keys, const __half* __restrict__ values,
                                                                 int n_tokens, int kv_heads, int q_heads, const QT* __restrict__ q,
                                                                 int n_splits, float scale, float* __restrict__ part_acc,
                                                                 float* __restrict__ part_ml) {
    constexpr int D = 32 * E;
    __shared__ float s_q[kDenseG][D];
    __shared__ __align__(16) float s_p[4][32][kDenseG];
    __shared__ float s_m[4][kDenseG], s_l[4][kDenseG];
    __shared__ float s_acc[4][kDenseG][D];

    const int tid = threadIdx.x, lane = tid & 31, wib = tid >> 5;
    const int G = q_heads / kv_heads;
    const int gchunks = (G + kDenseG - 1) / kDenseG;
    const int split = blockIdx.x, kvh = blockIdx.y / gchunks, gchunk = blockIdx.y - kvh * gchunks;
    const int g0 = gchunk * kDenseG;
    const int ng = min(kDenseG, G - g0);
    const int t0 = static_cast<int>(static_cast<long>(n_tokens) * split / n_splits);
    const int t1 = static_cast<int>(static_cast<long>(n_tokens) * (split + 1) / n_splits);

    for (int i = tid; i < kDenseG * D; i += 128) {
        const int g = i / D, d = i - g * D;
        float v = 0.f;
        if (g < ng) v = __half2float(__float2half_rn(static_cast<float>(q[(static_cast<size_t>(kvh) * G + g0 + g) * D + d])));
        s_q[g][d] = v;
    }
    __syncthreads();

    const size_t row = static_cast<size_t>(kv_heads) * D;   // halves per token
    float m[kDenseG], l[kDenseG], acc[kDenseG][E];
#pragma unroll
    for (int g = 0; g < kDenseG; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int j = 0; j < E; ++j) acc[g][j] = 0.f;
    }

    for (int tile = t0 + 32 * wib; tile < t1; tile += 128) {
        const int tok = tile + lane;
        const bool valid = tok < t1;
        // scores of this lane's token
        float s[kDenseG];
#pragma unroll
        for (int g = 0; g < kDenseG; ++g) s[g] = 0.f;
        if (valid) {
            const uint4* kr = reinterpret_cast<const uint4*>(keys + static_cast<size_t>(tok) * row + static_cast<size_t>(kvh) * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                const uint4 raw = __ldg(kr + c);
                const __half2* h = reinterpret_cast<const __half2*>(&raw);
                float kf[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(h[i]);
                    kf[2 * i] = f.x;
                    kf[2 * i + 1] = f.y;
                }
#pragma unroll
                for (int g = 0; g < kDenseG; ++g) {
                    const float4 qa = *reinterpret_cast<const float4*>(&s_q[g][8 * c]);
                    const float4 qb = *reinterpret_cast<const float4*>(&s_q[g][8 * c + 4]);
                    s[g] = fmaf(kf[0], qa.x, s[g]);
                    s[g] = fmaf(kf[1], qa.y, s[g]);
                    s[g] = fmaf(kf[2], qa.z, s[g]);
                    s[g] = fmaf(kf[3], qa.w, s[g]);
                    s[g] = fmaf(kf[4], qb.x, s[g]);
                    s[g] = fmaf(kf[5], qb.y, s[g]);
                    s[g] = fmaf(kf[6], qb.z, s[g]);
                    s[g] = fmaf(kf[7], qb.w, s[g]);
                }
            }
        }
        float corr[kDenseG];
#pragma unroll
        for (int g = 0; g < kDenseG; ++g) {
            const float sv = valid ? s[g] * scale : -INFINITY;
            float mx = sv;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float mn = fmaxf(m[g], mx);   // finite: the tile holds at least one token
            corr[g] = __expf(m[g] - mn);
            const float p = valid ? __expf(sv - mn) : 0.f;
            float ps = p;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
            l[g] = fmaf(l[g], corr[g], ps);
            m[g] = mn;
            s_p[wib][lane][g] = p;
        }
        __syncwarp();
#pragma unroll
        for (int g = 0; g < kDenseG; ++g)
#pragma unroll
            for (int j = 0; j < E; ++j) acc[g][j] *= corr[g];
        const int nt = min(32, t1 - tile);
        for (int t = 0; t < nt; ++t) {
            const __half* vr = values + static_cast<size_t>(tile + t) * row + static_cast<size_t>(kvh) * D + lane * E;
            float vf[E];
            if constexpr (E % 2 == 0) {
#pragma unroll
                for (int j = 0; j < E; j += 2) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(vr + j));
                    vf[j] = f.x;
                    vf[j + 1] = f.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < E; ++j) vf[j] = __half2float(vr[j]);
            }
            const float4 pa = *reinterpret_cast<const float4*>(&s_p[wib][t][0]);
            const float4 pb = *reinterpret_cast<const float4*>(&s_p[wib][t][4]);
            const float pp[kDenseG] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
            for (int g = 0; g < kDenseG; ++g)
#pragma unroll
                for (int j = 0; j < E; ++j) acc[g][j] = fmaf(pp[g], vf[j], acc[g][j]);
        }
        __syncwarp();
    }

    // merge the four warps of this CTA
#pragma unroll
    for (int g = 0; g < kDenseG; ++g) {
        if (lane == 0) {
            s_m[wib][g] = m[g];
            s_l[wib][g] = l[g];
        }
#pragma unroll
        for (int j = 0; j < E; ++j) s_acc[wib][g][lane * E + j] = acc[g][j];
    }
    __syncthreads();
    for (int idx = tid; idx < ng * D; idx += 128) {
        const int g = idx / D, e = idx - g * D;
        const float M = fmaxf(fmaxf(s_m[0][g], s_m[1][g]), fmaxf(s_m[2][g], s_m[3][g]));
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = (s_m[w][g] == -INFINITY) ? 0.f : __expf(s_m[w][g] - M);
            L = fmaf(s_l[w][g], f, L);
            A = fmaf(s_acc[w][g][e], f, A);
        }
        const size_t slot = (static_cast<size_t>(kvh) * G + g0 + g) * n_splits + split;
        part_acc[slot * D + e] = A;
        if (e == 0) {
            part_ml[slot * 2] = M;
            part_ml[slot * 2 + 1] = L;
        }
    }
}

__global__ void __launch_bounds__(128) dense_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                                            int q_heads, int D, int n_splits, __half* __restrict__ out) {
    const int h = blockIdx.x;
    if (h >= q_heads) return;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(static_cast<size_t>(h) * n_splits + s) * 2]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_ml[(static_cast<size_t>(h) * n_splits + s) * 2];
        if (ms != -INFINITY) L = fmaf(part_ml[(static_cast<size_t>(h) * n_splits + s) * 2 + 1], __expf(ms - M), L);
    }
    const float invL = L > 0.f ? 1.f / L : 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[(static_cast<size_t>(h) * n_splits + s) * 2];
            if (ms != -INFINITY) a = fmaf(part_acc[(static_cast<size_t>(h) * n_splits + s) * D + d], __expf(ms - M), a);
        }
        out[static_cast<size_t>(h) * D + d] = __float2half_rn(a * invL);
    }
}

}  // namespace

void launch_ring_write(const void* keys, const void* values, bool is_f16, long n_tokens, long src_token0, int row, int window,
                       long slot0, __half* ring_k, __half* ring_v, cudaStream_t stream) {
    if (n_tokens <= 0) return;
    const long total = n_tokens * row;
    const int blocks = static_cast<int>(std::min<long>((total + 255) / 256, 148L * 8));
    if (is_f16)
        ring_write_kernel<__half><<<blocks, 256, 0, stream>>>(static_cast<const __half*>(keys), static_cast<const __half*>(values), n_tokens,
                                                             src_token0, row, window, slot0, ring_k, ring_v);
    else
        ring_write_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(keys), static_cast<const float*>(values), n_tokens,
                                                            src_token0, row, window, slot0, ring_k, ring_v);
    TQ_CUDA(cudaGetLastError());
}

void launch_ring_read(const __half* ring, long n_tokens, int row, int window, long start, __half* out, cudaStream_t stream) {
    if (n_tokens <= 0) return;
    const long total = n_tokens * row;
    const int blocks = static_cast<int>(std::min<long>((total + 255) / 256, 148L * 8));
    ring_read_kernel<<<blocks, 256, 0, stream>>>(ring, n_tokens, row, window, start, out);
    TQ_CUDA(cudaGetLastError());
}

int dense_attention_splits(int n_tokens, int kv_heads, int q_heads, int sm_count) {
    const int G = q_heads / kv_heads;
    const int ctas_per_split = kv_heads * ((G + kDenseG - 1) / kDenseG);
    int n = (sm_count * 4 + ctas_per_split - 1) / ctas_per_split;
    n = std::min(n, std::max(1, n_tokens / 128));
    return std::max(1, std::min(n, 256));
}

size_t dense_attention_scratch_bytes(int q_heads, int head_dim, int n_splits) {
    return static_cast<size_t>(q_heads) * n_splits * (head_dim + 2) * sizeof(float);
}

void launch_dense_attention(const __half* keys, const __half* values, int n_tokens, int kv_heads, int head_dim, const void* q,
                            bool q_is_f16, int q_heads, int n_splits, void* scratch, __half* out, cudaStream_t stream) {
    TQ_REQUIRE(q_heads % kv_heads == 0, "window attention: query heads must be a multiple of KV heads");
    TQ_REQUIRE(n_tokens > 0 && n_splits >= 1, "window attention: empty range");
    const int G = q_heads / kv_heads;
    const dim3 grid(n_splits, kv_heads * ((G + kDenseG - 1) / kDenseG));
    const float scale = 1.0f / std::sqrt(static_cast<float>(head_dim));   // src/attention_dispatch.cpp:35
    float* part_acc = static_cast<float*>(scratch);
    float* part_ml = part_acc + static_cast<size_t>(q_heads) * n_splits * head_dim;
#define TQ_DENSE(EV)                                                                                                              \
    if (q_is_f16)                                                                                                                 \
        dense_attn_partial_kernel<EV, __half><<<grid, 128, 0, stream>>>(keys, values, n_tokens, kv_heads, q_heads,                  \
                                                                        static_cast<const __half*>(q), n_splits, scale, part_acc, \
                                                                        part_ml);                                                 \
    else                                                                                                                          \
        dense_attn_partial_kernel<EV, float><<<grid, 128, 0, stream>>>(keys, values, n_tokens, kv_heads, q_heads,                   \
                                                                       static_cast<const float*>(q), n_splits, scale, part_acc,   \
                                                                       part_ml);
    switch (head_dim) {
        case 32: TQ_DENSE(1) break;
        case 64: TQ_DENSE(2) break;
        case 128: TQ_DENSE(4) break;
        case 256: TQ_DENSE(8) break;
        default: throw Error("window attention: head_dim must be 32, 64, 128 or 256");
    }
#undef TQ_DENSE
    dense_combine_kernel<<<q_heads, 128, 0, stream>>>(part_acc, part_ml, q_heads, head_dim, n_splits, out);
    TQ_CUDA(cudaGetLastError());
}

}  // namespace tq
