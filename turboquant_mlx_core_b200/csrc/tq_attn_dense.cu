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
#include <cstdlib>

#include "tq_attn.cuh"
#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

template <typename InT>
__global__ void __launch_bounds__(256) ring_write_kernel(const InT* __restrict__ src_k, const InT* __restrict__ src_v, long n_tokens,
                                                         long src_token0, int row, int window, long slot0, __half* __restrict__ ring_k,
                                                         __half* __restrict__ ring_v) {
    pdl_wait_release();
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
        // value rows eight at a time: the eight loads are in flight together
        for (int tb = 0; tb < nt; tb += 8) {
            float vf[8][E];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int t = min(tb + u, nt - 1);   // rows past the end repeat the last one; their probabilities are zeroed below
                const __half* vr = values + static_cast<size_t>(tile + t) * row + static_cast<size_t>(kvh) * D + lane * E;
                if constexpr (E == 4) {
                    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(vr));
                    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    vf[u][0] = f0.x; vf[u][1] = f0.y; vf[u][2] = f1.x; vf[u][3] = f1.y;
                } else if constexpr (E == 8) {
                    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(vr));
                    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(h[j]);
                        vf[u][2 * j] = f.x;
                        vf[u][2 * j + 1] = f.y;
                    }
                } else if constexpr (E == 2) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(vr));
                    vf[u][0] = f.x; vf[u][1] = f.y;
                } else {
#pragma unroll
                    for (int j = 0; j < E; ++j) vf[u][j] = __half2float(vr[j]);
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int t = tb + u;
                const bool live = t < nt;
                const int ts = live ? t : nt - 1;
                const float4 pa = *reinterpret_cast<const float4*>(&s_p[wib][ts][0]);
                const float4 pb = *reinterpret_cast<const float4*>(&s_p[wib][ts][4]);
                const float pp[kDenseG] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
                for (int g = 0; g < kDenseG; ++g) {
                    const float pg = live ? pp[g] : 0.f;
#pragma unroll
                    for (int j = 0; j < E; ++j) acc[g][j] = fmaf(pg, vf[u][j], acc[g][j]);
                }
            }
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

// ---- head_dim 128 on the tensor cores ---------------------------------------------------------------
// One warp owns 16-token tiles; products are mma.sync.m16n8k16 (fp16 in, fp32 accumulate):
//   S^T[16 tokens x 8 heads]  = K[16 x 128] . Q^T[128 x 8]
//   O^T[128 dims x 8 heads]  += V^T[128 x 16] . P^T[16 x 8]
// Fragments come straight from global memory: thread (g, q) of a warp loads, for its two token rows g and
// g + 8, the 16 bytes at dims [32 j + 8 q, + 8) for j = 0..3 (eight rows x 64 contiguous bytes per load
// instruction) and uses the four fp16 pairs as the a0 / a2 registers of k-steps 2j and 2j + 1.  That is a
// permutation of the 128 dims inside each k-step (fragment column 2 q' + e of k-step 2 j + u holds dim
// 32 j + 8 q' + 4 u + e, column 8 + 2 q' + e the dim two further on); the query fragments use the same
// permutation, and the accumulator rows are mapped back when the partial result is written.
// V tiles are transposed in registers (movmatrix).  Softmax as in the compressed-cache kernels: a lazy
// reference maximum per head that moves only when a score exceeds it by more than kAttnSoftmaxSlack.
__device__ __forceinline__ void dense_mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t dense_movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t dense_pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// dim held by fragment column c (0..15) of k-step ks (0..7)
__host__ __device__ __forceinline__ int dense_frag_dim(int ks, int c) {
    return 32 * (ks >> 1) + 8 * ((c & 7) >> 1) + 4 * (ks & 1) + 2 * (c >> 3) + (c & 1);
}

template <typename QT>
__global__ void __launch_bounds__(128, 3) dense_attn_mma_kernel(const __half* __restrict__ keys, const __half* __restrict__ values,
                                                                int n_tokens, int kv_heads, int q_heads, const QT* __restrict__ q,
                                                                int n_splits, float scale, float* __restrict__ part_acc,
                                                                float* __restrict__ part_ml) {
    pdl_wait_release();
    constexpr int D = 128;
    __shared__ __half s_q[8][D + 8];
    __shared__ float s_m[4][8], s_l[4][8];
    __shared__ float s_acc[4][8][D + 4];

    const int tid = threadIdx.x, lane = tid & 31, wib = tid >> 5;
    const int g = lane >> 2, qd = lane & 3;
    const int G = q_heads / kv_heads;
    const int gchunks = (G + 7) / 8;
    const int split = blockIdx.x, kvh = blockIdx.y / gchunks, gchunk = blockIdx.y - kvh * gchunks;
    const int g0 = gchunk * 8;
    const int ng = min(8, G - g0);
    // splits in whole 16-token tiles
    const int all_tiles = (n_tokens + 15) >> 4;
    const int tile0 = static_cast<int>(static_cast<long>(all_tiles) * split / n_splits);
    const int tile1 = static_cast<int>(static_cast<long>(all_tiles) * (split + 1) / n_splits);

    for (int i = tid; i < 8 * D; i += 128) {
        const int h = i >> 7, d = i & (D - 1);
        float v = 0.f;
        if (h < ng) v = static_cast<float>(q[(static_cast<size_t>(kvh) * G + g0 + h) * D + d]);
        s_q[h][d] = __float2half_rn(v);
    }
    __syncthreads();
    uint32_t bq[16];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const int d0 = dense_frag_dim(ks, 2 * qd), d1 = dense_frag_dim(ks, 8 + 2 * qd);
        bq[2 * ks] = *reinterpret_cast<const uint32_t*>(&s_q[g][d0]);
        bq[2 * ks + 1] = *reinterpret_cast<const uint32_t*>(&s_q[g][d1]);
    }

    const size_t row = static_cast<size_t>(kv_heads) * D;   // halves per token
    const float sl2 = scale * 1.4426950408889634f;           // scores in the log2 domain
    const float slack = kAttnSoftmaxSlack * 1.4426950408889634f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // heads 2 qd, 2 qd + 1
    float acc[8][4];
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[mt][k] = 0.f;

    for (int tile = tile0 + wib; tile < tile1; tile += 4) {
        const int ta = tile * 16 + g, tb = ta + 8;
        const bool va = ta < n_tokens, vb = tb < n_tokens;
        const int ra = va ? ta : n_tokens - 1, rb = vb ? tb : n_tokens - 1;   // clamped: masked below
        const uint4* ka = reinterpret_cast<const uint4*>(keys + static_cast<size_t>(ra) * row + static_cast<size_t>(kvh) * D) + qd;
        const uint4* kb = reinterpret_cast<const uint4*>(keys + static_cast<size_t>(rb) * row + static_cast<size_t>(kvh) * D) + qd;
        const uint4* xa = reinterpret_cast<const uint4*>(values + static_cast<size_t>(ra) * row + static_cast<size_t>(kvh) * D) + qd;
        const uint4* xb = reinterpret_cast<const uint4*>(values + static_cast<size_t>(rb) * row + static_cast<size_t>(kvh) * D) + qd;
        uint4 fka[4], fkb[4], fva[4], fvb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            fka[j] = __ldg(ka + 4 * j);
            fkb[j] = __ldg(kb + 4 * j);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            fva[j] = __ldg(xa + 4 * j);
            fvb[j] = __ldg(xb + 4 * j);
        }
        float c1[4] = {0.f, 0.f, 0.f, 0.f}, c1b[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            dense_mma_f16(c1, fka[j].x, fkb[j].x, fka[j].y, fkb[j].y, bq[4 * j], bq[4 * j + 1]);
            dense_mma_f16(c1b, fka[j].z, fkb[j].z, fka[j].w, fkb[j].w, bq[4 * j + 2], bq[4 * j + 3]);
        }
        const float s00 = va ? (c1[0] + c1b[0]) * sl2 : -INFINITY, s01 = va ? (c1[1] + c1b[1]) * sl2 : -INFINITY;
        const float s10 = vb ? (c1[2] + c1b[2]) * sl2 : -INFINITY, s11 = vb ? (c1[3] + c1b[3]) * sl2 : -INFINITY;
        const float tm0 = fmaxf(s00, s10), tm1 = fmaxf(s01, s11);
        if (__any_sync(0xffffffffu, tm0 > m_run[0] + slack || tm1 > m_run[1] + slack)) {
            float mx0 = tm0, mx1 = tm1;
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
            }
            const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
            const float cr0 = mn0 == -INFINITY ? 1.f : exp2f(m_run[0] - mn0), cr1 = mn1 == -INFINITY ? 1.f : exp2f(m_run[1] - mn1);
            l_run[0] *= cr0;
            l_run[1] *= cr1;
            m_run[0] = mn0;
            m_run[1] = mn1;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                acc[mt][0] *= cr0;
                acc[mt][1] *= cr1;
                acc[mt][2] *= cr0;
                acc[mt][3] *= cr1;
            }
        }
        const float p00 = va ? exp2f(s00 - m_run[0]) : 0.f, p01 = va ? exp2f(s01 - m_run[1]) : 0.f;
        const float p10 = vb ? exp2f(s10 - m_run[0]) : 0.f, p11 = vb ? exp2f(s11 - m_run[1]) : 0.f;
        l_run[0] += p00 + p10;
        l_run[1] += p01 + p11;
        const uint32_t pb0 = dense_movmatrix_trans(dense_pack_half2(p00, p01));
        const uint32_t pb1 = dense_movmatrix_trans(dense_pack_half2(p10, p11));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            dense_mma_f16(acc[2 * j], dense_movmatrix_trans(fva[j].x), dense_movmatrix_trans(fva[j].y), dense_movmatrix_trans(fvb[j].x),
                          dense_movmatrix_trans(fvb[j].y), pb0, pb1);
            dense_mma_f16(acc[2 * j + 1], dense_movmatrix_trans(fva[j].z), dense_movmatrix_trans(fva[j].w), dense_movmatrix_trans(fvb[j].z),
                          dense_movmatrix_trans(fvb[j].w), pb0, pb1);
        }
    }

    // ---- merge the four warps, natural dim order ----
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], o);
        l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], o);
    }
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const int da = dense_frag_dim(ks, g), db = dense_frag_dim(ks, 8 + g);
        s_acc[wib][2 * qd][da] = acc[ks][0];
        s_acc[wib][2 * qd + 1][da] = acc[ks][1];
        s_acc[wib][2 * qd][db] = acc[ks][2];
        s_acc[wib][2 * qd + 1][db] = acc[ks][3];
    }
    if (g == 0) {
        s_m[wib][2 * qd] = m_run[0];
        s_m[wib][2 * qd + 1] = m_run[1];
        s_l[wib][2 * qd] = l_run[0];
        s_l[wib][2 * qd + 1] = l_run[1];
    }
    __syncthreads();
    for (int idx = tid; idx < ng * D; idx += 128) {
        const int h = idx >> 7, e = idx & (D - 1);
        const float M = fmaxf(fmaxf(s_m[0][h], s_m[1][h]), fmaxf(s_m[2][h], s_m[3][h]));
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = (s_m[w][h] == -INFINITY) ? 0.f : exp2f(s_m[w][h] - M);
            L = fmaf(s_l[w][h], f, L);
            A = fmaf(s_acc[w][h][e], f, A);
        }
        const size_t slot = (static_cast<size_t>(kvh) * G + g0 + h) * n_splits + split;
        part_acc[slot * D + e] = A;
        if (e == 0) {
            part_ml[slot * 2] = M * 0.6931471805599453f;   // natural-log domain, as dense_combine_kernel expects
            part_ml[slot * 2 + 1] = L;
        }
    }
}

__global__ void __launch_bounds__(128) dense_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                                            int q_heads, int D, int n_splits, __half* __restrict__ out) {
    pdl_wait_release();
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
        launch_pdl(ring_write_kernel<__half>, dim3(blocks), dim3(256), 0, stream, static_cast<const __half*>(keys),
                   static_cast<const __half*>(values), n_tokens, src_token0, row, window, slot0, ring_k, ring_v);
    else
        launch_pdl(ring_write_kernel<float>, dim3(blocks), dim3(256), 0, stream, static_cast<const float*>(keys),
                   static_cast<const float*>(values), n_tokens, src_token0, row, window, slot0, ring_k, ring_v);
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
    // one wave of resident CTAs (three per SM: the tensor-core kernel's register count allows no more)
    int n = (sm_count * 3) / ctas_per_split;
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
    static const bool cuda_core_only = std::getenv("TQ_WINDOW_ATTENTION_FMA") != nullptr;   // measurement switch: the fp32-FMA kernel at head_dim 128
    if (head_dim == 128 && !cuda_core_only) {
        if (q_is_f16)
            launch_pdl(dense_attn_mma_kernel<__half>, grid, dim3(128), 0, stream, keys, values, n_tokens, kv_heads, q_heads,
                       static_cast<const __half*>(q), n_splits, scale, part_acc, part_ml);
        else
            launch_pdl(dense_attn_mma_kernel<float>, grid, dim3(128), 0, stream, keys, values, n_tokens, kv_heads, q_heads,
                       static_cast<const float*>(q), n_splits, scale, part_acc, part_ml);
        launch_pdl(dense_combine_kernel, dim3(q_heads), dim3(128), 0, stream, part_acc, part_ml, q_heads, head_dim, n_splits, out);
        TQ_CUDA(cudaGetLastError());
        return;
    }
    switch (head_dim) {
        case 32: TQ_DENSE(1) break;
        case 64: TQ_DENSE(2) break;
        case 128: TQ_DENSE(4) break;
        case 256: TQ_DENSE(8) break;
        default: throw Error("window attention: head_dim must be 32, 64, 128 or 256");
    }
#undef TQ_DENSE
    launch_pdl(dense_combine_kernel, dim3(q_heads), dim3(128), 0, stream, part_acc, part_ml, q_heads, head_dim, n_splits, out);
    TQ_CUDA(cudaGetLastError());
}

}  // namespace tq
