// Compressed KV cache kernels: online encoder, range decoder, decode attention.
//
// Storage layout (device, per layer) is the reference's (include/turboquant/kv_cache.h:25-36,
// src/kv_cache.cpp:119-128): token-major records [token][head][...],
//   codes  : ceil(d/10) uint32 per vector, ten 3-bit codes per word, code j at bits 3*(j%10)
//   norms  : fp32 per vector
//   QJL    : ceil(d/32) uint32 sign words + fp32 residual norm per key vector
// so a snapshot in the reference's wire format is a plain copy.
#include <cmath>

#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

// 3-bit N(0,1) Lloyd-Max centroids and their midpoints (src/codebook.cpp:24-27, 49-57).
__constant__ float kC3[8] = {-2.152176f, -1.344318f, -0.756130f, -0.245379f, 0.245379f, 0.756130f, 1.344318f, 2.152176f};

__device__ __forceinline__ float load_as_f32(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float load_as_f32(const __half* p, size_t i) { return __half2float(p[i]); }

// ---- encoder (src/kv_cache.cpp:63-258) -----------------------------------------------------
// One warp per (token, head) vector of d = 32*E values.  Bit-exact: the two sums of
// squares are accumulated left to right by one lane, everything else is element-wise
// or the shared butterfly.
template <int E, typename InT>
__global__ void __launch_bounds__(128) kv_encode_kernel(const InT* __restrict__ x, long n_vec, uint32_t wht_seed,
                                                        uint32_t qjl_seed, int with_qjl, float scale, float inv_sqrt,
                                                        uint32_t* __restrict__ words, float* __restrict__ norms,
                                                        uint32_t* __restrict__ qjl_words, float* __restrict__ qjl_norms) {
    constexpr int D = 32 * E;
    constexpr int WPH = (D + 9) / 10;
    constexpr int QPH = D / 32;
    __shared__ float s_val[4][D];
    __shared__ uint8_t s_code[4][D];
    __shared__ uint32_t s_bits[4][QPH];
    __shared__ float s_bounds[7];
    __shared__ float s_cent[8];
    if (threadIdx.x < 8) s_cent[threadIdx.x] = kC3[threadIdx.x];
    if (threadIdx.x < 7) s_bounds[threadIdx.x] = __fmul_rn(__fadd_rn(kC3[threadIdx.x], kC3[threadIdx.x + 1]), 0.5f);
    __syncthreads();

    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const long warp0 = static_cast<long>(blockIdx.x) * 4 + wib;
    const long n_warps = static_cast<long>(gridDim.x) * 4;
    float sgn[E];
#pragma unroll
    for (int j = 0; j < E; ++j) sgn[j] = sign_value(wht_seed, static_cast<uint32_t>(lane * E + j));

    for (long vec = warp0; vec < n_vec; vec += n_warps) {
        float v[E];
#pragma unroll
        for (int j = 0; j < E; ++j) {
            v[j] = load_as_f32(x, static_cast<size_t>(vec) * D + lane * E + j);
            s_val[wib][lane * E + j] = v[j];
        }
        __syncwarp();
        float norm = 0.0f;
        if (lane == 0) {
            float acc = 0.0f;
            for (int j = 0; j < D; ++j) {
                const float t = s_val[wib][j];
                acc = __fadd_rn(acc, __fmul_rn(t, t));
            }
            norm = __fsqrt_rn(acc);
            norms[vec] = norm;
        }
        norm = __shfl_sync(0xffffffffu, norm, 0);
        const float inv_norm = (norm > 1e-10f) ? __fdiv_rn(1.0f, norm) : 0.0f;
#pragma unroll
        for (int j = 0; j < E; ++j) v[j] = __fmul_rn(__fmul_rn(v[j], inv_norm), sgn[j]);
        warp_fwht<E>(v, lane);
        __syncwarp();
        if (lane < QPH) s_bits[wib][lane] = 0u;
        __syncwarp();
        uint32_t my_bits = 0u;
#pragma unroll
        for (int j = 0; j < E; ++j) {
            v[j] = __fmul_rn(__fmul_rn(v[j], inv_sqrt), scale);
            int idx = 0;
#pragma unroll
            for (int b = 0; b < 7; ++b) idx += (s_bounds[b] < v[j]) ? 1 : 0;
            s_code[wib][lane * E + j] = static_cast<uint8_t>(idx);
            if (with_qjl) {
                const float r = __fsub_rn(v[j], s_cent[idx]);
                s_val[wib][lane * E + j] = r;
                const float s = qjl_sign_is_positive(qjl_seed, static_cast<uint32_t>(lane * E + j)) ? 1.0f : -1.0f;
                if (__fmul_rn(r, s) > 0.0f) my_bits |= 1u << j;
            }
        }
        if (with_qjl && my_bits) atomicOr(&s_bits[wib][(lane * E) >> 5], my_bits << ((lane * E) & 31));
        __syncwarp();
        if (with_qjl) {
            if (lane == 0) {
                float acc = 0.0f;
                for (int j = 0; j < D; ++j) {
                    const float t = s_val[wib][j];
                    acc = __fadd_rn(acc, __fmul_rn(t, t));
                }
                qjl_norms[vec] = __fsqrt_rn(acc);
            }
            if (lane < QPH) qjl_words[vec * QPH + lane] = s_bits[wib][lane];
        }
        for (int w = lane; w < WPH; w += 32) {
            uint32_t word = 0;
#pragma unroll
            for (int k = 0; k < 10; ++k) {
                const int e = w * 10 + k;
                if (e < D) word |= (static_cast<uint32_t>(s_code[wib][e]) & 7u) << (3 * k);
            }
            words[vec * WPH + w] = word;
        }
        __syncwarp();
    }
}

// ---- range decoder (src/kv_cache.cpp:292-365) -------------------------------------------------
template <int E>
__global__ void __launch_bounds__(128) kv_decode_kernel(const uint32_t* __restrict__ words, const float* __restrict__ norms,
                                                        long n_vec, uint32_t wht_seed, float inv_scale, float inv_sqrt,
                                                        __half* __restrict__ out) {
    constexpr int D = 32 * E;
    constexpr int WPH = (D + 9) / 10;
    const int lane = threadIdx.x & 31;
    const long warp0 = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
    float sg[E];
#pragma unroll
    for (int j = 0; j < E; ++j) sg[j] = __fmul_rn(inv_sqrt, sign_value(wht_seed, static_cast<uint32_t>(lane * E + j)));
    for (long vec = warp0; vec < n_vec; vec += n_warps) {
        const uint32_t* w = words + vec * WPH;
        float v[E];
#pragma unroll
        for (int j = 0; j < E; ++j) {
            const int e = lane * E + j;
            v[j] = __fmul_rn(kC3[(w[e / 10] >> ((e % 10) * 3)) & 7u], inv_scale);
        }
        warp_fwht<E>(v, lane);
        const float norm = norms[vec];
#pragma unroll
        for (int j = 0; j < E; ++j)
            out[static_cast<size_t>(vec) * D + lane * E + j] = __float2half_rn(__fmul_rn(__fmul_rn(v[j], sg[j]), norm));
    }
}

// ---- decode attention, first version -----------------------------------------------------------
// One query position per sequence; all G query heads of a KV head share one pass over
// that head's codes.  Scores are taken in the rotated domain (the query is rotated once,
// keys are never un-rotated), values are accumulated in the rotated domain and
// un-rotated once at the end.  Context is split across CTAs (and warps); partial
// (max, sum, accumulator) triples are merged by attn_combine_kernel.
constexpr int kAttnGMax = 8;

struct AttnSeq {
    const uint32_t* k_words;
    const uint32_t* v_words;
    const float* k_norms;
    const float* v_norms;
    const uint32_t* qjl_words;
    const float* qjl_norms;
    int start, end;
};

template <int E, typename QT>
__global__ void __launch_bounds__(128) attn_partial_kernel(const AttnSeq* __restrict__ seqs, const QT* __restrict__ q,
                                                           int q_heads, int kv_heads, int n_splits, uint32_t k_seed,
                                                           uint32_t qjl_seed, int use_qjl, float inv_sqrt,
                                                           float inv_scale_d, float attn_scale, float gamma,
                                                           float* __restrict__ part_acc, float* __restrict__ part_ml) {
    constexpr int D = 32 * E;
    constexpr int WPH = (D + 9) / 10;
    constexpr int QPH = D / 32;
    __shared__ float s_c[8];
    __shared__ float s_m[4][kAttnGMax], s_l[4][kAttnGMax];
    __shared__ float s_acc[4][kAttnGMax][D];
    if (threadIdx.x < 8) s_c[threadIdx.x] = kC3[threadIdx.x];
    __syncthreads();

    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int split = blockIdx.x, kvh = blockIdx.y % kv_heads, gchunk = blockIdx.y / kv_heads, seq = blockIdx.z;
    const int G = q_heads / kv_heads;
    const int g0 = gchunk * kAttnGMax;
    const int ng = min(kAttnGMax, G - g0);
    const AttnSeq S = seqs[seq];
    const int n_tok = S.end - S.start;
    const int t0 = S.start + static_cast<int>(static_cast<long>(n_tok) * split / n_splits);
    const int t1 = S.start + static_cast<int>(static_cast<long>(n_tok) * (split + 1) / n_splits);

    // rotated query: fp16-round, sign, butterfly, 1/sqrt(d)
    float qr[kAttnGMax][E], qs[kAttnGMax][E];
#pragma unroll
    for (int g = 0; g < kAttnGMax; ++g) {
        float v[E];
#pragma unroll
        for (int j = 0; j < E; ++j) {
            float t = 0.0f;
            if (g < ng) {
                const size_t qi = (static_cast<size_t>(seq) * q_heads + kvh * G + g0 + g) * D + lane * E + j;
                t = __half2float(__float2half_rn(static_cast<float>(q[qi])));
            }
            v[j] = t * sign_value(k_seed, static_cast<uint32_t>(lane * E + j));
        }
        warp_fwht<E>(v, lane);
#pragma unroll
        for (int j = 0; j < E; ++j) {
            qr[g][j] = v[j] * inv_sqrt;
            qs[g][j] = qjl_sign_is_positive(qjl_seed, static_cast<uint32_t>(lane * E + j)) ? qr[g][j] : -qr[g][j];
        }
    }

    float m[kAttnGMax], l[kAttnGMax], acc[kAttnGMax][E];
#pragma unroll
    for (int g = 0; g < kAttnGMax; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < E; ++j) acc[g][j] = 0.0f;
    }

    for (int t = t0 + wib; t < t1; t += 4) {
        const size_t rec = static_cast<size_t>(t) * kv_heads + kvh;
        const uint32_t* kw = S.k_words + rec * WPH;
        const uint32_t* vw = S.v_words + rec * WPH;
        float kc[E], vc[E], sgnbit[E];
        const uint32_t qword = use_qjl ? S.qjl_words[rec * QPH + ((lane * E) >> 5)] : 0u;
#pragma unroll
        for (int j = 0; j < E; ++j) {
            const int e = lane * E + j;
            kc[j] = s_c[(kw[e / 10] >> ((e % 10) * 3)) & 7u];
            vc[j] = s_c[(vw[e / 10] >> ((e % 10) * 3)) & 7u];
            sgnbit[j] = ((qword >> (e & 31)) & 1u) ? 1.0f : -1.0f;
        }
        const float kn = S.k_norms[rec] * inv_scale_d * attn_scale;
        const float vn = S.v_norms[rec];
        const float qn = use_qjl ? S.qjl_norms[rec] * gamma : 0.0f;
#pragma unroll
        for (int g = 0; g < kAttnGMax; ++g) {
            if (g < ng) {
                float d0 = 0.0f, d1 = 0.0f;
#pragma unroll
                for (int j = 0; j < E; ++j) {
                    d0 = fmaf(qr[g][j], kc[j], d0);
                    d1 = fmaf(qs[g][j], sgnbit[j], d1);
                }
                float dot = fmaf(qn, d1, d0);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                const float s = dot * kn;
                const float mn = fmaxf(m[g], s);
                const float corr = __expf(m[g] - mn);
                const float p = __expf(s - mn);
                l[g] = fmaf(l[g], corr, p);
                const float pv = p * vn;
#pragma unroll
                for (int j = 0; j < E; ++j) acc[g][j] = fmaf(acc[g][j], corr, pv * vc[j]);
                m[g] = mn;
            }
        }
    }

    // merge the 4 warps of this CTA
#pragma unroll
    for (int g = 0; g < kAttnGMax; ++g) {
        if (lane == 0) {
            s_m[wib][g] = m[g];
            s_l[wib][g] = l[g];
        }
#pragma unroll
        for (int j = 0; j < E; ++j) s_acc[wib][g][lane * E + j] = acc[g][j];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < ng * D; idx += blockDim.x) {
        const int g = idx / D, e = idx - g * D;
        float M = fmaxf(fmaxf(s_m[0][g], s_m[1][g]), fmaxf(s_m[2][g], s_m[3][g]));
        float L = 0.0f, A = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = (s_m[w][g] == -INFINITY) ? 0.0f : __expf(s_m[w][g] - M);
            L = fmaf(s_l[w][g], f, L);
            A = fmaf(s_acc[w][g][e], f, A);
        }
        const size_t slot = (static_cast<size_t>(seq) * q_heads + kvh * G + g0 + g) * n_splits + split;
        part_acc[slot * D + e] = A;
        if (e == 0) {
            part_ml[slot * 2] = M;
            part_ml[slot * 2 + 1] = L;
        }
    }
}

// Merge the context splits of one (sequence, query head) and un-rotate the value sum:
// out = (inv_sqrt*sign_v) o H(inv_scale_d * acc) / L.
template <int E>
__global__ void __launch_bounds__(128) attn_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                                           long n_rows, int n_splits, uint32_t v_seed, float inv_sqrt,
                                                           float inv_scale_d, __half* __restrict__ out) {
    constexpr int D = 32 * E;
    const int lane = threadIdx.x & 31;
    const long row = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (row >= n_rows) return;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(row * n_splits + s) * 2]);
    float L = 0.0f, v[E];
#pragma unroll
    for (int j = 0; j < E; ++j) v[j] = 0.0f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_ml[(row * n_splits + s) * 2];
        const float f = (ms == -INFINITY) ? 0.0f : __expf(ms - M);
        L = fmaf(part_ml[(row * n_splits + s) * 2 + 1], f, L);
#pragma unroll
        for (int j = 0; j < E; ++j) v[j] = fmaf(part_acc[(row * n_splits + s) * D + lane * E + j], f, v[j]);
    }
#pragma unroll
    for (int j = 0; j < E; ++j) v[j] *= inv_scale_d;
    warp_fwht<E>(v, lane);
    const float invL = (L > 0.0f) ? 1.0f / L : 0.0f;
#pragma unroll
    for (int j = 0; j < E; ++j)
        out[row * D + lane * E + j] =
            __float2half_rn(v[j] * inv_sqrt * sign_value(v_seed, static_cast<uint32_t>(lane * E + j)) * invL);
}

int grid_for_warps(long n_warp_items, int warps_per_block, int cap) {
    long want = (n_warp_items + warps_per_block - 1) / warps_per_block;
    if (want < 1) want = 1;
    return static_cast<int>(want < cap ? want : cap);
}

}  // namespace

#define TQ_D_SWITCH(D, MACRO)                                                      \
    switch (D) {                                                                   \
        case 32: MACRO(1) break;                                                   \
        case 64: MACRO(2) break;                                                   \
        case 128: MACRO(4) break;                                                  \
        case 256: MACRO(8) break;                                                  \
        case 512: MACRO(16) break;                                                 \
        default: throw Error("head_dim must be a power of two in [32, 512]");      \
    }

void launch_kv_encode(const void* x, bool x_is_f16, long n_vec, int head_dim, uint32_t wht_seed, uint32_t qjl_seed,
                      bool with_qjl, uint32_t* words, float* norms, uint32_t* qjl_words, float* qjl_norms,
                      cudaStream_t stream) {
    if (n_vec == 0) return;
    const float scale = std::sqrt(static_cast<float>(head_dim));             // src/kv_cache.cpp:72
    const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(head_dim));   // src/rotation.cpp:301
    const int grid = grid_for_warps(n_vec, 4, 148 * 16);
#define TQ_ENC(EV)                                                                                                      \
    if (x_is_f16)                                                                                                       \
        kv_encode_kernel<EV, __half><<<grid, 128, 0, stream>>>(static_cast<const __half*>(x), n_vec, wht_seed, qjl_seed, \
                                                               with_qjl ? 1 : 0, scale, inv_sqrt, words, norms,          \
                                                               qjl_words, qjl_norms);                                    \
    else                                                                                                                \
        kv_encode_kernel<EV, float><<<grid, 128, 0, stream>>>(static_cast<const float*>(x), n_vec, wht_seed, qjl_seed,   \
                                                              with_qjl ? 1 : 0, scale, inv_sqrt, words, norms,           \
                                                              qjl_words, qjl_norms);
    TQ_D_SWITCH(head_dim, TQ_ENC)
#undef TQ_ENC
    TQ_CUDA(cudaGetLastError());
}

void launch_kv_decode_f16(const uint32_t* words, const float* norms, long n_vec, int head_dim, uint32_t wht_seed,
                          __half* out, cudaStream_t stream) {
    if (n_vec == 0) return;
    const float inv_scale = 1.0f / std::sqrt(static_cast<float>(head_dim));  // src/kv_cache.cpp:302
    const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(head_dim));
    const int grid = grid_for_warps(n_vec, 4, 148 * 16);
#define TQ_DEC(EV) kv_decode_kernel<EV><<<grid, 128, 0, stream>>>(words, norms, n_vec, wht_seed, inv_scale, inv_sqrt, out);
    TQ_D_SWITCH(head_dim, TQ_DEC)
#undef TQ_DEC
    TQ_CUDA(cudaGetLastError());
}

size_t attn_scratch_bytes(int n_seqs, int q_heads, int head_dim, int n_splits) {
    return static_cast<size_t>(n_seqs) * q_heads * n_splits * (head_dim + 2) * sizeof(float);
}

void launch_kv_attention(const void* d_seqs, int n_seqs, const void* q, bool q_is_f16, int q_heads, int kv_heads,
                         int head_dim, int n_splits, uint32_t k_seed, uint32_t v_seed, uint32_t qjl_seed, bool use_qjl,
                         void* scratch, __half* out, cudaStream_t stream) {
    if (n_seqs == 0) return;
    TQ_REQUIRE(q_heads % kv_heads == 0, "query heads must be a multiple of KV heads");
    const int G = q_heads / kv_heads;
    const int gchunks = (G + kAttnGMax - 1) / kAttnGMax;
    const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(head_dim));
    const float inv_scale_d = 1.0f / std::sqrt(static_cast<float>(head_dim));
    const float attn_scale = 1.0f / std::sqrt(static_cast<float>(head_dim));  // src/attention_dispatch.cpp:35
    const float gamma = static_cast<float>(std::sqrt(2.0 / (3.14159265358979323846 * head_dim)));
    float* part_acc = static_cast<float*>(scratch);
    float* part_ml = part_acc + static_cast<size_t>(n_seqs) * q_heads * n_splits * head_dim;
    const dim3 grid(n_splits, kv_heads * gchunks, n_seqs);
    const long n_rows = static_cast<long>(n_seqs) * q_heads;
#define TQ_ATT(EV)                                                                                                       \
    if (q_is_f16)                                                                                                        \
        attn_partial_kernel<EV, __half><<<grid, 128, 0, stream>>>(static_cast<const AttnSeq*>(d_seqs),                    \
                                                                  static_cast<const __half*>(q), q_heads, kv_heads,      \
                                                                  n_splits, k_seed, qjl_seed, use_qjl ? 1 : 0, inv_sqrt,  \
                                                                  inv_scale_d, attn_scale, gamma, part_acc, part_ml);    \
    else                                                                                                                 \
        attn_partial_kernel<EV, float><<<grid, 128, 0, stream>>>(static_cast<const AttnSeq*>(d_seqs),                     \
                                                                 static_cast<const float*>(q), q_heads, kv_heads,        \
                                                                 n_splits, k_seed, qjl_seed, use_qjl ? 1 : 0, inv_sqrt,   \
                                                                 inv_scale_d, attn_scale, gamma, part_acc, part_ml);     \
    attn_combine_kernel<EV><<<static_cast<int>((n_rows + 3) / 4), 128, 0, stream>>>(part_acc, part_ml, n_rows, n_splits, \
                                                                                   v_seed, inv_sqrt, inv_scale_d, out);
    switch (head_dim) {
        case 32: TQ_ATT(1) break;
        case 64: TQ_ATT(2) break;
        case 128: TQ_ATT(4) break;
        case 256: TQ_ATT(8) break;
        default: throw Error("attention: head_dim must be 32, 64, 128 or 256");
    }
#undef TQ_ATT
    TQ_CUDA(cudaGetLastError());
}

}  // namespace tq
