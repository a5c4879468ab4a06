// Compressed KV cache kernels: online encoder, range decoder, decode attention.
//
// Storage layout (device, per layer) is the reference's (include/turboquant/kv_cache.h:25-36,
// src/kv_cache.cpp:119-128): token-major records [token][head][...],
//   codes  : ceil(d/10) uint32 per vector, ten 3-bit codes per word, code j at bits 3*(j%10)
//   norms  : fp32 per vector
//   QJL    : ceil(d/32) uint32 sign words + fp32 residual norm per key vector
// so a snapshot in the reference's wire format is a plain copy.
#include <cmath>
#include <cstdlib>

#include "tq_attn.cuh"
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
// Where the encoder writes: the input vectors are cut into segments of vec_per_seg consecutive
// vectors and segment s goes to seg[s] (one segment for an ordinary append; one per sequence when
// a decode step appends a token to many caches at once).
struct KvEncodeDst {
    uint32_t* words;
    float* norms;
    uint32_t* qjl_words;
    float* qjl_norms;
};
constexpr int kKvEncodeMaxSegments = 32;
template <int NSEG>
struct KvEncodeTableT {
    KvEncodeDst seg[NSEG];
};
using KvEncodeTable = KvEncodeTableT<kKvEncodeMaxSegments>;

// A second tensor (the values beside the keys of a decode step: x2, wht_seed2, tab2, never with residual bits) rides in
// the same launch as vectors n_vec .. n_vec + n_vec2 - 1.
// The segment tables are kernel parameters; NSEG is their capacity (1, 8 or 32 segments): a launch whose parameters
// run to kilobytes costs the host several microseconds more than a small one, and a decode step appends to one or
// a few sequences.
template <int E, typename InT, int NSEG>
__global__ void __launch_bounds__(128) kv_encode_kernel(const InT* __restrict__ x, long n_vec, uint32_t wht_seed,
                                                        uint32_t qjl_seed, int with_qjl_first, float scale, float inv_sqrt,
                                                        const __grid_constant__ KvEncodeTableT<NSEG> tab, long vec_per_seg,
                                                        const InT* __restrict__ x2, long n_vec2, uint32_t wht_seed2,
                                                        const __grid_constant__ KvEncodeTableT<NSEG> tab2) {
    pdl_wait_release();
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
    for (long gall = warp0; gall < n_vec + n_vec2; gall += n_warps) {
        const bool second = gall >= n_vec;
        const long gvec = second ? gall - n_vec : gall;
        const InT* const xs = second ? x2 : x;
        const uint32_t seed = second ? wht_seed2 : wht_seed;
        const int with_qjl = second ? 0 : with_qjl_first;
        float sgn[E];
#pragma unroll
        for (int j = 0; j < E; ++j) sgn[j] = sign_value(seed, static_cast<uint32_t>(lane * E + j));
        // destination of this vector: segment and position inside it
        const long sidx = gvec / vec_per_seg;
        const long vec = gvec - sidx * vec_per_seg;
        const KvEncodeDst& dst = second ? tab2.seg[sidx] : tab.seg[sidx];
        uint32_t* const words = dst.words;
        float* const norms = dst.norms;
        uint32_t* const qjl_words = dst.qjl_words;
        float* const qjl_norms = dst.qjl_norms;
        float v[E];
#pragma unroll
        for (int j = 0; j < E; ++j) {
            v[j] = load_as_f32(xs, static_cast<size_t>(gvec) * D + lane * E + j);
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

// The same encoder for bulk appends: a CTA takes VB vectors at a time through shared memory so that
// the two left-to-right sums of squares (the vector's norm and the residual's norm; their order is
// fixed by src/kv_cache.cpp:84-88, 226-231 and bit-exactness) run with ONE THREAD PER VECTOR, VB of
// them side by side, instead of one lane per warp while 31 wait.  The rotation, the codes and the
// sign bits are still done a warp per vector.  Rows of the staging array are one float longer than
// the vector: thread t walking row t then touches bank (t + j) % 32.
template <int E> struct KvBatch { static constexpr int kVecs = E <= 4 ? 128 : (E == 8 ? 64 : 32); };

constexpr int kKvBatchThreads = 512;   // 16 warps share a batch: the warp-per-vector part is latency-bound
template <int E, typename InT>
__global__ void __launch_bounds__(kKvBatchThreads) kv_encode_batch_kernel(const InT* __restrict__ x, long n_vec, uint32_t wht_seed,
                                                              uint32_t qjl_seed, int with_qjl, float scale, float inv_sqrt,
                                                              const __grid_constant__ KvEncodeTable tab, long vec_per_seg) {
    constexpr int D = 32 * E;
    constexpr int WPH = (D + 9) / 10;
    constexpr int QPH = D / 32;
    constexpr int VB = KvBatch<E>::kVecs;
    constexpr int RS = D + 1;   // row stride of the staging array, in floats
    extern __shared__ float s_stage[];          // [VB][RS]
    __shared__ float s_norm[VB];
    __shared__ uint8_t s_code[kKvBatchThreads / 32][D];
    __shared__ uint32_t s_bits[kKvBatchThreads / 32][QPH];
    __shared__ float s_bounds[7];
    __shared__ float s_cent[8];
    if (threadIdx.x < 8) s_cent[threadIdx.x] = kC3[threadIdx.x];
    if (threadIdx.x < 7) s_bounds[threadIdx.x] = __fmul_rn(__fadd_rn(kC3[threadIdx.x], kC3[threadIdx.x + 1]), 0.5f);

    const int tid = threadIdx.x, lane = tid & 31, wib = tid >> 5;
    float sgn[E];
#pragma unroll
    for (int j = 0; j < E; ++j) sgn[j] = sign_value(wht_seed, static_cast<uint32_t>(lane * E + j));

    for (long base = static_cast<long>(blockIdx.x) * VB; base < n_vec; base += static_cast<long>(gridDim.x) * VB) {
        const int nb = static_cast<int>(n_vec - base < VB ? n_vec - base : VB);
        __syncthreads();   // the previous batch has been consumed (and the tables are written)
        // 16-byte loads (the batch is contiguous in x and starts at a multiple of VB * D elements)
        constexpr int kPer = 16 / static_cast<int>(sizeof(InT));   // elements per load
        const InT* xb = x + static_cast<size_t>(base) * D;
        if (reinterpret_cast<uintptr_t>(xb) % 16 == 0) {
            for (int i = tid; i < nb * D / kPer; i += kKvBatchThreads) {
                const int e0 = i * kPer, vi = e0 / D, e = e0 - vi * D;
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xb) + i);
                float* dst = s_stage + vi * RS + e;
                if constexpr (sizeof(InT) == 2) {
                    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f = __half22float2(h[k]);
                        dst[2 * k] = f.x;
                        dst[2 * k + 1] = f.y;
                    }
                } else {
                    dst[0] = __uint_as_float(raw.x);
                    dst[1] = __uint_as_float(raw.y);
                    dst[2] = __uint_as_float(raw.z);
                    dst[3] = __uint_as_float(raw.w);
                }
            }
        } else {
            for (int i = tid; i < nb * D; i += kKvBatchThreads) {
                const int vi = i / D, e = i - vi * D;
                s_stage[vi * RS + e] = load_as_f32(x, static_cast<size_t>(base + vi) * D + e);
            }
        }
        __syncthreads();
        // ---- norms: one thread per vector, left to right ----
        if (tid < nb) {
            float acc = 0.0f;
            for (int j = 0; j < D; ++j) {
                const float t = s_stage[tid * RS + j];
                acc = __fadd_rn(acc, __fmul_rn(t, t));
            }
            const float norm = __fsqrt_rn(acc);
            s_norm[tid] = norm;
            const long gvec = base + tid, sidx = gvec / vec_per_seg;
            tab.seg[sidx].norms[gvec - sidx * vec_per_seg] = norm;
        }
        __syncthreads();
        // ---- rotation, codes, sign bits: a warp per vector ----
        for (int vi = wib; vi < nb; vi += kKvBatchThreads / 32) {
            const long gvec = base + vi, sidx = gvec / vec_per_seg, vec = gvec - sidx * vec_per_seg;
            const KvEncodeDst& dst = tab.seg[sidx];
            const float norm = s_norm[vi];
            const float inv_norm = (norm > 1e-10f) ? __fdiv_rn(1.0f, norm) : 0.0f;
            float v[E];
#pragma unroll
            for (int j = 0; j < E; ++j) v[j] = __fmul_rn(__fmul_rn(s_stage[vi * RS + lane * E + j], inv_norm), sgn[j]);
            warp_fwht<E>(v, lane);
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
                    s_stage[vi * RS + lane * E + j] = r;     // the residual replaces the vector
                    const float sg = qjl_sign_is_positive(qjl_seed, static_cast<uint32_t>(lane * E + j)) ? 1.0f : -1.0f;
                    if (__fmul_rn(r, sg) > 0.0f) my_bits |= 1u << j;
                }
            }
            if (with_qjl && my_bits) atomicOr(&s_bits[wib][(lane * E) >> 5], my_bits << ((lane * E) & 31));
            __syncwarp();
            if (with_qjl && lane < QPH) dst.qjl_words[vec * QPH + lane] = s_bits[wib][lane];
            for (int w = lane; w < WPH; w += 32) {
                uint32_t word = 0;
#pragma unroll
                for (int k = 0; k < 10; ++k) {
                    const int e = w * 10 + k;
                    if (e < D) word |= (static_cast<uint32_t>(s_code[wib][e]) & 7u) << (3 * k);
                }
                dst.words[vec * WPH + w] = word;
            }
            __syncwarp();
        }
        // ---- residual norms: one thread per vector again ----
        if (with_qjl) {
            __syncthreads();
            if (tid < nb) {
                float acc = 0.0f;
                for (int j = 0; j < D; ++j) {
                    const float t = s_stage[tid * RS + j];
                    acc = __fadd_rn(acc, __fmul_rn(t, t));
                }
                const long gvec = base + tid, sidx = gvec / vec_per_seg;
                tab.seg[sidx].qjl_norms[gvec - sidx * vec_per_seg] = __fsqrt_rn(acc);
            }
        }
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
        __align__(16) __half h[E];
#pragma unroll
        for (int j = 0; j < E; ++j) h[j] = __float2half_rn(__fmul_rn(__fmul_rn(v[j], sg[j]), norm));
        __half* dst = out + static_cast<size_t>(vec) * D + lane * E;
        constexpr int kBytes = E * 2;
        if (kBytes % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0) {
#pragma unroll
            for (int c = 0; c < (kBytes >= 16 ? kBytes / 16 : 1); ++c) reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(h)[c];
        } else if (kBytes == 8 && reinterpret_cast<uintptr_t>(dst) % 8 == 0) {
            *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(h);
        } else if (kBytes == 4 && reinterpret_cast<uintptr_t>(dst) % 4 == 0) {
            *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(h);
        } else {
#pragma unroll
            for (int j = 0; j < E; ++j) dst[j] = h[j];
        }
    }
}

// ---- decode attention, first version -----------------------------------------------------------
// One query position per sequence; all G query heads of a KV head share one pass over
// that head's codes.  Scores are taken in the rotated domain (the query is rotated once,
// keys are never un-rotated), values are accumulated in the rotated domain and
// un-rotated once at the end.  Context is split across CTAs (and warps); partial
// (max, sum, accumulator) triples are merged by attn_combine_kernel.
constexpr int kAttnGMax = 8;

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
                                                           float inv_scale_d, __half* __restrict__ out,
                                                           float* __restrict__ lse) {
    pdl_wait_release();
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
    // log of the softmax denominator: lets a caller merge results over disjoint token ranges
    if (lse != nullptr && lane == 0) lse[row] = (L > 0.0f) ? M + __logf(L) : -INFINITY;
#pragma unroll
    for (int j = 0; j < E; ++j)
        out[row * D + lane * E + j] =
            __float2half_rn(v[j] * inv_sqrt * sign_value(v_seed, static_cast<uint32_t>(lane * E + j)) * invL);
}

// ---- decode attention on the tensor cores (head_dim 128) ------------------------------------------
// One warp owns 16-token tiles.  Layouts (all mma.sync.m16n8k16, fp16 in, fp32 accumulate):
//   S^T[16 tokens x 8 heads]  = K[16 x 128]   . Qrot^T[128 x 8]      (8 MMAs, centroid part)
//   S2^T                       = Sgn[16 x 128] . Qsgn^T[128 x 8]      (8 MMAs, 1-bit residual part)
//   O^T[128 dims x 8 heads]   += V^T[128 x 16] . P^T[16 x 8]           (8 MMAs)
// so the 7 query heads of a GQA group fill the n = 8 side and no MMA row is wasted.
// Codes become fp16 fragments through a 64-entry table indexed by a PAIR of 3-bit codes (the
// reference packs ten codes per word, so pairs never straddle words); the table is replicated
// per lane in shared memory so lookups never bank-conflict.  Thread q of a quad owns the pairs
// of words q, q+4, q+8 and pair q of word 12; the resulting permutation of the 128 dims is
// the same on both operands of each product and is undone when the partial result is written.
// V tiles are looked up in [token x dim] order and transposed in registers (movmatrix).
constexpr int kMmaThreads = 128;
constexpr float kCentroidScale = kAttnCentroidScale;

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// First dim of pair `pidx` (0..15) owned by quad-thread q.
__host__ __device__ __forceinline__ int attn_pair_dim(int q, int pidx) {
    return pidx < 15 ? 10 * (q + 4 * (pidx / 5)) + 2 * (pidx % 5) : 120 + 2 * q;
}

template <typename QT>
__global__ void __launch_bounds__(kMmaThreads, 3) attn_mma_kernel(const AttnSeq* __restrict__ seqs, const QT* __restrict__ qv,
                                                               int q_heads, int kv_heads, int n_splits, uint32_t k_seed,
                                                               uint32_t qjl_seed, int use_qjl, float inv_sqrt,
                                                               float inv_scale_d, float attn_scale, float gamma,
                                                               float* __restrict__ part_acc, float* __restrict__ part_ml) {
    pdl_wait_release();
    constexpr int D = 128, WPH = 13, QPH = 4;
    // The pair table sits at a shared-window address that is a multiple of its size, so that
    // "table base + lane offset" and the scaled index occupy disjoint bits and one logic op
    // forms a lookup address.  The window offset of a static array is not under the program's
    // control, so the aligned address is chosen at run time inside a buffer of twice the size.
    __shared__ __align__(16) uint32_t s_tab[2 * 64 * 32];
    // rotated queries of this KV head's group, [head][32-dim word][dim in word], padded so that the
    // fragment set-up below reads without bank conflicts (bank = 4 g + word + dim)
    __shared__ float s_q[8][4][33];
    __shared__ float s_m[4][8], s_l[4][8];
    __shared__ float s_acc[4][8][D + 4];   // row stride 132: the publishing stores below hit 32 distinct banks

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y % kv_heads, gchunk = blockIdx.y / kv_heads, seq = blockIdx.z;
    const int G = q_heads / kv_heads;
    const int g0 = gchunk * 8;
    const int ng = min(8, G - g0);

    const uint32_t tab_addr = static_cast<uint32_t>(__cvta_generic_to_shared(s_tab));
    const uint32_t lut_addr = (tab_addr + 8191u) & ~8191u;           // pair table, [pair index][lane]
    uint32_t* const s_lut = s_tab + ((lut_addr - tab_addr) >> 2);
    for (int i = tid; i < 64 * 32; i += kMmaThreads) {
        const int idx = i >> 5;
        s_lut[i] = pack_half2(kCentroidScale * kC3[idx & 7], kCentroidScale * kC3[idx >> 3]);
    }
    // rotated queries: fp16-round, sign, butterfly, 1/sqrt(d)  (one warp per head)
    for (int h = warp; h < 8; h += 4) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float t = 0.f;
            if (h < ng) {
                const size_t qi = (static_cast<size_t>(seq) * q_heads + kvh * G + g0 + h) * D + lane * 4 + j;
                t = __half2float(__float2half_rn(static_cast<float>(qv[qi])));
            }
            v[j] = t * sign_value(k_seed, static_cast<uint32_t>(lane * 4 + j));
        }
        warp_fwht<4>(v, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) s_q[h][lane >> 3][(lane & 7) * 4 + j] = v[j] * inv_sqrt;
    }
    __syncthreads();

    // B fragments (head n = g): the centroid product uses this thread's pair dims; the sign
    // product pairs bits p and p + 16 of sign word q (dims 32 q + p, 32 q + p + 16), with the
    // key-side sign folded in.
    uint32_t bq[16], bs[16];
#pragma unroll
    for (int pidx = 0; pidx < 16; ++pidx) {
        const int d = attn_pair_dim(q, pidx);
        const float x0 = s_q[g][d >> 5][d & 31], x1 = s_q[g][(d + 1) >> 5][(d + 1) & 31];
        const float h0 = __half2float(__float2half_rn(x0)), h1 = __half2float(__float2half_rn(x1));
        bq[pidx] = pack_half2(h0, h1);
        const int e = 32 * q + pidx;
        const float s0 = qjl_sign_is_positive(qjl_seed, static_cast<uint32_t>(e)) ? 1.f : -1.f;
        const float s1 = qjl_sign_is_positive(qjl_seed, static_cast<uint32_t>(e + 16)) ? 1.f : -1.f;
        bs[pidx] = pack_half2(s_q[g][q][pidx] * s0, s_q[g][q][pidx + 16] * s1);
    }

    const AttnSeq S = seqs[seq];
    const int n_tok = S.end - S.start;
    const int t0 = S.start + static_cast<int>(static_cast<long>(n_tok) * split / n_splits);
    const int t1 = S.start + static_cast<int>(static_cast<long>(n_tok) * (split + 1) / n_splits);

    const uint32_t lut_base = lut_addr + static_cast<uint32_t>(lane) * 4u;
    auto lut_pair = [&](uint32_t word, int bit) -> uint32_t {
        // ((word >> bit) & 63) * 128 + lane * 4
        const uint32_t sh = bit >= 7 ? (word >> (bit - 7)) : (word << (7 - bit));
        uint32_t v;
        asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(lut_base | (sh & (63u << 7))));
        return v;
    };
    // Sign bits p and p + 16 of an INVERTED sign word -> fp16 pair (+-1, +-1) without a table:
    // a set bit of the inverted word becomes the fp16 sign bit of 1.0.
    auto sgn_pair = [&](uint32_t inv_word, int pp) -> uint32_t {
        const uint32_t sh = pp == 15 ? inv_word : (inv_word << (15 - pp));
        return (sh & 0x80008000u) | 0x3C003C00u;
    };
    // this thread's four code words of one token record, and the 16 pair fragments they hold
    auto load_words = [&](const uint32_t* rec, uint32_t (&w)[4]) {
        w[0] = __ldg(rec + q);
        w[1] = __ldg(rec + q + 4);
        w[2] = __ldg(rec + q + 8);
        w[3] = __ldg(rec + 12);
    };
    auto dequant16 = [&](const uint32_t (&w)[4], uint32_t (&out)[16]) {
        const uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3];
#pragma unroll
        for (int j = 0; j < 5; ++j) {
            out[j] = lut_pair(w0, 6 * j);
            out[5 + j] = lut_pair(w1, 6 * j);
            out[10 + j] = lut_pair(w2, 6 * j);
        }
        out[15] = lut_pair(w3 >> (6 * q), 0);
    };

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // heads 2q, 2q+1
    float acc[8][4];
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[mt][k] = 0.f;

    // Software pipeline over 16-token tiles: everything a tile reads from the cache (key words,
    // sign words, value words, the four norms) sits in registers when the tile starts, and each
    // register group is refilled for the NEXT tile right after its last use in this one, so every
    // load has a whole tile of work to hide behind and no extra registers are needed.  The refill
    // addresses are clamped, so the last tile's refills read valid (unused) records.
    // record index of this thread's two tokens of the tile starting at tb (clamped so loads stay
    // in range; tokens past the end are masked out of the scores)
    auto rec_of = [&](int tok) { return static_cast<size_t>(tok < t1 ? tok : t1 - 1) * kv_heads + kvh; };
    uint32_t kwa[4] = {0, 0, 0, 0}, kwb[4] = {0, 0, 0, 0}, vwa[4] = {0, 0, 0, 0}, vwb[4] = {0, 0, 0, 0};
    uint32_t wa_n = 0, wb_n = 0;
    float qa_n = 0.f, qb_n = 0.f, kna_n = 0.f, knb_n = 0.f, vna_n = 0.f, vnb_n = 0.f;
    if (t0 + warp * 16 < t1) {
        const size_t r0 = rec_of(t0 + warp * 16 + g), r1 = rec_of(t0 + warp * 16 + g + 8);
        load_words(S.k_words + r0 * WPH, kwa);
        load_words(S.k_words + r1 * WPH, kwb);
        load_words(S.v_words + r0 * WPH, vwa);
        load_words(S.v_words + r1 * WPH, vwb);
        if (use_qjl) {
            wa_n = __ldg(S.qjl_words + r0 * QPH + q);
            wb_n = __ldg(S.qjl_words + r1 * QPH + q);
            qa_n = __ldg(S.qjl_norms + r0);
            qb_n = __ldg(S.qjl_norms + r1);
        }
        kna_n = __ldg(S.k_norms + r0);
        knb_n = __ldg(S.k_norms + r1);
        vna_n = __ldg(S.v_norms + r0);
        vnb_n = __ldg(S.v_norms + r1);
    }
    for (int tb = t0 + warp * 16; tb < t1; tb += 64) {
        const int ta = tb + g, tbb = tb + g + 8;
        const bool va = ta < t1, vb = tbb < t1;
        const size_t na = rec_of(tb + 64 + g), nb = rec_of(tb + 64 + g + 8);  // this thread's records of the next tile
        const float kscale = inv_scale_d * attn_scale / kCentroidScale;
        const float kna = kna_n * kscale, knb = knb_n * kscale;
        kna_n = __ldg(S.k_norms + na);
        knb_n = __ldg(S.k_norms + nb);
        uint32_t wa = wa_n, wb = wb_n;
        float qa = qa_n, qb = qb_n;
        if (use_qjl) {
            wa_n = __ldg(S.qjl_words + na * QPH + q);
            wb_n = __ldg(S.qjl_words + nb * QPH + q);
            qa_n = __ldg(S.qjl_norms + na);
            qb_n = __ldg(S.qjl_norms + nb);
        }

        // ---- scores ----
        float c1[4] = {0.f, 0.f, 0.f, 0.f};
        {
            uint32_t ka[16], kb[16];
            dequant16(kwa, ka);
            dequant16(kwb, kb);
            load_words(S.k_words + na * WPH, kwa);  // the next tile's key words
            load_words(S.k_words + nb * WPH, kwb);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                mma_f16(c1, ka[2 * ks], kb[2 * ks], ka[2 * ks + 1], kb[2 * ks + 1], bq[2 * ks], bq[2 * ks + 1]);
            }
        }
        if (use_qjl) {
            float c2[4] = {0.f, 0.f, 0.f, 0.f};
            wa = ~wa;
            wb = ~wb;
            qa *= gamma * kCentroidScale;
            qb *= gamma * kCentroidScale;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                mma_f16(c2, sgn_pair(wa, 2 * ks), sgn_pair(wb, 2 * ks), sgn_pair(wa, 2 * ks + 1), sgn_pair(wb, 2 * ks + 1),
                        bs[2 * ks], bs[2 * ks + 1]);
            c1[0] = fmaf(qa, c2[0], c1[0]);
            c1[1] = fmaf(qa, c2[1], c1[1]);
            c1[2] = fmaf(qb, c2[2], c1[2]);
            c1[3] = fmaf(qb, c2[3], c1[3]);
        }
        // c1: (token g: heads 2q, 2q+1), (token g+8: heads 2q, 2q+1)
        float s00 = va ? c1[0] * kna : -INFINITY, s01 = va ? c1[1] * kna : -INFINITY;
        float s10 = vb ? c1[2] * knb : -INFINITY, s11 = vb ? c1[3] * knb : -INFINITY;

        // ---- online softmax per head (reduce over the 16 tokens = over g) ----
        float mx0 = fmaxf(s00, s10), mx1 = fmaxf(s01, s11);
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
        }
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float cr0 = __expf(m_run[0] - mn0), cr1 = __expf(m_run[1] - mn1);
        const float p00 = __expf(s00 - mn0), p01 = __expf(s01 - mn1), p10 = __expf(s10 - mn0), p11 = __expf(s11 - mn1);
        // this lane's share of the running sums (its two tokens); lanes are added up after the loop
        l_run[0] = fmaf(l_run[0], cr0, p00 + p10);
        l_run[1] = fmaf(l_run[1], cr1, p01 + p11);
        m_run[0] = mn0;
        m_run[1] = mn1;
        // once the running maxima have settled the correction is exactly 1: skip the rescale then
        if (__any_sync(0xffffffffu, cr0 != 1.f || cr1 != 1.f)) {
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                acc[mt][0] *= cr0;
                acc[mt][1] *= cr1;
                acc[mt][2] *= cr0;
                acc[mt][3] *= cr1;
            }
        }
        // P^T fragment: (tokens 2q, 2q+1 | 2q+8, 2q+9 ; head g) from (token g | g+8 ; heads 2q, 2q+1)
        const float vna = vna_n * (1.0f / kCentroidScale), vnb = vnb_n * (1.0f / kCentroidScale);
        vna_n = __ldg(S.v_norms + na);
        vnb_n = __ldg(S.v_norms + nb);
        const uint32_t pb0 = movmatrix_trans(pack_half2(p00 * vna, p01 * vna));
        const uint32_t pb1 = movmatrix_trans(pack_half2(p10 * vnb, p11 * vnb));

        // ---- values ----
        {
            uint32_t xa[16], xb[16];
            dequant16(vwa, xa);
            dequant16(vwb, xb);
            load_words(S.v_words + na * WPH, vwa);  // the next tile's value words
            load_words(S.v_words + nb * WPH, vwb);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                // V[token x dim] fragment of dim block ks -> V^T[dim x token] fragment
                const uint32_t a0 = movmatrix_trans(xa[2 * ks]);      // dims 0-7  x tokens 0-7
                const uint32_t a1 = movmatrix_trans(xa[2 * ks + 1]);  // dims 8-15 x tokens 0-7
                const uint32_t a2 = movmatrix_trans(xb[2 * ks]);      // dims 0-7  x tokens 8-15
                const uint32_t a3 = movmatrix_trans(xb[2 * ks + 1]);  // dims 8-15 x tokens 8-15
                mma_f16(acc[ks], a0, a1, a2, a3, pb0, pb1);
            }
        }
    }

    // ---- publish this warp's state in natural dim order, merge the 4 warps, write the partial ----
    // acc[mt]: (slot g: heads 2q, 2q+1), (slot g+8: heads 2q, 2q+1); slot -> dim through the pair map
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], o);
        l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], o);
    }
    if (g == 0) {
        s_m[warp][2 * q] = m_run[0];
        s_m[warp][2 * q + 1] = m_run[1];
        s_l[warp][2 * q] = l_run[0];
        s_l[warp][2 * q + 1] = l_run[1];
    }
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int slot = g + 8 * hf;                   // row of the m-tile
            const int qq = (slot & 7) >> 1, lowbit = slot & 1, half = slot >> 3;
            const int d = attn_pair_dim(qq, 2 * mt + half) + lowbit;
            s_acc[warp][2 * q][d] = acc[mt][2 * hf];
            s_acc[warp][2 * q + 1][d] = acc[mt][2 * hf + 1];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < ng * D; idx += kMmaThreads) {
        const int h = idx / D, e = idx - h * D;
        const float M = fmaxf(fmaxf(s_m[0][h], s_m[1][h]), fmaxf(s_m[2][h], s_m[3][h]));
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = (s_m[w][h] == -INFINITY) ? 0.f : __expf(s_m[w][h] - M);
            L = fmaf(s_l[w][h], f, L);
            A = fmaf(s_acc[w][h][e], f, A);
        }
        const size_t slot = (static_cast<size_t>(seq) * q_heads + kvh * G + g0 + h) * n_splits + split;
        part_acc[slot * D + e] = A;
        if (e == 0) {
            part_ml[slot * 2] = M;
            part_ml[slot * 2 + 1] = L;
        }
    }
}

// ---- decode attention, bulk-copy pipeline (head_dim 128) ----------------------------------------
// Same arithmetic as attn_mma_kernel, different data movement: a CTA owns a token range for GH KV heads at once,
// one warp per head.  The token-major storage makes the records of 16 tokens x all heads one
// contiguous slab per array, so a tile is fetched by six cp.async.bulk copies (key words, value
// words, sign words, three norm arrays) that complete on an mbarrier; a ring of kPipeStages tiles
// is in flight, no cache word passes through a register on its way in, and the warps read their
// records from shared memory without bank conflicts (token stride GH*13 words = 20 mod 32 for
// four heads).  With more KV heads than GH a CTA takes a group of GH heads and the tile is fetched
// as 16 per-token rows per array instead (16 lanes issue them).  Tiles are aligned to multiples
// of 16 tokens from the start of the layer's storage, whose capacity is a multiple of 16 tokens,
// so every copy source is 16-byte aligned and inside the allocation; tokens outside [start, end)
// are masked.  Every mbarrier wait is bounded: on a time-out the CTA raises *status, lets the
// copies in flight land, and returns without writing a result.
constexpr int kPipeStages = 4;
constexpr float kSoftmaxSlack = kAttnSoftmaxSlack;
constexpr int kPipeWarpsPerSm = 16;   // 128 registers per thread
constexpr unsigned long long kPipeWaitLimitNs = 200ull * 1000 * 1000;

__device__ __forceinline__ unsigned long long pipe_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool pipe_wait(uint32_t bar, uint32_t parity, volatile unsigned int* abort_flag) {
    unsigned long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t done;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (done) return true;
        if ((spin & 15) == 15 && *abort_flag) return false;
        if (spin == 64) t0 = pipe_timer_ns();
        if (spin > 64 && (spin & 63) == 0 && pipe_timer_ns() - t0 > kPipeWaitLimitNs) return false;
    }
}
__device__ __forceinline__ void pipe_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

template <int GH>
struct PipeLayout {
    static constexpr int kKBytes = 16 * GH * 52;     // key (and value) words of a tile
    static constexpr int kSBytes = 16 * GH * 16;     // sign words
    static constexpr int kNBytes = 16 * GH * 4;      // one norm array
    static constexpr int kOffV = kKBytes, kOffS = 2 * kKBytes, kOffKN = kOffS + kSBytes, kOffVN = kOffKN + kNBytes,
                         kOffQN = kOffVN + kNBytes;
    static constexpr int kStageBytes = kOffQN + kNBytes;
    static constexpr int kQStride = 136;             // halves per rotated query row
    static constexpr int kOffStages = 0;             // offsets into the dynamic shared memory
    static constexpr int kOffQ = kOffStages + kPipeStages * kStageBytes;
    static constexpr int kOffBars = kOffQ + GH * 8 * kQStride * 2;
    static constexpr int kSmemBytes = kOffBars + 2 * kPipeStages * 8;
    static_assert(kStageBytes % 16 == 0 && kKBytes % 16 == 0, "bulk copies move multiples of 16 bytes");
    static_assert(kPipeStages * kStageBytes >= GH * 8 * (128 + 4) * 4, "the result staging reuses the ring");
};

template <int GH, typename QT>
__global__ void __launch_bounds__(32 * GH, kPipeWarpsPerSm / GH) attn_pipe_kernel(const AttnSeq* __restrict__ seqs, const QT* __restrict__ qv,
                                                                    int q_heads, int kv_heads, int n_splits, uint32_t k_seed,
                                                                    uint32_t qjl_seed, int use_qjl, float inv_sqrt,
                                                                    float inv_scale_d, float attn_scale, float gamma,
                                                                    float* __restrict__ part_acc, float* __restrict__ part_ml,
                                                                    unsigned int* __restrict__ status) {
    pdl_wait_release();
    using LY = PipeLayout<GH>;
    constexpr int D = 128;
    extern __shared__ __align__(16) unsigned char pipe_smem[];
    // pair table [pair index][lane]: static, so its window address is an immediate of the lookup loads
    __shared__ __align__(16) uint32_t s_lut[64 * 32];
    __shared__ unsigned int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int G = q_heads / kv_heads;
    const int gchunks = (G + 7) / 8;
    const int split = blockIdx.x, grp = blockIdx.y / gchunks, gchunk = blockIdx.y - grp * gchunks, seq = blockIdx.z;
    const int kvh = grp * GH + warp;
    const int g0 = gchunk * 8;
    const int ng = min(8, G - g0);
    const bool rows_mode = kv_heads > GH;            // a head group of a wider cache: per-token rows

    const uint32_t raw_addr = static_cast<uint32_t>(__cvta_generic_to_shared(pipe_smem));
    unsigned char* const base = pipe_smem;
    __half* const s_q = reinterpret_cast<__half*>(base + LY::kOffQ) + warp * 8 * LY::kQStride;
    const uint32_t stage_addr = raw_addr + LY::kOffStages;
    const uint32_t bar_full = raw_addr + LY::kOffBars, bar_empty = bar_full + 8u * kPipeStages;

    const AttnSeq S = seqs[seq];
    const int first_tile = S.start >> 4, end_tile = (S.end + 15) >> 4;
    const int all_tiles = S.end > S.start ? end_tile - first_tile : 0;
    const int tile0 = first_tile + static_cast<int>(static_cast<long>(all_tiles) * split / n_splits);
    const int tile1 = first_tile + static_cast<int>(static_cast<long>(all_tiles) * (split + 1) / n_splits);
    const int n_tiles = tile1 - tile0;

    // one tile of the ring: expected bytes, then the copies (warp 0 only; all its lanes call)
    auto issue_tile = [&](int it) {
        const uint32_t dst = stage_addr + static_cast<uint32_t>(it % kPipeStages) * LY::kStageBytes;
        const uint32_t bar = bar_full + 8u * static_cast<uint32_t>(it % kPipeStages);
        const size_t tok = static_cast<size_t>(tile0 + it) * 16;
        if (lane == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(LY::kStageBytes) : "memory");
        __syncwarp();
        if (!rows_mode) {
            if (lane == 0) {
                const size_t rec = tok * GH;
                pipe_copy(dst, S.k_words + rec * 13, LY::kKBytes, bar);
                pipe_copy(dst + LY::kOffV, S.v_words + rec * 13, LY::kKBytes, bar);
                pipe_copy(dst + LY::kOffS, S.qjl_words + rec * 4, LY::kSBytes, bar);
                pipe_copy(dst + LY::kOffKN, S.k_norms + rec, LY::kNBytes, bar);
                pipe_copy(dst + LY::kOffVN, S.v_norms + rec, LY::kNBytes, bar);
                pipe_copy(dst + LY::kOffQN, S.qjl_norms + rec, LY::kNBytes, bar);
            }
        } else if (lane < 16) {
            const size_t rec = (tok + lane) * kv_heads + static_cast<size_t>(grp) * GH;
            pipe_copy(dst + lane * (GH * 52), S.k_words + rec * 13, GH * 52, bar);
            pipe_copy(dst + LY::kOffV + lane * (GH * 52), S.v_words + rec * 13, GH * 52, bar);
            pipe_copy(dst + LY::kOffS + lane * (GH * 16), S.qjl_words + rec * 4, GH * 16, bar);
            pipe_copy(dst + LY::kOffKN + lane * (GH * 4), S.k_norms + rec, GH * 4, bar);
            pipe_copy(dst + LY::kOffVN + lane * (GH * 4), S.v_norms + rec, GH * 4, bar);
            pipe_copy(dst + LY::kOffQN + lane * (GH * 4), S.qjl_norms + rec, GH * 4, bar);
        }
    };

    if (warp == 0) {
        if (lane == 0) {
            s_abort = 0u;
            for (int s = 0; s < kPipeStages; ++s) {
                asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_full + 8u * s), "r"(1) : "memory");
                asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_empty + 8u * s), "r"(GH) : "memory");
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        // the first tiles start moving while the tables below are set up
        for (int it = 0; it < min(kPipeStages, n_tiles); ++it) issue_tile(it);
    }
    for (int i = tid; i < 64 * 32; i += 32 * GH) {
        const int idx = i >> 5;
        s_lut[i] = pack_half2(kCentroidScale * kC3[idx & 7], kCentroidScale * kC3[idx >> 3]);
    }
    // rotated queries of this warp's KV head: fp16-round, sign, butterfly, 1/sqrt(d), fp16-round
    for (int h = 0; h < 8; ++h) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float t = 0.f;
            if (h < ng) {
                const size_t qi = (static_cast<size_t>(seq) * q_heads + kvh * G + g0 + h) * D + lane * 4 + j;
                t = __half2float(__float2half_rn(static_cast<float>(qv[qi])));
            }
            v[j] = t * sign_value(k_seed, static_cast<uint32_t>(lane * 4 + j));
        }
        warp_fwht<4>(v, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) s_q[h * LY::kQStride + lane * 4 + j] = __float2half_rn(v[j] * inv_sqrt);
    }
    __syncthreads();
    volatile unsigned int* abort_flag = &s_abort;

    // B fragments, as in attn_mma_kernel
    uint32_t bq[16], bs[16];
#pragma unroll
    for (int pidx = 0; pidx < 16; ++pidx) {
        const int d = attn_pair_dim(q, pidx);
        const __half2 hq = __halves2half2(s_q[g * LY::kQStride + d], s_q[g * LY::kQStride + d + 1]);
        bq[pidx] = *reinterpret_cast<const uint32_t*>(&hq);
        const int e = 32 * q + pidx;
        const float s0 = qjl_sign_is_positive(qjl_seed, static_cast<uint32_t>(e)) ? 1.f : -1.f;
        const float s1 = qjl_sign_is_positive(qjl_seed, static_cast<uint32_t>(e + 16)) ? 1.f : -1.f;
        bs[pidx] = pack_half2(__half2float(s_q[g * LY::kQStride + e]) * s0, __half2float(s_q[g * LY::kQStride + e + 16]) * s1);
    }

    const uint32_t lane_off = static_cast<uint32_t>(lane) * 4u;
    auto lut_pair = [&](uint32_t word, int bit) -> uint32_t {
        // byte offset ((word >> bit) & 63) * 128 + lane * 4: one shift, one logic op; the table's address is an immediate
        const uint32_t sh = bit >= 7 ? (word >> (bit - 7)) : (word << (7 - bit));
        return *reinterpret_cast<const uint32_t*>(reinterpret_cast<const unsigned char*>(s_lut) + ((sh & (63u << 7)) | lane_off));
    };
    auto sgn_pair = [&](uint32_t inv_word, int pp) -> uint32_t {
        const uint32_t sh = pp == 15 ? inv_word : (inv_word << (15 - pp));
        return (sh & 0x80008000u) | 0x3C003C00u;
    };
    auto dequant16 = [&](const uint32_t (&w)[4], uint32_t (&out)[16]) {
        const uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3];
#pragma unroll
        for (int j = 0; j < 5; ++j) {
            out[j] = lut_pair(w0, 6 * j);
            out[5 + j] = lut_pair(w1, 6 * j);
            out[10 + j] = lut_pair(w2, 6 * j);
        }
        out[15] = lut_pair(w3 >> (6 * q), 0);
    };

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float acc[8][4];
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[mt][k] = 0.f;

    // this thread's two records of a tile: tokens g and g + 8 of head `warp` of the group
    const int ra = g * GH + warp, rb = ra + 8 * GH;
    const float kscale = inv_scale_d * attn_scale / kCentroidScale;
    const float qscale = gamma * kCentroidScale;
    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
        const int s = it % kPipeStages;
        const uint32_t ph = static_cast<uint32_t>(it / kPipeStages) & 1u;
        if (warp == 0 && it > 0 && it - 1 + kPipeStages < n_tiles) {
            // the stage of the previous tile is free once every warp has read it: refill it
            if (!pipe_wait(bar_empty + 8u * ((it - 1) % kPipeStages), static_cast<uint32_t>((it - 1) / kPipeStages) & 1u, abort_flag)) {
                ok = false;
                break;
            }
            issue_tile(it - 1 + kPipeStages);
        }
        if (!pipe_wait(bar_full + 8u * s, ph, abort_flag)) {
            ok = false;
            break;
        }
        const unsigned char* st = base + LY::kOffStages + s * LY::kStageBytes;
        const uint32_t* sk = reinterpret_cast<const uint32_t*>(st);
        const uint32_t* sv = reinterpret_cast<const uint32_t*>(st + LY::kOffV);
        const uint32_t* ss = reinterpret_cast<const uint32_t*>(st + LY::kOffS);
        const float* skn = reinterpret_cast<const float*>(st + LY::kOffKN);
        const float* svn = reinterpret_cast<const float*>(st + LY::kOffVN);
        const float* sqn = reinterpret_cast<const float*>(st + LY::kOffQN);
        uint32_t kwa[4], kwb[4], vwa[4], vwb[4];
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            kwa[j] = sk[ra * 13 + q + 4 * j];
            kwb[j] = sk[rb * 13 + q + 4 * j];
            vwa[j] = sv[ra * 13 + q + 4 * j];
            vwb[j] = sv[rb * 13 + q + 4 * j];
        }
        kwa[3] = sk[ra * 13 + 12];
        kwb[3] = sk[rb * 13 + 12];
        vwa[3] = sv[ra * 13 + 12];
        vwb[3] = sv[rb * 13 + 12];
        uint32_t wa = 0, wb = 0;
        float qa = 0.f, qb = 0.f;
        if (use_qjl) {
            wa = ~ss[ra * 4 + q];
            wb = ~ss[rb * 4 + q];
            qa = sqn[ra] * qscale;
            qb = sqn[rb] * qscale;
        }
        const int ta = (tile0 + it) * 16 + g, tb = ta + 8;
        const bool va = ta >= S.start && ta < S.end, vb = tb >= S.start && tb < S.end;
        const float kna = skn[ra] * kscale, knb = skn[rb] * kscale;
        const float vna = va ? svn[ra] * (1.0f / kCentroidScale) : 0.f, vnb = vb ? svn[rb] * (1.0f / kCentroidScale) : 0.f;
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_empty + 8u * s) : "memory");

        // ---- scores (two accumulators per product: dependent chains of four MMAs, not eight) ----
        float c1[4] = {0.f, 0.f, 0.f, 0.f}, c1b[4] = {0.f, 0.f, 0.f, 0.f};
        {
            uint32_t ka[16], kb[16];
            dequant16(kwa, ka);
            dequant16(kwb, kb);
#pragma unroll
            for (int ks = 0; ks < 8; ks += 2) {
                mma_f16(c1, ka[2 * ks], kb[2 * ks], ka[2 * ks + 1], kb[2 * ks + 1], bq[2 * ks], bq[2 * ks + 1]);
                mma_f16(c1b, ka[2 * ks + 2], kb[2 * ks + 2], ka[2 * ks + 3], kb[2 * ks + 3], bq[2 * ks + 2], bq[2 * ks + 3]);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) c1[k] += c1b[k];
        if (use_qjl) {
            float c2[4] = {0.f, 0.f, 0.f, 0.f}, c2b[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 8; ks += 2) {
                mma_f16(c2, sgn_pair(wa, 2 * ks), sgn_pair(wb, 2 * ks), sgn_pair(wa, 2 * ks + 1), sgn_pair(wb, 2 * ks + 1),
                        bs[2 * ks], bs[2 * ks + 1]);
                mma_f16(c2b, sgn_pair(wa, 2 * ks + 2), sgn_pair(wb, 2 * ks + 2), sgn_pair(wa, 2 * ks + 3), sgn_pair(wb, 2 * ks + 3),
                        bs[2 * ks + 2], bs[2 * ks + 3]);
            }
            c1[0] = fmaf(qa, c2[0] + c2b[0], c1[0]);
            c1[1] = fmaf(qa, c2[1] + c2b[1], c1[1]);
            c1[2] = fmaf(qb, c2[2] + c2b[2], c1[2]);
            c1[3] = fmaf(qb, c2[3] + c2b[3], c1[3]);
        }
        const float s00 = va ? c1[0] * kna : -INFINITY, s01 = va ? c1[1] * kna : -INFINITY;
        const float s10 = vb ? c1[2] * knb : -INFINITY, s11 = vb ? c1[3] * knb : -INFINITY;

        // ---- online softmax per head, with a lazy reference: the running reference m_run only moves
        // (and the sums are only rescaled) when some score of the tile exceeds it by more than
        // kSoftmaxSlack, so the usual tile needs one vote instead of a reduction over the tokens.
        // Probabilities are then at most e^slack (7.4), still far from the fp16 range once
        // multiplied by a value norm.  Every tile of [tile0, tile1) holds a token of [start, end),
        // so the reference is finite from the first tile on.
        const float tm0 = fmaxf(s00, s10), tm1 = fmaxf(s01, s11);
        if (__any_sync(0xffffffffu, tm0 > m_run[0] + kSoftmaxSlack || tm1 > m_run[1] + kSoftmaxSlack)) {
            float mx0 = tm0, mx1 = tm1;
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
            }
            const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
            const float cr0 = __expf(m_run[0] - mn0), cr1 = __expf(m_run[1] - mn1);
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
        const float p00 = __expf(s00 - m_run[0]), p01 = __expf(s01 - m_run[1]);
        const float p10 = __expf(s10 - m_run[0]), p11 = __expf(s11 - m_run[1]);
        l_run[0] += p00 + p10;
        l_run[1] += p01 + p11;
        const uint32_t pb0 = movmatrix_trans(pack_half2(p00 * vna, p01 * vna));
        const uint32_t pb1 = movmatrix_trans(pack_half2(p10 * vnb, p11 * vnb));

        // ---- values ----
        {
            uint32_t xa[16], xb[16];
            dequant16(vwa, xa);
            dequant16(vwb, xb);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t a0 = movmatrix_trans(xa[2 * ks]);
                const uint32_t a1 = movmatrix_trans(xa[2 * ks + 1]);
                const uint32_t a2 = movmatrix_trans(xb[2 * ks]);
                const uint32_t a3 = movmatrix_trans(xb[2 * ks + 1]);
                mma_f16(acc[ks], a0, a1, a2, a3, pb0, pb1);
            }
        }
    }
    if (!ok) atomicExch(&s_abort, 1u);
    __syncthreads();   // every warp is past its last read of the ring (or has given up)
    if (s_abort) {
        // let whatever was requested land before the shared memory is released
        if (tid == 0) {
            *reinterpret_cast<volatile unsigned int*>(status) = 11u;   // may be host memory: a plain store, then a system fence
            __threadfence_system();
            const unsigned long long t0 = pipe_timer_ns();
            while (pipe_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        }
        __syncthreads();
        return;
    }

    // ---- publish: natural dim order through the (now idle) ring, one region per warp ----
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], o);
        l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], o);
    }
    float* const s_acc = reinterpret_cast<float*>(base + LY::kOffStages) + warp * 8 * (D + 4);
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int slot = g + 8 * hf;
            const int qq = (slot & 7) >> 1, lowbit = slot & 1, half = slot >> 3;
            const int d = attn_pair_dim(qq, 2 * mt + half) + lowbit;
            s_acc[(2 * q) * (D + 4) + d] = acc[mt][2 * hf];
            s_acc[(2 * q + 1) * (D + 4) + d] = acc[mt][2 * hf + 1];
        }
    }
    __syncwarp();
    const size_t slot0 = (static_cast<size_t>(seq) * q_heads + kvh * G + g0) * n_splits + split;
    for (int idx = lane; idx < ng * D; idx += 32) {
        const int h = idx >> 7, e = idx & (D - 1);
        part_acc[(slot0 + static_cast<size_t>(h) * n_splits) * D + e] = s_acc[h * (D + 4) + e];
    }
    if (g == 0) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int h = 2 * q + j;
            if (h < ng) {
                part_ml[(slot0 + static_cast<size_t>(h) * n_splits) * 2] = m_run[j];
                part_ml[(slot0 + static_cast<size_t>(h) * n_splits) * 2 + 1] = l_run[j];
            }
        }
    }
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
    KvEncodeSegment one{words, norms, qjl_words, qjl_norms};
    launch_kv_encode_segments(x, x_is_f16, n_vec, n_vec, head_dim, wht_seed, qjl_seed, with_qjl, &one, 1, stream);
}

// The warp-per-vector kernel on one tensor (n2 == 0) or on a tensor and a second one without residual bits.
template <int NSEG>
static void launch_kv_encode_small(const void* x, const void* x2, bool x_is_f16, long n_vec, long n2, long vec_per_seg, int head_dim,
                                   uint32_t seed, uint32_t seed2, uint32_t qjl_seed, bool with_qjl, const KvEncodeSegment* segs,
                                   const KvEncodeSegment* segs2, int n_segs, cudaStream_t stream) {
    KvEncodeTableT<NSEG> t1{}, t2{};
    for (int i = 0; i < n_segs; ++i) {
        t1.seg[i] = KvEncodeDst{segs[i].words, segs[i].norms, segs[i].qjl_words, segs[i].qjl_norms};
        if (n2 > 0) t2.seg[i] = KvEncodeDst{segs2[i].words, segs2[i].norms, nullptr, nullptr};
    }
    const float scale = std::sqrt(static_cast<float>(head_dim));             // src/kv_cache.cpp:72
    const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(head_dim));   // src/rotation.cpp:301
    const int grid = grid_for_warps(n_vec + n2, 4, 148 * 16);
#define TQ_ENC2(EV)                                                                                                                 \
    if (x_is_f16)                                                                                                                   \
        launch_pdl(kv_encode_kernel<EV, __half, NSEG>, dim3(grid), dim3(128), 0, stream, static_cast<const __half*>(x), n_vec, seed, qjl_seed, \
                                                                     with_qjl ? 1 : 0, scale, inv_sqrt, t1, vec_per_seg,            \
                                                                     static_cast<const __half*>(x2), n2, seed2, t2);                \
    else                                                                                                                            \
        launch_pdl(kv_encode_kernel<EV, float, NSEG>, dim3(grid), dim3(128), 0, stream, static_cast<const float*>(x), n_vec, seed, qjl_seed, \
                                                                    with_qjl ? 1 : 0, scale, inv_sqrt, t1, vec_per_seg,             \
                                                                    static_cast<const float*>(x2), n2, seed2, t2);
    TQ_D_SWITCH(head_dim, TQ_ENC2)
#undef TQ_ENC2
    TQ_CUDA(cudaGetLastError());
}

// Keys (with residual bits) and values of a few tokens in ONE launch of the warp-per-vector kernel; bulk appends
// keep one launch per tensor of the batched kernel.
void launch_kv_encode_pair_segments(const void* k, const void* v, bool x_is_f16, long n_vec, long vec_per_seg, int head_dim,
                                    uint32_t k_seed, uint32_t v_seed, uint32_t qjl_seed, const KvEncodeSegment* ksegs,
                                    const KvEncodeSegment* vsegs, int n_segs, cudaStream_t stream) {
    if (n_vec == 0) return;
    if (n_vec >= 512) {
        launch_kv_encode_segments(k, x_is_f16, n_vec, vec_per_seg, head_dim, k_seed, qjl_seed, true, ksegs, n_segs, stream);
        launch_kv_encode_segments(v, x_is_f16, n_vec, vec_per_seg, head_dim, v_seed, 0u, false, vsegs, n_segs, stream);
        return;
    }
    TQ_REQUIRE(n_segs >= 1 && n_segs <= kKvEncodeMaxSegments, "kv encode: 1..32 segments per launch");
    TQ_REQUIRE(vec_per_seg > 0 && (n_vec + vec_per_seg - 1) / vec_per_seg <= n_segs, "kv encode: segments do not cover the input");
    if (n_segs == 1) launch_kv_encode_small<1>(k, v, x_is_f16, n_vec, n_vec, vec_per_seg, head_dim, k_seed, v_seed, qjl_seed, true, ksegs, vsegs, n_segs, stream);
    else if (n_segs <= 8) launch_kv_encode_small<8>(k, v, x_is_f16, n_vec, n_vec, vec_per_seg, head_dim, k_seed, v_seed, qjl_seed, true, ksegs, vsegs, n_segs, stream);
    else launch_kv_encode_small<kKvEncodeMaxSegments>(k, v, x_is_f16, n_vec, n_vec, vec_per_seg, head_dim, k_seed, v_seed, qjl_seed, true, ksegs, vsegs, n_segs, stream);
}

void launch_kv_encode_segments(const void* x, bool x_is_f16, long n_vec, long vec_per_seg, int head_dim, uint32_t wht_seed,
                               uint32_t qjl_seed, bool with_qjl, const KvEncodeSegment* segs, int n_segs,
                               cudaStream_t stream) {
    if (n_vec == 0) return;
    TQ_REQUIRE(n_segs >= 1 && n_segs <= kKvEncodeMaxSegments, "kv encode: 1..32 segments per launch");
    TQ_REQUIRE(vec_per_seg > 0 && (n_vec + vec_per_seg - 1) / vec_per_seg <= n_segs, "kv encode: segments do not cover the input");
    KvEncodeTable tab{};
    for (int i = 0; i < n_segs; ++i) tab.seg[i] = KvEncodeDst{segs[i].words, segs[i].norms, segs[i].qjl_words, segs[i].qjl_norms};
    const float scale = std::sqrt(static_cast<float>(head_dim));             // src/kv_cache.cpp:72
    const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(head_dim));   // src/rotation.cpp:301
    // Bulk appends go through the batched kernel (one thread per vector for the sequential sums);
    // a handful of vectors (a decode step) keep the warp-per-vector kernel and its lower latency.
    if (n_vec >= 512) {
#define TQ_ENCB(EV)                                                                                                       \
    {                                                                                                                     \
        constexpr int kVB = KvBatch<EV>::kVecs;                                                                           \
        const int smem = kVB * (32 * EV + 1) * static_cast<int>(sizeof(float));                                           \
        long blocks = (n_vec + kVB - 1) / kVB;                                                                            \
        if (blocks > 148 * 3) blocks = 148 * 3;                                                                           \
        static bool configured[2][64] = {{false}};                                                                        \
        int dev = 0;                                                                                                      \
        TQ_CUDA(cudaGetDevice(&dev));                                                                                     \
        const int ti = x_is_f16 ? 0 : 1;                                                                                  \
        if (dev < 0 || dev >= 64 || !configured[ti][dev]) {                                                               \
            if (x_is_f16) TQ_CUDA(cudaFuncSetAttribute(kv_encode_batch_kernel<EV, __half>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
            else TQ_CUDA(cudaFuncSetAttribute(kv_encode_batch_kernel<EV, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));           \
            if (dev >= 0 && dev < 64) configured[ti][dev] = true;                                                         \
        }                                                                                                                 \
        if (x_is_f16)                                                                                                     \
            kv_encode_batch_kernel<EV, __half><<<static_cast<unsigned>(blocks), kKvBatchThreads, smem, stream>>>(                     \
                static_cast<const __half*>(x), n_vec, wht_seed, qjl_seed, with_qjl ? 1 : 0, scale, inv_sqrt, tab, vec_per_seg); \
        else                                                                                                              \
            kv_encode_batch_kernel<EV, float><<<static_cast<unsigned>(blocks), kKvBatchThreads, smem, stream>>>(                      \
                static_cast<const float*>(x), n_vec, wht_seed, qjl_seed, with_qjl ? 1 : 0, scale, inv_sqrt, tab, vec_per_seg);  \
    }
        TQ_D_SWITCH(head_dim, TQ_ENCB)
#undef TQ_ENCB
        TQ_CUDA(cudaGetLastError());
        return;
    }
    if (n_segs == 1) launch_kv_encode_small<1>(x, nullptr, x_is_f16, n_vec, 0, vec_per_seg, head_dim, wht_seed, 0u, qjl_seed, with_qjl, segs, nullptr, n_segs, stream);
    else if (n_segs <= 8) launch_kv_encode_small<8>(x, nullptr, x_is_f16, n_vec, 0, vec_per_seg, head_dim, wht_seed, 0u, qjl_seed, with_qjl, segs, nullptr, n_segs, stream);
    else launch_kv_encode_small<kKvEncodeMaxSegments>(x, nullptr, x_is_f16, n_vec, 0, vec_per_seg, head_dim, wht_seed, 0u, qjl_seed, with_qjl, segs, nullptr, n_segs, stream);
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

// KV heads one CTA of the bulk-copy pipeline kernel takes (0: that kernel does not apply).
static int attn_pipe_heads(int head_dim, int kv_heads) {
    if (head_dim != 128) return 0;
    if (kv_heads % 4 == 0) return 4;
    return (kv_heads == 1 || kv_heads == 2) ? kv_heads : 0;
}

// Plan of one attention call: which kernel, and how many context splits.
// kernel: 0 chooses, 1 forces the load-based kernels, 2 forces the bulk-copy pipeline (where it
// applies).  The pipeline pays a heavier per-CTA set-up (each warp rotates its own query group)
// and writes one partial per (head, split) for four heads per CTA, so it is chosen when every
// resident CTA slot still gets at least 512 tokens to walk; shorter jobs run the load-based
// kernel, whose four warps share one head's set-up.
// Splits: the launch runs in ceil(CTAs / resident CTAs) waves and a wave costs about (tokens a
// warp walks + a fixed set-up cost expressed in tokens); pick the count that minimises waves x
// cost.  Pipeline: a CTA is (sequence, group of KV heads, query-head group, split) and every warp
// walks the whole range of the split.  Load-based: a CTA is (sequence, KV head, query-head group,
// split) and its four warps share the range.
AttnPlan attn_make_plan(int n_seqs, int q_heads, int kv_heads, int head_dim, int max_tok, int sm_count, int kernel) {
    const int G = q_heads / kv_heads;
    const int gchunks = (G + kAttnGMax - 1) / kAttnGMax;
    if (kernel == 0) {
        static const int env_kernel = [] {
            const char* e = std::getenv("TQ_ATTENTION_KERNEL");
            return e ? std::atoi(e) : 0;
        }();
        kernel = env_kernel;
    }
    if (kernel == 3 && head_dim == 128 && kv_heads == 4) {
        // tensor-memory kernel: a CTA is (sequence, query-head group, split) over all four KV heads
        const long ctas_per_split = static_cast<long>(n_seqs) * gchunks;
        const long resident = static_cast<long>(sm_count) * kAttnTcCtasPerSm;
        const int max_splits = std::max(1, std::min(512, max_tok / 256));
        AttnPlan plan{1, 0, 1};
        double best = 1e300;
        for (int n = 1; n <= max_splits; ++n) {
            const long waves = (ctas_per_split * n + resident - 1) / resident;
            const double cost = static_cast<double>(waves) * (static_cast<double>(max_tok) / n + 256.0);
            if (cost < best * 0.999) {
                best = cost;
                plan.n_splits = n;
            }
        }
        return plan;
    }
    if (kernel == 3) kernel = 0;
    int gh = kernel == 1 ? 0 : attn_pipe_heads(head_dim, kv_heads);
    // A CTA that takes only some of the KV heads copies its tiles token by token (the records of a token's heads are
    // contiguous, a head group's are not): 32 x 8 heads x ctx 8192 then ran at 920 GB/s against 1610 GB/s for the
    // load-based kernel, so the pipeline is chosen only when one CTA takes all the heads.
    if (gh && kernel == 0 && gh != kv_heads) gh = 0;
    if (gh && kernel == 0) {
        const long slots = static_cast<long>(sm_count) * (kPipeWarpsPerSm / gh);
        const long ctas_at_512 = static_cast<long>(n_seqs) * (kv_heads / gh) * gchunks * (max_tok / 512);
        if (ctas_at_512 < slots) gh = 0;
    }
    const long ctas_per_split = gh ? static_cast<long>(n_seqs) * (kv_heads / gh) * gchunks : static_cast<long>(n_seqs) * kv_heads * gchunks;
    const long resident = static_cast<long>(sm_count) * (gh ? kPipeWarpsPerSm / gh : 3);
    const double walk = gh ? 1.0 : 0.25, setup = gh ? 96.0 : 40.0;
    const int min_tok = gh ? 128 : 256;
    const int max_splits = std::max(1, std::min(gh ? 512 : 128, max_tok / min_tok));
    AttnPlan plan{1, gh, 0};
    double best = 1e300;
    for (int n = 1; n <= max_splits; ++n) {
        const long waves = (ctas_per_split * n + resident - 1) / resident;
        const double cost = static_cast<double>(waves) * (walk * static_cast<double>(max_tok) / n + setup);
        if (cost < best * 0.999) {
            best = cost;
            plan.n_splits = n;
        }
    }
    return plan;
}

template <int GH, typename QT>
static void launch_attn_pipe(const AttnSeq* seqs, int n_seqs, const QT* q, int q_heads, int kv_heads, int n_splits, uint32_t k_seed,
                             uint32_t qjl_seed, bool use_qjl, float inv_sqrt, float inv_scale_d, float attn_scale, float gamma,
                             float* part_acc, float* part_ml, unsigned int* status, cudaStream_t stream) {
    // the opt-in shared-memory size is a per-device attribute of each instantiation
    static bool configured[64] = {false};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(attn_pipe_kernel<GH, QT>, cudaFuncAttributeMaxDynamicSharedMemorySize, PipeLayout<GH>::kSmemBytes));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int gchunks = (q_heads / kv_heads + kAttnGMax - 1) / kAttnGMax;
    const dim3 grid(n_splits, (kv_heads / GH) * gchunks, n_seqs);
    launch_pdl(attn_pipe_kernel<GH, QT>, grid, dim3(32 * GH), PipeLayout<GH>::kSmemBytes, stream, seqs, q, q_heads, kv_heads, n_splits, k_seed,
               qjl_seed, use_qjl ? 1 : 0, inv_sqrt, inv_scale_d, attn_scale, gamma, part_acc, part_ml, status);
}

void launch_kv_attention(const void* d_seqs, int n_seqs, const void* q, bool q_is_f16, int q_heads, int kv_heads,
                         int head_dim, AttnPlan plan, uint32_t k_seed, uint32_t v_seed, uint32_t qjl_seed, bool use_qjl,
                         void* scratch, __half* out, float* lse, unsigned int* status, cudaStream_t stream) {
    if (n_seqs == 0) return;
    const int n_splits = plan.n_splits;
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
    launch_pdl(attn_combine_kernel<EV>, dim3(static_cast<unsigned>((n_rows + 3) / 4)), dim3(128), 0, stream, part_acc, part_ml, n_rows, \
               n_splits, v_seed, inv_sqrt, inv_scale_d, out, lse);
    if (plan.tensor_memory) {
        launch_attn_tc(static_cast<const AttnSeq*>(d_seqs), n_seqs, q, q_is_f16, q_heads, kv_heads, n_splits, k_seed, qjl_seed, use_qjl,
                       inv_sqrt, inv_scale_d, attn_scale, gamma, part_acc, part_ml, status, stream);
        launch_pdl(attn_combine_kernel<4>, dim3(static_cast<unsigned>((n_rows + 3) / 4)), dim3(128), 0, stream, part_acc, part_ml, n_rows,
                   n_splits, v_seed, inv_sqrt, inv_scale_d, out, lse);
        TQ_CUDA(cudaGetLastError());
        return;
    }
    if (const int gh = plan.pipe_heads) {
        TQ_REQUIRE(gh == attn_pipe_heads(head_dim, kv_heads), "attention: plan does not match the cache shape");
        const AttnSeq* seqs = static_cast<const AttnSeq*>(d_seqs);
#define TQ_PIPE(GHV)                                                                                                            \
    if (q_is_f16)                                                                                                               \
        launch_attn_pipe<GHV, __half>(seqs, n_seqs, static_cast<const __half*>(q), q_heads, kv_heads, n_splits, k_seed, qjl_seed, \
                                      use_qjl, inv_sqrt, inv_scale_d, attn_scale, gamma, part_acc, part_ml, status, stream);    \
    else                                                                                                                        \
        launch_attn_pipe<GHV, float>(seqs, n_seqs, static_cast<const float*>(q), q_heads, kv_heads, n_splits, k_seed, qjl_seed,  \
                                     use_qjl, inv_sqrt, inv_scale_d, attn_scale, gamma, part_acc, part_ml, status, stream);
        if (gh == 4) {
            TQ_PIPE(4)
        } else if (gh == 2) {
            TQ_PIPE(2)
        } else {
            TQ_PIPE(1)
        }
#undef TQ_PIPE
        launch_pdl(attn_combine_kernel<4>, dim3(static_cast<unsigned>((n_rows + 3) / 4)), dim3(128), 0, stream, part_acc, part_ml, n_rows,
                   n_splits, v_seed, inv_sqrt, inv_scale_d, out, lse);
        TQ_CUDA(cudaGetLastError());
        return;
    }
    if (head_dim == 128) {
        if (q_is_f16)
            launch_pdl(attn_mma_kernel<__half>, grid, dim3(kMmaThreads), 0, stream, static_cast<const AttnSeq*>(d_seqs),
                       static_cast<const __half*>(q), q_heads, kv_heads, n_splits, k_seed, qjl_seed, use_qjl ? 1 : 0, inv_sqrt,
                       inv_scale_d, attn_scale, gamma, part_acc, part_ml);
        else
            launch_pdl(attn_mma_kernel<float>, grid, dim3(kMmaThreads), 0, stream, static_cast<const AttnSeq*>(d_seqs),
                       static_cast<const float*>(q), q_heads, kv_heads, n_splits, k_seed, qjl_seed, use_qjl ? 1 : 0, inv_sqrt,
                       inv_scale_d, attn_scale, gamma, part_acc, part_ml);
        launch_pdl(attn_combine_kernel<4>, dim3(static_cast<unsigned>((n_rows + 3) / 4)), dim3(128), 0, stream, part_acc, part_ml, n_rows,
                   n_splits, v_seed, inv_sqrt, inv_scale_d, out, lse);
        TQ_CUDA(cudaGetLastError());
        return;
    }
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
