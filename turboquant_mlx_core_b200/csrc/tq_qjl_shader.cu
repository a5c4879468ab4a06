// The two kernels of metal/turboquant_qjl.metal as CUDA kernels, arithmetic kept as the shader has it:
//   tq_qjl_compress (lines 52-137): one block per (head, token), one thread per projection row; the row of
//     the dense +-1 projection matrix comes from qjl_proj_sign's hash (lines 39-44); the dot product runs over
//     the columns in order; the residual's norm is the shader's shared-memory tree over proj_dim entries (only
//     the first min(head_dim, proj_dim) squares enter it, lines 91-96); sign bit = (dot >= 0), 32 per word.
//   tq_qjl_dot_correction (lines 163-216): matches = popcount(~(q ^ k)) summed over the words (unused high
//     bits of a last partial word are equal in both operands and so count as matches, as in the shader);
//     correction = sqrt(pi/2) / proj_dim * (2 * matches - proj_dim) * norm_k, evaluated left to right.
// The hash takes bit 0 of (h ^ h >> 16) * odd with h = seed ^ row * A ^ col * B: that bit is an XOR of a row term
// and a column term, so the projection matrix has rank one (sign(row, col) = a(row) * b(col)) and a vector's sign
// word is one fixed pattern or its complement.  Kept as the shader has it.
// This is the residual correction the reference ships as a shader; the KV cache's own 1-bit residual
// (src/kv_cache.cpp:215-258, a +-1 diagonal) is what the attention kernels read.
#include <cstdint>

#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

__device__ __forceinline__ float qjl_proj_sign(uint32_t seed, uint32_t proj_row, uint32_t col) {
    uint32_t h = seed ^ (proj_row * 2654435761u) ^ (col * 2246822519u);
    h ^= (h >> 16);
    h *= 0x45d9f3bu;
    return (h & 1u) ? 1.0f : -1.0f;
}

__global__ void __launch_bounds__(1024) qjl_compress_kernel(const float* __restrict__ residual, uint32_t head_dim, uint32_t num_heads,
                                                            uint32_t proj_dim, uint32_t proj_seed, uint32_t* __restrict__ signs_out,
                                                            float* __restrict__ norms_out) {
    __shared__ float shared_buf[1024];
    __shared__ uint32_t shared_signs[1024];
    const uint32_t tid = threadIdx.x, head_idx = blockIdx.x, token_idx = blockIdx.y;
    const size_t vec_offset = (static_cast<size_t>(token_idx) * num_heads + head_idx) * head_dim;
    float dot = 0.0f;
    for (uint32_t c = 0; c < head_dim; ++c) dot = __fadd_rn(dot, __fmul_rn(qjl_proj_sign(proj_seed, tid, c), residual[vec_offset + c]));
    if (tid < head_dim) {
        const float r = residual[vec_offset + tid];
        shared_buf[tid] = __fmul_rn(r, r);
    } else {
        shared_buf[tid] = 0.0f;
    }
    for (uint32_t stride = proj_dim / 2; stride > 0; stride >>= 1) {
        __syncthreads();
        if (tid < stride) shared_buf[tid] = __fadd_rn(shared_buf[tid], shared_buf[tid + stride]);
    }
    __syncthreads();
    if (tid == 0) norms_out[static_cast<size_t>(token_idx) * num_heads + head_idx] = __fsqrt_rn(shared_buf[0]);
    shared_signs[tid] = (dot >= 0.0f) ? 1u : 0u;
    __syncthreads();
    const uint32_t word_idx = tid / 32, bit_pos = tid % 32, words_per_vector = (proj_dim + 31) / 32;
    if (bit_pos == 0 && word_idx < words_per_vector) {
        uint32_t packed = 0;
        const uint32_t base = word_idx * 32;
        for (uint32_t i = 0; i < 32 && base + i < proj_dim; ++i) packed |= (shared_signs[base + i] & 1u) << i;
        signs_out[(static_cast<size_t>(token_idx) * num_heads + head_idx) * words_per_vector + word_idx] = packed;
    }
}

__global__ void __launch_bounds__(256) qjl_dot_correction_kernel(const uint32_t* __restrict__ signs_q, const uint32_t* __restrict__ signs_k,
                                                                 const float* __restrict__ norms_k, uint32_t proj_dim, uint32_t num_heads,
                                                                 uint32_t head_idx, uint32_t num_queries, uint32_t num_keys,
                                                                 float* __restrict__ corrections) {
    const uint32_t words_per_vec = (proj_dim + 31) / 32;
    const size_t total = static_cast<size_t>(num_queries) * num_keys;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t query_idx = static_cast<uint32_t>(i / num_keys), key_idx = static_cast<uint32_t>(i - static_cast<size_t>(query_idx) * num_keys);
        const uint32_t* q = signs_q + (static_cast<size_t>(query_idx) * num_heads + head_idx) * words_per_vec;
        const uint32_t* k = signs_k + (static_cast<size_t>(key_idx) * num_heads + head_idx) * words_per_vec;
        uint32_t total_matches = 0;
        for (uint32_t w = 0; w < words_per_vec; ++w) total_matches += __popc(~(q[w] ^ k[w]));
        const float signed_dot = __fsub_rn(static_cast<float>(2u * total_matches), static_cast<float>(proj_dim));
        const float norm = norms_k[static_cast<size_t>(key_idx) * num_heads + head_idx];
        corrections[i] = __fmul_rn(__fmul_rn(__fdiv_rn(1.2533141f, static_cast<float>(proj_dim)), signed_dot), norm);
    }
}

}  // namespace

void launch_qjl_compress(const float* d_residual, int num_tokens, int num_heads, int head_dim, int proj_dim, uint32_t seed,
                         uint32_t* d_signs, float* d_norms, cudaStream_t stream) {
    TQ_REQUIRE(proj_dim >= 1 && proj_dim <= 1024 && (proj_dim & (proj_dim - 1)) == 0, "qjl: proj_dim must be a power of two up to 1024");
    TQ_REQUIRE(num_heads >= 1 && head_dim >= 1 && num_tokens >= 0 && num_tokens <= 65535, "qjl: bad shape (at most 65535 tokens per call)");
    if (num_tokens == 0) return;
    qjl_compress_kernel<<<dim3(num_heads, num_tokens), proj_dim, 0, stream>>>(d_residual, head_dim, num_heads, proj_dim, seed, d_signs, d_norms);
    TQ_CUDA(cudaGetLastError());
}

void launch_qjl_dot_correction(const uint32_t* d_signs_q, const uint32_t* d_signs_k, const float* d_norms_k, int num_queries, int num_keys,
                               int num_heads, int head_idx, int proj_dim, float* d_corrections, cudaStream_t stream) {
    TQ_REQUIRE(proj_dim >= 1 && num_heads >= 1 && head_idx >= 0 && head_idx < num_heads, "qjl: bad shape");
    const size_t total = static_cast<size_t>(num_queries) * num_keys;
    if (total == 0) return;
    const int blocks = static_cast<int>(total + 255 < 148u * 8u * 256u ? (total + 255) / 256 : 148 * 8);
    qjl_dot_correction_kernel<<<blocks, 256, 0, stream>>>(d_signs_q, d_signs_k, d_norms_k, proj_dim, num_heads, head_idx, num_queries, num_keys,
                                                         d_corrections);
    TQ_CUDA(cudaGetLastError());
}

}  // namespace tq
