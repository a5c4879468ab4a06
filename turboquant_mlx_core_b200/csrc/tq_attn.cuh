// Shared by the decode-attention kernels (tq_kv_kernels.cu, tq_attn_tc.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace tq {

// One sequence of an attention call: the layer's storage (token-major records, see
// tq_kv_kernels.cu) and the token range [start, end) the query attends to.
struct AttnSeq {
    const uint32_t* k_words;
    const uint32_t* v_words;
    const float* k_norms;
    const float* v_norms;
    const uint32_t* qjl_words;
    const float* qjl_norms;
    int start, end;
};

// The pair tables hold kAttnCentroidScale * centroid: with this factor all four centroid
// magnitudes round to fp16 with a relative error below 1.4e-5 (unscaled: up to 3e-4, which the
// softmax amplifies); the factor is divided out of the key and value norms.
constexpr float kAttnCentroidScale = 1.1979075f;
// Lazy softmax reference: it only moves when a score exceeds it by more than this.
constexpr float kAttnSoftmaxSlack = 2.0f;

// Tensor-memory kernel (tq_attn_tc.cu): head_dim 128, four KV heads, up to 8 query heads per KV head
// and CTA.  Partials in the layout attn_combine_kernel reads.
void launch_attn_tc(const AttnSeq* seqs, int n_seqs, const void* q, bool q_is_f16, int q_heads, int kv_heads, int n_splits,
                    uint32_t k_seed, uint32_t qjl_seed, bool use_qjl, float inv_sqrt, float inv_scale_d, float attn_scale,
                    float gamma, float* part_acc, float* part_ml, unsigned int* status, cudaStream_t stream);
constexpr int kAttnTcCtasPerSm = 2;

// fp16 decode window (tq_attn_dense.cu): ring writes / reads and scaled-dot-product attention over a
// contiguous run of ring slots.  `row` = heads * head_dim.
void launch_ring_write(const void* keys, const void* values, bool is_f16, long n_tokens, long src_token0, int row, int window,
                       long slot0, __half* ring_k, __half* ring_v, cudaStream_t stream);
void launch_ring_read(const __half* ring, long n_tokens, int row, int window, long start, __half* out, cudaStream_t stream);
int dense_attention_splits(int n_tokens, int kv_heads, int q_heads, int sm_count);
size_t dense_attention_scratch_bytes(int q_heads, int head_dim, int n_splits);
void launch_dense_attention(const __half* keys, const __half* values, int n_tokens, int kv_heads, int head_dim, const void* q,
                            bool q_is_f16, int q_heads, int n_splits, void* scratch, __half* out, cudaStream_t stream);

}  // namespace tq
