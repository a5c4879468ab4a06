// Shared by the decode-attention kernels (tq_kv_kernels.cu, tq_attn_tc.cu).
#pragma once
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

}  // namespace tq
