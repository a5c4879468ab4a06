// Launchers of the sm_100a kernels (host-callable, asynchronous on `stream`).
// All pointers are device pointers unless stated otherwise.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>
#include <vector>

namespace tq {

// tq_wht.cu — blocked WHT of an fp32 [rows, cols] matrix (forward or inverse), bit-exact.
void launch_wht_rows(const float* in, float* out, long rows, int cols, uint32_t seed, uint32_t block, bool inverse,
                     cudaStream_t stream);

// tq_dequant.cu
// flags[0] is OR-ed with 1 when any residual byte is non-zero, flags[1] when a 5-bit-mode
// code does not fit the joint byte.
void launch_relayout(const uint8_t* packed_primary, const uint8_t* packed_residual, uint8_t* joint, long out, int in,
                     bool primary_5bit, unsigned int* flags, cudaStream_t stream);
void launch_unrelayout(const uint8_t* joint, uint8_t* packed_primary, uint8_t* packed_residual, long out, int in,
                       bool primary_5bit, cudaStream_t stream);
// tables: 256 fp32 (single rotation) or 512 fp32 (dual rotation: primary then residual).
void launch_dequant_f32(const uint8_t* joint, const float* norms, const float* tables, float* out, long rows, int in,
                        uint32_t block, uint32_t seed_p, uint32_t seed_r, bool dual, cudaStream_t stream);
void launch_dequant_f16(const uint8_t* joint, const float* norms, const float* tables, __half* out, long rows, int in,
                        uint32_t block, uint32_t seed_p, uint32_t seed_r, bool dual, cudaStream_t stream);

// tq_gemv.cu — fused dequantise + GEMV, 1..8 activation rows.  table: [n_planes, 256] fp32
// (one plane for shared rotation / primary only, two for dual rotation).
// scratch: gemv_scratch_bytes(out, in) bytes, zero-initialised once (the kernel leaves
// its counters at zero); may be NULL when that size is 0.  status: one device word,
// set non-zero by the kernel if its shared-memory layout assumption does not hold.
size_t gemv_scratch_bytes(int out, int in, int n_planes);
void launch_tq8_gemv(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y,
                     int out, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r,
                     void* scratch, unsigned int* status, int sm_count, cudaStream_t stream);

// The same with the fp16 result written to n_dst (1..8) buffers at once: destination d receives
// activation row n, output row r at dst[d][n * dst_stride + r].  Destinations may be other GPUs'
// memory mapped into this process (peer access / CUDA IPC): plain stores, no multicast.
// Fused all-gather of a row-sharded layer (gather != nullptr): the results are stored into dst[0]
// only; the CTA that completes the grid copies the block to dst[1..n_dst) with 16-byte stores and
// raises flag `signal_slot` of signal[0..n_signal) with the value ++(*epoch).  With n_wait > 0 every
// CTA waits (bounded) for wait_flags[0..n_wait) to reach *wait_epoch + 1 before it reads x, and the
// completing CTA advances *wait_epoch: a chain of such layers needs no separate exchange kernel.
struct GemvGather {
    unsigned int* epoch;
    const unsigned int* wait_flags;
    int n_wait;
    unsigned int* wait_epoch;
    // flag-in-data variant (ll_world > 0): every rank's packet buffer, this rank's own at [ll_rank]
    int ll_rank = 0, ll_world = 0;
    void* ll_base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
};
void launch_tq8_gemv_scatter(const uint8_t* codes, const float* norms, const float* table, const __half* x,
                             __half* const* dst, int n_dst, long dst_stride, int out, int in, int batch, uint32_t block,
                             int n_planes, uint32_t seed_p, uint32_t seed_r, void* scratch, unsigned int* status,
                             int sm_count, cudaStream_t stream, unsigned int* const* signal = nullptr, int signal_slot = 0,
                             unsigned int signal_value = 0, unsigned int* done_counter = nullptr,
                             const GemvGather* gather = nullptr, int n_signal = 0);
// Several matrices against the same activation (device fp16, 1..8 rows) in one launch: y of matrix i = its own
// [batch, out_i] buffer.  The matrices share in_features and the rotation mode; each brings its own scratch
// (gemv_scratch_bytes) and status word.
struct GemvGroupItem {
    const uint8_t* codes;
    const float* norms;
    const float* table;
    __half* y;
    int out, in;
    uint32_t block;
    int n_planes;
    uint32_t seed_p, seed_r;
    void* scratch;
    unsigned int* status;
};
void launch_tq8_gemv_group(const GemvGroupItem* items, int n, const __half* x, int batch, int sm_count, cudaStream_t stream);
// With `signal` (one flag array per destination): once the whole grid has stored its results,
// signal[d][signal_slot] = signal_value on every destination (release, system scope); `done_counter`
// must be a zero-initialised word in device memory (grid completion counter).  `status` may be
// page-locked host memory in every launcher of this file (kernels only store to it).  launch_peer_wait: one small kernel
// that waits, for at most a second, until flags[0..n) have all reached `value` (sets *status to
// 10 otherwise).
void launch_peer_wait(const unsigned int* flags, int n, unsigned int value, unsigned int* status, cudaStream_t stream);

// tq_gemv_staged.cu — the same operation with the codes staged through shared memory by bulk
// copies (cp.async.bulk + mbarrier), work balanced over CTAs to 4 KB, two CTAs per SM.
// scratch: gemv_staged_scratch_bytes(...) bytes, zero-initialised once.
size_t gemv_staged_scratch_bytes(int out, int in, int n_planes, int sm_count);
void launch_tq8_gemv_staged(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y,
                            int out, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r,
                            void* scratch, unsigned int* status, int sm_count, cudaStream_t stream);
size_t gemv_staged_scratch_need(int out, int in, int batch, int n_planes, int sm_count);
// Allocation-free variant over the library's built-in array (see launch_tq8_gemv_static).
bool gemv_staged_fits_static(int out, int in, int batch, int n_planes, int sm_count);
void launch_tq8_gemv_staged_static(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y,
                                   int out, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r,
                                   unsigned int* status, int sm_count, cudaStream_t stream);
void* gemv_static_scratch_address();   // device address of that array on the current device (tq_gemv.cu)
// The activation rotation of tq_gemv.cu alone: xrot = [n_planes, batch, in] fp32 (TF32-rounded).
void launch_rotate_x(const __half* x, float* xrot, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p,
                     uint32_t seed_r, cudaStream_t stream);

// Allocation-free variant: scratch is a fixed array in the library image
// (gemv_static_scratch_capacity() bytes); throws if the layer needs more.
size_t gemv_static_scratch_capacity();
void launch_tq8_gemv_static(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y,
                            int out, int in, int batch, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r,
                            unsigned int* status, int sm_count, cudaStream_t stream);

// tq_gemm.cu — fused dequantise + GEMM on tcgen05 / tensor memory for many activation rows
// (prefill).  x: [m, in] fp16, y: [m, out] fp16.  scratch: gemm_scratch_bytes(...) bytes (the
// rotated activation in fp16, plus fp32 partial sums when K is split over CTAs).  Needs in % 64 == 0 (gemm_supported).  status: one
// device word, set non-zero if the kernel refused to run or a bounded wait gave up.
bool gemm_supported(int in);
int gemm_k_splits(int out, int in, long m, int n_planes, int sm_count);
size_t gemm_scratch_bytes(int out, int in, long m, int n_planes, int sm_count);
// y_stride: elements between consecutive activation rows of y (0 = out).
void launch_tq8_gemm(const uint8_t* codes, const float* norms, const float* table, const __half* x, __half* y, int out,
                     int in, long m, uint32_t block, int n_planes, uint32_t seed_p, uint32_t seed_r, void* scratch,
                     unsigned int* status, int sm_count, cudaStream_t stream, long y_stride = 0);
// Several matrices against the same activation rows in one rotation launch, one GEMM launch and one split-K finish:
// y of matrix i = its own [m, out_i] buffer.  The matrices share in_features, the WHT block and the rotation mode; each
// brings its own scratch (gemm_scratch_bytes for its own shape) and status word.
struct GemmGroupItem {
    const uint8_t* codes;
    const float* norms;
    const float* table;
    __half* y;
    int out, in;
    uint32_t block;
    int n_planes;
    uint32_t seed_p, seed_r;
    void* scratch;
    unsigned int* status;
};
void launch_tq8_gemm_group(const GemmGroupItem* items, int n, const __half* x, long m, int sm_count, cudaStream_t stream);

// tq_quantize.cu — bit-exact weight quantiser.  derive_seeds hashes the sampled bytes
// of the fp32 weight (synchronises the stream).  launch_quantize_weight: cb_p / cb_r are
// HOST arrays; d_orig_norm_tmp is [out] fp32 and d_recon_tmp [out, in] fp32 scratch.
void derive_seeds(const float* d_weight, size_t n_elems, uint32_t* seed_primary, uint32_t* seed_residual,
                  cudaStream_t stream);
void launch_quantize_weight(const float* d_weight, long out, int in, const float* cb_p, int n_p, const float* cb_r,
                            int n_r, int primary_bits, int residual_bits, uint32_t block, bool shared_rotation,
                            uint32_t seed_p, uint32_t seed_r, uint8_t* d_packed_primary, uint8_t* d_packed_residual,
                            float* d_norms, float* d_orig_norm_tmp, float* d_recon_tmp, cudaStream_t stream);

// Row L2 norms with the quantiser's summation order (left to right in fp32).
void launch_row_norms(const float* d_matrix, float* d_out, long rows, int cols, cudaStream_t stream);

// tq_codebook_fit.cu — Lloyd-Max fit on the device and the per-layer sample extraction.
int launch_codebook_fit(const float* d_data, long n, int bits, int iterations, const float* init_centroids, float* centroids_out,
                        float* boundaries_out, cudaStream_t stream);
void launch_layer_samples(const float* d_weight, const float* d_row_norms, long rows, int in, uint32_t block, uint32_t seed_p,
                          const float* primary_centroids, int n_primary, float* d_scaled, float* d_residual, cudaStream_t stream);

// tq_qjl_shader.cu — the reference's QJL shader kernels (metal/turboquant_qjl.metal).
void launch_qjl_compress(const float* d_residual, int num_tokens, int num_heads, int head_dim, int proj_dim, uint32_t seed,
                         uint32_t* d_signs, float* d_norms, cudaStream_t stream);
void launch_qjl_dot_correction(const uint32_t* d_signs_q, const uint32_t* d_signs_k, const float* d_norms_k, int num_queries, int num_keys,
                               int num_heads, int head_idx, int proj_dim, float* d_corrections, cudaStream_t stream);

// tq_kv_kernels.cu — KV-cache encoder with several destinations: the n_vec input vectors
// ([n_vec, head_dim], contiguous) are cut into segments of vec_per_seg vectors and segment s is
// written to segs[s] (at most 32 segments per launch).  A decode step that appends one token to
// many sequences' caches is one launch for the keys and one for the values.
// How one decode-attention call runs (attn_make_plan in tq_kv_kernels.cu).
struct AttnPlan {
    int n_splits;     // context splits per sequence
    int pipe_heads;   // KV heads per CTA of the bulk-copy pipeline kernel; 0: load-based kernels
    int tensor_memory;   // 1: the tensor-memory kernel (tq_attn_tc.cu) instead of either
};

struct KvEncodeSegment {
    uint32_t* words;
    float* norms;
    uint32_t* qjl_words;  // may be NULL when with_qjl is false
    float* qjl_norms;
};
void launch_kv_encode_segments(const void* x, bool x_is_f16, long n_vec, long vec_per_seg, int head_dim, uint32_t wht_seed,
                               uint32_t qjl_seed, bool with_qjl, const KvEncodeSegment* segs, int n_segs,
                               cudaStream_t stream);
// keys (with residual bits) and values of the same tokens: one launch when there are fewer than 512 vectors
void launch_kv_encode_pair_segments(const void* k, const void* v, bool x_is_f16, long n_vec, long vec_per_seg, int head_dim,
                                    uint32_t k_seed, uint32_t v_seed, uint32_t qjl_seed, const KvEncodeSegment* ksegs,
                                    const KvEncodeSegment* vsegs, int n_segs, cudaStream_t stream);

// tq_peer.cu — exchange between ranks over peer-mapped memory (plain stores, flags with epochs).
void launch_exchange_broadcast(const void* src, void* const* dst, int n_dst, int rows, long row_bytes, long src_stride,
                               long dst_stride, unsigned int* const* signal, int n_signal, int slot, unsigned int* done,
                               unsigned int* epoch, cudaStream_t stream);
void launch_exchange_wait(const unsigned int* flags, int n, unsigned int* epoch, unsigned int* status, cudaStream_t stream);
// With norm_w: count is whole rows of `cols` elements, one CTA per row, which then also writes
// normed[row] = RMSNorm(out[row]) * norm_w (the bits launch_rmsnorm_f16 gives on out).
void launch_exchange_sum_f16(const __half* slots, int n_slots, long slot_stride, long count, const __half* residual, __half* out,
                             cudaStream_t stream, const __half* norm_w = nullptr, __half* normed = nullptr, int cols = 0,
                             float eps = 0.f);
void launch_exchange_wait_packets(const uint4* base, const unsigned int* epoch, unsigned int* wait_epoch, int rank, int world, long rows,
                                  int batch, __half* out, long out_stride, unsigned int* status, cudaStream_t stream);
void launch_exchange_sum_packets(const uint4* base, const unsigned int* epoch, unsigned int* wait_epoch, int rank, int world, long count,
                                 const __half* local, const __half* residual, __half* out, unsigned int* status, cudaStream_t stream,
                                 const __half* norm_w = nullptr, __half* normed = nullptr, int cols = 0, float eps = 0.f);
void launch_exchange_unpack_packets(const uint4* packets, long n_packets, __half* out, cudaStream_t stream);
void launch_exchange_merge_attention(const __half* outs, const float* lses, int parts, long rows, int dim, long part_stride_o,
                                     long part_stride_l, __half* out, cudaStream_t stream);

// tq_decoder_ops.cu — element-wise glue of a decoder layer (fp16 in / out, fp32 arithmetic).
void launch_rmsnorm_f16(const __half* x, const __half* weight, __half* y, long rows, int cols, float eps, cudaStream_t stream);
void launch_rope_f16(__half* x, const int* positions, long rows, int heads, int dim, float theta, cudaStream_t stream);
// queries [rows, q_heads, dim] and keys [rows, kv_heads, dim] in one launch
void launch_rope_qk_f16(__half* q, __half* k, const int* positions, long rows, int q_heads, int kv_heads, int dim, float theta,
                        cudaStream_t stream);
void launch_swiglu_f16(const __half* gate_up, __half* act, long rows, int inter, cudaStream_t stream);

// tq_misc.cu — small element-wise helpers.
void launch_f32_to_f16(const float* in, __half* out, long n, cudaStream_t stream);
void launch_f16_to_f32(const __half* in, float* out, long n, cudaStream_t stream);

}  // namespace tq
