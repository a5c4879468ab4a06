// Offline weight quantiser on the device, bit-identical to the reference's CPU route
// (quantize_weight, src/quantizer.cpp:41-261).
//
// Pipeline (all fp32, every operation rounded once, in the reference's order):
//   1. row norm   = sqrt(sum_j w*w), summed left to right            (:56-59)
//   2. w / max(norm, 1e-10)                                           (:62-66)
//   3. forward WHT with the primary seed, then * sqrt(in)             (:74-78)
//   4. primary code = #boundaries strictly below the value            (:83; src/codebook.cpp:295)
//   5. residual = value - centroid; shared rotation: code it in place;
//      dual rotation: * 1/sqrt(in), inverse WHT(primary seed), forward WHT(residual
//      seed), * sqrt(in), then code                                    (:118-148)
//   6. reconstruction in the normalised domain, its row norm (left-to-right sum again),
//      corrected norm = norm / max(recon_norm, 1e-10)                 (:162-248)
// One warp owns one (row, WHT block), so steps 2-6 never leave registers; the two row
// sums are separate passes because their summation order is sequential along the row.
// Content-derived seeds (FNV-1a over sampled bytes, :12-28) are computed on the host
// from a 4 KiB device gather.
#include <cmath>

#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

// sum_j m[r][j]^2, accumulated strictly left to right in fp32; out[r] = sqrt(sum).
// One warp per row: lanes read 32 consecutive columns (coalesced, four such pieces in flight) and
// square them; the running sum then takes the 32 squares in column order through lane
// broadcasts, every lane carrying the same sum.  Columns past the end contribute +0.0, which
// leaves a non-negative sum unchanged.  All rows run at once, so the matrix streams from HBM
// while each row's add chain (the order that makes the result bit-exact) stays serial.
__global__ void __launch_bounds__(256) row_norm_seq_kernel(const float* __restrict__ m, float* __restrict__ out,
                                                           long rows, int cols) {
    const int lane = threadIdx.x & 31;
    const long row = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (row >= rows) return;
    const float* src = m + row * cols;
    float acc = 0.0f;
    for (int c0 = 0; c0 < cols; c0 += 128) {
        float sq[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = c0 + 32 * u + lane;
            const float v = c < cols ? __ldg(src + c) : 0.0f;
            sq[u] = __fmul_rn(v, v);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, sq[u], j));
        }
    }
    if (lane == 0) out[row] = __fsqrt_rn(acc);
}

__global__ void corrected_norm_kernel(const float* __restrict__ orig, float* __restrict__ recon_inout, long rows) {
    const long r = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r < rows) recon_inout[r] = __fdiv_rn(orig[r], fmaxf(recon_inout[r], 1e-10f));
}

// The bytes derive_seed samples: byte i*stride of the fp32 weight buffer.
__global__ void gather_bytes_kernel(const uint8_t* __restrict__ bytes, size_t byte_count, size_t stride,
                                    uint8_t* __restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = bytes[static_cast<size_t>(i) * stride];
}

struct QuantTables {
    float cp[32], bp[31], cr[16], br[15];
    int n_p, n_r;
};

__device__ __forceinline__ int bin_of(float v, const float* bounds, int n_bounds) {
    int idx = 0;
    for (int i = 0; i < n_bounds; ++i) idx += (bounds[i] < v) ? 1 : 0;  // sorted, so this equals lower_bound
    return idx;
}

template <int E>
__global__ void __launch_bounds__(128) quantize_rows_kernel(
    const float* __restrict__ w, const float* __restrict__ orig_norm, uint8_t* __restrict__ packed_primary,
    uint8_t* __restrict__ packed_residual, float* __restrict__ recon, long rows, int blocks_per_row, uint32_t seed_p,
    uint32_t seed_r, int primary_bits, int residual_bits, int shared_rotation, float scale, float inv_scale,
    float inv_sqrt, const QuantTables tb) {
    __shared__ QuantTables t;
    if (threadIdx.x == 0) t = tb;
    __syncthreads();
    constexpr int BS = 32 * E;
    const int lane = threadIdx.x & 31;
    const long warp0 = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
    const long total = rows * blocks_per_row;
    const int in = blocks_per_row * BS;

    float sp[E], sr[E];
#pragma unroll
    for (int j = 0; j < E; ++j) {
        sp[j] = sign_value(seed_p, static_cast<uint32_t>(lane * E + j));
        sr[j] = sign_value(seed_r, static_cast<uint32_t>(lane * E + j));
    }

    for (long blk = warp0; blk < total; blk += n_warps) {
        const long row = blk / blocks_per_row;
        const int bcol = static_cast<int>(blk - row * blocks_per_row) * BS + lane * E;
        const size_t base = static_cast<size_t>(row) * in + bcol;
        const float safe = fmaxf(orig_norm[row], 1e-10f);
        float v[E];
#pragma unroll
        for (int j = 0; j < E; ++j) v[j] = __fmul_rn(__fdiv_rn(w[base + j], safe), sp[j]);
        warp_fwht<E>(v, lane);
        int cp_idx[E], cr_idx[E];
#pragma unroll
        for (int j = 0; j < E; ++j) {
            v[j] = __fmul_rn(__fmul_rn(v[j], inv_sqrt), scale);
            int idx = bin_of(v[j], t.bp, t.n_p - 1);
            if (idx >= t.n_p) idx = t.n_p - 1;
            cp_idx[j] = idx;
            cr_idx[j] = 0;
        }
        if (residual_bits > 0) {
            float r[E];
#pragma unroll
            for (int j = 0; j < E; ++j) r[j] = __fsub_rn(v[j], t.cp[cp_idx[j]]);
            if (!shared_rotation) {
#pragma unroll
                for (int j = 0; j < E; ++j) r[j] = __fmul_rn(r[j], inv_scale);
                warp_fwht<E>(r, lane);
#pragma unroll
                for (int j = 0; j < E; ++j) r[j] = __fmul_rn(__fmul_rn(r[j], __fmul_rn(inv_sqrt, sp[j])), sr[j]);
                warp_fwht<E>(r, lane);
#pragma unroll
                for (int j = 0; j < E; ++j) r[j] = __fmul_rn(__fmul_rn(r[j], inv_sqrt), scale);
            }
#pragma unroll
            for (int j = 0; j < E; ++j) {
                int idx = bin_of(r[j], t.br, t.n_r - 1);
                if (idx >= t.n_r) idx = t.n_r - 1;
                cr_idx[j] = idx & 0x0F;  // the reconstruction re-reads the packed nibble (:179-183)
            }
        }

        // ---- pack (src/quantizer.cpp:33-39, 94-111) ----
        if (primary_bits > 4) {
#pragma unroll
            for (int j = 0; j < E; ++j) packed_primary[base + j] = static_cast<uint8_t>(cp_idx[j]);
        }
        if constexpr (E >= 2) {
#pragma unroll
            for (int j = 0; j < E; j += 2) {
                if (primary_bits <= 4)
                    packed_primary[(base + j) >> 1] = static_cast<uint8_t>((cp_idx[j] & 0x0F) | ((cp_idx[j + 1] & 0x0F) << 4));
                packed_residual[(base + j) >> 1] = static_cast<uint8_t>(cr_idx[j] | (cr_idx[j + 1] << 4));
            }
        } else {
            const int p_hi = __shfl_down_sync(0xffffffffu, cp_idx[0], 1);
            const int r_hi = __shfl_down_sync(0xffffffffu, cr_idx[0], 1);
            if ((lane & 1) == 0) {
                if (primary_bits <= 4)
                    packed_primary[base >> 1] = static_cast<uint8_t>((cp_idx[0] & 0x0F) | ((p_hi & 0x0F) << 4));
                packed_residual[base >> 1] = static_cast<uint8_t>(cr_idx[0] | (r_hi << 4));
            }
        }

        // ---- reconstruction in the normalised domain (:162-235) ----
        float u[E];
        if (residual_bits > 0 && shared_rotation) {
#pragma unroll
            for (int j = 0; j < E; ++j)
                u[j] = __fmul_rn(__fadd_rn(t.cp[cp_idx[j]], t.cr[min(cr_idx[j], t.n_r - 1)]), inv_scale);
            warp_fwht<E>(u, lane);
#pragma unroll
            for (int j = 0; j < E; ++j) u[j] = __fmul_rn(u[j], __fmul_rn(inv_sqrt, sp[j]));
        } else {
#pragma unroll
            for (int j = 0; j < E; ++j) u[j] = __fmul_rn(t.cp[cp_idx[j]], inv_scale);
            warp_fwht<E>(u, lane);
#pragma unroll
            for (int j = 0; j < E; ++j) u[j] = __fmul_rn(u[j], __fmul_rn(inv_sqrt, sp[j]));
            if (residual_bits > 0) {
                float z[E];
#pragma unroll
                for (int j = 0; j < E; ++j) z[j] = __fmul_rn(t.cr[min(cr_idx[j], t.n_r - 1)], inv_scale);
                warp_fwht<E>(z, lane);
#pragma unroll
                for (int j = 0; j < E; ++j) u[j] = __fadd_rn(u[j], __fmul_rn(z[j], __fmul_rn(inv_sqrt, sr[j])));
            }
        }
#pragma unroll
        for (int j = 0; j < E; ++j) recon[base + j] = u[j];
    }
}

uint32_t fnv1a(const std::vector<uint8_t>& bytes, uint32_t salt) {
    uint32_t h = 2166136261u ^ salt;  // src/quantizer.cpp:18
    for (uint8_t b : bytes) {
        h ^= b;
        h *= 16777619u;
    }
    return h;
}

}  // namespace

void launch_row_norms(const float* d_matrix, float* d_out, long rows, int cols, cudaStream_t stream) {
    if (rows == 0) return;
    row_norm_seq_kernel<<<static_cast<int>((rows + 7) / 8), 256, 0, stream>>>(d_matrix, d_out, rows, cols);
    TQ_CUDA(cudaGetLastError());
}

void derive_seeds(const float* d_weight, size_t n_elems, uint32_t* seed_primary, uint32_t* seed_residual,
                  cudaStream_t stream) {
    const size_t byte_count = n_elems * sizeof(float);
    const size_t stride = byte_count > 4096 ? byte_count / 4096 : 1;  // src/quantizer.cpp:22
    const int n = byte_count ? static_cast<int>((byte_count + stride - 1) / stride) : 0;
    std::vector<uint8_t> sample(n);
    if (n) {
        uint8_t* d_sample = nullptr;
        TQ_CUDA(cudaMalloc(&d_sample, n));
        gather_bytes_kernel<<<(n + 255) / 256, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(d_weight), byte_count,
                                                                 stride, d_sample, n);
        cudaError_t e = cudaMemcpyAsync(sample.data(), d_sample, n, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        cudaFree(d_sample);
        TQ_CUDA(e);
    }
    *seed_primary = fnv1a(sample, 0u);
    *seed_residual = fnv1a(sample, 1u);
}

void launch_quantize_weight(const float* d_weight, long out, int in, const float* cb_p, int n_p, const float* cb_r,
                            int n_r, int primary_bits, int residual_bits, uint32_t block, bool shared_rotation,
                            uint32_t seed_p, uint32_t seed_r, uint8_t* d_packed_primary, uint8_t* d_packed_residual,
                            float* d_norms, float* d_orig_norm_tmp, float* d_recon_tmp, cudaStream_t stream) {
    TQ_REQUIRE(is_pow2(block) && block >= 32 && block <= 1024, "block_size must be a power of two in [32, 1024]");
    TQ_REQUIRE(in % static_cast<int>(block) == 0, "in_features must be divisible by block_size");
    TQ_REQUIRE(primary_bits >= 1 && primary_bits <= 5 && residual_bits >= 0 && residual_bits <= 4, "bad bit widths");
    TQ_REQUIRE(n_p >= 2 && n_p <= 32 && n_r >= 2 && n_r <= 16, "bad codebook size");
    TQ_REQUIRE(primary_bits > 4 || n_p <= 16, "a primary codebook above 16 entries needs primary_bits = 5");
    if (out == 0) return;
    QuantTables tb{};
    tb.n_p = n_p;
    tb.n_r = n_r;
    for (int i = 0; i < n_p; ++i) tb.cp[i] = cb_p[i];
    for (int i = 0; i < n_r; ++i) tb.cr[i] = cb_r[i];
    for (int i = 0; i + 1 < n_p; ++i) tb.bp[i] = (cb_p[i] + cb_p[i + 1]) * 0.5f;  // src/codebook.cpp:49-57
    for (int i = 0; i + 1 < n_r; ++i) tb.br[i] = (cb_r[i] + cb_r[i + 1]) * 0.5f;
    const float scale = std::sqrt(static_cast<float>(in));  // src/quantizer.cpp:51-52
    const float inv_scale = 1.0f / scale;
    const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(block));
    const int bpr = in / static_cast<int>(block);
    const long total = out * bpr;

    const int norm_grid = static_cast<int>((out + 7) / 8);  // 8 warps (rows) per CTA
    row_norm_seq_kernel<<<norm_grid, 256, 0, stream>>>(d_weight, d_orig_norm_tmp, out, in);
    TQ_CUDA(cudaGetLastError());
    if (residual_bits == 0) TQ_CUDA(cudaMemsetAsync(d_packed_residual, 0, static_cast<size_t>(out) * (in / 2), stream));
    long want = (total + 3) / 4;
    const int grid = static_cast<int>(want < 148L * 16 ? want : 148L * 16);
#define TQ_Q_CASE(EV)                                                                                                 \
    case 32 * EV:                                                                                                     \
        quantize_rows_kernel<EV><<<grid, 128, 0, stream>>>(d_weight, d_orig_norm_tmp, d_packed_primary,               \
                                                           d_packed_residual, d_recon_tmp, out, bpr, seed_p, seed_r,  \
                                                           primary_bits, residual_bits, shared_rotation ? 1 : 0,      \
                                                           scale, inv_scale, inv_sqrt, tb);                           \
        break;
    switch (block) {
        TQ_Q_CASE(1) TQ_Q_CASE(2) TQ_Q_CASE(4) TQ_Q_CASE(8) TQ_Q_CASE(16) TQ_Q_CASE(32)
        default: throw Error("unsupported WHT block size");
    }
#undef TQ_Q_CASE
    TQ_CUDA(cudaGetLastError());
    row_norm_seq_kernel<<<norm_grid, 256, 0, stream>>>(d_recon_tmp, d_norms, out, in);
    TQ_CUDA(cudaGetLastError());
    corrected_norm_kernel<<<static_cast<int>((out + 255) / 256), 256, 0, stream>>>(d_orig_norm_tmp, d_norms, out);
    TQ_CUDA(cudaGetLastError());
}

}  // namespace tq
