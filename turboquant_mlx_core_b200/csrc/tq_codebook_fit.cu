// Lloyd-Max codebook fit on the device (generate_codebook_from_data, src/codebook.cpp:99-143 and
// 158-267) and the sample extraction of the converter's per-layer fit (src/converter.cpp:291-368).
//
// One iteration = two launches on the same stream, no host round trip:
//   fit_partial_kernel   every thread bins its values by lower_bound over the current boundaries
//                        (a value equal to a boundary goes to the lower bin, as the CPU path of the
//                        reference and quantize() do) into a PRIVATE histogram in shared memory
//                        ([bin][thread]: no atomics, no bank conflicts), sums in double as the
//                        reference's CPU path; the block then folds its 256 histograms in a fixed order
//                        and writes one (sum, count) pair per bin;
//   fit_update_kernel    one warp folds the blocks' pairs in block order, moves each non-empty bin's
//                        centroid to its mean, recomputes the midpoints and raises a "converged" flag
//                        when no centroid moved by 1e-6 or more (src/codebook.cpp:68, 128-131).
// All `iterations` pairs of launches are enqueued at once; launches after convergence return at
// their first instruction.  Results are run-to-run identical (fixed summation orders).
#include <algorithm>
#include <cmath>
#include <cstdint>

#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

constexpr int kFitThreads = 256;
constexpr int kFitMaxBins = 32;
constexpr float kFitShiftThreshold = 1e-6f;   // src/codebook.cpp:68

struct FitState {
    float centroids[kFitMaxBins];
    float boundaries[kFitMaxBins];   // n - 1 used
    int n;
    int converged;
    int iterations_run;
};

__global__ void __launch_bounds__(kFitThreads) fit_partial_kernel(const float* __restrict__ data, long n_values,
                                                                   const FitState* __restrict__ state, double* __restrict__ part_sum,
                                                                   unsigned long long* __restrict__ part_count) {
    if (state->converged) return;
    extern __shared__ __align__(16) unsigned char fit_smem[];
    double* const h_sum = reinterpret_cast<double*>(fit_smem);                                             // [bin][thread]
    unsigned int* const h_cnt = reinterpret_cast<unsigned int*>(fit_smem + sizeof(double) * kFitMaxBins * kFitThreads);
    __shared__ float s_b[kFitMaxBins];
    const int tid = threadIdx.x;
    const int nc = state->n;
    if (tid < kFitMaxBins) s_b[tid] = tid < nc - 1 ? state->boundaries[tid] : INFINITY;
    for (int b = 0; b < nc; ++b) {
        h_sum[b * kFitThreads + tid] = 0.0;
        h_cnt[b * kFitThreads + tid] = 0u;
    }
    __syncthreads();
    // blocks take chunks of 2^14 values in turn; a thread's 32-bit count holds n / (blocks * 256) values
    const long chunk = 1L << 14;
    for (long c0 = static_cast<long>(blockIdx.x) * chunk; c0 < n_values; c0 += static_cast<long>(gridDim.x) * chunk) {
        const long c1 = c0 + chunk < n_values ? c0 + chunk : n_values;
        for (long i = c0 + tid; i < c1; i += kFitThreads) {
            const float x = __ldg(data + i);
            // number of boundaries strictly below x = std::lower_bound's index; the padding is +inf
            int idx = 0;
#pragma unroll
            for (int step = 16; step > 0; step >>= 1)
                if (s_b[idx + step - 1] < x) idx += step;
            if (idx >= nc) idx = nc - 1;
            h_sum[idx * kFitThreads + tid] += static_cast<double>(x);
            h_cnt[idx * kFitThreads + tid] += 1u;
        }
    }
    __syncthreads();
    // fold the 256 private histograms: warp w takes bins w, w + 8, ...; lane l adds threads l, l + 32, ...
    const int lane = tid & 31, warp = tid >> 5;
    for (int b = warp; b < nc; b += kFitThreads / 32) {
        double s = 0.0;
        unsigned long long c = 0;
        for (int t = lane; t < kFitThreads; t += 32) {
            s += h_sum[b * kFitThreads + t];
            c += h_cnt[b * kFitThreads + t];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            s += __shfl_down_sync(0xffffffffu, s, o);
            c += __shfl_down_sync(0xffffffffu, c, o);
        }
        if (lane == 0) {
            part_sum[static_cast<size_t>(blockIdx.x) * kFitMaxBins + b] = s;
            part_count[static_cast<size_t>(blockIdx.x) * kFitMaxBins + b] = c;
        }
    }
}

__global__ void __launch_bounds__(32) fit_update_kernel(FitState* __restrict__ state, const double* __restrict__ part_sum,
                                                        const unsigned long long* __restrict__ part_count, int n_blocks) {
    if (state->converged) return;
    const int b = threadIdx.x;
    const int nc = state->n;
    float shift = 0.f;
    float c_new = b < nc ? state->centroids[b] : 0.f;
    if (b < nc) {
        double s = 0.0;
        unsigned long long c = 0;
        for (int k = 0; k < n_blocks; ++k) {
            s += part_sum[static_cast<size_t>(k) * kFitMaxBins + b];
            c += part_count[static_cast<size_t>(k) * kFitMaxBins + b];
        }
        if (c > 0) {   // an empty bin keeps its centroid
            c_new = static_cast<float>(s / static_cast<double>(c));
            shift = fabsf(c_new - state->centroids[b]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) shift = fmaxf(shift, __shfl_xor_sync(0xffffffffu, shift, o));
    const float c_next = __shfl_down_sync(0xffffffffu, c_new, 1);
    if (b < nc) state->centroids[b] = c_new;
    if (b + 1 < nc) state->boundaries[b] = __fmul_rn(__fadd_rn(c_new, c_next), 0.5f);
    if (b == 0) {
        state->iterations_run += 1;
        if (shift < kFitShiftThreshold) state->converged = 1;
    }
}

// Rotated, scaled samples of a weight matrix and the residuals the shared primary codebook leaves
// (src/converter.cpp:303-357; the arithmetic is the quantiser's, src/quantizer.cpp:43-62, 117-120).
// One warp per (row, WHT block).  residual may be NULL.
struct SampleTables {
    float cp[32], bp[31];
    int n_p;
};

template <int E>
__global__ void __launch_bounds__(128) layer_samples_kernel(const float* __restrict__ w, const float* __restrict__ orig_norm, long rows,
                                                            int blocks_per_row, uint32_t seed_p, float scale, float inv_sqrt,
                                                            const SampleTables tb, float* __restrict__ scaled,
                                                            float* __restrict__ residual) {
    __shared__ SampleTables t;
    if (threadIdx.x == 0) t = tb;
    __syncthreads();
    constexpr int BS = 32 * E;
    const int lane = threadIdx.x & 31;
    const long warp0 = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
    const long total = rows * blocks_per_row;
    const int in = blocks_per_row * BS;
    float sp[E];
#pragma unroll
    for (int j = 0; j < E; ++j) sp[j] = sign_value(seed_p, static_cast<uint32_t>(lane * E + j));
    for (long blk = warp0; blk < total; blk += n_warps) {
        const long row = blk / blocks_per_row;
        const int bcol = static_cast<int>(blk - row * blocks_per_row) * BS + lane * E;
        const size_t base = static_cast<size_t>(row) * in + bcol;
        const float safe = fmaxf(orig_norm[row], 1e-10f);
        float v[E];
#pragma unroll
        for (int j = 0; j < E; ++j) v[j] = __fmul_rn(__fdiv_rn(w[base + j], safe), sp[j]);
        warp_fwht<E>(v, lane);
#pragma unroll
        for (int j = 0; j < E; ++j) {
            v[j] = __fmul_rn(__fmul_rn(v[j], inv_sqrt), scale);
            scaled[base + j] = v[j];
            if (residual != nullptr) {
                int idx = 0;
                for (int i = 0; i < t.n_p - 1; ++i) idx += (t.bp[i] < v[j]) ? 1 : 0;
                residual[base + j] = __fsub_rn(v[j], t.cp[idx]);
            }
        }
    }
}

}  // namespace

// Fits `bits`-bit centroids to d_data[n] starting from init_centroids (2^bits values, ascending).
// centroids_out / boundaries_out: host arrays of 2^bits and 2^bits - 1 floats.  Returns the iterations run.
int launch_codebook_fit(const float* d_data, long n, int bits, int iterations, const float* init_centroids, float* centroids_out,
                        float* boundaries_out, cudaStream_t stream) {
    TQ_REQUIRE(bits >= 1 && bits <= 5, "Unsupported bit width; must be 1-5");
    const int nc = 1 << bits;
    FitState h{};
    h.n = nc;
    for (int i = 0; i < nc; ++i) h.centroids[i] = init_centroids[i];
    for (int i = 0; i + 1 < nc; ++i) h.boundaries[i] = (init_centroids[i] + init_centroids[i + 1]) * 0.5f;
    int run = 0;
    if (n > 0 && iterations > 0) {
        int dev = 0, sms = 148;
        TQ_CUDA(cudaGetDevice(&dev));
        TQ_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        TQ_REQUIRE(n < (1L << 40), "tq_codebook_fit: at most 2^40 samples");
        const long chunks = (n + (1L << 14) - 1) >> 14;
        const int blocks = static_cast<int>(std::min<long>(chunks, 2L * sms));
        const size_t smem = (sizeof(double) + sizeof(unsigned int)) * kFitMaxBins * kFitThreads;
        static bool configured[64] = {false};
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            TQ_CUDA(cudaFuncSetAttribute(fit_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
        FitState* d_state = nullptr;
        double* d_sum = nullptr;
        unsigned long long* d_cnt = nullptr;
        TQ_CUDA(cudaMallocAsync(&d_state, sizeof(FitState), stream));
        TQ_CUDA(cudaMallocAsync(&d_sum, sizeof(double) * kFitMaxBins * blocks, stream));
        TQ_CUDA(cudaMallocAsync(&d_cnt, sizeof(unsigned long long) * kFitMaxBins * blocks, stream));
        TQ_CUDA(cudaMemcpyAsync(d_state, &h, sizeof h, cudaMemcpyHostToDevice, stream));
        for (int it = 0; it < iterations; ++it) {
            fit_partial_kernel<<<blocks, kFitThreads, smem, stream>>>(d_data, n, d_state, d_sum, d_cnt);
            fit_update_kernel<<<1, 32, 0, stream>>>(d_state, d_sum, d_cnt, blocks);
        }
        TQ_CUDA(cudaGetLastError());
        TQ_CUDA(cudaMemcpyAsync(&h, d_state, sizeof h, cudaMemcpyDeviceToHost, stream));
        TQ_CUDA(cudaFreeAsync(d_state, stream));
        TQ_CUDA(cudaFreeAsync(d_sum, stream));
        TQ_CUDA(cudaFreeAsync(d_cnt, stream));
        TQ_CUDA(cudaStreamSynchronize(stream));
        run = h.iterations_run;
    }
    for (int i = 0; i < nc; ++i) centroids_out[i] = h.centroids[i];
    if (boundaries_out)
        for (int i = 0; i + 1 < nc; ++i) boundaries_out[i] = (h.centroids[i] + h.centroids[i + 1]) * 0.5f;   // src/codebook.cpp:135-139
    return run;
}

void launch_layer_samples(const float* d_weight, const float* d_row_norms, long rows, int in, uint32_t block, uint32_t seed_p,
                          const float* primary_centroids, int n_primary, float* d_scaled, float* d_residual, cudaStream_t stream) {
    TQ_REQUIRE(is_pow2(block) && block >= 32 && block <= 1024, "block_size must be a power of two in [32, 1024]");
    TQ_REQUIRE(in % static_cast<int>(block) == 0, "in_features must be divisible by block_size");
    TQ_REQUIRE(n_primary >= 2 && n_primary <= 32, "bad codebook size");
    if (rows == 0) return;
    SampleTables tb{};
    tb.n_p = n_primary;
    for (int i = 0; i < n_primary; ++i) tb.cp[i] = primary_centroids[i];
    for (int i = 0; i + 1 < n_primary; ++i) tb.bp[i] = (primary_centroids[i] + primary_centroids[i + 1]) * 0.5f;
    const float scale = std::sqrt(static_cast<float>(in));
    const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(block));
    const int bpr = in / static_cast<int>(block);
    const long total = rows * bpr;
    const long want = (total + 3) / 4;
    const int grid = static_cast<int>(want < 148L * 16 ? want : 148L * 16);
#define TQ_S_CASE(EV)                                                                                                              \
    case 32 * EV:                                                                                                                  \
        layer_samples_kernel<EV><<<grid, 128, 0, stream>>>(d_weight, d_row_norms, rows, bpr, seed_p, scale, inv_sqrt, tb, d_scaled, \
                                                           d_residual);                                                            \
        break;
    switch (block) {
        TQ_S_CASE(1) TQ_S_CASE(2) TQ_S_CASE(4) TQ_S_CASE(8) TQ_S_CASE(16) TQ_S_CASE(32)
        default: throw Error("unsupported WHT block size");
    }
#undef TQ_S_CASE
    TQ_CUDA(cudaGetLastError());
}

}  // namespace tq
