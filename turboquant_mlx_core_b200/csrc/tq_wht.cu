// Blocked Walsh-Hadamard rotation of an fp32 matrix, bit-identical to the reference's
// CPU route (src/rotation.cpp:291-350):
//   forward: x *= sign; butterfly; x *= 1/sqrt(bs)
//   inverse: butterfly; x *= (1/sqrt(bs) * sign)
// One warp owns one block of bs = 32*E values (E consecutive values per lane), so the
// whole butterfly runs in registers and warp shuffles; global traffic is one read and
// one write of the matrix (HBM-bound, 8 B per element).
#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

template <int E>
__global__ void __launch_bounds__(256) wht_rows_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                       long total_blocks, uint32_t seed, float inv_sqrt, int inverse) {
    const int lane = threadIdx.x & 31;
    const long warp0 = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
    constexpr int BS = 32 * E;

    float sgn[E];
#pragma unroll
    for (int j = 0; j < E; ++j) sgn[j] = sign_value(seed, static_cast<uint32_t>(lane * E + j));

    for (long blk = warp0; blk < total_blocks; blk += n_warps) {
        const float* src = in + blk * BS + lane * E;
        float* dst = out + blk * BS + lane * E;
        float v[E];
        if constexpr (E >= 4) {
#pragma unroll
            for (int j = 0; j < E; j += 4) {
                float4 t = *reinterpret_cast<const float4*>(src + j);
                v[j] = t.x; v[j + 1] = t.y; v[j + 2] = t.z; v[j + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < E; ++j) v[j] = src[j];
        }
        if (!inverse) {
#pragma unroll
            for (int j = 0; j < E; ++j) v[j] = __fmul_rn(v[j], sgn[j]);
        }
        warp_fwht<E>(v, lane);
#pragma unroll
        for (int j = 0; j < E; ++j)
            v[j] = inverse ? __fmul_rn(v[j], __fmul_rn(inv_sqrt, sgn[j])) : __fmul_rn(v[j], inv_sqrt);
        if constexpr (E >= 4) {
#pragma unroll
            for (int j = 0; j < E; j += 4)
                *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < E; ++j) dst[j] = v[j];
        }
    }
}

void launch_wht_rows(const float* in, float* out, long rows, int cols, uint32_t seed, uint32_t block, bool inverse,
                     cudaStream_t stream) {
    TQ_REQUIRE(is_pow2(block) && block >= 32 && block <= 1024, "WHT block size must be a power of two in [32, 1024]");
    TQ_REQUIRE(cols % static_cast<int>(block) == 0, "in_features must be divisible by block_size");
    const long total_blocks = rows * (cols / static_cast<long>(block));
    if (total_blocks == 0) return;
    const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(block));  // src/rotation.cpp:301,333
    const int threads = 256;
    long want = (total_blocks + 7) / 8;
    int grid = static_cast<int>(want < 148L * 8 ? want : 148L * 8);
    if (grid < 1) grid = 1;
#define TQ_WHT_CASE(EV)                                                                                     \
    case 32 * EV:                                                                                           \
        wht_rows_kernel<EV><<<grid, threads, 0, stream>>>(in, out, total_blocks, seed, inv_sqrt, inverse);  \
        break;
    switch (block) {
        TQ_WHT_CASE(1) TQ_WHT_CASE(2) TQ_WHT_CASE(4) TQ_WHT_CASE(8) TQ_WHT_CASE(16) TQ_WHT_CASE(32)
        default: throw Error("unsupported WHT block size");
    }
#undef TQ_WHT_CASE
    TQ_CUDA(cudaGetLastError());
}

}  // namespace tq
