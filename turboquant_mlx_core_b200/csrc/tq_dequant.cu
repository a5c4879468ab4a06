// Weight-side kernels that must reproduce the reference bit for bit:
//   * relayout: the reference's two nibble planes -> one "joint" byte per weight
//     (primary code in the low bits, residual code above it), the layout every other
//     kernel streams;
//   * dequantize: joint codes -> fp32 / fp16 weights in the exact operation order of
//     dequantize_weight_cpu (src/dequantizer.cpp:52-256):
//        (centroid sum) * inv_scale -> butterfly -> * (inv_sqrt*sign) -> * norm.
// Both are pure HBM streams (1 B read per weight; 2 or 4 B written).
#include <cmath>

#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

// ---- relayout ---------------------------------------------------------------------
// 4-bit primary: packed byte k of a row holds codes 2k (low nibble) and 2k+1 (high
// nibble) in both planes (src/quantizer.cpp:33-39).  joint = p | r << 4.
// 5-bit primary: one primary code per byte, residual still nibble-packed (3-bit codes);
// joint = p | r << 5.
__global__ void relayout_kernel(const uint8_t* __restrict__ pp, const uint8_t* __restrict__ pr,
                                uint8_t* __restrict__ joint, long n_pairs, int pairs_per_row, int primary_5bit,
                                unsigned int* __restrict__ flags) {
    const size_t tpr = code_tiles_per_row(2 * pairs_per_row);
    unsigned int any_res = 0, bad = 0;
    for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_pairs;
         i += static_cast<long>(gridDim.x) * blockDim.x) {
        const uint32_t r = pr[i];
        any_res |= r;
        uint32_t j0, j1;
        if (!primary_5bit) {
            const uint32_t p = pp[i];
            j0 = (p & 0x0Fu) | ((r & 0x0Fu) << 4);
            j1 = (p >> 4) | (r & 0xF0u);
        } else {
            const uint32_t p0 = pp[2 * i], p1 = pp[2 * i + 1];
            // a residual code above 7 or a primary code above 31 does not fit the joint byte
            bad |= (r & 0x88u) | ((p0 | p1) & 0xE0u);
            j0 = (p0 & 0x1Fu) | ((r & 0x07u) << 5);
            j1 = (p1 & 0x1Fu) | (((r >> 4) & 0x07u) << 5);
        }
        const long row = i / pairs_per_row;
        const int col = 2 * static_cast<int>(i - row * pairs_per_row);
        *reinterpret_cast<uchar2*>(joint + code_offset(row, col, tpr)) =
            make_uchar2(static_cast<unsigned char>(j0), static_cast<unsigned char>(j1));
    }
    if (__any_sync(0xffffffffu, any_res != 0) && (threadIdx.x & 31) == 0) atomicOr(&flags[0], 1u);
    if (__any_sync(0xffffffffu, bad != 0) && (threadIdx.x & 31) == 0) atomicOr(&flags[1], 1u);
}

void launch_relayout(const uint8_t* packed_primary, const uint8_t* packed_residual, uint8_t* joint, long out, int in,
                     bool primary_5bit, unsigned int* flags, cudaStream_t stream) {
    const long n_pairs = out * (in / 2);
    if (n_pairs == 0) return;
    long want = (n_pairs + 255) / 256;
    int grid = static_cast<int>(want < 148L * 16 ? want : 148L * 16);
    // padding bytes of the tiled layout read as code 0
    TQ_CUDA(cudaMemsetAsync(joint, 0, code_bytes(out, in), stream));
    relayout_kernel<<<grid, 256, 0, stream>>>(packed_primary, packed_residual, joint, n_pairs, in / 2, primary_5bit ? 1 : 0, flags);
    TQ_CUDA(cudaGetLastError());
}

// Inverse of relayout (joint bytes -> the reference's two planes), used when a handle
// built on this device has to hand its codes back in the reference's format.
__global__ void unrelayout_kernel(const uint8_t* __restrict__ joint, uint8_t* __restrict__ pp,
                                  uint8_t* __restrict__ pr, long n_pairs, int pairs_per_row, int primary_5bit) {
    const size_t tpr = code_tiles_per_row(2 * pairs_per_row);
    for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_pairs;
         i += static_cast<long>(gridDim.x) * blockDim.x) {
        const long row = i / pairs_per_row;
        const int col = 2 * static_cast<int>(i - row * pairs_per_row);
        const uchar2 j = *reinterpret_cast<const uchar2*>(joint + code_offset(row, col, tpr));
        if (!primary_5bit) {
            pp[i] = static_cast<uint8_t>((j.x & 0x0F) | ((j.y & 0x0F) << 4));
            pr[i] = static_cast<uint8_t>((j.x >> 4) | (j.y & 0xF0));
        } else {
            pp[2 * i] = j.x & 0x1F;
            pp[2 * i + 1] = j.y & 0x1F;
            pr[i] = static_cast<uint8_t>((j.x >> 5) | ((j.y >> 5) << 4));
        }
    }
}

void launch_unrelayout(const uint8_t* joint, uint8_t* packed_primary, uint8_t* packed_residual, long out, int in,
                       bool primary_5bit, cudaStream_t stream) {
    const long n_pairs = out * (in / 2);
    if (n_pairs == 0) return;
    long want = (n_pairs + 255) / 256;
    int grid = static_cast<int>(want < 148L * 16 ? want : 148L * 16);
    unrelayout_kernel<<<grid, 256, 0, stream>>>(joint, packed_primary, packed_residual, n_pairs, in / 2, primary_5bit ? 1 : 0);
    TQ_CUDA(cudaGetLastError());
}

// ---- dequantize ---------------------------------------------------------------------
// One warp per (row, WHT block).  tables[0..255] is the single-rotation table
// (centroid sums, or primary centroids alone when no residual is present);
// for dual rotation tables[0..255] holds the primary centroid and tables[256..511]
// the residual centroid of each joint byte, and the two chains are rotated with their
// own sign vectors and added before the norm multiply (src/dequantizer.cpp:214-252).
template <int E, typename OutT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ joint, const float* __restrict__ norms,
                                                      const float* __restrict__ tables, OutT* __restrict__ out,
                                                      long rows, int blocks_per_row, uint32_t seed_p, uint32_t seed_r,
                                                      int dual, float inv_scale, float inv_sqrt) {
    __shared__ float lut[512];
    for (int i = threadIdx.x; i < (dual ? 512 : 256); i += blockDim.x) lut[i] = tables[i];
    __syncthreads();

    constexpr int BS = 32 * E;
    const int lane = threadIdx.x & 31;
    const long warp0 = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
    const long total = rows * blocks_per_row;

    float sp[E], sr[E];
#pragma unroll
    for (int j = 0; j < E; ++j) {
        sp[j] = __fmul_rn(inv_sqrt, sign_value(seed_p, static_cast<uint32_t>(lane * E + j)));
        sr[j] = __fmul_rn(inv_sqrt, sign_value(seed_r, static_cast<uint32_t>(lane * E + j)));
    }

    // A warp takes kAhead consecutive blocks per round and requests all their codes (and norms)
    // before it transforms the first one: with one 128-byte request per warp in flight the kernel
    // would be bound by load latency, not bandwidth.
    constexpr int kAhead = 4;
    constexpr int W = (E + 3) / 4;  // 32-bit words of codes per lane and block
    const size_t tiles_per_row = code_tiles_per_row(blocks_per_row * BS);
    for (long blk0 = warp0 * kAhead; blk0 < total; blk0 += n_warps * kAhead) {
        uint32_t raw[kAhead][W];
        float nrm[kAhead];
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const long blk = blk0 + u;
            nrm[u] = 0.f;
#pragma unroll
            for (int k = 0; k < W; ++k) raw[u][k] = 0u;
            if (blk < total) {
                const long row = blk / blocks_per_row;
                const int col = static_cast<int>(blk - row * blocks_per_row) * BS + lane * E;
                const uint8_t* src = joint + code_offset(row, col, tiles_per_row);
                nrm[u] = __ldg(norms + row);
                if constexpr (E >= 16) {
#pragma unroll
                    for (int j = 0; j < E / 16; ++j) {
                        const uint4 t = __ldg(reinterpret_cast<const uint4*>(src) + j);
                        raw[u][4 * j] = t.x; raw[u][4 * j + 1] = t.y; raw[u][4 * j + 2] = t.z; raw[u][4 * j + 3] = t.w;
                    }
                } else if constexpr (E == 8) {
                    const uint2 t = __ldg(reinterpret_cast<const uint2*>(src));
                    raw[u][0] = t.x; raw[u][1] = t.y;
                } else if constexpr (E == 4) {
                    raw[u][0] = __ldg(reinterpret_cast<const uint32_t*>(src));
                } else if constexpr (E == 2) {
                    raw[u][0] = __ldg(reinterpret_cast<const unsigned short*>(src));
                } else {
                    raw[u][0] = src[0];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
        const long blk = blk0 + u;
        if (blk >= total) break;
        uint8_t code[E];
#pragma unroll
        for (int k = 0; k < E; ++k) code[k] = static_cast<uint8_t>(raw[u][k >> 2] >> (8 * (k & 3)));

        const float norm = nrm[u];
        float v[E];
#pragma unroll
        for (int j = 0; j < E; ++j) v[j] = __fmul_rn(lut[code[j]], inv_scale);
        warp_fwht<E>(v, lane);
#pragma unroll
        for (int j = 0; j < E; ++j) v[j] = __fmul_rn(v[j], sp[j]);
        if (dual) {
            float u[E];
#pragma unroll
            for (int j = 0; j < E; ++j) u[j] = __fmul_rn(lut[256 + code[j]], inv_scale);
            warp_fwht<E>(u, lane);
#pragma unroll
            for (int j = 0; j < E; ++j) v[j] = __fadd_rn(v[j], __fmul_rn(u[j], sr[j]));
        }
        OutT* dst = out + blk * BS + lane * E;
        // a lane's E results are contiguous: store them with the widest aligned vector available
        __align__(16) OutT w[E];
#pragma unroll
        for (int j = 0; j < E; ++j) {
            const float f = __fmul_rn(v[j], norm);
            if constexpr (sizeof(OutT) == 4) w[j] = f;
            else w[j] = __float2half_rn(f);
        }
        constexpr int kBytes = E * static_cast<int>(sizeof(OutT));
        if constexpr (kBytes % 16 == 0) {
            if (reinterpret_cast<uintptr_t>(dst) % 16 == 0) {
#pragma unroll
                for (int c = 0; c < kBytes / 16; ++c) reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(w)[c];
                continue;
            }
        } else if constexpr (kBytes == 8) {
            if (reinterpret_cast<uintptr_t>(dst) % 8 == 0) {
                *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(w);
                continue;
            }
        } else if constexpr (kBytes == 4) {
            if (reinterpret_cast<uintptr_t>(dst) % 4 == 0) {
                *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(w);
                continue;
            }
        }
#pragma unroll
        for (int j = 0; j < E; ++j) dst[j] = w[j];
        }
    }
}

// The same for WHT blocks of up to 256 columns with 8 weights per lane: a warp takes 256
// consecutive columns of a row (lane l the columns 8l..8l+7: one 8-byte code load, one 16- or
// 32-byte store), butterfly stages below 8 stay in the lane, the rest are lane exchanges.  Same
// operations on the same operands in the same order as dequant_kernel, hence the same bits, at
// less than half the instructions per weight.
template <typename OutT>
__global__ void __launch_bounds__(256) dequant_wide_kernel(const uint8_t* __restrict__ joint, const float* __restrict__ norms,
                                                           const float* __restrict__ tables, OutT* __restrict__ out,
                                                           long rows, int in, int block, uint32_t seed_p, uint32_t seed_r,
                                                           int dual, float inv_scale, float inv_sqrt) {
    __shared__ float lut[512];
    for (int i = threadIdx.x; i < (dual ? 512 : 256); i += blockDim.x) lut[i] = tables[i];
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const long warp0 = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long n_warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
    const long groups_per_row = (in + 255) / 256;
    const long total = rows * groups_per_row;
    const size_t tiles_per_row = code_tiles_per_row(in);

    // the sign pattern repeats per block and blocks divide 256: it does not depend on the group
    float sp[8], sr[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t idx = static_cast<uint32_t>((8 * lane + j) & (block - 1));
        sp[j] = __fmul_rn(inv_sqrt, sign_value(seed_p, idx));
        sr[j] = __fmul_rn(inv_sqrt, sign_value(seed_r, idx));
    }
    const int lane_steps = block >> 3;  // lanes per WHT block

    auto fwht8 = [&](float (&v)[8], unsigned live) {
#pragma unroll
        for (int h = 1; h < 8; h <<= 1)
#pragma unroll
            for (int i = 0; i < 8; i += 2 * h)
#pragma unroll
                for (int j = i; j < i + h; ++j) {
                    const float a = v[j], b = v[j + h];
                    v[j] = __fadd_rn(a, b);
                    v[j + h] = __fsub_rn(a, b);
                }
        for (int m = 1; m < lane_steps; m <<= 1) {
            const bool upper = (lane & m) != 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float o = __shfl_xor_sync(live, v[j], m);
                v[j] = upper ? __fsub_rn(o, v[j]) : __fadd_rn(v[j], o);
            }
        }
    };

    constexpr int kAhead = 4;
    for (long g0 = warp0 * kAhead; g0 < total; g0 += n_warps * kAhead) {
        uint2 raw[kAhead];
        float nrm[kAhead];
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            raw[u] = make_uint2(0u, 0u);
            nrm[u] = 0.f;
            const long grp = g0 + u;
            if (grp < total) {
                const long row = grp / groups_per_row;
                const int col = static_cast<int>(grp - row * groups_per_row) * 256 + 8 * lane;
                nrm[u] = __ldg(norms + row);
                if (col < in) raw[u] = __ldg(reinterpret_cast<const uint2*>(joint + code_offset(row, col, tiles_per_row)));
            }
        }
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const long grp = g0 + u;
            if (grp >= total) break;
            const long row = grp / groups_per_row;
            const int col = static_cast<int>(grp - row * groups_per_row) * 256 + 8 * lane;
            const unsigned live = __ballot_sync(0xffffffffu, col < in);
            if (col >= in) continue;  // lanes past the row's end (whole blocks: their partners are out too)
            uint32_t code[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) code[k] = ((k < 4 ? raw[u].x : raw[u].y) >> (8 * (k & 3))) & 0xFFu;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(lut[code[j]], inv_scale);
            fwht8(v, live);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(v[j], sp[j]);
            if (dual) {
                float w2[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) w2[j] = __fmul_rn(lut[256 + code[j]], inv_scale);
                fwht8(w2, live);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = __fadd_rn(v[j], __fmul_rn(w2[j], sr[j]));
            }
            OutT* dst = out + row * in + col;
            __align__(16) OutT w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float f = __fmul_rn(v[j], nrm[u]);
                if constexpr (sizeof(OutT) == 4) w[j] = f;
                else w[j] = __float2half_rn(f);
            }
            if (reinterpret_cast<uintptr_t>(dst) % 16 == 0) {
#pragma unroll
                for (int c = 0; c < static_cast<int>(8 * sizeof(OutT) / 16); ++c)
                    reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(w)[c];
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) dst[j] = w[j];
            }
        }
    }
}

template <typename OutT>
static void launch_dequant_t(const uint8_t* joint, const float* norms, const float* tables, OutT* out, long rows, int in,
                             uint32_t block, uint32_t seed_p, uint32_t seed_r, bool dual, cudaStream_t stream) {
    TQ_REQUIRE(is_pow2(block) && block >= 32 && block <= 1024, "WHT block size must be a power of two in [32, 1024]");
    TQ_REQUIRE(in % static_cast<int>(block) == 0, "in_features must be divisible by block_size");
    const int bpr = in / static_cast<int>(block);
    const long total = rows * bpr;
    if (total == 0) return;
    const float inv_scale = 1.0f / std::sqrt(static_cast<float>(in));    // src/dequantizer.cpp:76
    const float inv_sqrt = 1.0f / std::sqrt(static_cast<float>(block));  // src/rotation.cpp:333
    if (block <= 256) {
        const long groups = rows * ((in + 255) / 256);
        const long want_w = (groups + 4 * 8 - 1) / (4 * 8);  // 8 warps per CTA, 4 groups per warp and round
        const int grid_w = static_cast<int>(want_w < 148L * 8 ? (want_w < 1 ? 1 : want_w) : 148L * 8);
        dequant_wide_kernel<OutT><<<grid_w, 256, 0, stream>>>(joint, norms, tables, out, rows, in, static_cast<int>(block),
                                                              seed_p, seed_r, dual ? 1 : 0, inv_scale, inv_sqrt);
        TQ_CUDA(cudaGetLastError());
        return;
    }
    long want = (total + 7) / 8;
    int grid = static_cast<int>(want < 148L * 8 ? want : 148L * 8);
#define TQ_DQ_CASE(EV)                                                                                            \
    case 32 * EV:                                                                                                 \
        dequant_kernel<EV, OutT><<<grid, 256, 0, stream>>>(joint, norms, tables, out, rows, bpr, seed_p, seed_r,  \
                                                           dual ? 1 : 0, inv_scale, inv_sqrt);                    \
        break;
    switch (block) {
        TQ_DQ_CASE(1) TQ_DQ_CASE(2) TQ_DQ_CASE(4) TQ_DQ_CASE(8) TQ_DQ_CASE(16) TQ_DQ_CASE(32)
        default: throw Error("unsupported WHT block size");
    }
#undef TQ_DQ_CASE
    TQ_CUDA(cudaGetLastError());
}

void launch_dequant_f32(const uint8_t* joint, const float* norms, const float* tables, float* out, long rows, int in,
                        uint32_t block, uint32_t seed_p, uint32_t seed_r, bool dual, cudaStream_t stream) {
    launch_dequant_t<float>(joint, norms, tables, out, rows, in, block, seed_p, seed_r, dual, stream);
}
void launch_dequant_f16(const uint8_t* joint, const float* norms, const float* tables, __half* out, long rows, int in,
                        uint32_t block, uint32_t seed_p, uint32_t seed_r, bool dual, cudaStream_t stream) {
    launch_dequant_t<__half>(joint, norms, tables, out, rows, in, block, seed_p, seed_r, dual, stream);
}

}  // namespace tq
