// Shared device/host helpers for the TurboQuant sm_100a kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace tq {

// ---- errors --------------------------------------------------------------------
// Host code throws; the C boundary catches and turns exceptions into status codes
// plus a thread-local message (no exception crosses the ABI).
struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

inline void cuda_check(cudaError_t e, const char* what, const char* file, int line) {
    if (e != cudaSuccess) {
        throw Error(std::string(what) + ": " + cudaGetErrorString(e) + " (" + file + ":" + std::to_string(line) + ")");
    }
}
#define TQ_CUDA(x) ::tq::cuda_check((x), #x, __FILE__, __LINE__)
#define TQ_REQUIRE(cond, msg)                    \
    do {                                         \
        if (!(cond)) throw ::tq::Error(msg);     \
    } while (0)

// ---- sign hash -----------------------------------------------------------------
// Same integer hash as the reference's make_signs (src/rotation.cpp:32-42): the index
// is the position inside the WHT block, so one sign vector serves every block and row.
__host__ __device__ __forceinline__ bool sign_is_positive(uint32_t seed, uint32_t i) {
    uint32_t h = seed * 2654435761u + i * 2246822519u;
    h ^= h >> 16;
    h *= 0x45d9f3bu;
    h ^= h >> 16;
    return (h & 1u) != 0u;
}
__host__ __device__ __forceinline__ float sign_value(uint32_t seed, uint32_t i) {
    return sign_is_positive(seed, i) ? 1.0f : -1.0f;
}

// QJL key-side sign (src/kv_cache.cpp:249-250): top bit of the un-avalanched hash.
__host__ __device__ __forceinline__ bool qjl_sign_is_positive(uint32_t seed, uint32_t d) {
    uint32_t h = seed * 2654435761u + d * 2246822519u;
    return (h >> 31) != 0u;
}

// Per-layer KV seeds (src/kv_cache.cpp:32-42). which: 1 = K rotation, 2 = V rotation, 3 = QJL.
__host__ __device__ __forceinline__ uint32_t kv_layer_seed(uint32_t layer, uint32_t which) {
    uint32_t h = layer;
    h ^= which + 0x9e3779b9u + (h << 6) + (h >> 2);
    h = (h ^ (h >> 16)) * 0x45d9f3bu;
    h = (h ^ (h >> 16)) * 0x45d9f3bu;
    h ^= h >> 16;
    return h;
}

// ---- warp-level Walsh-Hadamard butterfly -----------------------------------------
// One warp transforms one block of 32*E values; lane l holds elements [l*E, (l+1)*E).
// The add tree is the reference's (src/rotation.cpp:14-25): for h = 1, 2, 4, ... the
// pair (j, j+h) becomes (a+b, a-b) with a the lower index.  Stages h < E stay in
// registers; stages h >= E exchange with lane ^ (h/E).  Only __fadd_rn/__fsub_rn are
// used so nothing can be contracted into an FMA: results are bit-identical to the
// scalar loop.
template <int E>
__device__ __forceinline__ void warp_fwht(float (&v)[E], int lane) {
#pragma unroll
    for (int h = 1; h < E; h <<= 1) {
#pragma unroll
        for (int i = 0; i < E; i += 2 * h) {
#pragma unroll
            for (int j = i; j < i + h; ++j) {
                float a = v[j], b = v[j + h];
                v[j] = __fadd_rn(a, b);
                v[j + h] = __fsub_rn(a, b);
            }
        }
    }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const bool upper = (lane & m) != 0;
#pragma unroll
        for (int j = 0; j < E; ++j) {
            float other = __shfl_xor_sync(0xffffffffu, v[j], m);
            // lower lane: mine + other; upper lane: other - mine  (a is the lower index)
            v[j] = upper ? __fsub_rn(other, v[j]) : __fadd_rn(v[j], other);
        }
    }
}

__host__ __device__ __forceinline__ bool is_pow2(uint32_t v) { return v && !(v & (v - 1)); }

// ---- layout of the weight codes in HBM ------------------------------------------------
// One "joint" byte per weight, stored in tiles of 16 rows x 64 columns (1 KB, rows of a tile
// contiguous, 64 bytes each); tiles are row-major over the matrix, and the matrix is padded with
// zero bytes to whole tiles.  A warp of the decode kernel reads 16 rows x 16 bytes per load: in
// this order that is 2 x 512 contiguous bytes instead of 16 pieces of 64; a row's 64 columns of
// one tile stay contiguous for the row-wise readers (dequantiser, prefill GEMM).
constexpr int kCodeTileRows = 16, kCodeTileCols = 64, kCodeTileBytes = kCodeTileRows * kCodeTileCols;
__host__ __device__ __forceinline__ size_t code_tiles_per_row(int in) { return (static_cast<size_t>(in) + kCodeTileCols - 1) / kCodeTileCols; }
__host__ __device__ __forceinline__ size_t code_bytes(long out, int in) {
    return (static_cast<size_t>(out) + kCodeTileRows - 1) / kCodeTileRows * code_tiles_per_row(in) * kCodeTileBytes;
}
// Byte offset of (row, col); `tiles_per_row` = code_tiles_per_row(in).
__host__ __device__ __forceinline__ size_t code_offset(long row, int col, size_t tiles_per_row) {
    return ((static_cast<size_t>(row) >> 4) * tiles_per_row + (static_cast<size_t>(col) >> 6)) * kCodeTileBytes +
           (static_cast<size_t>(row) & 15) * kCodeTileCols + (static_cast<size_t>(col) & 63);
}

// Report a failure from a kernel.  The status word may live in page-locked HOST memory (so that
// the host reads it without a copy): a plain store followed by a system-scope fence, no atomic.
// Programmatic dependent launch for the small kernels of a decode step: launched with the attribute, a kernel's CTAs are
// set up while the kernel before it is still draining; they wait here until that kernel has completed (and its
// writes are visible) before they touch anything, and let the kernel after them start setting up in turn.
__device__ __forceinline__ void pdl_wait_release() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
}
template <typename Kernel, typename... Args>
inline void launch_pdl(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
}

// Threads of a CTA that normalises one row (the RMSNorm kernel and the row-wise all-reduce tails: the same count, so the
// same order of additions).  A decode step has a handful of rows: the row's latency, not the SM count, is what matters.
constexpr int kRowNormThreads = 1024;

// yr[:] = xr[:] * rsqrt(mean(xr[:]^2) + eps) * w for one row, by the whole CTA (up to 1024 threads, a multiple of 32;
// cols even).  Shared by the RMSNorm kernel and the all-reduce tails that normalise the row they have just summed, so
// the fused and the separate form give the same bits.
__device__ __forceinline__ void rmsnorm_row(const __half* xr, const __half* __restrict__ w, __half* yr, int cols, float eps) {
    float ss = 0.f;
    for (int c = threadIdx.x * 2; c < cols; c += blockDim.x * 2) {
        const float2 v = __half22float2(*reinterpret_cast<const __half2*>(xr + c));
        ss += v.x * v.x + v.y * v.y;
    }
    __shared__ float s_part[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) tot += s_part[i];   // fixed order
    const float scale = rsqrtf(tot / static_cast<float>(cols) + eps);
    for (int c = threadIdx.x * 2; c < cols; c += blockDim.x * 2) {
        const float2 v = __half22float2(*reinterpret_cast<const __half2*>(xr + c));
        const float2 g = __half22float2(*reinterpret_cast<const __half2*>(w + c));
        *reinterpret_cast<__half2*>(yr + c) = __floats2half2_rn(v.x * scale * g.x, v.y * scale * g.y);
    }
}

__device__ __forceinline__ void raise_status(unsigned int* status, unsigned int code) {
    *reinterpret_cast<volatile unsigned int*>(status) = code;
    __threadfence_system();
}

}  // namespace tq
