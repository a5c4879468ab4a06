// The element-wise glue of a decoder layer around the quantised linears and the compressed-cache
// attention: RMSNorm, rotary position embedding, SwiGLU.  The reference leaves these to MLX
// (mlx::core::fast::rms_norm / rope and plain array arithmetic in the host application); they are here
// so that a whole tensor-parallel decode step can be timed.  fp16 in and out, fp32 arithmetic;
// every kernel is memory-bound (a few bytes per element) and carries the programmatic-launch wait
// so that it can follow the kernels of this library without a launch gap.
#include <cmath>
#include <cstdint>

#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

namespace {

__device__ __forceinline__ void ops_dependency_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
}

// y[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * w      one CTA per row
__global__ void __launch_bounds__(kRowNormThreads) rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ w, __half* __restrict__ y,
                                                      int cols, float eps) {
    ops_dependency_sync();
    rmsnorm_row(x + static_cast<size_t>(blockIdx.x) * cols, w, y + static_cast<size_t>(blockIdx.x) * cols, cols, eps);
}

// Rotary embedding, "rotate half" convention: element i of a head pairs with element i + d/2;
// angle = position * theta^(-2 i / d).  x: [rows, heads, d] in place, positions: [rows].
// A second tensor x2 [rows, heads2, d] (the keys beside the queries) rides in the same launch: pairs beyond x's.
__global__ void __launch_bounds__(128) rope_kernel(__half* __restrict__ x, const int* __restrict__ positions, int heads, int dim,
                                                   float log2_theta, long total_pairs, __half* __restrict__ x2, int heads2, long total_pairs2) {
    ops_dependency_sync();
    const int half = dim >> 1;
    for (long i0 = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total_pairs + total_pairs2;
         i0 += static_cast<long>(gridDim.x) * blockDim.x) {
        const bool second = i0 >= total_pairs;
        const long i = second ? i0 - total_pairs : i0;
        __half* const xb = second ? x2 : x;
        const int hh = second ? heads2 : heads;
        const int p = static_cast<int>(i % half);
        const long vec = i / half;               // (row, head)
        const long row = vec / hh;
        const float inv_freq = exp2f(-log2_theta * (2.0f * static_cast<float>(p) / static_cast<float>(dim)));
        float s, c;
        sincosf(static_cast<float>(positions[row]) * inv_freq, &s, &c);
        __half* v = xb + vec * dim;
        const float a = __half2float(v[p]), b = __half2float(v[p + half]);
        v[p] = __float2half_rn(a * c - b * s);
        v[p + half] = __float2half_rn(b * c + a * s);
    }
}

// act[r, j] = silu(gate_up[r, j]) * gate_up[r, inter + j]      (gate rows first, then up rows)
__global__ void __launch_bounds__(256) swiglu_kernel(const __half* __restrict__ gate_up, __half* __restrict__ act, int inter, long rows) {
    ops_dependency_sync();
    const long total = rows * inter;
    for (long i = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) * 2; i < total; i += static_cast<long>(gridDim.x) * blockDim.x * 2) {
        const long r = i / inter, j = i - r * inter;
        const float2 g = __half22float2(*reinterpret_cast<const __half2*>(gate_up + r * 2 * inter + j));
        const float2 u = __half22float2(*reinterpret_cast<const __half2*>(gate_up + r * 2 * inter + inter + j));
        const float a = g.x / (1.0f + __expf(-g.x)) * u.x, b = g.y / (1.0f + __expf(-g.y)) * u.y;
        *reinterpret_cast<__half2*>(act + i) = __floats2half2_rn(a, b);
    }
}

cudaLaunchConfig_t ops_config(unsigned grid, unsigned block, cudaStream_t stream, cudaLaunchAttribute* attr) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cfg;
}

}  // namespace

void launch_rmsnorm_f16(const __half* x, const __half* weight, __half* y, long rows, int cols, float eps, cudaStream_t stream) {
    TQ_REQUIRE(x && weight && y, "rmsnorm: NULL argument");
    TQ_REQUIRE(cols > 0 && cols % 2 == 0, "rmsnorm: an even number of columns");
    if (rows == 0) return;
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = ops_config(static_cast<unsigned>(rows), kRowNormThreads, stream, attr);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, rmsnorm_kernel, x, weight, y, cols, eps));
}

void launch_rope_f16(__half* x, const int* positions, long rows, int heads, int dim, float theta, cudaStream_t stream) {
    TQ_REQUIRE(x && positions, "rope: NULL argument");
    TQ_REQUIRE(dim > 0 && dim % 2 == 0 && heads > 0 && theta > 1.0f, "rope: bad shape");
    if (rows == 0) return;
    const long pairs = rows * heads * (dim / 2);
    long blocks = (pairs + 127) / 128;
    if (blocks > 1184) blocks = 1184;
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = ops_config(static_cast<unsigned>(blocks), 128, stream, attr);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, rope_kernel, x, positions, heads, dim, std::log2(theta), pairs, static_cast<__half*>(nullptr), 1, 0L));
}

void launch_rope_qk_f16(__half* q, __half* k, const int* positions, long rows, int q_heads, int kv_heads, int dim, float theta,
                        cudaStream_t stream) {
    TQ_REQUIRE(q && k && positions, "rope: NULL argument");
    TQ_REQUIRE(dim > 0 && dim % 2 == 0 && q_heads > 0 && kv_heads > 0 && theta > 1.0f, "rope: bad shape");
    if (rows == 0) return;
    const long pairs_q = rows * q_heads * (dim / 2), pairs_k = rows * kv_heads * (dim / 2);
    long blocks = (pairs_q + pairs_k + 127) / 128;
    if (blocks > 1184) blocks = 1184;
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = ops_config(static_cast<unsigned>(blocks), 128, stream, attr);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, rope_kernel, q, positions, q_heads, dim, std::log2(theta), pairs_q, k, kv_heads, pairs_k));
}

void launch_swiglu_f16(const __half* gate_up, __half* act, long rows, int inter, cudaStream_t stream) {
    TQ_REQUIRE(gate_up && act, "swiglu: NULL argument");
    TQ_REQUIRE(inter > 0 && inter % 2 == 0, "swiglu: an even intermediate size");
    if (rows == 0) return;
    long blocks = (rows * inter / 2 + 255) / 256;
    if (blocks > 1184) blocks = 1184;
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = ops_config(static_cast<unsigned>(blocks), 256, stream, attr);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, swiglu_kernel, gate_up, act, inter, rows));
}

}  // namespace tq
