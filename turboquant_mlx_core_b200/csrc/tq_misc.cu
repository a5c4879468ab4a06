// Element-wise dtype conversions used at the API boundary (activations arrive as
// "any float type" and are cast to fp16 first, as src/dequantizer.cpp:691 does).
#include "tq_common.cuh"
#include "tq_kernels.cuh"

namespace tq {

__global__ void f32_to_f16_kernel(const float* __restrict__ in, __half* __restrict__ out, long n) {
    for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x)
        out[i] = __float2half_rn(in[i]);
}
__global__ void f16_to_f32_kernel(const __half* __restrict__ in, float* __restrict__ out, long n) {
    for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x)
        out[i] = __half2float(in[i]);
}

static int grid_for(long n) {
    long want = (n + 255) / 256;
    return static_cast<int>(want < 148L * 8 ? (want < 1 ? 1 : want) : 148L * 8);
}

void launch_f32_to_f16(const float* in, __half* out, long n, cudaStream_t stream) {
    if (n == 0) return;
    f32_to_f16_kernel<<<grid_for(n), 256, 0, stream>>>(in, out, n);
    TQ_CUDA(cudaGetLastError());
}
void launch_f16_to_f32(const __half* in, float* out, long n, cudaStream_t stream) {
    if (n == 0) return;
    f16_to_f32_kernel<<<grid_for(n), 256, 0, stream>>>(in, out, n);
    TQ_CUDA(cudaGetLastError());
}

}  // namespace tq
