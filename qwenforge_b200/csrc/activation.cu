// SwiGLU gate of the feed-forward: out[t][i] = silu(gu[t][i]) * gu[t][I + i], silu(x) = x / (1 + exp(-x)),
// evaluated in float32 on the fused [gate | up] projection.
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter, c = i % inter;
        const float g = Num<T>::to_f(gu[t * 2 * inter + c]);
        const float u = Num<T>::to_f(gu[t * 2 * inter + inter + c]);
        out[i] = Num<T>::from_f(g / (1.0f + expf(-g)) * u);
    }
}

QF_EXPORT int qf_swiglu(int is_bf16, const void* gu, void* out, int rows, int inter, cudaStream_t stream) {
    const size_t total = (size_t)rows * inter;
    if (total == 0) return 0;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (is_bf16)
        swiglu_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)gu, (bf16*)out, inter, total);
    else
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, (float*)out, inter, total);
    return (int)cudaGetLastError();
}
