// RMSNorm over the float32 residual stream, fused with the residual addition that precedes it:
//   hidden += delta (if delta is given);  out = hidden * rsqrt(mean(hidden^2) + eps) * weight
// The sum of squares, the reciprocal root and the scaling are float32; `out` has the activation type.
#include "common.cuh"

template <typename T>
__global__ void add_rms_norm_kernel(float* __restrict__ hidden, const T* __restrict__ delta,
                                    const T* __restrict__ weight, T* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
    float* h = hidden + (size_t)blockIdx.x * width;
    const T* d = delta ? delta + (size_t)blockIdx.x * width : nullptr;
    T* o = out + (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = h[c];
        if (d) {
            v += Num<T>::to_f(d[c]);
            h[c] = v;
        }
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    // each thread re-reads the columns it wrote itself
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = Num<T>::from_f(h[c] * inv * Num<T>::to_f(weight[c]));
}

template <typename T>
static int launch(float* hidden, const void* delta, const void* weight, void* out, int rows, int width, float eps,
                  cudaStream_t stream) {
    if (rows <= 0) return 0;
    add_rms_norm_kernel<T><<<rows, 256, 0, stream>>>(hidden, (const T*)delta, (const T*)weight, (T*)out, width, eps);
    return (int)cudaGetLastError();
}

QF_EXPORT int qf_add_rms_norm(int is_bf16, float* hidden, const void* delta, const void* weight, void* out, int rows,
                              int width, float eps, cudaStream_t stream) {
    return is_bf16 ? launch<bf16>(hidden, delta, weight, out, rows, width, eps, stream)
                   : launch<float>(hidden, delta, weight, out, rows, width, eps, stream);
}

template <typename T> __global__ void residual_add_kernel(float* __restrict__ hidden, const T* __restrict__ delta, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        hidden[i] += Num<T>::to_f(delta[i]);
}

// hidden += delta over n elements (the residual stream catching up with a pending update).
QF_EXPORT int qf_residual_add(int is_bf16, float* hidden, const void* delta, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    if (is_bf16)
        residual_add_kernel<bf16><<<blocks, 256, 0, stream>>>(hidden, (const bf16*)delta, n);
    else
        residual_add_kernel<float><<<blocks, 256, 0, stream>>>(hidden, (const float*)delta, n);
    return (int)cudaGetLastError();
}
