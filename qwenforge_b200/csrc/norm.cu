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
