// RMSNorm over the float32 residual stream, fused with the residual addition that precedes it:
//   hidden += delta (if delta is given);  out = hidden * rsqrt(mean(hidden^2) + eps) * weight
// The sum of squares, the reciprocal root and the scaling are float32; `out` has the activation type.
#include "common.cuh"

template <typename T>
__global__ void add_rms_norm_kernel(float* __restrict__ hidden, const T* __restrict__ delta,
                                    const T* __restrict__ weight, T* __restrict__ out, int width, float eps) {
    grid_chain_entry();
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

// The same with 16-byte accesses and the row kept in registers between the two passes: width % 4 == 0 and
// width <= 4 * 4 * blockDim (4096 at 256 threads).
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        uint2 r;
        *reinterpret_cast<__nv_bfloat162*>(&r.x) = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162*>(&r.y) = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

template <typename T>
__global__ void __launch_bounds__(256)
add_rms_norm_vec_kernel(float* __restrict__ hidden, const T* __restrict__ delta, const T* __restrict__ weight,
                        T* __restrict__ out, int width, float eps) {
    grid_chain_entry();
    __shared__ float scratch[33];
    float* h = hidden + (size_t)blockIdx.x * width;
    const T* d = delta ? delta + (size_t)blockIdx.x * width : nullptr;
    T* o = out + (size_t)blockIdx.x * width;
    const int n4 = width / 4;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int c = threadIdx.x + u * 256;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < n4) {
            v[u] = Vec4<float>::load(h + 4 * c);
            if (d) {
                const float4 dv = Vec4<T>::load(d + 4 * c);
                v[u].x += dv.x;
                v[u].y += dv.y;
                v[u].z += dv.z;
                v[u].w += dv.w;
                Vec4<float>::store(h + 4 * c, v[u]);
            }
            ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int c = threadIdx.x + u * 256;
        if (c < n4) {
            const float4 w = Vec4<T>::load(weight + 4 * c);
            Vec4<T>::store(o + 4 * c, make_float4(v[u].x * inv * w.x, v[u].y * inv * w.y, v[u].z * inv * w.z, v[u].w * inv * w.w));
        }
    }
}

// Narrow rows (width <= 1024, a multiple of 4): a warp per row, eight rows per block. The row stays in the lanes'
// registers, the sum of squares needs shuffles only, and a lane has up to eight independent 16-byte loads in flight, where
// a block per row had one load per thread and two block-wide barriers. Which kernel runs depends on the width alone, so a
// row's result does not depend on how many rows the step has.
#define NW_ROWS 8
#define NW_MAX 8   // 16-byte groups per lane
template <typename T>
__global__ void __launch_bounds__(NW_ROWS * 32)
add_rms_norm_warp_kernel(float* __restrict__ hidden, const T* __restrict__ delta, const T* __restrict__ weight,
                         T* __restrict__ out, int rows, int width, float eps) {
    grid_chain_entry();
    const int row = blockIdx.x * NW_ROWS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    float* h = hidden + (size_t)row * width;
    const T* d = delta ? delta + (size_t)row * width : nullptr;
    T* o = out + (size_t)row * width;
    const int n4 = width / 4;
    float4 v[NW_MAX], dv[NW_MAX];
#pragma unroll
    for (int u = 0; u < NW_MAX; ++u) {
        const int c = lane + 32 * u;
        v[u] = c < n4 ? Vec4<float>::load(h + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
        dv[u] = (d && c < n4) ? Vec4<T>::load(d + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < NW_MAX; ++u) {
        const int c = lane + 32 * u;
        if (d && c < n4) {
            v[u].x += dv[u].x;
            v[u].y += dv[u].y;
            v[u].z += dv[u].z;
            v[u].w += dv[u].w;
            Vec4<float>::store(h + 4 * c, v[u]);
        }
        ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)width + eps);
#pragma unroll
    for (int u = 0; u < NW_MAX; ++u) {
        const int c = lane + 32 * u;
        if (c < n4) {
            const float4 w = Vec4<T>::load(weight + 4 * c);
            Vec4<T>::store(o + 4 * c, make_float4(v[u].x * inv * w.x, v[u].y * inv * w.y, v[u].z * inv * w.z, v[u].w * inv * w.w));
        }
    }
}

template <typename T>
static int launch(float* hidden, const void* delta, const void* weight, void* out, int rows, int width, float eps,
                  cudaStream_t stream) {
    if (rows <= 0) return 0;
    const uintptr_t align = (uintptr_t)hidden | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out;
    if (width % 4 == 0 && width <= 4 * 32 * NW_MAX && align % 16 == 0) {
        return (int)launch_pdl(add_rms_norm_warp_kernel<T>, dim3((rows + NW_ROWS - 1) / NW_ROWS), dim3(NW_ROWS * 32), 0, stream, hidden, (const T*)delta, (const T*)weight,
                                                                                              (T*)out, rows, width, eps);
    }
    if (width % 4 == 0 && width <= 4096 && align % 16 == 0) {
        return (int)launch_pdl(add_rms_norm_vec_kernel<T>, dim3(rows), dim3(256), 0, stream, hidden, (const T*)delta, (const T*)weight, (T*)out, width, eps);
    }
    return (int)launch_pdl(add_rms_norm_kernel<T>, dim3(rows), dim3(256), 0, stream, hidden, (const T*)delta, (const T*)weight, (T*)out, width, eps);
}

QF_EXPORT int qf_add_rms_norm(int is_bf16, float* hidden, const void* delta, const void* weight, void* out, int rows,
                              int width, float eps, cudaStream_t stream) {
    return is_bf16 ? launch<bf16>(hidden, delta, weight, out, rows, width, eps, stream)
                   : launch<float>(hidden, delta, weight, out, rows, width, eps, stream);
}

template <typename T> __global__ void residual_add_kernel(float* __restrict__ hidden, const T* __restrict__ delta, long long n) {
    grid_chain_entry();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        hidden[i] += Num<T>::to_f(delta[i]);
}

// hidden += delta over n elements (the residual stream catching up with a pending update).
QF_EXPORT int qf_residual_add(int is_bf16, float* hidden, const void* delta, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long most = (long long)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 8;
    const int blocks = (int)((n + 255) / 256 < most ? (n + 255) / 256 : most);
    if (is_bf16)
        return (int)launch_pdl(residual_add_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, hidden, (const bf16*)delta, n);
    return (int)launch_pdl(residual_add_kernel<float>, dim3(blocks), dim3(256), 0, stream, hidden, (const float*)delta, n);
}
