// SwiGLU gate of the feed-forward: out[t][i] = silu(gu[t][i]) * gu[t][I + i], silu(x) = x / (1 + exp(-x)),
// evaluated in float32 on the fused [gate | up] projection.
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter, c = i % inter;
        const float g = Num<T>::to_f(gu[t * 2 * inter + c]);
        const float u = Num<T>::to_f(gu[t * 2 * inter + inter + c]);
        out[i] = Num<T>::from_f(g / (1.0f + expf(-g)) * u);
    }
}

// Eight bf16 elements per thread (16-byte loads and stores); needs inter % 8 == 0 and 16-byte aligned rows.
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int inter, size_t total8) {
    grid_chain_entry();
    const int per_row = inter / 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / per_row, c = (i % per_row) * 8;
        const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + c);
        const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + inter + c);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
        uint4 o4;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            o2[j] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + t * inter + c) = o4;
    }
}

QF_EXPORT int qf_swiglu(int is_bf16, const void* gu, void* out, int rows, int inter, cudaStream_t stream) {
    const size_t total = (size_t)rows * inter;
    if (total == 0) return 0;
    const size_t most = (size_t)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 16;  // blocks that a grid-stride loop is given
    const int blocks = (int)((total + 255) / 256 < most ? (total + 255) / 256 : most);
    int code;
    if (is_bf16 && inter % 8 == 0 && ((uintptr_t)gu % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
        const size_t total8 = total / 8;
        const int b8 = (int)((total8 + 255) / 256 < most ? (total8 + 255) / 256 : most);
        code = (int)launch_pdl(swiglu_bf16x8_kernel, dim3(b8), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out, inter, total8);
    } else if (is_bf16)
        code = (int)launch_pdl(swiglu_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out, inter, total);
    else
        code = (int)launch_pdl(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)out, inter, total);
    return code;
}
