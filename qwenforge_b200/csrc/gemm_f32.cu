// True 32-bit matrix product of the float32 path:  C[M][N] = A[M][K] * W[N][K]^T (+ bias[N]).
// FFMA only, no tensor cores, no TF32. Every output element is one chain of fused multiply-adds
// over k = 0 .. K-1 in that order, whatever M, the tiling or the batch: a row's result is bitwise
// the same however the rows were grouped into calls.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                float* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ float a_s[BK][BM + 1];
    __shared__ float w_s[BK][BN + 1];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k of each operand; 256 threads, 4 elements each
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx / BK, k = idx % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            a_s[k][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
            w_s[k][r] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = a_s[k][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = w_s[k][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty + 16 * i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx + 16 * j;
            if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j] + (bias ? bias[gn] : 0.f);
        }
    }
}

QF_EXPORT int qf_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K, int lda,
                          int ldw, int ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, W, bias, C, M, N, K, lda, ldw, ldc);
    return (int)cudaGetLastError();
}
