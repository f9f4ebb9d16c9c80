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

// The same product for 16 rows or fewer (decode steps), where tiles of 64 rows would be mostly padding and a handful of
// blocks would stream all the weights: a block takes 32 weight rows, a thread one weight row and two token rows. Every
// output element is still ONE chain of fused multiply-adds over k = 0 .. K-1 in that order (zeros beyond K add
// nothing), so its bits are those of the kernel above.
#define SN 32
#define SK 64
__global__ void __launch_bounds__(256)
gemm_f32_few_rows_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                         float* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ float w_s[SN][SK + 1];
    __shared__ float a_s[16][SK];
    const int n = threadIdx.x % SN, m0 = threadIdx.x / SN, m1 = m0 + 8;
    const int n0 = blockIdx.x * SN;
    float acc0 = 0.f, acc1 = 0.f;
    for (int k0 = 0; k0 < K; k0 += SK) {
#pragma unroll
        for (int i = 0; i < SN * SK / 256; ++i) {
            const int idx = threadIdx.x + i * 256, r = idx / SK, k = idx % SK;
            w_s[r][k] = (n0 + r < N && k0 + k < K) ? W[(size_t)(n0 + r) * ldw + k0 + k] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 16 * SK / 256; ++i) {
            const int idx = threadIdx.x + i * 256, r = idx / SK, k = idx % SK;
            a_s[r][k] = (r < M && k0 + k < K) ? A[(size_t)r * lda + k0 + k] : 0.f;
        }
        __syncthreads();
#pragma unroll 16
        for (int k = 0; k < SK; ++k) {
            const float w = w_s[n][k];
            acc0 = fmaf(a_s[m0][k], w, acc0);
            acc1 = fmaf(a_s[m1][k], w, acc1);
        }
        __syncthreads();
    }
    if (n0 + n < N) {
        const float b = bias ? bias[n0 + n] : 0.f;
        if (m0 < M) C[(size_t)m0 * ldc + n0 + n] = acc0 + b;
        if (m1 < M) C[(size_t)m1 * ldc + n0 + n] = acc1 + b;
    }
}

QF_EXPORT int qf_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K, int lda,
                          int ldw, int ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M <= 16) {
        gemm_f32_few_rows_kernel<<<(N + SN - 1) / SN, 256, 0, stream>>>(A, W, bias, C, M, N, K, lda, ldw, ldc);
        return (int)cudaGetLastError();
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, W, bias, C, M, N, K, lda, ldw, ldc);
    return (int)cudaGetLastError();
}
