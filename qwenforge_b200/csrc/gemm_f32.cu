// True 32-bit matrix product of the float32 path:  C[M][N] = A[M][K] * W[N][K]^T (+ bias[N]).
// FFMA only, no tensor cores, no TF32. Every output element is one chain of fused multiply-adds
// over k = 0 .. K-1 in that order, whatever M, the tiling or the batch: a row's result is bitwise
// the same however the rows were grouped into calls.
#include "mma.cuh"

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
// blocks would stream all the weights. A block takes 8 * NPT weight rows and all (up to 16) token rows: thread (n, m)
// owns the output elements (n + 8 i, m), each still ONE chain of fused multiply-adds over k = 0 .. K-1 in that order
// (zeros beyond K add nothing), so its bits are those of the kernel above. The chain is what bounds a block (4 cycles
// per k), so products of few weight rows are spread over N / 8 blocks (NPT = 1) and the others give a thread four
// chains (NPT = 4); the next columns of both operands arrive by cp.async, two stages ahead of the multiplication.
#define FR_N 8
#define FR_M 16
#define FR_STAGES 3
template <int NPT, int KC>
__global__ void __launch_bounds__(FR_N * FR_M)
gemm_f32_few_rows_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                         float* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc) {
    constexpr int LD = KC + 4;         // rows 16 bytes apart in the banks: 8 weight rows and 4 token rows read without conflicts
    constexpr int WR = FR_N * NPT;     // weight rows of a block
    __shared__ __align__(16) float w_s[FR_STAGES][WR][LD];
    __shared__ __align__(16) float a_s[FR_STAGES][FR_M][LD];
    const int n = threadIdx.x % FR_N, m = threadIdx.x / FR_N;
    const int n0 = blockIdx.x * WR;
    // whole 16-byte pieces go by cp.async when rows and K allow it; otherwise element by element
    const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) && ((((uintptr_t)A) | ((uintptr_t)W)) % 16 == 0);
    auto fetch = [&](int k0, int buf) {
        if (k0 >= K) return;
        if (vec) {
            for (int i = threadIdx.x; i < (WR + FR_M) * (KC / 4); i += FR_N * FR_M) {
                const int r = i / (KC / 4), k = (i % (KC / 4)) * 4;
                const bool is_w = r < WR;
                const int row = is_w ? n0 + r : r - WR;
                const bool ok = (is_w ? row < N : row < M) && k0 + k < K;
                const float* src = is_w ? W + (size_t)row * ldw + k0 + k : A + (size_t)row * lda + k0 + k;
                cp_async_16(is_w ? &w_s[buf][r][k] : &a_s[buf][r - WR][k], ok ? src : W, ok);
            }
        } else {
            for (int i = threadIdx.x; i < (WR + FR_M) * KC; i += FR_N * FR_M) {
                const int r = i / KC, k = i % KC;
                const bool is_w = r < WR;
                const int row = is_w ? n0 + r : r - WR;
                const bool ok = (is_w ? row < N : row < M) && k0 + k < K;
                const float v = ok ? (is_w ? W[(size_t)row * ldw + k0 + k] : A[(size_t)row * lda + k0 + k]) : 0.f;
                if (is_w) w_s[buf][r][k] = v;
                else a_s[buf][r - WR][k] = v;
            }
        }
    };
    float acc[NPT];
#pragma unroll
    for (int i = 0; i < NPT; ++i) acc[i] = 0.f;
    fetch(0, 0);
    cp_async_commit();
    fetch(KC, 1);
    cp_async_commit();
    for (int k0 = 0, turn = 0; k0 < K; k0 += KC, ++turn) {
        const int buf = turn % FR_STAGES;
        fetch(k0 + 2 * KC, (turn + 2) % FR_STAGES);   // its stage was read two turns ago, before that turn's last barrier
        cp_async_commit();
        cp_async_wait<2>();
        __syncthreads();
#pragma unroll 4
        for (int k = 0; k < KC; k += 4) {
            const float4 a = *reinterpret_cast<const float4*>(&a_s[buf][m][k]);
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
                const float4 w = *reinterpret_cast<const float4*>(&w_s[buf][n + FR_N * i][k]);
                acc[i] = fmaf(a.x, w.x, acc[i]);
                acc[i] = fmaf(a.y, w.y, acc[i]);
                acc[i] = fmaf(a.z, w.z, acc[i]);
                acc[i] = fmaf(a.w, w.w, acc[i]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if (m < M) {
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int col = n0 + n + FR_N * i;
            if (col < N) C[(size_t)m * ldc + col] = acc[i] + (bias ? bias[col] : 0.f);
        }
    }
}

QF_EXPORT int qf_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K, int lda,
                          int ldw, int ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M <= 16) {
        if (N <= 4096) gemm_f32_few_rows_kernel<1, 128><<<(N + 7) / 8, FR_N * FR_M, 0, stream>>>(A, W, bias, C, M, N, K, lda, ldw, ldc);
        else gemm_f32_few_rows_kernel<4, 64><<<(N + 31) / 32, FR_N * FR_M, 0, stream>>>(A, W, bias, C, M, N, K, lda, ldw, ldc);
        return (int)cudaGetLastError();
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, W, bias, C, M, N, K, lda, ldw, ldc);
    return (int)cudaGetLastError();
}
