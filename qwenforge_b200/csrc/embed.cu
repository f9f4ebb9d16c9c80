// Row gathers: token embedding into the float32 residual stream, and the gather of the
// rows whose logits are wanted.
#include "common.cuh"

template <typename T>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                    int vocab, int width, int* err) {
    grid_chain_entry();
    const int t = blockIdx.x;
    int id = ids[t];
    const bool bad = id < 0 || id >= vocab;
    if (bad) {
        if (threadIdx.x == 0) atomicOr(err, QF_ERR_TOKEN_RANGE);
        id = 0;
    }
    const T* row = table + (size_t)id * width;
    float* dst = out + (size_t)t * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = bad ? 0.f : Num<T>::to_f(row[c]);
}

// out[r] = hidden[rows[r]] (+ delta[rows[r]]): the residual stream with its pending update, at the wanted rows.
template <typename T>
__global__ void gather_rows_kernel(const float* __restrict__ hidden, const T* __restrict__ delta,
                                   const int* __restrict__ rows, float* __restrict__ out, int n_rows_in, int width,
                                   int* err) {
    grid_chain_entry();
    const int r = blockIdx.x;
    int src = rows[r];
    const bool bad = src < 0 || src >= n_rows_in;
    if (bad) {
        if (threadIdx.x == 0) atomicOr(err, QF_ERR_ROW_RANGE);
        src = 0;
    }
    const float* h = hidden + (size_t)src * width;
    const T* d = delta ? delta + (size_t)src * width : nullptr;
    float* dst = out + (size_t)r * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = h[c];
        if (d) v += Num<T>::to_f(d[c]);
        dst[c] = bad ? 0.f : v;
    }
}

// out[r] = rmsnorm(hidden[rows[r]] + delta[rows[r]]) * weight: the wanted rows of the residual stream with its pending
// update, normalised on the way out (what the output head reads). One block per wanted row; the row is read twice (the
// second time from the cache), so any width is taken. Launched as a programmatic dependent of the kernel before it.
template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_norm_kernel(const float* __restrict__ hidden, const T* __restrict__ delta, const int* __restrict__ rows,
                        const T* __restrict__ weight, T* __restrict__ out, int n_rows_in, int width, float eps, int* err) {
    __shared__ float scratch[33];
    grid_launch_dependents();
    const int r = blockIdx.x;
    int src = rows[r];
    const bool bad = src < 0 || src >= n_rows_in;
    if (bad) src = 0;
    grid_dependency_wait();
    if (bad && threadIdx.x == 0) atomicOr(err, QF_ERR_ROW_RANGE);
    const float* h = hidden + (size_t)src * width;
    const T* d = delta ? delta + (size_t)src * width : nullptr;
    T* dst = out + (size_t)r * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = h[c] + (d ? Num<T>::to_f(d[c]) : 0.f);
        ss += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = h[c] + (d ? Num<T>::to_f(d[c]) : 0.f);
        dst[c] = Num<T>::from_f(bad ? 0.f : v * inv * Num<T>::to_f(weight[c]));
    }
}

template <typename T>
static int gather_norm_launch(const float* hidden, const void* delta, const int* rows, const void* weight, void* out,
                              int n_out, int n_in, int width, float eps, int* err, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    return (int)launch_pdl(gather_rows_norm_kernel<T>, dim3(n_out), dim3(256), 0, stream, hidden, (const T*)delta, rows,
                           (const T*)weight, (T*)out, n_in, width, eps, err);
}

// delta (may be null), weight and out share a dtype (bfloat16 or float32); hidden is float32.
QF_EXPORT int qf_gather_rows_norm(int is_bf16, const float* hidden, const void* delta, const int* rows, const void* weight,
                                  void* out, int n_out, int n_in, int width, float eps, int* err, cudaStream_t stream) {
    return is_bf16 ? gather_norm_launch<bf16>(hidden, delta, rows, weight, out, n_out, n_in, width, eps, err, stream)
                   : gather_norm_launch<float>(hidden, delta, rows, weight, out, n_out, n_in, width, eps, err, stream);
}

template <typename T>
static int embed_launch(const int* ids, const void* table, float* out, int n_tokens, int vocab, int width, int* err,
                        cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    return (int)launch_pdl(embed_gather_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, ids, (const T*)table, out, vocab, width, err);
}

template <typename T>
static int gather_launch(const float* hidden, const void* delta, const int* rows, float* out, int n_out, int n_in,
                         int width, int* err, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    return (int)launch_pdl(gather_rows_kernel<T>, dim3(n_out), dim3(256), 0, stream, hidden, (const T*)delta, rows, out, n_in, width, err);
}

QF_EXPORT int qf_embed_gather(int is_bf16, const int* ids, const void* table, float* out, int n_tokens, int vocab,
                              int width, int* err, cudaStream_t stream) {
    return is_bf16 ? embed_launch<bf16>(ids, table, out, n_tokens, vocab, width, err, stream)
                   : embed_launch<float>(ids, table, out, n_tokens, vocab, width, err, stream);
}

QF_EXPORT int qf_gather_rows(int is_bf16, const float* hidden, const void* delta, const int* rows, float* out,
                             int n_out, int n_in, int width, int* err, cudaStream_t stream) {
    return is_bf16 ? gather_launch<bf16>(hidden, delta, rows, out, n_out, n_in, width, err, stream)
                   : gather_launch<float>(hidden, delta, rows, out, n_out, n_in, width, err, stream);
}
