// After the q/k/v projection: add the projection's bias (if given), rotate queries and keys (split-half rotary, angles in float32),
// write the queries out and append keys and values to the sequence's cache pages.
//   x' [j]        = x[j] * cos(a_j) - x[j + R/2] * sin(a_j)
//   x' [j + R/2]  = x[j + R/2] * cos(a_j) + x[j] * sin(a_j),   a_j = float(pos) * inv_freq[j],  j < R/2
// R (`rot_dim`) may be smaller than the head size; the remaining components pass through.
// inv_freq == nullptr means no rotation at all (another position encoding did its work before).
#include "common.cuh"

template <typename T>
__global__ void rope_cache_kernel(const T* __restrict__ qkv, const T* __restrict__ bias, int qkv_stride, const int* __restrict__ tok_seq,
                                  const int* __restrict__ tok_pos, const int* __restrict__ slots,
                                  const float* __restrict__ inv_freq, int rot_dim, int n_heads, T* __restrict__ q_out,
                                  KvSite<T> site, int write_cache, int* err) {
    const int t = blockIdx.x;
    const int D = site.head_dim, KVH = site.kv_heads;
    const int pos = tok_pos[t];
    const int slot = slots[tok_seq[t]];
    const T* row = qkv + (size_t)t * qkv_stride;
    const int half = rot_dim / 2;
    const int pass = D - rot_dim;  // unrotated tail of each head
    const int q_width = n_heads * D, kv_width = KVH * D;

    // cache rows of this token, one pointer per kind; nullptr where nothing is to be written
    const bool cache = write_cache && slot >= 0;
    if (cache && threadIdx.x == 0) {
        if (site.table[(long long)slot * site.table_stride + pos / QF_PAGE] < 0) atomicOr(err, QF_ERR_NO_PAGE);
    }

    // the token's sines and cosines once for all heads
    __shared__ float sin_s[128], cos_s[128];  // rot_dim <= head_dim <= 256
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf((float)pos * inv_freq[j], &sin_s[j], &cos_s[j]);
    __syncthreads();
    // work items: (head, j) rotation pairs of q and k heads, then pass-through and value elements
    const int rot_items = (n_heads + KVH) * half;
    for (int i = threadIdx.x; i < rot_items; i += blockDim.x) {
        const int head = i / half, j = i % half;
        const float s = sin_s[j], c = cos_s[j];
        const bool is_q = head < n_heads;
        const int src = is_q ? head * D : q_width + (head - n_heads) * D;
        float x1 = Num<T>::to_f(row[src + j]), x2 = Num<T>::to_f(row[src + j + half]);
        if (bias) {
            x1 += Num<T>::to_f(bias[src + j]);
            x2 += Num<T>::to_f(bias[src + j + half]);
        }
        const float o1 = x1 * c - x2 * s, o2 = x2 * c + x1 * s;
        if (is_q) {
            T* dst = q_out + (size_t)t * q_width + head * D;
            dst[j] = Num<T>::from_f(o1);
            dst[j + half] = Num<T>::from_f(o2);
        } else if (cache) {
            T* dst = kv_row(site, slot, pos, head - n_heads, 0);
            if (dst) {
                dst[j] = Num<T>::from_f(o1);
                dst[j + half] = Num<T>::from_f(o2);
            }
        }
    }
    // components beyond the rotated part
    const int pass_items = (n_heads + KVH) * pass;
    for (int i = threadIdx.x; i < pass_items; i += blockDim.x) {
        const int head = i / pass, j = rot_dim + i % pass;
        const bool is_q = head < n_heads;
        const int src = is_q ? head * D : q_width + (head - n_heads) * D;
        const T value = bias ? Num<T>::from_f(Num<T>::to_f(row[src + j]) + Num<T>::to_f(bias[src + j])) : row[src + j];
        if (is_q) {
            q_out[(size_t)t * q_width + head * D + j] = value;
        } else if (cache) {
            T* dst = kv_row(site, slot, pos, head - n_heads, 0);
            if (dst) dst[j] = value;
        }
    }
    if (cache) {
        for (int i = threadIdx.x; i < kv_width; i += blockDim.x) {
            T* dst = kv_row(site, slot, pos, i / D, 1);
            const int src = q_width + kv_width + i;
            if (dst) dst[i % D] = bias ? Num<T>::from_f(Num<T>::to_f(row[src]) + Num<T>::to_f(bias[src])) : row[src];
        }
    }
}

template <typename T>
static int launch(const void* qkv, const void* bias, int qkv_stride, const int* tok_seq, const int* tok_pos, const int* slots,
                  const float* inv_freq, int rot_dim, int n_heads, void* q_out, void* base, const int* table,
                  long long page_elems, int table_stride, int kv_heads, int head_dim, int write_cache, int n_tokens,
                  int* err, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    KvSite<T> site{(T*)base, table, page_elems, table_stride, kv_heads, head_dim};
    if (!inv_freq) rot_dim = 0;
    rope_cache_kernel<T><<<n_tokens, 256, 0, stream>>>((const T*)qkv, (const T*)bias, qkv_stride, tok_seq, tok_pos, slots, inv_freq,
                                                       rot_dim, n_heads, (T*)q_out, site, write_cache, err);
    return (int)cudaGetLastError();
}

// qkv: [n_tokens][qkv_stride] with q heads, then k heads, then v heads; bias: [(n_heads + 2 kv_heads) * head_dim] or null; q_out: [n_tokens][n_heads * head_dim].
QF_EXPORT int qf_rope_cache_write(int is_bf16, const void* qkv, const void* bias, int qkv_stride, const int* tok_seq, const int* tok_pos,
                                  const int* slots, const float* inv_freq, int rot_dim, int n_heads, void* q_out,
                                  void* base, const int* table, long long page_elems, int table_stride, int kv_heads,
                                  int head_dim, int write_cache, int n_tokens, int* err, cudaStream_t stream) {
    if (rot_dim < 0 || rot_dim > head_dim || (rot_dim & 1) || rot_dim > 256) return (int)cudaErrorInvalidValue;
    return is_bf16 ? launch<bf16>(qkv, bias, qkv_stride, tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, q_out, base,
                                  table, page_elems, table_stride, kv_heads, head_dim, write_cache, n_tokens, err,
                                  stream)
                   : launch<float>(qkv, bias, qkv_stride, tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, q_out, base,
                                   table, page_elems, table_stride, kv_heads, head_dim, write_cache, n_tokens, err,
                                   stream);
}
