// After the q/k/v projection: add the projection's bias (if given), rotate queries and keys (split-half rotary, angles in float32),
// write the queries out and append keys and values to the sequence's cache pages.
//   x' [j]        = x[j] * cos(a_j) - x[j + R/2] * sin(a_j)
//   x' [j + R/2]  = x[j + R/2] * cos(a_j) + x[j] * sin(a_j),   a_j = float(pos) * inv_freq[j],  j < R/2
// R (`rot_dim`) may be smaller than the head size; the remaining components pass through.
// inv_freq == nullptr means no rotation at all (another position encoding did its work before).
#include "common.cuh"

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <typename T>
__global__ void rope_cache_kernel(const T* __restrict__ qkv, const T* __restrict__ bias, int qkv_stride, const int* __restrict__ tok_seq,
                                  const int* __restrict__ tok_pos, const int* __restrict__ slots,
                                  const float* __restrict__ inv_freq, int rot_dim, int n_heads, T* __restrict__ q_out,
                                  KvSite<T> site, int write_cache, int* err) {
    grid_chain_entry();
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

// The same for bfloat16 with rows that 16-byte accesses can address (head size, rotated part and row stride
// multiples of 8 elements when halved): a block takes RC_TOKENS tokens, a thread eight components at a time.
#define RC_TOKENS 4
__global__ void __launch_bounds__(256)
rope_cache_vec_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ bias, int qkv_stride, const int* __restrict__ tok_seq,
                      const int* __restrict__ tok_pos, const int* __restrict__ slots, const float* __restrict__ inv_freq,
                      int rot_dim, int n_heads, bf16* __restrict__ q_out, KvSite<bf16> site, int write_cache, int n_tokens,
                      int* err) {
    grid_chain_entry();
    const int D = site.head_dim, KVH = site.kv_heads;
    const int half = rot_dim / 2, pass = D - rot_dim;
    const int q_width = n_heads * D, kv_width = KVH * D;
    const int t0 = blockIdx.x * RC_TOKENS, n_here = min(RC_TOKENS, n_tokens - t0);
    __shared__ float sin_s[RC_TOKENS][128], cos_s[RC_TOKENS][128];
    __shared__ int pos_s[RC_TOKENS];
    __shared__ long long page_s[RC_TOKENS];  // element offset of the token's page in the cache, -1: nothing to write
    if (threadIdx.x < n_here) {
        const int t = t0 + threadIdx.x, pos = tok_pos[t], slot = slots[tok_seq[t]];
        pos_s[threadIdx.x] = pos;
        long long offset = -1;
        if (write_cache && slot >= 0) {
            const int page = site.table[(long long)slot * site.table_stride + pos / QF_PAGE];
            if (page < 0) atomicOr(err, QF_ERR_NO_PAGE);
            else offset = (long long)page * site.page_elems + (long long)(pos % QF_PAGE) * D;
        }
        page_s[threadIdx.x] = offset;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_here * half; i += blockDim.x) {
        const int k = i / half, j = i % half;
        sincosf((float)pos_s[k] * inv_freq[j], &sin_s[k][j], &cos_s[k][j]);
    }
    __syncthreads();
    auto load8 = [&](const bf16* p, const bf16* b, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            v[2 * e] = f.x;
            v[2 * e + 1] = f.y;
        }
        if (b) {
            const uint4 braw = *reinterpret_cast<const uint4*>(b);
            const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&braw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(bh[e]);
                v[2 * e] += f.x;
                v[2 * e + 1] += f.y;
            }
        }
    };
    auto store8 = [&](bf16* p, const float (&v)[8]) {
        *reinterpret_cast<uint4*>(p) = make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
    };
    // work items per token: groups of eight rotation pairs of q and k heads, then groups of eight components that pass
    // through (the unrotated tail of q and k heads, and the values)
    const int rot_groups = (n_heads + KVH) * (half / 8);
    const int pass_groups = (n_heads + KVH) * (pass / 8) + kv_width / 8;
    const int per_token = rot_groups + pass_groups;
    for (int i = threadIdx.x; i < n_here * per_token; i += blockDim.x) {
        const int k = i / per_token, item = i % per_token, t = t0 + k;
        const bf16* row = qkv + (size_t)t * qkv_stride;
        const long long cache_off = page_s[k];
        if (item < rot_groups) {
            const int head = item / (half / 8), j = (item % (half / 8)) * 8;
            const bool is_q = head < n_heads;
            const int src = is_q ? head * D : q_width + (head - n_heads) * D;
            float x1[8], x2[8], o1[8], o2[8];
            load8(row + src + j, bias ? bias + src + j : nullptr, x1);
            load8(row + src + j + half, bias ? bias + src + j + half : nullptr, x2);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float s = sin_s[k][j + e], c = cos_s[k][j + e];
                o1[e] = x1[e] * c - x2[e] * s;
                o2[e] = x2[e] * c + x1[e] * s;
            }
            bf16* dst = nullptr;
            if (is_q) dst = q_out + (size_t)t * q_width + head * D;
            else if (cache_off >= 0) dst = site.base + cache_off + (long long)(head - n_heads) * QF_PAGE * D;
            if (dst) {
                store8(dst + j, o1);
                store8(dst + j + half, o2);
            }
        } else {
            int rest = item - rot_groups;
            const int head_groups = (n_heads + KVH) * (pass / 8);
            float v[8];
            if (rest < head_groups) {
                const int head = rest / (pass / 8), j = rot_dim + (rest % (pass / 8)) * 8;
                const bool is_q = head < n_heads;
                const int src = is_q ? head * D : q_width + (head - n_heads) * D;
                load8(row + src + j, bias ? bias + src + j : nullptr, v);
                if (is_q) store8(q_out + (size_t)t * q_width + head * D + j, v);
                else if (cache_off >= 0) store8(site.base + cache_off + (long long)(head - n_heads) * QF_PAGE * D + j, v);
            } else if (cache_off >= 0) {
                rest -= head_groups;
                const int c = rest * 8, src = q_width + kv_width + c;  // value component c of the token: head c / D
                load8(row + src, bias ? bias + src : nullptr, v);
                store8(site.base + cache_off + (long long)(KVH + c / D) * QF_PAGE * D + c % D, v);
            }
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
    if (sizeof(T) == 2 && head_dim % 16 == 0 && rot_dim % 16 == 0 && qkv_stride % 8 == 0 && head_dim <= 256 &&
        ((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)base | (uintptr_t)bias) % 16 == 0 && page_elems % 8 == 0) {
        return (int)launch_pdl(rope_cache_vec_kernel, dim3((n_tokens + RC_TOKENS - 1) / RC_TOKENS), dim3(256), 0, stream,
            (const bf16*)qkv, (const bf16*)bias, qkv_stride, tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, (bf16*)q_out,
            KvSite<bf16>{(bf16*)base, table, page_elems, table_stride, kv_heads, head_dim}, write_cache, n_tokens, err);
    }
    return (int)launch_pdl(rope_cache_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (const T*)qkv, (const T*)bias, qkv_stride, tok_seq, tok_pos, slots, inv_freq,
                                                       rot_dim, n_heads, (T*)q_out, site, write_cache, err);
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

// The rotation angles of a step, once for all its layers: table[t][j] = (cos, sin) of tok_pos[t] * inv_freq[j], float32,
// the same expression as in the kernels above.
__global__ void rope_table_kernel(const int* __restrict__ tok_pos, const float* __restrict__ inv_freq, int n_tokens, int half,
                                  float2* __restrict__ table) {
    grid_chain_entry();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens * half) return;
    float sn, c;
    sincosf((float)tok_pos[i / half] * inv_freq[i % half], &sn, &c);
    table[i] = make_float2(c, sn);
}

QF_EXPORT int qf_rope_table(const int* tok_pos, const float* inv_freq, int n_tokens, int half, void* table, cudaStream_t stream) {
    if (n_tokens <= 0 || half <= 0) return 0;
    const long long total = (long long)n_tokens * half;
    return (int)launch_pdl(rope_table_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, tok_pos, inv_freq, n_tokens, half, (float2*)table);
}
