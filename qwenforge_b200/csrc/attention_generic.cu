// Causal grouped-query attention over the paged cache, for any head size, group size, dtype and any
// mix of query lengths (whole prompts, continuations, single decoded tokens). Plain SIMT float32
// arithmetic: this is the kernel of the true 32-bit path and the fallback of the bf16 path for
// shapes the tensor-core kernels refuse.
//
// One block serves one (sequence, kv head, chunk of the query-head group, tile of query tokens).
// Each warp owns up to ROWS_PER_WARP query rows (a row = one token and one query head) and keeps
// their running maximum, sum and output accumulator in registers. Keys and values are staged
// through shared memory in tiles of 32 positions whose origin is always a multiple of 32, so the
// order of every row's arithmetic depends only on that row's own position and window: results
// are bitwise independent of what else is in the batch and of how the tokens were cut into steps.
//
// Query i at position p sees keys j with max(0, p - window + 1) <= j <= p (window 0: all j <= p).
#include <float.h>

#include "common.cuh"

#define KT 32               // keys per tile
#define WARPS 8
#define ROWS_PER_WARP 4
#define MAX_ROWS (WARPS * ROWS_PER_WARP)
#define MAX_DPL 8           // head_dim <= 32 * MAX_DPL

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, T* __restrict__ out, const int* __restrict__ cu_q,
                         const int* __restrict__ tok_pos, const int* __restrict__ slots, KvSite<T> site, int n_heads,
                         int group_chunk, int tokens_per_tile, float scale, int window, int* err) {
    extern __shared__ float smem[];
    const int D = site.head_dim, G = n_heads / site.kv_heads;
    const int chunks = (G + group_chunk - 1) / group_chunk;
    const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
    const int seq = blockIdx.z;
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    const int tile_tok0 = blockIdx.x * tokens_per_tile;
    if (tile_tok0 >= q_len) return;
    const int n_tok = min(tokens_per_tile, q_len - tile_tok0);
    const int g0 = chunk * group_chunk, n_g = min(group_chunk, G - g0);
    const int n_rows = n_tok * n_g;
    const int slot = slots[seq];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int q_width = n_heads * D;
    const int ldk = D + 1;

    float* q_s = smem;                      // [MAX_ROWS][D]
    float* k_s = q_s + MAX_ROWS * D;        // [KT][D + 1]
    float* v_s = k_s + KT * ldk;            // [KT][D + 1]

    // row r of this block: token tile_tok0 + r / n_g, query head kvh * G + g0 + r % n_g
    if (slot < 0) {  // a padding entry of the batch: defined output, no cache access
        for (int i = threadIdx.x; i < n_rows * D; i += blockDim.x) {
            const int r = i / D, d = i % D;
            const int t = q_begin + tile_tok0 + r / n_g, h = kvh * G + g0 + r % n_g;
            out[(size_t)t * q_width + h * D + d] = Num<T>::from_f(0.f);
        }
        return;
    }
    for (int i = threadIdx.x; i < n_rows * D; i += blockDim.x) {
        const int r = i / D, d = i % D;
        const int t = q_begin + tile_tok0 + r / n_g, h = kvh * G + g0 + r % n_g;
        q_s[r * D + d] = Num<T>::to_f(q[(size_t)t * q_width + h * D + d]);
    }

    // positions of the tile's tokens are consecutive: first_pos .. first_pos + n_tok - 1
    const int first_pos = tok_pos[q_begin + tile_tok0];
    const int last_pos = first_pos + n_tok - 1;
    const int lo_min = window > 0 ? max(0, first_pos - window + 1) : 0;

    float m[ROWS_PER_WARP], l[ROWS_PER_WARP], acc[ROWS_PER_WARP][MAX_DPL];
    int row_pos[ROWS_PER_WARP], row_lo[ROWS_PER_WARP];
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
        m[i] = -FLT_MAX;
        l[i] = 0.f;
#pragma unroll
        for (int dd = 0; dd < MAX_DPL; ++dd) acc[i][dd] = 0.f;
        const int r = warp + i * WARPS;
        row_pos[i] = r < n_rows ? first_pos + r / n_g : -1;
        row_lo[i] = window > 0 ? max(0, row_pos[i] - window + 1) : 0;
    }
    const int dpl = (D + 31) / 32;

    for (int k0 = (lo_min / KT) * KT; k0 <= last_pos; k0 += KT) {
        __syncthreads();  // the previous tile is consumed (and q_s is complete on the first pass)
        // stage keys k0 .. k0+KT-1 that some row may read; zero the rest so that 0 * garbage cannot arise
        for (int i = threadIdx.x; i < KT * D; i += blockDim.x) {
            const int j = i / D, d = i % D, kj = k0 + j;
            float kval = 0.f, vval = 0.f;
            if (kj >= lo_min && kj <= last_pos) {
                const T* kp = kv_row(site, slot, kj, kvh, 0);
                if (kp) {
                    kval = Num<T>::to_f(kp[d]);
                    vval = Num<T>::to_f(kp[(size_t)site.kv_heads * QF_PAGE * D + d]);
                } else if (d == 0) {
                    atomicOr(err, QF_ERR_NO_PAGE);
                }
            }
            k_s[j * ldk + d] = kval;
            v_s[j * ldk + d] = vval;
        }
        __syncthreads();
        const int kj = k0 + lane;
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) {
            const int r = warp + i * WARPS;
            if (r >= n_rows) continue;
            if (k0 > row_pos[i] || k0 + KT <= row_lo[i]) continue;  // no visible key of this tile (warp-uniform)
            const float* qr = q_s + r * D;
            const float* kr = k_s + lane * ldk;
            float s = 0.f;
            for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
            s *= scale;
            const bool visible = kj <= row_pos[i] && kj >= row_lo[i];
            s = visible ? s : -FLT_MAX;
            const float m_new = fmaxf(m[i], warp_max(s));
            const float p = visible ? expf(s - m_new) : 0.f;
            const float alpha = expf(m[i] - m_new);
            l[i] = l[i] * alpha + warp_sum(p);
            m[i] = m_new;
#pragma unroll
            for (int dd = 0; dd < MAX_DPL; ++dd) acc[i][dd] *= alpha;
            for (int j = 0; j < KT; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);  // every lane takes part, then uses it or not
#pragma unroll
                for (int dd = 0; dd < MAX_DPL; ++dd) {
                    const int d = lane + 32 * dd;
                    if (dd < dpl && d < D) acc[i][dd] = fmaf(pj, v_s[j * ldk + d], acc[i][dd]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
        const int r = warp + i * WARPS;
        if (r >= n_rows) continue;
        const int t = q_begin + tile_tok0 + r / n_g, h = kvh * G + g0 + r % n_g;
        const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
        for (int dd = 0; dd < MAX_DPL; ++dd) {
            const int d = lane + 32 * dd;
            if (dd < dpl && d < D) out[(size_t)t * q_width + h * D + d] = Num<T>::from_f(acc[i][dd] * inv);
        }
    }
}

template <typename T>
static int launch(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots, void* base,
                  const int* table, long long page_elems, int table_stride, int kv_heads, int head_dim, int n_heads,
                  int n_seqs, int max_q_len, float scale, int window, int* err, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (head_dim > 32 * MAX_DPL || kv_heads <= 0 || n_heads % kv_heads) return (int)cudaErrorInvalidValue;
    const int G = n_heads / kv_heads;
    const int group_chunk = G < MAX_ROWS ? G : MAX_ROWS;
    const int chunks = (G + group_chunk - 1) / group_chunk;
    int tokens_per_tile = MAX_ROWS / group_chunk;
    if (tokens_per_tile > max_q_len) tokens_per_tile = max_q_len;
    const size_t smem = (size_t)(MAX_ROWS * head_dim + 2 * KT * (head_dim + 1)) * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(attention_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    KvSite<T> site{(T*)base, table, page_elems, table_stride, kv_heads, head_dim};
    dim3 grid((max_q_len + tokens_per_tile - 1) / tokens_per_tile, kv_heads * chunks, n_seqs);
    attention_generic_kernel<T><<<grid, WARPS * 32, smem, stream>>>((const T*)q, (T*)out, cu_q, tok_pos, slots, site,
                                                                    n_heads, group_chunk, tokens_per_tile, scale,
                                                                    window, err);
    return (int)cudaGetLastError();
}

// q, out: [n_tokens][n_heads * head_dim]; cu_q: [n_seqs + 1] first token of each sequence in the flat batch;
// tok_pos: [n_tokens] absolute position of each token; slots: [n_seqs] cache slot of each sequence (-1: padding).
QF_EXPORT int qf_attention_generic(int is_bf16, const void* q, void* out, const int* cu_q, const int* tok_pos,
                                   const int* slots, void* base, const int* table, long long page_elems,
                                   int table_stride, int kv_heads, int head_dim, int n_heads, int n_seqs,
                                   int max_q_len, float scale, int window, int* err, cudaStream_t stream) {
    return is_bf16 ? launch<bf16>(q, out, cu_q, tok_pos, slots, base, table, page_elems, table_stride, kv_heads,
                                  head_dim, n_heads, n_seqs, max_q_len, scale, window, err, stream)
                   : launch<float>(q, out, cu_q, tok_pos, slots, base, table, page_elems, table_stride, kv_heads,
                                   head_dim, n_heads, n_seqs, max_q_len, scale, window, err, stream);
}
