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
//
// Steps of one token per sequence (decoding) give only sequences x kv heads blocks, each walking a whole sequence. For
// them the keys are cut into chunks of GEN_CHUNK positions at absolute multiples of GEN_CHUNK: a block per (sequence,
// kv head, chunk) leaves its rows' maximum, sum and unnormalised output in scratch, and a second kernel folds a row's
// chunks in rising order. Which chunks a row has depends on its own position and window only, so the result still
// does not depend on the batch (it differs by rounding from the unsplit kernel's).
#include <float.h>

#include "common.cuh"

#define KT 32               // keys per tile
#define WARPS 8
#define ROWS_PER_WARP 4
#define MAX_ROWS (WARPS * ROWS_PER_WARP)
#define MAX_DPL 8           // head_dim <= 32 * MAX_DPL
#define GEN_CHUNK 256       // keys per block of the split form; a multiple of KT

template <typename T, bool SPLIT>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, T* __restrict__ out, const int* __restrict__ cu_q,
                         const int* __restrict__ tok_pos, const int* __restrict__ slots, KvSite<T> site, int n_heads,
                         int group_chunk, int tokens_per_tile, float scale, int window, float* __restrict__ part_o,
                         float* __restrict__ part_ml, int* err) {
    extern __shared__ float smem[];
    const int D = site.head_dim, G = n_heads / site.kv_heads;
    const int chunks = (G + group_chunk - 1) / group_chunk;
    const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
    const int seq = blockIdx.z;
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    const int tile_tok0 = SPLIT ? 0 : blockIdx.x * tokens_per_tile;   // SPLIT: blockIdx.x is the chunk of keys
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
    if (SPLIT && slot < 0) return;  // the folding kernel writes the zeros
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

    int k_begin = (lo_min / KT) * KT, k_last = last_pos;
    if (SPLIT) {  // this block's chunk of keys; a chunk that no row sees leaves nothing (the fold knows which exist)
        const int c0 = blockIdx.x * GEN_CHUNK;
        if (c0 > last_pos || c0 + GEN_CHUNK <= lo_min) return;
        k_begin = max(k_begin, c0);
        k_last = min(k_last, c0 + GEN_CHUNK - 1);
    }
    for (int k0 = k_begin; k0 <= k_last; k0 += KT) {
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
        if (SPLIT) {
            const size_t at = ((size_t)seq * n_heads + h) * gridDim.x + blockIdx.x;
#pragma unroll
            for (int dd = 0; dd < MAX_DPL; ++dd) {
                const int d = lane + 32 * dd;
                if (dd < dpl && d < D) part_o[at * D + d] = acc[i][dd];
            }
            if (lane == 0) {
                part_ml[at * 2] = m[i];
                part_ml[at * 2 + 1] = l[i];
            }
            continue;
        }
        const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
        for (int dd = 0; dd < MAX_DPL; ++dd) {
            const int d = lane + 32 * dd;
            if (dd < dpl && d < D) out[(size_t)t * q_width + h * D + d] = Num<T>::from_f(acc[i][dd] * inv);
        }
    }
}

// Folds the chunks of every (sequence, head) of a decoding step, in rising order of the keys.
template <typename T>
__global__ void attention_generic_fold_kernel(T* __restrict__ out, const int* __restrict__ cu_q, const int* __restrict__ tok_pos,
                                              const int* __restrict__ slots, int n_heads, int D, int n_chunks, int window,
                                              const float* __restrict__ part_o, const float* __restrict__ part_ml) {
    const int h = blockIdx.x, seq = blockIdx.y, t = cu_q[seq];
    T* o = out + ((size_t)t * n_heads + h) * D;
    if (slots[seq] < 0) {
        for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] = Num<T>::from_f(0.f);
        return;
    }
    const int pos = tok_pos[t], lo = window > 0 ? max(0, pos - window + 1) : 0;
    const size_t row = ((size_t)seq * n_heads + h) * n_chunks;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float m = -FLT_MAX, l = 0.f, a = 0.f;
        for (int c = lo / GEN_CHUNK; c <= pos / GEN_CHUNK; ++c) {
            const float mc = part_ml[(row + c) * 2], lc = part_ml[(row + c) * 2 + 1];
            const float m_new = fmaxf(m, mc);
            const float alpha = expf(m - m_new), beta = expf(mc - m_new);
            l = l * alpha + lc * beta;
            a = a * alpha + part_o[(row + c) * D + d] * beta;
            m = m_new;
        }
        o[d] = Num<T>::from_f(l > 0.f ? a / l : 0.f);
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
    cudaError_t e = cudaFuncSetAttribute(attention_generic_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    KvSite<T> site{(T*)base, table, page_elems, table_stride, kv_heads, head_dim};
    dim3 grid((max_q_len + tokens_per_tile - 1) / tokens_per_tile, kv_heads * chunks, n_seqs);
    attention_generic_kernel<T, false><<<grid, WARPS * 32, smem, stream>>>((const T*)q, (T*)out, cu_q, tok_pos, slots, site,
                                                                           n_heads, group_chunk, tokens_per_tile, scale,
                                                                           window, nullptr, nullptr, err);
    return (int)cudaGetLastError();
}

template <typename T>
static int launch_decode(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots, void* base,
                         const int* table, long long page_elems, int table_stride, int kv_heads, int head_dim, int n_heads,
                         int n_seqs, int max_kv_len, float scale, int window, float* part_o, float* part_ml, int* err,
                         cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (head_dim > 32 * MAX_DPL || kv_heads <= 0 || n_heads % kv_heads || max_kv_len <= 0) return (int)cudaErrorInvalidValue;
    const int G = n_heads / kv_heads;
    const int group_chunk = G < MAX_ROWS ? G : MAX_ROWS;
    const int chunks = (G + group_chunk - 1) / group_chunk;
    const int n_chunks = (max_kv_len + GEN_CHUNK - 1) / GEN_CHUNK;
    const size_t smem = (size_t)(MAX_ROWS * head_dim + 2 * KT * (head_dim + 1)) * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(attention_generic_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    KvSite<T> site{(T*)base, table, page_elems, table_stride, kv_heads, head_dim};
    attention_generic_kernel<T, true><<<dim3(n_chunks, kv_heads * chunks, n_seqs), WARPS * 32, smem, stream>>>(
        (const T*)q, (T*)out, cu_q, tok_pos, slots, site, n_heads, group_chunk, 1, scale, window, part_o, part_ml, err);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    attention_generic_fold_kernel<T><<<dim3(n_heads, n_seqs), 64, 0, stream>>>((T*)out, cu_q, tok_pos, slots, n_heads, head_dim,
                                                                               n_chunks, window, part_o, part_ml);
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

// The same for a step of ONE token per sequence, cut into chunks of keys (see the top of the file). `max_kv_len`: an
// upper bound of any sequence's length after the step; scratch: part_o float32 [n_seqs * n_heads * n_chunks * head_dim],
// part_ml float32 [n_seqs * n_heads * n_chunks * 2] with n_chunks = ceil(max_kv_len / 256).
QF_EXPORT int qf_attention_generic_decode(int is_bf16, const void* q, void* out, const int* cu_q, const int* tok_pos,
                                          const int* slots, void* base, const int* table, long long page_elems,
                                          int table_stride, int kv_heads, int head_dim, int n_heads, int n_seqs,
                                          int max_kv_len, float scale, int window, float* part_o, float* part_ml, int* err,
                                          cudaStream_t stream) {
    return is_bf16 ? launch_decode<bf16>(q, out, cu_q, tok_pos, slots, base, table, page_elems, table_stride, kv_heads,
                                         head_dim, n_heads, n_seqs, max_kv_len, scale, window, part_o, part_ml, err, stream)
                   : launch_decode<float>(q, out, cu_q, tok_pos, slots, base, table, page_elems, table_stride, kv_heads,
                                          head_dim, n_heads, n_seqs, max_kv_len, scale, window, part_o, part_ml, err, stream);
}
