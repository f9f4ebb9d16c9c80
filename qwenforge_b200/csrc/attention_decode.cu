// Split-K flash decoding over the paged cache (bf16): one new token per sequence attends to its own
// cache; the key range of every (sequence, kv head) is cut into `n_splits` runs of whole pages that
// separate blocks reduce at once, so that a batch of a few sequences still fills the GPU.
//
// A block (4 warps) serves one (sequence, kv head, chunk of up to 16 query heads of the group, split).
// The query heads of the group are the 16 rows of an m16n8k16 tensor-core tile, so keys and values are
// read once for the whole group. Pages (64 positions: 64 x D keys, 64 x D values) stream through shared
// memory with double-buffered cp.async; each warp takes 16 keys of a page: S = Q K^T, online softmax in
// float32 (base-2 exponentials, the scale folded in), O += P V. Warps are merged in shared memory.
// With one split the block writes the output; otherwise it writes (max, sum, O) partials to scratch and
// takes a ticket: the block that draws the last ticket of its (sequence, kv head, chunk) merges all
// partials and resets the ticket counter. No block waits for another.
#include "mma.cuh"

#define DEC_WARPS 4
#define DEC_THREADS (DEC_WARPS * 32)

template <int D>
__global__ void __launch_bounds__(DEC_THREADS)
decode_split_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, const int* __restrict__ cu_q,
                    const int* __restrict__ tok_pos, const int* __restrict__ slots, KvSite<bf16> site, int n_heads,
                    int chunks, float scale_log2, int window, int n_splits, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int* __restrict__ counters, int* err) {
    constexpr int LD = D + 8;           // padded shared-memory row (bf16 elements): conflict-free ldmatrix
    constexpr int KS = D / 16;          // k-steps of Q K^T
    constexpr int NT = D / 8;           // n-tiles of P V
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* k_s = reinterpret_cast<bf16*>(smem_raw);             // [2][64][LD]
    bf16* v_s = k_s + 2 * QF_PAGE * LD;                        // [2][64][LD]
    __shared__ float m_s[DEC_WARPS][16], l_s[DEC_WARPS][16];
    __shared__ int ticket_s;

    const int split = blockIdx.x, seq = blockIdx.z;
    const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
    const int G = n_heads / site.kv_heads;
    const int g0 = chunk * 16, n_g = min(16, G - g0);
    const int head0 = kvh * G + g0;
    const int tok = cu_q[seq];
    const int slot = slots[seq];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int q_width = n_heads * D;
    bf16* out_row = out + (size_t)tok * q_width + (size_t)head0 * D;

    if (slot < 0) {  // padding entry: defined output, no cache access, no ticket
        if (split == 0)
            for (int i = threadIdx.x; i < n_g * D; i += DEC_THREADS) out_row[i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int L = tok_pos[tok] + 1;
    const int lo = window > 0 ? max(0, L - window) : 0;
    const int first_page = lo / QF_PAGE, last_page = (L - 1) / QF_PAGE;
    const int pps = (last_page - first_page + n_splits) / n_splits;  // ceil(pages / splits)
    const int p_begin = first_page + split * pps, p_end = min(p_begin + pps, last_page + 1);

    // Q fragments: row r = lane / 4 (and r + 8) is query head head0 + r; rows beyond the group are zero
    uint32_t qa[KS][4];
    {
        const int r0 = lane >> 2, r1 = r0 + 8, c = 2 * (lane & 3);
        const bf16* q0 = q + (size_t)tok * q_width + (size_t)(head0 + r0) * D;
        const bf16* q1 = q + (size_t)tok * q_width + (size_t)(head0 + r1) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qa[ks][0] = r0 < n_g ? *reinterpret_cast<const uint32_t*>(q0 + 16 * ks + c) : 0u;
            qa[ks][1] = r1 < n_g ? *reinterpret_cast<const uint32_t*>(q1 + 16 * ks + c) : 0u;
            qa[ks][2] = r0 < n_g ? *reinterpret_cast<const uint32_t*>(q0 + 16 * ks + 8 + c) : 0u;
            qa[ks][3] = r1 < n_g ? *reinterpret_cast<const uint32_t*>(q1 + 16 * ks + 8 + c) : 0u;
        }
    }

    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {QF_NEG_BIG, QF_NEG_BIG}, l_run[2] = {0.f, 0.f};

    const int* table_row = site.table + (long long)slot * site.table_stride;
    auto load_page = [&](int page_index, int buf) {
        const int page = table_row[page_index];
        const bool held = page >= 0;
        if (!held && threadIdx.x == 0) atomicOr(err, QF_ERR_NO_PAGE);
        const bf16* kp = site.base + (long long)(held ? page : 0) * site.page_elems + (long long)kvh * QF_PAGE * D;
        const bf16* vp = kp + (long long)site.kv_heads * QF_PAGE * D;
        constexpr int CH = D / 8;  // 16-byte chunks per row
        for (int i = threadIdx.x; i < QF_PAGE * CH; i += DEC_THREADS) {
            const int r = i / CH, c = (i % CH) * 8;
            cp_async_16(k_s + ((size_t)buf * QF_PAGE + r) * LD + c, kp + r * D + c, held);
            cp_async_16(v_s + ((size_t)buf * QF_PAGE + r) * LD + c, vp + r * D + c, held);
        }
    };

    if (p_begin < p_end) load_page(p_begin, 0);
    cp_async_commit();
    for (int p = p_begin; p < p_end; ++p) {
        const int buf = (p - p_begin) & 1;
        if (p + 1 < p_end) load_page(p + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* kb = k_s + (size_t)buf * QF_PAGE * LD;
        const bf16* vb = v_s + (size_t)buf * QF_PAGE * LD;
        const int key0 = p * QF_PAGE + 16 * warp;  // this warp's 16 keys
        if (key0 < L && key0 + 16 > lo) {
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t kf[4];
                ldmatrix_x4(kf, kb + (size_t)(16 * warp + (lane >> 4) * 8 + (lane & 7)) * LD + 16 * ks + ((lane >> 3) & 1) * 8);
                mma_bf16_16816(s[0], qa[ks], kf[0], kf[1]);
                mma_bf16_16816(s[1], qa[ks], kf[2], kf[3]);
            }
            float mx[2] = {QF_NEG_BIG, QF_NEG_BIG};
            bool ok[2][2];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int kj = key0 + 8 * t + 2 * (lane & 3) + e;
                    ok[t][e] = kj >= lo && kj < L;
                    s[t][e] = ok[t][e] ? s[t][e] * scale_log2 : QF_NEG_BIG;
                    s[t][2 + e] = ok[t][e] ? s[t][2 + e] * scale_log2 : QF_NEG_BIG;
                    mx[0] = fmaxf(mx[0], s[t][e]);
                    mx[1] = fmaxf(mx[1], s[t][2 + e]);
                }
            }
            float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                corr[r] = exp2f(m_run[r] - m_new);
                m_run[r] = m_new;
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    s[t][e] = ok[t][e] ? exp2f(s[t][e] - m_run[0]) : 0.f;
                    s[t][2 + e] = ok[t][e] ? exp2f(s[t][2 + e] - m_run[1]) : 0.f;
                    sum[0] += s[t][e];
                    sum[1] += s[t][2 + e];
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
                l_run[r] = l_run[r] * corr[r] + sum[r];
            }
            uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]), pack_bf16(s[1][0], s[1][1]),
                              pack_bf16(s[1][2], s[1][3])};
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, vb + (size_t)(16 * warp + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + 8 * nt + (lane >> 4) * 8);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    o[nt + h][0] *= corr[0];
                    o[nt + h][1] *= corr[0];
                    o[nt + h][2] *= corr[1];
                    o[nt + h][3] *= corr[1];
                }
                mma_bf16_16816(o[nt], pa, vf[0], vf[1]);
                mma_bf16_16816(o[nt + 1], pa, vf[2], vf[3]);
            }
        }
        __syncthreads();  // the buffer may be refilled by the next iteration's prefetch
    }
    cp_async_wait<0>();

    // ---- merge the four warps: common maximum, rescale, add up in shared memory
    if ((lane & 3) == 0) {
        m_s[warp][lane >> 2] = m_run[0];
        m_s[warp][(lane >> 2) + 8] = m_run[1];
    }
    __syncthreads();
    float* o_s = reinterpret_cast<float*>(smem_raw);  // [16][D] float32, over the key buffers (all reads are done)
    float m_all[2], f[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + 8 * r;
        m_all[r] = fmaxf(fmaxf(m_s[0][row], m_s[1][row]), fmaxf(m_s[2][row], m_s[3][row]));
        f[r] = exp2f(m_run[r] - m_all[r]);
    }
    if ((lane & 3) == 0) {
        l_s[warp][lane >> 2] = l_run[0] * f[0];
        l_s[warp][(lane >> 2) + 8] = l_run[1] * f[1];
    }
    for (int w = 0; w < DEC_WARPS; ++w) {
        if (warp == w) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int c = 8 * nt + 2 * (lane & 3), r0 = lane >> 2, r1 = r0 + 8;
                if (w == 0) {
                    o_s[r0 * D + c] = o[nt][0] * f[0];
                    o_s[r0 * D + c + 1] = o[nt][1] * f[0];
                    o_s[r1 * D + c] = o[nt][2] * f[1];
                    o_s[r1 * D + c + 1] = o[nt][3] * f[1];
                } else {
                    o_s[r0 * D + c] += o[nt][0] * f[0];
                    o_s[r0 * D + c + 1] += o[nt][1] * f[0];
                    o_s[r1 * D + c] += o[nt][2] * f[1];
                    o_s[r1 * D + c + 1] += o[nt][3] * f[1];
                }
            }
        }
        __syncthreads();
    }
    // block result: row r: maximum max_w m_s[w][r], sum sum_w l_s[w][r], numerator o_s[r][:]
    if (n_splits == 1) {
        for (int i = threadIdx.x; i < n_g * D; i += DEC_THREADS) {
            const int r = i / D;
            const float l = l_s[0][r] + l_s[1][r] + l_s[2][r] + l_s[3][r];
            out_row[i] = __float2bfloat16_rn(l > 0.f ? o_s[i] / l : 0.f);
        }
        return;
    }
    const size_t part_row0 = ((size_t)seq * n_heads + head0) * n_splits;  // partial index of (row 0, split 0)
    for (int i = threadIdx.x; i < n_g * D; i += DEC_THREADS) {
        const int r = i / D, d = i % D;
        part_o[(part_row0 + (size_t)r * n_splits + split) * D + d] = o_s[i];
    }
    if (threadIdx.x < n_g) {
        const int r = threadIdx.x;
        const float m = fmaxf(fmaxf(m_s[0][r], m_s[1][r]), fmaxf(m_s[2][r], m_s[3][r]));
        const float l = l_s[0][r] + l_s[1][r] + l_s[2][r] + l_s[3][r];
        part_ml[(part_row0 + (size_t)r * n_splits + split) * 2] = m;
        part_ml[(part_row0 + (size_t)r * n_splits + split) * 2 + 1] = l;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket_s = atomicAdd(counters + (size_t)seq * gridDim.y + blockIdx.y, 1);
    __syncthreads();
    if (ticket_s != n_splits - 1) return;
    // the last block of this (sequence, kv head, chunk): every partial is visible now
    __threadfence();
    if (threadIdx.x == 0) counters[(size_t)seq * gridDim.y + blockIdx.y] = 0;
    // (max, sum) of every (row, split) into shared memory with independent loads, then one warp per row turns
    // them into weights exp2(m - M) and the row's denominator
    float2* ml_s = reinterpret_cast<float2*>(smem_raw);  // [n_g][n_splits]; o_s has been written out above
    __syncthreads();
    for (int i = threadIdx.x; i < n_g * n_splits; i += DEC_THREADS)
        ml_s[i] = __ldcg(reinterpret_cast<const float2*>(part_ml) + part_row0 + i);
    __syncthreads();
    for (int r = warp; r < n_g; r += DEC_WARPS) {
        float m = QF_NEG_BIG;
        for (int sp = lane; sp < n_splits; sp += 32) m = fmaxf(m, ml_s[r * n_splits + sp].x);
        m = warp_max(m);
        float den = 0.f;
        for (int sp = lane; sp < n_splits; sp += 32) {
            const float2 v = ml_s[r * n_splits + sp];
            const float w = exp2f(v.x - m);
            den += w * v.y;
            ml_s[r * n_splits + sp].x = w;
        }
        den = warp_sum(den);
        if (lane == 0) l_s[0][r] = den;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_g * D; i += DEC_THREADS) {
        const int r = i / D, d = i % D;
        const float* po = part_o + (part_row0 + (size_t)r * n_splits) * D + d;
        float num = 0.f;
        for (int sp0 = 0; sp0 < n_splits; sp0 += 8) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = sp0 + j < n_splits ? __ldcg(po + (size_t)(sp0 + j) * D) : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (sp0 + j < n_splits) num += ml_s[r * n_splits + sp0 + j].x * v[j];
        }
        const float den = l_s[0][r];
        out_row[i] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    }
}

template <int D>
static int launch(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots, void* base,
                  const int* table, long long page_elems, int table_stride, int kv_heads, int n_heads, int n_seqs,
                  float scale, int window, int n_splits, float* part_o, float* part_ml, int* counters, int* err,
                  cudaStream_t stream) {
    const int G = n_heads / kv_heads, chunks = (G + 15) / 16;
    const size_t smem = (size_t)4 * QF_PAGE * (D + 8) * sizeof(bf16);
    cudaError_t e = cudaFuncSetAttribute(decode_split_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    KvSite<bf16> site{(bf16*)base, table, page_elems, table_stride, kv_heads, D};
    dim3 grid(n_splits, kv_heads * chunks, n_seqs);
    decode_split_kernel<D><<<grid, DEC_THREADS, smem, stream>>>((const bf16*)q, (bf16*)out, cu_q, tok_pos, slots, site,
                                                                n_heads, chunks, scale * 1.4426950408889634f, window,
                                                                n_splits, part_o, part_ml, counters, err);
    return (int)cudaGetLastError();
}

// Scratch (used when n_splits > 1): part_o float32 [n_seqs * n_heads * n_splits * head_dim], part_ml float32
// [n_seqs * n_heads * n_splits * 2], counters int32 [n_seqs * kv_heads * ceil(group / 16)], zero before the first
// call (the kernel leaves them zero). Returns cudaErrorInvalidValue for a head size without an instantiation.
QF_EXPORT int qf_attention_decode(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots,
                                  void* base, const int* table, long long page_elems, int table_stride, int kv_heads,
                                  int head_dim, int n_heads, int n_seqs, float scale, int window, int n_splits,
                                  float* part_o, float* part_ml, int* counters, int* err, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (kv_heads <= 0 || n_heads % kv_heads || n_splits < 1) return (int)cudaErrorInvalidValue;
#define QF_CASE(DIM)                                                                                                \
    case DIM:                                                                                                       \
        return launch<DIM>(q, out, cu_q, tok_pos, slots, base, table, page_elems, table_stride, kv_heads, n_heads, \
                           n_seqs, scale, window, n_splits, part_o, part_ml, counters, err, stream);
    switch (head_dim) {
        QF_CASE(32)
        QF_CASE(64)
        QF_CASE(96)
        QF_CASE(128)
        default:
            return (int)cudaErrorInvalidValue;
    }
#undef QF_CASE
}
