// Causal grouped-query flash attention for spans of new tokens over the paged cache (bf16): whole prompts of
// unequal lengths, and continuations whose earlier keys already lie in the cache. The span's own keys were
// written to the cache before this kernel runs, so all keys come from one place.
//
// A block serves 64 consecutive query tokens of one (sequence, query head) with G groups of 4 warps; in a group each
// warp owns 16 rows. Key/value pages (64 positions) of the head's kv head stream through shared memory with
// double-buffered cp.async, G pages per turn, from the first page that any row's window reaches to the page of the
// last row's own position; group g takes every G-th page, so a tile's chain of pages is 1 / G as long (a single
// prompt's last tile walks all of its pages while the SMs have room for more warps). At the end the groups' running
// maxima, sums and outputs of the same rows are merged through shared memory, lane by lane.
// S = Q K^T and O += P V run on the tensor cores (m16n8k16, bf16 in, float32 accumulate); the online softmax
// is float32 with base-2 exponentials (the scale folded in). A query at position p sees keys j with
// max(0, p - window + 1) <= j <= p.
#include "mma.cuh"

#define PF_WARPS 4
#define PF_THREADS (PF_WARPS * 32)
#define PF_BM 64

template <int D, int G>
__global__ void __launch_bounds__(PF_THREADS * G, (D <= 64 ? 4 : 2) / G)
prefill_flash_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, const int* __restrict__ cu_q,
                     const int* __restrict__ tok_pos, const int* __restrict__ slots, KvSite<bf16> site, int n_heads,
                     int n_seqs, int n_tiles, int wave, float scale_log2, int window, int* err) {
    grid_chain_entry();
    constexpr int LD = D + 8;
    constexpr int KS = D / 16;
    constexpr int NT = D / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* k_s = reinterpret_cast<bf16*>(smem_raw);  // [2][G][64][LD]
    bf16* v_s = k_s + 2 * G * QF_PAGE * LD;         // [2][G][64][LD]

    // Which (tile, head, sequence) this block serves. Tiles further down a prompt walk more pages, and the SMs hold
    // several blocks each, so what counts is that the blocks that share an SM have about the same work together:
    // blocks are taken in waves of `wave` (one block per SM), the first wave gets the longest tiles in falling order,
    // the second the next longest in rising order, and so on, so that the block that follows a long tile onto the same
    // SM is a short one.
    const int total = (int)gridDim.x, w = blockIdx.x / wave, j = blockIdx.x % wave;
    const int in_wave = min(wave, total - w * wave);
    const int item = w * wave + ((w & 1) ? in_wave - 1 - j : j);
    const int per_tile = n_heads * n_seqs;
    const int tile = n_tiles - 1 - item / per_tile, head = (item % per_tile) % n_heads, seq = (item % per_tile) / n_heads;
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    const int row0 = tile * PF_BM;
    if (row0 >= q_len) return;
    const int n_rows = min(PF_BM, q_len - row0);
    const int slot = slots[seq];
    const int lane = threadIdx.x & 31, warp = (threadIdx.x >> 5) % PF_WARPS, group = (threadIdx.x >> 5) / PF_WARPS;
    const int q_width = n_heads * D;
    const int kvh = head / (n_heads / site.kv_heads);

    if (slot < 0) {
        for (int i = threadIdx.x; i < n_rows * D; i += PF_THREADS * G)
            out[(size_t)(q_begin + row0 + i / D) * q_width + (size_t)head * D + i % D] = __float2bfloat16_rn(0.f);
        return;
    }
    const int pos0 = tok_pos[q_begin + row0];             // position of the tile's first row
    const int last_pos = pos0 + n_rows - 1;
    const int lo_min = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int p_begin = lo_min / QF_PAGE, p_end = last_pos / QF_PAGE + 1;

    // this thread's two rows
    const int r[2] = {16 * warp + (lane >> 2), 16 * warp + (lane >> 2) + 8};
    const bool row_ok[2] = {r[0] < n_rows, r[1] < n_rows};
    const int row_pos[2] = {pos0 + r[0], pos0 + r[1]};
    const int row_lo[2] = {window > 0 ? max(0, row_pos[0] - window + 1) : 0, window > 0 ? max(0, row_pos[1] - window + 1) : 0};
    // the warp's rows span positions [warp_first, warp_last]
    const int warp_first = pos0 + 16 * warp, warp_last = min(pos0 + 16 * warp + 15, last_pos);
    const int warp_lo = window > 0 ? max(0, warp_first - window + 1) : 0;
    const bool warp_active = 16 * warp < n_rows;

    uint32_t qa[KS][4];
    {
        const int c = 2 * (lane & 3);
        const bf16* q0 = q + (size_t)(q_begin + row0 + r[0]) * q_width + (size_t)head * D;
        const bf16* q1 = q + (size_t)(q_begin + row0 + r[1]) * q_width + (size_t)head * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qa[ks][0] = row_ok[0] ? *reinterpret_cast<const uint32_t*>(q0 + 16 * ks + c) : 0u;
            qa[ks][1] = row_ok[1] ? *reinterpret_cast<const uint32_t*>(q1 + 16 * ks + c) : 0u;
            qa[ks][2] = row_ok[0] ? *reinterpret_cast<const uint32_t*>(q0 + 16 * ks + 8 + c) : 0u;
            qa[ks][3] = row_ok[1] ? *reinterpret_cast<const uint32_t*>(q1 + 16 * ks + 8 + c) : 0u;
        }
    }
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {QF_NEG_BIG, QF_NEG_BIG}, l_run[2] = {0.f, 0.f};

    const int* table_row = site.table + (long long)slot * site.table_stride;
    // the pages of one turn: page first + g goes to group g's buffer; every thread helps to fetch all of them
    auto load_pages = [&](int first, int buf) {
        for (int gi = 0; gi < G; ++gi) {
            if (first + gi >= p_end) break;
            const int page = table_row[first + gi];
            const bool held = page >= 0;
            if (!held && threadIdx.x == 0) atomicOr(err, QF_ERR_NO_PAGE);
            const bf16* kp = site.base + (long long)(held ? page : 0) * site.page_elems + (long long)kvh * QF_PAGE * D;
            const bf16* vp = kp + (long long)site.kv_heads * QF_PAGE * D;
            constexpr int CH = D / 8;
            for (int i = threadIdx.x; i < QF_PAGE * CH; i += PF_THREADS * G) {
                const int rr = i / CH, c = (i % CH) * 8;
                cp_async_16(k_s + (((size_t)buf * G + gi) * QF_PAGE + rr) * LD + c, kp + rr * D + c, held);
                cp_async_16(v_s + (((size_t)buf * G + gi) * QF_PAGE + rr) * LD + c, vp + rr * D + c, held);
            }
        }
    };

    load_pages(p_begin, 0);
    cp_async_commit();
    for (int first = p_begin, turn = 0; first < p_end; first += G, ++turn) {
        const int buf = turn & 1;
        if (first + G < p_end) load_pages(first + G, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int p = first + group;
        const bf16* kb = k_s + ((size_t)buf * G + group) * QF_PAGE * LD;
        const bf16* vb = v_s + ((size_t)buf * G + group) * QF_PAGE * LD;
        const int key0 = p * QF_PAGE;
        if (p < p_end && warp_active && key0 <= warp_last && key0 + QF_PAGE > warp_lo) {
            float s[8][4];
#pragma unroll
            for (int t = 0; t < 8; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int t2 = 0; t2 < 4; ++t2) {  // 16 keys per ldmatrix.x4
                    uint32_t kf[4];
                    ldmatrix_x4(kf, kb + (size_t)(16 * t2 + (lane >> 4) * 8 + (lane & 7)) * LD + 16 * ks + ((lane >> 3) & 1) * 8);
                    mma_bf16_16816(s[2 * t2], qa[ks], kf[0], kf[1]);
                    mma_bf16_16816(s[2 * t2 + 1], qa[ks], kf[2], kf[3]);
                }
            }
            // a page that every row of the warp sees whole needs no mask
            const bool full = key0 + QF_PAGE - 1 <= warp_first && key0 >= (window > 0 ? max(0, warp_last - window + 1) : 0);
            float corr[2], sum[2] = {0.f, 0.f};
            if (full) {
                // the common case (every page left of the diagonal): no comparisons, one fused multiply-add and one
                // hardware exponential per score
                float mx[2] = {s[0][0], s[0][2]};
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    mx[0] = fmaxf(mx[0], fmaxf(s[t][0], s[t][1]));
                    mx[1] = fmaxf(mx[1], fmaxf(s[t][2], s[t][3]));
                }
                float neg_m[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                    const float m_new = fmaxf(m_run[i], mx[i] * scale_log2);
                    corr[i] = fast_exp2(m_run[i] - m_new);
                    m_run[i] = m_new;
                    neg_m[i] = -m_new;
                }
#pragma unroll
                for (int t = 0; t < 8; ++t) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        s[t][e] = fast_exp2(fmaf(s[t][e], scale_log2, neg_m[0]));
                        s[t][2 + e] = fast_exp2(fmaf(s[t][2 + e], scale_log2, neg_m[1]));
                        sum[0] += s[t][e];
                        sum[1] += s[t][2 + e];
                    }
                }
            } else {
                float mx[2] = {QF_NEG_BIG, QF_NEG_BIG};
#pragma unroll
                for (int t = 0; t < 8; ++t) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int kj = key0 + 8 * t + 2 * (lane & 3) + e;
                        const bool ok0 = kj <= row_pos[0] && kj >= row_lo[0];
                        const bool ok1 = kj <= row_pos[1] && kj >= row_lo[1];
                        s[t][e] = ok0 ? s[t][e] * scale_log2 : QF_NEG_BIG;
                        s[t][2 + e] = ok1 ? s[t][2 + e] * scale_log2 : QF_NEG_BIG;
                        mx[0] = fmaxf(mx[0], s[t][e]);
                        mx[1] = fmaxf(mx[1], s[t][2 + e]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                    const float m_new = fmaxf(m_run[i], mx[i]);
                    corr[i] = fast_exp2(m_run[i] - m_new);
                    m_run[i] = m_new;
                }
#pragma unroll
                for (int t = 0; t < 8; ++t) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        // a masked score is QF_NEG_BIG: its exponential is 0 unless the whole row is masked so far,
                        // in which case the maximum is QF_NEG_BIG too and the difference would be 0
                        s[t][e] = s[t][e] > 0.5f * QF_NEG_BIG ? fast_exp2(s[t][e] - m_run[0]) : 0.f;
                        s[t][2 + e] = s[t][2 + e] > 0.5f * QF_NEG_BIG ? fast_exp2(s[t][2 + e] - m_run[1]) : 0.f;
                        sum[0] += s[t][e];
                        sum[1] += s[t][2 + e];
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
                sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
                l_run[i] = l_run[i] * corr[i] + sum[i];
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                o[nt][0] *= corr[0];
                o[nt][1] *= corr[0];
                o[nt][2] *= corr[1];
                o[nt][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {  // 16 keys per step
                uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                  pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
                for (int nt = 0; nt < NT; nt += 2) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, vb + (size_t)(16 * kk + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + 8 * nt + (lane >> 4) * 8);
                    mma_bf16_16816(o[nt], pa, vf[0], vf[1]);
                    mma_bf16_16816(o[nt + 1], pa, vf[2], vf[3]);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if (G > 1) {
        // ---- merge the groups: a lane of group g > 0 leaves its maxima, sums and outputs where the lane of group 0 with
        // the same rows finds them (the page buffers are free: the loop ended with a block-wide barrier)
        constexpr int PER_LANE = NT * 4 + 4;
        float* merge = reinterpret_cast<float*>(smem_raw);  // [G - 1][PF_WARPS][PER_LANE][32]
        if (group > 0) {
            float* mine = merge + ((size_t)(group - 1) * PF_WARPS + warp) * PER_LANE * 32 + lane;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) mine[(nt * 4 + e) * 32] = o[nt][e];
            mine[(NT * 4 + 0) * 32] = m_run[0];
            mine[(NT * 4 + 1) * 32] = m_run[1];
            mine[(NT * 4 + 2) * 32] = l_run[0];
            mine[(NT * 4 + 3) * 32] = l_run[1];
        }
        __syncthreads();
        if (group > 0) return;
        for (int g = 1; g < G; ++g) {
            const float* theirs = merge + ((size_t)(g - 1) * PF_WARPS + warp) * PER_LANE * 32 + lane;
            float f_mine[2], f_theirs[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float m_other = theirs[(NT * 4 + i) * 32], l_other = theirs[(NT * 4 + 2 + i) * 32];
                const float m_new = fmaxf(m_run[i], m_other);
                f_mine[i] = fast_exp2(m_run[i] - m_new);     // both maxima QF_NEG_BIG (nothing seen): 2^0, sums stay 0
                f_theirs[i] = fast_exp2(m_other - m_new);
                m_run[i] = m_new;
                l_run[i] = l_run[i] * f_mine[i] + l_other * f_theirs[i];
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[nt][e] = o[nt][e] * f_mine[e >> 1] + theirs[(nt * 4 + e) * 32] * f_theirs[e >> 1];
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (!row_ok[i]) continue;
        const float inv = l_run[i] > 0.f ? 1.0f / l_run[i] : 0.f;
        bf16* dst = out + (size_t)(q_begin + row0 + r[i]) * q_width + (size_t)head * D + 2 * (lane & 3);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            *reinterpret_cast<uint32_t*>(dst + 8 * nt) = pack_bf16(o[nt][2 * i] * inv, o[nt][2 * i + 1] * inv);
    }
}

template <int D, int G>
static int launch_groups(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots, KvSite<bf16> site,
                         int n_heads, int n_seqs, int max_q_len, float scale, int window, int* err, cudaStream_t stream) {
    size_t smem = (size_t)4 * G * QF_PAGE * (D + 8) * sizeof(bf16);
    const size_t merge = (size_t)(G - 1) * PF_WARPS * (D / 8 * 4 + 4) * 32 * sizeof(float);
    if (smem < merge) smem = merge;
    cudaError_t e = cudaFuncSetAttribute(prefill_flash_kernel<D, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int n_tiles = (max_q_len + PF_BM - 1) / PF_BM;
    const long long blocks = (long long)n_tiles * n_heads * n_seqs;
    if (blocks > 0x7fffffffll) return (int)cudaErrorInvalidValue;
    return (int)launch_pdl(prefill_flash_kernel<D, G>, dim3((unsigned)blocks), dim3(PF_THREADS * G), smem, stream, (const bf16*)q,
                           (bf16*)out, cu_q, tok_pos, slots, site, n_heads, n_seqs, n_tiles, qf_sm_count(),
                           scale * 1.4426950408889634f, window, err);
}

template <int D>
static int launch(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots, void* base,
                  const int* table, long long page_elems, int table_stride, int kv_heads, int n_heads, int n_seqs,
                  int n_tokens, int max_q_len, int max_kv_len, float scale, int window, int* err, cudaStream_t stream) {
    KvSite<bf16> site{(bf16*)base, table, page_elems, table_stride, kv_heads, D};
    // Two groups of warps per tile when tiles walk many pages and all tiles find room on the SMs at once (a short
    // continuation over a long cache, one prompt of a few thousand tokens): what bounds the kernel then is the longest
    // tile's chain of pages, which two groups halve. With more tiles than room, the SMs are busy anyway and one group
    // per tile wastes nothing. Measured on one prompt of 2,048 tokens, 14 heads of 64 (448 tiles, room for 592): 55.5
    // microseconds with one group, 41.6 with two; 16 heads of 128 (512 tiles, room for 296): 73 against 94.
    // (tiles that hold rows: the grid also has blocks for the rows that shorter sequences lack, which end at once)
    const long long tiles = (long long)min((max_q_len + PF_BM - 1) / PF_BM * n_seqs, n_tokens / PF_BM + n_seqs) * n_heads;
    const int span = window > 0 && window + PF_BM < max_kv_len ? window + PF_BM : max_kv_len;
    const bool split = span >= 8 * QF_PAGE && tiles < (long long)qf_sm_count() * (D <= 64 ? 4 : 2);
    return split ? launch_groups<D, 2>(q, out, cu_q, tok_pos, slots, site, n_heads, n_seqs, max_q_len, scale, window, err, stream)
                 : launch_groups<D, 1>(q, out, cu_q, tok_pos, slots, site, n_heads, n_seqs, max_q_len, scale, window, err, stream);
}

// The arguments of the generic attention kernel, `n_tokens` (the rows of q: all sequences' new tokens) and `max_kv_len`,
// an upper bound of any sequence's length after this step (both only steer how a tile's pages are shared among warps);
// bf16 only. cudaErrorInvalidValue for a head size without an
// instantiation (the caller then uses the generic kernel).
QF_EXPORT int qf_attention_prefill(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots,
                                   void* base, const int* table, long long page_elems, int table_stride, int kv_heads,
                                   int head_dim, int n_heads, int n_seqs, int n_tokens, int max_q_len, int max_kv_len,
                                   float scale, int window, int* err, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (kv_heads <= 0 || n_heads % kv_heads) return (int)cudaErrorInvalidValue;
#define QF_CASE(DIM)                                                                                                 \
    case DIM:                                                                                                        \
        return launch<DIM>(q, out, cu_q, tok_pos, slots, base, table, page_elems, table_stride, kv_heads, n_heads,  \
                           n_seqs, n_tokens, max_q_len, max_kv_len, scale, window, err, stream);
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
