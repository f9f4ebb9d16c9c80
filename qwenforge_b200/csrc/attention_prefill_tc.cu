// Causal grouped-query flash attention for spans of new tokens over the paged cache on the fifth-generation tensor
// cores (tcgen05), bf16, head sizes 64 and 128. Same contract as the mma.sync kernel of attention_prefill.cu: the
// span's own keys are in the cache already, a query at position p sees keys max(0, p - window + 1) <= j <= p.
//
// A block of 128 threads serves 128 consecutive query tokens of one (sequence, query head); thread t owns query row
// t, which is lane t of the block's tensor memory. Per 64-position page of the head's kv head:
//   S = Q K^T     one thread issues D / 16 products of 128 x 64 x 16 into 64 columns of tensor memory; Q (once)
//                 and the page's keys come by tiled copies of the tensor memory accelerator, 128-byte swizzle
//   softmax       every thread loads its row of S (64 float32) into registers: maximum, base-2 exponentials and sum
//                 need no exchange between threads; the weights go to shared memory as bf16 in the swizzled
//                 K-major layout the tensor cores read
//   PV            four products of 128 x D x 16, the page's values read as they lie (MN-major), into D further columns
//   O             every thread folds its row of PV into its float32 running output, rescaled when the maximum moved
// Keys and values of the next page are on their way while a page is worked on (two stages), and S of the next page
// is issued together with PV, so that it is ready when the threads come back for it. Several blocks share an SM;
// one's exponentials overlap another's products. Every wait on a barrier is bounded: a wait that runs out sets
// QF_ERR_COPY_TIMEOUT, and the block still frees its tensor memory and returns. No copy uses cluster multicast.
#include "tcgen05.cuh"

#define TA_BM 128
#define TA_THREADS 128

template <int D>
__global__ void __launch_bounds__(TA_THREADS)
prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                  bf16* __restrict__ out, const int* __restrict__ cu_q, const int* __restrict__ tok_pos,
                  const int* __restrict__ slots, KvSite<bf16> site, int n_heads, float scale_log2, int window, int* err) {
    constexpr int CB = D / 64;                    // blocks of 64 columns in a row of Q, K or V
    constexpr int Q_BLOCK = TA_BM * 128;          // bytes of one [128][64] block of Q
    constexpr int KV_BLOCK = QF_PAGE * 128;       // bytes of one [64][64] block of a page's keys or values
    constexpr int KV_BYTES = CB * KV_BLOCK;
    constexpr int TMEM_COLS = D == 64 ? 128 : 256;  // S in columns 0..63, PV in columns 64..64 + D - 1
    constexpr int PV_COL = 64;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;                          // [CB][128][64]
    unsigned char* k_s = q_s + CB * Q_BLOCK;            // [2][CB][64][64]
    unsigned char* v_s = k_s + 2 * KV_BYTES;            // [2][CB][64][64]
    unsigned char* p_s = v_s + 2 * KV_BYTES;            // [128][64]
    __shared__ __align__(8) uint64_t bar_q, bar_kv[2], bar_s, bar_pv;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int seq = blockIdx.z, head = blockIdx.y;
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    const int tile = gridDim.x - 1 - blockIdx.x;  // long rows first
    const int row0 = tile * TA_BM;
    if (row0 >= q_len) return;
    const int n_rows = min(TA_BM, q_len - row0);
    const int slot = slots[seq];
    const int t = threadIdx.x, warp = t >> 5;
    const int q_width = n_heads * D;
    const int kvh = head / (n_heads / site.kv_heads);
    bf16* out_row = out + (size_t)(q_begin + row0 + t) * q_width + (size_t)head * D;
    if (slot < 0) {  // padding entry: defined output, no cache access
        if (t < n_rows)
            for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(out_row + c) = make_uint4(0, 0, 0, 0);
        return;
    }
    const int pos0 = tok_pos[q_begin + row0];  // position of the tile's first row; row t is at pos0 + t
    const int last_pos = pos0 + n_rows - 1;
    const int p_begin = (window > 0 ? max(0, pos0 - window + 1) : 0) / QF_PAGE, p_end = last_pos / QF_PAGE + 1;
    const int n_tiles = p_end - p_begin;
    const int row_pos = pos0 + t, row_lo = window > 0 ? max(0, row_pos - window + 1) : 0;
    const int* table_row = site.table + (long long)slot * site.table_stride;

    if (t == 0) {
        mbar_init(&bar_q, 1);
        mbar_init(&bar_kv[0], 1);
        mbar_init(&bar_kv[1], 1);
        mbar_init(&bar_s, 1);
        mbar_init(&bar_pv, 1);
        abort_s = 0;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);

    // ---- what thread 0 does besides owning row 0
    auto fetch_page = [&](int j) {  // keys and values of the j-th page of the run into stage j & 1
        const int stage = j & 1;
        int page = table_row[p_begin + j];
        if (page < 0) {  // a page the sequence does not hold: reported; some held memory is read instead
            atomicOr(err, QF_ERR_NO_PAGE);
            page = 0;
        }
        // row of the cache seen as one matrix [pages * 2 * kv_heads * 64][D]
        const long long k_row = ((long long)page * 2 * site.kv_heads + kvh) * QF_PAGE;
        const long long v_row = k_row + (long long)site.kv_heads * QF_PAGE;
        mbar_expect_tx(&bar_kv[stage], 2 * KV_BYTES);
#pragma unroll
        for (int cb = 0; cb < CB; ++cb) {
            tma_load_2d(k_s + stage * KV_BYTES + cb * KV_BLOCK, &kv_map, cb * 64, (int)k_row, &bar_kv[stage]);
            tma_load_2d(v_s + stage * KV_BYTES + cb * KV_BLOCK, &kv_map, cb * 64, (int)v_row, &bar_kv[stage]);
        }
    };
    auto issue_s = [&](int j) {  // S = Q K^T of page j; false if its keys did not arrive
        if (!mbar_wait(&bar_kv[j & 1], (j >> 1) & 1)) return false;
        tc_fence_after();
        const unsigned char* kb = k_s + (j & 1) * KV_BYTES;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {  // 16 columns = 32 bytes = 2 units of the descriptor's address field
            const uint64_t da = smem_desc_sw128(q_s + (ks / 4) * Q_BLOCK) + 2 * (ks % 4);
            const uint64_t db = smem_desc_sw128(kb + (ks / 4) * KV_BLOCK) + 2 * (ks % 4);
            umma_bf16(tmem, da, db, umma_idesc_bf16(TA_BM, QF_PAGE, false), ks > 0 ? 1u : 0u);
        }
        umma_commit(&bar_s);
        return true;
    };
    auto issue_pv = [&](int j) {  // PV of page j: weights [128][64 keys] K-major, values [64 keys][D] as they lie
        const unsigned char* vb = v_s + (j & 1) * KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < QF_PAGE / 16; ++kk) {  // 16 keys: 32 bytes of a weight row, two 8-row groups of the values
            const uint64_t da = smem_desc_sw128(p_s) + 2 * kk;
            const uint64_t db = smem_desc_mn_sw128(vb + kk * 2048, KV_BLOCK);
            umma_bf16(tmem + PV_COL, da, db, umma_idesc_bf16(TA_BM, D, true), kk > 0 ? 1u : 0u);
        }
        umma_commit(&bar_pv);
    };

    if (t == 0) {
        mbar_expect_tx(&bar_q, CB * Q_BLOCK);
#pragma unroll
        for (int cb = 0; cb < CB; ++cb) tma_load_2d(q_s + cb * Q_BLOCK, &q_map, head * D + cb * 64, q_begin + row0, &bar_q);
        fetch_page(0);
        if (n_tiles > 1) fetch_page(1);
        if (!mbar_wait(&bar_q, 0) || !issue_s(0)) abort_s = 1;
    }

    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    float m_run = QF_NEG_BIG, l_run = 0.f;

    for (int j = 0; j < n_tiles; ++j) {
        if (!mbar_wait(&bar_s, j & 1)) abort_s = 1;
        tc_fence_after();
        float s[QF_PAGE];
        {
            uint32_t raw[32];
            tmem_load_32(lane_base, raw);
#pragma unroll
            for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(raw[i]);
            tmem_load_32(lane_base + 32, raw);
#pragma unroll
            for (int i = 0; i < 32; ++i) s[32 + i] = __uint_as_float(raw[i]);
        }
        const int key0 = (p_begin + j) * QF_PAGE;
        // a page that every row of the block sees whole needs no mask
        const bool full = key0 + QF_PAGE - 1 <= pos0 && key0 >= (window > 0 ? max(0, pos0 + TA_BM - 1 - window + 1) : 0);
        float corr, sum = 0.f;
        if (full) {
            float mx = s[0];
#pragma unroll
            for (int i = 1; i < QF_PAGE; ++i) mx = fmaxf(mx, s[i]);
            const float m_new = fmaxf(m_run, mx * scale_log2);
            corr = fast_exp2(m_run - m_new);
            m_run = m_new;
#pragma unroll
            for (int i = 0; i < QF_PAGE; ++i) {
                s[i] = fast_exp2(fmaf(s[i], scale_log2, -m_new));
                sum += s[i];
            }
        } else {
            float mx = QF_NEG_BIG;
#pragma unroll
            for (int i = 0; i < QF_PAGE; ++i) {
                const int kj = key0 + i;
                s[i] = (kj <= row_pos && kj >= row_lo) ? s[i] * scale_log2 : QF_NEG_BIG;
                mx = fmaxf(mx, s[i]);
            }
            const float m_new = fmaxf(m_run, mx);
            corr = fast_exp2(m_run - m_new);
            m_run = m_new;
#pragma unroll
            for (int i = 0; i < QF_PAGE; ++i) {
                // a masked score is QF_NEG_BIG: its weight is 0 even while the running maximum is QF_NEG_BIG too
                s[i] = s[i] > 0.5f * QF_NEG_BIG ? fast_exp2(s[i] - m_new) : 0.f;
                sum += s[i];
            }
        }
        l_run = l_run * corr + sum;
        // the row of weights, bf16, 16-byte chunk c at chunk position c ^ (row % 8) of the row's 128 bytes
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint4 chunk = make_uint4(pack_bf16(s[8 * c], s[8 * c + 1]), pack_bf16(s[8 * c + 2], s[8 * c + 3]),
                                           pack_bf16(s[8 * c + 4], s[8 * c + 5]), pack_bf16(s[8 * c + 6], s[8 * c + 7]));
            *reinterpret_cast<uint4*>(p_s + t * 128 + ((c ^ (t & 7)) << 4)) = chunk;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor cores read what the threads wrote
        tc_fence_before();
        __syncthreads();  // every row of S has been read, every row of the weights written
        if (abort_s) break;
        if (t == 0) {
            tc_fence_after();
            issue_pv(j);
            if (j + 1 < n_tiles && !issue_s(j + 1)) abort_s = 1;
        }
        if (!mbar_wait(&bar_pv, j & 1)) abort_s = 1;
        tc_fence_after();
        // keys and values of page j have been read: their stage takes the page after next
        if (t == 0 && j + 2 < n_tiles) fetch_page(j + 2);
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t raw[32];
            tmem_load_32(lane_base + PV_COL + c0, raw);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[c0 + i] = fmaf(o[c0 + i], corr, __uint_as_float(raw[i]));
        }
    }
    if (abort_s && t == 0) atomicOr(err, QF_ERR_COPY_TIMEOUT);
    if (t < n_rows && !abort_s) {
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
        for (int c = 0; c < D; c += 8)
            *reinterpret_cast<uint4*>(out_row + c) =
                make_uint4(pack_bf16(o[c] * inv, o[c + 1] * inv), pack_bf16(o[c + 2] * inv, o[c + 3] * inv),
                           pack_bf16(o[c + 4] * inv, o[c + 5] * inv), pack_bf16(o[c + 6] * inv, o[c + 7] * inv));
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32  %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
}

template <int D>
static int launch(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots, void* base,
                  const int* table, long long page_elems, int table_stride, int kv_heads, int n_heads, int n_seqs,
                  int n_tokens, int max_q_len, float scale, int window, int* err, cudaStream_t stream) {
    // the cache pages must be what the map takes them for: [2][kv_heads][64][D] without gaps
    if (page_elems != 2ll * kv_heads * QF_PAGE * D) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)(D / 64) * TA_BM * 128 + 4 * (size_t)(D / 64) * QF_PAGE * 128 + TA_BM * 128 + 1024;
    cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    KvSite<bf16> site{(bf16*)base, table, page_elems, table_stride, kv_heads, D};
    CUtensorMap q_map = {}, kv_map = {};
    const long long q_width = (long long)n_heads * D;
    if (!qf_make_map_bf16(&q_map, q, n_tokens, q_width, q_width, TA_BM)) return (int)cudaErrorNotSupported;
    // The cache of this entry as one matrix of rows of D elements. The map is given more rows than any cache has
    // (its extent only bounds what a copy may address; copies address rows of held pages only).
    if (!qf_make_map_bf16(&kv_map, base, 1ll << 31, D, D, QF_PAGE)) return (int)cudaErrorNotSupported;
    dim3 grid((max_q_len + TA_BM - 1) / TA_BM, n_heads, n_seqs);
    prefill_tc_kernel<D><<<grid, TA_THREADS, smem, stream>>>(q_map, kv_map, (bf16*)out, cu_q, tok_pos, slots, site, n_heads,
                                                             scale * 1.4426950408889634f, window, err);
    return (int)cudaGetLastError();
}

// The arguments of qf_attention_prefill and the number of rows of q (n_tokens). cudaErrorInvalidValue for a head
// size other than 64 or 128, or for cache pages with gaps (the caller then uses another kernel).
QF_EXPORT int qf_attention_prefill_tc(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots,
                                      void* base, const int* table, long long page_elems, int table_stride, int kv_heads,
                                      int head_dim, int n_heads, int n_seqs, int n_tokens, int max_q_len, float scale,
                                      int window, int* err, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0 || n_tokens <= 0) return 0;
    if (kv_heads <= 0 || n_heads % kv_heads) return (int)cudaErrorInvalidValue;
    if (head_dim == 64)
        return launch<64>(q, out, cu_q, tok_pos, slots, base, table, page_elems, table_stride, kv_heads, n_heads, n_seqs,
                          n_tokens, max_q_len, scale, window, err, stream);
    if (head_dim == 128)
        return launch<128>(q, out, cu_q, tok_pos, slots, base, table, page_elems, table_stride, kv_heads, n_heads, n_seqs,
                           n_tokens, max_q_len, scale, window, err, stream);
    return (int)cudaErrorInvalidValue;
}
