// Causal grouped-query flash attention for spans of new tokens over the paged cache on the fifth-generation tensor
// cores (tcgen05), bf16, head sizes 64 and 128. Same contract as the mma.sync kernel of attention_prefill.cu: the
// span's own keys are in the cache already, a query at position p sees keys max(0, p - window + 1) <= j <= p.
//
// A block serves 128 consecutive query tokens of one (sequence, query head). Thread t of its first four warps owns
// query row t, which is lane t of the block's tensor memory; one thread of a fifth warp issues every copy and every
// product. Per 64-position page of the head's kv head:
//   S = Q K^T     D / 16 products of 128 x 64 x 16 into 64 columns of tensor memory; Q (once) and the page's keys
//                 come by tiled copies of the tensor memory accelerator, 128-byte swizzle
//   softmax       every row thread loads its row of S (64 float32) into registers and says so on a barrier of 128
//                 arrivals: S of the NEXT page is then multiplied under this page's softmax. Maximum, base-2
//                 exponentials and sum need no exchange between threads; the weights go to shared memory as bf16
//                 in the swizzled K-major layout the tensor cores read, and the thread arrives at a second barrier
//   PV            when all rows have arrived there: four products of 128 x D x 16, the page's values read as they
//                 lie (MN-major), ADDED to the running output O in D further columns of tensor memory
//   O             stays in tensor memory. The exponentials of a row are taken against a reference maximum that is
//                 only moved when the true maximum has grown by more than 2^8 since (weights stay below 256, well
//                 inside bf16 and float32); only then does the warp rescale its rows of O (load, multiply, store).
//                 Numerator and denominator carry the same reference, so the quotient at the end is unchanged.
// Keys and values of the page after next are fetched as soon as a page's products are done (two stages). There is
// no block-wide barrier inside the loop: rows and issuer hand over through shared-memory barriers. Several blocks
// share an SM; one's exponentials overlap another's products. Every wait on a barrier is bounded: a wait that runs
// out sets QF_ERR_COPY_TIMEOUT and ends the thread's loop, and the block still frees its tensor memory and returns.
// No copy uses cluster multicast.
// One prompt of a few thousand tokens gives too few blocks to fill the SMs, and its last tiles walk dozens of pages one
// after the other. With SPLIT two blocks (a cluster) share a tile: each takes every second page, and at the end the
// second block passes its rows' reference maxima, sums and outputs to the first through distributed shared memory
// (column by column, so that a warp's 32 rows make one 128-byte store; row by row the same transfer cost 17
// microseconds), which merges them with its own and writes the result.
#include <cooperative_groups.h>

#include "tcgen05.cuh"

#define TA_BM 128
#define TA_ROW_THREADS 128
#define TA_THREADS 160  // four warps of row threads and the issuing warp

template <int D, bool SPLIT>
__global__ void __launch_bounds__(TA_THREADS, D > 64 ? 2 : 3)
prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                  bf16* __restrict__ out, const int* __restrict__ cu_q, const int* __restrict__ tok_pos,
                  const int* __restrict__ slots, KvSite<bf16> site, int n_heads, int n_seqs, int row_tiles, int wave,
                  float scale_log2, int window, int* err) {
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
    // SPLIT: [D + 2][128] of the cluster's second block (a warp writes 32 neighbouring rows at once). It lies over Q and the pages' stages, which are free when both
    // blocks have left their loops (the first barrier of the cluster below).
    float* merge_s = reinterpret_cast<float*>(smem);
    constexpr int STRIDE = SPLIT ? 2 : 1;               // this block takes every STRIDE-th page of the tile
    const int rank = SPLIT ? (int)(blockIdx.x & 1) : 0;
    // Launched as a programmatic dependent: what a block works out and sets up before its first copy (its tile, the
    // barriers, its tensor memory) runs under the tail of the kernel before, which wrote the queries and the new keys
    // and values; they are read, and the output written, only after the wait.
    grid_launch_dependents();
    __shared__ __align__(8) uint64_t bar_q, bar_kv[2], bar_s, bar_sfree, bar_pv, bar_p;
    __shared__ uint32_t tmem_base_s;

    // Which (tile, head, sequence) this block serves (with SPLIT: this pair of blocks). Tiles further down a prompt walk
    // more pages and an SM holds two or three blocks, so the blocks are taken in waves of `wave` (one per SM): the first
    // wave gets the longest tiles in falling order, the second the next longest in rising order, and so on, so that the
    // blocks that share an SM have about the same work together.
    const int unit = SPLIT ? (int)(blockIdx.x / 2) : (int)blockIdx.x, units = SPLIT ? (int)(gridDim.x / 2) : (int)gridDim.x;
    const int w = unit / wave, in_wave = min(wave, units - w * wave), at = unit % wave;
    const int item = w * wave + ((w & 1) ? in_wave - 1 - at : at);
    const int per_tile = n_heads * n_seqs;
    const int tile = row_tiles - 1 - item / per_tile, head = (item % per_tile) % n_heads, seq = (item % per_tile) / n_heads;
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    const int row0 = tile * TA_BM;
    if (row0 >= q_len) return;
    const int n_rows = min(TA_BM, q_len - row0);
    const int slot = slots[seq];
    const int t = threadIdx.x, warp = t >> 5;
    const int q_width = n_heads * D;
    const int kvh = head / (n_heads / site.kv_heads);
    bf16* out_row = out + (size_t)(q_begin + row0 + t) * q_width + (size_t)head * D;
    if (slot < 0) {  // padding entry: defined output, no cache access
        grid_dependency_wait();
        if (t < n_rows)
            for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(out_row + c) = make_uint4(0, 0, 0, 0);
        return;
    }
    const int pos0 = tok_pos[q_begin + row0];  // position of the tile's first row; row t is at pos0 + t
    const int last_pos = pos0 + n_rows - 1;
    const int p_first = (window > 0 ? max(0, pos0 - window + 1) : 0) / QF_PAGE, p_end = last_pos / QF_PAGE + 1;
    const int p_begin = p_first + rank;  // this block's pages: p_begin, p_begin + STRIDE, ...
    const int n_tiles = p_end > p_begin ? (p_end - p_begin + STRIDE - 1) / STRIDE : 0;

    if (t == 0) {
        mbar_init(&bar_q, 1);
        mbar_init(&bar_kv[0], 1);
        mbar_init(&bar_kv[1], 1);
        mbar_init(&bar_s, 1);
        mbar_init(&bar_pv, 1);
        mbar_init(&bar_p, TA_ROW_THREADS);
        mbar_init(&bar_sfree, TA_ROW_THREADS);
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    grid_dependency_wait();
    const uint32_t tmem = tmem_base_s;
    bool timed_out = false;
    float m_ref = QF_NEG_BIG, l_run = 0.f;  // row threads: the reference maximum of the exponentials, and their sum
    // A warp waits as one: the loads and stores of tensor memory and the choice of the issuing lane are collective, so
    // the lanes of a warp must leave their loop together if a wait runs out.
    auto wait_all = [&](uint64_t* bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity)) != 0; };

    if (warp == 4) {
        {
            // ---- the issuing warp: copies and products. All lanes run the loop (uniform values); one lane issues.
            const bool leader = elect_one();
            const int* table_row = site.table + (long long)slot * site.table_stride;
            auto fetch_page = [&](int j) {  // keys and values of the j-th page of the run into stage j & 1
                const int stage = j & 1;
                int page = table_row[p_begin + j * STRIDE];
                if (page < 0) {  // a page the sequence does not hold: reported; some held memory is read instead
                    if (leader) atomicOr(err, QF_ERR_NO_PAGE);
                    page = 0;
                }
                // row of the cache seen as one matrix [pages * 2 * kv_heads * 64][D]
                const long long k_row = ((long long)page * 2 * site.kv_heads + kvh) * QF_PAGE;
                const long long v_row = k_row + (long long)site.kv_heads * QF_PAGE;
                if (leader) {
                    mbar_expect_tx(&bar_kv[stage], 2 * KV_BYTES);
#pragma unroll
                    for (int cb = 0; cb < CB; ++cb) {
                        tma_load_2d(k_s + stage * KV_BYTES + cb * KV_BLOCK, &kv_map, cb * 64, (int)k_row, &bar_kv[stage]);
                        tma_load_2d(v_s + stage * KV_BYTES + cb * KV_BLOCK, &kv_map, cb * 64, (int)v_row, &bar_kv[stage]);
                    }
                }
                __syncwarp();
            };
            // descriptors: an address field counts 16 bytes, so 16 columns of a K-major row (32 bytes) are 2 units
            const uint64_t desc_q = smem_desc_sw128(q_s), desc_p = smem_desc_sw128(p_s);
            const uint64_t desc_k = smem_desc_sw128(k_s), desc_v = smem_desc_mn_sw128(v_s, KV_BLOCK);
            constexpr uint32_t idesc_s = umma_idesc_bf16(TA_BM, QF_PAGE, false), idesc_pv = umma_idesc_bf16(TA_BM, D, true);
            auto issue_s = [&](int j) {  // S = Q K^T of page j; false if its keys did not arrive
                if (!wait_all(&bar_kv[j & 1], (j >> 1) & 1)) return false;
                tc_fence_after();
                const uint64_t dk = desc_k + (uint64_t)((j & 1) * (KV_BYTES >> 4));
                if (leader) {
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks)
                        umma_bf16(tmem, desc_q + (uint64_t)((ks / 4) * (Q_BLOCK >> 4) + 2 * (ks % 4)),
                                  dk + (uint64_t)((ks / 4) * (KV_BLOCK >> 4) + 2 * (ks % 4)), idesc_s, ks > 0 ? 1u : 0u);
                    umma_commit(&bar_s);
                }
                __syncwarp();
                return true;
            };
            if (leader && n_tiles > 0) {
                mbar_expect_tx(&bar_q, CB * Q_BLOCK);
#pragma unroll
                for (int cb = 0; cb < CB; ++cb) tma_load_2d(q_s + cb * Q_BLOCK, &q_map, head * D + cb * 64, q_begin + row0, &bar_q);
            }
            __syncwarp();
            if (n_tiles > 0) fetch_page(0);
            if (n_tiles > 1) fetch_page(1);
            if (n_tiles > 0) timed_out = !wait_all(&bar_q, 0) || !issue_s(0);
            for (int j = 0; j < n_tiles && !timed_out; ++j) {
                // as soon as every row holds its S in registers, S of the next page is multiplied under their softmax
                if (!wait_all(&bar_sfree, j & 1)) {
                    timed_out = true;
                    break;
                }
                tc_fence_after();
                if (j + 1 < n_tiles && !issue_s(j + 1)) {
                    timed_out = true;
                    break;
                }
                if (!wait_all(&bar_p, j & 1)) {  // every row has written its weights
                    timed_out = true;
                    break;
                }
                tc_fence_after();
                // PV of page j: weights [128][64 keys] K-major; values [64 keys][D] as they lie, 16 keys are two groups
                // of 8 rows (2048 bytes)
                const uint64_t dv = desc_v + (uint64_t)((j & 1) * (KV_BYTES >> 4));
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < QF_PAGE / 16; ++kk)
                        umma_bf16(tmem + PV_COL, desc_p + (uint64_t)(2 * kk), dv + (uint64_t)(kk * (2048 >> 4)), idesc_pv,
                                  (j > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(&bar_pv);
                }
                __syncwarp();
                if (j + 2 < n_tiles && !timed_out) {
                    // keys and values of page j have been read when its PV is done: their stage takes the page after next
                    if (!wait_all(&bar_pv, j & 1)) timed_out = true;
                    else fetch_page(j + 2);
                }
            }
        }
    } else {
        // ---- the row threads
        const int row_pos = pos0 + t, row_lo = window > 0 ? max(0, row_pos - window + 1) : 0;
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        for (int j = 0; j < n_tiles; ++j) {
            if (!wait_all(&bar_s, j & 1)) {
                timed_out = true;
                break;
            }
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
            tc_fence_before();
            mbar_arrive(&bar_sfree);  // S is in this thread's registers
            const int key0 = (p_begin + j * STRIDE) * QF_PAGE;
            // a page that every row of the block sees whole needs no mask
            const bool full = key0 + QF_PAGE - 1 <= pos0 && key0 >= (window > 0 ? max(0, pos0 + TA_BM - 1 - window + 1) : 0);
            float mx[4];  // four chains instead of one: the comparisons do not wait for each other
            if (full) {  // the scores stay unscaled; the scale is folded into the exponent below
#pragma unroll
                for (int i = 0; i < QF_PAGE; ++i) mx[i & 3] = i < 4 ? s[i] : fmaxf(mx[i & 3], s[i]);
#pragma unroll
                for (int i = 0; i < 4; ++i) mx[i] *= scale_log2;
            } else {
#pragma unroll
                for (int i = 0; i < QF_PAGE; ++i) {
                    const int kj = key0 + i;
                    s[i] = (kj <= row_pos && kj >= row_lo) ? s[i] * scale_log2 : QF_NEG_BIG;
                    mx[i & 3] = i < 4 ? s[i] : fmaxf(mx[i & 3], s[i]);
                }
            }
            const float m_true = fmaxf(m_ref, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])));
            // The reference maximum moves before the exponentials; O, which carries the old one, is rescaled after them,
            // when the products of the page before are surely done.
            float f_o = 1.0f;
            bool moved = false;
            if (j == 0) {
                m_ref = m_true;  // nothing to rescale yet: the first products overwrite O
            } else if (m_true - m_ref > 8.0f) {
                moved = true;
                f_o = fast_exp2(m_ref - m_true);
                m_ref = m_true;
                l_run *= f_o;
            }
            float part[4] = {0.f, 0.f, 0.f, 0.f};
            if (full) {
#pragma unroll
                for (int i = 0; i < QF_PAGE; ++i) {
                    s[i] = fast_exp2(fmaf(s[i], scale_log2, -m_ref));
                    part[i & 3] += s[i];
                }
            } else {
#pragma unroll
                for (int i = 0; i < QF_PAGE; ++i) {
                    // a masked score is QF_NEG_BIG: its weight is 0 even while the reference is QF_NEG_BIG too
                    s[i] = s[i] > 0.5f * QF_NEG_BIG ? fast_exp2(s[i] - m_ref) : 0.f;
                    part[i & 3] += s[i];
                }
            }
            l_run += (part[0] + part[1]) + (part[2] + part[3]);
            // the products of the page before read the weights' buffer and add to O: both must be done before this
            // thread writes either
            if (j > 0 && !wait_all(&bar_pv, (j - 1) & 1)) {
                timed_out = true;
                break;
            }
            if (__any_sync(0xffffffffu, moved)) {  // the warp's 32 rows of O are loaded and stored together
                tc_fence_after();
                // (16 columns at a time: the row of weights is still in this thread's registers)
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 16) {
                    uint32_t raw[16];
                    tmem_load_16(lane_base + PV_COL + c0, raw);
#pragma unroll
                    for (int i = 0; i < 16; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * f_o);
                    tmem_store_16(lane_base + PV_COL + c0, raw);
                }
                tmem_store_wait();
            }
            // the row of weights, bf16, 16-byte chunk c at chunk position c ^ (row % 8) of the row's 128 bytes
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint4 chunk = make_uint4(pack_bf16(s[8 * c], s[8 * c + 1]), pack_bf16(s[8 * c + 2], s[8 * c + 3]),
                                               pack_bf16(s[8 * c + 4], s[8 * c + 5]), pack_bf16(s[8 * c + 6], s[8 * c + 7]));
                *reinterpret_cast<uint4*>(p_s + t * 128 + ((c ^ (t & 7)) << 4)) = chunk;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor cores read what this thread wrote
            tc_fence_before();
            mbar_arrive(&bar_p);
        }
        if (!timed_out && n_tiles > 0 && !wait_all(&bar_pv, (n_tiles - 1) & 1)) timed_out = true;
        tc_fence_after();
        if (!SPLIT && !timed_out) {  // the loads are collective: every lane of the warp takes part, rows beyond the span store nothing
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t raw[32];
                tmem_load_32(lane_base + PV_COL + c0, raw);
                if (t < n_rows) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        float v[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(raw[c + i]) * inv;
                        *reinterpret_cast<uint4*>(out_row + c0 + c) =
                            make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
                    }
                }
            }
        }
    }
    if (SPLIT) {
        cooperative_groups::this_cluster().sync();  // every thread of both blocks: both have left their loops, their stages are free
        if (rank == 1 && warp < 4) {
            // this block's part of every row goes to the first block: output sums, reference maximum, sum of weights
            const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
            float* theirs = cooperative_groups::this_cluster().map_shared_rank(merge_s, 0) + t;
            const bool have = n_tiles > 0 && !timed_out;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 16) {
                uint32_t raw[16];
                if (have) tmem_load_16(lane_base + PV_COL + c0, raw);
#pragma unroll
                for (int i = 0; i < 16; ++i) theirs[(c0 + i) * TA_BM] = have ? __uint_as_float(raw[i]) : 0.f;
            }
            theirs[D * TA_BM] = have ? m_ref : QF_NEG_BIG;
            theirs[(D + 1) * TA_BM] = have ? l_run : 0.f;
        }
        cooperative_groups::this_cluster().sync();  // the second block's parts have arrived
        if (rank == 0 && warp < 4) {
            // merge: both parts carry a reference maximum of their own; the common one is the larger
            const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
            const float* theirs = merge_s + t;
            const float m_other = theirs[D * TA_BM], l_other = theirs[(D + 1) * TA_BM];
            const float m_all = fmaxf(m_ref, m_other);
            const float f_mine = fast_exp2(m_ref - m_all), f_theirs = fast_exp2(m_other - m_all);
            const float l_all = l_run * f_mine + l_other * f_theirs;
            const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
            const bool have = n_tiles > 0 && !timed_out;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t raw[32];
                if (have) tmem_load_32(lane_base + PV_COL + c0, raw);
                if (t < n_rows) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        float v[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            v[i] = ((have ? __uint_as_float(raw[c + i]) * f_mine : 0.f) + theirs[(c0 + c + i) * TA_BM] * f_theirs) * inv;
                        *reinterpret_cast<uint4*>(out_row + c0 + c) =
                            make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
                    }
                }
            }
        }
    }
    if (timed_out) atomicOr(err, QF_ERR_COPY_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 4)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32  %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
}

template <int D, bool SPLIT>
static int launch_variant(const CUtensorMap& q_map, const CUtensorMap& kv_map, void* out, const int* cu_q, const int* tok_pos,
                          const int* slots, KvSite<bf16> site, int n_heads, int n_seqs, int max_q_len, float scale, int window,
                          int* err, cudaStream_t stream) {
    size_t smem = (size_t)(D / 64) * TA_BM * 128 + 4 * (size_t)(D / 64) * QF_PAGE * 128 + TA_BM * 128 + 1024;
    auto kernel = prefill_tc_kernel<D, SPLIT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int row_tiles = (max_q_len + TA_BM - 1) / TA_BM;
    const long long blocks = (long long)row_tiles * n_heads * n_seqs * (SPLIT ? 2 : 1);
    if (blocks > 0x7fffffffll) return (int)cudaErrorInvalidValue;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)blocks);
    config.blockDim = dim3(TA_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = SPLIT ? 2 : 1;
    return (int)cudaLaunchKernelEx(&config, kernel, q_map, kv_map, (bf16*)out, cu_q, tok_pos, slots, site, n_heads, n_seqs,
                                   row_tiles, SPLIT ? qf_sm_count() / 2 : qf_sm_count(), scale * 1.4426950408889634f, window, err);
}

template <int D>
static int launch(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots, void* base,
                  const int* table, long long page_elems, int table_stride, int kv_heads, int n_heads, int n_seqs,
                  int n_tokens, int max_q_len, int max_kv_len, float scale, int window, int* err, cudaStream_t stream) {
    // the cache pages must be what the map takes them for: [2][kv_heads][64][D] without gaps
    if (page_elems != 2ll * kv_heads * QF_PAGE * D) return (int)cudaErrorInvalidValue;
    KvSite<bf16> site{(bf16*)base, table, page_elems, table_stride, kv_heads, D};
    CUtensorMap q_map = {}, kv_map = {};
    const long long q_width = (long long)n_heads * D;
    if (!qf_make_map_bf16(&q_map, q, n_tokens, q_width, q_width, TA_BM)) return (int)cudaErrorNotSupported;
    // The cache of this entry as one matrix of rows of D elements. The map is given more rows than any cache has
    // (its extent only bounds what a copy may address; copies address rows of held pages only).
    if (!qf_make_map_bf16(&kv_map, base, 1ll << 31, D, D, QF_PAGE)) return (int)cudaErrorNotSupported;
    // Two blocks per tile when a tile's chain of pages is what takes the time. Measured on one prompt, head size 64, 14
    // heads (three blocks fit an SM): 1,024 tokens 21 -> 17 microseconds, 2,048 tokens 38 -> 27, 3,072 tokens 54 -> 48,
    // 4,096 tokens no gain; so chains of 16 pages and more, while the pairs need no more than two rounds on the SMs.
    // Head size 128 (two blocks per SM, a merge twice as large): 8 tiles of 16 pages 24 -> 29 and pairs in two rounds 51 ->
    // 64, so chains of 32 pages and room for every pair at once.
    // (tiles that hold rows: the grid also has blocks for the rows that shorter sequences lack, which end at once)
    const long long blocks = (long long)min((max_q_len + TA_BM - 1) / TA_BM * n_seqs, n_tokens / TA_BM + n_seqs) * n_heads;
    const int span = window > 0 && window + TA_BM < max_kv_len ? window + TA_BM : max_kv_len;
    const long long room = (long long)qf_sm_count() * (D <= 64 ? 3 : 2);
    const bool split = D <= 64 ? span >= 16 * QF_PAGE && blocks <= room : span >= 32 * QF_PAGE && blocks * 2 <= room;
    return split ? launch_variant<D, true>(q_map, kv_map, out, cu_q, tok_pos, slots, site, n_heads, n_seqs, max_q_len, scale, window, err, stream)
                 : launch_variant<D, false>(q_map, kv_map, out, cu_q, tok_pos, slots, site, n_heads, n_seqs, max_q_len, scale, window, err, stream);
}

// The arguments of qf_attention_prefill (with `max_kv_len`, the bound that steers the sharing of a tile) and the number
// of rows of q (n_tokens). cudaErrorInvalidValue for a head
// size other than 64 or 128, or for cache pages with gaps (the caller then uses another kernel).
QF_EXPORT int qf_attention_prefill_tc(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots,
                                      void* base, const int* table, long long page_elems, int table_stride, int kv_heads,
                                      int head_dim, int n_heads, int n_seqs, int n_tokens, int max_q_len, int max_kv_len,
                                      float scale, int window, int* err, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0 || n_tokens <= 0) return 0;
    if (kv_heads <= 0 || n_heads % kv_heads) return (int)cudaErrorInvalidValue;
    if (head_dim == 64)
        return launch<64>(q, out, cu_q, tok_pos, slots, base, table, page_elems, table_stride, kv_heads, n_heads, n_seqs,
                          n_tokens, max_q_len, max_kv_len, scale, window, err, stream);
    if (head_dim == 128)
        return launch<128>(q, out, cu_q, tok_pos, slots, base, table, page_elems, table_stride, kv_heads, n_heads, n_seqs,
                           n_tokens, max_q_len, max_kv_len, scale, window, err, stream);
    return (int)cudaErrorInvalidValue;
}
