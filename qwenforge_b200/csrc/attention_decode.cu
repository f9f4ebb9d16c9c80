// Split-K flash decoding over the paged cache (bf16): one new token per sequence attends to its own
// cache; the key range of every (sequence, kv head) is cut into up to `n_splits` runs of whole pages that
// separate blocks reduce at once, so that a batch of a few sequences still fills the GPU. How many runs a sequence
// gets is decided on the device from the lengths of the batch (see the kernel's first lines): a long sequence among
// short ones gets more blocks, not longer ones.
//
// A block serves one (sequence, kv head, chunk of up to 16 query heads of the group, split). The query heads of
// the group are the 16 rows of an m16n8k16 tensor-core tile, so keys and values are read once for the whole
// group. Each WARP works alone on whole pages (64 positions: 64 x D keys, 64 x D values): the page arrives in two
// halves through the warp's own two shared-memory buffers (tiled TMA copies, or 16-byte asynchronous copies into
// padded rows; see below), then S = Q K^T, online softmax in float32 (base-2 exponentials, the scale folded in;
// halves that are seen whole skip the mask), O += P V. With eight warps a block has eight pages in flight and no
// block-wide barrier inside the loop. Halves that hold only positions before the new token are fetched before the
// kernel waits for the one that wrote the new token. At the end every warp leaves its rescaled sums in its own
// buffer and all threads add them up in warp order. With one split the block writes the output; otherwise it
// writes (max, sum, O) partials to scratch and takes a ticket: the block that draws the last ticket of its
// (sequence, kv head, chunk) folds all partials, two outputs per thread at once, and resets the ticket counter.
// No block waits for another. (Merging the splits of a thread-block cluster through distributed shared memory
// instead was measured slower, and so was a variant of sixteen warps with half a page each.)
// The kernel is launched as a programmatic dependent of the kernel before it.
#include <algorithm>

#include "tma.cuh"

// TMA: head sizes whose rows are a multiple of 128 bytes (64, 128) take the half pages by tiled copies of the tensor
// memory accelerator (128-byte swizzle; one copy per 64 columns for the keys and as many for the values, completing
// on the warp's own barrier with a bounded wait); other head sizes use 16-byte asynchronous copies into padded rows.
// ---- The plan of a step: which block takes which run of which sequence. The lengths live on the device (a captured
// graph replays these launches with other lengths every step), so one warp works the plan out once per step, for every
// layer whose attention has the same shape. A sequence of P pages is cut into ceil(P / target) runs of equal size,
// target being the pages per block at which the batch's pages fill the device's block slots once (and at least one
// page per warp of a block); where the rounding up gives more blocks than slots, target grows until they fit, so that
// no block waits for a free slot while others are done. Sequences of unequal lengths thus get blocks of about
// equal work, and a batch that fills the SMs unsplit stays unsplit.
// The plan starts with the number of runs of every sequence (n_seqs ints, padded to a multiple of four), for whoever
// folds the partial results later; the block records follow. Record j < n_pairs: x = sequence (batch entry; -1: no such
// block), y = run | runs << 16, z = the sequence's length with the new token, w = its cache slot (-1: a padding entry,
// whose one block writes zeros).
// The kernel does not let its dependents start early: whatever runs later in the stream may read the plan without
// waiting for anything but its own predecessor.
__global__ void __launch_bounds__(32)
decode_plan_kernel(const int* __restrict__ cu_q, const int* __restrict__ tok_pos, const int* __restrict__ slots, int n_seqs,
                   int kvc, int sms, int warps, int window, int max_splits, int4* __restrict__ plan_all, int n_pairs) {
    const int lane = threadIdx.x;
    int* runs = reinterpret_cast<int*>(plan_all);
    int4* plan = plan_all + (n_seqs + 3) / 4;
    auto length_of = [&](int s) -> int { return s < n_seqs && slots[s] >= 0 ? tok_pos[cu_q[s]] + 1 : 0; };
    auto pages_of = [&](int len) -> int {
        if (len <= 0) return 0;
        const int from = window > 0 ? max(0, len - window) : 0;
        return (len - 1) / QF_PAGE - from / QF_PAGE + 1;
    };
    auto runs_of = [&](int pages, float target) -> int {
        if (pages <= 0) return 1;
        int n = min(max((int)ceilf((float)pages / target), 1), max_splits);
        const int each = (pages + n - 1) / n;
        return (pages + each - 1) / each;  // no run without a page
    };
    auto warp_sum = [](int v) -> int {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        return v;
    };
    int total = 0;
    for (int s0 = 0; s0 < n_seqs; s0 += 32) total += pages_of(length_of(s0 + lane));
    total = warp_sum(total);
    float target = fmaxf((float)warps, (float)total * (float)kvc / (float)sms);
    for (int round = 0; round < 16; ++round) {
        int pairs = 0;
        for (int s0 = 0; s0 < n_seqs; s0 += 32) pairs += s0 + lane < n_seqs ? runs_of(pages_of(length_of(s0 + lane)), target) : 0;
        pairs = warp_sum(pairs);
        if (pairs <= n_seqs || (long long)pairs * kvc <= sms) break;
        if (round == 15) {
            target = 3.0e38f;  // one run each: always within the grid
            break;
        }
        target *= fmaxf(1.05f, (float)pairs * (float)kvc / (float)sms);
    }
    grid_dependency_wait();  // nothing is written before this; and when this kernel is done, so is everything before it
    int before = 0;
    for (int s0 = 0; s0 < n_seqs; s0 += 32) {
        const int s = s0 + lane;
        const int len = length_of(s);
        const int n = s < n_seqs ? runs_of(pages_of(len), target) : 0;
        int upto = n;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, upto, o);
            if (lane >= o) upto += t;
        }
        const int first = before + upto - n;
        if (s < n_seqs) runs[s] = n;
        for (int k = 0; k < n; ++k)
            if (first + k < n_pairs) plan[first + k] = make_int4(s, k | (n << 16), len, len > 0 ? slots[s] : -1);
        before += __shfl_sync(0xffffffffu, upto, 31);
    }
    for (int j = before + lane; j < n_pairs; j += 32) plan[j] = make_int4(-1, 0, 0, -1);
}

template <int D, int WARPS, bool TMA>
__global__ void __launch_bounds__(WARPS * 32)
decode_split_kernel(const __grid_constant__ CUtensorMap kv_map, const bf16* __restrict__ q, bf16* __restrict__ out,
                    const int* __restrict__ cu_q, const int4* __restrict__ plan, KvSite<bf16> site, int n_heads, int chunks, float scale_log2,
                    int window, int max_splits, int n_seqs, int fold_later, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int* __restrict__ counters, int* err, unsigned long long* stamps) {
    constexpr int DEC_WARPS = WARPS, DEC_THREADS = WARPS * 32;
    // measuring aid: if `stamps` is given, thread 0 leaves nanosecond time stamps of the block's phases in stamps[block][8]
    auto stamp = [&](int phase) {
        if (stamps && threadIdx.x == 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            stamps[(size_t)blockIdx.x * 8 + phase] = now;
        }
    };
    stamp(0);
    constexpr int LD = TMA ? D : D + 8;  // shared-memory row (bf16 elements): padded, or swizzled blocks of 64 columns
    constexpr int KS = D / 16;          // k-steps of Q K^T
    constexpr int NT = D / 8;           // n-tiles of P V
    constexpr int PAGE_BYTES = 2 * QF_PAGE * LD * 2;  // one warp's buffer: keys then values of a page
    extern __shared__ unsigned char smem_unaligned[];
    // the swizzle of the tiled copies is a function of the shared-memory address: buffers start on 1024 bytes
    unsigned char* smem_raw = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
    __shared__ float m_s[DEC_WARPS][16], l_s[DEC_WARPS][16];
    __shared__ int ticket_s;
    __shared__ __align__(8) uint64_t bars[DEC_WARPS][2];

    grid_launch_dependents();
    // ---- which (sequence, split) this block is: a record of the plan that decode_plan_kernel made from the lengths of
    // this step's batch (see there). The grid holds as many blocks as any batch of this shape can need; those beyond
    // the plan end here.
    const int kvc = site.kv_heads * chunks;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int4 record = __ldg(plan + (n_seqs + 3) / 4 + blockIdx.x / kvc);
    const int seq = record.x;
    if (seq < 0) return;
    const int split = record.y & 0xffff, n_splits = record.y >> 16;
    const int y = blockIdx.x % kvc;
    const int kvh = y / chunks, chunk = y % chunks;
    const int G = n_heads / site.kv_heads;
    const int g0 = chunk * 16, n_g = min(16, G - g0);
    const int head0 = kvh * G + g0;
    const int tok = cu_q[seq];
    const int slot = record.w;
    const int q_width = n_heads * D;
    bf16* out_row = out + (size_t)tok * q_width + (size_t)head0 * D;

    if (slot < 0) {  // padding entry: defined output (or a partial result that folds to zero), no cache access, no ticket
        grid_dependency_wait();
        if (split == 0 && !fold_later)
            for (int i = threadIdx.x; i < n_g * D; i += DEC_THREADS) out_row[i] = __float2bfloat16_rn(0.f);
        if (split == 0 && fold_later && threadIdx.x < n_g) {
            float* ml = part_ml + (((size_t)seq * n_heads + head0 + threadIdx.x) * max_splits) * 2;
            ml[0] = QF_NEG_BIG;
            ml[1] = 0.f;
        }
        return;
    }
    const int L = record.z;
    const int lo = window > 0 ? max(0, L - window) : 0;
    const int first_page = lo / QF_PAGE, last_page = (L - 1) / QF_PAGE;
    const int pps = (last_page - first_page + n_splits) / n_splits;  // ceil(pages / splits)
    const int p_begin = first_page + split * pps, p_end = min(p_begin + pps, last_page + 1);

    // ---- every warp works alone on whole pages: page p_begin + warp, then + WARPS, ... It takes a page in two halves
    // of 32 positions through two buffers, so that the second half (or the next page's first) is on its way while
    // the first is multiplied.
    constexpr int HALF = QF_PAGE / 2;
    constexpr int STAGE_ELEMS = 2 * HALF * LD;  // keys then values of half a page
    bf16* stage0 = reinterpret_cast<bf16*>(smem_raw + (size_t)warp * PAGE_BYTES);
    const int* table_row = site.table + (long long)slot * site.table_stride;
    const int my_pages = p_begin + warp < p_end ? (p_end - p_begin - warp + DEC_WARPS - 1) / DEC_WARPS : 0;
    const int n_halves = 2 * my_pages;
    // half i of this warp: page p_begin + warp + (i / 2) * WARPS, positions key0 .. key0 + 31
    // Element (row r, column c) of a staged half page: padded rows, or (TMA) blocks of 32 rows x 64 columns in which the
    // 16-byte chunk index is XORed with the row (the 128-byte swizzle the tiled copy writes).
    auto at = [&](const bf16* base, int r, int c) -> const bf16* {
        if (TMA) return base + (size_t)(c >> 6) * (HALF * 64) + (size_t)r * 64 + ((((c >> 3) & 7) ^ (r & 7)) << 3) + (c & 7);
        return base + (size_t)r * LD + c;
    };
    if (TMA && lane == 0) {
        mbar_init(&bars[warp][0], 1);
        mbar_init(&bars[warp][1], 1);
    }
    __syncwarp();
    auto half_live = [&](int i, int& page, int& key0) {
        if (i >= n_halves) return false;
        const int p = p_begin + warp + (i >> 1) * DEC_WARPS;
        key0 = p * QF_PAGE + (i & 1) * HALF;
        page = table_row[p];
        if (page < 0) {
            if (lane == 0 && (i & 1) == 0) atomicOr(err, QF_ERR_NO_PAGE);
            return false;
        }
        return key0 < L && key0 + HALF > lo;
    };
    auto issue = [&](int i) {
        int page, key0;
        if (half_live(i, page, key0)) {
            bf16* kb = stage0 + (size_t)(i & 1) * STAGE_ELEMS;
            bf16* vb = kb + HALF * LD;
            if (TMA) {
                if (lane == 0) {
                    // row of the cache seen as one matrix [pages * 2 * kv_heads * 64][D]
                    const long long k_row = ((long long)page * 2 * site.kv_heads + kvh) * QF_PAGE + (i & 1) * HALF;
                    const long long v_row = k_row + (long long)site.kv_heads * QF_PAGE;
                    uint64_t* bar = &bars[warp][i & 1];
                    mbar_expect_tx(bar, 2 * HALF * D * 2);
#pragma unroll
                    for (int cb = 0; cb < D / 64; ++cb) {
                        tma_load_2d(kb + (size_t)cb * HALF * 64, &kv_map, cb * 64, (int)k_row, bar);
                        tma_load_2d(vb + (size_t)cb * HALF * 64, &kv_map, cb * 64, (int)v_row, bar);
                    }
                }
            } else {
                const bf16* kp = site.base + (long long)page * site.page_elems + ((long long)kvh * QF_PAGE + (i & 1) * HALF) * D;
                const bf16* vp = kp + (long long)site.kv_heads * QF_PAGE * D;
                constexpr int CH = D / 8;  // 16-byte chunks per row
#pragma unroll 4
                for (int j = lane; j < HALF * CH; j += 32) {
                    const int r = j / CH, c = (j % CH) * 8;
                    cp_async_16(kb + (size_t)r * LD + c, kp + (size_t)r * D + c, true);
                    cp_async_16(vb + (size_t)r * LD + c, vp + (size_t)r * D + c, true);
                }
            }
        }
        if (!TMA) cp_async_commit();  // one group per half, empty when there is nothing to fetch
    };
    uint32_t uses_even = 0, uses_odd = 0;  // completed fetches into each buffer (the parity the next wait looks for)
    // Positions before the new token lie in the cache since earlier steps: the halves of the warp's first page that
    // hold only such positions are fetched before this kernel waits for the one that wrote the new token's query,
    // key and value.
    const int page0_end = (p_begin + warp + 1) * QF_PAGE;
    const int n_early = n_halves == 0 ? 0 : page0_end <= L - 1 ? 2 : page0_end - HALF <= L - 1 ? 1 : 0;
    for (int i = 0; i < n_early; ++i) issue(i);
    stamp(1);
    grid_dependency_wait();
    stamp(2);

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

    if (n_early == 0) issue(0);
    for (int i = 0; i < n_halves; ++i) {
        if (i + 1 >= n_early) issue(i + 1);
        int page_i, key0;
        const bool live = half_live(i, page_i, key0);
        if (TMA) {
            // the barrier of this buffer is on its (i / 2)-th use; only halves that were fetched are waited for
            const uint32_t parity = ((i & 1) ? uses_odd : uses_even) & 1;
            if (live && !mbar_wait(&bars[warp][i & 1], parity) && lane == 0) atomicOr(err, QF_ERR_COPY_TIMEOUT);
            if (live) {
                uses_even += (i & 1) ^ 1;
                uses_odd += i & 1;
            }
            if (i == 0) stamp(3);
        } else {
            cp_async_wait<1>();
            __syncwarp();  // each lane waited for its own copies; together the half page is complete
        }
        if (live) {
            const bf16* kb = stage0 + (size_t)(i & 1) * STAGE_ELEMS;
            const bf16* vb = kb + HALF * LD;
            float s[4][4];
#pragma unroll
            for (int t = 0; t < 4; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int t2 = 0; t2 < 2; ++t2) {  // 16 keys per ldmatrix.x4
                    uint32_t kf[4];
                    ldmatrix_x4(kf, at(kb, 16 * t2 + (lane >> 4) * 8 + (lane & 7), 16 * ks + ((lane >> 3) & 1) * 8));
                    mma_bf16_16816(s[2 * t2], qa[ks], kf[0], kf[1]);
                    mma_bf16_16816(s[2 * t2 + 1], qa[ks], kf[2], kf[3]);
                }
            }
            const bool full = key0 >= lo && key0 + HALF <= L;  // every key of the half is visible
            float mx[2] = {QF_NEG_BIG, QF_NEG_BIG};
            if (full) {
#pragma unroll
                for (int t = 0; t < 4; ++t) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[t][e] *= scale_log2;
                    mx[0] = fmaxf(mx[0], fmaxf(s[t][0], s[t][1]));
                    mx[1] = fmaxf(mx[1], fmaxf(s[t][2], s[t][3]));
                }
            } else {
#pragma unroll
                for (int t = 0; t < 4; ++t) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int kj = key0 + 8 * t + 2 * (lane & 3) + e;
                        const bool ok = kj >= lo && kj < L;
                        s[t][e] = ok ? s[t][e] * scale_log2 : QF_NEG_BIG;
                        s[t][2 + e] = ok ? s[t][2 + e] * scale_log2 : QF_NEG_BIG;
                        mx[0] = fmaxf(mx[0], s[t][e]);
                        mx[1] = fmaxf(mx[1], s[t][2 + e]);
                    }
                }
            }
            float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                corr[r] = fast_exp2(m_run[r] - m_new);
                m_run[r] = m_new;
            }
            // A live half holds a visible key, and the one token's heads all see the same keys: the running maximum is
            // a real score from here on, and a masked score (QF_NEG_BIG) gets the weight 2^(-huge) = 0.
#pragma unroll
            for (int t = 0; t < 4; ++t) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    s[t][e] = fast_exp2(s[t][e] - m_run[0]);
                    s[t][2 + e] = fast_exp2(s[t][2 + e] - m_run[1]);
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
            if (corr[0] != 1.f || corr[1] != 1.f) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    o[nt][0] *= corr[0];
                    o[nt][1] *= corr[0];
                    o[nt][2] *= corr[1];
                    o[nt][3] *= corr[1];
                }
            }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {  // 16 keys per step
                uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                  pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
                for (int nt = 0; nt < NT; nt += 2) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, at(vb, 16 * kk + ((lane >> 3) & 1) * 8 + (lane & 7), 8 * nt + (lane >> 4) * 8));
                    mma_bf16_16816(o[nt], pa, vf[0], vf[1]);
                    mma_bf16_16816(o[nt + 1], pa, vf[2], vf[3]);
                }
            }
        }
        __syncwarp();  // every lane has read this buffer before the copies of half i + 2 overwrite it
    }
    if (!TMA) cp_async_wait<0>();
    stamp(4);

    // ---- merge the warps: every warp leaves its numerators, rescaled to the block's maximum, in its own page buffer
    // (its copies are complete and nobody else read it); then all threads add the warps up, in warp order
    if ((lane & 3) == 0) {
        m_s[warp][lane >> 2] = m_run[0];
        m_s[warp][(lane >> 2) + 8] = m_run[1];
    }
    __syncthreads();
    constexpr int OLD = D + 8;  // float32 row stride (8 modulo 32): the 8-byte stores of a half warp meet no bank twice
    float* o_w = reinterpret_cast<float*>(smem_raw + (size_t)warp * PAGE_BYTES);  // [16][OLD]
    float f[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + 8 * r;
        float m_all = m_s[0][row];
#pragma unroll
        for (int w = 1; w < DEC_WARPS; ++w) m_all = fmaxf(m_all, m_s[w][row]);
        f[r] = exp2f(m_run[r] - m_all);
    }
    if ((lane & 3) == 0) {
        l_s[warp][lane >> 2] = l_run[0] * f[0];
        l_s[warp][(lane >> 2) + 8] = l_run[1] * f[1];
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int c = 8 * nt + 2 * (lane & 3), r0 = lane >> 2, r1 = r0 + 8;
        *reinterpret_cast<float2*>(o_w + r0 * OLD + c) = make_float2(o[nt][0] * f[0], o[nt][1] * f[0]);
        *reinterpret_cast<float2*>(o_w + r1 * OLD + c) = make_float2(o[nt][2] * f[1], o[nt][3] * f[1]);
    }
    __syncthreads();
    stamp(5);
    // block result: row r: maximum max_w m_s[w][r], sum sum_w l_s[w][r], numerator sum_w (warp w's buffer)[r][:]
    const size_t part_row0 = ((size_t)seq * n_heads + head0) * max_splits;  // partial index of (row 0, split 0)
    for (int i = threadIdx.x; i < n_g * D; i += DEC_THREADS) {
        const int r = i / D, d = i % D;
        float num = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) num += reinterpret_cast<const float*>(smem_raw + (size_t)w * PAGE_BYTES)[r * OLD + d];
        if (n_splits == 1 && !fold_later) {
            float l = 0.f;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) l += l_s[w][r];
            out_row[i] = __float2bfloat16_rn(l > 0.f ? num / l : 0.f);
        } else {
            part_o[(part_row0 + (size_t)r * max_splits + split) * D + d] = num;
        }
    }
    if (n_splits == 1 && !fold_later) return;
    if (threadIdx.x < n_g) {
        const int r = threadIdx.x;
        float m = m_s[0][r], l = 0.f;
#pragma unroll
        for (int w = 1; w < DEC_WARPS; ++w) m = fmaxf(m, m_s[w][r]);
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) l += l_s[w][r];
        part_ml[(part_row0 + (size_t)r * max_splits + split) * 2] = m;
        part_ml[(part_row0 + (size_t)r * max_splits + split) * 2 + 1] = l;
    }
    if (fold_later) {  // the kernel that comes next folds the partial results itself
        stamp(6);
        return;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = counters + (size_t)seq * kvc + y;
        const int ticket = atomicAdd(counter, 1);
        if (ticket == n_splits - 1) {
            // the last block of this (sequence, kv head, chunk): every partial is visible after this fence; the
            // block barrier below hands that on to the other threads
            __threadfence();
            *counter = 0;
        }
        ticket_s = ticket;
    }
    __syncthreads();
    stamp(6);
    if (ticket_s != n_splits - 1) return;
    // Every group of four output elements folds its row's partials in split order, eight at a time, keeping a running
    // maximum: out = sum_s exp2(m_s - M) o_s / sum_s exp2(m_s - M) l_s. A thread takes two groups at once, which covers
    // a block's whole output in one round at every head size, so that all of the fold's loads are in flight together.
    constexpr int D4 = D / 4;
    const int n_items = n_g * D4;
    for (int i0 = threadIdx.x; i0 < n_items; i0 += 2 * DEC_THREADS) {
        const float2* ml[2];
        const float4* po[2];
        bool live[2];
        float big[2] = {QF_NEG_BIG, QF_NEG_BIG}, den[2] = {0.f, 0.f};
        float4 num[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            const int i = i0 + x * DEC_THREADS;
            live[x] = i < n_items;
            const int r = live[x] ? i / D4 : 0, d4 = live[x] ? i % D4 : 0;
            ml[x] = reinterpret_cast<const float2*>(part_ml) + part_row0 + (size_t)r * max_splits;
            po[x] = reinterpret_cast<const float4*>(part_o + (part_row0 + (size_t)r * max_splits) * D) + d4;
        }
        for (int sp0 = 0; sp0 < n_splits; sp0 += 8) {
            float2 a[2][8];
            float4 v[2][8];
#pragma unroll
            for (int x = 0; x < 2; ++x)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const bool in = live[x] && sp0 + j < n_splits;
                    a[x][j] = in ? __ldcg(ml[x] + sp0 + j) : make_float2(QF_NEG_BIG, 0.f);
                    v[x][j] = in ? __ldcg(po[x] + (size_t)(sp0 + j) * D4) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                float top = big[x];
#pragma unroll
                for (int j = 0; j < 8; ++j) top = fmaxf(top, a[x][j].x);
                const float keep = exp2f(big[x] - top);
                den[x] *= keep;
                num[x].x *= keep;
                num[x].y *= keep;
                num[x].z *= keep;
                num[x].w *= keep;
                big[x] = top;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float w = exp2f(a[x][j].x - top);
                    den[x] += w * a[x][j].y;
                    num[x].x += w * v[x][j].x;
                    num[x].y += w * v[x][j].y;
                    num[x].z += w * v[x][j].z;
                    num[x].w += w * v[x][j].w;
                }
            }
        }
#pragma unroll
        for (int x = 0; x < 2; ++x)
            if (live[x]) {
                const float inv = den[x] > 0.f ? 1.f / den[x] : 0.f;
                uint2 packed;
                packed.x = pack_bf16(num[x].x * inv, num[x].y * inv);
                packed.y = pack_bf16(num[x].z * inv, num[x].w * inv);
                *reinterpret_cast<uint2*>(out_row + (size_t)(i0 + x * DEC_THREADS) * 4) = packed;
            }
    }
    stamp(7);
}

// Warps of a block: each has two half-page buffers (16 to 18 KB at D = 64, 33 to 35 KB at D = 128). Eight up to head
// size 64, four beyond. (Three at head size 128, so that two blocks share an SM and a batch of 64 sequences x 4 kv heads
// is resident at once instead of in two unequal waves, was measured: 537 MB in 104 microseconds against 99.)
constexpr int decode_warps(int d) { return d <= 64 ? 8 : 4; }
constexpr bool decode_tma(int d) { return d % 64 == 0; }
constexpr size_t decode_smem(int d) {
    return (size_t)decode_warps(d) * 2 * QF_PAGE * (decode_tma(d) ? d : d + 8) * sizeof(bf16) + 1024;
}

// Blocks of decode_split_kernel<D> that one SM holds at once (0: no kernel for this head size).
template <int D>
static int resident_blocks() {
    static int held = -1;
    if (held < 0) {
        auto kernel = decode_split_kernel<D, decode_warps(D), decode_tma(D)>;
        int n = 0;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem(D)) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, decode_warps(D) * 32, decode_smem(D)) != cudaSuccess)
            n = 1;
        held = n > 0 ? n : 1;
    }
    return held;
}

// Block slots of the device for this head size: what a plan may fill once.
static int decode_slots(int head_dim) {
    const int sms = qf_sm_count() > 0 ? qf_sm_count() : 1;
    switch (head_dim) {
        case 32: return sms * resident_blocks<32>();
        case 64: return sms * resident_blocks<64>();
        case 96: return sms * resident_blocks<96>();
        case 128: return sms * resident_blocks<128>();
        default: return 0;
    }
}

// (sequence, run) pairs of any plan: every sequence has one, and the runs beyond that fill the block slots at most once
static long long plan_pairs(int n_seqs, int kv_heads, int n_heads, int head_dim, int n_splits) {
    const long long kvc = (long long)kv_heads * ((n_heads / kv_heads + 15) / 16);
    return std::min((long long)n_seqs * n_splits, (long long)n_seqs + decode_slots(head_dim) / kvc);
}

// Blocks of the decode attention that the device holds at once at this head size (0: no kernel for this head size).
QF_EXPORT int qf_attention_decode_slots(int head_dim) { return decode_slots(head_dim); }

// Warps of a block at this head size: the pages that one run should hold at least (0: no kernel for this head size).
QF_EXPORT int qf_attention_decode_warps(int head_dim) {
    return head_dim == 32 || head_dim == 64 || head_dim == 96 || head_dim == 128 ? decode_warps(head_dim) : 0;
}

template <int D>
static int launch(const void* q, void* out, const int* cu_q, const int4* plan, void* base, const int* table,
                  long long page_elems, int table_stride, int kv_heads, int n_heads, int n_seqs, float scale, int window,
                  int n_splits, int fold_later, float* part_o, float* part_ml, int* counters, int* err,
                  unsigned long long* stamps, cudaStream_t stream) {
    constexpr int WARPS = decode_warps(D);
    constexpr bool TMA = decode_tma(D);
    const int G = n_heads / kv_heads, chunks = (G + 15) / 16;
    const size_t smem = decode_smem(D);
    cudaError_t e = cudaFuncSetAttribute(decode_split_kernel<D, WARPS, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    KvSite<bf16> site{(bf16*)base, table, page_elems, table_stride, kv_heads, D};
    CUtensorMap kv_map = {};
    if (TMA) {
        // The cache of this entry as one matrix of rows of D elements. The map is given more rows than any cache has
        // (its extent only bounds what a copy may address; copies address rows of held pages only).
        if (!qf_make_map_bf16(&kv_map, base, 1ll << 31, D, D, QF_PAGE / 2)) return (int)cudaErrorNotSupported;
    }
    dim3 grid((unsigned)(plan_pairs(n_seqs, kv_heads, n_heads, D, n_splits) * kv_heads * chunks));
    return (int)launch_pdl(decode_split_kernel<D, WARPS, TMA>, grid, dim3(WARPS * 32), smem, stream, kv_map, (const bf16*)q,
                           (bf16*)out, cu_q, plan, site, n_heads, chunks, scale * 1.4426950408889634f, window, n_splits,
                           n_seqs, fold_later, part_o, part_ml, counters, err, stamps);
}

// How many 16-byte units a plan of this shape holds (what qf_attention_decode_plan writes and qf_attention_decode
// reads): the sequences' numbers of runs, then the block records.
QF_EXPORT long long qf_attention_decode_plan_size(int n_seqs, int kv_heads, int n_heads, int head_dim, int n_splits) {
    if (n_seqs <= 0 || kv_heads <= 0 || n_heads % kv_heads || n_splits < 1 || !qf_attention_decode_warps(head_dim)) return 0;
    return (n_seqs + 3) / 4 + plan_pairs(n_seqs, kv_heads, n_heads, head_dim, n_splits);
}

// The plan of one step for attention of this shape (see decode_plan_kernel); the same plan serves every layer of the
// step that has this shape. `n_splits` is the most runs that one sequence may get.
QF_EXPORT int qf_attention_decode_plan(const int* cu_q, const int* tok_pos, const int* slots, int n_seqs, int kv_heads,
                                       int head_dim, int n_heads, int window, int n_splits, void* plan, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (kv_heads <= 0 || n_heads % kv_heads || n_splits < 1 || n_splits > 0x7fff || !qf_attention_decode_warps(head_dim))
        return (int)cudaErrorInvalidValue;
    const int kvc = kv_heads * ((n_heads / kv_heads + 15) / 16);
    return (int)launch_pdl(decode_plan_kernel, dim3(1), dim3(32), 0, stream, cu_q, tok_pos, slots, n_seqs, kvc,
                           decode_slots(head_dim), qf_attention_decode_warps(head_dim), window, n_splits, (int4*)plan,
                           (int)plan_pairs(n_seqs, kv_heads, n_heads, head_dim, n_splits));
}

// Scratch (used when n_splits > 1 or fold_later): part_o float32 [n_seqs * n_heads * n_splits * head_dim], part_ml
// float32 [n_seqs * n_heads * n_splits * 2], counters int32 [n_seqs * kv_heads * ceil(group / 16)], zero before the
// first call (the kernel leaves them zero; not used with fold_later). With fold_later the kernel stops at the partial
// results (every sequence's runs, as many as the plan's first part says) and writes no `out`: the caller's next
// kernel folds them. Returns cudaErrorInvalidValue for a head size without an instantiation.
static int decode_run(const void* q, void* out, const int* cu_q, const void* plan, void* base, const int* table,
                      long long page_elems, int table_stride, int kv_heads, int head_dim, int n_heads, int n_seqs,
                      float scale, int window, int n_splits, int fold_later, float* part_o, float* part_ml, int* counters,
                      int* err, unsigned long long* stamps, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (kv_heads <= 0 || n_heads % kv_heads || n_splits < 1 || !plan) return (int)cudaErrorInvalidValue;
    if (fold_later ? (!part_o || !part_ml) : !out) return (int)cudaErrorInvalidValue;
#define QF_CASE(DIM)                                                                                                   \
    case DIM:                                                                                                          \
        return launch<DIM>(q, out, cu_q, (const int4*)plan, base, table, page_elems, table_stride, kv_heads, n_heads, \
                           n_seqs, scale, window, n_splits, fold_later, part_o, part_ml, counters, err, stamps, stream);
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

QF_EXPORT int qf_attention_decode(const void* q, void* out, const int* cu_q, const void* plan, void* base,
                                  const int* table, long long page_elems, int table_stride, int kv_heads, int head_dim,
                                  int n_heads, int n_seqs, float scale, int window, int n_splits, int fold_later,
                                  float* part_o, float* part_ml, int* counters, int* err, cudaStream_t stream) {
    return decode_run(q, out, cu_q, plan, base, table, page_elems, table_stride, kv_heads, head_dim, n_heads, n_seqs, scale,
                      window, n_splits, fold_later, part_o, part_ml, counters, err, nullptr, stream);
}

// A measuring aid: the same launch, with every block's thread 0 writing nanosecond time stamps to stamps[block][8]:
// entry, early copies issued, the kernel before done, first half page arrived, pages done, warps merged, ticket drawn
// (or partial results written, with fold_later), fold done (the folding blocks only). The grid has
// kv_heads * ceil(group / 16) * (qf_attention_decode_plan_size(...) - ceil(n_seqs / 4)) blocks.
QF_EXPORT int qf_attention_decode_stamped(const void* q, void* out, const int* cu_q, const void* plan, void* base,
                                          const int* table, long long page_elems, int table_stride, int kv_heads,
                                          int head_dim, int n_heads, int n_seqs, float scale, int window, int n_splits,
                                          int fold_later, float* part_o, float* part_ml, int* counters, int* err,
                                          unsigned long long* stamps, cudaStream_t stream) {
    return decode_run(q, out, cu_q, plan, base, table, page_elems, table_stride, kv_heads, head_dim, n_heads, n_seqs, scale,
                      window, n_splits, fold_later, part_o, part_ml, counters, err, stamps, stream);
}

// ------------------------------------------------------------------------------------------------------------------
// The same split-K decode attention for callers that must not allocate (declared in attention_decode_noalloc.h).
// The partial results and the ticket counters live in ONE file-scope device array instead of caller-provided
// scratch. Every GPU that loads this library holds the array (QF_NOALLOC_BYTES, about 4.4 MB) until the process ends.
#include <stdio.h>

#include "attention_decode_noalloc.h"

#define QF_NOALLOC_PART_ML_FLOATS (QF_NOALLOC_MAX_ROWS * 2)
#define QF_NOALLOC_PART_O_FLOATS (QF_NOALLOC_MAX_ROWS * QF_NOALLOC_MAX_HEAD_DIM)
#define QF_NOALLOC_BYTES ((QF_NOALLOC_PART_O_FLOATS + QF_NOALLOC_PART_ML_FLOATS + QF_NOALLOC_MAX_COUNTERS + 4 * QF_NOALLOC_MAX_PAIRS) * 4)

// layout: [part_o floats][part_ml floats][counters ints][plan records of four ints]
static __device__ __align__(256) unsigned char qf_noalloc_scratch[QF_NOALLOC_BYTES];

#define QF_NOALLOC_MAX_DEVICES 64
static unsigned char* qf_noalloc_ptr[QF_NOALLOC_MAX_DEVICES];  // device address of the array, per device
static thread_local char qf_noalloc_message[256];

QF_EXPORT const char* qf_attention_decode_noalloc_error(void) { return qf_noalloc_message; }

QF_EXPORT int qf_attention_decode_noalloc(const void* q, void* out, const int* cu_q, const int* tok_pos,
                                          const int* slots, void* base, const int* table, long long page_elems,
                                          int table_stride, int kv_heads, int head_dim, int n_heads, int n_seqs,
                                          float scale, int window, int n_splits, int* err, cudaStream_t stream) {
    qf_noalloc_message[0] = 0;
    if (n_seqs <= 0) return 0;
    if (kv_heads <= 0 || n_heads % kv_heads || n_splits < 1 || n_splits > 128) {
        snprintf(qf_noalloc_message, sizeof qf_noalloc_message,
                 "qf_attention_decode_noalloc: bad shape (n_heads %d, kv_heads %d, n_splits %d)", n_heads, kv_heads, n_splits);
        return (int)cudaErrorInvalidValue;
    }
    const long long rows = (long long)n_seqs * n_heads * n_splits;
    const long long n_counters = (long long)n_seqs * kv_heads * ((n_heads / kv_heads + 15) / 16);
    const long long pairs = qf_attention_decode_plan_size(n_seqs, kv_heads, n_heads, head_dim, n_splits);
    if (pairs > QF_NOALLOC_MAX_PAIRS) {
        snprintf(qf_noalloc_message, sizeof qf_noalloc_message,
                 "qf_attention_decode_noalloc: a plan of %lld units of 16 bytes (limit %d): beyond the built-in scratch; "
                 "use fewer sequences per call or qf_attention_decode", pairs, QF_NOALLOC_MAX_PAIRS);
        return QF_NOALLOC_TOO_LARGE;
    }
    if (n_splits > 1 && (rows > QF_NOALLOC_MAX_ROWS || head_dim > QF_NOALLOC_MAX_HEAD_DIM || n_counters > QF_NOALLOC_MAX_COUNTERS)) {
        snprintf(qf_noalloc_message, sizeof qf_noalloc_message,
                 "qf_attention_decode_noalloc: n_seqs * n_heads * n_splits = %lld (limit %d), head_dim %d (limit %d), "
                 "counters %lld (limit %d): beyond the built-in scratch; use fewer splits or qf_attention_decode",
                 rows, QF_NOALLOC_MAX_ROWS, head_dim, QF_NOALLOC_MAX_HEAD_DIM, n_counters, QF_NOALLOC_MAX_COUNTERS);
        return QF_NOALLOC_TOO_LARGE;
    }
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= QF_NOALLOC_MAX_DEVICES) {
        snprintf(qf_noalloc_message, sizeof qf_noalloc_message, "qf_attention_decode_noalloc: device index %d not supported", device);
        return (int)cudaErrorInvalidDevice;
    }
    if (!qf_noalloc_ptr[device]) {
        // Set-up, once per device, with that device current: in host code the array's NAME is only a host-side
        // stand-in, not something a kernel may be given; its device address has to be asked for.
        unsigned char* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, qf_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            snprintf(qf_noalloc_message, sizeof qf_noalloc_message,
                     "qf_attention_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : (int)cudaErrorInvalidSymbol;
        }
        qf_noalloc_ptr[device] = p;
    }
    float* part_o = reinterpret_cast<float*>(qf_noalloc_ptr[device]);
    float* part_ml = part_o + QF_NOALLOC_PART_O_FLOATS;
    int* counters = reinterpret_cast<int*>(part_ml + QF_NOALLOC_PART_ML_FLOATS);
    void* plan = counters + QF_NOALLOC_MAX_COUNTERS;  // 16-byte aligned: every part before it is a multiple of 16 bytes
    if (n_splits > 1) {
        // the array keeps whatever the last call left: the ticket counters must start at zero
        e = cudaMemsetAsync(counters, 0, (size_t)n_counters * sizeof(int), stream);
        if (e != cudaSuccess) return (int)e;
    }
    int code = qf_attention_decode_plan(cu_q, tok_pos, slots, n_seqs, kv_heads, head_dim, n_heads, window, n_splits, plan, stream);
    if (code == 0)
        code = qf_attention_decode(q, out, cu_q, plan, base, table, page_elems, table_stride, kv_heads, head_dim, n_heads,
                                   n_seqs, scale, window, n_splits, 0, part_o, part_ml, counters, err, stream);
    if (code == (int)cudaErrorInvalidValue)
        snprintf(qf_noalloc_message, sizeof qf_noalloc_message,
                 "qf_attention_decode_noalloc: head_dim %d has no kernel (32, 64, 96, 128)", head_dim);
    return code;
}
