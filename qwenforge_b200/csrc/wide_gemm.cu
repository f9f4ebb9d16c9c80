// Weight-streaming matrix products for up to 64 token rows on the fifth-generation tensor cores (tcgen05):
//   out[m][n] = sum_k x[m][k] W[n][k],   bf16 in, float32 accumulation in tensor memory,
// computed as out^T = W x^T: 128 weight rows are the M side of `tcgen05.mma` (one accumulator lane each), the token
// rows its N side (16, 32, 48 or 64 columns of tensor memory), so a step of a few dozen sequences reads every
// weight once and wastes none of the instruction's shape. What surrounds the product is fused in, as in
// skinny_gemm.cu (whose SkinnyArgs this kernel takes; the input rows are always `x`, already normalised):
//   PLAIN     out (bf16 or float32) = product (+ bias)
//   RESIDUAL  hidden[m][n] += product                      (the float32 residual stream, in place)
//   SWIGLU    out[m][i] = silu(gate_i) * up_i              (a tile is 64 gate rows and the 64 matching up rows)
//   QKV       + bias, rotate q and k heads by position (float32 angles), q -> q_out, k and v -> cache pages
//             (a tile is 128 consecutive rows: whole heads, for head sizes that divide 128)
//
// One block computes one tile of 128 weight rows over its share of K. Warp 4 issues the copies: per 64 columns of K a
// stage of the ring receives the tile's weights (two boxes of 64 rows x 128 bytes) and the token rows (one box), by
// tiled copies of the tensor memory accelerator with the 128-byte swizzle the tensor cores read; the weights of the
// first stages are asked for before the kernel waits for the one before it (programmatic dependent launch). Warp 5
// issues the products, four of K = 16 per stage, and `tcgen05.commit` hands the stage back. Warps 0 to 3 own the
// accumulator's lanes: thread r reads the sums of weight row r for all token rows with `tcgen05.ld` and runs the
// sums across shared memory, token-major and with the two rows an epilogue needs together side by side (gate and up,
// component j and j + D/2 of a head); all six warps then run the epilogue, a thread per pair of rows. While the weights stream, those warps prepare what the epilogue needs
// (sines and cosines of every token's position, where each token's key and value go).
// Products of few tiles and a long K (a feed-forward's second product) are split along K over the blocks of a
// thread-block cluster: every block sends each owner its rows' partial sums through distributed shared memory, and
// the owners add them in rank order, so results do not change from run to run.
// Every wait on a barrier is bounded; one that runs out sets QF_ERR_COPY_TIMEOUT and the block still frees its tensor
// memory and returns. No copy uses cluster multicast.
#include <cooperative_groups.h>

#include "skinny_common.cuh"
#include "tcgen05.cuh"

#define WG_BM 128
#define WG_BK 64
#define WG_THREADS 192
#define WG_ROW_THREADS 128
#define WG_STAGES 6
#define WG_W_BYTES (WG_BM * WG_BK * 2)  // 16 KB of weights per stage
#define WG_MAX_TOK 64
#define WG_MAX_SPLIT 8

struct WideGeometry {
    int ntok;        // token columns of the accumulator: the row count rounded up to 16
    int tiles;       // tiles of 128 weight rows
    int ksplit;      // blocks of a cluster sharing a tile
    int slabs;       // 64-column slabs of K
    int slab_bytes;  // weights + token rows of one slab
    int group;       // slabs per stage of the ring
    int stage_bytes; // group * slab_bytes
    int stages;      // depth of the ring
    int pair_shift;  // log2 of the distance between the two tile rows an epilogue needs together
    unsigned long long* stamps;  // measuring aid: if not null, [blocks][8] nanosecond time stamps of a block's phases
};

__device__ __forceinline__ void stamp(const WideGeometry& geo, int slot) {
    if (geo.stamps) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        geo.stamps[(size_t)blockIdx.x * 8 + slot] = now;
    }
}

__device__ __forceinline__ void row_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(WG_ROW_THREADS) : "memory"); }

template <int EPI>
__global__ void __launch_bounds__(WG_THREADS, 1)
wide_gemm_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map, const SkinnyArgs a,
                 const WideGeometry geo) {
    namespace cg = cooperative_groups;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[WG_STAGES], empty_bar[WG_STAGES], acc_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int pos_s[WG_MAX_TOK];
    __shared__ long long dst_s[WG_MAX_TOK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) stamp(geo, 0);  // entry
    const int ntok = geo.ntok, ksplit = geo.ksplit;
    const int tile = blockIdx.x / ksplit, rank = blockIdx.x % ksplit;
    const int per = (geo.slabs + ksplit - 1) / ksplit;
    const int kb_begin = rank * per, kb_end = min(geo.slabs, kb_begin + per), n_kb = max(0, kb_end - kb_begin);
    // after the ring: what the epilogue exchanges (see below); the ring itself is free by then, but the partial sums of
    // other blocks of the cluster arrive while this block may still be multiplying, so they get room of their own
    unsigned char* ring = smem;
    float* extra = reinterpret_cast<float*>(ring + (size_t)geo.stages * geo.stage_bytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < geo.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(64));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    grid_launch_dependents();
    if (threadIdx.x == 0) stamp(geo, 1);  // barriers and tensor memory are set up
    const uint32_t tmem = tmem_base_s;
    bool timed_out = false;
    float v[WG_MAX_TOK];  // row threads: this lane's sums, one per token row
    const int D = a.head_dim;
    float* sums = extra;                                        // [ksplit][ntok][rows owned]: the (partial) sums, token-major
    float* cs = extra + (size_t)WG_BM * ntok;                   // QKV: [tokens][D / 2] pairs (cos, sin) of every token's angles

    // first weight row of the tile's two boxes of 64 rows
    int row0 = tile * WG_BM, row1 = row0 + 64;
    if (EPI == EPI_SWIGLU) {
        row0 = tile * 64;
        row1 = a.inter + tile * 64;
    }

    // A stage of the ring holds `group` consecutive slabs of K: its copies are issued together, slab after slab for the
    // same weight rows, so that the memory sees runs of group x 128 contiguous bytes per row instead of lone 128-byte
    // pieces a page apart (which it serves at a fraction of its bandwidth).
    const int group = geo.group, stages = geo.stages, slab_bytes = geo.slab_bytes;
    const int n_groups = (n_kb + group - 1) / group;
    if (warp == 4) {
        // ---- copies. All lanes run the loop; one issues.
        const bool leader = elect_one();
        auto slabs_of = [&](int gi) { return min(group, n_kb - gi * group); };
        auto load_w = [&](int gi, int s) {
            unsigned char* base = ring + (size_t)s * geo.stage_bytes;
            const int first = kb_begin + gi * group, count = slabs_of(gi);
            for (int half = 0; half < 2; ++half)
                for (int j = 0; j < count; ++j)
                    tma_load_2d(base + (size_t)j * slab_bytes + half * 64 * WG_BK * 2, &w_map, (first + j) * WG_BK, half ? row1 : row0,
                                &full_bar[s]);
        };
        auto load_x = [&](int gi, int s) {
            unsigned char* base = ring + (size_t)s * geo.stage_bytes;
            const int first = kb_begin + gi * group, count = slabs_of(gi);
            for (int j = 0; j < count; ++j)
                tma_load_2d(base + (size_t)j * slab_bytes + WG_W_BYTES, &x_map, (first + j) * WG_BK, 0, &full_bar[s]);
        };
        // weights are nobody's output: those of the first stages are on their way before the kernel before this one ends
        const int early = min(n_groups, stages);
        if (leader)
            for (int gi = 0; gi < early; ++gi) {
                mbar_expect_tx(&full_bar[gi], (uint32_t)(slabs_of(gi) * slab_bytes));
                load_w(gi, gi);
            }
        __syncwarp();
        grid_dependency_wait();
        if (leader) stamp(geo, 2);  // the kernel before this one is done
        if (leader)
            for (int gi = 0; gi < early; ++gi) load_x(gi, gi);
        __syncwarp();
        for (int gi = early; gi < n_groups; ++gi) {
            const int s = gi % stages;
            if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], ((gi / stages) - 1) & 1))) {
                timed_out = true;
                break;
            }
            if (leader) {
                mbar_expect_tx(&full_bar[s], (uint32_t)(slabs_of(gi) * slab_bytes));
                load_w(gi, s);
                load_x(gi, s);
            }
            __syncwarp();
        }
    } else if (warp == 5) {
        // ---- products
        const bool leader = elect_one();
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ntok >> 3) << 17) | ((uint32_t)(WG_BM >> 4) << 24);
        for (int gi = 0; gi < n_groups; ++gi) {
            const int s = gi % stages;
            if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], (gi / stages) & 1))) {
                timed_out = true;
                break;
            }
            tc_fence_after();
            if (leader && gi == 0) stamp(geo, 3);  // the first stage has arrived
            const int count = min(group, n_kb - gi * group);
            if (leader) {
                for (int j = 0; j < count; ++j) {
                    const unsigned char* w_s = ring + (size_t)s * geo.stage_bytes + (size_t)j * slab_bytes;
                    const uint64_t dw = smem_desc_sw128(w_s), dx = smem_desc_sw128(w_s + WG_W_BYTES);
#pragma unroll
                    for (int k4 = 0; k4 < WG_BK / 16; ++k4)
                        umma_bf16(tmem, dw + 2 * k4, dx + 2 * k4, idesc, (gi > 0 || j > 0 || k4 > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);
            }
            __syncwarp();
        }
        if (leader) umma_commit(&acc_bar);  // arrives when every product has finished (at once if there was none)
        __syncwarp();
    } else {
        // ---- the row threads: thread r owns accumulator lane r = weight row r of the tile
        const int r = threadIdx.x;
        if (EPI == EPI_QKV) {
            grid_dependency_wait();  // positions and page tables may be the work of the kernel before
            if (r < ntok) {
                int pos = 0;
                long long dst = -1;
                if (r < a.m) {
                    pos = a.tok_pos[r];
                    if (a.write_cache) {
                        const int slot = a.slots[a.tok_seq[r]];
                        if (slot >= 0) {
                            const int page = a.table[(long long)slot * a.table_stride + pos / QF_PAGE];
                            if (page < 0) atomicOr(a.err, QF_ERR_NO_PAGE);
                            else dst = (long long)page * a.page_elems + (long long)(pos % QF_PAGE) * D;
                        }
                    }
                }
                pos_s[r] = pos;
                dst_s[r] = dst;
            }
            row_barrier();
            if (a.inv_freq) {
                // thread r takes frequency r % (D / 2) for every (128 / (D / 2))-th token: no division in the loop
                const int half = D / 2, j = r & (half - 1), step = WG_ROW_THREADS / half;
                const float freq = a.inv_freq[j];
                for (int m = r / half; m < a.m; m += step) {
                    float sn, c;
                    sincosf((float)pos_s[m] * freq, &sn, &c);
                    cs[2 * (m * half + j)] = c;
                    cs[2 * (m * half + j) + 1] = sn;
                }
            }
            row_barrier();
        }
        if (!__all_sync(0xffffffffu, mbar_wait(&acc_bar, 0))) timed_out = true;
        tc_fence_after();
        if (threadIdx.x == 0) stamp(geo, 4);  // every product is done
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll
        for (int c0 = 0; c0 < WG_MAX_TOK; c0 += 32) {
            if (c0 < ntok && n_kb > 0 && !timed_out) {
                uint32_t raw[32];
                tmem_load_32(lane_base + c0, raw);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[c0 + i] = __uint_as_float(raw[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[c0 + i] = 0.f;
            }
        }
        // ---- every lane's sums go to the block that owns the lane's row (this block when K is not split), token-major,
        // with the two rows of a pair side by side: tile row r -> pair index (r without its bit `pair_shift`), half
        // (that bit). A pair is what an epilogue needs together: gate and up row, component j and j + D/2 of a head.
        const int lp = geo.pair_shift, P = 1 << lp;
        const int low = ((r >> (lp + 1)) << lp) | (r & (P - 1)), hi = (r >> lp) & 1;
        const int pairs_per_rank = 64 / ksplit, own = 2 * pairs_per_rank;
        const int q = low / pairs_per_rank, rl = 2 * (low % pairs_per_rank) + hi;
        float* mine = (ksplit > 1 ? cg::this_cluster().map_shared_rank(sums, q) : sums) + ((size_t)rank * ntok) * own + rl;
#pragma unroll
        for (int m = 0; m < WG_MAX_TOK; ++m)
            if (m < ntok) mine[(size_t)m * own] = v[m];
    }
    if (threadIdx.x == 0) stamp(geo, 5);  // this block's sums are on their way
    if (ksplit > 1) cg::this_cluster().sync();  // every thread of every block of the cluster: all partial sums have arrived
    else __syncthreads();
    if (threadIdx.x == 0) stamp(geo, 6);  // all sums have arrived
    {
        // ---- the owner's epilogue, by all six warps: a thread keeps one pair of rows (so that everything about the rows
        // is computed once) and walks the tokens; the threads of a warp hold neighbouring pairs, so they write
        // neighbouring features of one token
        grid_dependency_wait();  // the residual stream and the outputs belong to earlier kernels until now
        const int lp = geo.pair_shift, P = 1 << lp;
        const int ppr = 64 / ksplit, own = 2 * ppr;                      // pairs this block owns; a power of two
        const int p_local = threadIdx.x & (ppr - 1), m_first = threadIdx.x / ppr, m_step = WG_THREADS / ppr;
        const int low = rank * ppr + p_local;
        const int r_lo = ((low >> lp) << (lp + 1)) | (low & (P - 1));    // the pair's first tile row; the second is P further
        const int n0 = (EPI == EPI_SWIGLU ? tile * 64 : tile * WG_BM) + r_lo, n1 = n0 + P;
        const int width = EPI == EPI_SWIGLU ? a.inter : a.n;
        const bool in0 = n0 < width, in1 = EPI != EPI_SWIGLU && n1 < width;
        const float bias0 = (a.bias && in0) ? __bfloat162float(a.bias[n0]) : 0.f;
        const float bias1 = (a.bias && in1) ? __bfloat162float(a.bias[n1]) : 0.f;
        const float* pair_sums = sums + 2 * p_local;
        // QKV: n0 is component j < D/2 of head n0 / D (D a power of two), n1 its partner j + D/2
        const int d_shift = 31 - __clz(D > 0 ? D : 1), half = D / 2;
        const int head = EPI == EPI_QKV ? n0 >> d_shift : 0, j = EPI == EPI_QKV ? n0 & (D - 1) : 0;
        const bool rotated = EPI == EPI_QKV && a.inv_freq != nullptr && head < a.n_heads + a.kv_heads;
        constexpr int BATCH = 8;
        for (int mb = m_first; mb < a.m; mb += m_step * BATCH) {
            float x0[BATCH], x1[BATCH], res0[BATCH], res1[BATCH];
#pragma unroll
            for (int b = 0; b < BATCH; ++b) {
                const int m = mb + b * m_step;
                x0[b] = bias0;
                x1[b] = bias1;
                if (m < a.m) {
                    for (int src = 0; src < ksplit; ++src) {
                        const float2 part = *reinterpret_cast<const float2*>(pair_sums + ((size_t)src * ntok + m) * own);
                        x0[b] += part.x;
                        x1[b] += part.y;
                    }
                    if (EPI == EPI_RESIDUAL) {
                        res0[b] = in0 ? __ldcg(a.residual + (size_t)m * a.n + n0) : 0.f;
                        res1[b] = in1 ? __ldcg(a.residual + (size_t)m * a.n + n1) : 0.f;
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < BATCH; ++b) {
                const int m = mb + b * m_step;
                if (m >= a.m) break;
                if (EPI == EPI_SWIGLU) {
                    if (in0) reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + n0] = __float2bfloat16_rn(x0[b] / (1.0f + expf(-x0[b])) * x1[b]);
                } else if (EPI == EPI_RESIDUAL) {
                    if (in0) a.residual[(size_t)m * a.n + n0] = res0[b] + x0[b];
                    if (in1) a.residual[(size_t)m * a.n + n1] = res1[b] + x1[b];
                } else if (EPI == EPI_PLAIN) {
                    if (a.out_f32) {
                        float* o = reinterpret_cast<float*>(a.out) + (size_t)m * a.ldo;
                        if (in0) o[n0] = x0[b];
                        if (in1) o[n1] = x1[b];
                    } else {
                        bf16* o = reinterpret_cast<bf16*>(a.out) + (size_t)m * a.ldo;
                        if (in0) o[n0] = __float2bfloat16_rn(x0[b]);
                        if (in1) o[n1] = __float2bfloat16_rn(x1[b]);
                    }
                } else if (in0) {  // EPI_QKV
                    float y0 = x0[b], y1 = x1[b];
                    if (rotated) {
                        const float c = cs[2 * (m * half + j)], sn = cs[2 * (m * half + j) + 1];
                        y0 = x0[b] * c - x1[b] * sn;
                        y1 = x1[b] * c + x0[b] * sn;
                    }
                    bf16* dst = nullptr;
                    if (head < a.n_heads) dst = a.q_out + ((size_t)m * a.n_heads + head) * D;
                    else if (dst_s[m] >= 0) dst = a.kv_base + dst_s[m] + (long long)(head - a.n_heads) * QF_PAGE * D;  // keys, then values
                    if (dst) {
                        dst[j] = __float2bfloat16_rn(y0);
                        dst[j + half] = __float2bfloat16_rn(y1);
                    }
                }
            }
        }
    }
    if (threadIdx.x == 0) stamp(geo, 7);  // the epilogue is done
    if (timed_out && lane == 0) atomicOr(a.err, QF_ERR_COPY_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32  %0, %1;" ::"r"(tmem), "r"(64));
}

// ------------------------------------------------------------------------------------------------------------------
// Host side.

static int wide_tiles(int epilogue, const SkinnyArgs& a) {
    switch (epilogue) {
        case EPI_PLAIN:
        case EPI_RESIDUAL:
            return (a.n + WG_BM - 1) / WG_BM;
        case EPI_SWIGLU:
            if (a.inter <= 0 || a.n != 2 * a.inter || a.bias) return -1;
            return (a.inter + 63) / 64;
        case EPI_QKV:
            if (a.head_dim < 16 || WG_BM % a.head_dim || (a.inv_freq && a.rot_dim != a.head_dim) ||
                a.n != (a.n_heads + 2 * a.kv_heads) * a.head_dim)
                return -1;
            return (a.n + WG_BM - 1) / WG_BM;
    }
    return -1;
}

// The geometry of a product, or false if this kernel does not take it: 1 <= m <= 64 token rows `x` (bf16, rows a
// multiple of 8 elements apart, 16-byte aligned), K a multiple of 8, weight rows likewise.
static bool wide_plan(int epilogue, const SkinnyArgs& a, int sms, WideGeometry& geo, size_t& smem) {
    if (sms <= 0 || a.m < 1 || a.m > WG_MAX_TOK || a.k <= 0 || a.k % 8 || a.ldw % 8 || a.ldx % 8 || a.n <= 0 || !a.x) return false;
    if (((uintptr_t)a.w | (uintptr_t)a.x) % 16) return false;
    geo.tiles = wide_tiles(epilogue, a);
    if (geo.tiles < 1) return false;
    geo.ntok = (a.m + 15) / 16 * 16;
    geo.slabs = (a.k + WG_BK - 1) / WG_BK;
    geo.slab_bytes = WG_W_BYTES + geo.ntok * WG_BK * 2;
    // the rows an epilogue needs together: gate and up row (64 apart in a tile), components j and j + D/2 of a head
    int pair = 64;
    if (epilogue == EPI_QKV) pair = a.head_dim / 2;
    geo.pair_shift = 0;
    while ((1 << geo.pair_shift) < pair) ++geo.pair_shift;
    if ((1 << geo.pair_shift) != pair) return false;
    // K is split over the blocks of a cluster as far as that puts more SMs to streaming, while every block still has
    // two slabs or more to multiply
    geo.ksplit = 1;
    while (geo.ksplit < WG_MAX_SPLIT && geo.tiles * geo.ksplit * 2 <= sms && geo.slabs >= geo.ksplit * 4) geo.ksplit *= 2;
    const int per = (geo.slabs + geo.ksplit - 1) / geo.ksplit;
    size_t extra = (size_t)WG_BM * geo.ntok * 4;  // the (partial) sums on their way to the epilogue
    if (epilogue == EPI_QKV) extra += 2 * (size_t)WG_MAX_TOK * (a.head_dim / 2) * 4;
    // stages of four slabs (512 contiguous bytes per weight row and refill) while two of them fit, else of two, else one
    for (geo.group = 4; geo.group >= 1; geo.group /= 2) {
        geo.stage_bytes = geo.group * geo.slab_bytes;
        const int wanted = (per + geo.group - 1) / geo.group;
        const size_t room = 224 * 1024 - 1024 - extra;
        int fit = (int)(room / geo.stage_bytes);
        if (fit > WG_STAGES) fit = WG_STAGES;
        geo.stages = wanted < fit ? wanted : fit;
        if (geo.stages >= 2 || (geo.stages == 1 && wanted == 1)) break;
    }
    if (geo.group < 1 || geo.stages < 1) return false;
    geo.stamps = nullptr;
    smem = (size_t)geo.stages * geo.stage_bytes + extra + 1024;
    return smem <= 224 * 1024;
}

template <int EPI>
static int wide_launch(const SkinnyArgs& a, const WideGeometry& geo, size_t smem, cudaStream_t stream) {
    CUtensorMap w_map, x_map;
    if (!qf_make_map_bf16(&w_map, a.w, a.n, a.k, a.ldw, 64) || !qf_make_map_bf16(&x_map, a.x, a.m, a.k, a.ldx, geo.ntok))
        return (int)cudaErrorNotSupported;
    auto kernel = wide_gemm_kernel<EPI>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(geo.tiles * geo.ksplit);
    config.blockDim = dim3(WG_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = geo.ksplit;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = geo.ksplit > 1 ? 2 : 1;
    return (int)cudaLaunchKernelEx(&config, kernel, w_map, x_map, a, geo);
}

// One entry for all epilogues. cudaErrorInvalidValue: a shape this kernel does not take, nothing launched;
// cudaErrorNotSupported: the driver offers no tensor-map encoder.
QF_EXPORT int qf_wide_gemm(int epilogue, const SkinnyArgs* args, cudaStream_t stream) {
    WideGeometry geo;
    size_t smem = 0;
    if (!wide_plan(epilogue, *args, qf_sm_count(), geo, smem)) return (int)cudaErrorInvalidValue;
    switch (epilogue) {
        case EPI_PLAIN: return wide_launch<EPI_PLAIN>(*args, geo, smem, stream);
        case EPI_RESIDUAL: return wide_launch<EPI_RESIDUAL>(*args, geo, smem, stream);
        case EPI_SWIGLU: return wide_launch<EPI_SWIGLU>(*args, geo, smem, stream);
        case EPI_QKV: return wide_launch<EPI_QKV>(*args, geo, smem, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// A measuring aid: the same launch, with every block writing eight nanosecond time stamps (entry, set-up done, the
// kernel before done, first stage arrived, products done, sums sent, sums arrived, epilogue done) to stamps[block][8].
QF_EXPORT int qf_wide_gemm_stamped(int epilogue, const SkinnyArgs* args, unsigned long long* stamps, cudaStream_t stream) {
    WideGeometry geo;
    size_t smem = 0;
    if (!wide_plan(epilogue, *args, qf_sm_count(), geo, smem)) return (int)cudaErrorInvalidValue;
    geo.stamps = stamps;
    switch (epilogue) {
        case EPI_PLAIN: return wide_launch<EPI_PLAIN>(*args, geo, smem, stream);
        case EPI_RESIDUAL: return wide_launch<EPI_RESIDUAL>(*args, geo, smem, stream);
        case EPI_SWIGLU: return wide_launch<EPI_SWIGLU>(*args, geo, smem, stream);
        case EPI_QKV: return wide_launch<EPI_QKV>(*args, geo, smem, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// Whether `qf_wide_gemm` would run a product of these sizes on the current device (the number of blocks it would
// launch), or 0. Launches nothing; the pointers only say whether a bias and a rotation are given, and how the rows
// are aligned.
QF_EXPORT int qf_wide_gemm_takes(int epilogue, const SkinnyArgs* args) {
    WideGeometry geo;
    size_t smem = 0;
    return wide_plan(epilogue, *args, qf_sm_count(), geo, smem) ? geo.tiles * geo.ksplit : 0;
}
