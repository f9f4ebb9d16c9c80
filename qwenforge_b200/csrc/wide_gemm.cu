// Weight-streaming matrix products for up to 64 token rows on the fifth-generation tensor cores (tcgen05):
//   out[m][n] = sum_k x[m][k] W[n][k],   bf16 in, float32 accumulation in tensor memory,
// computed as out^T = W x^T: 128 weight rows are the M side of `tcgen05.mma` (one accumulator lane each), the token
// rows its N side (16, 32, 48 or 64 columns of tensor memory), so a step of a few dozen sequences reads every
// weight once and wastes none of the instruction's shape. What surrounds the product is fused in, as in
// skinny_gemm.cu (whose SkinnyArgs this kernel takes; the input rows are always `x`, already normalised):
//   PLAIN     out (bf16 or float32) = product (+ bias)
//   RESIDUAL  hidden[m][n] += product                      (the float32 residual stream, in place)
//   SWIGLU    out[m][i] = silu(gate_i) * up_i
//   QKV       + bias, rotate q and k heads by position (float32 angles), q -> q_out, k and v -> cache pages
//
// One block computes one tile over its share of K. A tile is 128 weight rows and one accumulator, or, where an epilogue
// needs two weight rows together, 2 x 128 rows and two accumulators whose lane r holds the two partners: gate row r
// and up row r of 128 features (SWIGLU); component j and component j + D/2 of a head, for 256 / D heads (QKV). So the
// thread that owns lane r finishes its outputs from its own registers, and neighbouring lanes write neighbouring
// features of a token.
// Warp 8 issues the copies: per 64 columns of K a slab of the ring receives the tile's weights and the token rows by
// tiled copies of the tensor memory accelerator with the 128-byte swizzle the tensor cores read; the weights of the
// first stages are asked for before the kernel waits for the one before it (programmatic dependent launch). Warp 9
// issues the products, four of K = 16 per slab and accumulator, and `tcgen05.commit` hands the stage back. Warps 0 to
// 15 own the accumulators' lanes (warp w: lanes 32 (w % 4) .. + 31 and token columns 16 (w / 4) .. + 15; an epilogue
// is a chain of dependent instructions per token, so it is spread over as many warps as the lanes allow): while the
// weights stream they fetch what the epilogue needs (the residual values they will add to, sines and cosines of every
// token's position, where each token's key and value go), then read their sums with `tcgen05.ld` and write the results.
// Products of few tiles and a long K (a feed-forward's second product) are split along K over the blocks of a
// thread-block cluster: the tokens are dealt out to the blocks, every block sends each owner its tokens' partial sums
// through distributed shared memory, and the owners add them in rank order, so results do not change from run to run.
// Every wait on a barrier is bounded; one that runs out sets QF_ERR_COPY_TIMEOUT and the block still frees its tensor
// memory and returns. No copy uses cluster multicast.
#include <cooperative_groups.h>

#include "skinny_common.cuh"
#include "tcgen05.cuh"

#define WG_BM 128
#define WG_BK 64
#define WG_ROW_WARPS 16
#define WG_ROW_THREADS (WG_ROW_WARPS * 32)
#define WG_THREADS (WG_ROW_THREADS + 64)
#define WG_STAGES 6
#define WG_ACC_BYTES (WG_BM * WG_BK * 2)  // 16 KB of weights per slab and accumulator
#define WG_MAX_TOK 64
#define WG_MAX_SPLIT 8
#define WG_SETS (WG_ROW_WARPS / 4)
#define WG_SET_TOK (WG_MAX_TOK / WG_SETS)  // token columns of one set of row warps: 16

struct WideGeometry {
    int ntok;        // token columns of an accumulator: the row count rounded up to 16
    int tiles;       // tiles of 128 accumulator lanes
    int accs;        // accumulators of a tile: 1, or 2 where the epilogue needs two weight rows together
    int box_rows;    // weight rows of one tiled copy
    int ksplit;      // blocks of a cluster sharing a tile
    int slabs;       // 64-column slabs of K
    int slab_bytes;  // weights + token rows of one slab
    int group;       // slabs per stage of the ring
    int stage_bytes; // group * slab_bytes
    int stages;      // depth of the ring
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
__device__ __forceinline__ float wide_silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <int EPI>
__global__ void __launch_bounds__(WG_THREADS, 1)
wide_gemm_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map, const SkinnyArgs a,
                 const WideGeometry geo) {
    namespace cg = cooperative_groups;
    constexpr int ACCS = (EPI == EPI_SWIGLU || EPI == EPI_QKV) ? 2 : 1;
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
    // after the ring: the partial sums that other blocks of the cluster send (they arrive while this block may still be
    // multiplying, so they get room of their own), then the angles of QKV
    unsigned char* ring = smem;
    const int tps = ntok / ksplit;                              // tokens this block owns when K is split
    float* sums = reinterpret_cast<float*>(ring + (size_t)geo.stages * geo.stage_bytes);  // [ksplit][tps][ACCS][128]
    float* cs = sums + (ksplit > 1 ? (size_t)ntok * ACCS * WG_BM : 0);                    // QKV: [tokens][D / 2] (cos, sin)

    if (threadIdx.x == 0) {
        for (int s = 0; s < geo.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(64 * ACCS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    grid_launch_dependents();
    if (threadIdx.x == 0) stamp(geo, 1);  // barriers and tensor memory are set up
    const uint32_t tmem = tmem_base_s;
    bool timed_out = false;
    const int D = a.head_dim, P = D / 2;

    // A stage of the ring holds `group` consecutive slabs of K: its copies are issued together, slab after slab for the
    // same weight rows, so that the memory sees runs of group x 128 contiguous bytes per row.
    const int group = geo.group, stages = geo.stages, slab_bytes = geo.slab_bytes;
    const int n_groups = (n_kb + group - 1) / group;
    // what the row threads keep from before the products to after them
    int tok_base = 0, tok_step = 1, tok_count = 0;  // the tokens this thread finishes: tok_base + i * tok_step, i < tok_count
    int n0 = 0, n1 = 0;                    // the weight rows of this thread's lane in accumulator 0 and 1
    bool in0 = false;
    float bias0 = 0.f, bias1 = 0.f;

    if (warp == WG_ROW_WARPS) {
        // ---- copies. All lanes run the loop; one issues.
        const bool leader = elect_one();
        auto slabs_of = [&](int gi) { return min(group, n_kb - gi * group); };
        auto load_w = [&](int gi, int s) {
            unsigned char* base = ring + (size_t)s * geo.stage_bytes;
            const int first = kb_begin + gi * group, count = slabs_of(gi), box = geo.box_rows, boxes = WG_BM / box;
            for (int acc = 0; acc < ACCS; ++acc)
                for (int b = 0; b < boxes; ++b) {
                    int row;  // first weight row of this box
                    if (EPI == EPI_SWIGLU) row = acc * a.inter + tile * WG_BM + b * box;
                    else if (EPI == EPI_QKV) row = (tile * boxes + b) * D + acc * P;   // a box is half a head
                    else row = tile * WG_BM + b * box;
                    for (int j = 0; j < count; ++j)
                        tma_load_2d(base + (size_t)j * slab_bytes + acc * WG_ACC_BYTES + (size_t)b * box * WG_BK * 2, &w_map,
                                    (first + j) * WG_BK, row, &full_bar[s]);
                }
        };
        auto load_x = [&](int gi, int s) {
            unsigned char* base = ring + (size_t)s * geo.stage_bytes;
            const int first = kb_begin + gi * group, count = slabs_of(gi);
            for (int j = 0; j < count; ++j)
                tma_load_2d(base + (size_t)j * slab_bytes + ACCS * WG_ACC_BYTES, &x_map, (first + j) * WG_BK, 0, &full_bar[s]);
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
    } else if (warp == WG_ROW_WARPS + 1) {
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
                    const uint64_t dx = smem_desc_sw128(w_s + ACCS * WG_ACC_BYTES);
#pragma unroll
                    for (int acc = 0; acc < ACCS; ++acc) {
                        const uint64_t dw = smem_desc_sw128(w_s + acc * WG_ACC_BYTES);
#pragma unroll
                        for (int k4 = 0; k4 < WG_BK / 16; ++k4)
                            umma_bf16(tmem + 64 * acc, dw + 2 * k4, dx + 2 * k4, idesc, (gi > 0 || j > 0 || k4 > 0) ? 1u : 0u);
                    }
                }
                umma_commit(&empty_bar[s]);
            }
            __syncwarp();
        }
        if (leader) umma_commit(&acc_bar);  // arrives when every product has finished (at once if there was none)
        __syncwarp();
    } else {
        // ---- the row threads: lane r of the accumulators is weight row n0 (and its partner n1)
        const int r = (warp & 3) * 32 + lane, set = warp >> 2;
        if (EPI == EPI_SWIGLU) {
            n0 = tile * WG_BM + r;
            n1 = a.inter + n0;
            in0 = n0 < a.inter;
        } else if (EPI == EPI_QKV) {
            n0 = (tile * (WG_BM / P) + r / P) * D + r % P;
            n1 = n0 + P;
            in0 = n0 < a.n;
        } else {
            n0 = tile * WG_BM + r;
            in0 = n0 < a.n;
        }
        // the tokens this thread finishes: its set's columns, or every fourth of the tokens this block owns
        if (ksplit > 1) {
            tok_base = rank * tps + set;
            tok_step = WG_SETS;
            tok_count = (min(tps, a.m - rank * tps) - set + WG_SETS - 1) / WG_SETS;
        } else {
            tok_base = set * WG_SET_TOK;
            tok_count = min(WG_SET_TOK, a.m - tok_base);
        }
        tok_count = max(0, tok_count);
        if (a.bias && in0) {
            bias0 = __bfloat162float(a.bias[n0]);
            if (EPI == EPI_QKV) bias1 = __bfloat162float(a.bias[n1]);
        }
        grid_dependency_wait();  // the residual stream, positions and page tables may be the work of the kernel before
        if (EPI == EPI_QKV) {
            const int t = threadIdx.x;
            if (t < ntok) {
                int pos = 0;
                long long dst = -1;
                if (t < a.m) {
                    pos = a.tok_pos[t];
                    if (a.write_cache) {
                        const int slot = a.slots[a.tok_seq[t]];
                        if (slot >= 0) {
                            const int page = a.table[(long long)slot * a.table_stride + pos / QF_PAGE];
                            if (page < 0) atomicOr(a.err, QF_ERR_NO_PAGE);
                            else dst = (long long)page * a.page_elems + (long long)(pos % QF_PAGE) * D;
                        }
                    }
                }
                pos_s[t] = pos;
                dst_s[t] = dst;
            }
            row_barrier();
            if (a.inv_freq) {
                // thread t takes frequency t % P for every (512 / P)-th token: no division in the loop
                const int j = t & (P - 1), step = WG_ROW_THREADS / P;
                const float freq = a.inv_freq[j];
                for (int m = t / P; m < a.m; m += step) {
                    float sn, c;
                    sincosf((float)pos_s[m] * freq, &sn, &c);
                    cs[2 * (m * P + j)] = c;
                    cs[2 * (m * P + j) + 1] = sn;
                }
            }
            row_barrier();
        }
        if (!__all_sync(0xffffffffu, mbar_wait(&acc_bar, 0))) timed_out = true;
        tc_fence_after();
        if (threadIdx.x == 0) stamp(geo, 4);  // every product is done
        if (ksplit > 1) {
            // ---- every token's partial sums go to the block that owns the token: [sender][token][accumulator][lane].
            // Loops over tokens stay loops (four tokens per turn): unrolled over all tokens, a warp would spend its time
            // fetching instructions that it runs once.
            const int col0 = set * WG_SET_TOK;
            const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + col0;
            int owner = col0 / tps, ml = col0 % tps;  // token col0 + i belongs to block `owner`, as its token `ml`
            for (int g = 0; g < WG_SET_TOK && col0 + g < ntok; g += 4) {
                uint32_t raw[ACCS][4];
#pragma unroll
                for (int acc = 0; acc < ACCS; ++acc) {
                    if (n_kb > 0 && !timed_out) tmem_load_4(lane_base + 64 * acc + g, raw[acc]);
                    else raw[acc][0] = raw[acc][1] = raw[acc][2] = raw[acc][3] = 0u;
                }
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    float* theirs = cg::this_cluster().map_shared_rank(sums, owner) + ((rank * tps + ml) * ACCS) * WG_BM + r;
#pragma unroll
                    for (int acc = 0; acc < ACCS; ++acc) theirs[acc * WG_BM] = __uint_as_float(raw[acc][t]);
                    if (++ml == tps) {
                        ml = 0;
                        ++owner;
                    }
                }
            }
        }
    }
    if (threadIdx.x == 0) stamp(geo, 5);              // this block's sums are on their way to their owners (if K is split)
    if (ksplit > 1) cg::this_cluster().sync();        // every thread of every block of the cluster: all partial sums have arrived
    if (threadIdx.x == 0) stamp(geo, 6);
    if (warp < WG_ROW_WARPS) {
        // ---- the epilogue, by the thread that owns the lane (every lane walks the loops: the loads from tensor memory are
        // the whole warp's; a lane beyond the last weight row just stores nothing). What does not depend on the token is computed once; per
        // token there remain an index, the arithmetic and the store.
        const int r = (warp & 3) * 32 + lane, set = warp >> 2;
        const int head = EPI == EPI_QKV ? n0 / D : 0, j = EPI == EPI_QKV ? n0 % D : 0;
        const bool rotated = EPI == EPI_QKV && a.inv_freq != nullptr && head < a.n_heads + a.kv_heads;
        const bool is_q = head < a.n_heads;
        const long long kv_off = (long long)(head - a.n_heads) * QF_PAGE * D + j;  // keys, then values
        const int q_off = head * D + j, q_width = a.n_heads * D;
        auto finish = [&](int m, float x0, float x1) {   // token m: this lane's sum x0 (and its partner's x1)
            if (!in0) return;
            x0 += bias0;
            if (EPI == EPI_SWIGLU) {
                reinterpret_cast<bf16*>(a.out)[m * a.ldo + n0] = __float2bfloat16_rn(wide_silu(x0) * x1);
            } else if (EPI == EPI_RESIDUAL) {
                atomicAdd(a.residual + (m * a.n + n0), x0);  // nobody else adds to this element: one float32 addition, no read first
            } else if (EPI == EPI_PLAIN) {
                if (a.out_f32) reinterpret_cast<float*>(a.out)[m * a.ldo + n0] = x0;
                else reinterpret_cast<bf16*>(a.out)[m * a.ldo + n0] = __float2bfloat16_rn(x0);
            } else {  // EPI_QKV
                x1 += bias1;
                float y0 = x0, y1 = x1;
                if (rotated) {
                    const float2 angle = *reinterpret_cast<const float2*>(cs + 2 * (m * P + j));  // (cos, sin)
                    y0 = x0 * angle.x - x1 * angle.y;
                    y1 = x1 * angle.x + x0 * angle.y;
                }
                bf16* dst = nullptr;
                if (is_q) dst = a.q_out + (m * q_width + q_off);
                else if (dst_s[m] >= 0) dst = a.kv_base + (dst_s[m] + kv_off);
                if (dst) {
                    dst[0] = __float2bfloat16_rn(y0);
                    dst[P] = __float2bfloat16_rn(y1);
                }
            }
        };
        if (ksplit > 1) {
            // this block's tokens, every fourth one; the senders' values are asked for at once and added in rank order
            for (int i = 0; i < tok_count; ++i) {
                const float* mine = sums + ((set + i * WG_SETS) * ACCS) * WG_BM + r;
                float total[ACCS];
#pragma unroll
                for (int acc = 0; acc < ACCS; ++acc) {
                    float part[WG_MAX_SPLIT];
#pragma unroll
                    for (int src = 0; src < WG_MAX_SPLIT; ++src) part[src] = src < ksplit ? mine[(src * tps * ACCS + acc) * WG_BM] : 0.f;
                    total[acc] = part[0];
#pragma unroll
                    for (int src = 1; src < WG_MAX_SPLIT; ++src) total[acc] += part[src];
                }
                finish(tok_base + i * tok_step, total[0], total[ACCS - 1]);
            }
        } else {
            // this set's token columns, four per turn, straight from tensor memory
            const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + tok_base;
            for (int g = 0; g < tok_count; g += 4) {
                uint32_t raw[ACCS][4];
#pragma unroll
                for (int acc = 0; acc < ACCS; ++acc) {
                    if (n_kb > 0 && !timed_out) tmem_load_4(lane_base + 64 * acc + g, raw[acc]);
                    else raw[acc][0] = raw[acc][1] = raw[acc][2] = raw[acc][3] = 0u;
                }
#pragma unroll
                for (int t = 0; t < 4; ++t)
                    if (g + t < tok_count) finish(tok_base + g + t, __uint_as_float(raw[0][t]), __uint_as_float(raw[ACCS - 1][t]));
            }
        }
    }
    if (threadIdx.x == 0) stamp(geo, 7);  // the epilogue is done
    if (timed_out && lane == 0) atomicOr(a.err, QF_ERR_COPY_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32  %0, %1;" ::"r"(tmem), "r"(64 * ACCS));
}

// ------------------------------------------------------------------------------------------------------------------
// Host side.

// The geometry of a product, or false if this kernel does not take it: 1 <= m <= 64 token rows `x` (bf16, rows a
// multiple of 8 elements apart, 16-byte aligned), K a multiple of 8, weight rows likewise; QKV: half a head divides
// 128 lanes and is 8 rows or more, and the whole head is rotated if any of it is.
static bool wide_plan(int epilogue, const SkinnyArgs& a, int sms, WideGeometry& geo, size_t& smem) {
    if (sms <= 0 || a.m < 1 || a.m > WG_MAX_TOK || a.k <= 0 || a.k % 8 || a.ldw % 8 || a.ldx % 8 || a.n <= 0 || !a.x) return false;
    if (((uintptr_t)a.w | (uintptr_t)a.x) % 16) return false;
    geo.accs = 1;
    geo.box_rows = 64;
    size_t angles = 0;
    switch (epilogue) {
        case EPI_PLAIN:
        case EPI_RESIDUAL:
            geo.tiles = (a.n + WG_BM - 1) / WG_BM;
            break;
        case EPI_SWIGLU:
            if (a.inter <= 0 || a.n != 2 * a.inter || a.bias) return false;
            geo.tiles = (a.inter + WG_BM - 1) / WG_BM;
            geo.accs = 2;
            break;
        case EPI_QKV: {
            const int half = a.head_dim / 2;
            if (a.head_dim < 16 || a.head_dim % 2 || half % 8 || WG_BM % half || (a.inv_freq && a.rot_dim != a.head_dim) ||
                a.n != (a.n_heads + 2 * a.kv_heads) * a.head_dim)
                return false;
            const int heads_per_tile = WG_BM / half;
            geo.tiles = (a.n_heads + 2 * a.kv_heads + heads_per_tile - 1) / heads_per_tile;
            geo.accs = 2;
            geo.box_rows = half;
            angles = 2 * (size_t)WG_MAX_TOK * half * 4;
            break;
        }
        default:
            return false;
    }
    if (geo.tiles < 1) return false;
    geo.ntok = (a.m + 15) / 16 * 16;
    geo.slabs = (a.k + WG_BK - 1) / WG_BK;
    geo.slab_bytes = geo.accs * WG_ACC_BYTES + geo.ntok * WG_BK * 2;
    // K is split over the blocks of a cluster as far as that puts more SMs to streaming, while every block still has
    // two slabs or more to multiply
    // (clusters of 8 need 8 free SMs of one processing cluster, of which a GPU of 148 SMs has about 14 at once; clusters
    // of 4 about 32: a split whose clusters do not all start together runs in two rounds and loses more than it gains)
    geo.ksplit = 1;
    while (geo.ksplit < WG_MAX_SPLIT && geo.tiles * geo.ksplit * 2 <= sms && geo.slabs >= geo.ksplit * 4 &&
           geo.tiles <= (geo.ksplit * 2 == 8 ? sms * 14 / 148 : sms * 32 / 148))
        geo.ksplit *= 2;
    const int per = (geo.slabs + geo.ksplit - 1) / geo.ksplit;
    const size_t extra = (geo.ksplit > 1 ? (size_t)geo.ntok * geo.accs * WG_BM * 4 : 0) + angles;
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
    if (!qf_make_map_bf16(&w_map, a.w, a.n, a.k, a.ldw, geo.box_rows) || !qf_make_map_bf16(&x_map, a.x, a.m, a.k, a.ldx, geo.ntok))
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

static int wide_run(int epilogue, const SkinnyArgs& a, unsigned long long* stamps, cudaStream_t stream) {
    WideGeometry geo;
    size_t smem = 0;
    if (!wide_plan(epilogue, a, qf_sm_count(), geo, smem)) return (int)cudaErrorInvalidValue;
    geo.stamps = stamps;
    switch (epilogue) {
        case EPI_PLAIN: return wide_launch<EPI_PLAIN>(a, geo, smem, stream);
        case EPI_RESIDUAL: return wide_launch<EPI_RESIDUAL>(a, geo, smem, stream);
        case EPI_SWIGLU: return wide_launch<EPI_SWIGLU>(a, geo, smem, stream);
        case EPI_QKV: return wide_launch<EPI_QKV>(a, geo, smem, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// One entry for all epilogues. cudaErrorInvalidValue: a shape this kernel does not take, nothing launched;
// cudaErrorNotSupported: the driver offers no tensor-map encoder.
QF_EXPORT int qf_wide_gemm(int epilogue, const SkinnyArgs* args, cudaStream_t stream) { return wide_run(epilogue, *args, nullptr, stream); }

// A measuring aid: the same launch, with every block writing eight nanosecond time stamps (entry, set-up done, the
// kernel before done, first stage arrived, products done, sums sent, sums arrived, epilogue done) to stamps[block][8].
QF_EXPORT int qf_wide_gemm_stamped(int epilogue, const SkinnyArgs* args, unsigned long long* stamps, cudaStream_t stream) {
    return wide_run(epilogue, *args, stamps, stream);
}

// Whether `qf_wide_gemm` would run a product of these sizes on the current device (the number of blocks it would
// launch), or 0. Launches nothing; the pointers only say whether a bias and a rotation are given, and how the rows
// are aligned.
QF_EXPORT int qf_wide_gemm_takes(int epilogue, const SkinnyArgs* args) {
    WideGeometry geo;
    size_t smem = 0;
    return wide_plan(epilogue, *args, qf_sm_count(), geo, smem) ? geo.tiles * geo.ksplit : 0;
}
