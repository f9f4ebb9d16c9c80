// Matrix products for many token rows on the fifth-generation tensor cores (tcgen05), bf16 in, float32
// accumulation in tensor memory:   C[M][N] = A[M][K] * W[N][K]^T
// with the feed-forward's gate fused in:  EPI_SWIGLU writes silu(gate) * up for W = [gate rows | up rows].
//
// One block computes one 128 x 128 or 128 x 256 tile of C. Operand tiles of 128 rows x 64 columns (128 bytes per row) are
// brought into shared memory by the tensor memory accelerator (2-D tiled copies with the 128-byte swizzle that
// the tensor cores read) through a ring of stages. Thread 0 of warp 0 issues the copies, thread 0 of warp 1 issues
// the tcgen05.mma instructions (four of K = 16 per stage) whose accumulator is 128 lanes x 128 or 256 columns of
// tensor memory; `tcgen05.commit` hands a stage back when its products have been read, and signals the epilogue at the
// end. All four warps then read their 32 accumulator lanes with tcgen05.ld, apply the epilogue and store.
// Two blocks fit an SM, so one block's epilogue overlaps the other's products. Every wait on a barrier is bounded;
// a wait that runs out sets QF_ERR_COPY_TIMEOUT, and the block still frees its tensor memory and returns.
// Copies use no cluster multicast; every block loads its own tiles.
#include "tcgen05.cuh"

enum { TC_PLAIN = 0, TC_SWIGLU = 1, TC_QKV = 2 };

// What the TC_QKV epilogue needs beside the product: W = [q heads | k heads | v heads] of head_dim rows each; the sums get
// the bias, q and k heads are rotated by the token's angles (a table [tokens][head_dim / 2] of (cos, sin) made once per
// step), q goes to q_out [tokens][n_heads * head_dim], k and v to the token's place in its sequence's cache page.
struct TcQkvArgs {
    const bf16* bias;        // [(n_heads + 2 kv_heads) * head_dim] or null
    const float2* angles;    // [tokens][head_dim / 2] (cos, sin), or null: no rotation
    const int* tok_pos;
    const int* tok_seq;
    const int* slots;
    bf16* q_out;
    bf16* kv_base;
    const int* table;
    long long page_elems;
    int table_stride, n_heads, kv_heads, head_dim, write_cache;
};

// One head (or half of one) of the TC_QKV epilogue for this thread's token row: P = D / 2 rotation pairs, W of them per
// turn from tensor memory columns `col` (first halves) and `col + P` (second halves).
template <int W>
__device__ __forceinline__ void qkv_head_turn(uint32_t lane_addr, int col, int P, const float* bias_s, const float2* angle_row,
                                              int first_pair, bool rotate, bf16* dst, bool store) {
    uint32_t lo[W], hi[W];
    if constexpr (W == 32) {
        tmem_load_32(lane_addr + col, lo);
        tmem_load_32(lane_addr + col + P, hi);
    } else {
        tmem_load_16(lane_addr + col, lo);
        tmem_load_16(lane_addr + col + P, hi);
    }
    if (!store) return;
    uint32_t o1[W / 2], o2[W / 2];
#pragma unroll
    for (int j = 0; j < W; j += 2) {
        float y1[2], y2[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float x1 = __uint_as_float(lo[j + e]) + bias_s[col + j + e], x2 = __uint_as_float(hi[j + e]) + bias_s[col + P + j + e];
            if (rotate) {
                const float2 a = angle_row[first_pair + j + e];  // (cos, sin)
                y1[e] = x1 * a.x - x2 * a.y;
                y2[e] = x2 * a.x + x1 * a.y;
            } else {
                y1[e] = x1;
                y2[e] = x2;
            }
        }
        o1[j / 2] = pack_bf16(y1[0], y1[1]);
        o2[j / 2] = pack_bf16(y2[0], y2[1]);
    }
#pragma unroll
    for (int j = 0; j < W / 2; j += 4) {
        *reinterpret_cast<uint4*>(dst + first_pair + 2 * j) = make_uint4(o1[j], o1[j + 1], o1[j + 2], o1[j + 3]);
        *reinterpret_cast<uint4*>(dst + P + first_pair + 2 * j) = make_uint4(o2[j], o2[j + 1], o2[j + 2], o2[j + 3]);
    }
}

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 128
// tile width BN: 128 (three stages of 32 KB, two blocks per SM) or 256 (four stages of 48 KB, one block per SM)
template <int BN> struct TcGeometry {
    static constexpr int stages = BN == 128 ? 3 : 4;
    static constexpr int stage_bytes = (TC_BM + BN) * TC_BK * 2;
    static constexpr size_t smem = (size_t)stages * stage_bytes + 1024;
};

// Instruction descriptor: float32 accumulator, bf16 A and B, both K-major, N = BN, M = 128.
template <int BN> __device__ __forceinline__ constexpr uint32_t tc_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

template <int EPI, int BN>
__global__ void __launch_bounds__(TC_THREADS)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, bf16* __restrict__ out,
               int M, int n_out, int K, int inter, int ldo, const TcQkvArgs qa, int* err) {
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
    constexpr int TC_STAGES = TcGeometry<BN>::stages, TC_STAGE_BYTES = TcGeometry<BN>::stage_bytes;
    constexpr int HALF = BN / 2;  // TC_SWIGLU: gate columns [0, HALF), up columns [HALF, BN)
    __shared__ __align__(8) uint64_t full_bar[TC_STAGES], empty_bar[TC_STAGES], acc_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ float bias_s[EPI == TC_QKV ? BN : 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x, tile_m = blockIdx.y;
    const int n_k = (K + TC_BK - 1) / TC_BK;
    // TC_QKV: where this thread's token row stands and where its key and value go (element offset in the cache, -1: nowhere)
    long long kv_at = -1;
    auto find_row = [&]() {
        const int row = tile_m * TC_BM + warp * 32 + lane;
        if (row < M && qa.write_cache) {
            const int slot = qa.slots[qa.tok_seq[row]], pos = qa.tok_pos[row];
            if (slot >= 0) {
                const int page = qa.table[(long long)slot * qa.table_stride + pos / QF_PAGE];
                if (page < 0) atomicOr(err, QF_ERR_NO_PAGE);
                else kv_at = (long long)page * qa.page_elems + (long long)(pos % QF_PAGE) * qa.head_dim;
            }
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
    }
    if (warp == 0) {  // one warp allocates the accumulator: 128 columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(BN));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = tmem_base_s;
    bool timed_out = false;

    if (warp == 0 && lane == 0) {
        // ---- producer: fill the ring with operand tiles
        for (int kb = 0; kb < n_k && !timed_out; ++kb) {
            const int s = kb % TC_STAGES;
            if (kb >= TC_STAGES && !mbar_wait(&empty_bar[s], ((kb / TC_STAGES) - 1) & 1)) {
                timed_out = true;
                break;
            }
            unsigned char* a_s = smem + (size_t)s * TC_STAGE_BYTES;
            unsigned char* b_s = a_s + TC_BM * TC_BK * 2;
            mbar_expect_tx(&full_bar[s], TC_STAGE_BYTES);
            tma_load_2d(a_s, &map_a, kb * TC_BK, tile_m * TC_BM, &full_bar[s]);
#pragma unroll
            for (int box = 0; box < BN / 64; ++box) {  // boxes of 64 weight rows
                int w_row = tile_n * BN + 64 * box;
                if (EPI == TC_SWIGLU)  // HALF gate rows, then the HALF matching up rows
                    w_row = 64 * box < HALF ? tile_n * HALF + 64 * box : inter + tile_n * HALF + (64 * box - HALF);
                tma_load_2d(b_s + (size_t)box * 64 * TC_BK * 2, &map_b, kb * TC_BK, w_row, &full_bar[s]);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- one thread issues the products
        for (int kb = 0; kb < n_k && !timed_out; ++kb) {
            const int s = kb % TC_STAGES;
            if (!mbar_wait(&full_bar[s], (kb / TC_STAGES) & 1)) {
                timed_out = true;
                break;
            }
            tc_fence_after();
            const unsigned char* a_s = smem + (size_t)s * TC_STAGE_BYTES;
            const unsigned char* b_s = a_s + TC_BM * TC_BK * 2;
            const uint64_t da = smem_desc_sw128(a_s), db = smem_desc_sw128(b_s);
#pragma unroll
            for (int k4 = 0; k4 < TC_BK / 16; ++k4)  // 16 columns = 32 bytes = 2 units of the address field
                umma_bf16(tmem_acc, da + 2 * k4, db + 2 * k4, tc_idesc<BN>(), (kb > 0 || k4 > 0) ? 1u : 0u);
            umma_commit(&empty_bar[s]);  // arrives when these products have finished reading the stage
        }
        umma_commit(&acc_bar);           // arrives when every product has finished
    } else if (EPI == TC_QKV) {
        // the other threads use the time of the products: the tile's bias values and their rows' places in the cache
        for (int i = threadIdx.x - (threadIdx.x > 32 ? 2 : 1); i < BN; i += TC_THREADS - 2) {
            const int col = tile_n * BN + i;
            bias_s[i] = (qa.bias && col < n_out) ? __bfloat162float(qa.bias[col]) : 0.f;
        }
        find_row();
    }
    if (EPI == TC_QKV && lane == 0 && warp < 2) find_row();  // the two issuing threads' own rows
    if (timed_out) atomicOr(err, QF_ERR_COPY_TIMEOUT);
    __syncwarp();

    // ---- epilogue: warp w owns accumulator lanes (= tile rows) 32 w .. 32 w + 31
    if (!mbar_wait(&acc_bar, 0) && lane == 0) atomicOr(err, QF_ERR_COPY_TIMEOUT);
    tc_fence_after();
    const int row = tile_m * TC_BM + warp * 32 + lane;
    const uint32_t lane_base = tmem_acc + ((uint32_t)(warp * 32) << 16);
    if (EPI == TC_QKV) {
        __syncthreads();  // the tile's bias values are in shared memory
        const int D = qa.head_dim, P = D / 2, total_heads = qa.n_heads + 2 * qa.kv_heads;
        const float2* angle_row = qa.angles ? qa.angles + (size_t)row * P : nullptr;
        for (int h = 0; h < BN / D; ++h) {   // the heads of this tile (the launch made sure that heads do not straddle tiles)
            const int head = tile_n * (BN / D) + h;
            if (head >= total_heads) break;
            const bool is_q = head < qa.n_heads, rotate = angle_row != nullptr && head < qa.n_heads + qa.kv_heads;
            bf16* dst = nullptr;
            if (row < M) {
                if (is_q) dst = qa.q_out + ((size_t)row * qa.n_heads + head) * D;
                else if (kv_at >= 0) dst = qa.kv_base + kv_at + (long long)(head - qa.n_heads) * QF_PAGE * D;  // keys, then values
            }
            // the loads from tensor memory are the whole warp's: every lane walks the turns, rows without a place store nothing
            if (P >= 32) {
                for (int first = 0; first < P; first += 32)
                    qkv_head_turn<32>(lane_base, h * D + first, P, bias_s, angle_row, first, rotate, dst, dst != nullptr);
            } else {
                qkv_head_turn<16>(lane_base, h * D, P, bias_s, angle_row, 0, rotate, dst, dst != nullptr);
            }
        }
    } else if (EPI == TC_SWIGLU) {
#pragma unroll
        for (int c0 = 0; c0 < HALF; c0 += 32) {
            uint32_t g[32], u[32];
            tmem_load_32(lane_base + c0, g);
            tmem_load_32(lane_base + HALF + c0, u);
            const int col = tile_n * HALF + c0;
            if (row < M && col < n_out) {
                uint32_t packed[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
                    packed[j] = pack_bf16(g0 / (1.0f + expf(-g0)) * __uint_as_float(u[2 * j]),
                                          g1 / (1.0f + expf(-g1)) * __uint_as_float(u[2 * j + 1]));
                }
                bf16* dst = out + (size_t)row * ldo + col;
                if (col + 32 <= n_out) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                } else {
                    for (int j = 0; j < n_out - col; ++j) dst[j] = reinterpret_cast<const bf16*>(packed)[j];
                }
            }
        }
    } else {
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t v[32];
            tmem_load_32(lane_base + c0, v);
            const int col = tile_n * BN + c0;
            if (row < M && col < n_out) {
                uint32_t packed[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) packed[j] = pack_bf16(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                bf16* dst = out + (size_t)row * ldo + col;
                if (col + 32 <= n_out) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                } else {
                    for (int j = 0; j < n_out - col; ++j) dst[j] = reinterpret_cast<const bf16*>(packed)[j];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32  %0, %1;" ::"r"(tmem_acc), "r"(BN));
}

// ------------------------------------------------------------------------------------------------------------------
// The persistent form, for products of many tiles: one block per SM walks tiles of 128 x 256 (tile index = block,
// block + blocks, ...; neighbouring blocks work on the same 256 weight rows, which the L2 then serves). The ring of
// stages runs on across tiles, and the accumulator is double: while the tensor cores fill one half of tensor memory
// (256 columns) with a tile's sums, eight epilogue warps read the other half, so a tile's epilogue and the start of
// the next tile's copies hide under products. Warp 0 issues copies, warp 1 products, warps 2 to 9 own the epilogue:
// warp w reads accumulator lanes 32 (w % 4) .. + 31 (the lanes a warp may read are fixed by its number) and one half
// of the tile's columns.
#define TP_THREADS 320
#define TP_EPI_WARPS 8
#define TP_BN 256
#define TP_STAGES 4
#define TP_STAGE_BYTES ((TC_BM + TP_BN) * TC_BK * 2)

__device__ __forceinline__ float fast_silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Tile t of the persistent walk. The blocks of the grid work on neighbouring t at any time, so the order decides what
// the L2 holds: tiles go by groups of `group_n` column tiles (their weight rows together fit in a quarter of the L2),
// and inside a group the column runs fastest, so that the blocks at work share a few row tiles of A and the group's
// weights, A streams through once per group, and the weights are read once. (With the row tile running fastest over
// the whole matrix, A was read again for every column tile once it outgrew the L2: 838 instead of 330 milliseconds
// for a 32,768-token step at Qwen2.5-7B sizes.)
__device__ __forceinline__ void tile_of(int t, int m_tiles, int n_tiles, int group_n, int& tile_m, int& tile_n) {
    const int per_group = group_n * m_tiles, g = t / per_group, first = g * group_n;
    const int width = min(group_n, n_tiles - first), local = t - g * per_group;
    tile_m = local / width;
    tile_n = first + local % width;
}

template <int EPI>
__global__ void __launch_bounds__(TP_THREADS, 1)
tc_gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          bf16* __restrict__ out, int M, int n_out, int K, int inter, int ldo, int m_tiles, int n_tiles, int group_n,
                          int* err) {
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
    constexpr int HALF = TP_BN / 2;  // TC_SWIGLU: gate columns [0, HALF), up columns [HALF, BN)
    __shared__ __align__(8) uint64_t full_bar[TP_STAGES], empty_bar[TP_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_k = (K + TC_BK - 1) / TC_BK, total = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TP_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], TP_EPI_WARPS);
        }
    }
    if (warp == 0) {  // both accumulators: all 512 columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(2 * TP_BN));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    bool timed_out = false;

    if (warp == 0) {
        // ---- copies: all lanes run the loops, one issues
        const bool leader = elect_one();
        int it = 0;
        for (int t = blockIdx.x; t < total && !timed_out; t += gridDim.x) {
            int tile_m, tile_n;
            tile_of(t, m_tiles, n_tiles, group_n, tile_m, tile_n);
            for (int kb = 0; kb < n_k; ++kb, ++it) {
                const int s = it % TP_STAGES;
                if (it >= TP_STAGES && !__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], ((it / TP_STAGES) - 1) & 1))) {
                    timed_out = true;
                    break;
                }
                if (leader) {
                    unsigned char* a_s = smem + (size_t)s * TP_STAGE_BYTES;
                    unsigned char* b_s = a_s + TC_BM * TC_BK * 2;
                    mbar_expect_tx(&full_bar[s], TP_STAGE_BYTES);
                    tma_load_2d(a_s, &map_a, kb * TC_BK, tile_m * TC_BM, &full_bar[s]);
                    // two boxes of 128 weight rows: the tile's halves, or HALF gate rows and the HALF matching up rows
                    const int w_row0 = EPI == TC_SWIGLU ? tile_n * HALF : tile_n * TP_BN;
                    const int w_row1 = EPI == TC_SWIGLU ? inter + tile_n * HALF : tile_n * TP_BN + HALF;
                    tma_load_2d(b_s, &map_b, kb * TC_BK, w_row0, &full_bar[s]);
                    tma_load_2d(b_s + (size_t)HALF * TC_BK * 2, &map_b, kb * TC_BK, w_row1, &full_bar[s]);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---- products
        const bool leader = elect_one();
        int it = 0, i = 0;
        for (int t = blockIdx.x; t < total && !timed_out; t += gridDim.x, ++i) {
            const int buf = i & 1;
            if (i >= 2 && !__all_sync(0xffffffffu, mbar_wait(&acc_empty[buf], ((i >> 1) - 1) & 1))) {  // the epilogue has read this half
                timed_out = true;
                break;
            }
            tc_fence_after();
            const uint32_t acc = tmem + (uint32_t)(buf * TP_BN);
            for (int kb = 0; kb < n_k; ++kb, ++it) {
                const int s = it % TP_STAGES;
                if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], (it / TP_STAGES) & 1))) {
                    timed_out = true;
                    break;
                }
                tc_fence_after();
                if (leader) {
                    const unsigned char* a_s = smem + (size_t)s * TP_STAGE_BYTES;
                    const uint64_t da = smem_desc_sw128(a_s), db = smem_desc_sw128(a_s + TC_BM * TC_BK * 2);
#pragma unroll
                    for (int k4 = 0; k4 < TC_BK / 16; ++k4)
                        umma_bf16(acc, da + 2 * k4, db + 2 * k4, tc_idesc<TP_BN>(), (kb > 0 || k4 > 0) ? 1u : 0u);
                    umma_commit(&empty_bar[s]);
                }
                __syncwarp();
            }
            if (timed_out) break;
            if (leader) umma_commit(&acc_full[buf]);  // arrives when the tile's products have finished
            __syncwarp();
        }
    } else {
        // ---- epilogue
        const int quad = warp & 3, half = (warp - 2) >> 2;
        int i = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++i) {
            const int buf = i & 1;
            int tile_m, tile_n;
            tile_of(t, m_tiles, n_tiles, group_n, tile_m, tile_n);
            if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (i >> 1) & 1))) {
                timed_out = true;
                break;
            }
            tc_fence_after();
            const int row = tile_m * TC_BM + quad * 32 + lane;
            const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * TP_BN);
            if (EPI == TC_SWIGLU) {
#pragma unroll
                for (int c0 = half * (HALF / 2); c0 < (half + 1) * (HALF / 2); c0 += 32) {
                    uint32_t g[32], u[32];
                    tmem_load_32(lane_base + c0, g);
                    tmem_load_32(lane_base + HALF + c0, u);
                    const int col = tile_n * HALF + c0;
                    if (row < M && col < n_out) {
                        uint32_t packed[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            packed[j] = pack_bf16(fast_silu(__uint_as_float(g[2 * j])) * __uint_as_float(u[2 * j]),
                                                  fast_silu(__uint_as_float(g[2 * j + 1])) * __uint_as_float(u[2 * j + 1]));
                        bf16* dst = out + (size_t)row * ldo + col;
                        if (col + 32 <= n_out) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                        } else {
                            for (int j = 0; j < n_out - col; ++j) dst[j] = reinterpret_cast<const bf16*>(packed)[j];
                        }
                    }
                }
            } else {
#pragma unroll
                for (int c0 = half * HALF; c0 < (half + 1) * HALF; c0 += 32) {
                    uint32_t v[32];
                    tmem_load_32(lane_base + c0, v);
                    const int col = tile_n * TP_BN + c0;
                    if (row < M && col < n_out) {
                        uint32_t packed[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) packed[j] = pack_bf16(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                        bf16* dst = out + (size_t)row * ldo + col;
                        if (col + 32 <= n_out) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                        } else {
                            for (int j = 0; j < n_out - col; ++j) dst[j] = reinterpret_cast<const bf16*>(packed)[j];
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);  // this warp has read its part of the half
        }
    }
    if (timed_out && lane == 0) atomicOr(err, QF_ERR_COPY_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32  %0, %1;" ::"r"(tmem), "r"(2 * TP_BN));
}

template <int EPI>
static int launch_persistent(const CUtensorMap& map_a, const CUtensorMap& map_b, void* out, int m, int n_out, int k, int inter,
                             int ldo, int m_tiles, int n_tiles, int* err, cudaStream_t stream) {
    const size_t smem = (size_t)TP_STAGES * TP_STAGE_BYTES + 1024;
    cudaError_t e = cudaFuncSetAttribute(tc_gemm_persistent_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int total = m_tiles * n_tiles, sms = qf_sm_count();
    // column tiles whose weight rows (256 rows of k) together take about 32 MB, a quarter of the L2; 4 at least
    long long group_n = (32ll << 20) / ((long long)TP_BN * k * 2);
    group_n = group_n < 4 ? 4 : group_n > n_tiles ? n_tiles : group_n;
    tc_gemm_persistent_kernel<EPI><<<total < sms ? total : sms, TP_THREADS, smem, stream>>>(map_a, map_b, (bf16*)out, m, n_out, k, inter,
                                                                                          ldo, m_tiles, n_tiles, (int)group_n, err);
    return (int)cudaGetLastError();
}

template <int EPI, int BN>
static int launch_tc(const CUtensorMap& map_a, const CUtensorMap& map_b, void* out, int m, int n_out, int k, int inter, int ldo,
                     int* err, dim3 grid, cudaStream_t stream) {
    const size_t smem = TcGeometry<BN>::smem;
    cudaError_t e = cudaFuncSetAttribute(tc_gemm_kernel<EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    tc_gemm_kernel<EPI, BN><<<grid, TC_THREADS, smem, stream>>>(map_a, map_b, (bf16*)out, m, n_out, k, inter, ldo, TcQkvArgs{}, err);
    return (int)cudaGetLastError();
}

static int g_persistent = 1;
// A measuring aid: 0 sends every product to the one-tile-per-block kernel.
QF_EXPORT void qf_tc_gemm_set_persistent(int on) { g_persistent = on; }

// Whether a product of these sizes has tiles for every SM and so runs in the persistent kernel (n as in qf_tc_gemm).
QF_EXPORT int qf_tc_gemm_is_persistent(int epilogue, int m, int n) {
    if (!g_persistent || m <= 0 || n <= 0) return 0;
    const long long m_tiles = (m + TC_BM - 1) / TC_BM;
    const long long n_tiles = epilogue == TC_SWIGLU ? (n / 2 + 127) / 128 : (n + 255) / 256;
    return m_tiles * n_tiles >= qf_sm_count();
}

// a [m][lda], w [n][ldw] (for TC_SWIGLU: n = 2 * inter, gate rows then up rows), out [m][ldo] with n columns
// (TC_SWIGLU: inter columns). Needs k, lda, ldw, ldo multiples of 8 and 16-byte aligned bases; for TC_SWIGLU
// inter a multiple of 8. Returns cudaErrorInvalidValue for what it does not take, cudaErrorNotSupported when
// the driver has no tensor-map encoder.
QF_EXPORT int qf_tc_gemm(int epilogue, const void* a, int lda, const void* w, int ldw, void* out, int ldo, int m, int n, int k,
                         int* err, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0 || k % 8 || lda % 8 || ldw % 8 || ldo % 8) return (int)cudaErrorInvalidValue;
    if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)out) % 16) return (int)cudaErrorInvalidValue;
    CUtensorMap map_a, map_b;
    if (!qf_make_map_bf16(&map_a, a, m, k, lda, TC_BM) || !qf_make_map_bf16(&map_b, w, n, k, ldw, 64)) return (int)cudaErrorNotSupported;
    // wide tiles when there are enough of them to fill the SMs; narrow ones otherwise
    const int out_cols = epilogue == TC_SWIGLU ? n / 2 : n;
    const int m_tiles = (m + TC_BM - 1) / TC_BM;
    if (epilogue == TC_SWIGLU) {
        if (n % 2 || (n / 2) % 8) return (int)cudaErrorInvalidValue;
        const int inter = n / 2;
        const bool wide = (long long)m_tiles * ((inter + 127) / 128) >= qf_sm_count();
        if (wide && g_persistent) {
            if (!qf_make_map_bf16(&map_b, w, n, k, ldw, 128)) return (int)cudaErrorNotSupported;  // boxes of 128 weight rows
            return launch_persistent<TC_SWIGLU>(map_a, map_b, out, m, inter, k, inter, ldo, m_tiles, (inter + 127) / 128, err, stream);
        }
        return wide ? launch_tc<TC_SWIGLU, 256>(map_a, map_b, out, m, inter, k, inter, ldo, err, dim3((inter + 127) / 128, m_tiles), stream)
                    : launch_tc<TC_SWIGLU, 128>(map_a, map_b, out, m, inter, k, inter, ldo, err, dim3((inter + 63) / 64, m_tiles), stream);
    }
    if (epilogue != TC_PLAIN) return (int)cudaErrorInvalidValue;
    const bool wide = (long long)m_tiles * ((out_cols + 255) / 256) >= qf_sm_count();
    if (wide && g_persistent) {
        if (!qf_make_map_bf16(&map_b, w, n, k, ldw, 128)) return (int)cudaErrorNotSupported;
        return launch_persistent<TC_PLAIN>(map_a, map_b, out, m, n, k, 0, ldo, m_tiles, (n + 255) / 256, err, stream);
    }
    return wide ? launch_tc<TC_PLAIN, 256>(map_a, map_b, out, m, n, k, 0, ldo, err, dim3((n + 255) / 256, m_tiles), stream)
                : launch_tc<TC_PLAIN, 128>(map_a, map_b, out, m, n, k, 0, ldo, err, dim3((n + 127) / 128, m_tiles), stream);
}


// The QKV product with bias, rotation and cache write in its epilogue (see TcQkvArgs): a [m][lda] against
// w [(n_heads + 2 kv_heads) * head_dim][ldw]. Head sizes 32, 64 and 128 (whole heads per tile of 128 columns); k, lda, ldw
// multiples of 8, 16-byte aligned bases, and rows of q_out and cache pages that keep 16-byte alignment. Returns
// cudaErrorInvalidValue for what it does not take, cudaErrorNotSupported when the driver has no tensor-map encoder.
QF_EXPORT int qf_tc_gemm_qkv(const void* a, int lda, const void* w, int ldw, int m, int k, const TcQkvArgs* args, int* err,
                             cudaStream_t stream) {
    const TcQkvArgs& q = *args;
    const int d = q.head_dim, n = (q.n_heads + 2 * q.kv_heads) * d;
    if (m <= 0 || n <= 0) return 0;
    if (d != 32 && d != 64 && d != 128) return (int)cudaErrorInvalidValue;
    if (k <= 0 || k % 8 || lda % 8 || ldw % 8 || q.page_elems % 8) return (int)cudaErrorInvalidValue;
    if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)q.q_out | (uintptr_t)q.kv_base) % 16) return (int)cudaErrorInvalidValue;
    CUtensorMap map_a, map_b;
    if (!qf_make_map_bf16(&map_a, a, m, k, lda, TC_BM) || !qf_make_map_bf16(&map_b, w, n, k, ldw, 64)) return (int)cudaErrorNotSupported;
    const size_t smem = TcGeometry<128>::smem;
    cudaError_t e = cudaFuncSetAttribute(tc_gemm_kernel<TC_QKV, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((n + 127) / 128, (m + TC_BM - 1) / TC_BM);
    tc_gemm_kernel<TC_QKV, 128><<<grid, TC_THREADS, smem, stream>>>(map_a, map_b, nullptr, m, n, k, 0, 0, q, err);
    return (int)cudaGetLastError();
}
