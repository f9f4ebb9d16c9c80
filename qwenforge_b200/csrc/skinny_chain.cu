// A chain of weight-streaming products for a handful of token rows in ONE persistent kernel: up to four products
// (each with the prologue and epilogue of skinny_gemm.cu: RMSNorm on the way in; QKV + rotation + cache write,
// SwiGLU, residual add or plain on the way out), each reading what the one before it wrote. In a decoder layer that
// is: attention output projection -> gate/up -> down -> the NEXT layer's query/key/value projection.
//
// Why one kernel: as separate launches each of these products is a short chain of dependent round trips (wait for
// the previous kernel, fetch the token rows, multiply, reduce, write) during which HBM idles, whatever its bytes.
// Here one block per SM stays resident for the whole chain. Its ninth warp does nothing but fetch: it walks the
// block's share of ALL the chain's weight tiles in order and keeps a ring of shared-memory stages full (bulk
// asynchronous copies completing on a 'full' barrier per stage), so the weights of a later product stream in while an
// earlier one is still being multiplied, across the points where the products wait for one another. Those points
// are barriers over the grid: the blocks that worked on product p count themselves in, and the blocks with work in
// product p + 1 wait for the count (a generation word; the wait is bounded and reports QF_ERR_BARRIER_TIMEOUT instead
// of spinning on). The host hands out the tiles so that every block streams about the same number of bytes over the
// whole chain. Inside a product, a block's tiles go to its eight product warps: with eight or more tiles a warp
// owns a tile (no reduction, no barrier); with fewer, the warps of a group take a tile's k-blocks in turn and the
// group adds its parts in warp order, so results do not change from run to run.
// The token rows stay in shared memory for a whole product (they are refetched per product: they are the previous
// product's output). Requirements: every K a multiple of 32; at most 8 (NT = 1) or 16 (NT = 2) token rows whose
// longest K fits beside three stages of the ring; at most CH_MAX_BLOCKS blocks. All blocks must be resident at once
// (one per SM; the launch asks for no more blocks than SMs).
#include "skinny_common.cuh"

#define CH_MAX_PHASES 4
#define CH_MAX_BLOCKS 160
#define CH_THREADS (SK_THREADS + 32)
#define CH_MAX_STAGES 8
#define CH_STAGE_BYTES (16 * SK_STAGE_STRIDE)
#define CH_BARRIER_TRIES 2000000

struct ChainPhase {
    SkinnyArgs a;
    int epilogue, norm;
    int tiles;      // 16-row weight tiles of this product
    int cpt;        // chunks of SK_CHUNK columns per tile
    int producers;  // blocks that have tiles of this product: the arrivals of the barrier after it
    int pad;
};

struct ChainArgs {  // a kernel parameter: at most 4 KB
    int n_phases, stages, x_bytes;
    int repeats;  // the products are run this many times over (weights, biases and norm weights advance by the strides below)
    long long w_step[CH_MAX_PHASES], bias_step[CH_MAX_PHASES], norm_step[CH_MAX_PHASES];  // elements per repeat
    unsigned* sync;  // [0] arrivals at the running barrier, [1] generation (barriers completed since the words were zeroed)
    int* err;
    ChainPhase phase[CH_MAX_PHASES];
    unsigned short begin[CH_MAX_PHASES][CH_MAX_BLOCKS];  // first tile of block b in product p
    unsigned short count[CH_MAX_PHASES][CH_MAX_BLOCKS];  // and how many
};

static_assert(sizeof(ChainArgs) <= 4096, "the chain's arguments travel as one kernel parameter");

__device__ __forceinline__ void tile_rows_of(int epilogue, const SkinnyArgs& a, int tile, int g, int& ra, int& rb) {
    switch (epilogue) {
        case EPI_SWIGLU: tile_rows<EPI_SWIGLU>(a, tile, g, ra, rb); break;
        case EPI_QKV: tile_rows<EPI_QKV>(a, tile, g, ra, rb); break;
        default: tile_rows<EPI_PLAIN>(a, tile, g, ra, rb); break;
    }
}

__device__ __forceinline__ unsigned load_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void group_barrier(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

// What a lane's epilogue reads from global memory, asked for before the products so that the epilogue ends in
// stores. The residual values were written by other blocks earlier in this kernel: they are read past L1.
template <int NT>
__device__ __forceinline__ void chain_prefetch(int epilogue, const SkinnyArgs& a, int tile, int g, int t, EpiloguePre<NT>& pre) {
    int ra, rb;
    tile_rows_of(epilogue, a, tile, g, ra, rb);
    if (a.bias && ra >= 0) pre.bias_a = __bfloat162float(a.bias[ra]);
    if (a.bias && rb >= 0) pre.bias_b = __bfloat162float(a.bias[rb]);
    if (epilogue == EPI_QKV && a.inv_freq && ra >= 0) pre.freq = a.inv_freq[ra % a.head_dim];
    if (epilogue == EPI_RESIDUAL) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int m = 8 * nt + 2 * t + e;
                pre.res[nt][e] = (m < a.m && ra >= 0) ? __ldcg(a.residual + (size_t)m * a.n + ra) : 0.f;
                pre.res[nt][2 + e] = (m < a.m && rb >= 0) ? __ldcg(a.residual + (size_t)m * a.n + rb) : 0.f;
            }
    }
}

template <int NT>
__global__ void __launch_bounds__(CH_THREADS, 1) skinny_chain_kernel(const __grid_constant__ ChainArgs c) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int MP = 8 * NT;
    __shared__ __align__(8) uint64_t full_bar[CH_MAX_STAGES], empty_bar[CH_MAX_STAGES];
    __shared__ float ss_s[16];
    __shared__ int pos_s[16];
    __shared__ long long dst_s[16];
    __shared__ unsigned gen_s;
    __shared__ int dead_s;
    const int stages = c.stages;
    unsigned char* ring = smem_raw;                                   // [stages][16][SK_STAGE_STRIDE]
    unsigned char* x_s = ring + (size_t)stages * CH_STAGE_BYTES;      // [MP][stride_x] of the running product
    float* red = reinterpret_cast<float*>(x_s + c.x_bytes);           // [SK_WARPS][NT * 4][32]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int block = blockIdx.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], SK_WARPS);
        }
        dead_s = 0;
    }
    __syncthreads();  // the only block-wide barrier of the kernel
    grid_launch_dependents();

    if (warp == SK_WARPS) {
        // ---- the fetching warp: every weight chunk this block will multiply, in the order in which it will; weights
        // are nobody's output, so nothing here waits for another kernel or another block
        int idx = 0;
        for (int rep = 0; rep < c.repeats; ++rep)
        for (int p = 0; p < c.n_phases; ++p) {
            const ChainPhase& ph = c.phase[p];
            const bf16* w_rep = ph.a.w + (size_t)rep * c.w_step[p];
            const int t0 = c.begin[p][block], n_mine = c.count[p][block];
            for (int tile = t0; tile < t0 + n_mine; ++tile) {
                int ra, rb;
                tile_rows_of(ph.epilogue, ph.a, tile, lane & 7, ra, rb);
                const int grow = lane < 16 ? (lane < 8 ? ra : rb) : -1;
                const unsigned rows_mask = __ballot_sync(0xffffffffu, grow >= 0);
                for (int ch = 0; ch < ph.cpt; ++ch, ++idx) {
                    const int s = idx % stages;
                    if (idx >= stages && !mbar_wait(&empty_bar[s], ((idx / stages) - 1) & 1)) {
                        if (lane == 0) atomicOr(c.err, QF_ERR_COPY_TIMEOUT);
                        return;
                    }
                    const uint32_t bytes = (uint32_t)min(SK_CHUNK, ph.a.k - ch * SK_CHUNK) * 2;
                    unsigned char* stage = ring + (size_t)s * CH_STAGE_BYTES;
                    if (lane == 0) mbar_expect_tx(&full_bar[s], bytes * __popc(rows_mask));
                    __syncwarp();
                    if (grow >= 0)
                        bulk_copy_g2s(stage + (size_t)lane * SK_STAGE_STRIDE, w_rep + (size_t)grow * ph.a.ldw + (size_t)ch * SK_CHUNK,
                                      bytes, &full_bar[s]);
                }
            }
        }
        return;
    }

    // ---- the eight product warps
    grid_dependency_wait();
    if (threadIdx.x == 0) gen_s = load_acquire(c.sync + 1);
    consumer_barrier();
    const unsigned gen0 = gen_s;
    int idx = 0;
    bool dead = false;  // a wait ran out: reported; from then on nothing waits, so that the kernel still ends
    for (int rep = 0; rep < c.repeats; ++rep)
    for (int p = 0; p < c.n_phases; ++p) {
        const ChainPhase& ph = c.phase[p];
        SkinnyArgs a = ph.a;
        a.w += (size_t)rep * c.w_step[p];
        if (a.bias) a.bias += (size_t)rep * c.bias_step[p];
        if (a.norm_w) a.norm_w += (size_t)rep * c.norm_step[p];
        const int t0 = c.begin[p][block], n_mine = c.count[p][block];
        if (n_mine == 0) continue;
        const int ordinal = rep * c.n_phases + p;  // products run before this one
        if (ordinal > 0) {
            // everything the earlier products wrote: the barrier after the one before is generation gen0 + ordinal
            if (threadIdx.x == 0 && !dead) {
                bool ok = false;
                for (int i = 0; i < CH_BARRIER_TRIES; ++i) {
                    if ((int)(load_acquire(c.sync + 1) - (gen0 + (unsigned)ordinal)) >= 0) {
                        ok = true;
                        break;
                    }
                    __nanosleep(32);
                }
                if (!ok) {
                    atomicOr(c.err, QF_ERR_BARRIER_TIMEOUT);
                    dead_s = 1;
                }
                __threadfence();
            }
            consumer_barrier();
            dead = dead || dead_s != 0;
        }
        // ---- the token rows of this product, normalised on the way if asked (as in skinny_gemm.cu); read past L1
        const int stride_x = pad_to_16_mod_128(a.k * 2);
        if (ph.norm) {
            for (int m = warp; m < MP; m += SK_WARPS) {
                bf16* dst = reinterpret_cast<bf16*>(x_s + (size_t)m * stride_x);
                float ss = 0.f;
                if (m < a.m) {
                    const float* h = a.hidden + (size_t)m * a.k;
                    for (int base = 0; base < a.k; base += 32 * 4 * 8) {
                        float4 x[8];
                        uint2 wv[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const int col = base + (u * 32 + lane) * 4;
                            const bool in = col < a.k;
                            x[u] = in ? __ldcg(reinterpret_cast<const float4*>(h + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
                            wv[u] = in ? *reinterpret_cast<const uint2*>(a.norm_w + col) : make_uint2(0u, 0u);
                        }
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const int col = base + (u * 32 + lane) * 4;
                            if (col >= a.k) continue;
                            ss += x[u].x * x[u].x + x[u].y * x[u].y + x[u].z * x[u].z + x[u].w * x[u].w;
                            const __nv_bfloat162 w01 = *reinterpret_cast<const __nv_bfloat162*>(&wv[u].x);
                            const __nv_bfloat162 w23 = *reinterpret_cast<const __nv_bfloat162*>(&wv[u].y);
                            uint2 o;
                            o.x = pack_bf16(x[u].x * __low2float(w01), x[u].y * __high2float(w01));
                            o.y = pack_bf16(x[u].z * __low2float(w23), x[u].w * __high2float(w23));
                            *reinterpret_cast<uint2*>(dst + col) = o;
                        }
                    }
                } else {
                    for (int col = lane * 8; col < a.k; col += 32 * 8) *reinterpret_cast<uint4*>(dst + col) = make_uint4(0, 0, 0, 0);
                }
                ss = warp_sum(ss);
                if (lane == 0) ss_s[m] = ss;
            }
        } else {
            // eight independent 16-byte loads per thread at a time: the rows come from L2, a round trip each
            const int pieces = a.k / 8, total = MP * pieces;
            for (int base = 0; base < total; base += SK_THREADS * 8) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = base + u * SK_THREADS + threadIdx.x;
                    const int m = i / pieces, col = (i % pieces) * 8;
                    v[u] = (i < total && m < a.m) ? __ldcg(reinterpret_cast<const uint4*>(a.x + (size_t)m * a.ldx + col))
                                                   : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = base + u * SK_THREADS + threadIdx.x;
                    if (i < total) *reinterpret_cast<uint4*>(x_s + (size_t)(i / pieces) * stride_x + (i % pieces) * 16) = v[u];
                }
            }
        }
        if (ph.epilogue == EPI_QKV && threadIdx.x < 16) {
            // where each token row's key and value go (positions, slots and page tables are complete before this kernel)
            const int m = threadIdx.x;
            int pos = 0;
            long long dst = -1;
            if (m < a.m) {
                pos = a.tok_pos[m];
                if (a.write_cache) {
                    const int slot = a.slots[a.tok_seq[m]];
                    if (slot >= 0) {
                        const int page = a.table[(long long)slot * a.table_stride + pos / QF_PAGE];
                        if (page < 0) atomicOr(a.err, QF_ERR_NO_PAGE);
                        else dst = (long long)page * a.page_elems + (long long)(pos % QF_PAGE) * a.head_dim;
                    }
                }
            }
            pos_s[m] = pos;
            dst_s[m] = dst;
        }
        consumer_barrier();  // the token rows are staged

        // ---- this block's tiles of the product: eight or more, a warp owns a tile; fewer, a group of warps shares one
        int gw = 1;  // warps per tile
        if (n_mine < 8) {
            int pow2 = 1;
            while (pow2 < n_mine) pow2 *= 2;
            gw = SK_WARPS / pow2;
        }
        const int groups = SK_WARPS / gw, my_group = warp / gw, sub = warp % gw;
        const int n_kb = a.k / 32;
        for (int j = 0; j < n_mine; ++j) {
            const bool mine = j % groups == my_group;
            float acc[NT][4];
#pragma unroll
            for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
            EpiloguePre<NT> pre;
            if (mine && sub == 0) chain_prefetch<NT>(ph.epilogue, a, t0 + j, g, t, pre);
            for (int ch = 0; ch < ph.cpt; ++ch, ++idx) {
                const int s = idx % stages;
                // every warp passes every stage in order (a stage is free again once all eight have left it)
                if (!dead && !mbar_wait(&full_bar[s], (idx / stages) & 1)) {
                    if (lane == 0) atomicOr(c.err, QF_ERR_COPY_TIMEOUT);
                    dead = true;
                }
                if (mine) {
                    const unsigned char* stage = ring + (size_t)s * CH_STAGE_BYTES;
                    const unsigned char* a_addr = stage + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * SK_STAGE_STRIDE + (lane >> 4) * 16;
                    const unsigned char* x_lane = x_lane_address(x_s + (size_t)ch * SK_CHUNK * 2, stride_x, lane, NT > 1);
                    const int kbs = min(SK_CHUNK / 32, n_kb - ch * (SK_CHUNK / 32));
                    for (int kb = sub; kb < kbs; kb += gw) mma_k_block<NT>(acc, a_addr, x_lane, stride_x, kb * 32);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[s]);
            }
            if (!mine) continue;
            if (gw > 1) {
                // the group's parts, added in warp order by its first warp
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) red[((size_t)warp * NT * 4 + nt * 4 + e) * 32 + lane] = acc[nt][e];
                group_barrier(2 + my_group, gw * 32);
                if (sub == 0) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float sum = 0.f;
                            for (int w = 0; w < gw; ++w) sum += red[((size_t)(warp + w) * NT * 4 + nt * 4 + e) * 32 + lane];
                            acc[nt][e] = sum;
                        }
                }
                group_barrier(2 + my_group, gw * 32);  // the parts have been read: the group's next tile may overwrite them
            }
            if (sub == 0) {
                const int tile = t0 + j;
#define CH_EPI(E)                                                                                            \
    if (ph.norm) skinny_epilogue<NT, E, true>(a, tile, g, t, acc, pre, ss_s, nullptr, 1, pos_s, dst_s);     \
    else skinny_epilogue<NT, E, false>(a, tile, g, t, acc, pre, ss_s, nullptr, 1, pos_s, dst_s);
                switch (ph.epilogue) {
                    case EPI_PLAIN: CH_EPI(EPI_PLAIN) break;
                    case EPI_RESIDUAL: CH_EPI(EPI_RESIDUAL) break;
                    case EPI_SWIGLU: CH_EPI(EPI_SWIGLU) break;
                    default: CH_EPI(EPI_QKV) break;
                }
#undef CH_EPI
            }
        }
        // ---- this block's part of product p is written: count it in (the last product has nobody waiting)
        if (ordinal + 1 < c.repeats * c.n_phases) {
            consumer_barrier();  // also keeps the token rows until every warp is done with them
            if (threadIdx.x == 0) {
                __threadfence();
                const unsigned before = atomicAdd(c.sync, 1u);
                if (before + 1 == (unsigned)ph.producers) {
                    c.sync[0] = 0;  // the words are ready for the next barrier before anyone can reach it
                    __threadfence();
                    atomicAdd(c.sync + 1, 1u);
                }
            }
        } else {
            consumer_barrier();
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// Host side.

struct ChainProduct {  // one product of a chain, as the caller describes it
    int epilogue, norm;
    SkinnyArgs a;
};

static int tiles_of(int epilogue, const SkinnyArgs& a) {
    switch (epilogue) {
        case EPI_PLAIN:
        case EPI_RESIDUAL:
            return (a.n + 15) / 16;
        case EPI_SWIGLU:
            if (a.inter <= 0 || a.inter % 8 || a.n != 2 * a.inter) return -1;
            return a.inter / 8;
        case EPI_QKV:
            if (a.head_dim <= 0 || a.head_dim % 16 || (a.inv_freq && a.rot_dim != a.head_dim) ||
                a.n != (a.n_heads + 2 * a.kv_heads) * a.head_dim)
                return -1;
            return (a.n_heads + 2 * a.kv_heads) * (a.head_dim / 16);
    }
    return -1;
}

// Fills the kernel's arguments for a chain; false if the chain does not fit this kernel (the caller then runs the
// products one by one). The tiles are handed out product by product, heaviest tiles first, each product's tiles to
// the blocks that have streamed least so far, so that over the whole chain every block streams about the same bytes.
static bool plan_chain(const ChainProduct* products, int n, int sms, ChainArgs& c, int& nt, size_t& smem) {
    if (n < 1 || n > CH_MAX_PHASES || sms <= 0) return false;
    const int blocks = sms < CH_MAX_BLOCKS ? sms : CH_MAX_BLOCKS;
    int m = products[0].a.m, k_max = 0;
    for (int p = 0; p < n; ++p) {
        const SkinnyArgs& a = products[p].a;
        if (a.m != m || a.m < 1 || a.m > 16 || a.k <= 0 || a.k % 32 || a.ldw % 8 || a.n <= 0) return false;
        if (!products[p].norm && a.ldx % 8) return false;
        const int tiles = tiles_of(products[p].epilogue, a);
        if (tiles < 1 || tiles > 65535) return false;
        if (a.k > k_max) k_max = a.k;
        c.phase[p].a = a;
        c.phase[p].epilogue = products[p].epilogue;
        c.phase[p].norm = products[p].norm;
        c.phase[p].tiles = tiles;
        c.phase[p].cpt = (a.k + SK_CHUNK - 1) / SK_CHUNK;
    }
    nt = m <= 8 ? 1 : 2;
    const size_t most = 224 * 1024;
    const size_t x_bytes = (size_t)8 * nt * pad_to_16_mod_128(k_max * 2), red = (size_t)SK_WARPS * nt * 4 * 32 * 4;
    if (x_bytes + red + 3 * (size_t)CH_STAGE_BYTES > most) return false;
    size_t stages = (most - x_bytes - red) / CH_STAGE_BYTES;
    if (stages > CH_MAX_STAGES) stages = CH_MAX_STAGES;
    c.n_phases = n;
    c.repeats = 1;
    for (int p = 0; p < CH_MAX_PHASES; ++p) c.w_step[p] = c.bias_step[p] = c.norm_step[p] = 0;
    c.stages = (int)stages;
    c.x_bytes = (int)x_bytes;
    smem = stages * CH_STAGE_BYTES + x_bytes + red;
    // hand out the tiles: `load` counts the chunks a block streams
    long long load[CH_MAX_BLOCKS] = {0};
    int order[CH_MAX_PHASES];
    for (int p = 0; p < n; ++p) order[p] = p;
    for (int i = 0; i < n; ++i)
        for (int j = i + 1; j < n; ++j)
            if (c.phase[order[j]].cpt > c.phase[order[i]].cpt) {
                const int tmp = order[i];
                order[i] = order[j];
                order[j] = tmp;
            }
    for (int i = 0; i < n; ++i) {
        const int p = order[i], w = c.phase[p].cpt, tiles = c.phase[p].tiles;
        // the lowest level such that the blocks below it can take all tiles
        long long lo = 0, hi = 0;
        for (int b = 0; b < blocks; ++b) hi = load[b] > hi ? load[b] : hi;
        hi += (long long)w * tiles;
        while (lo < hi) {
            const long long mid = (lo + hi) / 2;
            long long can = 0;
            for (int b = 0; b < blocks; ++b) can += mid > load[b] ? (mid - load[b]) / w : 0;
            if (can >= tiles) hi = mid;
            else lo = mid + 1;
        }
        int next = 0, left = tiles, producers = 0;
        for (int b = 0; b < blocks; ++b) {
            int take = (int)(lo > load[b] ? (lo - load[b]) / w : 0);
            if (take > left) take = left;
            c.begin[p][b] = (unsigned short)next;
            c.count[p][b] = (unsigned short)take;
            next += take;
            left -= take;
            load[b] += (long long)take * w;
            producers += take > 0;
        }
        if (left != 0) return false;
        c.phase[p].producers = producers;
    }
    return true;
}

template <int NT> static int launch_chain(const ChainArgs& c, int blocks, size_t smem, cudaStream_t stream) {
    auto kernel = skinny_chain_kernel<NT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_pdl(kernel, dim3(blocks), dim3(CH_THREADS), smem, stream, c);
}

// Runs `n` products (1..4) as one chain. `sync` points to two zero-initialised 32-bit words in device memory that
// belong to this stream's chains (they come back to a consistent state after every launch); `err` to the device error
// word. cudaErrorInvalidValue: the chain does not fit this kernel and nothing was launched.
QF_EXPORT int qf_skinny_chain(int n, const ChainProduct* products, unsigned* sync, int* err, cudaStream_t stream) {
    static ChainArgs c;  // filled and copied at launch; calls come from one host thread at a time (the GIL)
    int nt = 1;
    size_t smem = 0;
    const int sms = qf_sm_count();
    if (!plan_chain(products, n, sms, c, nt, smem)) return (int)cudaErrorInvalidValue;
    c.sync = sync;
    c.err = err;
    const int blocks = sms < CH_MAX_BLOCKS ? sms : CH_MAX_BLOCKS;
    return nt == 1 ? launch_chain<1>(c, blocks, smem, stream) : launch_chain<2>(c, blocks, smem, stream);
}

// The same chain run `repeats` times over in one launch, product p's weight, bias and norm weight advancing by
// steps[p], steps[4 + p], steps[8 + p] elements per repeat (stacked tensors); every other tensor is shared by the
// repeats. A measuring aid: how fast products follow one another once the blocks are resident and streaming.
QF_EXPORT int qf_skinny_chain_repeated(int n, const ChainProduct* products, int repeats, const long long* steps, unsigned* sync,
                                       int* err, cudaStream_t stream) {
    static ChainArgs c;
    int nt = 1;
    size_t smem = 0;
    const int sms = qf_sm_count();
    if (repeats < 1 || !plan_chain(products, n, sms, c, nt, smem)) return (int)cudaErrorInvalidValue;
    c.repeats = repeats;
    for (int p = 0; p < n; ++p) {
        c.w_step[p] = steps[p];
        c.bias_step[p] = steps[4 + p];
        c.norm_step[p] = steps[8 + p];
    }
    c.sync = sync;
    c.err = err;
    const int blocks = sms < CH_MAX_BLOCKS ? sms : CH_MAX_BLOCKS;
    return nt == 1 ? launch_chain<1>(c, blocks, smem, stream) : launch_chain<2>(c, blocks, smem, stream);
}

// Whether `qf_skinny_chain` would run these products (1) or refuse them (0). Launches nothing.
QF_EXPORT int qf_skinny_chain_takes(int n, const ChainProduct* products) {
    static ChainArgs c;
    int nt = 1;
    size_t smem = 0;
    return plan_chain(products, n, qf_sm_count(), c, nt, smem) ? 1 : 0;
}
