// Weight-streaming matrix products for a handful of token rows (decode steps): out[m][n] = sum_k x[m][k] W[n][k],
// M <= 16 rows, bf16 weights read once from HBM, with what surrounds the product fused in:
//   prologue  NORM     x = rmsnorm(hidden) * norm_weight, from the float32 residual stream (statistics in float32;
//                      the rows enter the product scaled by norm_weight, the sums are divided by the row's rms)
//   epilogue  PLAIN    out (bf16 or float32) = product (+ bias)
//             RESIDUAL hidden[m][n] += product            (the float32 residual stream, in place)
//             SWIGLU   out[m][i] = silu(gate_i) * up_i    (W = [gate rows | up rows])
//             QKV      + bias, rotate q and k heads by position (float32 angles), q -> q_out, k and v -> cache pages
//
// The product runs on the tensor cores as out^T = W x^T: 16 weight rows are the M side of an m16n8k16 tile and
// 8 token rows its N side. The kernel is a weight streamer: a block puts ALL the weight bytes it will need in
// flight at once (one bulk asynchronous copy per weight row, completing on a shared-memory barrier with a bounded
// wait), prepares its token rows while they fly, and only then multiplies. How many 16-row tiles a block takes,
// and over how many blocks of a thread-block cluster a tile's K is split, is planned on the host so that every SM
// streams and all blocks are resident in one wave. Partial sums are added in a fixed order: first the warps of a
// block, then the blocks of a cluster through distributed shared memory, so results do not change from run to run.
// It is launched as a programmatic dependent: the weight copies start while the previous kernel still runs.
// Products that do not fit one wave of blocks, or whose tiles are heavy, run in the second kernel of this file,
// which streams K through a ring of stages (see there).
// The 16 rows of a tile are chosen so that the two rows a lane holds (g and g + 8) are the pair its epilogue
// needs: component j and j + D/2 of a head for the rotation, gate row i and up row i for SwiGLU.
#include <cooperative_groups.h>

#include "skinny_common.cuh"

// Shared-memory geometry of one launch, computed on the host.
struct SkinnyPlan {
    int tpb;       // 16-row weight tiles per block
    int ksplit;    // blocks of a cluster that share a tile, each taking a slice of K
    int per;       // k-blocks (of 32) per slice
    int stride_w;  // bytes between weight rows in shared memory (16 modulo 128: conflict-free ldmatrix)
    int stride_x;  // bytes between token rows in shared memory (16 modulo 128: conflict-free fragment loads)
    int nblk;      // blocks (clusters) launched
};

template <int NT, int EPI, bool NORM>
__global__ void __launch_bounds__(SK_THREADS, 3) skinny_gemm_kernel(const SkinnyArgs a, const SkinnyPlan plan) {
    namespace cg = cooperative_groups;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t w_bar[1];
    __shared__ float ss_s[16];       // NORM: sum of squares of each token row over this block's slice
    __shared__ float ss_part[7][16]; // NORM: the same of the other blocks of the cluster, written into the first block
    __shared__ int pos_s[16];        // QKV: position of each token row
    __shared__ long long dst_s[16];  // QKV: element offset of the row's (page, position) in the cache, -1: nothing to write
    constexpr int MP = 8 * NT;
    const int tpb = plan.tpb, ksplit = plan.ksplit, per = plan.per;
    // weights [tpb * 16][stride_w]; the partial sums of the warps, red [SK_WARPS][NT * 4][32] floats, take their place
    // once the products are done
    const size_t w_bytes = max((size_t)tpb * 16 * plan.stride_w, (size_t)SK_WARPS * NT * 4 * 32 * 4);
    unsigned char* w_base = smem_raw;
    unsigned char* x_s = w_base + w_bytes;                                     // [MP][stride_x]
    float* part = reinterpret_cast<float*>(x_s + (size_t)MP * plan.stride_x);  // [ksplit - 1][tpb][NT * 4][32]
    float* red = reinterpret_cast<float*>(w_base);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int rank = ksplit > 1 ? (int)(blockIdx.x % ksplit) : 0;
    const int block0 = blockIdx.x / ksplit;
    const int n_kb = (a.k + 31) / 32;
    const int kb_begin = rank * per, kb_count = max(0, min(per, n_kb - kb_begin));
    const int k_begin = kb_begin * 32;
    const int kslice = per * 32;

    // ---- the weights of a tile batch go in flight at once: one bulk asynchronous copy per weight row slice, issued by
    // the lanes of warp 0 and completing on the buffer's shared-memory barrier; the other warps zero what no copy fills
    const int slice_bytes = max(0, min(per * 64, (a.k - k_begin) * 2));  // valid bytes of a row slice (multiple of 16)
    if (warp == 0) {  // warp 0 alone touches the barriers until the block-wide barrier after the token rows are staged
        if (lane == 0) mbar_init(&w_bar[0], 1);
        __syncwarp();
    }
    {
        unsigned char* w_s = w_base;
        const int block = block0;
        if (warp == 0) {
            uint32_t mine = 0;
            for (int row = lane; row < tpb * 16; row += 32) {
                int ra, rb;
                tile_rows<EPI>(a, block * tpb + (row >> 4), row & 7, ra, rb);
                if (((row & 15) < 8 ? ra : rb) >= 0) mine += slice_bytes;
            }
            const uint32_t total = warp_sum_u32(mine);
            if (lane == 0) mbar_expect_tx(&w_bar[0], total);
            __syncwarp();
            if (slice_bytes > 0)
                for (int row = lane; row < tpb * 16; row += 32) {
                    int ra, rb;
                    tile_rows<EPI>(a, block * tpb + (row >> 4), row & 7, ra, rb);
                    const int grow = (row & 15) < 8 ? ra : rb;
                    if (grow >= 0)
                        bulk_copy_g2s(w_s + (size_t)row * plan.stride_w, a.w + (size_t)grow * a.ldw + k_begin, slice_bytes,
                                      &w_bar[0]);
                }
        } else {
            // rows that do not exist, and the tail of a slice beyond K, must be zero: they meet zero token values
            const int tail16 = (per * 64 - slice_bytes) / 16;
            for (int row = warp - 1; row < tpb * 16; row += SK_WARPS - 1) {
                int ra, rb;
                tile_rows<EPI>(a, block * tpb + (row >> 4), row & 7, ra, rb);
                const bool exists = ((row & 15) < 8 ? ra : rb) >= 0;
                const int first = exists ? slice_bytes / 16 : 0, count = exists ? tail16 : per * 4;
                for (int c = lane; c < count; c += 32)
                    *reinterpret_cast<uint4*>(w_s + (size_t)row * plan.stride_w + (size_t)(first + c) * 16) = make_uint4(0, 0, 0, 0);
            }
        }
    }
    if (EPI == EPI_QKV && threadIdx.x >= SK_THREADS - 16) {
        // Where each token row goes: positions, slots and page tables are written by copies and by kernels that are not
        // launched as programmatic dependents, so they are complete before any kernel of this chain starts, and the
        // chain of dependent loads is walked here, before the wait, instead of by the lanes that write the cache.
        const int m = threadIdx.x - (SK_THREADS - 16);
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
    grid_launch_dependents();
    grid_dependency_wait();  // weights are nobody's output; everything below reads what earlier kernels wrote

    // ---- this block's slice of the token rows, normalised on the way if asked
    if (NORM) {
        // rmsnorm(x) W^T = (x * norm_weight) W^T / rms(x): the rows go into the product scaled by the norm weights only,
        // in one pass over this block's slice, and the row's 1 / rms, a float32 scalar, multiplies the sums in the
        // epilogue. A block adds up the squares of its own slice; the blocks of a cluster add theirs in rank order.
        for (int m = warp; m < MP; m += SK_WARPS) {
            bf16* dst = reinterpret_cast<bf16*>(x_s + (size_t)m * plan.stride_x);
            float ss = 0.f;
            if (m < a.m) {
                const float* h = a.hidden + (size_t)m * a.k;
                // column c of the slice is column k_begin + c of the row; the lane handles float4 groups u * 32 + lane,
                // eight independent 16-byte loads (a.k is a multiple of 8) of the row and of the weights at a time
                for (int base = 0; base < kslice; base += 32 * 4 * 8) {
                    float4 x[8];
                    uint2 wv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int c = base + (u * 32 + lane) * 4, kk = k_begin + c;
                        const bool in = c < kslice && kk < a.k;
                        x[u] = in ? *reinterpret_cast<const float4*>(h + kk) : make_float4(0.f, 0.f, 0.f, 0.f);
                        wv[u] = in ? *reinterpret_cast<const uint2*>(a.norm_w + kk) : make_uint2(0u, 0u);
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int c = base + (u * 32 + lane) * 4;
                        if (c >= kslice) continue;
                        ss += x[u].x * x[u].x + x[u].y * x[u].y + x[u].z * x[u].z + x[u].w * x[u].w;
                        const __nv_bfloat162 w01 = *reinterpret_cast<const __nv_bfloat162*>(&wv[u].x);
                        const __nv_bfloat162 w23 = *reinterpret_cast<const __nv_bfloat162*>(&wv[u].y);
                        uint2 o;
                        o.x = pack_bf16(x[u].x * __low2float(w01), x[u].y * __high2float(w01));
                        o.y = pack_bf16(x[u].z * __low2float(w23), x[u].w * __high2float(w23));
                        *reinterpret_cast<uint2*>(dst + c) = o;
                    }
                }
            } else {
                for (int c = lane; c < kslice; c += 32) dst[c] = __float2bfloat16_rn(0.f);
            }
            ss = warp_sum(ss);
            if (lane == 0) ss_s[m] = ss;
        }
    } else {
        const int chunks = kslice / 8;
        for (int i = threadIdx.x; i < MP * chunks; i += SK_THREADS) {
            const int m = i / chunks, c = (i % chunks) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (m < a.m && k_begin + c < a.k) v = *reinterpret_cast<const uint4*>(a.x + (size_t)m * a.ldx + k_begin + c);
            *reinterpret_cast<uint4*>(x_s + (size_t)m * plan.stride_x + c * 2) = v;
        }
    }
    __syncthreads();  // the token rows are staged
    const int wpt = SK_WARPS / tpb, tile_local = warp / wpt, sub = warp % wpt;
    const bool tile_leader = sub == 0;
    const unsigned char* w_s = w_base;
    const int block = block0;
    // What the epilogue reads from global memory is asked for now, so that it ends in stores, not in round trips
    EpiloguePre<NT> pre;
    if (tile_leader && rank == 0) skinny_epilogue_prefetch<NT, EPI>(a, block * tpb + tile_local, g, t, pre);
    if (!mbar_wait(&w_bar[0], 0) && lane == 0) atomicOr(a.err, QF_ERR_COPY_TIMEOUT);

    // ---- products: the warps of a tile take its k-blocks in turn
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const unsigned char* w_tile = w_s + (size_t)tile_local * 16 * plan.stride_w;
    const unsigned char* a_addr = w_tile + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * plan.stride_w + (lane >> 4) * 16;
    const unsigned char* x_lane = x_lane_address(x_s, plan.stride_x, lane, NT > 1);
    for (int kb = sub; kb < kb_count; kb += wpt) mma_k_block<NT>(acc, a_addr, x_lane, plan.stride_x, kb * 32);
    // ---- sum the warps of each tile in a fixed order, then the blocks of the cluster in rank order
    __syncthreads();  // every warp is done with this buffer's weights
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[((size_t)warp * NT * 4 + nt * 4 + e) * 32 + lane] = acc[nt][e];
    __syncthreads();
    if (tile_leader) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float s = 0.f;
                for (int w = 0; w < wpt; ++w) s += red[((size_t)(warp + w) * NT * 4 + nt * 4 + e) * 32 + lane];
                acc[nt][e] = s;
            }
    }
    if (ksplit > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        if (rank > 0 && tile_leader) {
            float* remote = cluster.map_shared_rank(part, 0) + ((size_t)(rank - 1) * tpb + tile_local) * NT * 4 * 32;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) remote[(nt * 4 + e) * 32 + lane] = acc[nt][e];
        }
        if (NORM && rank > 0 && threadIdx.x < MP) cluster.map_shared_rank(&ss_part[0][0], 0)[(rank - 1) * 16 + threadIdx.x] = ss_s[threadIdx.x];
        cluster.sync();
        if (rank == 0 && tile_leader) {
            for (int r = 1; r < ksplit; ++r) {
                const float* p = part + ((size_t)(r - 1) * tpb + tile_local) * NT * 4 * 32;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[nt][e] += p[(nt * 4 + e) * 32 + lane];
            }
        }
    }
    if (tile_leader && rank == 0)
        skinny_epilogue<NT, EPI, NORM>(a, block * tpb + tile_local, g, t, acc, pre, ss_s, ss_part, ksplit, pos_s, dst_s);
}

// ------------------------------------------------------------------------------------------------------------------
// The same products for weights that are too many for one wave of blocks (wide layers, the vocabulary): one block
// per SM walks its share of the 16-row tiles, and a tile's K comes in chunks of 1,024 columns through a ring of
// shared-memory stages. A ninth warp does nothing but fetch: it keeps the ring full across chunk and tile
// boundaries (bulk asynchronous copies, a 'full' barrier per stage counting bytes), so the memory pipe does not
// wait for the products; the eight product warps take the k-blocks of a chunk in turn, hand the stage back through
// its 'empty' barrier (one arrival per warp) and meet only at the end of a tile, to add up their sums and run the
// epilogue. There is no split of K over blocks and no cluster. The token rows stay in shared memory for the whole
// kernel, normalised as in the kernel above; when they are too long for that (a feed-forward's second product),
// their chunks travel through the ring beside the weights' (XS; rows that need the norm cannot).
// Requirements beyond the kernel above: K a multiple of 32.
struct StreamPlan {
    int stages;    // ring depth
    int n_chunks;  // chunks of SK_CHUNK columns per tile
    int stride_x;  // bytes between token rows in shared memory when they are resident
    int nblk;      // blocks launched; block b takes tiles b, b + nblk, ...
};
#define SK_STREAM_THREADS (SK_THREADS + 32)

template <int NT, int EPI, bool NORM, bool XS>
__global__ void __launch_bounds__(SK_STREAM_THREADS, 1) skinny_stream_kernel(const SkinnyArgs a, const StreamPlan plan, int tiles) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int MP = 8 * NT;
    constexpr int STAGE_ROWS = 16 + (XS ? MP : 0);
    constexpr int STAGE_BYTES = STAGE_ROWS * SK_STAGE_STRIDE;
    constexpr int MAX_STAGES = 16;
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES];
    __shared__ float ss_s[16];
    __shared__ int pos_s[16];
    __shared__ long long dst_s[16];
    const int stages = plan.stages, n_chunks = plan.n_chunks;
    unsigned char* ring = smem_raw;                                      // [stages][STAGE_ROWS][SK_STAGE_STRIDE]
    unsigned char* x_s = ring + (size_t)stages * STAGE_BYTES;            // [MP][stride_x] (not XS)
    float* red = reinterpret_cast<float*>(x_s + (XS ? 0 : (size_t)MP * plan.stride_x));  // [SK_WARPS][NT * 4][32]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int n_kb = a.k / 32;

    if (threadIdx.x == 0)
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], SK_WARPS);
        }
    if (EPI == EPI_QKV && threadIdx.x >= SK_THREADS - 16 && threadIdx.x < SK_THREADS) {
        // where each token row goes (see the kernel above: complete before any kernel of this chain starts)
        const int m = threadIdx.x - (SK_THREADS - 16);
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
    __syncthreads();  // barriers and row metadata are set; the only block-wide barrier of the kernel
    grid_launch_dependents();

    if (warp == SK_WARPS) {
        // ---- the fetching warp: lanes 0..15 copy the 16 weight rows of a stage, lanes 16.. the token rows (XS)
        if (XS) grid_dependency_wait();  // the token rows are the previous kernel's output; the weights are nobody's
        int idx = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += plan.nblk) {
            int ra, rb;
            tile_rows<EPI>(a, tile, lane & 7, ra, rb);
            const int grow = lane < 16 ? (lane < 8 ? ra : rb) : -1;
            const int xrow = (XS && lane >= 16 && lane - 16 < a.m) ? lane - 16 : -1;
            const unsigned rows_mask = __ballot_sync(0xffffffffu, grow >= 0 || xrow >= 0);
            for (int c = 0; c < n_chunks; ++c, ++idx) {
                const int s = idx % stages;
                if (idx >= stages && !mbar_wait(&empty_bar[s], ((idx / stages) - 1) & 1)) {
                    if (lane == 0) atomicOr(a.err, QF_ERR_COPY_TIMEOUT);
                    return;
                }
                const uint32_t bytes = (uint32_t)min(SK_CHUNK, a.k - c * SK_CHUNK) * 2;
                unsigned char* stage = ring + (size_t)s * STAGE_BYTES;
                if (lane == 0) mbar_expect_tx(&full_bar[s], bytes * __popc(rows_mask));
                __syncwarp();
                if (grow >= 0)
                    bulk_copy_g2s(stage + (size_t)lane * SK_STAGE_STRIDE, a.w + (size_t)grow * a.ldw + (size_t)c * SK_CHUNK, bytes, &full_bar[s]);
                if (xrow >= 0)
                    bulk_copy_g2s(stage + (size_t)(16 + xrow) * SK_STAGE_STRIDE, a.x + (size_t)xrow * a.ldx + (size_t)c * SK_CHUNK, bytes,
                                  &full_bar[s]);
            }
        }
        return;
    }

    // ---- the eight product warps
    grid_dependency_wait();
    if (!XS) {
        const int kpad = a.k;  // a multiple of 32: whole k-blocks, no padding needed
        if (NORM) {
            // as in the kernel above: the rows enter scaled by the norm weights, 1 / rms multiplies the sums at the end
            for (int m = warp; m < MP; m += SK_WARPS) {
                bf16* dst = reinterpret_cast<bf16*>(x_s + (size_t)m * plan.stride_x);
                float ss = 0.f;
                if (m < a.m) {
                    const float* h = a.hidden + (size_t)m * a.k;
                    for (int base = 0; base < kpad; base += 32 * 4 * 8) {
                        float4 x[8];
                        uint2 wv[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const int c = base + (u * 32 + lane) * 4;
                            const bool in = c < a.k;
                            x[u] = in ? *reinterpret_cast<const float4*>(h + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                            wv[u] = in ? *reinterpret_cast<const uint2*>(a.norm_w + c) : make_uint2(0u, 0u);
                        }
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const int c = base + (u * 32 + lane) * 4;
                            if (c >= kpad) continue;
                            ss += x[u].x * x[u].x + x[u].y * x[u].y + x[u].z * x[u].z + x[u].w * x[u].w;
                            const __nv_bfloat162 w01 = *reinterpret_cast<const __nv_bfloat162*>(&wv[u].x);
                            const __nv_bfloat162 w23 = *reinterpret_cast<const __nv_bfloat162*>(&wv[u].y);
                            uint2 o;
                            o.x = pack_bf16(x[u].x * __low2float(w01), x[u].y * __high2float(w01));
                            o.y = pack_bf16(x[u].z * __low2float(w23), x[u].w * __high2float(w23));
                            *reinterpret_cast<uint2*>(dst + c) = o;
                        }
                    }
                } else {
                    for (int c = lane * 8; c < kpad; c += 32 * 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
                }
                ss = warp_sum(ss);
                if (lane == 0) ss_s[m] = ss;
            }
        } else {
            const int chunks = kpad / 8;
            for (int i = threadIdx.x; i < MP * chunks; i += SK_THREADS) {
                const int m = i / chunks, c = (i % chunks) * 8;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (m < a.m && c < a.k) v = *reinterpret_cast<const uint4*>(a.x + (size_t)m * a.ldx + c);
                *reinterpret_cast<uint4*>(x_s + (size_t)m * plan.stride_x + c * 2) = v;
            }
        }
        consumer_barrier();  // the token rows are staged
    }
    int idx = 0;
    bool dead = false;  // a wait ran out: reported; the warp goes on without waiting, so that every barrier is still met
    for (int tile = blockIdx.x; tile < tiles; tile += plan.nblk) {
        EpiloguePre<NT> pre;
        if (warp < NT) skinny_epilogue_prefetch<NT, EPI>(a, tile, g, t, pre);
        float acc[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        for (int c = 0; c < n_chunks; ++c, ++idx) {
            const int s = idx % stages;
            if (!dead && !mbar_wait(&full_bar[s], (idx / stages) & 1)) {
                if (lane == 0) atomicOr(a.err, QF_ERR_COPY_TIMEOUT);
                dead = true;
            }
            const unsigned char* stage = ring + (size_t)s * STAGE_BYTES;
            const unsigned char* a_addr = stage + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * SK_STAGE_STRIDE + (lane >> 4) * 16;
            const unsigned char* x_base = XS ? stage + (size_t)16 * SK_STAGE_STRIDE : x_s + (size_t)c * SK_CHUNK * 2;
            const int x_stride = XS ? SK_STAGE_STRIDE : plan.stride_x;
            const int kbs = min(SK_CHUNK / 32, n_kb - c * (SK_CHUNK / 32));
            const unsigned char* x_lane = x_lane_address(x_base, x_stride, lane, NT > 1);
            for (int kb = warp; kb < kbs; kb += SK_WARPS) mma_k_block<NT>(acc, a_addr, x_lane, x_stride, kb * 32);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);  // this warp is done with the stage
        }
        // ---- the tile's sums: warp w adds up the parts of n-tile w in warp order and runs that n-tile's epilogue
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) red[((size_t)warp * NT * 4 + nt * 4 + e) * 32 + lane] = acc[nt][e];
        consumer_barrier();
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            if (warp == nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float sum = 0.f;
#pragma unroll
                    for (int w = 0; w < SK_WARPS; ++w) sum += red[((size_t)w * NT * 4 + nt * 4 + e) * 32 + lane];
                    acc[nt][e] = sum;
                }
            }
        consumer_barrier();  // the parts have been read: the next tile may overwrite them
        if (warp < NT) skinny_epilogue<NT, EPI, NORM>(a, tile, g, t, acc, pre, ss_s, nullptr, 1, pos_s, dst_s, warp);
    }
}

static size_t plan_smem(const SkinnyPlan& p, int nt) {
    size_t w = (size_t)p.tpb * 16 * p.stride_w;
    const size_t red = (size_t)SK_WARPS * nt * 4 * 32 * 4;
    if (w < red) w = red;  // the partial sums take the weights' place
    return w + (size_t)8 * nt * p.stride_x + (size_t)(p.ksplit - 1) * p.tpb * nt * 4 * 32 * 4;
}

// How a product is cut into blocks of the one-wave kernel: few tiles share their K among the blocks of a cluster so
// that every SM streams weights; many tiles are grouped so that all blocks are resident at once and the norm
// prologue is not repeated more often than needed. False: the product does not fit one wave.
static bool make_plan(int k, int tiles, int nt, int sms, SkinnyPlan& p) {
    const int n_kb = (k + 31) / 32;
    const size_t budget = 200 * 1024;
    auto fill = [&](int tpb, int ksplit) {
        p.tpb = tpb;
        p.ksplit = ksplit;
        p.per = (n_kb + ksplit - 1) / ksplit;
        p.stride_w = pad_to_16_mod_128(p.per * 64);
        p.stride_x = pad_to_16_mod_128(p.per * 64);
        p.nblk = (tiles + tpb - 1) / tpb;
        return plan_smem(p, nt);
    };
    if (tiles <= sms) {
        // K is split only as far as a block's weights need it: up to 48 KB a block has them in flight long before its
        // token rows are ready, and a cluster's exchange of partial sums would only add to the chain of waits
        int ksplit = 2 * sms / tiles;
        const int by_bytes = (int)(((size_t)16 * k * 2 + 48 * 1024 - 1) / (48 * 1024));
        if (ksplit > by_bytes) ksplit = by_bytes;
        if (ksplit > 4) ksplit = 4;
        while (ksplit > 1 && (n_kb + ksplit - 1) / ksplit < 4) --ksplit;
        if (ksplit == 3) ksplit = 2;
        for (; ksplit <= 8; ksplit *= 2)
            if (fill(1, ksplit) <= budget) return true;
        return false;
    }
    // every block resident at once, in one wave
    for (int tpb = 1; tpb <= 8; tpb *= 2) {
        const size_t smem = fill(tpb, 1);
        if (smem > budget) break;
        const int resident = (int)((227 * 1024) / (smem + 1024));
        const int blocks = (tiles + tpb - 1) / tpb;
        if (blocks <= sms * (resident > 3 ? 3 : resident)) return true;  // the launch bounds allow three blocks of 256 threads
    }
    // too many tiles for one wave: the streaming kernel's case
    return false;
}

// The streaming kernel's geometry for a product; false if it does not take the shape (K not a multiple of 32, or
// token rows that need the norm and do not fit beside three stages of the ring).
static bool make_stream_plan(int k, int tiles, int nt, bool norm, int sms, StreamPlan& sp, bool& xs, size_t& smem) {
    const size_t most = 224 * 1024;
    if (k % 32) return false;
    sp.n_chunks = (k + SK_CHUNK - 1) / SK_CHUNK;
    sp.stride_x = pad_to_16_mod_128(k * 2);
    sp.nblk = tiles < sms ? tiles : sms;
    const size_t red = (size_t)SK_WARPS * nt * 4 * 32 * 4, x_bytes = (size_t)8 * nt * sp.stride_x;
    // the token rows stay in shared memory while that leaves the ring four stages (three when they need the norm and
    // so cannot travel); rows that need no norm may travel through the ring instead
    const size_t stage = (size_t)16 * SK_STAGE_STRIDE, stage_xs = (size_t)(16 + 8 * nt) * SK_STAGE_STRIDE;
    const bool resident = red + x_bytes + (norm ? 3 : 4) * stage <= most;
    if (!resident && norm) return false;
    const size_t per_stage = resident ? stage : stage_xs, fixed = red + (resident ? x_bytes : 0);
    size_t stages = (most - fixed) / per_stage;
    if (stages > 16) stages = 16;
    if (stages < 3) return false;
    sp.stages = (int)stages;
    xs = !resident;
    smem = fixed + stages * per_stage;
    return true;
}

// Which kernel runs a product, and with which geometry. The one place that decides it: the launch and the
// host's question "would you take this shape" (`qf_skinny_gemm_takes`) both read it, so they cannot disagree.
enum { SK_NONE = 0, SK_WAVE = 1, SK_STREAM = 2, SK_STREAM_XS = 3 };
struct Decision {
    int kind = SK_NONE;
    int tiles = 0, nt = 1;
    SkinnyPlan wave;
    StreamPlan stream;
    size_t smem = 0;
};

// Requirements of every variant: 1 <= m <= 16; k, ldw (and ldx without the norm) multiples of 8; SWIGLU: inter a
// multiple of 8; QKV: head_dim a multiple of 16, rotation over the whole head.
static Decision decide(int epilogue, bool norm, const SkinnyArgs& a, int sms) {
    Decision d;
    if (sms <= 0 || a.m < 1 || a.m > 16 || a.k % 8 || a.ldw % 8 || a.k <= 0 || a.n <= 0) return d;
    if (!norm && a.ldx % 8) return d;
    switch (epilogue) {
        case EPI_PLAIN:
        case EPI_RESIDUAL:
            d.tiles = (a.n + 15) / 16;
            break;
        case EPI_SWIGLU:
            if (a.inter <= 0 || a.inter % 8 || a.n != 2 * a.inter) return d;
            d.tiles = a.inter / 8;
            break;
        case EPI_QKV:
            if (a.head_dim <= 0 || a.head_dim % 16 || (a.inv_freq && a.rot_dim != a.head_dim) ||
                a.n != (a.n_heads + 2 * a.kv_heads) * a.head_dim)
                return d;
            d.tiles = (a.n_heads + 2 * a.kv_heads) * (a.head_dim / 16);
            break;
        default:
            return d;
    }
    d.nt = a.m <= 8 ? 1 : 2;
    const bool planned = make_plan(a.k, d.tiles, d.nt, sms, d.wave);
    // The streaming kernel takes what does not fit one wave of blocks; and products of at least half as many tiles as
    // SMs whose tiles weigh 128 KB or more, where one block per tile streaming its whole K beats a cluster sharing it.
    const bool heavy_tiles = d.tiles <= sms && 2 * d.tiles > sms && (size_t)16 * a.k * 2 >= 128 * 1024;
    bool xs = false;
    if ((!planned || heavy_tiles) && make_stream_plan(a.k, d.tiles, d.nt, norm, sms, d.stream, xs, d.smem)) {
        d.kind = xs ? SK_STREAM_XS : SK_STREAM;
        return d;
    }
    if (!planned) return d;
    d.kind = SK_WAVE;
    d.smem = plan_smem(d.wave, d.nt);
    return d;
}

template <int NT, int EPI, bool NORM, bool XS>
static int launch_stream_variant(const SkinnyArgs& a, const Decision& d, cudaStream_t stream) {
    auto kernel = skinny_stream_kernel<NT, EPI, NORM, XS>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d.smem);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_pdl(kernel, dim3(d.stream.nblk), dim3(SK_STREAM_THREADS), d.smem, stream, a, d.stream, d.tiles);
}

template <int NT, int EPI, bool NORM> static int launch_one(const SkinnyArgs& a, const Decision& d, cudaStream_t stream) {
    if (d.kind == SK_STREAM) return launch_stream_variant<NT, EPI, NORM, false>(a, d, stream);
    if (d.kind == SK_STREAM_XS) return launch_stream_variant<NT, EPI, false, true>(a, d, stream);
    const SkinnyPlan& p = d.wave;
    auto kernel = skinny_gemm_kernel<NT, EPI, NORM>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d.smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(p.nblk * p.ksplit);
    config.blockDim = dim3(SK_THREADS);
    config.dynamicSmemBytes = d.smem;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = p.ksplit;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = p.ksplit > 1 ? 2 : 1;
    return (int)cudaLaunchKernelEx(&config, kernel, a, p);
}

template <int EPI, bool NORM> static int launch_epi(const SkinnyArgs& a, const Decision& d, cudaStream_t stream) {
    if (d.nt == 1) return launch_one<1, EPI, NORM>(a, d, stream);
    return launch_one<2, EPI, NORM>(a, d, stream);
}

// One entry for all variants. A shape that no kernel of this file takes returns cudaErrorInvalidValue and launches
// nothing; `qf_skinny_gemm_takes` answers the same question beforehand.
QF_EXPORT int qf_skinny_gemm(int epilogue, int norm, const SkinnyArgs* args, cudaStream_t stream) {
    const SkinnyArgs& a = *args;
    const Decision d = decide(epilogue, norm != 0, a, qf_sm_count());
    if (d.kind == SK_NONE) return (int)cudaErrorInvalidValue;
    switch (epilogue) {
        case EPI_PLAIN:
            return norm ? launch_epi<EPI_PLAIN, true>(a, d, stream) : launch_epi<EPI_PLAIN, false>(a, d, stream);
        case EPI_RESIDUAL:
            return norm ? launch_epi<EPI_RESIDUAL, true>(a, d, stream) : launch_epi<EPI_RESIDUAL, false>(a, d, stream);
        case EPI_SWIGLU:
            return norm ? launch_epi<EPI_SWIGLU, true>(a, d, stream) : launch_epi<EPI_SWIGLU, false>(a, d, stream);
        case EPI_QKV:
            return norm ? launch_epi<EPI_QKV, true>(a, d, stream) : launch_epi<EPI_QKV, false>(a, d, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// Whether `qf_skinny_gemm` would run a product of these sizes on the current device: 0 no; 1 the one-wave kernel;
// 2 the streaming kernel with the token rows resident; 3 the streaming kernel with the token rows travelling
// through the ring. Launches nothing. The sizes are those of the arguments: m token rows, weight [n][k] with rows
// `ldw` apart, input rows `ldx` apart (ignored with the norm), `inter` for SWIGLU, the head counts for QKV
// (`rotary` non-zero: the rotation is applied, over `rot_dim` components).
QF_EXPORT int qf_skinny_gemm_takes(int epilogue, int norm, int m, int n, int k, int ldw, int ldx, int inter, int n_heads,
                                   int kv_heads, int head_dim, int rotary, int rot_dim) {
    SkinnyArgs a = {};
    a.m = m;
    a.n = n;
    a.k = k;
    a.ldw = ldw;
    a.ldx = ldx;
    a.inter = inter;
    a.n_heads = n_heads;
    a.kv_heads = kv_heads;
    a.head_dim = head_dim;
    a.rot_dim = rot_dim;
    a.inv_freq = rotary ? reinterpret_cast<const float*>(&a) : nullptr;  // only tested against null
    return decide(epilogue, norm != 0, a, qf_sm_count()).kind;
}
