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
// The 16 rows of a tile are chosen so that the two rows a lane holds (g and g + 8) are the pair its epilogue
// needs: component j and j + D/2 of a head for the rotation, gate row i and up row i for SwiGLU.
#include <cooperative_groups.h>

#include "mma.cuh"

enum { EPI_PLAIN = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2, EPI_QKV = 3 };

struct SkinnyArgs {
    const bf16* w;        // [N][ldw]
    const bf16* bias;     // [N] or null
    int n, k, ldw, m;
    // input rows
    const bf16* x;        // [m][ldx] (no NORM)
    int ldx;
    const float* hidden;  // [m][k] (NORM)
    const bf16* norm_w;   // [k]
    float eps;
    // outputs
    void* out;            // PLAIN: [m][ldo] bf16 or float32; SWIGLU: [m][ldo] bf16
    int ldo, out_f32;
    float* residual;      // RESIDUAL: [m][n] float32, updated in place
    int inter;            // SWIGLU: rows of gate (= rows of up)
    // QKV
    int n_heads, kv_heads, head_dim, rot_dim, write_cache;
    const float* inv_freq;
    const int* tok_pos;
    const int* tok_seq;
    const int* slots;
    bf16* q_out;          // [m][n_heads * head_dim]
    bf16* kv_base;
    const int* table;
    long long page_elems;
    int table_stride;
    int* err;
};

template <int EPI> __device__ __forceinline__ void tile_rows(const SkinnyArgs& a, int tile, int g, int& ra, int& rb) {
    if (EPI == EPI_SWIGLU) {
        ra = tile * 8 + g;
        rb = a.inter + tile * 8 + g;
        if (ra >= a.inter) ra = rb = -1;
    } else if (EPI == EPI_QKV) {
        const int per_head = a.head_dim / 16, head = tile / per_head, j = (tile % per_head) * 8 + g;
        ra = head * a.head_dim + j;
        rb = ra + a.head_dim / 2;
        if (head >= a.n_heads + 2 * a.kv_heads) ra = rb = -1;
    } else {
        ra = tile * 16 + g;
        rb = ra + 8;
        if (ra >= a.n) ra = -1;
        if (rb >= a.n) rb = -1;
    }
}

// Shared-memory geometry of one launch, computed on the host.
struct SkinnyPlan {
    int tpb;       // 16-row weight tiles per block
    int ksplit;    // blocks of a cluster that share a tile, each taking a slice of K
    int per;       // k-blocks (of 32) per slice
    int stride_w;  // bytes between weight rows in shared memory (16 modulo 128: conflict-free ldmatrix)
    int stride_x;  // bytes between token rows in shared memory (16 modulo 128: conflict-free fragment loads)
    int rounds;    // tile batches a block works through, one after another, two weight buffers in turn (1: all at once)
    int nblk;      // blocks (clusters) launched; in round r a block takes tile batch  its index + r * nblk
};

static inline int pad_to_16_mod_128(int bytes) { return bytes + ((16 - bytes % 128) + 128) % 128; }

#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)

// STREAM: the block works through several tile batches (plan.rounds > 1); without it the loop and the second
// buffer compile away.
template <int NT, int EPI, bool NORM, bool STREAM>
__global__ void __launch_bounds__(SK_THREADS, 3) skinny_gemm_kernel(const SkinnyArgs a, const SkinnyPlan plan) {
    namespace cg = cooperative_groups;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t w_bar[2];
    __shared__ float ss_s[16];       // NORM: sum of squares of each token row over this block's slice
    __shared__ float ss_part[7][16]; // NORM: the same of the other blocks of the cluster, written into the first block
    __shared__ int pos_s[16];        // QKV: position of each token row
    __shared__ long long dst_s[16];  // QKV: element offset of the row's (page, position) in the cache, -1: nothing to write
    constexpr int MP = 8 * NT;
    const int tpb = plan.tpb, ksplit = plan.ksplit, per = plan.per, rounds = STREAM ? plan.rounds : 1;
    // weights [tpb * 16][stride_w], one buffer, or two when the block works through several tile batches
    const size_t w_bytes = rounds > 1 ? (size_t)tpb * 16 * plan.stride_w
                                      : max((size_t)tpb * 16 * plan.stride_w, (size_t)SK_WARPS * NT * 4 * 32 * 4);
    unsigned char* w_base = smem_raw;
    unsigned char* x_s = w_base + (rounds > 1 ? 2 : 1) * w_bytes;            // [MP][stride_x]
    float* part = reinterpret_cast<float*>(x_s + (size_t)MP * plan.stride_x);  // [ksplit - 1][tpb][NT * 4][32]
    // partial sums of the warps, red [SK_WARPS][NT * 4][32] floats: a single tile batch lends them the weights'
    // space once its products are done; with several batches the weights stay in use and red has its own space
    float* red = rounds > 1 ? part + (size_t)(ksplit - 1) * tpb * NT * 4 * 32 : reinterpret_cast<float*>(w_base);
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
        if (lane == 0) {
            mbar_init(&w_bar[0], 1);
            mbar_init(&w_bar[1], 1);
        }
        __syncwarp();
    }
    auto fetch = [&](int round) {
        unsigned char* w_s = w_base + (size_t)(round & 1) * w_bytes;
        const int block = block0 + round * plan.nblk;
        if (warp == 0) {
            uint32_t mine = 0;
            for (int row = lane; row < tpb * 16; row += 32) {
                int ra, rb;
                tile_rows<EPI>(a, block * tpb + (row >> 4), row & 7, ra, rb);
                if (((row & 15) < 8 ? ra : rb) >= 0) mine += slice_bytes;
            }
            const uint32_t total = warp_sum_u32(mine);
            if (lane == 0) mbar_expect_tx(&w_bar[round & 1], total);
            __syncwarp();
            if (slice_bytes > 0)
                for (int row = lane; row < tpb * 16; row += 32) {
                    int ra, rb;
                    tile_rows<EPI>(a, block * tpb + (row >> 4), row & 7, ra, rb);
                    const int grow = (row & 15) < 8 ? ra : rb;
                    if (grow >= 0)
                        bulk_copy_g2s(w_s + (size_t)row * plan.stride_w, a.w + (size_t)grow * a.ldw + k_begin, slice_bytes,
                                      &w_bar[round & 1]);
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
    };
    fetch(0);
    if (rounds > 1) fetch(1);
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
    for (int round = 0; round < rounds; ++round) {
    const unsigned char* w_s = w_base + (size_t)(round & 1) * w_bytes;
    const int block = block0 + round * plan.nblk;
    // What the epilogue reads from global memory is asked for now, so that it ends in stores, not in round trips:
    // bias and rotation frequency (constants), and for RESIDUAL the values this lane will add to
    float bias_a = 0.f, bias_b = 0.f, freq = 0.f;
    if (tile_leader && rank == 0) {
        int ra, rb;
        tile_rows<EPI>(a, block * tpb + tile_local, g, ra, rb);
        if (a.bias && ra >= 0) bias_a = __bfloat162float(a.bias[ra]);
        if (a.bias && rb >= 0) bias_b = __bfloat162float(a.bias[rb]);
        if (EPI == EPI_QKV && a.inv_freq && ra >= 0) freq = a.inv_freq[ra % a.head_dim];
    }
    float res[NT][4];
    if (EPI == EPI_RESIDUAL && tile_leader && rank == 0) {
        int ra, rb;
        tile_rows<EPI>(a, block * tpb + tile_local, g, ra, rb);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int m = 8 * nt + 2 * t + e;
                res[nt][e] = (m < a.m && ra >= 0) ? a.residual[(size_t)m * a.n + ra] : 0.f;
                res[nt][2 + e] = (m < a.m && rb >= 0) ? a.residual[(size_t)m * a.n + rb] : 0.f;
            }
    }
    if (!mbar_wait(&w_bar[round & 1], (round >> 1) & 1) && lane == 0) atomicOr(a.err, QF_ERR_COPY_TIMEOUT);

    // ---- products: the warps of a tile take its k-blocks in turn
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const unsigned char* w_tile = w_s + (size_t)tile_local * 16 * plan.stride_w;
    const unsigned char* a_addr = w_tile + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * plan.stride_w + (lane >> 4) * 16;
    for (int kb = sub; kb < kb_count; kb += wpt) {
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t af[4];
            ldmatrix_x4(af, a_addr + (kb * 32 + ks * 16) * 2);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const unsigned char* xr = x_s + (size_t)(8 * nt + g) * plan.stride_x + (kb * 32 + ks * 16 + 2 * t) * 2;
                mma_bf16_16816(acc[nt], af, *reinterpret_cast<const uint32_t*>(xr), *reinterpret_cast<const uint32_t*>(xr + 16));
            }
        }
    }
    // ---- sum the warps of each tile in a fixed order, then the blocks of the cluster in rank order
    __syncthreads();  // every warp is done with this buffer's weights
    if (round + 2 < rounds) fetch(round + 2);  // the batch after next goes into the buffer that has just been read
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
        if (rounds > 1) cluster.sync();  // the first block has read the partial sums before the next batch overwrites them
    }
    if (tile_leader && rank == 0) {
    int ra, rb;
    tile_rows<EPI>(a, block * tpb + tile_local, g, ra, rb);
    // this lane holds, for token rows m = 8 nt + 2t + {0, 1}: acc[nt][0..1] of weight row ra, acc[nt][2..3] of row rb
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int m = 8 * nt + 2 * t + e;
            if (m >= a.m) continue;
            float inv = 1.f;
            if (NORM) {
                float ss = ss_s[m];
                for (int r = 1; r < ksplit; ++r) ss += ss_part[r - 1][m];
                inv = 1.0f / sqrtf(ss / (float)a.k + a.eps);
            }
            const float va = acc[nt][e] * inv + bias_a, vb = acc[nt][2 + e] * inv + bias_b;
            if (EPI == EPI_PLAIN) {
                if (a.out_f32) {
                    float* o = reinterpret_cast<float*>(a.out) + (size_t)m * a.ldo;
                    if (ra >= 0) o[ra] = va;
                    if (rb >= 0) o[rb] = vb;
                } else {
                    bf16* o = reinterpret_cast<bf16*>(a.out) + (size_t)m * a.ldo;
                    if (ra >= 0) o[ra] = __float2bfloat16_rn(va);
                    if (rb >= 0) o[rb] = __float2bfloat16_rn(vb);
                }
            } else if (EPI == EPI_RESIDUAL) {
                float* h = a.residual + (size_t)m * a.n;
                if (ra >= 0) h[ra] = res[nt][e] + va;
                if (rb >= 0) h[rb] = res[nt][2 + e] + vb;
            } else if (EPI == EPI_SWIGLU) {
                if (ra >= 0)
                    reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + ra] = __float2bfloat16_rn(va / (1.0f + expf(-va)) * vb);
            } else if (ra >= 0) {  // EPI_QKV
                const int D = a.head_dim, head = ra / D, j = ra % D;  // rb is component j + D/2 of the same head
                float oa = va, ob = vb;
                const int pos = pos_s[m];
                if (head < a.n_heads + a.kv_heads && a.inv_freq) {
                    // rotation pairs j with j + rot/2; the tile pairs j with j + D/2: the same when rot_dim == head_dim
                    float s, c;
                    sincosf((float)pos * freq, &s, &c);
                    oa = va * c - vb * s;
                    ob = vb * c + va * s;
                }
                if (head < a.n_heads) {
                    bf16* qo = a.q_out + (size_t)m * a.n_heads * D + (size_t)head * D;
                    qo[j] = __float2bfloat16_rn(oa);
                    qo[j + D / 2] = __float2bfloat16_rn(ob);
                } else if (dst_s[m] >= 0) {  // keys are heads n_heads .., values follow them: [2][kv_heads] planes of a page
                    bf16* dst = a.kv_base + dst_s[m] + (long long)(head - a.n_heads) * QF_PAGE * D;
                    dst[j] = __float2bfloat16_rn(oa);
                    dst[j + D / 2] = __float2bfloat16_rn(ob);
                }
            }
        }
    }
    }  // the lanes that own outputs
    }  // tile batches
}

static size_t plan_smem(const SkinnyPlan& p, int nt) {
    size_t w = (size_t)p.tpb * 16 * p.stride_w;
    const size_t red = (size_t)SK_WARPS * nt * 4 * 32 * 4;
    if (p.rounds == 1 && w < red) w = red;  // a single batch lends the partial sums the weights' space
    return (p.rounds > 1 ? 2 * w + red : w) + (size_t)8 * nt * p.stride_x + (size_t)(p.ksplit - 1) * p.tpb * nt * 4 * 32 * 4;
}

// How a product is cut into blocks: few tiles share their K among the blocks of a cluster so that every SM streams
// weights; many tiles are grouped so that all blocks are resident at once (one wave) and the norm prologue is not
// repeated more often than needed.
static bool make_plan(const SkinnyArgs& a, int tiles, int nt, SkinnyPlan& p) {
    const int sms = 148, n_kb = (a.k + 31) / 32;
    const size_t budget = 200 * 1024, most = 224 * 1024;
    auto fill = [&](int tpb, int ksplit, int rounds) {
        p.tpb = tpb;
        p.ksplit = ksplit;
        p.per = (n_kb + ksplit - 1) / ksplit;
        p.stride_w = pad_to_16_mod_128(p.per * 64);
        p.stride_x = pad_to_16_mod_128(p.per * 64);
        p.rounds = rounds;
        p.nblk = (tiles + tpb - 1) / tpb;
        return plan_smem(p, nt);
    };
    if (tiles <= sms) {
        // K is split only as far as a block's weights need it: up to 48 KB a block has them in flight long before its
        // token rows are ready, and a cluster's exchange of partial sums would only add to the chain of waits
        int ksplit = 2 * sms / tiles;
        const int by_bytes = (int)(((size_t)16 * a.k * 2 + 48 * 1024 - 1) / (48 * 1024));
        if (ksplit > by_bytes) ksplit = by_bytes;
        if (ksplit > 4) ksplit = 4;
        while (ksplit > 1 && (n_kb + ksplit - 1) / ksplit < 4) --ksplit;
        if (ksplit == 3) ksplit = 2;
        for (; ksplit <= 8; ksplit *= 2)
            if (fill(1, ksplit, 1) <= budget) return true;
        return false;
    }
    // every block resident at once, in one wave
    for (int tpb = 1; tpb <= 8; tpb *= 2) {
        const size_t smem = fill(tpb, 1, 1);
        if (smem > budget) break;
        const int resident = (int)((227 * 1024) / (smem + 1024));
        const int blocks = (tiles + tpb - 1) / tpb;
        if (blocks <= sms * (resident > 3 ? 3 : resident)) return true;  // the launch bounds allow three blocks of 256 threads
    }
    // too many tiles for one wave: one block per SM (or cluster) streams its share of the tile batches through two
    // weight buffers, the token rows staged once; K is split over a cluster where two buffers of whole rows do not fit
    for (int ksplit = 1; ksplit <= 8; ksplit *= 2) {
        for (int tpb = 2; tpb >= 1; --tpb) {
            if (fill(tpb, ksplit, 2) > most) continue;
            const int batches = (tiles + tpb - 1) / tpb, nblk = sms / ksplit;
            p.nblk = batches < nblk ? batches : nblk;
            p.rounds = (batches + p.nblk - 1) / p.nblk;
            if (p.rounds == 1) fill(tpb, ksplit, 1), p.nblk = batches;
            return true;
        }
    }
    return false;
}

template <int NT, int EPI, bool NORM> static int launch_one(const SkinnyArgs& a, int tiles, cudaStream_t stream) {
    SkinnyPlan p;
    if (!make_plan(a, tiles, NT, p)) return (int)cudaErrorInvalidValue;
    const size_t smem = plan_smem(p, NT);
    auto kernel = p.rounds > 1 ? skinny_gemm_kernel<NT, EPI, NORM, true> : skinny_gemm_kernel<NT, EPI, NORM, false>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(p.nblk * p.ksplit);
    config.blockDim = dim3(SK_THREADS);
    config.dynamicSmemBytes = smem;
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

template <int EPI, bool NORM> static int launch_epi(const SkinnyArgs& a, int tiles, cudaStream_t stream) {
    if (a.m <= 8) return launch_one<1, EPI, NORM>(a, tiles, stream);
    return launch_one<2, EPI, NORM>(a, tiles, stream);
}

// One entry for all variants. Shapes that the kernel does not take return cudaErrorInvalidValue; the caller
// then uses the unfused kernels. Requirements: 1 <= m <= 16; k, ldw, ldx multiples of 8; 16-byte aligned rows;
// SWIGLU: inter a multiple of 8; QKV: head_dim a multiple of 16 and rot_dim == head_dim when inv_freq is given.
QF_EXPORT int qf_skinny_gemm(int epilogue, int norm, const SkinnyArgs* args, cudaStream_t stream) {
    const SkinnyArgs& a = *args;
    if (a.m < 1 || a.m > 16 || a.k % 8 || a.ldw % 8 || a.k <= 0 || a.n <= 0) return (int)cudaErrorInvalidValue;
    if (!norm && a.ldx % 8) return (int)cudaErrorInvalidValue;
    int tiles;
    switch (epilogue) {
        case EPI_PLAIN:
            tiles = (a.n + 15) / 16;
            return norm ? launch_epi<EPI_PLAIN, true>(a, tiles, stream) : launch_epi<EPI_PLAIN, false>(a, tiles, stream);
        case EPI_RESIDUAL:
            tiles = (a.n + 15) / 16;
            return norm ? launch_epi<EPI_RESIDUAL, true>(a, tiles, stream) : launch_epi<EPI_RESIDUAL, false>(a, tiles, stream);
        case EPI_SWIGLU:
            if (a.inter % 8 || a.n != 2 * a.inter) return (int)cudaErrorInvalidValue;
            tiles = a.inter / 8;
            return norm ? launch_epi<EPI_SWIGLU, true>(a, tiles, stream) : launch_epi<EPI_SWIGLU, false>(a, tiles, stream);
        case EPI_QKV:
            if (a.head_dim % 16 || (a.inv_freq && a.rot_dim != a.head_dim) ||
                a.n != (a.n_heads + 2 * a.kv_heads) * a.head_dim)
                return (int)cudaErrorInvalidValue;
            tiles = (a.n_heads + 2 * a.kv_heads) * (a.head_dim / 16);
            return norm ? launch_epi<EPI_QKV, true>(a, tiles, stream) : launch_epi<EPI_QKV, false>(a, tiles, stream);
    }
    return (int)cudaErrorInvalidValue;
}
