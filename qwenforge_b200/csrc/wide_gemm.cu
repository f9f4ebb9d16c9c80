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
// epilogue; where an epilogue pairs two weight rows (gate and up, component j and j + D/2 of a head) the partner's
// values cross through shared memory. While the weights stream, those warps prepare what the epilogue needs
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
    int stage_bytes; // weights + token rows of one stage
};

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
    const int ntok = geo.ntok, ksplit = geo.ksplit;
    const int tile = blockIdx.x / ksplit, rank = blockIdx.x % ksplit;
    const int per = (geo.slabs + ksplit - 1) / ksplit;
    const int kb_begin = rank * per, kb_end = min(geo.slabs, kb_begin + per), n_kb = max(0, kb_end - kb_begin);
    // after the ring: what the epilogue exchanges (see below); the ring itself is free by then, but the partial sums of
    // other blocks of the cluster arrive while this block may still be multiplying, so they get room of their own
    unsigned char* ring = smem;
    float* extra = reinterpret_cast<float*>(ring + (size_t)WG_STAGES * geo.stage_bytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < WG_STAGES; ++s) {
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
    const uint32_t tmem = tmem_base_s;
    bool timed_out = false;
    float v[WG_MAX_TOK];  // row threads: this lane's sums, one per token row
    const int D = a.head_dim;
    float* cs = extra;    // QKV: [tokens][D / 2] pairs (cos, sin) of every token's angles

    // first weight row of the tile's two boxes of 64 rows
    int row0 = tile * WG_BM, row1 = row0 + 64;
    if (EPI == EPI_SWIGLU) {
        row0 = tile * 64;
        row1 = a.inter + tile * 64;
    }

    if (warp == 4) {
        // ---- copies. All lanes run the loop; one issues.
        const bool leader = elect_one();
        auto load_w = [&](int kb, int s) {
            unsigned char* w_s = ring + (size_t)s * geo.stage_bytes;
            tma_load_2d(w_s, &w_map, kb * WG_BK, row0, &full_bar[s]);
            tma_load_2d(w_s + 64 * WG_BK * 2, &w_map, kb * WG_BK, row1, &full_bar[s]);
        };
        auto load_x = [&](int kb, int s) {
            tma_load_2d(ring + (size_t)s * geo.stage_bytes + WG_W_BYTES, &x_map, kb * WG_BK, 0, &full_bar[s]);
        };
        // weights are nobody's output: those of the first stages are on their way before the kernel before this one ends
        const int early = min(n_kb, WG_STAGES);
        if (leader)
            for (int i = 0; i < early; ++i) {
                mbar_expect_tx(&full_bar[i], (uint32_t)geo.stage_bytes);
                load_w(kb_begin + i, i);
            }
        __syncwarp();
        grid_dependency_wait();
        if (leader)
            for (int i = 0; i < early; ++i) load_x(kb_begin + i, i);
        __syncwarp();
        for (int i = early; i < n_kb; ++i) {
            const int s = i % WG_STAGES;
            if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], ((i / WG_STAGES) - 1) & 1))) {
                timed_out = true;
                break;
            }
            if (leader) {
                mbar_expect_tx(&full_bar[s], (uint32_t)geo.stage_bytes);
                load_w(kb_begin + i, s);
                load_x(kb_begin + i, s);
            }
            __syncwarp();
        }
    } else if (warp == 5) {
        // ---- products
        const bool leader = elect_one();
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ntok >> 3) << 17) | ((uint32_t)(WG_BM >> 4) << 24);
        for (int i = 0; i < n_kb; ++i) {
            const int s = i % WG_STAGES;
            if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], (i / WG_STAGES) & 1))) {
                timed_out = true;
                break;
            }
            tc_fence_after();
            const unsigned char* w_s = ring + (size_t)s * geo.stage_bytes;
            const uint64_t dw = smem_desc_sw128(w_s), dx = smem_desc_sw128(w_s + WG_W_BYTES);
            if (leader) {
#pragma unroll
                for (int k4 = 0; k4 < WG_BK / 16; ++k4) umma_bf16(tmem, dw + 2 * k4, dx + 2 * k4, idesc, (i > 0 || k4 > 0) ? 1u : 0u);
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
                const int half = D / 2;
                for (int i = r; i < a.m * half; i += WG_ROW_THREADS) {
                    const int m = i / half, j = i % half;
                    float s, c;
                    sincosf((float)pos_s[m] * a.inv_freq[j], &s, &c);
                    cs[2 * i] = c;
                    cs[2 * i + 1] = s;
                }
            }
            row_barrier();
        }
        if (!__all_sync(0xffffffffu, mbar_wait(&acc_bar, 0))) timed_out = true;
        tc_fence_after();
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
        if (EPI != EPI_QKV) grid_dependency_wait();  // the residual stream and the outputs belong to earlier kernels until now

        if (ksplit > 1) {
            // ---- K was split over the cluster (PLAIN and RESIDUAL only): block q owns rows [q * own, (q + 1) * own) of the
            // tile; everyone sends it their partial sums of those rows
            cg::cluster_group cluster = cg::this_cluster();
            const int own = WG_BM / ksplit, q = r / own, r_local = r % own;
            float* theirs = cluster.map_shared_rank(extra, q) + ((size_t)rank * own + r_local) * ntok;
#pragma unroll
            for (int m = 0; m < WG_MAX_TOK; ++m)
                if (m < ntok) theirs[m] = v[m];
        }
    }
    if (ksplit > 1) cg::this_cluster().sync();  // every thread of every block of the cluster: the partial sums have arrived
    if (warp < 4) {
        const int r = threadIdx.x;
        if (ksplit > 1) {
            // the owner adds its rows' partial sums in rank order
            const int own = WG_BM / ksplit;
            for (int i = r; i < own * a.m; i += WG_ROW_THREADS) {
                const int m = i / own, rl = i % own;
                float sum = 0.f;
                for (int src = 0; src < ksplit; ++src) sum += extra[((size_t)src * own + rl) * ntok + m];
                const int n = tile * WG_BM + rank * own + rl;
                if (n >= a.n) continue;
                if (a.bias) sum += __bfloat162float(a.bias[n]);
                if (EPI == EPI_RESIDUAL) a.residual[(size_t)m * a.n + n] += sum;
                else if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + n] = sum;
                else reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + n] = __float2bfloat16_rn(sum);
            }
        } else if (EPI == EPI_PLAIN || EPI == EPI_RESIDUAL) {
            const int n = tile * WG_BM + r;
            if (n < a.n) {
                const float bias = a.bias ? __bfloat162float(a.bias[n]) : 0.f;
#pragma unroll
                for (int m = 0; m < WG_MAX_TOK; ++m) {
                    if (m >= a.m) break;
                    const float value = v[m] + bias;
                    if (EPI == EPI_RESIDUAL) a.residual[(size_t)m * a.n + n] += value;
                    else if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + n] = value;
                    else reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + n] = __float2bfloat16_rn(value);
                }
            }
        } else if (EPI == EPI_SWIGLU) {
            // lanes 64..127 hold the up rows: they pass their sums to the gate rows' threads
            float* up = extra;  // [64][ntok + 1]
            if (r >= 64) {
#pragma unroll
                for (int m = 0; m < WG_MAX_TOK; ++m)
                    if (m < ntok) up[(size_t)(r - 64) * (ntok + 1) + m] = v[m];
            }
            row_barrier();
            const int i = tile * 64 + r;
            if (r < 64 && i < a.inter) {
#pragma unroll
                for (int m = 0; m < WG_MAX_TOK; ++m) {
                    if (m >= a.m) break;
                    const float gate = v[m], u = up[(size_t)r * (ntok + 1) + m];
                    reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + i] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * u);
                }
            }
        } else {  // EPI_QKV
            // row n of the projection is component j of head n / D; its rotation partner j +- D/2 lies in the same tile,
            // D/2 lanes away: all sums (bias added) cross through shared memory
            float* all = extra + 2 * (size_t)WG_MAX_TOK * (D / 2);  // [128][ntok + 1], behind the sines and cosines
            const int n = tile * WG_BM + r;
            const bool exists = n < a.n;
            const float bias = (a.bias && exists) ? __bfloat162float(a.bias[n]) : 0.f;
#pragma unroll
            for (int m = 0; m < WG_MAX_TOK; ++m)
                if (m < ntok) all[(size_t)r * (ntok + 1) + m] = v[m] + bias;
            row_barrier();
            if (exists) {
                const int head = n / D, j = n % D, half = D / 2;
                const bool rotated = a.inv_freq != nullptr && head < a.n_heads + a.kv_heads;
                const bool low = j < half;
                const float* partner = all + (size_t)(low ? r + half : r - half) * (ntok + 1);
#pragma unroll
                for (int m = 0; m < WG_MAX_TOK; ++m) {
                    if (m >= a.m) break;
                    float value = v[m] + bias;
                    if (rotated) {
                        const float c = cs[2 * (m * half + (low ? j : j - half))], s = cs[2 * (m * half + (low ? j : j - half)) + 1];
                        const float other = partner[m];
                        value = low ? value * c - other * s : value * c + other * s;
                    }
                    if (head < a.n_heads) {
                        a.q_out[(size_t)m * a.n_heads * D + (size_t)head * D + j] = __float2bfloat16_rn(value);
                    } else if (dst_s[m] >= 0) {  // keys are heads n_heads .., values follow: [2][kv_heads] planes of a page
                        a.kv_base[dst_s[m] + (long long)(head - a.n_heads) * QF_PAGE * D + j] = __float2bfloat16_rn(value);
                    }
                }
            }
        }
    }
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
    geo.stage_bytes = WG_W_BYTES + geo.ntok * WG_BK * 2;
    // K is split over a cluster when the tiles are few and heavy: a block should not stream much more than 256 KB,
    // as long as that does not ask for more blocks than there are SMs
    geo.ksplit = 1;
    if (epilogue == EPI_PLAIN || epilogue == EPI_RESIDUAL)
        while (geo.ksplit < WG_MAX_SPLIT && geo.tiles * geo.ksplit * 2 <= sms &&
               (size_t)WG_BM * a.k * 2 / geo.ksplit > 256 * 1024 && geo.slabs / (geo.ksplit * 2) >= 2)
            geo.ksplit *= 2;
    size_t extra = 0;
    if (geo.ksplit > 1) extra = (size_t)WG_BM * geo.ntok * 4;                                  // [ksplit][128 / ksplit][ntok]
    else if (epilogue == EPI_SWIGLU) extra = (size_t)64 * (geo.ntok + 1) * 4;
    else if (epilogue == EPI_QKV) extra = 2 * (size_t)WG_MAX_TOK * (a.head_dim / 2) * 4 + (size_t)WG_BM * (geo.ntok + 1) * 4;
    smem = (size_t)WG_STAGES * geo.stage_bytes + extra + 1024;
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

// Whether `qf_wide_gemm` would run a product of these sizes on the current device (the number of blocks it would
// launch), or 0. Launches nothing; the pointers only say whether a bias and a rotation are given, and how the rows
// are aligned.
QF_EXPORT int qf_wide_gemm_takes(int epilogue, const SkinnyArgs* args) {
    WideGeometry geo;
    size_t smem = 0;
    return wide_plan(epilogue, *args, qf_sm_count(), geo, smem) ? geo.tiles * geo.ksplit : 0;
}
