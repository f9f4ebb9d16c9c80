// Weight-streaming matrix products for a handful of token rows (decode steps): out[m][n] = sum_k x[m][k] W[n][k],
// M <= 16 rows, bf16 weights read once from HBM, with what surrounds the product fused in:
//   prologue  NORM     x = rmsnorm(hidden) * norm_weight, from the float32 residual stream (statistics in float32)
//   epilogue  PLAIN    out (bf16 or float32) = product (+ bias)
//             RESIDUAL hidden[m][n] += product            (the float32 residual stream, in place)
//             SWIGLU   out[m][i] = silu(gate_i) * up_i    (W = [gate rows | up rows])
//             QKV      + bias, rotate q and k heads by position (float32 angles), q -> q_out, k and v -> cache pages
//
// The product runs on the tensor cores as out^T = W x^T: 16 weight rows are the M side of an m16n8k16 tile and
// 8 token rows its N side, so no weight is touched twice and no shared-memory bandwidth is spent on it. A block
// owns 16 weight rows; its warps split K in interleaved blocks of 32 and are summed in a fixed order. Each lane
// loads 16 contiguous bytes of a weight row straight into the A fragments of two MMAs (the k order inside a
// block of 32 is permuted, identically for the x fragments, which does not change the sum's terms).
// The 16 rows of a block are chosen so that the two rows a lane holds (g and g + 8) are the pair its epilogue
// needs: component j and j + D/2 of a head for the rotation, gate row i and up row i for SwiGLU.
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
    } else {
        ra = tile * 16 + g;
        rb = ra + 8;
        if (ra >= a.n) ra = -1;
        if (rb >= a.n) rb = -1;
    }
}

template <int NT, int EPI, bool NORM, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) skinny_gemm_kernel(const SkinnyArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int MP = 8 * NT;  // token rows, padded
    const int kp = (a.k + 31) / 32 * 32;
    // row stride of x in shared memory: congruent to 64 bytes modulo 128, so that the eight (row, quarter) pairs
    // of a quarter-warp's 16-byte loads fall on distinct banks
    const int ldxs = kp + ((kp * 2) % 128 == 64 ? 0 : ((64 - (kp * 2) % 128 + 128) % 128) / 2);
    bf16* x_s = reinterpret_cast<bf16*>(smem_raw);                       // [MP][ldxs]
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)MP * ldxs * 2);  // [WARPS][NT * 4][32]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    int ra, rb;
    tile_rows<EPI>(a, blockIdx.x, g, ra, rb);
    const bf16* wa = a.w + (size_t)max(ra, 0) * a.ldw;
    const bf16* wb = a.w + (size_t)max(rb, 0) * a.ldw;
    const int n_kb = kp / 32;

    // ---- start the first weight loads, then prepare x while they fly
    constexpr int UNROLL = 4;
    uint4 fa[UNROLL], fb[UNROLL];
    auto load_w = [&](int kb0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int kb = kb0 + u * WARPS, kk = kb * 32 + t * 8;
            const bool ok = kb < n_kb && kk < a.k;
            fa[u] = (ok && ra >= 0) ? __ldcs(reinterpret_cast<const uint4*>(wa + kk)) : make_uint4(0, 0, 0, 0);
            fb[u] = (ok && rb >= 0) ? __ldcs(reinterpret_cast<const uint4*>(wb + kk)) : make_uint4(0, 0, 0, 0);
        }
    };
    load_w(warp);

    if (NORM) {
        for (int m = warp; m < MP; m += WARPS) {
            bf16* dst = x_s + (size_t)m * ldxs;
            if (m < a.m) {
                const float* h = a.hidden + (size_t)m * a.k;
                float ss = 0.f;
                for (int c = lane; c < a.k; c += 32) ss += h[c] * h[c];
                ss = warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss / (float)a.k + a.eps);
                for (int c = lane; c < kp; c += 32)
                    dst[c] = c < a.k ? __float2bfloat16_rn(h[c] * inv * __bfloat162float(a.norm_w[c])) : __float2bfloat16_rn(0.f);
            } else {
                for (int c = lane; c < kp; c += 32) dst[c] = __float2bfloat16_rn(0.f);
            }
        }
    } else {
        const int chunks = kp / 8;
        for (int i = threadIdx.x; i < MP * chunks; i += WARPS * 32) {
            const int m = i / chunks, c = (i % chunks) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (m < a.m && c < a.k) v = *reinterpret_cast<const uint4*>(a.x + (size_t)m * a.ldx + c);
            *reinterpret_cast<uint4*>(x_s + (size_t)m * ldxs + c) = v;
        }
    }
    __syncthreads();

    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    for (int kb0 = warp; kb0 < n_kb; kb0 += UNROLL * WARPS) {
        uint4 ca[UNROLL], cb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            ca[u] = fa[u];
            cb[u] = fb[u];
        }
        if (kb0 + UNROLL * WARPS < n_kb) load_w(kb0 + UNROLL * WARPS);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int kb = kb0 + u * WARPS;
            if (kb >= n_kb) break;
            // A fragments: rows g / g + 8; k slots (2t, 2t+1) and (2t+8, 2t+9) take this lane's 8 values in two MMAs
            const uint32_t a1[4] = {ca[u].x, cb[u].x, ca[u].y, cb[u].y};
            const uint32_t a2[4] = {ca[u].z, cb[u].z, ca[u].w, cb[u].w};
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 xv = *reinterpret_cast<const uint4*>(x_s + (size_t)(8 * nt + g) * ldxs + kb * 32 + t * 8);
                mma_bf16_16816(acc[nt], a1, xv.x, xv.y);
                mma_bf16_16816(acc[nt], a2, xv.z, xv.w);
            }
        }
    }
    // ---- sum the warps in a fixed order
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[((size_t)warp * NT * 4 + nt * 4 + e) * 32 + lane] = acc[nt][e];
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float s = 0.f;
            for (int w = 0; w < WARPS; ++w) s += red[((size_t)w * NT * 4 + nt * 4 + e) * 32 + lane];
            acc[nt][e] = s;
        }
    // this lane holds, for token rows m = 8 nt + 2t + {0, 1}: acc[nt][0..1] of weight row ra, acc[nt][2..3] of row rb
    const float bias_a = (a.bias && ra >= 0) ? __bfloat162float(a.bias[ra]) : 0.f;
    const float bias_b = (a.bias && rb >= 0) ? __bfloat162float(a.bias[rb]) : 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int m = 8 * nt + 2 * t + e;
            if (m >= a.m) continue;
            const float va = acc[nt][e] + bias_a, vb = acc[nt][2 + e] + bias_b;
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
                if (ra >= 0) h[ra] += va;
                if (rb >= 0) h[rb] += vb;
            } else if (EPI == EPI_SWIGLU) {
                if (ra >= 0)
                    reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + ra] = __float2bfloat16_rn(va / (1.0f + expf(-va)) * vb);
            } else {  // EPI_QKV
                const int D = a.head_dim, head = ra / D, j = ra % D;  // rb is component j + D/2 of the same head
                float oa = va, ob = vb;
                const int pos = a.tok_pos[m];
                if (head < a.n_heads + a.kv_heads && a.inv_freq) {
                    // rotation pairs j with j + rot/2; the tile pairs j with j + D/2: the same when rot_dim == head_dim
                    float s, c;
                    sincosf((float)pos * a.inv_freq[j], &s, &c);
                    oa = va * c - vb * s;
                    ob = vb * c + va * s;
                }
                if (head < a.n_heads) {
                    bf16* qo = a.q_out + (size_t)m * a.n_heads * D + (size_t)head * D;
                    qo[j] = __float2bfloat16_rn(oa);
                    qo[j + D / 2] = __float2bfloat16_rn(ob);
                } else if (a.write_cache) {
                    const int slot = a.slots[a.tok_seq[m]];
                    if (slot >= 0) {
                        const int which = head < a.n_heads + a.kv_heads ? 0 : 1;
                        const int h = head - a.n_heads - which * a.kv_heads;
                        const int page = a.table[(long long)slot * a.table_stride + pos / QF_PAGE];
                        if (page < 0) {
                            atomicOr(a.err, QF_ERR_NO_PAGE);
                        } else {
                            bf16* dst = a.kv_base + (long long)page * a.page_elems +
                                        ((long long)(which * a.kv_heads + h) * QF_PAGE + (pos % QF_PAGE)) * D;
                            dst[j] = __float2bfloat16_rn(oa);
                            dst[j + D / 2] = __float2bfloat16_rn(ob);
                        }
                    }
                }
            }
        }
    }
}

template <int NT, int EPI, bool NORM, int WARPS> static int launch_one(const SkinnyArgs& a, int tiles, cudaStream_t stream) {
    const int kp = (a.k + 31) / 32 * 32;
    const int ldxs = kp + ((kp * 2) % 128 == 64 ? 0 : ((64 - (kp * 2) % 128 + 128) % 128) / 2);
    const size_t smem = (size_t)8 * NT * ldxs * 2 + (size_t)WARPS * NT * 4 * 32 * 4;
    if (smem > 220 * 1024) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<NT, EPI, NORM, WARPS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    skinny_gemm_kernel<NT, EPI, NORM, WARPS><<<tiles, WARPS * 32, smem, stream>>>(a);
    return (int)cudaGetLastError();
}

template <int EPI, bool NORM> static int launch_epi(const SkinnyArgs& a, int tiles, cudaStream_t stream) {
    // few tiles: more warps per block share one tile's K; many tiles: fewer warps, more blocks per SM
    const bool wide = tiles < 400;
    if (a.m <= 8) return wide ? launch_one<1, EPI, NORM, 8>(a, tiles, stream) : launch_one<1, EPI, NORM, 4>(a, tiles, stream);
    return wide ? launch_one<2, EPI, NORM, 8>(a, tiles, stream) : launch_one<2, EPI, NORM, 4>(a, tiles, stream);
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
