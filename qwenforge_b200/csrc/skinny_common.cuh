// What the weight-streaming kernels for a few token rows share (skinny_gemm.cu, skinny_chain.cu): the argument
// block of one product, which weight rows make up a 16-row tile under each epilogue, and the epilogues themselves.
#pragma once
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

static __host__ __device__ inline int pad_to_16_mod_128(int bytes) { return bytes + ((16 - bytes % 128) + 128) % 128; }

#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)

// What a lane's epilogue reads from global memory, fetched before the products: bias and rotation frequency of its
// two weight rows (constants), and for RESIDUAL the values it will add to.
template <int NT> struct EpiloguePre {
    float bias_a = 0.f, bias_b = 0.f, freq = 0.f;
    float res[NT][4];
};

template <int NT, int EPI>
__device__ __forceinline__ void skinny_epilogue_prefetch(const SkinnyArgs& a, int tile, int g, int t, EpiloguePre<NT>& pre) {
    int ra, rb;
    tile_rows<EPI>(a, tile, g, ra, rb);
    if (a.bias && ra >= 0) pre.bias_a = __bfloat162float(a.bias[ra]);
    if (a.bias && rb >= 0) pre.bias_b = __bfloat162float(a.bias[rb]);
    if (EPI == EPI_QKV && a.inv_freq && ra >= 0) pre.freq = a.inv_freq[ra % a.head_dim];
    if (EPI == EPI_RESIDUAL) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int m = 8 * nt + 2 * t + e;
                pre.res[nt][e] = (m < a.m && ra >= 0) ? a.residual[(size_t)m * a.n + ra] : 0.f;
                pre.res[nt][2 + e] = (m < a.m && rb >= 0) ? a.residual[(size_t)m * a.n + rb] : 0.f;
            }
    }
}

// The epilogue of one 16-row tile, run by the 32 lanes that hold its sums. ss_s: sums of squares of the token rows
// over this block's K (NORM), ss_part: the same of the cluster's other blocks; pos_s, dst_s: position and cache
// offset of each token row (QKV).
template <int NT, int EPI, bool NORM>
__device__ __forceinline__ void skinny_epilogue(const SkinnyArgs& a, int tile, int g, int t, const float (&acc)[NT][4],
                                                const EpiloguePre<NT>& pre, const float* ss_s, const float (*ss_part)[16],
                                                int ksplit, const int* pos_s, const long long* dst_s, int only_nt = -1) {
    int ra, rb;
    tile_rows<EPI>(a, tile, g, ra, rb);
    const float bias_a = pre.bias_a, bias_b = pre.bias_b, freq = pre.freq;
    // this lane holds, for token rows m = 8 nt + 2t + {0, 1}: acc[nt][0..1] of weight row ra, acc[nt][2..3] of row rb
    // (`only_nt` >= 0: the caller holds the sums of that n-tile alone)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        if (only_nt >= 0 && nt != only_nt) continue;
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
                if (ra >= 0) h[ra] = pre.res[nt][e] + va;
                if (rb >= 0) h[rb] = pre.res[nt][2 + e] + vb;
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
}


// One k-block (32 columns) of a 16-row weight tile against NT n-tiles of 8 token rows, both in shared memory with rows
// a multiple of 128 bytes plus 16 apart (conflict-free ldmatrix). `a_lane` is this lane's ldmatrix address in the weight
// tile at column 0: row (lane & 7) + 8 * ((lane >> 3) & 1), plus 16 bytes for lanes 16..31. `x_lane` is this lane's
// address in the token rows at column 0 (`x_lane_address`): the token rows are read with ldmatrix as well, four 8 x 8
// blocks (two n-tiles, two halves of k) per instruction.
__device__ __forceinline__ const unsigned char* x_lane_address(const unsigned char* x_s, int x_stride, int lane, bool two_tiles) {
    const int row = (lane & 7) + (two_tiles ? ((lane >> 4) << 3) : 0);
    return x_s + (size_t)row * x_stride + ((lane >> 3) & 1) * 16;
}

template <int NT>
__device__ __forceinline__ void mma_k_block(float (&acc)[NT][4], const unsigned char* a_lane, const unsigned char* x_lane,
                                            int x_stride, int col) {
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
        uint32_t af[4];
        ldmatrix_x4(af, a_lane + (col + ks * 16) * 2);
        if (NT == 1) {
            uint32_t b[2];
            ldmatrix_x2(b, x_lane + (col + ks * 16) * 2);
            mma_bf16_16816(acc[0], af, b[0], b[1]);
        } else {
#pragma unroll
            for (int p = 0; p < NT / 2; ++p) {
                uint32_t b[4];
                ldmatrix_x4(b, x_lane + (size_t)p * 16 * x_stride + (col + ks * 16) * 2);
                mma_bf16_16816(acc[2 * p], af, b[0], b[1]);
                mma_bf16_16816(acc[2 * p + 1], af, b[2], b[3]);
            }
        }
    }
}

// The streaming kernels move K in chunks of SK_CHUNK columns through a ring of shared-memory stages.
#define SK_CHUNK 1024  // columns of a chunk: one bulk copy per row and chunk (2 KB); smaller copies are bound by their issue
#define SK_STAGE_STRIDE (SK_CHUNK * 2 + 16)  // bytes between rows of a stage (16 modulo 128: conflict-free ldmatrix)

// A barrier among the eight product warps only (the fetching warp does not take part).
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(SK_THREADS) : "memory"); }
