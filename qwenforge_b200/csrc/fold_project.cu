// The output projection of a decode step of few rows, fed with the decode attention's partial results as they are.
//
// Split-K decode attention leaves, per (sequence, head, run of pages), a numerator row and a (maximum, sum) pair in
// scratch. Folding them inside the attention kernel costs that kernel a second life after its pages are done: publish
// the partials, fence, draw a ticket, and the block with the last ticket reads everybody's partials back: three trips
// through the L2 with nothing else to do, about 3 of the kernel's 9 microseconds at batch 8. This kernel takes the
// fold on instead, where it costs one trip that the projection has to make anyway (it would load the attended rows
// at that point): hidden[r, :] += fold(partials of row r) @ W^T.
//
// So that no block reads more partials than it needs, the product is cut along K: block b owns the 32 inputs
// [32 b, 32 b + 32), which lie inside ONE head, folds exactly those (rows x 32 numerators from each run), multiplies
// them with its slice W[:, 32 b : 32 b + 32] (fetched by 16-byte asynchronous copies before the kernel waits for the
// attention kernel, since no kernel writes weights) on the tensor cores (mma.sync m16n8k16, float32 accumulation),
// and adds its [rows, N] share into the float32 residual stream with 16-byte vector reductions. The order in which
// the blocks' shares arrive is not fixed, so the stream's last bits can differ from run to run, as they do for every
// product that splits K across blocks.
//
// The fold itself is the attention kernel's own: eight runs at a time with a running maximum, base-2 exponentials,
// out = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s, rounded to bfloat16 like the attended rows it replaces.
#include "mma.cuh"

#define FP_KS 32        // inputs per block
#define FP_LD 40        // shared-memory row in bf16 elements: 80 bytes, so that eight rows of a ldmatrix meet no bank twice
#define FP_THREADS 256
#define FP_MAX_ROWS 16

struct FoldProjectArgs {
    const float* part_o;    // [rows * n_heads * max_splits][head_dim]
    const float* part_ml;   // [rows * n_heads * max_splits][2]
    const int* runs;        // [rows] how many runs each row's partials have (1 ..= max_splits)
    const bf16* w;          // [n][ldw], K = n_heads * head_dim inputs per output
    float* hidden;          // [rows][n]
    int rows, n, ldw, n_heads, head_dim, max_splits;
};

__global__ void __launch_bounds__(FP_THREADS) fold_project_kernel(FoldProjectArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* w_s = reinterpret_cast<bf16*>(smem_raw);                     // [n][FP_LD]
    bf16* x_s = w_s + (size_t)a.n * FP_LD;                             // [16][FP_LD]
    grid_launch_dependents();
    const int k0 = blockIdx.x * FP_KS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int c = threadIdx.x; c < a.n * (FP_KS / 8); c += FP_THREADS) {
        const int n = c / (FP_KS / 8), part = c % (FP_KS / 8);
        cp_async_16(w_s + (size_t)n * FP_LD + part * 8, a.w + (size_t)n * a.ldw + k0 + part * 8, true);
    }
    cp_async_commit();
    for (int i = threadIdx.x; i < 16 * FP_LD / 2; i += FP_THREADS) reinterpret_cast<uint32_t*>(x_s)[i] = 0u;
    grid_dependency_wait();
    __syncthreads();  // the zeros are in place before the folded rows go on top of them

    // ---- fold: thread (row, d) takes input k0 + d of its row over the row's runs
    const int head = k0 / a.head_dim, d0 = k0 % a.head_dim;
    for (int item = threadIdx.x; item < a.rows * FP_KS; item += FP_THREADS) {
        const int r = item / FP_KS, d = item % FP_KS;
        const int n_runs = min(max(a.runs[r], 1), a.max_splits);
        const size_t base = ((size_t)r * a.n_heads + head) * a.max_splits;
        const float2* ml = reinterpret_cast<const float2*>(a.part_ml) + base;
        const float* po = a.part_o + base * a.head_dim + d0 + d;
        float big = QF_NEG_BIG, den = 0.f, num = 0.f;
        for (int sp0 = 0; sp0 < n_runs; sp0 += 8) {
            float2 m[8];
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool in = sp0 + j < n_runs;
                m[j] = in ? __ldcg(ml + sp0 + j) : make_float2(QF_NEG_BIG, 0.f);
                v[j] = in ? __ldcg(po + (size_t)(sp0 + j) * a.head_dim) : 0.f;
            }
            float top = big;
#pragma unroll
            for (int j = 0; j < 8; ++j) top = fmaxf(top, m[j].x);
            const float keep = exp2f(big - top);
            den *= keep;
            num *= keep;
            big = top;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float w = exp2f(m[j].x - top);
                den += w * m[j].y;
                num += w * v[j];
            }
        }
        x_s[r * FP_LD + d] = __float2bfloat16_rn(den > 0.f ? num * (1.f / den) : 0.f);
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- product: warp w takes the outputs 16 g .. 16 g + 15 for g = w, w + 8, ...
    uint32_t xa[FP_KS / 16][4];
#pragma unroll
    for (int ks = 0; ks < FP_KS / 16; ++ks) ldmatrix_x4(xa[ks], x_s + (lane & 15) * FP_LD + 16 * ks + (lane >> 4) * 8);
    const int row = lane >> 2, pair = (lane & 3) >> 1;
    const bool odd = lane & 1;
    for (int g = warp; g < a.n / 16; g += FP_THREADS / 32) {
        float c[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < FP_KS / 16; ++ks) {
            uint32_t wf[4];
            ldmatrix_x4(wf, w_s + (size_t)(16 * g + (lane >> 4) * 8 + (lane & 7)) * FP_LD + 16 * ks + ((lane >> 3) & 1) * 8);
            mma_bf16_16816(c[0], xa[ks], wf[0], wf[1]);
            mma_bf16_16816(c[1], xa[ks], wf[2], wf[3]);
        }
        // Lane (row, q) holds columns 2q, 2q + 1 of both tiles of eight outputs. Neighbours swap one tile's pair, so
        // that the even lane has four adjacent columns of the first tile and the odd lane four of the second.
#pragma unroll
        for (int half = 0; half < 2; ++half) {  // accumulator rows `row` and `row + 8`
            const float s0 = odd ? c[0][2 * half] : c[1][2 * half], s1 = odd ? c[0][2 * half + 1] : c[1][2 * half + 1];
            const float r0 = __shfl_xor_sync(0xffffffffu, s0, 1), r1 = __shfl_xor_sync(0xffffffffu, s1, 1);
            const int r = row + 8 * half;
            if (r < a.rows) {
                const float4 sum = odd ? make_float4(r0, r1, c[1][2 * half], c[1][2 * half + 1])
                                       : make_float4(c[0][2 * half], c[0][2 * half + 1], r0, r1);
                float4* to = reinterpret_cast<float4*>(a.hidden + (size_t)r * a.n + 16 * g + (odd ? 8 : 0) + 4 * pair);
                atomicAdd(to, sum);
            }
        }
    }
}

static size_t fold_project_smem(int n) { return ((size_t)n + 16) * FP_LD * sizeof(bf16); }

// Whether the kernel takes the shape: the inputs of a block lie inside one head, the outputs come in groups of 16, the
// weight's rows start on 16 bytes, its slice fits into shared memory, and there are at most 16 rows.
QF_EXPORT int qf_fold_project_takes(int rows, int n, int ldw, int n_heads, int head_dim, const void* w, const void* hidden) {
    if (rows < 1 || rows > FP_MAX_ROWS || n < 16 || n % 16 || n_heads < 1 || head_dim < FP_KS || head_dim % FP_KS) return 0;
    if (ldw < n_heads * head_dim || ldw % 8) return 0;
    if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(hidden) & 15)) return 0;
    return fold_project_smem(n) <= 200 * 1024 ? 1 : 0;
}

QF_EXPORT int qf_fold_project(const FoldProjectArgs* args, cudaStream_t stream) {
    const FoldProjectArgs& a = *args;
    if (!qf_fold_project_takes(a.rows, a.n, a.ldw, a.n_heads, a.head_dim, a.w, a.hidden) || a.max_splits < 1)
        return (int)cudaErrorInvalidValue;
    const size_t smem = fold_project_smem(a.n);
    cudaError_t e = cudaFuncSetAttribute(fold_project_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_pdl(fold_project_kernel, dim3(a.n_heads * a.head_dim / FP_KS), dim3(FP_THREADS), smem, stream, a);
}
