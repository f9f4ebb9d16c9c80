// Next-token choice from float32 logits, one block per row.
//   temperature <= 0 : argmax, the lowest id on ties
//   temperature  > 0 : Gumbel-max,  argmax_i( logit_i / T - log(-log(u_i)) ), which draws i with
//                      probability softmax(logits / T)_i. u_i comes from a counter-based integer hash of
//                      (seed, sequence id, step, i), so a sequence's draws do not depend on the batch
//                      it is in, on its row in that batch, or on how many steps other sequences took.
#include <float.h>

#include "common.cuh"

__host__ __device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7FEB352Du;
    x ^= x >> 15;
    x *= 0x846CA68Bu;
    x ^= x >> 16;
    return x;
}

__device__ __forceinline__ uint32_t row_key(unsigned long long seed, long long seq_id, int step) {
    uint32_t key = mix32((uint32_t)seed ^ 0x9E3779B9u);
    key = mix32(key ^ (uint32_t)(seed >> 32));
    key = mix32(key ^ (uint32_t)seq_id);
    key = mix32(key ^ (uint32_t)((unsigned long long)seq_id >> 32) ^ 0x85EBCA6Bu);
    key = mix32(key ^ (uint32_t)step);
    return key;
}

// One block scans a chunk of one row's vocabulary; with several chunks per row the blocks leave their best
// (score, id) in scratch and take a ticket, and the block that draws the row's last ticket picks the row's best
// and resets the ticket counter. Ties go to the lowest id at every level, so the result does not depend on `chunks`.
__global__ void __launch_bounds__(256)
sample_kernel(const float* __restrict__ logits, int vocab, long long row_stride, float temperature,
              unsigned long long seed, const long long* __restrict__ seq_ids, const int* __restrict__ steps,
              int* __restrict__ out, int chunks, float* __restrict__ part_v, int* __restrict__ part_i,
              int* __restrict__ counters) {
    grid_chain_entry();
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    __shared__ int ticket;
    const int row = blockIdx.y, chunk = blockIdx.x;
    const float* x = logits + (size_t)row * row_stride;
    const bool sample = temperature > 0.f;
    const uint32_t key = sample ? row_key(seed, seq_ids[row], steps[row]) : 0u;
    const float inv_t = sample ? 1.0f / temperature : 1.0f;
    const int per = (((vocab + chunks - 1) / chunks) + 3) & ~3;  // a multiple of 4: chunks start on 16 bytes when rows do
    const int begin = min(vocab, chunk * per), end = min(vocab, begin + per);
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    auto consider = [&](float s, int i) {
        if (sample) {
            const uint32_t bits = mix32(key ^ mix32((uint32_t)i ^ 0x27D4EB2Fu));
            const float u = ((float)(bits >> 9) + 0.5f) * (1.0f / 8388608.0f);
            s = s * inv_t - logf(-logf(u));
        }
        if (s > bv || (s == bv && i < bi)) {
            bv = s;
            bi = i;
        }
    };
    int done = begin;  // ids below `done` have been considered by some thread
    if ((reinterpret_cast<uintptr_t>(x + begin) & 15) == 0) {
        // four 16-byte loads in flight per thread: the scan is a stream, not a chain of round trips
        const float4* x4 = reinterpret_cast<const float4*>(x + begin);
        const int n4 = (end - begin) / 4;
        for (int j0 = threadIdx.x; j0 < n4; j0 += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u * blockDim.x;
                v[u] = j < n4 ? x4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u * blockDim.x;
                if (j < n4) {
                    const int i = begin + 4 * j;
                    consider(v[u].x, i);
                    consider(v[u].y, i + 1);
                    consider(v[u].z, i + 2);
                    consider(v[u].w, i + 3);
                }
            }
        }
        done = begin + 4 * n4;
    }
    for (int i = done + threadIdx.x; i < end; i += blockDim.x) consider(x[i], i);
    auto better = [](float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) {
            bv = ov;
            bi = oi;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        best_v[warp] = bv;
        best_i[warp] = bi;
    }
    __syncthreads();
    if (warp != 0) return;
    const int nwarps = blockDim.x >> 5;
    bv = lane < nwarps ? best_v[lane] : -FLT_MAX;
    bi = lane < nwarps ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if (chunks == 1) {
        if (lane == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
        return;
    }
    if (lane == 0) {
        part_v[(size_t)row * chunks + chunk] = bv;
        part_i[(size_t)row * chunks + chunk] = bi;
        __threadfence();
        ticket = atomicAdd(counters + row, 1);
    }
    __syncwarp();
    if (ticket != chunks - 1) return;
    __threadfence();
    if (lane == 0) counters[row] = 0;
    bv = -FLT_MAX;
    bi = 0x7fffffff;
    for (int c = lane; c < chunks; c += 32) {
        const float v = __ldcg(part_v + (size_t)row * chunks + c);
        const int i = __ldcg(part_i + (size_t)row * chunks + c);
        if (better(v, i, bv, bi)) {
            bv = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if (lane == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

// logits: [rows][row_stride >= vocab] float32; seq_ids [rows] int64 and steps [rows] int32 are read only when sampling.
// chunks > 1 needs scratch: part_v float32 [rows * chunks], part_i int32 [rows * chunks], counters int32 [rows], zero
// before the first call (the kernel leaves them zero).
QF_EXPORT int qf_sample(const float* logits, int rows, int vocab, long long row_stride, float temperature,
                        unsigned long long seed, const long long* seq_ids, const int* steps, int* out, int chunks,
                        float* part_v, int* part_i, int* counters, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (chunks < 1 || (chunks > 1 && (!part_v || !part_i || !counters))) return (int)cudaErrorInvalidValue;
    return (int)launch_pdl(sample_kernel, dim3(chunks, rows), dim3(256), 0, stream, logits, vocab, row_stride, temperature, seed, seq_ids, steps, out,
                                                          chunks, part_v, part_i, counters);
}
