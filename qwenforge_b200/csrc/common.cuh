// Shared helpers of the sm_100a kernels: element types, conversions, warp reductions,
// the exported C calling convention and the cache addressing that every kernel uses.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

#define QF_EXPORT extern "C" __attribute__((visibility("default")))

// Tokens per cache page. The cache hands out storage in pages; a page holds the keys
// (or values) of QF_PAGE consecutive positions of one sequence for every kv head.
#define QF_PAGE 64

// Bits of the device error word (set with atomicOr, read by the host after a step).
#define QF_ERR_TOKEN_RANGE 1   // a token id outside the embedding table
#define QF_ERR_NO_PAGE 2       // a position whose cache page is not allocated
#define QF_ERR_ROW_RANGE 4     // a gathered row index outside the activations
#define QF_ERR_COPY_TIMEOUT 8  // a bulk copy did not complete within the wait limit
#define QF_ERR_BARRIER_TIMEOUT 16  // a barrier over the blocks of a persistent kernel was not reached within the wait limit

template <typename T> struct Num;
template <> struct Num<float> {
    static __device__ __forceinline__ float to_f(float x) { return x; }
    static __device__ __forceinline__ float from_f(float x) { return x; }
};
template <> struct Num<bf16> {
    static __device__ __forceinline__ float to_f(bf16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ bf16 from_f(float x) { return __float2bfloat16_rn(x); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ uint32_t warp_sum_u32(uint32_t v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` is 33 floats
// of shared memory. The order of the additions depends only on blockDim, never on the data.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Where one sequence's keys and values of one schedule entry lie.
//   base        first element of this entry's storage: [pages][2 (k,v)][kv_heads][QF_PAGE][head_dim]
//   page_elems  elements per page = 2 * kv_heads * QF_PAGE * head_dim
//   table       [slots][table_stride] page ids of each slot's logical pages, -1 where none is held
template <typename T> struct KvSite {
    T* base;
    const int* table;
    long long page_elems;
    int table_stride;
    int kv_heads;
    int head_dim;
};

// Pointer to head `h`'s key (which=0) or value (which=1) row at position `pos`; nullptr if that page is not held.
template <typename T>
__device__ __forceinline__ T* kv_row(const KvSite<T>& s, int slot, int pos, int h, int which) {
    const int page = s.table[(long long)slot * s.table_stride + pos / QF_PAGE];
    if (page < 0) return nullptr;
    return s.base + (long long)page * s.page_elems +
           ((long long)(which * s.kv_heads + h) * QF_PAGE + (pos % QF_PAGE)) * s.head_dim;
}

// Streaming multiprocessors of the current device, asked once per device (0 if the device cannot be asked): what
// grids, split counts and one-wave plans are sized by.
static inline int qf_sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached[dev] = n;
    }
    return cached[dev];
}

// Programmatic dependent launch. A kernel launched with `launch_pdl` may start while the kernel before it on the
// stream is still running; it must call grid_dependency_wait() before it reads anything that kernel wrote or
// writes anything at all. What it does before that call (fetching weights, which no kernel writes) overlaps the
// previous kernel's tail. grid_launch_dependents() lets the NEXT kernel start its own preamble early. Both are
// no-ops in a kernel that was launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The first statement of a small kernel that has nothing to do before its input is there: it lets the kernel after it
// start its own preamble (weight copies, page-table walks) at once, then waits for the kernel before it.
__device__ __forceinline__ void grid_chain_entry() {
    grid_launch_dependents();
    grid_dependency_wait();
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, KArgs(args)...);
}
