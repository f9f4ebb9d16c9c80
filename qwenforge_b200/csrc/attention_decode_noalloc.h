/* Split-K decode attention that allocates nothing.

   This entry point has no counterpart in the reference project (its decode attention gets its scratch
   tensors from PyTorch's allocator, student_engine.py:1022-1045). It exists for callers of this library
   that cannot allocate device memory at the moment they need attention: code running where every byte of
   the GPU was handed out up front (a fixed memory plan, an embedding host that forbids cudaMalloc after
   start-up), or code on a path where an allocation could block or fail in the middle of a step. Such a
   caller cannot create the scratch that qf_attention_decode wants for its partial results.

   qf_attention_decode_noalloc takes the arguments of qf_attention_decode without the three scratch
   pointers. Its scratch is one array inside the library, QF_NOALLOC_MAX_ROWS x QF_NOALLOC_MAX_HEAD_DIM
   floats plus small tables (about 4.4 MB), which every GPU that loads the library keeps until the
   process exits. The function calls no cudaMalloc, cudaFree or any allocating routine.

   n_splits is the most blocks that share one (sequence, kv head); the kernel gives each sequence as many of them
   as its share of the batch's pages asks for.

   Limits: n_seqs * n_heads * n_splits <= QF_NOALLOC_MAX_ROWS, head_dim <= QF_NOALLOC_MAX_HEAD_DIM,
   n_seqs * kv_heads * ceil(group / 16) <= QF_NOALLOC_MAX_COUNTERS (all only when n_splits > 1: one split
   needs no scratch), and in every call ceil(n_seqs / 4) + min(n_seqs * n_splits, n_seqs + SMs / (kv_heads * ceil(group / 16)))
   <= QF_NOALLOC_MAX_PAIRS (the plan of which block takes which run of which sequence). Larger calls return QF_NOALLOC_TOO_LARGE and qf_attention_decode_noalloc_error()
   says which limit was passed; nothing is launched.

   First call on a device: it looks up the array's device address (once per device, with that device
   current). Make that first call outside of any stream capture.

   All calls share the one array, and it keeps the previous call's contents; the function clears the
   part that has to start at zero (the ticket counters) on the given stream before it launches. Two calls
   whose kernels overlap on the GPU (different streams without an ordering between them) race on the
   array and give wrong results: order them.

   Return value: 0 on success, QF_NOALLOC_TOO_LARGE, or a CUDA error code (1 = a shape without a kernel). */
#pragma once
#include <cuda_runtime.h>

#define QF_NOALLOC_MAX_ROWS 8192
#define QF_NOALLOC_MAX_HEAD_DIM 128
#define QF_NOALLOC_MAX_COUNTERS 4096
#define QF_NOALLOC_MAX_PAIRS 8192
#define QF_NOALLOC_TOO_LARGE (-2)

#ifdef __cplusplus
extern "C" {
#endif

int qf_attention_decode_noalloc(const void* q, void* out, const int* cu_q, const int* tok_pos, const int* slots,
                                void* base, const int* table, long long page_elems, int table_stride, int kv_heads,
                                int head_dim, int n_heads, int n_seqs, float scale, int window, int n_splits, int* err,
                                cudaStream_t stream);

/* The message of the calling thread's last failed call ("" after a success). */
const char* qf_attention_decode_noalloc_error(void);

#ifdef __cplusplus
}
#endif
