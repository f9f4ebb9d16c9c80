// The host-free part of a decode step: after the sampling kernel has chosen each row's next token, record it,
// make it the next step's input, advance the row's position and counters, and retire rows that produced a stop
// token or spent their budget (a retired row's slot becomes -1: from then on it is a padding entry that touches
// no cache). With this kernel a whole decode step can be replayed from a CUDA graph without host work in between.
#include "common.cuh"

// out_tokens: [max_steps][n_rows], -1 where a row produced nothing. cursor[0]: steps recorded so far.
__global__ void decode_advance_kernel(const int* __restrict__ sampled, int* __restrict__ token_ids,
                                      int* __restrict__ tok_pos, int* __restrict__ slots, int* __restrict__ steps,
                                      const int* __restrict__ budgets, const int* __restrict__ stop_ids, int n_stop,
                                      int* __restrict__ out_tokens, int* __restrict__ cursor, int max_steps,
                                      int n_rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    const int at = cursor[0];
    if (r < n_rows && at < max_steps) {
        int produced = -1;
        if (slots[r] >= 0) {
            const int token = sampled[r];
            produced = token;
            token_ids[r] = token;
            tok_pos[r] += 1;
            const int made = steps[r] + 1;
            steps[r] = made;
            bool done = made >= budgets[r];
            for (int i = 0; i < n_stop; ++i) done = done || (stop_ids[i] == token);
            if (done) slots[r] = -1;
        }
        out_tokens[(size_t)at * n_rows + r] = produced;
    }
    // every thread of this launch has read cursor[0] before any block can see the increment of a LATER launch;
    // within this launch only one thread writes it, after a grid of one block (n_rows <= 1024)
    __syncthreads();
    if (r == 0 && at < max_steps) cursor[0] = at + 1;
}

QF_EXPORT int qf_decode_advance(const int* sampled, int* token_ids, int* tok_pos, int* slots, int* steps,
                                const int* budgets, const int* stop_ids, int n_stop, int* out_tokens, int* cursor,
                                int max_steps, int n_rows, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_rows > 1024) return (int)cudaErrorInvalidValue;  // one block, so that the cursor has one writer
    decode_advance_kernel<<<1, n_rows, 0, stream>>>(sampled, token_ids, tok_pos, slots, steps, budgets, stop_ids,
                                                    n_stop, out_tokens, cursor, max_steps, n_rows);
    return (int)cudaGetLastError();
}
