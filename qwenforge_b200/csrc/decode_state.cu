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
    grid_chain_entry();
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
    return (int)launch_pdl(decode_advance_kernel, dim3(1), dim3(n_rows), 0, stream, sampled, token_ids, tok_pos, slots, steps, budgets, stop_ids,
                                                    n_stop, out_tokens, cursor, max_steps, n_rows);
}

// The same step of the rows' state, and the NEXT step's first kernel with it: a block per row updates the row as above
// and then copies the embedding of the row's next input token into the float32 stream `hidden[row]`, so that the next
// step starts at its first layer. All blocks read the cursor before any block can move it: the block that draws the
// last ticket does that (and puts the ticket counter back to zero).
template <typename T>
__global__ void __launch_bounds__(128)
decode_advance_embed_kernel(const int* __restrict__ sampled, int* __restrict__ token_ids, int* __restrict__ tok_pos,
                            int* __restrict__ slots, int* __restrict__ steps, const int* __restrict__ budgets,
                            const int* __restrict__ stop_ids, int n_stop, int* __restrict__ out_tokens,
                            int* __restrict__ cursor, int max_steps, const T* __restrict__ table, int vocab, int width,
                            float* __restrict__ hidden, int* __restrict__ ticket, int* err) {
    grid_chain_entry();
    __shared__ int next_s, at_s;
    const int r = blockIdx.x, n_rows = gridDim.x;
    if (threadIdx.x == 0) {
        const int at = cursor[0];
        if (at < max_steps) {
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
        next_s = token_ids[r];
        at_s = at;
    }
    __syncthreads();
    int id = next_s;
    const bool bad = id < 0 || id >= vocab;
    if (bad) {
        if (threadIdx.x == 0) atomicOr(err, QF_ERR_TOKEN_RANGE);
        id = 0;
    }
    const T* row = table + (size_t)id * width;
    float* dst = hidden + (size_t)r * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = bad ? 0.f : Num<T>::to_f(row[c]);
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ticket, 1) == n_rows - 1) {
            *ticket = 0;
            if (at_s < max_steps) cursor[0] = at_s + 1;
        }
    }
}

// table [vocab][width] bfloat16 or float32, hidden float32 [n_rows][width], ticket one int that is zero before the first
// call (the kernel leaves it zero).
QF_EXPORT int qf_decode_advance_embed(const int* sampled, int* token_ids, int* tok_pos, int* slots, int* steps,
                                      const int* budgets, const int* stop_ids, int n_stop, int* out_tokens, int* cursor,
                                      int max_steps, int n_rows, int is_bf16, const void* table, int vocab, int width,
                                      float* hidden, int* ticket, int* err, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    int code;
    if (is_bf16)
        code = (int)launch_pdl(decode_advance_embed_kernel<bf16>, dim3(n_rows), dim3(128), 0, stream, sampled, token_ids, tok_pos, slots, steps, budgets,
                                                                     stop_ids, n_stop, out_tokens, cursor, max_steps,
                                                                     (const bf16*)table, vocab, width, hidden, ticket, err);
    else
        code = (int)launch_pdl(decode_advance_embed_kernel<float>, dim3(n_rows), dim3(128), 0, stream, sampled, token_ids, tok_pos, slots, steps, budgets,
                                                                      stop_ids, n_stop, out_tokens, cursor, max_steps,
                                                                      (const float*)table, vocab, width, hidden, ticket, err);
    return code;
}
