// Step preparation on the device: the token a request sampled last lives in a per-slot table, so that the next step
// can be enqueued before the host has read it. `feed` copies it into the step's input for the rows that ask for it;
// `store` files the step's sampled tokens (core/holon/core/executor.py:477-488, 606-617 do the same with indexing ops).
#include "common.cuh"

__global__ void feed_tokens_kernel(int32_t* __restrict__ token_ids, const int32_t* __restrict__ last_tokens,
                                   const int32_t* __restrict__ row_slot, const int32_t* __restrict__ query_start,
                                   const int32_t* __restrict__ from_last, int rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < rows && from_last[r]) token_ids[query_start[r]] = last_tokens[row_slot[r]];
}

__global__ void store_tokens_kernel(int32_t* __restrict__ last_tokens, const int32_t* __restrict__ slots,
                                    const int32_t* __restrict__ tokens, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) last_tokens[slots[i]] = tokens[i];
}

// For every row r with from_last[r] != 0: token_ids[query_start[r]] = last_tokens[row_slot[r]].
extern "C" int hb_feed_tokens(int32_t* token_ids, const int32_t* last_tokens, const int32_t* row_slot,
                              const int32_t* query_start, const int32_t* from_last, int rows, hb_stream stream) {
    if (rows == 0) return 0;
    feed_tokens_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>(token_ids, last_tokens, row_slot, query_start,
                                                                             from_last, rows);
    HB_LAUNCH_CHECK("feed_tokens");
    return 0;
}

// last_tokens[slots[i]] = tokens[i] for i < n.
extern "C" int hb_store_tokens(int32_t* last_tokens, const int32_t* slots, const int32_t* tokens, int n, hb_stream stream) {
    if (n == 0) return 0;
    store_tokens_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(last_tokens, slots, tokens, n);
    HB_LAUNCH_CHECK("store_tokens");
    return 0;
}
