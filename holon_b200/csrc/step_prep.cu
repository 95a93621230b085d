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

__global__ void scatter_rows_kernel(int32_t* __restrict__ table, const int32_t* __restrict__ slots,
                                    const int32_t* __restrict__ rows, int width, int table_rows) {
    const int slot = slots[blockIdx.x];
    if (slot < 0 || slot >= table_rows) return;
    for (int i = threadIdx.x; i < width; i += blockDim.x) table[(size_t)slot * width + i] = rows[(size_t)blockIdx.x * width + i];
}

// table[slots[i], :] = rows[i, :] for i < n (rows of `width` int32; slots outside [0, table_rows) are skipped).
extern "C" int hb_scatter_rows(int32_t* table, const int32_t* slots, const int32_t* rows, int n, int width, int table_rows,
                               hb_stream stream) {
    if (n == 0 || width == 0) return 0;
    scatter_rows_kernel<<<n, 128, 0, (cudaStream_t)stream>>>(table, slots, rows, width, table_rows);
    HB_LAUNCH_CHECK("scatter_rows");
    return 0;
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
