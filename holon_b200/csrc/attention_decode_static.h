// hb_attention_decode_bf16_static: decode attention for callers that cannot give the kernel scratch memory.
//
// This entry point has no counterpart in mxinO/holon; it exists for users of this library only.
//
// The split decode kernel (hb_attention_decode_bf16 in api.h) cuts each row's keys into parts and needs global
// scratch for the parts' partial results. Its normal caller, the Python engine, takes that scratch from torch's
// allocator on every call. Two kinds of caller cannot do that. A serving process that handed all free device memory
// to its cache pools at start has nothing left to allocate from, and an allocation that fails or stalls in the middle
// of serving is worse than a fixed cost paid once. And a program that reaches this library through the C symbol
// alone (another language, another runtime) has no allocator of ours to call and may not want to write one for a few
// megabytes. For them the scratch lives inside the library: a file-scope device array of
// HB_DECODE_STATIC_SCRATCH_FLOATS floats (8 MiB), which every GPU that loads the library holds until the process ends.
//
// Arguments and result are those of hb_attention_decode_bf16 without `scratch`. The call allocates nothing: no
// cudaMalloc, no cudaFree, no allocating library routine. A launch whose partial results would not fit the array
// (rows * heads * splits * (head_dim + 2) floats) is refused with HB_ERR_REFUSED and a message that names both
// numbers; use fewer splits or the entry point that takes scratch.
//
// Set-up: the first call on each device looks the array's device address up (cudaGetSymbolAddress, with the
// caller's current device) and remembers it per device; make that first call once at start, before any stream
// capture begins. Later calls on that device only launch.
//
// Sharing: all calls use the one array, and it keeps what the last call left there. Nothing in it has to start at
// zero: every launch writes each partial result before the merge reads it. But two calls that overlap on the GPU
// (different streams, no ordering between them) write the same cells and race; order such calls with events or keep
// them on one stream.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "api.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HB_DECODE_STATIC_SCRATCH_FLOATS (2u * 1024u * 1024u)

// The capacity of the built-in scratch, in floats.
size_t hb_attention_decode_static_capacity(void);

int hb_attention_decode_bf16_static(void* out, const void* q, const void* kv, const int32_t* block_table,
                                    int table_stride, const int32_t* row_slot, const int32_t* query_start,
                                    const int32_t* kv_len, int rows, int heads, int kv_heads, int head_dim,
                                    int pages, int page_size, float scale, int window, int splits, hb_stream stream);

#ifdef __cplusplus
}
#endif
