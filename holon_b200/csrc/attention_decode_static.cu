// The decode attention entry point that allocates nothing; see attention_decode_static.h for who needs it and why.
#include <mutex>

#include "attention_decode_static.h"
#include "common.cuh"

extern "C" size_t hb_attention_decode_scratch_floats(int rows, int heads, int head_dim, int splits);

// The partial results of the split kernel live here. In host code this name is only a handle for the runtime's symbol
// calls, not a device address: a kernel must be given what cudaGetSymbolAddress returns.
static __device__ __align__(256) float g_decode_scratch[HB_DECODE_STATIC_SCRATCH_FLOATS];

#define HB_MAX_DEVICES 64
static float* g_scratch_address[HB_MAX_DEVICES];        // by device ordinal; null until that device's first call
static std::mutex g_setup_lock;

// The array's address on the caller's current device, looked up once per device.
static int scratch_on_current_device(float** address) {
    int device = -1;
    HB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= HB_MAX_DEVICES) HB_REFUSE("attention_decode_bf16_static: device ordinal %d", device);
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (g_scratch_address[device] == nullptr) {
        void* p = nullptr;
        HB_CUDA(cudaGetSymbolAddress(&p, g_decode_scratch));
        g_scratch_address[device] = (float*)p;
    }
    *address = g_scratch_address[device];
    return 0;
}

extern "C" size_t hb_attention_decode_static_capacity(void) { return HB_DECODE_STATIC_SCRATCH_FLOATS; }

extern "C" int hb_attention_decode_bf16_static(void* out, const void* q, const void* kv, const int32_t* block_table,
                                               int table_stride, const int32_t* row_slot, const int32_t* query_start,
                                               const int32_t* kv_len, int rows, int heads, int kv_heads, int head_dim,
                                               int pages, int page_size, float scale, int window, int splits,
                                               hb_stream stream) {
    if (rows == 0) return 0;
    if (rows < 0 || heads < 1 || head_dim < 1 || splits < 1)
        HB_REFUSE("attention_decode_bf16_static: rows %d, heads %d, head_dim %d, splits %d", rows, heads, head_dim, splits);
    const size_t need = hb_attention_decode_scratch_floats(rows, heads, head_dim, splits);
    if (need > HB_DECODE_STATIC_SCRATCH_FLOATS)
        HB_REFUSE("attention_decode_bf16_static: %d rows x %d heads x %d splits at head_dim %d need %zu floats of "
                  "scratch, the built-in array holds %u; use fewer splits or hb_attention_decode_bf16 with your own scratch",
                  rows, heads, splits, head_dim, need, HB_DECODE_STATIC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (need) {
        const int rc = scratch_on_current_device(&scratch);
        if (rc) return rc;
    }
    return hb_attention_decode_bf16(out, scratch, q, kv, block_table, table_stride, row_slot, query_start, kv_len,
                                    rows, heads, kv_heads, head_dim, pages, page_size, scale, window, splits, stream);
}
