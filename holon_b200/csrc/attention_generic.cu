// Paged attention for any sizes on CUDA cores, 32-bit arithmetic throughout: the float32 engine's attention, and
// the bfloat16 engine's for shapes its tensor-core kernels refuse. One warp per (query token, query head).
// Each lane scores one key of a block of 32; the block's softmax weights then sweep the values, each lane owning
// every 32nd dimension of the output.
#include "common.cuh"

#define GEN_WARPS 4
#define GEN_MAX_PER_LANE 16          // head_dim up to 512

template <typename T>
__global__ void attention_generic_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ kv,
                                         const int32_t* __restrict__ block_table, int table_stride,
                                         const int32_t* __restrict__ row_slot, const int32_t* __restrict__ query_start,
                                         const int32_t* __restrict__ kv_len, int rows, int tokens, int heads,
                                         int kv_heads, int head_dim, int pages, int page_size, float scale,
                                         int window) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * GEN_WARPS + warp;
    if (item >= (long)tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item % heads);
    float* qs = smem + (size_t)warp * head_dim;

    int lo = 0, hi = rows;                           // the row b with query_start[b] <= t < query_start[b + 1]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (query_start[mid] <= t) lo = mid; else hi = mid;
    }
    const int b = lo;
    const int n = kv_len[b];
    T* o = out + ((size_t)t * heads + h) * head_dim;
    const int pos = n - query_start[b + 1] + t;       // the query's position in its sequence
    if (n <= 0 || pos < 0) {
        for (int d = lane; d < head_dim; d += 32) o[d] = from_f32<T>(0.f);
        return;
    }
    const T* qr = q + ((size_t)t * heads + h) * head_dim;
    for (int d = lane; d < head_dim; d += 32) qs[d] = to_f32(qr[d]) * scale;
    __syncwarp();

    const int hk = h / (heads / kv_heads);
    const int32_t* table = block_table + (size_t)row_slot[b] * table_stride;
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    float m = -INFINITY, l = 0.f, acc[GEN_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < GEN_MAX_PER_LANE; ++i) acc[i] = 0.f;

    for (int j0 = first; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= pos;
        long base = -1;                              // element offset of key j's row of this kv head
        if (valid) {
            const int page = table[j / page_size];
            if (page >= 0 && page < pages)
                base = ((((long)page * 2) * kv_heads + hk) * page_size + j % page_size) * head_dim;
        }
        float s = -INFINITY;
        if (base >= 0) {
            const T* kr = kv + base;
            float dot = 0.f;
            for (int d = 0; d < head_dim; ++d) dot += qs[d] * to_f32(kr[d]);
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = m_new == -INFINITY ? 1.f : expf(m - m_new);     // m = -inf at the start: exp(-inf) = 0
        const float p = base >= 0 ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < GEN_MAX_PER_LANE; ++i) acc[i] *= corr;
        const int count = min(32, pos - j0 + 1);
        const long v_shift = (long)kv_heads * page_size * head_dim;     // from a key row to its value row
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long bj = __shfl_sync(0xffffffffu, base, jj);
            if (bj < 0) continue;
            const T* vr = kv + bj + v_shift;
#pragma unroll
            for (int i = 0; i < GEN_MAX_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] += pj * to_f32(vr[d]);
            }
        }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < GEN_MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) o[d] = from_f32<T>(acc[i] * inv);
    }
}

extern "C" int hb_attention_generic(void* out, const void* q, const void* kv, int dtype, const int32_t* block_table,
                                    int table_stride, const int32_t* row_slot, const int32_t* query_start,
                                    const int32_t* kv_len, int rows, int tokens, int heads, int kv_heads,
                                    int head_dim, int pages, int page_size, float scale, int window,
                                    hb_stream stream) {
    if (tokens == 0 || rows == 0) return 0;
    if (head_dim > 32 * GEN_MAX_PER_LANE) HB_REFUSE("attention: head_dim %d is above %d", head_dim, 32 * GEN_MAX_PER_LANE);
    if (kv_heads < 1 || heads % kv_heads) HB_REFUSE("attention: %d heads are no multiple of %d kv heads", heads, kv_heads);
    cudaStream_t s = (cudaStream_t)stream;
    const long items = (long)tokens * heads;
    const unsigned blocks = (unsigned)((items + GEN_WARPS - 1) / GEN_WARPS);
    const size_t smem = (size_t)GEN_WARPS * head_dim * sizeof(float);
    if (dtype == HB_F32)
        attention_generic_kernel<float><<<blocks, GEN_WARPS * 32, smem, s>>>(
            (float*)out, (const float*)q, (const float*)kv, block_table, table_stride, row_slot, query_start, kv_len,
            rows, tokens, heads, kv_heads, head_dim, pages, page_size, scale, window);
    else if (dtype == HB_BF16)
        attention_generic_kernel<bf16><<<blocks, GEN_WARPS * 32, smem, s>>>(
            (bf16*)out, (const bf16*)q, (const bf16*)kv, block_table, table_stride, row_slot, query_start, kv_len,
            rows, tokens, heads, kv_heads, head_dim, pages, page_size, scale, window);
    else HB_REFUSE("attention: dtype %d", dtype);
    HB_LAUNCH_CHECK("attention_generic");
    return 0;
}
