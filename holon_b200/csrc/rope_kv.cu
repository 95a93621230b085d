// q/k RMSNorm per head + rotation + write of keys and values into the paged cache, one kernel.
// One warp per (token, head): query heads first, then key heads, then value heads (a plain copy).
#include "common.cuh"

template <typename T> struct Pair;
template <> struct Pair<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *(const float2*)p; }
    static __device__ __forceinline__ void store(float* p, float a, float b) { *(float2*)p = make_float2(a, b); }
};
template <> struct Pair<bf16> {
    static __device__ __forceinline__ float2 load(const bf16* p) { return __bfloat1622float2(*(const __nv_bfloat162*)p); }
    static __device__ __forceinline__ void store(bf16* p, float a, float b) { *(__nv_bfloat162*)p = __floats2bfloat162_rn(a, b); }
};

// VEC: head_dim and rotary_dim are multiples of 4, so a lane moves two neighbouring values at a time.
template <typename T, typename TW, bool VEC>
__global__ void qk_norm_rope_kv_write_kernel(T* __restrict__ q_out, const T* __restrict__ qkv,
                                             const int32_t* __restrict__ positions, const float* __restrict__ table,
                                             int rotary_dim, int max_positions, const TW* __restrict__ q_weight,
                                             const TW* __restrict__ k_weight, float eps, float offset,
                                             T* __restrict__ kv, const int32_t* __restrict__ write_index, int pages,
                                             int page_size, int heads, int kv_heads, int head_dim) {
    extern __shared__ float smem[];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int items = heads + (kv ? 2 * kv_heads : 0);
    float* y = smem + (size_t)warp * head_dim;
    for (int item = blockIdx.y * warps + warp; item < items; item += gridDim.y * warps) {
    __syncwarp();                                    // the buffer y is reused from one head to the next
    const int width = (heads + 2 * kv_heads) * head_dim;
    const T* src = qkv + (size_t)t * width + (size_t)item * head_dim;       // q heads, k heads, v heads in a row

    T* dst;
    const TW* weight = nullptr;
    bool rotate = false;
    if (item < heads) {
        dst = q_out + ((size_t)t * heads + item) * head_dim;
        weight = q_weight;
        rotate = true;
    } else {
        const int w = write_index[t];
        if (w < 0) continue;
        const int page = w / page_size, off = w % page_size;
        if (page >= pages) continue;
        const int is_v = item >= heads + kv_heads;
        const int head = item - heads - (is_v ? kv_heads : 0);
        dst = kv + ((((size_t)page * 2 + is_v) * kv_heads + head) * page_size + off) * head_dim;
        weight = is_v ? nullptr : k_weight;
        rotate = !is_v;
    }
    const int half = rotary_dim >> 1;
    if (VEC) {
        if (!rotate) {                               // values: copied as they are
            for (int d = lane * 2; d < head_dim; d += 64) {
                const float2 v = Pair<T>::load(src + d);        // (to 32-bit and back is exact)
                Pair<T>::store(dst + d, v.x, v.y);
            }
            continue;
        }
        float ss = 0.f;
        for (int d = lane * 2; d < head_dim; d += 64) {
            const float2 v = Pair<T>::load(src + d);
            y[d] = v.x; y[d + 1] = v.y;
            ss += v.x * v.x + v.y * v.y;
        }
        if (weight) {
            ss = warp_sum(ss);
            const float rstd = rsqrtf(ss / (float)head_dim + eps);
            for (int d = lane * 2; d < head_dim; d += 64) {
                const float2 w = Pair<TW>::load(weight + d);
                y[d] = rounded<T>(y[d] * rstd * (w.x + offset));
                y[d + 1] = rounded<T>(y[d + 1] * rstd * (w.y + offset));
            }
        }
        __syncwarp();
        int pos = positions[t];
        pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
        const float* cs = table + (size_t)pos * rotary_dim;
        for (int i = lane * 2; i < half; i += 64) {
            const float2 c = *(const float2*)(cs + i), sn = *(const float2*)(cs + half + i);
            const float a0 = y[i], a1 = y[i + 1], b0 = y[i + half], b1 = y[i + half + 1];
            Pair<T>::store(dst + i, a0 * c.x - b0 * sn.x, a1 * c.y - b1 * sn.y);
            Pair<T>::store(dst + i + half, b0 * c.x + a0 * sn.x, b1 * c.y + a1 * sn.y);
        }
        for (int d = rotary_dim + lane * 2; d < head_dim; d += 64) Pair<T>::store(dst + d, y[d], y[d + 1]);
        continue;
    }
    if (!rotate) {                                   // values: copied as they are
        for (int d = lane; d < head_dim; d += 32) dst[d] = src[d];
        continue;
    }
    float ss = 0.f;
    for (int d = lane; d < head_dim; d += 32) {
        const float v = to_f32(src[d]);
        y[d] = v;
        ss += v * v;
    }
    if (weight) {
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / (float)head_dim + eps);
        for (int d = lane; d < head_dim; d += 32) y[d] = rounded<T>(y[d] * rstd * (to_f32(weight[d]) + offset));
    }
    __syncwarp();
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
    const float* cs = table + (size_t)pos * rotary_dim;
    for (int i = lane; i < half; i += 32) {
        const float a = y[i], b = y[i + half], c = cs[i], s = cs[half + i];
        dst[i] = from_f32<T>(a * c - b * s);
        dst[i + half] = from_f32<T>(b * c + a * s);
    }
    for (int d = rotary_dim + lane; d < head_dim; d += 32) dst[d] = from_f32<T>(y[d]);
    }
}

// The production shape, bfloat16 with head_dim = rotary_dim = 128: eight lanes share one (token, head), each holding
// 8 values of the head's first half and the 8 it pairs with in the second half, so every access is 16 bytes wide,
// the norm's sum takes three shuffles and nothing goes through shared memory.
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 p = __bfloat1622float2(*(const __nv_bfloat162*)&w[i]);
        f[2 * i] = p.x; f[2 * i + 1] = p.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *(uint32_t*)&p;
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
template <typename TW> __device__ __forceinline__ void load_w8(const TW* w, float (&f)[8]);
template <> __device__ __forceinline__ void load_w8<bf16>(const bf16* w, float (&f)[8]) { unpack8(*(const uint4*)w, f); }
template <> __device__ __forceinline__ void load_w8<float>(const float* w, float (&f)[8]) {
    const float4 a = *(const float4*)w, b = *(const float4*)(w + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

template <typename TW>
__global__ void __launch_bounds__(256) qk_norm_rope_kv_write_d128_kernel(
        bf16* __restrict__ q_out, const bf16* __restrict__ qkv, const int32_t* __restrict__ positions,
        const float* __restrict__ table, int max_positions, const TW* __restrict__ q_weight,
        const TW* __restrict__ k_weight, float eps, float offset, bf16* __restrict__ kv,
        const int32_t* __restrict__ write_index, int pages, int page_size, int tokens, int heads, int kv_heads) {
    constexpr int D = 128, HALF = 64;
    const int items = heads + (kv ? 2 * kv_heads : 0);
    const long unit = (long)blockIdx.x * 32 + (threadIdx.x >> 3);   // one (token, head) per eight lanes
    const int sub = threadIdx.x & 7;
    const bool live = unit < (long)tokens * items;
    const int t = live ? (int)(unit / items) : 0, item = live ? (int)(unit % items) : 0;
    const bf16* src = qkv + (size_t)t * (heads + 2 * kv_heads) * D + (size_t)item * D;
    bf16* dst = nullptr;
    const TW* weight = nullptr;
    bool rotate = false;
    if (live) {
        if (item < heads) {
            dst = q_out + ((size_t)t * heads + item) * D;
            weight = q_weight;
            rotate = true;
        } else {
            const int w = write_index[t];
            const int page = w >= 0 ? w / page_size : -1, off = w >= 0 ? w % page_size : 0;
            if (page >= 0 && page < pages) {
                const int is_v = item >= heads + kv_heads;
                const int head = item - heads - (is_v ? kv_heads : 0);
                dst = kv + ((((size_t)page * 2 + is_v) * kv_heads + head) * page_size + off) * D;
                weight = is_v ? nullptr : k_weight;
                rotate = !is_v;
            }
        }
    }
    // Everything the rotation needs is asked for before the first result is used (the position first: the table row
    // hangs on it), so that a step of a few tokens pays two trips to memory instead of four.
    int pos = live && rotate ? positions[t] : 0;
    uint4 ra = make_uint4(0, 0, 0, 0), rb = ra;
    if (dst) { ra = *(const uint4*)(src + sub * 8); rb = *(const uint4*)(src + HALF + sub * 8); }
    float wa[8], wb[8], c[8], sn[8];
    if (dst && weight) {
        load_w8<TW>(weight + sub * 8, wa);
        load_w8<TW>(weight + HALF + sub * 8, wb);
    }
    if (dst && rotate) {
        pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
        const float* cs = table + (size_t)pos * D;
        load_w8<float>(cs + sub * 8, c);
        load_w8<float>(cs + HALF + sub * 8, sn);
    }
    if (dst && !rotate) {                             // values: copied as they are
        *(uint4*)(dst + sub * 8) = ra;
        *(uint4*)(dst + HALF + sub * 8) = rb;
    }
    float a[8], b[8];
    unpack8(ra, a);
    unpack8(rb, b);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + b[i] * b[i];
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);        // (every lane takes part: a group without work adds zeros)
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    if (!dst || !rotate) return;
    if (weight) {
        const float rstd = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            a[i] = rounded<bf16>(a[i] * rstd * (wa[i] + offset));
            b[i] = rounded<bf16>(b[i] * rstd * (wb[i] + offset));
        }
    }
    float oa[8], ob[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        oa[i] = a[i] * c[i] - b[i] * sn[i];
        ob[i] = b[i] * c[i] + a[i] * sn[i];
    }
    *(uint4*)(dst + sub * 8) = pack8(oa);
    *(uint4*)(dst + HALF + sub * 8) = pack8(ob);
}

template <typename T, typename TW>
static int launch(void* q_out, const void* qkv, const int32_t* positions, const float* table, int rotary_dim,
                  int max_positions, const void* qw, const void* kw, float eps, float offset, void* kv,
                  const int32_t* write_index, int pages, int page_size, int tokens, int heads, int kv_heads,
                  int head_dim, cudaStream_t s) {
    const int items = heads + (kv ? 2 * kv_heads : 0);
    if constexpr (sizeof(T) == 2) {
        const bool aligned = (((uintptr_t)q_out | (uintptr_t)qkv | (uintptr_t)table | (uintptr_t)qw | (uintptr_t)kw | (uintptr_t)kv) % 16) == 0;
        if (head_dim == 128 && rotary_dim == 128 && aligned && (long)tokens * items < (1l << 31)) {
            const unsigned blocks = (unsigned)(((long)tokens * items + 31) / 32);
            qk_norm_rope_kv_write_d128_kernel<TW><<<blocks, 256, 0, s>>>(
                (bf16*)q_out, (const bf16*)qkv, positions, table, max_positions, (const TW*)qw, (const TW*)kw, eps, offset,
                (bf16*)kv, write_index, pages, page_size, tokens, heads, kv_heads);
            HB_LAUNCH_CHECK("qk_norm_rope_kv_write");
            return 0;
        }
    }
    // Few tokens (decode): many small blocks, one head per warp. Many tokens: one block per token whose 8 warps walk
    // the heads, so that the launch is not made of tens of thousands of tiny blocks.
    const int warps = tokens >= 256 ? 8 : 4;
    dim3 grid(tokens, tokens >= 256 ? 1 : (items + warps - 1) / warps);
    const size_t smem = (size_t)warps * head_dim * sizeof(float);
    const bool vec = head_dim % 4 == 0 && rotary_dim % 4 == 0 &&
                     (((uintptr_t)q_out | (uintptr_t)qkv | (uintptr_t)table | (uintptr_t)qw | (uintptr_t)kw | (uintptr_t)kv) % 8 == 0);
    auto kernel = vec ? qk_norm_rope_kv_write_kernel<T, TW, true> : qk_norm_rope_kv_write_kernel<T, TW, false>;
    kernel<<<grid, warps * 32, smem, s>>>(
        (T*)q_out, (const T*)qkv, positions, table, rotary_dim, max_positions, (const TW*)qw, (const TW*)kw, eps,
        offset, (T*)kv, write_index, pages, page_size, heads, kv_heads, head_dim);
    HB_LAUNCH_CHECK("qk_norm_rope_kv_write");
    return 0;
}

extern "C" int hb_qk_norm_rope_kv_write(void* q_out, const void* qkv, int dtype, const int32_t* positions,
                                        const float* table, int rotary_dim, int max_positions, const void* q_weight,
                                        const void* k_weight, int weight_dtype, float eps, float offset, void* kv,
                                        const int32_t* write_index, int pages, int page_size, int tokens, int heads,
                                        int kv_heads, int head_dim, hb_stream stream) {
    if (tokens == 0) return 0;
    if (head_dim > 2048) HB_REFUSE("qk_norm_rope_kv_write: head_dim %d is above 2048", head_dim);
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
        HB_REFUSE("qk_norm_rope_kv_write: rotary_dim %d must be even and at most head_dim %d", rotary_dim, head_dim);
    if (rotary_dim && !table) HB_REFUSE("qk_norm_rope_kv_write: a rotation needs its table");
    if ((q_weight == nullptr) != (k_weight == nullptr)) HB_REFUSE("qk_norm_rope_kv_write: give both norm weights or none");
    if (kv && !write_index) HB_REFUSE("qk_norm_rope_kv_write: writing the cache needs write_index");
    cudaStream_t s = (cudaStream_t)stream;
#define HB_ARGS q_out, qkv, positions, table, rotary_dim, max_positions, q_weight, k_weight, eps, offset, kv, \
    write_index, pages, page_size, tokens, heads, kv_heads, head_dim, s
    if (dtype == HB_F32 && weight_dtype == HB_F32) return launch<float, float>(HB_ARGS);
    if (dtype == HB_BF16 && weight_dtype == HB_BF16) return launch<bf16, bf16>(HB_ARGS);
    if (dtype == HB_BF16 && weight_dtype == HB_F32) return launch<bf16, float>(HB_ARGS);
#undef HB_ARGS
    HB_REFUSE("qk_norm_rope_kv_write: no kernel for dtype %d with weight dtype %d", dtype, weight_dtype);
}
