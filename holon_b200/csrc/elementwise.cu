// Embedding gather, RMSNorm with the residual sum folded in, SwiGLU's activation.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[512] = "";
void hb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}
extern "C" const char* hb_last_error(void) { return g_error; }
extern "C" int hb_version(void) { return 1; }

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table, const int32_t* __restrict__ ids,
                             int hidden, int vocab) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* row = table + (size_t)(ok ? id : 0) * hidden;
    float* o = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = ok ? to_f32(row[i]) : 0.f;
}
// The same for a bfloat16 table whose rows are a multiple of 8 wide: 16 bytes a load, all of a thread's loads in flight
// before the first is used (a row of 4,096 is two loads a thread instead of sixteen in a row).
__global__ void embed_bf16x8_kernel(float* __restrict__ out, const bf16* __restrict__ table, const int32_t* __restrict__ ids,
                                    int hidden, int vocab) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const uint4* row = (const uint4*)(table + (size_t)(ok ? id : 0) * hidden);
    float4* o = (float4*)(out + (size_t)t * hidden);
    const int pieces = hidden >> 3;
    for (int i0 = threadIdx.x; i0 < pieces; i0 += 4 * blockDim.x) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * blockDim.x;
            v[u] = ok && i < pieces ? __ldg(row + i) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * blockDim.x;
            if (i < pieces) {
                const __nv_bfloat162* h = (const __nv_bfloat162*)&v[u];
                const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]), c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
                o[2 * i] = make_float4(a.x, a.y, b.x, b.y);
                o[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
            }
        }
    }
}

extern "C" int hb_embed(float* out, const void* table, int table_dtype, const int32_t* ids, int tokens, int hidden,
                        int vocab, hb_stream stream) {
    if (tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == HB_F32) embed_kernel<float><<<tokens, threads, 0, s>>>(out, (const float*)table, ids, hidden, vocab);
    else if (table_dtype == HB_BF16 && hidden % 8 == 0 && (((uintptr_t)table | (uintptr_t)out) % 16) == 0)
        embed_bf16x8_kernel<<<tokens, threads, 0, s>>>(out, (const bf16*)table, ids, hidden, vocab);
    else if (table_dtype == HB_BF16) embed_kernel<bf16><<<tokens, threads, 0, s>>>(out, (const bf16*)table, ids, hidden, vocab);
    else HB_REFUSE("embed: table dtype %d", table_dtype);
    HB_LAUNCH_CHECK("embed");
    return 0;
}

// ---------------------------------------------------------------- (add +) RMSNorm
// One block per output row. The row is kept in shared memory as 32-bit between the two passes.
// VEC: dim is a multiple of 4 and every pointer is 16-byte aligned per row, so a thread moves 4 values at a time.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) { const float4 x = *(const float4*)p; v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *(float4*)p = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
        const uint2 x = *(const uint2*)p;
        const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&x.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&x.y);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[4]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 x; x.x = *(uint32_t*)&a; x.y = *(uint32_t*)&b;
        *(uint2*)p = x;
    }
};

template <typename TH, typename TD, typename TW, bool VEC>
__global__ void add_rmsnorm_kernel(TD* __restrict__ out, TH* h, const TD* __restrict__ delta,
                                   const TW* __restrict__ weight, float eps, float offset,
                                   const int32_t* __restrict__ index, int dim) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t t = index ? (size_t)index[r] : (size_t)r;
    TH* hr = h + t * dim;
    const TD* dr = delta ? delta + t * dim : nullptr;
    const bool write_back = delta != nullptr && index == nullptr;
    float ss = 0.f;
    if (VEC && dim <= (int)blockDim.x * 4) {
        // A thread holds its (at most) four values in registers and reads the weight before the block-wide sum, so
        // that load's latency passes while the sum is formed; the values and their order are those of the loops below.
        const int i = threadIdx.x * 4;
        float v[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
        if (i < dim) {
            float d[4];
            Vec4<TH>::load(hr + i, v);
            if (dr) {
                Vec4<TD>::load(dr + i, d);
#pragma unroll
                for (int k = 0; k < 4; ++k) v[k] += d[k];
            }
            Vec4<TW>::load(weight + i, w);
            if (write_back) Vec4<TH>::store(hr + i, v);
            ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        }
        const float rstd = rsqrtf(block_sum(ss, scratch) / (float)dim + eps);
        if (i < dim) {
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = v[k] * rstd * (w[k] + offset);
            Vec4<TD>::store(out + (size_t)r * dim + i, v);
        }
        return;
    }
    if (VEC) {
        for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
            float v[4], d[4];
            Vec4<TH>::load(hr + i, v);
            if (dr) {
                Vec4<TD>::load(dr + i, d);
#pragma unroll
                for (int k = 0; k < 4; ++k) v[k] += d[k];
            }
            if (write_back) Vec4<TH>::store(hr + i, v);
            *(float4*)(row + i) = make_float4(v[0], v[1], v[2], v[3]);
            ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            float v = to_f32(hr[i]);
            if (dr) v += to_f32(dr[i]);
            if (write_back) hr[i] = from_f32<TH>(v);
            row[i] = v;
            ss += v * v;
        }
    }
    const float total = block_sum(ss, scratch);
    const float rstd = rsqrtf(total / (float)dim + eps);
    TD* o = out + (size_t)r * dim;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
            float w[4], v[4];
            Vec4<TW>::load(weight + i, w);
            const float4 x = *(const float4*)(row + i);
            v[0] = x.x * rstd * (w[0] + offset); v[1] = x.y * rstd * (w[1] + offset);
            v[2] = x.z * rstd * (w[2] + offset); v[3] = x.w * rstd * (w[3] + offset);
            Vec4<TD>::store(o + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x)
            o[i] = from_f32<TD>(row[i] * rstd * (to_f32(weight[i]) + offset));
    }
}

template <typename TH, typename TD, typename TW>
static int launch_add_rmsnorm(void* out, void* h, const void* delta, const void* weight, float eps, float offset,
                              const int32_t* index, int rows, int dim, cudaStream_t s) {
    const size_t smem = (size_t)dim * sizeof(float);
    if (smem > 200 * 1024) HB_REFUSE("rmsnorm: a row of %d values does not fit shared memory (limit 51200)", dim);
    const bool vec = dim % 4 == 0 && (((uintptr_t)out | (uintptr_t)h | (uintptr_t)delta | (uintptr_t)weight) % 16 == 0);
    auto kernel = vec ? add_rmsnorm_kernel<TH, TD, TW, true> : add_rmsnorm_kernel<TH, TD, TW, false>;
    if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int per = vec ? 4 : 1;
    int threads = dim >= 4096 * per ? 1024 : (dim >= 1024 * per ? 512 : (dim >= 256 * per ? 256 : 128));
    if (vec && dim <= 4096 && rows <= 256) threads = (dim / 4 + 31) / 32 * 32;   // few rows (latency counts): a row in one pass, four values a thread in registers
    kernel<<<rows, threads, smem, s>>>((TD*)out, (TH*)h, (const TD*)delta, (const TW*)weight, eps, offset, index, dim);
    HB_LAUNCH_CHECK("add_rmsnorm");
    return 0;
}

extern "C" int hb_add_rmsnorm(void* out, int out_dtype, void* h, int h_dtype, const void* delta, const void* weight,
                              int weight_dtype, float eps, float offset, const int32_t* index, int rows, int dim,
                              hb_stream stream) {
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (h_dtype != HB_F32 && delta) HB_REFUSE("add_rmsnorm: the residual stream must be float32 when a delta is added");
#define HB_CASE(H, D, W, TH, TD, TW) if (h_dtype == H && out_dtype == D && weight_dtype == W) \
    return launch_add_rmsnorm<TH, TD, TW>(out, h, delta, weight, eps, offset, index, rows, dim, s);
    HB_CASE(HB_F32, HB_F32, HB_F32, float, float, float)
    HB_CASE(HB_F32, HB_BF16, HB_BF16, float, bf16, bf16)
    HB_CASE(HB_F32, HB_BF16, HB_F32, float, bf16, float)
    HB_CASE(HB_BF16, HB_BF16, HB_BF16, bf16, bf16, bf16)
    HB_CASE(HB_BF16, HB_BF16, HB_F32, bf16, bf16, float)
#undef HB_CASE
    HB_REFUSE("add_rmsnorm: no kernel for dtypes h=%d out=%d weight=%d", h_dtype, out_dtype, weight_dtype);
}

// ---------------------------------------------------------------- silu(gate) * up
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter, c = i % inter;
        const float g = to_f32(gate_up[t * 2 * inter + c]), u = to_f32(gate_up[t * 2 * inter + inter + c]);
        out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
    }
}

// bfloat16 with inter a multiple of 8: a thread takes 8 gates and 8 ups as two 16-byte loads.
__global__ void silu_mul_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ gate_up, int inter, size_t groups) {
    const int per_row = inter >> 3;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / per_row, c = (i % per_row) << 3;
        const uint4 g4 = *(const uint4*)(gate_up + t * 2 * inter + c), u4 = *(const uint4*)(gate_up + t * 2 * inter + inter + c);
        const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 g = __bfloat1622float2(*(const __nv_bfloat162*)&gw[k]), u = __bfloat1622float2(*(const __nv_bfloat162*)&uw[k]);
            __nv_bfloat162 r = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y);
            ow[k] = *(uint32_t*)&r;
        }
        *(uint4*)(out + t * inter + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

extern "C" int hb_silu_mul(void* out, const void* gate_up, int dtype, int tokens, int inter, hb_stream stream) {
    const size_t total = (size_t)tokens * inter;
    if (total == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    if (dtype == HB_BF16 && inter % 8 == 0 && (((uintptr_t)out | (uintptr_t)gate_up) % 16 == 0)) {
        const size_t groups = total / 8;
        const int blocks = (int)((groups + threads - 1) / threads < 148 * 32 ? (groups + threads - 1) / threads : 148 * 32);
        silu_mul_bf16x8_kernel<<<blocks, threads, 0, s>>>((bf16*)out, (const bf16*)gate_up, inter, groups);
        HB_LAUNCH_CHECK("silu_mul");
        return 0;
    }
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == HB_F32) silu_mul_kernel<float><<<blocks, threads, 0, s>>>((float*)out, (const float*)gate_up, inter, total);
    else if (dtype == HB_BF16) silu_mul_kernel<bf16><<<blocks, threads, 0, s>>>((bf16*)out, (const bf16*)gate_up, inter, total);
    else HB_REFUSE("silu_mul: dtype %d", dtype);
    HB_LAUNCH_CHECK("silu_mul");
    return 0;
}
