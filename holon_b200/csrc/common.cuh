// Shared helpers of the kernels: storage types, conversions, warp and block reductions, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }
// The value after one rounding to the storage type, as 32-bit.
template <typename T> __device__ __forceinline__ float rounded(float x) { return to_f32(from_f32<T>(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                       // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = lane < warps ? scratch[lane] : 0.f;
        w = warp_sum(w);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = lane < warps ? scratch[lane] : -INFINITY;
        w = warp_max(w);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}

// Host side: remembers why a call was refused; hb_last_error() hands the text out.
void hb_set_error(const char* fmt, ...);
#define HB_REFUSE(...) do { hb_set_error(__VA_ARGS__); return HB_ERR_REFUSED; } while (0)
#define HB_LAUNCH_CHECK(name) do { cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) { \
    hb_set_error("%s: %s", name, cudaGetErrorString(e_)); return HB_ERR_CUDA; } } while (0)
#define HB_CUDA(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { \
    hb_set_error("%s: %s", #call, cudaGetErrorString(e_)); return HB_ERR_CUDA; } } while (0)
