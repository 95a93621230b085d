// What the weight-streaming products share: 16-byte loads of weights (streamed past the L1) and of activations, and
// the bfloat16 tensor-core step m16n8k16 with 32-bit sums.
#pragma once
#include "common.cuh"

__device__ __forceinline__ uint4 ld_stream16(const void* p, bool valid) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (valid) asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                            : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_cached16(const void* p, bool valid) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (valid) v = __ldg((const uint4*)p);
    return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

