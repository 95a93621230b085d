// out[m, n] = sum_k x[m, k] * w[n, k] for a few rows m (decode steps): bfloat16 operands, 32-bit sums.
//
// With at most 16 rows of x the product is bound by reading w once from HBM, so the kernel is built around that
// stream. The weight's rows are the M side of mma.sync m16n8k16 (16 rows of w per tile) and the few rows of x its
// 8-wide N side. Every lane reads w with 16-byte loads straight into A fragments: the 8 consecutive k values a lane
// loads from a row are used as two k-pairs of two consecutive mma steps, and x is loaded with the same permutation of
// k, so no shared-memory staging is needed. The 8 warps of a CTA take interleaved 32-wide k blocks of the same 16 or
// 32 rows and add their partial sums through shared memory in a fixed order.
// mode 1 computes SwiGLU's activation in the epilogue: the CTA's first tile holds 16 gate rows, its second the 16 up
// rows of the same columns, and it writes silu(gate) * up.
#include "common.cuh"

#define SK_WARPS 8

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

// MT tiles of 16 weight rows per CTA, NT tiles of 8 rows of x.
template <int MT, int NT, int SK_UNROLL, int MIN_CTAS>
__global__ void __launch_bounds__(SK_WARPS * 32, MIN_CTAS) gemm_skinny_kernel(void* __restrict__ out, int out_f32,
                                                                    const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                    int m, int n, int k, int mode, int inter) {
    __shared__ float red[SK_WARPS][MT * 16][NT * 8 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = lane >> 2, c = lane & 3;
    int row0[MT];                                        // first weight row of each tile
    int limit[MT];                                       // rows below this exist
    constexpr int HALF = MT > 1 ? MT / 2 : 1;           // mode 1: the CTA's gate tiles, then as many up tiles
    if (mode == 1) {
#pragma unroll
        for (int t = 0; t < HALF; ++t) {
            row0[t] = (blockIdx.x * HALF + t) * 16; limit[t] = inter;
            if (MT > 1) { row0[HALF + t] = inter + row0[t]; limit[HALF + t] = 2 * inter; }
        }
    } else {
#pragma unroll
        for (int t = 0; t < MT; ++t) { row0[t] = (blockIdx.x * MT + t) * 16; limit[t] = n; }
    }
    const bf16* wp[MT][2];
    bool wok[MT][2];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = row0[t] + r + 8 * h;
            wok[t][h] = row < limit[t];
            wp[t][h] = w + (size_t)(wok[t][h] ? row : 0) * k + c * 8;
        }
    const bf16* xp[NT];
    bool xok[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int row = t * 8 + r;
        xok[t] = row < m;
        xp[t] = x + (size_t)(xok[t] ? row : 0) * k + c * 8;
    }
    float acc[MT][NT][4];
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
        for (int b = 0; b < NT; ++b) acc[a][b][0] = acc[a][b][1] = acc[a][b][2] = acc[a][b][3] = 0.f;

    const int blocks = (k + 31) >> 5;                    // 32-wide k blocks; warp w takes w, w + 8, ...
    for (int kb = warp; kb < blocks; kb += SK_WARPS * SK_UNROLL) {
        uint4 wr[SK_UNROLL][MT][2], xr[SK_UNROLL][NT];
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u) {
            const int k0 = (kb + u * SK_WARPS) << 5;
            const bool kok = k0 + c * 8 < k;             // k is a multiple of 8: a 16-byte piece is whole or absent
#pragma unroll
            for (int t = 0; t < MT; ++t)
#pragma unroll
                for (int h = 0; h < 2; ++h) wr[u][t][h] = ld_stream16(wp[t][h] + k0, kok && wok[t][h]);
#pragma unroll
            for (int t = 0; t < NT; ++t) xr[u][t] = ld_cached16(xp[t] + k0, kok && xok[t]);
        }
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u)
#pragma unroll
            for (int a = 0; a < MT; ++a)
#pragma unroll
                for (int b = 0; b < NT; ++b) {
                    mma16816(acc[a][b], wr[u][a][0].x, wr[u][a][1].x, wr[u][a][0].y, wr[u][a][1].y, xr[u][b].x, xr[u][b].y);
                    mma16816(acc[a][b], wr[u][a][0].z, wr[u][a][1].z, wr[u][a][0].w, wr[u][a][1].w, xr[u][b].z, xr[u][b].w);
                }
    }
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
        for (int b = 0; b < NT; ++b) {
            red[warp][a * 16 + r][b * 8 + c * 2] = acc[a][b][0];
            red[warp][a * 16 + r][b * 8 + c * 2 + 1] = acc[a][b][1];
            red[warp][a * 16 + r + 8][b * 8 + c * 2] = acc[a][b][2];
            red[warp][a * 16 + r + 8][b * 8 + c * 2 + 1] = acc[a][b][3];
        }
    __syncthreads();
    const int rows_out = mode == 1 ? HALF * 16 : MT * 16;
    const int width = mode == 1 ? inter : n;
    for (int i = threadIdx.x; i < rows_out * m; i += SK_WARPS * 32) {
        const int rr = i % rows_out, tok = i / rows_out;
        float v = 0.f;
#pragma unroll
        for (int wv = 0; wv < SK_WARPS; ++wv) v += red[wv][rr][tok];
        int col = row0[0] + rr;
        if (MT > 1 && rr >= 16) col = row0[rr >> 4] + (rr & 15);
        if (mode == 1) {
            float u = 0.f;
#pragma unroll
            for (int wv = 0; wv < SK_WARPS; ++wv) u += red[wv][HALF * 16 + rr][tok];
            v = v / (1.f + expf(-v)) * u;
        }
        if (col < width) {
            if (out_f32) ((float*)out)[(size_t)tok * width + col] = v;
            else ((bf16*)out)[(size_t)tok * width + col] = __float2bfloat16_rn(v);
        }
    }
}

// mode 0: out [m, n] (bfloat16, or float32 when out_f32) = x [m, k] · w [n, k]ᵀ.
// mode 1: w is [2 * inter, k] with gate rows first; out [m, inter] = silu(x · gateᵀ) * (x · upᵀ); n is ignored.
// m at most 16, k a multiple of 8, all pointers 16-byte aligned.
extern "C" int hb_gemm_bf16_skinny(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode,
                                   int inter, hb_stream stream) {
    if (m == 0) return 0;
    if (m < 0 || m > 16) HB_REFUSE("gemm_bf16_skinny: %d rows; this kernel takes 1 to 16", m);
    if (k < 8 || k % 8) HB_REFUSE("gemm_bf16_skinny: k = %d is no multiple of 8", k);
    if ((((uintptr_t)out | (uintptr_t)x | (uintptr_t)w) % 16) != 0) HB_REFUSE("gemm_bf16_skinny: pointers must be 16-byte aligned");
    if (mode != 0 && mode != 1) HB_REFUSE("gemm_bf16_skinny: mode %d", mode);
    cudaStream_t s = (cudaStream_t)stream;
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        HB_CUDA(cudaGetDevice(&device));
        HB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    }
    const int nt = m <= 8 ? 1 : 2;
    if (mode == 1) {
        if (inter < 1) HB_REFUSE("gemm_bf16_skinny: inter = %d", inter);
        const int grid = (inter + 15) / 16;
        if (nt == 1) gemm_skinny_kernel<2, 1, 4, 2><<<grid, SK_WARPS * 32, 0, s>>>(out, out_f32, (const bf16*)x, (const bf16*)w, m, n, k, 1, inter);
        else gemm_skinny_kernel<2, 2, 4, 2><<<grid, SK_WARPS * 32, 0, s>>>(out, out_f32, (const bf16*)x, (const bf16*)w, m, n, k, 1, inter);
    } else {
        if (n < 1) HB_REFUSE("gemm_bf16_skinny: n = %d", n);
        const bool wide = n >= 32 * 2 * sms;             // enough rows to give every SM two CTAs of 32 rows
        const int grid = wide ? (n + 31) / 32 : (n + 15) / 16;
        if (wide && nt == 1) gemm_skinny_kernel<2, 1, 4, 2><<<grid, SK_WARPS * 32, 0, s>>>(out, out_f32, (const bf16*)x, (const bf16*)w, m, n, k, 0, 0);
        else if (wide) gemm_skinny_kernel<2, 2, 4, 2><<<grid, SK_WARPS * 32, 0, s>>>(out, out_f32, (const bf16*)x, (const bf16*)w, m, n, k, 0, 0);
        else if (nt == 1 && grid > 2 * sms && grid <= 3 * sms)       // one wave of three CTAs per SM instead of one and a bit of two
            gemm_skinny_kernel<1, 1, 4, 3><<<grid, SK_WARPS * 32, 0, s>>>(out, out_f32, (const bf16*)x, (const bf16*)w, m, n, k, 0, 0);
        else if (nt == 1) gemm_skinny_kernel<1, 1, 8, 2><<<grid, SK_WARPS * 32, 0, s>>>(out, out_f32, (const bf16*)x, (const bf16*)w, m, n, k, 0, 0);
        else gemm_skinny_kernel<1, 2, 8, 2><<<grid, SK_WARPS * 32, 0, s>>>(out, out_f32, (const bf16*)x, (const bf16*)w, m, n, k, 0, 0);
    }
    HB_LAUNCH_CHECK("gemm_bf16_skinny");
    return 0;
}
