// out[m, n] = sum_k x[m, k] * w[n, k] in true 32-bit on CUDA cores: no tensor cores, no reduced-precision mode.
// Every output element is summed over k in ascending order by one thread, whatever m and n are, so a row's result
// does not depend on how many other rows the batch holds. 64 x 64 tiles, 16 deep, 4 x 4 outputs per thread.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <bool VEC>
__global__ void __launch_bounds__(256) gemm_f32_kernel(float* __restrict__ out, const float* __restrict__ x,
                                                       const float* __restrict__ w, int m, int n, int k) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lr = tid >> 2, lk = (tid & 3) * 4;           // this thread loads 4 k-values of tile row lr
    const int ty = tid >> 4, tx = tid & 15;                 // and computes rows ty*4.., columns tx*4..
    float acc[4][4] = {};
    const int xr = m0 + lr, wr = n0 + lr;
    for (int k0 = 0; k0 < k; k0 += BK) {
        float xv[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
        const int kk = k0 + lk;
        if (VEC) {
            if (xr < m && kk < k) *(float4*)xv = *(const float4*)(x + (size_t)xr * k + kk);
            if (wr < n && kk < k) *(float4*)wv = *(const float4*)(w + (size_t)wr * k + kk);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (xr < m && kk + i < k) xv[i] = x[(size_t)xr * k + kk + i];
                if (wr < n && kk + i < k) wv[i] = w[(size_t)wr * k + kk + i];
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            xs[lk + i][lr] = xv[i];
            ws[lk + i][lr] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk2 = 0; kk2 < BK; ++kk2) {
            const float4 a = *(const float4*)&xs[kk2][ty * 4];
            const float4 b = *(const float4*)&ws[kk2][tx * 4];
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = m0 + ty * 4 + i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx * 4 + j;
            if (c < n) out[(size_t)r * n + c] = acc[i][j];
        }
    }
}

extern "C" int hb_gemm_f32(float* out, const float* x, const float* w, int m, int n, int k, hb_stream stream) {
    if (m == 0 || n == 0) return 0;
    if (k <= 0) HB_REFUSE("gemm_f32: k = %d", k);
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
    if (grid.y > 65535) HB_REFUSE("gemm_f32: %d rows are above the kernel's limit of %d", m, 65535 * BM);
    const bool vec = (k % 4 == 0) && (((uintptr_t)x | (uintptr_t)w) % 16 == 0);
    if (vec) gemm_f32_kernel<true><<<grid, 256, 0, s>>>(out, x, w, m, n, k);
    else gemm_f32_kernel<false><<<grid, 256, 0, s>>>(out, x, w, m, n, k);
    HB_LAUNCH_CHECK("gemm_f32");
    return 0;
}
