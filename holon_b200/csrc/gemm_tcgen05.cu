// bfloat16 GEMM on Blackwell's fifth-generation tensor cores: out[m, n] = sum_k x[m, k] * w[n, k].
//
// A CTA computes 128 x 256 tiles of the output, one after the other (one CTA per SM). Operands come in by TMA (cp.async.bulk.tensor, no multicast) as
// 64-wide k blocks into a ring of shared-memory stages in the 128-byte swizzled K-major layout; a single thread
// issues tcgen05.mma (kind::f16, M 128, N 256, K 16, four per stage) with the accumulator in tensor memory; four
// epilogue warps read it back with tcgen05.ld, 32 columns at a time, and write bfloat16 (or float32) rows.
// Warp roles: warp 0 producer (TMA), warp 1 MMA issue and TMEM allocation, warps 2-5 epilogue (warp w reads the
// TMEM lanes 32 (w mod 4) ..., which are the tile's rows).
// mode 1 is SwiGLU's first half: w is [2 inter, k] with gate rows first; the tile's first 128 accumulator columns
// come from gate rows n0.., the other 128 from up rows inter + n0.., and the epilogue writes silu(gate) * up.
//
// Every wait on an mbarrier is bounded: after HB_SPIN_LIMIT failed polls a thread records the place in the status
// word (hb_gemm_tcgen05_status reads and clears it), stops waiting, and the CTA still frees its tensor memory.
#include "tcgen05.cuh"

#define TC_BM 128
#define TC_BN 256
#define TC_BK 64
#define TC_STAGES 4
#define TC_A_BYTES (TC_BM * TC_BK * 2)
#define TC_B_BYTES (TC_BN * TC_BK * 2)
#define TC_STAGE_BYTES (TC_A_BYTES + TC_B_BYTES)
#define TC_SMEM (TC_STAGES * TC_STAGE_BYTES + 1024 + 256)
// Tile t of the launch: rows in bands of 16 tiles, inside a band the row index runs fastest, so that the CTAs that run
// side by side share few rows of x and few rows of w and both stay in L2.
struct TileAt { int m_tile, n_tile; };
__device__ __forceinline__ TileAt tile_at(int t, int tiles_m, int tiles_n) {
    constexpr int BAND = 16;
    const int per_band = BAND * tiles_n;
    const int band = t / per_band, within = t - band * per_band;
    const int rows = min(BAND, tiles_m - band * BAND);
    TileAt at;
    at.n_tile = within / rows;
    at.m_tile = band * BAND + within - at.n_tile * rows;
    return at;
}

// Persistent: each CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... Two accumulators of 256 columns alternate in
// tensor memory, so the epilogue of one tile runs while the tensor cores work on the next.
__global__ void __launch_bounds__(192, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                                                              const __grid_constant__ CUtensorMap map_w, void* __restrict__ out,
                                                              int out_f32, int m, int n, int k, int mode, int inter,
                                                              int tiles_m, int tiles_n) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;     // the swizzle pattern needs 1024-byte alignment
    const uint32_t bars = base + TC_STAGES * TC_STAGE_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * TC_STAGES;        // per stage: loaded / free again
    const uint32_t acc_full0 = bars + 16 * TC_STAGES, acc_empty0 = acc_full0 + 16;   // per accumulator: computed / read out
    const uint32_t slot = acc_empty0 + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (k + TC_BK - 1) / TC_BK;
    const int tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(2 * TC_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem) : "r"(slot));

    if (warp == 0) {
        if (lane == 0) {
            int kb_all = 0;                                           // k blocks loaded so far, over all tiles
            for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
                const TileAt at = tile_at(t, tiles_m, tiles_n);
                const int m0 = at.m_tile * TC_BM;
                const int w0 = mode == 1 ? at.n_tile * 128 : at.n_tile * TC_BN;
                const int w1 = mode == 1 ? inter + at.n_tile * 128 : w0 + 128;   // gate rows and the up rows of the same columns
                bool ok = true;
                for (int kb = 0; kb < kblocks && ok; ++kb, ++kb_all) {
                    const int s = kb_all % TC_STAGES;
                    ok = mbar_wait(empty0 + 8 * s, ((kb_all / TC_STAGES) & 1) ^ 1, 1);
                    if (!ok) break;
                    const uint32_t a = base + s * TC_STAGE_BYTES, b = a + TC_A_BYTES;
                    mbar_expect_tx(full0 + 8 * s, TC_STAGE_BYTES);
                    tma_load_2d(a, &map_x, full0 + 8 * s, kb * TC_BK, m0);
                    tma_load_2d(b, &map_w, full0 + 8 * s, kb * TC_BK, w0);
                    tma_load_2d(b + TC_B_BYTES / 2, &map_w, full0 + 8 * s, kb * TC_BK, w1);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // kind::f16: D float32 (bit 4), A and B bfloat16 (bits 7, 10), both K-major, N / 8 at bit 17, M / 16 at bit 24
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            int kb_all = 0, local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++local) {
                const int acc = local & 1, use = local >> 1;
                ok = mbar_wait(acc_empty0 + 8 * acc, (use & 1) ^ 1, 4);   // the epilogue has read this accumulator's last tile
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem + acc * TC_BN;
                for (int kb = 0; kb < kblocks; ++kb, ++kb_all) {
                    const int s = kb_all % TC_STAGES;
                    ok = mbar_wait(full0 + 8 * s, (kb_all / TC_STAGES) & 1, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a = base + s * TC_STAGE_BYTES, b = a + TC_A_BYTES;
                    const uint64_t da = tc_smem_desc(a), db = tc_smem_desc(b);
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; ++kk)          // 16 k values = 32 bytes further along each row
                        tc_mma(d, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb | kk) != 0);
                    tc_commit(empty0 + 8 * s);                        // the stage is free once these have read it
                }
                tc_commit(acc_full0 + 8 * acc);                       // arrives when every MMA above has finished
            }
        }
    } else {
        const int q = warp & 3;                                       // this warp's quarter of the TMEM lanes = tile rows
        const int width = mode == 1 ? inter : n;
        const int chunks = mode == 1 ? 4 : 8;
        int local = 0;
        for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++local) {
            const int acc = local & 1, use = local >> 1;
            const TileAt at = tile_at(t, tiles_m, tiles_n);
            const int row = at.m_tile * TC_BM + q * 32 + lane;
            const int col0 = mode == 1 ? at.n_tile * 128 : at.n_tile * TC_BN;
            if (!mbar_wait(acc_full0 + 8 * acc, use & 1, 3)) break;
            tc_fence_after();
            const uint32_t d = tmem + acc * TC_BN + ((uint32_t)(q * 32) << 16);
            for (int c = 0; c < chunks; ++c) {
                uint32_t r[32];
                tc_ld32(d + c * 32, r);
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                if (mode == 1) {
                    uint32_t u[32];
                    tc_ld32(d + 128 + c * 32, u);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = v[i] / (1.f + __expf(-v[i])) * __uint_as_float(u[i]);
                }
                if (c == chunks - 1) {                               // everything is in registers: hand the accumulator back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty0 + 8 * acc);
                }
                const int col = col0 + c * 32;
                if (row < m && col < width) {
                    if (out_f32) {
                        float* o = (float*)out + (size_t)row * width + col;
                        if (col + 32 <= width && (width & 3) == 0) {
#pragma unroll
                            for (int i = 0; i < 32; i += 4) *(float4*)(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                        } else {
                            for (int i = 0; i < 32 && col + i < width; ++i) o[i] = v[i];
                        }
                    } else {
                        bf16* o = (bf16*)out + (size_t)row * width + col;
                        if (col + 32 <= width && (width & 7) == 0) {
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                uint4 p;
                                __nv_bfloat162 a0 = __floats2bfloat162_rn(v[i], v[i + 1]), a1 = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
                                __nv_bfloat162 a2 = __floats2bfloat162_rn(v[i + 4], v[i + 5]), a3 = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
                                p.x = *(uint32_t*)&a0; p.y = *(uint32_t*)&a1; p.z = *(uint32_t*)&a2; p.w = *(uint32_t*)&a3;
                                *(uint4*)(o + i) = p;
                            }
                        } else {
                            for (int i = 0; i < 32 && col + i < width; ++i) o[i] = __float2bfloat16_rn(v[i]);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * TC_BN) : "memory");
    }
}

// ---------------------------------------------------------------- host side
static int encode_map(CUtensorMap* map, const void* ptr, int rows, int k, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                                              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) HB_REFUSE("gemm_tcgen05: cuTensorMapEncodeTiled failed with %d (rows %d, k %d)", (int)r, rows, k);
    return 0;
}

// Reads and clears the status word: 0, or (place << 28) | (block + 1) of the first wait that gave up
// (place 1 producer, 2 MMA, 3 epilogue). Synchronises the device.
HB_DEFINE_STATUS_MIRROR(hb_gemm_tcgen05_status_mirror)
extern "C" int hb_gemm_tcgen05_status(unsigned int* status) {
    HB_CUDA(cudaDeviceSynchronize());
    HB_CUDA(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(unsigned int)));
    const unsigned int zero = 0;
    HB_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(unsigned int)));
    return 0;
}

// mode 0: out [m, n] (bfloat16, or float32 when out_f32) = x [m, k] · w [n, k]ᵀ.
// mode 1: w is [2 inter, k], gate rows first; out [m, inter] = silu(x · gateᵀ) · (x · upᵀ).
// k a multiple of 8 (a row's bytes a multiple of 16); x, w 16-byte aligned.
extern "C" int hb_gemm_bf16_tcgen05(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode,
                                    int inter, hb_stream stream) {
    if (m == 0 || n == 0) return 0;
    if (k < 8 || k % 8) HB_REFUSE("gemm_tcgen05: k = %d is no multiple of 8", k);
    if ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) % 16) != 0) HB_REFUSE("gemm_tcgen05: pointers must be 16-byte aligned");
    if (mode != 0 && mode != 1) HB_REFUSE("gemm_tcgen05: mode %d", mode);
    if (mode == 1 && (inter < 1 || n != 2 * inter)) HB_REFUSE("gemm_tcgen05: mode 1 needs n = 2 inter (n %d, inter %d)", n, inter);
    CUtensorMap map_x, map_w;
    int rc = encode_map(&map_x, x, m, k, TC_BM);
    if (rc) return rc;
    rc = encode_map(&map_w, w, n, k, 128);
    if (rc) return rc;
    HB_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
    const int tiles_m = (m + TC_BM - 1) / TC_BM;
    const int tiles_n = mode == 1 ? (inter + 127) / 128 : (n + TC_BN - 1) / TC_BN;
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        HB_CUDA(cudaGetDevice(&device));
        HB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    }
    const long tiles = (long)tiles_m * tiles_n;
    const int grid = (int)(tiles < sms ? tiles : sms);
    gemm_tcgen05_kernel<<<grid, 192, TC_SMEM, (cudaStream_t)stream>>>(map_x, map_w, out, out_f32, m, n, k, mode, inter,
                                                                      tiles_m, tiles_n);
    HB_LAUNCH_CHECK("gemm_tcgen05");
    return 0;
}
