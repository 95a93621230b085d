// bfloat16 products of up to 64 rows (decode steps): out[m, n] = sum_k x[m, k] * w[n, k], bound by reading w once, with
// the work that follows the product in its epilogue, as in the mma.sync kernel for up to 16 rows. The kernel table sends
// SwiGLU's product here at every number of rows, the attention's first from 9 rows on, and from 17 rows on whatever
// HOLON_B200_MID says.
//
// The weight is the N side of tcgen05.mma: a tile is 256 rows of w (8 KB of weights an MMA of 16 k values, so the one
// issuing thread keeps up with the memory) against the rows of x on the M side (a box of 64 rows; the MMA's other 64
// rows read whatever follows in shared memory and land in tensor-memory lanes that nobody reads). n / 256 tiles are
// too few CTAs to pull the weight at HBM's pace, so a tile's k range is split over the CTAs of a thread-block
// cluster (up to 8): each streams its k blocks by TMA through a ring of five 40 KB stages into one accumulator,
// writes its partial sums to its own shared memory, and after a cluster barrier every CTA sums, in the fixed order of
// the ranks, its share of the tile's rows from all the CTAs' shared memory (distributed shared memory: no scratch in
// global memory, no second kernel, no atomics, the same bits whatever the timing). A CTA then holds whole rows of the
// tile, 256 columns each, which is what the epilogues want:
//   mode 0  out [m, n] (bfloat16 or float32)
//   mode 1  SwiGLU: the tile is 128 gate rows and the 128 up rows of the same columns; out [m, inter] = silu(g) u
//   mode 2  the attention's first product: per token and head (head_dim 32, 64 or 128: whole heads in a tile) the
//           RMSNorm of q and k, the rotation of half-split pairs and the write of k and v into the paged cache
//   mode 3  the product that ends a mixer or a feed-forward: h += bfloat16(product), out = bfloat16(h (w_next + o)),
//           ss_out [tiles, 64] = per tile and token the sum of squares of the tile's columns of the new h
// and in every mode ss_in: x lacks its norm's row scale (mode 3 of the product before left it out); the sums are
// scaled by rsqrt(sum over parts of ss_in / dim_in + eps_in) per token.
//
// Every wait on an mbarrier is bounded (tcgen05.cuh); a CTA whose wait gave up still walks through both cluster
// barriers and frees its tensor memory, so the others never wait for it.
#include "tcgen05.cuh"

#define MD_ROWS 64
#define MD_BN 256
#define MD_BK 64
#define MD_STAGES 5
#define MD_A_BYTES (MD_ROWS * MD_BK * 2)
#define MD_B_BYTES (MD_BN * MD_BK * 2)
#define MD_STAGE_BYTES (MD_A_BYTES + MD_B_BYTES)
#define MD_TAIL 384                                   // barriers, the tensor-memory slot, 64 row scales
#define MD_SMEM (MD_STAGES * MD_STAGE_BYTES + 1024 + MD_TAIL)
#define MD_PP 260                                     // floats a row of partial sums and of results: 16-byte pieces of rows that
                                                      // are 8 lanes apart fall into different banks
#define MD_THREADS 512

struct MidArgs {
    void* out; int out_f32, mode, inter;
    const float* ss_in; int parts_in, dim_in, stride_in; float eps_in;
    float* h; const void* next_weight; int next_weight_f32; float next_offset; float* ss_out;
    bf16* q_out; const int32_t* positions; const float* table; int max_positions;
    const void* q_weight; const void* k_weight; int weight_f32; float eps, offset;
    bf16* kv; const int32_t* write_index; int pages, page_size, heads, kv_heads, head_dim;
};

__device__ __forceinline__ float4 md_ld_peer4(const float* local, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_addr(local)), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ uint2 md_pack4(float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 p;
    p.x = *(uint32_t*)&lo; p.y = *(uint32_t*)&hi;
    return p;
}
__device__ __forceinline__ float md_weight(const void* w, int f32, int i) {
    return f32 ? ((const float*)w)[i] : to_f32(((const bf16*)w)[i]);
}

__global__ void __launch_bounds__(MD_THREADS, 1) gemm_mid_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                 const __grid_constant__ CUtensorMap map_w, int m, int n, int k,
                                                                 int csize, const __grid_constant__ MidArgs e) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;     // the swizzle pattern needs 1024-byte alignment
    unsigned char* base_ptr = smem_raw + (base - smem_addr(smem_raw));
    const uint32_t bars = base + MD_STAGES * MD_STAGE_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * MD_STAGES, acc_full = bars + 16 * MD_STAGES, slot = acc_full + 8;
    float* scale = (float*)(base_ptr + MD_STAGES * MD_STAGE_BYTES + 128);
    float* partial = (float*)base_ptr;                                // after the main loop, over the ring
    float* res = (float*)(base_ptr + MD_ROWS * MD_PP * 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
    const int tile = blockIdx.x / csize;
    const int kblocks = (k + MD_BK - 1) / MD_BK, per = (kblocks + csize - 1) / csize;
    const int kb0 = min(kblocks, (int)rank * per), kb1 = min(kblocks, kb0 + per), mine = kb1 - kb0;
    const int mode = e.mode;
    const int w0 = mode == 1 ? tile * 128 : tile * MD_BN;
    const int w1 = mode == 1 ? e.inter + tile * 128 : w0 + 128;      // gate rows and the up rows of the same columns

    // The producer thread makes the barriers itself and asks for its first stages at once: the weight is on its way
    // while the rest of the CTA sets up (tensor memory, the barrier below).
    const int share = (m + csize - 1) / csize;                        // this CTA's rows of the tile after the sum over the cluster
    const int r0 = min(m, (int)rank * share), r1 = min(m, r0 + share), rows = r1 - r0;
    auto load_stage = [&](int i) {
        const int s = i % MD_STAGES, kb = kb0 + i;
        const uint32_t a = base + s * MD_STAGE_BYTES, b = a + MD_A_BYTES;
        mbar_expect_tx(full0 + 8 * s, MD_STAGE_BYTES);
        tma_load_2d(a, &map_x, full0 + 8 * s, kb * MD_BK, 0);
        tma_load_2d(b, &map_w, full0 + 8 * s, kb * MD_BK, w0);
        tma_load_2d(b + MD_B_BYTES / 2, &map_w, full0 + 8 * s, kb * MD_BK, w1);
    };
    if (warp == 2 && lane == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_x) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_w) : "memory");
        for (int s = 0; s < MD_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        for (int i = 0; i < min(mine, MD_STAGES); ++i) load_stage(i);
    }
    if (warp == 3) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(MD_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem) : "r"(slot));

    // The scales of the rows of x, by the fourteen warps that neither load nor issue, while those two work: a warp a
    // row, a lane every 32nd part, summed over the warp in a fixed order. (One lane a row, all parts in turn, before the
    // barrier above held the first MMA back by the whole walk: 8 us at 16 rows and 256 parts.)
    if (warp != 2 && warp != 3) {
        if (e.ss_in != nullptr) {
            for (int row = warp < 2 ? warp : warp - 2; row < m; row += MD_THREADS / 32 - 2) {
                float ss = 0.f;
                for (int p = lane; p < e.parts_in; p += 32) ss += e.ss_in[p * e.stride_in + row];
                ss = warp_sum(ss);
                if (lane == 0) scale[row] = rsqrtf(ss / (float)e.dim_in + e.eps_in);
            }
        } else if (threadIdx.x < MD_ROWS) {
            scale[threadIdx.x] = 1.f;
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(MD_THREADS - 64) : "memory");    // (the fourteen warps: the scales are there)
    }

    // ---- the main loop: this CTA's k blocks of the tile
    if (warp == 2) {
        if (lane == 0) {
            for (int i = MD_STAGES; i < mine; ++i) {                  // (the first stages are on their way)
                if (!mbar_wait(empty0 + 8 * (i % MD_STAGES), ((i / MD_STAGES) & 1) ^ 1, 1)) break;
                load_stage(i);
            }
        }
    } else if (warp == 3) {
        if (lane == 0 && mine > 0) {
            // kind::f16: D float32 (bit 4), A and B bfloat16 (bits 7, 10), both K-major, N / 8 at bit 17, M / 16 at bit 24
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MD_BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            for (int i = 0; i < mine; ++i) {
                const int s = i % MD_STAGES;
                if (!mbar_wait(full0 + 8 * s, (i / MD_STAGES) & 1, 2)) break;
                tc_fence_after();
                const uint32_t a = base + s * MD_STAGE_BYTES, b = a + MD_A_BYTES;
                const uint64_t da = tc_smem_desc(a), db = tc_smem_desc(b);
#pragma unroll
                for (int kk = 0; kk < MD_BK / 16; ++kk)
                    tc_mma(tmem, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (i | kk) != 0);
                tc_commit(empty0 + 8 * s);
            }
            tc_commit(acc_full);                                      // arrives when every MMA above has finished
        }
    }
    // The warps whose quarter of the tensor-memory lanes holds rows of x (lanes 0 to 63): 0, 1, 4, 5, 8, 9, 12, 13. Each
    // reads two blocks of 32 columns of its 32 rows into partial[row][column] (one CTA a tile: scaled, straight into res).
    if ((warp & 3) < 2) {
        const int q = warp & 3, hf = warp >> 2, row = q * 32 + lane;
        bool ok = true;
        if (mine > 0) {
            ok = mbar_wait(acc_full, 0, 3);
            tc_fence_after();
        }
        float* to = csize == 1 ? res : partial;
        const float sc = csize == 1 && row < m ? scale[row] : 1.f;
        for (int c = hf * 2; c < hf * 2 + 2; ++c) {
            uint32_t r[32];
            if (mine > 0 && ok) {
                tc_ld32(tmem + ((uint32_t)(q * 32) << 16) + c * 32, r);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 32; i += 4)
                *(float4*)(to + row * MD_PP + c * 32 + i) = make_float4(__uint_as_float(r[i]) * sc, __uint_as_float(r[i + 1]) * sc,
                                                                         __uint_as_float(r[i + 2]) * sc, __uint_as_float(r[i + 3]) * sc);
        }
    }
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    if (csize > 1) {                                                            // (uniform over the cluster)
        asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");  // every CTA's partial sums are in its shared memory
    }
    for (int f = threadIdx.x; csize > 1 && f < rows * (MD_BN / 4); f += MD_THREADS) {      // four columns a thread
        const int rl = f >> 6, c4 = (f & 63) * 4;
        const float* p = partial + (r0 + rl) * MD_PP + c4;
        float4 part[8];
#pragma unroll
        for (int r2 = 0; r2 < 8; ++r2)                                         // all asked for, then summed in the order of the ranks
            part[r2] = r2 < csize ? md_ld_peer4(p, (uint32_t)r2) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 v = part[0];
#pragma unroll
        for (int r2 = 1; r2 < 8; ++r2)
            if (r2 < csize) { v.x += part[r2].x; v.y += part[r2].y; v.z += part[r2].z; v.w += part[r2].w; }
        const float sc = scale[r0 + rl];
        *(float4*)(res + rl * MD_PP + c4) = make_float4(v.x * sc, v.y * sc, v.z * sc, v.w * sc);
    }
    __syncwarp();
    if (csize > 1) asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");   // this CTA reads no other's shared memory any more
    __syncthreads();

    // ---- the epilogues: rows r0 .. r1 of the tile, 256 columns each, in res
    if (mode == 0) {
        const bool whole = (n & 3) == 0;
        for (int f = threadIdx.x; f < rows * (MD_BN / 4); f += MD_THREADS) {
            const int rl = f >> 6, c4 = (f & 63) * 4, gcol = tile * MD_BN + c4;
            if (gcol >= n) continue;
            const float4 v = *(const float4*)(res + rl * MD_PP + c4);
            const size_t at = (size_t)(r0 + rl) * n + gcol;
            if (whole) {                                              // (n a multiple of 4: the four columns exist and are aligned)
                if (e.out_f32) *(float4*)((float*)e.out + at) = v;
                else *(uint2*)((bf16*)e.out + at) = md_pack4(v.x, v.y, v.z, v.w);
            } else {
                const float a[4] = {v.x, v.y, v.z, v.w};
                for (int i = 0; i < 4 && gcol + i < n; ++i) {
                    if (e.out_f32) ((float*)e.out)[at + i] = a[i];
                    else ((bf16*)e.out)[at + i] = __float2bfloat16_rn(a[i]);
                }
            }
        }
    } else if (mode == 1) {
        const bool whole = (e.inter & 3) == 0;
        for (int f = threadIdx.x; f < rows * 32; f += MD_THREADS) {
            const int rl = f >> 5, c4 = (f & 31) * 4, gcol = tile * 128 + c4;
            if (gcol >= e.inter) continue;
            const float4 g = *(const float4*)(res + rl * MD_PP + c4), u = *(const float4*)(res + rl * MD_PP + 128 + c4);
            const float a[4] = {g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y,
                                g.z / (1.f + expf(-g.z)) * u.z, g.w / (1.f + expf(-g.w)) * u.w};
            bf16* o = (bf16*)e.out + (size_t)(r0 + rl) * e.inter + gcol;
            if (whole) *(uint2*)o = md_pack4(a[0], a[1], a[2], a[3]);
            else for (int i = 0; i < 4 && gcol + i < e.inter; ++i) o[i] = __float2bfloat16_rn(a[i]);
        }
    } else if (mode == 3) {
        const bool whole = (n & 3) == 0;
        for (int rl = warp; rl < rows; rl += MD_THREADS / 32) {       // a warp a row, a lane four columns at a time
            const int row = r0 + rl;
            float sq = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c4 = (lane + 32 * j) * 4, gcol = tile * MD_BN + c4;
                if (gcol >= n) continue;
                const float4 v = *(const float4*)(res + rl * MD_PP + c4);
                const size_t at = (size_t)row * n + gcol;
                const float a[4] = {v.x, v.y, v.z, v.w};
                float hn[4] = {0.f, 0.f, 0.f, 0.f}, y[4] = {0.f, 0.f, 0.f, 0.f};
                if (whole) {
                    const float4 before = *(const float4*)(e.h + at);
                    const float b[4] = {before.x, before.y, before.z, before.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        hn[i] = b[i] + rounded<bf16>(a[i]);
                        y[i] = hn[i] * (md_weight(e.next_weight, e.next_weight_f32, gcol + i) + e.next_offset);
                        sq += hn[i] * hn[i];
                    }
                    *(float4*)(e.h + at) = make_float4(hn[0], hn[1], hn[2], hn[3]);
                    *(uint2*)((bf16*)e.out + at) = md_pack4(y[0], y[1], y[2], y[3]);
                } else {
                    for (int i = 0; i < 4 && gcol + i < n; ++i) {
                        hn[i] = e.h[at + i] + rounded<bf16>(a[i]);
                        e.h[at + i] = hn[i];
                        ((bf16*)e.out)[at + i] =
                            __float2bfloat16_rn(hn[i] * (md_weight(e.next_weight, e.next_weight_f32, gcol + i) + e.next_offset));
                        sq += hn[i] * hn[i];
                    }
                }
            }
            sq = warp_sum(sq);
            if (lane == 0) e.ss_out[tile * MD_ROWS + row] = sq;
        }
    } else {                                                          // mode 2: a warp a (row, head)
        const int hd = e.head_dim, half = hd >> 1, per_tile = MD_BN / hd;
        for (int item = warp; item < rows * per_tile; item += MD_THREADS / 32) {
            const int rl = item / per_tile, hh = item - rl * per_tile, head = tile * per_tile + hh, row = r0 + rl;
            if (head >= e.heads + 2 * e.kv_heads) continue;
            const bool is_q = head < e.heads, is_v = head >= e.heads + e.kv_heads;
            const void* weight = is_q ? e.q_weight : e.k_weight;
            float* y = res + rl * MD_PP + hh * hd;                    // the head's columns of this row
            float ss = 0.f;
            for (int c = lane; c < hd; c += 32) {                     // the product as the separate kernel would read it
                const float v = rounded<bf16>(y[c]);
                y[c] = v;
                ss += v * v;
            }
            ss = warp_sum(ss);
            __syncwarp();
            const float rstd = rsqrtf(ss / (float)hd + e.eps);
            bf16* dst = nullptr;
            if (is_q) {
                dst = e.q_out + ((size_t)row * e.heads + head) * hd;
            } else if (e.kv) {
                const int w = e.write_index[row];
                const int page = w >= 0 ? w / e.page_size : -1, off = w >= 0 ? w % e.page_size : 0;
                const int kvh = head - e.heads - (is_v ? e.kv_heads : 0);
                if (page >= 0 && page < e.pages)
                    dst = e.kv + ((((size_t)page * 2 + is_v) * e.kv_heads + kvh) * e.page_size + off) * hd;
            }
            if (!dst) continue;
            if (is_v) {
                for (int c = lane; c < hd; c += 32) dst[c] = __float2bfloat16_rn(y[c]);
                continue;
            }
            int pos = e.positions[row];
            pos = pos < 0 ? 0 : (pos >= e.max_positions ? e.max_positions - 1 : pos);
            for (int c = lane; c < half; c += 32) {                   // a pair (c, c + half) a lane
                float a = y[c], b = y[c + half];
                if (weight) {
                    a = rounded<bf16>(a * rstd * (md_weight(weight, e.weight_f32, c) + e.offset));
                    b = rounded<bf16>(b * rstd * (md_weight(weight, e.weight_f32, c + half) + e.offset));
                }
                const float cs = e.table[(size_t)pos * hd + c], sn = e.table[(size_t)pos * hd + half + c];
                dst[c] = __float2bfloat16_rn(a * cs - b * sn);
                dst[c + half] = __float2bfloat16_rn(b * cs + a * sn);
            }
        }
    }
    __syncwarp();
    if (csize > 1) asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");     // nobody leaves while its shared memory may be read
    tc_fence_before();
    __syncthreads();
    if (warp == 3) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(MD_BN) : "memory");
    }
}

// ---------------------------------------------------------------- host side
static int md_encode_map(CUtensorMap* map, const void* ptr, int rows, int k, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {MD_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                                              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) HB_REFUSE("gemm_mid: cuTensorMapEncodeTiled failed with %d (rows %d, k %d)", (int)r, rows, k);
    return 0;
}

// Clusters of `csize` CTAs of this kernel that the device runs at once (0: that size cannot be launched).
static int md_capacity(int csize) {
    static int cached[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
    if (cached[csize] >= 0) return cached[csize];
    if (cudaFuncSetAttribute(gemm_mid_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MD_SMEM) != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(csize * 64);
    cfg.blockDim = dim3(MD_THREADS);
    cfg.dynamicSmemBytes = MD_SMEM;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = csize; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_mid_kernel, &cfg) != cudaSuccess) { cudaGetLastError(); clusters = 0; }
    return cached[csize] = clusters;
}

HB_DEFINE_STATUS_MIRROR(hb_gemm_mid_status_mirror)
extern "C" int hb_gemm_mid_status(unsigned int* status) {
    HB_CUDA(cudaDeviceSynchronize());
    HB_CUDA(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(unsigned int)));
    const unsigned int zero = 0;
    HB_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(unsigned int)));
    return 0;
}

static int md_launch(const void* x, const void* w, int m, int n, int k, int rows_w, int tiles, int split, const MidArgs& e,
                     cudaStream_t s) {
    if (m < 1 || m > MD_ROWS) HB_REFUSE("gemm_mid: %d rows; this kernel takes 1 to %d", m, MD_ROWS);
    if (k < 8 || k % 8) HB_REFUSE("gemm_mid: k = %d is no multiple of 8", k);
    if ((((uintptr_t)x | (uintptr_t)w) % 16) != 0) HB_REFUSE("gemm_mid: x and w must be 16-byte aligned");
    if (e.ss_in && (e.parts_in < 1 || e.dim_in < 1 || e.stride_in < m)) HB_REFUSE("gemm_mid: %d partial sums of stride %d over %d columns", e.parts_in, e.stride_in, e.dim_in);
    CUtensorMap map_x, map_w;
    int rc = md_encode_map(&map_x, x, m, k, MD_ROWS);
    if (rc) return rc;
    rc = md_encode_map(&map_w, w, rows_w, k, 128);
    if (rc) return rc;
    const int kblocks = (k + MD_BK - 1) / MD_BK;
    int csize = 1;                                        // the largest cluster whose CTAs all run at once and have k blocks to do
    if (split > 0) {
        csize = split;
    } else {
        for (int c = 8; c > 1; --c)
            if (2 * c <= kblocks && tiles <= md_capacity(c)) { csize = c; break; }
    }
    if (csize < 1 || csize > 8 || md_capacity(csize) < 1) HB_REFUSE("gemm_mid: clusters of %d CTAs cannot be launched", csize);
    HB_CUDA(cudaFuncSetAttribute(gemm_mid_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MD_SMEM));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * csize);
    cfg.blockDim = dim3(MD_THREADS);
    cfg.dynamicSmemBytes = MD_SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = csize; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    HB_CUDA(cudaLaunchKernelEx(&cfg, gemm_mid_kernel, map_x, map_w, m, n, k, csize, e));
    return 0;
}

// mode 0, 1, 3 as in the header of this file; ss_in [parts_in, stride_in] (null: x is normed); ss_out [ceil(n / 256), 64].
// `split`: CTAs a tile's k range is shared by (0: chosen). m 1 to 64, k a multiple of 8, pointers 16-byte aligned.
extern "C" int hb_gemm_bf16_mid(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode, int inter,
                                float* h, const void* next_weight, int next_weight_f32, float next_offset, float* ss_out,
                                const float* ss_in, int parts_in, int stride_in, float eps_in, int dim_in, int split,
                                hb_stream stream) {
    if (m == 0) return 0;
    if (mode != 0 && mode != 1 && mode != 3) HB_REFUSE("gemm_mid: mode %d", mode);
    if (mode == 1 && (inter < 1 || out_f32)) HB_REFUSE("gemm_mid: mode 1 needs inter and writes bfloat16");
    if (mode != 1 && n < 1) HB_REFUSE("gemm_mid: n = %d", n);
    if (mode == 3 && (!h || !next_weight || !ss_out || out_f32)) HB_REFUSE("gemm_mid: mode 3 needs h, the next norm's weight and ss_out, and writes bfloat16");
    if (((uintptr_t)out % 16) != 0) HB_REFUSE("gemm_mid: out must be 16-byte aligned");
    MidArgs e = {};
    e.out = out; e.out_f32 = out_f32; e.mode = mode; e.inter = inter;
    e.ss_in = ss_in; e.parts_in = parts_in; e.dim_in = dim_in; e.stride_in = stride_in; e.eps_in = eps_in;
    e.h = h; e.next_weight = next_weight; e.next_weight_f32 = next_weight_f32; e.next_offset = next_offset; e.ss_out = ss_out;
    const int tiles = mode == 1 ? (inter + 127) / 128 : (n + MD_BN - 1) / MD_BN;
    return md_launch(x, w, m, n, k, mode == 1 ? 2 * inter : n, tiles, split, e, (cudaStream_t)stream);
}

// The attention's first product for 17 to 64 tokens with the q/k norm, the rotation and the cache write in its
// epilogue (mode 2): arguments as hb_qkv_rope_skinny_linked, with the stride of ss_in.
extern "C" int hb_qkv_rope_mid(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions,
                               const float* table, int max_positions, const void* q_weight, const void* k_weight,
                               int weight_f32, float eps, float offset, void* kv, const int32_t* write_index, int pages,
                               int page_size, int heads, int kv_heads, int head_dim, const float* ss_in, int parts_in,
                               int stride_in, float eps_in, int dim_in, int split, hb_stream stream) {
    if (m == 0) return 0;
    if (head_dim != 32 && head_dim != 64 && head_dim != 128) HB_REFUSE("qkv_rope_mid: head_dim %d (32, 64 or 128)", head_dim);
    if (heads < 1 || kv_heads < 1) HB_REFUSE("qkv_rope_mid: %d heads, %d kv heads", heads, kv_heads);
    if (!q_out || !positions || !table || max_positions < 1) HB_REFUSE("qkv_rope_mid: q_out, positions and the table are needed");
    if ((q_weight == nullptr) != (k_weight == nullptr)) HB_REFUSE("qkv_rope_mid: both norm weights or none");
    if (kv && (!write_index || pages < 1 || page_size < 1)) HB_REFUSE("qkv_rope_mid: a cache needs write_index, pages and page_size");
    MidArgs e = {};
    e.mode = 2;
    e.ss_in = ss_in; e.parts_in = parts_in; e.dim_in = dim_in; e.stride_in = stride_in; e.eps_in = eps_in;
    e.q_out = (bf16*)q_out; e.positions = positions; e.table = table; e.max_positions = max_positions;
    e.q_weight = q_weight; e.k_weight = k_weight; e.weight_f32 = weight_f32; e.eps = eps; e.offset = offset;
    e.kv = (bf16*)kv; e.write_index = write_index; e.pages = pages; e.page_size = page_size;
    e.heads = heads; e.kv_heads = kv_heads; e.head_dim = head_dim;
    const int n = (heads + 2 * kv_heads) * head_dim;
    return md_launch(x, w, m, n, k, n, (n + MD_BN - 1) / MD_BN, split, e, (cudaStream_t)stream);
}
