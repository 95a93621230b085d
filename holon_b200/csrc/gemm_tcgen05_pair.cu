// bfloat16 GEMM on tcgen05 tensor cores with two CTAs on one tile: out[m, n] = sum_k x[m, k] * w[n, k].
//
// A cluster of two CTAs (two neighbouring SMs) computes 256 x 256 tiles with tcgen05.mma.cta_group::2: each CTA loads
// its own 128 rows of x and only its own 128 of the tile's 256 rows of w per 64-wide k block (32 KB a stage instead of
// the 48 KB a lone CTA needs for half the tile), the leader CTA's one thread issues the MMAs for both, and each CTA
// ends up with its 128 rows x 256 columns of the accumulator in its own tensor memory. Half the shared-memory traffic
// per flop is what lets the tensor pipe run near its rate; it also leaves room for six stages.
//   loads      warp 0 of either CTA: cp.async.bulk.tensor ... cta_group::2 (no multicast), completing on the LEADER's
//              "full" barrier, on which the leader's producer alone expects the bytes of both CTAs;
//   MMAs       warp 1 of the leader: four tcgen05.mma (M 256, N 256, K 16) a stage; tcgen05.commit with cluster
//              multicast frees the stage in both CTAs, and after a tile's last k block tells both CTAs' epilogues;
//   epilogue   warps 2-5 of either CTA read their CTA's accumulator (tcgen05.ld) and write its rows; the leader's
//              MMA thread reuses an accumulator after all eight epilogue warps (four of them in the peer, arriving
//              across the cluster) have read it. Two accumulators of 256 columns alternate.
// The tile's width bn is a launch parameter (a multiple of 16 up to 256; a multiple of 64 in mode 1): 256 unless a
// narrower tile fills the waves of 74 pairs so much better that it pays for its worse ratio of flops to bytes.
// mode 1 (SwiGLU's first half): the leader's rows of w are bn / 2 gate rows, the peer's the bn / 2 up rows of the same
// columns, so every CTA holds gate in its accumulator's first bn / 2 columns and up in the next bn / 2.
// Every wait is bounded (tcgen05.cuh); a CTA whose wait gave up records the place and still reaches the cluster
// barrier at the end, so its partner is not left waiting for it there.
#include "tcgen05.cuh"

#define TP_BM 128                                 // rows of x per CTA; the pair's tile has 256
#define TP_BN 256                                 // the widest tile; an accumulator's columns in tensor memory
#define TP_BK 64
#define TP_STAGES 6
#define TP_A_BYTES (TP_BM * TP_BK * 2)
#define TP_B_BYTES (128 * TP_BK * 2)              // a CTA's half of the tile's rows of w
#define TP_STAGE_BYTES (TP_A_BYTES + TP_B_BYTES)
#define TP_SMEM (TP_STAGES * TP_STAGE_BYTES + 1024 + 256)

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of this CTA's shared address `addr` inside CTA `rank`.
__device__ __forceinline__ uint32_t in_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// A tile load of a CTA pair: the data lands in this CTA, the bytes are counted on a barrier that may be the partner's.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once the MMAs issued so far have finished, on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}

// Tile t of the launch (256 x 256): bands of 8 tile rows, the row index fastest inside a band (see gemm_tcgen05.cu).
struct PairTile { int m_tile, n_tile; };
__device__ __forceinline__ PairTile pair_tile(int t, int tiles_m, int tiles_n) {
    constexpr int BAND = 8;
    const int per_band = BAND * tiles_n;
    const int band = t / per_band, within = t - band * per_band;
    const int rows = min(BAND, tiles_m - band * BAND);
    PairTile at;
    at.n_tile = within / rows;
    at.m_tile = band * BAND + within - at.n_tile * rows;
    return at;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         void* __restrict__ out, int out_f32, int m, int n, int k, int mode, int inter, int tiles_m,
                         int tiles_n, int bn) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;     // the swizzle pattern needs 1024-byte alignment
    const uint32_t bars = base + TP_STAGES * TP_STAGE_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * TP_STAGES;        // full: used in the leader only; empty: in both
    const uint32_t acc_full0 = bars + 16 * TP_STAGES, acc_empty0 = acc_full0 + 16;   // acc_empty: used in the leader only
    const uint32_t slot = acc_empty0 + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int kblocks = (k + TP_BK - 1) / TP_BK;
    const int tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TP_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, 8); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {                                                  // the same warp of both CTAs, as the pair's allocation asks
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(2 * TP_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync();                                                   // the partner's barriers exist before anything arrives on them
    tc_fence_after();
    uint32_t tmem;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem) : "r"(slot));

    if (warp == 0) {
        if (lane == 0) {
            int kb_all = 0;                                           // k blocks loaded so far, over all tiles
            for (int t = pair; t < tiles; t += pairs) {
                const PairTile at = pair_tile(t, tiles_m, tiles_n);
                const int m0 = at.m_tile * 2 * TP_BM + (int)rank * TP_BM;
                const int half = bn >> 1;                             // this CTA's rows of w
                const int w0 = mode == 1 ? (leader ? at.n_tile * half : inter + at.n_tile * half)
                                         : at.n_tile * bn + (int)rank * half;
                bool ok = true;
                for (int kb = 0; kb < kblocks && ok; ++kb, ++kb_all) {
                    const int s = kb_all % TP_STAGES;
                    ok = mbar_wait(empty0 + 8 * s, ((kb_all / TP_STAGES) & 1) ^ 1, 1);
                    if (!ok) break;
                    const uint32_t a = base + s * TP_STAGE_BYTES, b = a + TP_A_BYTES;
                    if (leader) mbar_expect_tx(full0 + 8 * s, 2 * (TP_A_BYTES + (bn >> 1) * TP_BK * 2));   // its own bytes and the partner's
                    const uint32_t bar = in_cta(full0 + 8 * s, 0);
                    tma_load_2d_pair(a, &map_x, bar, kb * TP_BK, m0);
                    tma_load_2d_pair(b, &map_w, bar, kb * TP_BK, w0);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // kind::f16: D float32 (bit 4), A and B bfloat16 (bits 7, 10), both K-major, N / 8 at bit 17, M / 16 at bit 24
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)((2 * TP_BM) >> 4) << 24);
            int kb_all = 0, local = 0;
            bool ok = true;
            for (int t = pair; t < tiles && ok; t += pairs, ++local) {
                const int acc = local & 1, use = local >> 1;
                ok = mbar_wait(acc_empty0 + 8 * acc, (use & 1) ^ 1, 4);   // both CTAs' epilogues have read this accumulator
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem + acc * TP_BN;
                for (int kb = 0; kb < kblocks; ++kb, ++kb_all) {
                    const int s = kb_all % TP_STAGES;
                    ok = mbar_wait(full0 + 8 * s, (kb_all / TP_STAGES) & 1, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a = base + s * TP_STAGE_BYTES, b = a + TP_A_BYTES;
                    const uint64_t da = tc_smem_desc(a), db = tc_smem_desc(b);
#pragma unroll
                    for (int kk = 0; kk < TP_BK / 16; ++kk)          // 16 k values = 32 bytes further along each row
                        tc_mma_pair(d, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb | kk) != 0);
                    tc_commit_pair(empty0 + 8 * s);                   // the stage is free in both CTAs once these have read it
                }
                tc_commit_pair(acc_full0 + 8 * acc);                  // both epilogues may read when every MMA above has finished
            }
        }
    } else {
        const int q = warp & 3;                                       // this warp's quarter of the TMEM lanes = the CTA's tile rows
        const int width = mode == 1 ? inter : n;
        const int span = mode == 1 ? bn >> 1 : bn;                    // output columns of a tile
        const int chunks = (span + 31) >> 5;
        const uint32_t acc_empty_leader = in_cta(acc_empty0, 0);
        int local = 0;
        for (int t = pair; t < tiles; t += pairs, ++local) {
            const int acc = local & 1, use = local >> 1;
            const PairTile at = pair_tile(t, tiles_m, tiles_n);
            const int row = at.m_tile * 2 * TP_BM + (int)rank * TP_BM + q * 32 + lane;
            const int col0 = at.n_tile * span;
            if (!mbar_wait(acc_full0 + 8 * acc, use & 1, 3)) break;
            tc_fence_after();
            const uint32_t d = tmem + acc * TP_BN + ((uint32_t)(q * 32) << 16);
            for (int c = 0; c < chunks; ++c) {
                uint32_t r[32];
                tc_ld32(d + c * 32, r);
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                if (mode == 1) {
                    uint32_t u[32];
                    tc_ld32(d + span + c * 32, u);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = v[i] / (1.f + __expf(-v[i])) * __uint_as_float(u[i]);
                }
                if (c == chunks - 1) {                               // everything is in registers: hand the accumulator back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(acc_empty_leader + 8 * acc);
                }
                const int col = col0 + c * 32;
                const int live = min(min(32, span - c * 32), width - col);    // columns of this chunk that exist
                if (row < m && live > 0) {
                    if (out_f32) {
                        float* o = (float*)out + (size_t)row * width + col;
                        if (live == 32 && (width & 3) == 0) {
#pragma unroll
                            for (int i = 0; i < 32; i += 4) *(float4*)(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                        } else {
                            for (int i = 0; i < live; ++i) o[i] = v[i];
                        }
                    } else {
                        bf16* o = (bf16*)out + (size_t)row * width + col;
                        if (live == 32 && (width & 7) == 0) {
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                uint4 p;
                                __nv_bfloat162 a0 = __floats2bfloat162_rn(v[i], v[i + 1]), a1 = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
                                __nv_bfloat162 a2 = __floats2bfloat162_rn(v[i + 4], v[i + 5]), a3 = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
                                p.x = *(uint32_t*)&a0; p.y = *(uint32_t*)&a1; p.z = *(uint32_t*)&a2; p.w = *(uint32_t*)&a3;
                                *(uint4*)(o + i) = p;
                            }
                        } else {
                            for (int i = 0; i < live; ++i) o[i] = __float2bfloat16_rn(v[i]);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync();                                                   // neither CTA leaves, or frees tensor memory, while the other may still use it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * TP_BN) : "memory");
    }
}

// ---------------------------------------------------------------- host side
static int encode_pair_map(CUtensorMap* map, const void* ptr, int rows, int k, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {TP_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                                              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) HB_REFUSE("gemm_tcgen05_pair: cuTensorMapEncodeTiled failed with %d (rows %d, k %d)", (int)r, rows, k);
    return 0;
}

// Reads and clears this kernel's status word: 0, or (place << 28) | (block + 1) of the first wait that gave up
// (place 1 producer, 2 and 4 MMA, 3 epilogue). Synchronises the device.
HB_DEFINE_STATUS_MIRROR(hb_gemm_tcgen05_pair_status_mirror)
extern "C" int hb_gemm_tcgen05_pair_status(unsigned int* status) {
    HB_CUDA(cudaDeviceSynchronize());
    HB_CUDA(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(unsigned int)));
    const unsigned int zero = 0;
    HB_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(unsigned int)));
    return 0;
}

// The same contract as hb_gemm_bf16_tcgen05 (gemm_tcgen05.cu), computed by pairs of CTAs.
static int forced_bn = 0;
// Tests: a fixed tile width for the launches that follow (0: chosen per launch again).
extern "C" int hb_gemm_tcgen05_pair_width(int bn) { forced_bn = bn; return 0; }

extern "C" int hb_gemm_bf16_tcgen05_pair(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode,
                                         int inter, hb_stream stream) {
    if (m == 0 || n == 0) return 0;
    if (k < 8 || k % 8) HB_REFUSE("gemm_tcgen05_pair: k = %d is no multiple of 8", k);
    if ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) % 16) != 0) HB_REFUSE("gemm_tcgen05_pair: pointers must be 16-byte aligned");
    if (mode != 0 && mode != 1) HB_REFUSE("gemm_tcgen05_pair: mode %d", mode);
    if (mode == 1 && (inter < 1 || n != 2 * inter)) HB_REFUSE("gemm_tcgen05_pair: mode 1 needs n = 2 inter (n %d, inter %d)", n, inter);
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        HB_CUDA(cudaGetDevice(&device));
        HB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    }
    // The tile width: 256 unless a narrower one saves more than a tenth by filling the waves better. A tile's time goes
    // with the larger of its MMA cycles (~ width) and its shared-memory traffic (~ 128 + width / 2: x's rows are loaded
    // whatever the width), which is why narrow tiles pay less than their width suggests (measured: 6144 columns in
    // tiles of 176 took 103 us against 87 us in tiles of 256). Widths are multiples of 16; mode 1 wants both halves
    // whole 32-column pieces of tensor memory, so multiples of 64.
    const int tiles_m = (m + 2 * TP_BM - 1) / (2 * TP_BM);
    const int span_all = mode == 1 ? inter : n, step = mode == 1 ? 64 : 16;
    int bn = forced_bn > 0 ? forced_bn : TP_BN;
    if (forced_bn <= 0) {
        auto cost = [&](int width) {
            const int span = mode == 1 ? width / 2 : width;
            const long tiles = (long)tiles_m * ((span_all + span - 1) / span);
            const int tile = width > 128 + width / 2 ? width : 128 + width / 2;
            return ((tiles + sms / 2 - 1) / (sms / 2)) * tile;
        };
        long best = cost(TP_BN) * 9 / 10;
        for (int cand = TP_BN - step; cand >= 128; cand -= step)
            if (cost(cand) < best) { best = cost(cand); bn = cand; }
    }
    if (bn < 32 || bn > TP_BN || bn % step) HB_REFUSE("gemm_tcgen05_pair: tile width %d (a multiple of %d up to %d)", bn, step, TP_BN);
    const int span = mode == 1 ? bn / 2 : bn;
    const int tiles_n = (span_all + span - 1) / span;
    CUtensorMap map_x, map_w;
    int rc = encode_pair_map(&map_x, x, m, k, TP_BM);
    if (rc) return rc;
    rc = encode_pair_map(&map_w, w, n, k, bn / 2);
    if (rc) return rc;
    HB_CUDA(cudaFuncSetAttribute(gemm_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM));
    const long tiles = (long)tiles_m * tiles_n;
    const int pairs = (int)(tiles < sms / 2 ? tiles : sms / 2);
    gemm_tcgen05_pair_kernel<<<2 * pairs, 192, TP_SMEM, (cudaStream_t)stream>>>(map_x, map_w, out, out_f32, m, n, k, mode,
                                                                              inter, tiles_m, tiles_n, bn);
    HB_LAUNCH_CHECK("gemm_tcgen05_pair");
    return 0;
}
