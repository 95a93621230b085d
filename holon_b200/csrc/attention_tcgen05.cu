// bfloat16 paged prefill attention on tcgen05 tensor cores, head size 128, pages of a multiple of 64 tokens.
//
// A CTA owns 256 queries of one head, as two groups of 128, and walks that row's 64-key tiles up to its diagonal; per group:
//   S = Q K^T    tcgen05.mma 128 x 64 x 16, eight per tile, Q and K in shared memory (TMA, 128-byte swizzle), S in one
//                of two 64-column tensor-memory buffers;
//   softmax      four warps, one query row per thread: tcgen05.ld of the row, mask, running maximum, 2^x, row sum, all
//                without a shuffle; the weights P go back to tensor memory as bfloat16 pairs, over the S they came from;
//   O += P V     tcgen05.mma 128 x 128 x 16, four per tile, P read from tensor memory, V from shared memory as an
//                MN-major operand (values are stored [key][d]), O in 128 tensor-memory columns for the whole walk.
// The running maximum is allowed to lag: O and the row sums are rescaled only when a row's maximum has grown by more
// than 2^8 since the last rescale (the weights stay below 256, which bfloat16 holds), so the tensor-memory round trip
// of O is rare. One thread issues the score MMAs of both groups, keeping S of tile j + 1 in flight while the
// softmax of tile j runs, and each group has a thread that issues its P V MMAs. Warp 0 loads by TMA (queries once;
// keys and values of a tile as four 64 x 64 boxes from the paged cache, found through the block table), warp 1 issues
// the score MMAs and owns the tensor memory, warps 10 and 11 issue the groups' P V MMAs, warps 2-5 and 6-9 are the
// groups' softmax and epilogue.
// Keys past a row's length are masked; they are read (a page is loaded whole), which is safe because cache pools start
// as zeros and only ever hold finite values. Every mbarrier wait is bounded (tcgen05.cuh).
#include "tcgen05.cuh"

#define AT_D 128
#define AT_BM 128                                 // queries per group; a CTA carries two groups
#define AT_GROUPS 2
#define AT_BN 64
#define AT_STAGES 3
#define AT_Q_BYTES (AT_BM * AT_D * 2)             // 32 KB a group: two [128 x 64] swizzled blocks
#define AT_KV_BYTES (AT_BN * AT_D * 2)            // 16 KB: two [64 x 64] swizzled blocks
#define AT_SMEM (AT_GROUPS * AT_Q_BYTES + AT_STAGES * 2 * AT_KV_BYTES + 1024 + 256)
#define AT_TMEM_COLS 512                          // per group: S0 [0, 64), S1 [64, 128), O [128, 256)
#define AT_RESCALE 8.0f
#define AT_MMA_WARP1 10                            // warps 10, 11: the groups' P V issuing warps; warps 2-9 are the softmax
#define AT_THREADS 384

__device__ __forceinline__ float at_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

// Two float32 in one 64-bit register, for the packed arithmetic of sm_100 (one instruction, two results).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// The same with the A operand in tensor memory (128 lanes x K/2 columns, two bfloat16 per column).
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

// Two groups of 128 queries share the CTA's key and value tiles; each has its own softmax warps (2-5 and 6-9), its own
// S, P and O, so that one group's softmax runs while the tensor cores work for the other.
__global__ void __launch_bounds__(AT_THREADS, 1) prefill_tcgen05_kernel(
        const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, bf16* __restrict__ out,
        const int32_t* __restrict__ block_table, int table_stride, const int32_t* __restrict__ row_slot,
        const int32_t* __restrict__ query_start, const int32_t* __restrict__ kv_len, int row0, int rows, int heads,
        int kv_heads, int pages, int page_size, float scale_log2, int window, int tile_q) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base, kv_s = q_s + AT_GROUPS * AT_Q_BYTES;
    const uint32_t bars = kv_s + AT_STAGES * 2 * AT_KV_BYTES;
    const uint32_t q_full = bars, kv_full0 = bars + 8, kv_empty0 = kv_full0 + 8 * AT_STAGES;
    // per group g and buffer i, at index (g * 2 + i): scores computed; weights written; weights read (O holds the tile)
    const uint32_t s_full0 = kv_empty0 + 8 * AT_STAGES, p_full0 = s_full0 + 32;
    const uint32_t p_empty0 = p_full0 + 32, o_full0 = p_empty0 + 32, slot = o_full0 + 16;
    __shared__ int s_row, s_q0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        int left = (int)blockIdx.y, found = -1, q0 = 0;      // blocks are handed out x first: every head's late query
                                                             // tiles (the longest walks) start before any short one
        for (int b = rows - 1; b >= row0; --b) {
            const int tiles = (query_start[b + 1] - query_start[b] + tile_q - 1) / tile_q;
            if (left < tiles) { found = b; q0 = (tiles - 1 - left) * tile_q; break; }
            left -= tiles;
        }
        s_row = found; s_q0 = q0;
        mbar_init(q_full, 1);
        for (int s = 0; s < AT_STAGES; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1 + AT_GROUPS); }
        for (int i = 0; i < 2 * AT_GROUPS; ++i) {
            mbar_init(s_full0 + 8 * i, 1);
            mbar_init(p_full0 + 8 * i, 4); mbar_init(p_empty0 + 8 * i, 1);
        }
        for (int g = 0; g < AT_GROUPS; ++g) mbar_init(o_full0 + 8 * g, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(AT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem) : "r"(slot));

    const int b = s_row;
    const int h = blockIdx.x, hk = h / (heads / kv_heads);
    int tile_lo = 0, t0 = 0, p0 = 0, n = 0, nq = 0;
    int g_tiles[AT_GROUPS] = {0, 0}, g_qn[AT_GROUPS] = {0, 0}, g_hi[AT_GROUPS] = {0, 0};
    if (b >= 0) {
        nq = query_start[b + 1] - query_start[b];
        n = kv_len[b];
        t0 = query_start[b] + s_q0;
        p0 = n - nq + s_q0;                                          // position of the CTA's first query
        const int lo = window > 0 ? max(0, p0 - window + 1) : 0;
        tile_lo = lo / AT_BN;
#pragma unroll
        for (int g = 0; g < AT_GROUPS; ++g) {
            g_qn[g] = max(0, min(AT_BM, min(nq - s_q0, tile_q) - g * AT_BM));   // queries of this group
            g_hi[g] = g_qn[g] ? min(n, p0 + g * AT_BM + g_qn[g]) : 0;   // keys below this are visible to some of them
            g_tiles[g] = g_qn[g] ? (g_hi[g] + AT_BN - 1) / AT_BN - tile_lo : 0;
        }
    }
    const int tiles = max(g_tiles[0], g_tiles[1]);

    if (b >= 0 && warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, AT_GROUPS * AT_Q_BYTES);
#pragma unroll
            for (int g = 0; g < AT_GROUPS; ++g) {                    // (a group without queries loads rows it never uses)
                tma_load_2d(q_s + g * AT_Q_BYTES, &map_q, q_full, h * AT_D, t0 + g * AT_BM);
                tma_load_2d(q_s + g * AT_Q_BYTES + AT_Q_BYTES / 2, &map_q, q_full, h * AT_D + 64, t0 + g * AT_BM);
            }
            const int32_t* table = block_table + (size_t)row_slot[b] * table_stride;
            for (int j = 0; j < tiles; ++j) {
                const int s = j % AT_STAGES;
                if (!mbar_wait(kv_empty0 + 8 * s, ((j / AT_STAGES) & 1) ^ 1, 1)) break;
                const int key0 = (tile_lo + j) * AT_BN;
                int page = table[key0 / page_size];
                page = page < 0 || page >= pages ? 0 : page;
                const int k_row = ((page * 2) * kv_heads + hk) * page_size + key0 % page_size;   // row of the flattened cache
                const int v_row = k_row + kv_heads * page_size;
                const uint32_t k_dst = kv_s + s * 2 * AT_KV_BYTES, v_dst = k_dst + AT_KV_BYTES;
                mbar_expect_tx(kv_full0 + 8 * s, 2 * AT_KV_BYTES);
                tma_load_2d(k_dst, &map_kv, kv_full0 + 8 * s, 0, k_row);
                tma_load_2d(k_dst + AT_KV_BYTES / 2, &map_kv, kv_full0 + 8 * s, 64, k_row);
                tma_load_2d(v_dst, &map_kv, kv_full0 + 8 * s, 0, v_row);
                tma_load_2d(v_dst + AT_KV_BYTES / 2, &map_kv, kv_full0 + 8 * s, 64, v_row);
            }
        }
    } else if (b >= 0 && (warp == 1 || warp >= AT_MMA_WARP1)) {
        if (lane == 0) {
            // Three issuing threads: one for the scores S = Q K^T of both groups, and for each group one for O += P V.
            // An MMA costs its issuing thread 60 to 200 cycles however small it is (a 128 x 64 x 16 one needs 32 cycles
            // of the tensor pipe), so a single thread with all 24 MMAs of a tile-step, or even one thread per group,
            // was the kernel's bound. (Four threads would need 416 threads a CTA, and the softmax warps their registers.)
            // kind::f16, D float32, A and B bfloat16; N / 8 at bit 17, M / 16 at bit 24; bit 16: B is MN-major
            const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_BN >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
            const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(AT_D >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
            if (warp == 1) {
                bool ok = mbar_wait(q_full, 0, 2);
                for (int j = 0; j < tiles && ok; ++j) {
                    const int s = j % AT_STAGES;
                    ok = mbar_wait(kv_full0 + 8 * s, (j / AT_STAGES) & 1, 3);
                    const uint32_t k_src = kv_s + s * 2 * AT_KV_BYTES;
                    for (int g = 0; g < AT_GROUPS && ok; ++g) {
                        if (j >= g_tiles[g]) continue;
                        const int gb = g * 2 + (j & 1);
                        // S_j overwrites S and P of tile j - 2: wait until P V of that tile has read them
                        if (j >= 2) ok = mbar_wait(p_empty0 + 8 * gb, ((j - 2) >> 1) & 1, 4);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t s_t = tmem + g * 256 + (j & 1) * AT_BN;
#pragma unroll
                        for (int kk = 0; kk < AT_D / 16; ++kk) {      // d 0..63 in the first block, 64..127 in the second
                            const uint32_t blk = kk >> 2, within = (kk & 3) * 2;
                            tc_mma_f16(s_t, tc_smem_desc(q_s + g * AT_Q_BYTES + blk * (AT_Q_BYTES / 2)) + within,
                                       tc_smem_desc(k_src + blk * (AT_KV_BYTES / 2)) + within, idesc_qk, kk != 0);
                        }
                        tc_commit(s_full0 + 8 * gb);
                    }
                    if (ok) tc_commit(kv_empty0 + 8 * s);             // the keys of the stage have been read (all three must arrive)
                }
            } else {
                const int g = warp - AT_MMA_WARP1;
                const int my_tiles = g_tiles[g];
                const uint32_t o_t = tmem + g * 256 + 2 * AT_BN;
                bool ok = true;
                for (int j = 0; j < tiles && ok; ++j) {               // (a group past its own last tile still paces the stages)
                    const int s = j % AT_STAGES, gb = g * 2 + (j & 1);
                    ok = mbar_wait(kv_full0 + 8 * s, (j / AT_STAGES) & 1, 3);
                    if (ok && j < my_tiles) {                         // O_g += P_g,j V_j
                        ok = mbar_wait(p_full0 + 8 * gb, (j >> 1) & 1, 5);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t v_src = kv_s + s * 2 * AT_KV_BYTES + AT_KV_BYTES;
                        const uint32_t p_t = tmem + g * 256 + (j & 1) * AT_BN;   // P lies over the first half of its own S
#pragma unroll
                        for (int kk = 0; kk < AT_BN / 16; ++kk)       // 16 keys a step: 8 columns along P, 16 rows down V
                            tc_mma_f16_ts(o_t, p_t + kk * 8, tc_smem_desc_mn(v_src + kk * 16 * 128, AT_KV_BYTES / 2), idesc_pv,
                                          (j | kk) != 0);
                        tc_commit(p_empty0 + 8 * gb);                 // P has been read; O_g holds tile j
                        if (j == my_tiles - 1) tc_commit(o_full0 + 8 * g);   // the group's last tile: its output is complete
                    }
                    if (ok) tc_commit(kv_empty0 + 8 * s);             // the values of the stage have been read
                }
                if (my_tiles == 0 || !ok) tc_commit(o_full0 + 8 * g);    // (nothing was issued for it, or the walk gave up)
            }
        }
    } else if (b >= 0 && warp < AT_MMA_WARP1) {
        const int g = (warp - 2) >> 2;                                // this warp's group of queries
        const int q = warp & 3;                                       // and its quarter of the TMEM lanes = query rows
        const int r = q * 32 + lane;                                  // this thread's query row within the group
        const int pos = p0 + g * AT_BM + r;                           // and its position
        const int hi = g_hi[g], qn = g_qn[g], my_tiles = g_tiles[g];
        const uint32_t lane_t = tmem + g * 256 + ((uint32_t)(q * 32) << 16);
        const uint32_t o_t = lane_t + 2 * AT_BN;
        float m_used = -INFINITY, l = 0.f;                            // in log2 units; the maximum may lag by AT_RESCALE
        bool ok = true;
        for (int j = 0; j < my_tiles && ok; ++j) {
            const int gb = g * 2 + (j & 1);
            ok = mbar_wait(s_full0 + 8 * gb, (j >> 1) & 1, 6);
            if (!ok) break;
            tc_fence_after();
            uint32_t sr[2][32];
            tc_ld32_nowait(lane_t + (j & 1) * AT_BN, sr[0]);
            tc_ld32_nowait(lane_t + (j & 1) * AT_BN + 32, sr[1]);
            tc_ld_wait();
            const int key0 = (tile_lo + j) * AT_BN;
            const bool edge = key0 + AT_BN - 1 > p0 + g * AT_BM || window > 0 || key0 + AT_BN > hi;
            if (edge) {
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = key0 + c * 32 + i;
                        if (!(key <= pos && key < hi && (window <= 0 || pos - key < window))) sr[c][i] = 0xff800000u;   // -inf
                    }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains instead of one of 64
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sr[c][i]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float mt = mx * scale_log2;
            const bool grow = mt > m_used + AT_RESCALE || (m_used == -INFINITY && mt > -INFINITY);
            if (__any_sync(0xffffffffu, grow)) {                      // rescale what is summed (whole warp: the TMEM ops are collective)
                const float m_new = grow ? mt : m_used;
                const float f = m_used == -INFINITY ? 0.f : at_ex2(m_used - m_new);
                if (j > 0) {
                    ok = mbar_wait(p_empty0 + 8 * (g * 2 + ((j - 1) & 1)), ((j - 1) >> 1) & 1, 7);   // O holds every tile before j
                    tc_fence_after();
                    if (ok) {
#pragma unroll
                        for (int c = 0; c < AT_D / 32; ++c) {
                            uint32_t o[32];
                            tc_ld32(o_t + c * 32, o);
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                            tc_st32(o_t + c * 32, o);
                        }
                    }
                }
                l *= f;
                m_used = m_new;
            }
            const float off = m_used == -INFINITY ? 0.f : -m_used;
            const uint64_t scale2 = pack2(scale_log2, scale_log2), off2 = pack2(off, off);
            uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};              // four chains of packed sums
            uint32_t pk[32];                                          // 64 weights as bfloat16 pairs
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float a, d;
                    unpack2(fma2(pack2(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1])), scale2, off2), a, d);
                    a = at_ex2(a);
                    d = at_ex2(d);
                    sum2[(i >> 1) & 3] = add2(sum2[(i >> 1) & 3], pack2(a, d));
                    __nv_bfloat162 pr = __floats2bfloat162_rn(a, d);
                    pk[c * 16 + i / 2] = *(uint32_t*)&pr;
                }
            {
                float lo, hi;
                unpack2(add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3])), lo, hi);
                l += lo + hi;
            }
            if (!ok) break;
            tc_st32(lane_t + (j & 1) * AT_BN, pk);                    // P over the S it came from: 32 columns of bfloat16 pairs
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full0 + 8 * gb);
        }
        if (ok) ok = mbar_wait(o_full0 + 8 * g, 0, 9);
        tc_fence_after();
        if (ok && qn > 0) {                                           // (the tensor-memory loads are warp-collective: no lane skips them)
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const bool keep = r < qn && my_tiles > 0 && l > 0.f;
            bf16* o_row = out + ((size_t)(t0 + g * AT_BM + (r < qn ? r : 0)) * heads + h) * AT_D;
#pragma unroll
            for (int c = 0; c < AT_D / 32; ++c) {
                uint32_t o[32];
                tc_ld32(o_t + c * 32, o);
                if (r < qn) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = keep ? __uint_as_float(o[i + e]) * inv : 0.f;
                        uint4 w;
                        __nv_bfloat162 a0 = __floats2bfloat162_rn(v[0], v[1]), a1 = __floats2bfloat162_rn(v[2], v[3]);
                        __nv_bfloat162 a2 = __floats2bfloat162_rn(v[4], v[5]), a3 = __floats2bfloat162_rn(v[6], v[7]);
                        w.x = *(uint32_t*)&a0; w.y = *(uint32_t*)&a1; w.z = *(uint32_t*)&a2; w.w = *(uint32_t*)&a3;
                        *(uint4*)(o_row + c * 32 + i) = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(AT_TMEM_COLS) : "memory");
    }
}

static int encode_2d(CUtensorMap* map, const void* ptr, uint64_t cols, uint64_t rows, uint32_t box_rows, const char* what) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                                              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) HB_REFUSE("attention_prefill_tcgen05: cuTensorMapEncodeTiled failed with %d for %s", (int)r, what);
    return 0;
}

HB_DEFINE_STATUS_MIRROR(hb_attention_tcgen05_status_mirror)
extern "C" int hb_attention_tcgen05_status(unsigned int* status) {
    HB_CUDA(cudaDeviceSynchronize());
    HB_CUDA(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(unsigned int)));
    const unsigned int zero = 0;
    HB_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(unsigned int)));
    return 0;
}

// Rows row0 .. rows - 1 of the batch; q_tiles is the sum of ceil(queries / tile_q) over them; tokens the step's token
// count. tile_q: 256 (both groups of a CTA at work) or 128 (one group: twice the CTAs, for steps whose tiles of 256
// would leave SMs idle).
extern "C" int hb_attention_prefill_tcgen05(void* out, const void* q, const void* kv, const int32_t* block_table,
                                            int table_stride, const int32_t* row_slot, const int32_t* query_start,
                                            const int32_t* kv_len, int row0, int rows, int q_tiles, int tokens, int heads,
                                            int kv_heads, int head_dim, int pages, int page_size, float scale, int window,
                                            int tile_q, hb_stream stream) {
    if (rows <= row0 || q_tiles == 0) return 0;
    if (tile_q != AT_BM && tile_q != AT_GROUPS * AT_BM) HB_REFUSE("attention_prefill_tcgen05: query tiles of %d (128 or 256)", tile_q);
    if (head_dim != AT_D) HB_REFUSE("attention_prefill_tcgen05: head_dim %d; this kernel is for %d", head_dim, AT_D);
    if (page_size % AT_BN) HB_REFUSE("attention_prefill_tcgen05: page size %d is no multiple of %d", page_size, AT_BN);
    if (kv_heads < 1 || heads % kv_heads) HB_REFUSE("attention_prefill_tcgen05: %d heads, %d kv heads", heads, kv_heads);
    if (q_tiles > 65535) HB_REFUSE("attention_prefill_tcgen05: %d query tiles in one step, above 65535", q_tiles);
    if (!(scale > 0.f)) HB_REFUSE("attention_prefill_tcgen05: the score scale must be positive");
    if ((((uintptr_t)q | (uintptr_t)kv | (uintptr_t)out) % 16) != 0) HB_REFUSE("attention_prefill_tcgen05: pointers must be 16-byte aligned");
    const uint64_t kv_rows = (uint64_t)pages * 2 * kv_heads * page_size;
    if (kv_rows > 0x7fffffffull) HB_REFUSE("attention_prefill_tcgen05: the cache has %llu rows, above 2^31", (unsigned long long)kv_rows);
    CUtensorMap map_q, map_kv;
    int rc = encode_2d(&map_q, q, (uint64_t)heads * AT_D, (uint64_t)tokens, AT_BM, "q");
    if (rc) return rc;
    rc = encode_2d(&map_kv, kv, AT_D, kv_rows, AT_BN, "the cache");
    if (rc) return rc;
    HB_CUDA(cudaFuncSetAttribute(prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM));
    prefill_tcgen05_kernel<<<dim3(heads, q_tiles), AT_THREADS, AT_SMEM, (cudaStream_t)stream>>>(
        map_q, map_kv, (bf16*)out, block_table, table_stride, row_slot, query_start, kv_len, row0, rows, heads, kv_heads,
        pages, page_size, scale * 1.4426950408889634f, window, tile_q);
    HB_LAUNCH_CHECK("attention_prefill_tcgen05");
    return 0;
}
