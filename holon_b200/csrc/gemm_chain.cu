// A chain of weight-streaming products in ONE persistent kernel, for the few rows of a decode step.
//
// A decode layer multiplies the same few rows by four weights one after the other (the mixer's last product, the
// feed-forward's two, the next mixer's first). As separate kernels each of them starts with an empty memory pipeline,
// ends in a tail, and cuts its weight into whole tiles that do not divide evenly among the SMs; at 10 to 40 us a
// product that costs a fifth to a third of its time. Here the products are phases of one kernel:
//
// - One CTA per SM stays for all phases (a cooperative launch: the CTAs wait for one another).
// - A phase's work is its weight cut into chunks of 16 rows x 256 columns (mode 1: 16 gate and 16 up rows). CTA c takes
//   the chunks [c C / G, (c + 1) C / G) of the C chunks in row-major order: every CTA streams the same number of bytes,
//   whatever the weight's shape. A tile (16 rows, all columns) that lies in several CTAs' ranges is summed by the CTA
//   that holds its first chunk: the others leave their partial sums in scratch memory and raise a flag; since a CTA
//   walks its range in ascending order, those partial sums were the first thing their CTAs did in the phase, and the
//   summing CTA reaches the tile last, so it all but never waits. The sum's order is fixed (ascending columns).
// - The weights come through a ring of shared-memory stages (a chunk of 16 rows x 512 bytes a stage), filled by four
//   producer warps with asynchronous 16-byte copies (cp.async, a row a warp instruction, completion counted on an
//   mbarrier; pieces past the weight's edge are written as zeros) as far ahead as the ring has room: 160 KB a CTA in
//   flight or waiting, whatever the consumers do. (The copy unit was tried first and cannot stream from DRAM at this
//   rate: TMA tile loads of a stage each gave 2.3 TB/s over all SMs whatever the ring's depth and even with consumers
//   that did nothing, sixteen bulk copies of 512 bytes a stage 1.2 TB/s; what it can keep in flight per SM is too
//   little for HBM's latency. Loads through the LSU are not so bounded.) The producer walks the CTA's chunks of ALL
//   phases without ever waiting for a phase to end: weights do not depend on what the phases compute. So the memory
//   pipeline stays full across tiles, across the barriers between phases and across products.
// - Eight consumer warps take the stages in turn (warp w the w-th, (w + 8)-th, ... chunk of a piece): a stage's 16
//   rows are the M side of mma.sync m16n8k16, every lane reads 16-byte pieces straight into A fragments, k permuted
//   the same way on both operands (as in gemm_skinny.cu), the few rows of x come from global memory as the N side
//   (a CTA meets each column of x once or twice only, so mostly from the L2; asked for a chunk ahead), and the 8
//   warps' partial sums are added through shared memory in a fixed order. Between phases the consumers pass a grid
//   barrier (a counter and a generation word in global memory): the next phase reads what this one wrote.
//
// Epilogues: mode 0 plain (bfloat16 or float32), mode 1 SwiGLU, mode 3 residual sum + next norm's weight + partial
// sums of squares; any mode scales its sums by the row scale its input still lacks (ss_in), as in gemm_skinny.cu.
//
// Measured (a layer's four products at Qwen3-8B sizes, 386 MB of weights, 8 rows, L2 replaced before): 102 us as one
// kernel against 89 us as four launches of gemm_skinny.cu (59 us is the weights at the copy bandwidth). The ring itself
// streams at HBM's pace (0.185 us a stage and SM); what is lost is about 10 us a phase around it: with one CTA an SM
// nothing streams for a CTA while its consumers sum a tile over warps and CTAs and write it out (two or three pieces a
// phase, each a chain of L2 round trips), and after a barrier the first x comes from the L2 before anything moves. The
// separate kernels hide the same work behind the other CTAs of the SM. And x: a CTA meets each column once or twice, and
// beside the ring the L1 has some 40 KB, so every chunk's rows of x come from the L2 (0.167 us a stage at 1 row, 0.185
// at 8, 0.26 at 16), where the separate kernels read x from the L1. So the kernel table queues products for this
// kernel only when asked to (HOLON_B200_CHAIN=1); the default stays a launch a product.
//
// Every wait (ring, barrier, flag) is bounded: after half a second the thread records the place (5: ring stage
// to fill, 4: ring stage to read, 6: barrier, 7: flag) in the status word and its host mirror (tcgen05.cuh); from then
// on nothing in the CTA waits any more, it lets its copies land and runs to its end.
#include "skinny.cuh"
#include "tcgen05.cuh"

#define CH_WARPS 8                               // consumer warps
#define CH_PRODUCERS 4                           // warps that feed the ring, each a stage in four (a power of two)
#define CH_CONSUMERS (CH_WARPS * 32)
#define CH_THREADS (CH_CONSUMERS + CH_PRODUCERS * 32)
#define CH_MAX_PHASES 8
#define CH_SCRATCH_FLOATS 512                    // per CTA: 32 rows x 16 tokens
#define CH_ROW_BYTES 576                         // a row's 256 columns (512 bytes) + 64: 16-byte reads of a quarter warp
#define CH_STAGE_BYTES (16 * CH_ROW_BYTES)       // (two rows, four pieces) then fall into 32 different banks
#define CH_STAGES 20
// A wait for a stage tells "filled" from "not yet" by one bit of the count of its fillings, so no waiter may be a whole
// turn of the ring behind what it waits for. That holds because a consumer warp's stages (8 or, with two stages a chunk,
// 16 apart) and the stage that held its ring slot before (CH_STAGES back) are all filled by the same producer warp, in
// order, and a producer thread's arrival at a stage's barrier comes only when all its earlier copies have landed too.
static_assert((CH_PRODUCERS & (CH_PRODUCERS - 1)) == 0 && CH_STAGES % CH_PRODUCERS == 0, "producer warps take stages in turn");
static_assert((CH_STAGES - CH_WARPS) % CH_PRODUCERS == 0 && CH_STAGES > 2 * CH_WARPS, "see above");
#define CH_DYNAMIC_SMEM (CH_STAGES * CH_STAGE_BYTES + 2 * CH_STAGES * 8 + 128)

struct ChainPhase {                              // (the host fills the same layout: hb_chain_phase in api.h)
    const bf16* w;                               // [n, k] (mode 1: [2 inter, k], gate rows first)
    const bf16* x;                               // [m, k]
    void* out;                                   // mode 0: [m, n]; mode 1: [m, inter]; mode 3: [m, n] bfloat16
    float* h;                                    // mode 3: [m, n] 32-bit stream, added into
    const void* next_weight;                     // mode 3: the next norm's weight [n]
    float* ss_out;                               // mode 3: [tiles, 16]
    const float* ss_in;                          // [parts_in, 16] or null
    int n, k, mode, inter, out_f32, next_weight_f32, parts_in, dim_in;
    float next_offset, eps_in;
    int tiles, chunks;                           // tiles of 16 output columns; 256-wide k chunks a tile
};

struct ChainArgs {
    ChainPhase phase[CH_MAX_PHASES];
    int phases, m;
    unsigned int* sync;                          // [0] arrivals at the current barrier, [1] generation
    float* scratch;                              // [ctas, CH_SCRATCH_FLOATS]
    unsigned int* flags;                         // [ctas]
};

struct Seg { int p, tile, c0, c1; };             // chunks c0 .. c1 - 1 of `tile` in phase p; p < 0: none

__device__ __forceinline__ uint4 ld_plain16(const void* p, bool valid) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);        // written earlier in this kernel by other CTAs: no read-only path
    if (valid) asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ long long chain_lo(const ChainPhase& ph, int cta, int ctas) {
    return (long long)cta * ((long long)ph.tiles * ph.chunks) / ctas;
}

// The first piece of work of CTA `cta` in phase `p` or a later one.
__device__ __forceinline__ Seg chain_first(const ChainArgs& a, int cta, int ctas, int p) {
    for (; p < a.phases; ++p) {
        const ChainPhase& ph = a.phase[p];
        const long long lo = chain_lo(ph, cta, ctas), hi = chain_lo(ph, cta + 1, ctas);
        if (lo < hi) {
            const int tile = (int)(lo / ph.chunks), c0 = (int)(lo % ph.chunks);
            const long long room = hi - lo;
            return Seg{p, tile, c0, (int)(room < ph.chunks - c0 ? c0 + room : ph.chunks)};
        }
    }
    return Seg{-1, 0, 0, 0};
}
__device__ __forceinline__ Seg chain_next(const ChainArgs& a, int cta, int ctas, const Seg& s) {
    const ChainPhase& ph = a.phase[s.p];
    const long long at = (long long)s.tile * ph.chunks + s.c1, hi = chain_lo(ph, cta + 1, ctas);
    if (at < hi) {                               // (a piece ends at its tile's end or at the range's: here the tile's)
        const long long room = hi - at;
        return Seg{s.p, s.tile + 1, 0, (int)(room < ph.chunks ? room : ph.chunks)};
    }
    return chain_first(a, cta, ctas, s.p + 1);
}

// 16 bytes from global to shared memory without a register in between; `bytes` 0: zeros, nothing is read.
__device__ __forceinline__ void copy_async16(uint32_t dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
// This thread's arrival at `bar`, made when all its copies asked for so far have landed.
__device__ __forceinline__ void copies_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(CH_CONSUMERS) : "memory"); }
__device__ __forceinline__ uint4 ld_shared16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
#define CH_WAIT_NS 500000000ull                  // half a second: no wait in this kernel is meant to last a millisecond

__device__ __forceinline__ unsigned long long chain_clock() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    return t;
}
// A wait for an mbarrier's phase, bounded in time, and skipped once any wait of the CTA has given up.
__device__ __forceinline__ void ring_wait(uint32_t bar, uint32_t parity, unsigned place, volatile int* gave_up) {
    unsigned long long began = 0;
    for (unsigned int spin = 0;; ++spin) {
        uint32_t done;
        // (test_wait, which never suspends the thread: a thread that try_wait has put to sleep is woken late, and a
        // producer that meets a full ring at every stage then fills one stage per such nap, whatever the ring's depth)
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return;
        if ((spin & 63u) == 63u) {
            if (*gave_up) return;
            const unsigned long long now = chain_clock();
            if (began == 0) began = now;
            else if (now - began > CH_WAIT_NS) break;
        }
    }
    tc_give_up(place);
    *gave_up = 1;
}
// The same for a word in global memory that another CTA writes: until `*word != unlike` (returns false if it gave up).
__device__ __forceinline__ bool word_wait(const unsigned int* word, unsigned int unlike, unsigned place, volatile int* gave_up) {
    unsigned long long began = 0;
    for (unsigned int spin = 0;; ++spin) {
        if (ld_acquire_u32(word) != unlike) return true;
        if ((spin & 63u) == 63u) {
            const unsigned long long now = chain_clock();
            if (began == 0) began = now;
            else if (now - began > CH_WAIT_NS) break;
        }
    }
    tc_give_up(place);
    *gave_up = 1;
    return false;
}

template <int NT>
__global__ void __launch_bounds__(CH_THREADS, 1) gemm_chain_kernel(const ChainArgs a) {
    extern __shared__ unsigned char ring[];                            // CH_STAGES stages, then their barriers
    __shared__ float red[CH_WARPS][32][NT * 8 + 1];
    __shared__ float total[32][NT * 8 + 1];
    __shared__ float scale_part[16][17];
    __shared__ float scale_in[16];
    __shared__ int gave_up_s;                        // a wait ran out: wait no more in this launch
    volatile int* gave_up = &gave_up_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = lane >> 2, c = lane & 3;
    const int cta = blockIdx.x, ctas = gridDim.x, m = a.m;
    const uint32_t ring0 = (smem_addr(ring) + 127u) & ~127u;
    const uint32_t full0 = ring0 + CH_STAGES * CH_STAGE_BYTES, empty0 = full0 + CH_STAGES * 8;
    if (threadIdx.x == 0) {
        gave_up_s = 0;
        for (int i = 0; i < CH_STAGES; ++i) {
            mbar_init(full0 + i * 8, 32);            // every thread of the stage's producer warp, when its copies have landed
            mbar_init(empty0 + i * 8, 1);            // the consumer warp that took the stage, when it has read it
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    if (warp >= CH_WARPS) {
        // ---- the producers: this CTA's chunks of every phase, as far ahead as the ring has room. Producer warp p fills
        // the stages p, p + 4, ... whole, sixteen rows each: a lone warp issues an instruction every few cycles at best,
        // so what a stage costs in instructions bounds the kernel (with one warp working out eight row addresses a
        // stage, a stage took 1,400 cycles); four warps on four stages at once, a row an add and a copy, keep ahead.
        const int p = warp - CH_WARPS;
        unsigned int before = 0;                                         // stages of the pieces before this one
        for (Seg s = chain_first(a, cta, ctas, 0); s.p >= 0 && !*gave_up; s = chain_next(a, cta, ctas, s)) {
            const ChainPhase& ph = a.phase[s.p];
            const int two = ph.mode == 1 ? 1 : 0, k = ph.k;
            const unsigned int stages = (unsigned int)(s.c1 - s.c0) << two;
            for (unsigned int q = (unsigned int)(p - (int)before) & (CH_PRODUCERS - 1); q < stages; q += CH_PRODUCERS) {
                const unsigned int it = before + q;
                const int j = s.c0 + (int)(q >> two), half = two ? (int)(q & 1u) : 0;
                const uint32_t stage = it % CH_STAGES, parity = (it / CH_STAGES) & 1u;
                if (lane == 0) ring_wait(empty0 + stage * 8, parity ^ 1u, 5u, gave_up);
                __syncwarp();
                const int first = (half ? ph.inter : 0) + s.tile * 16;
                const int limit = two ? (half ? 2 * ph.inter : ph.inter) : ph.n;
                const int rows = limit - first;                          // (16 or more: all of them)
                const int k0 = (j << 8) + lane * 8;
                const bool kok = k0 < k;
                const bf16* src = ph.w + (size_t)first * k + k0;
                const uint32_t dst = ring0 + stage * CH_STAGE_BYTES + lane * 16;
#pragma unroll
                for (int row = 0; row < 16; ++row) {
                    const bool ok = kok && row < rows;
                    copy_async16(dst + row * CH_ROW_BYTES, ok ? src : ph.w, ok ? 16u : 0u);
                    src += k;
                }
                copies_arrive(full0 + stage * 8);
            }
            before += stages;
        }
        asm volatile("cp.async.wait_all;\n" ::: "memory");
    } else {
        // ---- the consumers
        unsigned int it = 0;
        int phase_now = 0, phase_set = -1;
        auto barrier = [&]() {                       // all CTAs have finished phase `phase_now`
            consumer_sync();
            if (threadIdx.x == 0 && !*gave_up) {
                const unsigned int generation = ld_acquire_u32(a.sync + 1);
                __threadfence();
                if (atomicAdd(a.sync, 1u) == (unsigned int)ctas - 1) {
                    atomicExch(a.sync, 0u);
                    __threadfence();
                    atomicAdd(a.sync + 1, 1u);
                } else {
                    word_wait(a.sync + 1, generation, 6u, gave_up);
                }
                __threadfence();
            }
            consumer_sync();
            ++phase_now;
        };
        for (Seg cur = chain_first(a, cta, ctas, 0); cur.p >= 0; cur = chain_next(a, cta, ctas, cur)) {
            while (phase_now < cur.p) barrier();
            const ChainPhase& ph = a.phase[cur.p];
            if (phase_set != cur.p) {                // the row scale that this phase's x still lacks
                float mine = 0.f;                    // token (thread & 15): every 16th partial sum, in ascending order
                if (ph.ss_in)
                    for (int p2 = threadIdx.x >> 4; p2 < ph.parts_in; p2 += 16) mine += ph.ss_in[p2 * 16 + (threadIdx.x & 15)];
                scale_part[threadIdx.x >> 4][threadIdx.x & 15] = mine;
                consumer_sync();
                if (threadIdx.x < 16) {
                    float sum = 0.f;
#pragma unroll
                    for (int j = 0; j < 16; ++j) sum += scale_part[j][threadIdx.x];
                    scale_in[threadIdx.x] = ph.ss_in ? rsqrtf(sum / (float)ph.dim_in + ph.eps_in) : 1.f;
                }
                consumer_sync();
                phase_set = cur.p;
            }
            float acc[2][NT][4];
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int b = 0; b < NT; ++b) acc[t][b][0] = acc[t][b][1] = acc[t][b][2] = acc[t][b][3] = 0.f;
            const int halves = ph.mode == 1 ? 2 : 1;
            const bf16* xp[NT];
            bool xok[NT];
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                xok[t] = t * 8 + r < m;
                xp[t] = ph.x + (size_t)(xok[t] ? t * 8 + r : 0) * ph.k + c * 8;
            }
            // Warp w takes the piece's chunks w, w + 8, ... whole: eight warps on eight stages at a time (with all of
            // them on the same stage, a stage's wait, reads, steps and release were one dependent chain of 330 cycles).
            // Its rows of x for a chunk come from global memory, mostly from the L2 (a CTA meets each column of x once
            // or twice only); they are asked for one chunk of its own ahead (two ahead changed
            // nothing).
            uint4 xa[CH_WARPS][NT], xb[CH_WARPS][NT];
            float odd[2][NT][4];                     // the odd k blocks' sums: two chains of tensor-core steps, not one
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int b = 0; b < NT; ++b) odd[t][b][0] = odd[t][b][1] = odd[t][b][2] = odd[t][b][3] = 0.f;
            auto ask = [&](uint4 (&dst)[CH_WARPS][NT], int j) {
#pragma unroll
                for (int u = 0; u < CH_WARPS; ++u) {
                    const int k0 = (j * CH_WARPS + u) << 5;
#pragma unroll
                    for (int t = 0; t < NT; ++t) dst[u][t] = ld_plain16(xp[t] + k0, xok[t] && j < cur.c1 && k0 + c * 8 < ph.k);
                }
            };
            ask(xa, cur.c0 + warp);
            for (int j = cur.c0 + warp; j < cur.c1; j += CH_WARPS) {
                ask(xb, j + CH_WARPS);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (half < halves) {
                        const unsigned int mine = it + (unsigned int)((j - cur.c0) * halves + half);
                        const uint32_t stage = mine % CH_STAGES, parity = (mine / CH_STAGES) & 1u;
                        ring_wait(full0 + stage * 8, parity, 4u, gave_up);
                        const uint32_t at = ring0 + stage * CH_STAGE_BYTES + r * CH_ROW_BYTES + c * 16;
#pragma unroll
                        for (int u = 0; u < CH_WARPS; ++u) {
                            const uint4 lo = ld_shared16(at + u * 64), hi = ld_shared16(at + u * 64 + 8 * CH_ROW_BYTES);
#pragma unroll
                            for (int b = 0; b < NT; ++b) {
                                float (&sum)[4] = (u & 1) ? odd[half][b] : acc[half][b];
                                mma16816(sum, lo.x, hi.x, lo.y, hi.y, xa[u][b].x, xa[u][b].y);
                                mma16816(sum, lo.z, hi.z, lo.w, hi.w, xa[u][b].z, xa[u][b].w);
                            }
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty0 + stage * 8);
                    }
                }
#pragma unroll
                for (int u = 0; u < CH_WARPS; ++u)
#pragma unroll
                    for (int t = 0; t < NT; ++t) xa[u][t] = xb[u][t];
            }
            it += (unsigned int)((cur.c1 - cur.c0) * halves);
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int b = 0; b < NT; ++b)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[t][b][e] += odd[t][b][e];

            // ---- the piece's sums over the 8 warps, then over the CTAs that share the tile
            const int tile_rows = ph.mode == 1 ? 32 : 16;
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int b = 0; b < NT; ++b) {
                    red[warp][t * 16 + r][b * 8 + c * 2] = acc[t][b][0];
                    red[warp][t * 16 + r][b * 8 + c * 2 + 1] = acc[t][b][1];
                    red[warp][t * 16 + r + 8][b * 8 + c * 2] = acc[t][b][2];
                    red[warp][t * 16 + r + 8][b * 8 + c * 2 + 1] = acc[t][b][3];
                }
            consumer_sync();
            const bool whole = cur.c0 == 0 && cur.c1 == ph.chunks, summing = cur.c0 == 0;
            const long long tile_end = (long long)(cur.tile + 1) * ph.chunks;
            if (!whole && summing) {                 // wait for the CTAs that hold the rest of this tile
                if (threadIdx.x == 0)
                    for (int other = cta + 1; other < ctas && chain_lo(ph, other, ctas) < tile_end && !*gave_up; ++other) {
                        if (chain_lo(ph, other, ctas) == chain_lo(ph, other + 1, ctas)) continue;   // (it has no chunk at all)
                        word_wait(a.flags + other, 0u, 7u, gave_up);
                    }
                consumer_sync();
            }
            for (int i = threadIdx.x; i < tile_rows * (NT * 8); i += CH_CONSUMERS) {
                const int rr = i / (NT * 8), tok = i % (NT * 8);
                float v = 0.f;
#pragma unroll
                for (int wv = 0; wv < CH_WARPS; ++wv) v += red[wv][rr][tok];
                if (!whole && summing) {
                    for (int other = cta + 1; other < ctas && chain_lo(ph, other, ctas) < tile_end; ++other)
                        if (chain_lo(ph, other, ctas) < chain_lo(ph, other + 1, ctas))
                            v += __ldcg(a.scratch + (size_t)other * CH_SCRATCH_FLOATS + rr * 16 + tok);
                } else if (!whole) {
                    a.scratch[(size_t)cta * CH_SCRATCH_FLOATS + rr * 16 + tok] = v;
                }
                total[rr][tok] = v;
            }
            if (!whole && !summing) {                // this CTA's share of a tile that another CTA sums: hand it over
                __threadfence();
                consumer_sync();
                if (threadIdx.x == 0) st_release_u32(a.flags + cta, 1u);
            } else {
                consumer_sync();
                if (!whole && threadIdx.x == 0)      // the flags go down again for their CTAs' next use, a phase later
                    for (int other = cta + 1; other < ctas && chain_lo(ph, other, ctas) < tile_end; ++other)
                        if (chain_lo(ph, other, ctas) < chain_lo(ph, other + 1, ctas)) a.flags[other] = 0u;
                // ---- the tile's epilogue
                if (ph.mode == 3) {                  // 16 columns x up to 16 tokens: one thread each
                    const int rr = threadIdx.x & 15, tok = threadIdx.x >> 4, col = cur.tile * 16 + rr;
                    const bool live = tok < m && col < ph.n;
                    float hn = 0.f;
                    if (live) {
                        const float before = ph.h[(size_t)tok * ph.n + col];
                        const float wn = ph.next_weight_f32 ? ((const float*)ph.next_weight)[col] : to_f32(((const bf16*)ph.next_weight)[col]);
                        hn = before + rounded<bf16>(total[rr][tok] * scale_in[tok]);
                        ph.h[(size_t)tok * ph.n + col] = hn;
                        ((bf16*)ph.out)[(size_t)tok * ph.n + col] = __float2bfloat16_rn(hn * (wn + ph.next_offset));
                    }
                    float sq = hn * hn;              // over the token's 16 columns: lanes 0-15 or 16-31
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                    if (rr == 0) ph.ss_out[cur.tile * 16 + tok] = sq;
                } else {
                    const int width = ph.mode == 1 ? ph.inter : ph.n;
                    for (int i = threadIdx.x; i < 16 * m; i += CH_CONSUMERS) {
                        const int rr = i & 15, tok = i >> 4, col = cur.tile * 16 + rr;
                        float v = total[rr][tok] * scale_in[tok];
                        if (ph.mode == 1) v = v / (1.f + expf(-v)) * (total[16 + rr][tok] * scale_in[tok]);
                        if (col < width) {
                            if (ph.out_f32) ((float*)ph.out)[(size_t)tok * width + col] = v;
                            else ((bf16*)ph.out)[(size_t)tok * width + col] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
        }
        while (phase_now < a.phases - 1) barrier();
    }
    __syncthreads();
    if (*gave_up)                                    // copies that nobody waited for may still be on their way: let them land
        for (int i = 0; i < 50; ++i) __nanosleep(10000);
}

HB_DEFINE_STATUS_MIRROR(hb_gemm_chain_status_mirror)

extern "C" int hb_gemm_chain_status(unsigned int* status) {
    HB_CUDA(cudaDeviceSynchronize());
    HB_CUDA(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(unsigned int)));
    const unsigned int zero = 0;
    HB_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(unsigned int)));
    return 0;
}

// CTAs of the chain kernel that the current device runs at once (the most a launch may have).
extern "C" int hb_gemm_chain_capacity(void) {
    static int capacity = 0;
    if (capacity == 0) {
        int device = 0, sms = 0, one = 0, two = 0;
        if (cudaGetDevice(&device) != cudaSuccess) return 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
        if (cudaFuncSetAttribute(gemm_chain_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, CH_DYNAMIC_SMEM) != cudaSuccess) return 0;
        if (cudaFuncSetAttribute(gemm_chain_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, CH_DYNAMIC_SMEM) != cudaSuccess) return 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&one, gemm_chain_kernel<1>, CH_THREADS, CH_DYNAMIC_SMEM) != cudaSuccess) return 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&two, gemm_chain_kernel<2>, CH_THREADS, CH_DYNAMIC_SMEM) != cudaSuccess) return 0;
        capacity = sms * (one < two ? one : two);
    }
    return capacity;
}

// Runs `n_phases` products one after the other in one kernel (see the top of this file). phases[i] as in api.h;
// m rows, 1 to 16. sync: two words, zero before the first launch and left alone afterwards; scratch: `slots` x 512
// floats; flags: `slots` words, zero before the first launch. The launch has min(slots, hb_gemm_chain_capacity(), the
// largest phase's chunks) CTAs and is cooperative.
extern "C" int hb_gemm_chain(const hb_chain_phase* phases, int n_phases, int m, unsigned int* sync, float* scratch,
                             unsigned int* flags, int slots, int cooperative, hb_stream stream) {
    if (m == 0 || n_phases == 0) return 0;
    if (m < 0 || m > 16) HB_REFUSE("gemm_chain: %d rows; this kernel takes 1 to 16", m);
    if (n_phases < 0 || n_phases > CH_MAX_PHASES) HB_REFUSE("gemm_chain: %d phases; up to %d", n_phases, CH_MAX_PHASES);
    if (!sync || !scratch || !flags || slots < 1) HB_REFUSE("gemm_chain: sync, scratch and flags are needed");
    ChainArgs args = {};
    long long most = 1;
    for (int i = 0; i < n_phases; ++i) {
        const hb_chain_phase& p = phases[i];
        if (p.k < 8 || p.k % 8) HB_REFUSE("gemm_chain: phase %d: k = %d is no multiple of 8", i, p.k);
        if (p.mode != 0 && p.mode != 1 && p.mode != 3) HB_REFUSE("gemm_chain: phase %d: mode %d", i, p.mode);
        if ((((uintptr_t)p.out | (uintptr_t)p.x | (uintptr_t)p.w) % 16) != 0 || !p.out || !p.x || !p.w)
            HB_REFUSE("gemm_chain: phase %d: pointers must be given and 16-byte aligned", i);
        if (p.mode == 1 ? p.inter < 1 : p.n < 1) HB_REFUSE("gemm_chain: phase %d: n = %d, inter = %d", i, p.n, p.inter);
        if (p.mode == 3 && (!p.h || !p.next_weight || !p.ss_out || p.out_f32))
            HB_REFUSE("gemm_chain: phase %d: mode 3 needs h, the next norm's weight and ss_out, and writes bfloat16", i);
        if (p.mode == 1 && p.out_f32) HB_REFUSE("gemm_chain: phase %d: mode 1 writes bfloat16", i);
        if (p.ss_in && (p.parts_in < 1 || p.dim_in < 1)) HB_REFUSE("gemm_chain: phase %d: %d partial sums over %d columns", i, p.parts_in, p.dim_in);
        ChainPhase& q = args.phase[i];
        q.w = (const bf16*)p.w; q.x = (const bf16*)p.x; q.out = p.out; q.h = p.h; q.next_weight = p.next_weight;
        q.ss_out = p.ss_out; q.ss_in = p.ss_in; q.n = p.n; q.k = p.k; q.mode = p.mode; q.inter = p.inter; q.out_f32 = p.out_f32;
        q.next_weight_f32 = p.next_weight_f32; q.parts_in = p.parts_in; q.dim_in = p.dim_in; q.next_offset = p.next_offset;
        q.eps_in = p.eps_in;
        q.tiles = ((p.mode == 1 ? p.inter : p.n) + 15) / 16;
        q.chunks = (((p.k + 31) >> 5) + CH_WARPS - 1) / CH_WARPS;
        const long long all = (long long)q.tiles * q.chunks;
        most = all > most ? all : most;
    }
    args.phases = n_phases; args.m = m; args.sync = sync; args.scratch = scratch; args.flags = flags;



    const int capacity = hb_gemm_chain_capacity();
    if (capacity < 1) HB_REFUSE("gemm_chain: the device runs no CTA of this kernel");
    long long ctas = capacity < slots ? capacity : slots;
    ctas = most < ctas ? most : ctas;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned int)ctas);
    cfg.blockDim = dim3(CH_THREADS);
    cfg.dynamicSmemBytes = CH_DYNAMIC_SMEM;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeCooperative;
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = cooperative ? 1 : 0;
    if (m <= 8) HB_CUDA(cudaLaunchKernelEx(&cfg, gemm_chain_kernel<1>, args));
    else HB_CUDA(cudaLaunchKernelEx(&cfg, gemm_chain_kernel<2>, args));
    return 0;
}
