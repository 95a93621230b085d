// Several weight-streaming products of the same few rows in ONE launch, each CTA a tile of one of them, in order.
//
// The products of a decode layer follow one another on the same few rows (the mixer's last, the feed-forward's two,
// the next mixer's first): each needs what the one before wrote. As launches of their own, each starts when the one
// before has ended, with an empty memory pipeline. Here they are one grid. A CTA draws a ticket when it starts; the
// tickets 0 .. T0 - 1 are the tiles of the first product, the next T1 those of the second, and so on, so the CTAs of a
// product start as those of the product before leave their SMs, during its last wave. Such a CTA asks for the first
// weights of its tile at once (weights depend on nothing), then waits until a counter says that every tile of the
// product before is written, and goes on as gemm_skinny.cu's kernel does: the few rows of x from the L1, the tile's 16
// (or 16 + 16) rows of w as the M side of mma.sync m16n8k16, eight warps on interleaved k blocks, their sums added
// through shared memory in a fixed order, the same epilogues (mode 0 plain, mode 1 SwiGLU, mode 3 residual sum + next
// norm's weight + partial sums of squares; `ss_in` as there). So one product's start overlaps the other's end, inside
// one kernel, without a grid-wide barrier and without any CTA staying longer than its tile.
//
// A ticket is drawn with an atomic add, so whoever holds a lower one has started before: a CTA only ever waits for
// CTAs that run or have ended, never for one that has not been given an SM yet. The wait is bounded all the same (half
// a second; place 8 in the status word, tcgen05.cuh). The last CTA to end puts the counters back to zero.
#include "skinny.cuh"
#include "tcgen05.cuh"

#define TK_WARPS 8
#define TK_THREADS (TK_WARPS * 32)
#define TK_MAX_PHASES 4
#define TK_WAIT_NS 500000000ull

struct TicketPhase {
    const bf16* w; const bf16* x; void* out; float* h; const void* next_weight; float* ss_out; const float* ss_in;
    int n, k, mode, inter, out_f32, next_weight_f32, parts_in, dim_in;
    float next_offset, eps_in;
    int tiles, first;                            // tiles of 16 output columns; the first ticket of this product
};
struct TicketArgs {
    TicketPhase phase[TK_MAX_PHASES];
    int phases, m, total;
    unsigned int* state;                         // [0] tickets drawn, [1] CTAs ended, [2 + p] tiles of product p written
};

__device__ __forceinline__ uint4 tk_ld_plain16(const void* p, bool valid) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);        // (x may have been written by CTAs of this very launch: no read-only path)
    if (valid) asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned int tk_ld_acquire(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <int MT, int NT, int U>
__device__ __forceinline__ void ticket_tile(const TicketArgs& a, int p, int tile, float (*red)[32][NT * 8 + 1],
                                            float (*scale_part)[17], float* scale_in) {
    const TicketPhase& ph = a.phase[p];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = lane >> 2, c = lane & 3, m = a.m, k = ph.k;
    // ---- this tile's rows of w: asked for before anything else
    const bf16* wp[MT][2];
    bool wok[MT][2];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int base = ph.mode == 1 && t == 1 ? ph.inter : 0, limit = ph.mode == 1 ? base + ph.inter : ph.n;
            const int row = base + tile * 16 + r + 8 * h;
            wok[t][h] = row < limit;
            wp[t][h] = ph.w + (size_t)(wok[t][h] ? row : 0) * k + c * 8;
        }
    const int blocks = (k + 31) >> 5;                    // 32-wide k blocks; warp w takes w, w + 8, ...
    uint4 wr[U][MT][2];
    auto ask = [&](int kb) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k0 = (kb + u * TK_WARPS) << 5;
            const bool kok = k0 + c * 8 < k;
#pragma unroll
            for (int t = 0; t < MT; ++t)
#pragma unroll
                for (int h = 0; h < 2; ++h) wr[u][t][h] = ld_stream16(wp[t][h] + k0, kok && wok[t][h]);
        }
    };
    int kb = warp;
    if (kb < blocks) ask(kb);

    // ---- every tile of the product before must be written before its rows (and the stream) are read
    if (p > 0) {
        if (threadIdx.x == 0) {
            const unsigned int all = (unsigned int)a.phase[p - 1].tiles;
            unsigned long long began = 0;
            for (unsigned int spin = 0; tk_ld_acquire(a.state + 2 + (p - 1)) < all; ++spin)
                if ((spin & 63u) == 63u) {
                    unsigned long long now;
                    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(now));
                    if (began == 0) began = now;
                    else if (now - began > TK_WAIT_NS) { tc_give_up(8u); break; }
                }
            __threadfence();
        }
        __syncthreads();
    }
    float mine = 0.f;                                    // token (thread & 15): every 16th partial sum, in ascending order
    if (ph.ss_in)
        for (int p2 = threadIdx.x >> 4; p2 < ph.parts_in; p2 += 16) mine += ph.ss_in[p2 * 16 + (threadIdx.x & 15)];
    scale_part[threadIdx.x >> 4][threadIdx.x & 15] = mine;

    const bf16* xp[NT];
    bool xok[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        xok[t] = t * 8 + r < m;
        xp[t] = ph.x + (size_t)(xok[t] ? t * 8 + r : 0) * k + c * 8;
    }
    float acc[MT][NT][4];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int b = 0; b < NT; ++b) acc[t][b][0] = acc[t][b][1] = acc[t][b][2] = acc[t][b][3] = 0.f;
    constexpr int G = U * NT > 8 ? U / 2 : U;            // k blocks whose rows of x are held at a time (registers)
    while (kb < blocks) {
#pragma unroll
        for (int g = 0; g < U; g += G) {
            uint4 xr[G][NT];
#pragma unroll
            for (int u = 0; u < G; ++u) {
                const int k0 = (kb + (g + u) * TK_WARPS) << 5;
#pragma unroll
                for (int t = 0; t < NT; ++t) xr[u][t] = tk_ld_plain16(xp[t] + k0, xok[t] && k0 + c * 8 < k);
            }
#pragma unroll
            for (int u = 0; u < G; ++u)
#pragma unroll
                for (int t = 0; t < MT; ++t)
#pragma unroll
                    for (int b = 0; b < NT; ++b) {
                        mma16816(acc[t][b], wr[g + u][t][0].x, wr[g + u][t][1].x, wr[g + u][t][0].y, wr[g + u][t][1].y, xr[u][b].x, xr[u][b].y);
                        mma16816(acc[t][b], wr[g + u][t][0].z, wr[g + u][t][1].z, wr[g + u][t][0].w, wr[g + u][t][1].w, xr[u][b].z, xr[u][b].w);
                    }
        }
        kb += TK_WARPS * U;
        if (kb < blocks) ask(kb);
    }
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int b = 0; b < NT; ++b) {
            red[warp][t * 16 + r][b * 8 + c * 2] = acc[t][b][0];
            red[warp][t * 16 + r][b * 8 + c * 2 + 1] = acc[t][b][1];
            red[warp][t * 16 + r + 8][b * 8 + c * 2] = acc[t][b][2];
            red[warp][t * 16 + r + 8][b * 8 + c * 2 + 1] = acc[t][b][3];
        }
    __syncthreads();
    if (threadIdx.x < 16) {
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) sum += scale_part[j][threadIdx.x];
        scale_in[threadIdx.x] = ph.ss_in ? rsqrtf(sum / (float)ph.dim_in + ph.eps_in) : 1.f;
    }
    __syncthreads();
    if (ph.mode == 3) {                                  // 16 columns x up to 16 tokens: one thread each
        const int rr = threadIdx.x & 15, tok = threadIdx.x >> 4, col = tile * 16 + rr;
        const bool live = tok < m && col < ph.n;
        float hn = 0.f;
        if (live) {
            const float before = ph.h[(size_t)tok * ph.n + col];
            const float wn = ph.next_weight_f32 ? ((const float*)ph.next_weight)[col] : to_f32(((const bf16*)ph.next_weight)[col]);
            float v = 0.f;
#pragma unroll
            for (int wv = 0; wv < TK_WARPS; ++wv) v += red[wv][rr][tok];
            hn = before + rounded<bf16>(v * scale_in[tok]);
            ph.h[(size_t)tok * ph.n + col] = hn;
            ((bf16*)ph.out)[(size_t)tok * ph.n + col] = __float2bfloat16_rn(hn * (wn + ph.next_offset));
        }
        float sq = hn * hn;                              // over the token's 16 columns: lanes 0-15 or 16-31
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (rr == 0) ph.ss_out[tile * 16 + tok] = sq;
    } else {
        const int width = ph.mode == 1 ? ph.inter : ph.n;
        for (int i = threadIdx.x; i < 16 * m; i += TK_THREADS) {
            const int rr = i & 15, tok = i >> 4, col = tile * 16 + rr;
            float v = 0.f;
#pragma unroll
            for (int wv = 0; wv < TK_WARPS; ++wv) v += red[wv][rr][tok];
            v *= scale_in[tok];
            if (MT == 2) {
                float u = 0.f;
#pragma unroll
                for (int wv = 0; wv < TK_WARPS; ++wv) u += red[wv][16 + rr][tok];
                v = v / (1.f + expf(-v)) * (u * scale_in[tok]);
            }
            if (col < width) {
                if (ph.out_f32) ((float*)ph.out)[(size_t)tok * width + col] = v;
                else ((bf16*)ph.out)[(size_t)tok * width + col] = __float2bfloat16_rn(v);
            }
        }
    }
}

template <int NT>
__global__ void __launch_bounds__(TK_THREADS, 2) gemm_tickets_kernel(const TicketArgs a) {
    __shared__ float red[TK_WARPS][32][NT * 8 + 1];
    __shared__ float scale_part[16][17];
    __shared__ float scale_in[16];
    __shared__ unsigned int ticket_s;
    if (threadIdx.x == 0) ticket_s = atomicAdd(a.state, 1u);
    __syncthreads();
    const int ticket = (int)ticket_s;
    int p = 0;
    while (p + 1 < a.phases && ticket >= a.phase[p + 1].first) ++p;
    const int tile = ticket - a.phase[p].first;
    if (ticket < a.total) {
        if (a.phase[p].mode == 1) ticket_tile<2, NT, 4>(a, p, tile, red, scale_part, scale_in);
        else ticket_tile<1, NT, 8>(a, p, tile, red, scale_part, scale_in);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (ticket < a.total) atomicAdd(a.state + 2 + p, 1u);
        if (atomicAdd(a.state + 1, 1u) == gridDim.x - 1) {           // the last one out: nobody reads the counters any more
            for (int i = 0; i < 2 + TK_MAX_PHASES; ++i) a.state[i] = 0u;
            __threadfence();
        }
    }
}

HB_DEFINE_STATUS_MIRROR(hb_gemm_tickets_status_mirror)

extern "C" int hb_gemm_tickets_status(unsigned int* status) {
    HB_CUDA(cudaDeviceSynchronize());
    HB_CUDA(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(unsigned int)));
    const unsigned int zero = 0;
    HB_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(unsigned int)));
    return 0;
}

// Runs up to 4 products one after the other in one launch (see the top of this file). phases[i] as for hb_gemm_chain;
// m rows, 1 to 16. state: 2 + 4 words, zero before the first launch and left alone afterwards (the kernel puts them
// back to zero when it ends); not to be shared with a launch that may run at the same time.
extern "C" int hb_gemm_tickets(const hb_chain_phase* phases, int n_phases, int m, unsigned int* state, hb_stream stream) {
    if (m == 0 || n_phases == 0) return 0;
    if (m < 0 || m > 16) HB_REFUSE("gemm_tickets: %d rows; this kernel takes 1 to 16", m);
    if (n_phases < 0 || n_phases > TK_MAX_PHASES) HB_REFUSE("gemm_tickets: %d products; up to %d", n_phases, TK_MAX_PHASES);
    if (!state) HB_REFUSE("gemm_tickets: the counters are needed");
    TicketArgs args = {};
    int total = 0;
    for (int i = 0; i < n_phases; ++i) {
        const hb_chain_phase& p = phases[i];
        if (p.k < 8 || p.k % 8) HB_REFUSE("gemm_tickets: product %d: k = %d is no multiple of 8", i, p.k);
        if (p.mode != 0 && p.mode != 1 && p.mode != 3) HB_REFUSE("gemm_tickets: product %d: mode %d", i, p.mode);
        if ((((uintptr_t)p.out | (uintptr_t)p.x | (uintptr_t)p.w) % 16) != 0 || !p.out || !p.x || !p.w)
            HB_REFUSE("gemm_tickets: product %d: pointers must be given and 16-byte aligned", i);
        if (p.mode == 1 ? p.inter < 1 : p.n < 1) HB_REFUSE("gemm_tickets: product %d: n = %d, inter = %d", i, p.n, p.inter);
        if (p.mode == 3 && (!p.h || !p.next_weight || !p.ss_out || p.out_f32))
            HB_REFUSE("gemm_tickets: product %d: mode 3 needs h, the next norm's weight and ss_out, and writes bfloat16", i);
        if (p.mode == 1 && p.out_f32) HB_REFUSE("gemm_tickets: product %d: mode 1 writes bfloat16", i);
        if (p.ss_in && (p.parts_in < 1 || p.dim_in < 1)) HB_REFUSE("gemm_tickets: product %d: %d partial sums over %d columns", i, p.parts_in, p.dim_in);
        TicketPhase& q = args.phase[i];
        q.w = (const bf16*)p.w; q.x = (const bf16*)p.x; q.out = p.out; q.h = p.h; q.next_weight = p.next_weight;
        q.ss_out = p.ss_out; q.ss_in = p.ss_in; q.n = p.n; q.k = p.k; q.mode = p.mode; q.inter = p.inter; q.out_f32 = p.out_f32;
        q.next_weight_f32 = p.next_weight_f32; q.parts_in = p.parts_in; q.dim_in = p.dim_in; q.next_offset = p.next_offset;
        q.eps_in = p.eps_in;
        q.tiles = ((p.mode == 1 ? p.inter : p.n) + 15) / 16;
        q.first = total;
        total += q.tiles;
    }
    args.phases = n_phases; args.m = m; args.total = total; args.state = state;
    if (m <= 8) gemm_tickets_kernel<1><<<total, TK_THREADS, 0, (cudaStream_t)stream>>>(args);
    else gemm_tickets_kernel<2><<<total, TK_THREADS, 0, (cudaStream_t)stream>>>(args);
    HB_LAUNCH_CHECK("gemm_tickets");
    return 0;
}
