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
// mode 2 is the attention's first product with what follows it folded in: w is [q heads; k heads; v heads] x head_dim
// rows, the head_dim / 16 CTAs of a head form a thread-block cluster, and after the product they norm the head
// (RMSNorm over head_dim with the q or k weight), rotate it by its token's position (half-split pairs, whole head)
// and write queries to q_out and keys and values straight into their cache pages. The head's sum of squares and the
// rotation partner 64 columns away come from the other CTAs' shared memory. Values are rounded to bfloat16 where the
// separate kernels round them (after the product, after the norm), so the results are theirs.
// mode 3 folds the residual sum and the next RMSNorm into a product that ends a mixer or a feed-forward: the CTA adds
// its 16 columns (rounded to bfloat16, as the separate product's output is) into the 32-bit stream h, writes the new
// stream times the next norm's weight as bfloat16, and leaves the sum of squares of its columns per token. The
// product that consumes those rows (any mode, `NormLink::ss_in`) adds the partial sums up in a fixed order and scales
// its sums by rsqrt(mean + eps) per token: x · rstd · w == (x · w) · rstd, so the norm costs no kernel and no pass
// over the stream of its own.
// 17 to 32 rows run the same kernel with four 8-row tiles of x a warp (the *32 entry points): every CTA then reads
// four times the rows of x for its 16 rows of w, which a weight of a few MB does not feel (such products are their
// launch, and this one kernel stands for a product and the kernel after it) and a large one does; the kernel table
// sends only small weights here. Their partial sums of squares lie 32 to a part instead of 16.
#include "skinny.cuh"

#define SK_WARPS 8

struct RopeEpilogue {                              // what mode 2 needs beyond the product
    bf16* q_out;                                   // [m, heads, head_dim]
    const int32_t* positions;                      // [m]
    const float* table;                            // [max_positions, head_dim]: cosines, then sines
    const void* q_weight;                          // [head_dim] or null: no norm
    const void* k_weight;
    bf16* kv;                                      // [pages, 2, kv_heads, page_size, head_dim] or null: nothing is written
    const int32_t* write_index;                    // [m]: page * page_size + offset, negative: skip
    float eps, offset;
    int max_positions, weight_f32, pages, page_size, heads, kv_heads, head_dim;
};

struct NormLink {                                  // the residual stream and the norms around a product
    float* h;                                      // mode 3: [m, n] 32-bit stream, added into
    const void* next_weight;                       // mode 3: the next norm's weight [n]
    float* ss_out;                                 // mode 3: [grid, 16] sums of squares of the new stream, per CTA and token
    const float* ss_in;                            // any mode: [parts_in, 16] of the product that made x (null: x is normed)
    float next_offset, eps_in;
    int next_weight_f32, parts_in, dim_in;
    int stride_in, stride_out;                     // tokens a part of ss_in / ss_out holds (16, or 32 for the 32-row kernels)
};

__device__ __forceinline__ float ld_peer_f32(const float* local, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ void st_peer_f32(float* local, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_barrier_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// MT tiles of 16 weight rows per CTA, NT tiles of 8 rows of x.
template <int MT, int NT, int SK_UNROLL, int MIN_CTAS>
__global__ void __launch_bounds__(SK_WARPS * 32, MIN_CTAS) gemm_skinny_kernel(void* __restrict__ out, int out_f32,
                                                                    const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                    int m, int n, int k, int mode, int inter,
                                                                    const RopeEpilogue ep, const NormLink link) {
    constexpr int TOKP = NT <= 2 ? 16 : NT * 8;          // tokens the per-token arrays hold
    constexpr int SGROUPS = SK_WARPS * 32 / TOKP;        // threads that share a token's partial sums of squares
    __shared__ float red[SK_WARPS][MT * 16][NT * 8 + 1];
    __shared__ float scale_part[SGROUPS][TOKP + 1];
    __shared__ float scale_in[TOKP];                     // per token: what the rows of x still lack (1 without a link)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = lane >> 2, c = lane & 3;
    if (MT == 1 && mode == 2 && (int)(blockIdx.x / (ep.head_dim >> 4)) < ep.heads + ep.kv_heads)   // a head that is normed and rotated:
        asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");   // its CTAs say that they run (waited for in the epilogue)
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

    // Mode 2 with at most 16 tokens: what this thread's element of the epilogue reads from global memory (its token's
    // position, then the cosine and sine there; the norm weights of its column and of its partner; where the cache is
    // written) is asked for here, ahead of the weights: at the end of the CTA each would be a trip to the L2 in a row
    // (0.2 to 0.3 us a launch, measured back to back in a graph).
    float pf_cs = 1.f, pf_sn = 0.f, pf_w = 1.f, pf_wo = 1.f;
    int pf_write = -1;
    if (MT == 1 && NT <= 2 && mode == 2 && threadIdx.x < 16 * m) {
        const int per_head = ep.head_dim >> 4, rank = blockIdx.x % per_head, item = blockIdx.x / per_head;
        const int tok = threadIdx.x >> 4, col = rank * 16 + (threadIdx.x & 15), half = ep.head_dim >> 1;
        const bool is_q = item < ep.heads, is_v = item >= ep.heads + ep.kv_heads;
        const void* weight = is_q ? ep.q_weight : ep.k_weight;
        if (!is_v) {
            const int pair = col < half ? col : col - half, pcol = col < half ? col + half : col - half;
            if (weight) {
                pf_w = ep.weight_f32 ? ((const float*)weight)[col] : to_f32(((const bf16*)weight)[col]);
                pf_wo = ep.weight_f32 ? ((const float*)weight)[pcol] : to_f32(((const bf16*)weight)[pcol]);
            }
            int pos = ep.positions[tok];
            pos = pos < 0 ? 0 : (pos >= ep.max_positions ? ep.max_positions - 1 : pos);
            pf_cs = ep.table[(size_t)pos * ep.head_dim + pair];
            pf_sn = ep.table[(size_t)pos * ep.head_dim + half + pair];
        }
        if (!is_q && ep.kv) pf_write = ep.write_index[tok];
    }

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
    float ss_mine = 0.f;                                 // token (thread % TOKP): every SGROUPS-th partial sum, in ascending order
    if (link.ss_in)
        for (int p2 = threadIdx.x / TOKP; p2 < link.parts_in; p2 += SGROUPS) ss_mine += link.ss_in[p2 * link.stride_in + threadIdx.x % TOKP];
    scale_part[threadIdx.x / TOKP][threadIdx.x % TOKP] = ss_mine;
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
    if (threadIdx.x < TOKP) {
        float total = 0.f;
#pragma unroll
        for (int j = 0; j < SGROUPS; ++j) total += scale_part[j][threadIdx.x];
        scale_in[threadIdx.x] = link.ss_in ? rsqrtf(total / (float)link.dim_in + link.eps_in) : 1.f;
    }
    __syncthreads();
    if (MT == 1 && mode == 2) {
        // The CTAs of a head hand one another what they need by writing it into the others' shared memory (the head's
        // sums of squares to every CTA, the rotation partner's columns to the CTA half a head away), then meet at one
        // cluster barrier; nobody reads another's memory, so nobody waits for the others before it leaves. (The CTAs of a
        // cluster are known to run once the barrier of the kernel's first lines has completed.)
        __shared__ float res[NT * 8][16];                            // the product, rounded as the separate kernel's input is
        __shared__ float other_s[NT * 8][16];                        // the same of the CTA half a head away, written by it
        __shared__ float psum_all[8][NT * 8];                        // per CTA of the head: its share of each token's sum of squares
        const int per_head = ep.head_dim >> 4, rank = blockIdx.x % per_head, item = blockIdx.x / per_head;
        const bool is_q = item < ep.heads, is_v = item >= ep.heads + ep.kv_heads;
        const void* weight = is_q ? ep.q_weight : ep.k_weight;
        if (!is_v) asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");   // (the first lines' arrival: long complete)
        for (int i = threadIdx.x; i < 16 * m; i += SK_WARPS * 32) {
            const int rr = i & 15, tok = i >> 4;
            float v = 0.f;
#pragma unroll
            for (int wv = 0; wv < SK_WARPS; ++wv) v += red[wv][rr][tok];
            v = rounded<bf16>(v * scale_in[tok]);
            res[tok][rr] = v;
            if (!is_v) st_peer_f32(&other_s[tok][rr], rank ^ (per_head >> 1), v);
        }
        __syncthreads();
        if (threadIdx.x < m && weight && !is_v) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) ss += res[threadIdx.x][j] * res[threadIdx.x][j];
#pragma unroll
            for (int p2 = 0; p2 < 8; ++p2)
                if (p2 < per_head) st_peer_f32(&psum_all[rank][threadIdx.x], p2, ss);
        }
        if (!is_v) {                                                 // (the same for every CTA of a head)
            __syncwarp();
            cluster_barrier_all();                                   // what the others wrote here is here
        }
        const int half = ep.head_dim >> 1;
        __shared__ float rstd_s[NT * 8];
        if (threadIdx.x < m && weight && !is_v) {                    // the head's sum of squares, in the order of its CTAs
            float ss = 0.f;
#pragma unroll
            for (int p2 = 0; p2 < 8; ++p2) ss += p2 < per_head ? psum_all[p2][threadIdx.x] : 0.f;
            rstd_s[threadIdx.x] = rsqrtf(ss / (float)ep.head_dim + ep.eps);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < 16 * m; i += SK_WARPS * 32) {
            const int rr = i & 15, tok = i >> 4, col = rank * 16 + rr;          // column inside the head
            const int pair = col < half ? col : col - half, pcol = col < half ? col + half : col - half;
            float y = res[tok][rr], other = 0.f, w_mine = pf_w, w_other = pf_wo, cs = pf_cs, sn = pf_sn;
            int w = pf_write;
            if (!is_v) other = other_s[tok][rr];                      // the column half a head away
            if (NT > 2) {                                            // (more tokens than threads: nothing was asked for ahead)
                w_mine = w_other = 1.f; cs = 1.f; sn = 0.f; w = -1;
                if (!is_v) {
                    if (weight) {
                        w_mine = ep.weight_f32 ? ((const float*)weight)[col] : to_f32(((const bf16*)weight)[col]);
                        w_other = ep.weight_f32 ? ((const float*)weight)[pcol] : to_f32(((const bf16*)weight)[pcol]);
                    }
                    int pos = ep.positions[tok];
                    pos = pos < 0 ? 0 : (pos >= ep.max_positions ? ep.max_positions - 1 : pos);
                    cs = ep.table[(size_t)pos * ep.head_dim + pair];
                    sn = ep.table[(size_t)pos * ep.head_dim + half + pair];
                }
                if (!is_q && ep.kv) w = ep.write_index[tok];
            }
            bf16* dst = nullptr;
            if (is_q) {
                dst = ep.q_out + ((size_t)tok * ep.heads + item) * ep.head_dim + col;
            } else if (ep.kv) {
                const int page = w >= 0 ? w / ep.page_size : -1, off = w >= 0 ? w % ep.page_size : 0;
                const int head = item - ep.heads - (is_v ? ep.kv_heads : 0);
                if (page >= 0 && page < ep.pages)
                    dst = ep.kv + ((((size_t)page * 2 + is_v) * ep.kv_heads + head) * ep.page_size + off) * ep.head_dim + col;
            }
            if (!is_v) {
                if (weight) {
                    const float rstd = rstd_s[tok];
                    y = rounded<bf16>(y * rstd * (w_mine + ep.offset));
                    other = rounded<bf16>(other * rstd * (w_other + ep.offset));
                }
                y = col < half ? y * cs - other * sn : y * cs + other * sn;
            }
            if (dst) *dst = __float2bfloat16_rn(y);
        }
        return;
    }
    if (MT == 1 && mode == 3) {                                      // 16 columns x 16 tokens at a time: one thread each
        const int rr = threadIdx.x & 15, col = row0[0] + rr;
#pragma unroll
        for (int tok = threadIdx.x >> 4; tok < TOKP; tok += 16) {
            const bool live = tok < m && col < n;
            float hn = 0.f;
            if (live) {
                const float before = link.h[(size_t)tok * n + col];
                const float wn = link.next_weight_f32 ? ((const float*)link.next_weight)[col] : to_f32(((const bf16*)link.next_weight)[col]);
                float v = 0.f;
#pragma unroll
                for (int wv = 0; wv < SK_WARPS; ++wv) v += red[wv][rr][tok];
                hn = before + rounded<bf16>(v * scale_in[tok]);
                link.h[(size_t)tok * n + col] = hn;
                ((bf16*)out)[(size_t)tok * n + col] = __float2bfloat16_rn(hn * (wn + link.next_offset));
            }
            float sq = hn * hn;                                      // over the token's 16 columns: lanes 0-15 or 16-31
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (rr == 0) link.ss_out[blockIdx.x * link.stride_out + tok] = sq;   // (tokens beyond m: 0)
        }
        return;
    }
    const int rows_out = mode == 1 ? HALF * 16 : MT * 16;
    const int width = mode == 1 ? inter : n;
    for (int i = threadIdx.x; i < rows_out * m; i += SK_WARPS * 32) {
        const int rr = i % rows_out, tok = i / rows_out;
        float v = 0.f;
#pragma unroll
        for (int wv = 0; wv < SK_WARPS; ++wv) v += red[wv][rr][tok];
        v *= scale_in[tok];
        int col = row0[0] + rr;
        if (MT > 1 && rr >= 16) col = row0[rr >> 4] + (rr & 15);
        if (mode == 1) {
            float u = 0.f;
#pragma unroll
            for (int wv = 0; wv < SK_WARPS; ++wv) u += red[wv][HALF * 16 + rr][tok];
            v = v / (1.f + expf(-v)) * (u * scale_in[tok]);
        }
        if (col < width) {
            if (out_f32) ((float*)out)[(size_t)tok * width + col] = v;
            else ((bf16*)out)[(size_t)tok * width + col] = __float2bfloat16_rn(v);
        }
    }
}

// mode 0: out [m, n] (bfloat16, or float32 when out_f32) = x [m, k] · w [n, k]ᵀ.
// mode 1: w is [2 * inter, k] with gate rows first; out [m, inter] = silu(x · gateᵀ) * (x · upᵀ); n is ignored.
// mode 3: h [m, n] (float32) += bfloat16(x · wᵀ); out [m, n] = bfloat16(h · (next_weight + next_offset));
//         ss_out [ceil(n / 16), 16] = per CTA and token the sum of squares of the CTA's 16 columns of the new h.
// ss_in (any mode; null: none): x lacks its norm's row scale, rsqrt(sum of ss_in [parts_in, 16] over parts / dim_in +
// eps_in) per token; the product's sums are scaled by it.
// m at most 16, k a multiple of 8, all pointers 16-byte aligned.
static int skinny_product(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode, int inter,
                          float* h, const void* next_weight, int next_weight_f32, float next_offset, float* ss_out,
                          const float* ss_in, int parts_in, float eps_in, int dim_in, int most, hb_stream stream) {
    if (m == 0) return 0;
    if (m < 0 || m > most) HB_REFUSE("gemm_bf16_skinny: %d rows; this kernel takes 1 to %d", m, most);
    if (k < 8 || k % 8) HB_REFUSE("gemm_bf16_skinny: k = %d is no multiple of 8", k);
    if ((((uintptr_t)out | (uintptr_t)x | (uintptr_t)w) % 16) != 0) HB_REFUSE("gemm_bf16_skinny: pointers must be 16-byte aligned");
    if (mode != 0 && mode != 1 && mode != 3) HB_REFUSE("gemm_bf16_skinny: mode %d", mode);
    if (mode == 3 && (!h || !next_weight || !ss_out || out_f32)) HB_REFUSE("gemm_bf16_skinny: mode 3 needs h, the next norm's weight and ss_out, and writes bfloat16");
    if (ss_in && (parts_in < 1 || dim_in < 1)) HB_REFUSE("gemm_bf16_skinny: %d partial sums over %d columns", parts_in, dim_in);
    NormLink link = {};
    link.h = h; link.next_weight = next_weight; link.ss_out = ss_out; link.ss_in = ss_in; link.next_offset = next_offset;
    link.eps_in = eps_in; link.next_weight_f32 = next_weight_f32; link.parts_in = parts_in; link.dim_in = dim_in;
    link.stride_in = link.stride_out = most;             // (16 tokens a part, or 32: both sides of a link run the same kernels)
    cudaStream_t s = (cudaStream_t)stream;
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        HB_CUDA(cudaGetDevice(&device));
        HB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    }
    const int nt = m <= 8 ? 1 : 2;
#define HB_SK_ARGS(md, it) out, out_f32, (const bf16*)x, (const bf16*)w, m, n, k, md, it, RopeEpilogue{}, link
    if (most > 16) {                                     // the 32-row kernels: four tiles of x a warp
        if (mode == 1) {
            if (inter < 1) HB_REFUSE("gemm_bf16_skinny: inter = %d", inter);
            gemm_skinny_kernel<2, 4, 2, 2><<<(inter + 15) / 16, SK_WARPS * 32, 0, s>>>(HB_SK_ARGS(1, inter));
        } else {
            if (n < 1) HB_REFUSE("gemm_bf16_skinny: n = %d", n);
            gemm_skinny_kernel<1, 4, 4, 2><<<(n + 15) / 16, SK_WARPS * 32, 0, s>>>(HB_SK_ARGS(mode, 0));
        }
    } else if (mode == 1) {
        if (inter < 1) HB_REFUSE("gemm_bf16_skinny: inter = %d", inter);
        const int grid = (inter + 15) / 16;
        if (nt == 1) gemm_skinny_kernel<2, 1, 4, 2><<<grid, SK_WARPS * 32, 0, s>>>(HB_SK_ARGS(1, inter));
        else gemm_skinny_kernel<2, 2, 4, 2><<<grid, SK_WARPS * 32, 0, s>>>(HB_SK_ARGS(1, inter));
    } else {
        if (n < 1) HB_REFUSE("gemm_bf16_skinny: n = %d", n);
        const bool wide = mode == 0 && n >= 32 * 2 * sms;    // enough rows to give every SM two CTAs of 32 rows
        const int grid = wide ? (n + 31) / 32 : (n + 15) / 16;
        if (wide && nt == 1) gemm_skinny_kernel<2, 1, 4, 2><<<grid, SK_WARPS * 32, 0, s>>>(HB_SK_ARGS(0, 0));
        else if (wide) gemm_skinny_kernel<2, 2, 4, 2><<<grid, SK_WARPS * 32, 0, s>>>(HB_SK_ARGS(0, 0));
        else if (nt == 1 && grid > 2 * sms && grid <= 3 * sms)       // one wave of three CTAs per SM instead of one and a bit of two
            gemm_skinny_kernel<1, 1, 4, 3><<<grid, SK_WARPS * 32, 0, s>>>(HB_SK_ARGS(mode, 0));
        else if (nt == 1) gemm_skinny_kernel<1, 1, 8, 2><<<grid, SK_WARPS * 32, 0, s>>>(HB_SK_ARGS(mode, 0));
        else gemm_skinny_kernel<1, 2, 8, 2><<<grid, SK_WARPS * 32, 0, s>>>(HB_SK_ARGS(mode, 0));
    }
#undef HB_SK_ARGS
    HB_LAUNCH_CHECK("gemm_bf16_skinny");
    return 0;
}

extern "C" int hb_gemm_bf16_skinny_linked(void* out, int out_f32, const void* x, const void* w, int m, int n, int k,
                                          int mode, int inter, float* h, const void* next_weight, int next_weight_f32,
                                          float next_offset, float* ss_out, const float* ss_in, int parts_in,
                                          float eps_in, int dim_in, hb_stream stream) {
    return skinny_product(out, out_f32, x, w, m, n, k, mode, inter, h, next_weight, next_weight_f32, next_offset, ss_out,
                          ss_in, parts_in, eps_in, dim_in, 16, stream);
}

// The same for up to 32 rows (meant for 17 to 32, and for weights of a few MB: see the head of this file); ss_in and
// ss_out hold 32 tokens a part.
extern "C" int hb_gemm_bf16_skinny32(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode,
                                     int inter, float* h, const void* next_weight, int next_weight_f32, float next_offset,
                                     float* ss_out, const float* ss_in, int parts_in, float eps_in, int dim_in,
                                     hb_stream stream) {
    return skinny_product(out, out_f32, x, w, m, n, k, mode, inter, h, next_weight, next_weight_f32, next_offset, ss_out,
                          ss_in, parts_in, eps_in, dim_in, 32, stream);
}

extern "C" int hb_gemm_bf16_skinny(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode,
                                   int inter, hb_stream stream) {
    if (mode == 3) HB_REFUSE("gemm_bf16_skinny: mode 3 goes through hb_gemm_bf16_skinny_linked");
    return hb_gemm_bf16_skinny_linked(out, out_f32, x, w, m, n, k, mode, inter, nullptr, nullptr, 0, 0.f, nullptr, nullptr,
                                      0, 0.f, 0, stream);
}

template <typename Kernel>
static int launch_head_clusters(Kernel kernel, int grid, int per_head, cudaStream_t s, void* out, const bf16* x, const bf16* w,
                                int m, int n, int k, const RopeEpilogue& ep, const NormLink& link) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(SK_WARPS * 32);
    cfg.stream = s;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = per_head; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    HB_CUDA(cudaLaunchKernelEx(&cfg, kernel, out, 0, x, w, m, n, k, 2, 0, ep, link));
    return 0;
}

// The attention's first product for up to 16 tokens with the q/k norm, the rotation and the cache write in its
// epilogue (mode 2 above): x [m, k], w [(heads + 2 kv_heads) * head_dim, k]; q_out [m, heads, head_dim]; keys and
// values go to kv [pages, 2, kv_heads, page_size, head_dim] at write_index (kv null: they are dropped). head_dim 32, 64
// or 128 with the whole head rotated; weights of the norms bfloat16 or float32, or null for no norm.
// ss_in, parts_in, eps_in, dim_in: as for hb_gemm_bf16_skinny_linked (x lacks its norm's row scale).
static int skinny_qkv(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions, const float* table,
                      int max_positions, const void* q_weight, const void* k_weight, int weight_f32, float eps, float offset,
                      void* kv, const int32_t* write_index, int pages, int page_size, int heads, int kv_heads, int head_dim,
                      const float* ss_in, int parts_in, float eps_in, int dim_in, int most, hb_stream stream) {
    if (m == 0) return 0;
    if (m < 0 || m > most) HB_REFUSE("qkv_rope_skinny: %d rows; this kernel takes 1 to %d", m, most);
    if (k < 8 || k % 8) HB_REFUSE("qkv_rope_skinny: k = %d is no multiple of 8", k);
    if (head_dim != 32 && head_dim != 64 && head_dim != 128) HB_REFUSE("qkv_rope_skinny: head_dim %d (32, 64 or 128)", head_dim);
    if (heads < 1 || kv_heads < 1) HB_REFUSE("qkv_rope_skinny: %d heads, %d kv heads", heads, kv_heads);
    if ((((uintptr_t)x | (uintptr_t)w) % 16) != 0) HB_REFUSE("qkv_rope_skinny: x and w must be 16-byte aligned");
    if (!q_out || !positions || !table || max_positions < 1) HB_REFUSE("qkv_rope_skinny: q_out, positions and the table are needed");
    if ((q_weight == nullptr) != (k_weight == nullptr)) HB_REFUSE("qkv_rope_skinny: both norm weights or none");
    if (ss_in && (parts_in < 1 || dim_in < 1)) HB_REFUSE("qkv_rope_skinny: %d partial sums over %d columns", parts_in, dim_in);
    NormLink link = {};
    link.ss_in = ss_in; link.parts_in = parts_in; link.eps_in = eps_in; link.dim_in = dim_in;
    link.stride_in = link.stride_out = most;
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        HB_CUDA(cudaGetDevice(&device));
        HB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    }
    RopeEpilogue ep;
    ep.q_out = (bf16*)q_out; ep.positions = positions; ep.table = table; ep.q_weight = q_weight; ep.k_weight = k_weight;
    ep.kv = (bf16*)kv; ep.write_index = write_index; ep.eps = eps; ep.offset = offset; ep.max_positions = max_positions;
    ep.weight_f32 = weight_f32; ep.pages = pages; ep.page_size = page_size < 1 ? 1 : page_size; ep.heads = heads;
    ep.kv_heads = kv_heads; ep.head_dim = head_dim;
    const int per_head = head_dim / 16, n = (heads + 2 * kv_heads) * head_dim, grid = n / 16;
    cudaStream_t s = (cudaStream_t)stream;
    if (most > 16)
        return launch_head_clusters(gemm_skinny_kernel<1, 4, 4, 2>, grid, per_head, s, nullptr, (const bf16*)x, (const bf16*)w, m, n, k, ep, link);
    if (m <= 8 && grid > 2 * sms && grid <= 3 * sms)
        return launch_head_clusters(gemm_skinny_kernel<1, 1, 4, 3>, grid, per_head, s, nullptr, (const bf16*)x, (const bf16*)w, m, n, k, ep, link);
    if (m <= 8)
        return launch_head_clusters(gemm_skinny_kernel<1, 1, 8, 2>, grid, per_head, s, nullptr, (const bf16*)x, (const bf16*)w, m, n, k, ep, link);
    return launch_head_clusters(gemm_skinny_kernel<1, 2, 8, 2>, grid, per_head, s, nullptr, (const bf16*)x, (const bf16*)w, m, n, k, ep, link);
}

extern "C" int hb_qkv_rope_skinny_linked(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions,
                                         const float* table, int max_positions, const void* q_weight, const void* k_weight,
                                         int weight_f32, float eps, float offset, void* kv, const int32_t* write_index,
                                         int pages, int page_size, int heads, int kv_heads, int head_dim,
                                         const float* ss_in, int parts_in, float eps_in, int dim_in, hb_stream stream) {
    return skinny_qkv(q_out, x, w, m, k, positions, table, max_positions, q_weight, k_weight, weight_f32, eps, offset, kv,
                      write_index, pages, page_size, heads, kv_heads, head_dim, ss_in, parts_in, eps_in, dim_in, 16, stream);
}

// The same for up to 32 tokens; ss_in holds 32 tokens a part.
extern "C" int hb_qkv_rope_skinny32(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions,
                                    const float* table, int max_positions, const void* q_weight, const void* k_weight,
                                    int weight_f32, float eps, float offset, void* kv, const int32_t* write_index,
                                    int pages, int page_size, int heads, int kv_heads, int head_dim, const float* ss_in,
                                    int parts_in, float eps_in, int dim_in, hb_stream stream) {
    return skinny_qkv(q_out, x, w, m, k, positions, table, max_positions, q_weight, k_weight, weight_f32, eps, offset, kv,
                      write_index, pages, page_size, heads, kv_heads, head_dim, ss_in, parts_in, eps_in, dim_in, 32, stream);
}

extern "C" int hb_qkv_rope_skinny(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions,
                                  const float* table, int max_positions, const void* q_weight, const void* k_weight,
                                  int weight_f32, float eps, float offset, void* kv, const int32_t* write_index,
                                  int pages, int page_size, int heads, int kv_heads, int head_dim, hb_stream stream) {
    return hb_qkv_rope_skinny_linked(q_out, x, w, m, k, positions, table, max_positions, q_weight, k_weight, weight_f32,
                                     eps, offset, kv, write_index, pages, page_size, heads, kv_heads, head_dim, nullptr, 0,
                                     0.f, 0, stream);
}
