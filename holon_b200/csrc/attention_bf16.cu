// bfloat16 paged attention on tensor cores (mma.sync m16n8k16, 32-bit accumulation and softmax).
//
// Two kernels share the tile loader and the fragment code:
//  * decode: rows that bring one token. A CTA owns (row, kv head, split of the keys); the kv head's whole group of
//    query heads is the 16-row M tile, so keys and values are read once per group. Its four warps take 16 keys each of
//    every 64-key tile and keep their own running softmax; they are merged in shared memory at the end. With more than
//    one split the CTA writes (max, sum, unnormalised output) to scratch and a second kernel merges the splits in a
//    fixed order.
//  * prefill: rows that bring several tokens (prompt portions). A CTA owns 64 queries of one head, 16 per warp, and
//    walks the 64-key tiles up to its diagonal (FlashAttention-2 style).
// Head sizes are multiples of 16 up to 256 (template D_PAD 64 / 128 / 256 with a run-time head_dim inside it); any page
// size; any group size (groups above 16 heads take several CTAs). Keys outside a row's range are zero-filled on load
// and masked, so nothing is ever read from a page the row does not hold.
#include "common.cuh"

#define TILE_N 64

// ---------------------------------------------------------------- small PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                  // src-size 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&v;
}
__device__ __forceinline__ float ex2(float x) {   // 2^x; -inf gives 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Shared-memory tiles hold rows of D_PAD bf16 = D_PAD/8 chunks of 16 bytes; the chunk index is XOR-ed with the low
// three bits of the row so that ldmatrix's 8 rows fall into 8 different bank groups. Byte offset of (row, chunk):
template <int D_PAD> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)(row * (D_PAD * 2) + ((chunk ^ (row & 7)) << 4));
}

// Per-lane parts of the ldmatrix addresses, worked out once. A fragment of k-step (or d-step) `step` in a block of 16
// rows that starts at a multiple of 8 lies at  base + rows * (D_PAD * 2) + lane_row + ((step * 32) ^ lane_xor).
struct FragLanes {
    uint32_t a_row, a_xor;         // 16 x 16 A operand (queries): rows lane & 15, k-half lane >> 4
    uint32_t b_row, b_xor;         // two 8-wide B operands from [n][k] memory (keys): rows (lane & 7) + 8 (lane >> 4)
    uint32_t t_row, t_xor;         // two 8-wide B operands from [k][n] memory through .trans (values)
};
template <int D_PAD> __device__ __forceinline__ FragLanes frag_lanes(int lane) {
    const uint32_t x = lane & 7, rb = D_PAD * 2;
    FragLanes f;
    f.a_row = (lane & 15) * rb;                          f.a_xor = ((uint32_t)(lane >> 4) ^ x) << 4;
    f.b_row = ((lane & 7) + ((lane >> 4) << 3)) * rb;    f.b_xor = ((uint32_t)((lane >> 3) & 1) ^ x) << 4;
    f.t_row = ((lane & 7) + (((lane >> 3) & 1) << 3)) * rb;  f.t_xor = ((uint32_t)(lane >> 4) ^ x) << 4;
    return f;
}

struct KvView {
    const bf16* kv;                // [pages, 2, kv_heads, page_size, head_dim]
    const int32_t* table;          // this row's block-table row
    int pages, page_size, kv_heads, head_dim, hk;
    int page_shift;                // log2(page_size) when it is a power of two, else -1
};

static int log2_exact(int x) {
    int s = 0;
    while ((1 << s) < x) ++s;
    return (1 << s) == x ? s : -1;
}

// Loads keys [tile * 64, tile * 64 + 64) of one kv head into the tiles at shared addresses k_s / v_s; keys outside
// [lo, hi) become zeros. A thread copies the same 16-byte column of every (THREADS / chunks-per-row)-th key row.
template <int D_PAD, int THREADS>
__device__ __forceinline__ void load_kv_tile(uint32_t k_s, uint32_t v_s, const KvView& c, int tile, int lo, int hi) {
    constexpr int CPR = D_PAD / 8;                              // 16-byte chunks per shared-memory row
    constexpr int STEP = THREADS / CPR;                         // key rows covered per pass
    const int ch = threadIdx.x % CPR, r0 = threadIdx.x / CPR;
    if (ch >= (c.head_dim >> 3)) return;                        // columns past head_dim are never read
    const long head_stride = (long)c.page_size * c.head_dim;
    const long v_shift = (long)c.kv_heads * head_stride;
    const long head_base = (long)c.hk * head_stride + ch * 8;
#pragma unroll
    for (int r = r0; r < TILE_N; r += STEP) {
        const int j = tile * TILE_N + r;
        bool valid = j >= lo && j < hi;
        long off = 0;
        if (valid) {
            const int pi = c.page_shift >= 0 ? j >> c.page_shift : j / c.page_size;
            const int po = c.page_shift >= 0 ? j & (c.page_size - 1) : j - pi * c.page_size;
            const int page = c.table[pi];
            valid = page >= 0 && page < c.pages;
            off = (long)page * 2 * v_shift + head_base + (long)po * c.head_dim;
        }
        const uint32_t d = tile_off<D_PAD>(r, ch);
        cp_async16(k_s + d, c.kv + off, valid);
        cp_async16(v_s + d, c.kv + off + (valid ? v_shift : 0), valid);
    }
}

// The same when a page holds a whole number of 64-key tiles (a power of two of at least 64): the tile lies in one
// page, whose number the caller has read already (one table entry a tile instead of one a key row), and a key row's
// address is the tile's plus a multiple of head_dim.
template <int D_PAD, int THREADS>
__device__ __forceinline__ void load_kv_tile_in_page(uint32_t k_s, uint32_t v_s, const KvView& c, int tile, int lo, int hi,
                                                     int page) {
    constexpr int CPR = D_PAD / 8;
    constexpr int STEP = THREADS / CPR;
    const int ch = threadIdx.x % CPR, r0 = threadIdx.x / CPR;
    if (ch >= (c.head_dim >> 3)) return;
    const long head_stride = (long)c.page_size * c.head_dim;
    const long v_shift = (long)c.kv_heads * head_stride;
    const int j0 = tile * TILE_N;
    const bool page_ok = page >= 0 && page < c.pages;
    const bool whole = j0 >= lo && j0 + TILE_N <= hi;            // no key of the tile is outside the row's range
    const bf16* base = c.kv + ((long)(page_ok ? page : 0) * 2 * v_shift + (long)c.hk * head_stride + ch * 8 +
                               (long)(j0 & (c.page_size - 1)) * c.head_dim);
#pragma unroll
    for (int r = r0; r < TILE_N; r += STEP) {
        const bool valid = page_ok && (whole || (j0 + r >= lo && j0 + r < hi));
        const bf16* src = base + (valid ? (long)r * c.head_dim : 0);
        const uint32_t d = tile_off<D_PAD>(r, ch);
        cp_async16(k_s + d, src, valid);
        cp_async16(v_s + d, src + (valid ? v_shift : 0), valid);
    }
}

// Loads `rows` query rows of one head (row stride heads * head_dim elements) into a tile; the rest become zeros.
template <int D_PAD, int ROWS, int THREADS>
__device__ __forceinline__ void load_q_tile(uint32_t q_s, const bf16* q, long row_stride, int rows, int head_dim) {
    for (int i = threadIdx.x; i < ROWS * (D_PAD / 8); i += THREADS) {
        const int r = i / (D_PAD / 8), ch = i % (D_PAD / 8);
        const bool valid = r < rows && ch < (head_dim >> 3);
        cp_async16(q_s + tile_off<D_PAD>(r, ch), q + (valid ? (long)r * row_stride + ch * 8 : 0), valid);
    }
}

// One online-softmax update of a lane's two rows over NT 8-key blocks of raw scores `s` (masked ones are -inf):
// turns s into weights 2^((s - max) * scale), updates the running maxima and sums, returns the factors by which what
// was summed before must be scaled.
template <int NT>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float& m0, float& m1, float& l0, float& l1,
                                             float scale_log2, float& c0, float& c1) {
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
        mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float nb0 = n0 == -INFINITY ? 0.f : -n0 * scale_log2;    // a row with nothing yet: 2^(-inf) = 0 below
    const float nb1 = n1 == -INFINITY ? 0.f : -n1 * scale_log2;
    c0 = ex2(fmaf(m0, scale_log2, nb0));
    c1 = ex2(fmaf(m1, scale_log2, nb1));
    m0 = n0; m1 = n1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        s[nt][0] = ex2(fmaf(s[nt][0], scale_log2, nb0)); s[nt][1] = ex2(fmaf(s[nt][1], scale_log2, nb0));
        s[nt][2] = ex2(fmaf(s[nt][2], scale_log2, nb1)); s[nt][3] = ex2(fmaf(s[nt][3], scale_log2, nb1));
        sum0 += s[nt][0] + s[nt][1]; sum1 += s[nt][2] + s[nt][3];
    }
    l0 = l0 * c0 + sum0; l1 = l1 * c1 + sum1;                       // per-lane partial sums; quads are joined at the end
}

// ================================================================ decode
// One walk of the four warps over tiles [first, last) of one (row, kv head, 16-head tile of its group); the result
// goes to `out` (part_stride 0) or, unnormalised with its maximum and sum, to partial slot part_base + r * part_stride
// for the tile's r-th head. Ends with a barrier, so that the next walk of the same CTA may overwrite the tiles.
template <int D_PAD, int STAGES>
__device__ __forceinline__ void decode_walk(
        unsigned char* smem_raw, bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
        size_t part_base, int part_stride, const bf16* __restrict__ q, const bf16* __restrict__ kv,
        const int32_t* __restrict__ table, int t, int heads, int kv_heads, int head_dim, int pages, int page_size,
        int page_shift, float scale_log2, int hk, int group, int g0, int g, int first, int last, int lo, int n) {
    constexpr uint32_t TILE_BYTES = TILE_N * D_PAD * 2;
    const uint32_t q_s = smem_u32(smem_raw);                       // [16][D_PAD]
    const uint32_t k_s = q_s + 16 * D_PAD * 2;                     // [STAGES][64][D_PAD]
    const uint32_t v_s = k_s + STAGES * TILE_BYTES;                // [STAGES][64][D_PAD]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    KvView view{kv, table, pages, page_size, kv_heads, head_dim, hk, page_shift};
    const bool in_page = page_shift >= 6;                           // a 64-key tile lies in one page: one table entry a tile,
    const int tile_shift = page_shift - 6;                          // read one tile ahead of the load that needs it
    load_q_tile<D_PAD, 16, 128>(q_s, q + ((size_t)t * heads + (size_t)hk * group + g0) * head_dim, head_dim, g, head_dim);
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (first + s < last) {
            if (in_page) load_kv_tile_in_page<D_PAD, 128>(k_s + s * TILE_BYTES, v_s + s * TILE_BYTES, view, first + s, lo, n,
                                                          view.table[(first + s) >> tile_shift]);
            else load_kv_tile<D_PAD, 128>(k_s + s * TILE_BYTES, v_s + s * TILE_BYTES, view, first + s, lo, n);
        }
        cp_async_commit();
    }
    int page_ahead = in_page && first + STAGES - 1 < last ? view.table[(first + STAGES - 1) >> tile_shift] : 0;

    float o[D_PAD / 8][4];
#pragma unroll
    for (int i = 0; i < D_PAD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows lane/4 and lane/4 + 8
    const int ksteps = head_dim >> 4;
    const FragLanes f = frag_lanes<D_PAD>(lane);
    constexpr bool Q_IN_REGS = D_PAD <= 128;                        // larger heads keep the registers for the output
    uint32_t qf[Q_IN_REGS ? D_PAD / 16 : 1][4];
    bool q_loaded = false;
    const uint32_t warp_rows = warp * 16 * (D_PAD * 2);             // this warp's 16 keys inside a tile

    for (int tile = first; tile < last; ++tile) {
        const int stage = (tile - first) % STAGES;
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (tile + STAGES - 1 < last) {
            const int s2 = (tile - first + STAGES - 1) % STAGES;
            if (in_page) load_kv_tile_in_page<D_PAD, 128>(k_s + s2 * TILE_BYTES, v_s + s2 * TILE_BYTES, view, tile + STAGES - 1, lo, n,
                                                          page_ahead);
            else load_kv_tile<D_PAD, 128>(k_s + s2 * TILE_BYTES, v_s + s2 * TILE_BYTES, view, tile + STAGES - 1, lo, n);
        }
        cp_async_commit();
        if (in_page && tile + STAGES < last) page_ahead = view.table[(tile + STAGES) >> tile_shift];
        if (Q_IN_REGS && !q_loaded) {
#pragma unroll
            for (int ks = 0; ks < D_PAD / 16; ++ks)
                if (ks < ksteps) ldmatrix_x4(qf[Q_IN_REGS ? ks : 0], q_s + f.a_row + ((ks * 32) ^ f.a_xor));
            q_loaded = true;
        }
        const int key0 = tile * TILE_N + warp * 16;                 // this warp's 16 keys
        if (key0 >= n || key0 + 16 <= lo) continue;                 // (uniform per warp; the barrier is above)
        const uint32_t kt = k_s + stage * TILE_BYTES + warp_rows + f.b_row;
        const uint32_t vt = v_s + stage * TILE_BYTES + warp_rows + f.t_row;
        float s[2][4] = {};
#pragma unroll
        for (int ks = 0; ks < D_PAD / 16; ++ks) {
            if (ks < ksteps) {
                uint32_t a[4], kb[4];
                if (!Q_IN_REGS) ldmatrix_x4(a, q_s + f.a_row + ((ks * 32) ^ f.a_xor));
                ldmatrix_x4(kb, kt + ((ks * 32) ^ f.b_xor));
                mma_bf16(s[0], Q_IN_REGS ? qf[Q_IN_REGS ? ks : 0] : a, kb[0], kb[1]);
                mma_bf16(s[1], Q_IN_REGS ? qf[Q_IN_REGS ? ks : 0] : a, kb[2], kb[3]);
            }
        }
        if (key0 < lo || key0 + 16 > n) {                           // only a row's first and last keys need the mask
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                    if (j < lo || j >= n) s[nt][e] = -INFINITY;
                }
        }
        float c0, c1;
        softmax_step<2>(s, m0, m1, l0, l1, scale_log2, c0, c1);
        uint32_t p[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]), pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
        if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {      // the running maximum moved: rescale what is summed
#pragma unroll
            for (int i = 0; i < D_PAD / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
        }
#pragma unroll
        for (int dt = 0; dt < D_PAD / 16; ++dt) {
            if (dt < ksteps) {
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, vt + ((dt * 32) ^ f.t_xor));
                mma_bf16(o[2 * dt], p, vb[0], vb[1]);
                mma_bf16(o[2 * dt + 1], p, vb[2], vb[3]);
            }
        }
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();                                                // every warp is done with the tiles: reuse them

    // ---- merge the four warps: [warp][row][D_PAD] floats and [warp][row][2] (max, sum) in the tile memory
    float* wo = (float*)(smem_raw + 16 * D_PAD * 2);
    float* wml = wo + 4 * 16 * D_PAD;
    const int r0 = lane >> 2, cq = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < D_PAD / 8; ++i) {
        if (i * 8 < head_dim) {
            if (r0 < g) { wo[(warp * 16 + r0) * D_PAD + i * 8 + cq] = o[i][0]; wo[(warp * 16 + r0) * D_PAD + i * 8 + cq + 1] = o[i][1]; }
            if (r0 + 8 < g) { wo[(warp * 16 + r0 + 8) * D_PAD + i * 8 + cq] = o[i][2]; wo[(warp * 16 + r0 + 8) * D_PAD + i * 8 + cq + 1] = o[i][3]; }
        }
    }
    if ((lane & 3) == 0) {
        wml[(warp * 16 + r0) * 2] = m0; wml[(warp * 16 + r0) * 2 + 1] = l0;
        wml[(warp * 16 + r0 + 8) * 2] = m1; wml[(warp * 16 + r0 + 8) * 2 + 1] = l1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < g * head_dim; i += 128) {
        const int r = i / head_dim, d = i % head_dim;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, wml[(w * 16 + r) * 2]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = wml[(w * 16 + r) * 2];
            const float fw = mw == -INFINITY ? 0.f : ex2((mw - mm) * scale_log2);
            acc += fw * wo[(w * 16 + r) * D_PAD + d];
            l += fw * wml[(w * 16 + r) * 2 + 1];
        }
        const int h = hk * group + g0 + r;
        if (part_stride == 0) {
            out[((size_t)t * heads + h) * head_dim + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        } else if (part_stride < 0) {                               // left in shared memory for the CTA's cluster
            float* stage = wml + 4 * 16 * 2;                        // [16][D_PAD] sums, then [16][2] (max in log2 units, sum)
            stage[r * D_PAD + d] = acc;
            if (d == 0) { stage[16 * D_PAD + r * 2] = mm * scale_log2; stage[16 * D_PAD + r * 2 + 1] = l; }
        } else {
            const size_t slot = part_base + (size_t)r * part_stride;
            part_o[slot * head_dim + d] = acc;
            if (d == 0) { part_ml[slot * 2] = mm * scale_log2; part_ml[slot * 2 + 1] = l; }   // the maximum in log2 units
        }
    }
    __syncthreads();
}

// grid (rows, kv_heads * m_tiles, splits), 128 threads. m_tiles = ceil(group / 16).
template <int D_PAD, int STAGES>
__global__ void __launch_bounds__(128) decode_kernel(
        bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q,
        const bf16* __restrict__ kv, const int32_t* __restrict__ block_table, int table_stride,
        const int32_t* __restrict__ row_slot, const int32_t* __restrict__ query_start,
        const int32_t* __restrict__ kv_len, int heads, int kv_heads, int head_dim, int pages, int page_size,
        int page_shift, float scale_log2, int window, int splits) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int b = blockIdx.x, split = blockIdx.z;
    const int group = heads / kv_heads, m_tiles = (group + 15) / 16;
    const int hk = blockIdx.y / m_tiles, mt = blockIdx.y % m_tiles;
    const int g0 = mt * 16, g = min(16, group - g0);                // this CTA's query heads: hk * group + g0 + [0, g)
    const int n = kv_len[b];
    const int lo = window > 0 ? max(0, n - window) : 0;             // the one query sits at position n - 1
    const int tile_lo = lo / TILE_N, tile_hi = (n + TILE_N - 1) / TILE_N;
    const int per = (tile_hi - tile_lo + splits - 1) / splits;
    const int first = tile_lo + split * per, last = min(tile_hi, first + per);
    decode_walk<D_PAD, STAGES>(smem_raw, out, part_o, part_ml, ((size_t)b * heads + (size_t)hk * group + g0) * splits + split,
                               splits > 1 ? splits : 0, q, kv, block_table + (size_t)row_slot[b] * table_stride,
                               query_start[b], heads, kv_heads, head_dim, pages, page_size, page_shift, scale_log2, hk,
                               group, g0, g, first, last, lo, n);
}

// The same rows with the splits of a (row, kv head) as one thread-block cluster: each CTA leaves its partial result in
// its shared memory, and after a cluster barrier every CTA combines a share of the outputs from all of them through
// distributed shared memory, in the order of the splits. No scratch in global memory and no second kernel.
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

#define CL_RECV_BYTES 4096
template <int D_PAD, int STAGES> __host__ __device__ constexpr size_t decode_walk_bytes() {
    constexpr size_t tiles = (size_t)(16 + 2 * STAGES * TILE_N) * D_PAD * sizeof(bf16);
    constexpr size_t merge = 16 * D_PAD * sizeof(bf16) + (size_t)(4 * 16 * D_PAD + 4 * 16 * 2 + 16 * D_PAD + 16 * 2) * sizeof(float);
    return tiles > merge ? tiles : merge;
}
__device__ __forceinline__ void st_cluster_f32(const float* local, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(remote), "f"(v) : "memory");
}

template <int D_PAD, int STAGES>
__global__ void __launch_bounds__(128) decode_cluster_kernel(
        bf16* __restrict__ out, const bf16* __restrict__ q, const bf16* __restrict__ kv,
        const int32_t* __restrict__ block_table, int table_stride, const int32_t* __restrict__ row_slot,
        const int32_t* __restrict__ query_start, const int32_t* __restrict__ kv_len, int heads, int kv_heads,
        int head_dim, int pages, int page_size, int page_shift, float scale_log2, int window, int splits) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");   // (this CTA runs: waited for before anybody writes here)
    const int b = blockIdx.x, split = blockIdx.z;                   // the cluster is the z direction: split = rank in it
    const int group = heads / kv_heads, m_tiles = (group + 15) / 16;
    const int hk = blockIdx.y / m_tiles, mt = blockIdx.y % m_tiles;
    const int g0 = mt * 16, g = min(16, group - g0);
    const int n = kv_len[b];
    const int lo = window > 0 ? max(0, n - window) : 0;
    const int tile_lo = lo / TILE_N, tile_hi = (n + TILE_N - 1) / TILE_N;
    const int per = (tile_hi - tile_lo + splits - 1) / splits;
    const int first = tile_lo + split * per, last = min(tile_hi, first + per);
    const int t = query_start[b];
    decode_walk<D_PAD, STAGES>(smem_raw, out, nullptr, nullptr, 0, -1, q, kv, block_table + (size_t)row_slot[b] * table_stride,
                               t, heads, kv_heads, head_dim, pages, page_size, page_shift, scale_log2, hk, group, g0, g,
                               first, last, lo, n);
    const int total = g * head_dim, share = (total + splits - 1) / splits;
    __syncwarp();
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");     // every CTA of the cluster runs
    if ((size_t)(splits * share + splits * g * 2) * sizeof(float) <= CL_RECV_BYTES) {   // (the same for every CTA of the launch)
        // Every CTA writes, for each of the others, the share of its sums that the other combines (and its maxima and row
        // sums) into the other's shared memory, behind the walk's; after one barrier each combines what lies in its own
        // memory, in the order of the splits, and leaves: no CTA reads another's memory, none waits for the others' reads.
        const float* mine = (const float*)(smem_raw + 16 * D_PAD * 2) + 4 * 16 * D_PAD + 4 * 16 * 2;   // [16][D_PAD], then [16][2]
        float* recv_o = (float*)(smem_raw + decode_walk_bytes<D_PAD, STAGES>());                      // [splits][share]
        float* recv_ml = recv_o + splits * share;                                                    // [splits][g][2]
        for (int e = threadIdx.x; e < total; e += 128) {
            const int peer = e / share, r = e / head_dim, d = e - r * head_dim;
            st_cluster_f32(recv_o + split * share + (e - peer * share), peer, mine[r * D_PAD + d]);
        }
        for (int i = threadIdx.x; i < splits * g; i += 128) {
            const int peer = i / g, r = i - peer * g;
            st_cluster_f32(recv_ml + (split * g + r) * 2, peer, mine[16 * D_PAD + r * 2]);
            st_cluster_f32(recv_ml + (split * g + r) * 2 + 1, peer, mine[16 * D_PAD + r * 2 + 1]);
        }
        __syncwarp();
        cluster_barrier();
        for (int i = threadIdx.x; i < share; i += 128) {
            const int e = split * share + i;
            if (e >= total) break;
            const int r = e / head_dim, d = e % head_dim;
            float mm = -INFINITY;
            for (int s2 = 0; s2 < splits; ++s2) mm = fmaxf(mm, recv_ml[(s2 * g + r) * 2]);
            float acc = 0.f, l = 0.f;
            for (int s2 = 0; s2 < splits; ++s2) {                   // in the order of the splits
                const float ms = recv_ml[(s2 * g + r) * 2];
                const float fs = ms == -INFINITY ? 0.f : ex2(ms - mm);
                acc += fs * recv_o[s2 * share + i];
                l += fs * recv_ml[(s2 * g + r) * 2 + 1];
            }
            out[((size_t)t * heads + hk * group + g0 + r) * head_dim + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        }
        return;
    }
    cluster_barrier();                                              // every split's sums are in its shared memory
    const uint32_t stage = smem_u32(smem_raw) + 16 * D_PAD * 2 + (4 * 16 * D_PAD + 4 * 16 * 2) * 4;
    for (int i = threadIdx.x; i < share; i += 128) {
        const int e = split * share + i;
        if (e >= total) break;
        const int r = e / head_dim, d = e % head_dim;
        float mm = -INFINITY;
        for (int s2 = 0; s2 < splits; ++s2) mm = fmaxf(mm, ld_cluster_f32(stage + (16 * D_PAD + r * 2) * 4, s2));
        float acc = 0.f, l = 0.f;
        for (int s2 = 0; s2 < splits; ++s2) {                       // in the order of the splits
            const float ms = ld_cluster_f32(stage + (16 * D_PAD + r * 2) * 4, s2);
            const float fs = ms == -INFINITY ? 0.f : ex2(ms - mm);
            acc += fs * ld_cluster_f32(stage + (r * D_PAD + d) * 4, s2);
            l += fs * ld_cluster_f32(stage + (16 * D_PAD + r * 2 + 1) * 4, s2);
        }
        out[((size_t)t * heads + hk * group + g0 + r) * head_dim + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    }
    __syncwarp();
    cluster_barrier();                                              // nobody leaves while its shared memory may be read
}

// out[0 .. head_dim) = sum_i w_i o_i / sum_i w_i l_i over `count` partial results at slots base + i * stride,
// w_i = 2^(m_i - max m). 128 threads: the maximum first (every thread a share of the partials), then warp w sums the
// partials i = w, w + 4, ... with a lane per four values, and the four warps' sums are added in warp order; the
// order of the sums depends on `count` alone, so equal inputs give equal outputs.
__device__ __forceinline__ void merge_partials(bf16* __restrict__ out, const float* __restrict__ part_o,
                                               const float* __restrict__ part_ml, size_t base, size_t stride, int count,
                                               int head_dim) {
    __shared__ float red[4];
    __shared__ float sums[4][257];                                   // per warp: up to 256 values and the sum of weights
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float mm = -INFINITY;
    for (int i = threadIdx.x; i < count; i += 128) mm = fmaxf(mm, part_ml[(base + i * stride) * 2]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, d));
    if (lane == 0) red[warp] = mm;
    __syncthreads();
    mm = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    for (int d0 = 0; d0 < head_dim; d0 += 128) {                     // head sizes are multiples of 16: a lane's four values
        const int d = d0 + lane * 4;                                 // are all inside or all outside
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float l = 0.f;
        for (int i = warp; i < count; i += 4) {
            const size_t slot = base + i * stride;
            const float ms = part_ml[slot * 2];
            const float w = ms == -INFINITY ? 0.f : ex2(ms - mm);
            l += w * part_ml[slot * 2 + 1];
            if (d < head_dim) {
                const float4 o = *(const float4*)(part_o + slot * head_dim + d);
                acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
            }
        }
        if (d < head_dim) { sums[warp][lane * 4] = acc.x; sums[warp][lane * 4 + 1] = acc.y; sums[warp][lane * 4 + 2] = acc.z; sums[warp][lane * 4 + 3] = acc.w; }
        if (lane == 0) sums[warp][256] = l;
        __syncthreads();
        const int dd = d0 + (int)threadIdx.x;
        if (dd < head_dim) {
            const float total = ((sums[0][256] + sums[1][256]) + sums[2][256]) + sums[3][256];
            const float v = ((sums[0][threadIdx.x] + sums[1][threadIdx.x]) + sums[2][threadIdx.x]) + sums[3][threadIdx.x];
            out[dd] = __float2bfloat16_rn(total > 0.f ? v / total : 0.f);
        }
        __syncthreads();
    }
}

// out[t, h, :] from the partial results of (row, head)'s splits, in ascending order.
__global__ void decode_merge_kernel(bf16* __restrict__ out, const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, const int32_t* __restrict__ query_start,
                                    int heads, int head_dim, int splits) {
    const int b = blockIdx.x, h = blockIdx.y;
    merge_partials(out + ((size_t)query_start[b] * heads + h) * head_dim, part_o, part_ml,
                   ((size_t)b * heads + h) * splits, 1, splits, head_dim);
}

template <int D_PAD> static size_t decode_smem(int stages) {
    const size_t tiles = (size_t)(16 + 2 * stages * TILE_N) * D_PAD * sizeof(bf16);
    const size_t merge = 16 * D_PAD * sizeof(bf16) + (size_t)(4 * 16 * D_PAD + 4 * 16 * 2 + 16 * D_PAD + 16 * 2) * sizeof(float);
    return tiles > merge ? tiles : merge;
}
// The cluster kernel's shared memory: the walk's, and behind it what the other CTAs of the cluster write here.
template <int D_PAD> static size_t decode_cluster_smem(int stages) { return decode_smem<D_PAD>(stages) + CL_RECV_BYTES; }

template <int D_PAD, int STAGES>
static int launch_decode(bf16* out, float* part_o, float* part_ml, const bf16* q, const bf16* kv,
                         const int32_t* block_table, int table_stride, const int32_t* row_slot,
                         const int32_t* query_start, const int32_t* kv_len, int rows, int heads, int kv_heads,
                         int head_dim, int pages, int page_size, float scale, int window, int splits, cudaStream_t s) {
    auto kernel = decode_kernel<D_PAD, STAGES>;
    const size_t smem = decode_smem<D_PAD>(STAGES);
    HB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int group = heads / kv_heads, m_tiles = (group + 15) / 16;
    dim3 grid(rows, kv_heads * m_tiles, splits);
    kernel<<<grid, 128, smem, s>>>(out, part_o, part_ml, q, kv, block_table, table_stride, row_slot, query_start,
                                   kv_len, heads, kv_heads, head_dim, pages, page_size, log2_exact(page_size),
                                   scale * 1.4426950408889634f, window, splits);
    HB_LAUNCH_CHECK("attention_decode");
    if (splits > 1) {
        decode_merge_kernel<<<dim3(rows, heads), 128, 0, s>>>(out, part_o, part_ml, query_start, heads, head_dim, splits);
        HB_LAUNCH_CHECK("attention_decode_merge");
    }
    return 0;
}

// How many clusters of `splits` CTAs of the cluster kernel the GPU holds at once (0: none, or the size is refused).
// Sizes beyond the portable 8 are asked for first.
template <int D_PAD, int STAGES>
static int decode_cluster_capacity(int splits) {
    static int known[17] = {};                                       // per size: 0 unknown, else capacity + 1
    if (known[splits] == 0) {
        auto kernel = decode_cluster_kernel<D_PAD, STAGES>;
        const size_t smem = decode_cluster_smem<D_PAD>(STAGES);
        bool ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
        if (ok && splits > 8)
            ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 1, splits);
        cfg.blockDim = dim3(128);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr = {};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 1; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = splits;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (!ok || cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) {
            (void)cudaGetLastError();
            clusters = 0;
        }
        known[splits] = clusters + 1;
    }
    return known[splits] - 1;
}

template <int D_PAD, int STAGES>
static int launch_decode_cluster(bf16* out, const bf16* q, const bf16* kv, const int32_t* block_table, int table_stride,
                                 const int32_t* row_slot, const int32_t* query_start, const int32_t* kv_len, int rows,
                                 int heads, int kv_heads, int head_dim, int pages, int page_size, float scale, int window,
                                 int splits, cudaStream_t s) {
    auto kernel = decode_cluster_kernel<D_PAD, STAGES>;
    if (decode_cluster_capacity<D_PAD, STAGES>(splits) < 1)          // (sets the kernel's attributes at its first call)
        HB_REFUSE("attention_decode_bf16_cluster: this GPU places no cluster of %d CTAs", splits);
    const int group = heads / kv_heads, m_tiles = (group + 15) / 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows, kv_heads * m_tiles, splits);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = decode_cluster_smem<D_PAD>(STAGES);
    cfg.stream = s;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 1; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = splits;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    HB_CUDA(cudaLaunchKernelEx(&cfg, kernel, out, q, kv, block_table, table_stride, row_slot, query_start, kv_len, heads,
                               kv_heads, head_dim, pages, page_size, log2_exact(page_size), scale * 1.4426950408889634f,
                               window, splits));
    return 0;
}

// Clusters of `splits` CTAs that run at once for this head size; the planner lets splits merge inside the kernel only
// while every (row, kv head) has its cluster in that one wave.
extern "C" int hb_attention_decode_cluster_capacity(int head_dim, int splits) {
    if (splits < 2 || splits > 16 || head_dim < 16 || head_dim > 256) return 0;
    if (head_dim <= 64) return decode_cluster_capacity<64, 4>(splits);
    if (head_dim <= 128) return decode_cluster_capacity<128, 2>(splits);
    return decode_cluster_capacity<256, 2>(splits);
}

// The rows of hb_attention_decode_bf16 with 2 to 16 splits that merge inside the kernel (a cluster per row and kv
// head; more than 8 CTAs a cluster is the size the hardware allows beyond the portable one).
extern "C" int hb_attention_decode_bf16_cluster(void* out, const void* q, const void* kv, const int32_t* block_table,
                                                int table_stride, const int32_t* row_slot, const int32_t* query_start,
                                                const int32_t* kv_len, int rows, int heads, int kv_heads, int head_dim,
                                                int pages, int page_size, float scale, int window, int splits,
                                                hb_stream stream) {
    if (rows == 0) return 0;
    if (head_dim % 16 || head_dim > 256 || head_dim < 16)
        HB_REFUSE("attention_decode_bf16_cluster: head_dim %d is no multiple of 16 up to 256", head_dim);
    if (kv_heads < 1 || heads % kv_heads) HB_REFUSE("attention_decode_bf16_cluster: %d heads, %d kv heads", heads, kv_heads);
    if (splits < 2 || splits > 16) HB_REFUSE("attention_decode_bf16_cluster: %d splits (2 to 16, a cluster's size)", splits);
    if (!(scale > 0.f)) HB_REFUSE("attention_decode_bf16_cluster: the score scale must be positive");
    if (rows > 65535 * 32) HB_REFUSE("attention_decode_bf16_cluster: %d rows", rows);
    cudaStream_t s = (cudaStream_t)stream;
#define HB_ARGS (bf16*)out, (const bf16*)q, (const bf16*)kv, block_table, table_stride, row_slot, query_start, kv_len, rows, \
    heads, kv_heads, head_dim, pages, page_size, scale, window, splits, s
    if (head_dim <= 64) return launch_decode_cluster<64, 4>(HB_ARGS);
    if (head_dim <= 128) return launch_decode_cluster<128, 2>(HB_ARGS);
    return launch_decode_cluster<256, 2>(HB_ARGS);
#undef HB_ARGS
}

extern "C" size_t hb_attention_decode_scratch_floats(int rows, int heads, int head_dim, int splits) {
    return splits > 1 ? (size_t)rows * heads * splits * (head_dim + 2) : 0;
}

extern "C" int hb_attention_decode_bf16(void* out, float* scratch, const void* q, const void* kv,
                                        const int32_t* block_table, int table_stride, const int32_t* row_slot,
                                        const int32_t* query_start, const int32_t* kv_len, int rows, int heads,
                                        int kv_heads, int head_dim, int pages, int page_size, float scale, int window,
                                        int splits, hb_stream stream) {
    if (rows == 0) return 0;
    if (head_dim % 16 || head_dim > 256 || head_dim < 16)
        HB_REFUSE("attention_decode_bf16: head_dim %d is no multiple of 16 up to 256", head_dim);
    if (kv_heads < 1 || heads % kv_heads) HB_REFUSE("attention_decode_bf16: %d heads, %d kv heads", heads, kv_heads);
    if (splits < 1 || splits > 64) HB_REFUSE("attention_decode_bf16: %d splits (1 to 64)", splits);
    if (splits > 1 && !scratch) HB_REFUSE("attention_decode_bf16: more than one split needs scratch memory");
    if (!(scale > 0.f)) HB_REFUSE("attention_decode_bf16: the score scale must be positive");
    if (rows > 65535 * 32) HB_REFUSE("attention_decode_bf16: %d rows", rows);
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)rows * heads * splits * head_dim : nullptr;
    cudaStream_t s = (cudaStream_t)stream;
#define HB_ARGS (bf16*)out, part_o, part_ml, (const bf16*)q, (const bf16*)kv, block_table, table_stride, row_slot, \
    query_start, kv_len, rows, heads, kv_heads, head_dim, pages, page_size, scale, window, splits, s
    if (head_dim <= 64) return launch_decode<64, 4>(HB_ARGS);
    if (head_dim <= 128) return launch_decode<128, 2>(HB_ARGS);   // two stages: three CTAs fit an SM, which hides latency better than a third stage
    return launch_decode<256, 2>(HB_ARGS);
#undef HB_ARGS
}

// ================================================================ decode, the keys of all rows shared out evenly
// The 64-key tiles of every (row, kv head, 16-head tile) are numbered in one line, row by row; CTA c of C takes tiles
// [c T / C, (c + 1) T / C) of the T there are, in as many walks as that stretch touches (row, head) pairs. Every CTA
// reads the same number of keys whatever the rows' lengths are, and one wave of CTAs that fills the GPU does all of it.
// A walk's partial result goes to slot c + p (p the pair's number): along the line either c or p grows from one
// walk to the next, so the slots of a pair's walks are distinct and follow one another. The merge kernel works the
// same numbers out again. C is cut to T / 2 when there are fewer tiles than that (a CTA then has at least two).
#define HB_BALANCED_ROWS 256

struct BalancedPlan {
    long long tiles;               // T
    int ctas;                      // C
    int pairs_per_row;
};

// Tiles of row b: the ones that hold keys the row's query may see.
__device__ __forceinline__ int row_tiles(int n, int window, int* tile_lo) {
    const int lo = window > 0 ? max(0, n - window) : 0;
    *tile_lo = lo / TILE_N;
    return (n + TILE_N - 1) / TILE_N - lo / TILE_N;
}

// prefix[b] = tiles of rows before b, prefix[rows] their total; by warp 0, 32 rows a pass.
__device__ __forceinline__ void tile_prefix(int* prefix, const int32_t* __restrict__ kv_len, int rows, int window) {
    if (threadIdx.x < 32) {
        int carry = 0;
        for (int b0 = 0; b0 < rows; b0 += 32) {
            const int b = b0 + (int)threadIdx.x;
            int unused, v = b < rows ? row_tiles(kv_len[b], window, &unused) : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, v, d);
                if ((int)threadIdx.x >= d) v += up;
            }
            if (b < rows) prefix[b + 1] = carry + v;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
        if (threadIdx.x == 0) prefix[0] = 0;
    }
    __syncthreads();
}

__device__ __forceinline__ BalancedPlan balanced_plan(const int* prefix, int rows, int pairs_per_row, int max_ctas) {
    BalancedPlan plan;
    plan.pairs_per_row = pairs_per_row;
    plan.tiles = (long long)prefix[rows] * pairs_per_row;
    const long long want = plan.tiles / 2 > 1 ? plan.tiles / 2 : 1;
    plan.ctas = (int)(want < max_ctas ? want : max_ctas);
    return plan;
}

template <int D_PAD, int STAGES>
__global__ void __launch_bounds__(128, (D_PAD <= 64 ? 4 : D_PAD <= 128 ? 3 : 1)) decode_balanced_kernel(
        float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q,
        const bf16* __restrict__ kv, const int32_t* __restrict__ block_table, int table_stride,
        const int32_t* __restrict__ row_slot, const int32_t* __restrict__ query_start,
        const int32_t* __restrict__ kv_len, int rows, int heads, int kv_heads, int head_dim, int pages, int page_size,
        int page_shift, float scale_log2, int window) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int prefix[HB_BALANCED_ROWS + 1];
    tile_prefix(prefix, kv_len, rows, window);
    const int group = heads / kv_heads, m_tiles = (group + 15) / 16, gmax = min(16, group);
    const BalancedPlan plan = balanced_plan(prefix, rows, kv_heads * m_tiles, (int)gridDim.x);
    const int c = blockIdx.x;
    if (c >= plan.ctas) return;
    long long f = (long long)c * plan.tiles / plan.ctas;
    const long long end = (long long)(c + 1) * plan.tiles / plan.ctas;
    int b = 0;
    while (f < end) {
        while ((long long)prefix[b + 1] * plan.pairs_per_row <= f) ++b;          // the row this tile belongs to
        const int tiles_b = prefix[b + 1] - prefix[b];
        const long long in_row = f - (long long)prefix[b] * plan.pairs_per_row;
        const int pair = (int)(in_row / tiles_b), tile = (int)(in_row % tiles_b);
        const int count = (int)min((long long)(tiles_b - tile), end - f);
        const int hk = pair / m_tiles, mt = pair % m_tiles;
        const int g0 = mt * 16, g = min(16, group - g0);
        const int n = kv_len[b];
        int tile_lo;
        row_tiles(n, window, &tile_lo);
        const int lo = window > 0 ? max(0, n - window) : 0;
        const size_t slot = (size_t)c + (size_t)b * plan.pairs_per_row + pair;
        decode_walk<D_PAD, STAGES>(smem_raw, nullptr, part_o, part_ml, slot * gmax, 1, q, kv,
                                   block_table + (size_t)row_slot[b] * table_stride, query_start[b], heads, kv_heads,
                                   head_dim, pages, page_size, page_shift, scale_log2, hk, group, g0, g,
                                   tile_lo + tile, tile_lo + tile + count, lo, n);
        f += count;
    }
}

// out[t, h, :] from the partial results of the walks over (row, head)'s pair, in the order of the CTAs that made them.
__global__ void decode_balanced_merge_kernel(bf16* __restrict__ out, const float* __restrict__ part_o,
                                             const float* __restrict__ part_ml, const int32_t* __restrict__ query_start,
                                             const int32_t* __restrict__ kv_len, int rows, int heads, int kv_heads,
                                             int head_dim, int window, int max_ctas) {
    __shared__ int sums[2][4];
    const int b = blockIdx.x, h = blockIdx.y;
    int before = 0, total = 0, unused;                               // tiles of the rows before b, and of all rows
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
        const int v = row_tiles(kv_len[r], window, &unused);
        total += v;
        if (r < b) before += v;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        before += __shfl_xor_sync(0xffffffffu, before, d);
        total += __shfl_xor_sync(0xffffffffu, total, d);
    }
    if ((threadIdx.x & 31) == 0) { sums[0][threadIdx.x >> 5] = before; sums[1][threadIdx.x >> 5] = total; }
    __syncthreads();
    before = sums[0][0] + sums[0][1] + sums[0][2] + sums[0][3];
    total = sums[1][0] + sums[1][1] + sums[1][2] + sums[1][3];
    const int group = heads / kv_heads, m_tiles = (group + 15) / 16, gmax = min(16, group);
    const int pairs_per_row = kv_heads * m_tiles;
    const long long tiles = (long long)total * pairs_per_row;
    const long long want = tiles / 2 > 1 ? tiles / 2 : 1;
    const int ctas = (int)(want < max_ctas ? want : max_ctas);
    const int tiles_b = row_tiles(kv_len[b], window, &unused);
    const int hk = h / group, in_group = h - hk * group;
    const int pair = hk * m_tiles + in_group / 16, r = in_group % 16;
    const int t = query_start[b];
    if (tiles_b == 0) {
        for (int d = threadIdx.x; d < head_dim; d += blockDim.x) out[((size_t)t * heads + h) * head_dim + d] = __float2bfloat16_rn(0.f);
        return;
    }
    // CTA c owns tiles [c T / C, (c + 1) T / C): tile f belongs to the largest c with c T / C <= f
    const long long f_lo = (long long)before * pairs_per_row + (long long)pair * tiles_b, f_hi = f_lo + tiles_b - 1;
    const int c_lo = (int)(((f_lo + 1) * ctas - 1) / tiles), c_hi = (int)(((f_hi + 1) * ctas - 1) / tiles);
    const size_t p = (size_t)b * pairs_per_row + pair;
    merge_partials(out + ((size_t)t * heads + h) * head_dim, part_o, part_ml, ((size_t)c_lo + p) * gmax + r, gmax,
                   c_hi - c_lo + 1, head_dim);
}

template <int D_PAD, int STAGES>
static int launch_decode_balanced(bf16* out, float* part_o, float* part_ml, const bf16* q, const bf16* kv,
                                  const int32_t* block_table, int table_stride, const int32_t* row_slot,
                                  const int32_t* query_start, const int32_t* kv_len, int rows, int heads, int kv_heads,
                                  int head_dim, int pages, int page_size, float scale, int window, int ctas,
                                  cudaStream_t s) {
    auto kernel = decode_balanced_kernel<D_PAD, STAGES>;
    const size_t smem = decode_smem<D_PAD>(STAGES);
    HB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<ctas, 128, smem, s>>>(part_o, part_ml, q, kv, block_table, table_stride, row_slot, query_start, kv_len, rows,
                                   heads, kv_heads, head_dim, pages, page_size, log2_exact(page_size),
                                   scale * 1.4426950408889634f, window);
    HB_LAUNCH_CHECK("attention_decode_balanced");
    decode_balanced_merge_kernel<<<dim3(rows, heads), 128, 0, s>>>(out, part_o, part_ml, query_start, kv_len, rows, heads,
                                                                   kv_heads, head_dim, window, ctas);
    HB_LAUNCH_CHECK("attention_decode_balanced_merge");
    return 0;
}

// Floats of scratch for `ctas` CTAs: one partial (head_dim values, a maximum and a sum) per walk and head.
extern "C" size_t hb_attention_decode_balanced_scratch_floats(int rows, int heads, int kv_heads, int head_dim, int ctas) {
    const int group = heads / kv_heads, m_tiles = (group + 15) / 16, gmax = group < 16 ? group : 16;
    return ((size_t)ctas + (size_t)rows * kv_heads * m_tiles) * gmax * (head_dim + 2);
}

extern "C" int hb_attention_decode_bf16_balanced(void* out, float* scratch, const void* q, const void* kv,
                                                 const int32_t* block_table, int table_stride, const int32_t* row_slot,
                                                 const int32_t* query_start, const int32_t* kv_len, int rows, int heads,
                                                 int kv_heads, int head_dim, int pages, int page_size, float scale,
                                                 int window, int ctas, hb_stream stream) {
    if (rows == 0) return 0;
    if (head_dim % 16 || head_dim > 256 || head_dim < 16)
        HB_REFUSE("attention_decode_bf16_balanced: head_dim %d is no multiple of 16 up to 256", head_dim);
    if (kv_heads < 1 || heads % kv_heads) HB_REFUSE("attention_decode_bf16_balanced: %d heads, %d kv heads", heads, kv_heads);
    if (heads > 65535) HB_REFUSE("attention_decode_bf16_balanced: %d heads", heads);
    if (rows > HB_BALANCED_ROWS) HB_REFUSE("attention_decode_bf16_balanced: %d rows, at most %d", rows, HB_BALANCED_ROWS);
    if (ctas < 1 || ctas > 65535) HB_REFUSE("attention_decode_bf16_balanced: %d CTAs (1 to 65535)", ctas);
    if (!scratch) HB_REFUSE("attention_decode_bf16_balanced: needs scratch memory");
    if (!(scale > 0.f)) HB_REFUSE("attention_decode_bf16_balanced: the score scale must be positive");
    const size_t slots = hb_attention_decode_balanced_scratch_floats(rows, heads, kv_heads, head_dim, ctas) / (head_dim + 2);
    float* part_o = scratch;
    float* part_ml = scratch + slots * head_dim;
    cudaStream_t s = (cudaStream_t)stream;
#define HB_ARGS (bf16*)out, part_o, part_ml, (const bf16*)q, (const bf16*)kv, block_table, table_stride, row_slot, \
    query_start, kv_len, rows, heads, kv_heads, head_dim, pages, page_size, scale, window, ctas, s
    if (head_dim <= 64) return launch_decode_balanced<64, 4>(HB_ARGS);
    if (head_dim <= 128) return launch_decode_balanced<128, 2>(HB_ARGS);
    return launch_decode_balanced<256, 2>(HB_ARGS);
#undef HB_ARGS
}

// ================================================================ prefill
// grid (query tiles, heads), 128 threads; a CTA finds its (row, first query) by walking the rows' tile counts, the
// last tile first: under a causal mask the late queries of a row have the most keys, and they should start early.
template <int D_PAD>
__global__ void __launch_bounds__(128, (D_PAD <= 128 ? 3 : 1)) prefill_kernel(
        bf16* __restrict__ out, const bf16* __restrict__ q, const bf16* __restrict__ kv,
        const int32_t* __restrict__ block_table, int table_stride, const int32_t* __restrict__ row_slot,
        const int32_t* __restrict__ query_start, const int32_t* __restrict__ kv_len, int row0, int rows, int heads,
        int kv_heads, int head_dim, int pages, int page_size, int page_shift, float scale_log2, int window) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr uint32_t TILE_BYTES = TILE_N * D_PAD * 2;
    constexpr bool Q_IN_REGS = D_PAD <= 128;       // the queries then pass through the second stage's key tile
    const uint32_t k_s = smem_u32(smem_raw);                        // [2][64][D_PAD]
    const uint32_t v_s = k_s + 2 * TILE_BYTES;                      // [2][64][D_PAD]
    const uint32_t q_s = Q_IN_REGS ? k_s + TILE_BYTES : v_s + 2 * TILE_BYTES;
    __shared__ int s_row, s_q0;
    if (threadIdx.x == 0) {
        int left = (int)blockIdx.y, found = -1, q0 = 0;              // x is handed out first: all heads' late tiles (longest) start first
        for (int b = rows - 1; b >= row0; --b) {
            const int tiles = (query_start[b + 1] - query_start[b] + 63) >> 6;
            if (left < tiles) { found = b; q0 = (tiles - 1 - left) * 64; break; }
            left -= tiles;
        }
        s_row = found; s_q0 = q0;
    }
    __syncthreads();
    const int b = s_row;
    if (b < 0) return;
    const int h = blockIdx.x, hk = h / (heads / kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = query_start[b] + s_q0, nq = query_start[b + 1] - query_start[b];
    const int qn = min(64, nq - s_q0);                              // queries in this tile
    const int n = kv_len[b];
    const int p0 = n - nq + s_q0;                                   // position of the tile's first query
    const int hi = min(n, p0 + qn);                                 // keys below hi are visible to someone here
    const int lo = window > 0 ? max(0, p0 - window + 1) : 0;
    const int tile_lo = lo / TILE_N, tile_hi = (hi + TILE_N - 1) / TILE_N;

    KvView view{kv, block_table + (size_t)row_slot[b] * table_stride, pages, page_size, kv_heads, head_dim, hk, page_shift};
    const int ksteps = head_dim >> 4;
    const FragLanes f = frag_lanes<D_PAD>(lane);
    const uint32_t warp_rows = warp * 16 * (D_PAD * 2);
    uint32_t qf[Q_IN_REGS ? D_PAD / 16 : 1][4];

    load_q_tile<D_PAD, 64, 128>(q_s, q + ((size_t)t0 * heads + h) * head_dim, (long)heads * head_dim, qn, head_dim);
    cp_async_commit();
    if (tile_lo < tile_hi) load_kv_tile<D_PAD, 128>(k_s, v_s, view, tile_lo, lo, hi);
    cp_async_commit();
    if (Q_IN_REGS) {
        cp_async_wait<1>();                                         // the queries have landed (the first keys may not)
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < D_PAD / 16; ++ks)
            if (ks < ksteps) ldmatrix_x4(qf[Q_IN_REGS ? ks : 0], q_s + warp_rows + f.a_row + ((ks * 32) ^ f.a_xor));
        __syncthreads();                                            // before the second stage is filled with keys
    }

    float o[D_PAD / 8][4];
#pragma unroll
    for (int i = 0; i < D_PAD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int pos0 = p0 + warp * 16 + (lane >> 2), pos1 = pos0 + 8;  // this lane's two query positions

    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int stage = (tile - tile_lo) & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (tile + 1 < tile_hi)
            load_kv_tile<D_PAD, 128>(k_s + (stage ^ 1) * TILE_BYTES, v_s + (stage ^ 1) * TILE_BYTES, view, tile + 1, lo, hi);
        cp_async_commit();
        const int key0 = tile * TILE_N;
        if (warp * 16 >= qn) continue;                              // a warp without queries
        if (key0 > p0 + warp * 16 + 15) continue;                   // every key of the tile is in this warp's future
        const uint32_t kt = k_s + stage * TILE_BYTES + f.b_row;
        const uint32_t vt = v_s + stage * TILE_BYTES + f.t_row;
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D_PAD / 16; ++ks) {
            if (ks < ksteps) {
                uint32_t a[4];
                if (!Q_IN_REGS) ldmatrix_x4(a, q_s + warp_rows + f.a_row + ((ks * 32) ^ f.a_xor));
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t kb[4];
                    ldmatrix_x4(kb, kt + np * 16 * (D_PAD * 2) + ((ks * 32) ^ f.b_xor));
                    mma_bf16(s[2 * np], Q_IN_REGS ? qf[Q_IN_REGS ? ks : 0] : a, kb[0], kb[1]);
                    mma_bf16(s[2 * np + 1], Q_IN_REGS ? qf[Q_IN_REGS ? ks : 0] : a, kb[2], kb[3]);
                }
            }
        }
        if (key0 + TILE_N - 1 > p0 + warp * 16 || window > 0 || key0 + TILE_N > hi) {     // the diagonal, a window, the end
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const int pos = e < 2 ? pos0 : pos1;
                    if (!(j <= pos && j < hi && (window <= 0 || pos - j < window))) s[nt][e] = -INFINITY;
                }
        }
        float c0, c1;
        softmax_step<8>(s, m0, m1, l0, l1, scale_log2, c0, c1);
        if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {
#pragma unroll
            for (int i = 0; i < D_PAD / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {                            // 16 keys at a time
            uint32_t p[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                             pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
            for (int dt = 0; dt < D_PAD / 16; ++dt) {
                if (dt < ksteps) {
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, vt + kk * 16 * (D_PAD * 2) + ((dt * 32) ^ f.t_xor));
                    mma_bf16(o[2 * dt], p, vb[0], vb[1]);
                    mma_bf16(o[2 * dt + 1], p, vb[2], vb[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    const int r0 = warp * 16 + (lane >> 2), cq = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < D_PAD / 8; ++i) {
        if (i * 8 < head_dim) {
            if (r0 < qn) *(uint32_t*)(out + ((size_t)(t0 + r0) * heads + h) * head_dim + i * 8 + cq) = pack_bf16(o[i][0] * i0, o[i][1] * i0);
            if (r0 + 8 < qn) *(uint32_t*)(out + ((size_t)(t0 + r0 + 8) * heads + h) * head_dim + i * 8 + cq) = pack_bf16(o[i][2] * i1, o[i][3] * i1);
        }
    }
}

template <int D_PAD>
static int launch_prefill(bf16* out, const bf16* q, const bf16* kv, const int32_t* block_table, int table_stride,
                          const int32_t* row_slot, const int32_t* query_start, const int32_t* kv_len, int row0,
                          int rows, int q_tiles, int heads, int kv_heads, int head_dim, int pages, int page_size,
                          float scale, int window, cudaStream_t s) {
    auto kernel = prefill_kernel<D_PAD>;
    const size_t smem = (size_t)(4 * TILE_N + (D_PAD <= 128 ? 0 : 64)) * D_PAD * sizeof(bf16);
    HB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (q_tiles > 65535) HB_REFUSE("attention_prefill: %d query tiles in one step, above 65535", q_tiles);
    kernel<<<dim3(heads, q_tiles), 128, smem, s>>>(out, q, kv, block_table, table_stride, row_slot, query_start,
                                                   kv_len, row0, rows, heads, kv_heads, head_dim, pages, page_size,
                                                   log2_exact(page_size), scale * 1.4426950408889634f, window);
    HB_LAUNCH_CHECK("attention_prefill");
    return 0;
}

// Rows row0 .. rows - 1 of the batch; q_tiles is the sum of ceil(queries / 64) over them.
extern "C" int hb_attention_prefill_bf16(void* out, const void* q, const void* kv, const int32_t* block_table,
                                         int table_stride, const int32_t* row_slot, const int32_t* query_start,
                                         const int32_t* kv_len, int row0, int rows, int q_tiles, int heads,
                                         int kv_heads, int head_dim, int pages, int page_size, float scale,
                                         int window, hb_stream stream) {
    if (rows <= row0 || q_tiles == 0) return 0;
    if (head_dim % 16 || head_dim > 256 || head_dim < 16)
        HB_REFUSE("attention_prefill_bf16: head_dim %d is no multiple of 16 up to 256", head_dim);
    if (kv_heads < 1 || heads % kv_heads) HB_REFUSE("attention_prefill_bf16: %d heads, %d kv heads", heads, kv_heads);
    if (heads > 65535) HB_REFUSE("attention_prefill_bf16: %d heads", heads);
    if (!(scale > 0.f)) HB_REFUSE("attention_prefill_bf16: the score scale must be positive");
    cudaStream_t s = (cudaStream_t)stream;
#define HB_ARGS (bf16*)out, (const bf16*)q, (const bf16*)kv, block_table, table_stride, row_slot, query_start, kv_len, \
    row0, rows, q_tiles, heads, kv_heads, head_dim, pages, page_size, scale, window, s
    if (head_dim <= 64) return launch_prefill<64>(HB_ARGS);
    if (head_dim <= 128) return launch_prefill<128>(HB_ARGS);
    return launch_prefill<256>(HB_ARGS);
#undef HB_ARGS
}
