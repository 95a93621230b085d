// The C interface of the kernel library. Every function enqueues work on `stream` and returns at once:
// 0 on success, HB_ERR_REFUSED for sizes or types a kernel does not take (hb_last_error() says which),
// HB_ERR_CUDA when the launch itself failed. Pointers are device pointers unless a comment says otherwise.
// dtype codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HB_F32 0
#define HB_BF16 1
#define HB_ERR_REFUSED 1
#define HB_ERR_CUDA 2

typedef void* hb_stream;

const char* hb_last_error(void);
int hb_version(void);

// out[t, :] = float(table[ids[t], :]); ids outside [0, vocab) give a row of zeros.
int hb_embed(float* out, const void* table, int table_dtype, const int32_t* ids, int tokens, int hidden, int vocab,
             hb_stream stream);

// Row r reads row t = index ? index[r] : r of h (and of delta when given): v = h[t] + delta[t];
// out[r] = v * rsqrt(mean(v^2) + eps) * (weight + offset), rounded once. With delta and without index, h[t] = v is
// written back (h must then be float32). h_dtype may be bfloat16 only without delta (a plain norm).
int hb_add_rmsnorm(void* out, int out_dtype, void* h, int h_dtype, const void* delta, const void* weight,
                   int weight_dtype, float eps, float offset, const int32_t* index, int rows, int dim,
                   hb_stream stream);

// out[t, i] = silu(gate_up[t, i]) * gate_up[t, inter + i], in 32-bit, rounded once.
int hb_silu_mul(void* out, const void* gate_up, int dtype, int tokens, int inter, hb_stream stream);

// Per token and head: RMSNorm over the head (if weights are given), rounding, rotation of the first rotary_dim
// dimensions in half-split pairs with cos|sin rows of `table` [max_positions, rotary_dim], rounding. q goes to q_out
// [tokens, heads, head_dim]; k and v go to kv [pages, 2, kv_heads, page_size, head_dim] at write_index = page *
// page_size + offset (a negative or out-of-range index skips the token). kv may be null (q only).
int hb_qk_norm_rope_kv_write(void* q_out, const void* qkv, int dtype, const int32_t* positions, const float* table,
                             int rotary_dim, int max_positions, const void* q_weight, const void* k_weight,
                             int weight_dtype, float eps, float offset, void* kv, const int32_t* write_index,
                             int pages, int page_size, int tokens, int heads, int kv_heads, int head_dim,
                             hb_stream stream);

// Attention of the step's new rows over the paged cache, any sizes, on CUDA cores with 32-bit arithmetic.
// Row b owns query rows query_start[b] .. query_start[b+1], the last ones of its kv_len[b] tokens; a query at position
// p sees keys j <= p, with window > 0 only p - j < window.
int hb_attention_generic(void* out, const void* q, const void* kv, int dtype, const int32_t* block_table,
                         int table_stride, const int32_t* row_slot, const int32_t* query_start,
                         const int32_t* kv_len, int rows, int tokens, int heads, int kv_heads, int head_dim,
                         int pages, int page_size, float scale, int window, hb_stream stream);

// bfloat16 attention on tensor cores for rows that bring one token each (rows 0 .. rows - 1 of the batch). The keys of
// a row are cut into `splits` parts that run side by side; with more than one split, `scratch` must hold
// hb_attention_decode_scratch_floats(...) floats: the parts' partial results, merged by a second kernel.
// head_dim: a multiple of 16 up to 256.
size_t hb_attention_decode_scratch_floats(int rows, int heads, int head_dim, int splits);
int hb_attention_decode_bf16(void* out, float* scratch, const void* q, const void* kv, const int32_t* block_table,
                             int table_stride, const int32_t* row_slot, const int32_t* query_start,
                             const int32_t* kv_len, int rows, int heads, int kv_heads, int head_dim, int pages,
                             int page_size, float scale, int window, int splits, hb_stream stream);

// The same rows with 2 to 16 splits whose CTAs form a thread-block cluster and merge through distributed shared memory
// inside the kernel: no scratch, no second kernel. hb_attention_decode_cluster_capacity: clusters of that many CTAs
// that the GPU runs at once for this head size (0: none).
int hb_attention_decode_cluster_capacity(int head_dim, int splits);
int hb_attention_decode_bf16_cluster(void* out, const void* q, const void* kv, const int32_t* block_table,
                                     int table_stride, const int32_t* row_slot, const int32_t* query_start,
                                     const int32_t* kv_len, int rows, int heads, int kv_heads, int head_dim, int pages,
                                     int page_size, float scale, int window, int splits, hb_stream stream);

// The same rows with the keys of all of them shared out evenly over `ctas` CTAs (one wave that fills the GPU): each
// takes the same number of 64-key tiles, across rows and heads where its stretch crosses them, so rows of any lengths
// cost what their sum costs. At most 256 rows. `scratch`: hb_attention_decode_balanced_scratch_floats(...) floats.
size_t hb_attention_decode_balanced_scratch_floats(int rows, int heads, int kv_heads, int head_dim, int ctas);
int hb_attention_decode_bf16_balanced(void* out, float* scratch, const void* q, const void* kv,
                                      const int32_t* block_table, int table_stride, const int32_t* row_slot,
                                      const int32_t* query_start, const int32_t* kv_len, int rows, int heads,
                                      int kv_heads, int head_dim, int pages, int page_size, float scale, int window,
                                      int ctas, hb_stream stream);

// bfloat16 attention on tensor cores for rows row0 .. rows - 1, each bringing any number of tokens. q_tiles: at least
// the sum over these rows of ceil(tokens / 64).
int hb_attention_prefill_bf16(void* out, const void* q, const void* kv, const int32_t* block_table, int table_stride,
                              const int32_t* row_slot, const int32_t* query_start, const int32_t* kv_len, int row0,
                              int rows, int q_tiles, int heads, int kv_heads, int head_dim, int pages, int page_size,
                              float scale, int window, hb_stream stream);

// The same rows on tcgen05 tensor cores (scores and output in tensor memory, operands by TMA): head_dim 128, page
// sizes that are multiples of 64. q_tiles: the sum over the rows of ceil(tokens / tile_q); tokens: all tokens of the
// step; tile_q: 256, or 128 for twice the CTAs at half the work each (steps with few query tiles).
// hb_attention_tcgen05_status synchronises the device and returns (and clears) the kernel's bounded-wait status word.
int hb_attention_prefill_tcgen05(void* out, const void* q, const void* kv, const int32_t* block_table, int table_stride,
                                 const int32_t* row_slot, const int32_t* query_start, const int32_t* kv_len, int row0,
                                 int rows, int q_tiles, int tokens, int heads, int kv_heads, int head_dim, int pages,
                                 int page_size, float scale, int window, int tile_q, hb_stream stream);
int hb_attention_tcgen05_status(unsigned int* status);

// out[m, n] = sum_k x[m, k] * w[n, k], all float32, sums in a fixed order that does not depend on m's neighbours.
int hb_gemm_f32(float* out, const float* x, const float* w, int m, int n, int k, hb_stream stream);

// bfloat16 product for at most 16 rows of x, bound by reading w once. mode 0: out [m, n] (bfloat16, or float32 when
// out_f32) = x [m, k] · w [n, k]ᵀ. mode 1: w is [2 inter, k], gate rows first; out [m, inter] = silu(x · gateᵀ) ·
// (x · upᵀ). k a multiple of 8; pointers 16-byte aligned.
int hb_gemm_bf16_skinny(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode, int inter,
                        hb_stream stream);

// The same kernel with the norms around the product folded in. mode 3: h [m, n] (float32) += bfloat16(x · wᵀ),
// out [m, n] = bfloat16(h · (next_weight + next_offset)), ss_out [ceil(n / 16), 16] = sums of squares of the new h
// per 16 columns and token. ss_in (any mode; null: none): x is such an `out` and lacks its row scale
// rsqrt(sum of ss_in [parts_in, 16] over parts / dim_in + eps_in), which is applied to the product's sums.
int hb_gemm_bf16_skinny_linked(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode,
                               int inter, float* h, const void* next_weight, int next_weight_f32, float next_offset,
                               float* ss_out, const float* ss_in, int parts_in, float eps_in, int dim_in,
                               hb_stream stream);

// The attention's first product for up to 16 tokens with what follows it in one kernel: x [m, k] times
// w [(heads + 2 kv_heads) * head_dim, k], then per head the q/k RMSNorm (weights bfloat16 or, with weight_f32, float32;
// null: no norm), the rotation of the whole head by the token's position (table [max_positions, head_dim], cosines
// then sines) and the write of queries to q_out [m, heads, head_dim] and of keys and values into their cache pages.
// head_dim 32, 64 or 128. The head_dim / 16 CTAs of a head are a thread-block cluster.
int hb_qkv_rope_skinny(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions,
                       const float* table, int max_positions, const void* q_weight, const void* k_weight, int weight_f32,
                       float eps, float offset, void* kv, const int32_t* write_index, int pages, int page_size, int heads,
                       int kv_heads, int head_dim, hb_stream stream);
int hb_qkv_rope_skinny_linked(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions,
                              const float* table, int max_positions, const void* q_weight, const void* k_weight,
                              int weight_f32, float eps, float offset, void* kv, const int32_t* write_index, int pages,
                              int page_size, int heads, int kv_heads, int head_dim, const float* ss_in, int parts_in,
                              float eps_in, int dim_in, hb_stream stream);
// The same two for up to 32 rows (four 8-row tiles of x a warp; meant for 17 to 32 rows and weights of a few MB, where a
// product is its launch): ss_in and ss_out hold 32 tokens a part.
int hb_gemm_bf16_skinny32(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode, int inter,
                          float* h, const void* next_weight, int next_weight_f32, float next_offset, float* ss_out,
                          const float* ss_in, int parts_in, float eps_in, int dim_in, hb_stream stream);
int hb_qkv_rope_skinny32(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions,
                         const float* table, int max_positions, const void* q_weight, const void* k_weight, int weight_f32,
                         float eps, float offset, void* kv, const int32_t* write_index, int pages, int page_size, int heads,
                         int kv_heads, int head_dim, const float* ss_in, int parts_in, float eps_in, int dim_in,
                         hb_stream stream);

// Several products of the same few rows, one after the other, as phases of ONE persistent kernel (csrc/gemm_chain.cu):
// the weight stream keeps running across them. A phase is a product of hb_gemm_bf16_skinny_linked (modes 0, 1, 3, same
// meanings of the fields); a phase may read what an earlier phase wrote. sync: two words, zero before the first
// launch; scratch: `slots` x 512 floats; flags: `slots` words, zero before the first launch; none of them may be
// shared with a launch that runs at the same time. hb_gemm_chain_capacity: the most CTAs a launch can have.
typedef struct {
    const void* w; const void* x; void* out; float* h; const void* next_weight; float* ss_out; const float* ss_in;
    int n, k, mode, inter, out_f32, next_weight_f32, parts_in, dim_in;
    float next_offset, eps_in;
} hb_chain_phase;
int hb_gemm_chain_capacity(void);
int hb_gemm_chain(const hb_chain_phase* phases, int n_phases, int m, unsigned int* sync, float* scratch,
                  unsigned int* flags, int slots, int cooperative, hb_stream stream);
int hb_gemm_chain_status(unsigned int* status);

// The same products in one launch whose CTAs each take one tile of one product, in the products' order (tickets drawn
// at the start; csrc/gemm_tickets.cu): a product's CTAs start while the one before ends, ask for their weights and
// wait for its last tile. Up to 4 products; state: 6 words, zero before the first launch.
int hb_gemm_tickets(const hb_chain_phase* phases, int n_phases, int m, unsigned int* state, hb_stream stream);
int hb_gemm_tickets_status(unsigned int* status);

// bfloat16 product on tcgen05 tensor cores with TMA loads and the accumulator in tensor memory (128 x 256 tiles).
// Same arguments and modes as hb_gemm_bf16_skinny, any m. hb_gemm_tcgen05_status synchronises the device and
// returns (and clears) a status word that is non-zero if a bounded wait inside the kernel ever gave up.
int hb_gemm_bf16_tcgen05(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode, int inter,
                         hb_stream stream);
int hb_gemm_tcgen05_status(unsigned int* status);

// The same product by pairs of CTAs on neighbouring SMs (tcgen05 cta_group::2: 256 x 256 tiles, each CTA loading half
// of both operands); same arguments and modes, its own status word.
int hb_gemm_bf16_tcgen05_pair(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode,
                              int inter, hb_stream stream);
int hb_gemm_tcgen05_pair_status(unsigned int* status);
int hb_gemm_tcgen05_pair_width(int bn);             // tests: fix the tile width (0: chosen per launch)

// bfloat16 products of 1 to 64 rows with the following work in their epilogue (csrc/gemm_mid.cu): weight tiles of
// 256 rows on tcgen05, a tile's k range split over a thread-block cluster of `split` CTAs (0: chosen; 1 to 8) that
// sum their partial results through distributed shared memory. mode 0 plain, 1 SwiGLU (w [2 inter, k], gate rows
// first; out [m, inter]), 3 residual sum and next norm (h [m, n] float32 += product; out = bfloat16(h (next_weight +
// next_offset)); ss_out [ceil(n / 256), 64] partial sums of squares of the new h). ss_in [parts_in, stride_in] (null:
// none): x lacks its norm's row scale rsqrt(sum over parts / dim_in + eps_in). hb_qkv_rope_mid: the attention's first
// product with q/k norm, rotation and cache write (arguments as hb_qkv_rope_skinny_linked).
int hb_gemm_bf16_mid(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode, int inter,
                     float* h, const void* next_weight, int next_weight_f32, float next_offset, float* ss_out,
                     const float* ss_in, int parts_in, int stride_in, float eps_in, int dim_in, int split,
                     hb_stream stream);
int hb_qkv_rope_mid(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions, const float* table,
                    int max_positions, const void* q_weight, const void* k_weight, int weight_f32, float eps, float offset,
                    void* kv, const int32_t* write_index, int pages, int page_size, int heads, int kv_heads, int head_dim,
                    const float* ss_in, int parts_in, int stride_in, float eps_in, int dim_in, int split, hb_stream stream);
int hb_gemm_mid_status(unsigned int* status);

// The waits inside the tcgen05 kernels are bounded; one that gives up records (place << 28) | (block + 1) in its
// kernel file's status word (the *_status functions above read those, synchronising) and in one word of page-locked
// host memory that hb_status_word hands out: the host reads it without a copy or a synchronisation, after a step's
// completion event, and may write 0 to it. hb_status_selftest enqueues a wait of `polls` polls on a barrier nobody
// arrives at (place 15): it runs out within microseconds and lets tests see what the host does then.
int hb_status_word(unsigned int** host);
int hb_status_word_device(unsigned int** device);   // the same word as the device addresses it (for a part's own kernel files)
int hb_status_selftest(int polls, hb_stream stream);

// The token each request sampled last, kept on the device by slot. feed: for every row r with from_last[r] != 0,
// token_ids[query_start[r]] = last_tokens[row_slot[r]]. store: last_tokens[slots[i]] = tokens[i] for i < n.
int hb_feed_tokens(int32_t* token_ids, const int32_t* last_tokens, const int32_t* row_slot, const int32_t* query_start,
                   const int32_t* from_last, int rows, hb_stream stream);
int hb_store_tokens(int32_t* last_tokens, const int32_t* slots, const int32_t* tokens, int n, hb_stream stream);

// Block-table rows that changed on the host, uploaded packed: table[slots[i], :] = rows[i, :] for i < n.
int hb_scatter_rows(int32_t* table, const int32_t* slots, const int32_t* rows, int n, int width, int table_rows,
                    hb_stream stream);

// One token per logits row: arg max where temperature is 0, else a draw from softmax(logits / temperature) after the
// filters (when `filtered`), by inverse CDF in vocabulary order with the uniform of (seed, position).
int hb_sample(int32_t* tokens, const float* logits, const float* temperature, const int32_t* top_k,
              const float* top_p, const float* min_p, const int32_t* seed_lo, const int32_t* seed_hi,
              const int32_t* position, int filtered, int rows, int vocab, hb_stream stream);

// Log-probabilities of the raw logits per row: chosen[r] of tokens[r], and the k most likely tokens ranked (equal
// logits by ascending id) as top_ids / top [rows, k]; places beyond the row's finite entries hold id -1 and -inf.
int hb_logprobs(float* chosen, int32_t* top_ids, float* top, const float* logits, const int32_t* tokens, int rows,
                int vocab, int k, hb_stream stream);

#ifdef __cplusplus
}
#endif
