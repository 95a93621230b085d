// Sampling: one block per logits row. Greedy rows take the arg max (the lowest index among equals). Sampled rows
// draw from softmax(logits / temperature) by inverse CDF in vocabulary order: the first token whose cumulative mass
// exceeds u * total, u a hash of (seed, position). Filters keep a set of tokens first: the top_k largest, then the
// smallest set of the most likely whose mass reaches top_p (of the kept mass), then those at least min_p times as
// likely as the best. Each filter is a threshold on the logit, found by a bitwise search over the order-preserving
// integer image of the float, with one deterministic block reduction per bit; no sort, no atomics on floats.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
    return x;
}
__device__ __forceinline__ float uniform_of(uint32_t lo, uint32_t hi, uint32_t pos) {
    const uint32_t h = mix32(mix32(lo) ^ hi ^ mix32(pos));
    const float u = ((float)(h >> 8) + 0.5f) * 5.9604644775390625e-08f;          // 2^-24
    return fminf(u, 1.f - 5.9604644775390625e-08f);
}
// Floats to integers that sort the same way.
__device__ __forceinline__ uint32_t key_of(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned block_count(unsigned v, unsigned* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        unsigned w = lane < (SAMPLE_THREADS >> 5) ? scratch[lane] : 0u;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(
        int32_t* __restrict__ tokens, const float* __restrict__ logits, const float* __restrict__ temperature,
        const int32_t* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
        const int32_t* __restrict__ seed_lo, const int32_t* __restrict__ seed_hi, const int32_t* __restrict__ position,
        int filtered, int vocab) {
    __shared__ float scratch[33];
    __shared__ unsigned uscratch[33];
    __shared__ float warp_mass[SAMPLE_THREADS / 32];
    __shared__ int best_index[33];
    __shared__ int chosen;
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)r * vocab;
    const float temp = temperature[r];

    // ---- the largest logit and its first index
    float best = -INFINITY;
    int arg = vocab;
    if ((vocab & 3) == 0 && (((uintptr_t)x) & 15) == 0) {           // four logits a load, two loads in flight a thread
        const float4* x4 = (const float4*)x;
        const int pieces = vocab >> 2;
        for (int i0 = tid; i0 < pieces; i0 += 2 * SAMPLE_THREADS) {
            const int i1 = i0 + SAMPLE_THREADS;
            const float4 a = x4[i0];
            const float4 b = i1 < pieces ? x4[i1] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            const float va[4] = {a.x, a.y, a.z, a.w}, vb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) if (va[e] > best) { best = va[e]; arg = i0 * 4 + e; }   // (ascending indices: the first of equals)
#pragma unroll
            for (int e = 0; e < 4; ++e) if (vb[e] > best) { best = vb[e]; arg = i1 * 4 + e; }
        }
    } else {
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
            const float v = x[i];
            if (v > best) { best = v; arg = i; }
        }
    }
    const float top = block_max(best, scratch);
    int cand = best == top ? arg : vocab;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    if (lane == 0) best_index[warp] = cand;
    __syncthreads();
    if (warp == 0) {
        int c = lane < (SAMPLE_THREADS >> 5) ? best_index[lane] : vocab;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c = min(c, __shfl_xor_sync(0xffffffffu, c, o));
        if (lane == 0) best_index[32] = c;
    }
    __syncthreads();
    if (temp == 0.f || !(top > -INFINITY)) {
        if (tid == 0) tokens[r] = best_index[32] < vocab ? best_index[32] : 0;
        return;
    }

    const float inv_t = 1.f / temp;
    const float shift = top * inv_t;                     // mass of token i: exp(x_i / T - shift)
    uint32_t floor_key = 0;                              // tokens with key_of(x) >= floor_key are kept ...
    float least = 0.f;                                   // ... if their mass relative to the best is at least this
    if (filtered) {
        const int k = top_k[r];
        if (k > 0 && k < vocab) {                        // the k-th largest key: the largest c with count(key >= c) >= k
            uint32_t c = 0;
            for (int bit = 31; bit >= 0; --bit) {
                const uint32_t trial = c | (1u << bit);
                unsigned n = 0;
                for (int i = tid; i < vocab; i += SAMPLE_THREADS) n += key_of(x[i]) >= trial;
                if (block_count(n, uscratch) >= (unsigned)k) c = trial;
            }
            floor_key = c;
        }
        const float p = top_p[r];
        if (p < 1.f) {                                   // the largest c with mass(key >= c) > p * kept mass
            float z = 0.f;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
                const float v = x[i];
                if (key_of(v) >= floor_key) z += expf(v * inv_t - shift);
            }
            const float target = p * block_sum(z, scratch);
            const uint32_t at_least = floor_key;          // the answer is searched from 0 and never falls below the top-k floor
            uint32_t c = 0;
            for (int bit = 31; bit >= 0; --bit) {
                const uint32_t trial = c | (1u << bit);
                if (trial <= at_least) { c = trial; continue; }
                float mass = 0.f;
                for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
                    const float v = x[i];
                    if (key_of(v) >= trial) mass += expf(v * inv_t - shift);
                }
                if (block_sum(mass, scratch) > target) c = trial;
            }
            floor_key = c > at_least ? c : at_least;
        }
        if (min_p[r] > 0.f) least = min_p[r];          // exp(x/T - shift) >= min_p, tested token by token below
    }

    // ---- the draw: warp w owns the contiguous span [w * span, (w + 1) * span)
    const int warps = SAMPLE_THREADS >> 5;
    const int span = ((vocab + warps - 1) / warps + 31) & ~31;
    const int begin = warp * span, end = min(vocab, begin + span);
    float mass = 0.f;
    for (int i = begin + lane; i < end; i += 32) {
        const float v = x[i];
        if (key_of(v) >= floor_key) { const float e = expf(v * inv_t - shift); if (e >= least) mass += e; }
    }
    mass = warp_sum(mass);
    if (lane == 0) warp_mass[warp] = mass;
    if (tid == 0) chosen = -1;
    __syncthreads();
    float before = 0.f, total = 0.f;                     // every thread sums the warps' masses in the same order
    for (int w = 0; w < warps; ++w) {
        if (w == warp) before = total;
        total += warp_mass[w];
    }
    const float u = uniform_of((uint32_t)seed_lo[r], (uint32_t)seed_hi[r], (uint32_t)position[r]);
    const float target = u * total;
    // the first warp whose running total exceeds the target holds the token
    const bool mine = before <= target && before + warp_mass[warp] > target;
    if (mine) {
        float run = before;
        int found = -1;
        for (int i0 = begin; i0 < end && found < 0; i0 += 32) {
            const int i = i0 + lane;
            float q = 0.f;
            if (i < end) {
                const float v = x[i];
                if (key_of(v) >= floor_key) { const float e = expf(v * inv_t - shift); if (e >= least) q = e; }
            }
            float inc = q;                               // inclusive scan over the 32 lanes
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += up;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, q > 0.f && run + inc > target);
            if (hit) found = i0 + __ffs(hit) - 1;
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (found < 0) {                                 // rounding kept the running sum at the target: the last kept token
            for (int i0 = ((end - 1 - begin) & ~31) + begin; i0 >= begin && found < 0; i0 -= 32) {
                const int i = i0 + lane;
                const bool kept = i < end && key_of(x[i]) >= floor_key && expf(x[i] * inv_t - shift) >= least;
                const unsigned any = __ballot_sync(0xffffffffu, kept);
                if (any) found = i0 + 31 - __clz(any);
            }
        }
        if (lane == 0) chosen = found;
    }
    __syncthreads();
    if (tid == 0) tokens[r] = chosen >= 0 ? chosen : best_index[32];
}

extern "C" int hb_sample(int32_t* tokens, const float* logits, const float* temperature, const int32_t* top_k,
                         const float* top_p, const float* min_p, const int32_t* seed_lo, const int32_t* seed_hi,
                         const int32_t* position, int filtered, int rows, int vocab, hb_stream stream) {
    if (rows == 0) return 0;
    if (vocab < 1) HB_REFUSE("sample: vocab = %d", vocab);
    sample_kernel<<<rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(tokens, logits, temperature, top_k, top_p, min_p,
                                                                    seed_lo, seed_hi, position, filtered, vocab);
    HB_LAUNCH_CHECK("sample");
    return 0;
}

// Log-probabilities of the raw logits (before temperature and filters), one block per row: the chosen token's, and
// the `k` most likely tokens ranked, equal logits by ascending id (std/holon_std/sampling/sampler.py:118-126:
// log_softmax, gather, topk). The largest logit and the sum of exponentials come from block reductions in a fixed
// order; the ranking takes one pass over the row per place, each looking for the best entry after the one before.
__global__ void __launch_bounds__(SAMPLE_THREADS) logprobs_kernel(
        float* __restrict__ chosen, int32_t* __restrict__ top_ids, float* __restrict__ top,
        const float* __restrict__ logits, const int32_t* __restrict__ tokens, int vocab, int k) {
    __shared__ float fs[SAMPLE_THREADS / 32 + 1];
    __shared__ int is[SAMPLE_THREADS / 32 + 1];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)r * vocab;
    auto block_best = [&](float v, int i) {                         // the largest v, the lowest i among equals
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, i, o);
            if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
        }
        __syncthreads();
        if (lane == 0) { fs[warp] = v; is[warp] = i; }
        __syncthreads();
        if (warp == 0) {
            v = lane < SAMPLE_THREADS / 32 ? fs[lane] : -INFINITY;
            i = lane < SAMPLE_THREADS / 32 ? is[lane] : 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, v, o);
                const int oi = __shfl_xor_sync(0xffffffffu, i, o);
                if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
            }
            if (lane == 0) { fs[SAMPLE_THREADS / 32] = v; is[SAMPLE_THREADS / 32] = i; }
        }
        __syncthreads();
    };
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = x[i];
        if (v > best) { best = v; arg = i; }                        // (ascending i: the first of equals stays)
    }
    block_best(best, arg);
    const float top_v = fs[SAMPLE_THREADS / 32];
    const int top_i = is[SAMPLE_THREADS / 32];
    float sum = 0.f;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) sum += expf(x[i] - top_v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncthreads();
    if (lane == 0) fs[warp] = sum;
    __syncthreads();
    if (tid == 0) {
        float total = 0.f;
        for (int w = 0; w < SAMPLE_THREADS / 32; ++w) total += fs[w];
        fs[SAMPLE_THREADS / 32] = top_v + logf(total);
    }
    __syncthreads();
    const float lse = fs[SAMPLE_THREADS / 32];
    if (tid == 0) chosen[r] = x[tokens[r]] - lse;
    float prev_v = top_v;
    int prev_i = top_i;
    for (int j = 0; j < k; ++j) {
        if (j) {
            best = -INFINITY; arg = 0x7fffffff;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
                const float v = x[i];
                const bool after = v < prev_v || (v == prev_v && i > prev_i);
                if (after && v > best) { best = v; arg = i; }
            }
            block_best(best, arg);
            prev_v = fs[SAMPLE_THREADS / 32];
            prev_i = is[SAMPLE_THREADS / 32];
        }
        if (tid == 0) {
            const bool have = prev_i != 0x7fffffff;                  // fewer than k entries (or only NaN) left: -inf, id -1
            top_ids[(size_t)r * k + j] = have ? prev_i : -1;
            top[(size_t)r * k + j] = have ? prev_v - lse : -INFINITY;
        }
    }
}

extern "C" int hb_logprobs(float* chosen, int32_t* top_ids, float* top, const float* logits, const int32_t* tokens,
                           int rows, int vocab, int k, hb_stream stream) {
    if (rows == 0) return 0;
    if (vocab < 1 || k < 0 || k > vocab) HB_REFUSE("logprobs: vocab = %d, k = %d", vocab, k);
    logprobs_kernel<<<rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(chosen, top_ids, top, logits, tokens, vocab, k);
    HB_LAUNCH_CHECK("logprobs");
    return 0;
}
