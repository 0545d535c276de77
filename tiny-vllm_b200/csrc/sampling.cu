// Next-token sampling, one block per row of logits: greedy argmax, or temperature
// with optional top-k and top-p and an exponential race as the draw.
//
// Follows tinyvllm/sampling.py: argmax for temperature 0 (:42-43); scores =
// (logits - max) / temperature in float32 (:82-104); the k largest scores stay
// (:107-112); softmax over them; a token stays under top-p while the mass of the
// tokens sorted before it does not exceed top_p (:125-139); the draw is
// argmax(p / noise), noise ~ Exp(1) (:141-157).  Ties go to the smaller token id.
// Ties exactly at the top-p boundary all stay.
//
// The noise is counter-based instead of a generator carried from step to step:
// token i of draw number n of a request with seed s takes word i % 4 of
// Philox-4x32-10(counter = (i / 4, n_lo, n_hi, 0), key = (s_lo, s_hi)),
// u = ((word >> 9) + 0.5) / 2^23, noise = -log(u).  A request's tokens thus do not
// depend on what else is in the batch or on the order of the rows.
//
// No sort: thresholds are found by bisection over the ordered bit pattern of the
// scores, each probe being one pass over the row.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ uint32_t ordered_key(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int delta = 16; delta > 0; delta >>= 1) v += __shfl_xor_sync(0xffffffffu, v, delta);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int total = lane < (SAMPLE_THREADS >> 5) ? scratch[lane] : 0;
#pragma unroll
    for (int delta = 16; delta > 0; delta >>= 1) total += __shfl_xor_sync(0xffffffffu, total, delta);
    return total;
}

// argmax of (value, smaller index wins ties) over the block; every thread gets it
__device__ __forceinline__ void block_argmax(float& value, int& index, float* vals, int* idxs) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int delta = 16; delta > 0; delta >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, value, delta);
        const int oi = __shfl_xor_sync(0xffffffffu, index, delta);
        if (ov > value || (ov == value && oi < index)) { value = ov; index = oi; }
    }
    __syncthreads();
    if (lane == 0) { vals[warp] = value; idxs[warp] = index; }
    __syncthreads();
    value = lane < (SAMPLE_THREADS >> 5) ? vals[lane] : -INFINITY;
    index = lane < (SAMPLE_THREADS >> 5) ? idxs[lane] : 0x7fffffff;
#pragma unroll
    for (int delta = 16; delta > 0; delta >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, value, delta);
        const int oi = __shfl_xor_sync(0xffffffffu, index, delta);
        if (ov > value || (ov == value && oi < index)) { value = ov; index = oi; }
    }
}

template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS, 1)
sample_rows_kernel(const T* logits, int64_t row_stride, int vocab,   // logits: from the kernel before
                   const int* __restrict__ packed, int capacity, int* __restrict__ tokens) {
    __shared__ float fscratch[32];
    __shared__ int iscratch[32];
    pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const T* x = logits + (int64_t)row * row_stride;

    float best = -INFINITY;
    int best_index = 0x7fffffff;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = to_float<T>(x[i]);
        if (v > best) { best = v; best_index = i; }
    }
    block_argmax(best, best_index, fscratch, iscratch);
    const float temp = __int_as_float(packed[row]);
    if (!(temp > 0.0f) || best_index == 0x7fffffff) {
        if (tid == 0) tokens[row] = best_index == 0x7fffffff ? 0 : best_index;
        return;
    }
    const float row_max = best;
#define SCORE(i) __fdiv_rn(__fsub_rn(to_float<T>(x[i]), row_max), temp)

    // ---- top-k: the k-th largest key, then how many of its equals stay
    const int k = packed[2 * capacity + row];
    const bool use_k = k > 0 && k < vocab;
    uint32_t k_key = 0;
    int k_index_limit = vocab;
    if (use_k) {
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t candidate = k_key | (1u << bit);
            int count = 0;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) count += ordered_key(SCORE(i)) >= candidate;
            if (block_sum_int(count, iscratch) >= k) k_key = candidate;
        }
        int greater = 0, equal = 0;
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
            const uint32_t key = ordered_key(SCORE(i));
            greater += key > k_key;
            equal += key == k_key;
        }
        greater = block_sum_int(greater, iscratch);
        equal = block_sum_int(equal, iscratch);
        const int wanted = k - greater;
        if (equal > wanted) {              // ties: the first `wanted` of them by token id
            int lo = 0, hi = vocab;
            while (lo < hi) {
                const int mid = lo + (hi - lo) / 2;
                int count = 0;
                for (int i = tid; i < mid; i += SAMPLE_THREADS) count += ordered_key(SCORE(i)) == k_key;
                if (block_sum_int(count, iscratch) >= wanted) hi = mid; else lo = mid + 1;
            }
            k_index_limit = lo;
        }
    }
#define KEPT_K(key, i) (!use_k || (key) > k_key || ((key) == k_key && (i) < k_index_limit))

    // ---- top-p: the smallest key kappa with mass(keys above kappa) <= top_p
    const float p_limit = __int_as_float(packed[capacity + row]);
    uint32_t p_key = 0;
    if (p_limit < 1.0f) {
        float part = 0.0f;
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
            const float s = SCORE(i);
            if (KEPT_K(ordered_key(s), i)) part += expf(s);
        }
        const float total = block_sum(part, fscratch);
        uint32_t lo = 0, hi = 0xffffffffu;
        while (lo < hi) {
            const uint32_t mid = lo + (hi - lo) / 2;
            float above = 0.0f;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
                const float s = SCORE(i);
                const uint32_t key = ordered_key(s);
                if (key > mid && KEPT_K(key, i)) above += expf(s);
            }
            above = block_sum(above, fscratch);
            if (__fdiv_rn(above, total) <= p_limit) hi = mid; else lo = mid + 1;
        }
        p_key = lo;
    }

    // ---- the race
    const uint32_t seed_lo = (uint32_t)packed[3 * capacity + row], seed_hi = (uint32_t)packed[4 * capacity + row];
    const uint32_t draw_lo = (uint32_t)packed[5 * capacity + row], draw_hi = (uint32_t)packed[6 * capacity + row];
    float win = -INFINITY;
    int win_index = 0x7fffffff;
    // a thread takes four consecutive tokens at a time: they share one Philox block
    for (int quad = tid; quad * 4 < vocab; quad += SAMPLE_THREADS) {
        uint32_t words[4];
        philox4x32_10((uint32_t)quad, draw_lo, draw_hi, 0u, seed_lo, seed_hi, words);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = quad * 4 + e;
            if (i >= vocab) break;
            const float s = SCORE(i);
            const uint32_t key = ordered_key(s);
            if (key < p_key || !KEPT_K(key, i)) continue;
            const float u = __fmul_rn(__fadd_rn((float)(words[e] >> 9), 0.5f), 1.0f / 8388608.0f);
            const float ratio = __fdiv_rn(expf(s), -logf(u));
            if (ratio > win) { win = ratio; win_index = i; }
        }
    }
    block_argmax(win, win_index, fscratch, iscratch);
    if (tid == 0) tokens[row] = win_index == 0x7fffffff ? best_index : win_index;
#undef SCORE
#undef KEPT_K
}

// packed: int32 [7, capacity], field-major: temperature and top_p as float bits, top_k,
// seed low/high word, draw-counter low/high word; row r reads column r.
extern "C" int tvb_sample_rows(const void* logits, long long row_stride, int rows, int vocab,
                               const int* packed, int capacity, int* tokens, int dtype, int pdl,
                               void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || capacity < rows) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    TvbLaunch launch(dim3(rows), dim3(SAMPLE_THREADS), 0, s, pdl);
    cudaError_t e;
    if (dtype == TVB_F32)
        e = cudaLaunchKernelEx(&launch.config, sample_rows_kernel<float>, (const float*)logits,
                               (int64_t)row_stride, vocab, packed, capacity, tokens);
    else if (dtype == TVB_BF16)
        e = cudaLaunchKernelEx(&launch.config, sample_rows_kernel<bf16>, (const bf16*)logits,
                               (int64_t)row_stride, vocab, packed, capacity, tokens);
    else
        return TVB_BAD_ARGUMENT;
    return e == cudaSuccess ? tvb_last_error() : (int)e;
}
