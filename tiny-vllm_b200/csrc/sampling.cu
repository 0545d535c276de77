// Next-token sampling, a cluster of 8 CTAs per row of logits (each takes an eighth of the
// vocabulary; partial results meet through distributed shared memory): greedy argmax, or
// temperature with optional top-k and top-p and an exponential race as the draw.
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

#include <cstdint>

#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SAMPLE_THREADS 256
#define SAMPLE_WARPS (SAMPLE_THREADS / 32)
#define SAMPLE_CTAS 8           // CTAs (one cluster) that share a row

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

// What the CTAs of a row's cluster tell one another: every reduction below ends with each CTA's
// partial result in slot [buffer][rank] of every CTA's copy, written through distributed shared
// memory, and one cluster barrier; the buffers alternate, so a slot is not written again before
// every CTA has read it (it has to pass the barrier in between).
struct SampleShared {
    float warp_f[SAMPLE_WARPS];
    int warp_i[SAMPLE_WARPS];
    float part_f[2][SAMPLE_CTAS];
    int part_i[2][SAMPLE_CTAS];
};

struct RowTeam {
    cg::cluster_group cluster;
    SampleShared* sh;
    int rank;
    int phase;

    // partial (f, i) of this CTA, held by thread 0, to every CTA of the cluster; then the barrier
    __device__ __forceinline__ void publish(float f, int i) {
        if (threadIdx.x == 0) {
#pragma unroll
            for (int r = 0; r < SAMPLE_CTAS; ++r) {
                SampleShared* other = cluster.map_shared_rank(sh, r);
                other->part_f[phase][rank] = f;
                other->part_i[phase][rank] = i;
            }
        }
        cluster.sync();
    }

    __device__ __forceinline__ int sum(int v) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int delta = 16; delta > 0; delta >>= 1) v += __shfl_xor_sync(0xffffffffu, v, delta);
        __syncthreads();
        if (lane == 0) sh->warp_i[warp] = v;
        __syncthreads();
        int total = 0;
#pragma unroll
        for (int w = 0; w < SAMPLE_WARPS; ++w) total += sh->warp_i[w];
        publish(0.0f, total);
        total = 0;
#pragma unroll
        for (int r = 0; r < SAMPLE_CTAS; ++r) total += sh->part_i[phase][r];
        phase ^= 1;
        return total;
    }

    // warps, then CTAs, in a fixed order
    __device__ __forceinline__ float sum(float v) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        v = warp_sum(v);
        __syncthreads();
        if (lane == 0) sh->warp_f[warp] = v;
        __syncthreads();
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < SAMPLE_WARPS; ++w) total = __fadd_rn(total, sh->warp_f[w]);
        publish(total, 0);
        total = 0.0f;
#pragma unroll
        for (int r = 0; r < SAMPLE_CTAS; ++r) total = __fadd_rn(total, sh->part_f[phase][r]);
        phase ^= 1;
        return total;
    }

    // argmax of (value, smaller index wins ties); every thread of every CTA gets it
    __device__ __forceinline__ void argmax(float& value, int& index) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int delta = 16; delta > 0; delta >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, value, delta);
            const int oi = __shfl_xor_sync(0xffffffffu, index, delta);
            if (ov > value || (ov == value && oi < index)) { value = ov; index = oi; }
        }
        __syncthreads();
        if (lane == 0) { sh->warp_f[warp] = value; sh->warp_i[warp] = index; }
        __syncthreads();
        value = sh->warp_f[0]; index = sh->warp_i[0];
#pragma unroll
        for (int w = 1; w < SAMPLE_WARPS; ++w) {
            const float ov = sh->warp_f[w];
            const int oi = sh->warp_i[w];
            if (ov > value || (ov == value && oi < index)) { value = ov; index = oi; }
        }
        publish(value, index);
        value = sh->part_f[phase][0]; index = sh->part_i[phase][0];
#pragma unroll
        for (int r = 1; r < SAMPLE_CTAS; ++r) {
            const float ov = sh->part_f[phase][r];
            const int oi = sh->part_i[phase][r];
            if (ov > value || (ov == value && oi < index)) { value = ov; index = oi; }
        }
        phase ^= 1;
    }
};

template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const T* logits, int64_t row_stride, int vocab,   // logits: from the kernel before
                   const int* __restrict__ packed, int capacity, int* __restrict__ tokens) {
    __shared__ SampleShared shared;
    RowTeam team{cg::this_cluster(), &shared, (int)(blockIdx.x % SAMPLE_CTAS), 0};
    cluster_arrive();                       // this CTA runs; waited for before the first remote store
    pdl_wait();
    const int row = blockIdx.x / SAMPLE_CTAS, tid = threadIdx.x;
    const T* x = logits + (int64_t)row * row_stride;
    // this CTA's part of the row: whole groups of four tokens (they share a block of noise)
    const int part = ((vocab + SAMPLE_CTAS - 1) / SAMPLE_CTAS + 3) / 4 * 4;
    const int begin = min(vocab, team.rank * part), end = min(vocab, begin + part);

    float best = -INFINITY;
    int best_index = 0x7fffffff;
    int scalar_from = begin;
    if (sizeof(T) == 4 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        // float32 rows on a 16-byte boundary: four logits a load (begin is a multiple of four)
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const int quads_end = end / 4;
#pragma unroll 4
        for (int q = begin / 4 + tid; q < quads_end; q += SAMPLE_THREADS) {
            const float4 v = x4[q];
            if (v.x > best) { best = v.x; best_index = 4 * q; }
            if (v.y > best) { best = v.y; best_index = 4 * q + 1; }
            if (v.z > best) { best = v.z; best_index = 4 * q + 2; }
            if (v.w > best) { best = v.w; best_index = 4 * q + 3; }
        }
        scalar_from = max(begin, quads_end * 4);
    }
    for (int i = scalar_from + tid; i < end; i += SAMPLE_THREADS) {
        const float v = to_float<T>(x[i]);
        if (v > best || (v == best && i < best_index)) { best = v; best_index = i; }
    }
    cluster_wait();
    team.argmax(best, best_index);
    const float temp = __int_as_float(packed[row]);
    if (!(temp > 0.0f) || best_index == 0x7fffffff) {           // the same in every CTA of the row
        if (tid == 0 && team.rank == 0) tokens[row] = best_index == 0x7fffffff ? 0 : best_index;
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
            for (int i = begin + tid; i < end; i += SAMPLE_THREADS) count += ordered_key(SCORE(i)) >= candidate;
            if (team.sum(count) >= k) k_key = candidate;
        }
        int greater = 0, equal = 0;
        for (int i = begin + tid; i < end; i += SAMPLE_THREADS) {
            const uint32_t key = ordered_key(SCORE(i));
            greater += key > k_key;
            equal += key == k_key;
        }
        greater = team.sum(greater);
        equal = team.sum(equal);
        const int wanted = k - greater;
        if (equal > wanted) {              // ties: the first `wanted` of them by token id
            int lo = 0, hi = vocab;
            while (lo < hi) {
                const int mid = lo + (hi - lo) / 2;
                int count = 0;
                for (int i = begin + tid; i < min(end, mid); i += SAMPLE_THREADS) count += ordered_key(SCORE(i)) == k_key;
                if (team.sum(count) >= wanted) hi = mid; else lo = mid + 1;
            }
            k_index_limit = lo;
        }
    }
#define KEPT_K(key, i) (!use_k || (key) > k_key || ((key) == k_key && (i) < k_index_limit))

    // ---- top-p: the smallest key kappa with mass(keys above kappa) <= top_p
    const float p_limit = __int_as_float(packed[capacity + row]);
    uint32_t p_key = 0;
    if (p_limit < 1.0f) {
        float mass = 0.0f;
        for (int i = begin + tid; i < end; i += SAMPLE_THREADS) {
            const float s = SCORE(i);
            if (KEPT_K(ordered_key(s), i)) mass += expf(s);
        }
        const float total = team.sum(mass);
        uint32_t lo = 0, hi = 0xffffffffu;
        while (lo < hi) {
            const uint32_t mid = lo + (hi - lo) / 2;
            float above = 0.0f;
            for (int i = begin + tid; i < end; i += SAMPLE_THREADS) {
                const float s = SCORE(i);
                const uint32_t key = ordered_key(s);
                if (key > mid && KEPT_K(key, i)) above += expf(s);
            }
            above = team.sum(above);
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
    for (int quad = begin / 4 + tid; begin < end && quad * 4 < end; quad += SAMPLE_THREADS) {
        uint32_t words[4];
        philox4x32_10((uint32_t)quad, draw_lo, draw_hi, 0u, seed_lo, seed_hi, words);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = quad * 4 + e;
            if (i >= end) break;
            const float s = SCORE(i);
            const uint32_t key = ordered_key(s);
            if (key < p_key || !KEPT_K(key, i)) continue;
            const float u = __fmul_rn(__fadd_rn((float)(words[e] >> 9), 0.5f), 1.0f / 8388608.0f);
            const float ratio = __fdiv_rn(expf(s), -logf(u));
            if (ratio > win) { win = ratio; win_index = i; }
        }
    }
    team.argmax(win, win_index);
    if (tid == 0 && team.rank == 0) tokens[row] = win_index == 0x7fffffff ? best_index : win_index;
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
    TvbLaunch launch(dim3(rows * SAMPLE_CTAS), dim3(SAMPLE_THREADS), 0, s, pdl, SAMPLE_CTAS);
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
