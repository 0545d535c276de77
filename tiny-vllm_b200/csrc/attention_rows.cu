// Paged causal attention, one warp per (query token, query head): the kernel of
// the float32 path and of every head size the tiled kernels do not take.
//
// The query at position p of a request attends the keys lo..p of that request
// (lo = max(0, p - window + 1) with a window, else 0) through the request's
// block table: key j of kv head g lies at row (table[j / page] * num_kv + g) * page + j % page
// of the cache [pages, num_kv, page, head_dim].  Query head
// h reads kv head h / (num_q / num_kv) (tinyvllm/kernels/paged_decode.cu:120).
// Scores, softmax and the output sum are float32 (:302-356, :457-465).
//
// Keys are processed in chunks of ATTN_CHUNK keys that start at absolute
// multiples of ATTN_CHUNK; every chunk gives a partial (max, sum, output) and the
// partials are merged in ascending order.  A row's arithmetic is therefore the
// same whether its chunks are walked by one warp (mode "rows", prompts) or by
// one warp per chunk with the partials in scratch memory and a merge kernel
// (mode "split", few rows with long contexts): the result at a position does not
// depend on how the tokens were cut into steps or batched.
#include "common.cuh"

#define ATTN_CHUNK 256
#define ATTN_MAX_DIMS 8      // head_dim <= 256: lane l owns dims l, l + 32, ...
#define ATTN_WARPS 4

struct Partial {
    float max, sum;
    float out[ATTN_MAX_DIMS];
};

// running (M, L, O) <- merge with a chunk's (m, l, o); explicit operations so that
// both callers compile to the same arithmetic.
__device__ __forceinline__ void merge_partial(Partial& total, const Partial& part) {
    const float new_max = fmaxf(total.max, part.max);
    const float scale_total = total.max == -INFINITY ? 0.0f : expf(__fsub_rn(total.max, new_max));
    const float scale_part = part.max == -INFINITY ? 0.0f : expf(__fsub_rn(part.max, new_max));
    total.sum = __fadd_rn(__fmul_rn(total.sum, scale_total), __fmul_rn(part.sum, scale_part));
#pragma unroll
    for (int i = 0; i < ATTN_MAX_DIMS; ++i)
        total.out[i] = __fadd_rn(__fmul_rn(total.out[i], scale_total), __fmul_rn(part.out[i], scale_part));
    total.max = new_max;
}


// q . k over one head in ascending order of the dimension; 16-byte loads when the
// head is a whole number of them (the order of additions is the same either way).
template <typename T>
__device__ __forceinline__ float dot_head(const float* __restrict__ q_shared, const T* __restrict__ k,
                                          int head_dim);
template <>
__device__ __forceinline__ float dot_head<float>(const float* __restrict__ q_shared,
                                                 const float* __restrict__ k, int head_dim) {
    float dot = 0.0f;
    if (head_dim % 4 == 0) {
        const float4* k4 = reinterpret_cast<const float4*>(k);
        for (int i = 0; i < head_dim / 4; ++i) {
            const float4 v = k4[i];
            dot = __fmaf_rn(q_shared[4 * i + 0], v.x, dot);
            dot = __fmaf_rn(q_shared[4 * i + 1], v.y, dot);
            dot = __fmaf_rn(q_shared[4 * i + 2], v.z, dot);
            dot = __fmaf_rn(q_shared[4 * i + 3], v.w, dot);
        }
    } else {
        for (int i = 0; i < head_dim; ++i) dot = __fmaf_rn(q_shared[i], k[i], dot);
    }
    return dot;
}
template <>
__device__ __forceinline__ float dot_head<bf16>(const float* __restrict__ q_shared,
                                                const bf16* __restrict__ k, int head_dim) {
    float dot = 0.0f;
    if (head_dim % 8 == 0) {
        const uint4* k8 = reinterpret_cast<const uint4*>(k);
        for (int i = 0; i < head_dim / 8; ++i) {
            const uint4 v = k8[i];
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                // a bfloat16 is the upper half of a float32
                dot = __fmaf_rn(q_shared[8 * i + 2 * w], __uint_as_float(words[w] << 16), dot);
                dot = __fmaf_rn(q_shared[8 * i + 2 * w + 1], __uint_as_float(words[w] & 0xffff0000u), dot);
            }
        }
    } else {
        for (int i = 0; i < head_dim; ++i) dot = __fmaf_rn(q_shared[i], __bfloat162float(k[i]), dot);
    }
    return dot;
}

// One chunk of keys [first, last] (inclusive, inside one ATTN_CHUNK block) for one row.
template <typename T>
__device__ __forceinline__ void attend_chunk(
    Partial& part, const float* __restrict__ q_shared, const T* __restrict__ key_cache,
    const T* __restrict__ value_cache, const int* __restrict__ table, int first, int last,
    int kv_head, int num_kv, int head_dim, int page_size, float scale, int lane) {
    part.max = -INFINITY;
    part.sum = 0.0f;
#pragma unroll
    for (int i = 0; i < ATTN_MAX_DIMS; ++i) part.out[i] = 0.0f;
    for (int base = first - first % 32; base <= last; base += 32) {
        const int j = base + lane;
        const bool valid = j >= first && j <= last;
        int64_t slot = 0;
        float score = -INFINITY;
        if (valid) {
            slot = ((int64_t)table[j / page_size] * num_kv + kv_head) * page_size + j % page_size;
            const T* k = key_cache + slot * head_dim;
            score = __fmul_rn(dot_head<T>(q_shared, k, head_dim), scale);
        }
        const float tile_max = warp_max(score);          // at least one key of a tile is valid
        const float new_max = fmaxf(part.max, tile_max);
        const float rescale = part.max == -INFINITY ? 0.0f : expf(__fsub_rn(part.max, new_max));
        const float p = valid ? expf(__fsub_rn(score, new_max)) : 0.0f;
        part.sum = __fadd_rn(__fmul_rn(part.sum, rescale), warp_sum(p));
#pragma unroll
        for (int i = 0; i < ATTN_MAX_DIMS; ++i) part.out[i] = __fmul_rn(part.out[i], rescale);
        const int count = min(32, last - base + 1);
        for (int jj = max(0, first - base); jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int64_t sj = __shfl_sync(0xffffffffu, slot, jj);
            const T* v = value_cache + sj * head_dim;
#pragma unroll
            for (int i = 0; i < ATTN_MAX_DIMS; ++i) {
                const int dim = lane + 32 * i;
                if (dim < head_dim) part.out[i] = __fmaf_rn(pj, to_float<T>(v[dim]), part.out[i]);
            }
        }
        part.max = new_max;
    }
}

// mode rows: grid.x covers (token, head) rows, grid.y = 1, each warp walks all chunks.
// mode split: grid.y = chunk index; partials go to scratch.
template <typename T, bool SPLIT>
__global__ void paged_attention_rows_kernel(
    const T* __restrict__ q, int64_t q_token_stride, const T* __restrict__ key_cache,
    const T* __restrict__ value_cache, const int* __restrict__ block_tables, int table_stride,
    const int* __restrict__ token_row, const int* __restrict__ positions, T* __restrict__ out,
    float* __restrict__ scratch, int max_chunks, int tokens, int num_q, int num_kv, int head_dim,
    int page_size, int window, float scale) {
    __shared__ float q_shared[ATTN_WARPS][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * ATTN_WARPS + warp;
    if (row >= (int64_t)tokens * num_q) return;
    const int token = (int)(row / num_q), head = (int)(row % num_q);
    const int position = positions[token];
    const int request = token_row[token];
    T* out_row = out + row * head_dim;
    if (request < 0 || position < 0) {            // padding row of a captured batch
        if (!SPLIT || blockIdx.y == 0)
            for (int i = lane; i < head_dim; i += 32) out_row[i] = from_float<T>(0.0f);
        return;
    }
    const int lo = window > 0 ? max(0, position - window + 1) : 0;
    const int first_chunk = lo / ATTN_CHUNK, last_chunk = position / ATTN_CHUNK;
    if (SPLIT && ((int)blockIdx.y < first_chunk || (int)blockIdx.y > last_chunk)) return;
    const T* q_row = q + (int64_t)token * q_token_stride + (int64_t)head * head_dim;
    for (int i = lane; i < head_dim; i += 32) q_shared[warp][i] = to_float<T>(q_row[i]);
    __syncwarp();
    const int* table = block_tables + (int64_t)request * table_stride;
    const int kv_head = head / (num_q / num_kv);

    if (SPLIT) {
        const int chunk = blockIdx.y;
        Partial part;
        attend_chunk<T>(part, q_shared[warp], key_cache, value_cache, table,
                        max(lo, chunk * ATTN_CHUNK), min(position, chunk * ATTN_CHUNK + ATTN_CHUNK - 1),
                        kv_head, num_kv, head_dim, page_size, scale, lane);
        float* dst = scratch + (row * max_chunks + chunk) * (int64_t)(head_dim + 2);
        if (lane == 0) { dst[0] = part.max; dst[1] = part.sum; }
#pragma unroll
        for (int i = 0; i < ATTN_MAX_DIMS; ++i) {
            const int dim = lane + 32 * i;
            if (dim < head_dim) dst[2 + dim] = part.out[i];
        }
    } else {
        Partial total;
        total.max = -INFINITY;
        total.sum = 0.0f;
#pragma unroll
        for (int i = 0; i < ATTN_MAX_DIMS; ++i) total.out[i] = 0.0f;
        for (int chunk = first_chunk; chunk <= last_chunk; ++chunk) {
            Partial part;
            attend_chunk<T>(part, q_shared[warp], key_cache, value_cache, table,
                            max(lo, chunk * ATTN_CHUNK), min(position, chunk * ATTN_CHUNK + ATTN_CHUNK - 1),
                            kv_head, num_kv, head_dim, page_size, scale, lane);
            merge_partial(total, part);
        }
#pragma unroll
        for (int i = 0; i < ATTN_MAX_DIMS; ++i) {
            const int dim = lane + 32 * i;
            if (dim < head_dim) out_row[dim] = from_float<T>(__fdiv_rn(total.out[i], total.sum));
        }
    }
}

template <typename T>
__global__ void merge_attention_rows_kernel(const float* __restrict__ scratch, int max_chunks,
                                            const int* __restrict__ token_row,
                                            const int* __restrict__ positions, T* __restrict__ out,
                                            int tokens, int num_q, int head_dim, int window) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * ATTN_WARPS + warp;
    if (row >= (int64_t)tokens * num_q) return;
    const int token = (int)(row / num_q);
    const int position = positions[token];
    if (token_row[token] < 0 || position < 0) return;     // zeros were written by the first kernel
    const int lo = window > 0 ? max(0, position - window + 1) : 0;
    Partial total;
    total.max = -INFINITY;
    total.sum = 0.0f;
#pragma unroll
    for (int i = 0; i < ATTN_MAX_DIMS; ++i) total.out[i] = 0.0f;
    // The scratch holds max_chunks partials a row.  A caller whose max_chunks is too small for this
    // row's position gets the row as NaN: the first kernel wrote no partial beyond max_chunks - 1,
    // and reading on would take the next row's (or leave the buffer).
    const int last_chunk = position / ATTN_CHUNK;
    if (last_chunk >= max_chunks) {
        T* bad_row = out + row * head_dim;
        for (int dim = lane; dim < head_dim; dim += 32) bad_row[dim] = from_float<T>(__int_as_float(0x7fc00000));
        return;
    }
    for (int chunk = lo / ATTN_CHUNK; chunk <= last_chunk; ++chunk) {
        const float* src = scratch + (row * max_chunks + chunk) * (int64_t)(head_dim + 2);
        Partial part;
        part.max = src[0];
        part.sum = src[1];
#pragma unroll
        for (int i = 0; i < ATTN_MAX_DIMS; ++i) {
            const int dim = lane + 32 * i;
            part.out[i] = dim < head_dim ? src[2 + dim] : 0.0f;
        }
        merge_partial(total, part);
    }
    T* out_row = out + row * head_dim;
#pragma unroll
    for (int i = 0; i < ATTN_MAX_DIMS; ++i) {
        const int dim = lane + 32 * i;
        if (dim < head_dim) out_row[dim] = from_float<T>(__fdiv_rn(total.out[i], total.sum));
    }
}

extern "C" int tvb_attention_chunk_keys() { return ATTN_CHUNK; }

// scratch floats the split mode needs: tokens * num_q * max_chunks * (head_dim + 2)
extern "C" long long tvb_attention_rows_scratch_floats(int tokens, int num_q, int head_dim, int max_chunks) {
    return (long long)tokens * num_q * max_chunks * (head_dim + 2);
}

// max_chunks = 0 selects mode rows (no scratch).  Otherwise max_chunks must be at
// least ceil((largest position + 1) / ATTN_CHUNK) of the batch and scratch must hold
// tokens * num_q * max_chunks * (head_dim + 2) floats.  The host cannot see the positions:
// a row whose position needs more chunks than max_chunks is written as NaN (and nothing
// outside the stated scratch is read or written).
extern "C" int tvb_attention_rows(const void* q, long long q_token_stride, const void* key_cache,
                                  const void* value_cache, const int* block_tables, int table_stride,
                                  const int* token_row, const int* positions, void* out,
                                  float* scratch, int max_chunks, int tokens, int num_q, int num_kv,
                                  int head_dim, int page_size, int window, float scale, int dtype,
                                  void* stream) {
    if (tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim > 32 * ATTN_MAX_DIMS || num_q <= 0 || num_kv <= 0 ||
        num_q % num_kv || page_size <= 0 || max_chunks < 0 || max_chunks > 65535 ||
        (max_chunks > 0 && !scratch))
        return TVB_BAD_ARGUMENT;
    const int64_t rows = (int64_t)tokens * num_q;
    const int64_t blocks = (rows + ATTN_WARPS - 1) / ATTN_WARPS;
    if (blocks > 2147483647LL) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((unsigned)blocks, max_chunks > 0 ? max_chunks : 1);
#define LAUNCH_ROWS(T)                                                                              \
    do {                                                                                            \
        if (max_chunks > 0) {                                                                       \
            paged_attention_rows_kernel<T, true><<<grid, ATTN_WARPS * 32, 0, s>>>(                  \
                (const T*)q, q_token_stride, (const T*)key_cache, (const T*)value_cache,            \
                block_tables, table_stride, token_row, positions, (T*)out, scratch, max_chunks,     \
                tokens, num_q, num_kv, head_dim, page_size, window, scale);                         \
            merge_attention_rows_kernel<T><<<(unsigned)blocks, ATTN_WARPS * 32, 0, s>>>(            \
                scratch, max_chunks, token_row, positions, (T*)out, tokens, num_q, head_dim, window); \
        } else {                                                                                    \
            paged_attention_rows_kernel<T, false><<<grid, ATTN_WARPS * 32, 0, s>>>(                 \
                (const T*)q, q_token_stride, (const T*)key_cache, (const T*)value_cache,            \
                block_tables, table_stride, token_row, positions, (T*)out, scratch, max_chunks,     \
                tokens, num_q, num_kv, head_dim, page_size, window, scale);                         \
        }                                                                                           \
    } while (0)
    if (dtype == TVB_F32) LAUNCH_ROWS(float);
    else if (dtype == TVB_BF16) LAUNCH_ROWS(bf16);
    else return TVB_BAD_ARGUMENT;
#undef LAUNCH_ROWS
    return tvb_last_error();
}

// ------------------------------------------------ entry point that allocates nothing
// See attention_rows_static.h for who needs this and how to use it.
#include "attention_rows_static.h"

// The scratch of the split mode, held by every GPU that loads this library until exit.
static __device__ __align__(256) float tvb_static_scratch[TVB_STATIC_SCRATCH_FLOATS];

// In host code `tvb_static_scratch` is only a stand-in for the symbol, not a device address:
// the address is asked for once per device, with that device current, and kept here.
#define TVB_STATIC_MAX_DEVICES 64
static float* tvb_static_scratch_address[TVB_STATIC_MAX_DEVICES];

static int tvb_static_scratch_of_current_device(float** address) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= TVB_STATIC_MAX_DEVICES) return TVB_BAD_ARGUMENT;
    if (!tvb_static_scratch_address[device]) {
        float* found = nullptr;
        e = cudaGetSymbolAddress((void**)&found, tvb_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!found) return (int)cudaErrorInvalidSymbol;
        tvb_static_scratch_address[device] = found;
    }
    *address = tvb_static_scratch_address[device];
    return 0;
}

extern "C" long long tvb_attention_rows_static_capacity(void) { return TVB_STATIC_SCRATCH_FLOATS; }

extern "C" const char* tvb_attention_rows_static_error(int code) {
    if (code == 0) return "ok";
    if (code == TVB_STATIC_SCRATCH_TOO_SMALL)
        return "the partials of this batch (tokens * num_q * max_chunks * (head_dim + 2) floats) do not fit "
               "into the library's built-in scratch of 4 Mi floats; use tvb_attention_rows with a buffer of "
               "your own, or fewer tokens per call";
    if (code == TVB_BAD_ARGUMENT)
        return "sizes this kernel does not take (or max_chunks == 0, which needs no scratch: call "
               "tvb_attention_rows)";
    return cudaGetErrorString((cudaError_t)code);
}

extern "C" int tvb_attention_rows_static(const void* q, long long q_token_stride, const void* key_cache,
                                         const void* value_cache, const int* block_tables, int table_stride,
                                         const int* token_row, const int* positions, void* out,
                                         int max_chunks, int tokens, int num_q, int num_kv, int head_dim,
                                         int page_size, int window, float scale, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    // bounds first, so that the product below cannot overflow
    if (max_chunks <= 0 || max_chunks > 65535 || num_q <= 0 || num_q > 65535 || head_dim <= 0 ||
        head_dim > 32 * ATTN_MAX_DIMS)
        return TVB_BAD_ARGUMENT;
    if (tokens > TVB_STATIC_SCRATCH_FLOATS) return TVB_STATIC_SCRATCH_TOO_SMALL;      // every token needs floats
    if (tvb_attention_rows_scratch_floats(tokens, num_q, head_dim, max_chunks) > TVB_STATIC_SCRATCH_FLOATS)
        return TVB_STATIC_SCRATCH_TOO_SMALL;
    float* scratch = nullptr;
    const int status = tvb_static_scratch_of_current_device(&scratch);
    if (status != 0) return status;
    // the launcher below only checks sizes and launches the two kernels
    return tvb_attention_rows(q, q_token_stride, key_cache, value_cache, block_tables, table_stride,
                              token_row, positions, out, scratch, max_chunks, tokens, num_q, num_kv,
                              head_dim, page_size, window, scale, dtype, stream);
}
