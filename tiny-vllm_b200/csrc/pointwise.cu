// Memory-bound kernels of a decoder step: embedding rows, (residual +) RMSNorm,
// SiLU(gate) * up, rotary tables, and per-head q/k RMSNorm + rotation fused with
// the write of keys and values into their cache pages.
//
// Formulas and rounding points follow tinyvllm/kernels/pointwise.cu:94-116
// (rotation), :153-211 (RMSNorm), :274-285 (SiLU * up) and
// tinyvllm/kernels/kv_store.cu:26-90 (cache write).  Sums, the reciprocal root
// and the rotation run in float32; 1/sqrt is the correctly rounded division of a
// correctly rounded root, so that the float32 path shows no approximation.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                  T* __restrict__ out, int width, int vocab) {
    const int row = blockIdx.x;
    int id = ids[row];
    if (id < 0 || id >= vocab) id = 0;   // the host validates ids; padding rows carry 0
    const T* src = table + (int64_t)id * width;
    T* dst = out + (int64_t)row * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

extern "C" int tvb_embed_rows(const void* table, const int* ids, void* out, int rows, int width,
                              int vocab, int dtype, void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || vocab <= 0) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == TVB_F32)
        embed_rows_kernel<float><<<rows, threads, 0, s>>>((const float*)table, ids, (float*)out, width, vocab);
    else if (dtype == TVB_BF16)
        embed_rows_kernel<bf16><<<rows, threads, 0, s>>>((const bf16*)table, ids, (bf16*)out, width, vocab);
    else
        return TVB_BAD_ARGUMENT;
    return tvb_last_error();
}

// -------------------------------------------------------------------- RMSNorm
// One block per output row.  `gather` (optional) picks the input row of each
// output row, so the last norm runs on the wanted rows only.  With `residual`
// the rounded sum x + residual is normalised and, if `residual_out` is given,
// stored as the new residual stream.
template <typename T, typename W>
__global__ void rms_norm_kernel(const T* x, const T* residual,   // written by the kernel before
                                
                                const W* __restrict__ weight, T* __restrict__ y,
                                T* __restrict__ residual_out, const int* __restrict__ gather,
                                int width, float eps) {
    extern __shared__ float row_values[];
    __shared__ float scratch[32];
    pdl_wait();
    pdl_launch_dependents();
    const int out_row = blockIdx.x;
    const int in_row = gather ? gather[out_row] : out_row;
    const T* xr = x + (int64_t)in_row * width;
    const T* rr = residual ? residual + (int64_t)in_row * width : nullptr;
    float part = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = to_float<T>(xr[i]);
        if (rr) v = round_to<T>(__fadd_rn(v, to_float<T>(rr[i])));
        row_values[i] = v;
        part = __fadd_rn(part, __fmul_rn(v, v));
    }
    const float total = block_sum(part, scratch);
    const float variance = __fmul_rn(total, 1.0f / (float)width);
    const float inverse_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(variance, eps)));
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = row_values[i];
        if (residual_out) residual_out[(int64_t)out_row * width + i] = from_float<T>(v);
        const float normalised = round_to<T>(__fmul_rn(v, inverse_rms));
        y[(int64_t)out_row * width + i] = from_float<T>(__fmul_rn(normalised, to_float<W>(weight[i])));
    }
}

template <typename T, typename W>
static int launch_rms_norm(const void* x, const void* residual, const void* weight, void* y,
                           void* residual_out, const int* gather, int rows, int width, float eps,
                           int pdl, cudaStream_t s) {
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return TVB_BAD_ARGUMENT;
    auto kernel = rms_norm_kernel<T, W>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : (width >= 128 ? 128 : 32));
    TvbLaunch launch(dim3(rows), dim3(threads), smem, s, pdl);
    cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, (const T*)x, (const T*)residual,
                                       (const W*)weight, (T*)y, (T*)residual_out, gather, width, eps);
    return e == cudaSuccess ? tvb_last_error() : (int)e;
}

// weight_dtype may differ from dtype: a norm weight stored in 32-bit stays 32-bit.
extern "C" int tvb_rms_norm(const void* x, const void* residual, const void* weight, void* y,
                            void* residual_out, const int* gather, int rows, int width, float eps,
                            int dtype, int weight_dtype, int pdl, void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TVB_F32 && weight_dtype == TVB_F32)
        return launch_rms_norm<float, float>(x, residual, weight, y, residual_out, gather, rows, width, eps, pdl, s);
    if (dtype == TVB_BF16 && weight_dtype == TVB_BF16)
        return launch_rms_norm<bf16, bf16>(x, residual, weight, y, residual_out, gather, rows, width, eps, pdl, s);
    if (dtype == TVB_BF16 && weight_dtype == TVB_F32)
        return launch_rms_norm<bf16, float>(x, residual, weight, y, residual_out, gather, rows, width, eps, pdl, s);
    return TVB_BAD_ARGUMENT;
}

// --------------------------------------------------------------- SiLU(gate)*up
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
    const int64_t row = blockIdx.y;
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= inter) return;
    const T* src = gate_up + row * 2 * inter;
    const float gate = to_float<T>(src[col]);
    const float up = to_float<T>(src[col + inter]);
    const float activated = round_to<T>(__fdiv_rn(gate, __fadd_rn(1.0f, expf(-gate))));
    out[row * inter + col] = from_float<T>(__fmul_rn(activated, up));
}

extern "C" int tvb_silu_mul(const void* gate_up, void* out, int rows, int inter, int dtype, void* stream) {
    if (rows <= 0) return 0;
    if (inter <= 0 || rows > 65535 * 32) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    // grid.y is limited to 65535 rows; longer batches go in slices
    for (int first = 0; first < rows; first += 65535) {
        const int count = rows - first < 65535 ? rows - first : 65535;
        dim3 grid((inter + 255) / 256, count);
        if (dtype == TVB_F32)
            silu_mul_kernel<float><<<grid, 256, 0, s>>>((const float*)gate_up + (int64_t)first * 2 * inter,
                                                        (float*)out + (int64_t)first * inter, inter);
        else if (dtype == TVB_BF16)
            silu_mul_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)gate_up + (int64_t)first * 2 * inter,
                                                       (bf16*)out + (int64_t)first * inter, inter);
        else
            return TVB_BAD_ARGUMENT;
    }
    return tvb_last_error();
}

// --------------------------------------------------------------- rotary tables
// cos/sin of position * inv_freq[j] in float32, [positions, half]
// (tinyvllm/layers.py:192-226).  inv_freq comes from the host.
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float* __restrict__ cos_out,
                                  float* __restrict__ sin_out, int positions, int half) {
    const int64_t index = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= (int64_t)positions * half) return;
    const int p = (int)(index / half), j = (int)(index % half);
    const float angle = __fmul_rn((float)p, inv_freq[j]);
    cos_out[index] = cosf(angle);
    sin_out[index] = sinf(angle);
}

extern "C" int tvb_rope_table(const float* inv_freq, float* cos_out, float* sin_out, int positions,
                              int half, void* stream) {
    if (positions <= 0 || half <= 0) return TVB_BAD_ARGUMENT;
    const int64_t total = (int64_t)positions * half;
    rope_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        inv_freq, cos_out, sin_out, positions, half);
    return tvb_last_error();
}

// ------------------------------------- q/k norm + rotation + cache write, fused
// One warp per (token, head) over the packed projection row
// [q heads | k heads | v heads].  q heads are normalised and rotated in place;
// k heads are normalised, rotated and written to the key cache [pages, num_kv, page,
// head_dim] at the token's slot (page * page_size + offset); v heads are copied to the
// value cache.  Lane l holds the pairs
// (j, j + d/2) for j = l, l + 32, ...  Null norm weights skip the norm, null
// tables skip the rotation, null slots (or a negative slot) skip the writes.
#define QK_MAX_PAIRS 4   // head_dim <= 256

template <typename T, typename W>
__global__ void qk_norm_rope_store_kernel(
    T* __restrict__ qkv, const W* __restrict__ q_weight, const W* __restrict__ k_weight,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table,
    const int* __restrict__ positions, const int* __restrict__ slots,
    T* __restrict__ key_cache, T* __restrict__ value_cache,
    int tokens, int num_q, int num_kv, int head_dim, int page_size, int table_positions, float eps) {
    const int heads = num_q + 2 * num_kv;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= (int64_t)tokens * heads) return;
    const int lane = threadIdx.x & 31;
    const int token = (int)(row / heads), head = (int)(row % heads);
    const int half = head_dim >> 1;
    T* src = qkv + ((int64_t)token * heads + head) * head_dim;
    const int slot = slots ? slots[token] : -1;

    if (head >= num_q + num_kv) {            // a value head: plain copy
        if (slot < 0) return;
        T* dst = value_cache + (((int64_t)(slot / page_size) * num_kv + (head - num_q - num_kv)) * page_size +
                                slot % page_size) * head_dim;
        for (int i = lane; i < head_dim; i += 32) dst[i] = src[i];
        return;
    }
    const bool is_key = head >= num_q;
    if (is_key && slot < 0) return;
    const W* weight = is_key ? k_weight : q_weight;

    float first[QK_MAX_PAIRS], second[QK_MAX_PAIRS];
    float squares = 0.0f;
#pragma unroll
    for (int i = 0; i < QK_MAX_PAIRS; ++i) {
        const int j = lane + 32 * i;
        first[i] = second[i] = 0.0f;
        if (j < half) {
            first[i] = to_float<T>(src[j]);
            second[i] = to_float<T>(src[j + half]);
            squares = __fadd_rn(squares, __fadd_rn(__fmul_rn(first[i], first[i]),
                                                   __fmul_rn(second[i], second[i])));
        }
    }
    if (weight) {
        squares = warp_sum(squares);
        const float variance = __fmul_rn(squares, 1.0f / (float)head_dim);
        const float inverse_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(variance, eps)));
#pragma unroll
        for (int i = 0; i < QK_MAX_PAIRS; ++i) {
            const int j = lane + 32 * i;
            if (j < half) {
                first[i] = round_to<T>(__fmul_rn(round_to<T>(__fmul_rn(first[i], inverse_rms)),
                                                 to_float<W>(weight[j])));
                second[i] = round_to<T>(__fmul_rn(round_to<T>(__fmul_rn(second[i], inverse_rms)),
                                                  to_float<W>(weight[j + half])));
            }
        }
    }
    T* dst = is_key ? key_cache + (((int64_t)(slot / page_size) * num_kv + (head - num_q)) * page_size +
                                   slot % page_size) * head_dim
                    : src;
    int position = positions[token];
    if (position < 0) position = 0;
    if (position >= table_positions) position = table_positions - 1;   // the host refuses these
#pragma unroll
    for (int i = 0; i < QK_MAX_PAIRS; ++i) {
        const int j = lane + 32 * i;
        if (j < half) {
            float a = first[i], b = second[i];
            if (cos_table) {
                const float c = round_to<T>(cos_table[(int64_t)position * half + j]);
                const float s = round_to<T>(sin_table[(int64_t)position * half + j]);
                const float ac = round_to<T>(__fmul_rn(a, c)), bs = round_to<T>(__fmul_rn(b, s));
                const float bc = round_to<T>(__fmul_rn(b, c)), as = round_to<T>(__fmul_rn(a, s));
                a = __fsub_rn(ac, bs);
                b = __fadd_rn(bc, as);
            }
            dst[j] = from_float<T>(a);
            dst[j + half] = from_float<T>(b);
        }
    }
}

template <typename T, typename W>
static int launch_qk(void* qkv, const void* qw, const void* kw, const float* cos_table,
                     const float* sin_table, const int* positions, const int* slots, void* key_cache,
                     void* value_cache, int tokens, int num_q, int num_kv, int head_dim, int page_size,
                     int table_positions, float eps, cudaStream_t s) {
    const int64_t rows = (int64_t)tokens * (num_q + 2 * num_kv);
    const int warps = 4;
    qk_norm_rope_store_kernel<T, W><<<(unsigned)((rows + warps - 1) / warps), warps * 32, 0, s>>>(
        (T*)qkv, (const W*)qw, (const W*)kw, cos_table, sin_table, positions, slots, (T*)key_cache,
        (T*)value_cache, tokens, num_q, num_kv, head_dim, page_size, table_positions, eps);
    return tvb_last_error();
}

extern "C" int tvb_qk_norm_rope_store(void* qkv, const void* q_weight, const void* k_weight,
                                      const float* cos_table, const float* sin_table,
                                      const int* positions, const int* slots, void* key_cache,
                                      void* value_cache, int tokens, int num_q, int num_kv,
                                      int head_dim, int page_size, int table_positions, float eps,
                                      int dtype, int weight_dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim % 2 || head_dim > 64 * QK_MAX_PAIRS || num_q <= 0 || num_kv < 0 ||
        (slots && page_size <= 0))
        return TVB_BAD_ARGUMENT;
    if ((int64_t)tokens * (num_q + 2 * num_kv) / 4 + 1 > 2147483647LL) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TVB_F32 && weight_dtype == TVB_F32)
        return launch_qk<float, float>(qkv, q_weight, k_weight, cos_table, sin_table, positions, slots,
                                       key_cache, value_cache, tokens, num_q, num_kv, head_dim, page_size,
                                       table_positions, eps, s);
    if (dtype == TVB_BF16 && weight_dtype == TVB_BF16)
        return launch_qk<bf16, bf16>(qkv, q_weight, k_weight, cos_table, sin_table, positions, slots,
                                     key_cache, value_cache, tokens, num_q, num_kv, head_dim, page_size,
                                     table_positions, eps, s);
    if (dtype == TVB_BF16 && weight_dtype == TVB_F32)
        return launch_qk<bf16, float>(qkv, q_weight, k_weight, cos_table, sin_table, positions, slots,
                                      key_cache, value_cache, tokens, num_q, num_kv, head_dim, page_size,
                                      table_positions, eps, s);
    return TVB_BAD_ARGUMENT;
}
