// bfloat16 fast paths of the memory-bound kernels, for rows that are whole numbers of 16-byte
// words: every access is a 16- or 8-byte one and a row lives in registers between the sum of
// squares and the scaling, so each byte crosses the memory system once.  Same arithmetic and
// rounding points as the general kernels in pointwise.cu (tinyvllm/kernels/pointwise.cu:94-116,
// :153-211, :274-285; tinyvllm/kernels/kv_store.cu:26-90).
#include "common.cuh"

// -------------------------------------------------------------------- RMSNorm
// TPR threads share a row (32: one warp, 8 rows a CTA; 64, 128; 256: the whole CTA).  A thread holds up to
// 4 words of 8 values.  `x` and `residual` come from the kernel before: coherent loads.
#define NORM_WORDS 4

template <int TPR, typename W>
__global__ void __launch_bounds__(256)
rms_norm_bf16_kernel(const bf16* x, const bf16* residual, const W* __restrict__ weight,
                     bf16* __restrict__ y, bf16* __restrict__ residual_out,
                     const int* __restrict__ gather, int rows, int width, float eps) {
    __shared__ float scratch[32];
    __shared__ float row_parts[8];
    pdl_wait();
    pdl_launch_dependents();
    const int rows_per_cta = 256 / TPR;
    const int out_row = blockIdx.x * rows_per_cta + threadIdx.x / TPR;
    const int lane = threadIdx.x % TPR;
    const bool live = out_row < rows;
    const int in_row = live ? (gather ? gather[out_row] : out_row) : 0;
    const bf16* xr = x + (int64_t)in_row * width;
    const bf16* rr = residual ? residual + (int64_t)in_row * width : nullptr;
    float values[NORM_WORDS][8];
    float squares = 0.0f;
#pragma unroll
    for (int i = 0; i < NORM_WORDS; ++i) {
        const int at = (lane + i * TPR) * 8;
        if (live && at < width) {
            unpack_bf16x8(ld_global_16(xr + at), values[i]);
            if (rr) {
                float other[8];
                unpack_bf16x8(ld_global_16(rr + at), other);
#pragma unroll
                for (int e = 0; e < 8; ++e) values[i][e] = round_to<bf16>(__fadd_rn(values[i][e], other[e]));
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) squares = __fadd_rn(squares, __fmul_rn(values[i][e], values[i][e]));
            if (residual_out) *reinterpret_cast<uint4*>(residual_out + (int64_t)out_row * width + at) = pack_bf16x8(values[i]);
        }
    }
    if (TPR == 32) {
        squares = warp_sum(squares);
    } else if (TPR == 256) {
        squares = block_sum(squares, scratch);
    } else {
        // TPR / 32 warps share a row: their sums meet in shared memory and are added in warp order
        squares = warp_sum(squares);
        if ((threadIdx.x & 31) == 0) row_parts[threadIdx.x >> 5] = squares;
        __syncthreads();
        const int first_warp = (threadIdx.x / TPR) * (TPR / 32);
        squares = 0.0f;
#pragma unroll
        for (int w = 0; w < TPR / 32; ++w) squares = __fadd_rn(squares, row_parts[first_warp + w]);
    }
    const float inverse_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(squares, 1.0f / (float)width), eps)));
#pragma unroll
    for (int i = 0; i < NORM_WORDS; ++i) {
        const int at = (lane + i * TPR) * 8;
        if (live && at < width) {
            float out[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
                out[e] = __fmul_rn(round_to<bf16>(__fmul_rn(values[i][e], inverse_rms)), to_float<W>(weight[at + e]));
            *reinterpret_cast<uint4*>(y + (int64_t)out_row * width + at) = pack_bf16x8(out);
        }
    }
}

extern "C" int tvb_rms_norm_bf16_supports(int width) { return width > 0 && width % 8 == 0 && width <= 8 * NORM_WORDS * 256; }

extern "C" int tvb_rms_norm_bf16(const void* x, const void* residual, const void* weight, void* y,
                                 void* residual_out, const int* gather, int rows, int width, float eps,
                                 int weight_dtype, int pdl, void* stream) {
    if (rows <= 0) return 0;
    if (!tvb_rms_norm_bf16_supports(width)) return TVB_BAD_ARGUMENT;
    // threads that share a row: the fewer rows, the more, so that the GPU is filled either way
    // (measured at width 1024: 8192 rows 32 or 64, 2048 rows 64, 512 rows 128, few rows 256); a
    // thread holds at most NORM_WORDS words, which bounds the width a narrow team takes
    int tpr = rows >= 4096 ? 32 : rows >= 1024 ? 64 : rows >= 256 ? 128 : 256;
    while (width > 8 * NORM_WORDS * tpr) tpr *= 2;
    const int rows_per_cta = 256 / tpr;
    TvbLaunch launch(dim3((rows + rows_per_cta - 1) / rows_per_cta), dim3(256), 0, (cudaStream_t)stream, pdl);
    cudaError_t e;
#define NORM_LAUNCH(TPR, WT)                                                                          \
    e = cudaLaunchKernelEx(&launch.config, rms_norm_bf16_kernel<TPR, WT>, (const bf16*)x,             \
                           (const bf16*)residual, (const WT*)weight, (bf16*)y, (bf16*)residual_out,   \
                           gather, rows, width, eps)
#define NORM_BY_TPR(WT)                                        \
    do {                                                       \
        if (tpr == 32) NORM_LAUNCH(32, WT);                    \
        else if (tpr == 64) NORM_LAUNCH(64, WT);               \
        else if (tpr == 128) NORM_LAUNCH(128, WT);             \
        else NORM_LAUNCH(256, WT);                             \
    } while (0)
    if (weight_dtype == TVB_F32) NORM_BY_TPR(float);
    else if (weight_dtype == TVB_BF16) NORM_BY_TPR(bf16);
    else return TVB_BAD_ARGUMENT;
#undef NORM_BY_TPR
#undef NORM_LAUNCH
    return e == cudaSuccess ? tvb_last_error() : (int)e;
}

// --------------------------------------------------------------- SiLU(gate)*up
__global__ void __launch_bounds__(256)
silu_mul_bf16_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, int64_t rows, int inter) {
    const int words = inter / 8;
    const int64_t total = rows * words;
    for (int64_t index = (int64_t)blockIdx.x * 256 + threadIdx.x; index < total; index += (int64_t)gridDim.x * 256) {
        const int64_t row = index / words;
        const int col = (int)(index % words) * 8;
        const bf16* src = gate_up + row * 2 * inter + col;
        float gate[8], up[8], result[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(src), gate);
        unpack_bf16x8(*reinterpret_cast<const uint4*>(src + inter), up);
#pragma unroll
        for (int e = 0; e < 8; ++e)
            result[e] = __fmul_rn(round_to<bf16>(__fdiv_rn(gate[e], __fadd_rn(1.0f, expf(-gate[e])))), up[e]);
        *reinterpret_cast<uint4*>(out + row * inter + col) = pack_bf16x8(result);
    }
}

extern "C" int tvb_silu_mul_bf16(const void* gate_up, void* out, int rows, int inter, void* stream) {
    if (rows <= 0) return 0;
    if (inter <= 0 || inter % 8) return TVB_BAD_ARGUMENT;
    const int64_t total = (int64_t)rows * (inter / 8);
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    silu_mul_bf16_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const bf16*)gate_up, (bf16*)out, rows, inter);
    return tvb_last_error();
}

// ------------------------------------- q/k norm + rotation + cache write, fused
// LANES = head_dim / 8 lanes share a (token, head) row: lane l holds 4 values of the first half
// (at 4 l) and the 4 values they pair with in the second half.  head_dim is 16, 32, 64, 128 or 256.
template <int HEAD_DIM, typename W>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_bf16_kernel(bf16* __restrict__ qkv, const W* __restrict__ q_weight,
                               const W* __restrict__ k_weight, const float* __restrict__ cos_table,
                               const float* __restrict__ sin_table, const int* __restrict__ positions,
                               const int* __restrict__ slots, bf16* __restrict__ key_cache,
                               bf16* __restrict__ value_cache, int tokens, int num_q, int num_kv,
                               int page_size, int table_positions, float eps) {
    constexpr int HALF = HEAD_DIM / 2;
    constexpr int LANES = HEAD_DIM / 8;
    const int heads = num_q + 2 * num_kv;
    const int64_t row = ((int64_t)blockIdx.x * 256 + threadIdx.x) / LANES;
    const int lane = threadIdx.x % LANES;
    const bool live = row < (int64_t)tokens * heads;
    const int token = live ? (int)(row / heads) : 0, head = live ? (int)(row % heads) : 0;
    bf16* src = qkv + ((int64_t)token * heads + head) * HEAD_DIM + 4 * lane;
    const int slot = slots && live ? slots[token] : -1;
    const bool is_value = head >= num_q + num_kv, is_key = !is_value && head >= num_q;
    float a[4], b[4];
    {
        const uint2 lo = live ? *reinterpret_cast<const uint2*>(src) : make_uint2(0, 0);
        const uint2 hi = live ? *reinterpret_cast<const uint2*>(src + HALF) : make_uint2(0, 0);
        a[0] = __uint_as_float(lo.x << 16); a[1] = __uint_as_float(lo.x & 0xffff0000u);
        a[2] = __uint_as_float(lo.y << 16); a[3] = __uint_as_float(lo.y & 0xffff0000u);
        b[0] = __uint_as_float(hi.x << 16); b[1] = __uint_as_float(hi.x & 0xffff0000u);
        b[2] = __uint_as_float(hi.y << 16); b[3] = __uint_as_float(hi.y & 0xffff0000u);
    }
    const W* weight = is_key ? k_weight : q_weight;
    // every lane of the warp takes part in the shuffles, whatever its row is
    float squares = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) squares = __fadd_rn(squares, __fadd_rn(__fmul_rn(a[e], a[e]), __fmul_rn(b[e], b[e])));
#pragma unroll
    for (int delta = LANES / 2; delta > 0; delta >>= 1) squares += __shfl_xor_sync(0xffffffffu, squares, delta);
    if (!live) return;
    bf16* dst = src;
    if (is_value || is_key) {
        if (slot < 0) return;
        bf16* cache = is_value ? value_cache : key_cache;
        const int kv_head = is_value ? head - num_q - num_kv : head - num_q;
        dst = cache + (((int64_t)(slot / page_size) * num_kv + kv_head) * page_size + slot % page_size) * HEAD_DIM +
              4 * lane;
    }
    if (!is_value) {
        if (weight) {
            const float inverse_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(squares, 1.0f / (float)HEAD_DIM), eps)));
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                a[e] = round_to<bf16>(__fmul_rn(round_to<bf16>(__fmul_rn(a[e], inverse_rms)), to_float<W>(weight[4 * lane + e])));
                b[e] = round_to<bf16>(__fmul_rn(round_to<bf16>(__fmul_rn(b[e], inverse_rms)), to_float<W>(weight[4 * lane + e + HALF])));
            }
        }
        if (cos_table) {
            int position = positions[token];
            position = position < 0 ? 0 : (position >= table_positions ? table_positions - 1 : position);
            const float4 c4 = *reinterpret_cast<const float4*>(cos_table + (int64_t)position * HALF + 4 * lane);
            const float4 s4 = *reinterpret_cast<const float4*>(sin_table + (int64_t)position * HALF + 4 * lane);
            const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float c = round_to<bf16>(cs[e]), s = round_to<bf16>(sn[e]);
                const float ac = round_to<bf16>(__fmul_rn(a[e], c)), bs = round_to<bf16>(__fmul_rn(b[e], s));
                const float bc = round_to<bf16>(__fmul_rn(b[e], c)), as = round_to<bf16>(__fmul_rn(a[e], s));
                a[e] = __fsub_rn(ac, bs);
                b[e] = __fadd_rn(bc, as);
            }
        }
    }
    *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]));
    *reinterpret_cast<uint2*>(dst + HALF) = make_uint2(pack_bf16x2(b[0], b[1]), pack_bf16x2(b[2], b[3]));
}

extern "C" int tvb_qk_norm_rope_store_bf16_supports(int head_dim) {
    return head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256;
}

extern "C" int tvb_qk_norm_rope_store_bf16(void* qkv, const void* q_weight, const void* k_weight,
                                           const float* cos_table, const float* sin_table,
                                           const int* positions, const int* slots, void* key_cache,
                                           void* value_cache, int tokens, int num_q, int num_kv,
                                           int head_dim, int page_size, int table_positions, float eps,
                                           int weight_dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (!tvb_qk_norm_rope_store_bf16_supports(head_dim) || num_q <= 0 || num_kv < 0 || (slots && page_size <= 0))
        return TVB_BAD_ARGUMENT;
    const int64_t threads = (int64_t)tokens * (num_q + 2 * num_kv) * (head_dim / 8);
    const int64_t blocks = (threads + 255) / 256;
    if (blocks > 2147483647LL) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
#define QK_LAUNCH(D, WT)                                                                                   \
    qk_norm_rope_store_bf16_kernel<D, WT><<<(unsigned)blocks, 256, 0, s>>>(                                \
        (bf16*)qkv, (const WT*)q_weight, (const WT*)k_weight, cos_table, sin_table, positions, slots,      \
        (bf16*)key_cache, (bf16*)value_cache, tokens, num_q, num_kv, page_size, table_positions, eps)
#define QK_BY_DIM(WT)                                     \
    do {                                                  \
        if (head_dim == 16) QK_LAUNCH(16, WT);            \
        else if (head_dim == 32) QK_LAUNCH(32, WT);       \
        else if (head_dim == 64) QK_LAUNCH(64, WT);       \
        else if (head_dim == 128) QK_LAUNCH(128, WT);     \
        else QK_LAUNCH(256, WT);                          \
    } while (0)
    if (weight_dtype == TVB_F32) QK_BY_DIM(float);
    else if (weight_dtype == TVB_BF16) QK_BY_DIM(bf16);
    else return TVB_BAD_ARGUMENT;
    return tvb_last_error();
}
