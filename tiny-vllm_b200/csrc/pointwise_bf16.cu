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
    // all loads of the row first (they are ordered with the stores below, so a load after a store
    // would wait for a second trip to memory)
    uint4 x_words[NORM_WORDS], r_words[NORM_WORDS];
#pragma unroll
    for (int i = 0; i < NORM_WORDS; ++i) {
        const int at = (lane + i * TPR) * 8;
        x_words[i] = r_words[i] = make_uint4(0u, 0u, 0u, 0u);
        if (live && at < width) {
            x_words[i] = ld_global_16(xr + at);
            if (rr) r_words[i] = ld_global_16(rr + at);
        }
    }
#pragma unroll
    for (int i = 0; i < NORM_WORDS; ++i) {
        const int at = (lane + i * TPR) * 8;
        if (live && at < width) {
            unpack_bf16x8(x_words[i], values[i]);
            if (rr) {
                float other[8];
                unpack_bf16x8(r_words[i], other);
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
// One warp per token.  LANES = head_dim / 16 lanes share a head: lane l holds 8 values of the first
// half (at 8 l) and the 8 they pair with in the second half, so every access is 16 bytes.  The
// warp's 32 / LANES groups of lanes take the token's heads in turn (q, then k, then v), four heads
// of a group at a time with all their loads issued before the first is used; position, cache slot,
// rotation angles and norm weights are read once per thread, not once per head.
// head_dim is 16, 32, 64, 128 or 256.
template <int HEAD_DIM, typename W>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_bf16_kernel(bf16* __restrict__ qkv, const W* __restrict__ q_weight,
                               const W* __restrict__ k_weight, const float* __restrict__ cos_table,
                               const float* __restrict__ sin_table, const int* __restrict__ positions,
                               const int* __restrict__ slots, bf16* __restrict__ key_cache,
                               bf16* __restrict__ value_cache, int tokens, int num_q, int num_kv,
                               int page_size, int table_positions, float eps) {
    constexpr int HALF = HEAD_DIM / 2;
    constexpr int LANES = HEAD_DIM / 16;
    constexpr int GROUPS = 32 / LANES;
    constexpr int BATCH = 4;
    const int heads = num_q + 2 * num_kv;
    const int token = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (token >= tokens) return;                 // the whole warp
    const int lane = threadIdx.x & 31;
    const int group = lane / LANES, l = lane % LANES;
    const int slot = slots ? slots[token] : -1;
    const bool rotated = cos_table != nullptr;
    // Every intermediate of the rotation is a bfloat16 (the product of two bfloat16 is exact in
    // float32, so rounding it once is the packed instruction's own rounding): it runs on pairs.
    __nv_bfloat162 cs[4], sn[4];
    float wq_lo[8], wq_hi[8], wk_lo[8], wk_hi[8];
    if (rotated) {
        int position = positions[token];
        position = position < 0 ? 0 : (position >= table_positions ? table_positions - 1 : position);
        const float4* c4 = reinterpret_cast<const float4*>(cos_table + (int64_t)position * HALF + 8 * l);
        const float4* s4 = reinterpret_cast<const float4*>(sin_table + (int64_t)position * HALF + 8 * l);
        const float4 c_lo = c4[0], c_hi = c4[1], s_lo = s4[0], s_hi = s4[1];
        cs[0] = __floats2bfloat162_rn(c_lo.x, c_lo.y), cs[1] = __floats2bfloat162_rn(c_lo.z, c_lo.w);
        cs[2] = __floats2bfloat162_rn(c_hi.x, c_hi.y), cs[3] = __floats2bfloat162_rn(c_hi.z, c_hi.w);
        sn[0] = __floats2bfloat162_rn(s_lo.x, s_lo.y), sn[1] = __floats2bfloat162_rn(s_lo.z, s_lo.w);
        sn[2] = __floats2bfloat162_rn(s_hi.x, s_hi.y), sn[3] = __floats2bfloat162_rn(s_hi.z, s_hi.w);
    }
    const bool normed = q_weight != nullptr;     // the two weights come together
    if (normed) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            wq_lo[e] = to_float<W>(q_weight[8 * l + e]), wq_hi[e] = to_float<W>(q_weight[HALF + 8 * l + e]);
            wk_lo[e] = to_float<W>(k_weight[8 * l + e]), wk_hi[e] = to_float<W>(k_weight[HALF + 8 * l + e]);
        }
    }
    // position, slot, angles and weights do not come from the kernel before this one; the projection does
    pdl_wait();
    pdl_launch_dependents();
    bf16* row = qkv + (int64_t)token * heads * HEAD_DIM + 8 * l;
    const int64_t cache_row = slot >= 0 ? ((int64_t)(slot / page_size) * num_kv * page_size + slot % page_size) : 0;

    // every lane goes round the same number of times: the shuffles below are warp-wide
    // (the CTAs of a token's row of the grid share its heads: batches blockIdx.y, blockIdx.y + gridDim.y, ...)
    for (int first = blockIdx.y * GROUPS * BATCH; first < heads; first += gridDim.y * GROUPS * BATCH) {
        uint4 lo[BATCH], hi[BATCH];
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const int head = first + i * GROUPS + group;
            lo[i] = hi[i] = make_uint4(0u, 0u, 0u, 0u);
            if (head < heads) {
                lo[i] = *reinterpret_cast<const uint4*>(row + (int64_t)head * HEAD_DIM);
                hi[i] = *reinterpret_cast<const uint4*>(row + (int64_t)head * HEAD_DIM + HALF);
            }
        }
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const int head = first + i * GROUPS + group;
            const bool live = head < heads;
            const bool is_value = head >= num_q + num_kv, is_key = !is_value && head >= num_q;
            __align__(16) __nv_bfloat162 a2[4];
            __align__(16) __nv_bfloat162 b2[4];
            *reinterpret_cast<uint4*>(a2) = lo[i];
            *reinterpret_cast<uint4*>(b2) = hi[i];
            float squares = 0.0f;
            if (normed) {            // the same for the whole warp
                float a[8], b[8];
                unpack_bf16x8(lo[i], a);
                unpack_bf16x8(hi[i], b);
#pragma unroll
                for (int e = 0; e < 8; ++e) squares = __fadd_rn(squares, __fadd_rn(__fmul_rn(a[e], a[e]), __fmul_rn(b[e], b[e])));
#pragma unroll
                for (int delta = LANES / 2; delta > 0; delta >>= 1) squares += __shfl_xor_sync(0xffffffffu, squares, delta);
                if (live && !is_value) {
                    const float inverse_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(squares, 1.0f / (float)HEAD_DIM), eps)));
                    const float* w_lo = is_key ? wk_lo : wq_lo;
                    const float* w_hi = is_key ? wk_hi : wq_hi;
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        // round(round(x * inverse rms) * weight), two values at a time
                        const float2 x = __bfloat1622float2(__floats2bfloat162_rn(__fmul_rn(a[2 * p], inverse_rms), __fmul_rn(a[2 * p + 1], inverse_rms)));
                        const float2 y = __bfloat1622float2(__floats2bfloat162_rn(__fmul_rn(b[2 * p], inverse_rms), __fmul_rn(b[2 * p + 1], inverse_rms)));
                        a2[p] = __floats2bfloat162_rn(__fmul_rn(x.x, w_lo[2 * p]), __fmul_rn(x.y, w_lo[2 * p + 1]));
                        b2[p] = __floats2bfloat162_rn(__fmul_rn(y.x, w_hi[2 * p]), __fmul_rn(y.y, w_hi[2 * p + 1]));
                    }
                }
            }
            if (!live) continue;
            bf16* dst = row + (int64_t)head * HEAD_DIM;
            if (is_value || is_key) {
                if (slot < 0) continue;
                const int kv_head = is_value ? head - num_q - num_kv : head - num_q;
                dst = (is_value ? value_cache : key_cache) + (cache_row + (int64_t)kv_head * page_size) * HEAD_DIM + 8 * l;
            }
            if (!is_value && rotated) {
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const __nv_bfloat162 ac = __hmul2(a2[p], cs[p]), bs = __hmul2(b2[p], sn[p]);
                    const __nv_bfloat162 bc = __hmul2(b2[p], cs[p]), as = __hmul2(a2[p], sn[p]);
                    a2[p] = __hsub2(ac, bs);
                    b2[p] = __hadd2(bc, as);
                }
            }
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(a2);
            *reinterpret_cast<uint4*>(dst + HALF) = *reinterpret_cast<const uint4*>(b2);
        }
    }
}

static int tvb_sm_count_pointwise() {
    static int count = 0;
    if (count == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
            count = 1;
    }
    return count;
}

extern "C" int tvb_qk_norm_rope_store_bf16_supports(int head_dim) {
    return head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256;
}

extern "C" int tvb_qk_norm_rope_store_bf16(void* qkv, const void* q_weight, const void* k_weight,
                                           const float* cos_table, const float* sin_table,
                                           const int* positions, const int* slots, void* key_cache,
                                           void* value_cache, int tokens, int num_q, int num_kv,
                                           int head_dim, int page_size, int table_positions, float eps,
                                           int weight_dtype, int pdl, void* stream) {
    if (tokens <= 0) return 0;
    if (!tvb_qk_norm_rope_store_bf16_supports(head_dim) || num_q <= 0 || num_kv < 0 || (slots && page_size <= 0))
        return TVB_BAD_ARGUMENT;
    if (head_dim % 8 || ((num_q + 2 * num_kv) * head_dim) % 8) return TVB_BAD_ARGUMENT;
    const int64_t blocks = ((int64_t)tokens + 7) / 8;         // a warp per token, eight to a block
    cudaStream_t s = (cudaStream_t)stream;
    // With few tokens (a warp each) the heads of a token are shared out over more CTAs: a batch of
    // heads (four per group of lanes) per CTA along y while the grid stays within one CTA an SM
    // (256 tokens, 32 heads of 128: 4.6 us against 6.2).  Beyond that the kernel moves its bytes at
    // the rate of L2 and a second CTA per token only repeats the angles and weights (2,048 tokens:
    // 9.3 us against 8.3).
    const int lanes = head_dim / 16, batch_heads = (32 / lanes) * 4;
    int along_y = (num_q + 2 * num_kv + batch_heads - 1) / batch_heads;
    const long long room = (long long)tvb_sm_count_pointwise() / (blocks > 0 ? blocks : 1);
    if (along_y > room) along_y = room < 1 ? 1 : (int)room;
    TvbLaunch launch(dim3((unsigned)blocks, (unsigned)along_y), dim3(256), 0, s, pdl);
    cudaError_t launched = cudaSuccess;
#define QK_LAUNCH(D, WT)                                                                                   \
    launched = cudaLaunchKernelEx(&launch.config, qk_norm_rope_store_bf16_kernel<D, WT>,                   \
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
    return launched == cudaSuccess ? tvb_last_error() : (int)launched;
}
