// Prefill attention for bfloat16: tiles of 64 consecutive query tokens of one request
// against the paged cache, on the tensor cores, with an online softmax in float32.
//
// Stands where the reference calls torch's scaled_dot_product_attention per request
// and, for a continued prompt, first gathers the whole history into a contiguous
// copy (tinyvllm/runtime/attention.py:112-147, tinyvllm/paged_kv.py:111-127): here
// keys and values are read from their pages inside the kernel, and every portion of
// every request of the step is one launch.
//
// A CTA of 4 warps takes one tile of queries and one q head; each warp owns 16 query
// rows.  Keys are walked in tiles of 32 that start at absolute multiples of 32, so a
// row's arithmetic does not depend on how the prompt was cut.  K and V tiles are
// brought in with cp.async (two stages), S = Q K^T and O += P V are mma.sync
// m16n8k16 with float32 accumulators, P is rounded to bfloat16 for the second
// product while the denominator sums the unrounded values (as
// tinyvllm/kernels/paged_decode.cu:322-356 does for decode).
#include "common.cuh"

#define PF_BM 64
#define PF_BN 32
#define PF_WARPS 4
#define PF_PAD 8        // bfloat16 of padding per shared-memory row: ldmatrix without bank conflicts

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_address(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_address(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HEAD_DIM>
__global__ void __launch_bounds__(PF_WARPS * 32, 3)
prefill_attention_kernel(const bf16* __restrict__ q, int64_t q_token_stride,
                         const bf16* __restrict__ key_cache, const bf16* __restrict__ value_cache,
                         const int* __restrict__ block_tables, int table_stride,
                         const int* __restrict__ positions, const int* __restrict__ tile_row,
                         const int* __restrict__ tile_first, const int* __restrict__ tile_count,
                         bf16* __restrict__ out, int num_q, int num_kv, int page_size, int window,
                         float scale) {
    constexpr int ROW = HEAD_DIM + PF_PAD;                 // bfloat16 per shared row
    constexpr int CHUNKS = HEAD_DIM / 8;                   // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char shared_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(shared_raw);                         // [64][ROW]
    bf16* k_s = q_s + PF_BM * ROW;                                           // [2][64][ROW]
    bf16* v_s = k_s + 2 * PF_BN * ROW;                                       // [2][64][ROW]
    int* slot_s = reinterpret_cast<int*>(v_s + 2 * PF_BN * ROW);             // [2][64]

    // later tiles of a request see more keys: they are launched first, the short ones fill the tail
    const int tile = gridDim.x - 1 - blockIdx.x, head = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int request = tile_row[tile], first_token = tile_first[tile], count = tile_count[tile];
    const int first_position = positions[first_token];
    const int kv_head = head / (num_q / num_kv);
    const int* table = block_tables + (int64_t)request * table_stride;
    const int last_position = first_position + count - 1;
    const int lo_first = window > 0 ? max(0, first_position - window + 1) : 0;
    const int key_begin = lo_first / PF_BN * PF_BN;
    const int tiles = (last_position - key_begin) / PF_BN + 1;

    // ---- Q tile (rows past `count` are zero)
    for (int index = tid; index < PF_BM * CHUNKS; index += PF_WARPS * 32) {
        const int r = index / CHUNKS, c = index % CHUNKS;
        const bf16* src = q + (int64_t)(first_token + min(r, count - 1)) * q_token_stride +
                          (int64_t)head * HEAD_DIM + c * 8;
        cp_async_16(q_s + r * ROW + c * 8, src, r < count);
    }
    cp_async_commit();

    // row of each key of tile t in the cache [pages, num_kv, page, head_dim] for this kv head, -1 if none
    auto stage_slots = [&](int t, int buffer) {
        if (tid < PF_BN) {
            const int key = key_begin + t * PF_BN + tid;
            int slot = -1;
            if (key <= last_position) {
                const int page = table[key / page_size];
                if (page >= 0) slot = (page * num_kv + kv_head) * page_size + key % page_size;
            }
            slot_s[buffer * PF_BN + tid] = slot;
        }
    };
    auto load_tile = [&](int buffer) {
        for (int index = tid; index < PF_BN * CHUNKS; index += PF_WARPS * 32) {
            const int r = index / CHUNKS, c = index % CHUNKS;
            const int slot = slot_s[buffer * PF_BN + r];
            const int64_t offset = (int64_t)max(slot, 0) * HEAD_DIM + c * 8;
            cp_async_16(k_s + (buffer * PF_BN + r) * ROW + c * 8, key_cache + offset, slot >= 0);
            cp_async_16(v_s + (buffer * PF_BN + r) * ROW + c * 8, value_cache + offset, slot >= 0);
        }
        cp_async_commit();
    };

    stage_slots(0, 0);
    __syncthreads();
    load_tile(0);

    // ---- Q fragments stay in registers for the whole walk
    cp_async_wait<1>();                                   // the Q tile (the first group) has landed
    __syncthreads();
    uint32_t q_frag[HEAD_DIM / 16][4];
#pragma unroll
    for (int ks = 0; ks < HEAD_DIM / 16; ++ks) {
        const int matrix = lane >> 3;
        const int r = warp * 16 + (lane & 7) + (matrix & 1) * 8;
        const int c = ks * 16 + (matrix >> 1) * 8;
        ldmatrix_x4(q_frag[ks], q_s + r * ROW + c);
    }

    const int g = lane >> 2, t4 = lane & 3;
    const int row_a = warp * 16 + g, row_b = row_a + 8;          // the two query rows this thread holds
    const int pos_a = first_position + row_a, pos_b = first_position + row_b;
    const int lo_a = window > 0 ? max(0, pos_a - window + 1) : 0;
    const int lo_b = window > 0 ? max(0, pos_b - window + 1) : 0;
    float o_acc[HEAD_DIM / 8][4];
#pragma unroll
    for (int n = 0; n < HEAD_DIM / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o_acc[n][i] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
    const float scale_log2 = scale * 1.4426950408889634f;

    for (int t = 0; t < tiles; ++t) {
        const int buffer = t & 1;
        if (t + 1 < tiles) stage_slots(t + 1, buffer ^ 1);
        cp_async_wait<0>();
        __syncthreads();                                  // tile t is in shared memory; slots of t + 1 too
        if (t + 1 < tiles) load_tile(buffer ^ 1);

        const bf16* k_tile = k_s + buffer * PF_BN * ROW;
        const bf16* v_tile = v_s + buffer * PF_BN * ROW;
        float s_acc[PF_BN / 8][4];
#pragma unroll
        for (int n = 0; n < PF_BN / 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) s_acc[n][i] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < HEAD_DIM / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < PF_BN / 16; ++np) {
                uint32_t b[4];
                const int matrix = lane >> 3;
                const int key = np * 16 + (matrix >> 1) * 8 + (lane & 7);
                const int dim = ks * 16 + (matrix & 1) * 8;
                ldmatrix_x4(b, k_tile + key * ROW + dim);
                mma_bf16(s_acc[2 * np], q_frag[ks], b[0], b[1]);
                mma_bf16(s_acc[2 * np + 1], q_frag[ks], b[2], b[3]);
            }
        }

        // ---- mask and online softmax (rows a and b of this thread; a row is spread over 4 threads)
        const int key0 = key_begin + t * PF_BN;
        const bool full = key0 + PF_BN - 1 <= first_position + warp * 16 &&      // below every diagonal
                          key0 >= (window > 0 ? max(0, first_position + warp * 16 + 15 - window + 1) : 0);
        float tile_max_a = -INFINITY, tile_max_b = -INFINITY;
#pragma unroll
        for (int n = 0; n < PF_BN / 8; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = key0 + n * 8 + 2 * t4 + (i & 1);
                const bool upper = i < 2;
                float s = s_acc[n][i] * scale_log2;
                if (!full) {
                    const bool ok = upper ? (key <= pos_a && key >= lo_a) : (key <= pos_b && key >= lo_b);
                    if (!ok) s = -INFINITY;
                }
                s_acc[n][i] = s;
                if (upper) tile_max_a = fmaxf(tile_max_a, s); else tile_max_b = fmaxf(tile_max_b, s);
            }
        }
        tile_max_a = fmaxf(tile_max_a, __shfl_xor_sync(0xffffffffu, tile_max_a, 1));
        tile_max_a = fmaxf(tile_max_a, __shfl_xor_sync(0xffffffffu, tile_max_a, 2));
        tile_max_b = fmaxf(tile_max_b, __shfl_xor_sync(0xffffffffu, tile_max_b, 1));
        tile_max_b = fmaxf(tile_max_b, __shfl_xor_sync(0xffffffffu, tile_max_b, 2));
        const float new_a = fmaxf(m_a, tile_max_a), new_b = fmaxf(m_b, tile_max_b);
        // a row that has seen no key yet keeps the reference 0 so that no inf - inf appears
        const float ref_a = new_a == -INFINITY ? 0.0f : new_a, ref_b = new_b == -INFINITY ? 0.0f : new_b;
        const float rescale_a = exp2f(m_a - ref_a), rescale_b = exp2f(m_b - ref_b);
        m_a = new_a;
        m_b = new_b;
        float sum_a = 0.0f, sum_b = 0.0f;
        uint32_t p_frag[PF_BN / 16][4];
#pragma unroll
        for (int n = 0; n < PF_BN / 8; ++n) {
            const float p0 = exp2f(s_acc[n][0] - ref_a), p1 = exp2f(s_acc[n][1] - ref_a);
            const float p2 = exp2f(s_acc[n][2] - ref_b), p3 = exp2f(s_acc[n][3] - ref_b);
            sum_a += p0 + p1;
            sum_b += p2 + p3;
            p_frag[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            p_frag[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_a = l_a * rescale_a + sum_a;
        l_b = l_b * rescale_b + sum_b;
#pragma unroll
        for (int n = 0; n < HEAD_DIM / 8; ++n) {
            o_acc[n][0] *= rescale_a; o_acc[n][1] *= rescale_a;
            o_acc[n][2] *= rescale_b; o_acc[n][3] *= rescale_b;
        }

        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < PF_BN / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < HEAD_DIM / 16; ++dp) {
                uint32_t b[4];
                const int matrix = lane >> 3;
                const int key = kk * 16 + (matrix & 1) * 8 + (lane & 7);
                const int dim = dp * 16 + (matrix >> 1) * 8;
                ldmatrix_x4_trans(b, v_tile + key * ROW + dim);
                mma_bf16(o_acc[2 * dp], p_frag[kk], b[0], b[1]);
                mma_bf16(o_acc[2 * dp + 1], p_frag[kk], b[2], b[3]);
            }
        }
    }

    // ---- the four threads of a row hold partial sums of its denominator
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float inv_a = 1.0f / l_a, inv_b = 1.0f / l_b;
    bf16* out_a = out + ((int64_t)(first_token + row_a) * num_q + head) * HEAD_DIM;
    bf16* out_b = out + ((int64_t)(first_token + row_b) * num_q + head) * HEAD_DIM;
#pragma unroll
    for (int n = 0; n < HEAD_DIM / 8; ++n) {
        const int dim = n * 8 + 2 * t4;
        if (row_a < count)
            *reinterpret_cast<uint32_t*>(out_a + dim) = pack_bf16(o_acc[n][0] * inv_a, o_acc[n][1] * inv_a);
        if (row_b < count)
            *reinterpret_cast<uint32_t*>(out_b + dim) = pack_bf16(o_acc[n][2] * inv_b, o_acc[n][3] * inv_b);
    }
}

extern "C" int tvb_attention_prefill_tile_tokens() { return PF_BM; }

extern "C" int tvb_attention_prefill_supports(int head_dim, int num_q, int num_kv) {
    return (head_dim == 64 || head_dim == 128) && num_kv > 0 && num_q % num_kv == 0;
}

template <int HEAD_DIM>
static int launch_prefill(const void* q, long long q_token_stride, const void* key_cache,
                          const void* value_cache, const int* block_tables, int table_stride,
                          const int* positions, const int* tile_row, const int* tile_first,
                          const int* tile_count, void* out, int tiles, int num_q, int num_kv,
                          int page_size, int window, float scale, cudaStream_t stream) {
    constexpr int ROW = HEAD_DIM + PF_PAD;
    const size_t shared = (size_t)(PF_BM + 4 * PF_BN) * ROW * sizeof(bf16) + 2 * PF_BN * sizeof(int);
    auto kernel = prefill_attention_kernel<HEAD_DIM>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(tiles, num_q);
    kernel<<<grid, PF_WARPS * 32, shared, stream>>>(
        (const bf16*)q, q_token_stride, (const bf16*)key_cache, (const bf16*)value_cache, block_tables,
        table_stride, positions, tile_row, tile_first, tile_count, (bf16*)out, num_q, num_kv, page_size,
        window, scale);
    return tvb_last_error();
}

// tile_row / tile_first / tile_count: per tile the request's row in block_tables, the flat index
// of its first query token and the number of query tokens (1..64); the tokens of a tile stand at
// consecutive positions.  q holds the (normalised, rotated) query heads of token t at
// t * q_token_stride elements.
extern "C" int tvb_attention_prefill(const void* q, long long q_token_stride, const void* key_cache,
                                     const void* value_cache, const int* block_tables, int table_stride,
                                     const int* positions, const int* tile_row, const int* tile_first,
                                     const int* tile_count, void* out, int tiles, int num_q, int num_kv,
                                     int head_dim, int page_size, int window, float scale, void* stream) {
    if (tiles <= 0) return 0;
    if (!tvb_attention_prefill_supports(head_dim, num_q, num_kv) || page_size <= 0 || num_q > 65535 ||
        (q_token_stride * 2) % 16 != 0)
        return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64)
        return launch_prefill<64>(q, q_token_stride, key_cache, value_cache, block_tables, table_stride,
                                  positions, tile_row, tile_first, tile_count, out, tiles, num_q, num_kv,
                                  page_size, window, scale, s);
    return launch_prefill<128>(q, q_token_stride, key_cache, value_cache, block_tables, table_stride,
                               positions, tile_row, tile_first, tile_count, out, tiles, num_q, num_kv,
                               page_size, window, scale, s);
}
