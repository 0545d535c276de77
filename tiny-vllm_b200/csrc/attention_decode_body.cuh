// This file is the body of the libraries attention_decode_<head size>_<norm weight type>.cu: each of
// them defines TVB_DECODE_HEAD_DIM (64, 128 or 256) and TVB_DECODE_WEIGHT (float or bf16) and
// includes it, so that a model compiles the one combination it uses (a sixth of the templates).
//
// Decode attention for bfloat16: one new token per request, fused from the packed
// projection to the attention output.
//
// One launch does what the general path does in three: per-head RMSNorm and
// rotation of the new q and k (tinyvllm/kernels/pointwise.cu:324-450), the write of
// the new k and v into their cache page (tinyvllm/kernels/kv_store.cu:26-90) and
// paged GQA attention (tinyvllm/kernels/paged_decode.cu:85-466).  Unlike the
// reference kernel (one CTA per request and q head, no split over the context,
// :586-590) a CTA serves HPB q heads that share one kv head, so keys and values
// are read once per group, and the context is split over a thread-block cluster of
// up to 8 CTAs.  Every CTA stores its partial (max, sum, output) into the shared
// memory of the cluster's first CTA (distributed shared memory), which merges them
// in rank order: no scratch in global memory and no second kernel.
//
// Every warp walks its keys in tiles through a ring of cp.async stages of its own in shared
// memory (16-byte chunks swizzled by the key, so that ldmatrix reads them without bank conflicts);
// the cache slots of its keys are looked up once, up front, and the first stage is in flight
// before the kernel waits for the projection (keys and values already in the cache do not depend
// on it, nor do the norm weights and the rotation's table row, which are asked for up front too).
// The products are mma.sync m16n8k16 with float32 accumulators, in one of two arrangements:
//
// * head size 128, tiles of 16 keys: the KEYS are the rows of the first product, S^T = K Q^T (the
//   CTA's up to 8 q heads are its 8 columns), and the k of the second, O^T += V^T P^T, whose b
//   operand P^T comes from the first product's accumulators by two 8 x 8 transposes in registers
//   (movmatrix).  Every row of every product and every accumulator register is in use: 16 products
//   and 16 ldmatrix for 16 keys, and the loop waits for memory, not for its own instructions.
// * the other head sizes, tiles of 8 keys: the q heads are the rows of both products (rows past
//   the heads are zero) and the second product's k of 16 is the tile's 8 keys and 8 zeros: 48
//   products for 16 keys.  Measured on head size 128 this form was bound by each warp's chain of
//   about 300 instructions a tile (`ncu`: no memory stall, 0.4 instructions a cycle and scheduler).
//
// Few warps and small tiles keep several CTAs on an SM (three of four warps or four of three with
// 16-key tiles; grids smaller than the GPU get one CTA of eight warps an SM).  Softmax is
// float32; P is rounded to bfloat16 for the second product while the denominator sums the
// unrounded values (as tinyvllm/kernels/paged_decode.cu:322-356 does).  The size of a piece
// follows from the request's own position (and window) alone and is a whole number of tiles:
// pieces of a request differ by one tile at most, so the CTAs of a cluster reach its barrier
// together (pieces of whole multiples of 64 keys left the last CTAs of a cluster with little or
// nothing to do, and the others waiting).
#include <cooperative_groups.h>
#include <type_traits>

#include "common.cuh"

namespace cg = cooperative_groups;

// Keys of a stage: TILE is a template parameter of the kernel.  8: the q heads are the rows of the
// products' tiles and the keys their columns (the second product's k = 16 is half zeros); 16: the
// keys are the rows of the first product (S^T = K Q^T) and the k of the second (O^T += V^T P^T),
// the q heads the columns of both.
// DEC_STAGES, the stages of each warp's ring of keys and values in shared memory, is a template
// parameter of the kernel (2 with tiles of 8 keys).
#define DEC_MAX_SPLITS 8

// Where things lie in a CTA's dynamic shared memory (byte offsets; worked out by the launcher).
// Only what a launch needs is there: partials for `splits` CTAs, not for the largest cluster; the
// list of cache slots holds one entry per tile of 8 keys where a tile lies inside one page (pages
// of a multiple of 8 tokens), else one per key; and the warps' partial outputs reuse the rings
// once the keys have been walked.  The less a CTA takes, the more of them share an SM (up to the
// four that the registers allow) whatever the context limit, the cluster size and the number of q
// heads a CTA serves.  (A third stage of the rings, which this leaves room for, was measured and
// is slower at every batch size, also where it costs no residency.)
struct DecodeLayout {
    int q;            // float [HPB][HEAD_DIM]: normalised, rotated, rounded q heads
    int v_new;        // float [HEAD_DIM]: the new value as stored
    int s_new;        // float [HPB]: score of the new key for each head
    int warp_m;       // float [DEC_WARPS][HPB]
    int warp_l;
    int part_m;       // float [splits][HPB]: partials of every CTA of the cluster; only the first CTA's
    int part_l;       //   copy is used, the others write theirs into it
    int part_o;       // float [splits][HPB][HEAD_DIM]
    int ring;         // per warp: DEC_STAGES x (keys, values) x [TILE keys][HEAD_DIM] bfloat16, chunk c of key k at
                      //   c ^ (k & 7); after the loop the warp's partial output float [HPB][HEAD_DIM] lies here
    int slots;        // int [DEC_WARPS][warp_slot_capacity]
    int total;        // bytes
};

static DecodeLayout decode_layout(int head_dim, int hpb, int warps, int splits, int warp_slots, int tile, int stages) {
    DecodeLayout l;
    int at = 0;
    auto take = [&](int bytes) { const int here = at; at += (bytes + 15) / 16 * 16; return here; };
    l.q = take(hpb * head_dim * 4);
    l.v_new = take(head_dim * 4);
    l.s_new = take(hpb * 4);
    l.warp_m = take(warps * hpb * 4);
    l.warp_l = take(warps * hpb * 4);
    l.part_m = take(splits * hpb * 4);
    l.part_l = take(splits * hpb * 4);
    l.part_o = take(splits * hpb * head_dim * 4);
    l.ring = take(warps * stages * 2 * tile * head_dim * 2);
    l.slots = take(warps * warp_slots * 4);
    l.total = at;
    return l;
}

__device__ __forceinline__ void dec_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_address(p)));
}
__device__ __forceinline__ void dec_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_address(p)));
}
// d += a . b for a 16 x 16 tile whose rows 8..15 are zero (a1 = a3 = 0)
__device__ __forceinline__ void dec_mma(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    const uint32_t zero = 0u;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(zero), "r"(a2), "r"(zero), "r"(b0), "r"(b1));
}

// d (16 x 8) += a (16 x 16) . b (16 x 8), all four registers of a and d in use
__device__ __forceinline__ void dec_mma_full(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// The transpose of an 8 x 8 matrix of 16-bit values held as a product's fragment (lane l: row l / 4,
// columns 2 (l % 4) and the next): afterwards lane l holds rows 2 (l % 4) and the next of column l / 4.
__device__ __forceinline__ uint32_t dec_transpose_8x8(uint32_t v) {
    uint32_t t;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(t) : "r"(v));
    return t;
}

// One head of the new token in a warp's registers: lane l holds elements l + 32 i of the first half
// (a) and of the second half (b).  The steps below are RMSNorm and half-split rotation with the
// roundings of tinyvllm/kernels/pointwise.cu:324-450 (every intermediate rounded to bfloat16).
template <int HEAD_DIM>
struct HeadRegs {
    static constexpr int HALF = HEAD_DIM / 2;
    static constexpr int PAIRS = (HALF + 31) / 32;
    float a[PAIRS], b[PAIRS];
};

// What the steps need beside the head itself; it does not depend on the kernel before this one, so
// it is asked for before the wait on that kernel.
template <int HEAD_DIM>
struct HeadConstants {
    HeadRegs<HEAD_DIM> q_weight, k_weight, cos, sin;      // cos, sin: rounded to bfloat16
};

template <int HEAD_DIM, typename W>
__device__ __forceinline__ void load_head_weight(HeadRegs<HEAD_DIM>& to, const W* __restrict__ weight, int lane) {
#pragma unroll
    for (int i = 0; i < HeadRegs<HEAD_DIM>::PAIRS; ++i) {
        const int j = lane + 32 * i;
        const bool in = weight != nullptr && j < HeadRegs<HEAD_DIM>::HALF;
        to.a[i] = in ? to_float<W>(weight[j]) : 1.0f;
        to.b[i] = in ? to_float<W>(weight[j + HeadRegs<HEAD_DIM>::HALF]) : 1.0f;
    }
}

// `src` was written by the kernel before this one: read with plain coherent loads that are all in
// flight together (volatile ones would go one after the other, a latency each).
template <int HEAD_DIM>
__device__ __forceinline__ void load_head(HeadRegs<HEAD_DIM>& to, const unsigned short* src, int lane) {
#pragma unroll
    for (int i = 0; i < HeadRegs<HEAD_DIM>::PAIRS; ++i) {
        const int j = lane + 32 * i;
        const bool in = j < HeadRegs<HEAD_DIM>::HALF;
        to.a[i] = in ? bf16_bits_to_float(ld_global_u16(src + j)) : 0.0f;
        to.b[i] = in ? bf16_bits_to_float(ld_global_u16(src + j + HeadRegs<HEAD_DIM>::HALF)) : 0.0f;
    }
}

template <int HEAD_DIM>
__device__ __forceinline__ void norm_rotate_head(HeadRegs<HEAD_DIM>& x, bool normed, const HeadRegs<HEAD_DIM>& weight,
                                                 float eps, bool rotated, const HeadRegs<HEAD_DIM>& cos,
                                                 const HeadRegs<HEAD_DIM>& sin) {
    constexpr int PAIRS = HeadRegs<HEAD_DIM>::PAIRS;
    if (normed) {
        float squares = 0.0f;
#pragma unroll
        for (int i = 0; i < PAIRS; ++i)
            squares = __fadd_rn(squares, __fadd_rn(__fmul_rn(x.a[i], x.a[i]), __fmul_rn(x.b[i], x.b[i])));
        squares = warp_sum(squares);
        const float inverse_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(squares, 1.0f / (float)HEAD_DIM), eps)));
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) {
            x.a[i] = round_to<bf16>(__fmul_rn(round_to<bf16>(__fmul_rn(x.a[i], inverse_rms)), weight.a[i]));
            x.b[i] = round_to<bf16>(__fmul_rn(round_to<bf16>(__fmul_rn(x.b[i], inverse_rms)), weight.b[i]));
        }
    }
    if (rotated) {
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) {
            const float c = cos.a[i], s = sin.a[i];
            const float xc = round_to<bf16>(__fmul_rn(x.a[i], c)), ys = round_to<bf16>(__fmul_rn(x.b[i], s));
            const float yc = round_to<bf16>(__fmul_rn(x.b[i], c)), xs = round_to<bf16>(__fmul_rn(x.a[i], s));
            x.a[i] = round_to<bf16>(__fsub_rn(xc, ys));
            x.b[i] = round_to<bf16>(__fadd_rn(yc, xs));
        }
    }
}

// the head to [HEAD_DIM] floats (shared memory) or bfloat16 (a row of the cache)
template <int HEAD_DIM, typename T>
__device__ __forceinline__ void store_head(const HeadRegs<HEAD_DIM>& x, T* to, int lane) {
#pragma unroll
    for (int i = 0; i < HeadRegs<HEAD_DIM>::PAIRS; ++i) {
        const int j = lane + 32 * i;
        if (j < HeadRegs<HEAD_DIM>::HALF) {
            if constexpr (std::is_same<T, float>::value) {
                to[j] = x.a[i];
                to[j + HeadRegs<HEAD_DIM>::HALF] = x.b[i];
            } else {
                to[j] = __float2bfloat16_rn(x.a[i]);
                to[j + HeadRegs<HEAD_DIM>::HALF] = __float2bfloat16_rn(x.b[i]);
            }
        }
    }
}

// RESIDENT: the CTAs that are to share an SM, which caps the registers.  The loop wants about 150
// and is up to a tenth faster with them than with 128 and spills, so the cap follows the grid:
// four CTAs of four warps an SM (128 registers) only where the grid needs them, three (160) for
// grids of up to three CTAs an SM, none for the eight-warp CTAs of grids smaller than the GPU and
// for a head of 256, which keeps its output tile in twice the registers.  With 16-key tiles
// (twice the ring per warp) the larger grids get CTAs of three warps, four to an SM.
//
// FAR (one request with a long context, where clusters of the largest size that fits would leave
// half of the SMs idle): the keys of a request that holds `far.from` or more are cut `far.groups`
// times more finely and every group of `splits` pieces has a cluster of its own; the first CTA of
// a cluster leaves its merged piece (maximum, denominator, sums) in global memory and counts itself
// in; the cluster that finds all others counted merges the groups in their order and stores the
// result.  Nobody waits: a cluster that is not last is done.  With fewer keys the first group's
// cluster does everything as without FAR and the others leave at once.
struct FarArgs {
    int groups;          // clusters per (request, kv head, block of q heads)
    int from;            // keys from which a request is cut over all groups
    float* pieces;       // [requests][gridDim.y / groups][groups][HPB][HEAD_DIM + 2]
    int* arrived;        // [requests][gridDim.y / groups], zero between launches
};

template <int HEAD_DIM, int HPB, int DEC_WARPS, int RESIDENT, int TILE, int DEC_STAGES, typename W, bool FAR = false>
__global__ void __launch_bounds__(DEC_WARPS * 32, RESIDENT)
decode_attention_kernel(const bf16* qkv, const W* __restrict__ q_weight,
                        const W* __restrict__ k_weight, float eps, const float* __restrict__ cos_table,
                        const float* __restrict__ sin_table, int table_positions,
                        const int* __restrict__ positions, const int* __restrict__ token_row,
                        const int* __restrict__ slots, bf16* __restrict__ key_cache,
                        bf16* __restrict__ value_cache, const int* __restrict__ block_tables,
                        int table_stride, int page_size, bf16* __restrict__ out, int num_q, int num_kv,
                        int window, float scale, int write_cache, int warp_slot_capacity, int heads_here,
                        DecodeLayout layout, FarArgs far) {
    // heads_here <= HPB q heads of one kv head are this CTA's (HPB is what the tile and the shared
    // arrays hold; rows past heads_here stay zero): groups of 3, 5, 6 or 7 heads run on the next size up
    constexpr int CPR = HEAD_DIM / 8;          // 16-byte chunks of a key's row
    constexpr int KPI = 32 / CPR;              // keys a warp copies per instruction
    constexpr int WARP_KEYS = TILE;
    static_assert(HPB <= 8 && 32 % CPR == 0 && TILE % KPI == 0 && HEAD_DIM % 32 == 0 && (TILE == 8 || TILE == 16), "shape of the tile");
    extern __shared__ __align__(16) unsigned char shared_raw[];
    constexpr int TILE_WORDS = TILE * HEAD_DIM / 8;                 // 16-byte words of a tile of keys
    // the arrays of the layout, worked out where they are used (nothing of this stays in registers
    // through the loop over the keys)
#define q_s (reinterpret_cast<float*>(shared_raw + layout.q))                  /* [HPB][HEAD_DIM] */
#define v_new_s (reinterpret_cast<float*>(shared_raw + layout.v_new))
#define s_new_s (reinterpret_cast<float*>(shared_raw + layout.s_new))
#define warp_m_s (reinterpret_cast<float*>(shared_raw + layout.warp_m))        /* [DEC_WARPS][HPB] */
#define warp_l_s (reinterpret_cast<float*>(shared_raw + layout.warp_l))
    auto ring_of = [&](int w, int stage, int which) {
        return reinterpret_cast<uint4*>(shared_raw + layout.ring) + ((w * DEC_STAGES + stage) * 2 + which) * TILE_WORDS;
    };
    auto warp_o_of = [&](int w) { return reinterpret_cast<float*>(ring_of(w, 0, 0)); };     // [HPB][HEAD_DIM], after the loop
    int* slot_s = reinterpret_cast<int*>(shared_raw + layout.slots);

    cg::cluster_group cluster = cg::this_cluster();
    const int split = blockIdx.x;              // = rank in the cluster
    const int splits = gridDim.x;
    const int group = num_q / num_kv;
    const int blocks_per_kv = group / heads_here;
    const int y_block = FAR ? blockIdx.y / far.groups : blockIdx.y;       // (kv head, block of its q heads)
    const int far_group = FAR ? blockIdx.y % far.groups : 0;
    const int kv_head = y_block / blocks_per_kv;
    const int first_q_head = kv_head * group + (y_block % blocks_per_kv) * heads_here;
    const int request = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = num_q + 2 * num_kv;
    // The block table's row is asked into L1 while position and row are on their way (in a step of
    // decoded tokens only, request i is row i; a wrong guess costs nothing): the look-up of the
    // pages then does not wait for a second trip to L2.
    if (threadIdx.x * 32 < table_stride && threadIdx.x < 64)
        asm volatile("prefetch.global.L1 [%0];\n" ::"l"(block_tables + (int64_t)request * table_stride + threadIdx.x * 32));
    const int position = positions[request];
    const int row = token_row[request];
    bf16* out_row = out + ((int64_t)request * num_q + first_q_head) * HEAD_DIM;
    if (row < 0 || position < 0) {              // padding: the whole cluster leaves together
        pdl_wait();
        if (split == 0 && far_group == 0)
            for (int i = threadIdx.x; i < heads_here * HEAD_DIM; i += blockDim.x) out_row[i] = __float2bfloat16_rn(0.0f);
        return;
    }
    // groups of pieces that this request is cut into: all of them from far.from keys on
    int far_groups = 1;
    if constexpr (FAR) {
        const int keys = window > 0 ? min(position + 1, window) : position + 1;
        far_groups = keys >= far.from ? far.groups : 1;
        if (far_group >= far_groups) return;    // the whole cluster
    }
    const int pieces = splits * far_groups, piece = far_group * splits + split;

    // Every CTA says that it runs; the stores into the first CTA's shared memory at the end wait
    // until all of them have said so.
    cluster_arrive_relaxed();

    // What the new token's heads are normalised and rotated with does not come from the kernel
    // before this one: asked for now, it is there when that kernel has ended.
    const bool cached_new = write_cache == 2;   // the new key and value are in the cache, q is ready
    HeadRegs<HEAD_DIM> q_norm_weight, k_norm_weight, cos_regs, sin_regs;
    load_head_weight<HEAD_DIM, W>(q_norm_weight, q_weight, lane);
    load_head_weight<HEAD_DIM, W>(k_norm_weight, k_weight, lane);
    {
        const int table_row = min(position, table_positions - 1);
        const float* cos_row = cos_table ? cos_table + (int64_t)table_row * (HEAD_DIM / 2) : nullptr;
        const float* sin_row = sin_table ? sin_table + (int64_t)table_row * (HEAD_DIM / 2) : nullptr;
#pragma unroll
        for (int i = 0; i < HeadRegs<HEAD_DIM>::PAIRS; ++i) {
            const int j = lane + 32 * i;
            const bool in = cos_row != nullptr && j < HEAD_DIM / 2;
            cos_regs.a[i] = in ? round_to<bf16>(cos_row[j]) : 1.0f;
            sin_regs.a[i] = in ? round_to<bf16>(sin_row[j]) : 0.0f;
            cos_regs.b[i] = sin_regs.b[i] = 0.0f;          // unused
        }
    }

    // ---- the keys [lo, position] are cut into `splits` pieces of a size that depends on this
    // request alone; piece `split` is this CTA's.  Keys [first, last] of it are in the cache.
    const int lo = window > 0 ? max(0, position - window + 1) : 0;
    const int range_first = lo - lo % 64;
    const int split_keys = ((position - range_first + pieces) / pieces + TILE - 1) / TILE * TILE;
    const int own_piece = (position - range_first) / split_keys;     // holds the new token
    const int base = range_first + piece * split_keys;
    const int first = max(lo, base);
    // write_cache 2: the new token's key and value are in the cache already (and q is ready): it is
    // a key like the others, nothing of it is taken from the projection
    const int last = min(cached_new ? position : position - 1, base + split_keys - 1);
    const int sub = lane % CPR;                 // which 16-byte chunk of a key's row this lane copies
    const int key_in_instr = lane / CPR;
    const int* table = block_tables + (int64_t)row * table_stride;
    // the cache is [pages, num_kv, page, head_dim]: a key's row for this kv head
    const int64_t row_stride = HEAD_DIM;
    const bf16* k_base = key_cache + sub * 8;
    const bf16* v_base = value_cache + sub * 8;

    // The piece is walked in sub-tiles of WARP_KEYS keys; warp w takes sub-tiles w, w + 4, ...
    const int sub_tiles = last >= first ? (last - base) / WARP_KEYS + 1 : 0;
    int first_tile = max(0, (first - base) / WARP_KEYS);
    first_tile += (warp - first_tile % DEC_WARPS + DEC_WARPS) % DEC_WARPS;
    int mine = first_tile < sub_tiles ? (sub_tiles - 1 - first_tile) / DEC_WARPS + 1 : 0;

    // Cache rows of this warp's keys, looked up once: where a tile of 8 keys lies inside one page,
    // the row of the tile's first key (-1: the page is not there); else one row per key (-1: no key).
    const bool by_tile = page_size % TILE == 0;
    mine = min(mine, by_tile ? warp_slot_capacity : warp_slot_capacity / WARP_KEYS);     // sized for the context limit
    int* my_slots = slot_s + warp * warp_slot_capacity;
    if (by_tile) {
        for (int e = lane; e < mine; e += 32) {
            const int key0 = base + (first_tile + e * DEC_WARPS) * WARP_KEYS;
            const int page = table[key0 / page_size];
            my_slots[e] = page >= 0 ? (page * num_kv + kv_head) * page_size + key0 % page_size : -1;
        }
    } else {
        for (int e = lane; e < mine * WARP_KEYS; e += 32) {
            const int key = base + (first_tile + (e / WARP_KEYS) * DEC_WARPS) * WARP_KEYS + e % WARP_KEYS;
            int slot = -1;
            if (key >= first && key <= last) {
                const int page = table[key / page_size];
                if (page >= 0) slot = (page * num_kv + kv_head) * page_size + key % page_size;
            }
            my_slots[e] = slot;
        }
    }
    __syncwarp();

    auto issue = [&](int i) {                   // the i-th sub-tile of this warp into stage i % DEC_STAGES
        uint4* keys_to = ring_of(warp, i % DEC_STAGES, 0);
        uint4* values_to = ring_of(warp, i % DEC_STAGES, 1);
        const int key0 = base + (first_tile + i * DEC_WARPS) * WARP_KEYS;
#pragma unroll
        for (int u = 0; u < TILE / KPI; ++u) {
            const int key = u * KPI + key_in_instr;
            int slot;
            if (by_tile) {
                const int tile_slot = my_slots[i];
                slot = (tile_slot >= 0 && key0 + key >= first && key0 + key <= last) ? tile_slot + key : -1;
            } else {
                slot = my_slots[i * WARP_KEYS + key];
            }
            const int64_t offset = (int64_t)max(slot, 0) * row_stride;
            const int at = key * CPR + (sub ^ (key & 7));
            cp_async_16(keys_to + at, k_base + offset, slot >= 0);
            cp_async_16(values_to + at, v_base + offset, slot >= 0);
        }
    };
#pragma unroll
    for (int i = 0; i < DEC_STAGES - 1; ++i) {  // in flight before anything of this step is needed
        if (i < mine) issue(i);
        cp_async_commit();
    }

    // ---- the new token.  A warp takes q heads warp, warp + DEC_WARPS, ... of this CTA.  In the CTA
    // whose piece holds the new token it also normalises and rotates the new key for itself (the
    // same arithmetic in every warp) and has the head's score with it at once, without a round
    // through shared memory; the warp of head 0 stores the key, the last warp the value.
    pdl_wait();                                 // the projection comes from the kernel before this one
    {
        const unsigned short* token = reinterpret_cast<const unsigned short*>(qkv) + (int64_t)request * heads * HEAD_DIM;
        const bool new_here = piece == own_piece && !cached_new;
        const bool stores = write_cache == 1 && (y_block % blocks_per_kv) == 0;
        int64_t cache_at = -1;
        if (new_here && stores) {
            const int slot = slots[request];
            if (slot >= 0) cache_at = (((int64_t)(slot / page_size) * num_kv + kv_head) * page_size + slot % page_size) * HEAD_DIM;
        }
        const bool normed = q_weight != nullptr, rotated = cos_table != nullptr;
        HeadRegs<HEAD_DIM> q_head, k_head;
        const bool has_q = warp < heads_here;
        if (has_q) load_head<HEAD_DIM>(q_head, token + (int64_t)(first_q_head + warp) * HEAD_DIM, lane);
        if (new_here && has_q) load_head<HEAD_DIM>(k_head, token + (int64_t)(num_q + kv_head) * HEAD_DIM, lane);
        if (new_here && warp == DEC_WARPS - 1) {
            const unsigned short* v = token + (int64_t)(num_q + num_kv + kv_head) * HEAD_DIM;
            // the loads first: they are ordered with the stores, and one after a store would be
            // another trip to memory
            unsigned short bits[HEAD_DIM / 32];
#pragma unroll
            for (int i = 0; i < HEAD_DIM / 32; ++i) bits[i] = ld_global_u16(v + lane + 32 * i);
#pragma unroll
            for (int i = 0; i < HEAD_DIM / 32; ++i) {
                v_new_s[lane + 32 * i] = bf16_bits_to_float(bits[i]);
                if (cache_at >= 0) reinterpret_cast<unsigned short*>(value_cache + cache_at)[lane + 32 * i] = bits[i];
            }
        }
        if (new_here && has_q) {
            norm_rotate_head<HEAD_DIM>(k_head, normed, k_norm_weight, eps, rotated, cos_regs, sin_regs);
            if (warp == 0 && cache_at >= 0) store_head<HEAD_DIM, bf16>(k_head, key_cache + cache_at, lane);
        }
        for (int h = warp; h < heads_here; h += DEC_WARPS) {
            if (h != warp) load_head<HEAD_DIM>(q_head, token + (int64_t)(first_q_head + h) * HEAD_DIM, lane);
            norm_rotate_head<HEAD_DIM>(q_head, normed, q_norm_weight, eps, rotated, cos_regs, sin_regs);
            store_head<HEAD_DIM, float>(q_head, q_s + h * HEAD_DIM, lane);
            if (new_here) {                     // the head's score with the new key: elements in ascending order a lane
                float dot = 0.0f;
#pragma unroll
                for (int i = 0; i < HeadRegs<HEAD_DIM>::PAIRS; ++i) dot = __fmaf_rn(q_head.a[i], k_head.a[i], dot);
#pragma unroll
                for (int i = 0; i < HeadRegs<HEAD_DIM>::PAIRS; ++i) dot = __fmaf_rn(q_head.b[i], k_head.b[i], dot);
                dot = warp_sum(dot);
                if (lane == 0) s_new_s[h] = __fmul_rn(dot, scale);
            }
        }
    }
    __syncthreads();

    // ---- q as the a operand: row g of the tile is q head g (zero past HPB), two registers a k step
    const int g = lane >> 2, t4 = lane & 3;
    uint32_t q_frag[HEAD_DIM / 16][2];
#pragma unroll
    for (int ks = 0; ks < HEAD_DIM / 16; ++ks) {
        q_frag[ks][0] = q_frag[ks][1] = 0u;
        if (g < heads_here) {
            const float* qh = q_s + g * HEAD_DIM + ks * 16 + 2 * t4;
            q_frag[ks][0] = pack_bf16x2(qh[0], qh[1]);
            q_frag[ks][1] = pack_bf16x2(qh[8], qh[9]);
        }
    }
    if constexpr (TILE == 16) {
        // ---- keys as rows.  S^T[key][head] = K Q^T: the tile's 16 keys are the rows, the CTA's q heads
        // the 8 columns (q_frag is the b operand as it stands: head g, dimensions 2 t4.. of the k
        // step); O^T[dimension][head] += V^T P^T with the keys as k.  A lane holds heads 2 t4 and
        // 2 t4 + 1: of keys g and g + 8 in S^T, of dimensions g and g + 8 of every 16 in O^T.
        float m_run[2] = {-INFINITY, -INFINITY};    // of heads 2 t4, 2 t4 + 1; the same in the 8 lanes of a t4
        float l_run[2] = {0.0f, 0.0f};              // this lane's share (its keys g, g + 8 of every tile)
        float o_run[HEAD_DIM / 16][4];
#pragma unroll
        for (int n = 0; n < HEAD_DIM / 16; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) o_run[n][e] = 0.0f;
        // lane l of an ldmatrix names a row of one of its four 8 x 8 matrices: matrix l / 8, row l % 8
        const int matrix = lane >> 3, matrix_row = lane & 7;
        // K as the a operand: matrices (keys 0..7 | 8..15) x (chunk 2 ks | 2 ks + 1) in that order
        const int k_key = matrix_row + 8 * (matrix & 1);
        const int k_row = k_key * CPR, k_flip = (matrix >> 1) ^ matrix_row;          // chunk ^ (key & 7) = 2 ks ^ k_flip
        // V^T as the a operand (transposing loads): matrices (chunk 2 mt | 2 mt + 1) x (keys 0..7 | 8..15)
        const int v_key = matrix_row + 8 * (matrix >> 1);
        const int v_row = v_key * CPR, v_flip = (matrix & 1) ^ matrix_row;

        // A tile that lies inside a page and inside the piece is copied from one address: what a lane
        // adds to it does not change from tile to tile (chunk `sub` of keys key_in_instr,
        // key_in_instr + KPI, ...; with u KPI + key_in_instr for the key, its place in the stage is
        // (lane_place ^ (u KPI & 7)) + u KPI CPR: one XOR and constants).
        const uint32_t my_ring = smem_address(ring_of(warp, 0, 0));
        const uint32_t lane_place = key_in_instr * CPR + (sub ^ key_in_instr);
        const bf16* k_lane = key_cache + (key_in_instr * HEAD_DIM + sub * 8);
        const bf16* v_lane = value_cache + (key_in_instr * HEAD_DIM + sub * 8);
        auto issue_whole = [&](int i) {
            const int key0 = base + (first_tile + i * DEC_WARPS) * WARP_KEYS;
            const int tile_slot = by_tile ? my_slots[i] : -1;
            if (tile_slot < 0 || key0 < first || key0 + TILE - 1 > last) {           // the whole warp
                issue(i);
                return;
            }
            const uint32_t keys_to = my_ring + (uint32_t)((i % DEC_STAGES) * 2 * TILE_WORDS * 16);
            const bf16* k_from = k_lane + (int64_t)tile_slot * HEAD_DIM;
            const bf16* v_from = v_lane + (int64_t)tile_slot * HEAD_DIM;
#pragma unroll
            for (int u = 0; u < TILE / KPI; ++u) {
                const uint32_t to = keys_to + ((lane_place ^ ((u * KPI) & 7)) + u * KPI * CPR) * 16;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(to), "l"(k_from + u * KPI * HEAD_DIM));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(to + TILE_WORDS * 16), "l"(v_from + u * KPI * HEAD_DIM));
            }
        };

        for (int i = 0; i < mine; ++i) {
            if (i + DEC_STAGES - 1 < mine) issue_whole(i + DEC_STAGES - 1);
            cp_async_commit();
            cp_async_wait<DEC_STAGES - 1>();        // sub-tile i has landed ...
            __syncwarp();                           // ... for every lane of the warp
            const uint4* k_tile = ring_of(warp, i % DEC_STAGES, 0);
            const uint4* v_tile = ring_of(warp, i % DEC_STAGES, 1);
            const int key0 = base + (first_tile + i * DEC_WARPS) * WARP_KEYS;

            // even and odd k steps sum apart: a product waits for the one two before it only
            float s_even[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s_odd[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int ks = 0; ks < HEAD_DIM / 16; ks += 2) {
                uint32_t a_even[4], a_odd[4];
                dec_ldmatrix_x4(a_even, k_tile + k_row + ((2 * ks) ^ k_flip));
                dec_ldmatrix_x4(a_odd, k_tile + k_row + ((2 * ks + 2) ^ k_flip));
                dec_mma_full(s_even, a_even, q_frag[ks][0], q_frag[ks][1]);
                dec_mma_full(s_odd, a_odd, q_frag[ks + 1][0], q_frag[ks + 1][1]);
            }
            // online softmax per head (column): this lane holds keys g (e = 0) and g + 8 (e = 1)
            float score[2][2];                      // [key e][head j]
            float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + g + 8 * e;
                const bool valid = key >= first && key <= last;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    score[e][j] = valid ? __fmul_rn(__fadd_rn(s_even[2 * e + j], s_odd[2 * e + j]), scale) : -INFINITY;
                    tile_max[j] = fmaxf(tile_max[j], score[e][j]);
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                tile_max[j] = fmaxf(tile_max[j], __shfl_xor_sync(0xffffffffu, tile_max[j], 4));
                tile_max[j] = fmaxf(tile_max[j], __shfl_xor_sync(0xffffffffu, tile_max[j], 8));
                tile_max[j] = fmaxf(tile_max[j], __shfl_xor_sync(0xffffffffu, tile_max[j], 16));
            }
            float rescale[2], prob[2][2];
            bool changed = false;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float new_max = fmaxf(m_run[j], tile_max[j]);            // finite: the sub-tile has a valid key
                rescale[j] = m_run[j] == -INFINITY ? 0.0f : __expf(m_run[j] - new_max);
                changed = changed || new_max != m_run[j];
                m_run[j] = new_max;
#pragma unroll
                for (int e = 0; e < 2; ++e) prob[e][j] = score[e][j] == -INFINITY ? 0.0f : __expf(score[e][j] - new_max);
                l_run[j] = l_run[j] * rescale[j] + (prob[0][j] + prob[1][j]);
            }
            // P^T as the b operand: the transposes of P[keys 0..7][heads] and P[keys 8..15][heads]
            const uint32_t p_lo = dec_transpose_8x8(pack_bf16x2(prob[0][0], prob[0][1]));
            const uint32_t p_hi = dec_transpose_8x8(pack_bf16x2(prob[1][0], prob[1][1]));
            if (__any_sync(0xffffffffu, changed)) {
#pragma unroll
                for (int n = 0; n < HEAD_DIM / 16; ++n) {
                    o_run[n][0] *= rescale[0]; o_run[n][1] *= rescale[1];
                    o_run[n][2] *= rescale[0]; o_run[n][3] *= rescale[1];
                }
            }
#pragma unroll
            for (int mt = 0; mt < HEAD_DIM / 16; ++mt) {
                uint32_t a[4];
                dec_ldmatrix_x4_trans(a, v_tile + v_row + ((2 * mt) ^ v_flip));
                dec_mma_full(o_run[mt], a, p_lo, p_hi);
            }
            __syncwarp();                           // the stage may be filled again
        }
        pdl_launch_dependents();

        // ---- the warp's partial result to where its ring was; the lanes' shares of the denominators
        // are added up over the 8 lanes of a t4 first
        cp_async_wait<0>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 4);
            l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 8);
            l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 16);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int head = 2 * t4 + j;
            if (head < heads_here) {
                float* mine_o = warp_o_of(warp) + head * HEAD_DIM;
#pragma unroll
                for (int n = 0; n < HEAD_DIM / 16; ++n) {
                    mine_o[n * 16 + g] = o_run[n][j];
                    mine_o[n * 16 + g + 8] = o_run[n][2 + j];
                }
                if (g == 0) { warp_m_s[warp * HPB + head] = m_run[j]; warp_l_s[warp * HPB + head] = l_run[j]; }
            }
        }
    } else {
        float m_run = -INFINITY, l_run = 0.0f;      // of row g; the four lanes of a row hold the same
        float o_run[HEAD_DIM / 8][4];               // [n tile][row g: columns 2 t4, 2 t4 + 1 | row g + 8: unused]
#pragma unroll
        for (int n = 0; n < HEAD_DIM / 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) o_run[n][i] = 0.0f;

        for (int i = 0; i < mine; ++i) {
            // the next sub-tile is asked for before this one is waited for (asking after the products
            // instead, with every stage filled up front, measured 1 % slower on the whole step)
            if (i + DEC_STAGES - 1 < mine) issue(i + DEC_STAGES - 1);
            cp_async_commit();
            cp_async_wait<DEC_STAGES - 1>();        // sub-tile i has landed ...
            __syncwarp();                           // ... for every lane of the warp
            const uint4* k_tile = ring_of(warp, i % DEC_STAGES, 0);
            const uint4* v_tile = ring_of(warp, i % DEC_STAGES, 1);
            const int key0 = base + (first_tile + i * DEC_WARPS) * WARP_KEYS;

            // S[row][key] for the 8 keys of the tile
            float s_acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            {
                const int key = lane & 7;
#pragma unroll
                for (int ks2 = 0; ks2 < HEAD_DIM / 32; ++ks2) {
                    uint32_t b[4];
                    const int chunk = ks2 * 4 + (lane >> 3);
                    dec_ldmatrix_x4(b, k_tile + key * CPR + (chunk ^ key));
                    dec_mma(s_acc, q_frag[2 * ks2][0], q_frag[2 * ks2][1], b[0], b[1]);
                    dec_mma(s_acc, q_frag[2 * ks2 + 1][0], q_frag[2 * ks2 + 1][1], b[2], b[3]);
                }
            }
            // online softmax of row g over the 8 keys (this lane holds keys 2 t4, 2 t4 + 1)
            float score[2];
            bool valid[2];
            float tile_max = -INFINITY;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + 2 * t4 + e;
                valid[e] = key >= first && key <= last;
                score[e] = valid[e] ? __fmul_rn(s_acc[e], scale) : -INFINITY;
                tile_max = fmaxf(tile_max, score[e]);
            }
            tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
            tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
            const float new_max = fmaxf(m_run, tile_max);          // finite: the sub-tile has a valid key
            const float rescale = m_run == -INFINITY ? 0.0f : __expf(m_run - new_max);
            const bool moved = __any_sync(0xffffffffu, new_max != m_run);
            m_run = new_max;
            float prob[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) prob[e] = valid[e] ? __expf(score[e] - new_max) : 0.0f;
            float sum = prob[0] + prob[1];
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l_run = l_run * rescale + sum;
            const uint32_t p_lo = pack_bf16x2(prob[0], prob[1]);            // keys 0..7; k 8..15 of the product are zero
            if (moved) {
#pragma unroll
                for (int n = 0; n < HEAD_DIM / 8; ++n) { o_run[n][0] *= rescale; o_run[n][1] *= rescale; }
            }
            // O += P V, 32 head dimensions (four n tiles) per ldmatrix
#pragma unroll
            for (int n4 = 0; n4 < HEAD_DIM / 32; ++n4) {
                uint32_t b[4];
                const int key = lane & 7;
                const int chunk = n4 * 4 + (lane >> 3);
                dec_ldmatrix_x4_trans(b, v_tile + key * CPR + (chunk ^ key));
#pragma unroll
                for (int m = 0; m < 4; ++m) dec_mma(o_run[4 * n4 + m], p_lo, 0u, b[m], 0u);
            }
            __syncwarp();                           // the stage may be filled again
        }
        pdl_launch_dependents();

        // ---- the warps' partial results, merged below in a fixed order; a warp's output goes where its
        // ring was (every tile it asked for has been used)
        cp_async_wait<0>();
        __syncwarp();
        if (g < heads_here) {
            float* mine_o = warp_o_of(warp) + g * HEAD_DIM;
#pragma unroll
            for (int n = 0; n < HEAD_DIM / 8; ++n) {
                mine_o[n * 8 + 2 * t4] = o_run[n][0];
                mine_o[n * 8 + 2 * t4 + 1] = o_run[n][1];
            }
            if (t4 == 0) { warp_m_s[warp * HPB + g] = m_run; warp_l_s[warp * HPB + g] = l_run; }
        }
    }
    __syncthreads();
    cluster_wait();
    unsigned char* first_cta = cluster.map_shared_rank(shared_raw, 0);
    float* first_part_m = reinterpret_cast<float*>(first_cta + layout.part_m);       // [splits][HPB]
    float* first_part_l = reinterpret_cast<float*>(first_cta + layout.part_l);
    float* first_part_o = reinterpret_cast<float*>(first_cta + layout.part_o);       // [splits][HPB][HEAD_DIM]
    const float* part_m_s = reinterpret_cast<const float*>(shared_raw + layout.part_m);
    const float* part_l_s = reinterpret_cast<const float*>(shared_raw + layout.part_l);
    const float* part_o_s = reinterpret_cast<const float*>(shared_raw + layout.part_o);
    for (int index = threadIdx.x; index < heads_here * HEAD_DIM; index += blockDim.x) {
        const int h = index / HEAD_DIM, dim = index % HEAD_DIM;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, warp_m_s[w * HPB + h]);
        float l = 0.0f, o = 0.0f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = warp_m_s[w * HPB + h] == -INFINITY ? 0.0f : __expf(warp_m_s[w * HPB + h] - m);
            l += warp_l_s[w * HPB + h] * f;
            o += warp_o_of(w)[h * HEAD_DIM + dim] * f;
        }
        if (piece == own_piece && !cached_new) {   // the new token itself, from shared memory
            const float s = s_new_s[h];
            const float new_max = fmaxf(m, s);
            const float f_old = m == -INFINITY ? 0.0f : __expf(m - new_max);
            const float f_new = __expf(s - new_max);
            l = l * f_old + f_new;
            o = o * f_old + f_new * v_new_s[dim];
            m = new_max;
        }
        if (splits == 1) {                         // nothing to merge with: the same value the merge below gives
            out_row[index] = __float2bfloat16_rn(o / l);
            continue;
        }
        first_part_o[(split * HPB + h) * HEAD_DIM + dim] = o;   // a store into the first CTA's shared memory
        if (dim == 0) { first_part_m[split * HPB + h] = m; first_part_l[split * HPB + h] = l; }
    }

    if (splits == 1) return;

    // ---- the first CTA merges the pieces in rank order
    cluster.sync();
    if (split == 0) {
        // FAR, a request cut over several clusters: this cluster's merged piece goes to global memory
        float* far_mine = nullptr;
        if constexpr (FAR) {
            if (far_groups > 1)
                far_mine = far.pieces + (((int64_t)request * (gridDim.y / far.groups) + y_block) * far.groups + far_group) *
                                            (HPB * (HEAD_DIM + 2));
        }
        for (int index = threadIdx.x; index < heads_here * HEAD_DIM; index += blockDim.x) {
            const int h = index / HEAD_DIM, dim = index % HEAD_DIM;
            float l = 0.0f, o = 0.0f;
            float top = -INFINITY;             // FAR: the maximum that l and o are relative to
            if constexpr (HPB >= 2) {
                // unrolled over the largest cluster, so that the loads and exponentials of all pieces
                // are in flight together; the sums keep the rank order.  (With one q head a CTA the
                // registers of this form would cost the kernel its fourth CTA per SM.)
                float pm[DEC_MAX_SPLITS], pl[DEC_MAX_SPLITS], po[DEC_MAX_SPLITS];
                float m = -INFINITY;
#pragma unroll
                for (int r = 0; r < DEC_MAX_SPLITS; ++r) {
                    const bool in = r < splits;
                    pm[r] = in ? part_m_s[r * HPB + h] : -INFINITY;
                    pl[r] = in ? part_l_s[r * HPB + h] : 0.0f;
                    po[r] = in ? part_o_s[(r * HPB + h) * HEAD_DIM + dim] : 0.0f;
                    m = fmaxf(m, pm[r]);
                }
#pragma unroll
                for (int r = 0; r < DEC_MAX_SPLITS; ++r) {
                    const float f = pm[r] == -INFINITY ? 0.0f : __expf(pm[r] - m);
                    l += pl[r] * f;
                    o += po[r] * f;
                }
                if constexpr (FAR) top = m;
            } else {
                float m = -INFINITY;
                for (int r = 0; r < splits; ++r) m = fmaxf(m, part_m_s[r * HPB + h]);
                for (int r = 0; r < splits; ++r) {
                    const float pm = part_m_s[r * HPB + h];
                    const float f = pm == -INFINITY ? 0.0f : __expf(pm - m);
                    l += part_l_s[r * HPB + h] * f;
                    o += part_o_s[(r * HPB + h) * HEAD_DIM + dim] * f;
                }
                if constexpr (FAR) top = m;
            }
            if constexpr (FAR) {
                if (far_mine) {
                    float* head = far_mine + h * (HEAD_DIM + 2);
                    head[dim] = o;
                    if (dim == 0) { head[HEAD_DIM] = top; head[HEAD_DIM + 1] = l; }
                    continue;
                }
            }
            out_row[index] = __float2bfloat16_rn(o / l);
        }
        if constexpr (FAR) {
            if (far_mine) {
                // Count this cluster in; the one that finds all others counted has their pieces
                // before it (the fences order each cluster's stores before its count, and the
                // last one's loads after it) and merges them in the order of the groups.
                int* last_s = reinterpret_cast<int*>(shared_raw + layout.s_new);      // free by now
                __threadfence();
                __syncthreads();
                if (threadIdx.x == 0) {
                    int* count = far.arrived + (int64_t)request * (gridDim.y / far.groups) + y_block;
                    const int before = atomicAdd(count, 1);
                    const int last = before == far_groups - 1;
                    if (last) *count = 0;                  // for the next launch
                    *last_s = last;
                }
                __syncthreads();
                if (*last_s == 0) return;
                __threadfence();
                const float* all = far_mine - (int64_t)far_group * (HPB * (HEAD_DIM + 2));
                for (int index = threadIdx.x; index < heads_here * HEAD_DIM; index += blockDim.x) {
                    const int h = index / HEAD_DIM, dim = index % HEAD_DIM;
                    float m = -INFINITY;
                    for (int r = 0; r < far_groups; ++r)
                        m = fmaxf(m, __ldcg(all + (r * HPB + h) * (HEAD_DIM + 2) + HEAD_DIM));
                    float l = 0.0f, o = 0.0f;
                    for (int r = 0; r < far_groups; ++r) {
                        const float* head = all + (r * HPB + h) * (HEAD_DIM + 2);
                        const float pm = __ldcg(head + HEAD_DIM);
                        const float f = pm == -INFINITY ? 0.0f : __expf(pm - m);
                        l += __ldcg(head + HEAD_DIM + 1) * f;
                        o += __ldcg(head + dim) * f;
                    }
                    out_row[index] = __float2bfloat16_rn(o / l);
                }
            }
        }
    }
}

// entries of a warp's list of cache slots: one per tile of 8 keys where tiles lie inside pages, else
// one per key; sized for the longest piece a request of max_context tokens is cut into
#undef q_s
#undef v_new_s
#undef s_new_s
#undef warp_m_s
#undef warp_l_s

template <int DEC_WARPS, int TILE>
static int decode_warp_slot_capacity(int max_context, int splits, int page_size) {
    const int split_keys = ((max_context + 64 + splits - 1) / splits + TILE - 1) / TILE * TILE;
    const int tiles = split_keys / (TILE * DEC_WARPS) + 2;
    return page_size % TILE == 0 ? tiles : tiles * TILE;
}

template <int HEAD_DIM, int HPB, int DEC_WARPS, int RESIDENT, int TILE, int DEC_STAGES, typename W, bool FAR = false>
static int launch_decode(const void* qkv, const void* q_weight, const void* k_weight, float eps,
                         const float* cos_table, const float* sin_table, int table_positions,
                         const int* positions, const int* token_row, const int* slots, void* key_cache,
                         void* value_cache, const int* block_tables, int table_stride, int page_size,
                         void* out, int requests, int num_q, int num_kv, int window, float scale,
                         int splits, int write_cache, int max_context, int pdl, cudaStream_t stream, int heads_here,
                         int sm_count, int* clusters_that_fit = nullptr, FarArgs far = FarArgs{1, 0, nullptr, nullptr}) {
    auto kernel = decode_attention_kernel<HEAD_DIM, HPB, DEC_WARPS, RESIDENT, TILE, DEC_STAGES, W, FAR>;
    if (FAR != (far.groups > 1) || (FAR && (splits < 2 || !far.pieces || !far.arrived))) return TVB_BAD_ARGUMENT;
    const int warp_slots = decode_warp_slot_capacity<DEC_WARPS, TILE>(max_context, splits, page_size);
    const DecodeLayout layout = decode_layout(HEAD_DIM, HPB, DEC_WARPS, splits, warp_slots, TILE, DEC_STAGES);
    if (layout.total > 200 * 1024) return TVB_BAD_ARGUMENT;
    static int configured = 0;                   // the largest size asked for so far, per instantiation
    if (layout.total > configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = 200 * 1024;
    }
    TvbLaunch launch(dim3(splits, num_kv * ((num_q / num_kv) / heads_here) * far.groups, requests), dim3(DEC_WARPS * 32),
                     (size_t)layout.total, stream, pdl, splits);
    if (clusters_that_fit) {
        // Not a launch: how many clusters of this shape the GPU holds at once (the CTAs of a cluster
        // need SMs of one GPC; remembered per cluster size and shared memory).
        static int known[DEC_MAX_SPLITS + 1][2] = {};          // [splits] = {shared bytes, clusters}
        if (known[splits][0] != layout.total || known[splits][1] <= 0) {
            int clusters = 0;
            cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &launch.config);
            if (e != cudaSuccess) { cudaGetLastError(); clusters = 0; }
            known[splits][0] = layout.total;
            known[splits][1] = clusters;
        }
        *clusters_that_fit = known[splits][1];
        return 0;
    }
    cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, (const bf16*)qkv, (const W*)q_weight, (const W*)k_weight, eps,
                                       cos_table, sin_table, table_positions, positions, token_row, slots,
                                       (bf16*)key_cache, (bf16*)value_cache, block_tables, table_stride, page_size,
                                       (bf16*)out, num_q, num_kv, window, scale, write_cache, warp_slots, heads_here,
                                       layout, far);
    return e == cudaSuccess ? tvb_last_error() : (int)e;
}

// q heads of one kv head that a CTA serves: as many of the group as a tile holds (8 at head sizes
// up to 128, else 4), so that the keys are read as few times as possible: the largest divisor of the
// group within that.  A group of 5 (40 q heads on 8 kv heads) gives 5, a group of 12 gives 6.
static int decode_heads_per_cta(int group, int head_dim) {
    const int most = head_dim <= 128 ? 8 : 4;
    for (int heads = most < group ? most : group; heads > 1; --heads)
        if (group % heads == 0) return heads;
    return 1;
}

template <typename T> constexpr int tvb_dtype_tag_of();
template <> constexpr int tvb_dtype_tag_of<float>() { return TVB_F32; }
template <> constexpr int tvb_dtype_tag_of<bf16>() { return TVB_BF16; }

// 1 if this library takes the shape: its head size; any whole number of q heads per kv head.
extern "C" int tvb_attention_decode_supports(int head_dim, int num_q, int num_kv, int splits) {
    if (head_dim != TVB_DECODE_HEAD_DIM) return 0;
    if (num_kv <= 0 || num_q <= 0 || num_q % num_kv) return 0;
    return splits >= 1 && splits <= DEC_MAX_SPLITS;
}

// qkv: [requests, (num_q + 2 num_kv) * head_dim] bfloat16, the raw projection of one token per
// request.  Caches: [pages, num_kv, page_size, head_dim].  weight_dtype: TVB_BF16 or TVB_F32 (norm weights; null pointers skip the norm).
// splits (1..8) is the cluster size: the number of pieces every request's keys are cut into.
// max_context bounds position + 1 of every request (it sizes the list of cache slots a warp keeps).
// write_cache: 0 the new key and value are used but not stored, 1 they are stored in slot slots[i],
// 2 they are in the cache already, as the other keys are, and q comes normalised and rotated (the
// decoded tokens of a step that also holds prompt portions, after the pass that prepares all its tokens).
// fits_wide != null: nothing is launched; *fits_wide says whether this call would run as CTAs of
// eight warps with all its clusters on the GPU at once.
static int decode_dispatch(const void* qkv, const void* q_weight, const void* k_weight, float eps,
                           const float* cos_table, const float* sin_table, int table_positions,
                           const int* positions, const int* token_row, const int* slots,
                           void* key_cache, void* value_cache, const int* block_tables,
                           int table_stride, int page_size, void* out, int requests, int num_q,
                           int num_kv, int head_dim, int window, float scale, int splits,
                           int write_cache, int max_context, int weight_dtype, int pdl,
                           void* stream, int* fits_wide, FarArgs far = FarArgs{1, 0, nullptr, nullptr}) {
    if (fits_wide) *fits_wide = 0;
    if (far.groups < 1 || (far.groups > 1 && (head_dim != 128 || splits < 2))) return TVB_BAD_ARGUMENT;
    if (requests <= 0) return 0;
    if (!tvb_attention_decode_supports(head_dim, num_q, num_kv, splits) || page_size <= 0 ||
        requests > 65535 || max_context <= 0)
        return TVB_BAD_ARGUMENT;
    const int group = num_q / num_kv;
    // q heads a CTA serves (they share its keys); the tile that holds them is the next of 1, 2, 4, 8.
    // With eight heads no key is read twice.
    const int heads_here = decode_heads_per_cta(group, head_dim);
    const int hpb = heads_here <= 1 ? 1 : heads_here <= 2 ? 2 : heads_here <= 4 ? 4 : 8;
    cudaStream_t s = (cudaStream_t)stream;
    // The shape of a CTA follows the grid.  A grid of fewer CTAs than SMs (one or two requests) gets
    // eight warps a CTA, each with half as many keys to walk (batch 1, context 2,100: 10.3 us against
    // 12.8 us) and no register cap; grids of up to three CTAs an SM get four warps and three CTAs an
    // SM (160 registers, no spills); larger ones four CTAs an SM: of four warps with 8-key tiles, of
    // three with 16-key tiles (whose rings are twice as large).
    static int sm_count = 0;
    if (sm_count == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
            sm_count = 0;
    }
    // (eight warps a CTA only if every cluster is on the GPU at once: clusters of 8 CTAs of that
    // size fit 14 to 16 times, not 148 / 8 times, and a second round of them doubles the time)
    const long long clusters = (long long)requests * num_kv * (group / heads_here) * far.groups;
    const bool wide = head_dim <= 128 && clusters * splits <= sm_count;
    int wide_room = 0;
    const bool roomy = (long long)requests * num_kv * (group / heads_here) * splits <= 3ll * sm_count;
#define DECODE_ARGS qkv, q_weight, k_weight, eps, cos_table, sin_table, table_positions, positions, \
                    token_row, slots, key_cache, value_cache, block_tables, table_stride, page_size, out, \
                    requests, num_q, num_kv, window, scale, splits, write_cache, max_context, pdl, s, heads_here, \
                    sm_count
#define DECODE_BY_WARPS(D, H, WT)                                       \
    do {                                                                \
        if constexpr (D == 128) {                                             \
            const bool all_at_once = wide && launch_decode<128, H, 8, 1, 16, 2, WT>(DECODE_ARGS, &wide_room) == 0 && clusters <= wide_room; \
            if (fits_wide) { *fits_wide = all_at_once ? 1 : 0; return 0; }        \
            if (far.groups > 1) {                                                 \
                /* several clusters a request: only as CTAs of eight warps that are all on the GPU at once */ \
                if (!all_at_once) return TVB_BAD_ARGUMENT;                        \
                return launch_decode<128, H, 8, 1, 16, 2, WT, true>(DECODE_ARGS, nullptr, far); \
            }                                                                     \
            if (all_at_once) return launch_decode<128, H, 8, 1, 16, 2, WT>(DECODE_ARGS); \
            if (roomy) return launch_decode<128, H, 4, 3, 16, 2, WT>(DECODE_ARGS); \
            return launch_decode<128, H, 3, 4, 16, 2, WT>(DECODE_ARGS);       \
        } else {                                                              \
            const bool all_at_once = wide && launch_decode<D, H, 8, 1, 8, 2, WT>(DECODE_ARGS, &wide_room) == 0 && clusters <= wide_room; \
            if (fits_wide) { *fits_wide = all_at_once ? 1 : 0; return 0; }        \
            if (all_at_once) return launch_decode<D, H, 8, 1, 8, 2, WT>(DECODE_ARGS); \
            if (roomy) return launch_decode<D, H, 4, (D > 128 ? 1 : 3), 8, 2, WT>(DECODE_ARGS); \
            return launch_decode<D, H, 4, (D > 128 ? 1 : 4), 8, 2, WT>(DECODE_ARGS);            \
        }                                                                     \
    } while (0)
#define DECODE_BY_HPB(D, WT)                                            \
    do {                                                                \
        if (hpb == 1) DECODE_BY_WARPS(D, 1, WT);                        \
        if (hpb == 2) DECODE_BY_WARPS(D, 2, WT);                        \
        if (hpb == 8) DECODE_BY_WARPS(D, 8, WT);                        \
        DECODE_BY_WARPS(D, 4, WT);                                      \
    } while (0)
    // this library holds one head size and one type of norm weights
    if (head_dim != TVB_DECODE_HEAD_DIM || weight_dtype != tvb_dtype_tag_of<TVB_DECODE_WEIGHT>()) return TVB_BAD_ARGUMENT;
    DECODE_BY_HPB(TVB_DECODE_HEAD_DIM, TVB_DECODE_WEIGHT);
    return TVB_BAD_ARGUMENT;
}

extern "C" int tvb_attention_decode(const void* qkv, const void* q_weight, const void* k_weight, float eps,
                                    const float* cos_table, const float* sin_table, int table_positions,
                                    const int* positions, const int* token_row, const int* slots,
                                    void* key_cache, void* value_cache, const int* block_tables,
                                    int table_stride, int page_size, void* out, int requests, int num_q,
                                    int num_kv, int head_dim, int window, float scale, int splits,
                                    int write_cache, int max_context, int weight_dtype, int pdl,
                                    void* stream) {
    return decode_dispatch(qkv, q_weight, k_weight, eps, cos_table, sin_table, table_positions, positions, token_row,
                           slots, key_cache, value_cache, block_tables, table_stride, page_size, out, requests, num_q,
                           num_kv, head_dim, window, scale, splits, write_cache, max_context, weight_dtype, pdl,
                           stream, nullptr);
}

// 1 if `requests` rows cut into `splits` pieces run as CTAs of eight warps with every cluster on the
// GPU at once (the form that keeps most bytes in flight per SM when the grid is small); 0 if not,
// or if the shape is not taken.  Launches nothing.
extern "C" int tvb_attention_decode_fits_wide(int requests, int num_q, int num_kv, int head_dim, int page_size,
                                              int splits, int max_context, int weight_dtype) {
    int fits = 0;
    const int code = decode_dispatch(nullptr, nullptr, nullptr, 0.0f, nullptr, nullptr, 0, nullptr, nullptr, nullptr,
                                     nullptr, nullptr, nullptr, 0, page_size, nullptr, requests, num_q, num_kv,
                                     head_dim, 0, 1.0f, splits, 1, max_context, weight_dtype, 0, nullptr, &fits);
    return code == 0 ? fits : 0;
}

// The same with a long request cut over `far_groups` clusters per (kv head, block of q heads), from
// `far_from` keys on (head size 128; every cluster must be on the GPU at once, which
// tvb_attention_decode_fits_wide answers for requests * far_groups rows).  far_pieces: float
// [tvb_attention_decode_far_floats(...)], scratch; far_arrived: int [requests * num_q] or more, zero
// before the first launch (every launch leaves it zero).
extern "C" int tvb_attention_decode_far(const void* qkv, const void* q_weight, const void* k_weight, float eps,
                                        const float* cos_table, const float* sin_table, int table_positions,
                                        const int* positions, const int* token_row, const int* slots,
                                        void* key_cache, void* value_cache, const int* block_tables,
                                        int table_stride, int page_size, void* out, int requests, int num_q,
                                        int num_kv, int head_dim, int window, float scale, int splits,
                                        int write_cache, int max_context, int weight_dtype, int pdl,
                                        int far_groups, int far_from, float* far_pieces, int* far_arrived,
                                        void* stream) {
    if (far_groups < 2 || far_from < 1 || !far_pieces || !far_arrived) return TVB_BAD_ARGUMENT;
    return decode_dispatch(qkv, q_weight, k_weight, eps, cos_table, sin_table, table_positions, positions, token_row,
                           slots, key_cache, value_cache, block_tables, table_stride, page_size, out, requests, num_q,
                           num_kv, head_dim, window, scale, splits, write_cache, max_context, weight_dtype, pdl,
                           stream, nullptr, FarArgs{far_groups, far_from, far_pieces, far_arrived});
}

// floats of scratch that tvb_attention_decode_far needs
extern "C" long long tvb_attention_decode_far_floats(int requests, int num_q, int num_kv, int head_dim, int far_groups) {
    if (num_kv <= 0 || num_q <= 0 || num_q % num_kv || requests <= 0 || far_groups < 1) return 0;
    const int heads_here = decode_heads_per_cta(num_q / num_kv, head_dim);
    const int hpb = heads_here <= 1 ? 1 : heads_here <= 2 ? 2 : heads_here <= 4 ? 4 : 8;
    return (long long)requests * (num_q / heads_here) * far_groups * hpb * (head_dim + 2);
}
