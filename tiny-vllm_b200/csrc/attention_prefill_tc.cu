// Prefill attention for bfloat16 and head size 128 on the fifth-generation tensor cores:
// tiles of up to 128 consecutive query tokens of one request and one q head against the paged
// cache.  S = Q K^T and O += P V are tcgen05.mma with the accumulators in tensor memory; Q, K
// and V tiles arrive through tensor-map copies (K and V page by page, straight from the cache
// [pages, kv_heads, page_size, 128]) in the 128-byte swizzle.  256 threads, two per query row
// (64 keys of a block each), read S from tensor memory, apply the mask and the online softmax in
// float32 and write P as bfloat16 into shared memory for the second product.  O stays in tensor
// memory over all blocks of a tile; a row's part of it is scaled there only when the row's
// maximum has grown by more than 2^8 since the reference that its exponentials use was set (the
// denominator carries the same reference, so the quotient is the same softmax).
//
// Roles: warp 0 issues the copies (lane p the page p of a block), warp 1 one thread issues the
// products, warps 2..9 are the softmax rows.  S is double-buffered, so S of block j + 1 is
// computed while the rows work on block j.  Keys are walked in blocks that start at
// absolute multiples of 128, so a row's arithmetic does not depend on how the prompt was cut.
// Persistent CTAs take (tile, head) items, the tiles sorted by the host with the longest first.
//
// Stands where the reference calls torch's scaled_dot_product_attention per request after
// gathering the history into a contiguous copy (tinyvllm/runtime/attention.py:112-147,
// tinyvllm/paged_kv.py:111-127).  P is rounded to bfloat16 for the second product while the
// denominator sums the unrounded values (as tinyvllm/kernels/paged_decode.cu:322-356 does).
//
// Whole pages are copied: cache slots past a request's last key are read and multiplied by zero,
// so they must hold finite values (a cache that starts as zeros and only receives finite keys
// and values does).
//
// Every wait on an mbarrier is bounded (see tc5.cuh); a wait that gives up is reported by
// tvb_attention_prefill_tc_status.
#include <mutex>
#include <unordered_map>

#include "tc5.cuh"

namespace {

constexpr int QT = 128;                      // query rows of a tile = lanes of tensor memory
constexpr int KT = 128;                      // keys of a block
constexpr int HD = 128;                      // head size
constexpr int HALF_BYTES = 128 * 64 * 2;     // [128 rows, 64 values] bfloat16: one swizzled sub-tile
constexpr int TILE_BYTES = 2 * HALF_BYTES;   // a Q, K, V or P tile
constexpr int SLOTS = 4;                     // ring of K / V tiles
constexpr int THREADS = 320;
constexpr int ROW_WARPS = 8;
constexpr uint32_t TMEM_COLS = 512;          // S0 S1 O, 128 float32 columns each (a power of two is allocated)
constexpr float RESCALE_STEP = 8.0f;         // log2 of the growth of a row's maximum that moves its reference

// barrier numbers
constexpr int B_Q_FULL = 0, B_Q_EMPTY = 1, B_KV_FULL = 2, B_KV_EMPTY = B_KV_FULL + SLOTS,
              B_S_FULL = B_KV_EMPTY + SLOTS, B_S_EMPTY = B_S_FULL + 2, B_P_FULL = B_S_EMPTY + 2,
              B_O_DONE = B_P_FULL + 1, B_O_FREE = B_O_DONE + 1, B_PAIR = B_O_FREE + 1, BARRIERS = B_PAIR + 4;
constexpr int EXCHANGE_BYTES = 2 * QT * 2 * 4;      // [buffer][row][half] float
constexpr int SHARED_BYTES = TILE_BYTES * (1 + SLOTS + 1) + EXCHANGE_BYTES + BARRIERS * 8 + 16 + 1024;

__device__ int tvb_attention_prefill_tc_status_word = 0;

struct Item {
    int first, count, p0, head, kv_head, block0, blocks, valid_pages;
    const int* table;
};

__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// 32 lanes x 32 consecutive float32 columns back into tensor memory.
__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* block_tables, int table_stride,
                            const int* positions, const int* tile_row, const int* tile_first, const int* tile_count,
                            bf16* out, int64_t out_stride, int num_tiles, int num_q, int num_kv, int page_size,
                            int window, float scale_log2) {
    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (smem_address(raw_shared) + 1023u) & ~1023u;
    uint8_t* aligned = raw_shared + (base - smem_address(raw_shared));
    const uint32_t q_at = base;
    const uint32_t kv_at = base + TILE_BYTES;
    const uint32_t p_at = kv_at + SLOTS * TILE_BYTES;
    uint8_t* p_generic = aligned + TILE_BYTES * (1 + SLOTS);
    float* exchange = reinterpret_cast<float*>(aligned + TILE_BYTES * (1 + SLOTS + 1));      // [2][QT][2]
    const uint32_t bars = p_at + TILE_BYTES + EXCHANGE_BYTES;
    auto bar = [&](int i) { return bars + 8u * i; };
    uint32_t* tmem_base_slot =
        reinterpret_cast<uint32_t*>(aligned + TILE_BYTES * (1 + SLOTS + 1) + EXCHANGE_BYTES + BARRIERS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    int* status = &tvb_attention_prefill_tc_status_word;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int items = num_tiles * num_q;
    const int pages_per_block = KT / page_size;

    if (threadIdx.x == 0) {
        for (int i = 0; i < BARRIERS; ++i) {
            const bool by_rows = (i >= B_S_EMPTY && i < B_S_EMPTY + 2) || i == B_P_FULL || i == B_O_FREE;
            mbar_init(bar(i), by_rows ? ROW_WARPS : (i >= B_PAIR ? 2 : 1));
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
    }
    if (warp == 1) tmem_alloc(smem_address(tmem_base_slot), TMEM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;

    // The items of this CTA: rounds go forth and back over the CTAs, so that the CTA with the
    // longest item of one round gets the shortest of the next.
    auto item_of = [&](int round, Item& it) -> bool {
        const int g = (int)gridDim.x, c = (int)blockIdx.x;
        const int index = round * g + ((round & 1) ? g - 1 - c : c);
        if (index >= items) return false;
        const int tile = index / num_q;
        it.head = index % num_q;
        it.kv_head = it.head / (num_q / num_kv);
        it.first = tile_first[tile];
        it.count = tile_count[tile];
        it.p0 = positions[it.first];
        it.table = block_tables + (int64_t)tile_row[tile] * table_stride;
        const int lowest = window > 0 ? max(0, it.p0 - window + 1) : 0;
        it.block0 = lowest / KT;
        it.blocks = (it.p0 + it.count + KT - 1) / KT - it.block0;
        it.valid_pages = (it.p0 + it.count + page_size - 1) / page_size;
        return true;
    };

    if (warp == 0) {
        // ---- copies, in the order in which the products use the tiles: K0, K1, V0, K2, V1, ...
        // The whole warp takes part: lane p looks up page p of a block and issues its two copies;
        // lane 0 waits for the slot (with the limit) and arms the barrier.
        uint32_t ring = 0;
        int done_items = 0;
        bool alive = true;
        auto lane_wait = [&](int barrier, uint32_t parity, int code) -> bool {
            int ready = lane == 0 ? (int)mbar_wait(bar(barrier), parity, abort_flag, status, code) : 1;
            return __shfl_sync(0xffffffffu, ready, 0) != 0;
        };
        // page of this lane in `block`; -1 (a coordinate that reads zeros) past the request's keys
        auto page_of = [&](const Item& it, int block) -> int {
            const int index = block * pages_per_block + lane;
            return lane < pages_per_block && index < it.valid_pages ? __ldg(it.table + index) : -1;
        };
        auto load_tile = [&](const CUtensorMap* map, const Item& it, int page) -> bool {
            const int slot = ring % SLOTS;
            const uint32_t phase = (ring / SLOTS) & 1u;
            if (!lane_wait(B_KV_EMPTY + slot, phase ^ 1u, 1)) return false;
            if (lane == 0) mbar_arrive_expect(bar(B_KV_FULL + slot), TILE_BYTES);
            __syncwarp();
            if (lane < pages_per_block) {
                const uint32_t dst = kv_at + slot * TILE_BYTES + (uint32_t)(lane * page_size * 128);
                tma_load_4d(dst, map, 0, 0, it.kv_head, page, bar(B_KV_FULL + slot));
                tma_load_4d(dst + HALF_BYTES, map, 64, 0, it.kv_head, page, bar(B_KV_FULL + slot));
            }
            ++ring;
            return true;
        };
        for (int round = 0; alive; ++round) {
            Item it;
            if (!item_of(round, it)) break;
            // pages of the block whose V is next, of the block whose K is next, and of the one after
            int page_v = page_of(it, it.block0);
            int page_k = it.blocks > 1 ? page_of(it, it.block0 + 1) : -1;
            if (!lane_wait(B_Q_EMPTY, (done_items & 1u) ^ 1u, 2)) break;
            if (lane == 0) {
                mbar_arrive_expect(bar(B_Q_FULL), TILE_BYTES);
                tma_load_2d(q_at, &map_q, it.head * HD, it.first, bar(B_Q_FULL));
                tma_load_2d(q_at + HALF_BYTES, &map_q, it.head * HD + 64, it.first, bar(B_Q_FULL));
            }
            alive = load_tile(&map_k, it, page_v);
            for (int j = 0; j < it.blocks && alive; ++j) {
                const int page_after = j + 2 < it.blocks ? page_of(it, it.block0 + j + 2) : -1;
                if (j + 1 < it.blocks) alive = load_tile(&map_k, it, page_k);
                if (alive) alive = load_tile(&map_v, it, page_v);
                page_v = page_k;
                page_k = page_after;
            }
            ++done_items;
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- products
            constexpr uint32_t idesc_qk = instruction_descriptor_bf16(QT, KT, false);
            constexpr uint32_t idesc_pv = instruction_descriptor_bf16(QT, HD, true);
            uint32_t ring = 0, g = 0;
            int done_items = 0;
            bool alive = true;
            // S[g & 1] = Q K^T for global block g
            auto issue_qk = [&](uint32_t gi) -> bool {
                const int slot = ring % SLOTS;
                const uint32_t phase = (ring / SLOTS) & 1u, b = gi & 1u, use = (gi >> 1) & 1u;
                if (!mbar_wait(bar(B_KV_FULL + slot), phase, abort_flag, status, 3)) return false;
                if (!mbar_wait(bar(B_S_EMPTY + b), use ^ 1u, abort_flag, status, 4)) return false;
                tc_fence_after_sync();
                const uint32_t k_tile = kv_at + slot * TILE_BYTES;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t half = (kk / 4) * HALF_BYTES, step = 2u * (kk % 4);
                    tc_mma(tmem_base + b * KT, tile_descriptor(q_at + half) + step,
                           tile_descriptor(k_tile + half) + step, idesc_qk, kk != 0);
                }
                tc_commit(bar(B_KV_EMPTY + slot));
                tc_commit(bar(B_S_FULL + b));
                ++ring;
                return true;
            };
            // O (+)= P V for global block g; the first block of an item starts O afresh
            auto issue_pv = [&](uint32_t gi, bool first_of_item) -> bool {
                const int slot = ring % SLOTS;
                const uint32_t phase = (ring / SLOTS) & 1u;
                if (!mbar_wait(bar(B_KV_FULL + slot), phase, abort_flag, status, 5)) return false;
                if (!mbar_wait(bar(B_P_FULL), gi & 1u, abort_flag, status, 6)) return false;
                if (first_of_item && !mbar_wait(bar(B_O_FREE), (done_items & 1u) ^ 1u, abort_flag, status, 7))
                    return false;
                tc_fence_after_sync();
                const uint32_t v_tile = kv_at + slot * TILE_BYTES, p_tile = p_at;
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk) {
                    // 16 keys: 32 bytes inside a row of P, two 1024-byte atoms of V
                    const uint32_t half = (kk / 4) * HALF_BYTES, step = 2u * (kk % 4);
                    tc_mma(tmem_base + 2 * KT, tile_descriptor(p_tile + half) + step,
                           tile_descriptor_mn_major(v_tile + kk * 2048, HALF_BYTES), idesc_pv,
                           !(first_of_item && kk == 0));
                }
                tc_commit(bar(B_KV_EMPTY + slot));
                tc_commit(bar(B_O_DONE));
                ++ring;
                return true;
            };
            for (int round = 0; alive; ++round) {
                Item it;
                if (!item_of(round, it)) break;
                if (!mbar_wait(bar(B_Q_FULL), done_items & 1u, abort_flag, status, 8)) break;
                tc_fence_after_sync();
                alive = issue_qk(g);
                if (alive && it.blocks == 1) tc_commit(bar(B_Q_EMPTY));
                for (int j = 0; j < it.blocks && alive; ++j) {
                    if (j + 1 < it.blocks) {
                        alive = issue_qk(g + j + 1);
                        if (alive && j + 2 == it.blocks) tc_commit(bar(B_Q_EMPTY));
                    }
                    if (alive) alive = issue_pv(g + j, j == 0);
                }
                g += it.blocks;
                ++done_items;
            }
        }
        __syncwarp();
    } else {
        // ---- softmax rows: two threads per query row, 64 keys of a block each.  Warps 2..9: the
        // warp's number modulo 4 names the 32 lanes of tensor memory it may read, warps w and w + 4
        // share them and take the first and the second 64 columns.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_address = tmem_base + ((uint32_t)(quarter * 32) << 16);
        // every lane waits (with the limit); the warp goes on only if all of them saw the phase
        auto warp_wait = [&](int barrier, uint32_t parity, int code) -> bool {
            const bool seen = mbar_wait(bar(barrier), parity, abort_flag, status, code);
            return __all_sync(0xffffffffu, seen);
        };
        auto warp_arrive = [&](int barrier) {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(barrier));
        };
        // the two warps that share 32 query rows meet (a bounded wait, as everywhere)
        uint32_t pair_phase = 0;
        auto pair_sync = [&]() -> bool {
            warp_arrive(B_PAIR + quarter);
            const bool met = warp_wait(B_PAIR + quarter, pair_phase, 14);
            pair_phase ^= 1u;
            return met;
        };
        uint32_t g = 0;
        int done_items = 0;
        bool alive = true;
        for (int round = 0; alive; ++round) {
            Item it;
            if (!item_of(round, it)) break;
            const int q_pos = it.p0 + row;
            const int lowest = window > 0 ? q_pos - window + 1 : 0;      // first key this row sees
            float reference = -INFINITY;      // what the exponentials of this row subtract (in log2 units)
            float l = 0.0f;                   // this thread's part of the denominator
            for (int j = 0; j < it.blocks && alive; ++j) {
                const uint32_t gi = g + j, b = gi & 1u, use = (gi >> 1) & 1u;
                const int key0 = (it.block0 + j) * KT + half * 64;
                if (!warp_wait(B_S_FULL + b, use, 10)) { alive = false; break; }
                tc_fence_after_sync();
                uint32_t v[64];
                tmem_load_32(lane_address + b * KT + half * 64, v);
                tmem_load_32(lane_address + b * KT + half * 64 + 32, v + 32);
                tmem_load_wait();
                // S is not read again: the products of the block after next may overwrite it
                tc_fence_before_sync();
                warp_arrive(B_S_EMPTY + b);
                // below every row's diagonal and inside every row's window: no mask
                const bool full = key0 + 63 <= it.p0 && (window <= 0 || key0 >= it.p0 + QT - 1 - window + 1);
                float s[64];
                float part[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                if (full) {
#pragma unroll
                    for (int e = 0; e < 64; ++e) {
                        s[e] = __uint_as_float(v[e]) * scale_log2;
                        part[e & 3] = fmaxf(part[e & 3], s[e]);
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 64; ++e) {
                        const int key = key0 + e;
                        s[e] = key > q_pos || key < lowest ? -INFINITY : __uint_as_float(v[e]) * scale_log2;
                        part[e & 3] = fmaxf(part[e & 3], s[e]);
                    }
                }
                const float mine = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
                float* shared_max = exchange + (b * QT + row) * 2;
                shared_max[half] = mine;
                if (!pair_sync()) { alive = false; break; }
                const float block_max = fmaxf(mine, shared_max[half ^ 1]);
                // the reference moves when the maximum has outgrown it by more than 2^RESCALE_STEP
                const bool moves = block_max > reference + RESCALE_STEP || (reference == -INFINITY && block_max > -INFINITY);
                float factor = 1.0f;
                if (moves) {
                    factor = exp2_fast(reference - block_max);       // 0 for a row that had seen no key
                    reference = block_max;
                    l *= factor;
                }
                // a row that has seen no key yet subtracts 0 so that no inf - inf appears
                const float subtract = reference == -INFINITY ? 0.0f : reference;
                uint4 packed[8];
                float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int e = 0; e < 64; e += 8) {
                    float p[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        p[i] = exp2_fast(s[e + i] - subtract);
                        sums[i & 3] += p[i];
                    }
                    packed[e / 8] = pack_bf16x8(p);
                }
                l += (sums[0] + sums[1]) + (sums[2] + sums[3]);
                // The product of the block before has finished: P may be overwritten and O scaled.  Every
                // completion of O_DONE is waited for in turn (a parity wait cannot tell a phase from the one
                // two before it).
                if (j > 0 && !warp_wait(B_O_DONE, (gi - 1) & 1u, 12)) { alive = false; break; }
                if (j > 0 && __any_sync(0xffffffffu, moves)) {
                    // scale this thread's 64 columns of O where the products so far have left them
                    tc_fence_after_sync();
#pragma unroll
                    for (int c = 0; c < 64; c += 32) {
                        uint32_t o[32];
                        tmem_load_32(lane_address + 2 * KT + half * 64 + c, o);
                        tmem_load_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * factor);
                        tmem_store_32(lane_address + 2 * KT + half * 64 + c, o);
                    }
                    tmem_store_wait();
                    tc_fence_before_sync();
                }
                // row-major [128 rows, 64 keys], 16-byte chunks swizzled by the row
                uint8_t* p_row = p_generic + half * HALF_BYTES + row * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(p_row + ((c ^ (row & 7)) * 16)) = packed[c];
                fence_async_shared();
                warp_arrive(B_P_FULL);
            }
            if (!alive) break;
            // ---- the tile's result: O / (both halves of the denominator)
            const uint32_t last = g + it.blocks - 1;
            float* shared_sum = exchange + ((last & 1u) * QT + row) * 2;
            if (!pair_sync()) break;                  // the maxima of the last block have been read
            shared_sum[half] = l;
            if (!pair_sync()) break;
            const float total = l + shared_sum[half ^ 1];
            if (!warp_wait(B_O_DONE, last & 1u, 13)) break;
            tc_fence_after_sync();
            uint32_t o[64];
            tmem_load_32(lane_address + 2 * KT + half * 64, o);
            tmem_load_32(lane_address + 2 * KT + half * 64 + 32, o + 32);
            tmem_load_wait();
            tc_fence_before_sync();
            warp_arrive(B_O_FREE);
            g += it.blocks;
            ++done_items;
            if (row < it.count) {
                const float inverse = total > 0.0f ? 1.0f / total : 0.0f;
                bf16* out_row = out + (int64_t)(it.first + row) * out_stride + it.head * HD + half * 64;
#pragma unroll
                for (int e = 0; e < 64; e += 8) {
                    float f[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(o[e + i]) * inverse;
                    *reinterpret_cast<uint4*>(out_row + e) = pack_bf16x8(f);
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // copies or products may still be in flight towards this CTA's memory: give them time
        const long long started = clock64();
        while (clock64() - started < 400000) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_free(tmem_base, TMEM_COLS);
    }
}

struct MapKey {
    const void* p;
    long long pages;
    int kv_heads, page_size;
    bool operator==(const MapKey& o) const {
        return p == o.p && pages == o.pages && kv_heads == o.kv_heads && page_size == o.page_size;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.p) ^ (size_t)(k.pages * 131 + k.kv_heads * 17 + k.page_size);
    }
};

// Map of a cache [pages, kv_heads, page_size, 128]: boxes of one page of one kv head, 64 values wide.
bool cache_map(CUtensorMap* map, const void* cache, long long pages, int kv_heads, int page_size) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> known;
    static std::mutex guard;
    std::lock_guard<std::mutex> lock(guard);
    const MapKey key{cache, pages, kv_heads, page_size};
    auto found = known.find(key);
    if (found != known.end()) {
        *map = found->second;
        return true;
    }
    const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)page_size, (cuuint64_t)kv_heads, (cuuint64_t)pages};
    const cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)page_size * HD * 2,
                                   (cuuint64_t)kv_heads * page_size * HD * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)page_size, 1, 1};
    if (!tvb_make_map(map, cache, 4, dims, strides, box)) return false;
    if (known.size() > 4096) known.clear();
    known.emplace(key, *map);
    return true;
}

}  // namespace

extern "C" int tvb_attention_prefill_tc_tile_tokens() { return QT; }

// Head size 128, pages of 8 to 128 tokens (a power of two), q heads a multiple of kv heads.
extern "C" int tvb_attention_prefill_tc_supports(int head_dim, int num_q, int num_kv, int page_size) {
    return head_dim == HD && num_q > 0 && num_kv > 0 && num_q % num_kv == 0 && page_size >= 8 && page_size <= KT &&
           (page_size & (page_size - 1)) == 0;
}

// 0, or which wait gave up in some launch since the last call; reading clears it.  Synchronises.
extern "C" int tvb_attention_prefill_tc_status() {
    int value = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&value, tvb_attention_prefill_tc_status_word, sizeof(int)) != cudaSuccess) return -1;
    if (value != 0) cudaMemcpyToSymbol(tvb_attention_prefill_tc_status_word, &zero, sizeof(int));
    return value;
}

// q: [tokens, q_token_stride] bfloat16, the q heads of token t at q + t * q_token_stride (norm and
// rotation applied); key_cache, value_cache: [pages, num_kv, page_size, 128]; block_tables
// [rows, table_stride]; positions [tokens]; tile_row / tile_first / tile_count [num_tiles]: request
// row, first flat token and number of tokens (<= 128) of each tile, longest context first;
// out [tokens, num_q * 128].  window 0: none.
extern "C" int tvb_attention_prefill_tc(const void* q, long long q_token_stride, long long tokens,
                                        const void* key_cache, const void* value_cache, long long pages,
                                        const int* block_tables, int table_stride, const int* positions,
                                        const int* tile_row, const int* tile_first, const int* tile_count,
                                        int num_tiles, void* out, int num_q, int num_kv, int head_dim, int page_size,
                                        int window, float scale, void* stream) {
    if (num_tiles <= 0 || tokens <= 0) return 0;
    if (!tvb_attention_prefill_tc_supports(head_dim, num_q, num_kv, page_size) || q_token_stride % 8 ||
        ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)key_cache & 15) || ((uintptr_t)value_cache & 15) ||
        pages <= 0 || window < 0)
        return TVB_BAD_ARGUMENT;
    const int sms = tvb_sm_count();
    if (sms <= 0) return (int)cudaErrorInvalidDevice;
    CUtensorMap map_q, map_k, map_v;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)num_q * HD, (cuuint64_t)tokens};
        const cuuint64_t strides[1] = {(cuuint64_t)q_token_stride * 2};
        const cuuint32_t box[2] = {64, QT};
        if (!tvb_make_map(&map_q, q, 2, dims, strides, box)) return (int)cudaErrorNotSupported;
    }
    if (!cache_map(&map_k, key_cache, pages, num_kv, page_size) ||
        !cache_map(&map_v, value_cache, pages, num_kv, page_size))
        return (int)cudaErrorNotSupported;
    auto kernel = attention_prefill_tc_kernel;
    static bool configured[64] = {false};
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64 && !configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SHARED_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured[device] = true;
    }
    const long long items = (long long)num_tiles * num_q;
    const int ctas = (int)(items < sms ? items : sms);
    TvbLaunch launch(dim3(ctas), dim3(THREADS), SHARED_BYTES, (cudaStream_t)stream, 0);
    cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, map_q, map_k, map_v, block_tables, table_stride,
                                       positions, tile_row, tile_first, tile_count, (bf16*)out,
                                       (int64_t)num_q * HD, num_tiles, num_q, num_kv, page_size, window,
                                       scale * 1.4426950408889634f);
    return (int)e;
}
