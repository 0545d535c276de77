// Prefill attention for bfloat16 and head size 128 on the fifth-generation tensor cores:
// tiles of up to 128 consecutive query tokens of one request and one q head against the paged
// cache.  S = Q K^T and O += P V are tcgen05.mma with the accumulators in tensor memory; Q, K
// and V tiles arrive through tensor-map copies (K and V page by page, straight from the cache
// [pages, kv_heads, page_size, 128]) in the 128-byte swizzle.
//
// The blocks of 128 keys of a tile go alternately to two groups of 128 softmax threads (one
// thread per query row).  Each group has its own S and its own O in tensor memory, with its own
// running reference and denominator, so the two chains (read S, mask, maximum, exponentials in
// float32, P as bfloat16) do not wait for each other: one group's exponentials run under the
// other's waits.  P never leaves tensor memory: a thread writes its row of P over the columns of
// S it has read (two bfloat16 per column), and the second product takes its a operand from there.  A row's part of O
// is scaled in tensor memory only when the row's maximum has grown by more than 2^8 since the
// reference that its exponentials use was set (the denominator carries the same reference).  At
// the end of a tile the first group merges the two accumulators:
// (O_a 2^(m_a - m) + O_b 2^(m_b - m)) / (l_a 2^(m_a - m) + l_b 2^(m_b - m)).
//
// Roles: warp 0 issues the copies (lane p the page p of a block), one thread of warp 1 issues the
// products Q K^T and one thread of warp 10 the products P V (each has its own waits and commits
// to do between products, and the tensor pipe takes the other's meanwhile), warps 2..5 and 6..9
// are the two softmax groups.  Keys are walked in blocks that start
// at absolute multiples of 128, even blocks to the first group, so a row's arithmetic does not
// depend on how the prompt was cut.  Persistent CTAs take (tile, head) items, the tiles sorted by
// the host with the longest first.
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
constexpr int SLOTS = 5;                     // ring of K / V tiles
constexpr int THREADS = 352;                 // copy warp, issuer of Q K^T, 8 softmax warps, issuer of P V
constexpr int GROUP_WARPS = 4;               // warps of one softmax group
constexpr uint32_t TMEM_COLS = 512;          // S_a S_b O_a O_b, 128 float32 columns each
constexpr float RESCALE_STEP = 8.0f;         // log2 of the growth of a row's maximum that moves its reference

// barrier numbers; [2] = one per softmax group
constexpr int B_Q_FULL = 0, B_Q_EMPTY = 1, B_KV_FULL = 2, B_KV_EMPTY = B_KV_FULL + SLOTS,
              B_S_FULL = B_KV_EMPTY + SLOTS, B_P_FULL = B_S_FULL + 2, B_P_READ = B_P_FULL + 2,
              B_O_LAST = B_P_READ + 2, B_O_FREE = B_O_LAST + 2, B_SECOND_DONE = B_O_FREE + 2, B_FIRST_TOOK = B_SECOND_DONE + 1,
              BARRIERS = B_FIRST_TOOK + 1;
constexpr int EXCHANGE_BYTES = QT * 2 * 4;          // [row][reference, denominator] of the second group
constexpr int SHARED_BYTES = TILE_BYTES * (1 + SLOTS) + EXCHANGE_BYTES + BARRIERS * 8 + 16 + 1024;

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

template <bool PAIRED>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_k_run,
                            const __grid_constant__ CUtensorMap map_v_run, int run, const int* block_tables, int table_stride,
                            const int* positions, const int* tile_row, const int* tile_first, const int* tile_count,
                            bf16* out, int64_t out_stride, int num_tiles, int num_q, int num_kv, int page_size,
                            int window, float scale_log2) {
    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (smem_address(raw_shared) + 1023u) & ~1023u;
    uint8_t* aligned = raw_shared + (base - smem_address(raw_shared));
    // PAIRED: two q heads of one kv head at a time, one softmax group each, both on every block of
    // keys: a K or V tile in shared memory serves both (two Q tiles and a ring of four; else one
    // and five).
    constexpr int RING = PAIRED ? SLOTS - 1 : SLOTS;
    const uint32_t q_at = base;
    const uint32_t kv_at = base + (PAIRED ? 2 : 1) * TILE_BYTES;
    float* exchange = reinterpret_cast<float*>(aligned + TILE_BYTES * (1 + SLOTS));      // [QT][2]
    const uint32_t bars = base + (1 + SLOTS) * TILE_BYTES + EXCHANGE_BYTES;
    auto bar = [&](int i) { return bars + 8u * i; };
    uint32_t* tmem_base_slot =
        reinterpret_cast<uint32_t*>(aligned + TILE_BYTES * (1 + SLOTS) + EXCHANGE_BYTES + BARRIERS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    int* status = &tvb_attention_prefill_tc_status_word;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_tile = PAIRED ? num_q / 2 : num_q;       // items of a tile of tokens
    const int items = num_tiles * per_tile;
    const int pages_per_block = KT / page_size;

    if (threadIdx.x == 0) {
        for (int i = 0; i < BARRIERS; ++i) {
            const bool by_group = (i >= B_P_FULL && i < B_P_FULL + 2) || (i >= B_O_FREE && i < B_O_FREE + 2) ||
                                  i == B_SECOND_DONE || i == B_FIRST_TOOK;
            mbar_init(bar(i), by_group ? GROUP_WARPS : 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
        if (!PAIRED && run > 1) {
            prefetch_tensormap(&map_k_run);
            prefetch_tensormap(&map_v_run);
        }
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
        const int tile = index / per_tile;
        it.head = (index % per_tile) * (PAIRED ? 2 : 1);
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
            const int slot = ring % RING;
            const uint32_t phase = (ring / RING) & 1u;
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
        // The same for one head an item, where the products wait for their tiles: small pages that
        // lie one after the other in the cache come in one copy of `run` pages (a copy of 2 KB costs
        // the copy unit nearly what one of 4 KB does: 1.5 us a block of 128 keys with pages of 16
        // tokens copied singly, 1.15 us in pairs); a run that is broken, or reaches past the
        // request's pages, comes page by page.  With two heads an item the copies are not what the
        // products wait for, and this longer code on a warp that shares its issue slots with two
        // softmax warps cost 6 % there (8,192 tokens: 302 against 281 us).
        auto load_tile_runs = [&](const CUtensorMap* map, const CUtensorMap* map_run, const Item& it, int page) -> bool {
            const int slot = ring % RING;
            const uint32_t phase = (ring / RING) & 1u;
            if (!lane_wait(B_KV_EMPTY + slot, phase ^ 1u, 1)) return false;
            if (lane == 0) mbar_arrive_expect(bar(B_KV_FULL + slot), TILE_BYTES);
            bool together = false;
            if (run > 1) {
                const int place = lane & (run - 1);
                const int leader_page = __shfl_sync(0xffffffffu, page, lane - place);
                const bool in_place = page >= 0 && leader_page >= 0 && page == leader_page + place;
                const uint32_t run_lanes = ((1u << run) - 1u) << (lane - place);
                together = (__ballot_sync(0xffffffffu, in_place) & run_lanes) == run_lanes;
            }
            __syncwarp();
            if (lane < pages_per_block) {
                const uint32_t dst = kv_at + slot * TILE_BYTES + (uint32_t)(lane * page_size * 128);
                if (!together) {
                    tma_load_4d(dst, map, 0, 0, it.kv_head, page, bar(B_KV_FULL + slot));
                    tma_load_4d(dst + HALF_BYTES, map, 64, 0, it.kv_head, page, bar(B_KV_FULL + slot));
                } else if ((lane & (run - 1)) == 0) {
                    tma_load_4d(dst, map_run, 0, 0, it.kv_head, page, bar(B_KV_FULL + slot));
                    tma_load_4d(dst + HALF_BYTES, map_run, 64, 0, it.kv_head, page, bar(B_KV_FULL + slot));
                }
            }
            ++ring;
            return true;
        };
        pdl_wait();                             // q, keys and values come from the kernel before this one
        if constexpr (PAIRED) {
            // the tiles of an item in the order K0, V0, K1, V1, ...
            for (int round = 0; alive; ++round) {
                Item it;
                if (!item_of(round, it)) break;
                int page = page_of(it, it.block0);
                if (!lane_wait(B_Q_EMPTY, (done_items & 1u) ^ 1u, 2)) break;
                if (lane == 0) {
                    mbar_arrive_expect(bar(B_Q_FULL), 2 * TILE_BYTES);
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        tma_load_2d(q_at + b * TILE_BYTES, &map_q, (it.head + b) * HD, it.first, bar(B_Q_FULL));
                        tma_load_2d(q_at + b * TILE_BYTES + HALF_BYTES, &map_q, (it.head + b) * HD + 64, it.first, bar(B_Q_FULL));
                    }
                }
                for (int j = 0; j < it.blocks && alive; ++j) {
                    const int page_after = j + 1 < it.blocks ? page_of(it, it.block0 + j + 1) : -1;
                    alive = load_tile(&map_k, it, page);
                    if (alive) alive = load_tile(&map_v, it, page);
                    page = page_after;
                }
                ++done_items;
            }
        } else {
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
                alive = load_tile_runs(&map_k, &map_k_run, it, page_v);
                for (int j = 0; j < it.blocks && alive; ++j) {
                    const int page_after = j + 2 < it.blocks ? page_of(it, it.block0 + j + 2) : -1;
                    if (j + 1 < it.blocks) alive = load_tile_runs(&map_k, &map_k_run, it, page_k);
                    if (alive) alive = load_tile_runs(&map_v, &map_v_run, it, page_v);
                    page_v = page_k;
                    page_k = page_after;
                }
                ++done_items;
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 10) {
        // ---- products.  The tiles of an item with n blocks come through the ring in the order K0, K1,
        // V0, K2, V1, ..., V(n-1): K of block j is the item's tile 2 j - 1 (0 for j = 0), V of block j
        // its tile 2 j + 2 (2 n - 1 for the last).  Block j belongs to softmax group j & 1.
        if (PAIRED && lane == 0 && warp == 1) {
            // both groups' S = Q K^T of every block: K of block j is the item's tile 2 j
            constexpr uint32_t idesc_qk = instruction_descriptor_bf16(QT, KT, false);
            uint32_t ring_base = 0, used = 0, done_items = 0;
            bool alive = true;
            for (int round = 0; alive; ++round) {
                Item it;
                if (!item_of(round, it)) break;
                if (!mbar_wait(bar(B_Q_FULL), done_items & 1u, abort_flag, status, 8)) break;
                for (int j = 0; j < it.blocks && alive; ++j) {
                    const uint32_t n = used + j;                        // every group's n-th block
                    const uint32_t tile = ring_base + 2 * j;
                    const uint32_t slot = tile % RING, phase = (tile / RING) & 1u;
                    if (!mbar_wait(bar(B_KV_FULL + slot), phase, abort_flag, status, 3)) { alive = false; break; }
                    const uint32_t k_tile = kv_at + slot * TILE_BYTES;
#pragma unroll
                    for (uint32_t b = 0; b < 2; ++b) {
                        // S of the group is also where its P lies: the product that read P of the block
                        // before must have finished
                        if (n > 0 && !mbar_wait(bar(B_P_READ + b), (n - 1) & 1u, abort_flag, status, 4)) { alive = false; break; }
                        // The second group starts an item when the first has its first block's softmax
                        // behind it: from then on one group's softmax runs under the other's products
                        // (started together, both would do their softmax at the same time, on the same
                        // issue slots and special-function unit, and the tensor cores would wait for both).
                        if (b == 1 && j == 0 && !mbar_wait(bar(B_P_FULL), n & 1u, abort_flag, status, 9)) { alive = false; break; }
                        tc_fence_after_sync();
#pragma unroll
                        for (int kk = 0; kk < HD / 16; ++kk) {
                            const uint32_t half = (kk / 4) * HALF_BYTES, step = 2u * (kk % 4);
                            tc_mma(tmem_base + b * KT, tile_descriptor(q_at + b * TILE_BYTES + half) + step,
                                   tile_descriptor(k_tile + half) + step, idesc_qk, kk != 0);
                        }
                        tc_commit(bar(B_S_FULL + b));
                    }
                    if (alive) tc_commit(bar(B_KV_EMPTY + slot));
                }
                if (alive) tc_commit(bar(B_Q_EMPTY));
                ring_base += 2 * it.blocks;
                used += it.blocks;
                ++done_items;
            }
        } else if (PAIRED && lane == 0) {
            // both groups' O += P V of every block: V of block j is the item's tile 2 j + 1
            constexpr uint32_t idesc_pv = instruction_descriptor_bf16(QT, HD, true);
            uint32_t ring_base = 0, used = 0, done_items = 0;
            bool alive = true;
            for (int round = 0; alive; ++round) {
                Item it;
                if (!item_of(round, it)) break;
                for (int j = 0; j < it.blocks && alive; ++j) {
                    const uint32_t n = used + j;
                    const uint32_t tile = ring_base + 2 * j + 1;
                    const uint32_t slot = tile % RING, phase = (tile / RING) & 1u;
                    const bool first_of_item = j == 0, last_of_item = j + 1 == it.blocks;
                    if (!mbar_wait(bar(B_KV_FULL + slot), phase, abort_flag, status, 5)) { alive = false; break; }
                    const uint32_t v_tile = kv_at + slot * TILE_BYTES;
#pragma unroll
                    for (uint32_t b = 0; b < 2; ++b) {
                        if (!mbar_wait(bar(B_P_FULL + b), n & 1u, abort_flag, status, 6)) { alive = false; break; }
                        if (first_of_item && !mbar_wait(bar(B_O_FREE + b), (done_items & 1u) ^ 1u, abort_flag, status, 7)) {
                            alive = false;
                            break;
                        }
                        tc_fence_after_sync();
#pragma unroll
                        for (int kk = 0; kk < KT / 16; ++kk) {
                            tc_mma_a_in_tmem(tmem_base + 2 * KT + b * HD, tmem_base + b * KT + kk * 8,
                                             tile_descriptor_mn_major(v_tile + kk * 2048, HALF_BYTES), idesc_pv,
                                             !(first_of_item && kk == 0));
                        }
                        tc_commit(bar(B_P_READ + b));
                        if (last_of_item) tc_commit(bar(B_O_LAST + b));
                    }
                    if (alive) tc_commit(bar(B_KV_EMPTY + slot));
                }
                ring_base += 2 * it.blocks;
                used += it.blocks;
                ++done_items;
            }
        } else if (lane == 0 && warp == 1) {
            constexpr uint32_t idesc_qk = instruction_descriptor_bf16(QT, KT, false);
            uint32_t ring_base = 0, used_a = 0, used_b = 0, done_items = 0;
            bool alive = true;
            for (int round = 0; alive; ++round) {
                Item it;
                if (!item_of(round, it)) break;
                if (!mbar_wait(bar(B_Q_FULL), done_items & 1u, abort_flag, status, 8)) break;
                for (int j = 0; j < it.blocks; ++j) {
                    const uint32_t b = j & 1u;
                    const uint32_t n = (b ? used_b : used_a) + j / 2;      // the group's n-th block
                    const uint32_t tile = ring_base + (j == 0 ? 0 : 2 * j - 1);
                    const uint32_t slot = tile % SLOTS, phase = (tile / SLOTS) & 1u;
                    if (!mbar_wait(bar(B_KV_FULL + slot), phase, abort_flag, status, 3)) { alive = false; break; }
                    // S of the group is also where its P lies: the product that read P of the block before
                    // must have finished
                    if (n > 0 && !mbar_wait(bar(B_P_READ + b), (n - 1) & 1u, abort_flag, status, 4)) { alive = false; break; }
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
                }
                if (alive) tc_commit(bar(B_Q_EMPTY));
                ring_base += 2 * it.blocks;
                used_a += (it.blocks + 1) / 2;
                used_b += it.blocks / 2;
                ++done_items;
            }
        } else if (lane == 0) {
            constexpr uint32_t idesc_pv = instruction_descriptor_bf16(QT, HD, true);
            uint32_t ring_base = 0, used_a = 0, used_b = 0, done_items = 0;
            bool alive = true;
            for (int round = 0; alive; ++round) {
                Item it;
                if (!item_of(round, it)) break;
                for (int j = 0; j < it.blocks; ++j) {
                    const uint32_t b = j & 1u;
                    const uint32_t n = (b ? used_b : used_a) + j / 2;
                    const uint32_t tile = ring_base + (j + 1 < it.blocks ? 2 * j + 2 : 2 * it.blocks - 1);
                    const uint32_t slot = tile % SLOTS, phase = (tile / SLOTS) & 1u;
                    const bool first_of_item = j < 2, last_of_item = j + 2 >= it.blocks;
                    if (!mbar_wait(bar(B_KV_FULL + slot), phase, abort_flag, status, 5)) { alive = false; break; }
                    if (!mbar_wait(bar(B_P_FULL + b), n & 1u, abort_flag, status, 6)) { alive = false; break; }
                    if (first_of_item && !mbar_wait(bar(B_O_FREE + b), (done_items & 1u) ^ 1u, abort_flag, status, 7)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t v_tile = kv_at + slot * TILE_BYTES;
#pragma unroll
                    for (int kk = 0; kk < KT / 16; ++kk) {
                        // 16 keys: 8 columns of P (two bfloat16 a column, over S), two 1024-byte atoms of V
                        tc_mma_a_in_tmem(tmem_base + 2 * KT + b * HD, tmem_base + b * KT + kk * 8,
                                         tile_descriptor_mn_major(v_tile + kk * 2048, HALF_BYTES), idesc_pv,
                                         !(first_of_item && kk == 0));
                    }
                    tc_commit(bar(B_KV_EMPTY + slot));
                    tc_commit(bar(B_P_READ + b));
                    if (last_of_item) tc_commit(bar(B_O_LAST + b));
                }
                ring_base += 2 * it.blocks;
                used_a += (it.blocks + 1) / 2;
                used_b += it.blocks / 2;
                ++done_items;
            }
        }
        __syncwarp();
    } else {
        // ---- softmax rows: group 0 = warps 2..5 takes the even blocks of a tile, group 1 = warps 6..9
        // the odd ones; a warp's number modulo 4 names the 32 lanes of tensor memory it may read.
        const int quarter = warp & 3, group = (warp - 2) >> 2;
        pdl_wait();                             // before this kernel's first write to global memory
        const int row = quarter * 32 + lane;
        const uint32_t lane_address = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t s_address = lane_address + group * KT;
        const uint32_t o_address = lane_address + 2 * KT + group * HD;
        // every lane waits (with the limit); the warp goes on only if all of them saw the phase
        auto warp_wait = [&](int barrier, uint32_t parity, int code) -> bool {
            const bool seen = mbar_wait(bar(barrier), parity, abort_flag, status, code);
            return __all_sync(0xffffffffu, seen);
        };
        auto warp_arrive = [&](int barrier) {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(barrier));
        };
        uint32_t used = 0;                    // blocks this group has taken so far
        uint32_t finals = 0;                  // tiles in which this group had blocks
        uint32_t done_items = 0;
        bool alive = true;
        for (int round = 0; alive; ++round) {
            Item it;
            if (!item_of(round, it)) break;
            const int q_pos = it.p0 + row;
            const int lowest = window > 0 ? q_pos - window + 1 : 0;      // first key this row sees
            float reference = -INFINITY;      // what the exponentials of this row subtract (in log2 units)
            float l = 0.0f;                   // the denominator of this group's blocks
            for (int j = PAIRED ? 0 : group; j < it.blocks && alive; j += PAIRED ? 1 : 2, ++used) {
                const uint32_t parity = used & 1u;
                const int key0 = (it.block0 + j) * KT;
                const bool has_previous = j >= (PAIRED ? 1 : 2);
                if (!warp_wait(B_S_FULL + group, parity, 10)) { alive = false; break; }
                tc_fence_after_sync();
                // below every row's diagonal and inside every row's window: no mask
                const bool full = key0 + KT - 1 <= it.p0 && (window <= 0 || key0 >= it.p0 + QT - 1 - window + 1);
                // ---- first pass over S: the block's maximum of this row
                float part[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < KT; c += 64) {
                    uint32_t v[64];
                    tmem_load_32(s_address + c, v);
                    tmem_load_32(s_address + c + 32, v + 32);
                    tmem_load_wait();
                    if (full) {
#pragma unroll
                        for (int e = 0; e < 64; ++e) part[e & 3] = fmaxf(part[e & 3], __uint_as_float(v[e]));
                    } else {
#pragma unroll
                        for (int e = 0; e < 64; ++e) {
                            const int key = key0 + c + e;
                            part[e & 3] = fmaxf(part[e & 3], key > q_pos || key < lowest ? -INFINITY : __uint_as_float(v[e]));
                        }
                    }
                }
                // scale > 0: the maximum of the scaled scores is the scaled maximum
                const float block_max = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])) * scale_log2;
                // the reference moves when the maximum has outgrown it by more than 2^RESCALE_STEP
                const bool moves = block_max > reference + RESCALE_STEP || (reference == -INFINITY && block_max > -INFINITY);
                float factor = 1.0f;
                if (moves) {
                    factor = exp2_fast(reference - block_max);       // 0 for a row that had seen no key
                    reference = block_max;
                    l *= factor;
                }
                // S of this block is there, so every product issued before it has finished, the one into this
                // group's O among them: O may be scaled.
                if (has_previous && __any_sync(0xffffffffu, moves)) {
#pragma unroll
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t o[32];
                        tmem_load_32(o_address + c, o);
                        tmem_load_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * factor);
                        tmem_store_32(o_address + c, o);
                    }
                }
                // ---- second pass: exponentials; P (two bfloat16 a column) over the columns of S just read
                // a row that has seen no key yet subtracts 0 so that no inf - inf appears
                const float subtract = reference == -INFINITY ? 0.0f : reference;
                float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int c = 0; c < KT; c += 64) {
                    uint32_t v[64];
                    tmem_load_32(s_address + c, v);
                    tmem_load_32(s_address + c + 32, v + 32);
                    tmem_load_wait();
                    uint32_t packed[32];
                    if (full) {
#pragma unroll
                        for (int e = 0; e < 64; e += 2) {
                            const float p0 = exp2_fast(fmaf(__uint_as_float(v[e]), scale_log2, -subtract));
                            const float p1 = exp2_fast(fmaf(__uint_as_float(v[e + 1]), scale_log2, -subtract));
                            sums[e & 3] += p0;
                            sums[(e & 3) + 1] += p1;
                            packed[e / 2] = pack_bf16x2(p0, p1);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 64; e += 2) {
                            const int key = key0 + c + e;
                            const float p0 = key > q_pos || key < lowest
                                                 ? 0.0f : exp2_fast(fmaf(__uint_as_float(v[e]), scale_log2, -subtract));
                            const float p1 = key + 1 > q_pos || key + 1 < lowest
                                                 ? 0.0f : exp2_fast(fmaf(__uint_as_float(v[e + 1]), scale_log2, -subtract));
                            sums[e & 3] += p0;
                            sums[(e & 3) + 1] += p1;
                            packed[e / 2] = pack_bf16x2(p0, p1);
                        }
                    }
                    tmem_store_32(s_address + c / 2, packed);
                }
                l += (sums[0] + sums[1]) + (sums[2] + sums[3]);
                tmem_store_wait();
                tc_fence_before_sync();
                warp_arrive(B_P_FULL + group);
            }
            if (!alive) break;
            if constexpr (PAIRED) {
                // ---- the group's own head: O over its denominator, when the last product into O has finished
                if (!warp_wait(B_O_LAST + group, finals & 1u, 13)) break;
                ++finals;
                const float inverse = l > 0.0f ? 1.0f / l : 0.0f;
                tc_fence_after_sync();
                bf16* out_row = out + (int64_t)(it.first + row) * out_stride + (it.head + group) * HD;
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    uint32_t a[32];
                    tmem_load_32(o_address + c, a);
                    tmem_load_wait();
                    if (c + 32 == HD) {
                        tc_fence_before_sync();
                        warp_arrive(B_O_FREE + group);
                    }
                    if (row < it.count) {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            float f[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(a[e + i]) * inverse;
                            *reinterpret_cast<uint4*>(out_row + c + e) = pack_bf16x8(f);
                        }
                    }
                }
                ++done_items;
                continue;
            }
            const int own_blocks = (it.blocks - group + 1) / 2;
            // the last product into this group's O has finished
            if (own_blocks > 0) {
                if (!warp_wait(B_O_LAST + group, finals & 1u, 13)) break;
                ++finals;
            }
            if (group == 1) {
                // hand reference and denominator to the first group (which has taken those of the tile before)
                if (done_items > 0 && !warp_wait(B_FIRST_TOOK, (done_items - 1) & 1u, 16)) break;
                exchange[row * 2] = reference;
                exchange[row * 2 + 1] = l;
                warp_arrive(B_SECOND_DONE);
            } else {
                // ---- the tile's result: both accumulators on the larger reference, over both denominators
                if (!warp_wait(B_SECOND_DONE, done_items & 1u, 17)) break;
                const float other_reference = exchange[row * 2], other_l = exchange[row * 2 + 1];
                warp_arrive(B_FIRST_TOOK);
                const float top = fmaxf(reference, other_reference);
                const float mine = reference == -INFINITY ? 0.0f : exp2_fast(reference - top);
                const float theirs = other_reference == -INFINITY ? 0.0f : exp2_fast(other_reference - top);
                const float total = l * mine + other_l * theirs;
                const float inverse = total > 0.0f ? 1.0f / total : 0.0f;
                const float weight_a = mine * inverse, weight_b = theirs * inverse;
                const bool second_used = it.blocks > 1;            // else O of the second group holds nothing of this tile
                tc_fence_after_sync();
                bf16* out_row = out + (int64_t)(it.first + row) * out_stride + it.head * HD;
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    uint32_t a[32], b[32];
                    tmem_load_32(lane_address + 2 * KT + c, a);
                    if (second_used) tmem_load_32(lane_address + 2 * KT + HD + c, b);
                    tmem_load_wait();
                    if (c + 32 == HD) {
                        tc_fence_before_sync();
                        warp_arrive(B_O_FREE);
                        warp_arrive(B_O_FREE + 1);
                    }
                    if (row < it.count) {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            float f[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                f[i] = __uint_as_float(a[e + i]) * weight_a;
                                if (second_used) f[i] = fmaf(__uint_as_float(b[e + i]), weight_b, f[i]);
                            }
                            *reinterpret_cast<uint4*>(out_row + c + e) = pack_bf16x8(f);
                        }
                    }
                }
            }
            ++done_items;
        }
    }

    pdl_launch_dependents();
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
    int kv_heads, page_size, run;
    bool operator==(const MapKey& o) const {
        return p == o.p && pages == o.pages && kv_heads == o.kv_heads && page_size == o.page_size && run == o.run;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.p) ^ (size_t)(k.pages * 131 + k.kv_heads * 17 + k.page_size + k.run * 7919);
    }
};

// Map of a cache [pages, kv_heads, page_size, 128]: boxes of `run` pages of one kv head, 64 values wide.
bool cache_map(CUtensorMap* map, const void* cache, long long pages, int kv_heads, int page_size, int run) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> known;
    static std::mutex guard;
    std::lock_guard<std::mutex> lock(guard);
    const MapKey key{cache, pages, kv_heads, page_size, run};
    auto found = known.find(key);
    if (found != known.end()) {
        *map = found->second;
        return true;
    }
    const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)page_size, (cuuint64_t)kv_heads, (cuuint64_t)pages};
    const cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)page_size * HD * 2,
                                   (cuuint64_t)kv_heads * page_size * HD * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)page_size, 1, (cuuint32_t)run};
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
                                        int window, float scale, int pdl, void* stream) {
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
    // pages of fewer than 32 tokens come two or four to a copy where they lie together (one head an item)
    int run = 32 / page_size < 1 ? 1 : 32 / page_size;
    while (run > 1 && run > pages) run /= 2;
    CUtensorMap map_k_run, map_v_run;
    if (!cache_map(&map_k, key_cache, pages, num_kv, page_size, 1) ||
        !cache_map(&map_v, value_cache, pages, num_kv, page_size, 1) ||
        !cache_map(&map_k_run, key_cache, pages, num_kv, page_size, run) ||
        !cache_map(&map_v_run, value_cache, pages, num_kv, page_size, run))
        return (int)cudaErrorNotSupported;
    // Two q heads of a kv head per item where the heads pair up: every K and V tile then serves both
    // (one head an item is bound by the copies of K and V: 64 KB a block for 8.4 MFLOP).  With few
    // items (a prompt of 2,048 tokens of 16 heads: 128 pairs for 148 CTAs) single heads spread
    // better: 39.7 against 47.9 us; at 8,192 tokens pairs take 285 against 382 us.
    const bool paired = (num_q / num_kv) % 2 == 0 && (long long)num_tiles * (num_q / 2) * 2 >= 3ll * sms;
    auto kernel = paired ? attention_prefill_tc_kernel<true> : attention_prefill_tc_kernel<false>;
    static bool configured[2][64] = {{false}};
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64 && !configured[paired][device]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SHARED_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured[paired][device] = true;
    }
    const long long items = (long long)num_tiles * (paired ? num_q / 2 : num_q);
    const int ctas = (int)(items < sms ? items : sms);
    TvbLaunch launch(dim3(ctas), dim3(THREADS), SHARED_BYTES, (cudaStream_t)stream, pdl);
    cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, map_q, map_k, map_v, map_k_run, map_v_run, run, block_tables, table_stride,
                                       positions, tile_row, tile_first, tile_count, (bf16*)out,
                                       (int64_t)num_q * HD, num_tiles, num_q, num_kv, page_size, window,
                                       scale * 1.4426950408889634f);
    return (int)e;
}
