// out[m, n] = x[m, k] . w[n, k]^T for bfloat16 operands with FEW rows of x (decode, up to 128) and
// a LARGE weight: the product is bound by reading w once from memory, and the kernel is a stream
// of w through the fifth-generation tensor cores.
//
// The roles of the operands are swapped: 128 rows of w are the m side of tcgen05.mma (the lanes
// of tensor memory), the rows of x (padded to 16, 32, 64 or 128) its n side, so that a tile of w
// fills the instruction whatever the batch.  w and x tiles arrive through tensor-map copies
// (cp.async.bulk.tensor, 128-byte swizzle) into a ring of stages that holds about 190 KB in
// flight per SM; one thread issues the copies, one the products, four warps read the
// accumulators.
//
// Work is cut evenly, not by tiles: the (tile of 128 rows of w, block of 64 values of k) pairs
// are numbered tile by tile and every CTA takes an equal, consecutive share of them ("stream-k"),
// so every SM reads the same number of bytes whatever n and k are.  A CTA whose share starts or
// ends inside a tile leaves its partial sums (float32) in a workspace; the CTA that arrives last
// at a tile (counters per tile, no waiting) adds the partial sums in the order of k and stores
// the result, so the sum does not depend on which CTA that was.
//
// Modes: bfloat16 result (optionally added to the residual stream: round(round(product) +
// stream)), float32 result (logits), and the packed feed-forward input w = [gate (n rows) |
// up (n rows)] with the result round(round(SiLU(gate)) * up) (tinyvllm/layers.py:274-285).
// Stands where the reference calls F.linear (tinyvllm/layers.py:84-85).
//
// Every wait on an mbarrier is bounded (tc5.cuh); a wait that gives up is reported by
// tvb_gemm_stream_status.  One launch at a time may use a workspace (launches of one stream do).
#include <mutex>
#include <unordered_map>

#include "tc5.cuh"

namespace {

constexpr int BW = 128;                 // rows of w of a tile = lanes of tensor memory
constexpr int BK = 64;                  // 64 bfloat16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;            // warp 0 copies, warp 1 issues, warps 2..5 read the accumulators
constexpr int EPILOGUE_WARPS = 4;
constexpr int STAGE_BUDGET = 196608;    // bytes of operand stages
constexpr int MAX_STAGES = 12;

enum { MODE_BF16 = 0, MODE_F32 = 1, MODE_SILU = 2 };
enum { GAVE_UP_EMPTY = 1, GAVE_UP_FULL = 2, GAVE_UP_ACC_EMPTY = 3, GAVE_UP_ACC_FULL = 4 };

__device__ int tvb_gemm_stream_status_word = 0;

template <int XN, int SETS> struct Shape {
    static constexpr int W_BYTES = BW * BK * 2;
    static constexpr int X_BYTES = XN * BK * 2;
    static constexpr int STAGE_BYTES = SETS * W_BYTES + X_BYTES;
    static constexpr int STAGES = STAGE_BUDGET / STAGE_BYTES < MAX_STAGES ? STAGE_BUDGET / STAGE_BYTES : MAX_STAGES;
    static constexpr int SET_COLS = XN < 32 ? 32 : XN;          // columns of tensor memory of one accumulator
    static constexpr int ACC_COLS = SETS * SET_COLS;            // gate and up side by side
    static constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;         // two of them: one is read while the other fills
    static constexpr int BARRIERS = 2 * STAGES + 4;
    static constexpr int SHARED_BYTES = STAGES * STAGE_BYTES + BARRIERS * 8 + 32 + 1024;
    static constexpr int SLOT_FLOATS = SETS * XN * BW;          // partial sums of a tile: [set][row of x][row of w]
};

// The share of CTA `c` of `ctas` in `units` consecutive units starts here.
__device__ __host__ __forceinline__ long long share_start(long long c, long long units, long long ctas) {
    return c * units / ctas;
}
// The CTA whose share holds unit u (shares are not empty: ctas <= units).
__device__ __forceinline__ int owner_of(long long u, long long units, long long ctas) {
    return (int)(((u + 1) * ctas + units - 1) / units - 1);
}

struct Segment {
    int tile, kb0, kb1;     // blocks [kb0, kb1) of k of this tile
    bool whole;             // the whole tile: stored directly
    int which;              // else: 0 if it is the first piece of the CTA's share, 1 if not (then it is the last)
};

// Walks the segments of this CTA's share: the piece of a tile at its start, then the piece of a tile
// at its end, then the whole tiles between them.  The pieces come first so that the sums other
// CTAs wait for are in the workspace early, and adding them up runs beside the stream of whole
// tiles and not after it.
struct Walk {
    long long u0, u1;
    int k_blocks, first_tile, count, index;
    __device__ Walk(long long units, int k_blocks_) : k_blocks(k_blocks_), index(0) {
        u0 = share_start(blockIdx.x, units, gridDim.x);
        u1 = share_start(blockIdx.x + 1, units, gridDim.x);
        first_tile = (int)(u0 / k_blocks);
        count = u1 > u0 ? (int)((u1 - 1) / k_blocks) - first_tile + 1 : 0;     // tiles the share touches
    }
    __device__ bool next(Segment& s) {
        if (index >= count) return false;
        const int j = index == 0 ? 0 : index == 1 ? count - 1 : index - 1;     // in the order of k: 0, 1, ..., count - 1
        ++index;
        s.tile = first_tile + j;
        const long long tile_start = (long long)s.tile * k_blocks;
        const long long from = j == 0 ? u0 : tile_start, to = u1 < tile_start + k_blocks ? u1 : tile_start + k_blocks;
        s.kb0 = (int)(from - tile_start);
        s.kb1 = (int)(to - tile_start);
        s.whole = s.kb0 == 0 && s.kb1 == k_blocks;
        s.which = j == 0 ? 0 : 1;
        return true;
    }
};

template <int XN, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, void* out,
                   int64_t ldo, int m, int n, int k, int up_offset, const bf16* add_stream, float* workspace,
                   int* counters) {
    constexpr int SETS = MODE == MODE_SILU ? 2 : 1;
    using S = Shape<XN, SETS>;
    constexpr int STAGES = S::STAGES;

    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (smem_address(raw_shared) + 1023u) & ~1023u;
    uint8_t* aligned = raw_shared + (base - smem_address(raw_shared));
    const uint32_t bars = base + STAGES * S::STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(aligned + STAGES * S::STAGE_BYTES + S::BARRIERS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    int* status = &tvb_gemm_stream_status_word;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = (n + BW - 1) / BW;
    const int k_blocks = (k + BK - 1) / BK;
    const long long units = (long long)tiles * k_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), EPILOGUE_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_x);
    }
    __syncthreads();                            // the barriers are there
    // The copy thread starts at once; tensor memory is allocated under its first copies and its
    // address goes to the five warps that use it through a barrier of their own.
    uint32_t tmem_base = 0;
    if (warp >= 1) {
        if (warp == 1) tmem_alloc(smem_address(tmem_base_slot), S::TMEM_COLS);
        tc_fence_before_sync();
        asm volatile("bar.sync 1, %0;\n" ::"n"(THREADS - 32) : "memory");
        tc_fence_after_sync();
        tmem_base = *tmem_base_slot;
    }

    if (warp == 0) {
        if (lane == 0) {
            // ---- copies: a stage = 128 rows of w (of gate and of up) and the rows of x for 64 values
            // of k.  x comes from the kernel before this one: under programmatic dependent launch the
            // first weights are asked for before the wait on that kernel.
            int stage = 0; uint32_t phase = 0;
            bool alive = true, waited = false;
            Walk walk(units, k_blocks);
            Segment seg;
            while (alive && walk.next(seg)) {
                const int n0 = seg.tile * BW;
                for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status, GAVE_UP_EMPTY)) { alive = false; break; }
                    const uint32_t w_at = base + stage * S::STAGE_BYTES, x_at = w_at + SETS * S::W_BYTES;
                    mbar_arrive_expect(full_bar(stage), S::STAGE_BYTES);
                    tma_load_2d(w_at, &map_w, kb * BK, n0, full_bar(stage));
                    if (SETS == 2) tma_load_2d(w_at + S::W_BYTES, &map_w, kb * BK, up_offset + n0, full_bar(stage));
                    if (!waited) { pdl_wait(); waited = true; }
                    tma_load_2d(x_at, &map_x, kb * BK, 0, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- products: D[128 rows of w, rows of x] += w tile . x tile^T, four per set and stage
            constexpr uint32_t idesc = instruction_descriptor_bf16(BW, XN, false);
            int stage = 0; uint32_t phase = 0;
            bool alive = true;
            int local = 0;
            Walk walk(units, k_blocks);
            Segment seg;
            while (alive && walk.next(seg)) {
                const int acc = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1u;
                ++local;
                if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag, status, GAVE_UP_ACC_EMPTY)) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * S::ACC_COLS);
                for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, status, GAVE_UP_FULL)) { alive = false; break; }
                    tc_fence_after_sync();
                    const uint32_t w_at = base + stage * S::STAGE_BYTES, x_at = w_at + SETS * S::W_BYTES;
                    const uint64_t x_desc = tile_descriptor(x_at);
#pragma unroll
                    for (int set = 0; set < SETS; ++set) {
                        const uint64_t w_desc = tile_descriptor(w_at + set * S::W_BYTES);
#pragma unroll
                        for (int kk = 0; kk < BK / UMMA_K; ++kk)
                            tc_mma(d_tmem + (uint32_t)(set * S::SET_COLS), w_desc + 2u * kk, x_desc + 2u * kk, idesc,
                                   (uint32_t)(kb != seg.kb0 || kk != 0));
                    }
                    tc_commit(empty_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (alive) tc_commit(acc_full_bar(acc));
            }
        }
        __syncwarp();
    } else {
        // ---- the accumulators: warp w reads the 32 lanes of tensor memory that its number modulo 4
        // names; thread = row of w (a column of the result)
        const int quarter = warp & 3;
        const int row_local = quarter * 32 + lane;
        int local = 0;
        pdl_wait();
        Walk walk(units, k_blocks);
        Segment seg;
        // The result for rows [c, c + 32) of x of this thread's row of w, from `v` (and `u` for up).
        auto store = [&](int n_index, int c, const float* v, const float* u) {
            if (n_index >= n) return;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int row = c + j;
                if (row >= m) continue;
                if (MODE == MODE_F32) {
                    reinterpret_cast<float*>(out)[(int64_t)row * ldo + n_index] = v[j];
                } else if (MODE == MODE_SILU) {
                    const float gate = v[j], up = u[j];
                    const float activated = round_to<bf16>(__fdividef(gate, 1.0f + __expf(-gate)));
                    reinterpret_cast<bf16*>(out)[(int64_t)row * ldo + n_index] = __float2bfloat16_rn(__fmul_rn(activated, up));
                } else {
                    float value = round_to<bf16>(v[j]);
                    if (add_stream) value = __fadd_rn(value, __bfloat162float(add_stream[(int64_t)row * n + n_index]));
                    reinterpret_cast<bf16*>(out)[(int64_t)row * ldo + n_index] = __float2bfloat16_rn(value);
                }
            }
        };
        while (walk.next(seg)) {
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1u;
            ++local;
            const int n_index = seg.tile * BW + row_local;
            // one lane waits with the limit and tells the others, so that the warp stays whole
            int ready = lane == 0 ? (int)mbar_wait(acc_full_bar(acc), acc_phase, abort_flag, status, GAVE_UP_ACC_FULL) : 1;
            ready = __shfl_sync(0xffffffffu, ready, 0);
            if (!ready) break;
            for (int tries = 0; tries < 1024 && !mbar_try(acc_full_bar(acc), acc_phase); ++tries) {}
            __syncwarp();
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * S::ACC_COLS);
            if (seg.whole) {
                for (int c = 0; c < XN && c < m; c += 32) {
                    uint32_t v[32], u[32];
                    tmem_load_32(taddr + (uint32_t)c, v);
                    if (SETS == 2) tmem_load_32(taddr + (uint32_t)(S::SET_COLS + c), u);
                    tmem_load_wait();
                    store(n_index, c, reinterpret_cast<const float*>(v), reinterpret_cast<const float*>(u));
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(acc));
                continue;
            }
            // ---- a piece of a tile.  Every warp works for its own 32 rows of w, with a counter per
            // tile and warp of the pieces whose sums are in the workspace: no warp waits for another.
            // If all the other pieces are there, this warp adds them to its own sums (still in
            // tensor memory) in the order of k and stores the result; else it leaves its sums in
            // the workspace ([set][row of x][row of w]) and counts itself, and if it was the last
            // to do so after all, it adds up as well.
            const long long tile_first = (long long)seg.tile * k_blocks;
            const int c_first = owner_of(tile_first, units, gridDim.x);
            const int others = owner_of(tile_first + k_blocks - 1, units, gridDim.x) - c_first;
            int* counter = counters + seg.tile * EPILOGUE_WARPS + quarter;
            int finish = 0;
            if (lane == 0) finish = *reinterpret_cast<volatile int*>(counter) == others;
            finish = __shfl_sync(0xffffffffu, finish, 0);
            const bool own_in_tensor_memory = finish != 0;
            if (!finish) {
                float* mine = workspace + (int64_t)(blockIdx.x * 2 + seg.which) * S::SLOT_FLOATS;
                for (int c = 0; c < XN && c < m; c += 32) {
#pragma unroll
                    for (int set = 0; set < SETS; ++set) {
                        uint32_t v[32];
                        tmem_load_32(taddr + (uint32_t)(set * S::SET_COLS + c), v);
                        tmem_load_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (c + j < m) mine[(set * XN + c + j) * BW + row_local] = __uint_as_float(v[j]);
                    }
                }
                // the accumulator may be filled again while the sums find their way
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(acc));
                __threadfence();
                __syncwarp();
                if (lane == 0) finish = atomicAdd(counter, 1) == others;
                finish = __shfl_sync(0xffffffffu, finish, 0);
            }
            if (finish) {
                if (lane == 0) *counter = 0;               // for the next launch
                __threadfence();
                const int me = (int)blockIdx.x, c_last = c_first + others;
                // the sums of piece `piece` for rows [c, c + 32) of x, added to v (and u)
                auto add_piece = [&](int piece, int c, float* v, float* u) {
                    const int which = share_start(piece, units, gridDim.x) >= tile_first ? 0 : 1;
                    const float* theirs = workspace + (int64_t)(piece * 2 + which) * S::SLOT_FLOATS;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        // every row of the chunk, also those past m (never stored): a condition on m here
                        // would put a branch around every load, and they would go one after the other
                        if (c + j < XN) {
                            v[j] += __ldcg(theirs + (c + j) * BW + row_local);
                            if (SETS == 2) u[j] += __ldcg(theirs + (XN + c + j) * BW + row_local);
                        }
                    }
                };
                for (int c = 0; c < XN && c < m; c += 32) {
                    float v[32], u[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = u[j] = 0.0f;
                    if (own_in_tensor_memory) {
                        uint32_t own[32], own_up[32];
                        tmem_load_32(taddr + (uint32_t)c, own);
                        if (SETS == 2) tmem_load_32(taddr + (uint32_t)(S::SET_COLS + c), own_up);
                        for (int piece = c_first; piece < me; ++piece) add_piece(piece, c, v, u);
                        tmem_load_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            v[j] += __uint_as_float(own[j]);
                            if (SETS == 2) u[j] += __uint_as_float(own_up[j]);
                        }
                        for (int piece = me + 1; piece <= c_last; ++piece) add_piece(piece, c, v, u);
                    } else {
                        for (int piece = c_first; piece <= c_last; ++piece) add_piece(piece, c, v, u);
                    }
                    store(n_index, c, v, u);
                }
            }
            if (own_in_tensor_memory) {
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(acc));
            }
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
        tmem_free(tmem_base, S::TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host side
// Map of a row-major bfloat16 matrix [rows, cols] with `ld` elements between rows; boxes of
// 64 columns x box_rows rows.
bool make_map(CUtensorMap* map, const void* p, long long rows, long long cols, long long ld, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    return tvb_make_map(map, p, 2, dims, strides, box);
}

template <int XN, int MODE>
int launch_stream(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, long long ldo, int m, int n, int k,
                  int up_offset, const void* add_stream, float* workspace, int* counters, int ctas, int pdl,
                  cudaStream_t stream) {
    constexpr int SETS = MODE == MODE_SILU ? 2 : 1;
    using S = Shape<XN, SETS>;
    auto kernel = gemm_stream_kernel<XN, MODE>;
    static bool configured[64] = {false};
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64 && !configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SHARED_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured[device] = true;
    }
    TvbLaunch launch(dim3(ctas), dim3(THREADS), S::SHARED_BYTES, stream, pdl);
    cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, map_w, map_x, out, (int64_t)ldo, m, n, k, up_offset,
                                       (const bf16*)add_stream, workspace, counters);
    return (int)e;
}

int padded_rows(int m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }

int ctas_for(int n, int k) {
    const int sms = tvb_sm_count();
    const long long units = (long long)((n + BW - 1) / BW) * ((k + BK - 1) / BK);
    // a share of fewer than four blocks of k is all set-up
    long long ctas = units / 4;
    if (ctas > sms) ctas = sms;
    return ctas < 1 ? 1 : (int)ctas;
}

}  // namespace

extern "C" int tvb_gemm_stream_max_rows() { return BW; }

// Floats of workspace and ints of counters (zeroed once by the caller, left zeroed by every
// launch) that a product of these sizes needs.
extern "C" long long tvb_gemm_stream_workspace_floats(int m, int n, int k, int mode) {
    const int sets = mode == MODE_SILU ? 2 : 1;
    return (long long)ctas_for(n, k) * 2 * sets * padded_rows(m) * BW;
}
extern "C" int tvb_gemm_stream_counters(int n) { return (n + BW - 1) / BW * EPILOGUE_WARPS; }

extern "C" int tvb_gemm_stream_supports(int m, int n, int k, long long ldx, long long ldw, long long ldo) {
    return m > 0 && m <= BW && n > 0 && k > 0 && k % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldo > 0;
}

// 0, or which wait gave up in some launch since the last call (1 stage to fill, 2 stage to read,
// 3 accumulator to fill, 4 accumulator to read); reading clears it.  Synchronises the device.
extern "C" int tvb_gemm_stream_status() {
    int value = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&value, tvb_gemm_stream_status_word, sizeof(int)) != cudaSuccess) return -1;
    if (value != 0) cudaMemcpyToSymbol(tvb_gemm_stream_status_word, &zero, sizeof(int));
    return value;
}

// mode 0: out[m, n] bfloat16 = x . w^T (w has n rows); add_stream (may be null, contiguous [m, n]
// bfloat16): out = round(round(product) + add_stream).  mode 1: out float32.  mode 2: w = [gate
// (n rows) | up (n rows)], out[m, n] = SiLU(gate) * up.  x and w are bfloat16 with 16-byte aligned
// rows, m <= 128.  workspace / counters: as tvb_gemm_stream_workspace_floats / _counters say;
// the counters are zero before the first launch and zero again after every launch.
extern "C" int tvb_gemm_stream(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo,
                               int m, int n, int k, int mode, const void* add_stream, float* workspace,
                               int* counters, int pdl, void* stream) {
    if (m <= 0 || n <= 0) return 0;
    if (!tvb_gemm_stream_supports(m, n, k, ldx, ldw, ldo) || mode < 0 || mode > 2 || ((uintptr_t)x & 15) ||
        ((uintptr_t)w & 15) || !workspace || !counters || (add_stream && mode != MODE_BF16))
        return TVB_BAD_ARGUMENT;
    if (tvb_sm_count() <= 0) return (int)cudaErrorInvalidDevice;
    const int xn = padded_rows(m);
    const int ctas = ctas_for(n, k);
    const long long w_rows = mode == MODE_SILU ? 2ll * n : n;

    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, x, m, k, ldx, xn)) return (int)cudaErrorNotSupported;
    {
        // weights keep their address: their maps are made once
        struct Key { const void* p; long long rows, ld; int k; };
        struct Hash { size_t operator()(const Key& q) const {
            return std::hash<const void*>()(q.p) ^ (size_t)(q.rows * 31 + q.ld * 17 + q.k * 7); } };
        struct Equal { bool operator()(const Key& a, const Key& b) const {
            return a.p == b.p && a.rows == b.rows && a.ld == b.ld && a.k == b.k; } };
        static std::unordered_map<Key, CUtensorMap, Hash, Equal> cache;
        static std::mutex guard;
        std::lock_guard<std::mutex> lock(guard);
        const Key key{w, w_rows, ldw, k};
        auto found = cache.find(key);
        if (found == cache.end()) {
            if (!make_map(&map_w, w, w_rows, k, ldw, BW)) return (int)cudaErrorNotSupported;
            if (cache.size() > 4096) cache.clear();
            cache.emplace(key, map_w);
        } else {
            map_w = found->second;
        }
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int up_offset = mode == MODE_SILU ? n : 0;
#define STREAM(XN, MODE) \
    launch_stream<XN, MODE>(map_w, map_x, out, ldo, m, n, k, up_offset, add_stream, workspace, counters, ctas, pdl, s)
#define BY_ROWS(MODE)                          \
    do {                                       \
        if (xn == 16) return STREAM(16, MODE); \
        if (xn == 32) return STREAM(32, MODE); \
        if (xn == 64) return STREAM(64, MODE); \
        return STREAM(128, MODE);              \
    } while (0)
    if (mode == MODE_BF16) BY_ROWS(MODE_BF16);
    if (mode == MODE_F32) BY_ROWS(MODE_F32);
    BY_ROWS(MODE_SILU);
}
