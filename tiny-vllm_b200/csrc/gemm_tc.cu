// out[m, n] = x[m, k] . w[n, k]^T for bfloat16 operands with many rows (prefill), on the
// fifth-generation tensor cores: tcgen05.mma with the accumulator in tensor memory, operand
// tiles brought into shared memory by the tensor-map copy engine (cp.async.bulk.tensor) in the
// 128-byte swizzle that the matrix descriptors name, a ring of mbarriers between the copy
// thread, the issuing thread and four epilogue warps, and two accumulators so that the
// epilogue of one tile runs under the products of the next.  One persistent CTA per SM walks
// the tiles.
//
// Modes: 0 stores bfloat16 [m, n]; 2 is the packed feed-forward input: w = [gate (n rows) |
// up (n rows)], a tile holds the same columns of both and the epilogue stores
// round(round(SiLU(gate)) * up), so the [m, 2n] intermediate never reaches memory.
//
// The reference calls a library (cuBLAS through torch.nn.functional.linear,
// tinyvllm/layers.py:84-85 and :274-285 for the activation) for these products.
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT_CYCLES the waiting thread records which
// wait gave up in tvb_gemm_tc_status, raises the CTA's abort flag, every role leaves its loop,
// the CTA waits a fixed time for copies still in flight, frees its tensor memory and returns.
#include <mutex>
#include <unordered_map>

#include "tc5.cuh"

namespace {

constexpr int BM = 128;                 // rows of a tile = lanes of tensor memory
constexpr int BK = 64;                  // 64 bfloat16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;              // k of one tcgen05.mma.kind::f16
constexpr int THREADS = 192;            // warp 0 copies, warp 1 issues, warps 2..5 epilogue
constexpr int EPILOGUE_WARPS = 4;
constexpr int STAGE_BUDGET = 196608;    // bytes of operand stages

enum { MODE_BF16 = 0, MODE_SILU = 2 };
enum { GAVE_UP_EMPTY = 1, GAVE_UP_FULL = 2, GAVE_UP_ACC_EMPTY = 3, GAVE_UP_ACC_FULL = 4 };

__device__ int tvb_gemm_tc_status_word = 0;

template <int BN> struct Tile {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = STAGE_BUDGET / STAGE_BYTES;
    static constexpr int BARRIERS = 2 * STAGES + 4;
    // stages (1024-aligned), barriers, tensor-memory base, abort flag; 1024 spare to align
    static constexpr int SHARED_BYTES = STAGES * STAGE_BYTES + BARRIERS * 8 + 16 + 1024;
};

template <int BN> __device__ __forceinline__ constexpr uint32_t instruction_descriptor() {
    return instruction_descriptor_bf16(BM, BN, false);
}

template <int BN, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               bf16* out, int64_t ldo, int m, int n, int k, int up_offset) {
    using T = Tile<BN>;
    constexpr int STAGES = T::STAGES;
    constexpr int OUT_COLS = MODE == MODE_SILU ? BN / 2 : BN;   // output columns of a tile
    constexpr uint32_t TMEM_COLS = 2 * BN;                     // two accumulators
    static_assert(BN == 128 || BN == 256, "tile widths 128 and 256");

    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (smem_address(raw_shared) + 1023u) & ~1023u;
    uint8_t* aligned = raw_shared + (base - smem_address(raw_shared));
    const uint32_t bars = base + STAGES * T::STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(aligned + STAGES * T::STAGE_BYTES + T::BARRIERS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (m + BM - 1) / BM, tiles_n = (n + OUT_COLS - 1) / OUT_COLS;
    const int tiles = tiles_m * tiles_n;
    const int k_blocks = (k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), EPILOGUE_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_w);
    }
    if (warp == 1) tmem_alloc(smem_address(tmem_base_slot), TMEM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;

    // x comes from the kernel before this one in the stream: under programmatic dependent
    // launch the copy thread waits for it after its first copy of weights, the epilogue warps
    // before their first store; set-up and the first weights overlap that kernel's end.

    if (warp == 0) {
        if (lane == 0) {
            // ---- copies: one stage = rows of x and rows of w for 64 values of k
            int stage = 0; uint32_t phase = 0;
            bool alive = true, waited = false;
            for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * OUT_COLS;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, &tvb_gemm_tc_status_word, GAVE_UP_EMPTY)) { alive = false; break; }
                    const uint32_t a_at = base + stage * T::STAGE_BYTES, b_at = a_at + T::A_BYTES;
                    mbar_arrive_expect(full_bar(stage), T::STAGE_BYTES);
                    tma_load_2d(b_at, &map_w, kb * BK, n0, full_bar(stage));
                    if (MODE == MODE_SILU)
                        tma_load_2d(b_at + T::B_BYTES / 2, &map_w, kb * BK, up_offset + n0, full_bar(stage));
                    if (!waited) { pdl_wait(); waited = true; }
                    tma_load_2d(a_at, &map_x, kb * BK, m0, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- products: four tcgen05.mma per stage, the stage is handed back when they finish
            constexpr uint32_t idesc = instruction_descriptor<BN>();
            int stage = 0; uint32_t phase = 0;
            bool alive = true;
            int local = 0;
            for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ++local) {
                const int acc = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1u;
                if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag, &tvb_gemm_tc_status_word, GAVE_UP_ACC_EMPTY)) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, &tvb_gemm_tc_status_word, GAVE_UP_FULL)) { alive = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_at = base + stage * T::STAGE_BYTES, b_at = a_at + T::A_BYTES;
                    const uint64_t a_desc = tile_descriptor(a_at), b_desc = tile_descriptor(b_at);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        // 16 values of k further: 32 bytes inside the swizzled row, 2 in address units
                        tc_mma(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc, (kb | kk) != 0);
                    }
                    tc_commit(empty_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (alive) tc_commit(acc_full_bar(acc));
            }
        }
        __syncwarp();
    } else {
        // ---- epilogue: warp w reads the 32 lanes of tensor memory that its number modulo 4 names
        const int quarter = warp & 3;
        int local = 0;
        pdl_wait();
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1u;
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * OUT_COLS;
            // one lane waits with the limit and tells the others, so that the warp stays whole
            int ready = lane == 0 ? (int)mbar_wait(acc_full_bar(acc), acc_phase, abort_flag, &tvb_gemm_tc_status_word, GAVE_UP_ACC_FULL) : 1;
            ready = __shfl_sync(0xffffffffu, ready, 0);
            if (!ready) break;
            for (int tries = 0; tries < 1024 && !mbar_try(acc_full_bar(acc), acc_phase); ++tries) {}
            __syncwarp();
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
            const int row = m0 + quarter * 32 + lane;
            bf16* out_row = out + (int64_t)row * ldo + n0;
            // the load of the next 32 columns is in flight while these are converted and stored
            uint32_t v[2][32], u[2][32];
            tmem_load_32(taddr, v[0]);
            if (MODE == MODE_SILU) tmem_load_32(taddr + (uint32_t)(BN / 2), u[0]);
#pragma unroll
            for (int c = 0; c < OUT_COLS; c += 32) {
                const int cur = (c / 32) & 1;
                tmem_load_wait();
                if (c + 32 < OUT_COLS) {
                    tmem_load_32(taddr + (uint32_t)(c + 32), v[cur ^ 1]);
                    if (MODE == MODE_SILU) tmem_load_32(taddr + (uint32_t)(BN / 2 + c + 32), u[cur ^ 1]);
                }
                float f[32];
                if (MODE == MODE_SILU) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float gate = __uint_as_float(v[cur][j]), up = __uint_as_float(u[cur][j]);
                        // 2^x and the quotient to within two units of the last place of float32,
                        // then rounded to bfloat16's eight bits
                        const float activated = round_to<bf16>(__fdividef(gate, 1.0f + __expf(-gate)));
                        f[j] = __fmul_rn(activated, up);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[cur][j]);
                }
                if (row < m) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (n0 + c + j < n)      // n is a multiple of 8: a group of 8 is inside or outside
                            *reinterpret_cast<uint4*>(out_row + c + j) = pack_bf16x8(f + j);
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(acc));
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

// ------------------------------------------------------------------ host side
// Map of a row-major bfloat16 matrix [rows, cols] with `ld` elements between rows; boxes of
// 64 columns x box_rows rows.
bool make_map(CUtensorMap* map, const void* p, long long rows, long long cols, long long ld, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    return tvb_make_map(map, p, 2, dims, strides, box);
}

int sm_count() { return tvb_sm_count(); }

template <int BN, int MODE>
int launch_tc(const CUtensorMap& map_x, const CUtensorMap& map_w, void* out, long long ldo, int m, int n, int k,
              int up_offset, int ctas, int pdl, cudaStream_t stream) {
    auto kernel = gemm_tc_kernel<BN, MODE>;
    static bool configured[64] = {false};
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64 && !configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Tile<BN>::SHARED_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured[device] = true;
    }
    TvbLaunch launch(dim3(ctas), dim3(THREADS), Tile<BN>::SHARED_BYTES, stream, pdl);
    cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, map_x, map_w, (bf16*)out, (int64_t)ldo, m, n, k,
                                       up_offset);
    return (int)e;
}

}  // namespace

// Whether tvb_gemm_tc takes a product of these sizes (the caller uses another kernel if not).
extern "C" int tvb_gemm_tc_supports(int m, int n, int k, long long ldx, long long ldw, long long ldo) {
    return m > 0 && n > 0 && k > 0 && k % 8 == 0 && n % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldo % 8 == 0;
}

// 0, or which wait gave up in some launch since the last call (1 stage to fill, 2 stage to read,
// 3 accumulator to fill, 4 accumulator to read); reading clears it.  Synchronises the device.
extern "C" int tvb_gemm_tc_status() {
    int value = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&value, tvb_gemm_tc_status_word, sizeof(int)) != cudaSuccess) return -1;
    if (value != 0) cudaMemcpyToSymbol(tvb_gemm_tc_status_word, &zero, sizeof(int));
    return value;
}

// mode 0: out[m, n] = x . w^T (w has n rows).  mode 2: w = [gate (n rows) | up (n rows)],
// out[m, n] = SiLU(gate) * up.  x, w, out are bfloat16 with 16-byte aligned rows.
// tile_n: 0 lets the launcher choose, 128 or 256 forces the width of a tile.
extern "C" int tvb_gemm_tc(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo,
                           int m, int n, int k, int mode, int tile_n, int pdl, void* stream) {
    if (m <= 0 || n <= 0) return 0;
    if (!tvb_gemm_tc_supports(m, n, k, ldx, ldw, ldo) || (mode != MODE_BF16 && mode != MODE_SILU) ||
        ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15))
        return TVB_BAD_ARGUMENT;
    const int sms = sm_count();
    if (sms <= 0) return (int)cudaErrorInvalidDevice;
    const int tiles_m = (m + BM - 1) / BM;
    const int out_cols_256 = mode == MODE_SILU ? 128 : 256;
    int bn = tile_n;
    if (bn == 0) bn = tiles_m * ((n + out_cols_256 - 1) / out_cols_256) >= sms ? 256 : 128;
    if (bn != 128 && bn != 256) return TVB_BAD_ARGUMENT;
    const int out_cols = mode == MODE_SILU ? bn / 2 : bn;
    const int tiles = tiles_m * ((n + out_cols - 1) / out_cols);
    const int ctas = tiles < sms ? tiles : sms;
    const long long w_rows = mode == MODE_SILU ? 2ll * n : n;

    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, x, m, k, ldx, BM)) return (int)cudaErrorNotSupported;
    {
        // weights keep their address: their maps are made once
        struct Key { const void* p; long long rows, ld; int k, box; };
        struct Hash { size_t operator()(const Key& q) const {
            return std::hash<const void*>()(q.p) ^ (size_t)(q.rows * 31 + q.ld * 17 + q.k * 7 + q.box); } };
        struct Equal { bool operator()(const Key& a, const Key& b) const {
            return a.p == b.p && a.rows == b.rows && a.ld == b.ld && a.k == b.k && a.box == b.box; } };
        static std::unordered_map<Key, CUtensorMap, Hash, Equal> cache;
        static std::mutex guard;
        std::lock_guard<std::mutex> lock(guard);
        const Key key{w, w_rows, ldw, k, out_cols};
        auto found = cache.find(key);
        if (found == cache.end()) {
            if (!make_map(&map_w, w, w_rows, k, ldw, out_cols)) return (int)cudaErrorNotSupported;
            if (cache.size() > 4096) cache.clear();
            cache.emplace(key, map_w);
        } else {
            map_w = found->second;
        }
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int up_offset = mode == MODE_SILU ? n : 0;
    if (bn == 256) {
        if (mode == MODE_SILU) return launch_tc<256, MODE_SILU>(map_x, map_w, out, ldo, m, n, k, up_offset, ctas, pdl, s);
        return launch_tc<256, MODE_BF16>(map_x, map_w, out, ldo, m, n, k, up_offset, ctas, pdl, s);
    }
    if (mode == MODE_SILU) return launch_tc<128, MODE_SILU>(map_x, map_w, out, ldo, m, n, k, up_offset, ctas, pdl, s);
    return launch_tc<128, MODE_BF16>(map_x, map_w, out, ldo, m, n, k, up_offset, ctas, pdl, s);
}
