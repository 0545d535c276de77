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
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

constexpr int BM = 128;                 // rows of a tile = lanes of tensor memory
constexpr int BK = 64;                  // 64 bfloat16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;              // k of one tcgen05.mma.kind::f16
constexpr int THREADS = 192;            // warp 0 copies, warp 1 issues, warps 2..5 epilogue
constexpr int EPILOGUE_WARPS = 4;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;   // about a second of SM clock
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

// ---- mbarriers
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
// True when the phase completed; false when the CTA gives up (this wait ran out or another did).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_try(bar, parity)) return true;
    const long long started = clock64();
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_try(bar, parity)) return true;
        if ((spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - started > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                atomicCAS(&tvb_gemm_tc_status_word, 0, code);
                return false;
            }
        }
    }
}

// ---- tensor-map copies: box {BK columns, rows} at (column x, row y) into shared memory
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory and tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t result_in_shared, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(result_in_shared), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// All tcgen05.mma issued so far by this thread arrive on `bar` when they have finished.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] . B[smem]^T, 128 x N x 16, bfloat16 in, float32 out.
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 32 consecutive float32 columns: thread i of the warp gets lane (base lane + i).
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor of a k-major tile whose rows are 128 bytes, stored in the
// 128-byte swizzle: groups of 8 rows lie 1024 bytes apart (stride offset), the leading offset
// is not used by this layout, descriptor version 1, layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t tile_descriptor(uint32_t shared_address) {
    return (uint64_t)((shared_address >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: float32 accumulator (1 at bit 4), bfloat16 a and b (1 at bits 7 and
// 10), both k-major (bits 15, 16 zero), n / 8 at bit 17, m / 16 at bit 24.
template <int BN> __device__ __forceinline__ constexpr uint32_t instruction_descriptor() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
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
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, GAVE_UP_EMPTY)) { alive = false; break; }
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
                if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag, GAVE_UP_ACC_EMPTY)) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, GAVE_UP_FULL)) { alive = false; break; }
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
            int ready = lane == 0 ? (int)mbar_wait(acc_full_bar(acc), acc_phase, abort_flag, GAVE_UP_ACC_FULL) : 1;
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
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &result) !=
                cudaSuccess || result != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

// Map of a row-major bfloat16 matrix [rows, cols] with `ld` elements between rows; boxes of
// 64 columns x box_rows rows, 128-byte swizzle, zeros outside the matrix.
bool make_map(CUtensorMap* map, const void* p, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p), dims, strides, box,
                  element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
    static int counts[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
    if (counts[device] == 0) cudaDeviceGetAttribute(&counts[device], cudaDevAttrMultiProcessorCount, device);
    return counts[device];
}

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
