// Building blocks of the tcgen05 kernels: mbarriers with bounded waits, tensor-map copies,
// tensor-memory allocation, tcgen05.mma / commit / ld, shared-memory matrix descriptors.
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT_CYCLES the waiting thread stores which
// wait gave up in *status_word (if it still holds 0), raises the CTA's abort flag and returns
// false; every other wait of the CTA then returns false as well.
#pragma once

#include <cuda.h>

#include "common.cuh"

constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;   // about a second of SM clock

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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status_word,
                                          int code) {
    if (mbar_try(bar, parity)) return true;
    const long long started = clock64();
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_try(bar, parity)) return true;
        if ((spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - started > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                atomicCAS(status_word, 0, code);
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
// The same with the a operand in tensor memory: lane = row, one 32-bit column = two consecutive
// bfloat16 of k (16 values of k = 8 columns from `a_tmem` on).
__device__ __forceinline__ void tc_mma_a_in_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
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
// 32 lanes x 32 consecutive 32-bit columns from registers into tensor memory.
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
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }


// Four-dimensional box (the paged cache: head size, page, kv head, page number).
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}
// Writes of this thread to shared memory become visible to the copy engine and the tensor cores.
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// Shared-memory matrix descriptor of a k-major tile whose rows are 128 bytes, stored in the
// 128-byte swizzle: groups of 8 rows lie 1024 bytes apart (stride offset), the leading offset
// is not used by this layout, descriptor version 1, layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t tile_descriptor(uint32_t shared_address) {
    return (uint64_t)((shared_address >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// The same for an operand whose rows along m/n are contiguous (the values of a key: 64 head
// dimensions = 128 bytes per key, 8 keys = one 1024-byte swizzle atom): atoms along k (groups of 8
// keys) lie 1024 bytes apart (stride offset), atoms along m/n (the next 64 dimensions)
// `leading_bytes` apart.
__device__ __forceinline__ uint64_t tile_descriptor_mn_major(uint32_t shared_address, uint32_t leading_bytes) {
    return (uint64_t)((shared_address >> 4) & 0x3fffu) | ((uint64_t)((leading_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: float32 accumulator (1 at bit 4), bfloat16 a and b (1 at
// bits 7 and 10), a k-major (bit 15 zero), b k-major or m/n-major (bit 16), n / 8 at bit 17,
// m / 16 at bit 24.
__device__ __forceinline__ constexpr uint32_t instruction_descriptor_bf16(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// ---- host side: tensor maps through the driver entry point (no link against the driver library)
typedef CUresult (*TvbEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline TvbEncodeTiled tvb_encode_tiled() {
    static TvbEncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &result) !=
                cudaSuccess || result != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<TvbEncodeTiled>(p);
    }();
    return fn;
}

// Map of a bfloat16 tensor of `rank` dimensions (innermost first), `strides` in bytes for the
// dimensions after the first, boxes of `box` elements, 128-byte swizzle, zeros outside the tensor.
static inline bool tvb_make_map(CUtensorMap* map, const void* p, int rank, const cuuint64_t* dims,
                                const cuuint64_t* strides, const cuuint32_t* box) {
    TvbEncodeTiled encode = tvb_encode_tiled();
    if (!encode) return false;
    const cuuint32_t element_strides[5] = {1, 1, 1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(p), dims, strides, box,
                  element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static inline int tvb_sm_count() {
    static int counts[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
    if (counts[device] == 0) cudaDeviceGetAttribute(&counts[device], cudaDevAttrMultiProcessorCount, device);
    return counts[device];
}
