// Shared helpers of the sm_100a kernels: storage types, rounding, reductions.
//
// Every launcher is an extern "C" function that takes raw device pointers, sizes,
// a storage-type tag and a CUDA stream, and returns 0, a cudaError_t (> 0) or
// TVB_BAD_ARGUMENT (< 0) for sizes it refuses.  All arithmetic is float32; the
// storage type only decides what is loaded, stored and rounded in between.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TVB_F32 0
#define TVB_BF16 1
#define TVB_BAD_ARGUMENT (-1)

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

// Round to the storage type and come back: the value a later kernel would load.
template <typename T> __device__ __forceinline__ float round_to(float v) {
    return to_float<T>(from_float<T>(v));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int delta = 16; delta > 0; delta >>= 1) v += __shfl_xor_sync(0xffffffffu, v, delta);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int delta = 16; delta > 0; delta >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, delta));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch`
// holds 32 floats.  The order of additions depends on the block size only.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = lane < warps ? scratch[lane] : 0.0f;
    return warp_sum(total);
}

// ---- asynchronous 16-byte copies from global to shared memory
__device__ __forceinline__ uint32_t smem_address(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
// With valid == false nothing is read and the 16 destination bytes become zero.
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_address(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// ---- eight bfloat16 in one 16-byte word
__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint4 pack_bf16x8(const float* f) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                      pack_bf16x2(f[6], f[7]));
}

// ---- the cluster's barrier in two halves: arrive early, wait where the others are needed
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
// The same without ordering any memory access: for "this CTA runs", said at a kernel's start, where
// nothing has been written that another CTA will read (a release would make the warp wait for its
// loads in flight).
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }

// ---- programmatic dependent launch: a kernel launched with the attribute may start while the
// kernel before it in the stream still runs.  It must call pdl_wait() before it reads what that
// kernel wrote and before its own first write to global memory; pdl_launch_dependents() lets
// the kernel after it start.  Without the attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

// A kernel that runs under programmatic dependent launch must not read what its predecessor
// writes through pointers the compiler may treat as read-only for the kernel's whole life
// (const __restrict__ turns loads into ld.global.nc, which may be hoisted above the wait or be
// served from a stale read-only cache).  Such inputs are plain pointers, read with these.
__device__ __forceinline__ float bf16_bits_to_float(unsigned short bits) {
    return __uint_as_float((uint32_t)bits << 16);
}
__device__ __forceinline__ float ld_global_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];\n" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned short ld_global_u16(const void* p) {
    unsigned short v;
    asm volatile("ld.global.cg.u16 %0, [%1];\n" : "=h"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_global_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Ask for the 128-byte line at p to be brought into L2; nothing waits for it.
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p)); }

// Every thread of the grid takes its share of the lines of [p, p + bytes).
__device__ __forceinline__ void prefetch_l2_range(const void* p, long long bytes) {
    if (!p || bytes <= 0) return;
    const long long threads = (long long)gridDim.x * gridDim.y * gridDim.z * blockDim.x;
    const long long me = ((long long)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;
    for (long long line = me; line * 128 < bytes; line += threads)
        prefetch_l2(reinterpret_cast<const char*>(p) + line * 128);
}

// Launch configuration with the optional attributes: cluster size along x, programmatic
// stream serialisation.
struct TvbLaunch {
    cudaLaunchConfig_t config;
    cudaLaunchAttribute attributes[2];
    TvbLaunch(dim3 grid, dim3 block, size_t shared, cudaStream_t stream, int pdl, int cluster_x = 0) {
        config = cudaLaunchConfig_t{};
        config.gridDim = grid;
        config.blockDim = block;
        config.dynamicSmemBytes = shared;
        config.stream = stream;
        int count = 0;
        if (cluster_x > 0) {
            attributes[count].id = cudaLaunchAttributeClusterDimension;
            attributes[count].val.clusterDim.x = cluster_x;
            attributes[count].val.clusterDim.y = 1;
            attributes[count].val.clusterDim.z = 1;
            ++count;
        }
        if (pdl) {
            attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attributes[count].val.programmaticStreamSerializationAllowed = 1;
            ++count;
        }
        config.attrs = attributes;
        config.numAttrs = count;
    }
};

static inline int tvb_last_error() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
