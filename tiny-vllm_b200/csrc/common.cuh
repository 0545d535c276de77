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

static inline int tvb_last_error() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
