// A one-CTA kernel that waits, with the bounded wait of tc5.cuh, on an mbarrier that nothing
// arrives on: the way to see, without a fault and without a hang, that a wait of the tcgen05
// kernels which is never satisfied ends by itself, records its code and lets the kernel return
// with the context intact.  The reference has no counterpart (its kernels have no such waits).
#include "tc5.cuh"

namespace {

__device__ int tvb_wait_probe_status_word = 0;

__global__ void wait_probe_kernel(int code, int* gave_up_after_ms) {
    __shared__ __align__(8) unsigned long long barrier;
    __shared__ int abort_flag;
    const uint32_t bar = smem_address(&barrier);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const long long started = clock64();
        const bool completed = mbar_wait(bar, 0, &abort_flag, &tvb_wait_probe_status_word, code);
        // SM clock in kHz is not known here: report cycles / 1e6 (about half a millisecond each)
        *gave_up_after_ms = completed ? -1 : (int)((clock64() - started) / 1000000);
    }
    __syncthreads();
    // every other thread of the CTA sees the flag and would leave its loop
    if (threadIdx.x == 32 && abort_flag != 1) *gave_up_after_ms = -2;
}

}  // namespace

// Launches the probe, waits for it, returns the status word it left (and clears it); `cycles_e6`
// receives how long the wait lasted in millions of SM cycles (-1: the barrier completed, which
// cannot be; -2: the abort flag was not seen).  Takes about a second.
extern "C" int tvb_wait_probe(int code, int* cycles_e6, void* stream) {
    int* device_value = nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    if (cudaMallocAsync(&device_value, sizeof(int), s) != cudaSuccess) return -1;
    wait_probe_kernel<<<1, 64, 0, s>>>(code, device_value);
    int status = 0, zero = 0;
    cudaError_t e = cudaMemcpyAsync(cycles_e6, device_value, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFreeAsync(device_value, s);
    if (e != cudaSuccess) return -(int)e - 100;
    if (cudaMemcpyFromSymbol(&status, tvb_wait_probe_status_word, sizeof(int)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(tvb_wait_probe_status_word, &zero, sizeof(int));
    return status;
}
