// C[M,N] = A[M,K] . W[N,K]^T on the float32 cores: the matrix product of the true
// 32-bit path (no tensor cores, no reduced-precision mode), for any M, N, K.
//
// Each output element is the sum over k = 0..K-1 in ascending order, one fused
// multiply-add per k, whatever M is: a row's result does not depend on which
// other rows are in the batch.  Stands where the reference calls F.linear
// (tinyvllm/layers.py:84-85).
#include "common.cuh"

#define TILE_M 64
#define TILE_N 64
#define TILE_K 16

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_nt_simt_kernel(const TI* __restrict__ a, int64_t lda, const TI* __restrict__ w, int64_t ldw,
                    TO* __restrict__ c, int64_t ldc, int m, int n, int k) {
    __shared__ float a_tile[TILE_K][TILE_M + 4];
    __shared__ float w_tile[TILE_K][TILE_N + 4];
    const int tid = threadIdx.x;
    const int row0 = blockIdx.y * TILE_M, col0 = blockIdx.x * TILE_N;
    const int ty = tid / 16, tx = tid % 16;           // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    const int load_row = tid / 4;                      // 64 rows, 4 threads per row
    const int load_k = (tid % 4) * 4;                  // 4 consecutive k per thread
    for (int k0 = 0; k0 < k; k0 += TILE_K) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = k0 + load_k + i;
            const int ar = row0 + load_row, wr = col0 + load_row;
            a_tile[load_k + i][load_row] = (ar < m && kk < k) ? to_float<TI>(a[(int64_t)ar * lda + kk]) : 0.0f;
            w_tile[load_k + i][load_row] = (wr < n && kk < k) ? to_float<TI>(w[(int64_t)wr * ldw + kk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TILE_K; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = a_tile[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = w_tile[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = col0 + tx * 4 + j;
            if (col < n) c[(int64_t)r * ldc + col] = from_float<TO>(acc[i][j]);
        }
    }
}

// in_dtype: type of A and W; out_dtype: type of C (float32 output from bfloat16
// inputs serves the logits).
extern "C" int tvb_gemm_nt_simt(const void* a, long long lda, const void* w, long long ldw, void* c,
                                long long ldc, int m, int n, int k, int in_dtype, int out_dtype,
                                void* stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0) return TVB_BAD_ARGUMENT;
    dim3 grid((n + TILE_N - 1) / TILE_N, (m + TILE_M - 1) / TILE_M);
    if (grid.y > 65535) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == TVB_F32 && out_dtype == TVB_F32)
        gemm_nt_simt_kernel<float, float><<<grid, 256, 0, s>>>((const float*)a, lda, (const float*)w, ldw,
                                                               (float*)c, ldc, m, n, k);
    else if (in_dtype == TVB_BF16 && out_dtype == TVB_BF16)
        gemm_nt_simt_kernel<bf16, bf16><<<grid, 256, 0, s>>>((const bf16*)a, lda, (const bf16*)w, ldw,
                                                             (bf16*)c, ldc, m, n, k);
    else if (in_dtype == TVB_BF16 && out_dtype == TVB_F32)
        gemm_nt_simt_kernel<bf16, float><<<grid, 256, 0, s>>>((const bf16*)a, lda, (const bf16*)w, ldw,
                                                              (float*)c, ldc, m, n, k);
    else
        return TVB_BAD_ARGUMENT;
    return tvb_last_error();
}
