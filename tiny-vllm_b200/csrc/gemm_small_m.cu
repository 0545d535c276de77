// out[M,N] = x[M,K] . W[N,K]^T for a handful of rows (decode): a weight-streaming
// kernel.  With M <= 32 every weight is used once, so the product is bound by reading
// W from HBM; the kernel is built around that read, not around the arithmetic.
//
// The transposed product C^T[n, m] = W[n, :] . x[m, :] goes through mma.sync
// m16n8k16 (bfloat16 in, float32 accumulate): 16 rows of W are the A operand, 8 rows of x
// the B operand, so a batch of up to 8 fills one instruction exactly and nothing of W is
// staged in shared memory.  A thread loads 16 bytes (8 consecutive k) of two W rows and of
// one x row per 32-wide k block; which k a fragment slot stands for is permuted the same way
// in both operands, which a dot product does not notice, so the 16-byte loads feed two
// instructions without any shuffle.
//
// Work is cut as (N / 16 row tiles) x (k blocks dealt round-robin to the 4 warps of the KS CTAs
// of a thread-block cluster).  Warps, then CTAs (through distributed shared memory, in rank
// order) add their partial tiles, so the sum order is fixed and nothing is staged in global
// memory.  Loads of W are issued before the wait on the previous kernel of the stream
// (programmatic dependent launch), since weights do not depend on it.
//
// Epilogues: bfloat16 or float32 result, or SiLU(gate) * up for a packed [gate | up] weight
// (tinyvllm/kernels/pointwise.cu:274-285) so that the activation never goes to memory.
// Stands where the reference calls F.linear (tinyvllm/layers.py:84-85).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

#define SM_WARPS 4
#define SM_BATCH 4            // k blocks a warp has in flight

#define MODE_BF16 0
#define MODE_F32 1
#define MODE_SILU 2

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_16(const bf16* p, bool ok) {
    return ok ? *reinterpret_cast<const uint4*>(p) : make_uint4(0u, 0u, 0u, 0u);
}

// NT: number of 8-row groups of x (M <= 8 NT).  SETS: 1, or 2 for the gate and up rows.
template <int NT, int MODE>
__global__ void __launch_bounds__(SM_WARPS * 32)
gemm_small_m_kernel(const bf16* __restrict__ x, int64_t ldx, const bf16* __restrict__ w, int64_t ldw,
                    void* __restrict__ out, int64_t ldo, int m, int n, int k, int up_offset) {
    constexpr int SETS = MODE == MODE_SILU ? 2 : 1;
    constexpr int MP = 8 * NT;
    __shared__ float warp_part[SM_WARPS][SETS][16][MP];
    __shared__ float cta_part[SETS][16][MP];

    cg::cluster_group cluster = cg::this_cluster();
    const int rank = blockIdx.x, ranks = gridDim.x;
    const int n0 = blockIdx.y * 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int k_blocks = (k + 31) / 32;
    const int stride = ranks * SM_WARPS;

    const bf16* w_lo[SETS];
    const bf16* w_hi[SETS];
    bool lo_ok[SETS], hi_ok[SETS];
#pragma unroll
    for (int s = 0; s < SETS; ++s) {
        const int row = n0 + g + s * up_offset;
        lo_ok[s] = n0 + g < n;
        hi_ok[s] = n0 + g + 8 < n;
        w_lo[s] = w + (int64_t)(lo_ok[s] ? row : 0) * ldw + 8 * t4;
        w_hi[s] = w + (int64_t)(hi_ok[s] ? row + 8 : 0) * ldw + 8 * t4;
    }
    float acc[SETS][NT][4];
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[s][j][i] = 0.0f;

    bool waited = false;
    for (int kb0 = rank * SM_WARPS + warp; kb0 < k_blocks; kb0 += stride * SM_BATCH) {
        uint4 a_lo[SM_BATCH][SETS], a_hi[SM_BATCH][SETS];
#pragma unroll
        for (int u = 0; u < SM_BATCH; ++u) {
            const int kb = kb0 + u * stride;
            const bool k_ok = kb < k_blocks && kb * 32 + 8 * t4 + 8 <= k;
#pragma unroll
            for (int s = 0; s < SETS; ++s) {
                a_lo[u][s] = load_16(w_lo[s] + kb * 32, k_ok && lo_ok[s]);
                a_hi[u][s] = load_16(w_hi[s] + kb * 32, k_ok && hi_ok[s]);
            }
        }
        if (!waited) {               // the weights are on their way; now the previous kernel's output
            asm volatile("griddepcontrol.wait;\n" ::: "memory");
            waited = true;
        }
#pragma unroll
        for (int u = 0; u < SM_BATCH; ++u) {
            const int kb = kb0 + u * stride;
            const bool k_ok = kb < k_blocks && kb * 32 + 8 * t4 + 8 <= k;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int row = 8 * j + g;
                const uint4 b = load_16(x + (int64_t)row * ldx + kb * 32 + 8 * t4, k_ok && row < m);
#pragma unroll
                for (int s = 0; s < SETS; ++s) {
                    mma_16816(acc[s][j], a_lo[u][s].x, a_hi[u][s].x, a_lo[u][s].y, a_hi[u][s].y, b.x, b.y);
                    mma_16816(acc[s][j], a_lo[u][s].z, a_hi[u][s].z, a_lo[u][s].w, a_hi[u][s].w, b.z, b.w);
                }
            }
        }
    }
    if (!waited) asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::);

    // ---- warps of the CTA, then CTAs of the cluster, in a fixed order
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            warp_part[warp][s][g][8 * j + 2 * t4] = acc[s][j][0];
            warp_part[warp][s][g][8 * j + 2 * t4 + 1] = acc[s][j][1];
            warp_part[warp][s][g + 8][8 * j + 2 * t4] = acc[s][j][2];
            warp_part[warp][s][g + 8][8 * j + 2 * t4 + 1] = acc[s][j][3];
        }
    __syncthreads();
    for (int index = threadIdx.x; index < SETS * 16 * MP; index += SM_WARPS * 32) {
        float total = 0.0f;
#pragma unroll
        for (int wi = 0; wi < SM_WARPS; ++wi) total += (&warp_part[wi][0][0][0])[index];
        (&cta_part[0][0][0])[index] = total;
    }
    cluster.sync();
    if (rank == 0) {
        // thread -> (row of x, column of the tile), columns fastest: 16 consecutive outputs per row
        for (int index = threadIdx.x; index < 16 * MP; index += SM_WARPS * 32) {
            const int col = index % 16, row = index / 16;
            float value[SETS];
#pragma unroll
            for (int s = 0; s < SETS; ++s) {
                float total = 0.0f;
                for (int r = 0; r < ranks; ++r) {
                    const float* other = cluster.map_shared_rank(&cta_part[0][0][0], r);
                    total += other[(s * 16 + col) * MP + row];
                }
                value[s] = total;
            }
            if (row < m && n0 + col < n) {
                const int64_t at = (int64_t)row * ldo + n0 + col;
                if (MODE == MODE_F32) {
                    reinterpret_cast<float*>(out)[at] = value[0];
                } else if (MODE == MODE_BF16) {
                    reinterpret_cast<bf16*>(out)[at] = __float2bfloat16_rn(value[0]);
                } else {
                    const float gate = value[0], up = value[SETS - 1];
                    const float activated = round_to<bf16>(__fdiv_rn(gate, __fadd_rn(1.0f, expf(-gate))));
                    reinterpret_cast<bf16*>(out)[at] = __float2bfloat16_rn(__fmul_rn(activated, up));
                }
            }
        }
    }
    cluster.sync();
}

template <int NT, int MODE>
static int launch_small_m(const void* x, long long ldx, const void* w, long long ldw, void* out,
                          long long ldo, int m, int n, int k, int up_offset, int ranks, int pdl,
                          cudaStream_t stream) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(ranks, (n + 15) / 16);
    config.blockDim = dim3(SM_WARPS * 32);
    config.dynamicSmemBytes = 0;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = ranks;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    config.numAttrs = 1;
    if (pdl) {
        attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[1].val.programmaticStreamSerializationAllowed = 1;
        config.numAttrs = 2;
    }
    config.attrs = attributes;
    cudaError_t e = cudaLaunchKernelEx(&config, gemm_small_m_kernel<NT, MODE>, (const bf16*)x, (int64_t)ldx,
                                       (const bf16*)w, (int64_t)ldw, out, (int64_t)ldo, m, n, k, up_offset);
    return e == cudaSuccess ? tvb_last_error() : (int)e;
}

extern "C" int tvb_gemm_small_m_max_rows() { return 32; }

// mode: 0 bfloat16 result [m, n]; 1 float32 result [m, n]; 2 SiLU(gate) * up, w = [gate (n rows) |
// up (n rows)] and the result is [m, n].  k must be a multiple of 8 and rows 16-byte aligned.
// pdl != 0 launches with programmatic stream serialisation (the kernel before it in the stream
// must then be one that tolerates an early start of this one: this kernel only reads weights
// before it waits).
extern "C" int tvb_gemm_small_m(const void* x, long long ldx, const void* w, long long ldw, void* out,
                                long long ldo, int m, int n, int k, int mode, int pdl, void* stream) {
    if (m <= 0 || n <= 0) return 0;
    if (m > 32 || k <= 0 || k % 8 || ldx % 8 || ldw % 8 || mode < 0 || mode > 2 || n > 65535 * 16)
        return TVB_BAD_ARGUMENT;
    const int k_blocks = (k + 31) / 32;
    // enough CTAs per row tile that every warp has about one batch of k blocks, at most 8 per cluster
    // (a power of two)
    const int wanted = (k_blocks + SM_WARPS * SM_BATCH - 1) / (SM_WARPS * SM_BATCH);
    int ranks = 1;
    while (ranks < wanted && ranks < 8) ranks *= 2;
    const int up_offset = mode == MODE_SILU ? n : 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = (m + 7) / 8;
#define SMALL_M(NT, MODE) launch_small_m<NT, MODE>(x, ldx, w, ldw, out, ldo, m, n, k, up_offset, ranks, pdl, s)
#define BY_NT(MODE)                                  \
    do {                                             \
        if (nt == 1) return SMALL_M(1, MODE);        \
        if (nt == 2) return SMALL_M(2, MODE);        \
        if (nt == 3) return SMALL_M(3, MODE);        \
        return SMALL_M(4, MODE);                     \
    } while (0)
    if (mode == MODE_BF16) BY_NT(MODE_BF16);
    if (mode == MODE_F32) BY_NT(MODE_F32);
    BY_NT(MODE_SILU);
}
