// This file is the body of the libraries gemm_small_m_nt<1..4>.cu: each defines TVB_SMALL_M_NT (the
// number of 8-row groups of x it is compiled for) and includes it, so that a decode step compiles
// the templates of its own batch size only.
//
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
// Work is cut as (N / 16 row tiles) x (k blocks dealt round-robin to the 4 warps of the CTAs
// of a thread-block cluster).  Warps add their partial tiles, every CTA stores its sum into the
// shared memory of the cluster's first CTA (distributed shared memory), and after one cluster
// barrier that CTA adds them in rank order: the sum order is fixed, nothing is staged in global
// memory, and the other CTAs are done at the barrier.  Loads of W are issued before the wait on
// the previous kernel of the stream (programmatic dependent launch), since weights do not depend
// on it, and the kernel behind this one is released at once, so that it can do the same.
//
// Prologue (optional): x = RMSNorm(h + residual) computed by every CTA for itself into
// shared memory while its weights are in flight (tinyvllm/kernels/pointwise.cu:153-211);
// the first CTA also stores the new residual stream.  Epilogues: bfloat16 or float32
// result, or SiLU(gate) * up for a packed [gate | up] weight (:274-285), so that neither
// the normalised input nor the activation goes through memory.
//
// A pre-norm between two products without a kernel of its own: the first product (a part's
// output projection) adds its result to the residual stream on the way out and stores, for
// every row, the sum of squares of the 16 columns of each of its tiles.  The second (the next
// part's input projection) multiplies its x fragments by the norm weight as it loads them and
// applies the row's inverse RMS, a factor of the whole row, to the finished sums: only the CTA
// that writes a tile reads the partial sums (in a fixed order), it asks for them at its start
// and needs them at its end.  (Every CTA reading them before its first product cost as much as
// the norm kernel: hundreds of CTAs ask for the same 2 KB.)  The rounding differs from the norm
// kernel's in one place: round(stream * weight) enters the product, where the kernel rounds
// stream * inverse RMS first and the product with the weight second.
// Stands where the reference calls F.linear (tinyvllm/layers.py:84-85).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

#define SM_WARPS 4
#define SM_BATCH 4            // k blocks a warp has in flight
#define SM_PAD 32             // bfloat16 of padding per row of x in shared memory (no bank conflicts)

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

struct NormArgs {
    const bf16* residual;       // null: x = RMSNorm(h), the stream is h itself (written by an earlier kernel)
    const void* weight;         // [k], bfloat16 or float32
    bf16* residual_out;         // null: not stored
    float eps;
    const float* squares;       // NORM 3, 4: [square_tiles][8 NT] partial sums of squares of the rows of x
    int square_tiles;
};

// The epilogue that adds the product to the residual stream (MODE_BF16 only).
struct StreamArgs {
    const bf16* stream;         // [m, n] contiguous; null: the plain epilogue
    float* squares_out;         // [tiles of 16 columns][8 NT]: sums of squares of the new stream
};

// NT: number of 8-row groups of x (M <= 8 NT).  NORM: 0 none; 1 bfloat16 weight, 2 float32 weight:
// the prologue normalises x + residual; 3, 4 (bfloat16, float32 weight): x is the stream, its
// fragments are multiplied by the norm weight and the results by the rows' inverse RMS, from the
// sums of squares the product before stored.
template <int NT, int MODE, int NORM>
__global__ void __launch_bounds__(SM_WARPS * 32)
gemm_small_m_kernel(const bf16* x, int64_t ldx, const bf16* __restrict__ w, int64_t ldw,
                    void* __restrict__ out, int64_t ldo, int m, int n, int k, int up_offset, NormArgs norm,
                    StreamArgs into, const void* __restrict__ next_weight, long long next_bytes) {
    constexpr int SETS = MODE == MODE_SILU ? 2 : 1;
    constexpr int MP = 8 * NT;
    __shared__ float warp_part[SM_WARPS][SETS][16][MP];
    // partial tiles of every CTA of the cluster; only the first CTA's copy is used: the others store
    // theirs into it through distributed shared memory
    constexpr int MAX_RANKS = NT <= 2 ? 8 : 4;
    __shared__ float cluster_part[MAX_RANKS][SETS][16][MP];
    constexpr bool PROLOGUE_NORM = NORM == 1 || NORM == 2;
    constexpr bool SCALED = NORM >= 3;
    extern __shared__ __align__(16) unsigned char dynamic_shared[];
    bf16* x_s = reinterpret_cast<bf16*>(dynamic_shared);       // [MP][k + SM_PAD] when NORM

    cg::cluster_group cluster = cg::this_cluster();
    const int rank = blockIdx.x, ranks = gridDim.x;
    // Every CTA says that it runs; before the first store into another CTA's shared memory the
    // epilogue makes sure that all of them have said so.
    cluster_arrive_relaxed();
    const int n0 = blockIdx.y * 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int k_blocks = (k + 31) / 32;
    const int stride = ranks * SM_WARPS;
    const int x_row = k + SM_PAD;

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

    constexpr int SQUARE_LOADS = 4;      // tiles of the stream's sums of squares a lane asks for up front
    float row_squares[SCALED ? NT : 1][SQUARE_LOADS];
    bool ready = false;          // the previous kernel's output may be read (and the norm is done)
    for (int kb0 = rank * SM_WARPS + warp; kb0 < k_blocks || !ready; kb0 += stride * SM_BATCH) {
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
        if (!ready) {                // the weights are on their way; now the previous kernel's output
            // The kernel behind this one may start now: what it does before its own wait (the
            // decode attention looks up cache slots and starts streaming keys, a product its
            // weights) runs beside this product, which leaves most of the memory system idle.
            pdl_launch_dependents();
            prefetch_l2_range(next_weight, next_bytes);   // and those of the product after this one
            pdl_wait();
            if (SCALED && rank == 0) {
                // The rows' sums of squares are needed at the very end only (the inverse RMS is a factor
                // of the whole row of x, so it is applied to the finished sums): asked for now, by the
                // CTA that writes the tile; lane `col` of a row's 16 takes tiles col, col + 16, ...
#pragma unroll
                for (int i = 0; i < NT; ++i) {
                    const int index = threadIdx.x + i * SM_WARPS * 32;
                    const int col = index % 16, row = index / 16;
#pragma unroll
                    for (int q = 0; q < SQUARE_LOADS; ++q) {
                        const int t = col + 16 * q;
                        row_squares[i][q] = t < norm.square_tiles ? ld_global_f32(norm.squares + (int64_t)t * MP + row) : 0.0f;
                    }
                }
            }
            if (PROLOGUE_NORM) {
                // every CTA normalises all rows for itself: warp w takes rows w, w + 4, ...
                for (int row = warp; row < MP; row += SM_WARPS) {
                    bf16* dst = x_s + row * x_row;
                    if (row >= m) {
                        for (int i = lane * 8; i < k; i += 256) *reinterpret_cast<uint4*>(dst + i) = make_uint4(0, 0, 0, 0);
                        continue;
                    }
                    const bf16* h = x + (int64_t)row * ldx;
                    const bf16* r = norm.residual ? norm.residual + (int64_t)row * k : nullptr;
                    float squares = 0.0f;
                    for (int i = lane * 8; i < k; i += 256) {
                        float v[8], rv[8];
                        unpack_bf16x8(ld_global_16(h + i), v);
                        if (r) {
                            unpack_bf16x8(ld_global_16(r + i), rv);
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] = round_to<bf16>(__fadd_rn(v[e], rv[e]));
                        }
#pragma unroll
                        for (int e = 0; e < 8; ++e) squares = __fadd_rn(squares, __fmul_rn(v[e], v[e]));
                        const uint4 merged = pack_bf16x8(v);
                        *reinterpret_cast<uint4*>(dst + i) = merged;      // the stream, normalised below
                        if (norm.residual_out && rank == 0 && blockIdx.y == 0)
                            *reinterpret_cast<uint4*>(norm.residual_out + (int64_t)row * k + i) = merged;
                    }
                    squares = warp_sum(squares);
                    const float inverse_rms =
                        __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(squares, 1.0f / (float)k), norm.eps)));
                    for (int i = lane * 8; i < k; i += 256) {
                        float v[8];
                        unpack_bf16x8(*reinterpret_cast<const uint4*>(dst + i), v);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float weight = NORM == 2 ? reinterpret_cast<const float*>(norm.weight)[i + e]
                                                           : __bfloat162float(reinterpret_cast<const bf16*>(norm.weight)[i + e]);
                            v[e] = __fmul_rn(round_to<bf16>(__fmul_rn(v[e], inverse_rms)), weight);
                        }
                        *reinterpret_cast<uint4*>(dst + i) = pack_bf16x8(v);
                    }
                }
                __syncthreads();
            }
        }
        // ---- the x fragments of this batch: all loads first, so that their latencies overlap
        uint4 b_all[SM_BATCH][NT];
        float norm_weight[SCALED ? SM_BATCH : 1][8];
#pragma unroll
        for (int u = 0; u < SM_BATCH; ++u) {
            const int kb = kb0 + u * stride;
            const bool k_ok = kb < k_blocks && kb * 32 + 8 * t4 + 8 <= k;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int row = 8 * j + g;
                if (PROLOGUE_NORM) b_all[u][j] = k_ok ? *reinterpret_cast<const uint4*>(x_s + row * x_row + kb * 32 + 8 * t4)
                                                      : make_uint4(0u, 0u, 0u, 0u);
                else b_all[u][j] = k_ok && row < m ? ld_global_16(x + (int64_t)row * ldx + kb * 32 + 8 * t4)
                                                   : make_uint4(0u, 0u, 0u, 0u);
            }
            if (SCALED) {
                const int at = k_ok ? kb * 32 + 8 * t4 : 0;
                if (NORM == 4) {
                    const float4 lo = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(norm.weight) + at);
                    const float4 hi = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(norm.weight) + at + 4);
                    norm_weight[u][0] = lo.x, norm_weight[u][1] = lo.y, norm_weight[u][2] = lo.z, norm_weight[u][3] = lo.w;
                    norm_weight[u][4] = hi.x, norm_weight[u][5] = hi.y, norm_weight[u][6] = hi.z, norm_weight[u][7] = hi.w;
                } else {
                    unpack_bf16x8(*reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(norm.weight) + at), norm_weight[u]);
                }
            }
        }
        if (!ready) {
            ready = true;
        }
#pragma unroll
        for (int u = 0; u < SM_BATCH; ++u) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                uint4 b = b_all[u][j];
                if (SCALED) {
                    float v[8];
                    unpack_bf16x8(b, v);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], norm_weight[u][e]);
                    b = pack_bf16x8(v);
                }
#pragma unroll
                for (int s = 0; s < SETS; ++s) {
                    mma_16816(acc[s][j], a_lo[u][s].x, a_hi[u][s].x, a_lo[u][s].y, a_hi[u][s].y, b.x, b.y);
                    mma_16816(acc[s][j], a_lo[u][s].z, a_hi[u][s].z, a_lo[u][s].w, a_hi[u][s].w, b.z, b.w);
                }
            }
        }
    }

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
    cluster_wait();
    {
        float* slot_at_first = cluster.map_shared_rank(&cluster_part[0][0][0][0], 0) + rank * (SETS * 16 * MP);
        for (int index = threadIdx.x; index < SETS * 16 * MP; index += SM_WARPS * 32) {
            float total = 0.0f;
#pragma unroll
            for (int wi = 0; wi < SM_WARPS; ++wi) total += (&warp_part[wi][0][0][0])[index];
            slot_at_first[index] = total;       // a store into the first CTA's shared memory
        }
    }
    // thread -> (row of x, column of the tile), columns fastest: 16 consecutive outputs per row; what the
    // epilogue adds from the stream is asked for before the barrier, so that it arrives meanwhile
    float from_stream[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        const int index = threadIdx.x + i * SM_WARPS * 32;
        const int col = index % 16, row = index / 16;
        from_stream[i] = 0.0f;
        if (MODE == MODE_BF16 && rank == 0 && into.stream && row < m && n0 + col < n)
            from_stream[i] = bf16_bits_to_float(ld_global_u16(into.stream + (int64_t)row * n + n0 + col));
    }
    cluster.sync();                             // every CTA's stores have arrived; the others are done
    if (rank == 0) {
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int index = threadIdx.x + i * SM_WARPS * 32;
            const int col = index % 16, row = index / 16;
            float value[SETS];
#pragma unroll
            for (int s = 0; s < SETS; ++s) {
                float total = 0.0f;
                for (int r = 0; r < ranks; ++r) total += cluster_part[r][s][col][row];
                value[s] = total;
            }
            if (SCALED) {
                // sum of squares of the row: this lane's tiles in ascending order, then the 16 lanes of the row
                float squares = 0.0f;
#pragma unroll
                for (int q = 0; q < SQUARE_LOADS; ++q) squares = __fadd_rn(squares, row_squares[i][q]);
                for (int t = col + 16 * SQUARE_LOADS; t < norm.square_tiles; t += 16)
                    squares = __fadd_rn(squares, ld_global_f32(norm.squares + (int64_t)t * MP + row));
#pragma unroll
                for (int delta = 8; delta > 0; delta >>= 1) squares = __fadd_rn(squares, __shfl_xor_sync(0xffffffffu, squares, delta));
                const float inverse_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(squares, 1.0f / (float)k), norm.eps)));
#pragma unroll
                for (int s = 0; s < SETS; ++s) value[s] = __fmul_rn(value[s], inverse_rms);
            }
            if (row < m && n0 + col < n) {
                const int64_t at = (int64_t)row * ldo + n0 + col;
                if (MODE == MODE_F32) {
                    reinterpret_cast<float*>(out)[at] = value[0];
                } else if (MODE == MODE_BF16) {
                    if (!into.stream) reinterpret_cast<bf16*>(out)[at] = __float2bfloat16_rn(value[0]);
                } else {
                    const float gate = value[0], up = value[SETS - 1];
                    const float activated = round_to<bf16>(__fdiv_rn(gate, __fadd_rn(1.0f, expf(-gate))));
                    reinterpret_cast<bf16*>(out)[at] = __float2bfloat16_rn(__fmul_rn(activated, up));
                }
            }
            if (MODE == MODE_BF16 && into.stream) {
                // the new residual stream and, over the 16 columns of this tile (16 consecutive lanes),
                // its sum of squares for the norm that the next product applies
                float added = 0.0f;
                if (row < m && n0 + col < n) {
                    added = round_to<bf16>(__fadd_rn(round_to<bf16>(value[0]), from_stream[i]));
                    reinterpret_cast<bf16*>(out)[(int64_t)row * ldo + n0 + col] = __float2bfloat16_rn(added);
                }
                float squares = __fmul_rn(added, added);
#pragma unroll
                for (int delta = 8; delta > 0; delta >>= 1) squares = __fadd_rn(squares, __shfl_xor_sync(0xffffffffu, squares, delta));
                if (col == 0) into.squares_out[(int64_t)blockIdx.y * MP + row] = squares;
            }
        }
    }
}

template <int NT, int MODE, int NORM>
static int launch_small_m(const void* x, long long ldx, const void* w, long long ldw, void* out,
                          long long ldo, int m, int n, int k, int up_offset, int ranks, int pdl,
                          NormArgs norm, StreamArgs into, const void* next_weight, long long next_bytes,
                          cudaStream_t stream) {
    auto kernel = gemm_small_m_kernel<NT, MODE, NORM>;
    size_t dynamic = 0;
    if (NORM == 1 || NORM == 2) {
        dynamic = (size_t)8 * NT * (k + SM_PAD) * sizeof(bf16);
        if (dynamic > 160 * 1024) return TVB_BAD_ARGUMENT;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dynamic);
        if (e != cudaSuccess) return (int)e;
    }
    TvbLaunch launch(dim3(ranks, (n + 15) / 16), dim3(SM_WARPS * 32), dynamic, stream, pdl, ranks);
    cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, (const bf16*)x, (int64_t)ldx, (const bf16*)w,
                                       (int64_t)ldw, out, (int64_t)ldo, m, n, k, up_offset, norm, into,
                                       next_weight, next_bytes);
    return e == cudaSuccess ? tvb_last_error() : (int)e;
}

extern "C" int tvb_gemm_small_m_max_rows() { return 32; }

// mode: 0 bfloat16 result [m, n]; 1 float32 result [m, n]; 2 SiLU(gate) * up, w = [gate (n rows) |
// up (n rows)] and the result is [m, n].  k must be a multiple of 8 and rows 16-byte aligned.
//
// norm_weight != null: x is replaced by RMSNorm(x + residual) * norm_weight (residual may be null;
// both are contiguous [m, k]); residual_out (may be null) receives the rounded sum.
// norm_weight_dtype: TVB_BF16 or TVB_F32.
//
// row_squares != null (with norm_weight, without residual): x is the residual stream itself and
// row_squares [square_tiles][m rounded up to 8] holds partial sums of squares of its rows, as a
// launch with add_stream stored them; the result is that of RMSNorm(x) * norm_weight, computed as
// (round(x * norm_weight) . w^T) * inverse RMS of the row.  norm_weight is 16-byte aligned.
// add_stream != null (mode 0): out = round(round(product) + add_stream) (both contiguous [m, n] is
// assumed for add_stream), and squares_out [ceil(n / 16)][m rounded up to 8] receives the sums of
// squares of out over each tile of 16 columns.
//
// next_weight / next_bytes (may be null / 0): memory the grid asks to be brought into L2 while it
// works, typically the weight of the product that follows.
//
// pdl != 0 launches with programmatic stream serialisation: the kernel may start while the kernel
// before it in the stream still runs; it reads nothing but weights before it waits for that kernel.
extern "C" int tvb_gemm_small_m(const void* x, long long ldx, const void* w, long long ldw, void* out,
                                long long ldo, int m, int n, int k, int mode, const void* residual,
                                const void* norm_weight, void* residual_out, float eps,
                                int norm_weight_dtype, const float* row_squares, int square_tiles,
                                const void* add_stream, float* squares_out, const void* next_weight,
                                long long next_bytes, int pdl, void* stream) {
    if (m <= 0 || n <= 0) return 0;
    if (m > 32 || k <= 0 || k % 8 || ldx % 8 || ldw % 8 || mode < 0 || mode > 2 || n > 65535 * 16)
        return TVB_BAD_ARGUMENT;
    if (norm_weight && ldx != k) return TVB_BAD_ARGUMENT;
    if (row_squares && (!norm_weight || residual || residual_out || square_tiles <= 0)) return TVB_BAD_ARGUMENT;
    if (add_stream && (mode != MODE_BF16 || !squares_out)) return TVB_BAD_ARGUMENT;
    const int k_blocks = (k + 31) / 32;
    // enough CTAs per row tile that every warp has about one batch of k blocks, at most 8 per
    // cluster (a power of two)
    const int wanted = (k_blocks + SM_WARPS * SM_BATCH - 1) / (SM_WARPS * SM_BATCH);
    const int max_ranks = m <= 16 ? 8 : 4;      // what the kernel's shared memory holds partial tiles of
    int ranks = 1;
    while (ranks < wanted && ranks < max_ranks) ranks *= 2;
    const int up_offset = mode == MODE_SILU ? n : 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = (m + 7) / 8;
    NormArgs norm = {(const bf16*)residual, norm_weight, (bf16*)residual_out, eps, row_squares, square_tiles};
    StreamArgs into = {(const bf16*)add_stream, squares_out};
    if (norm_weight && norm_weight_dtype != TVB_F32 && norm_weight_dtype != TVB_BF16) return TVB_BAD_ARGUMENT;
    const int norm_kind = !norm_weight ? 0 : (norm_weight_dtype == TVB_F32 ? 2 : 1) + (row_squares ? 2 : 0);
#define SMALL_M(NT, MODE, NORM) \
    launch_small_m<NT, MODE, NORM>(x, ldx, w, ldw, out, ldo, m, n, k, up_offset, ranks, pdl, norm, into, \
                                   next_weight, next_bytes, s)
#define BY_NORM(NT, MODE)                                   \
    do {                                                    \
        if (norm_kind == 0) return SMALL_M(NT, MODE, 0);    \
        if (norm_kind == 1) return SMALL_M(NT, MODE, 1);    \
        if (norm_kind == 2) return SMALL_M(NT, MODE, 2);    \
        if (norm_kind == 3) return SMALL_M(NT, MODE, 3);    \
        return SMALL_M(NT, MODE, 4);                        \
    } while (0)
    // this library holds one number of 8-row groups
    if (nt != TVB_SMALL_M_NT) return TVB_BAD_ARGUMENT;
#define BY_NT(MODE) BY_NORM(TVB_SMALL_M_NT, MODE)
    if (mode == MODE_BF16) BY_NT(MODE_BF16);
    if (mode == MODE_F32) BY_NT(MODE_F32);
    BY_NT(MODE_SILU);
}
