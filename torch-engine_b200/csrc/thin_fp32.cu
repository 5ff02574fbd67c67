// FP32-accurate products with a thin left operand (M <= 16 rows) on the FP32 units.
//
// C[M,N] = A[M,K] . B[K,N] with M <= 16 reads every element of B once and uses it M times: 2.M FLOP per 4 bytes, far
// below what the tensor cores need to be worth their set-up.  In 3xTF32 mode the tensor-core path pads the 16 rows to
// a 128-row MMA, issues three MMAs per k-step and rewrites every landed tile of B as hi / lo planes in shared memory:
// 0.121 ms at 16 x 8192 x 8192, 2.5x the TF32-mode time of the same product, with HBM at a third of its rate.  The
// product is memory-bound, so it is computed here as what it is: each thread owns four consecutive columns of C and
// all M rows (64 accumulators), streams its columns of B from global memory with 16-byte loads, eight rows of B in
// flight per thread (a warp reads 512 contiguous bytes per k), and takes the M values of A for that k as broadcast
// reads from shared memory.  Arithmetic is FP32 FMA (the packed two-lane
// instruction of sm_100, each lane rounded as a scalar fma) in ascending k
// within a K slice, i.e. what the reference's cuBLAS FP32 path and its CPU loop compute (reference
// src/tensor/tensor.h:690-698, :795-836), not a split: the mode's promise is FP32 accuracy, and this is FP32.
//
// K is cut into slices so that a few CTAs per SM exist (the grid is column blocks x slices); every slice writes a
// partial [M, N] tile to the split-K scratch and the common reduction adds the slices in slice order and applies
// the epilogue (scale, bias, GELU, residual), as for the tensor-core kernels.
// Limits: one product (no batch), A with K contiguous, B with N contiguous, M <= 16; everything else stays on the
// tensor-core path.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_common.cuh"

namespace te {

namespace {

constexpr int THIN_M = 16;          // rows of A a thread accumulates
constexpr int THIN_COLS = 512;      // columns of C per CTA: four consecutive ones per thread
constexpr int THIN_THREADS = 128;
constexpr int THIN_KC = 128;        // k extent of one staged chunk of A
constexpr int THIN_UNROLL = 16;     // k steps whose loads of B are issued before the first FMA

struct ThinParams {
    const float* a; long long lda;
    const float* b; long long ldb;
    float* partial;                  // [slices][M][N]
    int M, N, K;
    int k_per_slice;                 // multiple of THIN_UNROLL
};

// Two FP32 FMAs in one instruction (sm_100 packed form): d.lo = a.lo * b.lo + d.lo, d.hi = a.hi * b.hi + d.hi, each
// rounded like a scalar fma.rn.  The kernel is bound by instruction issue, not by the FP32 lanes, so halving the
// FMA instructions is what the packed form buys.
__device__ __forceinline__ void fma2(unsigned long long& d, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ unsigned long long pair_of(float x) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void unpack(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__global__ void __launch_bounds__(THIN_THREADS) thin_fp32_kernel(const ThinParams p) {
    __shared__ __align__(16) float a_sm[THIN_KC][THIN_M];        // [k][m]: the M values of one k are one 64-byte row
    griddep_wait();
    const int t = threadIdx.x;
    const int c0 = blockIdx.x * THIN_COLS + 4 * t;               // this thread's four consecutive columns (N % 4 == 0)
    const bool live = c0 < p.N;
    const int k_begin = blockIdx.y * p.k_per_slice;
    const int k_end = min(k_begin + p.k_per_slice, p.K);
    // accumulators as pairs of rows (m, m + 1): acc[c][q] holds rows 2q and 2q + 1 of column c0 + c
    unsigned long long acc[4][THIN_M / 2];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int q = 0; q < THIN_M / 2; ++q) acc[c][q] = 0ull;       // two +0.0f
    // staging map: 16 threads cover the rows of one k, a warp covers two k (conflict-free shared-memory writes)
    const int sm_m = t & 15, sm_k = t >> 4;
    // columns past N read the last four columns instead (their sums are not stored): the loads need no predicate
    const float* bcol = p.b + (live ? c0 : p.N - 4);
    for (int kc = k_begin; kc < k_end; kc += THIN_KC) {
        __syncthreads();             // the previous chunk has been consumed
#pragma unroll
        for (int j = 0; j < THIN_KC / 8; ++j) {
            const int kk = sm_k + 8 * j, k = kc + kk;
            a_sm[kk][sm_m] = (sm_m < p.M && k < k_end) ? __ldg(p.a + (long long)sm_m * p.lda + k) : 0.0f;
        }
        __syncthreads();
        const int chunk = min(THIN_KC, k_end - kc);
        for (int kk = 0; kk < chunk; kk += THIN_UNROLL) {
            float4 v[THIN_UNROLL];
            const float* r = bcol + (long long)(kc + kk) * p.ldb;
            if (kk + THIN_UNROLL <= chunk) {         // uniform: all but the last group of the last slice
#pragma unroll
                for (int u = 0; u < THIN_UNROLL; ++u) v[u] = __ldg(reinterpret_cast<const float4*>(r + (long long)u * p.ldb));
            } else {
#pragma unroll
                for (int u = 0; u < THIN_UNROLL; ++u)        // rows of A past the slice are zero; B is not read there
                    v[u] = kk + u < chunk ? __ldg(reinterpret_cast<const float4*>(r + (long long)u * p.ldb)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < THIN_UNROLL; ++u) {
                const ulonglong2* row = reinterpret_cast<const ulonglong2*>(&a_sm[kk + u][0]);
                const unsigned long long w0 = pair_of(v[u].x), w1 = pair_of(v[u].y), w2 = pair_of(v[u].z), w3 = pair_of(v[u].w);
#pragma unroll
                for (int q = 0; q < THIN_M / 4; ++q) {
                    const ulonglong2 a = row[q];             // rows 4q .. 4q + 3 of A at this k
                    fma2(acc[0][2 * q], a.x, w0); fma2(acc[0][2 * q + 1], a.y, w0);
                    fma2(acc[1][2 * q], a.x, w1); fma2(acc[1][2 * q + 1], a.y, w1);
                    fma2(acc[2][2 * q], a.x, w2); fma2(acc[2][2 * q + 1], a.y, w2);
                    fma2(acc[3][2 * q], a.x, w3); fma2(acc[3][2 * q + 1], a.y, w3);
                }
            }
        }
    }
    if (!live) return;
    float* out = p.partial + (long long)blockIdx.y * p.M * p.N + c0;
#pragma unroll
    for (int q = 0; q < THIN_M / 2; ++q) {
        float lo[4], hi[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) unpack(acc[c][q], lo[c], hi[c]);
        if (2 * q < p.M) *reinterpret_cast<float4*>(out + (long long)(2 * q) * p.N) = make_float4(lo[0], lo[1], lo[2], lo[3]);
        if (2 * q + 1 < p.M) *reinterpret_cast<float4*>(out + (long long)(2 * q + 1) * p.N) = make_float4(hi[0], hi[1], hi[2], hi[3]);
    }
}

// ---- the same product with B staged by TMA ---------------------------------------------------------------------
// Above, what bounds the kernel is the bytes of B a thread can keep in flight in registers (96 KB per SM).  Here a
// producer warp lands 8-row x 1024-column slabs of B in a ring of six 32 KB shared-memory stages (160 KB in flight per
// SM, no register cost), eight consumer warps read their four columns of a slab back with one 16-byte load per k and
// keep the same 64 accumulators.  One CTA per SM; used when the grid of column blocks x K slices fills the GPU.
constexpr int TT_CONSUMERS = 256;
constexpr int TT_THREADS = TT_CONSUMERS + 32;
constexpr int TT_COLS = 4 * TT_CONSUMERS;            // 1024 columns of C per CTA
constexpr int TT_KS = 8;                              // rows of B per stage
constexpr int TT_BOX_COLS = 256;                      // a TMA box is at most 256 elements wide
constexpr int TT_BOXES = TT_COLS / TT_BOX_COLS;
constexpr int TT_STAGE_BYTES = TT_KS * TT_COLS * 4;   // 32 KB
constexpr int TT_STAGES = 6;
constexpr int TT_SMEM_BYTES = TT_STAGES * TT_STAGE_BYTES + THIN_KC * THIN_M * 4 + 256 + 128;

__global__ void __launch_bounds__(TT_THREADS, 1) thin_fp32_tma_kernel(const __grid_constant__ CUtensorMap tm_b, const ThinParams p, int* status) {
    extern __shared__ uint8_t tt_smem[];
    const uint32_t raw = smem_u32(tt_smem);
    const uint32_t ring = (raw + 127u) & ~127u;
    const uint32_t a_addr = ring + TT_STAGES * TT_STAGE_BYTES;
    float (*a_sm)[THIN_M] = reinterpret_cast<float (*)[THIN_M]>(tt_smem + (a_addr - raw));
    const uint32_t bar_full = a_addr + THIN_KC * THIN_M * 4;
    const uint32_t bar_empty = bar_full + 8 * TT_STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tt_smem + (bar_empty + 8 * TT_STAGES - raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < TT_STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, TT_CONSUMERS / 32);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tm_b);
    }
    __syncthreads();
    griddep_launch_dependents();
    griddep_wait();
    const int k_begin = blockIdx.y * p.k_per_slice;
    const int k_end = min(k_begin + p.k_per_slice, p.K);
    const int stages = (k_end - k_begin + TT_KS - 1) / TT_KS;
    const int col0 = blockIdx.x * TT_COLS;
    if (warp == TT_CONSUMERS / 32) {
        // ------------------------------------------------------------ producer: slabs of B, K ascending
        if (lane == 0) {
            for (int i = 0; i < stages; ++i) {
                const int s = i % TT_STAGES;
                if (!wait_bounded(bar_empty + 8 * s, ((i / TT_STAGES) & 1) ^ 1, abort_flag, status, WAIT_THIN_EMPTY)) break;
                mbar_arrive_expect_tx(bar_full + 8 * s, TT_STAGE_BYTES);     // rows past K and columns past N arrive as zeros
#pragma unroll
                for (int b = 0; b < TT_BOXES; ++b)
                    tma_load_4d(ring + s * TT_STAGE_BYTES + b * (TT_KS * TT_BOX_COLS * 4), &tm_b, bar_full + 8 * s,
                                col0 + b * TT_BOX_COLS, k_begin + i * TT_KS, 0, 0);
            }
            if (*abort_flag) {      // copies already issued still write shared memory: let them land
                const uint64_t t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 200000ull) {
                }
            }
        }
    } else {
        // ------------------------------------------------------------ consumers: four columns x 16 rows each
        const int t = threadIdx.x;
        const int c0 = col0 + 4 * t;
        unsigned long long acc[4][THIN_M / 2];
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int q = 0; q < THIN_M / 2; ++q) acc[c][q] = 0ull;
        const int sm_m = t & 15, sm_k = t >> 4;                           // 16 k rows of A per staging pass
        // this thread's 16 bytes of a slab row: box t / 64, 16-byte unit t % 64
        const uint32_t b_off = (uint32_t)(t >> 6) * (TT_KS * TT_BOX_COLS * 4) + (uint32_t)(t & 63) * 16;
        // A warp whose wait ran out keeps walking the loop for the two barriers of every A chunk (the other warps
        // count on all 256 threads there) and does nothing else.
        bool ok = true;
        for (int i = 0; i < stages; ++i) {
            const int kk0 = (i * TT_KS) % THIN_KC;
            if (kk0 == 0) {          // next 128 k of A: [k][m], zeros past the slice and past M
                asm volatile("bar.sync 1, %0;" ::"n"(TT_CONSUMERS) : "memory");
                const int kc = k_begin + i * TT_KS;
                if (ok) {
#pragma unroll
                    for (int j = 0; j < THIN_KC / 16; ++j) {
                        const int kk = sm_k + 16 * j, k = kc + kk;
                        a_sm[kk][sm_m] = (sm_m < p.M && k < k_end) ? __ldg(p.a + (long long)sm_m * p.lda + k) : 0.0f;
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(TT_CONSUMERS) : "memory");
            }
            if (!ok) continue;
            const int s = i % TT_STAGES;
            ok = wait_bounded(bar_full + 8 * s, (i / TT_STAGES) & 1, abort_flag, status, WAIT_THIN_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) continue;
            const uint32_t slab = ring + s * TT_STAGE_BYTES + b_off;
            float4 v[TT_KS];
#pragma unroll
            for (int u = 0; u < TT_KS; ++u) v[u] = ld_shared_v4(slab + u * (TT_BOX_COLS * 4));
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);                 // the slab is in registers
#pragma unroll
            for (int u = 0; u < TT_KS; ++u) {
                const ulonglong2* row = reinterpret_cast<const ulonglong2*>(&a_sm[kk0 + u][0]);
                const unsigned long long w0 = pair_of(v[u].x), w1 = pair_of(v[u].y), w2 = pair_of(v[u].z), w3 = pair_of(v[u].w);
#pragma unroll
                for (int q = 0; q < THIN_M / 4; ++q) {
                    const ulonglong2 a = row[q];
                    fma2(acc[0][2 * q], a.x, w0); fma2(acc[0][2 * q + 1], a.y, w0);
                    fma2(acc[1][2 * q], a.x, w1); fma2(acc[1][2 * q + 1], a.y, w1);
                    fma2(acc[2][2 * q], a.x, w2); fma2(acc[2][2 * q + 1], a.y, w2);
                    fma2(acc[3][2 * q], a.x, w3); fma2(acc[3][2 * q + 1], a.y, w3);
                }
            }
        }
        if (ok && c0 < p.N) {
            float* out = p.partial + (long long)blockIdx.y * p.M * p.N + c0;
#pragma unroll
            for (int q = 0; q < THIN_M / 2; ++q) {
                float lo[4], hi[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) unpack(acc[c][q], lo[c], hi[c]);
                if (2 * q < p.M) *reinterpret_cast<float4*>(out + (long long)(2 * q) * p.N) = make_float4(lo[0], lo[1], lo[2], lo[3]);
                if (2 * q + 1 < p.M) *reinterpret_cast<float4*>(out + (long long)(2 * q + 1) * p.N) = make_float4(hi[0], hi[1], hi[2], hi[3]);
            }
        }
    }
}

}  // namespace

// Returns TE_OK when the product was issued here, -1 when it is outside this form's limits (the caller then takes the
// tensor-core path), or an error status.
int launch_thin_fp32(te_b200_ctx* ctx, const GemmProblem& g, cudaStream_t stream) {
    if (g.batch_inner * g.batch_outer != 1 || g.M < 1 || g.M > THIN_M || g.K < 256 || g.N < 512) return -1;
    if (g.a.mn_major || !g.b.mn_major || g.preact) return -1;
    if ((g.N & 3) || (g.b.ld & 3) || (reinterpret_cast<uintptr_t>(g.b.ptr) & 15) || (reinterpret_cast<uintptr_t>(g.split_ws) & 15)) return -1;
    if (g.N > INT32_MAX || g.K > INT32_MAX) return -1;
    // B staged by TMA (one CTA per SM) when its grid of 1024-column blocks x K slices fills most of the GPU
    {
        const long long cb = (g.N + TT_COLS - 1) / TT_COLS;
        long long sl = ctx->sm_count / cb;
        if (sl > g.K / 128) sl = g.K / 128;
        if (sl > 64) sl = 64;
        if (sl >= 2 && cb * sl * 10 >= (long long)ctx->sm_count * 8) {
            long long k_per = (g.K + sl - 1) / sl;
            k_per = (k_per + 15) / 16 * 16;
            sl = (g.K + k_per - 1) / k_per;
            CUtensorMap mb;
            const int64_t strides[3] = {0, 0, g.b.ld};
            if (sl >= 2 && g.split_ws && (size_t)sl * (size_t)g.M * (size_t)g.N * sizeof(float) <= g.split_ws_bytes &&
                make_bhtc_map(ctx, &mb, g.b.ptr, g.N, g.K, 1, 1, strides, TT_BOX_COLS, TT_KS, CU_TENSOR_MAP_SWIZZLE_NONE)) {
                int& attr = ctx->kernel_state[reinterpret_cast<const void*>(thin_fp32_tma_kernel)];
                if (attr < TT_SMEM_BYTES) {
                    cudaError_t ea = cudaFuncSetAttribute(thin_fp32_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TT_SMEM_BYTES);
                    if (ea != cudaSuccess) return cuda_fail(ea, "cudaFuncSetAttribute(thin_fp32_tma_kernel)");
                    attr = TT_SMEM_BYTES;
                }
                ThinParams p;
                p.a = g.a.ptr; p.lda = g.a.ld;
                p.b = g.b.ptr; p.ldb = g.b.ld;
                p.partial = g.split_ws;
                p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K;
                p.k_per_slice = (int)k_per;
                cudaError_t e = launch_pdl(thin_fp32_tma_kernel, dim3((unsigned)cb, (unsigned)sl), dim3(TT_THREADS), (size_t)TT_SMEM_BYTES, stream,
                                           mb, p, ctx->d_status);
                if (e != cudaSuccess) return cuda_fail(e, "thin_fp32_tma_kernel launch");
                ctx->launches += 1;
                return finish_split(ctx, g, (int)sl, stream);
            }
        }
    }
    const long long col_blocks = (g.N + THIN_COLS - 1) / THIN_COLS;
    // about three CTAs per SM (each keeps 16 KB of B in flight), at least 128 k per slice, at least two slices (the
    // reduction applies the epilogue)
    long long slices = (3LL * ctx->sm_count + col_blocks - 1) / col_blocks;
    if (slices > g.K / 128) slices = g.K / 128;
    if (slices > 64) slices = 64;
    if (slices < 2) return -1;
    long long k_per = (g.K + slices - 1) / slices;
    k_per = (k_per + THIN_UNROLL - 1) / THIN_UNROLL * THIN_UNROLL;
    slices = (g.K + k_per - 1) / k_per;
    if (slices < 2 || col_blocks > INT32_MAX) return -1;
    if (!g.split_ws || (size_t)slices * (size_t)g.M * (size_t)g.N * sizeof(float) > g.split_ws_bytes) return -1;
    ThinParams p;
    p.a = g.a.ptr; p.lda = g.a.ld;
    p.b = g.b.ptr; p.ldb = g.b.ld;
    p.partial = g.split_ws;
    p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K;
    p.k_per_slice = (int)k_per;
    cudaError_t e = launch_pdl(thin_fp32_kernel, dim3((unsigned)col_blocks, (unsigned)slices), dim3(THIN_THREADS), 0, stream, p);
    if (e != cudaSuccess) return cuda_fail(e, "thin_fp32_kernel launch");
    ctx->launches += 1;
    return finish_split(ctx, g, (int)slices, stream);
}

}  // namespace te
