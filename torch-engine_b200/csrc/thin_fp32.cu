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
// Limits: one product (no batch), A with K contiguous, M <= 16, K >= 256, N >= 512; everything else stays on the
// tensor-core path.  B with N contiguous (a row-major right operand) takes the kernels below; B with K contiguous
// (Linear's weight, [N, K]) takes the pair of kernels further down, which run the lanes along k instead.
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

// MR: rows of A a thread accumulates (8 for M <= 8, else 16); the staged A keeps 16-row pitch either way.
template <int MR>
__global__ void __launch_bounds__(THIN_THREADS) thin_fp32_kernel(const ThinParams p) {
    __shared__ __align__(16) float a_sm[THIN_KC][THIN_M];        // [k][m]: the M values of one k are one 64-byte row
    griddep_wait();
    const int t = threadIdx.x;
    const int c0 = blockIdx.x * THIN_COLS + 4 * t;               // this thread's four consecutive columns (N % 4 == 0)
    const bool live = c0 < p.N;
    const int k_begin = blockIdx.y * p.k_per_slice;
    const int k_end = min(k_begin + p.k_per_slice, p.K);
    // accumulators as pairs of rows (m, m + 1): acc[c][q] holds rows 2q and 2q + 1 of column c0 + c
    unsigned long long acc[4][MR / 2];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int q = 0; q < MR / 2; ++q) acc[c][q] = 0ull;       // two +0.0f
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
                for (int q = 0; q < MR / 4; ++q) {
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
    for (int q = 0; q < MR / 2; ++q) {
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

template <int MR>
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
        unsigned long long acc[4][MR / 2];
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int q = 0; q < MR / 2; ++q) acc[c][q] = 0ull;
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
                for (int q = 0; q < MR / 4; ++q) {
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
            for (int q = 0; q < MR / 2; ++q) {
                float lo[4], hi[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) unpack(acc[c][q], lo[c], hi[c]);
                if (2 * q < p.M) *reinterpret_cast<float4*>(out + (long long)(2 * q) * p.N) = make_float4(lo[0], lo[1], lo[2], lo[3]);
                if (2 * q + 1 < p.M) *reinterpret_cast<float4*>(out + (long long)(2 * q + 1) * p.N) = make_float4(hi[0], hi[1], hi[2], hi[3]);
            }
        }
    }
}


// ---- the Linear layout: C[M,N] = X[M,K] . W[N,K]^T, both operands with K contiguous --------------------------------------
// Here a row of W is one column of C, so the lanes of a warp run along k (their loads of a row of W are one contiguous
// 128-byte line) and the sum over k ends with a reduction over the lanes.  A warp task is eight rows of W over one K
// slice: every lane keeps 8 x 16 accumulators (as 64 row pairs (m, m + 1)), reads per step four k (k = base + 32.j + lane)
// of each of the eight rows -- the next step's 32 values are requested before the current ones are used -- and takes
// the sixteen values of X for a k as four 16-byte reads of shared memory, where the CTA has laid its K slice of X out
// as [k][m] with a pitch of 20 floats (consecutive k then fall in distinct bank groups).  Eight rows per task is what
// keeps the shared-memory reads (64 wavefronts per step) under the FMA issue (256 packed FMAs per step).  The task ends
// with a halving exchange over the lanes (128 values -> 4 per lane in 124 shuffles, the same tree for every task) and
// 4 stores per lane into the slice's partial tile; the common reduction adds the slices and applies the epilogue.
constexpr int NT_ROWS = 8;
constexpr int NT_WARPS = 8;
constexpr int NT_THREADS = NT_WARPS * 32;
constexpr int NT_PITCH = 20;                // floats per k of the staged X slice: 16 rows + 4 of padding
constexpr int NT_STEP = 128;                // k per warp step: four per lane
constexpr int NT_KMAX = 2048;               // K slice of X held in shared memory (160 KB)

struct ThinNtParams {
    const float* x; long long ldx;
    const float* w; long long ldw;
    float* partial;                  // [slices][M][N]
    int M, N, K;
    int k_per_slice;                 // multiple of NT_STEP, <= NT_KMAX
    int rows_per_cta;                // multiple of NT_ROWS
};

template <int HALF>
__device__ __forceinline__ void halve_over_lanes(float* v, int off, bool up) {
#pragma unroll
    for (int i = 0; i < HALF; ++i) {
        const float send = up ? v[i] : v[i + HALF];
        const float keep = up ? v[i + HALF] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
}

__device__ __forceinline__ void nt_load_step(float (&w)[NT_ROWS][4], const float* const (&row)[NT_ROWS], int k, int k_end) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int kj = k + 32 * j;
        const bool in = kj < k_end;                 // past the slice the X rows are zero, W is not read
#pragma unroll
        for (int r = 0; r < NT_ROWS; ++r) w[r][j] = in ? __ldg(row[r] + kj) : 0.0f;
    }
}

template <int MP>
__device__ __forceinline__ void nt_fma_step(unsigned long long (&acc)[NT_ROWS][MP], const float (&w)[NT_ROWS][4], const float* x_lane) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const ulonglong2* xr = reinterpret_cast<const ulonglong2*>(x_lane + 32 * j * NT_PITCH);
        ulonglong2 x[MP / 2];                        // rows 0 .. 2 MP - 1 of X at this k, as pairs
#pragma unroll
        for (int q = 0; q < MP / 2; ++q) x[q] = xr[q];
#pragma unroll
        for (int r = 0; r < NT_ROWS; ++r) {
            const unsigned long long wp = pair_of(w[r][j]);
#pragma unroll
            for (int q = 0; q < MP / 2; ++q) {
                fma2(acc[r][2 * q], x[q].x, wp);
                fma2(acc[r][2 * q + 1], x[q].y, wp);
            }
        }
    }
}

// End of a warp task: the lanes' 8 x 2 MP sums are added over the lanes by a halving exchange (the same tree for every
// task), after which lane l holds entries l V / 32 .. of v[r * 2 MP + m], and stored into the slice's partial tile.
template <int MP>
__device__ __forceinline__ void nt_reduce_store(const unsigned long long (&acc)[NT_ROWS][MP], int lane, int n_first, int slice, const ThinNtParams& p) {
    constexpr int V = NT_ROWS * 2 * MP, PER = V / 32;
    float v[V];
#pragma unroll
    for (int r = 0; r < NT_ROWS; ++r)
#pragma unroll
        for (int q = 0; q < MP; ++q) unpack(acc[r][q], v[r * 2 * MP + 2 * q], v[r * 2 * MP + 2 * q + 1]);
    halve_over_lanes<V / 2>(v, 16, lane & 16);
    halve_over_lanes<V / 4>(v, 8, lane & 8);
    halve_over_lanes<V / 8>(v, 4, lane & 4);
    halve_over_lanes<V / 16>(v, 2, lane & 2);
    halve_over_lanes<V / 32>(v, 1, lane & 1);
    const int n = n_first + (lane * PER) / (2 * MP), m0 = (lane * PER) % (2 * MP);
    if (n < p.N) {
        float* out = p.partial + ((long long)slice * p.M + m0) * p.N + n;
#pragma unroll
        for (int j = 0; j < PER; ++j)
            if (m0 + j < p.M) out[(long long)j * p.N] = v[j];
    }
}

// The same stores with zeros: the second partial slot of a task that one CTA computed alone.
template <int MP>
__device__ __forceinline__ void nt_store_zeros(int lane, int n_first, int slot, const ThinNtParams& p) {
    constexpr int PER = NT_ROWS * 2 * MP / 32;
    const int n = n_first + (lane * PER) / (2 * MP), m0 = (lane * PER) % (2 * MP);
    if (n < p.N) {
        float* out = p.partial + ((long long)slot * p.M + m0) * p.N + n;
#pragma unroll
        for (int j = 0; j < PER; ++j)
            if (m0 + j < p.M) out[(long long)j * p.N] = 0.0f;
    }
}

// The CTA's K slice of X, [m][k] in global memory, laid out as [k][m] in shared memory; rows past M and k past the
// slice are zero.  A thread owns every 256th k and has its sixteen loads of a k in flight together.
__device__ __forceinline__ void nt_stage_x(float* x_sm, const ThinNtParams& p, int k_begin, int k_len, int k_pad, int t) {
#pragma unroll 2
    for (int k = t; k < k_pad; k += NT_THREADS) {
        float v[THIN_M];
#pragma unroll
        for (int m = 0; m < THIN_M; ++m) v[m] = (m < p.M && k < k_len) ? __ldg(p.x + (long long)m * p.ldx + k_begin + k) : 0.0f;
        float4* dst = reinterpret_cast<float4*>(x_sm + k * NT_PITCH);
#pragma unroll
        for (int q = 0; q < THIN_M / 4; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    }
}

template <int MP>
__global__ void __launch_bounds__(NT_THREADS, 1) thin_nt_fp32_kernel(const ThinNtParams p) {
    extern __shared__ __align__(16) float nt_x[];               // [k_per_slice][NT_PITCH]
    griddep_launch_dependents();
    griddep_wait();
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int k_begin = blockIdx.y * p.k_per_slice;
    const int k_end = min(k_begin + p.k_per_slice, p.K);
    const int k_len = k_end - k_begin;
    const int k_pad = (k_len + NT_STEP - 1) / NT_STEP * NT_STEP;
    nt_stage_x(nt_x, p, k_begin, k_len, k_pad, t);
    __syncthreads();
    const int row_begin = blockIdx.x * p.rows_per_cta;
    const int row_end = min(row_begin + p.rows_per_cta, p.N);
    const int steps = k_pad / NT_STEP;
    for (int n0 = row_begin + warp * NT_ROWS; n0 < row_end; n0 += NT_WARPS * NT_ROWS) {
        const float* row[NT_ROWS];                               // rows past N read the last row (their sums are not stored)
#pragma unroll
        for (int r = 0; r < NT_ROWS; ++r) row[r] = p.w + (long long)min(n0 + r, p.N - 1) * p.ldw + k_begin + lane;
        unsigned long long acc[NT_ROWS][MP];
#pragma unroll
        for (int r = 0; r < NT_ROWS; ++r)
#pragma unroll
            for (int q = 0; q < MP; ++q) acc[r][q] = 0ull;
        float wa[NT_ROWS][4], wb[NT_ROWS][4];
        const float* x_lane = nt_x + lane * NT_PITCH;
        nt_load_step(wa, row, 0, k_len - lane);                  // "k < k_len - lane" is "k + lane < k_len"
        for (int s = 0; s < steps; s += 2) {
            if (s + 1 < steps) nt_load_step(wb, row, (s + 1) * NT_STEP, k_len - lane);
            nt_fma_step(acc, wa, x_lane + s * NT_STEP * NT_PITCH);
            if (s + 1 < steps) {
                if (s + 2 < steps) nt_load_step(wa, row, (s + 2) * NT_STEP, k_len - lane);
                nt_fma_step(acc, wb, x_lane + (s + 1) * NT_STEP * NT_PITCH);
            }
        }
        nt_reduce_store<MP>(acc, lane, n0, blockIdx.y, p);
    }
}


// The same warp task with W staged by TMA: 64-row x 128-k tiles of W (the eight tasks of the CTA's eight warps, one
// step) land in a ring of four 32 KB stages, so the bytes in flight cost no registers, and the warps read their values
// of W back from shared memory (lanes along k: conflict-free).  There is no producer warp -- a ninth warp would cap
// the kernel at 168 registers, under what 128 accumulators need: lane 0 of warp 0 refills a stage one step after the
// warps took its tile into registers (three tiles stay in flight).  One CTA per SM; a CTA takes a contiguous range of
// the (K slice, 64-row group) list, slice-major, and restages its slice of X when the range crosses into the next
// slice.  Needs W on 16-byte boundaries (pointer and leading dimension).
constexpr int NTT_THREADS = NT_THREADS;
constexpr int NTT_GROUP = NT_WARPS * NT_ROWS;                 // 64 rows of W per stage
constexpr int NTT_STAGE_BYTES = NTT_GROUP * NT_STEP * 4;      // 32 KB
constexpr int NTT_STAGES = 4;
constexpr int NTT_KMAX = 1024;                                // K slice of X held in shared memory (80 KB)
constexpr int NTT_SMEM_BYTES = 128 + NTT_STAGES * NTT_STAGE_BYTES + NTT_KMAX * NT_PITCH * 4 + 16 * NTT_STAGES + 16;

struct ThinNtTmaParams {
    ThinNtParams q;                  // rows_per_cta unused
    int slices, groups;              // K slices, 64-row groups of W
};

// Walks the tiles of a CTA's task range in the order they are consumed.
struct NtTileCursor {
    int t, s, steps, k_begin, grp;
    __device__ __forceinline__ void open(const ThinNtTmaParams& pp, int task) {
        t = task; s = 0;
        const int slice = t / pp.groups;
        grp = t - slice * pp.groups;
        k_begin = slice * pp.q.k_per_slice;
        steps = (min(pp.q.k_per_slice, pp.q.K - k_begin) + NT_STEP - 1) / NT_STEP;
    }
    __device__ __forceinline__ void next(const ThinNtTmaParams& pp, int t_end) {
        if (++s == steps && t + 1 < t_end) open(pp, t + 1);
    }
};

template <int MP>
__global__ void __launch_bounds__(NTT_THREADS, 1) thin_nt_tma_kernel(const __grid_constant__ CUtensorMap tm_w, const ThinNtTmaParams pp, int* status) {
    extern __shared__ uint8_t ntt_smem[];
    const ThinNtParams& p = pp.q;
    const uint32_t raw = smem_u32(ntt_smem);
    const uint32_t ring = (raw + 127u) & ~127u;
    const uint32_t x_addr = ring + NTT_STAGES * NTT_STAGE_BYTES;
    float* x_sm = reinterpret_cast<float*>(ntt_smem + (x_addr - raw));
    const uint32_t bar_full = x_addr + NTT_KMAX * NT_PITCH * 4;
    const uint32_t bar_empty = bar_full + 8 * NTT_STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(ntt_smem + (bar_empty + 8 * NTT_STAGES - raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool feeder = threadIdx.x == 0;
    if (feeder) {
        for (int s = 0; s < NTT_STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, NT_WARPS);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tm_w);
    }
    __syncthreads();
    griddep_launch_dependents();
    griddep_wait();
    const long long tasks = (long long)pp.slices * pp.groups;
    const int t_begin = (int)(tasks * blockIdx.x / gridDim.x), t_end = (int)(tasks * (blockIdx.x + 1) / gridDim.x);
    if (t_begin >= t_end) return;
    // the feeder's view: tiles of this CTA in consumption order, `fed` of `tiles` issued so far
    NtTileCursor cur;
    int tiles = 0, fed = 0;
    if (feeder) {
        for (int t = t_begin; t < t_end; ++t) {
            cur.open(pp, t);
            tiles += cur.steps;
        }
        cur.open(pp, t_begin);
        for (; fed < NTT_STAGES && fed < tiles; ++fed) {          // k past K and rows past N arrive as zeros
            mbar_arrive_expect_tx(bar_full + 8 * fed, NTT_STAGE_BYTES);
            tma_load_4d(ring + fed * NTT_STAGE_BYTES, &tm_w, bar_full + 8 * fed, cur.k_begin + cur.s * NT_STEP, cur.grp * NTT_GROUP, 0, 0);
            cur.next(pp, t_end);
        }
    }
    const float* x_lane = x_sm + lane * NT_PITCH;
    const uint32_t w_off = (uint32_t)(warp * NT_ROWS) * (NT_STEP * 4) + (uint32_t)lane * 4;
    int cur_slice = -1, i = 0;
    // A warp whose wait ran out keeps walking the task list for the two barriers around every restaging of X (the
    // other warps count on all 256 threads there) and does nothing else.
    bool ok = true;
    for (int t = t_begin; t < t_end; ++t) {
        const int slice = t / pp.groups, grp = t - slice * pp.groups;
        const int k_begin = slice * p.k_per_slice;
        const int k_len = min(p.k_per_slice, p.K - k_begin);
        const int steps = (k_len + NT_STEP - 1) / NT_STEP;
        if (slice != cur_slice) {
            cur_slice = slice;
            __syncthreads();
            if (ok) nt_stage_x(x_sm, p, k_begin, k_len, steps * NT_STEP, threadIdx.x);
            __syncthreads();
        }
        if (!ok) continue;
        unsigned long long acc[NT_ROWS][MP];
#pragma unroll
        for (int r = 0; r < NT_ROWS; ++r)
#pragma unroll
            for (int q = 0; q < MP; ++q) acc[r][q] = 0ull;
        for (int s = 0; s < steps; ++s, ++i) {
            const int st = i % NTT_STAGES;
            bool mine = wait_bounded(bar_full + 8 * st, (i / NTT_STAGES) & 1, abort_flag, status, WAIT_THIN_FULL);
            const uint32_t wt = ring + st * NTT_STAGE_BYTES + w_off;
            float w[NT_ROWS][4];                                         // the warp's share of the tile, then release it
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int r = 0; r < NT_ROWS; ++r) w[r][j] = ld_shared_f32(wt + r * (NT_STEP * 4) + j * 128);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * st);
            if (feeder && i >= 1 && fed < tiles) {                       // refill the stage of the previous step
                const int sp = (i - 1) % NTT_STAGES;
                mine = mine && wait_bounded(bar_empty + 8 * sp, ((i - 1) / NTT_STAGES) & 1, abort_flag, status, WAIT_THIN_EMPTY);
                if (mine) {
                    mbar_arrive_expect_tx(bar_full + 8 * sp, NTT_STAGE_BYTES);
                    tma_load_4d(ring + sp * NTT_STAGE_BYTES, &tm_w, bar_full + 8 * sp, cur.k_begin + cur.s * NT_STEP, cur.grp * NTT_GROUP, 0, 0);
                    cur.next(pp, t_end);
                    ++fed;
                }
            }
            ok = __all_sync(0xffffffffu, mine);
            if (!ok) break;
            nt_fma_step<MP>(acc, w, x_lane + s * NT_STEP * NT_PITCH);
        }
        if (!ok) continue;
        nt_reduce_store<MP>(acc, lane, grp * NTT_GROUP + warp * NT_ROWS, slice, p);
    }
    if (feeder && *abort_flag) {      // copies already issued still write shared memory: let them land
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {
        }
    }
}


// For large W the ring is what limits the rate (three 32 KB tiles in flight per SM against the latency of a loaded
// HBM), and the 80 KB slice of X is what limits the ring.  This form takes X out of the way: a small kernel first
// writes X transposed, [k][20] (16 rows + 4 floats of padding, the shared-memory pitch), and the tile of X for a
// step then arrives by TMA together with the tile of W (10 KB beside 32 KB).  Five stages, no CTA-wide staging, and
// the K slices can be as long as the balance over the SMs allows, so fewer reductions over the lanes.  Costs one
// more launch; used when W is large.
constexpr int NTX_STAGES = 5;
constexpr int NTX_W_BYTES = NTT_GROUP * NT_STEP * 4;          // 32 KB
constexpr int NTX_X_BYTES = NT_STEP * NT_PITCH * 4;           // 10 KB
constexpr int NTX_STAGE_BYTES = NTX_W_BYTES + NTX_X_BYTES;
constexpr int NTX_SMEM_BYTES = 128 + NTX_STAGES * NTX_STAGE_BYTES + 16 * NTX_STAGES + 16;

__global__ void __launch_bounds__(256) thin_nt_transpose_x_kernel(const float* __restrict__ x, long long ldx, int M, int K, float* __restrict__ xt) {
    griddep_launch_dependents();
    griddep_wait();
    const int k = blockIdx.x * 256 + threadIdx.x;
    if (k >= K) return;
    float v[THIN_M];
#pragma unroll
    for (int m = 0; m < THIN_M; ++m) v[m] = m < M ? __ldg(x + (long long)m * ldx + k) : 0.0f;
    float4* dst = reinterpret_cast<float4*>(xt + (long long)k * NT_PITCH);
#pragma unroll
    for (int q = 0; q < THIN_M / 4; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    dst[THIN_M / 4] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// The tile list of the product: K slices outermost, then 64-row groups of W, then the steps of a slice (the last
// slice may be shorter).  A CTA takes a contiguous range of it, cut at tile granularity so that every SM gets the same
// number of steps; a task cut by a range boundary is finished by the next CTA, and its two parts go to two partial
// slots (slot 2.slice for the CTA that began the task, 2.slice + 1 for the one that continued it -- zeros when one CTA
// did it all), which the common reduction adds in slot order.  The launcher keeps a task no longer than a range, so
// no task has three parts.
struct NtxParams {
    ThinNtParams q;                  // k_per_slice = 128 * steps_full; rows_per_cta unused
    int groups, slices, steps_full, steps_last;
    long long tiles_full;            // groups * steps_full * (slices - 1)
    long long tiles;
};

struct NtxCursor {
    int slice, grp, s, steps;
    __device__ __forceinline__ void open(const NtxParams& pp, long long g) {
        if (g < pp.tiles_full) {
            const long long per = (long long)pp.groups * pp.steps_full;
            slice = (int)(g / per);
            const int r = (int)(g - slice * per);
            grp = r / pp.steps_full; s = r - grp * pp.steps_full; steps = pp.steps_full;
        } else {
            const int r = (int)(g - pp.tiles_full);
            slice = pp.slices - 1;
            grp = r / pp.steps_last; s = r - grp * pp.steps_last; steps = pp.steps_last;
        }
    }
    __device__ __forceinline__ void next(const NtxParams& pp) {
        if (++s < steps) return;
        s = 0;
        if (++grp < pp.groups) return;
        grp = 0;
        ++slice;
        steps = slice == pp.slices - 1 ? pp.steps_last : pp.steps_full;
    }
};

template <int MP>
__global__ void __launch_bounds__(NTT_THREADS, 1) thin_nt_tma_xt_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                                                                          const NtxParams pp, int* status) {
    extern __shared__ uint8_t ntx_smem[];
    const ThinNtParams& p = pp.q;
    const uint32_t raw = smem_u32(ntx_smem);
    const uint32_t ring = (raw + 127u) & ~127u;
    const uint32_t bar_full = ring + NTX_STAGES * NTX_STAGE_BYTES;
    const uint32_t bar_empty = bar_full + 8 * NTX_STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(ntx_smem + (bar_empty + 8 * NTX_STAGES - raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool feeder = threadIdx.x == 0;
    if (feeder) {
        for (int s = 0; s < NTX_STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, NT_WARPS);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tm_w);
        tma_prefetch_desc(&tm_x);
    }
    __syncthreads();
    griddep_launch_dependents();
    griddep_wait();
    const long long g_begin = pp.tiles * blockIdx.x / gridDim.x, g_end = pp.tiles * (blockIdx.x + 1) / gridDim.x;
    const int tiles = (int)(g_end - g_begin);
    if (tiles <= 0) return;
    NtxCursor feed = {}, cc;
    int fed = 0;
    // one tile of W (k past K and rows past N arrive as zeros) and the same k of the transposed X into a stage
    auto feed_stage = [&](int st) {
        const uint32_t dst = ring + st * NTX_STAGE_BYTES, bar = bar_full + 8 * st;
        const int k = feed.slice * p.k_per_slice + feed.s * NT_STEP;
        mbar_arrive_expect_tx(bar, NTX_STAGE_BYTES);
        tma_load_4d(dst, &tm_w, bar, k, feed.grp * NTT_GROUP, 0, 0);
        tma_load_4d(dst + NTX_W_BYTES, &tm_x, bar, 0, k, 0, 0);
        feed.next(pp);
        ++fed;
    };
    if (feeder) {
        feed.open(pp, g_begin);
        while (fed < NTX_STAGES && fed < tiles) feed_stage(fed);
    }
    const uint32_t w_off = (uint32_t)(warp * NT_ROWS) * (NT_STEP * 4) + (uint32_t)lane * 4;
    const uint8_t* x_lane0 = ntx_smem + (ring - raw) + NTX_W_BYTES + lane * (NT_PITCH * 4);
    cc.open(pp, g_begin);
    bool began_here = cc.s == 0;             // the task under way was begun by this CTA
    unsigned long long acc[NT_ROWS][MP];
#pragma unroll
    for (int r = 0; r < NT_ROWS; ++r)
#pragma unroll
        for (int q = 0; q < MP; ++q) acc[r][q] = 0ull;
    for (int i = 0; i < tiles; ++i) {
        const int st = i % NTX_STAGES;
        const bool mine = wait_bounded(bar_full + 8 * st, (i / NTX_STAGES) & 1, abort_flag, status, WAIT_THIN_FULL);
        if (!__all_sync(0xffffffffu, mine)) break;
        const uint32_t wt = ring + st * NTX_STAGE_BYTES + w_off;
        float w[NT_ROWS][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int r = 0; r < NT_ROWS; ++r) w[r][j] = ld_shared_f32(wt + r * (NT_STEP * 4) + j * 128);
        if (feeder && i >= 1 && fed < tiles) {                       // refill the stage of the previous step
            const int sp = (i - 1) % NTX_STAGES;
            if (wait_bounded(bar_empty + 8 * sp, ((i - 1) / NTX_STAGES) & 1, abort_flag, status, WAIT_THIN_EMPTY)) feed_stage(sp);
        }
        nt_fma_step<MP>(acc, w, reinterpret_cast<const float*>(x_lane0 + st * NTX_STAGE_BYTES));
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * st);              // W and X of the stage have been read
        const bool task_ends = cc.s + 1 == cc.steps;
        if (task_ends || i + 1 == tiles) {
            const int n_first = cc.grp * NTT_GROUP + warp * NT_ROWS;
            nt_reduce_store<MP>(acc, lane, n_first, 2 * cc.slice + (began_here ? 0 : 1), p);
            if (task_ends && began_here) nt_store_zeros<MP>(lane, n_first, 2 * cc.slice + 1, p);
            began_here = true;
#pragma unroll
            for (int r = 0; r < NT_ROWS; ++r)
#pragma unroll
                for (int q = 0; q < MP; ++q) acc[r][q] = 0ull;
        }
        cc.next(pp);
    }
    if (feeder && *abort_flag) {      // copies already issued still write shared memory: let them land
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {
        }
    }
}

}  // namespace

// The Linear layout (W as [N, K]): a grid of row blocks x K slices of one CTA per SM.
// MP: row pairs of X the kernels accumulate (4 for M <= 8, 8 for M <= 16).
template <int MP>
static int launch_thin_nt_mp(te_b200_ctx* ctx, const GemmProblem& g, cudaStream_t stream) {
    if (g.N > INT32_MAX || g.K > INT32_MAX || !g.split_ws) return -1;
    // large W with 16-byte rows: X transposed by a small kernel, tiles of W and X by TMA, ranges of the tile list cut
    // at tile granularity (see thin_nt_tma_xt_kernel)
    if ((double)g.N * (double)g.K >= 8.0e6 && g.K >= 1024) {
        const long long groups = (g.N + NTT_GROUP - 1) / NTT_GROUP;
        const long long steps_total = (g.K + NT_STEP - 1) / NT_STEP;
        const long long total = groups * steps_total;
        const long long grid = total < ctx->sm_count ? total : ctx->sm_count;
        // the fewest K slices whose tasks are no longer than a CTA's range (then a task has at most two parts)
        long long sl = 0, steps_full = 0;
        for (long long c = 1; c <= 16 && !sl; ++c) {
            const long long sf = (steps_total + c - 1) / c;
            if (sf <= total / grid && (steps_total + sf - 1) / sf == c) { sl = c; steps_full = sf; }
        }
        const size_t partial_bytes = ((size_t)(2 * sl) * (size_t)g.M * (size_t)g.N * sizeof(float) + 255) & ~size_t(255);
        const size_t xt_bytes = (size_t)g.K * NT_PITCH * sizeof(float);
        CUtensorMap mw, mx;
        const int64_t w_strides[3] = {0, 0, g.b.ld}, x_strides[3] = {0, 0, NT_PITCH};
        float* xt = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(g.split_ws) + partial_bytes);
        if (sl && total <= INT32_MAX && partial_bytes + xt_bytes <= g.split_ws_bytes && !(reinterpret_cast<uintptr_t>(g.split_ws) & 15) &&
            make_bhtc_map(ctx, &mw, g.b.ptr, g.K, g.N, 1, 1, w_strides, NT_STEP, NTT_GROUP, CU_TENSOR_MAP_SWIZZLE_NONE) &&
            make_bhtc_map(ctx, &mx, xt, NT_PITCH, g.K, 1, 1, x_strides, NT_PITCH, NT_STEP, CU_TENSOR_MAP_SWIZZLE_NONE)) {
            int& attr = ctx->kernel_state[reinterpret_cast<const void*>(thin_nt_tma_xt_kernel<MP>)];
            if (attr < NTX_SMEM_BYTES) {
                cudaError_t ea = cudaFuncSetAttribute(thin_nt_tma_xt_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, NTX_SMEM_BYTES);
                if (ea != cudaSuccess) return cuda_fail(ea, "cudaFuncSetAttribute(thin_nt_tma_xt_kernel)");
                attr = NTX_SMEM_BYTES;
            }
            cudaError_t e = launch_pdl(thin_nt_transpose_x_kernel, dim3((unsigned)((g.K + 255) / 256)), dim3(256), (size_t)0, stream,
                                       g.a.ptr, (long long)g.a.ld, (int)g.M, (int)g.K, xt);
            if (e != cudaSuccess) return cuda_fail(e, "thin_nt_transpose_x_kernel launch");
            NtxParams pp;
            pp.q.x = g.a.ptr; pp.q.ldx = g.a.ld;
            pp.q.w = g.b.ptr; pp.q.ldw = g.b.ld;
            pp.q.partial = g.split_ws;
            pp.q.M = (int)g.M; pp.q.N = (int)g.N; pp.q.K = (int)g.K;
            pp.q.k_per_slice = (int)(steps_full * NT_STEP);
            pp.q.rows_per_cta = 0;
            pp.groups = (int)groups; pp.slices = (int)sl;
            pp.steps_full = (int)steps_full;
            pp.steps_last = (int)(steps_total - steps_full * (sl - 1));
            pp.tiles_full = groups * steps_full * (sl - 1);
            pp.tiles = total;
            e = launch_pdl(thin_nt_tma_xt_kernel<MP>, dim3((unsigned)grid), dim3(NTT_THREADS), (size_t)NTX_SMEM_BYTES, stream, mw, mx, pp, ctx->d_status);
            if (e != cudaSuccess) return cuda_fail(e, "thin_nt_tma_xt_kernel launch");
            ctx->launches += 2;
            return finish_split(ctx, g, (int)(2 * sl), stream);
        }
    }
    // W staged by TMA (one CTA per SM over the list of K slices x 64-row groups) when that list fills most of the GPU
    {
        long long sl = (g.K + NTT_KMAX - 1) / NTT_KMAX;
        if (sl < 2) sl = 2;
        const long long k_per = ((g.K + sl - 1) / sl + NT_STEP - 1) / NT_STEP * NT_STEP;
        sl = (g.K + k_per - 1) / k_per;
        const long long groups = (g.N + NTT_GROUP - 1) / NTT_GROUP;
        const long long tasks = sl * groups;
        CUtensorMap mw;
        const int64_t strides[3] = {0, 0, g.b.ld};
        if (sl >= 2 && sl <= 64 && tasks * 10 >= (long long)ctx->sm_count * 8 && tasks <= INT32_MAX &&
            (size_t)sl * (size_t)g.M * (size_t)g.N * sizeof(float) <= g.split_ws_bytes &&
            make_bhtc_map(ctx, &mw, g.b.ptr, g.K, g.N, 1, 1, strides, NT_STEP, NTT_GROUP, CU_TENSOR_MAP_SWIZZLE_NONE)) {
            int& attr = ctx->kernel_state[reinterpret_cast<const void*>(thin_nt_tma_kernel<MP>)];
            if (attr < NTT_SMEM_BYTES) {
                cudaError_t ea = cudaFuncSetAttribute(thin_nt_tma_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, NTT_SMEM_BYTES);
                if (ea != cudaSuccess) return cuda_fail(ea, "cudaFuncSetAttribute(thin_nt_tma_kernel)");
                attr = NTT_SMEM_BYTES;
            }
            ThinNtTmaParams pp;
            pp.q.x = g.a.ptr; pp.q.ldx = g.a.ld;
            pp.q.w = g.b.ptr; pp.q.ldw = g.b.ld;
            pp.q.partial = g.split_ws;
            pp.q.M = (int)g.M; pp.q.N = (int)g.N; pp.q.K = (int)g.K;
            pp.q.k_per_slice = (int)k_per;
            pp.q.rows_per_cta = 0;
            pp.slices = (int)sl; pp.groups = (int)groups;
            const unsigned grid = (unsigned)(tasks < ctx->sm_count ? tasks : ctx->sm_count);
            cudaError_t e = launch_pdl(thin_nt_tma_kernel<MP>, dim3(grid), dim3(NTT_THREADS), (size_t)NTT_SMEM_BYTES, stream, mw, pp, ctx->d_status);
            if (e != cudaSuccess) return cuda_fail(e, "thin_nt_tma_kernel launch");
            ctx->launches += 1;
            return finish_split(ctx, g, (int)sl, stream);
        }
    }
    // slices of at most NT_KMAX k, at least two (the reduction applies the epilogue); row blocks fill the SMs
    long long slices = (g.K + NT_KMAX - 1) / NT_KMAX;
    if (slices < 2) slices = 2;
    long long k_per = ((g.K + slices - 1) / slices + NT_STEP - 1) / NT_STEP * NT_STEP;
    slices = (g.K + k_per - 1) / k_per;
    if (slices < 2 || slices > 64) return -1;
    long long row_blocks = ctx->sm_count / slices;
    if (row_blocks < 1) row_blocks = 1;
    const long long task_rows = NT_WARPS * NT_ROWS;
    long long rows_per = ((g.N + row_blocks - 1) / row_blocks + task_rows - 1) / task_rows * task_rows;
    row_blocks = (g.N + rows_per - 1) / rows_per;
    if ((size_t)slices * (size_t)g.M * (size_t)g.N * sizeof(float) > g.split_ws_bytes) return -1;
    const int smem = (int)(k_per * NT_PITCH * sizeof(float));
    int& attr = ctx->kernel_state[reinterpret_cast<const void*>(thin_nt_fp32_kernel<MP>)];
    if (attr < smem) {
        cudaError_t ea = cudaFuncSetAttribute(thin_nt_fp32_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, NT_KMAX * NT_PITCH * (int)sizeof(float));
        if (ea != cudaSuccess) return cuda_fail(ea, "cudaFuncSetAttribute(thin_nt_fp32_kernel)");
        attr = NT_KMAX * NT_PITCH * (int)sizeof(float);
    }
    ThinNtParams p;
    p.x = g.a.ptr; p.ldx = g.a.ld;
    p.w = g.b.ptr; p.ldw = g.b.ld;
    p.partial = g.split_ws;
    p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K;
    p.k_per_slice = (int)k_per;
    p.rows_per_cta = (int)rows_per;
    cudaError_t e = launch_pdl(thin_nt_fp32_kernel<MP>, dim3((unsigned)row_blocks, (unsigned)slices), dim3(NT_THREADS), (size_t)smem, stream, p);
    if (e != cudaSuccess) return cuda_fail(e, "thin_nt_fp32_kernel launch");
    ctx->launches += 1;
    return finish_split(ctx, g, (int)slices, stream);
}

static int launch_thin_nt(te_b200_ctx* ctx, const GemmProblem& g, cudaStream_t stream) {
    return g.M <= 8 ? launch_thin_nt_mp<4>(ctx, g, stream) : launch_thin_nt_mp<8>(ctx, g, stream);
}

// The row-major right operand (B as [K, N]).
template <int MR>
static int launch_thin_nn(te_b200_ctx* ctx, const GemmProblem& g, cudaStream_t stream) {
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
                int& attr = ctx->kernel_state[reinterpret_cast<const void*>(thin_fp32_tma_kernel<MR>)];
                if (attr < TT_SMEM_BYTES) {
                    cudaError_t ea = cudaFuncSetAttribute(thin_fp32_tma_kernel<MR>, cudaFuncAttributeMaxDynamicSharedMemorySize, TT_SMEM_BYTES);
                    if (ea != cudaSuccess) return cuda_fail(ea, "cudaFuncSetAttribute(thin_fp32_tma_kernel)");
                    attr = TT_SMEM_BYTES;
                }
                ThinParams p;
                p.a = g.a.ptr; p.lda = g.a.ld;
                p.b = g.b.ptr; p.ldb = g.b.ld;
                p.partial = g.split_ws;
                p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K;
                p.k_per_slice = (int)k_per;
                cudaError_t e = launch_pdl(thin_fp32_tma_kernel<MR>, dim3((unsigned)cb, (unsigned)sl), dim3(TT_THREADS), (size_t)TT_SMEM_BYTES, stream,
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
    cudaError_t e = launch_pdl(thin_fp32_kernel<MR>, dim3((unsigned)col_blocks, (unsigned)slices), dim3(THIN_THREADS), 0, stream, p);
    if (e != cudaSuccess) return cuda_fail(e, "thin_fp32_kernel launch");
    ctx->launches += 1;
    return finish_split(ctx, g, (int)slices, stream);
}

// Returns TE_OK when the product was issued here, -1 when it is outside this form's limits (the caller then takes the
// tensor-core path), or an error status.
int launch_thin_fp32(te_b200_ctx* ctx, const GemmProblem& g, cudaStream_t stream) {
    if (g.batch_inner * g.batch_outer != 1 || g.M < 1 || g.M > THIN_M || g.K < 256 || g.N < 512) return -1;
    if (g.a.mn_major || g.preact) return -1;
    if (!g.b.mn_major) return launch_thin_nt(ctx, g, stream);
    return g.M <= 8 ? launch_thin_nn<8>(ctx, g, stream) : launch_thin_nn<16>(ctx, g, stream);
}

}  // namespace te
