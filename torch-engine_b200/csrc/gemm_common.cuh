// Device-side pieces shared by the GEMM kernels (single-CTA and CTA-pair forms): tile constants, kernel
// parameters, the bounded mbarrier wait, the tile raster and the fused epilogue.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"
#include "te_internal.h"

namespace te {

constexpr int BM = 128;
constexpr int BK = 32;                       // floats per k-block = one 128-byte swizzle row
constexpr int UMMA_K = 8;                    // tf32 K per tcgen05.mma
constexpr int A_PLANE_BYTES = BM * BK * 4;   // 16 KiB
constexpr int SMEM_RING_BUDGET = 192 * 1024;
constexpr int SMEM_AUX_BYTES = 512;          // mbarriers, TMEM slot, abort flag
constexpr int GROUP_M = 16;                  // raster: tiles advance down 16 m-blocks, then one n-block over
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;   // default limit of a bounded wait; a context may set another
// Warp roles: warps 0-7 drain accumulators (warp w reads TMEM lanes 32*(w%4).., columns of half w/4),
// warp 8 issues TMA loads, warp 9 allocates TMEM and issues MMAs.
constexpr int EPI_WARPS = 8;
constexpr int PRODUCER_WARP = 8;
constexpr int MMA_WARP = 9;
constexpr int CTA_THREADS = 320;
constexpr int CONVERTER_THREADS = 128;       // warps 10-13 of the kernels that split fp32 into tf32 hi/lo in shared memory

enum : int {  // where a bounded wait gave up (stored in the device status word)
    WAIT_PRODUCER_EMPTY = 101,
    WAIT_MMA_FULL = 102,
    WAIT_MMA_TMEM_EMPTY = 103,
    WAIT_EPI_TMEM_FULL = 104,
    WAIT_TEARDOWN = 105,
    WAIT_CONVERTER_FULL = 106,
    WAIT_THIN_FULL = 107,        // thin FP32 product: a consumer warp waiting for a stage of B
    WAIT_THIN_EMPTY = 108        // ... its producer waiting for a stage to be released
};

// How an epilogue thread's 32 consecutive columns of one row reach global memory.
//   STORE_DIRECT  16-byte or scalar stores: any leading dimension, alignment and ragged N;
//   STORE_TMA     the warp's 32 x 32 block is staged in shared memory and leaves as one TMA tensor store;
//   STORE_SECTOR  each thread writes its row piece with 32-byte stores (st.global.v8.f32), one whole L2 sector per
//                 store: no shared-memory staging, no proxy fence, no wait for a staging tile to drain.  Needs 32-byte
//                 aligned rows (base, ldc and batch strides multiples of 8 floats) and N a multiple of 8.
enum : int { STORE_DIRECT = 0, STORE_TMA = 1, STORE_SECTOR = 2 };

// Epilogue forms a GEMM kernel is compiled for.  The bare product (EPI_PLAIN) and the residual form are separate
// instances because epilogue code that is present but not taken still costs registers and drain time on products
// whose epilogue is not hidden behind a long main loop.
enum : int { EPI_GENERAL = 0, EPI_PLAIN = 1, EPI_RESIDUAL = 2 };

struct GemmParams {
    int M, N, K;
    int tiles_m, tiles_n;
    int batch_inner, num_batches;
    int a_mul_inner, a_mul_outer, b_mul_inner, b_mul_outer;  // 0 = broadcast, 1 = indexed
    long long ldc, c_stride_inner, c_stride_outer;
    float* c;
    float* preact;
    const float* bias;
    const float* residual;   // optional, same layout as c: added last (may alias c: accumulation)
    float alpha;
    int scale_mode;
    int epilogue;
    int* status;
    int tma_store;   // how outputs leave: STORE_DIRECT (any layout), STORE_TMA (staged in shared memory), STORE_SECTOR
    // Split K: every output tile is computed by k_splits work units, each over kb_per_split k-blocks, each writing
    // its partial tile to slice `split` of a scratch buffer (split_stride elements apart); a reduction kernel adds
    // the slices in order and applies the epilogue.  k_splits == 1: no scratch, kb_per_split = all k-blocks.
    int k_splits, kb_per_split;
    int batch_outer_n;          // number of outer batches (coordinate base of the split in the output tensor map)
    long long split_stride;
};

struct WorkUnit {
    int batch, m_blk, n_blk, split, kb0, kb1;
};


template <int BN, int NPL>
struct TileCfg {
    static constexpr int B_PLANE_BYTES = BN * BK * 4;
    static constexpr int STAGE_BYTES = NPL * (A_PLANE_BYTES + B_PLANE_BYTES);
    static constexpr int STAGES = SMEM_RING_BUDGET / STAGE_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;  // two accumulator buffers of BN fp32 columns
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 8 * 32 * 128 + SMEM_AUX_BYTES + 1024;  // ring + 8 epilogue staging tiles + barriers + alignment slack
    static_assert(STAGES >= 2, "need at least a double buffer");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
    static_assert(TMEM_COLS >= 32 && TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM columns");
};

// round-to-nearest (ties away) fp32 -> tf32, low 13 mantissa bits cleared: exactly representable on the tensor core
__device__ __forceinline__ float to_tf32_rn(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u & 0xFFFFE000u);
}

// The same rounding with integer instructions: half a tf32 ulp added to the magnitude bits, low 13 bits cleared.
// Equal to to_tf32_rn for every finite input and for infinity; a NaN may come out as another NaN or, with a mantissa
// of all ones, as zero, so this form is for values whose NaN case is already decided elsewhere (the lo part
// x - hi of a hi / lo split: a NaN x makes hi a NaN, and the product with it).  It keeps the conversion unit, which
// issues a quarter as many lanes per clock as the integer unit, free for the hi parts.
__device__ __forceinline__ float to_tf32_rn_finite(float x) {
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
}

__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                             int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    // The limit lives next to the status word (bytes 8..15 of the status area); 0 means the default.  Only this slow
    // path reads it.
    const uint64_t set_limit = *reinterpret_cast<const volatile unsigned long long*>(status + 2);
    const uint64_t limit = set_limit ? set_limit : WAIT_LIMIT_NS;
    uint32_t polls = 0;
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++polls & 0x3F) == 0) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > limit) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tile_coords(int t, const GemmParams& p, int& batch, int& m_blk, int& n_blk) {
    const int per_batch = p.tiles_m * p.tiles_n;
    batch = t / per_batch;
    const int r = t - batch * per_batch;
    const int group_span = GROUP_M * p.tiles_n;
    const int g = r / group_span;
    const int first_m = g * GROUP_M;
    const int gm = min(p.tiles_m - first_m, GROUP_M);
    const int in_group = r - g * group_span;
    m_blk = first_m + in_group % gm;
    n_blk = in_group / gm;
}

__device__ __forceinline__ void decode_unit(int u, const GemmParams& p, int kblocks, WorkUnit& w) {
    const int t = u / p.k_splits;
    w.split = u - t * p.k_splits;
    tile_coords(t, p, w.batch, w.m_blk, w.n_blk);
    w.kb0 = w.split * p.kb_per_split;
    w.kb1 = min(w.kb0 + p.kb_per_split, kblocks);
}

__device__ __forceinline__ float gelu_tanh(float x) {
    // Same function as gelu_forward_kernel (reference src/cuda/elementwise_cuda.cu:2701-2707), 0.5 x (1 + tanh(z)) with
    // z = 0.79788456 (x + 0.044715 x^3).  Since 0.5 (1 + tanh(z)) = 1 / (1 + exp(-2z)), one fast exponential and one
    // fast division do it (absolute error ~1e-7; the epilogue evaluates this for every output element, so it has to
    // stay cheaper than the main loop).
    const float u = x * x;
    const float m2z = x * fmaf(u, -2.0f * 0.7978845608f * 0.044715f, -2.0f * 0.7978845608f);    // -2z
    return __fdividef(x, 1.0f + __expf(m2z));
}

constexpr int EPI_STAGE_BYTES = 32 * 128;   // one warp's staging tile: 32 rows x 32 floats, 128-byte swizzled

struct EpilogueRow {
    float* c_row;      // start of this thread's output row
    float* pre_row;    // same row of the optional pre-activation output
    const float* res_row;   // same row of the optional residual input
    bool row_ok;       // row < M
    bool vec_ok;       // 16-byte stores are legal
    bool sector_ok;    // STORE_SECTOR: 32-byte stores straight from registers
    // TMA-store path (used when the output can be described by a tensor map)
    bool tma_ok;
    uint32_t stage;            // this warp's staging tile in shared memory
    const CUtensorMap* tm_c;
    const CUtensorMap* tm_pre;
    int row0;                  // first of the 32 rows this warp owns
    int bi, bo;                // batch coordinates
};

// The warp's 32 x 32 block goes through shared memory so that global memory is written in whole 128-byte lines by
// the TMA unit instead of 32 scattered 16-byte pieces per store instruction.  Lane 0 owns the bulk group.
// With `alternate` the caller switches between two staging tiles (er.stage and er.stage + EPI_STAGE_BYTES, chosen by
// `which`), so only the store before the previous one has to have drained.
// With `add` the tile is added onto what global memory holds (cp.reduce.async.bulk) instead of replacing it.
__device__ __forceinline__ void stage_and_store32(const float* v, int col0, const EpilogueRow& er, const CUtensorMap* tm,
                                                  int lane, bool alternate = false, int which = 0, bool add = false) {
    if (lane == 0) {
        if (alternate) bulk_wait_read_all_but_one();
        else bulk_wait_read_all();           // the previous store has finished reading the staging tile
    }
    __syncwarp();
    const uint32_t stage = er.stage + (alternate ? which * EPI_STAGE_BYTES : 0);
    const uint32_t row_addr = stage + lane * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t unit = uint32_t(j) ^ (uint32_t(lane) & 7u);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + unit * 16), "f"(v[4 * j]), "f"(v[4 * j + 1]),
                     "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                     : "memory");
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        if (add) tma_reduce_add_4d(tm, stage, col0, er.row0, er.bi, er.bo);
        else tma_store_4d(tm, stage, col0, er.row0, er.bi, er.bo);
        bulk_commit_group();
    }
}

// 32 consecutive floats of one row, 32-byte aligned, as whole sectors; `left` = columns up to N (a multiple of 8).
__device__ __forceinline__ void store_row32_sectors(float* dst, const float* v, int left) {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        if (j < left)
            asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + j), "f"(v[j]), "f"(v[j + 1]),
                         "f"(v[j + 2]), "f"(v[j + 3]), "f"(v[j + 4]), "f"(v[j + 5]), "f"(v[j + 6]), "f"(v[j + 7])
                         : "memory");
    }
}

// The bare product's way out: sector stores from registers, or the staged TMA store.
__device__ __forceinline__ void plain_store32(const float* v, int col0, const EpilogueRow& er, const GemmParams& p, int lane) {
    if (er.sector_ok) {
        if (er.row_ok) store_row32_sectors(er.c_row + col0, v, p.N - col0);
    } else if (er.row0 < p.M) {
        stage_and_store32(v, col0, er, er.tm_c, lane);
    }
}

// This thread's 32 residual values (its row, columns col0 .. col0+31); zeros outside the matrix.
__device__ __forceinline__ void load_residual32(float* r, int col0, const EpilogueRow& er, const GemmParams& p) {
    if (er.row_ok && er.vec_ok && col0 + 32 <= p.N) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const float4 t = *reinterpret_cast<const float4*>(er.res_row + col0 + j);
            r[j] = t.x; r[j + 1] = t.y; r[j + 2] = t.z; r[j + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = (er.row_ok && col0 + j < p.N) ? er.res_row[col0 + j] : 0.0f;
    }
}

// scale -> (+bias) -> [store pre-activation] -> (GELU) -> (+residual) -> store, for 32 consecutive columns of one row.
template <bool RES = false>
__device__ __forceinline__ void epilogue_store32(float* v, int col0, const EpilogueRow& er, const GemmParams& p, int lane) {
    float res[RES ? 32 : 1];
    if constexpr (RES) {
        // issued first so that the loads are in flight during the arithmetic below (the residual may alias the
        // output: every element is read here, by the thread that writes it later)
        if (p.residual) load_residual32(res, col0, er, p);
        else {
#pragma unroll
            for (int j = 0; j < 32; ++j) res[j] = 0.0f;
        }
    }
    // One uniform branch around each loop: written per element, the compiler predicates the (long) division sequence
    // into every element of every call, scaled or not (measured: +200 instructions per 32 x 32 block).
    const int scale_mode = p.scale_mode;
    if (scale_mode == TE_SCALE_MUL) {
        const float alpha = p.alpha;
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= alpha;
    } else if (scale_mode == TE_SCALE_DIV) {
        const float alpha = p.alpha;
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = v[j] / alpha;
    }
    if (p.bias) {
        // every thread of the warp needs the same 32 bias values: eight 16-byte loads from one address per
        // instruction (a broadcast out of L1), instead of a shuffle per output element
        const float* bp = p.bias + col0;
        if (col0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(bp) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 t = __ldg(reinterpret_cast<const float4*>(bp + j));
                v[j] += t.x; v[j + 1] += t.y; v[j + 2] += t.z; v[j + 3] += t.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += (col0 + j < p.N) ? __ldg(bp + j) : 0.0f;
        }
    }
    if (er.sector_ok) {   // warp-uniform
        if (!er.row_ok) return;
        if (er.pre_row) store_row32_sectors(er.pre_row + col0, v, p.N - col0);
        if (p.epilogue == TE_EPI_BIAS_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
        }
        if constexpr (RES) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += res[j];
        }
        store_row32_sectors(er.c_row + col0, v, p.N - col0);
        return;
    }
    if (er.tma_ok) {   // warp-uniform
        if (er.row0 >= p.M) return;   // nothing of this warp's 32 rows exists: issue no store at all
        if (p.preact) stage_and_store32(v, col0, er, er.tm_pre, lane);
        if (p.epilogue == TE_EPI_BIAS_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
        }
        if constexpr (RES) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += res[j];
        }
        stage_and_store32(v, col0, er, er.tm_c, lane);
        return;
    }
    if (!er.row_ok) return;
    const bool full_chunk = col0 + 32 <= p.N;
    if (er.pre_row) {
        if (full_chunk && er.vec_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(er.pre_row + col0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) er.pre_row[col0 + j] = v[j];
        }
    }
    if (p.epilogue == TE_EPI_BIAS_GELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
    }
    if constexpr (RES) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += res[j];
    }
    if (full_chunk && er.vec_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(er.c_row + col0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) er.c_row[col0 + j] = v[j];
    }
}

// Host: 4-D tensor map {contiguous index, strided index, batch_inner, batch_outer} of one operand; box_rows is the
// number of lines a K-major box carries (an MN-major box is always 32 x 32).
int make_operand_map(te_b200_ctx* ctx, CUtensorMap* out, const float* ptr, const Operand& op, int64_t K,
                     int box_rows, int64_t batch_inner, int64_t batch_outer);
// Host: tensor maps {column, row, batch_inner, batch_outer} of the output (and of the optional pre-activation
// output) for the TMA-store epilogue.  Returns false when the output cannot be described (odd ldc, misaligned base);
// the kernels then store directly.
bool make_output_maps(te_b200_ctx* ctx, const GemmProblem& g, int k_splits, CUtensorMap* tm_c, CUtensorMap* tm_pre);
// Host: the store mode for this output (fills the tensor maps when it is STORE_TMA; they are valid dummies otherwise).
int choose_store_mode(te_b200_ctx* ctx, const GemmProblem& g, int k_splits, CUtensorMap* tm_c, CUtensorMap* tm_pre);
// Fills the kernel parameters that do not depend on the tile shape.
void fill_common_params(GemmParams& p, const te_b200_ctx* ctx, const GemmProblem& g);

// attention_sm100.cu.  Host: tensor map {cols, T, H, B} of a [B, H, T, cols] view with unit last-dim stride and element
// strides strides_bht for B, H, T.  Returns false when TMA cannot address the view.
bool make_bhtc_map(te_b200_ctx* ctx, CUtensorMap* out, const float* ptr, int64_t cols, int64_t T, int64_t H, int64_t B,
                   const int64_t* strides_bht, int box_cols, int box_rows, CUtensorMapSwizzle swz);

// gemm_sm100_2cta.cu: the CTA-pair (cta_group::2) TF32 kernel, tiles 256 x bn with bn in {128, 192, 256}.
int launch_gemm_2cta(te_b200_ctx* ctx, const GemmProblem& g, int bn, int k_splits, cudaStream_t stream);

// Split-K plumbing shared by both kernels (gemm_sm100.cu).  prepare_split rewrites `kernel_problem` so that the GEMM
// kernel writes raw partial tiles into the scratch of `g`, and fills the split fields of `p`; finish_split launches the
// reduction that adds the slices and applies the epilogue of `g`.
void prepare_split(const GemmProblem& g, int k_splits, GemmProblem& kernel_problem, GemmParams& p);
int finish_split(te_b200_ctx* ctx, const GemmProblem& g, int k_splits, cudaStream_t stream);

}  // namespace te
