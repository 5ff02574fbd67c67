// Fused scaled-dot attention forward for sm_100a:  O = softmax(Q.K^T / sqrt(d)) . V, one tile = one (batch, head) and
// one block of 128 query rows, with the score matrix kept in tensor memory.  Persistent: one CTA per SM walks the tiles
// and fetches the next tile's operands while the current tile is in its softmax.
//
// Reference semantics: ScaledDot::forward (reference src/nn/scaledot.cpp:8-27): S = Q.K^T, S / sqrt(d) (a division),
// softmax over the last dimension with max subtraction and division by the row sum (reference
// src/tensor/tensor.cpp:1246-1283), then P.V; no mask, no dropout.  The probabilities P are also written out,
// because SoftmaxBackward and the backward GEMMs consume them.
//
// Why fused: unfused, the [B,H,T,T] score tensor crosses HBM four times (S written, softmax read + write, P read):
// 200 of the 252 MB the attention configuration moves.  Here S never leaves the SM; only P is written, once.
//
// Per CTA (320 threads), for every tile:
//   warp 8      TMA loads of the Q block (128 x d), all keys K (T x d) and all values V (T x d) into shared memory;
//   warp 9      S = Q.K^T with tcgen05.mma (both operands K-major) into TMEM columns [0, Tp); later O = P.V with
//               the A operand read from TMEM (P, written back by the softmax warps) and V as an MN-major operand;
//   warps 0-7   two warps per 32 query rows, each owning half of the key columns: row maximum, exp and row sum
//               straight from TMEM (the halves exchange maxima and sums through four spare TMEM columns), exp written back
//               to TMEM as the PV operand, P = exp / sum and finally O / sum staged through shared memory and
//               TMA-stored.
// Limits of this form: TF32 mode, T <= 256 keys (one TMEM pass, no running rescale), d in {32, 64}; other problems
// take the unfused path (two batched GEMMs + softmax kernel).  All waits are bounded as in the GEMM kernels.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>

#include "gemm_common.cuh"

namespace te {

constexpr int ATT_MAX_T = 256;
constexpr int ATT_O_COL = 256;     // TMEM column where the output accumulator starts
constexpr int ATT_EPI_WARPS = 8;    // two warps per TMEM lane quadrant, each owning half of the columns

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct AttnParams {
    int T, d, H, B;
    int t_pad;        // T rounded up to 16: N of the score MMA, K extent of the PV MMA
    int tiles_q;      // 128-row query blocks per head
    int total_tiles;  // B * H * tiles_q
    float scale;      // sqrt(d)
    int* status;
};

__global__ void __launch_bounds__(CTA_THREADS, 1)
attention_tf32_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_p,
                      const __grid_constant__ CUtensorMap tm_o, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    const int dchunks = p.d / 32;
    const uint32_t q_smem = base;                                         // dchunks x [128 rows x 128 B]
    const uint32_t k_smem = q_smem + dchunks * (128 * 128);               // dchunks x [256 rows x 128 B]
    const uint32_t v_smem = k_smem + dchunks * (ATT_MAX_T * 128);         // dchunks x [256 key rows x 128 B], MN-major
    const uint32_t stage_smem = v_smem + dchunks * (ATT_MAX_T * 128);     // 2 staging tiles per softmax warp
    const uint32_t aux_addr = stage_smem + 2 * ATT_EPI_WARPS * EPI_STAGE_BYTES;
    uint8_t* aux = smem_raw + (aux_addr - raw_addr);
    // One barrier per hand-off; tile i of this CTA completes phase i of each, so waits use parity i & 1.
    const uint32_t bar_qk = aux_addr;          // Q and K of the tile have landed            (producer -> MMA)
    const uint32_t bar_v = aux_addr + 8;       // V has landed                               (producer -> MMA)
    const uint32_t bar_s = aux_addr + 16;      // score MMAs done: S readable, Q/K buffers reusable (MMA -> softmax, producer)
    const uint32_t bar_p = aux_addr + 24;      // exponentials are in TMEM                   (8 softmax warps -> MMA)
    const uint32_t bar_o = aux_addr + 32;      // PV MMAs done: O readable, V buffer reusable (MMA -> softmax, producer)
    const uint32_t bar_td = aux_addr + 48;     // teardown
    const uint32_t bar_x1 = aux_addr + 56;     // row maxima of both column halves written   (8 softmax warps)
    const uint32_t bar_x2 = aux_addr + 64;     // row sums written                           (8 softmax warps)
    const uint32_t bar_sfree = aux_addr + 72;  // S columns no longer read                   (8 softmax warps -> MMA)
    const uint32_t bar_ofree = aux_addr + 80;  // O columns no longer read                   (8 softmax warps -> MMA)
    const uint32_t tmem_slot_addr = aux_addr + 40;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aux + 40);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aux + 44);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(bar_qk, 1);
        mbar_init(bar_v, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_p, ATT_EPI_WARPS);
        mbar_init(bar_o, 1);
        mbar_init(bar_td, 1);
        mbar_init(bar_x1, ATT_EPI_WARPS);
        mbar_init(bar_x2, ATT_EPI_WARPS);
        mbar_init(bar_sfree, ATT_EPI_WARPS);
        mbar_init(bar_ofree, ATT_EPI_WARPS);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(tmem_slot_addr, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    griddep_launch_dependents();   // persistent grid, every CTA resident: the next kernel may move in as CTAs exit
    griddep_wait();                // the prologue above overlapped the previous kernel's tail; global memory from here on

    // Persistent: this CTA handles tiles blockIdx.x, blockIdx.x + gridDim.x, ...  While the softmax of tile i runs,
    // the producer already fetches Q and K of tile i+1 (their buffers are free once the score MMAs are done).
    if (warp == PRODUCER_WARP) {
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            int i = 0;
            for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x, ++i) {
                const int qb = t % p.tiles_q, bh = t / p.tiles_q;
                const int h = bh % p.H, b = bh / p.H, q0 = qb * 128;
                if (i > 0 && !wait_bounded(bar_s, (i - 1) & 1, abort_flag, p.status, WAIT_PRODUCER_EMPTY)) break;
                mbar_arrive_expect_tx(bar_qk, dchunks * (128 * 128 + ATT_MAX_T * 128));
                for (int c = 0; c < dchunks; ++c) {
                    tma_load_4d(q_smem + c * (128 * 128), &tm_q, bar_qk, 32 * c, q0, h, b);
                    tma_load_4d(k_smem + c * (ATT_MAX_T * 128), &tm_k, bar_qk, 32 * c, 0, h, b);
                }
                if (i > 0 && !wait_bounded(bar_o, (i - 1) & 1, abort_flag, p.status, WAIT_PRODUCER_EMPTY)) break;
                mbar_arrive_expect_tx(bar_v, dchunks * (ATT_MAX_T * 128));
                for (int c = 0; c < dchunks; ++c)
                    for (int kb = 0; kb < ATT_MAX_T / 32; ++kb)
                        tma_load_4d(v_smem + c * (ATT_MAX_T * 128) + kb * (32 * 128), &tm_v, bar_v, 32 * c, 32 * kb, h, b);
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            const uint32_t idesc_s = make_idesc_tf32(128, p.t_pad, false, false);
            const uint32_t idesc_o = make_idesc_tf32(128, p.d, false, true);
            int i = 0;
            for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x, ++i) {
                const uint32_t par = i & 1, prev = (i - 1) & 1;
                // S columns: the previous tile's PV MMAs (which read them) and its probability pass must be over
                if (i > 0 && !(wait_bounded(bar_o, prev, abort_flag, p.status, WAIT_MMA_TMEM_EMPTY) &&
                               wait_bounded(bar_sfree, prev, abort_flag, p.status, WAIT_MMA_TMEM_EMPTY))) break;
                if (!wait_bounded(bar_qk, par, abort_flag, p.status, WAIT_MMA_FULL)) break;
                tc_fence_after_sync();
                for (int c = 0; c < dchunks; ++c) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t da = make_smem_desc(q_smem + c * (128 * 128) + j * 32, 16, 1024, SMEM_LAYOUT_SW128);
                        const uint64_t db = make_smem_desc(k_smem + c * (ATT_MAX_T * 128) + j * 32, 16, 1024, SMEM_LAYOUT_SW128);
                        umma_tf32(tmem_base, da, db, idesc_s, (c | j) != 0);
                    }
                }
                umma_commit(bar_s);
                if (!(wait_bounded(bar_p, par, abort_flag, p.status, WAIT_MMA_TMEM_EMPTY) &&
                      wait_bounded(bar_v, par, abort_flag, p.status, WAIT_MMA_FULL))) break;
                // O columns: the previous tile's output must have been read out
                if (i > 0 && !wait_bounded(bar_ofree, prev, abort_flag, p.status, WAIT_MMA_TMEM_EMPTY)) break;
                tc_fence_after_sync();
                for (int kk = 0; kk < p.t_pad / 8; ++kk) {
                    const uint64_t dv = make_smem_desc(v_smem + kk * 1024, ATT_MAX_T * 128, 512, SMEM_LAYOUT_SW128_BASE32B);
                    umma_tf32_a_tmem(tmem_base + ATT_O_COL, tmem_base + kk * 8, dv, idesc_o, kk != 0);
                }
                umma_commit(bar_o);
            }
            umma_commit(bar_td);   // nothing of this thread's MMAs may be in flight when TMEM is freed
        }
    } else {
        // ---------------------------------------------------------------- softmax + output (warps 0-7)
        const int quad = warp & 3, half = warp >> 2;
        const uint32_t t_row = tmem_base + (uint32_t(quad * 32) << 16);
        const uint32_t x_col = t_row + ATT_O_COL + 64;             // 4 spare columns: max[half 0,1], sum[half 0,1]
        const int nchunks = (p.t_pad + 31) / 32;
        const int c_begin = half ? (nchunks + 1) / 2 : 0;          // this warp's share of the 32-column chunks
        const int c_end = half ? nchunks : (nchunks + 1) / 2;
        // Scores are scaled by multiplying with 1/sqrt(d) and exponentiated with the ex2 unit: this kernel runs in
        // TF32 mode only, where the scores carry ~1e-3 relative error already, and the per-element cost of the
        // softmax is on the critical path of the CTA.
        const float k2 = (1.0f / p.scale) * 1.4426950408889634f;   // log2(e) / sqrt(d)
        int stores = 0;   // staging tiles alternate over ALL stores of this warp
        int i = 0;
        for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x, ++i) {
            const uint32_t par = i & 1;
            const int qb = t % p.tiles_q, bh = t / p.tiles_q;
            const int h = bh % p.H, b = bh / p.H, q0 = qb * 128;
            bool ok = wait_bounded(bar_s, par, abort_flag, p.status, WAIT_EPI_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            // pass 1: row maximum of the raw scores (the scale is positive, so the maximum commutes with it)
            float m = -INFINITY;
            for (int cc = c_begin; cc < c_end; ++cc) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_row + cc * 32, r);
                tmem_ld_wait();
                if ((cc + 1) * 32 <= p.T) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) m = fmaxf(m, __uint_as_float(r[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (cc * 32 + j < p.T) m = fmaxf(m, __uint_as_float(r[j]));
                }
            }
            // The two warps of a row group own the same TMEM lanes: they exchange through two spare columns.
            tmem_st_32x32b_x1(x_col + half, __float_as_uint(m));
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_x1);
            ok = wait_bounded(bar_x1, par, abort_flag, p.status, WAIT_EPI_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            m = fmaxf(m, __uint_as_float(tmem_ld_32x32b_x1(x_col + (half ^ 1))));
            tmem_ld_wait();
            const float mk = m * k2;
            // pass 2: e = exp(s - m), row sum; e goes back to TMEM as the A operand of P.V
            float sum = 0.0f;
            for (int cc = c_begin; cc < c_end; ++cc) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_row + cc * 32, r);
                tmem_ld_wait();
                if ((cc + 1) * 32 <= p.T) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float e = ex2_approx(fmaf(__uint_as_float(r[j]), k2, -mk));
                        sum += e;
                        r[j] = __float_as_uint(e);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float e = 0.0f;
                        if (cc * 32 + j < p.T) {
                            e = ex2_approx(fmaf(__uint_as_float(r[j]), k2, -mk));
                            sum += e;
                        }
                        r[j] = __float_as_uint(e);
                    }
                }
                tmem_st_32x32b_x32(t_row + cc * 32, r);
            }
            tmem_st_32x32b_x1(x_col + 2 + half, __float_as_uint(sum));
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_p);      // this warp's part of the PV operand is in place
                mbar_arrive(bar_x2);
            }
            ok = wait_bounded(bar_x2, par, abort_flag, p.status, WAIT_EPI_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            sum += __uint_as_float(tmem_ld_32x32b_x1(x_col + 2 + (half ^ 1)));
            tmem_ld_wait();
            const float inv_sum = 1.0f / sum;
            EpilogueRow er;
            er.c_row = nullptr; er.pre_row = nullptr; er.res_row = nullptr; er.row_ok = true; er.vec_ok = false; er.tma_ok = true; er.sector_ok = false;
            er.stage = stage_smem + warp * 2 * EPI_STAGE_BYTES;
            er.tm_c = &tm_p; er.tm_pre = &tm_p;
            er.row0 = q0 + quad * 32;
            er.bi = h; er.bo = b;
            // pass 3: P = e / sum, written out once (while the tensor core computes P.V from the same columns)
            for (int cc = c_begin; cc < c_end && cc * 32 < p.T; ++cc) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_row + cc * 32, r);
                tmem_ld_wait();
                if (er.row0 < p.T) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * inv_sum;
                    stage_and_store32(v, cc * 32, er, &tm_p, lane, true, (stores++) & 1);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sfree);     // the S columns may be overwritten by the next tile's scores
            ok = wait_bounded(bar_o, par, abort_flag, p.status, WAIT_EPI_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            const int o_begin = half ? (dchunks + 1) / 2 : 0, o_end = half ? dchunks : (dchunks + 1) / 2;
            for (int cc = o_begin; cc < o_end; ++cc) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_row + ATT_O_COL + cc * 32, r);
                tmem_ld_wait();
                if (er.row0 < p.T) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * inv_sum;
                    stage_and_store32(v, cc * 32, er, &tm_o, lane, true, (stores++) & 1);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_ofree);     // the O columns may be overwritten by the next tile's P.V
        }
        if (lane == 0) bulk_wait_read_all();   // shared memory may go away once the stores have read it
    }

    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) {
        if (lane == 0) {   // teardown barrier: every MMA of this CTA has completed
            const uint64_t t0 = global_timer_ns();
            while (!mbar_try_wait(bar_td, 0)) {
                if (global_timer_ns() - t0 > WAIT_LIMIT_NS) {
                    atomicCAS(p.status, 0, (int)WAIT_TEARDOWN);
                    break;
                }
            }
        }
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

// [B, H, T, cols] view with unit last-dim stride -> map {cols, T, H, B}.
bool make_bhtc_map(te_b200_ctx* ctx, CUtensorMap* out, const float* ptr, int64_t cols, int64_t T, int64_t H,
                          int64_t B, const int64_t* strides_bht, int box_cols, int box_rows, CUtensorMapSwizzle swz) {
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return false;
    const int64_t sT = strides_bht[2], sH = strides_bht[1], sB = strides_bht[0];
    if ((T > 1 && ((sT & 3) || sT < cols)) || (H > 1 && ((sH & 3) || sH == 0)) || (B > 1 && ((sB & 3) || sB == 0))) return false;
    const cuuint64_t row_bytes = (cuuint64_t)(T > 1 ? sT : ((cols + 3) & ~int64_t(3))) * 4;
    const uint64_t dims[4] = {(uint64_t)cols, (uint64_t)T, (uint64_t)H, (uint64_t)B};
    const uint64_t strides[3] = {row_bytes, H > 1 ? (uint64_t)sH * 4 : row_bytes, B > 1 ? (uint64_t)sB * 4 : row_bytes};
    const uint32_t box[4] = {(uint32_t)box_cols, (uint32_t)box_rows, 1, 1};
    return encode_tiled_cached(ctx, out, ptr, dims, strides, box, (int)swz, (int)CU_TENSOR_MAP_L2_PROMOTION_L2_256B) == 0;
}

// Returns TE_OK when the fused kernel was launched, -1 when this problem is outside its limits (the caller then
// takes the unfused path), or an error status.
int launch_attention_fused(te_b200_ctx* ctx, const te_attn_desc* t, cudaStream_t stream) {
    if (t->precision != TE_PREC_TF32) return -1;
    if (t->T > ATT_MAX_T || (t->T & 3) || (t->d != 32 && t->d != 64)) return -1;
    if (t->B * t->H * ((t->T + 127) / 128) > INT32_MAX) return -1;
    CUtensorMap mq, mk, mv, mp, mo;
    const int64_t p_strides[3] = {t->H * t->T * t->T, t->T * t->T, t->T};
    if (!make_bhtc_map(ctx, &mq, t->q, t->d, t->T, t->H, t->B, t->q_strides, 32, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (!make_bhtc_map(ctx, &mk, t->k, t->d, t->T, t->H, t->B, t->k_strides, 32, 256, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (!make_bhtc_map(ctx, &mv, t->v, t->d, t->T, t->H, t->B, t->v_strides, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return -1;
    if (!make_bhtc_map(ctx, &mp, t->p_out, t->T, t->T, t->H, t->B, p_strides, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (!make_bhtc_map(ctx, &mo, t->o, t->d, t->T, t->H, t->B, t->o_strides, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    AttnParams p;
    p.T = (int)t->T; p.d = (int)t->d; p.H = (int)t->H; p.B = (int)t->B;
    p.t_pad = (int)((t->T + 15) & ~int64_t(15));
    p.tiles_q = (int)((t->T + 127) / 128);
    p.scale = sqrtf((float)t->d);
    p.status = ctx->d_status;
    const int dchunks = p.d / 32;
    const int smem = 1024 + dchunks * (128 * 128 + 2 * ATT_MAX_T * 128) + 2 * ATT_EPI_WARPS * EPI_STAGE_BYTES + 128;
    if (smem > 232448) return -1;
    int& attr_smem = ctx->kernel_state[reinterpret_cast<const void*>(attention_tf32_kernel)];
    if (attr_smem < smem) {
        cudaError_t e = cudaFuncSetAttribute(attention_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(attention)");
        attr_smem = smem;
    }
    p.total_tiles = (int)(t->B * t->H * p.tiles_q);
    const int grid = p.total_tiles < ctx->sm_count ? p.total_tiles : ctx->sm_count;
    launch_pdl(attention_tf32_kernel, dim3(grid), dim3(CTA_THREADS), smem, stream, mq, mk, mv, mp, mo, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "attention_tf32_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

}  // namespace te
