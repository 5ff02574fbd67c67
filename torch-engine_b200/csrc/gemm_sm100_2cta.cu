// CTA-pair form of the TF32 GEMM: two neighbouring SMs (a cluster of 2 CTAs) compute one 256 x 256 output tile
// with tcgen05.mma.cta_group::2.
//
// Why: the single-CTA kernel streams (128 + 256) x 32 floats = 48 KB into shared memory for every 128x256x32
// block of work and is limited by how fast shared memory can be filled, not by the tensor pipe.  In the pair form
// each CTA loads its own 128 rows of A and only HALF of the B block (128 of the 256 columns); the instruction
// reads both halves straight out of the two CTAs' shared memories.  Per CTA that is 32 KB for the same amount of
// tensor work, and no load is broadcast between CTAs.
//
// Roles per CTA are as in the single-CTA kernel (warps 0-7 epilogue, warp 8 TMA producer, warp 9 MMA), with the
// pair protocol on top:
//   * "full" barriers live in the leader CTA (cluster rank 0): both producers post their byte counts there;
//   * the leader's MMA lane issues for the pair and commits to the "empty" and "accumulator full" barriers of
//     BOTH CTAs;
//   * each CTA's epilogue drains its own 128 accumulator rows from its own TMEM and both report to the leader's
//     "accumulator empty" barrier.
// Every wait is bounded as in the single-CTA kernel; the CTAs leave together through a cluster barrier.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "gemm_common.cuh"

namespace te {

constexpr int PAIR_BM = 256;   // rows of one pair tile (128 per CTA)

// NW = 1: the tile is 256 x BN and tensor memory holds two accumulator buffers, so the epilogue of one tile overlaps
// the main loop of the next.  NW = 2 ("wide"): the tile is 256 x 2 BN, computed by two MMAs per k-step into two
// accumulators side by side; A is fetched once for twice the columns (a third fewer bytes per flop into shared
// memory), at the price of a single accumulator buffer: the next tile's MMAs wait for the epilogue.
template <int BN, int NPL, int NW = 1>
struct PairCfg {
    static constexpr int TILE_N = NW * BN;
    static constexpr int B_HALF_BYTES = (TILE_N / 2) * BK * 4;
    static constexpr int STAGE_BYTES = NPL * (A_PLANE_BYTES + B_HALF_BYTES);      // per CTA; NPL = 2: tf32 hi and lo planes
    static constexpr int STAGES = SMEM_RING_BUDGET / STAGE_BYTES;
    static constexpr int ACC_BUFS = NW == 1 ? 2 : 1;
    static constexpr int TMEM_COLS = ACC_BUFS * TILE_N <= 256 ? 256 : 512;   // allocations are powers of two
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * EPI_STAGE_BYTES + SMEM_AUX_BYTES + 1024;
    static_assert(STAGES >= 2 && STAGES <= 12, "ring depth");
    static_assert(ACC_BUFS * TILE_N <= TMEM_COLS && BN % 64 == 0 && (NW == 1 || NPL == 1), "TMEM columns");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

// EPI_PLAIN: the output is the bare product going out through TMA stores (no scale, bias, pre-activation output or GELU).
// Compiling that case separately keeps the general epilogue's code out of it, which is worth 2-11 % on the products
// whose epilogue is not hidden behind a long main loop (16384x384x384: 16.9 -> 15.1 us) and 2 % on 8192^3.
template <int BN, int NPL, bool A_MN, bool B_MN, int NW = 1, int EPI = EPI_GENERAL>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(CTA_THREADS, 1)
gemm_tf32_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a_lo,
                      const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_b_lo,
                      const __grid_constant__ CUtensorMap tm_c, const __grid_constant__ CUtensorMap tm_pre,
                      const GemmParams p) {
    using Cfg = PairCfg<BN, NPL, NW>;
    constexpr int TN = Cfg::TILE_N;           // columns of one tile
    constexpr int ACC_BUFS = Cfg::ACC_BUFS;
    constexpr bool CHUNKED = (NPL == 2);      // 3xTF32: sum K in chunks in TMEM, add the chunks in registers
    constexpr int CHUNK_KB = 8;
    constexpr int B_HALF_BYTES = Cfg::B_HALF_BYTES;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr int HALF_N = BN / 2;
    constexpr uint32_t IDESC = make_idesc_tf32(PAIR_BM, BN, A_MN, B_MN);
    constexpr uint32_t MN_CHUNK_BYTES = BK * 128;
    constexpr uint32_t A_LBO = A_MN ? MN_CHUNK_BYTES : 16, A_SBO = A_MN ? 512 : 1024, A_KSTEP = A_MN ? 1024 : UMMA_K * 4;
    constexpr uint32_t B_LBO = B_MN ? MN_CHUNK_BYTES : 16, B_SBO = B_MN ? 512 : 1024, B_KSTEP = B_MN ? 1024 : UMMA_K * 4;
    constexpr uint32_t A_LAYOUT = A_MN ? SMEM_LAYOUT_SW128_BASE32B : SMEM_LAYOUT_SW128;
    constexpr uint32_t B_LAYOUT = B_MN ? SMEM_LAYOUT_SW128_BASE32B : SMEM_LAYOUT_SW128;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t ring = (raw_addr + 1023u) & ~1023u;
    const uint32_t epi_stage = ring + STAGES * STAGE_BYTES;       // EPI_WARPS staging tiles, 1024-byte aligned
    uint8_t* aux = smem_raw + (ring - raw_addr) + STAGES * STAGE_BYTES + EPI_WARPS * EPI_STAGE_BYTES;
    const uint32_t aux_addr = epi_stage + EPI_WARPS * EPI_STAGE_BYTES;
    // aux: full[STAGES] | empty[STAGES] | tmem_full[2] | tmem_empty[2] | teardown | slot | abort
    const uint32_t bar_full = aux_addr;
    const uint32_t bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tmem_full = bar_empty + 8 * STAGES;
    const uint32_t bar_tmem_empty = bar_tmem_full + 16;
    const uint32_t bar_teardown = bar_tmem_empty + 16;
    const uint32_t tmem_slot_addr = bar_teardown + 8;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aux + (tmem_slot_addr - aux_addr));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aux + (tmem_slot_addr - aux_addr) + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 2);           // leader's copy is the one in use: one arrival per producer
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tmem_full + 8 * i, 1);
            mbar_init(bar_tmem_empty + 8 * i, 2 * EPI_WARPS);   // leader's copy: the epilogue warps of both CTAs
        }
        mbar_init(bar_teardown, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == PRODUCER_WARP && lane == 0) {
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        if (NPL == 2) {
            tma_prefetch_desc(&tm_a_lo);
            tma_prefetch_desc(&tm_b_lo);
        }
    }
    if (warp == MMA_WARP) {
        tmem_alloc_pair(tmem_slot_addr, Cfg::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                               // partner's barriers are initialised before anyone signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched only the pair's shared and tensor memory, so it may overlap the tail of the kernel
    // ahead in the stream; from here on global memory is read and written.
    griddep_launch_dependents();
    griddep_wait();

    const int total_units = p.tiles_m * p.tiles_n * p.num_batches * p.k_splits;
    const int kblocks = (p.K + BK - 1) / BK;

    if (warp == PRODUCER_WARP) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int u = pair; u < total_units && ok; u += num_pairs) {
                WorkUnit w;
                decode_unit(u, p, kblocks, w);
                const int batch = w.batch, m_blk = w.m_blk, n_blk = w.n_blk;
                const int bo = batch / p.batch_inner, bi = batch - bo * p.batch_inner;
                const int a_ci = bi * p.a_mul_inner, a_co = bo * p.a_mul_outer;
                const int b_ci = bi * p.b_mul_inner, b_co = bo * p.b_mul_outer;
                const int m0 = m_blk * PAIR_BM + (int)rank * BM;       // this CTA's 128 rows of A
                const int n0 = n_blk * TN + (int)rank * HALF_N;        // this CTA's half of the B columns (of every sub-tile)
                for (int kb = w.kb0; kb < w.kb1; ++kb, ++issued) {
                    const int s = issued % STAGES;
                    const uint32_t phase = (issued / STAGES) & 1;
                    if (!wait_bounded(bar_empty + 8 * s, phase ^ 1, abort_flag, p.status, WAIT_PRODUCER_EMPTY)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = map_to_cta(bar_full + 8 * s, 0);     // the leader's barrier
                    mbar_arrive_expect_tx_cluster(full, STAGE_BYTES);
                    const uint32_t sa = ring + s * STAGE_BYTES;
                    const uint32_t sb = sa + NPL * A_PLANE_BYTES;
                    const int k0 = kb * BK;
#pragma unroll
                    for (int pl = 0; pl < NPL; ++pl) {
                        const CUtensorMap* ma = pl ? &tm_a_lo : &tm_a;
                        const CUtensorMap* mb = pl ? &tm_b_lo : &tm_b;
                        const uint32_t pa = sa + pl * A_PLANE_BYTES, pb = sb + pl * B_HALF_BYTES;
                        if (A_MN) {
#pragma unroll
                            for (int c = 0; c < BM / 32; ++c)
                                tma_load_4d_pair(pa + c * MN_CHUNK_BYTES, ma, full, m0 + 32 * c, k0, a_ci, a_co);
                        } else {
                            tma_load_4d_pair(pa, ma, full, k0, m0, a_ci, a_co);
                        }
#pragma unroll
                        for (int sub = 0; sub < NW; ++sub) {      // sub-tile `sub` takes columns n0 + sub * BN ..
                            if (B_MN) {
#pragma unroll
                                for (int c = 0; c < HALF_N / 32; ++c)
                                    tma_load_4d_pair(pb + (sub * (HALF_N / 32) + c) * MN_CHUNK_BYTES, mb, full, n0 + sub * BN + 32 * c, k0, b_ci, b_co);
                            } else {
                                tma_load_4d_pair(pb + sub * (HALF_N * BK * 4), mb, full, k0, n0 + sub * BN, b_ci, b_co);
                            }
                        }
                    }
                }
            }
            if (!ok || *abort_flag) {
                // Copies already issued still write this CTA's shared memory: give them time to land before leaving.
                const uint64_t t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 200000ull) {
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            int consumed = 0;
            int acc_idx = 0;
            bool ok = true;
            for (int u = pair; u < total_units && ok; u += num_pairs) {
                WorkUnit w;
                decode_unit(u, p, kblocks, w);
                int kb = w.kb0;
                do {   // one pass per accumulator buffer: this unit's whole K range, or one chunk of it
                    const int kb_end = CHUNKED ? min(kb + CHUNK_KB, w.kb1) : w.kb1;
                    const int buf = ACC_BUFS == 2 ? (acc_idx & 1) : 0;
                    const uint32_t acc_phase = ACC_BUFS == 2 ? ((acc_idx >> 1) & 1) : (acc_idx & 1);
                    if (!wait_bounded(bar_tmem_empty + 8 * buf, acc_phase ^ 1, abort_flag, p.status,
                                      WAIT_MMA_TMEM_EMPTY)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * TN;
                    const int kb_first = kb;
                    for (; kb < kb_end; ++kb, ++consumed) {
                        const int s = consumed % STAGES;
                        if (!wait_bounded(bar_full + 8 * s, (consumed / STAGES) & 1, abort_flag, p.status, WAIT_MMA_FULL)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t sa = ring + s * STAGE_BYTES;
                        const uint32_t sb = sa + NPL * A_PLANE_BYTES;
#pragma unroll
                        for (int j = 0; j < BK / UMMA_K; ++j) {
                            const uint64_t a_hi = make_smem_desc(sa + j * A_KSTEP, A_LBO, A_SBO, A_LAYOUT);
                            const uint64_t b_hi = make_smem_desc(sb + j * B_KSTEP, B_LBO, B_SBO, B_LAYOUT);
                            const uint32_t acc0 = ((kb - kb_first) | j) != 0;
                            if (NPL == 2) {
                                const uint64_t a_lo = make_smem_desc(sa + A_PLANE_BYTES + j * A_KSTEP, A_LBO, A_SBO, A_LAYOUT);
                                const uint64_t b_lo = make_smem_desc(sb + B_HALF_BYTES + j * B_KSTEP, B_LBO, B_SBO, B_LAYOUT);
                                umma_tf32_pair(d_tmem, a_lo, b_hi, IDESC, acc0);   // small terms first
                                umma_tf32_pair(d_tmem, a_hi, b_lo, IDESC, 1);
                                umma_tf32_pair(d_tmem, a_hi, b_hi, IDESC, 1);
                            } else {
                                umma_tf32_pair(d_tmem, a_hi, b_hi, IDESC, acc0);
                                if (NW == 2) {     // second sub-tile: the other half of this CTA pair's B rows, next BN columns
                                    constexpr uint32_t SUB = B_MN ? (HALF_N / 32) * MN_CHUNK_BYTES : HALF_N * BK * 4;
                                    const uint64_t b2 = make_smem_desc(sb + SUB + j * B_KSTEP, B_LBO, B_SBO, B_LAYOUT);
                                    umma_tf32_pair(d_tmem + BN, a_hi, b2, IDESC, acc0);
                                }
                            }
                        }
                        umma_commit_pair(bar_empty + 8 * s, 3);        // frees the stage in both CTAs
                    }
                    if (!ok) break;
                    umma_commit_pair(bar_tmem_full + 8 * buf, 3);      // accumulator ready in both CTAs
                    ++acc_idx;
                } while (kb < w.kb1);
            }
            umma_commit_pair(bar_teardown, 1);
            const uint64_t t0 = global_timer_ns();
            while (!mbar_try_wait(bar_teardown, 0)) {
                if (global_timer_ns() - t0 > WAIT_LIMIT_NS) {
                    atomicCAS(p.status, 0, (int)WAIT_TEARDOWN);
                    break;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 0-7, both CTAs)
        int acc_idx = 0;
        bool ok = true;
        for (int u = pair; u < total_units && ok; u += num_pairs) {
            WorkUnit w;
            decode_unit(u, p, kblocks, w);
            const int batch = w.batch, m_blk = w.m_blk, n_blk = w.n_blk;
            const int bo = batch / p.batch_inner, bi = batch - bo * p.batch_inner;
            const int row = m_blk * PAIR_BM + (int)rank * BM + (warp & 3) * 32 + lane;
            const int n0 = n_blk * TN;
            const long long batch_off = (long long)bo * p.c_stride_outer + (long long)bi * p.c_stride_inner +
                                        (long long)w.split * p.split_stride;
            EpilogueRow er;
            er.c_row = p.c + batch_off + (long long)row * p.ldc;
            er.pre_row = p.preact ? p.preact + batch_off + (long long)row * p.ldc : nullptr;
            er.res_row = p.residual ? p.residual + batch_off + (long long)row * p.ldc : nullptr;
            er.row_ok = row < p.M;
            er.vec_ok = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.c + batch_off) & 15) == 0) &&
                        (!p.preact || (reinterpret_cast<uintptr_t>(p.preact + batch_off) & 15) == 0) &&
                        (!p.residual || (reinterpret_cast<uintptr_t>(p.residual + batch_off) & 15) == 0);
            er.tma_ok = p.tma_store == STORE_TMA;
            er.sector_ok = p.tma_store == STORE_SECTOR;
            er.stage = epi_stage + warp * EPI_STAGE_BYTES;
            er.tm_c = &tm_c;
            er.tm_pre = &tm_pre;
            er.row0 = m_blk * PAIR_BM + (int)rank * BM + (warp & 3) * 32;
            er.bi = bi;
            er.bo = w.split * p.batch_outer_n + bo;
            const uint32_t empty_leader = map_to_cta(bar_tmem_empty, 0);
            if (CHUNKED) {
                // Two-level accumulation (see the single-CTA kernel): chunk sums from TMEM are added in registers.
                constexpr int NACC = CHUNKED ? BN / 2 : 1;     // this warp's half of the tile's columns
                const int nh = n0 + (warp >> 2) * (BN / 2);
                float acc[NACC];
#pragma unroll
                for (int j = 0; j < NACC; ++j) acc[j] = 0.0f;
                const int chunks = w.kb1 > w.kb0 ? (w.kb1 - w.kb0 + CHUNK_KB - 1) / CHUNK_KB : 1;
                for (int ch = 0; ch < chunks && ok; ++ch, ++acc_idx) {
                    const int buf = acc_idx & 1;
                    ok = wait_bounded(bar_tmem_full + 8 * buf, (acc_idx >> 1) & 1, abort_flag, p.status, WAIT_EPI_TMEM_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t t_row = tmem_base + (uint32_t((warp & 3) * 32) << 16) + buf * BN + (warp >> 2) * (BN / 2);
                    if (p.K > 0) {
#pragma unroll
                        for (int cc = 0; cc < NACC / 32; ++cc) {
                            if (nh + cc * 32 < p.N) {   // warp-uniform
                                uint32_t r[32];
                                tmem_ld_32x32b_x32(t_row + cc * 32, r);
                                tmem_ld_wait();
#pragma unroll
                                for (int j = 0; j < 32; ++j) acc[cc * 32 + j] += __uint_as_float(r[j]);
                            }
                        }
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(empty_leader + 8 * buf);
                }
                if (ok) {
#pragma unroll
                    for (int cc = 0; cc < NACC / 32; ++cc) {
                        const int col0 = nh + cc * 32;
                        if (col0 < p.N) {
                            if constexpr (EPI == EPI_PLAIN) {
                                plain_store32(&acc[cc * 32], col0, er, p, lane);
                            } else {
                                epilogue_store32<EPI == EPI_RESIDUAL>(&acc[cc * 32], col0, er, p, lane);
                            }
                        }
                    }
                }
            } else {
                const int buf = ACC_BUFS == 2 ? (acc_idx & 1) : 0;
                const uint32_t acc_phase = ACC_BUFS == 2 ? ((acc_idx >> 1) & 1) : (acc_idx & 1);
                ok = wait_bounded(bar_tmem_full + 8 * buf, acc_phase, abort_flag, p.status, WAIT_EPI_TMEM_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t t_row = tmem_base + (uint32_t((warp & 3) * 32) << 16) + buf * TN;
#pragma unroll 1
                for (int cc = (warp >> 2) * (TN / 64); cc < ((warp >> 2) + 1) * (TN / 64); ++cc) {
                    const int col0 = n0 + cc * 32;
                    if (col0 >= p.N) break;
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(t_row + cc * 32, r);
                    tmem_ld_wait();
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = p.K > 0 ? __uint_as_float(r[j]) : 0.0f;
                    if constexpr (EPI == EPI_PLAIN) {
                        plain_store32(v, col0, er, p, lane);
                    } else {
                        epilogue_store32<EPI == EPI_RESIDUAL>(v, col0, er, p, lane);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(empty_leader + 8 * buf);
                ++acc_idx;
            }
        }
    }

    if (warp < EPI_WARPS && lane == 0) bulk_wait_all();   // this warp's output stores are complete
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();          // nobody leaves while the partner may still touch this CTA's memory or barriers
    if (warp == MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    }
}

// One-time set-up of a pair-kernel instance in this context; *out_pairs receives how many CTA pairs can be resident.
template <int BN, int NPL, bool A_MN, bool B_MN, int NW, int EPI>
static int ensure_pair_kernel(te_b200_ctx* ctx, int* out_pairs) {
    using Cfg = PairCfg<BN, NPL, NW>;
    auto kernel = gemm_tf32_pair_kernel<BN, NPL, A_MN, B_MN, NW, EPI>;
    // kernel_state of a pair kernel: 0 = untouched, otherwise the number of CTA pairs that can be resident at once
    int& max_pairs = ctx->kernel_state[reinterpret_cast<const void*>(kernel)];
    if (max_pairs == 0) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(max dynamic shared memory)");
        // pairs must sit on neighbouring SMs, so the count can be below SMs / 2
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(ctx->sm_count & ~1, 1, 1);
        cfg.blockDim = dim3(CTA_THREADS, 1, 1);
        cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        cudaError_t eo = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
        if (eo != cudaSuccess || n < 1) { cudaGetLastError(); n = ctx->sm_count / 2; }
        max_pairs = n;
    }
    *out_pairs = max_pairs;
    return TE_OK;
}

int prepare_pair_3xtf32_kernel(te_b200_ctx* ctx) {
    int pairs = 0;
    return ensure_pair_kernel<256, 2, false, false, 1, EPI_RESIDUAL>(ctx, &pairs);
}

template <int BN, int NPL, bool A_MN, bool B_MN, int NW, int EPI>
static int launch_pair_impl(te_b200_ctx* ctx, const GemmProblem& g_in, int k_splits, cudaStream_t stream);

// The bare-product kernel serves the calls whose output a tensor map can describe and that ask for nothing but the
// product (split-K partial tiles included); everything else takes the general one.
template <int BN, int NPL, bool A_MN, bool B_MN, int NW = 1>
static int launch_pair_variant(te_b200_ctx* ctx, const GemmProblem& g, int k_splits, cudaStream_t stream) {
    const bool bare = k_splits > 1 || (!g.bias && !g.preact && !g.residual && g.scale_mode == TE_SCALE_NONE && g.epilogue == TE_EPI_NONE);
    if (NPL == 1 && bare) {
        // does a tensor map describe the output?  (the encoding itself is cached in the context, so the launcher's own
        // call below costs a table look-up)
        GemmProblem k = g;
        GemmParams scratch;
        CUtensorMap probe_c, probe_pre;
        fill_common_params(scratch, ctx, g);
        prepare_split(g, k_splits, k, scratch);
        if (make_output_maps(ctx, k, k_splits, &probe_c, &probe_pre))
            return launch_pair_impl<BN, NPL, A_MN, B_MN, NW, EPI_PLAIN>(ctx, g, k_splits, stream);
    }
    // 3xTF32 (NPL = 2) has one instance, which carries the residual input
    if (NPL == 2 || (g.residual && k_splits == 1)) return launch_pair_impl<BN, NPL, A_MN, B_MN, NW, EPI_RESIDUAL>(ctx, g, k_splits, stream);
    if constexpr (NPL == 1) return launch_pair_impl<BN, NPL, A_MN, B_MN, NW, EPI_GENERAL>(ctx, g, k_splits, stream);
    return TE_ERR_BAD_ARGUMENT;   // not reached
}

template <int BN, int NPL, bool A_MN, bool B_MN, int NW, int EPI>
static int launch_pair_impl(te_b200_ctx* ctx, const GemmProblem& g_in, int k_splits, cudaStream_t stream) {
    using Cfg = PairCfg<BN, NPL, NW>;
    auto kernel = gemm_tf32_pair_kernel<BN, NPL, A_MN, B_MN, NW, EPI>;
    int max_pairs = 0;
    if (int rc0 = ensure_pair_kernel<BN, NPL, A_MN, B_MN, NW, EPI>(ctx, &max_pairs)) return rc0;
    GemmProblem g = g_in;
    CUtensorMap ma, mal, mb, mbl;
    int rc;
    if ((rc = make_operand_map(ctx, &ma, g.a.ptr, g.a, g.K, BM, g.batch_inner, g.batch_outer))) return rc;
    if ((rc = make_operand_map(ctx, &mb, g.b.ptr, g.b, g.K, BN / 2, g.batch_inner, g.batch_outer))) return rc;
    if (NPL == 2) {
        if ((rc = make_operand_map(ctx, &mal, g.a_lo, g.a, g.K, BM, g.batch_inner, g.batch_outer))) return rc;
        if ((rc = make_operand_map(ctx, &mbl, g.b_lo, g.b, g.K, BN / 2, g.batch_inner, g.batch_outer))) return rc;
    } else {
        mal = ma;
        mbl = mb;
    }
    GemmParams p;
    fill_common_params(p, ctx, g);
    prepare_split(g_in, k_splits, g, p);       // with k_splits > 1 the kernel writes raw partial tiles to scratch
    CUtensorMap mc, mpre;
    p.tma_store = choose_store_mode(ctx, g, k_splits, &mc, &mpre);
    if (EPI == EPI_PLAIN && !p.tma_store) {
        set_error("internal: the bare-product kernel was chosen for an output no tensor map describes");
        return TE_ERR_BAD_ARGUMENT;
    }
    p.tiles_m = (int)((g.M + PAIR_BM - 1) / PAIR_BM);
    p.tiles_n = (int)((g.N + Cfg::TILE_N - 1) / Cfg::TILE_N);
    const long long total = (long long)p.tiles_m * p.tiles_n * p.num_batches * k_splits;
    const int pairs = (int)(total < max_pairs ? total : max_pairs);
    cudaError_t e = launch_pdl(kernel, dim3((unsigned)(2 * pairs)), dim3(CTA_THREADS), Cfg::SMEM_BYTES, stream, ma, mal, mb, mbl, mc, mpre, p);
    if (e != cudaSuccess) return cuda_fail(e, "gemm_tf32_pair_kernel launch");
    ctx->launches += 1;
    return k_splits > 1 ? finish_split(ctx, g_in, k_splits, stream) : TE_OK;
}

template <int BN, int NW = 1>
static int launch_pair_bn(te_b200_ctx* ctx, const GemmProblem& g, int k_splits, cudaStream_t stream) {
    if (!g.a.mn_major && !g.b.mn_major) return launch_pair_variant<BN, 1, false, false, NW>(ctx, g, k_splits, stream);
    if (!g.a.mn_major && g.b.mn_major) return launch_pair_variant<BN, 1, false, true, NW>(ctx, g, k_splits, stream);
    if (g.a.mn_major && !g.b.mn_major) return launch_pair_variant<BN, 1, true, false, NW>(ctx, g, k_splits, stream);
    return launch_pair_variant<BN, 1, true, true, NW>(ctx, g, k_splits, stream);
}

int launch_gemm_2cta(te_b200_ctx* ctx, const GemmProblem& g, int bn, int k_splits, cudaStream_t stream) {
    if (g.a_lo) return launch_pair_variant<256, 2, false, false>(ctx, g, k_splits, stream);   // 3xTF32: packed K-major planes
    if (bn == 128) return launch_pair_bn<128>(ctx, g, k_splits, stream);
    if (bn == 192) return launch_pair_bn<192>(ctx, g, k_splits, stream);
    if (bn == 384) return launch_pair_bn<192, 2>(ctx, g, k_splits, stream);   // wide tiles: two accumulators side by side
    if (bn == 512) return launch_pair_bn<256, 2>(ctx, g, k_splits, stream);
    return launch_pair_bn<256>(ctx, g, k_splits, stream);
}

}  // namespace te
