// FP32-in / FP32-out GEMM for sm_100a on the 5th-generation tensor cores.
//
//   C[b] = epilogue( scale( A[b] . B[b] ) ),  A: M x K,  B: K x N,  C: M x N row-major.
//
// One persistent CTA per SM walks a list of 128 x BN output tiles.  Inside a CTA the work is
// split by warp role:
//   warps 0-7  epilogue: tcgen05.ld the finished accumulator out of TMEM, apply scale / bias /
//              GELU, store to global memory;
//   warp  8    producer: one lane issues TMA tensor loads (128-byte swizzle, each CTA for itself) of the
//              A and B k-blocks into a ring of shared-memory stages;
//   warp  9    MMA: one lane issues tcgen05.mma kind::tf32 (128 x BN x 8 per instruction) from
//              shared-memory descriptors into one of two TMEM accumulator buffers, so the
//              epilogue of tile i overlaps the main loop of tile i+1.
// Stage hand-off is by mbarriers (full: TMA bytes landed; empty: tcgen05.commit after the MMAs
// that read the stage).  Every wait is bounded: after ~2 s a waiter records an error code in a
// device status word, raises a CTA-wide abort flag, and all roles fall through to the teardown
// that drains outstanding copies/MMAs and frees TMEM.
//
// Operands are either K-major (K contiguous: a row-major A, a column-major B) or MN-major (a
// column-major A, a row-major B).  Both are read in place by TMA; ragged M/N/K edges rely on
// TMA zero fill and a predicated epilogue.  In 3xTF32 mode each operand comes as two tf32 planes
// (hi, lo) and every k-step issues lo.hi + hi.lo + hi.hi into the same accumulator; because the tensor
// core's fp32 adder truncates, K is summed in chunks of 256 in TMEM and the chunks are added in registers.
//
// Where this sits in the reference: it is the device side of Tensor::cuda_matmul_impl_f32
// (reference src/tensor/tensor.h:614-793), replacing cublasSgemm(/StridedBatched) and
// matmul_kernel_double_buffered_cpasync (reference src/cuda/elementwise_cuda.cu:842-1005).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <type_traits>

#include "gemm_common.cuh"

namespace te {


// EPI_PLAIN: the output is the bare product going out through TMA stores (no scale, bias, pre-activation output or
// GELU); the general epilogue's code costs registers and drain time even when none of its branches is taken.
// EPI_RESIDUAL: the general epilogue plus a residual input added last.
// SPLIT (3xTF32 only): the operands arrive as they are in memory; TMA fills the first plane of a stage with the raw
// fp32 tile and four converter warps (warps 10-13) rewrite it in place as hi = round-to-nearest tf32(x) and write
// lo = round-to-nearest tf32(x - hi) into the second plane, then hand the stage to the MMA warp.  Same numbers as the
// packing pre-pass, without its workspace and without its extra pass over global memory.
template <int BN, int NPL, bool A_MN, bool B_MN, int EPI = EPI_GENERAL, bool SPLIT = false>
__global__ void __launch_bounds__(SPLIT ? CTA_THREADS + CONVERTER_THREADS : CTA_THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a_lo,
                 const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_b_lo,
                 const __grid_constant__ CUtensorMap tm_c, const __grid_constant__ CUtensorMap tm_pre,
                 const GemmParams p) {
    using Cfg = TileCfg<BN, NPL>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int B_PLANE_BYTES = Cfg::B_PLANE_BYTES;
    constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr uint32_t IDESC = make_idesc_tf32(BM, BN, A_MN, B_MN);
    constexpr bool CHUNKED = (NPL == 2);      // 3xTF32: sum K in chunks, add the chunks in registers
    constexpr int CHUNK_KB = 8;               // k-blocks per chunk = 256 values of K
    static_assert(!CHUNKED || BN <= 256, "chunked accumulation keeps BN/2 floats per thread in registers");
    static_assert(!SPLIT || NPL == 2, "the in-kernel split produces the second plane of a two-plane stage");
    // Descriptor geometry.
    // K-major (TMA SWIZZLE_128B): rows of 128 B, 8-row groups 1024 B apart (SBO); one MMA advances 32 B along K.
    // MN-major (TMA SWIZZLE_128B_ATOM_32B): every k index is a 128-byte row of 32 consecutive MN elements;
    // 4-row groups are 512 B apart (SBO), 32-element MN chunks are BK*128 B apart (LBO); one MMA (8 k) advances 1024 B.
    constexpr uint32_t MN_CHUNK_BYTES = BK * 128;
    constexpr uint32_t A_LBO = A_MN ? MN_CHUNK_BYTES : 16, A_SBO = A_MN ? 512 : 1024, A_KSTEP = A_MN ? 1024 : UMMA_K * 4;
    constexpr uint32_t B_LBO = B_MN ? MN_CHUNK_BYTES : 16, B_SBO = B_MN ? 512 : 1024, B_KSTEP = B_MN ? 1024 : UMMA_K * 4;
    constexpr uint32_t A_LAYOUT = A_MN ? SMEM_LAYOUT_SW128_BASE32B : SMEM_LAYOUT_SW128;
    constexpr uint32_t B_LAYOUT = B_MN ? SMEM_LAYOUT_SW128_BASE32B : SMEM_LAYOUT_SW128;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t ring = (raw_addr + 1023u) & ~1023u;           // 128B swizzle wants 1024-byte aligned tiles
    const uint32_t epi_stage = ring + STAGES * STAGE_BYTES;       // EPI_WARPS staging tiles, 1024-byte aligned
    uint8_t* aux = smem_raw + (ring - raw_addr) + STAGES * STAGE_BYTES + EPI_WARPS * EPI_STAGE_BYTES;
    const uint32_t aux_addr = epi_stage + EPI_WARPS * EPI_STAGE_BYTES;
    // aux layout (8-byte slots): full[STAGES] | empty[STAGES] | conv[STAGES] | tmem_full[2] | tmem_empty[2] | teardown | slot | abort
    const uint32_t bar_full = aux_addr;
    const uint32_t bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_conv = bar_empty + 8 * STAGES;          // SPLIT: the converter warps have produced hi and lo
    const uint32_t bar_tmem_full = bar_conv + 8 * STAGES;
    const uint32_t bar_tmem_empty = bar_tmem_full + 16;
    const uint32_t bar_teardown = bar_tmem_empty + 16;
    const uint32_t tmem_slot_addr = bar_teardown + 8;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aux + (tmem_slot_addr - aux_addr));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aux + (tmem_slot_addr - aux_addr) + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
            mbar_init(bar_conv + 8 * s, CONVERTER_THREADS / 32);   // one arrival per converter warp
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tmem_full + 8 * i, 1);
            mbar_init(bar_tmem_empty + 8 * i, EPI_WARPS);   // one arrival per epilogue warp
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
        tmem_alloc(tmem_slot_addr, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched only this CTA's shared and tensor memory, so it may overlap the tail of the kernel
    // ahead in the stream; from here on global memory is read and written.
    griddep_launch_dependents();
    griddep_wait();

    const int total_units = p.tiles_m * p.tiles_n * p.num_batches * p.k_splits;
    const int kblocks = (p.K + BK - 1) / BK;

    if (warp == PRODUCER_WARP) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
                WorkUnit w;
                decode_unit(u, p, kblocks, w);
                const int batch = w.batch, m_blk = w.m_blk, n_blk = w.n_blk;
                const int bo = batch / p.batch_inner, bi = batch - bo * p.batch_inner;
                const int a_ci = bi * p.a_mul_inner, a_co = bo * p.a_mul_outer;
                const int b_ci = bi * p.b_mul_inner, b_co = bo * p.b_mul_outer;
                const int m0 = m_blk * BM, n0 = n_blk * BN;
                for (int kb = w.kb0; kb < w.kb1; ++kb, ++issued) {
                    const int s = issued % STAGES;
                    const uint32_t phase = (issued / STAGES) & 1;
                    if (!wait_bounded(bar_empty + 8 * s, phase ^ 1, abort_flag, p.status, WAIT_PRODUCER_EMPTY)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = bar_full + 8 * s;
                    mbar_arrive_expect_tx(full, SPLIT ? STAGE_BYTES / 2 : STAGE_BYTES);
                    const uint32_t sa = ring + s * STAGE_BYTES;
                    const uint32_t sb = sa + NPL * A_PLANE_BYTES;
                    const int k0 = kb * BK;
#pragma unroll
                    for (int pl = 0; pl < (SPLIT ? 1 : NPL); ++pl) {
                        const CUtensorMap* ma = pl ? &tm_a_lo : &tm_a;
                        const CUtensorMap* mb = pl ? &tm_b_lo : &tm_b;
                        if (A_MN) {
#pragma unroll
                            for (int c = 0; c < BM / 32; ++c)
                                tma_load_4d(sa + pl * A_PLANE_BYTES + c * MN_CHUNK_BYTES, ma, full,
                                            m0 + 32 * c, k0, a_ci, a_co);
                        } else {
                            tma_load_4d(sa + pl * A_PLANE_BYTES, ma, full, k0, m0, a_ci, a_co);
                        }
                        if (B_MN) {
#pragma unroll
                            for (int c = 0; c < BN / 32; ++c)
                                tma_load_4d(sb + pl * B_PLANE_BYTES + c * MN_CHUNK_BYTES, mb, full,
                                            n0 + 32 * c, k0, b_ci, b_co);
                        } else {
                            tma_load_4d(sb + pl * B_PLANE_BYTES, mb, full, k0, n0, b_ci, b_co);
                        }
                    }
                }
            }
            if (!ok || *abort_flag) {
                // Drain: copies already issued still write shared memory; wait (bounded) for them.
                const int first = issued > STAGES ? issued - STAGES : 0;
                for (int i = first; i < issued; ++i) {
                    const uint64_t t0 = global_timer_ns();
                    while (!mbar_try_wait(bar_full + 8 * (i % STAGES), (i / STAGES) & 1)) {
                        if (global_timer_ns() - t0 > WAIT_LIMIT_NS) break;
                    }
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int consumed = 0;
            int acc_idx = 0;   // accumulator hand-offs so far (one per tile, or one per K chunk when CHUNKED)
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
                WorkUnit w;
                decode_unit(u, p, kblocks, w);
                int kb = w.kb0;
                do {   // one pass per accumulator buffer: this unit's whole K range, or one chunk of it
                    const int kb_end = CHUNKED ? min(kb + CHUNK_KB, w.kb1) : w.kb1;
                    const int buf = acc_idx & 1;
                    if (!wait_bounded(bar_tmem_empty + 8 * buf, ((acc_idx >> 1) & 1) ^ 1, abort_flag, p.status,
                                      WAIT_MMA_TMEM_EMPTY)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * BN;
                    const int kb_first = kb;
                    for (; kb < kb_end; ++kb, ++consumed) {
                        const int s = consumed % STAGES;
                        if (!wait_bounded((SPLIT ? bar_conv : bar_full) + 8 * s, (consumed / STAGES) & 1, abort_flag, p.status,
                                          WAIT_MMA_FULL)) {
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
                                const uint64_t b_lo = make_smem_desc(sb + B_PLANE_BYTES + j * B_KSTEP, B_LBO, B_SBO, B_LAYOUT);
                                umma_tf32(d_tmem, a_lo, b_hi, IDESC, acc0);   // small terms first
                                umma_tf32(d_tmem, a_hi, b_lo, IDESC, 1);
                                umma_tf32(d_tmem, a_hi, b_hi, IDESC, 1);
                            } else {
                                umma_tf32(d_tmem, a_hi, b_hi, IDESC, acc0);
                            }
                        }
                        umma_commit(bar_empty + 8 * s);   // stage reusable once these MMAs have read it
                    }
                    if (!ok) break;
                    umma_commit(bar_tmem_full + 8 * buf);
                    ++acc_idx;
                } while (kb < w.kb1);
            }
            // All MMAs issued by this thread must be finished before TMEM is freed.
            umma_commit(bar_teardown);
            const uint64_t t0 = global_timer_ns();
            while (!mbar_try_wait(bar_teardown, 0)) {
                if (global_timer_ns() - t0 > WAIT_LIMIT_NS) {
                    atomicCAS(p.status, 0, (int)WAIT_TEARDOWN);
                    break;
                }
            }
        }
    } else if (SPLIT && warp > MMA_WARP) {
        // ------------------------------------------------------------ converters (warps 10-13, SPLIT only)
        // A stage is [A raw->hi | A lo | B raw->hi | B lo]; whatever the operand's layout, the lo plane mirrors the hi
        // plane byte for byte, so the conversion walks both planes as flat arrays of 16-byte pieces.
        const int ct = threadIdx.x - (MMA_WARP + 1) * 32;
        int converted = 0;
        bool ok = true;
        constexpr int A_PIECES = A_PLANE_BYTES / 16 / CONVERTER_THREADS, B_PIECES = B_PLANE_BYTES / 16 / CONVERTER_THREADS;
        // Rows of a K-major A tile past the end of the matrix (a thin M: 16 rows in a 128-row tile) hold the zeros TMA
        // filled in and belong to output rows that are never stored: they are not converted.  Their lo rows are
        // zeroed once here so that the MMAs of those rows read numbers.
        if (!A_MN) {
            for (int st = 0; st < STAGES; ++st) {
                float4* a_lo = reinterpret_cast<float4*>(smem_raw + (ring - raw_addr) + st * STAGE_BYTES) + A_PIECES * CONVERTER_THREADS;
#pragma unroll
                for (int i = 0; i < A_PIECES; ++i) a_lo[ct + i * CONVERTER_THREADS] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
            WorkUnit w;
            decode_unit(u, p, kblocks, w);
            // 16-byte pieces of the A plane that hold rows of the matrix: a row is 128 bytes, rows come in swizzle
            // groups of eight
            int a_valid = A_PIECES * CONVERTER_THREADS;
            if (!A_MN) {
                const long long rows_left = p.M - (long long)w.m_blk * BM;
                if (rows_left < BM) a_valid = (int)((rows_left + 7) / 8) * 64;
            }
            for (int kb = w.kb0; kb < w.kb1 && ok; ++kb, ++converted) {
                const int s = converted % STAGES;
                ok = wait_bounded(bar_full + 8 * s, (converted / STAGES) & 1, abort_flag, p.status, WAIT_CONVERTER_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                // all loads of a plane are issued before the first conversion, so that their latencies overlap
                float4* a_hi = reinterpret_cast<float4*>(smem_raw + (ring - raw_addr) + s * STAGE_BYTES);
                float4* b_hi = a_hi + 2 * (A_PLANE_BYTES / 16);
                auto split_plane = [&](float4* hi_plane, auto pieces_tag, int valid) {
                    constexpr int PIECES = decltype(pieces_tag)::value;      // 16-byte pieces per thread
                    float4* lo_plane = hi_plane + PIECES * CONVERTER_THREADS;
                    float4 x[PIECES];
#pragma unroll
                    for (int i = 0; i < PIECES; ++i)
                        if (ct + i * CONVERTER_THREADS < valid) x[i] = hi_plane[ct + i * CONVERTER_THREADS];
#pragma unroll
                    for (int i = 0; i < PIECES; ++i) {
                        if (ct + i * CONVERTER_THREADS >= valid) continue;
                        float4 hi, lo;
                        hi.x = to_tf32_rn(x[i].x); hi.y = to_tf32_rn(x[i].y); hi.z = to_tf32_rn(x[i].z); hi.w = to_tf32_rn(x[i].w);
                        lo.x = to_tf32_rn_finite(x[i].x - hi.x); lo.y = to_tf32_rn_finite(x[i].y - hi.y);
                        lo.z = to_tf32_rn_finite(x[i].z - hi.z); lo.w = to_tf32_rn_finite(x[i].w - hi.w);
                        hi_plane[ct + i * CONVERTER_THREADS] = hi;
                        lo_plane[ct + i * CONVERTER_THREADS] = lo;
                    }
                };
                split_plane(a_hi, std::integral_constant<int, A_PIECES>{}, a_valid);
                split_plane(b_hi, std::integral_constant<int, B_PIECES>{}, B_PIECES * CONVERTER_THREADS);
                fence_proxy_async_smem();      // the tensor core reads these planes through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_conv + 8 * s);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 0-7)
        int acc_idx = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
            WorkUnit w;
            decode_unit(u, p, kblocks, w);
            const int batch = w.batch, m_blk = w.m_blk, n_blk = w.n_blk;
            const int bo = batch / p.batch_inner, bi = batch - bo * p.batch_inner;
            const int row = m_blk * BM + (warp & 3) * 32 + lane;
            const int n0 = n_blk * BN;
            const long long batch_off = (long long)bo * p.c_stride_outer + (long long)bi * p.c_stride_inner +
                                        (long long)w.split * p.split_stride;
            EpilogueRow er;
            er.c_row = p.c + batch_off + (long long)row * p.ldc;
            er.pre_row = p.preact ? p.preact + batch_off + (long long)row * p.ldc : nullptr;
            er.res_row = p.residual ? p.residual + batch_off + (long long)row * p.ldc : nullptr;
            er.row_ok = row < p.M;
            // 16-byte stores need every row start aligned: aligned batch base and ldc a multiple of 4.
            er.vec_ok = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.c + batch_off) & 15) == 0) &&
                        (!p.preact || (reinterpret_cast<uintptr_t>(p.preact + batch_off) & 15) == 0) &&
                        (!p.residual || (reinterpret_cast<uintptr_t>(p.residual + batch_off) & 15) == 0);
            er.tma_ok = p.tma_store == STORE_TMA;
            er.sector_ok = p.tma_store == STORE_SECTOR;
            er.stage = epi_stage + warp * EPI_STAGE_BYTES;
            er.tm_c = &tm_c;
            er.tm_pre = &tm_pre;
            er.row0 = m_blk * BM + (warp & 3) * 32;
            er.bi = bi;
            er.bo = w.split * p.batch_outer_n + bo;
            if (CHUNKED) {
                // Two-level accumulation: the tensor core sums CHUNK_KB k-blocks in TMEM (its fp32 adder
                // truncates, which biases long sums), the partial sums are then added here in registers with
                // round-to-nearest.  This keeps the 3xTF32 result at FP32 accuracy for any K.
                constexpr int NACC = CHUNKED ? BN / 2 : 1;     // this warp's half of the tile's columns
                const int nh = n0 + (warp >> 2) * (BN / 2);
                float acc[NACC];
#pragma unroll
                for (int j = 0; j < NACC; ++j) acc[j] = 0.0f;
                const int chunks = w.kb1 > w.kb0 ? (w.kb1 - w.kb0 + CHUNK_KB - 1) / CHUNK_KB : 1;
                for (int ch = 0; ch < chunks && ok; ++ch, ++acc_idx) {
                    const int buf = acc_idx & 1;
                    ok = wait_bounded(bar_tmem_full + 8 * buf, (acc_idx >> 1) & 1, abort_flag, p.status,
                                      WAIT_EPI_TMEM_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t t_row = tmem_base + (uint32_t((warp & 3) * 32) << 16) + buf * BN;
                    if (p.K > 0) {
#pragma unroll
                        for (int cc = 0; cc < NACC / 32; ++cc) {
                            if (nh + cc * 32 < p.N) {   // warp-uniform
                                uint32_t r[32];
                                tmem_ld_32x32b_x32(t_row + (warp >> 2) * (BN / 2) + cc * 32, r);
                                tmem_ld_wait();
#pragma unroll
                                for (int j = 0; j < 32; ++j) acc[cc * 32 + j] += __uint_as_float(r[j]);
                            }
                        }
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_tmem_empty + 8 * buf);
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
                const int buf = acc_idx & 1;
                ok = wait_bounded(bar_tmem_full + 8 * buf, (acc_idx >> 1) & 1, abort_flag, p.status,
                                  WAIT_EPI_TMEM_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t t_row = tmem_base + (uint32_t((warp & 3) * 32) << 16) + buf * BN;
#pragma unroll 1
                for (int cc = (warp >> 2) * (BN / 64); cc < ((warp >> 2) + 1) * (BN / 64); ++cc) {
                    const int col0 = n0 + cc * 32;
                    if (col0 >= p.N) break;   // warp-uniform
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
                // Hand the accumulator buffer back to the MMA warp.
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tmem_empty + 8 * buf);
                ++acc_idx;
            }
        }
    }

    if (warp < EPI_WARPS && lane == 0) bulk_wait_all();   // this warp's output stores are complete
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host side ---

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

// A training step encodes the same few hundred maps again every iteration (same pointers, shapes and strides); the
// context keeps the last encodings in a small direct-mapped table so that a repeat costs a hash and a 128-byte copy
// instead of a driver call.  The key holds every argument of the encoder, so a hit is exact.
int encode_tiled_cached(te_b200_ctx* ctx, void* out_map, const void* ptr, const uint64_t dims[4], const uint64_t strides[3],
                        const uint32_t box[4], int swizzle, int l2_promotion) {
    uint64_t key[16] = {reinterpret_cast<uint64_t>(ptr), dims[0], dims[1], dims[2], dims[3], strides[0], strides[1], strides[2],
                        (uint64_t)box[0] | ((uint64_t)box[1] << 32), (uint64_t)box[2] | ((uint64_t)box[3] << 32),
                        (uint64_t)(uint32_t)swizzle | ((uint64_t)(uint32_t)l2_promotion << 32), 0, 0, 0, 0, 0};
    uint64_t h = 0x9E3779B97F4A7C15ull;
    for (int i = 0; i < 11; ++i) h = (h ^ key[i]) * 0xFF51AFD7ED558CCDull, h ^= h >> 29;
    TensorMapCacheEntry& e = ctx->tmap_cache[h & 255];
    if (e.valid && memcmp(e.key, key, sizeof key) == 0) {
        memcpy(out_map, e.map, 128);
        ctx->tmap_hits += 1;
        return 0;
    }
    cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
    cuuint64_t st[3] = {strides[0], strides[1], strides[2]};
    cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMap m;
    EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), d, st, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    (CUtensorMapSwizzle)swizzle, (CUtensorMapL2promotion)l2_promotion, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return (int)r;
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    memcpy(out_map, &m, 128);
    memcpy(e.key, key, sizeof key);
    memcpy(e.map, &m, 128);
    e.valid = true;
    ctx->tmap_misses += 1;
    return 0;
}

bool operand_tma_ok(const Operand& op, int64_t K, int64_t batch_inner, int64_t batch_outer) {
    if (reinterpret_cast<uintptr_t>(op.ptr) & 15) return false;
    const int64_t strided_extent = op.mn_major ? K : op.rows;
    if (strided_extent > 1 && (op.ld & 3)) return false;   // the pitch of a single-line slice is never used
    if (batch_inner > 1 && (op.stride_inner & 3)) return false;
    if (batch_outer > 1 && (op.stride_outer & 3)) return false;
    return true;
}

// 4-D map {contiguous index, strided index, batch_inner, batch_outer}.  Broadcast (stride 0) levels get
// extent 1; the kernel multiplies their coordinate by 0.
int make_operand_map(te_b200_ctx* ctx, CUtensorMap* out, const float* ptr, const Operand& op,
                            int64_t K, int box_rows, int64_t batch_inner, int64_t batch_outer) {
    const int64_t k_extent = K > 0 ? K : 1;   // K == 0 issues no loads but the map must still be valid
    const int64_t contiguous_extent = op.mn_major ? op.rows : k_extent;
    const int64_t strided_extent = op.mn_major ? k_extent : op.rows;
    const int64_t e2 = (batch_inner > 1 && op.stride_inner != 0) ? batch_inner : 1;
    const int64_t e3 = (batch_outer > 1 && op.stride_outer != 0) ? batch_outer : 1;
    const uint64_t dims[4] = {(uint64_t)contiguous_extent, (uint64_t)strided_extent, (uint64_t)e2, (uint64_t)e3};
    // A slice with one line may carry any pitch; the map still needs a legal one.
    const int64_t ld = strided_extent > 1 ? op.ld : ((contiguous_extent + 3) & ~int64_t(3));
    const uint64_t row_bytes = (uint64_t)ld * 4;
    const uint64_t strides[3] = {row_bytes,
                                 e2 > 1 ? (uint64_t)op.stride_inner * 4 : row_bytes,
                                 e3 > 1 ? (uint64_t)op.stride_outer * 4 : row_bytes};
    const uint32_t box[4] = {(uint32_t)BK, (uint32_t)(op.mn_major ? BK : box_rows), 1, 1};
    const int r = encode_tiled_cached(ctx, out, ptr, dims, strides, box,
                                      (int)(op.mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B),
                                      (int)CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (r != 0) {
        char msg[256];
        snprintf(msg, sizeof msg,
                 "cuTensorMapEncodeTiled failed (%d): dims {%llu,%llu,%llu,%llu} ld %lld ptr %p", r,
                 (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
                 (unsigned long long)dims[3], (long long)op.ld, (const void*)ptr);
        set_error(msg);
        return TE_ERR_CUDA;
    }
    return TE_OK;
}

static bool make_one_output_map(te_b200_ctx* ctx, CUtensorMap* out, float* ptr, const GemmProblem& g, int k_splits) {
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return false;
    if (g.N & 3) return false;   // the store unit clips a row at 16-byte granularity: a ragged last quad would spill past N
    if (g.M > 1 && (g.ldc & 3)) return false;
    if (g.batch_inner > 1 && ((g.c_stride_inner & 3) || g.c_stride_inner == 0)) return false;
    if (g.batch_outer * k_splits > 1 && ((g.c_stride_outer & 3) || g.c_stride_outer == 0)) return false;
    const int64_t ld = g.M > 1 ? g.ldc : ((g.N + 3) & ~int64_t(3));
    // split-K scratch is laid out [split][outer][inner][M][N] dense, so splits extend the outer batch dimension
    const int64_t outer_n = g.batch_outer * k_splits;
    const uint64_t dims[4] = {(uint64_t)g.N, (uint64_t)g.M, (uint64_t)g.batch_inner, (uint64_t)outer_n};
    const uint64_t row_bytes = (uint64_t)ld * 4;
    const uint64_t strides[3] = {row_bytes, g.batch_inner > 1 ? (uint64_t)g.c_stride_inner * 4 : row_bytes,
                                 outer_n > 1 ? (uint64_t)g.c_stride_outer * 4 : row_bytes};
    const uint32_t box[4] = {32, 32, 1, 1};
    return encode_tiled_cached(ctx, out, ptr, dims, strides, box, (int)CU_TENSOR_MAP_SWIZZLE_128B,
                               (int)CU_TENSOR_MAP_L2_PROMOTION_NONE) == 0;
}

bool make_output_maps(te_b200_ctx* ctx, const GemmProblem& g, int k_splits, CUtensorMap* tm_c, CUtensorMap* tm_pre) {
    if (!make_one_output_map(ctx, tm_c, g.c, g, k_splits)) return false;
    if (g.preact) {
        if (!make_one_output_map(ctx, tm_pre, g.preact, g, k_splits)) return false;
    } else {
        *tm_pre = *tm_c;
    }
    return true;
}

// 32-byte stores need every row start on a sector boundary.
static bool sector_store_ok(const GemmProblem& g, int k_splits) {
    auto ok_ptr = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 31) == 0; };
    if ((g.N & 7) || !ok_ptr(g.c) || (g.preact && !ok_ptr(g.preact))) return false;
    if (g.M > 1 && (g.ldc & 7)) return false;
    if (g.batch_inner > 1 && (g.c_stride_inner & 7)) return false;
    if (g.batch_outer * k_splits > 1 && (g.c_stride_outer & 7)) return false;
    return true;
}

#ifndef TE_PREFER_SECTOR_STORES
#define TE_PREFER_SECTOR_STORES 0
#endif

int choose_store_mode(te_b200_ctx* ctx, const GemmProblem& g, int k_splits, CUtensorMap* tm_c, CUtensorMap* tm_pre) {
    const bool tma = make_output_maps(ctx, g, k_splits, tm_c, tm_pre);
    const bool sector = sector_store_ok(g, k_splits);
    if (!tma) {
        // the kernels take tensor maps as parameters whether they use them or not
        memset(tm_c, 0, sizeof(CUtensorMap));
        memset(tm_pre, 0, sizeof(CUtensorMap));
    }
    if (sector && (TE_PREFER_SECTOR_STORES || !tma)) return STORE_SECTOR;
    return tma ? STORE_TMA : STORE_DIRECT;
}

void fill_common_params(GemmParams& p, const te_b200_ctx* ctx, const GemmProblem& g) {
    p.tma_store = 0;
    p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K;
    p.tiles_m = p.tiles_n = 0;
    p.batch_inner = (int)g.batch_inner;
    p.num_batches = (int)(g.batch_inner * g.batch_outer);
    p.a_mul_inner = (g.batch_inner > 1 && g.a.stride_inner != 0) ? 1 : 0;
    p.a_mul_outer = (g.batch_outer > 1 && g.a.stride_outer != 0) ? 1 : 0;
    p.b_mul_inner = (g.batch_inner > 1 && g.b.stride_inner != 0) ? 1 : 0;
    p.b_mul_outer = (g.batch_outer > 1 && g.b.stride_outer != 0) ? 1 : 0;
    p.ldc = g.ldc; p.c_stride_inner = g.c_stride_inner; p.c_stride_outer = g.c_stride_outer;
    p.c = g.c; p.preact = g.preact; p.bias = g.bias; p.residual = g.residual;
    p.alpha = g.alpha; p.scale_mode = g.scale_mode; p.epilogue = g.epilogue;
    p.status = ctx->d_status;
    p.k_splits = 1;
    p.kb_per_split = (int)((g.K + BK - 1) / BK);
    p.batch_outer_n = (int)g.batch_outer;
    p.split_stride = 0;
}

void prepare_split(const GemmProblem& g, int k_splits, GemmProblem& kp, GemmParams& p) {
    if (k_splits <= 1) return;
    const int kblocks = (int)((g.K + BK - 1) / BK);
    const int64_t batches = g.batch_inner * g.batch_outer;
    // the kernel writes raw sums into dense scratch [split][outer][inner][M][N]; the epilogue runs in the reduction
    kp.c = g.split_ws;
    kp.ldc = g.N;
    kp.c_stride_inner = g.M * g.N;
    kp.c_stride_outer = g.batch_inner * g.M * g.N;
    kp.preact = nullptr; kp.bias = nullptr; kp.residual = nullptr; kp.scale_mode = TE_SCALE_NONE; kp.epilogue = TE_EPI_NONE;
    p.c = kp.c; p.ldc = kp.ldc; p.c_stride_inner = kp.c_stride_inner; p.c_stride_outer = kp.c_stride_outer;
    p.preact = nullptr; p.bias = nullptr; p.residual = nullptr; p.scale_mode = TE_SCALE_NONE; p.epilogue = TE_EPI_NONE;
    p.k_splits = k_splits;
    p.kb_per_split = (kblocks + k_splits - 1) / k_splits;
    p.split_stride = batches * g.M * g.N;
}

// out = epilogue( sum over splits, in split order, of the partial tiles ): deterministic, streaming, HBM-bound.
struct SplitReduceParams {
    const float* partial;
    long long split_stride;
    int k_splits;
    long long M, N, batch_inner, total;       // total = batches * M * N
    float* c; float* preact; const float* bias; const float* residual;
    long long ldc, c_stride_inner, c_stride_outer;
    float alpha; int scale_mode; int epilogue;
};

// VEC = 4: N, ldc and the batch strides are multiples of 4 and every pointer is 16-byte aligned, so a thread owns four
// consecutive columns of one row.  The partial tiles sit in L2 (they were just written); what a thread waits for is
// the latency of its loads, so four splits are fetched before the first is added -- in split order all the same.
template <int VEC>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const SplitReduceParams r) {
    griddep_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long total_v = r.total / VEC;
    // the output is one dense block in the order of the partial tiles: no index arithmetic beyond the column
    const bool dense = r.ldc == r.N && (r.total == r.M * r.N ||
                                        (r.c_stride_inner == r.M * r.N &&
                                         (r.total == r.batch_inner * r.M * r.N || r.c_stride_outer == r.batch_inner * r.M * r.N)));
    for (long long iv = (long long)blockIdx.x * blockDim.x + threadIdx.x; iv < total_v; iv += stride) {
        const long long i = iv * VEC;
        float v[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[e] = 0.0f;
        auto fetch = [&](int s, float* dst) {
            const float* src = r.partial + s * r.split_stride + i;
            if (VEC == 4) {
                const float4 t = *reinterpret_cast<const float4*>(src);
                dst[0] = t.x; dst[1] = t.y; dst[2] = t.z; dst[3] = t.w;
            } else {
                dst[0] = *src;
            }
        };
        int s = 0;
        for (; s + 4 <= r.k_splits; s += 4) {
            float t0[VEC], t1[VEC], t2[VEC], t3[VEC];
            fetch(s, t0); fetch(s + 1, t1); fetch(s + 2, t2); fetch(s + 3, t3);
#pragma unroll
            for (int e = 0; e < VEC; ++e) { v[e] += t0[e]; v[e] += t1[e]; v[e] += t2[e]; v[e] += t3[e]; }
        }
        for (; s < r.k_splits; ++s) {
            float t0[VEC];
            fetch(s, t0);
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] += t0[e];
        }
        long long n, o;
        if (r.total <= 0x7fffffffLL) {      // 32-bit index arithmetic where it fits
            const unsigned iu = (unsigned)i, N = (unsigned)r.N, M = (unsigned)r.M;
            const unsigned rowb = iu / N;
            n = iu - rowb * N;
            if (dense) {
                o = i;
            } else {
                const unsigned batch = rowb / M, row = rowb - batch * M;
                const unsigned bo = batch / (unsigned)r.batch_inner, bi = batch - bo * (unsigned)r.batch_inner;
                o = bo * r.c_stride_outer + bi * r.c_stride_inner + (long long)row * r.ldc + n;
            }
        } else {
            n = i % r.N;
            const long long row = (i / r.N) % r.M, batch = i / (r.N * r.M);
            const long long bo = batch / r.batch_inner, bi = batch - bo * r.batch_inner;
            o = bo * r.c_stride_outer + bi * r.c_stride_inner + row * r.ldc + n;
        }
        if (r.scale_mode == TE_SCALE_MUL) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] *= r.alpha;
        } else if (r.scale_mode == TE_SCALE_DIV) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = v[e] / r.alpha;
        }
        if (r.bias) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] += r.bias[n + e];
        }
        auto store = [&](float* base) {
            if (VEC == 4) *reinterpret_cast<float4*>(base + o) = make_float4(v[0], v[1], v[2], v[3]);
            else base[o] = v[0];
        };
        if (r.preact) store(r.preact);
        if (r.epilogue == TE_EPI_BIAS_GELU) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = gelu_tanh(v[e]);
        }
        if (r.residual) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] += r.residual[o + e];
        }
        store(r.c);
    }
}

int finish_split(te_b200_ctx* ctx, const GemmProblem& g, int k_splits, cudaStream_t stream) {
    SplitReduceParams r;
    r.partial = g.split_ws;
    r.M = g.M; r.N = g.N; r.batch_inner = g.batch_inner;
    r.total = g.batch_inner * g.batch_outer * g.M * g.N;
    r.split_stride = r.total;
    r.k_splits = k_splits;
    r.c = g.c; r.preact = g.preact; r.bias = g.bias; r.residual = g.residual;
    r.ldc = g.ldc; r.c_stride_inner = g.c_stride_inner; r.c_stride_outer = g.c_stride_outer;
    r.alpha = g.alpha; r.scale_mode = g.scale_mode; r.epilogue = g.epilogue;
    const uintptr_t ptr_bits = reinterpret_cast<uintptr_t>(r.partial) | reinterpret_cast<uintptr_t>(r.c) | reinterpret_cast<uintptr_t>(r.preact) |
                               reinterpret_cast<uintptr_t>(r.bias) | reinterpret_cast<uintptr_t>(r.residual);
    const bool vec = ((r.N | r.ldc | r.c_stride_inner | r.c_stride_outer) & 3) == 0 && (ptr_bits & 15) == 0;
    long long blocks = (r.total / (vec ? 4 : 1) + 255) / 256;
    if (blocks > (long long)ctx->sm_count * 16) blocks = (long long)ctx->sm_count * 16;
    if (blocks < 1) blocks = 1;
    if (vec) launch_pdl(splitk_reduce_kernel<4>, dim3((unsigned)blocks), dim3(256), 0, stream, r);
    else launch_pdl(splitk_reduce_kernel<1>, dim3((unsigned)blocks), dim3(256), 0, stream, r);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "splitk_reduce_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

// One-time set-up of a kernel instance in this context: the dynamic shared memory limit (which also makes the
// runtime load the kernel's module).
template <int BN, int NPL, bool A_MN, bool B_MN, bool SPLIT = false>
static int ensure_kernel_attributes(te_b200_ctx* ctx) {
    using Cfg = TileCfg<BN, NPL>;
    // 3xTF32 (NPL = 2) has one instance, which carries the residual input; TF32 has all three epilogue forms
    int& attr_done = ctx->kernel_state[reinterpret_cast<const void*>(gemm_tf32_kernel<BN, NPL, A_MN, B_MN, EPI_RESIDUAL, SPLIT>)];
    if (attr_done) return TE_OK;
    cudaError_t e = cudaFuncSetAttribute(gemm_tf32_kernel<BN, NPL, A_MN, B_MN, EPI_RESIDUAL, SPLIT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e == cudaSuccess && NPL == 1)
        e = cudaFuncSetAttribute(gemm_tf32_kernel<BN, 1, A_MN, B_MN, EPI_PLAIN>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, TileCfg<BN, 1>::SMEM_BYTES);
    if (e == cudaSuccess && NPL == 1)
        e = cudaFuncSetAttribute(gemm_tf32_kernel<BN, 1, A_MN, B_MN, EPI_GENERAL>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, TileCfg<BN, 1>::SMEM_BYTES);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(max dynamic shared memory)");
    attr_done = 1;
    return TE_OK;
}

int prepare_3xtf32_kernels(te_b200_ctx* ctx) {
    int rc;
    if ((rc = ensure_kernel_attributes<64, 2, false, false>(ctx))) return rc;
    if ((rc = ensure_kernel_attributes<128, 2, false, false>(ctx))) return rc;
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, splitk_reduce_kernel<4>);      // loads the kernel
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, splitk_reduce_kernel<1>);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncGetAttributes(splitk_reduce_kernel)");
    if ((rc = prepare_pair_3xtf32_kernel(ctx))) return rc;
    return prepare_pack_kernels();
}

template <int BN, int NPL, bool A_MN, bool B_MN, bool SPLIT = false>
static int launch_variant(te_b200_ctx* ctx, const GemmProblem& g_in, int k_splits, cudaStream_t stream) {
    GemmProblem g = g_in;
    using Cfg = TileCfg<BN, NPL>;
    if (int rc0 = ensure_kernel_attributes<BN, NPL, A_MN, B_MN, SPLIT>(ctx)) return rc0;
    CUtensorMap ma, mal, mb, mbl;
    int rc;
    if ((rc = make_operand_map(ctx, &ma, g.a.ptr, g.a, g.K, BM, g.batch_inner, g.batch_outer))) return rc;
    if ((rc = make_operand_map(ctx, &mb, g.b.ptr, g.b, g.K, BN, g.batch_inner, g.batch_outer))) return rc;
    if (NPL == 2 && !SPLIT) {
        if ((rc = make_operand_map(ctx, &mal, g.a_lo, g.a, g.K, BM, g.batch_inner, g.batch_outer))) return rc;
        if ((rc = make_operand_map(ctx, &mbl, g.b_lo, g.b, g.K, BN, g.batch_inner, g.batch_outer))) return rc;
    } else {
        mal = ma;
        mbl = mb;
    }
    GemmParams p;
    fill_common_params(p, ctx, g);
    prepare_split(g_in, k_splits, g, p);       // with k_splits > 1 the kernel writes raw partial tiles to scratch
    CUtensorMap mc, mpre;
    p.tma_store = choose_store_mode(ctx, g, k_splits, &mc, &mpre);
    p.tiles_m = (int)((g.M + BM - 1) / BM);
    p.tiles_n = (int)((g.N + BN - 1) / BN);
    const long long total = (long long)p.tiles_m * p.tiles_n * p.num_batches * k_splits;
    const int grid = (int)(total < ctx->sm_count ? total : ctx->sm_count);
    // The bare-product kernel serves the calls whose output a tensor map describes and that ask for nothing but the
    // product (split-K partial tiles included).
    const bool bare = NPL == 1 && p.tma_store &&
                      (k_splits > 1 || (!g.bias && !g.preact && !g.residual && g.scale_mode == TE_SCALE_NONE && g.epilogue == TE_EPI_NONE));
    auto kernel = gemm_tf32_kernel<BN, NPL, A_MN, B_MN, EPI_RESIDUAL, SPLIT>;
    if constexpr (NPL == 1) {
        if (bare) kernel = gemm_tf32_kernel<BN, 1, A_MN, B_MN, EPI_PLAIN>;
        else if (!p.residual) kernel = gemm_tf32_kernel<BN, 1, A_MN, B_MN, EPI_GENERAL>;
    }
    const int threads = SPLIT ? CTA_THREADS + CONVERTER_THREADS : CTA_THREADS;
    cudaError_t e = launch_pdl(kernel, dim3((unsigned)grid), dim3(threads), Cfg::SMEM_BYTES, stream, ma, mal, mb, mbl, mc, mpre, p);
    if (e != cudaSuccess) return cuda_fail(e, "gemm_tf32_kernel launch");
    ctx->launches += 1;
    return k_splits > 1 ? finish_split(ctx, g_in, k_splits, stream) : TE_OK;
}

template <int BN>
static int launch_bn(te_b200_ctx* ctx, const GemmProblem& g, int k_splits, cudaStream_t stream) {
    if (g.split_in_kernel) {   // 3xTF32 on the operands as they are: the kernel splits hi / lo in shared memory
        constexpr int B2 = BN <= 128 ? BN : 128;
        if (!g.a.mn_major && !g.b.mn_major) return launch_variant<B2, 2, false, false, true>(ctx, g, k_splits, stream);
        if (!g.a.mn_major && g.b.mn_major) return launch_variant<B2, 2, false, true, true>(ctx, g, k_splits, stream);
        if (g.a.mn_major && !g.b.mn_major) return launch_variant<B2, 2, true, false, true>(ctx, g, k_splits, stream);
        return launch_variant<B2, 2, true, true, true>(ctx, g, k_splits, stream);
    }
    if (g.a_lo) {   // 3xTF32 on packed planes (always K-major)
        if constexpr (BN <= 128) return launch_variant<BN, 2, false, false>(ctx, g, k_splits, stream);
        else return launch_variant<128, 2, false, false>(ctx, g, k_splits, stream);
    }
    if (!g.a.mn_major && !g.b.mn_major) return launch_variant<BN, 1, false, false>(ctx, g, k_splits, stream);
    if (!g.a.mn_major && g.b.mn_major) return launch_variant<BN, 1, false, true>(ctx, g, k_splits, stream);
    if (g.a.mn_major && !g.b.mn_major) return launch_variant<BN, 1, true, false>(ctx, g, k_splits, stream);
    return launch_variant<BN, 1, true, true>(ctx, g, k_splits, stream);
}

// Tile-shape choice.  Larger tiles move fewer bytes into shared memory per flop (the pair tile least of all) but
// give fewer tiles; with too few tiles most SMs idle.  The estimate below is waves x (k-blocks x time per k-block
// + a fixed per-tile cost) with per-k-block times measured on 8192^3 for each shape (ns): they encode that the
// small shapes are bound by filling shared memory, not by the tensor pipe.  When a problem has few tiles but a long
// K (a thin M, a weight gradient over many tokens), K is additionally split over several work units per tile.

TileChoice choose_tile(const te_b200_ctx* ctx, const GemmProblem& g_in) {
    // 3xTF32 is recognised by its lo planes; a problem that is split inside the kernel has none but is costed the same
    // way and is limited to the single-CTA kernel
    GemmProblem g = g_in;
    static const float three_x_marker = 0.0f;
    if (g.split_in_kernel) g.a_lo = &three_x_marker;
    const int kblocks = (int)((g.K + BK - 1) / BK);
    const double batches = (double)(g.batch_inner * g.batch_outer);
    // ns per k-block of one tile in TF32 mode and in 3xTF32 mode (two planes per operand, three MMAs per k-step,
    // fewer and larger pipeline stages), fixed ns per tile
    struct Cand { int bn; bool pair; double ns_per_kblock; double ns_per_kblock_3x; double fixed_ns; };
    // (the 256 x 192 pair tile exists for N = 384 and the like, where 256-wide tiles would be a quarter padding;
    // measured on 16384x384x384: 16.3 us against 18.0 us.  The wide pair tiles -- 256 x 512 and 256 x 384, two
    // accumulators side by side, A fetched once for both -- move a third fewer bytes per flop into shared memory but
    // cannot overlap the epilogue with the next tile: 8192^3 1.55 ms against 1.78 ms, 4096^3 0.190 against 0.214 ms,
    // 8192x512x8192 0.169 against 0.140 ms; their figures below are fitted to those ratios.)
    const Cand cands[7] = {{256, true, 405.0, 1400.0, 3000.0}, {512, true, 695.0, 1e9, 8300.0}, {384, true, 618.0, 1e9, 8300.0},
                           {192, true, 355.0, 1e9, 3000.0}, {256, false, 432.0, 1e9, 3000.0},
                           {128, false, 350.0, 804.0, 2000.0}, {64, false, 291.0, 520.0, 1500.0}};
    const int split_options[8] = {1, 2, 3, 4, 6, 8, 12, 16};
    const double out_bytes = batches * (double)g.M * (double)g.N * 4.0;
    TileChoice best{64, false, 1};
    double best_t = 1e300;
    for (const Cand& c : cands) {
        if (c.pair && (g.M <= 128 || g.N <= 128 || g.split_in_kernel)) continue;
        if (c.pair && g.a_lo && kblocks < 160) continue;         // measured: the 3-stage pair form of 3xTF32 pays off from K ~ 5000
        if (g.a_lo && !c.pair && c.bn > 128) continue;           // 3xTF32, single CTA: two 96 KB stages would be too few
        if (g.a_lo && c.pair && c.bn != 256) continue;           // 3xTF32 pair form exists for 256-wide tiles only
        // wide tiles: the exposed epilogue needs a long main loop to pay (measured: 8192x1024x8192 and 16384x1024x4096
        // lose 4-20 % with them, 4096x2048x4096 gains 20 %, everything from K = 4096 on gains 13-30 %)
        if (c.bn > 256 && kblocks < 64) {
            // ... except a single wave of 256 x 384 tiles, whose epilogue is exposed only once (16384x1536x384: 37.5 us
            // against 40.7 us with 192-wide tiles)
            const long long wide_tiles = ((g.M + 255) / 256) * ((g.N + c.bn - 1) / c.bn) * (long long)batches;
            if (!(c.bn == 384 && kblocks >= 32 && wide_tiles <= ctx->sm_count / 2)) continue;
        }
        if (c.bn > 64 && g.N <= c.bn / 2) continue;              // more than half of the tile would be padding
        const double tm = (double)((g.M + (c.pair ? 255 : 127)) / (c.pair ? 256 : 128));
        const double tn = (double)((g.N + c.bn - 1) / c.bn);
        const double tiles = tm * tn * batches;
        const double slots = c.pair ? ctx->sm_count / 2 : ctx->sm_count;
        const double ns_kb = g.a_lo ? c.ns_per_kblock_3x : c.ns_per_kblock;
        const double fixed = g.a_lo && c.pair ? 2.0 * c.fixed_ns : c.fixed_ns;
        for (int S : split_options) {
            if (S > 1) {
                // every split needs a few k-blocks of its own, the scratch must hold S copies of the output, and the
                // last split must not be empty
                if (kblocks < 4 * S || !g.split_ws || out_bytes * S > (double)g.split_ws_bytes) break;
                const int per = (kblocks + S - 1) / S;
                if ((S - 1) * per >= kblocks) continue;
            }
            const double units = tiles * S;
            const double waves = (double)(long long)((units + slots - 1) / slots);
            const double kb_unit = (double)((kblocks + S - 1) / S);
            double t = waves * (kb_unit * ns_kb + fixed);
            if (S > 1) t += 4000.0 + out_bytes * (S + 1) / 4000.0;     // reduction: launch + (S reads + 1 write) at ~4 TB/s
            if (t < best_t) { best_t = t; best = TileChoice{c.bn, c.pair, S}; }
        }
    }
    return best;
}

// Self-test of the bounded wait every kernel of the library uses: one warp initialises an mbarrier that nothing ever
// arrives at and waits on it.  The wait runs out after the context's limit, records STATUS_SELFTEST_WAIT in the status
// word and the kernel returns normally -- no trap, no fault, the context stays usable.
__global__ void __launch_bounds__(32) wait_selftest_kernel(int* status) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    griddep_wait();
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_barrier_init();
        wait_bounded(smem_u32(&bar), 0, &abort_flag, status, STATUS_SELFTEST_WAIT);
    }
}

int launch_wait_selftest(te_b200_ctx* ctx, cudaStream_t stream) {
    cudaError_t e = launch_pdl(wait_selftest_kernel, dim3(1), dim3(32), 0, stream, ctx->d_status);
    if (e != cudaSuccess) return cuda_fail(e, "wait_selftest_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

int launch_gemm(te_b200_ctx* ctx, const GemmProblem& g, cudaStream_t stream) {
    const TileChoice c = choose_tile(ctx, g);
    if (c.pair) return launch_gemm_2cta(ctx, g, c.bn, c.k_splits, stream);
    if (c.bn == 256) return launch_bn<256>(ctx, g, c.k_splits, stream);
    if (c.bn == 128) return launch_bn<128>(ctx, g, c.k_splits, stream);
    return launch_bn<64>(ctx, g, c.k_splits, stream);
}

}  // namespace te
