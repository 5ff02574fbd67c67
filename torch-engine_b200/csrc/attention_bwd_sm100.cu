// Fused backward of the scaled-dot attention for sm_100a: from dO, the saved probabilities P and Q, K, V, O it produces
// dQ, dK and dV of one (batch, head) per tile without writing dP or dS to global memory.
//
// Reference semantics: the backward graph of ScaledDot::forward (reference src/nn/scaledot.cpp:8-27):
//   MatMulBackward of P.V      dV = P^T.dO,  dP = dO.V^T                     (src/core/grad_fn.cpp:126-139)
//   SoftmaxBackward            dZ = P o (dP - rowsum(P o dP))                (src/core/grad_fn.cpp:569-665)
//   DivBackward                dS = dZ / sqrt(d)                             (src/core/grad_fn.cpp:142-156)
//   MatMulBackward of Q.K^T    dQ = dS.K,    dK = dS^T.Q
// rowsum(P o dP) equals rowsum(dO o O) (O = P.V), which needs no reduction over keys.
//
// Why fused: unfused, the [B,H,T,T] tensors cross HBM eight times (P twice, dP written, read and rewritten as dS, dS
// read twice) against once here (P), beside the [B,H,T,d] operands.
//
// Everything is computed in the transposed frame, with KEYS on the 128 TMEM lanes, so that the two products whose
// left operand is transposed (P^T.dO and dS^T.Q) take it straight from tensor memory.  For key block j and query block
// i (128 x 128 each; T <= 256, so at most 2 x 2 steps per tile):
//   MMA 1   dP^T = V_j . dO_i^T                        -> TMEM columns [0,128)
//   warps   P^T from global memory (lane = key: a warp reads 128 contiguous bytes of one row of P), then
//           dS^T = P^T o (dP^T - D_query) / sqrt(d)    -> TMEM [0,128) in place, P^T -> TMEM [128,256),
//           and dS^T also into shared memory in the M-major operand layout (for dQ, whose left operand is dS)
//   MMA 2   dQ_i += dS   . K_j    (A from shared)      -> TMEM [384 + 64 i, ..)
//   MMA 3   dV_j += P^T  . dO_i   (A from TMEM)        -> TMEM [256,320)
//   MMA 4   dK_j += dS^T . Q_i    (A from TMEM)        -> TMEM [320,384)
// The dQ product goes first because it is the only reader of the dS^T tile in shared memory: once it is done the next
// step's block of P may land there, while MMAs 3 and 4 are still running.
// A tile is one head (all key blocks in turn) or, when that fills the SMs better (p.split_keys; for example 192 heads
// on 148 SMs), one (head, key block): dV_j / dK_j are complete either way, and the two tiles of a head add their dQ
// onto memory that the row-dot pre-pass has filled with zeros (cp.reduce.async.bulk, fp32 add): with exactly two
// addends per element the result does not depend on which arrives first.
// dV_j and dK_j leave after the last query block, dQ after the last key block, through TMA stores staged in the
// dO / Q operand buffers (free at that point; for d = 32 they are too small and the dS^T region is used instead).
// Warp roles as in the forward kernel: warp 8 TMA producer, warp 9 MMA issue, warps 0-7 element work and output
// (warp w: TMEM lanes 32 (w % 4).., query-column half w / 4).  All waits are bounded.
// Limits: TF32 mode, T <= 256, T % 4 == 0, d in {32, 64}; other problems take the GEMM sequence.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "gemm_common.cuh"

namespace te {

constexpr int BWD_COL_DP = 0;
constexpr int BWD_COL_P = 128;
constexpr int BWD_COL_DV = 256;
constexpr int BWD_COL_DK = 320;
constexpr int BWD_COL_DQ = 384;
constexpr int BWD_CHUNK = 128 * 128;     // bytes of one [128 rows x 32 floats] operand chunk

struct AttnBwdParams {
    int T, d, H, B;
    int nblk;          // 128-row blocks per head (1 or 2)
    int split_keys;    // 1: a tile is one (head, key block) and dQ is added onto zero-filled memory by the two tiles of a head
    int total_tiles;   // B * H, or B * H * nblk with split_keys
    float inv_scale;   // 1 / sqrt(d)
    int pbox;          // rows and columns of the P box: min(T, 128)
    const float* dvec; // [B,H,T]: rowsum(dO o O), written by rowdot_bht_kernel
    int* status;
};

// D[b,h,t] = sum_c dO[b,h,t,c] * O[b,h,t,c] (= rowsum(P o dP), the inner product SoftmaxBackward subtracts).  A row is
// d/4 float4 wide, so one warp instruction covers 32/(d/4) whole rows; partial dot products meet by shuffles.
// `zero` (optional): a third [B,H,T,d] view that is filled with zeros in the same pass (the dQ buffer when two tiles
// per head add their parts onto it).
__global__ void __launch_bounds__(256) rowdot_bht_kernel(const float* __restrict__ x, long long xs0, long long xs1, long long xs2,
                                                         const float* __restrict__ y, long long ys0, long long ys1, long long ys2,
                                                         float* __restrict__ out, int H, int T, int d, long long rows,
                                                         float* __restrict__ zero, long long zs0, long long zs1, long long zs2) {
    griddep_wait();
    const int lane = threadIdx.x & 31;
    const int f4 = d >> 2, rpi = 32 / f4;
    const int sub = lane / f4, col = lane - sub * f4;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long g = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); g * rpi < rows; g += warps) {
        const long long r = g * rpi + sub;
        float acc = 0.0f;
        if (r < rows) {
            const long long bh = r / T;
            const int t = (int)(r - bh * T), h = (int)(bh % H);
            const long long b = bh / H;
            const float4 a = __ldg(reinterpret_cast<const float4*>(x + b * xs0 + h * xs1 + t * xs2) + col);
            const float4 c = __ldg(reinterpret_cast<const float4*>(y + b * ys0 + h * ys1 + t * ys2) + col);
            acc = a.x * c.x + a.y * c.y + a.z * c.z + a.w * c.w;
            if (zero) reinterpret_cast<float4*>(zero + b * zs0 + h * zs1 + t * zs2)[col] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int off = f4 >> 1; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (col == 0 && r < rows) out[r] = acc;
    }
}

__global__ void __launch_bounds__(CTA_THREADS, 1)
attention_bwd_tf32_kernel(const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_dok, const __grid_constant__ CUtensorMap tm_dom,
                          const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_dq,
                          const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                          const __grid_constant__ CUtensorMap tm_p, const AttnBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    const int dchunks = p.d / 32;
    const uint32_t opnd = dchunks * BWD_CHUNK;                 // bytes of one [128 x d] operand tile
    const uint32_t v_smem = base;                              // V_j, K-major           (A of MMA 1)
    const uint32_t k_smem = v_smem + opnd;                     // K_j, N-major 32x32 boxes (B of MMA 4)
    const uint32_t dok_smem = k_smem + opnd;                   // dO_i, K-major          (B of MMA 1)
    const uint32_t dom_smem = dok_smem + opnd;                 // dO_i, N-major          (B of MMA 2)
    const uint32_t q_smem = dom_smem + opnd;                   // Q_i, N-major           (B of MMA 3)
    const uint32_t ds_smem = q_smem + opnd;                    // dS^T as the M-major A of MMA 4: 4 chunks of 32 queries
    const uint32_t d_addr = ds_smem + 4 * BWD_CHUNK;           // D[256]
    const uint32_t aux_addr = d_addr + 1024;
    float* d_sm = reinterpret_cast<float*>(smem_raw + (d_addr - raw_addr));
    uint8_t* aux = smem_raw + (aux_addr - raw_addr);
    const uint32_t bar_a = aux_addr;           // operands of MMA 1 have landed: dO_i K-major (and V_j)   (producer -> MMA)
    const uint32_t bar_b = aux_addr + 8;       // operands of MMAs 2-4: dO_i N-major, Q_i (and K_j)       (producer -> MMA)
    const uint32_t bar_dp = aux_addr + 16;     // MMA 1 done: dP^T readable                        (MMA -> warps)
    const uint32_t bar_ds = aux_addr + 24;     // P^T, dS^T in TMEM and dS^T in shared memory      (8 warps -> MMA)
    const uint32_t bar_step = aux_addr + 32;   // MMAs 2-4 done: operand buffers and ds reusable   (MMA -> producer, warps)
    const uint32_t bar_free = aux_addr + 40;   // dV/dK (and at a tile's end dQ) read out          (8 warps -> MMA)
    const uint32_t bar_d = aux_addr + 48;      // D of the tile written                            (8 warps)
    const uint32_t bar_td = aux_addr + 56;     // teardown
    const uint32_t bar_p = aux_addr + 64;      // the step's block of P has landed in the dS^T region (producer -> warps)
    const uint32_t bar_pr = aux_addr + 72;     // every warp has taken its P values: the region may be rewritten (8 warps)
    const uint32_t tmem_slot_addr = aux_addr + 80;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aux + 80);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aux + 84);
    const uint32_t bar_dsfree = aux_addr + 88; // the dQ product has read dS^T: the region may take the next P block (MMA -> producer)
    // Output staging: in the dO (N-major) + Q buffers when they hold 64 KB together, else in the dS^T region.
    const bool stage_in_operands = dchunks == 2;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(bar_a, 1);
        mbar_init(bar_b, 1);
        mbar_init(bar_dp, 1);
        mbar_init(bar_ds, EPI_WARPS);
        mbar_init(bar_step, 1);
        mbar_init(bar_free, EPI_WARPS);
        mbar_init(bar_d, EPI_WARPS);
        mbar_init(bar_td, 1);
        mbar_init(bar_p, 1);
        mbar_init(bar_pr, EPI_WARPS);
        mbar_init(bar_dsfree, 1);
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
    const int nblk = p.nblk;
    // tile -> head and the key blocks [jb, je) it covers
    const int units_per_head = p.split_keys ? nblk : 1;
    auto tile_head = [&](int t) { return t / units_per_head; };
    auto tile_jb = [&](int t) { return p.split_keys ? t % units_per_head : 0; };
    auto tile_je = [&](int t) { return p.split_keys ? t % units_per_head + 1 : nblk; };

    if (warp == PRODUCER_WARP) {
        if (lane == 0) {
            tma_prefetch_desc(&tm_v);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_dok);
            tma_prefetch_desc(&tm_dom);
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_p);
            int s = 0;   // steps issued by this CTA so far (phase of the per-step barriers)
            int jc = 0;  // key blocks finished by this CTA so far (phase of bar_free)
            bool ok = true;
            // The step's 128 x 128 block of P is copied into the (still unused) dS^T region, from where the element
            // warps take it transposed; the block of the NEXT step is pulled into L2 a step ahead.
            if ((int)blockIdx.x < p.total_tiles)
                tma_prefetch_l2_4d(&tm_p, 128 * tile_jb(blockIdx.x), 0, tile_head(blockIdx.x) % p.H, tile_head(blockIdx.x) / p.H);
            for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
                const int h = tile_head(t) % p.H, b = tile_head(t) / p.H;
                const int jb = tile_jb(t), je = tile_je(t);
                for (int j = jb; j < je && ok; ++j) {
                    for (int i = 0; i < nblk; ++i, ++s) {
                        // Every buffer is single.  The operands of MMA 1 are free as soon as the previous step's MMA 1 is
                        // done, so they are fetched while that step is still in its element work and MMAs 2-4.
                        if (s > 0 && !wait_bounded(bar_dp, (s - 1) & 1, abort_flag, p.status, WAIT_PRODUCER_EMPTY)) {
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(bar_a, i == 0 ? 2 * opnd : opnd);
                        for (int c = 0; c < dchunks; ++c) {
                            tma_load_4d(dok_smem + c * BWD_CHUNK, &tm_dok, bar_a, 32 * c, 128 * i, h, b);
                            if (i == 0) tma_load_4d(v_smem + c * BWD_CHUNK, &tm_v, bar_a, 32 * c, 128 * j, h, b);
                        }
                        // The dS^T region takes the step's P block.  It is free once the previous step's dQ product is done
                        // and, where outputs are staged in it, once the stores of a key block's last step have read them.
                        // The operands of MMAs 3-4 follow when all of the previous step's MMAs are done and, where the
                        // outputs are staged in their buffers, the stores have read those.
                        const bool after_outputs = s > 0 && i == 0;
                        if (s > 0 && !wait_bounded(bar_dsfree, (s - 1) & 1, abort_flag, p.status, WAIT_PRODUCER_EMPTY)) {
                            ok = false;
                            break;
                        }
                        const bool p_first = !(after_outputs && !stage_in_operands);
                        if (p_first) {
                            mbar_arrive_expect_tx(bar_p, p.pbox * p.pbox * 4);
                            tma_load_4d(ds_smem, &tm_p, bar_p, 128 * j, 128 * i, h, b);
                        }
                        if (s > 0 && !wait_bounded(bar_step, (s - 1) & 1, abort_flag, p.status, WAIT_PRODUCER_EMPTY)) {
                            ok = false;
                            break;
                        }
                        if (after_outputs) {
                            if (!wait_bounded(bar_free, jc & 1, abort_flag, p.status, WAIT_PRODUCER_EMPTY)) {
                                ok = false;
                                break;
                            }
                            ++jc;
                        }
                        if (!p_first) {
                            mbar_arrive_expect_tx(bar_p, p.pbox * p.pbox * 4);
                            tma_load_4d(ds_smem, &tm_p, bar_p, 128 * j, 128 * i, h, b);
                        }
                        mbar_arrive_expect_tx(bar_b, i == 0 ? 3 * opnd : 2 * opnd);
                        for (int c = 0; c < dchunks; ++c) {
                            for (int kb = 0; kb < 4; ++kb) {
                                tma_load_4d(dom_smem + c * BWD_CHUNK + kb * 4096, &tm_dom, bar_b, 32 * c, 128 * i + 32 * kb, h, b);
                                tma_load_4d(q_smem + c * BWD_CHUNK + kb * 4096, &tm_q, bar_b, 32 * c, 128 * i + 32 * kb, h, b);
                                if (i == 0)
                                    tma_load_4d(k_smem + c * BWD_CHUNK + kb * 4096, &tm_k, bar_b, 32 * c, 128 * j + 32 * kb, h, b);
                            }
                        }
                        if (!ok) break;
                        {   // P block of the step after this one
                            int ni = i + 1, nj = j, nt = t;
                            if (ni == nblk) { ni = 0; ++nj; }
                            if (nj == je) {
                                nt += gridDim.x;
                                nj = nt < p.total_tiles ? tile_jb(nt) : 0;
                            }
                            if (nt < p.total_tiles) tma_prefetch_l2_4d(&tm_p, 128 * nj, 128 * ni, tile_head(nt) % p.H, tile_head(nt) / p.H);
                        }
                    }
                }
            }
            if (!ok || *abort_flag) {   // copies already issued still write shared memory: let them land
                const uint64_t t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 200000ull) {
                }
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            const uint32_t idesc_dp = make_idesc_tf32(128, 128, false, false);
            const uint32_t idesc_ta = make_idesc_tf32(128, p.d, false, true);     // A from TMEM, B N-major
            const uint32_t idesc_dq = make_idesc_tf32(128, p.d, true, true);      // A M-major, B N-major
            int s = 0, jc = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
                const int jb = tile_jb(t), je = tile_je(t);
                for (int j = jb; j < je && ok; ++j, ++jc) {
                    for (int i = 0; i < nblk; ++i, ++s) {
                        if (!wait_bounded(bar_a, s & 1, abort_flag, p.status, WAIT_MMA_FULL)) { ok = false; break; }
                        tc_fence_after_sync();
                        for (int c = 0; c < dchunks; ++c) {
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk) {
                                const uint64_t da = make_smem_desc(v_smem + c * BWD_CHUNK + kk * 32, 16, 1024, SMEM_LAYOUT_SW128);
                                const uint64_t db = make_smem_desc(dok_smem + c * BWD_CHUNK + kk * 32, 16, 1024, SMEM_LAYOUT_SW128);
                                umma_tf32(tmem_base + BWD_COL_DP, da, db, idesc_dp, (c | kk) != 0);
                            }
                        }
                        umma_commit(bar_dp);
                        if (!(wait_bounded(bar_ds, s & 1, abort_flag, p.status, WAIT_MMA_TMEM_EMPTY) &&
                              wait_bounded(bar_b, s & 1, abort_flag, p.status, WAIT_MMA_FULL))) { ok = false; break; }
                        // dV / dK accumulators (and, at a new tile, dQ) must have been read out
                        if (i == 0 && jc > 0 && !wait_bounded(bar_free, (jc - 1) & 1, abort_flag, p.status, WAIT_MMA_TMEM_EMPTY)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
#pragma unroll
                        for (int kk = 0; kk < 16; ++kk) {
                            const uint64_t da = make_smem_desc(ds_smem + kk * 1024, BWD_CHUNK, 512, SMEM_LAYOUT_SW128_BASE32B);
                            const uint64_t db = make_smem_desc(k_smem + kk * 1024, BWD_CHUNK, 512, SMEM_LAYOUT_SW128_BASE32B);
                            umma_tf32(tmem_base + BWD_COL_DQ + i * 64, da, db, idesc_dq, j != jb || kk != 0);
                        }
                        umma_commit(bar_dsfree);
#pragma unroll
                        for (int kk = 0; kk < 16; ++kk) {
                            const uint64_t db = make_smem_desc(dom_smem + kk * 1024, BWD_CHUNK, 512, SMEM_LAYOUT_SW128_BASE32B);
                            umma_tf32_a_tmem(tmem_base + BWD_COL_DV, tmem_base + BWD_COL_P + kk * 8, db, idesc_ta, (i | kk) != 0);
                        }
#pragma unroll
                        for (int kk = 0; kk < 16; ++kk) {
                            const uint64_t db = make_smem_desc(q_smem + kk * 1024, BWD_CHUNK, 512, SMEM_LAYOUT_SW128_BASE32B);
                            umma_tf32_a_tmem(tmem_base + BWD_COL_DK, tmem_base + BWD_COL_DP + kk * 8, db, idesc_ta, (i | kk) != 0);
                        }
                        umma_commit(bar_step);
                    }
                }
            }
            umma_commit(bar_td);   // nothing of this thread's MMAs may be in flight when TMEM is freed
        }
    } else {
        // ---------------------------------------------------------------- element work + outputs (warps 0-7)
        const int quad = warp & 3, half = warp >> 2;
        const uint32_t t_row = tmem_base + (uint32_t(quad * 32) << 16);
        const int krow = quad * 32 + lane;                       // this thread's key row within the key block
        const uint32_t swz = uint32_t(lane & 3) << 1;            // 32-byte-atom swizzle of that row, in 16-byte units
        // This warp's two 4 KB output staging tiles: blocks of the dO (N-major) + Q buffers, or of the dS^T tile.
        const uint32_t my_blk0 = (stage_in_operands ? dom_smem : ds_smem) + (half * 2) * BWD_CHUNK + quad * 4096;
        int s = 0, jc = 0, tc = 0;
        bool ok = true;
        EpilogueRow er;
        er.c_row = nullptr; er.pre_row = nullptr; er.res_row = nullptr; er.row_ok = true; er.vec_ok = false; er.tma_ok = true; er.sector_ok = false;
        er.tm_c = nullptr; er.tm_pre = nullptr;
        int stores = 0;
        for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++tc) {
            const int head = tile_head(t), h = head % p.H, b = head / p.H;
            const int jb = tile_jb(t), je = tile_je(t);
            er.bi = h; er.bo = b;
            // D of this head's queries: fetched now, published to the other warps just before its first use
            const float d_mine = (int)threadIdx.x < p.T ? __ldg(p.dvec + (size_t)head * p.T + threadIdx.x) : 0.0f;
            for (int j = jb; j < je && ok; ++j, ++jc) {
                for (int i = 0; i < nblk; ++i, ++s) {
                    // P^T for this thread's key and its 64 queries, out of the block the producer copied in
                    float pt[64];
                    ok = wait_bounded(bar_p, s & 1, abort_flag, p.status, WAIT_EPI_TMEM_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    {
                        const int q0 = half * 64;                // row of the block; rows and keys past T hold zeros or are skipped
                        const uint32_t src = ds_smem + (uint32_t(q0) * p.pbox + krow) * 4;
#pragma unroll
                        for (int c = 0; c < 64; ++c)
                            pt[c] = (krow < p.pbox && q0 + c < p.pbox) ? ld_shared_f32(src + uint32_t(c) * p.pbox * 4) : 0.0f;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_pr);
                    if (i == 0 && j == jb) {
                        // every warp is past the previous tile's last element pass (its outputs were read after that
                        // step's MMAs, which waited for all eight warps), so the D array may be rewritten
                        d_sm[threadIdx.x] = d_mine;
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_d);
                        ok = wait_bounded(bar_d, tc & 1, abort_flag, p.status, WAIT_EPI_TMEM_FULL);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                    }
                    ok = wait_bounded(bar_dp, s & 1, abort_flag, p.status, WAIT_EPI_TMEM_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
                    ok = wait_bounded(bar_pr, s & 1, abort_flag, p.status, WAIT_EPI_TMEM_FULL);   // nobody still reads P
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
#pragma unroll
                    for (int c2 = 0; c2 < 2; ++c2) {
                        const int cc = half * 2 + c2;            // 32-query chunk of the block
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(t_row + BWD_COL_DP + cc * 32, r);
                        tmem_ld_wait();
                        uint32_t pr[32];
#pragma unroll
                        for (int q = 0; q < 32; ++q) {
                            const float pv = pt[c2 * 32 + q];
                            const float dsv = pv * (__uint_as_float(r[q]) - d_sm[i * 128 + cc * 32 + q]) * p.inv_scale;
                            pr[q] = __float_as_uint(pv);
                            r[q] = __float_as_uint(dsv);
                        }
                        tmem_st_32x32b_x32(t_row + BWD_COL_P + cc * 32, pr);
                        tmem_st_32x32b_x32(t_row + BWD_COL_DP + cc * 32, r);
                        const uint32_t row_addr = ds_smem + cc * BWD_CHUNK + krow * 128;
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + ((uint32_t(u) ^ swz) << 4)),
                                         "r"(r[4 * u]), "r"(r[4 * u + 1]), "r"(r[4 * u + 2]), "r"(r[4 * u + 3])
                                         : "memory");
                    }
                    tmem_st_wait();
                    tc_fence_before_sync();
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_ds);
                    if (i != nblk - 1) continue;
                    // ---- last query block of this key block: dV_j and dK_j are complete once this step's MMAs are done
                    ok = wait_bounded(bar_step, s & 1, abort_flag, p.status, WAIT_EPI_TMEM_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
                    er.row0 = j * 128 + quad * 32;
                    for (int item = half; item < 2 * dchunks; item += 2) {
                        const int which = item / dchunks, c = item % dchunks;      // 0: dV, 1: dK
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(t_row + (which ? BWD_COL_DK : BWD_COL_DV) + c * 32, r);
                        tmem_ld_wait();
                        if (er.row0 < p.T) {
                            er.stage = my_blk0 + ((stores++) & 1) * BWD_CHUNK;
                            stage_and_store32(reinterpret_cast<const float*>(r), c * 32, er, which ? &tm_dk : &tm_dv, lane, true, 0);
                        }
                    }
                    if (j == je - 1) {   // last key block of the tile: its dQ (whole, or this key block's part) goes out as well
                        for (int item = half; item < nblk * dchunks; item += 2) {
                            const int qi = item / dchunks, c = item % dchunks;
                            uint32_t r[32];
                            tmem_ld_32x32b_x32(t_row + BWD_COL_DQ + qi * 64 + c * 32, r);
                            tmem_ld_wait();
                            er.row0 = qi * 128 + quad * 32;
                            if (er.row0 < p.T) {
                                er.stage = my_blk0 + ((stores++) & 1) * BWD_CHUNK;
                                stage_and_store32(reinterpret_cast<const float*>(r), c * 32, er, &tm_dq, lane, true, 0, p.split_keys != 0);
                            }
                        }
                    }
                    tc_fence_before_sync();
                    if (lane == 0) bulk_wait_read_all();       // the staging blocks go back to the producer
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_free);
                }
            }
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

static bool aligned16_view(const float* ptr, const int64_t* s) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (s[0] & 3) == 0 && (s[1] & 3) == 0 && (s[2] & 3) == 0;
}

// Returns TE_OK when the fused kernel was launched, -1 when this problem is outside its limits (the caller then takes
// the GEMM sequence), or an error status.
int launch_attention_backward_fused(te_b200_ctx* ctx, const te_attn_bwd_desc* t, cudaStream_t stream) {
    if (t->precision != TE_PREC_TF32 || !t->o) return -1;
    if (t->T > 256 || (t->T & 3) || (t->d != 32 && t->d != 64)) return -1;
    if (t->B * t->H > INT32_MAX) return -1;
    if (!aligned16_view(t->o, t->o_strides) || !aligned16_view(t->d_o, t->d_o_strides)) return -1;
    if (reinterpret_cast<uintptr_t>(t->p) & 15) return -1;
    CUtensorMap mv, mk, mdok, mdom, mq, mdq, mdk, mdv, mp;
    const auto K_MAJOR = CU_TENSOR_MAP_SWIZZLE_128B, N_MAJOR = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
    if (!make_bhtc_map(ctx, &mv, t->v, t->d, t->T, t->H, t->B, t->v_strides, 32, 128, K_MAJOR)) return -1;
    if (!make_bhtc_map(ctx, &mk, t->k, t->d, t->T, t->H, t->B, t->k_strides, 32, 32, N_MAJOR)) return -1;
    if (!make_bhtc_map(ctx, &mdok, t->d_o, t->d, t->T, t->H, t->B, t->d_o_strides, 32, 128, K_MAJOR)) return -1;
    if (!make_bhtc_map(ctx, &mdom, t->d_o, t->d, t->T, t->H, t->B, t->d_o_strides, 32, 32, N_MAJOR)) return -1;
    if (!make_bhtc_map(ctx, &mq, t->q, t->d, t->T, t->H, t->B, t->q_strides, 32, 32, N_MAJOR)) return -1;
    if (!make_bhtc_map(ctx, &mdq, t->dq, t->d, t->T, t->H, t->B, t->dq_strides, 32, 32, K_MAJOR)) return -1;
    if (!make_bhtc_map(ctx, &mdk, t->dk, t->d, t->T, t->H, t->B, t->dk_strides, 32, 32, K_MAJOR)) return -1;
    if (!make_bhtc_map(ctx, &mdv, t->dv, t->d, t->T, t->H, t->B, t->dv_strides, 32, 32, K_MAJOR)) return -1;
    const int64_t p_strides[3] = {t->H * t->T * t->T, t->T * t->T, t->T};
    if (!make_bhtc_map(ctx, &mp, t->p, t->T, t->T, t->H, t->B, p_strides, (int)(t->T < 128 ? t->T : 128),
                       (int)(t->T < 128 ? t->T : 128), CU_TENSOR_MAP_SWIZZLE_NONE)) return -1;
    AttnBwdParams p;
    p.T = (int)t->T; p.d = (int)t->d; p.H = (int)t->H; p.B = (int)t->B;
    p.nblk = (int)((t->T + 127) / 128);
    {
        // steps a CTA runs with one tile per head (nblk^2 each) against one tile per (head, key block) (nblk each)
        const long long heads = t->B * t->H, sms = ctx->sm_count;
        const long long per_head = ((heads + sms - 1) / sms) * p.nblk * p.nblk;
        const long long per_key_block = ((heads * p.nblk + sms - 1) / sms) * p.nblk;
        p.split_keys = (p.nblk == 2 && per_key_block < per_head && heads * p.nblk <= INT32_MAX) ? 1 : 0;
    }
    p.total_tiles = (int)(t->B * t->H) * (p.split_keys ? p.nblk : 1);
    p.inv_scale = 1.0f / sqrtf((float)t->d);
    p.pbox = (int)(t->T < 128 ? t->T : 128);
    p.status = ctx->d_status;
    // D lives at the end of the context workspace
    const long long rows = (long long)t->B * t->H * t->T;
    const size_t d_bytes = ((size_t)rows * sizeof(float) + 255) & ~size_t(255);
    if (d_bytes > ctx->workspace_bytes) return -1;
    float* dvec = reinterpret_cast<float*>(static_cast<char*>(ctx->workspace) + ctx->workspace_bytes - d_bytes);
    p.dvec = dvec;
    {
        const int rpi = 32 / ((int)t->d / 4);
        long long blocks = (rows + 8 * rpi - 1) / (8 * rpi);
        if (blocks > (long long)ctx->sm_count * 16) blocks = (long long)ctx->sm_count * 16;
        launch_pdl(rowdot_bht_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, t->d_o, t->d_o_strides[0], t->d_o_strides[1], t->d_o_strides[2],
                                                                 t->o, t->o_strides[0], t->o_strides[1], t->o_strides[2], dvec,
                                                                 (int)t->H, (int)t->T, (int)t->d, rows,
                                                                 p.split_keys ? t->dq : (float*)nullptr, t->dq_strides[0], t->dq_strides[1], t->dq_strides[2]);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "rowdot_bht_kernel launch");
        ctx->launches += 1;
    }
    const int dchunks = p.d / 32;
    const int smem = 1024 + 5 * dchunks * BWD_CHUNK + 4 * BWD_CHUNK + 1024 + 128;
    if (smem > 232448) return -1;
    int& attr_smem = ctx->kernel_state[reinterpret_cast<const void*>(attention_bwd_tf32_kernel)];
    if (attr_smem < smem) {
        cudaError_t e = cudaFuncSetAttribute(attention_bwd_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(attention backward)");
        attr_smem = smem;
    }
    const int grid = p.total_tiles < ctx->sm_count ? p.total_tiles : ctx->sm_count;
    launch_pdl(attention_bwd_tf32_kernel, dim3(grid), dim3(CTA_THREADS), smem, stream, mv, mk, mdok, mdom, mq, mdq, mdk, mdv, mp, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "attention_bwd_tf32_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

}  // namespace te
