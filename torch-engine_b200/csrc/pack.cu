// Operand packing pre-pass.
//
// Rewrites one GEMM operand (any of: row-/column-major, any leading dimension, two-level batch
// strides) as dense K-major planes  dst[batch][row][kp]  with kp = K rounded up to 4 floats, so that
// the TMA path of the GEMM kernel can always address it.  Two uses:
//   * copy  - an operand whose base address or strides are not multiples of 16 bytes (for example
//             the [tokens, 65] logits gradient of the language-model head);
//   * split - 3xTF32: hi = round-to-nearest tf32(x), lo = round-to-nearest tf32(x - hi); both planes
//             are exactly representable in tf32, so the tensor core consumes them unchanged.
// Pure streaming work: bound by HBM bandwidth (reads 4 B, writes 4 or 8 B per element).
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_common.cuh"
#include "pdl.cuh"
#include "te_internal.h"

namespace te {

struct PackParams {
    const float* src;
    float* dst_hi;
    float* dst_lo;
    long long rows, K, kp, ld;
    long long stride_inner, stride_outer;   // source batch strides (elements)
    long long batch_inner, num_batches;     // packed batches are enumerated outer-major
};

template <bool MN_MAJOR, bool SPLIT>
__global__ void __launch_bounds__(256) pack_operand_kernel(const PackParams p) {
    griddep_wait();
    __shared__ float tile[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;          // 32 x 8
    const long long k0 = (long long)blockIdx.x * 32;
    // grid.y / grid.z are capped at 65535: blocks walk the remaining row blocks and batches (block-uniform loops)
    for (long long batch = blockIdx.z; batch < p.num_batches; batch += gridDim.z) {
        const long long bo = batch / p.batch_inner, bi = batch - bo * p.batch_inner;
        const float* src = p.src + bo * p.stride_outer + bi * p.stride_inner;
        const long long plane = batch * p.rows * p.kp;
        for (long long r0 = (long long)blockIdx.y * 32; r0 < p.rows; r0 += (long long)gridDim.y * 32) {
            if (MN_MAJOR) {
                // coalesced along the row index; transpose through shared memory
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const long long k = k0 + ty + 8 * i, r = r0 + tx;
                    tile[ty + 8 * i][tx] = (k < p.K && r < p.rows) ? src[k * p.ld + r] : 0.0f;
                }
                __syncthreads();
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const long long r = r0 + ty + 8 * i, k = k0 + tx;
                if (r >= p.rows || k >= p.kp) continue;
                float x;
                if (MN_MAJOR) x = tile[tx][ty + 8 * i];
                else x = (k < p.K) ? src[r * p.ld + k] : 0.0f;
                const long long o = plane + r * p.kp + k;
                if (SPLIT) {
                    const float hi = to_tf32_rn(x);
                    p.dst_hi[o] = hi;
                    p.dst_lo[o] = to_tf32_rn(x - hi);
                } else {
                    p.dst_hi[o] = x;
                }
            }
            if (MN_MAJOR) __syncthreads();   // the tile is rewritten by the next iteration
        }
    }
}

// K-major source whose rows are 16-byte aligned: no transpose needed, four k per thread with 16-byte accesses.
template <bool SPLIT>
__global__ void __launch_bounds__(256) pack_rows_vec4_kernel(const PackParams p, long long quads_per_row, long long total) {
    griddep_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long q = i % quads_per_row;
        const long long rb = i / quads_per_row;           // row index over all batches
        const long long r = rb % p.rows;
        const long long batch = rb / p.rows;
        const long long bo = batch / p.batch_inner, bi = batch - bo * p.batch_inner;
        const float* src = p.src + bo * p.stride_outer + bi * p.stride_inner + r * p.ld + 4 * q;
        float4 x;
        if (4 * q + 4 <= p.K) {
            x = *reinterpret_cast<const float4*>(src);
        } else {
            x.x = 4 * q + 0 < p.K ? src[0] : 0.0f;
            x.y = 4 * q + 1 < p.K ? src[1] : 0.0f;
            x.z = 4 * q + 2 < p.K ? src[2] : 0.0f;
            x.w = 0.0f;
        }
        const long long o = rb * p.kp + 4 * q;
        if (SPLIT) {
            float4 hi, lo;
            hi.x = to_tf32_rn(x.x); hi.y = to_tf32_rn(x.y); hi.z = to_tf32_rn(x.z); hi.w = to_tf32_rn(x.w);
            lo.x = to_tf32_rn(x.x - hi.x); lo.y = to_tf32_rn(x.y - hi.y); lo.z = to_tf32_rn(x.z - hi.z); lo.w = to_tf32_rn(x.w - hi.w);
            *reinterpret_cast<float4*>(p.dst_hi + o) = hi;
            *reinterpret_cast<float4*>(p.dst_lo + o) = lo;
        } else {
            *reinterpret_cast<float4*>(p.dst_hi + o) = x;
        }
    }
}

// Makes the runtime load the packing kernels now (a first launch would otherwise do it).
int prepare_pack_kernels() {
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, pack_rows_vec4_kernel<true>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, pack_operand_kernel<true, true>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, pack_operand_kernel<false, true>);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncGetAttributes(pack kernels)");
    return TE_OK;
}

int launch_pack(te_b200_ctx* ctx, const Operand& src, int64_t K, int64_t batch_inner, int64_t batch_outer,
                float* dst_hi, float* dst_lo, bool split, cudaStream_t stream) {
    // Broadcast levels are packed once.
    const int64_t bi = (batch_inner > 1 && src.stride_inner != 0) ? batch_inner : 1;
    const int64_t bo = (batch_outer > 1 && src.stride_outer != 0) ? batch_outer : 1;
    PackParams p;
    p.src = src.ptr; p.dst_hi = dst_hi; p.dst_lo = dst_lo;
    p.rows = src.rows; p.K = K; p.kp = (K + 3) & ~int64_t(3); p.ld = src.ld;
    p.stride_inner = src.stride_inner; p.stride_outer = src.stride_outer;
    p.batch_inner = bi;
    p.num_batches = bi * bo;
    if (src.rows == 0 || K == 0) return TE_OK;
    const int64_t nb = bi * bo;
    const bool rows_aligned = !src.mn_major && (reinterpret_cast<uintptr_t>(src.ptr) & 15) == 0 && (src.ld & 3) == 0 &&
                              (bi == 1 || (src.stride_inner & 3) == 0) && (bo == 1 || (src.stride_outer & 3) == 0);
    if (rows_aligned) {
        const long long quads = p.kp / 4, total = quads * src.rows * nb;
        long long blocks = (total + 255) / 256;
        if (blocks > (long long)ctx->sm_count * 32) blocks = (long long)ctx->sm_count * 32;
        if (split) launch_pdl(pack_rows_vec4_kernel<true>, dim3((unsigned)blocks), dim3(256), 0, stream, p, quads, total);
        else launch_pdl(pack_rows_vec4_kernel<false>, dim3((unsigned)blocks), dim3(256), 0, stream, p, quads, total);
        cudaError_t ev = cudaGetLastError();
        if (ev != cudaSuccess) return cuda_fail(ev, "pack_rows_vec4_kernel launch");
        ctx->launches += 1;
        return TE_OK;
    }
    const int64_t row_blocks = (src.rows + 31) / 32;
    dim3 grid((unsigned)((p.kp + 31) / 32), (unsigned)(row_blocks < 65535 ? row_blocks : 65535), (unsigned)(nb < 65535 ? nb : 65535));
    dim3 block(32, 8);
    if (src.mn_major) {
        if (split) launch_pdl(pack_operand_kernel<true, true>, dim3(grid), dim3(block), 0, stream, p);
        else launch_pdl(pack_operand_kernel<true, false>, dim3(grid), dim3(block), 0, stream, p);
    } else {
        if (split) launch_pdl(pack_operand_kernel<false, true>, dim3(grid), dim3(block), 0, stream, p);
        else launch_pdl(pack_operand_kernel<false, false>, dim3(grid), dim3(block), 0, stream, p);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "pack_operand_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

}  // namespace te
