// Row-wise and elementwise kernels that sit between / behind the GEMMs on the matmul path:
// last-dim softmax (forward, backward), tanh-GELU (forward, backward) and the column sum that
// produces a bias gradient.  All are HBM-bound streaming kernels: one warp per softmax row with the
// row held in registers (one read, one write of the row), 16-byte accesses for the elementwise ones.
#include <cuda_runtime.h>
#include <stdint.h>

#include "pdl.cuh"
#include "te_internal.h"

namespace te {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Softmax over the last dimension with max subtraction, as Tensor::softmax does
// (reference src/tensor/tensor.cpp:1164-1296; CUDA kernel src/cuda/elementwise_cuda.cu:2424-2448).
// ITEMS * 32 >= cols: the row lives in registers.  ITEMS == 0: generic three-pass loop.
template <int ITEMS>
__global__ void __launch_bounds__(256) softmax_rows_kernel(const float* in, float* out,   // in may alias out
                                                          
                                                           long long rows, int cols) {
    griddep_wait();
    const int lane = threadIdx.x & 31;
    const long long warps_per_grid = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
         row += warps_per_grid) {
        const float* x = in + row * cols;
        float* y = out + row * cols;
        if (ITEMS > 0) {
            float v[ITEMS > 0 ? ITEMS : 1];
            float m = -__int_as_float(0x7f800000);
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) {
                const int c = lane + 32 * i;
                v[i] = c < cols ? x[c] : -__int_as_float(0x7f800000);
                m = fmaxf(m, v[i]);
            }
            m = warp_max(m);
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) {
                const int c = lane + 32 * i;
                v[i] = c < cols ? expf(v[i] - m) : 0.0f;
                s += v[i];
            }
            s = warp_sum(s);
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) {
                const int c = lane + 32 * i;
                if (c < cols) y[c] = v[i] / s;
            }
        } else {
            float m = -__int_as_float(0x7f800000);
            for (int c = lane; c < cols; c += 32) m = fmaxf(m, x[c]);
            m = warp_max(m);
            float s = 0.0f;
            for (int c = lane; c < cols; c += 32) {
                const float e = expf(x[c] - m);
                y[c] = e;
                s += e;
            }
            s = warp_sum(s);
            for (int c = lane; c < cols; c += 32) y[c] = y[c] / s;
        }
    }
}

// Same softmax for rows of V4 * 128 floats that start on 16-byte boundaries: every lane moves whole float4s, which
// keeps four times as many bytes in flight per instruction as the scalar form.
template <int V4>
__global__ void __launch_bounds__(256) softmax_rows_vec4_kernel(const float* in, float* out, long long rows) {
    griddep_wait();
    constexpr int cols = V4 * 128;
    const int lane = threadIdx.x & 31;
    const long long warps_per_grid = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
         row += warps_per_grid) {
        const float4* x = reinterpret_cast<const float4*>(in + row * cols);
        float4* y = reinterpret_cast<float4*>(out + row * cols);
        float4 v[V4];
        float m = -__int_as_float(0x7f800000);
#pragma unroll
        for (int i = 0; i < V4; ++i) {
            v[i] = x[lane + 32 * i];
            m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
        }
        m = warp_max(m);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < V4; ++i) {
            v[i].x = expf(v[i].x - m); v[i].y = expf(v[i].y - m); v[i].z = expf(v[i].z - m); v[i].w = expf(v[i].w - m);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
        s = warp_sum(s);
#pragma unroll
        for (int i = 0; i < V4; ++i) {
            v[i].x = v[i].x / s; v[i].y = v[i].y / s; v[i].z = v[i].z / s; v[i].w = v[i].w / s;
            y[lane + 32 * i] = v[i];
        }
    }
}

// dx = s * (dy - <dy, s>) per row (reference src/cuda/elementwise_cuda.cu:2450-2467).
// dx may be the same buffer as dy: every element is read and then written by the one lane that owns it.
__global__ void __launch_bounds__(256) softmax_backward_rows_kernel(const float* __restrict__ s, const float* dy,
                                                                    float* dx, long long rows, int cols) {
    griddep_wait();
    const int lane = threadIdx.x & 31;
    const long long warps_per_grid = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
         row += warps_per_grid) {
        const float* sr = s + row * cols;
        const float* gr = dy + row * cols;
        float* o = dx + row * cols;
        float dot = 0.0f;
        for (int c = lane; c < cols; c += 32) dot += gr[c] * sr[c];
        dot = warp_sum(dot);
        for (int c = lane; c < cols; c += 32) o[c] = sr[c] * (gr[c] - dot);
    }
}

__device__ __forceinline__ float gelu_fwd(float x) {
    const float x3 = x * x * x;
    return 0.5f * x * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x3)));
}
// Derivative as written in gelu_backward_kernel (reference src/cuda/elementwise_cuda.cu:2709-2724).
__device__ __forceinline__ float gelu_bwd(float x, float dy) {
    const float c = 0.7978845608f, k = 0.044715f;
    const float z = c * (x + k * x * x * x);
    const float t = tanhf(z);
    const float sech_sq = 1.0f - t * t;
    const float inner = c * (1.0f + 3.0f * k * x * x);
    return dy * (0.5f * (1.0f + t) * (1.0f + x * sech_sq * inner));
}

__global__ void __launch_bounds__(256) gelu_kernel(const float* __restrict__ x, float* __restrict__ y, long long n) {
    griddep_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] = gelu_fwd(x[i]);
}
// 16-byte aligned buffers, n4 = n / 4 vectors, four vectors in flight per thread.
constexpr int GELU_UNROLL = 4;
__global__ void __launch_bounds__(256) gelu_vec4_kernel(const float4* __restrict__ x, float4* __restrict__ y, long long n4) {
    griddep_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += stride * GELU_UNROLL) {
        float4 xv[GELU_UNROLL];
#pragma unroll
        for (int u = 0; u < GELU_UNROLL; ++u) {
            const long long i = i0 + u * stride;
            if (i < n4) xv[u] = x[i];
        }
#pragma unroll
        for (int u = 0; u < GELU_UNROLL; ++u) {
            const long long i = i0 + u * stride;
            if (i < n4) y[i] = make_float4(gelu_fwd(xv[u].x), gelu_fwd(xv[u].y), gelu_fwd(xv[u].z), gelu_fwd(xv[u].w));
        }
    }
}
// dx may be the same buffer as dy (each element is read, then written, by one thread).
__global__ void __launch_bounds__(256) gelu_backward_kernel(const float* __restrict__ x, const float* dy, float* dx, long long n) {
    griddep_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dx[i] = gelu_bwd(x[i], dy[i]);
}
// The same for 16-byte aligned buffers, n4 = n / 4 vectors: because dx may alias dy the compiler cannot move loads
// above stores by itself, so each thread first loads the operands of GELU_BWD_UNROLL vectors and then writes them --
// enough loads in flight to reach the HBM rate, and still every element is read before it is written.
constexpr int GELU_BWD_UNROLL = 4;
__global__ void __launch_bounds__(256) gelu_backward_vec4_kernel(const float4* __restrict__ x, const float4* dy, float4* dx, long long n4) {
    griddep_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += stride * GELU_BWD_UNROLL) {
        float4 xv[GELU_BWD_UNROLL], gv[GELU_BWD_UNROLL];
#pragma unroll
        for (int u = 0; u < GELU_BWD_UNROLL; ++u) {
            const long long i = i0 + u * stride;
            if (i < n4) { xv[u] = x[i]; gv[u] = dy[i]; }
        }
#pragma unroll
        for (int u = 0; u < GELU_BWD_UNROLL; ++u) {
            const long long i = i0 + u * stride;
            if (i < n4) {
                float4 r;
                r.x = gelu_bwd(xv[u].x, gv[u].x); r.y = gelu_bwd(xv[u].y, gv[u].y);
                r.z = gelu_bwd(xv[u].z, gv[u].z); r.w = gelu_bwd(xv[u].w, gv[u].w);
                dx[i] = r;
            }
        }
    }
}

__device__ __forceinline__ bool colsum_is_last_block(unsigned* counter, unsigned slabs, bool* flag_smem);

// Sum of the slab partials warp, warp + 8, ... of four columns, added in ascending slab order.  The partials were
// written by other blocks (read through L2); four are fetched before the first is added, because what the finishing
// block waits for is the latency of these loads.
__device__ __forceinline__ float4 slab_partials_in_order(const float* partial_col, long long cols, int warp, int slabs) {
    float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
    int sl = warp;
    for (; sl + 24 < slabs; sl += 32) {
        float4 t[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) t[u] = __ldcg(reinterpret_cast<const float4*>(partial_col + (long long)(sl + 8 * u) * cols));
#pragma unroll
        for (int u = 0; u < 4; ++u) { s4.x += t[u].x; s4.y += t[u].y; s4.z += t[u].z; s4.w += t[u].w; }
    }
    for (; sl < slabs; sl += 8) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(partial_col + (long long)sl * cols));
        s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
    }
    return s4;
}

// dx = dy * gelu'(x) over a dense [rows, cols] matrix AND the column sums of dx in the same pass (the bias gradient of
// the Linear that produced x: FeedForward's first Linear, src/nn/ffn.cpp:12-14 / src/core/grad_fn.cpp:93-102).  Thread
// layout of colsum_slab_vec4_kernel: a block owns 128 columns and a slab of rows, its eight warps stride the rows four
// at a time (eight 16-byte loads in flight per thread); slab sums go to `partial`, the last block of a column block
// adds them in slab order.  dx may alias dy (each element is read before it is written, by the same thread).
__global__ void __launch_bounds__(256) gelu_backward_colsum_kernel(const float* __restrict__ x, const float* dy, float* dx,
                                                                   long long rows, long long cols, long long rows_per_slab,
                                                                   float* __restrict__ partial, int slabs, unsigned* counters,
                                                                   float* out) {
    griddep_wait();
    __shared__ float4 red[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long col = (long long)blockIdx.x * 128 + lane * 4;
    const long long r0 = (long long)blockIdx.y * rows_per_slab;
    const long long r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < cols) {
        for (long long r = r0 + warp; r < r1; r += 32) {
            float4 xv[4], gv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long rr = r + 8 * u;
                if (rr < r1) {
                    xv[u] = *reinterpret_cast<const float4*>(x + rr * cols + col);
                    gv[u] = *reinterpret_cast<const float4*>(dy + rr * cols + col);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long rr = r + 8 * u;
                if (rr < r1) {
                    float4 t;
                    t.x = gelu_bwd(xv[u].x, gv[u].x); t.y = gelu_bwd(xv[u].y, gv[u].y);
                    t.z = gelu_bwd(xv[u].z, gv[u].z); t.w = gelu_bwd(xv[u].w, gv[u].w);
                    *reinterpret_cast<float4*>(dx + rr * cols + col) = t;
                    acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
                }
            }
        }
    }
    red[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && col < cols) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float4 v = red[w][lane];
            t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        }
        *reinterpret_cast<float4*>(partial + (long long)blockIdx.y * cols + col) = t;
    }
    __shared__ bool last;
    if (!colsum_is_last_block(counters + blockIdx.x, (unsigned)slabs, &last)) return;
    float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < cols)
        s4 = slab_partials_in_order(partial + col, cols, warp, slabs);
    __syncthreads();
    red[warp][lane] = s4;
    __syncthreads();
    if (warp == 0 && col < cols) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float4 v = red[w][lane];
            t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        }
        *reinterpret_cast<float4*>(out + col) = t;
    }
}

// out[j] = sum over rows of in[i*ld + j].  One block owns 32 columns; its 32 row-lanes stride the rows,
// then a shared-memory tree adds the 32 partials in a fixed order (deterministic, unlike an atomicAdd).
__global__ void __launch_bounds__(1024) colsum_kernel(const float* __restrict__ in, long long rows, long long cols,
                                                      long long ld, float* out, int accumulate) {
    griddep_wait();
    __shared__ float part[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const long long col = (long long)blockIdx.x * 32 + tx;
    float acc = 0.0f;
    if (col < cols)
        for (long long r = ty; r < rows; r += 32) acc += in[r * ld + col];
    part[ty][tx] = acc;
    __syncthreads();
    for (int h = 16; h > 0; h >>= 1) {
        if (ty < h) part[ty][tx] += part[ty + h][tx];
        __syncthreads();
    }
    if (ty == 0 && col < cols) out[col] = accumulate ? out[col] + part[0][tx] : part[0][tx];
}

// Form for tall inputs: slab s of the rows is summed into partial[s][col] (same thread layout as above), then the
// slabs are added in order.  Deterministic, and enough blocks to pull the full HBM bandwidth.
// The block that finishes a column block last (counted through `counters`, one zero-initialised word per column block,
// reset to zero by that block) adds the slabs' partial sums in a fixed order: warp w adds slabs w, w + 8, ... ascending,
// then the eight warp sums are added in warp order.  One launch, and the same result bits on every run.
__device__ __forceinline__ bool colsum_is_last_block(unsigned* counter, unsigned slabs, bool* flag_smem) {
    __threadfence();                 // this thread's partial sums are visible before the count goes up
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0) {
        const unsigned prev = atomicAdd(counter, 1u);
        *flag_smem = (prev == slabs - 1);
        if (prev == slabs - 1) *counter = 0;      // ready for the next call
    }
    __syncthreads();
    if (*flag_smem) __threadfence();
    return *flag_smem;
}

__global__ void __launch_bounds__(1024) colsum_slab_kernel(const float* __restrict__ in, long long rows, long long cols,
                                                           long long ld, long long rows_per_slab, float* __restrict__ partial,
                                                           int slabs, unsigned* counters, float* out, int accumulate) {
    griddep_wait();
    __shared__ float part[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const long long col = (long long)blockIdx.x * 32 + tx;
    const long long r0 = (long long)blockIdx.y * rows_per_slab;
    const long long r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
    float acc = 0.0f;
    if (col < cols)
        for (long long r = r0 + ty; r < r1; r += 32) acc += in[r * ld + col];
    part[ty][tx] = acc;
    __syncthreads();
    for (int h = 16; h > 0; h >>= 1) {
        if (ty < h) part[ty][tx] += part[ty + h][tx];
        __syncthreads();
    }
    if (ty == 0 && col < cols) partial[(long long)blockIdx.y * cols + col] = part[0][tx];
    __shared__ bool last;
    if (!colsum_is_last_block(counters + blockIdx.x, (unsigned)slabs, &last)) return;
    // warps 0-7 add the slabs (warp w: w, w + 8, ...), then the eight sums are added in warp order
    if (ty < 8) {
        float t = 0.0f;
        if (col < cols)
            for (int sl = ty; sl < slabs; sl += 8) t += __ldcg(partial + (long long)sl * cols + col);
        part[ty][tx] = t;
    }
    __syncthreads();
    if (ty == 0 && col < cols) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += part[w][tx];
        out[col] = accumulate ? out[col] + t : t;
    }
}
// Slab sums with 16-byte loads (cols and ld multiples of 4, 16-byte aligned base): a block owns 128 columns, its eight
// warps stride the rows of the slab four rows at a time (16 KB of loads in flight per block), every lane keeps four
// column sums; the warps' sums are added in warp order through shared memory.
__global__ void __launch_bounds__(256) colsum_slab_vec4_kernel(const float* __restrict__ in, long long rows, long long cols,
                                                               long long ld, long long rows_per_slab, float* __restrict__ partial,
                                                               int slabs, unsigned* counters, float* out, int accumulate) {
    griddep_wait();
    __shared__ float4 red[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long col = (long long)blockIdx.x * 128 + lane * 4;
    const long long r0 = (long long)blockIdx.y * rows_per_slab;
    const long long r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < cols) {
        const float* base = in + col;
        long long r = r0 + warp;
        for (; r + 24 < r1; r += 32) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(base + r * ld));
            const float4 b = __ldg(reinterpret_cast<const float4*>(base + (r + 8) * ld));
            const float4 c = __ldg(reinterpret_cast<const float4*>(base + (r + 16) * ld));
            const float4 d = __ldg(reinterpret_cast<const float4*>(base + (r + 24) * ld));
            acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
            acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
            acc.x += c.x; acc.y += c.y; acc.z += c.z; acc.w += c.w;
            acc.x += d.x; acc.y += d.y; acc.z += d.z; acc.w += d.w;
        }
        for (; r < r1; r += 8) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(base + r * ld));
            acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
        }
    }
    red[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && col < cols) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float4 x = red[w][lane];
            t.x += x.x; t.y += x.y; t.z += x.z; t.w += x.w;
        }
        *reinterpret_cast<float4*>(partial + (long long)blockIdx.y * cols + col) = t;
    }
    __shared__ bool last;
    if (!colsum_is_last_block(counters + blockIdx.x, (unsigned)slabs, &last)) return;
    float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < cols)
        s4 = slab_partials_in_order(partial + col, cols, warp, slabs);
    __syncthreads();                 // red[] is reused
    red[warp][lane] = s4;
    __syncthreads();
    if (warp == 0 && col < cols) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float4 x = red[w][lane];
            t.x += x.x; t.y += x.y; t.z += x.z; t.w += x.w;
        }
        float4* o = reinterpret_cast<float4*>(out + col);
        if (accumulate) {
            const float4 prev = *o;
            t.x += prev.x; t.y += prev.y; t.z += prev.z; t.w += prev.w;
        }
        *o = t;
    }
}

// ---- q / k / v parameter packing ---------------------------------------------------------------------------------
// Three equally sized weights and three equally sized biases gathered into one buffer  w0 | w1 | w2 | b0 | b1 | b2
// (PACK), or that buffer scattered back to six places (gradients; ACC adds to what is there).  A NULL source packs
// zeros, a NULL destination is skipped.  VEC = 4 needs wn and bn multiples of 4 and 16-byte aligned pointers.
struct SixSegments { float* w[3]; float* b[3]; };
template <bool PACK, int VEC>
__global__ void __launch_bounds__(256) qkv_segments_kernel(SixSegments seg, float* packed, long long wn, long long bn, int acc) {
    griddep_wait();
    const long long total = 3 * (wn + bn) / VEC;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += stride) {
        const long long i = v * VEC;
        float* base;
        long long j;
        if (i < 3 * wn) { const int s = (int)(i / wn); base = seg.w[s]; j = i - s * wn; }
        else { const long long r = i - 3 * wn; const int s = (int)(r / bn); base = seg.b[s]; j = r - s * bn; }
        if (VEC == 4) {
            float4* pk = reinterpret_cast<float4*>(packed + i);
            if (PACK) {
                *pk = base ? *reinterpret_cast<const float4*>(base + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            } else if (base) {
                float4 g = *pk;
                float4* dst = reinterpret_cast<float4*>(base + j);
                if (acc) { const float4 o = *dst; g.x += o.x; g.y += o.y; g.z += o.z; g.w += o.w; }
                *dst = g;
            }
        } else {
            if (PACK) packed[i] = base ? base[j] : 0.f;
            else if (base) base[j] = acc ? base[j] + packed[i] : packed[i];
        }
    }
}

static int grid_for(long long work_items, int per_block, int sm_count) {
    long long blocks = (work_items + per_block - 1) / per_block;
    const long long cap = (long long)sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

int launch_softmax_rows(te_b200_ctx* ctx, const float* in, float* out, int64_t rows, int64_t cols, cudaStream_t st) {
    if (rows == 0 || cols == 0) return TE_OK;
    const int grid = grid_for(rows, 8, ctx->sm_count);
    const int c = (int)cols;
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (aligned && (cols == 128 || cols == 256 || cols == 512 || cols == 1024)) {
        if (cols == 128) launch_pdl(softmax_rows_vec4_kernel<1>, dim3(grid), dim3(256), 0, st, in, out, rows);
        else if (cols == 256) launch_pdl(softmax_rows_vec4_kernel<2>, dim3(grid), dim3(256), 0, st, in, out, rows);
        else if (cols == 512) launch_pdl(softmax_rows_vec4_kernel<4>, dim3(grid), dim3(256), 0, st, in, out, rows);
        else launch_pdl(softmax_rows_vec4_kernel<8>, dim3(grid), dim3(256), 0, st, in, out, rows);
    } else if (cols <= 32) launch_pdl(softmax_rows_kernel<1>, dim3(grid), dim3(256), 0, st, in, out, rows, c);
    else if (cols <= 64) launch_pdl(softmax_rows_kernel<2>, dim3(grid), dim3(256), 0, st, in, out, rows, c);
    else if (cols <= 128) launch_pdl(softmax_rows_kernel<4>, dim3(grid), dim3(256), 0, st, in, out, rows, c);
    else if (cols <= 256) launch_pdl(softmax_rows_kernel<8>, dim3(grid), dim3(256), 0, st, in, out, rows, c);
    else if (cols <= 512) launch_pdl(softmax_rows_kernel<16>, dim3(grid), dim3(256), 0, st, in, out, rows, c);
    else if (cols <= 1024) launch_pdl(softmax_rows_kernel<32>, dim3(grid), dim3(256), 0, st, in, out, rows, c);
    else launch_pdl(softmax_rows_kernel<0>, dim3(grid), dim3(256), 0, st, in, out, rows, c);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "softmax_rows_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

int launch_softmax_backward_rows(te_b200_ctx* ctx, const float* s, const float* dy, float* dx, int64_t rows,
                                 int64_t cols, cudaStream_t st) {
    if (rows == 0 || cols == 0) return TE_OK;
    launch_pdl(softmax_backward_rows_kernel, dim3(grid_for(rows, 8, ctx->sm_count)), dim3(256), 0, st, s, dy, dx, rows, (int)cols);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "softmax_backward_rows_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

int launch_gelu(te_b200_ctx* ctx, const float* x, float* y, int64_t n, cudaStream_t st) {
    if (n == 0) return TE_OK;
    if ((n & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0)
        launch_pdl(gelu_vec4_kernel, dim3(grid_for(n / 4 / GELU_UNROLL + 1, 256, ctx->sm_count)), dim3(256), 0, st,
                   reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), (long long)(n / 4));
    else
        launch_pdl(gelu_kernel, dim3(grid_for(n, 256, ctx->sm_count)), dim3(256), 0, st, x, y, n);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "gelu_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

int launch_gelu_backward(te_b200_ctx* ctx, const float* x, const float* dy, float* dx, int64_t n, cudaStream_t st) {
    if (n == 0) return TE_OK;
    const bool vec = (n & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) |
                                        reinterpret_cast<uintptr_t>(dx)) & 15) == 0;
    if (vec)
        launch_pdl(gelu_backward_vec4_kernel, dim3(grid_for(n / 4 / GELU_BWD_UNROLL + 1, 256, ctx->sm_count)), dim3(256), 0, st,
                   reinterpret_cast<const float4*>(x), reinterpret_cast<const float4*>(dy), reinterpret_cast<float4*>(dx),
                   (long long)(n / 4));
    else
        launch_pdl(gelu_backward_kernel, dim3(grid_for(n, 256, ctx->sm_count)), dim3(256), 0, st, x, dy, dx, n);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "gelu_backward_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

// dx = dy * gelu'(x) and colsum_out = column sums of dx, x / dy / dx dense [rows, cols].  One launch where the layout
// allows the fused kernel, otherwise the two kernels one after the other.
int launch_gelu_backward_colsum(te_b200_ctx* ctx, const float* x, const float* dy, float* dx, int64_t rows, int64_t cols,
                                float* colsum_out, cudaStream_t st) {
    if (rows == 0 || cols == 0) return TE_OK;
    const long long cb = (cols + 127) / 128;
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx) |
                           reinterpret_cast<uintptr_t>(colsum_out)) & 15) == 0;
    long long slabs = ((long long)ctx->sm_count * 4 + cb - 1) / cb;
    if (slabs > rows / 64) slabs = rows / 64;
    if (slabs > 65535) slabs = 65535;
    if ((cols & 3) == 0 && aligned && slabs >= 1 && (size_t)(slabs * cols * 4) <= ctx->workspace_bytes && cb <= STATUS_COUNTER_WORDS) {
        const long long rows_per_slab = (rows + slabs - 1) / slabs;
        slabs = (rows + rows_per_slab - 1) / rows_per_slab;
        unsigned* counters = reinterpret_cast<unsigned*>(ctx->d_status) + STATUS_COUNTER_WORD;
        launch_pdl(gelu_backward_colsum_kernel, dim3((unsigned)cb, (unsigned)slabs), dim3(256), 0, st, x, dy, dx, (long long)rows,
                   (long long)cols, rows_per_slab, static_cast<float*>(ctx->workspace), (int)slabs, counters, colsum_out);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "gelu_backward_colsum_kernel launch");
        ctx->launches += 1;
        return TE_OK;
    }
    if (int rc = launch_gelu_backward(ctx, x, dy, dx, rows * cols, st)) return rc;
    return launch_colsum(ctx, dx, rows, cols, cols, colsum_out, false, st);
}

int launch_colsum(te_b200_ctx* ctx, const float* in, int64_t rows, int64_t cols, int64_t ld, float* out, bool accumulate,
                  cudaStream_t st) {
    if (cols == 0) return TE_OK;
    dim3 block(32, 32);
    unsigned* counters = reinterpret_cast<unsigned*>(ctx->d_status) + STATUS_COUNTER_WORD;
    const bool vec = (cols & 3) == 0 && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(out) & 15) == 0 && rows >= 512;
    if (vec) {
        // enough (column block, row slab) pairs for ~4 blocks per SM, at least 64 rows per slab
        const long long cb = (cols + 127) / 128;
        long long slabs = ((long long)ctx->sm_count * 4 + cb - 1) / cb;
        if (slabs > rows / 64) slabs = rows / 64;
        if (slabs < 1) slabs = 1;
        if (slabs > 65535) slabs = 65535;
        if ((size_t)(slabs * cols * 4) <= ctx->workspace_bytes && cb <= STATUS_COUNTER_WORDS) {
            const long long rows_per_slab = (rows + slabs - 1) / slabs;
            slabs = (rows + rows_per_slab - 1) / rows_per_slab;
            float* partial = static_cast<float*>(ctx->workspace);
            launch_pdl(colsum_slab_vec4_kernel, dim3((unsigned)cb, (unsigned)slabs), dim3(256), 0, st, in, rows, cols, ld,
                       rows_per_slab, partial, (int)slabs, counters, out, accumulate ? 1 : 0);
            cudaError_t ev = cudaGetLastError();
            if (ev != cudaSuccess) return cuda_fail(ev, "colsum_slab_vec4_kernel launch");
            ctx->launches += 1;
            return TE_OK;
        }
    }
    const long long col_blocks = (cols + 31) / 32;
    // enough (column block, row slab) pairs for ~4 blocks per SM, at least 256 rows per slab
    long long slabs = ((long long)ctx->sm_count * 4 + col_blocks - 1) / col_blocks;
    if (slabs > rows / 256) slabs = rows / 256;
    if (slabs > 65535) slabs = 65535;
    if (slabs > 1 && (size_t)(slabs * cols * 4) <= ctx->workspace_bytes && col_blocks <= STATUS_COUNTER_WORDS) {
        const long long rows_per_slab = (rows + slabs - 1) / slabs;
        slabs = (rows + rows_per_slab - 1) / rows_per_slab;
        float* partial = static_cast<float*>(ctx->workspace);
        launch_pdl(colsum_slab_kernel, dim3(dim3((unsigned)col_blocks, (unsigned)slabs)), dim3(block), 0, st, in, rows, cols, ld,
                   rows_per_slab, partial, (int)slabs, counters, out, accumulate ? 1 : 0);
        cudaError_t e2 = cudaGetLastError();
        if (e2 != cudaSuccess) return cuda_fail(e2, "colsum_slab_kernel launch");
        ctx->launches += 1;
        return TE_OK;
    }
    launch_pdl(colsum_kernel, dim3((unsigned)col_blocks), dim3(block), 0, st, in, rows, cols, ld, out, accumulate ? 1 : 0);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "colsum_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

static int launch_qkv_segments(te_b200_ctx* ctx, bool pack, float* const w[3], float* const b[3], float* packed, int64_t wn,
                               int64_t bn, bool accumulate, cudaStream_t st) {
    if (wn + bn == 0) return TE_OK;
    SixSegments seg;
    uintptr_t bits = reinterpret_cast<uintptr_t>(packed);
    for (int i = 0; i < 3; ++i) {
        seg.w[i] = w[i]; seg.b[i] = b[i];
        bits |= reinterpret_cast<uintptr_t>(w[i]) | reinterpret_cast<uintptr_t>(b[i]);
    }
    const bool vec = (bits & 15) == 0 && (wn & 3) == 0 && (bn & 3) == 0;
    const long long items = 3 * (wn + bn) / (vec ? 4 : 1);
    const dim3 grid(grid_for(items, 256, ctx->sm_count)), block(256);
    const int acc = accumulate ? 1 : 0;
    if (pack && vec) launch_pdl(qkv_segments_kernel<true, 4>, grid, block, 0, st, seg, packed, (long long)wn, (long long)bn, acc);
    else if (pack) launch_pdl(qkv_segments_kernel<true, 1>, grid, block, 0, st, seg, packed, (long long)wn, (long long)bn, acc);
    else if (vec) launch_pdl(qkv_segments_kernel<false, 4>, grid, block, 0, st, seg, packed, (long long)wn, (long long)bn, acc);
    else launch_pdl(qkv_segments_kernel<false, 1>, grid, block, 0, st, seg, packed, (long long)wn, (long long)bn, acc);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "qkv_segments_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

// packed = w0 | w1 | w2 | b0 | b1 | b2  (wn floats per weight, bn per bias; NULL sources pack zeros)
int launch_pack_qkv(te_b200_ctx* ctx, const float* const w[3], const float* const b[3], float* packed, int64_t wn, int64_t bn,
                    cudaStream_t st) {
    float* wm[3]; float* bm[3];
    for (int i = 0; i < 3; ++i) { wm[i] = const_cast<float*>(w[i]); bm[i] = const_cast<float*>(b[i]); }
    return launch_qkv_segments(ctx, true, wm, bm, packed, wn, bn, false, st);
}
// the reverse, for gradients: NULL destinations are skipped, accumulate adds to the destinations
int launch_unpack_qkv(te_b200_ctx* ctx, const float* packed, float* const w[3], float* const b[3], int64_t wn, int64_t bn,
                      bool accumulate, cudaStream_t st) {
    return launch_qkv_segments(ctx, false, w, b, const_cast<float*>(packed), wn, bn, accumulate, st);
}

}  // namespace te
