// The GPT step's kernels around the matmuls: LayerNorm forward / backward, token embedding (+ positional table)
// forward / backward and the mean cross-entropy with its gradient.  All are streaming kernels bound by HBM bandwidth
// (bytes per element in the comments); every reduction is done in a fixed order, so results are bit-reproducible
// (the reference's CUDA versions accumulate with atomicAdd: src/cuda/elementwise_cuda.cu:2546-2550, :2605, :2648).
//
// Reference semantics:
//   LayerNorm::forward / LayerNormBackward      src/nn/layernorm.cpp:19-82, src/core/grad_fn.cpp:405-538
//   Embedding::forward / EmbeddingBackward      src/nn/embedding.cpp:18-60, src/core/grad_fn.cpp:688-760,
//                                               token + positional sum of GPT::forward, src/nn/gpt.cpp:30-69
//   crossEntropyLoss::forward_batched / CrossEntropyBatchedBackward
//                                               src/loss/CrossEntropyLoss.cpp:47-127, src/core/grad_fn.cpp:271-346
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "pdl.cuh"
#include "te_internal.h"

namespace te {

namespace {


__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// A row of up to 1024 floats held by one warp: N groups per lane, a group being one float4 (VEC: the row is a
// multiple of 4 long and 16-byte aligned) or one float.  Element e of group g sits in column
//   VEC:  g * 128 + lane * 4 + e        scalar:  g * 32 + lane.
template <int N, bool VEC>
struct RowRegs {
    static constexpr int W = VEC ? 4 : 1;
    float v[N * W];
    __device__ __forceinline__ static int col(int g, int e, int lane) { return VEC ? g * 128 + lane * 4 + e : g * 32 + lane; }
    __device__ __forceinline__ void load(const float* row, int cols, int lane) {
#pragma unroll
        for (int g = 0; g < N; ++g) {
            const int c = col(g, 0, lane);
            if constexpr (VEC) {
                const float4 x = c < cols ? __ldg(reinterpret_cast<const float4*>(row + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
                v[g * 4] = x.x; v[g * 4 + 1] = x.y; v[g * 4 + 2] = x.z; v[g * 4 + 3] = x.w;
            } else {
                v[g] = c < cols ? __ldg(row + c) : 0.0f;
            }
        }
    }
    __device__ __forceinline__ void store(float* row, int cols, int lane) const {
#pragma unroll
        for (int g = 0; g < N; ++g) {
            const int c = col(g, 0, lane);
            if (c >= cols) continue;
            if constexpr (VEC) *reinterpret_cast<float4*>(row + c) = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
            else row[c] = v[g];
        }
    }
};

// ------------------------------------------------------------------------------------------------ LayerNorm
// Forward: 4 B read + 4 B written per element.  One warp per row, the row stays in registers.
template <int N, bool VEC>
__global__ void __launch_bounds__(256) layernorm_forward_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                const float* __restrict__ beta, float* __restrict__ y,
                                                                long long rows, int cols, float eps) {
    griddep_wait();
    using R = RowRegs<N, VEC>;
    const int lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    R g, b;
    g.load(gamma, cols, lane);
    b.load(beta, cols, lane);
    const float inv_n = 1.0f / (float)cols;
    for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        R xr;
        xr.load(x + r * cols, cols, lane);
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < N * R::W; ++k) s += xr.v[k];
        const float mean = warp_sum_f(s) * inv_n;
        float q = 0.0f;
#pragma unroll
        for (int k = 0; k < N * R::W; ++k) {
            const float d = R::col(k / R::W, k % R::W, lane) < cols ? xr.v[k] - mean : 0.0f;
            q += d * d;
        }
        const float inv_std = 1.0f / sqrtf(warp_sum_f(q) * inv_n + eps);
#pragma unroll
        for (int k = 0; k < N * R::W; ++k) xr.v[k] = (xr.v[k] - mean) * inv_std * g.v[k] + b.v[k];
        xr.store(y + r * cols, cols, lane);
    }
}

// Backward: 8 B read + 4 B written per element.  Each warp walks its rows, writes dx and keeps the column sums of
// dy * x_hat and dy for its rows in registers; the block adds its warps' sums through shared memory and writes one
// partial row pair; layernorm_param_grad_kernel adds the partials of all blocks in block order.
template <int N, bool VEC, bool AHEAD>
__global__ void __launch_bounds__(256, (N <= 2 || (N == 3 && !AHEAD)) ? 2 : 1) layernorm_backward_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                 const float* __restrict__ dy, float* dx, const float* dx_residual,
                                                                 float* __restrict__ partial, long long rows, int cols, float eps,
                                                                 int want_dx_sum) {
    griddep_wait();
    using R = RowRegs<N, VEC>;
    extern __shared__ float red[];     // [8 warps][cols]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    R g, dg, db, ds;       // ds: column sums of the result dx (asked for by want_dx_sum)
    g.load(gamma, cols, lane);
#pragma unroll
    for (int k = 0; k < N * R::W; ++k) dg.v[k] = db.v[k] = ds.v[k] = 0.0f;
    const float inv_n = 1.0f / (float)cols;
    // the next row's loads are issued before the current row's arithmetic (four dependent warp reductions per row):
    // a warp otherwise has nothing in flight while it computes
    long long r = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    // (AHEAD: rows of at most 256 floats, and of 257-384 floats at one block per SM when there is a residual to fetch;
    // longer rows have no registers to spare for a second row)
    R xn, gn;
    if (AHEAD && r < rows) {
        xn.load(x + r * cols, cols, lane);
        gn.load(dy + r * cols, cols, lane);
    }
    for (; r < rows; r += warps) {
        R xr, gy, res;
        if constexpr (AHEAD) {
            xr = xn; gy = gn;
        } else {
            xr.load(x + r * cols, cols, lane);
            gy.load(dy + r * cols, cols, lane);
        }
        if (AHEAD && dx_residual) res.load(dx_residual + r * cols, cols, lane);     // needed last: in flight during the arithmetic
        if (AHEAD && r + warps < rows) {
            xn.load(x + (r + warps) * cols, cols, lane);
            gn.load(dy + (r + warps) * cols, cols, lane);
        }
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < N * R::W; ++k) s += xr.v[k];
        const float mean = warp_sum_f(s) * inv_n;
        float q = 0.0f;
#pragma unroll
        for (int k = 0; k < N * R::W; ++k) {
            const float d = R::col(k / R::W, k % R::W, lane) < cols ? xr.v[k] - mean : 0.0f;
            xr.v[k] = d;
            q += d * d;
        }
        const float inv_std = 1.0f / sqrtf(warp_sum_f(q) * inv_n + eps);
        float m1 = 0.0f, m2 = 0.0f;
#pragma unroll
        for (int k = 0; k < N * R::W; ++k) {
            const float xh = xr.v[k] * inv_std;
            xr.v[k] = xh;
            dg.v[k] += gy.v[k] * xh;
            db.v[k] += gy.v[k];
            const float gdy = g.v[k] * gy.v[k];
            gy.v[k] = gdy;
            m1 += gdy;
            m2 += gdy * xh;
        }
        m1 = warp_sum_f(m1) * inv_n;
        m2 = warp_sum_f(m2) * inv_n;
#pragma unroll
        for (int k = 0; k < N * R::W; ++k) xr.v[k] = (gy.v[k] - m1 - xr.v[k] * m2) * inv_std;
        if (dx_residual) {     // the gradient arriving over the branch that bypasses this LayerNorm (may be dx itself)
            if constexpr (!AHEAD) gy.load(dx_residual + r * cols, cols, lane);
#pragma unroll
            for (int k = 0; k < N * R::W; ++k) xr.v[k] += AHEAD ? res.v[k] : gy.v[k];
        }
        if (want_dx_sum) {
#pragma unroll
            for (int k = 0; k < N * R::W; ++k) ds.v[k] += R::col(k / R::W, k % R::W, lane) < cols ? xr.v[k] : 0.0f;
        }
        xr.store(dx + r * cols, cols, lane);
    }
    // block sums of the two column accumulators, warps added in warp order
    auto block_sum = [&](const R& acc, int which) {
        __syncthreads();
#pragma unroll
        for (int k = 0; k < N * R::W; ++k) {
            const int c = R::col(k / R::W, k % R::W, lane);
            if (c < cols) red[warp * cols + c] = acc.v[k];
        }
        __syncthreads();
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            float t = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += red[w * cols + c];
            partial[((long long)blockIdx.x * 3 + which) * cols + c] = t;
        }
    };
    block_sum(dg, 0);
    block_sum(db, 1);
    if (want_dx_sum) block_sum(ds, 2);
}

// One block per 32 columns: warp w adds the partial rows w, w + 8, ... in ascending order, then the eight warp sums
// are added in warp order.
__global__ void __launch_bounds__(256) layernorm_param_grad_kernel(const float* __restrict__ partial, int blocks, int cols,
                                                                   float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                                   float* __restrict__ dx_colsum) {
    griddep_wait();
    __shared__ float red[3][8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    float a = 0.0f, b = 0.0f, s = 0.0f;
    if (c < cols) {
        // what a warp waits for is the latency of its loads: four partial rows are fetched before the first is added
        // (in ascending row order all the same)
        const long long row_stride = 3LL * cols;
        const float* base = partial + c;
        int i = warp;
        for (; i + 24 < blocks; i += 32) {
            float ta[4], tb[4], ts[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float* row = base + (long long)(i + 8 * u) * row_stride;
                ta[u] = row[0];
                tb[u] = row[cols];
                ts[u] = dx_colsum ? row[2 * cols] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) { a += ta[u]; b += tb[u]; s += ts[u]; }
        }
        for (; i < blocks; i += 8) {
            a += partial[((long long)i * 3) * cols + c];
            b += partial[((long long)i * 3 + 1) * cols + c];
            if (dx_colsum) s += partial[((long long)i * 3 + 2) * cols + c];
        }
    }
    red[0][warp][lane] = a;
    red[1][warp][lane] = b;
    red[2][warp][lane] = s;
    __syncthreads();
    if (warp == 0 && c < cols) {
        float ta = 0.0f, tb = 0.0f, ts = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            ta += red[0][w][lane];
            tb += red[1][w][lane];
            ts += red[2][w][lane];
        }
        if (dgamma) dgamma[c] = ta;
        if (dbeta) dbeta[c] = tb;
        if (dx_colsum) dx_colsum[c] = ts;
    }
}

// ------------------------------------------------------------------------------------------------ embedding
// out[i][:] = table[tokens[i]][:] + pos[i % T][:]   (pos optional).  4 B written per element, reads mostly from L2.
template <bool VEC>
__global__ void __launch_bounds__(256) embedding_forward_kernel(const float* __restrict__ table, const long long* __restrict__ tokens,
                                                                const float* __restrict__ pos, float* __restrict__ out, long long n,
                                                                int T, int D, long long vocab, int* status) {
    griddep_wait();
    const int per_row = VEC ? D / 4 : D;
    const long long total = n * per_row;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const long long i = idx / per_row;
        const int j = (int)(idx - i * per_row);
        const long long tok = tokens[i];
        const bool ok = tok >= 0 && tok < vocab;
        if (!ok && j == 0) atomicCAS(status, 0, te::STATUS_BAD_EMBEDDING_INDEX);
        if (VEC) {
            float4 v = ok ? __ldg(reinterpret_cast<const float4*>(table + tok * D) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (pos) {
                const float4 q = __ldg(reinterpret_cast<const float4*>(pos + (i % T) * D) + j);
                v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
            }
            reinterpret_cast<float4*>(out + i * D)[j] = v;
        } else {
            float v = ok ? __ldg(table + tok * D + j) : 0.0f;
            if (pos) v += __ldg(pos + (i % T) * D + j);
            out[i * D + j] = v;
        }
    }
}

// dtable[v][c] = sum over the positions i with tokens[i] == v, in ascending i, of dout[i][c]: one block per
// (vocabulary row, 128 columns).  The block scans the token ids 128 at a time and appends the matching positions, in
// order, to a list in shared memory (warp votes + prefix counts); whenever the list is full, and at the end, every
// thread (one per column) adds the listed rows of dout, eight loads in flight at a time, strictly in list order.
// Suits the small vocabularies of the reference's character-level models; the scan costs vocab * n / 128 block steps.
constexpr int EMB_LIST = 1024;
constexpr int EMB_SUB = 4;               // sub-chunks of 128 token ids scanned per round (one barrier pair per round)

__global__ void __launch_bounds__(128) embedding_backward_kernel(const long long* __restrict__ tokens, const float* __restrict__ dout,
                                                                 float* __restrict__ dtable, long long n, int D) {
    griddep_wait();
    __shared__ int list[EMB_LIST + EMB_SUB * 128];
    __shared__ int warp_count[EMB_SUB][4];
    const long long v = blockIdx.x;
    const int c = blockIdx.y * 128 + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float acc = 0.0f;
    int filled = 0;                                       // entries in the list (uniform over the block)
    long long list_base = 0;                              // positions in the list are stored relative to this
    auto consume = [&]() {
        const float* col = dout + list_base * D + c;
        int k = 0;
        for (; k + 8 <= filled; k += 8) {
            float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] = c < D ? __ldg(col + (long long)list[k + u] * D) : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; ++u) acc += x[u];
        }
        for (; k < filled; ++k) acc += c < D ? __ldg(col + (long long)list[k] * D) : 0.0f;
    };
    for (long long base = 0; base < n; base += EMB_SUB * 128) {
        if (filled == 0) list_base = base;
        bool hit[EMB_SUB];
        unsigned m[EMB_SUB];
#pragma unroll
        for (int s = 0; s < EMB_SUB; ++s) {                 // the loads of a round are independent
            const long long i = base + s * 128 + threadIdx.x;
            hit[s] = i < n && tokens[i] == v;
        }
#pragma unroll
        for (int s = 0; s < EMB_SUB; ++s) {
            m[s] = __ballot_sync(0xffffffffu, hit[s]);
            if (lane == 0) warp_count[s][warp] = __popc(m[s]);
        }
        __syncthreads();
        int offset = filled;
#pragma unroll
        for (int s = 0; s < EMB_SUB; ++s) {                 // positions are appended in ascending token order
            int before = 0, total = 0;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const int cnt = warp_count[s][w];
                if (w < warp) before += cnt;
                total += cnt;
            }
            if (hit[s]) list[offset + before + __popc(m[s] & ((1u << lane) - 1u))] = (int)(base + s * 128 + threadIdx.x - list_base);
            offset += total;
        }
        filled = offset;
        __syncthreads();                                  // list entries visible; warp_count may be rewritten
        if (filled >= EMB_LIST) {
            consume();
            filled = 0;
            __syncthreads();                              // everyone is done with the list before it is refilled
        }
    }
    consume();
    if (c < D) dtable[v * D + c] = acc;
}

// ------------------------------------------------------------------------------------------------ cross-entropy
// One warp per row of logits: max, sum of exp, loss of the row and (optionally) grad = (softmax - one_hot) * scale.
// The row losses of a block are added in double, warp by warp, into one partial per block; the finish kernel adds
// the partials in block order and divides by the row count.  4 B read (three cached passes) + 4 B written per logit.
__global__ void __launch_bounds__(256) cross_entropy_rows_kernel(const float* __restrict__ logits, const long long* __restrict__ targets,
                                                                 float* __restrict__ grad, float scale, double* __restrict__ partial,
                                                                 long long rows, int V, int* status) {
    griddep_wait();
    __shared__ double block_part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    double mine = 0.0;
    for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + warp; r < rows; r += warps) {
        const float* row = logits + r * V;
        long long tgt = targets[r];
        if (tgt < 0 || tgt >= V) {
            if (lane == 0) atomicCAS(status, 0, te::STATUS_BAD_TARGET_INDEX);
            tgt = 0;
        }
        float m = -INFINITY;
        for (int c = lane; c < V; c += 32) m = fmaxf(m, row[c]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float s = 0.0f;
        for (int c = lane; c < V; c += 32) s += expf(row[c] - m);
        s = warp_sum_f(s);
        if (lane == 0) mine += (double)(-row[tgt] + (m + logf(s)));
        if (grad) {
            float* g = grad + r * V;
            for (int c = lane; c < V; c += 32) {
                const float p = expf(row[c] - m) / s;
                g[c] = (p - (c == tgt ? 1.0f : 0.0f)) * scale;
            }
        }
    }
    if (lane == 0) block_part[warp] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < 8; ++w) t += block_part[w];
        partial[blockIdx.x] = t;
    }
}

// One warp: lane l adds the block partials l, l + 32, ... in ascending order, then the 32 lane sums meet in a fixed
// shuffle tree.
__global__ void cross_entropy_finish_kernel(const double* __restrict__ partial, int blocks, long long rows, float* __restrict__ loss) {
    griddep_wait();
    const int lane = threadIdx.x;
    double t = 0.0;
    for (int i = lane; i < blocks; i += 32) t += partial[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) *loss = (float)(t / (double)rows);
}

int row_grid(long long rows, int sm_count, int per_sm) {
    long long blocks = (rows + 7) / 8;
    const long long cap = (long long)sm_count * per_sm;
    if (blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

#define TE_LN_DISPATCH(CALL)                                             \
    if (vec) {                                                           \
        const int n = (cols + 127) / 128;                                \
        if (n <= 1) { CALL(1, true); } else if (n <= 2) { CALL(2, true); } else if (n <= 3) { CALL(3, true); }   \
        else if (n <= 4) { CALL(4, true); } else if (n <= 6) { CALL(6, true); } else { CALL(8, true); }          \
    } else {                                                             \
        const int n = (cols + 31) / 32;                                  \
        if (n <= 1) { CALL(1, false); } else if (n <= 2) { CALL(2, false); } else if (n <= 4) { CALL(4, false); } \
        else if (n <= 8) { CALL(8, false); } else if (n <= 16) { CALL(16, false); } else { CALL(32, false); }    \
    }

int launch_layernorm_forward(te_b200_ctx* ctx, const float* x, const float* gamma, const float* beta, float* y,
                             int64_t rows, int64_t cols64, float eps, cudaStream_t st) {
    if (rows == 0 || cols64 == 0) return TE_OK;
    if (cols64 > 1024) {
        set_error("LayerNorm rows longer than 1024 elements are not supported");
        return TE_ERR_BAD_ARGUMENT;
    }
    const int cols = (int)cols64;
    const bool vec = (cols & 3) == 0 && aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta);
    const int grid = row_grid(rows, ctx->sm_count, 8);
#define CALL(N, V) launch_pdl(layernorm_forward_kernel<N, V>, dim3(grid), dim3(256), 0, st, x, gamma, beta, y, rows, cols, eps)
    TE_LN_DISPATCH(CALL)
#undef CALL
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "layernorm_forward_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

int launch_layernorm_backward(te_b200_ctx* ctx, const float* x, const float* gamma, const float* dy, float* dx,
                              const float* dx_residual, float* dgamma, float* dbeta, float* dx_colsum, int64_t rows, int64_t cols64,
                              float eps, cudaStream_t st) {
    if (cols64 == 0) return TE_OK;
    if (cols64 > 1024) {
        set_error("LayerNorm rows longer than 1024 elements are not supported");
        return TE_ERR_BAD_ARGUMENT;
    }
    const int cols = (int)cols64;
    const bool vec = (cols & 3) == 0 && aligned16(x) && aligned16(dy) && aligned16(dx) && aligned16(gamma) &&
                     (!dx_residual || aligned16(dx_residual));
    // rows of 257-384 floats with a residual keep two rows per warp in registers and run one block per SM
    const bool mid = vec && cols > 256 && cols <= 384 && dx_residual;
    const int grid = row_grid(rows, ctx->sm_count, mid ? 1 : 2);
    const size_t need = (size_t)grid * 3 * cols * sizeof(float);
    if (need > ctx->workspace_bytes) {
        set_error("context workspace too small for the LayerNorm parameter-gradient partials");
        return TE_ERR_WORKSPACE;
    }
    float* partial = static_cast<float*>(ctx->workspace);
    const size_t smem = (size_t)8 * cols * sizeof(float);
#define CALL(N, V)                                                                                                                        \
    if (N <= 2 || (N == 3 && V && mid))                                                                                                   \
        launch_pdl(layernorm_backward_kernel<N, V, (N <= 3)>, dim3(grid), dim3(256), smem, st, x, gamma, dy, dx, dx_residual, partial, rows, cols, eps, dx_colsum ? 1 : 0); \
    else                                                                                                                                  \
        launch_pdl(layernorm_backward_kernel<N, V, false>, dim3(grid), dim3(256), smem, st, x, gamma, dy, dx, dx_residual, partial, rows, cols, eps, dx_colsum ? 1 : 0);
    TE_LN_DISPATCH(CALL)
#undef CALL
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "layernorm_backward_kernel launch");
    launch_pdl(layernorm_param_grad_kernel, dim3((cols + 31) / 32), dim3(256), 0, st, partial, grid, cols, dgamma, dbeta, dx_colsum);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "layernorm_param_grad_kernel launch");
    ctx->launches += 2;
    return TE_OK;
}

int launch_embedding_forward(te_b200_ctx* ctx, const float* table, const int64_t* tokens, const float* pos, float* out,
                             int64_t n, int64_t T, int64_t D, int64_t vocab, cudaStream_t st) {
    if (n == 0 || D == 0) return TE_OK;
    const bool vec = (D & 3) == 0 && aligned16(table) && aligned16(out) && (!pos || aligned16(pos));
    const long long total = n * (vec ? D / 4 : D);
    long long blocks = (total + 255) / 256;
    if (blocks > (long long)ctx->sm_count * 16) blocks = (long long)ctx->sm_count * 16;
    const long long* tk = reinterpret_cast<const long long*>(tokens);
    if (vec) launch_pdl(embedding_forward_kernel<true>, dim3((unsigned)blocks), dim3(256), 0, st, table, tk, pos, out, n, (int)(T > 0 ? T : 1), (int)D, vocab, ctx->d_status);
    else launch_pdl(embedding_forward_kernel<false>, dim3((unsigned)blocks), dim3(256), 0, st, table, tk, pos, out, n, (int)(T > 0 ? T : 1), (int)D, vocab, ctx->d_status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "embedding_forward_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

int launch_embedding_backward(te_b200_ctx* ctx, const int64_t* tokens, const float* dout, float* dtable, int64_t n,
                              int64_t D, int64_t vocab, cudaStream_t st) {
    if (vocab == 0 || D == 0) return TE_OK;
    if (vocab > INT32_MAX || (D + 127) / 128 > 65535) {
        set_error("embedding backward: table too large");
        return TE_ERR_BAD_ARGUMENT;
    }
    dim3 grid((unsigned)vocab, (unsigned)((D + 127) / 128));
    launch_pdl(embedding_backward_kernel, dim3(grid), dim3(128), 0, st, reinterpret_cast<const long long*>(tokens), dout, dtable, n, (int)D);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "embedding_backward_kernel launch");
    ctx->launches += 1;
    return TE_OK;
}

int launch_cross_entropy(te_b200_ctx* ctx, const float* logits, const int64_t* targets, float* loss, float* grad,
                         float upstream, int64_t rows, int64_t V, cudaStream_t st) {
    if (rows == 0 || V == 0) return TE_OK;
    if (V > INT32_MAX) {
        set_error("cross-entropy: vocabulary too large");
        return TE_ERR_BAD_ARGUMENT;
    }
    const int grid = row_grid(rows, ctx->sm_count, 2);
    if ((size_t)grid * sizeof(double) > ctx->workspace_bytes) {
        set_error("context workspace too small for the cross-entropy partial sums");
        return TE_ERR_WORKSPACE;
    }
    double* partial = static_cast<double*>(ctx->workspace);
    const float scale = upstream / (float)rows;      // CrossEntropyBatchedBackward: upstream / N (grad_fn.cpp:295)
    launch_pdl(cross_entropy_rows_kernel, dim3(grid), dim3(256), 0, st, logits, reinterpret_cast<const long long*>(targets), grad, scale, partial,
                                                    rows, (int)V, ctx->d_status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "cross_entropy_rows_kernel launch");
    ctx->launches += 1;
    if (loss) {
        launch_pdl(cross_entropy_finish_kernel, dim3(1), dim3(32), 0, st, partial, grid, rows, loss);
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "cross_entropy_finish_kernel launch");
        ctx->launches += 1;
    }
    return TE_OK;
}

}  // namespace te
