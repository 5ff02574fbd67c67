/*
 * te_oracle.c -- CPU restatement of the reference's FP32 matmul path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker for the CUDA backend: tests, the smoke check and the cpu_baseline /
 * reference legs of the benchmark may call it; the product library never does.
 *
 * Parity status: PINNED.  Each function below follows the reference lines it cites, is checked
 * bit-for-bit against the reference's own CPU code compiled from its sources (ref_driver.cpp ->
 * _ref/libref_cpu.so, by tests/test_oracle_cpu.py) and against the known-answer vectors of the reference's
 * tests (tests/golden/reference_known_answers.json).
 *
 * Arithmetic notes that make bit-exactness possible: the reference accumulates C[i][j] in memory
 * as `C += a_ik * b_kj` with k strictly ascending (the 64-wide blocking of tensor.h:818-835 never
 * reorders k for a fixed (i,j)), in float, with separate multiply and add (built without FMA
 * contraction: -ffp-contract=off here, plain x86-64 -O2 there).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

enum { ORACLE_OK = 0, ORACLE_ERR_NDIM = 3, ORACLE_ERR_INNER = 4, ORACLE_ERR_BROADCAST = 5, ORACLE_ERR_ARG = 1 };

/* One 2-D slice, real strides of the last two dims: Tensor::tiled_matmul_2d (src/tensor/tensor.h:795-836).
 * C is dense row-major with ldc = N and is accumulated into (the caller zeroes it, tensor.h:577). */
static void slice_matmul(const float* A, int64_t lda, int64_t inner_a, const float* B, int64_t ldb,
                         int64_t inner_b, float* C, int64_t M, int64_t K, int64_t N) {
    for (int64_t i = 0; i < M; ++i) {
        float* crow = C + i * N;
        for (int64_t k = 0; k < K; ++k) {
            const float a_ik = A[i * lda + k * inner_a];
            const float* brow = B + k * ldb;
            if (inner_b == 1) {
                for (int64_t j = 0; j < N; ++j) crow[j] += a_ik * brow[j];
            } else {
                for (int64_t j = 0; j < N; ++j) crow[j] += a_ik * brow[j * inner_b];
            }
        }
    }
}

/* Tensor::matmul -> matmul_impl<float> on the CPU (src/tensor/tensor.cpp:761-785, src/tensor/tensor.h:529-612):
 * >= 2-D check (:536), inner-dim check (:546), NumPy broadcast of batch dims (broadcast_shapes, :838-865),
 * per-batch offsets with size-1 dims pinned to index 0 (compute_batch_offset, :867-906).
 * c must hold prod(batch) * M * N floats; out_shape has room for 8 entries. */
ORACLE_API int oracle_matmul_nd_f32(const float* a, const int64_t* a_shape, const int64_t* a_strides, int a_ndim,
                                    const float* b, const int64_t* b_shape, const int64_t* b_strides, int b_ndim,
                                    float* c, int64_t* out_shape, int* out_ndim) {
    if (a_ndim < 2 || b_ndim < 2) return ORACLE_ERR_NDIM;
    if (a_ndim > 8 || b_ndim > 8) return ORACLE_ERR_ARG;
    const int64_t M = a_shape[a_ndim - 2], Ka = a_shape[a_ndim - 1];
    const int64_t Kb = b_shape[b_ndim - 2], N = b_shape[b_ndim - 1];
    if (Ka != Kb) return ORACLE_ERR_INNER;
    const int nba = a_ndim - 2, nbb = b_ndim - 2, nb = nba > nbb ? nba : nbb;
    int64_t ext[8];
    for (int i = 0; i < nb; ++i) {
        const int64_t da = i < nba ? a_shape[nba - 1 - i] : 1;
        const int64_t db = i < nbb ? b_shape[nbb - 1 - i] : 1;
        if (da != db && da != 1 && db != 1) return ORACLE_ERR_BROADCAST;
        ext[nb - 1 - i] = da > db ? da : db;
    }
    if (out_ndim) *out_ndim = nb + 2;
    if (out_shape) {
        for (int i = 0; i < nb; ++i) out_shape[i] = ext[i];
        out_shape[nb] = M;
        out_shape[nb + 1] = N;
    }
    if (!c) return ORACLE_OK;
    int64_t batches = 1;
    for (int i = 0; i < nb; ++i) batches *= ext[i];
    memset(c, 0, (size_t)(batches * M * N) * sizeof(float));
    const int64_t lda = a_strides[a_ndim - 2], inner_a = a_strides[a_ndim - 1];
    const int64_t ldb = b_strides[b_ndim - 2], inner_b = b_strides[b_ndim - 1];
    for (int64_t flat = 0; flat < batches; ++flat) {
        int64_t idx[8];
        int64_t rem = flat;
        for (int i = nb - 1; i >= 0; --i) { idx[i] = rem % ext[i]; rem /= ext[i]; }
        int64_t off_a = 0, off_b = 0;
        for (int i = 0; i < nba; ++i) {
            const int pos = nb - nba + i;
            off_a += (a_shape[i] == 1 ? 0 : idx[pos]) * a_strides[i];
        }
        for (int i = 0; i < nbb; ++i) {
            const int pos = nb - nbb + i;
            off_b += (b_shape[i] == 1 ? 0 : idx[pos]) * b_strides[i];
        }
        slice_matmul(a + off_a, lda, inner_a, b + off_b, ldb, inner_b, c + flat * M * N, M, Ka, N);
    }
    return ORACLE_OK;
}

/* Rows [row_begin, row_end) of a dense 2-D product; lets a test or the CPU baseline split one large
 * product over host threads without changing any element's summation order. */
ORACLE_API void oracle_matmul_rows_f32(const float* a, int64_t lda, int64_t inner_a, const float* b, int64_t ldb,
                                       int64_t inner_b, float* c, int64_t M, int64_t K, int64_t N,
                                       int64_t row_begin, int64_t row_end) {
    (void)M;
    memset(c + row_begin * N, 0, (size_t)((row_end - row_begin) * N) * sizeof(float));
    slice_matmul(a + row_begin * lda, lda, inner_a, b, ldb, inner_b, c + row_begin * N, row_end - row_begin, K, N);
}

/* Same product with double accumulation: the arbiter when two float results disagree. */
ORACLE_API void oracle_matmul_rows_f64acc(const float* a, int64_t lda, int64_t inner_a, const float* b, int64_t ldb,
                                          int64_t inner_b, double* c, int64_t K, int64_t N, int64_t row_begin,
                                          int64_t row_end) {
    for (int64_t i = row_begin; i < row_end; ++i) {
        double* crow = c + i * N;
        for (int64_t j = 0; j < N; ++j) crow[j] = 0.0;
        for (int64_t k = 0; k < K; ++k) {
            const double a_ik = a[i * lda + k * inner_a];
            for (int64_t j = 0; j < N; ++j) crow[j] += a_ik * (double)b[k * ldb + j * inner_b];
        }
    }
}

/* y[r][j] = x[r][j] + bias[j]: the broadcast add of Linear::forward (src/nn/linear.cpp:22, Tensor::operator+). */
ORACLE_API void oracle_add_bias_f32(float* y, const float* bias, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t j = 0; j < cols; ++j) y[r * cols + j] = y[r * cols + j] + bias[j];
}

/* Tensor::gelu on the CPU evaluates in double and casts (src/tensor/tensor.h:444-455). */
ORACLE_API void oracle_gelu_f32(const float* x, float* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        const double v = (double)x[i];
        const double v3 = v * v * v;
        y[i] = (float)(0.5 * v * (1.0 + tanh(0.7978845608 * (v + 0.044715 * v3))));
    }
}

/* GeluBackward on the CPU evaluates in float (src/core/grad_fn.cpp:186-199). */
ORACLE_API void oracle_gelu_backward_f32(const float* x, const float* dy, float* dx, int64_t n) {
    const float c = 0.7978845608f, k = 0.044715f;
    for (int64_t i = 0; i < n; ++i) {
        const float v = x[i];
        const float x_cubed = v * v * v;
        const float z = c * (v + k * x_cubed);
        const float t = tanhf(z);
        const float sech_sq = 1.0f - t * t;
        const float inner = c * (1.0f + 3.0f * k * v * v);
        const float g = 0.5f * (1.0f + t) * (1.0f + v * sech_sq * inner);
        dx[i] = dy[i] * g;
    }
}

/* Last-dim softmax, CPU path: max, exp and running float sum in index order, then divide by the sum
 * (src/tensor/tensor.cpp:1246-1283). */
ORACLE_API void oracle_softmax_rows_f32(const float* x, float* y, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        float* yr = y + r * cols;
        float m = -INFINITY;
        for (int64_t i = 0; i < cols; ++i) m = xr[i] > m ? xr[i] : m;
        float s = 0.0f;
        for (int64_t i = 0; i < cols; ++i) {
            const float e = expf(xr[i] - m);
            yr[i] = e;
            s += e;
        }
        for (int64_t i = 0; i < cols; ++i) yr[i] /= s;
    }
}

/* dx = s * (dy - sum_j dy_j s_j): the softmax Jacobian product of SoftmaxBackward
 * (src/core/grad_fn.cpp:569-665; device form src/cuda/elementwise_cuda.cu:2450-2467). */
ORACLE_API void oracle_softmax_backward_rows_f32(const float* s, const float* dy, float* dx, int64_t rows,
                                                 int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        float dot = 0.0f;
        for (int64_t i = 0; i < cols; ++i) dot += dy[r * cols + i] * s[r * cols + i];
        for (int64_t i = 0; i < cols; ++i) dx[r * cols + i] = s[r * cols + i] * (dy[r * cols + i] - dot);
    }
}

/* out[j] = sum_i in[i][j], rows added in ascending order: what reduce_gradient -> Tensor::sum(0) yields for a
 * bias gradient (src/core/grad_fn.cpp:13-58). */
ORACLE_API void oracle_colsum_f32(const float* in, int64_t rows, int64_t cols, int64_t ld, float* out) {
    for (int64_t j = 0; j < cols; ++j) out[j] = 0.0f;
    for (int64_t i = 0; i < rows; ++i)
        for (int64_t j = 0; j < cols; ++j) out[j] += in[i * ld + j];
}

/* ---- the GPT step's kernels around the matmuls (LayerNorm, embedding, cross-entropy) ------------------------- */

/* LayerNorm::forward on the CPU (src/nn/layernorm.cpp:56-82): float mean, biased float variance, division by
 * sqrt(var + eps), then * gamma + beta. */
ORACLE_API void oracle_layernorm_forward(const float* x, const float* gamma, const float* beta, float* y,
                                         int64_t rows, int64_t D, float eps) {
    for (int64_t i = 0; i < rows; ++i) {
        const float* xr = x + i * D;
        float mean = 0.0f;
        for (int64_t j = 0; j < D; ++j) mean += xr[j];
        mean /= D;
        float variance = 0.0f;
        for (int64_t j = 0; j < D; ++j) {
            const float diff = xr[j] - mean;
            variance += diff * diff;
        }
        variance /= D;
        const float std_dev = sqrtf(variance + eps);
        for (int64_t j = 0; j < D; ++j) {
            const float normalized = (xr[j] - mean) / std_dev;
            y[i * D + j] = normalized * gamma[j] + beta[j];
        }
    }
}

/* LayerNormBackward::backward on the CPU (src/core/grad_fn.cpp:474-538): rows in ascending order accumulate
 * d_gamma and d_beta in float; dx = (gamma*dy - mean(gamma*dy) - x_hat*mean(gamma*dy*x_hat)) / std. */
ORACLE_API void oracle_layernorm_backward(const float* x, const float* gamma, const float* dy, float* dx,
                                          float* dgamma, float* dbeta, float* x_hat_scratch, int64_t rows,
                                          int64_t D, float eps) {
    const float N = (float)D;
    float* x_hat = x_hat_scratch;
    for (int64_t j = 0; j < D; ++j) dgamma[j] = dbeta[j] = 0.0f;
    for (int64_t b = 0; b < rows; ++b) {
        const float* xr = x + b * D;
        const float* dyr = dy + b * D;
        float* dxr = dx + b * D;
        float mean = 0.0f;
        for (int64_t j = 0; j < D; ++j) mean += xr[j];
        mean /= N;
        float var = 0.0f;
        for (int64_t j = 0; j < D; ++j) {
            const float d = xr[j] - mean;
            var += d * d;
        }
        var /= N;
        const float std_val = sqrtf(var + eps);
        for (int64_t j = 0; j < D; ++j) x_hat[j] = (xr[j] - mean) / std_val;
        for (int64_t j = 0; j < D; ++j) {
            dgamma[j] += dyr[j] * x_hat[j];
            dbeta[j] += dyr[j];
        }
        float mean_g_dy = 0.0f, mean_g_dy_xhat = 0.0f;
        for (int64_t j = 0; j < D; ++j) {
            const float g_dy = gamma[j] * dyr[j];
            mean_g_dy += g_dy;
            mean_g_dy_xhat += g_dy * x_hat[j];
        }
        mean_g_dy /= N;
        mean_g_dy_xhat /= N;
        for (int64_t j = 0; j < D; ++j)
            dxr[j] = (gamma[j] * dyr[j] - mean_g_dy - x_hat[j] * mean_g_dy_xhat) / std_val;
    }
}

/* crossEntropyLoss::forward_batched on the CPU (src/loss/CrossEntropyLoss.cpp:100-124): per row float max, float
 * sum of expf, the row losses added in double in row order, mean cast to float. */
ORACLE_API float oracle_cross_entropy_forward(const float* logits, const int64_t* targets, int64_t rows, int64_t V) {
    double total = 0.0;
    for (int64_t n = 0; n < rows; ++n) {
        const float* row = logits + n * V;
        float max_logit = row[0];
        for (int64_t v = 1; v < V; ++v) max_logit = row[v] > max_logit ? row[v] : max_logit;
        float sum_exp = 0.0f;
        for (int64_t v = 0; v < V; ++v) sum_exp += expf(row[v] - max_logit);
        const float log_sum_exp = max_logit + logf(sum_exp);
        total += (double)(-row[targets[n]] + log_sum_exp);
    }
    return (float)(total / (double)rows);
}

/* CrossEntropyBatchedBackward::backward on the CPU (src/core/grad_fn.cpp:295, :322-343):
 * grad = (softmax - one_hot) * (upstream / rows). */
ORACLE_API void oracle_cross_entropy_backward(const float* logits, const int64_t* targets, float upstream,
                                              float* grad, int64_t rows, int64_t V) {
    const float scale = upstream / (float)rows;
    for (int64_t n = 0; n < rows; ++n) {
        const float* row = logits + n * V;
        float max_logit = row[0];
        for (int64_t v = 1; v < V; ++v) max_logit = row[v] > max_logit ? row[v] : max_logit;
        float sum_exp = 0.0f;
        for (int64_t v = 0; v < V; ++v) sum_exp += expf(row[v] - max_logit);
        for (int64_t v = 0; v < V; ++v) {
            const float softmax_val = expf(row[v] - max_logit) / sum_exp;
            const float one_hot = (v == targets[n]) ? 1.0f : 0.0f;
            grad[n * V + v] = (softmax_val - one_hot) * scale;
        }
    }
}

/* Token embedding lookup plus the broadcast positional table, as GPT::forward composes them
 * (src/nn/embedding.cpp:51-59, src/nn/gpt.cpp:30-69): out[i][j] = table[tokens[i]][j] + pos[i % T][j].
 * pos may be NULL (plain Embedding::forward).  Returns non-zero for an index out of range. */
ORACLE_API int oracle_embedding_forward(const float* table, const int64_t* tokens, const float* pos, float* out,
                                        int64_t n, int64_t T, int64_t D, int64_t vocab) {
    for (int64_t i = 0; i < n; ++i) {
        const int64_t idx = tokens[i];
        if (idx < 0 || idx >= vocab) return ORACLE_ERR_ARG;
        for (int64_t j = 0; j < D; ++j)
            out[i * D + j] = pos ? table[idx * D + j] + pos[(i % T) * D + j] : table[idx * D + j];
    }
    return ORACLE_OK;
}

/* EmbeddingBackward::backward on the CPU (src/core/grad_fn.cpp:745-757): rows of the upstream gradient are added
 * into the table gradient in token order; out-of-range indices are skipped. */
ORACLE_API void oracle_embedding_backward(const int64_t* tokens, const float* dout, float* dtable, int64_t n,
                                          int64_t D, int64_t vocab) {
    for (int64_t k = 0; k < vocab * D; ++k) dtable[k] = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        const int64_t idx = tokens[i];
        if (idx < 0 || idx >= vocab) continue;
        for (int64_t j = 0; j < D; ++j) dtable[idx * D + j] += dout[i * D + j];
    }
}
