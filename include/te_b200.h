/*
 * te_b200.h -- C ABI of the B200 (sm_100a) FP32 matmul backend for TorchEngine.
 *
 * Every entry point is plain C: pointers, sizes, int status codes.  Nothing here
 * throws, allocates on behalf of the caller in the hot call, or synchronises the
 * device unless the comment says so.  Device pointers are raw addresses already
 * offset by the caller, exactly as the reference passes them to its own
 * launchers (reference src/cuda/elementwise_cuda.h:90 and src/tensor/tensor.h:646-648).
 *
 * Matrices are described the way reference src/tensor/tensor.h:623-627
 * (`cublas_params`) accepts them: every 2-D slice is row-major (last-dim stride 1)
 * or column-major (second-last-dim stride 1) with an explicit leading dimension
 * in elements.  Anything else is TE_ERR_UNSUPPORTED_LAYOUT, the C spelling of the
 * reference's "CUDA matmul only supports row- or column-major 2D slices".
 */
#ifndef TE_B200_H
#define TE_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define TE_API __attribute__((visibility("default")))
#else
#define TE_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (0 = ok) ------------------------------------------------ */
enum {
    TE_OK = 0,
    TE_ERR_BAD_ARGUMENT = 1,        /* null pointer, negative size, bad enum          */
    TE_ERR_UNSUPPORTED_LAYOUT = 2,  /* slice is neither row- nor column-major          */
    TE_ERR_SHAPE_NDIM = 3,          /* "Matmul requires tensors with at least 2 dimensions" (tensor.h:537) */
    TE_ERR_SHAPE_INNER = 4,         /* "Inner dimensions must match for matmul"       (tensor.h:547) */
    TE_ERR_SHAPE_BROADCAST = 5,     /* "Batch dimensions are not broadcastable"       (tensor.h:858) */
    TE_ERR_WORKSPACE = 6,           /* context workspace too small for this call       */
    TE_ERR_CUDA = 7,                /* a CUDA runtime / driver call failed             */
    TE_ERR_DEVICE_TIMEOUT = 8,      /* a bounded device-side wait gave up              */
    TE_ERR_NO_DEVICE = 9            /* library loaded on a machine without a usable GPU */
};

enum { TE_ROW_MAJOR = 0, TE_COL_MAJOR = 1 };
/* TE_PREC_TF32: operands rounded to tf32 by the tensor core (max relative error ~1e-3).  TE_PREC_3XTF32: the
 * FP32-accurate mode (<= 1e-5, typically 2e-6): hi / lo tf32 split with three tensor-core products per term; a product
 * with at most 16 rows, which is bound by reading B once, is computed with FP32 FMAs instead (same accuracy class,
 * error ~4e-7), for a row-major B and for Linear's weight layout alike. */
enum { TE_PREC_TF32 = 0, TE_PREC_3XTF32 = 1 };
enum { TE_EPI_NONE = 0, TE_EPI_BIAS = 1, TE_EPI_BIAS_GELU = 2 };
enum { TE_SCALE_NONE = 0, TE_SCALE_MUL = 1, TE_SCALE_DIV = 2 };

typedef struct te_b200_ctx te_b200_ctx;   /* one per device; owns the workspace   */
typedef void* te_stream_t;                /* a cudaStream_t; NULL = legacy default */

/*
 * One (optionally strided-batched) GEMM:  C[b] = epi( scale( A[b] . B[b] ) ) [+ R[b]].
 * A[b] is M x K, B[b] is K x N, C[b] is M x N row-major with leading dim ldc.
 * Replaces the argument lists of cublasSgemm / cublasSgemmStridedBatched as the
 * reference issues them (src/tensor/tensor.h:690-698, :756-765) and of
 * cuda_matmul_double_buffered_cpasync (src/cuda/elementwise_cuda.h:90).
 *
 * Batches are indexed on two levels, outer x inner, so that attention operands
 * viewed as [B,H,T,d] with strides [T*E, d, E, 1] need no copy
 * (src/nn/multi_head_attention.cpp:19-42).  A stride of 0 broadcasts the operand
 * (the Linear weight of src/nn/linear.cpp:21 under a 3-D input).
 */
typedef struct te_gemm_desc {
    int64_t M, N, K;
    const float* a;            /* device */
    const float* b;            /* device */
    float*       c;            /* device, fully overwritten (beta = 0) */
    int64_t lda, ldb, ldc;     /* elements */
    int32_t a_major, b_major;  /* TE_ROW_MAJOR: (i,j) at i*ld+j;  TE_COL_MAJOR: (i,j) at i+j*ld */
    int64_t batch_outer, batch_inner;          /* >= 1 each; total = outer*inner */
    int64_t a_stride_outer, a_stride_inner;    /* elements; 0 = broadcast        */
    int64_t b_stride_outer, b_stride_inner;
    int64_t c_stride_outer, c_stride_inner;
    float   alpha;             /* used when scale_mode != TE_SCALE_NONE */
    int32_t scale_mode;        /* TE_SCALE_DIV reproduces `S / sqrt(d)` of src/nn/scaledot.cpp:22 */
    int32_t epilogue;          /* TE_EPI_*; bias has N entries, added per column (src/nn/linear.cpp:22) */
    const float* bias;         /* device or NULL */
    float*  preact_out;        /* optional: value before GELU (what GeluBackward needs,
                                  src/core/grad_fn.cpp:169); same layout as c; NULL to skip */
    const float* residual;     /* optional, same layout as c (ldc and the c batch strides), added last:
                                  c = act(scale(A.B) + bias) + residual.  The `x + sublayer(x)` adds of
                                  src/nn/transformer_block.cpp:15-35, and, with residual == c, the gradient
                                  accumulation `*grad = *grad + g` of src/tensor/tensor.cpp:1138-1142.
                                  May alias c (each element is read before it is written); NULL to skip */
    int32_t precision;         /* TE_PREC_* */
    int32_t reserved;
} te_gemm_desc;

/* ---- context --------------------------------------------------------------- */

/* Creates the per-device context on `device` and reserves `workspace_bytes` of
 * device scratch (operand packing for 3xTF32 and for operands TMA cannot address).
 * Replaces the process-wide lazily created cuBLAS handle of
 * src/core/cuda_utils.cpp:48-55.  Returns TE_ERR_NO_DEVICE when no GPU is usable.
 * Calls that take the context launch on the caller's stream: `device` must be the calling
 * thread's current device then (they return TE_ERR_BAD_ARGUMENT otherwise).  A context is
 * used by one thread and one stream at a time (its scratch is shared by its calls). */
TE_API int te_b200_init(int device, size_t workspace_bytes, te_b200_ctx** out_ctx);
TE_API int te_b200_destroy(te_b200_ctx* ctx);

/* Scratch bytes a call with this descriptor needs (0 when operands are used in place). */
TE_API int te_b200_gemm_workspace_size(const te_gemm_desc* d, size_t* out_bytes);

/* Number of kernels of this library launched through `ctx` since creation. */
TE_API int64_t te_b200_launch_count(const te_b200_ctx* ctx);

/* Human-readable text for the last non-zero status returned on this thread. */
TE_API const char* te_b200_last_error(void);
/* Fixed message for a status code; the shape errors repeat the reference's text. */
TE_API const char* te_b200_status_string(int status);

/* After a stream has been synchronised: returns TE_ERR_DEVICE_TIMEOUT if any kernel
 * launched through ctx gave up a bounded wait since the last call, else TE_OK. */
TE_API int te_b200_check_device_status(te_b200_ctx* ctx);

/* Every wait inside a kernel of this library (on an mbarrier that a copy, the tensor core or another warp
 * completes) is bounded: when it runs out the kernel records where, winds down and returns, and
 * te_b200_check_device_status reports TE_ERR_DEVICE_TIMEOUT.  This sets the bound for kernels launched through ctx
 * afterwards (0 = the default of two seconds).  Synchronises `stream`.  No reference counterpart: the reference's
 * kernels contain no waits (src/cuda/elementwise_cuda.cu). */
TE_API int te_b200_set_wait_limit_ns(te_b200_ctx* ctx, uint64_t limit_ns, te_stream_t stream);
/* Launches a one-warp kernel that waits, with that bound, on a barrier nothing arrives at: after synchronising,
 * te_b200_check_device_status returns TE_ERR_DEVICE_TIMEOUT ("... site code 901") and the context works as before.
 * The kernel returns by itself; nothing traps, faults or hangs.  Proves the failure path of the waits end to end. */
TE_API int te_b200_selftest_wait_timeout(te_b200_ctx* ctx, te_stream_t stream);

/* ---- GEMM ------------------------------------------------------------------ */

/* Asynchronous on `stream`.  Replaces the body of Tensor::cuda_matmul_impl_f32
 * (src/tensor/tensor.h:614-793) for one uniformly strided group of batches. */
TE_API int te_b200_gemm_f32(te_b200_ctx* ctx, const te_gemm_desc* d, te_stream_t stream);

/* N-D matmul with NumPy batch broadcasting over raw shape/stride arrays (strides in
 * elements), i.e. Tensor::matmul -> matmul_impl<float> -> cuda_matmul_impl_f32
 * (src/tensor/tensor.cpp:761-785, src/tensor/tensor.h:529-612, :838-906).
 * `c` is a fresh contiguous [batch..., M, N] buffer.  out_shape (capacity 8) and
 * out_ndim receive the result shape when non-NULL.  If `c` is NULL only the shape is
 * computed and validated (no GPU needed). */
TE_API int te_b200_matmul_nd(te_b200_ctx* ctx,
                      const float* a, const int64_t* a_shape, const int64_t* a_strides, int a_ndim,
                      const float* b, const int64_t* b_shape, const int64_t* b_strides, int b_ndim,
                      float* c, int64_t* out_shape, int* out_ndim,
                      int precision, te_stream_t stream);

/* The 3xTF32 GEMM for callers that may not allocate device memory.  No counterpart in the reference (its
 * launchers allocate freely, src/cuda/elementwise_cuda.cu:2302-2346).  Some hosts cannot call cudaMalloc, or let
 * a library call it for them: a plugin inside a framework whose allocator owns the device, a loop with a
 * fixed memory budget, code that has already started capturing its streams.  For them this entry point
 * needs no te_b200_ctx and calls no allocator: the tf32 hi/lo planes go into one fixed device array of
 * TE_B200_STATIC_SCRATCH_BYTES inside the library image.  The CUDA runtime reserves that array on a GPU when it
 * loads this part of the library there, which (with the default lazy loading) is during the first call on that
 * device; from then on the GPU holds it until the process exits.
 *   - d->precision must be TE_PREC_3XTF32; the device that is current when called is used.
 *   - This entry always reads tf32 hi / lo planes out of the array: two planes of M x K4 and two of N x K4 floats per
 *     batch (K4 = K rounded up to 4), each rounded up to 256 bytes.  A problem that needs more than
 *     TE_B200_STATIC_SCRATCH_BYTES is refused with TE_ERR_WORKSPACE; nothing is launched.  (te_b200_gemm_workspace_size
 *     describes the context path, which needs no plane storage for thin and small problems.)
 *   - The first successful call on a device does all one-time work (the load above, the array's address, and the
 *     attributes of every kernel any problem shape can reach): make it before any stream capture begins and while
 *     the device still has the array's size free.  If it fails, the next call tries again.
 *   - Calls share the array, which keeps the previous call's contents; each call rewrites what it reads
 *     (planes, status word), but calls that overlap on the GPU race.  Serialise them on one stream.
 *   - host_status (optional) receives, asynchronously on `stream`, 0 or the code of a device-side wait
 *     that gave up; read it after synchronising the stream.  It is the target of a device-to-host copy: use pinned
 *     memory, and it must be pinned (or NULL) if the stream is being captured.  An empty problem (M or N zero)
 *     launches nothing and stores 0 at once. */
#define TE_B200_STATIC_SCRATCH_BYTES (64ll << 20)
TE_API int te_b200_gemm_3xtf32_static(const te_gemm_desc* d, te_stream_t stream, int* host_status);

/* Same GEMM with HOST buffers: copies A and B to the device, runs, copies C back and
 * synchronises.  This is the call a CPU-resident reference Tensor would make
 * (Tensor::toDevice + matmul + toDevice back, src/tensor/tensor.cpp:308-340). */
TE_API int te_b200_gemm_f32_host(te_b200_ctx* ctx, const te_gemm_desc* d_host);

/* ---- row operations around the attention GEMMs ----------------------------- */

/* out[r,:] = softmax(in[r,:]) over `cols` contiguous floats, rows*cols dense.
 * Replaces cuda_softmax_forward (src/cuda/elementwise_cuda.cu:2424-2448, :2469). in may equal out. */
TE_API int te_b200_softmax_rows_f32(te_b200_ctx* ctx, const float* in, float* out,
                             int64_t rows, int64_t cols, te_stream_t stream);
/* dx = s * (dy - sum(dy*s)) per row.  Replaces cuda_softmax_backward (:2450-2467, :2476). */
TE_API int te_b200_softmax_backward_rows_f32(te_b200_ctx* ctx, const float* s, const float* dy, float* dx,
                                      int64_t rows, int64_t cols, te_stream_t stream);
/* y = gelu_tanh(x).  Replaces cuda_gelu (:2701-2707, :2726). */
TE_API int te_b200_gelu_f32(te_b200_ctx* ctx, const float* x, float* y, int64_t n, te_stream_t stream);
/* dx = dy * gelu'(x) with x the pre-activation.  Replaces cuda_gelu_backward (:2709-2724, :2732). */
TE_API int te_b200_gelu_backward_f32(te_b200_ctx* ctx, const float* x, const float* dy, float* dx,
                              int64_t n, te_stream_t stream);
/* out[j] = sum_i in[i*ld + j], i < rows, j < cols: the bias gradient that AddBackward obtains
 * through reduce_gradient -> cuda_sum_dim (src/core/grad_fn.cpp:13-58, :93-102). */
TE_API int te_b200_colsum_f32(te_b200_ctx* ctx, const float* in, int64_t rows, int64_t cols, int64_t ld,
                       float* out, te_stream_t stream);

/* ---- fused callers ---------------------------------------------------------- */

/* Y[rows,out] = act(X[rows,in] . W[out,in]^T + bias).  Linear::forward (src/nn/linear.cpp:14-23)
 * with the bias add, and optionally FeedForward's GELU (src/nn/ffn.cpp:12-16), in the epilogue.
 * gelu != 0 selects bias+GELU; preact (optional) receives X.W^T+bias. */
TE_API int te_b200_linear_forward(te_b200_ctx* ctx, const float* x, const float* w, const float* bias,
                           float* y, float* preact, int64_t rows, int64_t in_features,
                           int64_t out_features, int gelu, int precision, te_stream_t stream);
/* dX = dY.W, dW[out,in] = dY^T.X (one GEMM with K = rows, written directly as [out,in]),
 * db = column sums of dY.  MatMulBackward + AddBackward + TransposeBackward of the Linear graph
 * (src/core/grad_fn.cpp:93-102, :126-139, :397-403).  Any of dx/dw/db may be NULL. */
TE_API int te_b200_linear_backward(te_b200_ctx* ctx, const float* x, const float* w, const float* dy,
                            float* dx, float* dw, float* db, int64_t rows, int64_t in_features,
                            int64_t out_features, int precision, te_stream_t stream);
/* The same when x is the output of a GELU whose pre-activation is x_preact [rows,in] (the second
 * Linear of FeedForward, src/nn/ffn.cpp:12-16): dx receives the gradient with respect to the
 * PRE-activation, dX o gelu'(x_preact): the dX product followed by GeluBackward
 * (src/core/grad_fn.cpp:169-204) in place, one call for both.  (Folding GeluBackward into the
 * product's epilogue was built and measured: a second [rows,in] input read in the epilogue costs this
 * short-K product more than the separate pass does -- 16384 x 384 -> 1536 goes from 42 to 63 us with a
 * residual-like input against 49 us for the pass -- because the product is bound by what an SM takes in
 * from L2, and the extra tile competes with the operand tiles for it.)
 * x_preact == NULL: identical to te_b200_linear_backward. */
TE_API int te_b200_linear_backward_gelu(te_b200_ctx* ctx, const float* x, const float* x_preact,
                                 const float* w, const float* dy, float* dx, float* dw, float* db,
                                 int64_t rows, int64_t in_features, int64_t out_features,
                                 int precision, te_stream_t stream);

/* The general form of the two calls above.  dx_residual (optional, [rows,in]) is added into dx: the gradient that
 * reaches the Linear's input over a parallel branch (the `x + sublayer(x)` of src/nn/transformer_block.cpp:15-35);
 * it may be dx itself, which chains the input gradients of several Linears reading the same x.  accumulate != 0
 * adds dW and db to the buffers' contents instead of overwriting them -- the `*grad = *grad + g` of the autograd
 * engine (src/tensor/tensor.cpp:1138-1142) folded into the producing kernels.  x_preact as in _gelu (it excludes
 * dx_residual).  dx_colsum (optional, [in]) receives the column sums of the returned dx: the bias gradient of the
 * Linear whose output x (or x_preact) is, i.e. what its AddBackward would obtain through reduce_gradient
 * (src/core/grad_fn.cpp:13-58, :93-102); with x_preact it comes out of the GeluBackward pass itself. */
TE_API int te_b200_linear_backward_ex(te_b200_ctx* ctx, const float* x, const float* x_preact, const float* w,
                               const float* dy, float* dx, const float* dx_residual, float* dx_colsum, float* dw,
                               float* db, int accumulate, int64_t rows, int64_t in_features,
                               int64_t out_features, int precision, te_stream_t stream);

/* O = softmax(Q.K^T / sqrt(d)) . V for Q,K,V viewed as [B,H,T,d] with explicit element
 * strides (last-dim stride must be 1).  ScaledDot::forward (src/nn/scaledot.cpp:8-27).
 * p_out is a dense [B,H,T,T] buffer that receives the probabilities (SoftmaxBackward and
 * the backward GEMMs need them); o is dense [B,H,T,d] with strides o_strides. */
typedef struct te_attn_desc {
    int64_t B, H, T, d;
    const float* q; const float* k; const float* v;
    int64_t q_strides[3];   /* element strides of dims B, H, T (dim d has stride 1) */
    int64_t k_strides[3];
    int64_t v_strides[3];
    float* p_out;           /* [B,H,T,T] dense, required */
    float* o;               /* output */
    int64_t o_strides[3];
    int32_t precision;
    int32_t reserved;
} te_attn_desc;
TE_API int te_b200_attention_forward(te_b200_ctx* ctx, const te_attn_desc* d, te_stream_t stream);

/* Gradients of the call above given dO: the backward of ScaledDot::forward's graph
 * (MatMulBackward of P.V and of Q.K^T, src/core/grad_fn.cpp:126-139; SoftmaxBackward,
 * :569-665; DivBackward, :142-156) as one call:
 *     dV = P^T.dO      dP = dO.V^T      dS = P o (dP - rowsum(P o dP)) / sqrt(d)
 *     dQ = dS.K        dK = dS^T.Q
 * p is the dense [B,H,T,T] probability tensor the forward call wrote; o its output (used for
 * rowsum(P o dP) = rowsum(dO o O) by the fused kernel; may be NULL, which selects the unfused
 * path).  q, k, v, o, d_o and the outputs dq, dk, dv are [B,H,T,d] views with element strides
 * for B, H, T and unit stride over d.  The unfused path keeps dP/dS ([B,H,T,T] floats) in the
 * context workspace. */
typedef struct te_attn_bwd_desc {
    int64_t B, H, T, d;
    const float* q; const float* k; const float* v;
    int64_t q_strides[3];
    int64_t k_strides[3];
    int64_t v_strides[3];
    const float* p;         /* [B,H,T,T] dense */
    const float* o;         /* forward output, optional */
    int64_t o_strides[3];
    const float* d_o;       /* gradient of the output */
    int64_t d_o_strides[3];
    float* dq; float* dk; float* dv;
    int64_t dq_strides[3];
    int64_t dk_strides[3];
    int64_t dv_strides[3];
    int32_t precision;
    int32_t reserved;
} te_attn_bwd_desc;
TE_API int te_b200_attention_backward(te_b200_ctx* ctx, const te_attn_bwd_desc* d, te_stream_t stream);

/* MultiHeadAttention::forward (src/nn/multi_head_attention.cpp:19-42) as one call: the three input projections
 * (bias in the GEMM epilogue), scaled-dot attention on the head views [B,H,T,E/H] of the [B,T,E] projections
 * (strides [T*E, E/H, E]: no copy), the head outputs written straight back in merged [B,T,E] order, and the output
 * projection, optionally with the block's residual input added (src/nn/transformer_block.cpp:20-24).
 * Weights are [E,E] as Linear stores them ([out,in], src/nn/linear.cpp:7); biases [E] or NULL.  q, k, v, p, attn are
 * caller-owned buffers the backward call needs again.
 *
 * One-GEMM form of the three projections: with wqkv given (scratch of 3*E*E + 3*E floats) and q, k, v the three column
 * blocks of ONE [B,T,3E] buffer (k == q + E, v == q + 2E, ld_qkv == 3*E), the call gathers the three weights and
 * biases into wqkv ([3E,E] then [3E]) and computes x . Wqkv^T + bqkv in one product; every element is the same dot
 * product as in the three-GEMM form.  ld_qkv == 0 or E: q, k, v are three dense [B,T,E] buffers. */
typedef struct te_mha_desc {
    int64_t B, T, E, H;
    const float* x;                                  /* [B,T,E] */
    const float *wq, *bq, *wk, *bk, *wv, *bv, *wo, *bo;
    float *q, *k, *v;                                /* the projections, row stride ld_qkv */
    float* p;                                        /* [B,H,T,T] attention probabilities */
    float* attn;                                     /* [B,T,E] merged head outputs (input of the out projection) */
    float* y;                                        /* [B,T,E] result */
    const float* residual;                           /* optional [B,T,E], added to y */
    int32_t precision;
    int32_t reserved;
    float* wqkv;                                     /* optional scratch, see above */
    int64_t ld_qkv;                                  /* row stride of q, k, v: 0 / E (dense) or 3*E */
} te_mha_desc;
TE_API int te_b200_mha_forward(te_b200_ctx* ctx, const te_mha_desc* d, te_stream_t stream);

/* Backward of the call above: the graph MatMulBackward/AddBackward of four Linears, TransposeBackward and
 * ReshapeBackward of the head split and merge, and the attention core (src/core/grad_fn.cpp:93-156, :397-403,
 * :559-665).  dq, dk, dv, dattn are caller-owned [B,T,E] scratch.  dx = dx_residual + dq.Wq + dk.Wk + dv.Wv.
 * Parameter gradients are [E,E] / [E] like the parameters; NULL skips one; accumulate != 0 adds to their contents.
 *
 * One-GEMM form (see the forward call): with wqkv (as the forward call left it) and dwqkv (scratch, 3*E*E + 3*E
 * floats) given, ld_qkv == 3*E, and dq, dk, dv the column blocks of one [B,T,3E] buffer like q, k, v, the call runs
 * dx = dx_residual + dQKV . Wqkv as one K = 3E product, dWqkv = dQKV^T . x as one product and the three bias
 * gradients as one column sum, then scatters dwqkv to the six gradient pointers. */
typedef struct te_mha_bwd_desc {
    int64_t B, T, E, H;
    const float* x;
    const float *wq, *wk, *wv, *wo;
    const float *q, *k, *v, *p, *attn;               /* as the forward call left them */
    const float* dy;                                 /* [B,T,E] */
    float* dx;                                       /* [B,T,E] */
    const float* dx_residual;                        /* optional [B,T,E] */
    float *dwq, *dbq, *dwk, *dbk, *dwv, *dbv, *dwo, *dbo;
    float *dq, *dk, *dv, *dattn;                     /* scratch; dq, dk, dv with row stride ld_qkv */
    int32_t accumulate;
    int32_t precision;
    const float* wqkv;                               /* optional, see above */
    float* dwqkv;                                    /* optional scratch */
    int64_t ld_qkv;                                  /* row stride of q, k, v, dq, dk, dv: 0 / E or 3*E */
} te_mha_bwd_desc;
TE_API int te_b200_mha_backward(te_b200_ctx* ctx, const te_mha_bwd_desc* d, te_stream_t stream);

/* ---- the GPT step's kernels around the matmuls ------------------------------- */
/* Not matmuls, but what a training step of the reference's GPT runs between them; with the
 * GEMMs and attention on this backend they were what bounded the step.  All reductions run in
 * a fixed order (the reference's CUDA kernels use atomicAdd). */

/* y = (x - mean) / sqrt(var + eps) * gamma + beta over the last dimension of x [rows, cols],
 * biased variance.  LayerNorm::forward (src/nn/layernorm.cpp:19-82; kernel
 * src/cuda/elementwise_cuda.cu:2497-2521).  cols <= 1024. */
TE_API int te_b200_layernorm_forward(te_b200_ctx* ctx, const float* x, const float* gamma,
                              const float* beta, float* y, int64_t rows, int64_t cols, float eps,
                              te_stream_t stream);
/* {dx, dgamma, dbeta} from x, gamma and the upstream gradient dy; mean and variance are
 * recomputed from x as LayerNormBackward::backward does (src/core/grad_fn.cpp:405-538; kernel
 * elementwise_cuda.cu:2523-2568).  dgamma / dbeta may be NULL.  Uses the context workspace. */
TE_API int te_b200_layernorm_backward(te_b200_ctx* ctx, const float* x, const float* gamma,
                               const float* dy, float* dx, float* dgamma, float* dbeta,
                               int64_t rows, int64_t cols, float eps, te_stream_t stream);
/* The same with dx_residual ([rows, cols], optional) added into dx: in a pre-LN block the gradient of the block's
 * input is the LayerNorm's dx plus the gradient that bypasses it over the residual branch
 * (src/nn/transformer_block.cpp:15-35; AddBackward, src/core/grad_fn.cpp:93-102).  May be dx itself.
 * dx_colsum (optional, [cols]) receives the column sums of the returned dx -- the bias gradient of the Linear whose
 * output feeds the residual stream at this point -- accumulated beside dgamma and dbeta in the same pass. */
TE_API int te_b200_layernorm_backward_ex(te_b200_ctx* ctx, const float* x, const float* gamma,
                                  const float* dy, float* dx, const float* dx_residual, float* dgamma,
                                  float* dbeta, float* dx_colsum, int64_t rows, int64_t cols, float eps,
                                  te_stream_t stream);
/* out[i][:] = table[tokens[i]][:] (+ pos[i % seq_len][:] when pos is not NULL) for n int64
 * tokens: Embedding::forward (src/nn/embedding.cpp:18-60) with the positional sum of
 * GPT::forward (src/nn/gpt.cpp:30-69) folded in.  An index outside [0, vocab) writes zeros and
 * is reported by te_b200_check_device_status ("Embedding index out of range"). */
TE_API int te_b200_embedding_forward(te_b200_ctx* ctx, const float* table, const int64_t* tokens,
                              const float* pos, float* out, int64_t n, int64_t seq_len,
                              int64_t dim, int64_t vocab, te_stream_t stream);
/* dtable[v][:] = sum of dout[i][:] over the positions with tokens[i] == v, added in ascending i
 * (the order of EmbeddingBackward's CPU loop, src/core/grad_fn.cpp:745-757); dtable is fully
 * overwritten.  Cost grows with vocab * n: meant for the reference's small vocabularies. */
TE_API int te_b200_embedding_backward(te_b200_ctx* ctx, const int64_t* tokens, const float* dout,
                               float* dtable, int64_t n, int64_t dim, int64_t vocab,
                               te_stream_t stream);
/* Mean cross-entropy of logits [rows, vocab] against int64 targets [rows] into the device float
 * *loss (may be NULL), and, when dlogits is not NULL, its gradient
 * (softmax - one_hot) * upstream / rows.  crossEntropyLoss::forward_batched
 * (src/loss/CrossEntropyLoss.cpp:47-127) and CrossEntropyBatchedBackward
 * (src/core/grad_fn.cpp:271-346).  Uses the context workspace. */
TE_API int te_b200_cross_entropy(te_b200_ctx* ctx, const float* logits, const int64_t* targets,
                          float* loss, float* dlogits, float upstream, int64_t rows, int64_t vocab,
                          te_stream_t stream);

/* ---- introspection --------------------------------------------------------- */

/* Which kernel form te_b200_gemm_f32 would use for this problem on a GPU with `sm_count` SMs
 * and `scratch_bytes` of context workspace left for split-K partials: tile width (64, 128,
 * 192, 256, 384 or 512 columns), whether the CTA-pair (cta_group::2, 256-row tiles) or the single-CTA
 * (128-row tiles) kernel runs, and into how many work units K is split.  Pure host
 * arithmetic (the tile cost model); needs no GPU and no context.  No reference counterpart:
 * the reference's dispatcher has one kernel per backend (src/tensor/tensor.h:652-698). */
TE_API int te_b200_gemm_plan(const te_gemm_desc* d, int sm_count, size_t scratch_bytes,
                      int* tile_n, int* cta_pair, int* k_splits);

/* ---- sharding helpers (multi-GPU: one process per GPU) ----------------------- */

/* Splits `total` units (N columns, or batch indices) over `world` ranks in blocks that are
 * multiples of `align` (the last rank takes the ragged tail).  No reference counterpart:
 * the reference has no multi-device code (README.md:47). */
TE_API int te_b200_shard_range(int64_t total, int world, int rank, int64_t align,
                        int64_t* out_begin, int64_t* out_count);

/* ---- multi-GPU driver (one process per GPU, NCCL over NVLink) -------------------- */
/* None of this has a counterpart in the reference (no multi-device code, README.md:47).  Computing a shard needs no
 * exchange; these calls move data AROUND the products.  NCCL is bound at run time (libnccl.so.2). */
typedef struct te_b200_comm te_b200_comm;

/* 128 bytes identifying a new communicator: rank 0 creates them, the caller hands them to every rank (a file, a
 * socket, torch.distributed's store ...). */
#define TE_B200_COMM_ID_BYTES 128
TE_API int te_b200_comm_unique_id(void* out_id);
/* Joins rank `rank` of `world` (collective: every rank calls it); ctx's device must be current. */
TE_API int te_b200_comm_init(te_b200_ctx* ctx, const void* id, int world, int rank, te_b200_comm** out_comm);
TE_API int te_b200_comm_destroy(te_b200_comm* comm);
TE_API int te_b200_comm_rank(const te_b200_comm* comm, int* world, int* rank);

/* Reassembles C [M,N] (row-major, pitch ld_full) on every rank from the ranks' column blocks as
 * te_b200_shard_range(N, world, r, align) assigns them.  c_local is this rank's dense [M, n_local] block; staging
 * holds M*N floats.  One all-gather of the blocks as they are, then one re-tile kernel.  Asynchronous on `stream`. */
TE_API int te_b200_all_gather_columns(te_b200_comm* comm, const float* c_local, int64_t M, int64_t N, int64_t align,
                               float* staging, float* c_full, int64_t ld_full, te_stream_t stream);
/* The same for row blocks of a dense [rows, cols] matrix, in place: this rank's rows
 * (te_b200_shard_range(rows, world, rank, align)) are already at their position inside `full`. */
TE_API int te_b200_all_gather_rows(te_b200_comm* comm, float* full, int64_t rows, int64_t cols, int64_t align,
                            te_stream_t stream);
/* The one exchange of a data-parallel training step (every rank ran forward + backward on its own slice of the batch,
 * with a mean loss over `local_rows` rows): grads (n floats on the device) becomes the row-weighted average of the
 * ranks' gradients, i.e. the gradient of the mean loss over the whole batch.  One all-reduce of the gradient and one of
 * the row count, in place, asynchronous on `stream`.  A rank with local_rows == 0 contributes nothing.  (The reference
 * has no multi-device code; its single-device step divides by the batch's rows in CrossEntropyBatchedBackward,
 * src/core/grad_fn.cpp:295.) */
TE_API int te_b200_all_reduce_batch_mean(te_b200_comm* comm, float* grads, int64_t n, int64_t local_rows, te_stream_t stream);
/* te_b200_gemm_f32_host for `world` ranks that all hold the same HOST operands (row-major A [M,K] and B [K,N]): each
 * rank copies 1/world of A's rows and its column block of B (te_b200_shard_range(N, world, rank, column_align)) to
 * its GPU, the ranks replicate A over NVLink, each multiplies and copies its columns of C back into its host C.
 * Per GPU, PCIe carries 1/world of the bytes.  Collective; synchronises before returning. */
TE_API int te_b200_gemm_f32_host_sharded(te_b200_comm* comm, const te_gemm_desc* d_host, int64_t column_align);

#ifdef __cplusplus
}
#endif
#endif /* TE_B200_H */
