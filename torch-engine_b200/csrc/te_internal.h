// Internal (C++) interfaces between the C-ABI layer and the CUDA translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>
#include <unordered_map>
#include "te_b200.h"

namespace te {

// One GEMM operand as the kernel sees it: logical [rows, K] where rows is the M (for A) or
// N (for B) extent.  mn_major == false: K is the contiguous index (element (r,k) at r*ld + k).
// mn_major == true: the row index is contiguous (element (r,k) at k*ld + r).
struct Operand {
    const float* ptr = nullptr;
    bool mn_major = false;
    int64_t rows = 0;
    int64_t ld = 0;
    int64_t stride_inner = 0, stride_outer = 0;  // elements; 0 = broadcast over that batch level
};

struct GemmProblem {
    int64_t M = 0, N = 0, K = 0;
    int64_t batch_inner = 1, batch_outer = 1;
    Operand a, b;                 // raw fp32 (TF32 mode) or the tf32 "hi" planes (3xTF32)
    const float* a_lo = nullptr;  // 3xTF32 on packed planes: "lo" planes with the geometry of a / b
    const float* b_lo = nullptr;
    bool split_in_kernel = false; // 3xTF32 on raw operands: the kernel derives hi / lo itself (single-CTA kernel only)
    float* c = nullptr;
    int64_t ldc = 0, c_stride_inner = 0, c_stride_outer = 0;
    float* preact = nullptr;
    const float* bias = nullptr;
    const float* residual = nullptr;   // optional, layout of c; added last; may alias c
    float alpha = 1.0f;
    int scale_mode = TE_SCALE_NONE;
    int epilogue = TE_EPI_NONE;
    // scratch the launcher may use for split-K partial tiles (may be null / 0)
    float* split_ws = nullptr;
    size_t split_ws_bytes = 0;
};

}  // namespace te

// One encoded tensor map and the arguments it was encoded from (context-local cache, see encode_tiled_cached).
struct TensorMapCacheEntry {
    uint64_t key[16];
    unsigned char map[128];
    bool valid = false;
};

struct te_b200_ctx {
    int device = 0;
    int sm_count = 0;
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
    // Device status area (STATUS_AREA_BYTES; the static-scratch entry point has the first 256 bytes only).  Word 0: code
    // written by a kernel whose bounded wait gave up (or that met a bad index).  Bytes 8..15: the wait limit in
    // nanoseconds every bounded wait reads on its slow path (0 = default).  Words STATUS_COUNTER_WORD..: arrival
    // counters of the column-sum kernel, zero between launches.
    int* d_status = nullptr;
    int64_t launches = 0;
    uint64_t wait_limit_ns = 0;   // host copy of the limit stored in the status area (0 = default)
    // Per-kernel one-time state of THIS context, keyed by the kernel's address: 1 once its attributes are set; for
    // the CTA-pair kernels the number of pairs that can be resident at once.
    std::unordered_map<const void*, int> kernel_state;
    // Recently encoded tensor maps: a repeated step (same pointers, shapes and strides) skips the driver's encoder.
    TensorMapCacheEntry tmap_cache[256];
    int64_t tmap_hits = 0, tmap_misses = 0;
    void* encode_tiled = nullptr; // cuTensorMapEncodeTiled, resolved through the runtime
    void* host_stage = nullptr;   // grow-only device staging used by the host-buffer entry point
    size_t host_stage_bytes = 0;
    // host-buffer entry point: copy-in, compute and copy-out streams plus per-block events (created on first use)
    cudaStream_t host_streams[3] = {nullptr, nullptr, nullptr};
    cudaEvent_t host_events[33] = {};
    bool host_pipe_ready = false;
};

namespace te {

void set_error(const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);

// cuTensorMapEncodeTiled for a 4-D fp32 tensor through the context's cache.  Returns the driver's CUresult (0 = ok).
int encode_tiled_cached(te_b200_ctx* ctx, void* out_map, const void* ptr, const uint64_t dims[4], const uint64_t strides[3],
                        const uint32_t box[4], int swizzle, int l2_promotion);

constexpr int STATUS_AREA_BYTES = 8192;
constexpr int STATUS_COUNTER_WORD = 16;
constexpr int STATUS_COUNTER_WORDS = STATUS_AREA_BYTES / 4 - STATUS_COUNTER_WORD;

// Device status codes that are not wait sites.
constexpr int STATUS_BAD_EMBEDDING_INDEX = 201;   // "Embedding index out of range" (src/nn/embedding.cpp:53-55)
constexpr int STATUS_BAD_TARGET_INDEX = 202;      // cross-entropy target outside [0, vocab)
constexpr int STATUS_SELFTEST_WAIT = 901;         // the wait self-test's barrier, which nobody arrives at

// True when TMA can address the operand in place (16-byte aligned base, strides multiple of 16 B).
bool operand_tma_ok(const Operand& op, int64_t K, int64_t batch_inner, int64_t batch_outer);

// gemm_sm100.cu
int launch_gemm(te_b200_ctx* ctx, const GemmProblem& p, cudaStream_t stream);
int launch_wait_selftest(te_b200_ctx* ctx, cudaStream_t stream);
// Loads every kernel a 3xTF32 GEMM can reach (both single-CTA tile widths, the CTA-pair form, the split-K reduction,
// the packing kernels) and sets their attributes in this context, so that no later call does first-use work.
int prepare_3xtf32_kernels(te_b200_ctx* ctx);
int prepare_pair_3xtf32_kernel(te_b200_ctx* ctx);   // gemm_sm100_2cta.cu
int prepare_pack_kernels();                         // pack.cu
// The kernel form launch_gemm picks: tile width, CTA-pair or single-CTA kernel, K splits.  Uses only the extents, the
// precision (a_lo set or not), the scratch size of `p` and ctx->sm_count; touches no device.
struct TileChoice { int bn; bool pair; int k_splits; };
// 3xTF32: where the tf32 hi / lo parts of the operands come from.  Splitting inside the kernel (converter warps rewrite
// every landed stage in shared memory) needs no plane storage and no extra pass over global memory, but a tile of A is
// converted again for every tile of N it meets (and B for every tile of M), and the conversion shares the shared-memory
// bandwidth the tensor core feeds from.  Measured: it wins where one extent is thin (16x8192x8192: 0.138 against
// 0.275 ms) and on small problems (no two extra launches); the packing pre-pass wins on large squares (4096^3: 0.72
// against 0.96 ms).
// A left operand stored M-major (a weight gradient dY^T . X) would have to be transposed by the packing pass, which
// costs more than the split in shared memory up to a larger size (384x16384x1536: 0.125 against 0.206 ms,
// 3072x4096x768: 0.126 against 0.140 ms).
inline bool three_x_split_in_kernel(int64_t M, int64_t N, int64_t K, bool a_m_major) {
    const int64_t thin = M < N ? M : N;
    const double mnk = (double)M * (double)N * (double)K;
    return thin <= 256 || mnk <= 2147483648.0 || (a_m_major && mnk <= 17179869184.0);
}
TileChoice choose_tile(const te_b200_ctx* ctx, const GemmProblem& p);

// attention_sm100.cu: fused QK^T -> softmax -> PV.  Returns -1 when the problem is outside the fused kernel's limits.
int launch_attention_fused(te_b200_ctx* ctx, const te_attn_desc* t, cudaStream_t stream);
// attention_bwd_sm100.cu: fused backward of the same.  Returns -1 when the problem is outside the fused kernel's limits.
int launch_attention_backward_fused(te_b200_ctx* ctx, const te_attn_bwd_desc* t, cudaStream_t stream);

// pack.cu: writes dense K-major planes [batch_outer][batch_inner][rows][kp] (kp = K rounded up to 4).
// split == false: dst_hi receives a copy.  split == true: dst_hi / dst_lo receive the tf32 hi / lo parts.
int launch_pack(te_b200_ctx* ctx, const Operand& src, int64_t K, int64_t batch_inner,
                int64_t batch_outer, float* dst_hi, float* dst_lo, bool split, cudaStream_t stream);

// rowops.cu
int launch_softmax_rows(te_b200_ctx*, const float*, float*, int64_t rows, int64_t cols, cudaStream_t);
int launch_softmax_backward_rows(te_b200_ctx*, const float* s, const float* dy, float* dx,
                                 int64_t rows, int64_t cols, cudaStream_t);
int launch_gelu(te_b200_ctx*, const float*, float*, int64_t n, cudaStream_t);
int launch_gelu_backward(te_b200_ctx*, const float* x, const float* dy, float* dx, int64_t n,
                         cudaStream_t);
int launch_gelu_backward_colsum(te_b200_ctx*, const float* x, const float* dy, float* dx, int64_t rows, int64_t cols,
                                float* colsum_out, cudaStream_t);
int launch_colsum(te_b200_ctx*, const float* in, int64_t rows, int64_t cols, int64_t ld, float* out, bool accumulate,
                  cudaStream_t);
// FP32-FMA form of a thin (M <= 16) FP32-accurate product; -1 when the problem is outside its limits.
int launch_thin_fp32(te_b200_ctx*, const te::GemmProblem& g, cudaStream_t st);
int launch_pack_qkv(te_b200_ctx*, const float* const w[3], const float* const b[3], float* packed, int64_t wn, int64_t bn,
                    cudaStream_t st);
int launch_unpack_qkv(te_b200_ctx*, const float* packed, float* const w[3], float* const b[3], int64_t wn, int64_t bn,
                      bool accumulate, cudaStream_t st);

// norm_embed_loss.cu: the GPT step's kernels around the matmuls
int launch_layernorm_forward(te_b200_ctx*, const float* x, const float* gamma, const float* beta, float* y, int64_t rows,
                             int64_t cols, float eps, cudaStream_t);
int launch_layernorm_backward(te_b200_ctx*, const float* x, const float* gamma, const float* dy, float* dx,
                              const float* dx_residual, float* dgamma, float* dbeta, float* dx_colsum, int64_t rows, int64_t cols,
                              float eps, cudaStream_t);
int launch_embedding_forward(te_b200_ctx*, const float* table, const int64_t* tokens, const float* pos, float* out, int64_t n,
                             int64_t T, int64_t D, int64_t vocab, cudaStream_t);
int launch_embedding_backward(te_b200_ctx*, const int64_t* tokens, const float* dout, float* dtable, int64_t n, int64_t D,
                              int64_t vocab, cudaStream_t);
int launch_cross_entropy(te_b200_ctx*, const float* logits, const int64_t* targets, float* loss, float* grad, float upstream,
                         int64_t rows, int64_t V, cudaStream_t);

}  // namespace te
