// Multi-GPU driver of the matmul path: one process per GPU, one communicator per context.
//
// The path shards without any exchange while computing: a large product by N column blocks (every rank holds all of A
// and its own columns of B), batched products by batch index.  What this file adds is the traffic AROUND the
// products, over NCCL (NVLink / NVSwitch):
//   * te_b200_all_gather_columns  reassembles C [M,N] on every rank from the ranks' column blocks: the blocks travel
//     as they are (contiguous [M, n_r] pieces) into a staging buffer [rank][M][n_r] and one kernel re-tiles them into
//     row-major [M,N];
//   * te_b200_all_gather_rows     the same for row blocks (contiguous in a row-major matrix: no re-tile), used to
//     replicate A when every rank uploaded only its share of it;
//   * te_b200_gemm_f32_host_sharded  the host-buffer entry point for N ranks: each rank copies M/world rows of A and
//     its column block of B over PCIe, the ranks replicate A over NVLink, each multiplies its block and copies its
//     columns of C back.  PCIe carries 1/world of the bytes per GPU; the replication costs NVLink time only.
// No kernel here or elsewhere reads another GPU's memory; peers are reached through NCCL only.
//
// NCCL is bound at run time (dlopen of libnccl.so.2): inside a process that already loaded an NCCL (for example
// through torch) that copy is used, otherwise the system's.  The reference has no counterpart of any of this: it has
// no multi-device code (README.md:47).
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>

#include "pdl.cuh"
#include "te_internal.h"

namespace {

// The handful of NCCL entry points used, with the types of nccl.h (ncclResult_t and ncclDataType_t are ints; a
// communicator is an opaque pointer; the unique id is 128 bytes passed by value).
struct NcclId { char internal[128]; };
typedef int (*GetUniqueIdFn)(NcclId*);
typedef int (*CommInitRankFn)(void**, int, NcclId, int);
typedef int (*CommDestroyFn)(void*);
typedef int (*AllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*SendFn)(const void*, size_t, int, int, void*, cudaStream_t);
typedef int (*RecvFn)(void*, size_t, int, int, void*, cudaStream_t);
typedef int (*GroupFn)(void);
typedef const char* (*ErrStrFn)(int);
constexpr int NCCL_FLOAT32 = 7, NCCL_FLOAT64 = 8, NCCL_SUM = 0;

struct NcclApi {
    void* handle = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    AllGatherFn all_gather = nullptr;
    AllReduceFn all_reduce = nullptr;
    SendFn send = nullptr;
    RecvFn recv = nullptr;
    GroupFn group_start = nullptr, group_end = nullptr;
    ErrStrFn error_string = nullptr;
};

NcclApi g_nccl;

int load_nccl() {
    if (g_nccl.handle) return TE_OK;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        te::set_error(std::string("cannot load libnccl.so.2: ") + dlerror());
        return TE_ERR_CUDA;
    }
    NcclApi a;
    a.get_unique_id = reinterpret_cast<GetUniqueIdFn>(dlsym(h, "ncclGetUniqueId"));
    a.comm_init_rank = reinterpret_cast<CommInitRankFn>(dlsym(h, "ncclCommInitRank"));
    a.comm_destroy = reinterpret_cast<CommDestroyFn>(dlsym(h, "ncclCommDestroy"));
    a.all_gather = reinterpret_cast<AllGatherFn>(dlsym(h, "ncclAllGather"));
    a.all_reduce = reinterpret_cast<AllReduceFn>(dlsym(h, "ncclAllReduce"));
    a.send = reinterpret_cast<SendFn>(dlsym(h, "ncclSend"));
    a.recv = reinterpret_cast<RecvFn>(dlsym(h, "ncclRecv"));
    a.group_start = reinterpret_cast<GroupFn>(dlsym(h, "ncclGroupStart"));
    a.group_end = reinterpret_cast<GroupFn>(dlsym(h, "ncclGroupEnd"));
    a.error_string = reinterpret_cast<ErrStrFn>(dlsym(h, "ncclGetErrorString"));
    if (!a.get_unique_id || !a.comm_init_rank || !a.comm_destroy || !a.all_gather || !a.all_reduce || !a.send || !a.recv || !a.group_start ||
        !a.group_end || !a.error_string) {
        te::set_error("libnccl.so.2 lacks an entry point this driver needs");
        return TE_ERR_CUDA;
    }
    a.handle = h;
    g_nccl = a;
    return TE_OK;
}

int nccl_fail(int r, const char* what) {
    te::set_error(std::string(what) + ": " + (g_nccl.error_string ? g_nccl.error_string(r) : "NCCL error"));
    return TE_ERR_CUDA;
}

int bad(const char* msg) {
    te::set_error(msg);
    return TE_ERR_BAD_ARGUMENT;
}

// staging [rank][M][n_rank] (rank r's piece starts at M * first_col(r)) -> out [M][N] row-major.  16-byte accesses when
// every block width, the row pitch and both bases allow it.  HBM-bound: 4 B read + 4 B written per element.
struct RetileParams {
    const float* staging;
    float* out;
    long long M, N, ldo;
    long long block;      // columns per rank (the last rank may own fewer)
};

template <int VEC>
__global__ void __launch_bounds__(256) retile_columns_kernel(const RetileParams p) {
    te::griddep_wait();
    const long long per_row = p.N / VEC;
    const long long total = p.M * per_row;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long row = i / per_row, col = (i - row * per_row) * VEC;
        const long long c0 = (col / p.block) * p.block;
        const long long width = (c0 + p.block <= p.N) ? p.block : p.N - c0;
        const float* src = p.staging + p.M * c0 + row * width + (col - c0);
        float* dst = p.out + row * p.ldo + col;
        if (VEC == 4) *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
        else *dst = *src;
    }
}

}  // namespace

// x *= s, and *rows = r: every rank weights its gradient by the number of rows it averaged over ...
__global__ void __launch_bounds__(256) scale_set_rows_kernel(float* x, long long n, float s, double* rows, double r) {
    te::griddep_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] *= s;
    if (blockIdx.x == 0 && threadIdx.x == 0) *rows = r;
}
// ... and after the sums over the ranks, x /= total rows.
__global__ void __launch_bounds__(256) divide_by_rows_kernel(float* x, long long n, const double* rows) {
    te::griddep_wait();
    const float inv = (float)(1.0 / *rows);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] *= inv;
}

struct te_b200_comm {
    te_b200_ctx* ctx = nullptr;
    void* nccl = nullptr;
    int world = 1, rank = 0;
    // host-sharded entry point: grow-only device buffers (A replicated, this rank's B and C blocks)
    float* dev_a = nullptr;
    float* dev_b = nullptr;
    float* dev_c = nullptr;
    size_t dev_a_bytes = 0, dev_b_bytes = 0, dev_c_bytes = 0;
    double* dev_rows = nullptr;         // row count of the data-parallel gradient average (one double)
    cudaStream_t stream = nullptr;
};

static int check_comm(const te_b200_comm* c) {
    if (!c || !c->ctx) return bad("communicator is NULL");
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != c->ctx->device) return bad("the communicator's device is not the current device");
    return TE_OK;
}

extern "C" {

int te_b200_comm_unique_id(void* out_id) {
    if (!out_id) return bad("out_id is NULL");
    if (int rc = load_nccl()) return rc;
    NcclId id;
    int r = g_nccl.get_unique_id(&id);
    if (r) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(out_id, &id, sizeof id);
    return TE_OK;
}

int te_b200_comm_init(te_b200_ctx* ctx, const void* id, int world, int rank, te_b200_comm** out) {
    if (!ctx || !id || !out || world < 1 || rank < 0 || rank >= world) return bad("comm_init: bad argument");
    *out = nullptr;
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != ctx->device) return bad("comm_init: the context's device is not the current device");
    if (int rc = load_nccl()) return rc;
    te_b200_comm* c = new te_b200_comm();
    c->ctx = ctx; c->world = world; c->rank = rank;
    NcclId nid;
    memcpy(&nid, id, sizeof nid);
    int r = g_nccl.comm_init_rank(&c->nccl, world, nid, rank);
    if (r) { delete c; return nccl_fail(r, "ncclCommInitRank"); }
    cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { g_nccl.comm_destroy(c->nccl); delete c; return te::cuda_fail(e, "cudaStreamCreateWithFlags"); }
    *out = c;
    return TE_OK;
}

int te_b200_comm_destroy(te_b200_comm* c) {
    if (!c) return TE_OK;
    if (c->stream) { cudaStreamSynchronize(c->stream); cudaStreamDestroy(c->stream); }
    if (c->dev_a) cudaFree(c->dev_a);
    if (c->dev_b) cudaFree(c->dev_b);
    if (c->dev_c) cudaFree(c->dev_c);
    if (c->dev_rows) cudaFree(c->dev_rows);
    if (c->nccl) g_nccl.comm_destroy(c->nccl);
    delete c;
    return TE_OK;
}

int te_b200_comm_rank(const te_b200_comm* c, int* world, int* rank) {
    if (!c) return bad("communicator is NULL");
    if (world) *world = c->world;
    if (rank) *rank = c->rank;
    return TE_OK;
}

// Exchanges pieces of unequal size: rank r contributes `counts[r]` floats, stored at recv + offsets[r] on every rank.
static int all_gather_v(te_b200_comm* c, const float* send, float* recv, const std::vector<int64_t>& counts,
                        const std::vector<int64_t>& offsets, cudaStream_t st) {
    bool equal = true;
    for (int r = 1; r < c->world; ++r) equal = equal && counts[r] == counts[0] && offsets[r] == r * counts[0];
    int rr;
    if (equal) {
        if (counts[0] == 0) return TE_OK;
        if ((rr = g_nccl.all_gather(send, recv, (size_t)counts[0], NCCL_FLOAT32, c->nccl, st))) return nccl_fail(rr, "ncclAllGather");
        return TE_OK;
    }
    if ((rr = g_nccl.group_start())) return nccl_fail(rr, "ncclGroupStart");
    for (int peer = 0; peer < c->world; ++peer) {
        if (counts[c->rank] > 0 && (rr = g_nccl.send(send, (size_t)counts[c->rank], NCCL_FLOAT32, peer, c->nccl, st))) return nccl_fail(rr, "ncclSend");
        if (counts[peer] > 0 && (rr = g_nccl.recv(recv + offsets[peer], (size_t)counts[peer], NCCL_FLOAT32, peer, c->nccl, st))) return nccl_fail(rr, "ncclRecv");
    }
    if ((rr = g_nccl.group_end())) return nccl_fail(rr, "ncclGroupEnd");
    return TE_OK;
}

int te_b200_all_gather_columns(te_b200_comm* c, const float* c_local, int64_t M, int64_t N, int64_t align, float* staging,
                               float* c_full, int64_t ld_full, te_stream_t stream) {
    if (int rc = check_comm(c)) return rc;
    if (M < 0 || N < 0 || align < 1 || ld_full < N) return bad("all_gather_columns: bad extents");
    if (M == 0 || N == 0) return TE_OK;
    if (!staging || !c_full) return bad("all_gather_columns: NULL pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    std::vector<int64_t> counts(c->world), offsets(c->world);
    int64_t block = 0;
    for (int r = 0; r < c->world; ++r) {
        int64_t b = 0, n = 0;
        te_b200_shard_range(N, c->world, r, align, &b, &n);
        counts[r] = M * n;
        offsets[r] = M * b;
        if (r == 0) block = n;
    }
    if (block == 0) return bad("all_gather_columns: rank 0 owns no columns");
    if (!c_local && counts[c->rank] > 0) return bad("all_gather_columns: NULL pointer");     // a rank that owns nothing may pass NULL
    if (int rc = all_gather_v(c, c_local, staging, counts, offsets, st)) return rc;
    RetileParams p;
    p.staging = staging; p.out = c_full; p.M = M; p.N = N; p.ldo = ld_full; p.block = block;
    const bool vec = (block & 3) == 0 && (N & 3) == 0 && (ld_full & 3) == 0 && (reinterpret_cast<uintptr_t>(staging) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(c_full) & 15) == 0;
    const long long total = M * (vec ? N / 4 : N);
    long long blocks = (total + 255) / 256;
    if (blocks > (long long)c->ctx->sm_count * 16) blocks = (long long)c->ctx->sm_count * 16;
    cudaError_t e = vec ? te::launch_pdl(retile_columns_kernel<4>, dim3((unsigned)blocks), dim3(256), 0, st, p)
                        : te::launch_pdl(retile_columns_kernel<1>, dim3((unsigned)blocks), dim3(256), 0, st, p);
    if (e != cudaSuccess) return te::cuda_fail(e, "retile_columns_kernel launch");
    c->ctx->launches += 1;
    return TE_OK;
}

int te_b200_all_gather_rows(te_b200_comm* c, float* full, int64_t rows, int64_t cols, int64_t align, te_stream_t stream) {
    if (int rc = check_comm(c)) return rc;
    if (rows < 0 || cols < 0 || align < 1) return bad("all_gather_rows: bad extents");
    if (rows == 0 || cols == 0) return TE_OK;
    if (!full) return bad("all_gather_rows: NULL pointer");
    std::vector<int64_t> counts(c->world), offsets(c->world);
    for (int r = 0; r < c->world; ++r) {
        int64_t b = 0, n = 0;
        te_b200_shard_range(rows, c->world, r, align, &b, &n);
        counts[r] = n * cols;
        offsets[r] = b * cols;
    }
    // in place: this rank's rows already sit at their position inside `full`
    return all_gather_v(c, full + offsets[c->rank], full, counts, offsets, static_cast<cudaStream_t>(stream));
}

int te_b200_all_reduce_batch_mean(te_b200_comm* c, float* grads, int64_t n, int64_t local_rows, te_stream_t stream) {
    if (int rc = check_comm(c)) return rc;
    if (n < 0 || local_rows < 0) return bad("all_reduce_batch_mean: negative count");
    if (n == 0) return TE_OK;
    if (!grads) return bad("all_reduce_batch_mean: NULL pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!c->dev_rows) {
        cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->dev_rows), 2 * sizeof(double));
        if (e != cudaSuccess) return te::cuda_fail(e, "cudaMalloc(row count)");
    }
    long long blocks = (n + 255) / 256;
    if (blocks > (long long)c->ctx->sm_count * 16) blocks = (long long)c->ctx->sm_count * 16;
    cudaError_t e = te::launch_pdl(scale_set_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, st, grads, (long long)n, (float)local_rows,
                                   c->dev_rows, (double)local_rows);
    if (e != cudaSuccess) return te::cuda_fail(e, "scale_set_rows_kernel launch");
    int rr;
    if (c->world > 1) {
        if ((rr = g_nccl.all_reduce(grads, grads, (size_t)n, NCCL_FLOAT32, NCCL_SUM, c->nccl, st))) return nccl_fail(rr, "ncclAllReduce");
        if ((rr = g_nccl.all_reduce(c->dev_rows, c->dev_rows, 1, NCCL_FLOAT64, NCCL_SUM, c->nccl, st))) return nccl_fail(rr, "ncclAllReduce");
    }
    e = te::launch_pdl(divide_by_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, st, grads, (long long)n, (const double*)c->dev_rows);
    if (e != cudaSuccess) return te::cuda_fail(e, "divide_by_rows_kernel launch");
    c->ctx->launches += 2;
    return TE_OK;
}

static int grow(float** buf, size_t* have, size_t need) {
    if (need <= *have) return TE_OK;
    if (*buf) cudaFree(*buf);
    *buf = nullptr; *have = 0;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(buf), need);
    if (e != cudaSuccess) return te::cuda_fail(e, "cudaMalloc(sharded host staging)");
    *have = need;
    return TE_OK;
}

int te_b200_gemm_f32_host_sharded(te_b200_comm* c, const te_gemm_desc* h, int64_t column_align) {
    if (int rc = check_comm(c)) return rc;
    if (!h) return bad("gemm descriptor is NULL");
    if (h->batch_outer != 1 || h->batch_inner != 1 || h->a_major != TE_ROW_MAJOR || h->b_major != TE_ROW_MAJOR)
        return bad("the sharded host entry takes one row-major A . row-major B product");
    if (h->residual || h->preact_out) return bad("the sharded host entry takes no residual or pre-activation output");
    if (h->M <= 0 || h->N <= 0 || h->K <= 0 || !h->a || !h->b || !h->c) return bad("the sharded host entry needs a non-empty problem");
    if (h->lda < h->K || h->ldb < h->N || h->ldc < h->N || column_align < 1) return bad("leading dimension smaller than the row");
    const int64_t M = h->M, N = h->N, K = h->K;
    int64_t n0 = 0, nc = 0, r0 = 0, rc_rows = 0;
    te_b200_shard_range(N, c->world, c->rank, column_align, &n0, &nc);
    te_b200_shard_range(M, c->world, c->rank, 1, &r0, &rc_rows);
    int rc;
    if ((rc = grow(&c->dev_a, &c->dev_a_bytes, (size_t)M * K * 4))) return rc;
    // B block, followed by this rank's slice of the bias
    if ((rc = grow(&c->dev_b, &c->dev_b_bytes, ((size_t)K + 1) * (nc ? nc : 1) * 4))) return rc;
    if ((rc = grow(&c->dev_c, &c->dev_c_bytes, (size_t)M * (nc ? nc : 1) * 4))) return rc;
    cudaStream_t st = c->stream;
    cudaError_t e;
    // this rank's rows of A (a contiguous range of a dense A goes as one copy) and its columns of B, over PCIe
    if (rc_rows > 0) {
        e = cudaMemcpy2DAsync(c->dev_a + r0 * K, (size_t)K * 4, h->a + r0 * h->lda, (size_t)h->lda * 4, (size_t)K * 4, (size_t)rc_rows,
                              cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return te::cuda_fail(e, "H2D rows of A");
    }
    if (nc > 0) {
        e = cudaMemcpy2DAsync(c->dev_b, (size_t)nc * 4, h->b + n0, (size_t)h->ldb * 4, (size_t)nc * 4, (size_t)K, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return te::cuda_fail(e, "H2D columns of B");
    }
    // replicate A over NVLink
    if (c->world > 1 && (rc = te_b200_all_gather_rows(c, c->dev_a, M, K, 1, st))) { cudaStreamSynchronize(st); return rc; }
    if (nc > 0) {
        te_gemm_desc d = *h;
        d.N = nc;
        d.a = c->dev_a; d.lda = K;
        d.b = c->dev_b; d.ldb = nc;
        d.c = c->dev_c; d.ldc = nc;
        if (h->bias) {
            float* dev_bias = c->dev_b + K * nc;
            e = cudaMemcpyAsync(dev_bias, h->bias + n0, (size_t)nc * 4, cudaMemcpyHostToDevice, st);
            if (e != cudaSuccess) { cudaStreamSynchronize(st); return te::cuda_fail(e, "H2D bias"); }
            d.bias = dev_bias;
        }
        if ((rc = te_b200_gemm_f32(c->ctx, &d, st))) { cudaStreamSynchronize(st); return rc; }
        e = cudaMemcpy2DAsync(h->c + n0, (size_t)h->ldc * 4, c->dev_c, (size_t)nc * 4, (size_t)nc * 4, (size_t)M, cudaMemcpyDeviceToHost, st);
        if (e != cudaSuccess) { cudaStreamSynchronize(st); return te::cuda_fail(e, "D2H columns of C"); }
    }
    if ((e = cudaStreamSynchronize(st)) != cudaSuccess) return te::cuda_fail(e, "cudaStreamSynchronize");
    return te_b200_check_device_status(c->ctx);
}

}  // extern "C"
