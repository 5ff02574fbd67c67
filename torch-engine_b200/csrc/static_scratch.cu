// te_b200_gemm_3xtf32_static: the 3xTF32 GEMM for callers that must not allocate device memory.
//
// Who needs it: a host that runs inside someone else's memory plan -- a plugin called from a framework whose
// allocator owns the whole device, a real-time loop, code between cudaStreamBeginCapture/EndCapture set-up
// phases, or a process whose memory budget was fixed at start-up.  Such callers cannot create the usual
// context (te_b200_init calls cudaMalloc for the workspace and the status word) and cannot let a library
// call cudaMalloc or cudaFree behind their back, because that either fails, or synchronises the device, or
// breaks their accounting.
//
// What it does instead: the tf32 hi/lo planes that the 3xTF32 kernel reads are written into ONE fixed
// array in device global memory that is part of this library's image.  Nothing here calls cudaMalloc,
// cudaFree, or any routine that allocates (no torch, no cuBLAS).  The array is not free, though: the CUDA
// runtime loads a library's device code lazily, and loading the part that holds the array is what reserves
// its TE_B200_STATIC_SCRATCH_BYTES (plus the code of the kernels) on that GPU, until the process exits.
// That load happens inside the FIRST call on each device (or earlier, if the process runs with
// CUDA_MODULE_LOADING=EAGER); it is the one moment at which this entry point needs free device memory,
// and on a device that has none left it fails with TE_ERR_CUDA -- the next call tries again.
//
// Rules for the caller:
//   * The first successful call on each device does all one-time work: it resolves the array's device
//     address (cudaGetSymbolAddress with that device current), the driver's tensor-map encoder, and loads
//     and configures every kernel any later problem shape can reach (both single-CTA tile widths, the
//     CTA-pair form, the split-K reduction, the packing kernels).  Make that first call outside any
//     stream capture; later calls, whatever their shape, do no first-use work.
//   * All calls on one device share the array; it keeps whatever the previous call left.  Everything a call
//     reads from it is rewritten by that call first (the planes by the packing pass, the status word by a
//     memset on the stream), but two calls that overlap on the GPU (different streams) race on it.
//   * Problems whose planes do not fit are refused with TE_ERR_WORKSPACE before anything is launched.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "te_internal.h"

// 256 bytes of status area followed by the plane storage.
static __device__ __align__(256) unsigned char g_static_scratch[256 + TE_B200_STATIC_SCRATCH_BYTES];

namespace {

constexpr int MAX_DEVICES = 16;

struct DeviceSlot {
    std::mutex lock;
    bool ready = false;            // set once the set-up has succeeded; a failed set-up is retried by the next call
    unsigned char* base = nullptr; // DEVICE address of g_static_scratch on this device
    te_b200_ctx ctx;               // host-side bookkeeping only; nothing in it is allocated on the device
};
DeviceSlot g_slots[MAX_DEVICES];

inline int64_t round_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

int setup_device(int dev, DeviceSlot* slot) {
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return te::cuda_fail(e, "cudaGetDeviceProperties");
    if (prop.major != 10) {
        te::set_error("this backend is built for sm_100a only");
        return TE_ERR_NO_DEVICE;
    }
    // In host code `g_static_scratch` names a host-side shadow, not device memory: ask the runtime for the
    // address the array has on the device that is current right now.
    void* dptr = nullptr;
    e = cudaGetSymbolAddress(&dptr, g_static_scratch);
    if (e != cudaSuccess || !dptr) {
        cudaGetLastError();
        return te::cuda_fail(e, "cudaGetSymbolAddress(static scratch; loading it reserves the array on this device)");
    }
    slot->base = static_cast<unsigned char*>(dptr);
    cudaDriverEntryPointQueryResult q;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &slot->ctx.encode_tiled, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !slot->ctx.encode_tiled) {
        te::set_error("cuTensorMapEncodeTiled is not available from this driver");
        return TE_ERR_CUDA;
    }
    slot->ctx.device = dev;
    slot->ctx.sm_count = prop.multiProcessorCount;
    slot->ctx.d_status = reinterpret_cast<int*>(slot->base);
    slot->ctx.workspace = slot->base + 256;
    slot->ctx.workspace_bytes = TE_B200_STATIC_SCRATCH_BYTES;
    // Load and configure every kernel a later call may launch, so that none of them does first-use work.
    return te::prepare_3xtf32_kernels(&slot->ctx);
}

}  // namespace

extern "C" int te_b200_gemm_3xtf32_static(const te_gemm_desc* d, te_stream_t stream, int* host_status) {
    using namespace te;
    size_t need = 0;
    int rc = te_b200_gemm_workspace_size(d, &need);   // validates the descriptor as te_b200_gemm_f32 does
    if (rc) return rc;
    if (d->precision != TE_PREC_3XTF32) {
        set_error("te_b200_gemm_3xtf32_static runs the 3xTF32 mode only; set precision = TE_PREC_3XTF32");
        return TE_ERR_BAD_ARGUMENT;
    }
    // This entry always reads hi / lo planes out of the scratch array (the context path splits thin and small problems
    // inside the kernel and reports no scratch for them): what has to fit is counted here, plane by plane, exactly as
    // the packing loop below lays the planes out.
    need = 0;
    if (d->K > 0 && d->M > 0 && d->N > 0) {
        const int64_t kp = round_up(d->K, 4);
        const int64_t rows[2] = {d->M, d->N};
        const int64_t si[2] = {d->a_stride_inner, d->b_stride_inner}, so[2] = {d->a_stride_outer, d->b_stride_outer};
        for (int i = 0; i < 2; ++i) {
            const int64_t bi = (d->batch_inner > 1 && si[i] != 0) ? d->batch_inner : 1;
            const int64_t bo = (d->batch_outer > 1 && so[i] != 0) ? d->batch_outer : 1;
            const double planes = 2.0 * (double)bi * (double)bo * (double)rows[i] * (double)kp * 4.0;
            if (planes > 4.0 * (double)TE_B200_STATIC_SCRATCH_BYTES) { need = SIZE_MAX; break; }
            need += 2 * (size_t)round_up(bi * bo * rows[i] * kp * 4, 256);
        }
    }
    if (need > (size_t)TE_B200_STATIC_SCRATCH_BYTES) {
        char msg[200];
        snprintf(msg, sizeof msg, "problem needs %zu bytes of plane storage; the static scratch array holds %lld",
                 need, (long long)TE_B200_STATIC_SCRATCH_BYTES);
        set_error(msg);
        return TE_ERR_WORKSPACE;
    }
    if (d->M == 0 || d->N == 0) {
        if (host_status) *host_status = 0;    // nothing was launched, so nothing can have timed out
        return TE_OK;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_error("no CUDA device is current; this backend has no CPU path");
        return TE_ERR_NO_DEVICE;
    }
    if (dev < 0 || dev >= MAX_DEVICES) {
        set_error("device ordinal beyond the static slot table");
        return TE_ERR_BAD_ARGUMENT;
    }
    DeviceSlot* slot = &g_slots[dev];
    {
        std::lock_guard<std::mutex> guard(slot->lock);
        if (!slot->ready) {
            if ((rc = setup_device(dev, slot))) return rc;     // not latched: the next call tries again
            slot->ready = true;
        }
    }
    te_b200_ctx* ctx = &slot->ctx;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // The status word must start at zero; the array keeps the previous call's contents.
    if ((e = cudaMemsetAsync(ctx->d_status, 0, sizeof(int), st)) != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(status)");

    GemmProblem g;
    g.M = d->M; g.N = d->N; g.K = d->K;
    g.batch_inner = d->batch_inner; g.batch_outer = d->batch_outer;
    g.a.ptr = d->a; g.a.mn_major = (d->a_major == TE_COL_MAJOR); g.a.rows = d->M; g.a.ld = d->lda;
    g.a.stride_inner = d->a_stride_inner; g.a.stride_outer = d->a_stride_outer;
    g.b.ptr = d->b; g.b.mn_major = (d->b_major == TE_ROW_MAJOR); g.b.rows = d->N; g.b.ld = d->ldb;
    g.b.stride_inner = d->b_stride_inner; g.b.stride_outer = d->b_stride_outer;
    g.c = d->c; g.ldc = d->ldc; g.c_stride_inner = d->c_stride_inner; g.c_stride_outer = d->c_stride_outer;
    g.preact = d->preact_out; g.bias = d->bias; g.residual = d->residual; g.alpha = d->alpha; g.scale_mode = d->scale_mode;
    g.epilogue = d->epilogue;

    unsigned char* cursor = static_cast<unsigned char*>(ctx->workspace);
    if (d->K > 0) {
        const int64_t kp = round_up(d->K, 4);
        Operand* ops[2] = {&g.a, &g.b};
        const float** los[2] = {&g.a_lo, &g.b_lo};
        for (int i = 0; i < 2; ++i) {
            Operand& op = *ops[i];
            const int64_t bi = (d->batch_inner > 1 && op.stride_inner != 0) ? d->batch_inner : 1;
            const int64_t bo = (d->batch_outer > 1 && op.stride_outer != 0) ? d->batch_outer : 1;
            const int64_t bytes = round_up(bi * bo * op.rows * kp * 4, 256);
            float* hi = reinterpret_cast<float*>(cursor);
            float* lo = reinterpret_cast<float*>(cursor + bytes);
            cursor += 2 * bytes;
            if ((rc = launch_pack(ctx, op, d->K, d->batch_inner, d->batch_outer, hi, lo, true, st))) return rc;
            Operand packed;
            packed.ptr = hi; packed.mn_major = false; packed.rows = op.rows; packed.ld = kp;
            packed.stride_inner = (d->batch_inner > 1 && op.stride_inner != 0) ? op.rows * kp : 0;
            packed.stride_outer = (d->batch_outer > 1 && op.stride_outer != 0) ? bi * op.rows * kp : 0;
            op = packed;
            *los[i] = lo;
        }
    } else {
        g.a.ptr = g.b.ptr = reinterpret_cast<const float*>(cursor);   // never read: K == 0 issues no loads
        g.a.mn_major = g.b.mn_major = false;
        g.a.ld = g.b.ld = 4;
        g.a.stride_inner = g.a.stride_outer = g.b.stride_inner = g.b.stride_outer = 0;
        g.a_lo = g.a.ptr; g.b_lo = g.b.ptr;
    }
    if ((rc = launch_gemm(ctx, g, st))) return rc;
    if (host_status) {
        if ((e = cudaMemcpyAsync(host_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, st)) != cudaSuccess)
            return cuda_fail(e, "cudaMemcpyAsync(status)");
    }
    return TE_OK;
}
