// Programmatic dependent launch, used by every kernel of the library.
//
// A kernel launched with the programmatic-stream-serialization attribute (launch_pdl below) may be scheduled before the
// kernel ahead of it in the stream has finished: its CTAs take over SMs as those of the earlier kernel exit, and the
// launch latency and any prologue are hidden behind the earlier kernel's tail.  griddep_wait() blocks until that
// earlier kernel has completed and its memory is visible; every kernel executes it before its first access to global
// memory.  griddep_launch_dependents() lets the kernel BEHIND this one be scheduled as soon as every CTA of this grid
// has issued it or exited; only the persistent kernels (all CTAs resident at once) issue it early, the others leave it
// to their exit.  Building with -DTE_NO_PDL turns both into no-ops and the launches into ordinary ones.
#pragma once
#include <cuda_runtime.h>

namespace te {

#ifndef TE_NO_PDL
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
constexpr int TE_PDL_ALLOWED = 1;
#else
__device__ __forceinline__ void griddep_wait() {}
__device__ __forceinline__ void griddep_launch_dependents() {}
constexpr int TE_PDL_ALLOWED = 0;
#endif

template <typename Kernel, typename... Args>
inline cudaError_t launch_pdl(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = TE_PDL_ALLOWED;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace te
