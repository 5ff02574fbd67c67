"""Builds libte_b200.so (the C-ABI shared library) in-tree with nvcc for sm_100a.

The arch is passed as `-gencode arch=compute_100a,code=sm_100a`: the tcgen05 / TMA PTX the
kernels use only assembles for the architecture-specific target.  No torch headers are involved;
the library links the CUDA runtime statically and resolves the one driver symbol it needs
(cuTensorMapEncodeTiled) at run time.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libte_b200.so")
SOURCES = ["gemm_sm100.cu", "gemm_sm100_2cta.cu", "attention_sm100.cu", "attention_bwd_sm100.cu", "pack.cu", "rowops.cu", "norm_embed_loss.cu", "api.cu", "static_scratch.cu", "dist.cu", "thin_fp32.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compiles every .cu under csrc/ and links libte_b200.so.  Returns the library path."""
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(ROOT, "include", "te_b200.h"))
    objs = []
    procs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(CSRC, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed on " + src)
    if force or procs or _stale(LIB, objs):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
        subprocess.run(cmd, check=True)
    return LIB


ADAPTER_BENCH_SRC = os.path.join(HERE, "benchmarks", "adapter_step_benchmark.cpp")
ADAPTER_BENCH = os.path.join(HERE, "benchmarks", "adapter_step_benchmark")


def build_adapter_benchmark(out=ADAPTER_BENCH):
    """Compiles benchmarks/adapter_step_benchmark.cpp (the C++ adapter's transformer-block step, caching allocator
    against cudaMalloc per tensor) against libte_b200.so.  Returns the program's path."""
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    deps = [ADAPTER_BENCH_SRC, os.path.join(ROOT, "include", "te_b200.hpp"), os.path.join(ROOT, "include", "te_b200.h")]
    if _stale(out, deps):
        cmd = ["g++", "-std=c++17", "-O2", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(cuda, "include"),
               ADAPTER_BENCH_SRC, "-o", out, "-L" + HERE, "-lte_b200", "-L" + os.path.join(cuda, "lib64"), "-lcudart",
               "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath," + os.path.join(cuda, "lib64")]
        subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_adapter_benchmark())
