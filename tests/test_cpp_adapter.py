"""The header-only C++ host adapter (include/te_b200.hpp): it must compile against the C ABI everywhere, and on
a GPU its test program -- the counterpart of the reference's plain-main CUDA matmul check -- must pass."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "matmul_tensor_test.cpp")
LIBDIR = os.path.join(ROOT, "torch-engine_b200")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build(out):
    cmd = ["g++", "-std=c++17", "-O1", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(CUDA, "include"), SRC,
           "-o", out, "-L" + LIBDIR, "-lte_b200", "-L" + os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + LIBDIR, "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    subprocess.run(cmd, check=True, capture_output=True, text=True)


def test_adapter_compiles_and_links(tmp_path):
    from torch_engine_b200 import lib
    lib.load()                      # the shared library must exist
    _build(str(tmp_path / "matmul_tensor_test"))


@pytest.mark.gpu
def test_adapter_program_passes_on_gpu(tmp_path):
    exe = str(tmp_path / "matmul_tensor_test")
    _build(exe)
    for prec in ("tf32", "3xtf32"):
        r = subprocess.run([exe], capture_output=True, text=True, timeout=120,
                           env=dict(os.environ, TENSOR_GEMM_PRECISION=prec))
        assert r.returncode == 0, r.stdout + r.stderr
        assert "All C++ adapter checks passed." in r.stdout


def _load_build():
    import importlib.util
    spec = importlib.util.spec_from_file_location("te_build", os.path.join(LIBDIR, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_adapter_benchmark_compiles(tmp_path):
    from torch_engine_b200 import lib
    lib.load()
    exe = _load_build().build_adapter_benchmark(str(tmp_path / "adapter_step_benchmark"))
    assert os.path.exists(exe)


@pytest.mark.gpu
def test_adapter_benchmark_runs_both_allocator_modes(tmp_path):
    """The transformer-block step of the C++ adapter gives the same result with the caching allocator and with a
    cudaMalloc per tensor, and the caching mode calls cudaMalloc for no tensor once it is warm."""
    import json
    exe = _load_build().build_adapter_benchmark(str(tmp_path / "adapter_step_benchmark"))
    r = subprocess.run([exe, "3", "2", "2", "128", "128", "4"], capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, LD_LIBRARY_PATH=LIBDIR + ":" + os.environ.get("LD_LIBRARY_PATH", "")))
    assert r.returncode == 0, r.stdout + r.stderr
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [l["allocator"] for l in lines] == ["caching", "cudaMalloc_per_tensor"]
    assert lines[0]["cuda_mallocs_per_step"] == 0 and lines[0]["cache_hits_per_step"] > 50
    assert lines[1]["cuda_mallocs_per_step"] > 50 and lines[1]["cache_hits_per_step"] == 0
    assert lines[0]["checksum"] == lines[1]["checksum"]
