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
