"""te_b200_gemm_3xtf32_static: the 3xTF32 GEMM whose scratch is a fixed device array inside the library, for
callers that may not allocate device memory.  Called through the C ABI, twice in a row (the array keeps the
first call's contents, the second call must not be disturbed by them), and compared with the ordinary
context-based entry point.  This file sorts last so that a run stopping at the first failure has already run
everything else; it also passes on its own in a fresh process."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.gpu_util import TOL_REL, rel_err
from torch_engine_b200 import lib as L

pytestmark = pytest.mark.gpu


def _desc(a, b, c):
    M, K = a.shape
    N = b.shape[1]
    d = L.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.a, d.b, d.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    d.lda, d.ldb, d.ldc = K, N, N
    d.batch_outer = d.batch_inner = 1
    d.alpha = 1.0
    d.precision = L.TE_PREC_3XTF32
    return d


def test_static_scratch_entry_matches_context_entry(backend):
    lib = L.load()
    g = torch.Generator(device="cuda").manual_seed(123)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two different problems back to back: the second reuses the array the first one filled
    for (M, K, N) in [(300, 200, 260), (129, 515, 77)]:
        a = torch.rand(M, K, device="cuda", generator=g) * 2 - 1
        b = torch.rand(K, N, device="cuda", generator=g) * 2 - 1
        want = torch.empty(M, N, device="cuda")
        backend.gemm(_desc(a, b, want))
        got = torch.full((M, N), float("nan"), device="cuda")
        status = C.c_int(-1)
        L.check(lib.te_b200_gemm_3xtf32_static(C.byref(_desc(a, b, got)), stream, C.byref(status)))
        torch.cuda.synchronize()
        assert status.value == 0
        assert rel_err(got.cpu().numpy(), want.cpu().numpy()) <= TOL_REL["3xtf32"]
        ref = (a.double() @ b.double()).cpu().numpy()          # float64 arbiter
        assert rel_err(got.cpu().numpy(), ref) <= TOL_REL["3xtf32"]
    backend.check_device_status()


def test_static_scratch_entry_allocates_nothing_after_its_first_call():
    """The first call on a device loads the library's device code (which reserves the scratch array) and configures
    every kernel variant; from the second call on, the free device memory must not move, whatever the shape: a thin
    product (split K), a 64-wide tile, a 128-wide tile, and a long-K product that takes the CTA-pair form."""
    lib = L.load()
    g = torch.Generator(device="cuda").manual_seed(5)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    shapes = [(64, 64, 64), (16, 4096, 256), (200, 300, 100), (512, 512, 512), (512, 5120, 512)]
    ops = []
    for (M, K, N) in shapes:
        a = torch.rand(M, K, device="cuda", generator=g) * 2 - 1
        b = torch.rand(K, N, device="cuda", generator=g) * 2 - 1
        ops.append((a, b, torch.empty(M, N, device="cuda")))
    status = torch.zeros(1, dtype=torch.int32).pin_memory()
    sp = C.cast(status.data_ptr(), C.POINTER(C.c_int))
    a, b, c = ops[0]
    L.check(lib.te_b200_gemm_3xtf32_static(C.byref(_desc(a, b, c)), stream, sp))   # first call: one-time work
    torch.cuda.synchronize()
    for a, b, c in ops[1:]:
        free_before = torch.cuda.mem_get_info()[0]     # taken per call: torch's own allocator may grow in between
        L.check(lib.te_b200_gemm_3xtf32_static(C.byref(_desc(a, b, c)), stream, sp))
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        assert torch.cuda.mem_get_info()[0] == free_before
        ref = (a.double() @ b.double()).cpu().numpy()
        assert rel_err(c.cpu().numpy(), ref) <= TOL_REL["3xtf32"]
    # an empty problem launches nothing and reports 0 at once
    flag = C.c_int(-1)
    d = _desc(ops[0][0], ops[0][1], ops[0][2])
    d.M = 0
    L.check(lib.te_b200_gemm_3xtf32_static(C.byref(d), stream, C.byref(flag)))
    assert flag.value == 0


def test_static_scratch_entry_refuses_what_does_not_fit():
    lib = L.load()
    a = torch.zeros(16, 16, device="cuda")
    d = _desc(a, a, a)
    d.M = d.N = d.K = 8192             # planes would need 1 GiB
    d.lda = d.ldb = d.ldc = 8192
    rc = lib.te_b200_gemm_3xtf32_static(C.byref(d), None, None)
    assert rc == L.TE_ERR_WORKSPACE
    assert b"static scratch array holds" in lib.te_b200_last_error()
    # a thin product too: the context path needs no plane storage for it (it splits inside the kernel), this entry
    # always packs planes, so the 2 x 268 MB of B's planes are refused here
    d = _desc(a, a, a)
    d.M, d.N, d.K = 16, 8192, 8192
    d.lda = d.ldb = d.ldc = 8192
    assert lib.te_b200_gemm_3xtf32_static(C.byref(d), None, None) == L.TE_ERR_WORKSPACE
    assert b"static scratch array holds" in lib.te_b200_last_error()
    d = _desc(a, a, a)
    d.precision = L.TE_PREC_TF32
    assert lib.te_b200_gemm_3xtf32_static(C.byref(d), None, None) == L.TE_ERR_BAD_ARGUMENT
