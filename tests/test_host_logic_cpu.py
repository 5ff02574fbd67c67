"""Host-side logic of the C-ABI library that needs no GPU: symbol export, shape/broadcast rules and error
texts of Tensor::matmul, descriptor validation, workspace sizing, shard ranges, and the loud failure when
no GPU is present."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from torch_engine_b200 import lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "te_b200.h")).read()
    declared = set(re.findall(r"TE_API\s+[\w\s\*]+?\b(te_b200_\w+)\s*\(", header))
    assert len(declared) >= 19
    lib = L.load()
    for name in sorted(declared):
        assert hasattr(lib, name), name
    assert declared == set(L.SIGNATURES), declared ^ set(L.SIGNATURES)


def test_struct_sizes_match_header_layout(tmp_path):
    """sizeof and the offset of the last field of every descriptor, as a C compiler lays include/te_b200.h out,
    against the ctypes mirrors in lib.py."""
    import subprocess
    src = tmp_path / "sizes.c"
    src.write_text("""
#include <stdio.h>
#include <stddef.h>
#include "te_b200.h"
int main(void) {
    printf("%zu %zu\\n", sizeof(te_gemm_desc), offsetof(te_gemm_desc, precision));
    printf("%zu %zu\\n", sizeof(te_attn_desc), offsetof(te_attn_desc, precision));
    printf("%zu %zu\\n", sizeof(te_attn_bwd_desc), offsetof(te_attn_bwd_desc, precision));
    printf("%zu %zu\\n", sizeof(te_mha_desc), offsetof(te_mha_desc, precision));
    printf("%zu %zu\\n", sizeof(te_mha_bwd_desc), offsetof(te_mha_bwd_desc, precision));
    return 0;
}
""")
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    rows = [tuple(int(v) for v in line.split()) for line in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split("\n") if line]
    mirrors = [L.GemmDesc, L.AttnDesc, L.AttnBwdDesc, L.MhaDesc, L.MhaBwdDesc]
    assert len(rows) == len(mirrors)
    for (size, off), m in zip(rows, mirrors):
        assert C.sizeof(m) == size, m.__name__
        assert getattr(m, "precision").offset == off, m.__name__


@pytest.mark.parametrize("a,b", [((2, 3), (3, 4)), ((2, 2, 3), (2, 3, 2)), ((1, 2, 3), (3, 3, 4)), ((2, 1, 4, 3), (5, 3, 6)),
                                 ((4, 6, 8), (8, 10)), ((7, 1, 2, 5, 6), (3, 1, 6, 2))])
def test_result_shape_matches_numpy_broadcasting(a, b):
    def strides(s):
        st, run = [], 1
        for d in reversed(s):
            st.append(run)
            run *= d
        return tuple(reversed(st))
    assert L.matmul_shape(a, strides(a), b, strides(b)) == np.matmul(np.zeros(a), np.zeros(b)).shape


@pytest.mark.parametrize("a,b,code,msg", [
    ((3,), (3, 2), L.TE_ERR_SHAPE_NDIM, "Matmul requires tensors with at least 2 dimensions"),
    ((2, 3), (2, 2), L.TE_ERR_SHAPE_INNER, "Inner dimensions must match for matmul"),
    ((3, 2, 3), (2, 3, 4), L.TE_ERR_SHAPE_BROADCAST, "Batch dimensions are not broadcastable"),
    ((2, 2, 3), (3, 3, 4), L.TE_ERR_SHAPE_BROADCAST, "Batch dimensions are not broadcastable"),
])
def test_shape_errors_repeat_the_reference_text(a, b, code, msg):
    with pytest.raises(L.BackendError) as e:
        L.matmul_shape(a, (1,) * len(a), b, (1,) * len(b))
    assert e.value.status == code and str(e.value) == msg
    assert L.status_string(code) == msg


def test_unsupported_layout_text():
    assert L.status_string(L.TE_ERR_UNSUPPORTED_LAYOUT) == "CUDA matmul only supports row- or column-major 2D slices"


def _desc(**kw):
    d = L.GemmDesc()
    d.M, d.N, d.K = 64, 64, 64
    d.a = d.b = d.c = 0x1000
    d.lda = d.ldb = d.ldc = 64
    d.batch_outer = d.batch_inner = 1
    d.alpha = 1.0
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def _ws(d):
    n = C.c_size_t()
    rc = L.load().te_b200_gemm_workspace_size(C.byref(d), C.byref(n))
    return rc, n.value


def test_descriptor_validation():
    assert _ws(_desc())[0] == L.TE_OK
    assert _ws(_desc(M=-1))[0] == L.TE_ERR_BAD_ARGUMENT
    assert _ws(_desc(batch_inner=0))[0] == L.TE_ERR_BAD_ARGUMENT
    assert _ws(_desc(a_major=2))[0] == L.TE_ERR_UNSUPPORTED_LAYOUT
    assert _ws(_desc(lda=8))[0] == L.TE_ERR_UNSUPPORTED_LAYOUT       # ld smaller than the row
    assert _ws(_desc(precision=7))[0] == L.TE_ERR_BAD_ARGUMENT
    assert _ws(_desc(epilogue=L.TE_EPI_BIAS))[0] == L.TE_ERR_BAD_ARGUMENT   # bias epilogue without a bias
    assert _ws(_desc(epilogue=3))[0] == L.TE_ERR_BAD_ARGUMENT
    assert _ws(_desc(c=0))[0] == L.TE_ERR_BAD_ARGUMENT
    assert _ws(_desc(a_stride_inner=-4))[0] == L.TE_ERR_BAD_ARGUMENT


def test_workspace_sizing():
    # aligned operands in TF32 mode are read in place
    assert _ws(_desc()) == (L.TE_OK, 0)
    # 3xTF32 splits hi / lo inside the kernel for thin and small products: no plane storage ...
    assert _ws(_desc(precision=L.TE_PREC_3XTF32)) == (L.TE_OK, 0)
    thin = dict(M=16, N=8192, K=8192, lda=8192, ldb=8192, ldc=8192, precision=L.TE_PREC_3XTF32)
    assert _ws(_desc(**thin)) == (L.TE_OK, 0)
    # ... large ones read packed hi+lo planes of both operands: 2 * 2 * 2048*2048*4 bytes
    big = dict(M=2048, N=2048, K=2048, lda=2048, ldb=2048, ldc=2048, precision=L.TE_PREC_3XTF32)
    assert _ws(_desc(**big)) == (L.TE_OK, 4 * 2048 * 2048 * 4)
    # an operand TMA cannot address is still copied once (not split) in 3xTF32 mode
    assert _ws(_desc(M=64, K=65, N=64, lda=65, ldb=64, precision=L.TE_PREC_3XTF32))[1] == 64 * 68 * 4
    # a leading dimension that is not a multiple of 4 floats cannot be addressed by TMA -> one packed copy of A
    rc, n = _ws(_desc(M=64, K=65, N=64, lda=65, ldb=64))
    assert rc == L.TE_OK and n == 64 * 68 * 4
    # a misaligned base pointer likewise
    assert _ws(_desc(b=0x1004))[1] == 64 * 64 * 4
    # broadcast operands are packed once
    rc, n = _ws(_desc(batch_inner=8, a=0x1004, a_stride_inner=64 * 64, b=0x2004, b_stride_inner=0, c_stride_inner=64 * 64))
    assert n == (8 + 1) * 64 * 64 * 4
    # empty problems need nothing
    assert _ws(_desc(M=0))[1] == 0
    # a left operand stored M-major (a weight gradient dY^T . X) is split inside the kernel up to M*N*K = 2^34 ...
    wgrad = dict(M=384, N=1536, K=16384, a_major=L.TE_COL_MAJOR, lda=384, ldb=1536, ldc=1536, precision=L.TE_PREC_3XTF32)
    assert _ws(_desc(**wgrad)) == (L.TE_OK, 0)
    # ... the same extents with a K-major left operand read packed planes
    assert _ws(_desc(**dict(wgrad, a_major=L.TE_ROW_MAJOR, lda=16384)))[1] == 2 * (384 + 1536) * 16384 * 4


def test_static_entry_counts_its_own_planes():
    """The no-allocation entry always packs hi / lo planes into its fixed array, whatever the context path would do
    with the same problem: a thin product whose planes exceed the array is refused on the host, before any CUDA call."""
    lib = L.load()
    thin = _desc(M=16, N=8192, K=8192, lda=8192, ldb=8192, ldc=8192, precision=L.TE_PREC_3XTF32)
    assert _ws(thin) == (L.TE_OK, 0)
    assert lib.te_b200_gemm_3xtf32_static(C.byref(thin), None, None) == L.TE_ERR_WORKSPACE
    assert b"static scratch array holds" in lib.te_b200_last_error()


@pytest.mark.parametrize("total,world,align", [(8192, 8, 256), (8192, 4, 256), (65, 4, 1), (16, 8, 1), (16, 3, 1), (1000, 8, 128),
                                               (5, 8, 1), (0, 2, 1)])
def test_shard_ranges_partition_exactly(total, world, align):
    covered = 0
    for r in range(world):
        b, n = L.shard_range(total, world, r, align)
        assert b == covered and n >= 0
        if n and b + n < total:
            assert n % align == 0
        covered += n
    assert covered == total


def test_shard_range_rejects_bad_arguments():
    for args in [(-1, 2, 0, 1), (8, 0, 0, 1), (8, 2, 2, 1), (8, 2, 0, 0)]:
        with pytest.raises(L.BackendError):
            L.shard_range(*args)


def test_init_fails_loudly_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = L.load().te_b200_init(0, 1 << 20, C.byref(h))
    assert rc == L.TE_ERR_NO_DEVICE and not h.value
    assert b"no CPU path" in L.load().te_b200_last_error()
    from torch_engine_b200 import ops
    with pytest.raises(L.BackendError):
        ops.Backend(0)


def test_null_context_is_rejected():
    d = _desc()
    assert L.load().te_b200_gemm_f32(None, C.byref(d), None) == L.TE_ERR_BAD_ARGUMENT
    assert L.load().te_b200_softmax_rows_f32(None, None, None, 1, 1, None) == L.TE_ERR_BAD_ARGUMENT


def _plan(M, K, N, prec=None, batch=1, sm=148, scratch=1 << 30):
    d = _desc(M=M, K=K, N=N, lda=K, ldb=N, ldc=N, batch_inner=batch, a_stride_inner=M * K, b_stride_inner=K * N,
              c_stride_inner=M * N, precision=L.TE_PREC_TF32 if prec is None else prec)
    bn, pair, splits = C.c_int(), C.c_int(), C.c_int()
    rc = L.load().te_b200_gemm_plan(C.byref(d), sm, scratch, C.byref(bn), C.byref(pair), C.byref(splits))
    assert rc == L.TE_OK
    return bn.value, bool(pair.value), splits.value


def test_tile_cost_model_choices():
    """The tile choice is host arithmetic: pin the decisions the measurements behind it led to."""
    assert _plan(8192, 8192, 8192) == (512, True, 1)                   # the headline shape: wide 256 x 512 CTA-pair tiles
    assert _plan(2048, 2048, 2048) == (256, True, 1)                   # too few tiles for the wide form to pay
    assert _plan(8192, 512, 8192) == (256, True, 1)                    # short K: the wide form's exposed epilogue loses
    assert _plan(16384, 1536, 384) == (384, True, 1)                   # one wave of 256 x 384 tiles
    assert _plan(8192, 1024, 8192) == (256, True, 1)                   # 32 k-blocks: too short for the wide form
    assert _plan(16384, 384, 384) == (192, True, 1)                    # N = 384: two 192-wide tiles, not 256 + half-empty 256
    assert _plan(16384, 384, 1536) == (256, True, 1)
    assert _plan(4096, 768, 3072) == (256, True, 1)
    bn, pair, splits = _plan(16, 8192, 8192)                           # thin M: single-CTA kernel, K split over several units
    assert not pair and splits > 1
    assert _plan(16, 8192, 8192, scratch=0)[2] == 1                    # no scratch, no split
    bn, pair, splits = _plan(384, 16384, 384)                          # weight gradient: few tiles, long K
    assert splits > 1
    assert _plan(100, 64, 100)[1] is False                             # fits one 128-row tile: no pair
    assert _plan(8192, 8192, 8192, prec=L.TE_PREC_3XTF32) == (256, True, 1)
    bn, pair, splits = _plan(2048, 2048, 2048, prec=L.TE_PREC_3XTF32)  # 3xTF32 below K ~ 5000: single-CTA form, <= 128 wide
    assert not pair and bn <= 128
    for shape in [(1, 1, 1), (1000, 3, 7), (5, 100000, 5), (256, 512, 192)]:
        bn, pair, splits = _plan(*shape)
        assert bn in (64, 128, 192, 256, 384, 512) and splits >= 1
    d = _desc(M=-1)
    assert L.load().te_b200_gemm_plan(C.byref(d), 148, 0, None, None, None) == L.TE_ERR_BAD_ARGUMENT
