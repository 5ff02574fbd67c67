"""GPU parity of the GEMM path, through the C ABI, against the oracle (the reference's CPU FP32 matmul).

Tolerances: max|C-Cref|/max|Cref| <= 2e-3 in TF32 mode and <= 1e-5 in 3xTF32 mode (tests/gpu_util.py);
where the reference's own test states a tolerance (1e-4*K absolute, src/tests/cuda_test.cpp:383) it is
checked as well."""
import ctypes as C
import json
import os

import numpy as np
import pytest
import torch

from oracle import binding
from tests import golden_cases as gc
from tests.gpu_util import TOL_REL, assert_close, rel_err
from torch_engine_b200 import lib as L

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
PRECS = ["tf32", "3xtf32"]


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.fixture(scope="module")
def known():
    with open(os.path.join(GOLD, "reference_known_answers.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("name", ["matmul_2x3_3x4", "matmul_transposed_a", "matmul_batched_3d", "matmul_f32_2x3_3x2"])
def test_reference_known_answers(backend, known, name, prec):
    k = known[name]
    a = dev(np.array(k["a"], dtype=np.float32).reshape(k["a_shape"]))
    if "a_transpose" in k:
        a = a.transpose(*k["a_transpose"])
    b = dev(np.array(k["b"], dtype=np.float32).reshape(k["b_shape"]))
    c = backend.matmul(a, b, precision=prec).cpu().numpy()
    # small integers are exact in tf32, so even the fast mode must hit the reference's tolerance
    assert np.abs(c.ravel() - np.array(k["expected"], dtype=np.float32)).max() <= max(k["tol"], 1e-6)


def test_reference_throw_cases(backend, known):
    for t in known["throws"]:
        with pytest.raises(L.BackendError) as e:
            backend.matmul(torch.zeros(t["a_shape"], device="cuda"), torch.zeros(t["b_shape"], device="cuda"))
        assert str(e.value) == t["message"]
    with pytest.raises(L.BackendError) as e:
        backend.matmul(torch.zeros(3, device="cuda"), torch.zeros(3, 2, device="cuda"))
    assert e.value.status == L.TE_ERR_SHAPE_NDIM
    # neither row- nor column-major slice (tensor.h:626)
    a = torch.zeros(8, 16, device="cuda")[:, ::2]
    with pytest.raises(L.BackendError) as e:
        backend.matmul(a, torch.zeros(8, 4, device="cuda"))
    assert e.value.status == L.TE_ERR_UNSUPPORTED_LAYOUT
    assert str(e.value) == "CUDA matmul only supports row- or column-major 2D slices"
    with pytest.raises(L.BackendError) as e:
        backend.matmul(torch.zeros(2, 2, device="cuda", dtype=torch.float64), torch.zeros(2, 2, device="cuda", dtype=torch.float64))
    assert "only supports Float32" in str(e.value)


@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("name", sorted(gc.MATMUL_CASES))
def test_golden_matmul_cases(backend, name, prec):
    gold = np.load(os.path.join(GOLD, "matmul_cases.npz"))[name]
    a, va, b, vb = gc.build_matmul_inputs(gc.MATMUL_CASES[name])
    c = backend.matmul(gc.apply_view_torch(dev(a), va), gc.apply_view_torch(dev(b), vb), precision=prec)
    assert tuple(c.shape) == gold.shape and c.is_contiguous()
    assert_close(c.cpu().numpy(), gold, prec, name)


def _layouts(a, b):
    """The four operand layouts of one logical product (views over differently stored copies)."""
    at = a.t().contiguous().t()      # column-major A
    bt = b.t().contiguous().t()      # column-major B
    return {"row.row": (a, b), "row.col": (a, bt), "col.row": (at, b), "col.col": (at, bt)}


@pytest.mark.parametrize("prec", PRECS)
def test_ragged_shapes_all_layouts(backend, oracle, known, prec):
    extra = [[1, 1, 1], [5, 3, 7], [100, 77, 65], [130, 40, 260], [257, 33, 129], [64, 1000, 8]]
    ref_cases = known["ragged_mkn"]["cases"]
    for M, K, N in ref_cases + extra:
        rng = binding.SeededRng(42)
        a, b = rng.uniform((M, K)), rng.uniform((K, N))
        ref = oracle.matmul_2d_threads(a, b)
        for lay, (ta, tb) in _layouts(dev(a), dev(b)).items():
            c = backend.matmul(ta, tb, precision=prec).cpu().numpy()
            assert_close(c, ref, prec, f"{M}x{K}x{N} {lay}")
            if [M, K, N] in ref_cases:
                assert np.abs(c - ref).max() < 1e-4 * K, "reference tolerance 1e-4*K (cuda_test.cpp:383)"
    backend.check_device_status()


@pytest.mark.parametrize("prec", PRECS)
def test_config1_512_cubed(backend, oracle, prec):
    g = np.load(os.path.join(GOLD, "c1_512_samples.npz"))
    rng = binding.SeededRng(42)
    a, b = rng.uniform((512, 512)), rng.uniform((512, 512))
    c = backend.matmul(dev(a), dev(b), precision=prec).cpu().numpy()
    ref = oracle.matmul_2d_threads(a, b)
    assert_close(c, ref, prec, "512^3")
    # the committed samples come from the reference's own CPU run
    samp = c[g["idx"][:, 0], g["idx"][:, 1]]
    assert np.abs(samp - g["values"]).max() / np.abs(ref).max() <= TOL_REL[prec]


def test_empty_and_degenerate(backend):
    z = lambda *s: torch.zeros(*s, device="cuda")
    assert backend.matmul(z(0, 8), z(8, 4)).shape == (0, 4)
    assert backend.matmul(z(4, 8), z(8, 0)).shape == (4, 0)
    # K == 0: the reference memsets the result to zero (tensor.h:577)
    c = torch.full((4, 6), float("nan"), device="cuda")
    out = backend.matmul(torch.ones(4, 0, device="cuda"), torch.ones(0, 6, device="cuda"))
    assert out.shape == (4, 6) and torch.count_nonzero(out).item() == 0
    backend.check_device_status()


@pytest.mark.parametrize("prec", PRECS)
def test_guard_band_untouched(backend, oracle, prec):
    """C is written through ldc > N into a NaN-poisoned buffer: only the M x N window may change."""
    M, K, N, ldc = 200, 96, 150, 160
    rng = binding.SeededRng(1)
    a, b = rng.uniform((M, K)), rng.uniform((K, N))
    buf = torch.full((M + 8, ldc), float("nan"), device="cuda")
    d = L.GemmDesc()
    d.M, d.N, d.K = M, N, K
    ta, tb = dev(a), dev(b)
    d.a, d.b, d.c = ta.data_ptr(), tb.data_ptr(), buf[4:].data_ptr()
    d.lda, d.ldb, d.ldc = K, N, ldc
    d.batch_outer = d.batch_inner = 1
    d.precision = L.TE_PREC_TF32 if prec == "tf32" else L.TE_PREC_3XTF32
    backend.gemm(d)
    backend.check_device_status()
    out = buf.cpu().numpy()
    assert np.isnan(out[:4]).all() and np.isnan(out[4 + M:]).all() and np.isnan(out[4:4 + M, N:]).all()
    assert_close(out[4:4 + M, :N], oracle.matmul(a, b), prec, "guard band window")


@pytest.mark.parametrize("prec", PRECS)
def test_operands_tma_cannot_address(backend, oracle, prec):
    """Odd leading dimensions and a base pointer off 16-byte alignment take the packing pre-pass."""
    rng = binding.SeededRng(5)
    M, K, N = 70, 65, 33            # the language-model-head shapes have N = 65
    a, b = rng.uniform((M, K)), rng.uniform((K, N))
    ref = oracle.matmul(a, b)
    ta, tb = dev(a), dev(b)
    for lay, (x, y) in _layouts(ta, tb).items():
        assert_close(backend.matmul(x, y, precision=prec).cpu().numpy(), ref, prec, "odd ld " + lay)
    # misaligned base: slice off one leading float of a padded buffer
    pad = torch.zeros(M * 72 + 1, device="cuda")
    am = pad[1:].view(M, 72)[:, :64]
    am.copy_(dev(a[:, :64]))
    b64 = dev(rng.uniform((64, 40)))
    assert (am.data_ptr() % 16) != 0
    assert_close(backend.matmul(am, b64, precision=prec).cpu().numpy(), oracle.matmul(a[:, :64].copy(), b64.cpu().numpy()),
                 prec, "misaligned base")
    backend.check_device_status()


@pytest.mark.parametrize("prec", PRECS)
def test_nd_broadcast_and_unmergeable_batches(backend, oracle, prec):
    g = torch.Generator(device="cpu").manual_seed(3)
    cases = []
    a = torch.randn(2, 1, 40, 24, generator=g); b = torch.randn(3, 24, 36, generator=g); cases.append((a, b))
    # three batch levels that cannot be merged (A is a permuted view): exercises the host loop over outer levels
    a = torch.randn(3, 2, 4, 16, 24, generator=g).permute(1, 0, 2, 3, 4); b = torch.randn(2, 3, 4, 24, 20, generator=g); cases.append((a, b))
    # Linear-style: 3-D input against a broadcast 2-D transposed weight
    a = torch.randn(4, 50, 32, generator=g); b = torch.randn(48, 32, generator=g).t(); cases.append((a, b))
    for a, b in cases:
        ref = oracle.matmul(a.numpy(), b.numpy())
        c = backend.matmul(a.cuda(), b.cuda(), precision=prec)
        assert tuple(c.shape) == ref.shape
        assert_close(c.cpu().numpy(), ref, prec, f"{tuple(a.shape)}@{tuple(b.shape)}")


@pytest.mark.parametrize("prec", PRECS)
def test_epilogues(backend, oracle, prec):
    rng = binding.SeededRng(9)
    M, K, N = 150, 72, 200
    a, b = rng.normal((M, K)), rng.normal((K, N), 0.0, 0.2)
    bias = rng.normal((N,), 0.0, 0.5)
    base = oracle.matmul(a, b)
    ta, tb, tbias = dev(a), dev(b), dev(bias)

    def run(**kw):
        c = torch.empty(M, N, device="cuda")
        pre = torch.empty(M, N, device="cuda") if kw.pop("want_pre", False) else None
        d = L.GemmDesc()
        d.M, d.N, d.K = M, N, K
        d.a, d.b, d.c = ta.data_ptr(), tb.data_ptr(), c.data_ptr()
        d.lda, d.ldb, d.ldc = K, N, N
        d.batch_outer = d.batch_inner = 1
        d.alpha = 1.0
        d.precision = L.TE_PREC_TF32 if prec == "tf32" else L.TE_PREC_3XTF32
        if pre is not None:
            d.preact_out = pre.data_ptr()
        for k, v in kw.items():
            setattr(d, k, v)
        backend.gemm(d)
        return c.cpu().numpy(), (pre.cpu().numpy() if pre is not None else None)

    c, _ = run(scale_mode=L.TE_SCALE_DIV, alpha=8.0)
    assert_close(c, (base / np.float32(8.0)).astype(np.float32), prec, "divide")
    c, _ = run(scale_mode=L.TE_SCALE_MUL, alpha=0.37)
    assert_close(c, (base * np.float32(0.37)).astype(np.float32), prec, "multiply")
    c, _ = run(epilogue=L.TE_EPI_BIAS, bias=tbias.data_ptr())
    assert_close(c, oracle.add_bias(base, bias), prec, "bias")
    c, pre = run(epilogue=L.TE_EPI_BIAS_GELU, bias=tbias.data_ptr(), want_pre=True)
    pre_ref = oracle.add_bias(base, bias)
    assert_close(pre, pre_ref, prec, "pre-activation")
    # GELU is 1.13-Lipschitz: the GEMM error passes through, plus the reference's own 1e-4 GELU tolerance
    assert np.abs(c - oracle.gelu(pre_ref)).max() <= 1.2 * TOL_REL[prec] * np.abs(pre_ref).max() + 1e-4
    # and GELU of the kernel's own pre-activation matches the formula tightly
    assert np.abs(c - oracle.gelu(pre)).max() <= 1e-5
    backend.check_device_status()


@pytest.mark.parametrize("n,rows", [(2048, 24), (4096, 16), (8192, 12)])
@pytest.mark.parametrize("prec", PRECS)
def test_large_squares_sampled_rows(backend, oracle, n, rows, prec):
    """Full-size products checked on sampled rows against a float64-accumulated oracle (the summation-order
    noise of any float32 result at K=8192 is itself ~1e-6, so float64 is the arbiter here)."""
    g = torch.Generator(device="cuda").manual_seed(42)
    a = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
    b = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
    c = backend.matmul(a, b, precision=prec)
    backend.check_device_status()
    pick = np.linspace(0, n - 1, rows).astype(int)
    ref = oracle.matmul_f64(a.cpu().numpy(), b.cpu().numpy(), rows=pick.tolist())[pick]
    assert_close(c[pick].cpu().numpy(), ref, prec, f"{n}^3 rows")
    # size-independent property: the column-major-B form of the same product agrees with the row-major form
    c2 = backend.matmul(a, b.t().contiguous().t(), precision=prec)
    assert rel_err(c2.cpu().numpy(), c.cpu().numpy()) <= 2 * TOL_REL[prec]


def test_largest_sweep_square_16384(backend, oracle):
    """16384^3 (1 GiB per operand): sampled rows against the float64 oracle in both modes, and two size-independent
    properties: scaling A by a power of two scales C exactly, and the N-column-sharded evaluation (what each GPU of a
    multi-GPU run computes) reproduces the unsharded columns bit for bit."""
    n = 16384
    g = torch.Generator(device="cuda").manual_seed(42)
    a = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
    b = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
    pick = np.linspace(0, n - 1, 6).astype(int)
    ref = oracle.matmul_f64(a[pick].cpu().numpy(), b.cpu().numpy())
    c = backend.matmul(a, b, precision="tf32")
    assert_close(c[pick].cpu().numpy(), ref, "tf32", "16384^3 tf32")
    c4 = backend.matmul(a * 4.0, b, precision="tf32")
    assert torch.equal(c4[pick], c[pick] * 4.0), "power-of-two scaling must be exact"
    shard = backend.matmul(a, b[:, 4096:8192], precision="tf32")
    assert torch.equal(shard, c[:, 4096:8192]), "column shard differs from the unsharded product"
    del c4, shard
    c3 = backend.matmul(a, b, precision="3xtf32")
    assert_close(c3[pick].cpu().numpy(), ref, "3xtf32", "16384^3 3xtf32")
    backend.check_device_status()


@pytest.mark.parametrize("shape", [(8192, 512, 8192), (8192, 8192, 512), (16, 8192, 8192)])
def test_skinny_sweep_shapes(backend, oracle, shape):
    M, K, N = shape
    g = torch.Generator(device="cuda").manual_seed(42)
    a = torch.rand(M, K, device="cuda", generator=g) * 2 - 1
    b = torch.rand(K, N, device="cuda", generator=g) * 2 - 1
    pick = np.linspace(0, M - 1, min(M, 12)).astype(int)
    ref = oracle.matmul_f64(a.cpu().numpy(), b.cpu().numpy(), rows=pick.tolist())[pick]
    for prec in PRECS:
        c = backend.matmul(a, b, precision=prec)
        assert_close(c[pick].cpu().numpy(), ref, prec, f"{shape}")
    backend.check_device_status()


@pytest.mark.parametrize("prec", PRECS)
def test_split_k_paths(backend, oracle, prec):
    """Few output tiles and a long K: the launcher splits K over several work units per tile, the partial tiles go
    to scratch and a reduction kernel adds them and applies the epilogue.  Covers the TMA-stored and the directly
    stored partials (N not a multiple of 4), batches, the pair kernel (M, N > 128) and the fused epilogue."""
    rng = binding.SeededRng(17)
    for (B, M, K, N) in [(1, 96, 4096, 200), (1, 40, 3000, 198), (3, 64, 2048, 72), (1, 384, 8192, 320), (1, 16, 8192, 1024)]:
        a = rng.normal((B, M, K)) if B > 1 else rng.normal((M, K))
        b = rng.normal((K, N), 0.0, 0.1)
        bias = rng.normal((N,), 0.0, 0.5)
        ref = oracle.matmul(a, b) if B > 1 else oracle.matmul_2d_threads(a, b)
        n0 = backend.launches
        c = backend.matmul(dev(a), dev(b), precision=prec)
        used = backend.launches - n0
        assert used >= 2, "expected the split-K path (GEMM + reduction)"
        assert_close(c.cpu().numpy(), ref, prec, f"split-K {B}x{M}x{K}x{N}")
        if B == 1:   # epilogue applied by the reduction kernel
            y, pre = backend.linear_forward(dev(a), dev(np.ascontiguousarray(b.T)), dev(bias), gelu=True, want_preact=True,
                                            precision=prec)
            pre_ref = oracle.add_bias(ref, bias)
            assert_close(pre.cpu().numpy(), pre_ref, prec, "split-K pre-activation")
            assert np.abs(y.cpu().numpy() - oracle.gelu(pre.cpu().numpy())).max() <= 1e-5
    backend.check_device_status()


def test_host_buffer_entry_point(backend, oracle):
    rng = binding.SeededRng(42)
    M, K, N = 300, 128, 260
    a, b = rng.uniform((M, K)), rng.uniform((K, N))
    c = np.zeros((M, N), dtype=np.float32)
    d = L.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.a, d.b, d.c = a.ctypes.data, b.ctypes.data, c.ctypes.data
    d.lda, d.ldb, d.ldc = K, N, N
    d.batch_outer = d.batch_inner = 1
    d.precision = L.TE_PREC_3XTF32
    backend.gemm_host(d)
    assert_close(c, oracle.matmul(a, b), "3xtf32", "host entry")
    # a tall product in TF32 mode takes the row-block pipeline (copy-in / multiply / copy-out overlapped)
    M, K, N = 2500, 192, 520
    a, b, bias = rng.uniform((M, K)), rng.uniform((K, N)), rng.uniform((N,))
    c = np.full((M, N), np.nan, dtype=np.float32)
    pre = np.full((M, N), np.nan, dtype=np.float32)
    d = L.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.a, d.b, d.c = a.ctypes.data, b.ctypes.data, c.ctypes.data
    d.lda, d.ldb, d.ldc = K, N, N
    d.batch_outer = d.batch_inner = 1
    d.precision = L.TE_PREC_TF32
    d.epilogue, d.bias, d.preact_out = L.TE_EPI_BIAS_GELU, bias.ctypes.data, pre.ctypes.data
    backend.gemm_host(d)
    pre_ref = oracle.add_bias(oracle.matmul_2d_threads(a, b), bias)
    assert_close(pre, pre_ref, "tf32", "pipelined host entry, pre-activation")
    assert np.abs(c - oracle.gelu(pre)).max() <= 1e-5


@pytest.mark.parametrize("M,K,N", [(16, 8192, 8192), (1, 4100, 2048), (7, 1000, 516), (16, 300, 1024)])
def test_thin_rows_fp32_accurate_mode(backend, M, K, N):
    """At most 16 rows in the FP32-accurate mode: the memory-bound FP32-FMA form (two launches: the product in K
    slices, the reduction with the epilogue).  Error against float64 at FP32 level, K tails and column tails
    included; scale, bias + GELU and residual come out of the reduction like for the tensor-core kernels; the
    same call with a layout the form does not take (N not a multiple of 4, a batch) gives the same numbers."""
    g = torch.Generator(device="cuda").manual_seed(M * 131 + K)
    a = torch.rand(M, K, device="cuda", generator=g) * 2 - 1
    b = torch.rand(K, N, device="cuda", generator=g) * 2 - 1
    ref = a.double() @ b.double()
    n0 = backend.launches
    c = backend.matmul(a, b, precision="3xtf32")
    assert backend.launches == n0 + 2
    assert float((c.double() - ref).abs().max() / ref.abs().max()) <= 2e-6
    # a row-strided A (a slice of a wider matrix) and a B that is a column block of a wider matrix
    wide_a = torch.rand(M, K + 8, device="cuda", generator=g)
    wide_b = torch.rand(K, N + 64, device="cuda", generator=g)
    a2, b2 = wide_a[:, 4:4 + K], wide_b[:, 32:32 + N]
    c2 = backend.matmul(a2, b2, precision="3xtf32")
    ref2 = a2.double() @ b2.double()
    assert float((c2.double() - ref2).abs().max() / ref2.abs().max()) <= 2e-6
    # epilogue forms
    bias = torch.randn(N, device="cuda", generator=g)
    res = torch.randn(M, N, device="cuda", generator=g)
    out = torch.empty(M, N, device="cuda")
    d = L.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.a, d.b, d.c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    d.lda, d.ldb, d.ldc = K, N, N
    d.batch_outer = d.batch_inner = 1
    d.alpha, d.scale_mode = 4.0, L.TE_SCALE_DIV
    d.bias, d.epilogue, d.residual = bias.data_ptr(), L.TE_EPI_BIAS_GELU, res.data_ptr()
    d.precision = L.TE_PREC_3XTF32
    backend.gemm(d)
    want = torch.nn.functional.gelu(ref / 4.0 + bias.double(), approximate="tanh") + res.double()
    assert float((out.double() - want).abs().max()) <= 2e-6 * float(want.abs().max()) + 2e-6
    # outside the form's limits the tensor-core path answers, within the mode's tolerance of the same reference
    b_odd = b[:, :N - 1].contiguous()
    c_odd = backend.matmul(a, b_odd, precision="3xtf32")
    assert float((c_odd.double() - ref[:, :N - 1]).abs().max() / ref.abs().max()) <= 1e-5
    backend.check_device_status()


@pytest.mark.parametrize("M,K,N,pad", [(16, 4096, 4096, 0), (8, 2048, 8192, 0), (3, 1000, 1536, 0), (13, 1031, 777, 0),
                                       (16, 1024, 1024, 3), (1, 8192, 512, 0), (11, 4100, 3000, 0), (16, 8192, 1100, 3), (4, 1024, 9600, 0),
                                       (16, 16384, 512, 0)])
def test_thin_rows_linear_layout_fp32_accurate_mode(backend, M, K, N, pad):
    """The same mode for Linear's layout, X[M,K] . W[N,K]^T with at most 16 rows of X: two launches (lanes along k
    with a fixed reduction tree over the lanes, then the K-slice reduction with the epilogue), three for a large W
    (X transposed first, so that its tiles arrive by TMA beside those of W).  W on 16-byte rows is staged by TMA; an
    odd K or an odd leading dimension (pad) takes the plain-load form.  Error against float64 at
    FP32 level for both, with bias + GELU from the reduction."""
    g = torch.Generator(device="cuda").manual_seed(M * 137 + K + pad)
    x = torch.rand(M, K, device="cuda", generator=g) * 2 - 1
    w = (torch.rand(N, K + pad, device="cuda", generator=g) * 2 - 1)[:, :K]
    ref = x.double() @ w.double().t()
    # a large W takes one more launch (X transposed for the TMA tiles) unless N is too small for that form's ranges
    allowed = (2, 3) if N * K >= 8e6 and K >= 1024 and pad == 0 else (2,)
    n0 = backend.launches
    c = backend.matmul(x, w.t(), precision="3xtf32")
    assert backend.launches - n0 in allowed
    assert float((c.double() - ref).abs().max() / ref.abs().max()) <= 2e-6
    if pad == 0:
        bias = torch.randn(N, device="cuda", generator=g)
        n0 = backend.launches
        y = backend.linear_forward(x, w, bias, gelu=True, precision="3xtf32")
        assert backend.launches - n0 in allowed
        want = torch.nn.functional.gelu(ref + bias.double(), approximate="tanh")
        assert float((y.double() - want).abs().max()) <= 2e-6 * float(want.abs().max()) + 2e-6
    # repeated calls give the same bits (no atomics, one reduction tree)
    assert torch.equal(c, backend.matmul(x, w.t(), precision="3xtf32"))
    backend.check_device_status()


def test_launch_counter_moves(backend):
    n0 = backend.launches
    backend.matmul(torch.ones(8, 8, device="cuda"), torch.ones(8, 8, device="cuda"))
    assert backend.launches == n0 + 1
    backend.matmul(torch.ones(8, 8, device="cuda"), torch.ones(8, 8, device="cuda"), precision="3xtf32")
    assert backend.launches == n0 + 2      # the 3xTF32 mode splits hi / lo inside the kernel: one launch as well
    big = torch.ones(2048, 8192, device="cuda")
    n1 = backend.launches
    backend.matmul(big, big.t().contiguous(), precision="3xtf32")
    assert backend.launches == n1 + 3      # long K, large M and N: the CTA-pair form behind two packing passes


def test_pair_tiles_192_wide(backend, oracle):
    """N in (256, 384] with enough rows takes the 256 x 192 CTA-pair tile in TF32 mode (no quarter-empty 256-wide
    tiles): all four layouts, ragged N and M, a long K, the fused Linear epilogue and a batched product."""
    for M, K, N in [(1024, 384, 384), (600, 100, 330), (512, 2100, 384), (4096, 64, 260)]:
        rng = binding.SeededRng(M + N)
        a, b = rng.uniform((M, K)), rng.uniform((K, N))
        ref = oracle.matmul_2d_threads(a, b)
        for lay, (ta, tb) in _layouts(dev(a), dev(b)).items():
            assert_close(backend.matmul(ta, tb, precision="tf32").cpu().numpy(), ref, "tf32", f"{M}x{K}x{N} {lay}")
    rng = binding.SeededRng(17)
    x, w, bias = rng.normal((2048, 96)), rng.normal((384, 96), 0.0, 0.2), rng.normal((384,), 0.0, 0.5)
    y, pre = backend.linear_forward(dev(x), dev(w), dev(bias), gelu=True, want_preact=True, precision="tf32")
    y_ref, pre_ref = oracle.linear(x, w, bias, gelu=True)
    assert_close(pre.cpu().numpy(), pre_ref, "tf32", "Linear 96->384 pre-activation")
    assert_close(y.cpu().numpy(), y_ref, "tf32", "Linear 96->384 + GELU")
    a, b = rng.uniform((3, 512, 48)), rng.uniform((3, 48, 384))
    assert_close(backend.matmul(dev(a), dev(b), precision="tf32").cpu().numpy(), oracle.matmul(a, b), "tf32", "batched 3x512x48x384")
    backend.check_device_status()


def test_wide_pair_tiles(backend, oracle):
    """Long K with enough tiles takes the wide CTA-pair tiles in TF32 mode (256 x 512 or 256 x 384: two accumulators side
    by side, one accumulator buffer): all four layouts, ragged M and N (a second tile that is mostly padding, a tile
    whose second half is empty), the fused Linear epilogue, a batched product, and bit-reproducibility."""
    # 256 x 512 tiles: (3000, 2100, 3000), (4000, 2048, 2000), (6000, 2048, 1300); 256 x 384 tiles: (3000, 2080, 2304),
    # (4000, 2100, 1300) and, as a single wave from 32 k-blocks on, (16384, 1536, 384)
    for M, K, N in [(3000, 2100, 3000), (4000, 2048, 2000), (6000, 2048, 1300), (3000, 2080, 2304), (4000, 2100, 1300), (16384, 1536, 384)]:
        rng = binding.SeededRng(M + N + 1)
        a, b = rng.uniform((M, K)), rng.uniform((K, N))
        ref = oracle.matmul_2d_threads(a, b)
        for lay, (ta, tb) in _layouts(dev(a), dev(b)).items():
            c = backend.matmul(ta, tb, precision="tf32")
            assert_close(c.cpu().numpy(), ref, "tf32", f"{M}x{K}x{N} {lay}")
            assert torch.equal(c, backend.matmul(ta, tb, precision="tf32")), "two runs differ"
    rng = binding.SeededRng(23)
    x, w, bias = rng.normal((4096, 2048)), rng.normal((2048, 2048), 0.0, 0.05), rng.normal((2048,), 0.0, 0.5)
    y, pre = backend.linear_forward(dev(x), dev(w), dev(bias), gelu=True, want_preact=True, precision="tf32")
    y_ref, pre_ref = oracle.linear(x, w, bias, gelu=True)
    assert_close(pre.cpu().numpy(), pre_ref, "tf32", "Linear 2048->2048 pre-activation")
    assert_close(y.cpu().numpy(), y_ref, "tf32", "Linear 2048->2048 + GELU")
    a, b = rng.uniform((2, 4096, 2048)), rng.uniform((2, 2048, 2048))     # 2 x 64 wide tiles
    assert_close(backend.matmul(dev(a), dev(b), precision="tf32").cpu().numpy(), oracle.matmul(a, b), "tf32", "batched 2x4096x2048x2048")
    backend.check_device_status()
