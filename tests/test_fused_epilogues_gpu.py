"""GPU parity of what the GEMM epilogues and the fused callers absorb from the reference's graph: the residual adds of
src/nn/transformer_block.cpp:15-35 and the gradient accumulation of src/tensor/tensor.cpp:1138-1142 (`residual` of
te_gemm_desc), MultiHeadAttention as one call forward and backward, the FeedForward chain, LayerNorm backward with the
gradient of the bypassing branch, the single-launch column sum, packing of many small batches, and the bounded-wait
failure path.  Goldens come from the reference's own CPU autograd (tests/golden/nn_cases.npz)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import binding
from tests import golden_cases as gc
from tests.gpu_util import TOL_REL, rel_err, rel_err_floored
from torch_engine_b200 import lib as L

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
PRECS = ["tf32", "3xtf32"]
ATTN_TOL = {"tf32": 1e-2, "3xtf32": 2e-5}      # two chained GEMMs around an exponential
CHAIN_TOL = {"tf32": 2e-2, "3xtf32": 1e-4}     # gradients through 4-12 chained GEMMs


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _desc(a, b, c, prec, bias=None, residual=None, epilogue=L.TE_EPI_NONE):
    M, K = a.shape
    N = b.shape[1]
    d = L.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.a, d.b, d.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    d.lda, d.ldb, d.ldc = a.stride(0), b.stride(0), c.stride(0)
    d.batch_outer = d.batch_inner = 1
    d.alpha = 1.0
    d.bias = bias.data_ptr() if bias is not None else None
    d.residual = residual.data_ptr() if residual is not None else None
    d.epilogue = epilogue
    d.precision = L.TE_PREC_TF32 if prec == "tf32" else L.TE_PREC_3XTF32
    return d


# single-CTA tiles, CTA-pair tiles, wide pair tiles (K >= 2048), split K (thin M), an output no tensor map describes
RESIDUAL_SHAPES = [(96, 200, 72), (512, 256, 384), (1024, 4096, 1024), (16, 4096, 512), (300, 128, 130), (260, 64, 65)]


@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("mkn", RESIDUAL_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_gemm_residual_and_in_place_accumulation(backend, mkn, prec):
    M, K, N = mkn
    g = torch.Generator(device="cuda").manual_seed(M + K + N)
    a = torch.rand(M, K, device="cuda", generator=g) * 2 - 1
    b = torch.rand(K, N, device="cuda", generator=g) * 2 - 1
    bias = torch.rand(N, device="cuda", generator=g)
    r = torch.randn(M, N, device="cuda", generator=g) * 3
    ref = a.double() @ b.double()
    scale = float(ref.abs().max())
    tol = TOL_REL[prec] * scale
    c = torch.empty(M, N, device="cuda")
    backend.gemm(_desc(a, b, c, prec, residual=r))
    assert float((c.double() - (ref + r.double())).abs().max()) <= tol
    backend.gemm(_desc(a, b, c, prec, bias=bias, residual=r, epilogue=L.TE_EPI_BIAS))
    assert float((c.double() - (ref + bias.double() + r.double())).abs().max()) <= tol
    # c += a.b : the residual is the output itself, twice in a row
    acc = r.clone()
    backend.gemm(_desc(a, b, acc, prec, residual=acc))
    backend.gemm(_desc(a, b, acc, prec, residual=acc))
    assert float((acc.double() - (r.double() + 2 * ref)).abs().max()) <= 2 * tol
    backend.check_device_status()


@pytest.mark.parametrize("prec", PRECS)
def test_linear_backward_with_branch_gradient_and_accumulation(backend, prec):
    nn = gc.nn_inputs()["linear"]
    gold = np.load(os.path.join(GOLD, "nn_cases.npz"))
    x, w, dy = dev(nn["x"]), dev(nn["w"]), dev(nn["dy"])
    branch = torch.randn_like(x)
    dw0 = torch.randn_like(w)
    db0 = torch.randn(w.shape[0], device="cuda")
    dw, db = dw0.clone(), db0.clone()
    dx, _, _ = backend.linear_backward(x, w, dy, precision=prec, dx_residual=branch, accumulate_into=(dw, db))
    assert rel_err((dx - branch).cpu().numpy(), gold["linear.dx"]) <= 2 * TOL_REL[prec]
    assert rel_err((dw - dw0).cpu().numpy(), gold["linear.dw"]) <= 2 * TOL_REL[prec]
    assert np.abs((db - db0).cpu().numpy() - gold["linear.db"]).max() <= 1e-4
    backend.check_device_status()


@pytest.mark.parametrize("prec", PRECS)
def test_feed_forward_goldens(backend, prec):
    """FeedForward forward and backward (src/nn/ffn.cpp:12-16) against the reference's autograd: Linear+GELU with the
    pre-activation kept, Linear; backward through te_b200_linear_backward_ex (x_preact form) and the plain form."""
    f = gc.nn_inputs()["ffn"]
    gold = np.load(os.path.join(GOLD, "nn_cases.npz"))
    x, w1, b1, w2, b2, dy = (dev(f[k]) for k in ("x", "w1", "b1", "w2", "b2", "dy"))
    h, pre = backend.linear_forward(x, w1, b1, gelu=True, want_preact=True, precision=prec)
    y = backend.linear_forward(h, w2, b2, precision=prec)
    assert rel_err(y.cpu().numpy(), gold["ffn.y"]) <= 3 * TOL_REL[prec]
    d_pre, dw2, db2 = backend.linear_backward(h, w2, dy, precision=prec, gelu_preact=pre)
    dx, dw1, db1 = backend.linear_backward(x, w1, d_pre, precision=prec)
    for got, name in ((dx, "dx"), (dw1, "dw1"), (db1, "db1"), (dw2, "dw2"), (db2, "db2")):
        assert rel_err(got.cpu().numpy(), gold[f"ffn.{name}"]) <= 3 * TOL_REL[prec], name
    # the first Linear's bias gradient as a by-product of the GeluBackward pass (column sums of d_pre)
    d_pre2, _, _, db1_fused = backend.linear_backward(h, w2, dy, precision=prec, gelu_preact=pre, want_dx_colsum=True)
    assert torch.equal(d_pre2, d_pre)
    assert rel_err(db1_fused.cpu().numpy(), gold["ffn.db1"]) <= 3 * TOL_REL[prec]
    backend.check_device_status()


@pytest.mark.parametrize("one_gemm", [True, False], ids=["qkv_one_gemm", "qkv_three_gemms"])
@pytest.mark.parametrize("prec", PRECS)
def test_multi_head_attention_goldens(backend, prec, one_gemm):
    """te_b200_mha_forward / _backward against MultiHeadAttention::forward + backward of the reference (CPU autograd),
    with the three input projections as one product against the gathered weights and as three products."""
    m = gc.nn_inputs()["mha"]
    gold = np.load(os.path.join(GOLD, "nn_cases.npz"))
    x, dy = dev(m["x"]), dev(m["dy"])
    params = [dev(p) for p in m["params"]]
    y, saved = backend.mha_forward(x, params, m["H"], precision=prec, one_projection_gemm=one_gemm)
    assert rel_err(y.cpu().numpy(), gold["mha.y"]) <= ATTN_TOL[prec]
    dx, grads = backend.mha_backward(saved, dy, precision=prec)
    assert rel_err(dx.cpu().numpy(), gold["mha.dx"]) <= CHAIN_TOL[prec]
    # the key-projection bias gradient is zero in exact arithmetic: what any implementation returns there is rounding
    # noise of sums of O(1) terms, so it is measured against the scale of the other gradients
    gmax = max(float(np.abs(gold[f"mha.dparam{i}"]).max()) for i in range(8))
    for i, g in enumerate(grads):
        floor = gmax if float(np.abs(gold[f"mha.dparam{i}"]).max()) < 1e-3 * gmax else 0.0
        assert rel_err_floored(g.cpu().numpy(), gold[f"mha.dparam{i}"], floor) <= CHAIN_TOL[prec], i
    # with the block's residual input and the gradient of the bypassing branch
    y2, saved2 = backend.mha_forward(x, params, m["H"], residual=x, precision=prec, one_projection_gemm=one_gemm)
    assert rel_err((y2 - x).cpu().numpy(), gold["mha.y"]) <= ATTN_TOL[prec]
    dx2, _ = backend.mha_backward(saved2, dy, dx_residual=dy, precision=prec)
    assert rel_err((dx2 - dy).cpu().numpy(), gold["mha.dx"]) <= CHAIN_TOL[prec]
    backend.check_device_status()


def test_multi_head_attention_projection_forms_agree(backend):
    """One product against the gathered [3E,E] weight computes each projection element as the same dot product as the
    three-product form: the forward results are identical; so are the parameter gradients of the projections (the
    same products, the same column sums).  Bad layouts of the one-product form are refused."""
    torch.manual_seed(5)
    B, T, E, H = 3, 128, 256, 4
    x = torch.randn(B, T, E, device="cuda")
    dy = torch.randn(B, T, E, device="cuda")
    params = []
    for _ in range(4):
        params += [torch.randn(E, E, device="cuda") / 16, torch.randn(E, device="cuda")]
    y1, s1 = backend.mha_forward(x, params, H, one_projection_gemm=True)
    y3, s3 = backend.mha_forward(x, params, H, one_projection_gemm=False)
    assert s1["qkv"].shape == (B, T, 3 * E) and s1["q"].stride() == (T * 3 * E, 3 * E, 1)
    packed_w = s1["wqkv"][:3 * E * E].reshape(3, E, E)
    packed_b = s1["wqkv"][3 * E * E:].reshape(3, E)
    for i in range(3):
        assert torch.equal(packed_w[i], params[2 * i]) and torch.equal(packed_b[i], params[2 * i + 1])
        assert torch.equal(s1["qkv"][:, :, i * E:(i + 1) * E], s3[("q", "k", "v")[i]]), i
    assert torch.equal(s1["p"], s3["p"]) and torch.equal(y1, y3)
    dx1, g1 = backend.mha_backward(s1, dy)
    dx3, g3 = backend.mha_backward(s3, dy)
    for i in range(8):
        # projection weight gradients: split-K slices differ between a [3E,E] and an [E,E] product, so the sums
        # are the same terms in another order
        assert rel_err(g1[i].cpu().numpy(), g3[i].cpu().numpy()) <= 1e-5, i
    assert rel_err(dx1.cpu().numpy(), dx3.cpu().numpy()) <= 1e-5    # one K = 3E sum against three chained K = E sums
    m = L.MhaDesc()
    m.B, m.T, m.E, m.H = B, T, E, H
    m.x = x.data_ptr()
    for n, t in zip(("wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo"), params):
        setattr(m, n, t.data_ptr())
    q = s1["qkv"].data_ptr()
    m.q, m.k, m.v, m.p, m.attn, m.y = q, q + 4 * E, q + 8 * E, s1["p"].data_ptr(), s1["attn"].data_ptr(), y1.data_ptr()
    m.ld_qkv = 3 * E                      # the scratch is missing
    assert backend._lib.te_b200_mha_forward(backend._ctx, C.byref(m), None) == L.TE_ERR_BAD_ARGUMENT
    m.wqkv, m.k = s1["wqkv"].data_ptr(), q + 8 * E      # k is not the second column block
    assert backend._lib.te_b200_mha_forward(backend._ctx, C.byref(m), None) == L.TE_ERR_BAD_ARGUMENT
    m.k, m.ld_qkv = q + 4 * E, 2 * E
    assert backend._lib.te_b200_mha_forward(backend._ctx, C.byref(m), None) == L.TE_ERR_BAD_ARGUMENT
    backend.check_device_status()


@pytest.mark.parametrize("prec", PRECS)
def test_scaled_dot_backward_on_head_views_goldens(backend, prec):
    """dQ, dK, dV for operands taken as MultiHeadAttention's head views, against the reference's autograd."""
    s = gc.nn_inputs()["scaled_dot"]
    gold = np.load(os.path.join(GOLD, "nn_cases.npz"))
    B, H, T, d = s["B"], s["H"], s["T"], s["d"]
    heads = lambda t: dev(t).view(B, T, H, d).transpose(1, 2)
    q, k, v = heads(s["q"]), heads(s["k"]), heads(s["v"])
    o, p = backend.scaled_dot(q, k, v, precision=prec)
    assert rel_err(o.cpu().numpy(), gold["scaled_dot_views.o"]) <= ATTN_TOL[prec]
    dq, dk, dv = backend.scaled_dot_backward(q, k, v, p, dev(s["d_o"]), o=o, precision=prec, head_major_out=False)
    # the goldens are gradients of the [B,T,E] base tensors: the head-minor memory order of these views
    for got, name in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        flat = got.transpose(1, 2).contiguous().reshape(-1).cpu().numpy()
        assert rel_err(flat, gold[f"scaled_dot_views.{name}"]) <= CHAIN_TOL[prec], name
    backend.check_device_status()


def test_layernorm_backward_adds_the_bypassing_gradient(backend, oracle):
    c = gc.step_op_inputs()["ln"]["ln384"]
    x, gamma, dy = dev(c["x"]), dev(c["gamma"]), dev(c["dy"])
    branch = torch.randn_like(x)
    dx0, dg0, db0 = backend.layernorm_backward(x, gamma, dy)
    dx1, dg1, db1 = backend.layernorm_backward(x, gamma, dy, dx_residual=branch)
    assert torch.equal(dg0, dg1) and torch.equal(db0, db1)
    assert float((dx1 - (dx0 + branch)).abs().max()) <= 1e-6
    dx_ref, _, _ = oracle.layernorm_backward(c["x"], c["gamma"], c["dy"])
    assert np.abs(dx0.cpu().numpy() - dx_ref).max() <= 2e-5
    # column sums of the result (the bias gradient of the Linear feeding the residual stream) out of the same pass
    dx2, dg2, db2, sums = backend.layernorm_backward(x, gamma, dy, dx_residual=branch, want_dx_colsum=True)
    assert torch.equal(dx2, dx1) and torch.equal(dg2, dg1) and torch.equal(db2, db1)
    want = dx1.double().reshape(-1, dx1.shape[-1]).sum(dim=0)
    assert float((sums.double() - want).abs().max()) <= 1e-5 * max(1.0, float(want.abs().max()))
    backend.check_device_status()


@pytest.mark.parametrize("rows,cols", [(16384, 384), (16384, 1536), (16384, 65), (700, 132), (5, 7), (4096, 4000)])
def test_colsum_single_launch_is_deterministic_and_accumulates(backend, oracle, rows, cols):
    rng = binding.SeededRng(rows + cols)
    x = rng.normal((rows, cols))
    tx = dev(x)
    n0 = backend.launches
    s1 = backend.colsum(tx)
    assert backend.launches - n0 == 1
    s2 = backend.colsum(tx)
    assert torch.equal(s1, s2)                                  # fixed summation order: the same bits every run
    ref = x.astype(np.float64).sum(axis=0)
    assert rel_err(s1.cpu().numpy(), ref) <= 1e-5
    # accumulate form, through the Linear backward entry (db += column sums of dy)
    w = torch.zeros(cols, 8, device="cuda")
    xin = torch.zeros(rows, 8, device="cuda")
    db = torch.full((cols,), 2.0, device="cuda")
    dw = torch.zeros_like(w)
    backend.linear_backward(xin, w, tx, need_dx=False, accumulate_into=(dw, db))
    assert rel_err((db - 2.0).cpu().numpy(), ref) <= 1e-5
    backend.check_device_status()


def test_3xtf32_many_small_batches(backend):
    """More than 65535 batches in one call: the packing pre-pass of the 3xTF32 mode walks them instead of refusing."""
    Bn, M, K, N = 70000, 4, 8, 4
    g = torch.Generator(device="cuda").manual_seed(9)
    a = torch.rand(Bn, M, K, device="cuda", generator=g) * 2 - 1
    b = torch.rand(Bn, K, N, device="cuda", generator=g) * 2 - 1
    ref = torch.bmm(a.double(), b.double())
    for prec in PRECS:
        c = backend.matmul(a, b, precision=prec)
        assert float((c.double() - ref).abs().max()) <= TOL_REL[prec] * float(ref.abs().max())
    # a column-major operand takes the transposing pack kernel, whose grid is capped in y and z
    at = torch.rand(Bn, K, M, device="cuda", generator=g).transpose(1, 2)
    c = backend.matmul(at, b, precision="3xtf32")
    assert float((c.double() - torch.bmm(at.double(), b.double())).abs().max()) <= 1e-5 * float(ref.abs().max())
    backend.check_device_status()


def test_bounded_wait_runs_out_and_the_context_survives(backend):
    """A kernel waits on a barrier nothing arrives at, with a 1 ms bound: it returns by itself, the status word carries
    the site code, te_b200_check_device_status reports TE_ERR_DEVICE_TIMEOUT and clears it -- ten times in a row --
    and a GEMM on the same context afterwards is correct."""
    backend.check_device_status()
    backend.set_wait_limit_ns(1_000_000)
    try:
        for _ in range(10):
            backend.selftest_wait_timeout()
            with pytest.raises(L.BackendError) as err:
                backend.check_device_status()
            assert err.value.status == L.TE_ERR_DEVICE_TIMEOUT
            assert "site code 901" in str(err.value)
            backend.check_device_status()                      # the word was cleared by the failing check
    finally:
        backend.set_wait_limit_ns(0)
    a = torch.rand(300, 200, device="cuda") * 2 - 1
    b = torch.rand(200, 260, device="cuda") * 2 - 1
    c = backend.matmul(a, b, precision="3xtf32")
    assert rel_err(c.cpu().numpy(), (a.double() @ b.double()).cpu().numpy()) <= TOL_REL["3xtf32"]
    backend.check_device_status()


def test_cross_entropy_bad_target_has_its_own_message(backend):
    logits = torch.zeros(2, 3, 5, device="cuda")
    targets = torch.tensor([[0, 1, 9], [2, 3, 4]], device="cuda")
    backend.cross_entropy(logits, targets)
    with pytest.raises(L.BackendError, match="Cross-entropy target index out of range"):
        backend.check_device_status()
    backend.check_device_status()
