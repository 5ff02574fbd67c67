"""GPU parity of the callers of the GEMM path: Linear (+GELU) forward/backward, scaled-dot attention with
contiguous and head-view operands, and the row kernels between the GEMMs.  All through the C ABI."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import binding
from tests import golden_cases as gc
from tests.gpu_util import TOL_REL, assert_close, rel_err

# Attention chains two GEMMs around an exp: a logit error e becomes a relative error ~e in the probabilities.
# In TF32 mode the logits (|S| up to ~6 after scaling) carry ~7e-4*|QK^T|, so the composed tolerance is looser
# than the single-GEMM 2e-3; in 3xTF32 mode the single-GEMM bound still holds with a small factor.
ATTN_TOL = {"tf32": 1e-2, "3xtf32": 2e-5}

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
PRECS = ["tf32", "3xtf32"]


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.fixture(scope="module")
def nn_gold():
    return np.load(os.path.join(GOLD, "nn_cases.npz"))


@pytest.fixture(scope="module")
def known():
    with open(os.path.join(GOLD, "reference_known_answers.json")) as f:
        return json.load(f)


def test_gelu_and_softmax_value_tables(backend, oracle, known):
    x = np.array(known["gelu_inputs"]["x"], dtype=np.float32)
    y = backend.gelu(dev(x)).cpu().numpy()
    assert np.abs(y - oracle.gelu(x)).max() <= known["gelu_inputs"]["tol"]
    dy = np.linspace(-1, 1, x.size).astype(np.float32)
    assert np.abs(backend.gelu_backward(dev(x), dev(dy)).cpu().numpy() - oracle.gelu_backward(x, dy)).max() <= 1e-5
    row = np.array(known["softmax_rows"]["row"], dtype=np.float32)
    s = backend.softmax(dev(np.tile(row, (3, 1)))).cpu().numpy()
    assert np.abs(s - oracle.softmax(np.tile(row, (3, 1)))).max() <= known["softmax_rows"]["tol"]
    x3 = (np.arange(24) % 4).astype(np.float32).reshape(2, 3, 4)
    assert np.abs(backend.softmax(dev(x3)).cpu().numpy() - oracle.softmax(x3)).max() <= 1e-5
    g = backend.softmax_backward(dev(s), torch.ones(3, 4, device="cuda")).cpu().numpy()
    assert np.abs(g).max() <= 1e-6


@pytest.mark.parametrize("cols", [1, 7, 32, 33, 64, 200, 256, 1000, 1024, 1500, 4097])
def test_softmax_rows_vs_oracle(backend, oracle, cols):
    rng = binding.SeededRng(cols)
    x = rng.normal((37, cols), 0.0, 3.0)
    s = backend.softmax(dev(x)).cpu().numpy()
    ref = oracle.softmax(x)
    assert np.abs(s - ref).max() <= 1e-5          # the reference's own softmax tolerance
    dy = rng.normal((37, cols))
    assert np.abs(backend.softmax_backward(dev(ref), dev(dy)).cpu().numpy() - oracle.softmax_backward(ref, dy)).max() <= 1e-5


def test_colsum_and_elementwise_vs_oracle(backend, oracle):
    rng = binding.SeededRng(4)
    x = rng.normal((1000, 77))
    assert np.abs(backend.colsum(dev(x)).cpu().numpy() - oracle.colsum(x)).max() <= 1e-3
    # the 16-byte-load form (column count a multiple of 4, tall input), the GPT configuration's bias gradients among
    # them; ragged slab and column-block tails; against float64 sums (the float order differs from the oracle's)
    for rows, cols in ((16384, 384), (16384, 1536), (4099, 260), (513, 4), (70000, 132)):
        y = rng.normal((rows, cols))
        got = backend.colsum(dev(y))
        assert torch.equal(got, backend.colsum(dev(y))), "two runs differ"
        ref64 = y.astype(np.float64).sum(0)
        assert np.abs(got.cpu().numpy() - ref64).max() <= 2e-5 * np.abs(y).sum(0).max(), (rows, cols)
    v = rng.normal((12345,), 0.0, 2.0)
    assert np.abs(backend.gelu(dev(v)).cpu().numpy() - oracle.gelu(v)).max() <= 1e-5
    dy = rng.normal((12345,))
    assert np.abs(backend.gelu_backward(dev(v), dev(dy)).cpu().numpy() - oracle.gelu_backward(v, dy)).max() <= 1e-5
    # lengths that take the vector kernels: a ragged last round of a small grid, and more vectors than one round of
    # the capped grid covers
    for n in (4 * 100003, 4 * 5000003):
        v, dy = rng.normal((n,), 0.0, 2.0), rng.normal((n,))
        assert np.abs(backend.gelu(dev(v)).cpu().numpy() - oracle.gelu(v)).max() <= 1e-5, n
        assert np.abs(backend.gelu_backward(dev(v), dev(dy)).cpu().numpy() - oracle.gelu_backward(v, dy)).max() <= 1e-5, n


@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("rows,in_f,out_f", [(4096, 1536, 384), (4096, 2048, 2048), (300, 100, 40), (257, 77, 33), (64, 8, 4)])
def test_linear_backward_through_gelu(backend, oracle, prec, rows, in_f, out_f):
    """The second Linear of FeedForward: dx comes back as the gradient of the GELU's pre-activation.  Reference
    composition: dH = dY . W (MatMulBackward), then GeluBackward on the pre-activation (grad_fn.cpp:169-204)."""
    rng = binding.SeededRng(rows + in_f)
    pre, w, dy = rng.normal((rows, in_f)), rng.normal((out_f, in_f), 0.0, 0.2), rng.normal((rows, out_f))
    h = oracle.gelu(pre)
    d_pre, dw, db = backend.linear_backward(dev(h), dev(w), dev(dy), precision=prec, gelu_preact=dev(pre))
    want = oracle.gelu_backward(pre, oracle.matmul_2d_threads(dy, w))
    assert_close(d_pre.cpu().numpy(), want, prec, "gradient of the pre-activation")
    plain_dx, dw2, db2 = backend.linear_backward(dev(h), dev(w), dev(dy), precision=prec)
    assert torch.equal(dw, dw2) and torch.equal(db, db2)
    # the same two kernels issued separately give the same bits
    two_step = backend.gelu_backward(dev(pre), plain_dx)
    assert torch.equal(d_pre, two_step)
    backend.check_device_status()


@pytest.mark.parametrize("prec", PRECS)
def test_linear_golden_forward_backward(backend, nn_gold, prec):
    lin = gc.nn_inputs()["linear"]
    x, w, b, dy = (dev(lin[k]) for k in ("x", "w", "b", "dy"))
    y = backend.linear_forward(x, w, b, precision=prec)
    assert tuple(y.shape) == nn_gold["linear.y"].shape
    assert_close(y.cpu().numpy(), nn_gold["linear.y"], prec, "Linear y")
    yg, pre = backend.linear_forward(x, w, b, gelu=True, want_preact=True, precision=prec)
    assert_close(pre.cpu().numpy(), nn_gold["linear_gelu.preact"], prec, "pre-activation")
    assert np.abs(yg.cpu().numpy() - nn_gold["linear_gelu.y"]).max() <= 1.2 * TOL_REL[prec] * np.abs(nn_gold["linear_gelu.preact"]).max() + 1e-4
    dx, dw, db = backend.linear_backward(x, w, dy, precision=prec)
    assert_close(dx.cpu().numpy(), nn_gold["linear.dx"], prec, "dX")
    assert_close(dw.cpu().numpy(), nn_gold["linear.dw"], prec, "dW")
    assert np.abs(db.cpu().numpy() - nn_gold["linear.db"]).max() <= 1e-4
    # with GELU: the upstream gradient first passes GeluBackward on the pre-activation
    dpre = backend.gelu_backward(pre, dy)
    dx2, dw2, db2 = backend.linear_backward(x, w, dpre, precision=prec)
    assert_close(dx2.cpu().numpy(), nn_gold["linear_gelu.dx"], prec, "dX through GELU")
    assert_close(dw2.cpu().numpy(), nn_gold["linear_gelu.dw"], prec, "dW through GELU")
    assert_close(db2.cpu().numpy(), nn_gold["linear_gelu.db"], prec, "db through GELU")
    backend.check_device_status()


@pytest.mark.parametrize("prec", PRECS)
def test_config3_mlp_linear_full_size(backend, oracle, prec):
    """X [4096,768] ~ N(0,1), W [3072,768] ~ N(0,0.02), bias zeros, dY ~ N(0,1); seed 42, order X, W, dY."""
    rng = binding.SeededRng(42)
    x, w, dy = rng.normal((4096, 768)), rng.normal((3072, 768), 0.0, 0.02), rng.normal((4096, 3072))
    bias = np.zeros(3072, dtype=np.float32)
    tx, tw, tb, tdy = dev(x), dev(w), dev(bias), dev(dy)
    y, pre = backend.linear_forward(tx, tw, tb, gelu=True, want_preact=True, precision=prec)
    pre_ref = oracle.matmul_2d_threads(x, w.T)
    assert_close(pre.cpu().numpy(), pre_ref, prec, "X.W^T")
    assert np.abs(y.cpu().numpy() - oracle.gelu(pre_ref)).max() <= 1.2 * TOL_REL[prec] * np.abs(pre_ref).max() + 1e-4
    dx, dw, db = backend.linear_backward(tx, tw, tdy, precision=prec)
    assert_close(dx.cpu().numpy(), oracle.matmul_2d_threads(dy, w), prec, "dX = dY.W")
    pick = np.linspace(0, 3071, 48).astype(int)
    dw_ref = oracle.matmul_f64(np.ascontiguousarray(dy.T), x, rows=pick.tolist())[pick]
    assert_close(dw.cpu().numpy()[pick], dw_ref, prec, "dW = dY^T.X (sampled rows, float64 arbiter)")
    assert rel_err(db.cpu().numpy(), dy.astype(np.float64).sum(axis=0)) <= 1e-5
    backend.check_device_status()


@pytest.mark.parametrize("prec", PRECS)
def test_scaled_dot_golden_contiguous_and_head_views(backend, nn_gold, prec):
    s = gc.nn_inputs()["scaled_dot"]
    B, H, T, d = s["B"], s["H"], s["T"], s["d"]
    q, k, v = (dev(s[n]) for n in "qkv")
    o, p = backend.scaled_dot(q.view(B, H, T, d), k.view(B, H, T, d), v.view(B, H, T, d), precision=prec)
    assert rel_err(o.cpu().numpy(), nn_gold["scaled_dot_contig.o"]) <= ATTN_TOL[prec]
    heads = lambda t: t.view(B, T, H, d).transpose(1, 2)     # strides [T*E, d, E, 1]
    o2, _ = backend.scaled_dot(heads(q), heads(k), heads(v), precision=prec)
    assert rel_err(o2.cpu().numpy(), nn_gold["scaled_dot_views.o"]) <= ATTN_TOL[prec]
    assert np.abs(p.sum(dim=-1).cpu().numpy() - 1).max() <= 1e-5


@pytest.mark.parametrize("prec", PRECS)
def test_config2_attention_full_size(backend, oracle, prec):
    """Q,K,V [16,12,256,64] ~ N(0,1) from seed 42 in the order Q, K, V."""
    rng = binding.SeededRng(42)
    shape = (16, 12, 256, 64)
    q, k, v = rng.normal(shape), rng.normal(shape), rng.normal(shape)
    o, p = backend.scaled_dot(dev(q), dev(k), dev(v), precision=prec)
    backend.check_device_status()
    sub = slice(0, 3)      # the oracle is single-threaded: check three batch entries (36 heads) in full
    o_ref, p_ref = oracle.scaled_dot(q[sub], k[sub], v[sub])
    assert rel_err(o[sub].cpu().numpy(), o_ref) <= ATTN_TOL[prec]
    # probabilities: softmax amplifies a logit error e to ~e*p; logits are O(10) here
    assert np.abs(p[sub].cpu().numpy() - p_ref).max() <= (3e-2 if prec == "tf32" else 2e-5)
    # batch-sharded evaluation (what each GPU does) equals the unsharded one
    o_hi, _ = backend.scaled_dot(dev(q[8:]), dev(k[8:]), dev(v[8:]), precision=prec)
    assert torch.equal(o_hi, o[8:])


@pytest.mark.parametrize("shape", [(2, 3, 100, 32), (1, 2, 200, 64), (2, 2, 256, 32), (1, 2, 64, 64), (1, 1, 4, 32),
                                   (1, 1, 260, 64), (1, 2, 128, 48)])
@pytest.mark.parametrize("prec", PRECS)
def test_scaled_dot_shapes_fused_and_unfused(backend, oracle, shape, prec):
    """Key counts up to 256 with head size 32 or 64 take the fused kernel in TF32 mode (ragged T included); the last two
    shapes and the 3xTF32 mode take the two-GEMM path.  Both must agree with the reference composition."""
    rng = binding.SeededRng(shape[2] * 7 + shape[3])
    q, k, v = rng.normal(shape), rng.normal(shape), rng.normal(shape)
    tq, tk, tv = dev(q), dev(k), dev(v)
    n0 = backend.launches
    o, p = backend.scaled_dot(tq, tk, tv, precision=prec)
    launches = backend.launches - n0
    backend.check_device_status()
    fused = prec == "tf32" and shape[2] <= 256 and shape[2] % 4 == 0 and shape[3] in (32, 64)
    assert launches == (1 if fused else 3), launches      # 3xTF32 splits hi / lo inside the GEMM kernel: no packing passes
    o_ref, p_ref = oracle.scaled_dot(q, k, v)
    assert rel_err(o.cpu().numpy(), o_ref) <= ATTN_TOL[prec]
    assert np.abs(p.cpu().numpy() - p_ref).max() <= (3e-2 if prec == "tf32" else 2e-5)
    assert np.abs(p.sum(dim=-1).cpu().numpy() - 1).max() <= 1e-5
    # head views of a [B, T, H*d] projection, as MultiHeadAttention builds them
    B, H, T, d = shape
    heads = lambda x: torch.from_numpy(np.ascontiguousarray(np.swapaxes(x, 1, 2))).cuda().view(B, T, H * d).view(B, T, H, d).transpose(1, 2)
    o2, _ = backend.scaled_dot(heads(q), heads(k), heads(v), precision=prec)
    assert rel_err(o2.cpu().numpy(), o_ref) <= ATTN_TOL[prec]
