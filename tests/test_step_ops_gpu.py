"""GPU parity of the GPT step's kernels around the matmuls -- LayerNorm, token embedding (+ positional table) and the
mean cross-entropy, forward and backward -- through the C ABI, against the reference's own CPU results
(tests/golden/step_ops.npz) and the oracle on larger seeded inputs; plus the attention backward against the gradients the
reference's autograd produced for ScaledDot.

Tolerances (max|x - ref| / max|ref| unless stated): LayerNorm forward and dx 1e-5 (the row mean and variance are summed
in a different order and 1/sqrt is multiplied instead of dividing by sqrt); dgamma / dbeta 2e-5 (column sums over all
rows, added in block order instead of row order); cross-entropy loss 1e-6 absolute, its gradient 1e-6; embedding forward
and backward bit for bit (same additions in the same order)."""
import os

import numpy as np
import pytest
import torch

from oracle import binding
from tests import golden_cases as gc
from tests.gpu_util import rel_err
from torch_engine_b200 import lib as L

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(GOLD, "step_ops.npz"))


@pytest.mark.parametrize("tag", ["ln48", "ln50", "ln384"])
def test_layernorm_against_reference_golden(backend, gold, tag):
    c = gc.step_op_inputs()["ln"][tag]
    y = backend.layernorm(dev(c["x"]), dev(c["gamma"]), dev(c["beta"]))
    assert rel_err(y.cpu().numpy(), gold[f"{tag}.y"]) <= 1e-5
    dx, dg, db = backend.layernorm_backward(dev(c["x"]), dev(c["gamma"]), dev(c["dy"]))
    assert rel_err(dx.cpu().numpy(), gold[f"{tag}.dx"]) <= 1e-5
    assert rel_err(dg.cpu().numpy(), gold[f"{tag}.dgamma"]) <= 2e-5
    assert rel_err(db.cpu().numpy(), gold[f"{tag}.dbeta"]) <= 2e-5


@pytest.mark.parametrize("rows,cols", [(16384, 384), (4097, 768), (1000, 1024), (777, 130), (33, 1), (5, 1023)])
def test_layernorm_against_oracle_sizes(backend, oracle, rows, cols):
    """The GPT configuration's [16384, 384] activations, rows that do not fill the last block, the longest supported
    row, and row lengths that take the scalar path (not a multiple of 4)."""
    rng = binding.SeededRng(rows + cols)
    x, dy = rng.normal((rows, cols), 0.1, 1.3), rng.normal((rows, cols))
    gamma, beta = rng.normal((cols,), 1.0, 0.2), rng.normal((cols,), 0.0, 0.3)
    y = backend.layernorm(dev(x), dev(gamma), dev(beta))
    assert rel_err(y.cpu().numpy(), oracle.layernorm(x, gamma, beta)) <= 1e-5
    dx, dg, db = backend.layernorm_backward(dev(x), dev(gamma), dev(dy))
    dx2, dg2, db2 = backend.layernorm_backward(dev(x), dev(gamma), dev(dy))
    assert torch.equal(dx, dx2) and torch.equal(dg, dg2) and torch.equal(db, db2), "two runs differ"
    dx_r, dg_r, db_r = oracle.layernorm_backward(x, gamma, dy)
    assert rel_err(dx.cpu().numpy(), dx_r) <= 1e-5
    # column sums over `rows` terms: float rounding of the sum grows with sqrt(rows); compare against float64 sums too
    x64 = x.astype(np.float64)
    xh = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5)
    assert rel_err(dg.cpu().numpy(), (dy * xh).sum(0)) <= 2e-5
    assert rel_err(db.cpu().numpy(), dy.astype(np.float64).sum(0)) <= 2e-5
    assert rel_err(dg.cpu().numpy(), dg_r) <= 1e-4 and rel_err(db.cpu().numpy(), db_r) <= 1e-4
    backend.check_device_status()


def test_layernorm_rejects_long_rows(backend):
    with pytest.raises(L.BackendError) as e:
        backend.layernorm(torch.zeros(2, 1025, device="cuda"), torch.ones(1025, device="cuda"), torch.zeros(1025, device="cuda"))
    assert "not supported" in str(e.value)


def test_cross_entropy_against_reference_golden_and_oracle(backend, oracle, gold):
    ce = gc.step_op_inputs()["ce"]
    loss, grad = backend.cross_entropy(dev(ce["logits"]), dev(ce["targets"]))
    assert abs(float(loss) - float(gold["ce.loss"])) <= 1e-6
    assert rel_err(grad.cpu().numpy(), gold["ce.dlogits"]) <= 1e-6
    # the GPT configuration: 16384 rows of 65 logits
    rng = binding.SeededRng(5)
    logits, targets = rng.normal((64, 256, 65), 0.0, 3.0), rng.tokens((64, 256), 65)
    loss, grad = backend.cross_entropy(dev(logits), dev(targets))
    loss2, grad2 = backend.cross_entropy(dev(logits), dev(targets))
    assert torch.equal(loss, loss2) and torch.equal(grad, grad2), "two runs differ"
    assert abs(float(loss) - float(oracle.cross_entropy(logits, targets))) <= 2e-6
    assert rel_err(grad.cpu().numpy(), oracle.cross_entropy_backward(logits, targets)) <= 1e-6
    # a large vocabulary (strided loops over the row) and an upstream gradient other than 1
    logits, targets = rng.normal((37, 5000), 0.0, 2.0), rng.tokens((37,), 5000)
    loss, grad = backend.cross_entropy(dev(logits), dev(targets), upstream=0.5)
    assert abs(float(loss) - float(oracle.cross_entropy(logits, targets))) <= 2e-6
    assert rel_err(grad.cpu().numpy(), oracle.cross_entropy_backward(logits, targets, upstream=0.5)) <= 1e-6
    backend.check_device_status()


def test_embedding_against_reference_golden_and_oracle(backend, oracle, gold):
    e = gc.step_op_inputs()["emb"]
    out = backend.embedding(dev(e["table"]), dev(e["tokens"]))
    assert np.array_equal(out.cpu().numpy(), gold["emb.out"])
    dtable = backend.embedding_backward(dev(e["tokens"]), dev(e["dout"]), 65)
    assert np.array_equal(dtable.cpu().numpy(), gold["emb.dtable"])
    with_pos = backend.embedding(dev(e["table"]), dev(e["tokens"]), pos=dev(e["pos"]))
    assert np.array_equal(with_pos.cpu().numpy(), oracle.embedding(e["table"], e["tokens"], pos=e["pos"]))
    # the GPT configuration (vocab 65, 16384 tokens, E 384) and an odd width that takes the scalar path
    rng = binding.SeededRng(9)
    for vocab, shape, dim in ((65, (64, 256), 384), (300, (7, 33), 50)):
        table, tokens = rng.normal((vocab, dim)), rng.tokens(shape, vocab)
        pos, dout = rng.normal((shape[1], dim)), rng.normal(shape + (dim,))
        out = backend.embedding(dev(table), dev(tokens), pos=dev(pos))
        assert np.array_equal(out.cpu().numpy(), oracle.embedding(table, tokens, pos=pos))
        dtable = backend.embedding_backward(dev(tokens), dev(dout), vocab)
        assert np.array_equal(dtable.cpu().numpy(), oracle.embedding_backward(tokens, dout, vocab))
    backend.check_device_status()


def test_embedding_index_out_of_range_is_reported(backend):
    table = torch.ones(10, 8, device="cuda")
    out = backend.embedding(table, torch.tensor([[1, 10, 3]], device="cuda"))
    torch.cuda.synchronize()
    with pytest.raises(L.BackendError) as e:
        backend.check_device_status()
    assert str(e.value) == "Embedding index out of range"          # the text of src/nn/embedding.cpp:54
    assert float(out[0, 1].abs().sum()) == 0.0 and float(out[0, 0].sum()) == 8.0
    backend.check_device_status()                                   # the status word was cleared


@pytest.mark.parametrize("prec", ["tf32", "3xtf32"])
def test_attention_backward_against_reference_autograd(backend, gold, prec):
    """dQ, dK, dV of ScaledDot as the reference's own autograd computed them on the CPU: [1, 2, 64, 32] (the fused
    kernel in TF32 mode, the GEMM sequence in 3xTF32 mode) and the [2, 3, 16, 8] case of nn_cases.npz (GEMM sequence)."""
    a = gc.step_op_inputs()["att"]
    q, k, v, d_o = (dev(a[n]) for n in ("q", "k", "v", "d_o"))
    o, p = backend.scaled_dot(q, k, v, precision=prec)
    got = backend.scaled_dot_backward(q, k, v, p, d_o, o=o, precision=prec)
    tol = 1e-2 if prec == "tf32" else 2e-5
    for name, g in zip(("dq", "dk", "dv"), got):
        assert rel_err(g.cpu().numpy(), gold[f"att.{name}"]) <= tol, name
    nn_gold = np.load(os.path.join(GOLD, "nn_cases.npz"))
    s = gc.nn_inputs()["scaled_dot"]
    shape = (s["B"], s["H"], s["T"], s["d"])
    q, k, v = (dev(s[n]).view(shape) for n in "qkv")
    o, p = backend.scaled_dot(q, k, v, precision=prec)
    got = backend.scaled_dot_backward(q, k, v, p, dev(s["d_o"]), o=o, precision=prec)
    for name, g in zip(("dq", "dk", "dv"), got):
        assert rel_err(g.cpu().numpy(), nn_gold[f"scaled_dot_contig.{name}"].reshape(shape)) <= tol, name
    backend.check_device_status()
