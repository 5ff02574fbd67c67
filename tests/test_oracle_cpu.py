"""The oracle (plain-C restatement) against everything that pins it: the reference's known-answer vectors,
the golden fixtures produced by the reference's own CPU code, and -- where the compiled reference is
present -- the reference itself, bit for bit."""
import json
import os

import numpy as np
import pytest

from oracle import binding
from tests import golden_cases as gc

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def known():
    with open(os.path.join(GOLD, "reference_known_answers.json")) as f:
        return json.load(f)


def _arr(vals, shape):
    return np.array(vals, dtype=np.float32).reshape(shape)


@pytest.mark.parametrize("name", ["matmul_2x3_3x4", "matmul_transposed_a", "matmul_batched_3d", "matmul_f32_2x3_3x2"])
def test_known_answer_matmul(oracle, known, name):
    k = known[name]
    a = _arr(k["a"], k["a_shape"])
    if "a_transpose" in k:
        a = np.swapaxes(a, *k["a_transpose"])
    c = oracle.matmul(a, _arr(k["b"], k["b_shape"]))
    assert np.abs(c.ravel() - np.array(k["expected"], dtype=np.float32)).max() <= k["tol"]


def test_known_throw_cases(oracle, known):
    for t in known["throws"]:
        a = np.zeros(t["a_shape"], dtype=np.float32)
        b = np.zeros(t["b_shape"], dtype=np.float32)
        with pytest.raises(binding.OracleError) as e:
            oracle.matmul(a, b)
        assert str(e.value) == t["message"], t["source"]
    with pytest.raises(binding.OracleError) as e:
        oracle.matmul(np.zeros(3, dtype=np.float32), np.zeros((3, 2), dtype=np.float32))
    assert str(e.value) == "Matmul requires tensors with at least 2 dimensions"


def test_known_shapes(oracle, known):
    for s in known["shapes"]:
        c = oracle.matmul(np.ones(s["a_shape"], dtype=np.float32), np.ones(s["b_shape"], dtype=np.float32))
        assert list(c.shape) == s["out_shape"]


def test_gelu_value_table(oracle, known):
    x = np.array(known["gelu_inputs"]["x"], dtype=np.float32)
    ref = 0.5 * x.astype(np.float64) * (1 + np.tanh(0.7978845608 * (x.astype(np.float64) + 0.044715 * x.astype(np.float64) ** 3)))
    assert np.abs(oracle.gelu(x) - ref).max() <= known["gelu_inputs"]["tol"]


def test_softmax_known_rows(oracle, known):
    row = np.array(known["softmax_rows"]["row"], dtype=np.float32)
    e = np.exp(row - row.max())
    expected = e / e.sum()
    x = np.tile(row, (3, 1))
    s = oracle.softmax(x)
    assert np.abs(s - expected).max() <= known["softmax_rows"]["tol"]
    assert np.abs(s.sum(axis=1) - 1).max() <= 1e-5
    # all-ones upstream gradient -> zero input gradient (src/tests/cuda_softmax_tensor_test.cpp, test 3)
    assert np.abs(oracle.softmax_backward(s, np.ones_like(s))).max() <= 1e-6


@pytest.mark.parametrize("name", sorted(gc.MATMUL_CASES))
def test_matmul_golden_bit_exact(oracle, name):
    gold = np.load(os.path.join(GOLD, "matmul_cases.npz"))
    a, va, b, vb = gc.build_matmul_inputs(gc.MATMUL_CASES[name])
    c = oracle.matmul(gc.apply_view_numpy(a, va), gc.apply_view_numpy(b, vb))
    assert c.shape == gold[name].shape
    assert np.array_equal(c, gold[name]), "oracle differs from the reference CPU result"


def test_c1_512_samples_bit_exact(oracle):
    g = np.load(os.path.join(GOLD, "c1_512_samples.npz"))
    rng = binding.SeededRng(42)
    a = rng.uniform((512, 512))
    b = rng.uniform((512, 512))
    c = oracle.matmul_2d_threads(a, b)
    assert np.array_equal(c[g["idx"][:, 0], g["idx"][:, 1]], g["values"])
    assert c.astype(np.float64).sum() == g["checksum"]
    assert np.abs(c.astype(np.float64)).sum() == g["abs_checksum"]
    assert np.array_equal(c, oracle.matmul(a, b)), "threaded row split changed a summation order"


def test_linear_golden(oracle):
    g = np.load(os.path.join(GOLD, "nn_cases.npz"))
    lin = gc.nn_inputs()["linear"]
    y, pre = oracle.linear(lin["x"], lin["w"], lin["b"], gelu=False)
    assert np.array_equal(y, g["linear.y"])
    yg, pre = oracle.linear(lin["x"], lin["w"], lin["b"], gelu=True)
    assert np.array_equal(pre, g["linear_gelu.preact"])
    assert np.array_equal(yg, g["linear_gelu.y"])
    # backward of y = x.w^T + b: dx = dy.w, dw^T = x^T.dy per batch then summed, db = column sums
    dy = lin["dy"]
    dx = oracle.matmul(dy, lin["w"])          # dY . (W^T)^T
    assert np.array_equal(dx, g["linear.dx"])
    db = oracle.colsum(dy.reshape(-1, dy.shape[-1]))
    assert np.allclose(db, g["linear.db"], rtol=0, atol=1e-5)
    dw = oracle.matmul(dy.reshape(-1, dy.shape[-1]).T, lin["x"].reshape(-1, lin["x"].shape[-1]))
    assert np.allclose(dw, g["linear.dw"], rtol=0, atol=1e-4)   # the reference sums per-batch products: order differs
    # gelu variant: upstream gradient first goes through GeluBackward
    dpre = oracle.gelu_backward(g["linear_gelu.preact"], dy)
    assert np.array_equal(oracle.matmul(dpre, lin["w"]), g["linear_gelu.dx"])


def test_scaled_dot_golden(oracle):
    g = np.load(os.path.join(GOLD, "nn_cases.npz"))
    s = gc.nn_inputs()["scaled_dot"]
    B, H, T, d = s["B"], s["H"], s["T"], s["d"]
    q, k, v = (s[n].reshape(B, H, T, d) for n in "qkv")
    o, p = oracle.scaled_dot(q, k, v)
    assert np.array_equal(o, g["scaled_dot_contig.o"])
    view = lambda t: np.swapaxes(t.reshape(B, T, H, d), 1, 2)
    o2, _ = oracle.scaled_dot(view(s["q"]), view(s["k"]), view(s["v"]))
    assert np.array_equal(o2, g["scaled_dot_views.o"])


@pytest.mark.skipif(not binding.Reference.available(), reason="compiled reference not present")
def test_oracle_equals_reference_random_views(oracle):
    ref = binding.Reference()
    rng = np.random.default_rng(3)
    for trial in range(12):
        M, K, N = (int(x) for x in rng.integers(1, 70, 3))
        a = rng.uniform(-1, 1, (K, M) if trial % 2 else (M, K)).astype(np.float32)
        b = rng.uniform(-1, 1, (N, K) if trial % 3 == 0 else (K, N)).astype(np.float32)
        va = binding.ref_view(a.shape, transpose=(0, 1) if trial % 2 else None)
        vb = binding.ref_view(b.shape, transpose=(0, 1) if trial % 3 == 0 else None)
        c_ref = ref.matmul(a, va, b, vb)
        c = oracle.matmul(gc.apply_view_numpy(a, va), gc.apply_view_numpy(b, vb))
        assert np.array_equal(c, c_ref)
    x = rng.normal(size=(5, 37)).astype(np.float32)
    r = ref.linear(x, rng.normal(size=(11, 37)).astype(np.float32) * 0 + 1, np.zeros(11, dtype=np.float32), gelu=True)
    assert np.array_equal(oracle.gelu(r["preact"]), r["y"])
    assert ref.matmul_i32([[1, 2], [3, 4]], [[5, 6], [7, 8]]).ravel().tolist() == [19, 22, 43, 50]


def test_seeded_rng_matches_reference_first_values():
    # std::mt19937(42) + uniform_real_distribution<float>(-1,1): the stream every reference benchmark draws from
    r = binding.SeededRng(42)
    v = r.uniform((4,))
    assert np.allclose(v, [-0.25091976, 0.593086, 0.9014286, -0.63313043], atol=1e-7)


def test_step_op_restatements_match_reference_golden(oracle):
    """LayerNorm, embedding and cross-entropy restatements against outputs of the compiled reference
    (tests/golden/step_ops.npz, written by tests/golden/make_golden_step_ops.py): bit for bit."""
    g = np.load(os.path.join(GOLD, "step_ops.npz"))
    inp = gc.step_op_inputs()
    for tag, c in inp["ln"].items():
        assert np.array_equal(oracle.layernorm(c["x"], c["gamma"], c["beta"]), g[f"{tag}.y"]), tag
        dx, dg, db = oracle.layernorm_backward(c["x"], c["gamma"], c["dy"])
        assert np.array_equal(dx, g[f"{tag}.dx"]) and np.array_equal(dg, g[f"{tag}.dgamma"]) and np.array_equal(db, g[f"{tag}.dbeta"]), tag
    ce = inp["ce"]
    assert oracle.cross_entropy(ce["logits"], ce["targets"]) == g["ce.loss"]
    assert np.array_equal(oracle.cross_entropy_backward(ce["logits"], ce["targets"]), g["ce.dlogits"])
    e = inp["emb"]
    assert np.array_equal(oracle.embedding(e["table"], e["tokens"]), g["emb.out"])
    assert np.array_equal(oracle.embedding_backward(e["tokens"], e["dout"], 65), g["emb.dtable"])
    assert np.array_equal(oracle.embedding(e["table"], e["tokens"], pos=e["pos"]),
                          (g["emb.out"] + e["pos"][None]).astype(np.float32))
    with pytest.raises(binding.OracleError):
        oracle.embedding(e["table"], np.array([[65]]))
    a = inp["att"]
    o, _ = oracle.scaled_dot(a["q"], a["k"], a["v"])
    assert np.array_equal(o, g["att.o"])
