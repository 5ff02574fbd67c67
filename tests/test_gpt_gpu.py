"""The GPT training-step caller with every matmul on the CUDA backend, against the reference's own CPU step.
Tiny configuration: full logits and all gradients from tests/golden/gpt_tiny.npz.  Benchmark configuration 4
(6 layers, d_model 384, 6 heads, context 256, vocab 65, batch 64): loss, norms and sampled entries of every gradient from
tests/golden/gpt_c4.npz, and the COMPLETE gradient tensors of the token embedding, the final LayerNorm, the head and block 2
from tests/golden/gpt_c4_full.npz (one reference CPU run of 12 minutes, tests/golden/make_golden_c4.py)."""
import os

import numpy as np
import pytest
import torch

from tests import golden_cases as gc

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")

# A training step chains ~150 GEMMs through LayerNorms and softmaxes.  In TF32 mode the per-GEMM 7e-4 input rounding
# accumulates; in 3xTF32 mode the step stays at FP32 accuracy.  Gradient errors are measured per tensor in max-norm
# relative to that tensor's largest gradient entry.
LOSS_TOL = {"tf32": 2e-3, "3xtf32": 1e-4}
GRAD_TOL = {"tf32": 3e-2, "3xtf32": 2e-4}


def _floor(global_absmax):
    """Some gradients are zero in exact arithmetic (the key-projection bias: softmax ignores a constant added to
    every key score) and hold only rounding noise in any implementation; their scale is floored at 1e-3 of the
    largest gradient entry of the whole model."""
    return 1e-3 * global_absmax


def _per_tensor_rel(got, want, layout):
    worst, where, off = 0.0, -1, 0
    floor = _floor(float(np.abs(want).max()))
    for t, (size, _) in enumerate(layout):
        g, w = got[off:off + size], want[off:off + size]
        e = float(np.abs(g - w).max() / max(float(np.abs(w).max()), floor))
        if e > worst:
            worst, where = e, t
        off += size
    return worst, where


@pytest.mark.parametrize("prec", ["tf32", "3xtf32"])
def test_tiny_gpt_step_matches_reference(backend, prec):
    from torch_engine_b200 import gpt
    g = np.load(os.path.join(GOLD, "gpt_tiny.npz"))
    cfg = gc.GPT_TINY
    layout = [tuple(x) for x in g["layout"].tolist()]
    flat, tokens, targets = gc.gpt_tiny_inputs(layout)
    loss, logits, grads = gpt.gpt_step(backend, torch.from_numpy(flat).cuda(), torch.from_numpy(tokens).cuda(),
                                       torch.from_numpy(targets).cuda(), cfg["vocab"], cfg["E"], cfg["H"], cfg["L"],
                                       cfg["ff"], prec)
    backend.check_device_status()
    assert abs(float(loss) - float(g["loss"])) <= LOSS_TOL[prec]
    assert np.abs(logits.cpu().numpy() - g["logits"]).max() <= GRAD_TOL[prec] * np.abs(g["logits"]).max()
    worst, where = _per_tensor_rel(grads.cpu().numpy(), g["grads"], layout)
    assert worst <= GRAD_TOL[prec], f"gradient tensor {where} (GPT::parameters() order) off by {worst:.3e}"


@pytest.mark.parametrize("prec", ["tf32", "3xtf32"])
def test_config4_gpt_step_matches_reference(backend, prec):
    from torch_engine_b200 import gpt
    path = os.path.join(GOLD, "gpt_c4.npz")
    assert os.path.exists(path), "run tests/golden/make_golden_c4.py where the reference sources are available"
    g = np.load(path)
    cfg = gc.GPT_C4
    layout = [tuple(x) for x in g["layout"].tolist()]
    flat, tokens, targets = gc.gpt_c4_inputs(layout)
    n0 = backend.launches
    loss, logits, grads = gpt.gpt_step(backend, torch.from_numpy(flat).cuda(), torch.from_numpy(tokens).cuda(),
                                       torch.from_numpy(targets).cuda(), cfg["vocab"], cfg["E"], cfg["H"], cfg["L"],
                                       cfg["ff"], prec)
    backend.check_device_status()
    assert backend.launches - n0 >= 147, "49 forward and 98 backward GEMMs are expected on the backend"
    assert abs(float(loss) - float(g["loss"])) <= LOSS_TOL[prec]
    lg = logits.cpu().numpy().ravel()
    assert np.abs(lg[g["logits_idx"]] - g["logits_val"]).max() <= GRAD_TOL[prec] * np.abs(g["logits_val"]).max()
    gr = grads.cpu().numpy()
    off = 0
    floor = _floor(float(g["grad_absmax"].max()))
    for t, (size, _) in enumerate(layout):
        seg = gr[off:off + size]
        idx = g["grad_idx"][64 * t:64 * (t + 1)]
        want = g["grad_val"][64 * t:64 * (t + 1)]
        scale = max(float(g["grad_absmax"][t]), floor)
        assert np.abs(gr[idx] - want).max() <= GRAD_TOL[prec] * scale, f"gradient tensor {t}"
        norm = np.linalg.norm(seg.astype(np.float64))
        assert abs(norm - g["grad_norm"][t]) <= GRAD_TOL[prec] * max(g["grad_norm"][t], floor * np.sqrt(size)), f"gradient norm {t}"
        off += size
    # complete tensors: embedding, block 2 (LayerNorms, query / output projections, every bias, 32 rows of the second
    # FeedForward weight), final LayerNorm and head
    full = np.load(os.path.join(GOLD, "gpt_c4_full.npz"))
    starts = np.concatenate([[0], np.cumsum([size for size, _ in layout])])
    for t in full["tensors"].tolist():
        want = full["grad_%d" % t]
        first = int(full["first_%d" % t])
        got = gr[starts[t] + first:starts[t] + first + want.size]
        scale = max(float(g["grad_absmax"][t]), floor)
        assert np.abs(got - want).max() <= GRAD_TOL[prec] * scale, f"complete gradient tensor {t}"
