"""Runs the reference's own CPU GPT step at the size of benchmark config 4 (6 layers, d_model 384, 6 heads, context
256, vocab 65, batch 64, ffDim 4*384) ONCE and stores a small fixture: the loss, and for the logits and every
parameter gradient its L2 norm, absolute maximum and 64 sampled entries.  Takes 10-20 minutes of one host core.

    python tests/golden/make_golden_c4.py          # needs the reference sources (builds oracle/_ref)
"""
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import binding  # noqa: E402
from tests.golden_cases import GPT_C4, gpt_c4_inputs  # noqa: E402


def main():
    binding.build()
    ref = binding.Reference()
    c = GPT_C4
    layout = ref.gpt_param_layout(c["vocab"], c["max_seq"], c["E"], c["H"], c["L"], c["ff"])
    flat, tokens, targets = gpt_c4_inputs(layout)
    t0 = time.time()
    loss, logits, grads = ref.gpt_step(c["vocab"], c["max_seq"], c["E"], c["H"], c["L"], c["ff"], flat, tokens, targets,
                                       want_grads=True, want_logits=True)
    print("reference CPU step: %.1f s, loss %.7f" % (time.time() - t0, loss))
    rng = np.random.default_rng(11)
    out = {"loss": np.float32(loss), "layout": np.array(layout, dtype=np.int64), "seconds": np.float64(time.time() - t0)}
    lidx = rng.integers(0, logits.size, 256)
    out["logits_idx"], out["logits_val"] = lidx, logits.ravel()[lidx]
    out["logits_norm"] = np.float64(np.linalg.norm(logits.astype(np.float64)))
    off = 0
    norms, maxes, idxs, vals = [], [], [], []
    for size, _rank in layout:
        g = grads[off:off + size]
        norms.append(np.linalg.norm(g.astype(np.float64)))
        maxes.append(np.abs(g).max())
        idx = rng.integers(0, size, 64)
        idxs.append(idx + off)
        vals.append(g[idx])
        off += size
    out.update(grad_norm=np.array(norms), grad_absmax=np.array(maxes), grad_idx=np.concatenate(idxs),
               grad_val=np.concatenate(vals))
    np.savez_compressed(os.path.join(HERE, "gpt_c4.npz"), **out)
    print("written", os.path.join(HERE, "gpt_c4.npz"))


if __name__ == "__main__":
    main()
