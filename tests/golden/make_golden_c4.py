"""Runs the reference's own CPU GPT step at the size of benchmark config 4 (6 layers, d_model 384, 6 heads, context
256, vocab 65, batch 64, ffDim 4*384) ONCE and stores a small fixture: the loss, and for the logits and every
parameter gradient its L2 norm, absolute maximum and 64 sampled entries (gpt_c4.npz), and, in gpt_c4_full.npz, the
complete gradient tensors of the token embedding, the final LayerNorm, the head and of block 2 (its two LayerNorms, the
query and output projections, every bias, and the first 32 rows of the second FeedForward weight).  Takes 10-20 minutes
of one host core.

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
    # complete tensors: index in GPT::parameters() order -> (first element, count) inside that tensor
    E, ff, nl = c["E"], c["ff"], c["L"]
    blk = 1 + 16 * 2                       # block 2: ln1 g,b | wq,bq,wk,bk,wv,bv,wo,bo | ln2 g,b | w1,c1,w2,c2
    tail = 1 + 16 * nl                     # final ln g,b | head w,b
    whole = [0, blk, blk + 1, blk + 2, blk + 3, blk + 5, blk + 7, blk + 8, blk + 9, blk + 10, blk + 11, blk + 13, blk + 15,
             tail, tail + 1, tail + 2, tail + 3]
    pick = {t: (0, layout[t][0]) for t in whole}
    pick[blk + 14] = (0, 32 * ff)          # the first 32 of the E rows of w2 [E, ff]
    starts = np.concatenate([[0], np.cumsum([sz for sz, _ in layout])])
    full = {"tensors": np.array(sorted(pick), dtype=np.int64)}
    for t in sorted(pick):
        first, count = pick[t]
        full["first_%d" % t] = np.int64(first)
        full["grad_%d" % t] = grads[starts[t] + first:starts[t] + first + count].copy()
    np.savez_compressed(os.path.join(HERE, "gpt_c4_full.npz"), **full)
    print("written", os.path.join(HERE, "gpt_c4_full.npz"), os.path.getsize(os.path.join(HERE, "gpt_c4_full.npz")), "bytes")


if __name__ == "__main__":
    main()
