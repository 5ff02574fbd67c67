"""Generates step_ops.npz from the reference's own CPU implementation: LayerNorm forward + backward, Embedding forward
+ backward, crossEntropyLoss::forward_batched + backward, and ScaledDot forward + backward on a [1, 2, 64, 32] case
(inside the limits of the fused attention kernels).  Inputs are regenerated from the seed by the tests
(tests/golden_cases.step_op_inputs); only the reference's outputs are stored.

    python tests/golden/make_golden_step_ops.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import binding  # noqa: E402
from tests.golden_cases import step_op_inputs  # noqa: E402


def main():
    binding.build()
    ref = binding.Reference()
    inp = step_op_inputs()
    res = {}
    for tag, c in inp["ln"].items():
        r = ref.layernorm(c["x"], c["gamma"], c["beta"], eps=1e-5, dy=c["dy"])
        for k, v in r.items():
            res[f"{tag}.{k}"] = v
    ce = inp["ce"]
    r = ref.cross_entropy(ce["logits"], ce["targets"])
    res["ce.loss"], res["ce.dlogits"] = r["loss"], r["dlogits"]
    e = inp["emb"]
    r = ref.embedding(e["table"], e["tokens"], dout=e["dout"])
    res["emb.out"], res["emb.dtable"] = r["out"], r["dtable"]
    a = inp["att"]
    shape = (a["B"], a["H"], a["T"], a["d"])
    v = binding.ref_view(shape)
    r = ref.scaled_dot(a["q"], v, a["k"], v, a["v"], v, shape, d_o=a["d_o"])
    for k, val in r.items():
        res[f"att.{k}"] = val
    out = os.path.join(HERE, "step_ops.npz")
    np.savez_compressed(out, **res)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
