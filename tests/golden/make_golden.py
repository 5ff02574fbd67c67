"""Generates the golden fixtures in this directory from the reference's own CPU implementation.

Run where the reference sources are available (it builds oracle/_ref/libref_cpu.so from them in place):

    python tests/golden/make_golden.py

Outputs (small, committed):
    reference_known_answers.json  known-answer vectors transcribed from the reference's own tests
    matmul_cases.npz              Tensor::matmul on seeded inputs: dense, transposed views, batched,
                                  broadcast, attention head views
    c1_512_samples.npz            config "512^3": sampled entries + float64 checksum of the reference result
    nn_cases.npz                  Linear / FeedForward / ScaledDot / MultiHeadAttention forward+backward
    gpt_tiny.npz                  one forward+backward of a 2-layer GPT: loss, logits, all gradients
Inputs are regenerated from the seed by the tests (oracle.binding.SeededRng), so only outputs are stored,
except where an input is cheap to keep.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import binding  # noqa: E402
from tests.golden_cases import (MATMUL_CASES, build_matmul_inputs, gpt_tiny_inputs, GPT_TINY,  # noqa: E402
                                nn_inputs)


def known_answers():
    """Transcribed by reading the reference tests as text (file:line in each entry)."""
    return {
        "matmul_2x3_3x4": {"source": "src/tests/cuda_matmul_tensor_test.cpp:14-35",
                           "a": [1, 2, 3, 4, 5, 6], "a_shape": [2, 3],
                           "b": list(range(1, 13)), "b_shape": [3, 4],
                           "expected": [38, 44, 50, 56, 83, 98, 113, 128], "tol": 1e-5},
        "matmul_transposed_a": {"source": "src/tests/cuda_matmul_tensor_test.cpp:37-53",
                                "a": [1, 2, 3, 4, 5, 6], "a_shape": [3, 2], "a_transpose": [0, 1],
                                "b": list(range(1, 13)), "b_shape": [3, 4],
                                "expected": [61, 70, 79, 88, 76, 88, 100, 112], "tol": 1e-5},
        "matmul_batched_3d": {"source": "src/tests/cuda_matmul_tensor_test.cpp:55-99",
                              "a": list(range(1, 13)), "a_shape": [2, 2, 3],
                              "b": list(range(1, 25)), "b_shape": [2, 3, 4],
                              "expected": [38, 44, 50, 56, 83, 98, 113, 128, 416, 440, 464, 488, 569, 602, 635, 668],
                              "tol": 1e-4},
        "matmul_f32_2x3_3x2": {"source": "src/tests/tensor_test.cpp:537-569",
                               "a": [1, 2, 3, 4, 5, 6], "a_shape": [2, 3],
                               "b": [1, 2, 3, 4, 5, 6], "b_shape": [3, 2],
                               "expected": [22, 28, 49, 64], "tol": 0.0},
        "matmul_i32_2x2": {"source": "src/tests/tensor_test.cpp:571-595",
                           "a": [1, 2, 3, 4], "b": [5, 6, 7, 8], "expected": [19, 22, 43, 50]},
        "throws": [
            {"source": "src/tests/tensor_test.cpp:597-602", "a_shape": [2, 3], "b_shape": [2, 2],
             "message": "Inner dimensions must match for matmul"},
            {"source": "src/tests/tensor_test.cpp:683-691", "a_shape": [3, 2, 3], "b_shape": [2, 3, 4],
             "message": "Batch dimensions are not broadcastable"},
            {"source": "src/tests/tensor_test.cpp:718-725", "a_shape": [2, 2, 3], "b_shape": [3, 3, 4],
             "message": "Batch dimensions are not broadcastable"},
        ],
        "shapes": [
            {"source": "src/tests/tensor_test.cpp:693-716", "a_shape": [1, 2, 3], "b_shape": [3, 3, 4],
             "out_shape": [3, 2, 4]},
        ],
        "ragged_mkn": {"source": "src/tests/cuda_test.cpp:486-496 (M, K, N); seed 42 uniform(-1,1); tol 1e-4*K abs",
                       "cases": [[33, 128, 128], [129, 128, 128], [128, 128, 132], [128, 136, 128], [129, 256, 512],
                                 [256, 128, 512], [128, 256, 512]]},
        "gelu_inputs": {"source": "src/tests/cuda_gelu_tensor_test.cpp:31-34, tol 1e-4 (:55)",
                        "x": [0.0, 1.0, -1.0, 2.0, -2.0, 0.5, -0.5, 3.0, -3.0, 0.1, -0.1, 1.5], "tol": 1e-4},
        "softmax_rows": {"source": "src/tests/cuda_softmax_tensor_test.cpp:16-65, tol 1e-5 (:34)",
                         "row": [1.0, 2.0, 3.0, 4.0], "tol": 1e-5},
    }


def main():
    binding.build()
    ref = binding.Reference()
    with open(os.path.join(HERE, "reference_known_answers.json"), "w") as f:
        json.dump(known_answers(), f, indent=1)

    # ---- Tensor::matmul cases --------------------------------------------------------------
    out = {}
    for name, case in MATMUL_CASES.items():
        a, va, b, vb = build_matmul_inputs(case)
        out[name] = ref.matmul(a, va, b, vb)
    np.savez_compressed(os.path.join(HERE, "matmul_cases.npz"), **out)

    # ---- config 1: 512^3, seed 42 uniform(-1,1), A then B ----------------------------------
    rng = binding.SeededRng(42)
    a = rng.uniform((512, 512))
    b = rng.uniform((512, 512))
    c = ref.matmul(a, binding.ref_view(a.shape), b, binding.ref_view(b.shape))
    idx = np.random.default_rng(7).integers(0, 512, size=(256, 2))
    np.savez_compressed(os.path.join(HERE, "c1_512_samples.npz"), idx=idx, values=c[idx[:, 0], idx[:, 1]],
                        checksum=np.float64(c.astype(np.float64).sum()),
                        abs_checksum=np.float64(np.abs(c.astype(np.float64)).sum()))

    # ---- nn-level cases ----------------------------------------------------------------------
    nn = nn_inputs()
    res = {}
    lin = nn["linear"]
    for tag, gelu in (("linear", False), ("linear_gelu", True)):
        r = ref.linear(lin["x"], lin["w"], lin["b"], gelu=gelu, dy=lin["dy"])
        for k, v in r.items():
            res[f"{tag}.{k}"] = v
    f = nn["ffn"]
    r = ref.ffn(f["x"], f["w1"], f["b1"], f["w2"], f["b2"], dy=f["dy"])
    for k, v in r.items():
        res[f"ffn.{k}"] = v
    s = nn["scaled_dot"]
    B, H, T, d = s["B"], s["H"], s["T"], s["d"]
    # contiguous [B,H,T,d] operands
    vq = binding.ref_view((B, H, T, d))
    r = ref.scaled_dot(s["q"], vq, s["k"], vq, s["v"], vq, (B, H, T, d), d_o=s["d_o"])
    for k, v in r.items():
        res[f"scaled_dot_contig.{k}"] = v
    # the MultiHeadAttention head views: base [B,T,E] -> view [B,T,H,d] -> transpose_view(1,2)
    vm = binding.ref_view((B, T, H * d), view=(B, T, H, d), transpose=(1, 2))
    r = ref.scaled_dot(s["q"], vm, s["k"], vm, s["v"], vm, (B, H, T, d), d_o=s["d_o"])
    for k, v in r.items():
        res[f"scaled_dot_views.{k}"] = v
    m = nn["mha"]
    r = ref.mha(m["x"], m["params"], m["H"], dy=m["dy"])
    res["mha.y"], res["mha.dx"] = r["y"], r["dx"]
    for i, g in enumerate(r["dparams"]):
        res[f"mha.dparam{i}"] = g
    np.savez_compressed(os.path.join(HERE, "nn_cases.npz"), **res)

    # ---- tiny GPT step -----------------------------------------------------------------------
    cfg = GPT_TINY
    layout = ref.gpt_param_layout(cfg["vocab"], cfg["max_seq"], cfg["E"], cfg["H"], cfg["L"], cfg["ff"])
    flat, tokens, targets = gpt_tiny_inputs(layout)
    loss, logits, grads = ref.gpt_step(cfg["vocab"], cfg["max_seq"], cfg["E"], cfg["H"], cfg["L"], cfg["ff"], flat,
                                       tokens, targets, want_grads=True, want_logits=True)
    np.savez_compressed(os.path.join(HERE, "gpt_tiny.npz"), loss=np.float32(loss), logits=logits, grads=grads,
                        layout=np.array(layout, dtype=np.int64))
    print("golden fixtures written to", HERE)
    for fn in sorted(os.listdir(HERE)):
        print("  %-34s %8d bytes" % (fn, os.path.getsize(os.path.join(HERE, fn))))


if __name__ == "__main__":
    main()
