"""Seeded input definitions shared by tests/golden/make_golden.py (which stores the reference's outputs)
and by the tests (which regenerate the same inputs and compare)."""
import numpy as np

from oracle import binding

# name -> recipe.  "a"/"b": (base shape, view shape or None, transpose or None, second transpose or None)
MATMUL_CASES = {
    "dense_64x48x80": dict(a=((64, 80), None, None, None), b=((80, 48), None, None, None), dist="uniform"),
    "ragged_33x20x17": dict(a=((33, 17), None, None, None), b=((17, 20), None, None, None), dist="uniform"),
    "a_transposed": dict(a=((40, 24), None, (0, 1), None), b=((40, 36), None, None, None), dist="uniform"),
    "b_transposed_linear_weight": dict(a=((12, 40), None, None, None), b=((28, 40), None, (1, 0), None), dist="normal"),
    "batched_3d": dict(a=((3, 10, 12), None, None, None), b=((3, 12, 9), None, None, None), dist="uniform"),
    "broadcast_1_vs_3": dict(a=((1, 6, 5), None, None, None), b=((3, 5, 7), None, None, None), dist="uniform"),
    "broadcast_2d_weight": dict(a=((4, 6, 8), None, None, None), b=((8, 10), None, None, None), dist="normal"),
    "broadcast_4d_mixed": dict(a=((2, 1, 5, 6), None, None, None), b=((3, 6, 4), None, None, None), dist="uniform"),
    # attention head views: [B,T,E] -> view [B,T,H,hd] -> transpose_view(1,2); K additionally transpose_view(2,3)
    "mha_qk_views": dict(a=((2, 16, 24), (2, 16, 3, 8), (1, 2), None), b=((2, 16, 24), (2, 16, 3, 8), (1, 2), (2, 3)),
                         dist="normal"),
    "mha_pv_views": dict(a=((2, 3, 16, 16), None, None, None), b=((2, 16, 24), (2, 16, 3, 8), (1, 2), None),
                         dist="normal"),
}


def _draw(rng, shape, dist):
    return rng.uniform(shape) if dist == "uniform" else rng.normal(shape)


def build_matmul_inputs(case, seed=42):
    """Returns (a_base, a_recipe, b_base, b_recipe): dense base arrays (A drawn first, then B) and RefView recipes."""
    rng = binding.SeededRng(seed)
    (sa, va, ta, ta2), (sb, vb, tb, tb2) = case["a"], case["b"]
    a = _draw(rng, sa, case["dist"])
    b = _draw(rng, sb, case["dist"])
    return a, binding.ref_view(sa, va, ta, ta2), b, binding.ref_view(sb, vb, tb, tb2)


def apply_view_numpy(base, recipe):
    """The numpy view equivalent to a RefView recipe (for the oracle and for torch via the same ops)."""
    t = base
    if recipe.view_ndim:
        t = t.reshape(tuple(recipe.view_shape[i] for i in range(recipe.view_ndim)))
    if recipe.t1 >= 0:
        t = np.swapaxes(t, recipe.t1, recipe.t2)
    if recipe.t3 >= 0:
        t = np.swapaxes(t, recipe.t3, recipe.t4)
    return t


def apply_view_torch(base, recipe):
    t = base
    if recipe.view_ndim:
        t = t.view(tuple(recipe.view_shape[i] for i in range(recipe.view_ndim)))
    if recipe.t1 >= 0:
        t = t.transpose(recipe.t1, recipe.t2)
    if recipe.t3 >= 0:
        t = t.transpose(recipe.t3, recipe.t4)
    return t


def nn_inputs(seed=42):
    rng = binding.SeededRng(seed)
    lin = dict(x=rng.normal((3, 7, 20)), w=rng.normal((28, 20), 0.0, 0.2), b=rng.normal((28,), 0.0, 0.5),
               dy=rng.normal((3, 7, 28)))
    E, FF = 16, 40
    ffn = dict(x=rng.normal((2, 9, E)), w1=rng.normal((FF, E), 0.0, 0.3), b1=rng.normal((FF,), 0.0, 0.1),
               w2=rng.normal((E, FF), 0.0, 0.3), b2=rng.normal((E,), 0.0, 0.1), dy=rng.normal((2, 9, E)))
    B, H, T, d = 2, 3, 16, 8
    sd = dict(B=B, H=H, T=T, d=d, q=rng.normal((B * H * T * d,)), k=rng.normal((B * H * T * d,)),
              v=rng.normal((B * H * T * d,)), d_o=rng.normal((B, H, T, d)))
    Em, Hm = 24, 3
    params = []
    for _ in range(4):
        params.append(rng.normal((Em, Em), 0.0, 0.2))
        params.append(rng.normal((Em,), 0.0, 0.1))
    mha = dict(x=rng.normal((2, 10, Em)), params=params, H=Hm, dy=rng.normal((2, 10, Em)))
    return dict(linear=lin, ffn=ffn, scaled_dot=sd, mha=mha)


def step_op_inputs(seed=7):
    """Inputs of the LayerNorm / embedding / cross-entropy cases (the GPT step's kernels around the matmuls) and of
    one attention backward case inside the fused kernel's limits."""
    rng = binding.SeededRng(seed)
    ln = {}
    for tag, shape in (("ln48", (5, 7, 48)), ("ln50", (4, 6, 50)), ("ln384", (2, 5, 384))):
        D = shape[-1]
        ln[tag] = dict(x=rng.normal(shape, 0.3, 1.7), gamma=rng.normal((D,), 1.0, 0.3), beta=rng.normal((D,), 0.0, 0.2),
                       dy=rng.normal(shape))
    ce = dict(logits=rng.normal((3, 9, 65), 0.0, 2.5), targets=rng.tokens((3, 9), 65))
    emb = dict(table=rng.normal((65, 24)), tokens=rng.tokens((4, 10), 65), dout=rng.normal((4, 10, 24)),
               pos=rng.normal((10, 24)))
    B, H, T, d = 1, 2, 64, 32
    att = dict(B=B, H=H, T=T, d=d, q=rng.normal((B, H, T, d)), k=rng.normal((B, H, T, d)), v=rng.normal((B, H, T, d)),
               d_o=rng.normal((B, H, T, d)))
    return dict(ln=ln, ce=ce, emb=emb, att=att)


GPT_TINY = dict(vocab=65, max_seq=16, E=32, H=4, L=2, ff=128, batch=3, seq=16)


def gpt_param_kinds(n_layers):
    """Kind of each tensor in GPT::parameters() order (reference src/nn/gpt.cpp:88-113,
    src/nn/transformer_block.cpp:37-62): 'w' weight matrix, 'b' bias, 'g' LayerNorm gain, 'beta' LayerNorm shift."""
    kinds = ["w"]                                   # token embedding; the positional embedding has no parameters
    for _ in range(n_layers):
        kinds += ["g", "beta"] + ["w", "b"] * 4 + ["g", "beta"] + ["w", "b"] * 2
    kinds += ["g", "beta", "w", "b"]
    return kinds


def gpt_init_params(layout, n_layers, rng):
    """Flat parameter vector: weights N(0, 0.02), LayerNorm gain 1 / shift 0, biases 0."""
    kinds = gpt_param_kinds(n_layers)
    assert len(kinds) == len(layout), (len(kinds), len(layout))
    parts = []
    for (size, _rank), kind in zip(layout, kinds):
        if kind == "w":
            parts.append(rng.normal((size,), 0.0, 0.02))
        elif kind == "g":
            parts.append(np.ones(size, dtype=np.float32))
        else:
            parts.append(np.zeros(size, dtype=np.float32))
    return np.concatenate(parts)


def gpt_tiny_inputs(layout, seed=42):
    cfg = GPT_TINY
    rng = binding.SeededRng(seed)
    flat = gpt_init_params(layout, cfg["L"], rng)
    tokens = rng.tokens((cfg["batch"], cfg["seq"]), cfg["vocab"])
    targets = rng.tokens((cfg["batch"], cfg["seq"]), cfg["vocab"])
    return flat, tokens, targets


# Benchmark config 4.  ffDim is 4*E, the ratio of every preset of the reference (scripts/run_benchmark_suite.py:22-26).
GPT_C4 = dict(vocab=65, max_seq=256, E=384, H=6, L=6, ff=1536, batch=64, seq=256)


def gpt_c4_inputs(layout, seed=42):
    cfg = GPT_C4
    rng = binding.SeededRng(seed)
    flat = gpt_init_params(layout, cfg["L"], rng)
    tokens = rng.tokens((cfg["batch"], cfg["seq"]), cfg["vocab"])
    targets = rng.tokens((cfg["batch"], cfg["seq"]), cfg["vocab"])
    return flat, tokens, targets
