"""GPU parity of te_b200_attention_backward: the backward graph of ScaledDot::forward (MatMulBackward of P.V and of
Q.K^T, SoftmaxBackward, DivBackward; reference src/core/grad_fn.cpp:126-156, :569-665).

The arbiter here is those formulas evaluated in float64 on the same inputs and the same saved probabilities, so that
only the backward's own arithmetic is measured:  dV = P^T.dO,  dP = dO.V^T,  dZ = P o (dP - rowsum(P o dP)),
dS = dZ / sqrt(d),  dQ = dS.K,  dK = dS^T.Q.  Tolerances (max|x - ref| / max|ref| per output): 5e-3 in TF32 mode
(two chained TF32 products), 2e-5 in 3xTF32 mode.  End to end against the reference's own CPU autograd the same call
is covered by the GPT-step golden tests (tests/test_gpt_gpu.py), whose attention gradients all pass through it."""
import math

import numpy as np
import pytest
import torch

from tests.gpu_util import rel_err

pytestmark = pytest.mark.gpu
TOL = {"tf32": 5e-3, "3xtf32": 2e-5}


def _case(shape, seed, views=False):
    B, H, T, d = shape
    g = torch.Generator(device="cuda").manual_seed(seed)
    if views:     # head views of [B, T, H*d] projections, strides [T*E, d, E, 1] (multi_head_attention.cpp:27-33)
        mk = lambda: torch.randn(B, T, H * d, device="cuda", generator=g).view(B, T, H, d).transpose(1, 2)
    else:
        mk = lambda: torch.randn(B, H, T, d, device="cuda", generator=g)
    q, k, v, d_o = mk(), mk(), mk(), mk()
    s = (q.double() @ k.double().transpose(-1, -2)) / math.sqrt(d)
    p = torch.softmax(s, dim=-1).float().contiguous()
    o = (p.double() @ v.double()).float()
    if views:
        o = o.transpose(1, 2).contiguous().transpose(1, 2)
    return q, k, v, p, o, d_o


def _reference(q, k, v, p, d_o):
    q, k, v, p, d_o = (t.double() for t in (q, k, v, p, d_o))
    dv = p.transpose(-1, -2) @ d_o
    dp = d_o @ v.transpose(-1, -2)
    dz = p * (dp - (p * dp).sum(dim=-1, keepdim=True))
    ds = dz / math.sqrt(q.shape[-1])
    return ds @ k, ds.transpose(-1, -2) @ q, dv


def _check(got, ref, prec, what):
    for name, g, r in zip(("dq", "dk", "dv"), got, ref):
        e = rel_err(g.cpu().numpy(), r.cpu().numpy())
        assert e <= TOL[prec], f"{what} {name}: {e:.3e} > {TOL[prec]:.0e} ({prec})"


FUSED_SHAPES = [(2, 3, 256, 64), (2, 3, 128, 64), (1, 2, 64, 32), (2, 2, 200, 64), (1, 1, 4, 32), (3, 2, 256, 32),
                (1, 5, 132, 64)]


@pytest.mark.parametrize("views", [False, True], ids=["dense", "head_views"])
@pytest.mark.parametrize("shape", FUSED_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_fused_backward_tf32(backend, shape, views):
    q, k, v, p, o, d_o = _case(shape, 5 + shape[2], views)
    n0 = backend.launches
    got = backend.scaled_dot_backward(q, k, v, p, d_o, o=o, precision="tf32")
    assert backend.launches - n0 == 2, "the row-dot pre-pass and the fused kernel should have taken this problem"
    backend.check_device_status()
    _check(got, _reference(q, k, v, p, d_o), "tf32", f"fused {shape}")
    again = backend.scaled_dot_backward(q, k, v, p, d_o, o=o, precision="tf32")
    for a, b in zip(got, again):
        assert torch.equal(a, b), "two runs differ"


@pytest.mark.parametrize("prec", ["tf32", "3xtf32"])
@pytest.mark.parametrize("shape", [(2, 3, 256, 64), (1, 2, 300, 64), (2, 2, 100, 48), (1, 1, 5, 7)],
                         ids=lambda s: "x".join(map(str, s)))
def test_unfused_backward(backend, shape, prec):
    """3xTF32 mode, more than 256 keys, other head sizes, or no forward output at hand: four batched GEMMs and the
    softmax-backward kernel, with dP / dS in the context workspace."""
    q, k, v, p, o, d_o = _case(shape, 11 + shape[2])
    got = backend.scaled_dot_backward(q, k, v, p, d_o, o=None, precision=prec)
    backend.check_device_status()
    _check(got, _reference(q, k, v, p, d_o), prec, f"unfused {shape}")


def test_fused_and_unfused_agree_and_many_tiles(backend):
    """More (batch, head) tiles than SMs, so every CTA walks several tiles and the barrier phases wrap."""
    shape = (40, 6, 256, 64)
    q, k, v, p, o, d_o = _case(shape, 3, views=True)
    fused = backend.scaled_dot_backward(q, k, v, p, d_o, o=o, precision="tf32")
    plain = backend.scaled_dot_backward(q, k, v, p, d_o, o=None, precision="tf32")
    backend.check_device_status()
    ref = _reference(q, k, v, p, d_o)
    _check(fused, ref, "tf32", "fused 40x6")
    _check(plain, ref, "tf32", "unfused 40x6")


def test_key_block_tiles_are_reproducible(backend):
    """192 heads on 148 SMs run as one tile per (head, key block): the two tiles of a head add their parts of dQ onto
    memory the pre-pass zeroed.  Two addends per element, so the sum does not depend on their order: repeated calls
    agree bit for bit, whatever the output buffer held before, and the values match the reference."""
    shape = (16, 12, 256, 64)
    q, k, v, p, o, d_o = _case(shape, 5)
    first = backend.scaled_dot_backward(q, k, v, p, d_o, o=o, precision="tf32")
    junk = [torch.full_like(t, float("nan")) for t in first]       # the next outputs are likely to reuse such blocks
    del junk
    for _ in range(3):
        again = backend.scaled_dot_backward(q, k, v, p, d_o, o=o, precision="tf32")
        for a, b in zip(first, again):
            assert torch.equal(a, b)
    backend.check_device_status()
    _check(first, _reference(q, k, v, p, d_o), "tf32", "key-block tiles 16x12")


def test_outputs_written_in_token_major_layout(backend):
    """head_major_out=False: O, dQ, dK, dV land in [B,T,H,d] memory (the layout of the head-split views), values equal."""
    shape = (3, 4, 256, 64)
    q, k, v, p, o, d_o = _case(shape, 23, views=True)
    for prec in ("tf32", "3xtf32"):
        o1, p1 = backend.scaled_dot(q, k, v, precision=prec)
        o2, p2 = backend.scaled_dot(q, k, v, precision=prec, head_major_out=False)
        assert o2.transpose(1, 2).is_contiguous() and torch.equal(o1, o2) and torch.equal(p1, p2)
        g1 = backend.scaled_dot_backward(q, k, v, p, d_o, o=o, precision=prec)
        g2 = backend.scaled_dot_backward(q, k, v, p, d_o, o=o, precision=prec, head_major_out=False)
        for a, b in zip(g1, g2):
            assert b.transpose(1, 2).is_contiguous() and torch.equal(a, b)
    backend.check_device_status()


def test_backward_through_forward_outputs(backend):
    """The pair as a caller uses it: p and o come from this backend's own forward call."""
    shape = (4, 6, 256, 64)
    q, k, v, _, _, d_o = _case(shape, 17, views=True)
    o, p = backend.scaled_dot(q, k, v, precision="tf32")
    got = backend.scaled_dot_backward(q, k, v, p, d_o, o=o, precision="tf32")
    qd, kd, vd = (t.double().detach().requires_grad_(True) for t in (q, k, v))
    s = (qd @ kd.transpose(-1, -2)) / math.sqrt(shape[3])
    (torch.softmax(s, dim=-1) @ vd).backward(d_o.double())
    for name, g, r in zip(("dq", "dk", "dv"), got, (qd.grad, kd.grad, vd.grad)):
        assert rel_err(g.cpu().numpy(), r.cpu().numpy()) <= 1e-2, name     # forward's TF32 error in p adds to it
