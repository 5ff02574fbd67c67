"""Seeded random shapes through the C ABI against float64: the forms whose limits are easy to get wrong -- thin
FP32-accurate products (both layouts of the right operand) around their row / column / alignment limits, the fused attention kernels around their
sequence-length and head-size limits (dense operands and MultiHeadAttention head views), and MultiHeadAttention with
its three input projections as one product against three.

Tolerances: 1e-5 (FP32-accurate mode, max-norm relative); attention in TF32 mode 2e-2 on O, 3e-2 absolute on P and
1e-2 on the gradients (three to five chained TF32 products per value); the two MultiHeadAttention forms agree to 1e-4
(same products, sums in another order)."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(x, y):
    return float((x.double() - y).abs().max() / (y.abs().max() + 1e-9))


def test_thin_products_around_the_limits(backend):
    rnd = random.Random(7)
    g = torch.Generator(device="cuda").manual_seed(7)
    for _ in range(48):
        M = rnd.randint(1, 18)                                        # 17 and 18 rows take the tensor cores
        K = rnd.choice([256, 257, 300, 511, 1000, 4097, 8192])
        N = rnd.choice([512, 516, 1024, 2052, 4096, 1000, 1002])     # 1002: not a multiple of 4, tensor cores again
        pad_a, pad_b = rnd.choice([0, 4, 7]), rnd.choice([0, 4, 8])
        a = (torch.rand(M, K + pad_a, device="cuda", generator=g) * 2 - 1)[:, :K]
        b = (torch.rand(K, N + pad_b, device="cuda", generator=g) * 2 - 1)[:, :N]
        c = backend.matmul(a, b, precision="3xtf32")
        assert _rel(c, a.double() @ b.double()) <= 1e-5, (M, K, N, pad_a, pad_b)
    backend.check_device_status()


def test_thin_linear_layout_around_the_limits(backend):
    """X[M,K] . W[N,K]^T with M <= 16 in FP32-accurate mode (lanes along k, W staged by TMA when its rows sit on
    16-byte boundaries, by plain loads otherwise): through Linear with bias / GELU and through matmul on W's
    transposed view."""
    rnd = random.Random(17)
    g = torch.Generator(device="cuda").manual_seed(17)
    for it in range(48):
        M = rnd.randint(1, 18)                                        # 17 and 18 rows take the tensor cores
        K = rnd.choice([256, 257, 300, 511, 1000, 1024, 2049, 4097, 8192])
        N = rnd.choice([512, 513, 1000, 1024, 2052, 3001, 4096])
        pad_x, pad_w = rnd.choice([0, 4, 7]), rnd.choice([0, 4, 3])   # a pad of 3 or an odd K takes W off 16-byte rows
        x = (torch.rand(M, K + pad_x, device="cuda", generator=g) * 2 - 1)[:, :K]
        w = (torch.rand(N, K + pad_w, device="cuda", generator=g) * 2 - 1)[:, :K]
        ref = x.double() @ w.double().t()
        c = backend.matmul(x, w.t(), precision="3xtf32")
        assert _rel(c, ref) <= 1e-5, (M, K, N, pad_x, pad_w)
        if it % 3 == 0:
            bias = torch.rand(N, device="cuda", generator=g)
            gelu = it % 2 == 0
            y = backend.linear_forward(x.contiguous(), w.contiguous(), bias, gelu=gelu, precision="3xtf32")
            want = ref + bias.double()
            if gelu:
                want = torch.nn.functional.gelu(want, approximate="tanh")
            assert _rel(y, want) <= 1e-5, (M, K, N, gelu)
    backend.check_device_status()


def test_attention_around_the_limits(backend):
    rnd = random.Random(11)
    g = torch.Generator(device="cuda").manual_seed(11)
    for _ in range(32):
        B, H = rnd.randint(1, 5), rnd.randint(1, 7)
        T, d = rnd.choice([4, 64, 128, 132, 200, 252, 256]), rnd.choice([32, 64])
        q, k, v, d_o = (torch.randn(B, H, T, d, device="cuda", generator=g) for _ in range(4))
        if rnd.random() < 0.5:      # head views of [B, T, H*d] memory, as MultiHeadAttention produces them
            q, k, v, d_o = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (q, k, v, d_o))
        o, p = backend.scaled_dot(q, k, v)
        s = (q.double() @ k.double().transpose(-1, -2)) / (d ** 0.5)
        p_ref = torch.softmax(s, -1)
        assert float((o.double() - p_ref @ v.double()).abs().max()) <= 2e-2, (B, H, T, d)
        assert float((p.double() - p_ref).abs().max()) <= 3e-2, (B, H, T, d)
        dq, dk, dv = backend.scaled_dot_backward(q, k, v, p, d_o, o=o)
        P, dO = p.double(), d_o.double()
        dP = dO @ v.double().transpose(-1, -2)
        dS = P * (dP - (P * dP).sum(-1, keepdim=True)) / (d ** 0.5)
        for got, want in ((dq, dS @ k.double()), (dk, dS.transpose(-1, -2) @ q.double()), (dv, P.transpose(-1, -2) @ dO)):
            assert _rel(got, want) <= 1e-2, (B, H, T, d)
    backend.check_device_status()


def test_multi_head_attention_projection_forms_on_random_sizes(backend):
    rnd = random.Random(13)
    g = torch.Generator(device="cuda").manual_seed(13)
    for _ in range(10):
        B, T = rnd.randint(1, 4), rnd.choice([16, 100, 128, 256])
        H, hd = rnd.choice([1, 2, 4, 6]), rnd.choice([32, 64])
        E = H * hd
        x, dy = (torch.randn(B, T, E, device="cuda", generator=g) for _ in range(2))
        params = []
        for _ in range(4):
            params += [torch.randn(E, E, device="cuda", generator=g) / (E ** 0.5), torch.randn(E, device="cuda", generator=g)]
        y1, s1 = backend.mha_forward(x, params, H, one_projection_gemm=True)
        y3, s3 = backend.mha_forward(x, params, H, one_projection_gemm=False)
        assert torch.equal(y1, y3), (B, T, H, hd)
        dx1, g1 = backend.mha_backward(s1, dy)
        dx3, g3 = backend.mha_backward(s3, dy)
        assert _rel(dx1, dx3.double()) <= 1e-4, (B, T, H, hd)
        for a, b in zip(g1, g3):
            assert _rel(a, b.double()) <= 1e-4, (B, T, H, hd)
    backend.check_device_status()
