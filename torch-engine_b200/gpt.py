"""The GPT training-step caller of the matmul path (reference src/benchmarks/gpt_benchmark_gpu.cpp:230-236 without
the optimizer): GPT::forward (src/nn/gpt.cpp:26-86) -> crossEntropyLoss::forward_batched
(src/loss/CrossEntropyLoss.cpp:47-127) -> backward.

The step is an explicit schedule of C-ABI calls over buffers allocated once per configuration: nothing in it is a
torch operator, torch only owns the memory.  Per pre-LN block (src/nn/transformer_block.cpp:15-35):

  forward   LayerNorm -> te_b200_mha_forward (the three projections as one product against the gathered [3E,E]
            weight, attention on head views, out projection, the block's residual input added in the last GEMM's
            epilogue) -> LayerNorm -> Linear+GELU (pre-activation kept) ->
            Linear with the second residual in its epilogue;
  backward  te_b200_linear_backward_ex twice (the first hands back the gradient of the GELU's pre-activation and,
            from the same pass, its column sums = the bias gradient of the first FeedForward Linear),
            te_b200_layernorm_backward_ex (adds the gradient that bypasses the LayerNorm over the residual branch, and
            sums its result over the rows = the bias gradient of the Linear that fed the residual stream there),
            te_b200_mha_backward, te_b200_layernorm_backward_ex.

Every parameter is used once per step, so each gradient is written once, straight into its slice of one flat
gradient vector in GPT::parameters() order (src/nn/gpt.cpp:88-113): no accumulation pass and no concatenation.
Token embedding with the positional sum (src/nn/embedding.cpp:18-60, src/nn/gpt.cpp:30-69), the mean cross-entropy with
its gradient and the embedding gradient are backend kernels as well.
"""
import ctypes as C

import torch

from . import lib as L
from .ops import _prec

_POS_TABLES = {}


def positional_table(seq_len, d_model, device):
    """PositionalEmbedding::init_positional_embeddings (src/nn/positional_embedding.cpp:18-36): the exponent uses
    the column index itself for even and odd columns alike.  Built once per (length, width, device), as the reference
    builds it in the constructor."""
    key = (seq_len, d_model, str(device))
    if key not in _POS_TABLES:
        _POS_TABLES[key] = _positional_table(seq_len, d_model).to(device)
    return _POS_TABLES[key]


def _positional_table(seq_len, d_model):
    pos = torch.arange(seq_len, dtype=torch.float32).unsqueeze(1)
    i = torch.arange(d_model, dtype=torch.float32).unsqueeze(0)
    div = torch.exp(torch.log(torch.tensor(10000.0)) * (2.0 * (i / 2.0)) / float(d_model))
    ang = pos / div
    return torch.where((torch.arange(d_model) % 2 == 0).unsqueeze(0), torch.sin(ang), torch.cos(ang))


def param_shapes(vocab, E, n_layers, ff):
    """Shapes of GPT::parameters() in order: token table, per block {ln1 g/b, q/k/v/out Linear w/b, ln2 g/b, ffn w1/b1/w2/b2},
    final LayerNorm g/b, head w/b."""
    shapes = [(vocab, E)]
    for _ in range(n_layers):
        shapes += [(E,), (E,)] + [(E, E), (E,)] * 4 + [(E,), (E,)] + [(ff, E), (ff,), (E, ff), (E,)]
    shapes += [(E,), (E,), (vocab, E), (vocab,)]
    return shapes


def _numel(shape):
    n = 1
    for d in shape:
        n *= d
    return n


class GptStep:
    """Buffers and call schedule of one forward + loss + backward for a fixed (model, batch, sequence) configuration."""

    def __init__(self, be, vocab, E, H, n_layers, ff, B, T, prec="tf32"):
        self.be, self.cfg = be, (vocab, E, H, n_layers, ff, B, T, prec)
        self.prec = _prec(prec)
        dev = be.torch_device
        f32 = dict(dtype=torch.float32, device=dev)
        self.shapes = param_shapes(vocab, E, n_layers, ff)
        self.offsets, off = [], 0
        for s in self.shapes:
            self.offsets.append(off)
            off += _numel(s)
        self.n_params = off
        self.grads = torch.empty(off, **f32)
        bte = lambda: torch.empty(B, T, E, **f32)
        self.x = [bte() for _ in range(n_layers + 1)]          # block inputs; x[0] is the embedding output
        self.layers = []
        for _ in range(n_layers):
            # qkv: the three projections as column blocks of one buffer (one GEMM against the gathered weights wqkv)
            self.layers.append(dict(h1=bte(), qkv=torch.empty(B, T, 3 * E, **f32), wqkv=torch.empty(3 * E * E + 3 * E, **f32),
                                    attn=bte(), y1=bte(), h2=bte(), p=torch.empty(B, H, T, T, **f32),
                                    pre=torch.empty(B, T, ff, **f32), f=torch.empty(B, T, ff, **f32)))
        self.hf = bte()
        self.logits = torch.empty(B, T, vocab, **f32)
        self.dlogits = torch.empty(B, T, vocab, **f32)
        self.loss = torch.empty(1, **f32)
        # backward scratch
        self.dxa, self.dxb, self.dh = bte(), bte(), bte()
        self.dqkv, self.dattn = torch.empty(B, T, 3 * E, **f32), bte()
        self.dwqkv = torch.empty(3 * E * E + 3 * E, **f32)
        self.dpre = torch.empty(B, T, ff, **f32)
        self.pos = positional_table(T, E, dev)

    def _p(self, flat, i):
        return flat.data_ptr() + 4 * self.offsets[i]

    def _g(self, i):
        return self.grads.data_ptr() + 4 * self.offsets[i]

    def run(self, flat_params, tokens, targets):
        """Returns (loss [1], logits [B,T,vocab], flat gradient); all three are buffers of this object."""
        vocab, E, H, n_layers, ff, B, T, _ = self.cfg
        be, lib, ctx, prec = self.be, self.be._lib, self.be._ctx, self.prec
        st = be._stream()
        rows = B * T
        ptr = lambda t: C.c_void_p(t.data_ptr())
        P = lambda i: C.c_void_p(self._p(flat_params, i))
        G = lambda i: C.c_void_p(self._g(i))
        eps = 1e-5
        assert flat_params.numel() == self.n_params and flat_params.is_contiguous()
        assert tokens.shape == (B, T) and tokens.dtype == torch.int64 and targets.dtype == torch.int64
        tokens, targets = tokens.contiguous(), targets.contiguous()

        # ---- forward ----------------------------------------------------------------------------------------
        L.check(lib.te_b200_embedding_forward(ctx, P(0), ptr(tokens), ptr(self.pos), ptr(self.x[0]), rows, T, E, vocab, st))
        for l, a in enumerate(self.layers):
            i = 1 + 16 * l          # ln1 g,b | wq,bq,wk,bk,wv,bv,wo,bo | ln2 g,b | w1,c1,w2,c2
            L.check(lib.te_b200_layernorm_forward(ctx, ptr(self.x[l]), P(i), P(i + 1), ptr(a["h1"]), rows, E, eps, st))
            m = L.MhaDesc()
            m.B, m.T, m.E, m.H = B, T, E, H
            m.x = a["h1"].data_ptr()
            for n, j in zip(("wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo"), range(i + 2, i + 10)):
                setattr(m, n, self._p(flat_params, j))
            q = a["qkv"].data_ptr()
            m.q, m.k, m.v, m.ld_qkv, m.wqkv = q, q + 4 * E, q + 8 * E, 3 * E, a["wqkv"].data_ptr()
            m.p, m.attn = a["p"].data_ptr(), a["attn"].data_ptr()
            m.y, m.residual, m.precision = a["y1"].data_ptr(), self.x[l].data_ptr(), prec
            L.check(lib.te_b200_mha_forward(ctx, C.byref(m), st))                       # y1 = x + MHA(LN1(x))
            L.check(lib.te_b200_layernorm_forward(ctx, ptr(a["y1"]), P(i + 10), P(i + 11), ptr(a["h2"]), rows, E, eps, st))
            L.check(lib.te_b200_linear_forward(ctx, ptr(a["h2"]), P(i + 12), P(i + 13), ptr(a["f"]), ptr(a["pre"]), rows, E, ff,
                                               1, prec, st))                           # f = gelu(h2.W1^T + c1)
            d = L.GemmDesc()                                                            # x' = y1 + f.W2^T + c2
            d.M, d.N, d.K = rows, E, ff
            d.a, d.lda, d.a_major = a["f"].data_ptr(), ff, L.TE_ROW_MAJOR
            d.b, d.ldb, d.b_major = self._p(flat_params, i + 14), ff, L.TE_COL_MAJOR
            d.c, d.ldc = self.x[l + 1].data_ptr(), E
            d.batch_outer = d.batch_inner = 1
            d.alpha, d.bias, d.epilogue = 1.0, self._p(flat_params, i + 15), L.TE_EPI_BIAS
            d.residual, d.precision = a["y1"].data_ptr(), prec
            L.check(lib.te_b200_gemm_f32(ctx, C.byref(d), st))
        i = 1 + 16 * n_layers      # final ln g,b | head w,b
        L.check(lib.te_b200_layernorm_forward(ctx, ptr(self.x[n_layers]), P(i), P(i + 1), ptr(self.hf), rows, E, eps, st))
        L.check(lib.te_b200_linear_forward(ctx, ptr(self.hf), P(i + 2), P(i + 3), ptr(self.logits), None, rows, E, vocab, 0, prec, st))
        L.check(lib.te_b200_cross_entropy(ctx, ptr(self.logits), ptr(targets), ptr(self.loss), ptr(self.dlogits), 1.0, rows,
                                          vocab, st))                                  # mean over B*T, gradient in the same pass

        # ---- backward ---------------------------------------------------------------------------------------
        L.check(lib.te_b200_linear_backward_ex(ctx, ptr(self.hf), None, P(i + 2), ptr(self.dlogits), ptr(self.dh), None, None,
                                               G(i + 2), G(i + 3), 0, rows, E, vocab, prec, st))
        # the gradient of x[L] is also the upstream gradient of the last block's second FeedForward Linear: its bias
        # gradient (column sums) comes out of this pass
        c2_last = G(1 + 16 * (n_layers - 1) + 15) if n_layers > 0 else None
        L.check(lib.te_b200_layernorm_backward_ex(ctx, ptr(self.x[n_layers]), P(i), ptr(self.dh), ptr(self.dxa), None, G(i),
                                                  G(i + 1), c2_last, rows, E, eps, st))
        for l in range(n_layers - 1, -1, -1):      # dxa holds the gradient of x[l+1]
            a = self.layers[l]
            i = 1 + 16 * l
            # FeedForward: dW2 (its bias gradient came with dxa), d_pre with GeluBackward and the column sums of d_pre
            # (= bias gradient of the first Linear) in one pass, then the first Linear's dX and dW
            L.check(lib.te_b200_linear_backward_ex(ctx, ptr(a["f"]), ptr(a["pre"]), P(i + 14), ptr(self.dxa), ptr(self.dpre), None,
                                                   G(i + 13), G(i + 14), None, 0, rows, ff, E, prec, st))
            L.check(lib.te_b200_linear_backward_ex(ctx, ptr(a["h2"]), None, P(i + 12), ptr(self.dpre), ptr(self.dh), None, None,
                                                   G(i + 12), None, 0, rows, E, ff, prec, st))
            # gradient of y1 = dxa + LayerNorm backward; its column sums are the output projection's bias gradient
            L.check(lib.te_b200_layernorm_backward_ex(ctx, ptr(a["y1"]), P(i + 10), ptr(self.dh), ptr(self.dxb), ptr(self.dxa),
                                                      G(i + 10), G(i + 11), G(i + 9), rows, E, eps, st))
            m = L.MhaBwdDesc()
            m.B, m.T, m.E, m.H = B, T, E, H
            m.x = a["h1"].data_ptr()
            m.wq, m.wk, m.wv, m.wo = (self._p(flat_params, j) for j in (i + 2, i + 4, i + 6, i + 8))
            q, dq = a["qkv"].data_ptr(), self.dqkv.data_ptr()
            m.q, m.k, m.v, m.ld_qkv, m.wqkv = q, q + 4 * E, q + 8 * E, 3 * E, a["wqkv"].data_ptr()
            m.p, m.attn = a["p"].data_ptr(), a["attn"].data_ptr()
            m.dy, m.dx, m.dx_residual = self.dxb.data_ptr(), self.dh.data_ptr(), None
            for n, j in zip(("dwq", "dbq", "dwk", "dbk", "dwv", "dbv", "dwo"), range(i + 2, i + 9)):
                setattr(m, n, self._g(j))
            m.dbo = None                                                               # came with the LayerNorm backward above
            m.dq, m.dk, m.dv, m.dattn, m.dwqkv = dq, dq + 4 * E, dq + 8 * E, self.dattn.data_ptr(), self.dwqkv.data_ptr()
            m.accumulate, m.precision = 0, prec
            L.check(lib.te_b200_mha_backward(ctx, C.byref(m), st))                     # gradient of LN1's output
            # gradient of x[l]; for l > 0 its column sums are the bias gradient of block l-1's second FeedForward Linear
            c2_prev = G(1 + 16 * (l - 1) + 15) if l > 0 else None
            L.check(lib.te_b200_layernorm_backward_ex(ctx, ptr(self.x[l]), P(i), ptr(self.dh), ptr(self.dxa), ptr(self.dxb), G(i),
                                                      G(i + 1), c2_prev, rows, E, eps, st))
        L.check(lib.te_b200_embedding_backward(ctx, ptr(tokens), ptr(self.dxa), G(0), rows, E, vocab, st))
        return self.loss, self.logits, self.grads


def gpt_step(be, flat_params, tokens, targets, vocab, E, H, n_layers, ff, prec="tf32", grad_sync=None):
    """One forward + backward.  Returns (loss, logits, flat gradient in parameter order).  grad_sync, if given, is
    called with (flat gradient, token rows of this rank) before returning: the data-parallel exchange
    (sharding.all_reduce_batch_mean_).  The buffers belong to a GptStep kept on the backend per configuration, so
    the results of one call are overwritten by the next call with the same configuration."""
    B, T = tokens.shape
    key = (vocab, E, H, n_layers, ff, B, T, prec)
    plans = be.__dict__.setdefault("_gpt_steps", {})
    if key not in plans:
        plans[key] = GptStep(be, vocab, E, H, n_layers, ff, B, T, prec)
    loss, logits, grads = plans[key].run(flat_params, tokens, targets)
    if grad_sync is not None:
        grad_sync(grads, tokens.numel())
    return loss.reshape(()), logits, grads
