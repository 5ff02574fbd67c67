"""The GPT training-step caller of the matmul path (reference src/benchmarks/gpt_benchmark_gpu.cpp:230-236 without
the optimizer): GPT::forward (src/nn/gpt.cpp:26-86) -> crossEntropyLoss::forward_batched
(src/loss/CrossEntropyLoss.cpp:47-127) -> backward.

Every matmul of the step runs on this backend through the C ABI:
  * Linear forward / backward (src/nn/linear.cpp:14-23, src/core/grad_fn.cpp:93-139) as the fused calls
    te_b200_linear_forward / te_b200_linear_backward, the FeedForward GELU (src/nn/ffn.cpp:12-16) in the epilogue;
  * ScaledDot::forward (src/nn/scaledot.cpp:8-27) on the head views of MultiHeadAttention::forward
    (src/nn/multi_head_attention.cpp:19-42, strides [T*E, hd, E, 1], no copies, no mask), and its backward
    (MatMulBackward x2, DivBackward, SoftmaxBackward) as te_b200_attention_backward.
The step's kernels around the matmuls run on the backend as well: token embedding with the positional sum
(src/nn/embedding.cpp:18-60, src/nn/gpt.cpp:30-69), pre-LN LayerNorm forward / backward (src/nn/layernorm.cpp:19-82,
src/core/grad_fn.cpp:405-538) and the mean cross-entropy with its gradient (src/loss/CrossEntropyLoss.cpp:47-127,
src/core/grad_fn.cpp:271-346).  Residual adds, the head merge copy and gradient accumulation stay stock torch ops.
Parameters come in GPT::parameters() order (src/nn/gpt.cpp:88-113).
"""

import torch


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, be, prec, gelu):
        if gelu:
            y, pre = be.linear_forward(x, w, b, gelu=True, want_preact=True, precision=prec)
        else:
            y, pre = be.linear_forward(x, w, b, precision=prec), None
        ctx.save_for_backward(x, w, pre if pre is not None else x.new_empty(0))
        ctx.be, ctx.prec, ctx.gelu = be, prec, gelu
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, pre = ctx.saved_tensors
        be = ctx.be
        dy = dy.contiguous()
        if ctx.gelu:
            dy = be.gelu_backward(pre, dy)       # GeluBackward consumes the pre-activation (grad_fn.cpp:169-204)
        dx, dw, db = be.linear_backward(x, w, dy, precision=ctx.prec)
        return dx, dw, db, None, None, None


class _FeedForward(torch.autograd.Function):
    """FeedForward::forward (src/nn/ffn.cpp:12-16): Linear -> GELU -> Linear.  Forward keeps the pre-activation of the
    GELU; backward asks the second Linear for the gradient of that pre-activation directly (one call: dX product, then
    GeluBackward in place)."""
    @staticmethod
    def forward(ctx, x, w1, c1, w2, c2, be, prec):
        h, pre = be.linear_forward(x, w1, c1, gelu=True, want_preact=True, precision=prec)
        y = be.linear_forward(h, w2, c2, precision=prec)
        ctx.save_for_backward(x, w1, w2, h, pre)
        ctx.be, ctx.prec = be, prec
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w1, w2, h, pre = ctx.saved_tensors
        be, prec = ctx.be, ctx.prec
        dy = dy.contiguous()
        d_pre, dw2, dc2 = be.linear_backward(h, w2, dy, precision=prec, gelu_preact=pre)
        dx, dw1, dc1 = be.linear_backward(x, w1, d_pre, precision=prec)
        return dx, dw1, dc1, dw2, dc2, None, None


class _ScaledDot(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, be, prec):
        o, p = be.scaled_dot(q, k, v, precision=prec, head_major_out=False)     # written as [B,T,H,hd]: the merge is a view
        ctx.save_for_backward(q, k, v, p, o)
        ctx.be, ctx.prec = be, prec
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, p, o = ctx.saved_tensors
        dq, dk, dv = ctx.be.scaled_dot_backward(q, k, v, p, d_o, o=o, precision=ctx.prec, head_major_out=False)
        return dq, dk, dv, None, None


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g, b, be, eps):
        ctx.save_for_backward(x, g)
        ctx.be, ctx.eps = be, eps
        return be.layernorm(x, g, b, eps)

    @staticmethod
    def backward(ctx, dy):
        x, g = ctx.saved_tensors
        dx, dg, db = ctx.be.layernorm_backward(x, g, dy, ctx.eps)
        return dx, dg, db, None, None


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, tokens, pos, be):
        ctx.save_for_backward(tokens)
        ctx.be, ctx.vocab = be, table.shape[0]
        return be.embedding(table, tokens, pos)

    @staticmethod
    def backward(ctx, dout):
        (tokens,) = ctx.saved_tensors
        return ctx.be.embedding_backward(tokens, dout, ctx.vocab), None, None, None


class _CrossEntropy(torch.autograd.Function):
    """Loss and gradient come out of one pass over the logits; backward scales the stored gradient by the upstream
    value (1 for a plain loss.backward())."""
    @staticmethod
    def forward(ctx, logits, targets, be):
        loss, grad = be.cross_entropy(logits, targets)
        ctx.save_for_backward(grad)
        return loss.reshape(())

    @staticmethod
    def backward(ctx, upstream):
        (grad,) = ctx.saved_tensors
        return grad * upstream, None, None


def linear(be, x, w, b, prec, gelu=False):
    return _Linear.apply(x, w, b, be, prec, gelu)


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


def layer_norm(be, x, g, b, eps=1e-5):
    """LayerNorm::forward (src/nn/layernorm.cpp:19-77): biased variance, (x-mean)/sqrt(var+eps)*g+b."""
    return _LayerNorm.apply(x, g, b, be, eps)


def split_params(flat, vocab, E, n_layers, ff):
    """Views of a flat parameter vector in GPT::parameters() order, as leaf tensors that require grad."""
    shapes = [(vocab, E)]
    for _ in range(n_layers):
        shapes += [(E,), (E,)] + [(E, E), (E,)] * 4 + [(E,), (E,)] + [(ff, E), (ff,), (E, ff), (E,)]
    shapes += [(E,), (E,), (vocab, E), (vocab,)]
    out, off = [], 0
    for s in shapes:
        n = 1
        for d in s:
            n *= d
        out.append(flat[off:off + n].view(s).detach().requires_grad_(True))     # a leaf over the same storage, no copy
        off += n
    assert off == flat.numel(), (off, flat.numel())
    return out


def gpt_forward(be, params, tokens, E, H, n_layers, prec="tf32"):
    """Logits [B, T, vocab] of the pre-LN, unmasked GPT of the reference."""
    B, T = tokens.shape
    hd = E // H
    it = iter(params)
    emb = next(it)
    x = _Embedding.apply(emb, tokens, positional_table(T, E, tokens.device), be)   # gpt.cpp:29-68
    for _ in range(n_layers):                                                     # transformer_block.cpp:15-35
        g1, b1 = next(it), next(it)
        wq, bq, wk, bk, wv, bv, wo, bo = (next(it) for _ in range(8))
        g2, b2 = next(it), next(it)
        w1, c1, w2, c2 = (next(it) for _ in range(4))
        h = layer_norm(be, x, g1, b1)
        heads = lambda t: t.view(B, T, H, hd).transpose(1, 2)                      # zero-copy head views
        q, k, v = (heads(linear(be, h, w, b, prec)) for w, b in ((wq, bq), (wk, bk), (wv, bv)))
        o = _ScaledDot.apply(q, k, v, be, prec)                                    # [B,H,T,hd]
        o = o.transpose(1, 2).reshape(B, T, E)
        x = x + linear(be, o, wo, bo, prec)
        h = layer_norm(be, x, g2, b2)
        x = x + _FeedForward.apply(h, w1, c1, w2, c2, be, prec)
    gf, bf, wh, bh = (next(it) for _ in range(4))
    return linear(be, layer_norm(be, x, gf, bf), wh, bh, prec)


def gpt_step(be, flat_params, tokens, targets, vocab, E, H, n_layers, ff, prec="tf32", grad_sync=None):
    """One forward + backward.  Returns (loss, logits, flat gradient in parameter order).  grad_sync, if given, is
    called with (flat gradient, token rows of this rank) before returning: the data-parallel exchange
    (sharding.all_reduce_batch_mean_)."""
    params = split_params(flat_params, vocab, E, n_layers, ff)
    logits = gpt_forward(be, params, tokens, E, H, n_layers, prec)
    loss = _CrossEntropy.apply(logits, targets, be)                                             # mean over B*T
    loss.backward()
    grads = torch.cat([p.grad.reshape(-1) for p in params])
    if grad_sync is not None:
        grad_sync(grads, tokens.numel())
    return loss.detach(), logits.detach(), grads
