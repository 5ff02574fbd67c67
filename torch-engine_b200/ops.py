"""Tensor-level host mirror of the reference operators on the matmul path.

Each method corresponds to one reference call and forwards to the C ABI (lib.py); torch tensors are
used only as device-memory holders (data_ptr, shape, stride) and for the current CUDA stream.

    Backend.matmul          Tensor::matmul                        (reference src/tensor/tensor.cpp:761-785)
    Backend.linear_forward  Linear::forward (+ FeedForward GELU)  (src/nn/linear.cpp:14-23, src/nn/ffn.cpp:12-16)
    Backend.linear_backward MatMulBackward/AddBackward/TransposeBackward of that graph (src/core/grad_fn.cpp:93-139)
    Backend.scaled_dot      ScaledDot::forward                    (src/nn/scaledot.cpp:8-27)
    Backend.scaled_dot_backward  its backward graph                (src/core/grad_fn.cpp:126-156, :569-665)
    Backend.mha_forward / mha_backward  MultiHeadAttention::forward and its backward graph
                                                                  (src/nn/multi_head_attention.cpp:19-42)
    Backend.softmax / softmax_backward / gelu / gelu_backward / colsum: the kernels between the GEMMs.
    Backend.layernorm / layernorm_backward / embedding / embedding_backward / cross_entropy: the GPT step's kernels
        around the matmuls (src/nn/layernorm.cpp, src/nn/embedding.cpp, src/loss/CrossEntropyLoss.cpp).
"""
import ctypes as C

import torch

from . import lib as L

_PREC = {"tf32": L.TE_PREC_TF32, "3xtf32": L.TE_PREC_3XTF32, L.TE_PREC_TF32: L.TE_PREC_TF32,
         L.TE_PREC_3XTF32: L.TE_PREC_3XTF32}


def _prec(p):
    try:
        return _PREC[p]
    except KeyError:
        raise ValueError("precision must be 'tf32' or '3xtf32'")


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _i64(seq):
    n = max(len(seq), 1)
    return (C.c_int64 * n)(*seq)


class Backend:
    """One per device: owns the C context (workspace, status word).  Not thread-safe; calls that use the
    workspace (3xTF32, operands TMA cannot address) must not overlap on different streams."""

    def __init__(self, device=0, workspace_bytes=2 << 30):
        self._lib = L.load()
        self.device = int(device)
        h = C.c_void_p()
        L.check(self._lib.te_b200_init(self.device, workspace_bytes, C.byref(h)))
        self._ctx = h
        self.torch_device = torch.device("cuda", self.device)

    def close(self):
        if getattr(self, "_ctx", None):
            self._lib.te_b200_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.torch_device).cuda_stream)

    def _check_f32_cuda(self, *ts):
        for t in ts:
            if t is None:
                continue
            if t.dtype != torch.float32:
                raise L.BackendError(L.TE_ERR_BAD_ARGUMENT, "CUDA matmul currently only supports Float32")
            if not t.is_cuda:
                raise L.BackendError(L.TE_ERR_BAD_ARGUMENT, "tensor is not on the GPU; this backend has no CPU path")

    @property
    def launches(self):
        return int(self._lib.te_b200_launch_count(self._ctx))

    def check_device_status(self):
        """Synchronises and raises if a kernel gave up a bounded wait."""
        torch.cuda.synchronize(self.torch_device)
        L.check(self._lib.te_b200_check_device_status(self._ctx))

    def set_wait_limit_ns(self, limit_ns):
        """Bound of every device-side wait of kernels launched through this context from now on (0 = default, 2 s)."""
        L.check(self._lib.te_b200_set_wait_limit_ns(self._ctx, int(limit_ns), self._stream()))

    def selftest_wait_timeout(self):
        """Launches the kernel whose bounded wait is meant to run out; check_device_status() then raises
        BackendError with status TE_ERR_DEVICE_TIMEOUT."""
        L.check(self._lib.te_b200_selftest_wait_timeout(self._ctx, self._stream()))

    # ------------------------------------------------------------------ GEMM
    def gemm(self, desc):
        """Raw strided-batched GEMM from a filled lib.GemmDesc."""
        L.check(self._lib.te_b200_gemm_f32(self._ctx, C.byref(desc), self._stream()))

    def gemm_host(self, desc):
        """Same with host pointers in the descriptor (copies in, runs, copies out, synchronises)."""
        L.check(self._lib.te_b200_gemm_f32_host(self._ctx, C.byref(desc)))

    def workspace_size(self, desc):
        n = C.c_size_t()
        L.check(self._lib.te_b200_gemm_workspace_size(C.byref(desc), C.byref(n)))
        return n.value

    def matmul(self, a, b, precision="tf32"):
        """a.matmul(b) with NumPy batch broadcasting; a and b may be any strided views whose last two
        dims form a row- or column-major slice.  Returns a fresh contiguous tensor."""
        self._check_f32_cuda(a, b)
        out_shape = L.matmul_shape(tuple(a.shape), tuple(a.stride()), tuple(b.shape), tuple(b.stride()))
        c = torch.empty(out_shape, dtype=torch.float32, device=a.device)
        L.check(self._lib.te_b200_matmul_nd(
            self._ctx, _ptr(a), _i64(a.shape), _i64(a.stride()), a.dim(),
            _ptr(b), _i64(b.shape), _i64(b.stride()), b.dim(),
            _ptr(c), None, None, _prec(precision), self._stream()))
        return c

    # ------------------------------------------------------------------ Linear
    def linear_forward(self, x, w, bias=None, gelu=False, want_preact=False, precision="tf32"):
        """y = act(x . w^T + bias); x [..., in] contiguous, w [out, in].  Returns y or (y, preact)."""
        self._check_f32_cuda(x, w, bias)
        x = x.contiguous()
        out_f, in_f = w.shape
        rows = x.numel() // in_f if in_f else 0
        y = torch.empty(x.shape[:-1] + (out_f,), dtype=torch.float32, device=x.device)
        pre = torch.empty_like(y) if want_preact else None
        L.check(self._lib.te_b200_linear_forward(self._ctx, _ptr(x), _ptr(w.contiguous()), _ptr(bias), _ptr(y),
                                                 _ptr(pre), rows, in_f, out_f, int(bool(gelu)), _prec(precision),
                                                 self._stream()))
        return (y, pre) if want_preact else y

    def linear_backward(self, x, w, dy, precision="tf32", need_dx=True, need_dw=True, need_db=True, gelu_preact=None,
                        dx_residual=None, accumulate_into=None, want_dx_colsum=False):
        """(dx, dw[out,in], db[out]) for y = x . w^T + b given dy.  With gelu_preact (x = gelu(gelu_preact), the second
        Linear of FeedForward) dx is the gradient of that pre-activation: the dX product, then GeluBackward in place.
        dx_residual ([rows, in]) is added into dx.  accumulate_into = (dw, db) adds the parameter gradients to those
        tensors in place (and returns them) instead of writing fresh ones.  want_dx_colsum appends the column sums of dx
        (the bias gradient of the Linear that produced x) to the result."""
        self._check_f32_cuda(x, w, dy, gelu_preact, dx_residual)
        x = x.contiguous()
        dy = dy.contiguous()
        out_f, in_f = w.shape
        rows = x.numel() // in_f if in_f else 0
        dx = torch.empty_like(x) if need_dx else None
        if accumulate_into is not None:
            dw, db = accumulate_into
            self._check_f32_cuda(dw, db)
        else:
            dw = torch.empty_like(w) if need_dw else None
            db = torch.empty(out_f, dtype=torch.float32, device=x.device) if need_db else None
        if gelu_preact is not None and (gelu_preact.shape != x.shape or not gelu_preact.is_contiguous()):
            raise L.BackendError(L.TE_ERR_BAD_ARGUMENT, "gelu_preact must be contiguous and shaped like x")
        if dx_residual is not None and (dx_residual.shape != x.shape or not dx_residual.is_contiguous()):
            raise L.BackendError(L.TE_ERR_BAD_ARGUMENT, "dx_residual must be contiguous and shaped like x")
        dxs = torch.empty(in_f, dtype=torch.float32, device=x.device) if want_dx_colsum else None
        L.check(self._lib.te_b200_linear_backward_ex(self._ctx, _ptr(x), _ptr(gelu_preact), _ptr(w.contiguous()), _ptr(dy),
                                                     _ptr(dx), _ptr(dx_residual), _ptr(dxs), _ptr(dw), _ptr(db),
                                                     int(accumulate_into is not None), rows, in_f, out_f, _prec(precision),
                                                     self._stream()))
        return (dx, dw, db, dxs) if want_dx_colsum else (dx, dw, db)

    # ------------------------------------------------------------------ multi-head attention
    def mha_forward(self, x, params, heads, residual=None, precision="tf32", one_projection_gemm=True):
        """MultiHeadAttention::forward for x [B,T,E]; params in parameters() order (wq,bq,wk,bk,wv,bv,wo,bo).
        Returns (y, saved) where saved holds what mha_backward needs.  one_projection_gemm: the three projections as
        one product against the gathered [3E,E] weight (q, k, v are then column blocks of one [B,T,3E] buffer);
        False runs them as three products into three dense buffers."""
        self._check_f32_cuda(x, residual, *params)
        x = x.contiguous()
        B, T, E = x.shape
        new = lambda *shape: torch.empty(shape, dtype=torch.float32, device=x.device)
        saved = dict(x=x, p=new(B, heads, T, T), attn=new(B, T, E), params=[t.contiguous() for t in params], heads=heads,
                     fused=bool(one_projection_gemm))
        if one_projection_gemm:
            saved["qkv"], saved["wqkv"] = new(B, T, 3 * E), new(3 * E * E + 3 * E)
            saved["q"], saved["k"], saved["v"] = (saved["qkv"][:, :, i * E:(i + 1) * E] for i in range(3))
        else:
            saved["q"], saved["k"], saved["v"] = new(B, T, E), new(B, T, E), new(B, T, E)
        y = new(B, T, E)
        m = L.MhaDesc()
        m.B, m.T, m.E, m.H = B, T, E, heads
        m.x = x.data_ptr()
        for n, t in zip(("wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo"), saved["params"]):
            setattr(m, n, t.data_ptr())
        for n in ("q", "k", "v", "p", "attn"):
            setattr(m, n, saved[n].data_ptr())
        if one_projection_gemm:
            m.ld_qkv, m.wqkv = 3 * E, saved["wqkv"].data_ptr()
        m.y = y.data_ptr()
        m.residual = residual.contiguous().data_ptr() if residual is not None else None
        m.precision = _prec(precision)
        L.check(self._lib.te_b200_mha_forward(self._ctx, C.byref(m), self._stream()))
        return y, saved

    def mha_backward(self, saved, dy, dx_residual=None, precision="tf32"):
        """(dx, [dwq, dbq, dwk, dbk, dwv, dbv, dwo, dbo]) for the call that produced `saved`."""
        self._check_f32_cuda(dy, dx_residual)
        x = saved["x"]
        dy = dy.contiguous()
        B, T, E = x.shape
        dx = torch.empty_like(x)
        grads = [torch.empty_like(t) for t in saved["params"]]
        dattn = torch.empty_like(x)
        m = L.MhaBwdDesc()
        m.B, m.T, m.E, m.H = B, T, E, saved["heads"]
        m.x = x.data_ptr()
        m.wq, m.wk, m.wv, m.wo = (saved["params"][i].data_ptr() for i in (0, 2, 4, 6))
        for n in ("q", "k", "v", "p", "attn"):
            setattr(m, n, saved[n].data_ptr())
        m.dy, m.dx = dy.data_ptr(), dx.data_ptr()
        m.dx_residual = dx_residual.contiguous().data_ptr() if dx_residual is not None else None
        for n, t in zip(("dwq", "dbq", "dwk", "dbk", "dwv", "dbv", "dwo", "dbo"), grads):
            setattr(m, n, t.data_ptr())
        if saved["fused"]:
            dqkv, dwqkv = torch.empty_like(saved["qkv"]), torch.empty_like(saved["wqkv"])
            m.dq, m.dk, m.dv = (dqkv.data_ptr() + 4 * E * i for i in range(3))
            m.ld_qkv, m.wqkv, m.dwqkv = 3 * E, saved["wqkv"].data_ptr(), dwqkv.data_ptr()
        else:
            scratch = [torch.empty_like(x) for _ in range(3)]
            m.dq, m.dk, m.dv = (t.data_ptr() for t in scratch)
        m.dattn = dattn.data_ptr()
        m.accumulate, m.precision = 0, _prec(precision)
        L.check(self._lib.te_b200_mha_backward(self._ctx, C.byref(m), self._stream()))
        return dx, grads

    # ------------------------------------------------------------------ attention
    def scaled_dot(self, q, k, v, precision="tf32", head_major_out=True):
        """softmax(q . k^T / sqrt(d)) . v for [B,H,T,d] views with unit last-dim stride (for example the
        MultiHeadAttention head views with strides [T*E, d, E, 1]).  Returns (o [B,H,T,d], p).  o is contiguous, or with
        head_major_out=False a view over [B,T,H,d] memory, so that the head merge of MultiHeadAttention::forward
        (transpose + reshape, src/nn/multi_head_attention.cpp:36-38) needs no copy."""
        self._check_f32_cuda(q, k, v)
        if q.dim() != 4 or q.shape != k.shape or q.shape != v.shape:
            raise L.BackendError(L.TE_ERR_BAD_ARGUMENT, "scaled_dot expects q, k, v of one [B,H,T,d] shape")
        for t in (q, k, v):
            if t.stride(3) != 1:
                raise L.BackendError(L.TE_ERR_UNSUPPORTED_LAYOUT, L.status_string(L.TE_ERR_UNSUPPORTED_LAYOUT))
        B, H, T, d = q.shape
        p = torch.empty((B, H, T, T), dtype=torch.float32, device=q.device)
        if head_major_out:
            o = torch.empty((B, H, T, d), dtype=torch.float32, device=q.device)
        else:
            o = torch.empty((B, T, H, d), dtype=torch.float32, device=q.device).transpose(1, 2)
        desc = L.AttnDesc()
        desc.B, desc.H, desc.T, desc.d = B, H, T, d
        desc.q, desc.k, desc.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
        desc.q_strides = (C.c_int64 * 3)(*q.stride()[:3])
        desc.k_strides = (C.c_int64 * 3)(*k.stride()[:3])
        desc.v_strides = (C.c_int64 * 3)(*v.stride()[:3])
        desc.p_out, desc.o = p.data_ptr(), o.data_ptr()
        desc.o_strides = (C.c_int64 * 3)(*o.stride()[:3])
        desc.precision = _prec(precision)
        L.check(self._lib.te_b200_attention_forward(self._ctx, C.byref(desc), self._stream()))
        return o, p

    def scaled_dot_backward(self, q, k, v, p, d_o, o=None, precision="tf32", head_major_out=True):
        """(dq, dk, dv) of scaled_dot given the gradient d_o of its output, the probabilities p it returned and
        (optionally) its output o: MatMulBackward x2, SoftmaxBackward and DivBackward of the reference graph
        (src/core/grad_fn.cpp:126-156, :569-665).  With o the fused kernel may run; without it the GEMM sequence.
        head_major_out=False returns views over [B,T,H,d] memory (the layout the head-split views came from)."""
        self._check_f32_cuda(q, k, v, p, d_o, o)
        B, H, T, d = q.shape
        if p.shape != (B, H, T, T) or not p.is_contiguous():
            raise L.BackendError(L.TE_ERR_BAD_ARGUMENT, "scaled_dot_backward expects dense probabilities [B,H,T,T]")
        if d_o.stride(3) != 1:
            d_o = d_o.contiguous()
        for t in (q, k, v) + ((o,) if o is not None else ()):
            if t.shape != q.shape or t.stride(3) != 1:
                raise L.BackendError(L.TE_ERR_UNSUPPORTED_LAYOUT, L.status_string(L.TE_ERR_UNSUPPORTED_LAYOUT))
        if head_major_out:
            dq, dk, dv = (torch.empty((B, H, T, d), dtype=torch.float32, device=q.device) for _ in range(3))
        else:
            dq, dk, dv = (torch.empty((B, T, H, d), dtype=torch.float32, device=q.device).transpose(1, 2) for _ in range(3))
        desc = L.AttnBwdDesc()
        desc.B, desc.H, desc.T, desc.d = B, H, T, d
        desc.q, desc.k, desc.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
        desc.q_strides = (C.c_int64 * 3)(*q.stride()[:3])
        desc.k_strides = (C.c_int64 * 3)(*k.stride()[:3])
        desc.v_strides = (C.c_int64 * 3)(*v.stride()[:3])
        desc.p = p.data_ptr()
        desc.o = o.data_ptr() if o is not None else None
        desc.o_strides = (C.c_int64 * 3)(*(o.stride()[:3] if o is not None else (0, 0, 0)))
        desc.d_o = d_o.data_ptr()
        desc.d_o_strides = (C.c_int64 * 3)(*d_o.stride()[:3])
        desc.dq, desc.dk, desc.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        desc.dq_strides = (C.c_int64 * 3)(*dq.stride()[:3])
        desc.dk_strides = (C.c_int64 * 3)(*dk.stride()[:3])
        desc.dv_strides = (C.c_int64 * 3)(*dv.stride()[:3])
        desc.precision = _prec(precision)
        L.check(self._lib.te_b200_attention_backward(self._ctx, C.byref(desc), self._stream()))
        return dq, dk, dv

    # ------------------------------------------------------------------ the GPT step's kernels around the matmuls
    def layernorm(self, x, gamma, beta, eps=1e-5):
        """LayerNorm::forward over the last dimension (src/nn/layernorm.cpp:19-82)."""
        self._check_f32_cuda(x, gamma, beta)
        x = x.contiguous()
        y = torch.empty_like(x)
        cols = x.shape[-1]
        rows = x.numel() // cols if cols else 0
        L.check(self._lib.te_b200_layernorm_forward(self._ctx, _ptr(x), _ptr(gamma.contiguous()), _ptr(beta.contiguous()),
                                                    _ptr(y), rows, cols, eps, self._stream()))
        return y

    def layernorm_backward(self, x, gamma, dy, eps=1e-5, dx_residual=None, want_dx_colsum=False):
        """(dx, dgamma, dbeta) of LayerNormBackward::backward (src/core/grad_fn.cpp:405-538); dx_residual is added to dx;
        want_dx_colsum appends the column sums of dx."""
        self._check_f32_cuda(x, gamma, dy, dx_residual)
        x, dy = x.contiguous(), dy.contiguous()
        cols = x.shape[-1]
        rows = x.numel() // cols if cols else 0
        dx = torch.empty_like(x)
        dg = torch.empty(cols, dtype=torch.float32, device=x.device)
        db = torch.empty(cols, dtype=torch.float32, device=x.device)
        dxs = torch.empty(cols, dtype=torch.float32, device=x.device) if want_dx_colsum else None
        L.check(self._lib.te_b200_layernorm_backward_ex(self._ctx, _ptr(x), _ptr(gamma.contiguous()), _ptr(dy), _ptr(dx),
                                                        _ptr(dx_residual.contiguous() if dx_residual is not None else None),
                                                        _ptr(dg), _ptr(db), _ptr(dxs), rows, cols, eps, self._stream()))
        return (dx, dg, db, dxs) if want_dx_colsum else (dx, dg, db)

    def embedding(self, table, tokens, pos=None):
        """table[tokens] (+ pos[t]) for int64 tokens [..., T]: Embedding::forward with GPT::forward's positional sum
        (src/nn/embedding.cpp:18-60, src/nn/gpt.cpp:30-69)."""
        self._check_f32_cuda(table, pos)
        if tokens.dtype != torch.int64:
            raise L.BackendError(L.TE_ERR_BAD_ARGUMENT, "Embedding input must be Int64")
        tokens = tokens.contiguous()
        table = table.contiguous()
        vocab, dim = table.shape
        out = torch.empty(tuple(tokens.shape) + (dim,), dtype=torch.float32, device=table.device)
        T = tokens.shape[-1] if tokens.dim() else 1
        L.check(self._lib.te_b200_embedding_forward(self._ctx, _ptr(table), _ptr(tokens), _ptr(pos.contiguous() if pos is not None else None),
                                                    _ptr(out), tokens.numel(), T, dim, vocab, self._stream()))
        return out

    def embedding_backward(self, tokens, dout, vocab):
        """Table gradient of EmbeddingBackward::backward (src/core/grad_fn.cpp:688-760), rows added in token order."""
        self._check_f32_cuda(dout)
        tokens, dout = tokens.contiguous(), dout.contiguous()
        dim = dout.shape[-1]
        dtable = torch.empty((vocab, dim), dtype=torch.float32, device=dout.device)
        L.check(self._lib.te_b200_embedding_backward(self._ctx, _ptr(tokens), _ptr(dout), _ptr(dtable), tokens.numel(), dim,
                                                     vocab, self._stream()))
        return dtable

    def cross_entropy(self, logits, targets, want_grad=True, upstream=1.0):
        """(mean loss as a 1-element device tensor, dlogits or None): crossEntropyLoss::forward_batched and its
        backward (src/loss/CrossEntropyLoss.cpp:47-127, src/core/grad_fn.cpp:271-346)."""
        self._check_f32_cuda(logits)
        if targets.dtype != torch.int64:
            raise L.BackendError(L.TE_ERR_BAD_ARGUMENT, "cross-entropy targets must be Int64")
        logits, targets = logits.contiguous(), targets.contiguous()
        vocab = logits.shape[-1]
        rows = logits.numel() // vocab if vocab else 0
        loss = torch.empty(1, dtype=torch.float32, device=logits.device)
        grad = torch.empty_like(logits) if want_grad else None
        L.check(self._lib.te_b200_cross_entropy(self._ctx, _ptr(logits), _ptr(targets), _ptr(loss), _ptr(grad), upstream, rows,
                                                vocab, self._stream()))
        return loss, grad

    # ------------------------------------------------------------------ row / elementwise ops
    def softmax(self, x):
        self._check_f32_cuda(x)
        x = x.contiguous()
        y = torch.empty_like(x)
        cols = x.shape[-1]
        rows = x.numel() // cols if cols else 0
        L.check(self._lib.te_b200_softmax_rows_f32(self._ctx, _ptr(x), _ptr(y), rows, cols, self._stream()))
        return y

    def softmax_backward(self, s, dy):
        self._check_f32_cuda(s, dy)
        s, dy = s.contiguous(), dy.contiguous()
        dx = torch.empty_like(s)
        cols = s.shape[-1]
        rows = s.numel() // cols if cols else 0
        L.check(self._lib.te_b200_softmax_backward_rows_f32(self._ctx, _ptr(s), _ptr(dy), _ptr(dx), rows, cols,
                                                            self._stream()))
        return dx

    def gelu(self, x):
        self._check_f32_cuda(x)
        x = x.contiguous()
        y = torch.empty_like(x)
        L.check(self._lib.te_b200_gelu_f32(self._ctx, _ptr(x), _ptr(y), x.numel(), self._stream()))
        return y

    def gelu_backward(self, x, dy):
        self._check_f32_cuda(x, dy)
        x, dy = x.contiguous(), dy.contiguous()
        dx = torch.empty_like(x)
        L.check(self._lib.te_b200_gelu_backward_f32(self._ctx, _ptr(x), _ptr(dy), _ptr(dx), x.numel(), self._stream()))
        return dx

    def colsum(self, x2d):
        self._check_f32_cuda(x2d)
        x2d = x2d.contiguous()
        rows, cols = x2d.shape
        out = torch.empty(cols, dtype=torch.float32, device=x2d.device)
        L.check(self._lib.te_b200_colsum_f32(self._ctx, _ptr(x2d), rows, cols, cols, _ptr(out), self._stream()))
        return out
