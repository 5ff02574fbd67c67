"""numpy-facing ctypes bindings of the checkers.  TEST INFRASTRUCTURE ONLY.

`Oracle`    - liboracle.so, the plain-C restatement (te_oracle.c); built by `make -C oracle`.
`Reference` - _ref/libref_cpu.so, the reference's own CPU path compiled from its sources (ref_driver.cpp).
              Present only where it was built; it travels as a prebuilt file.
`ReferenceCuda` - _ref_cuda/libref_cuda.so, the reference's CUDA path built for sm_100a with the
              TENSOR_GEMM_BACKEND=b200 binding applied (same driver, USE_CUDA): the reference's own Tensor / nn /
              autograd code on the GPU under its cuBLAS, `custom` or `b200` GEMM backend.  Needs a GPU to run.
Only tests/, the smoke check and the benchmark's CPU legs may import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_PATH = os.path.join(_HERE, "liboracle.so")
REF_PATH = os.path.join(_HERE, "_ref", "libref_cpu.so")
REF_CUDA_PATH = os.path.join(_HERE, "_ref_cuda", "libref_cuda.so")
REF_CUDA_MATMUL_TEST = os.path.join(_HERE, "_ref_cuda", "cuda_matmul_tensor_test")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")


def build(reference_root="/root/reference"):
    """Runs the Makefile: liboracle.so always; _ref/libref_cpu.so and (once libte_b200.so exists) the patched CUDA
    build _ref_cuda/ when the reference sources are present."""
    subprocess.run(["make", "-s", "-C", _HERE, "-j8", "REF=" + reference_root, "all", "ref_cuda"], check=True)


def _i64(seq):
    return (C.c_int64 * max(len(seq), 1))(*[int(s) for s in seq])


def _fptr(a):
    return a.ctypes.data_as(C.c_void_p)


class OracleError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(msg)
        self.code = code


_ORACLE_ERR = {3: "Matmul requires tensors with at least 2 dimensions", 4: "Inner dimensions must match for matmul",
               5: "Batch dimensions are not broadcastable", 1: "bad argument"}


class Oracle:
    def __init__(self):
        if not os.path.exists(ORACLE_PATH):
            build()
        self.lib = C.CDLL(ORACLE_PATH)

    def matmul(self, a, b):
        """a @ b for float32 numpy arrays of any strides (views allowed), reference CPU summation order."""
        assert a.dtype == np.float32 and b.dtype == np.float32
        es = 4
        a_str = [s // es for s in a.strides]
        b_str = [s // es for s in b.strides]
        out_shape = (C.c_int64 * 8)()
        nd = C.c_int()
        rc = self.lib.oracle_matmul_nd_f32(None, _i64(a.shape), _i64(a_str), a.ndim, None, _i64(b.shape), _i64(b_str),
                                           b.ndim, None, out_shape, C.byref(nd))
        if rc:
            raise OracleError(rc, _ORACLE_ERR.get(rc, "error"))
        shape = tuple(out_shape[i] for i in range(nd.value))
        c = np.empty(shape, dtype=np.float32)
        rc = self.lib.oracle_matmul_nd_f32(_fptr(a), _i64(a.shape), _i64(a_str), a.ndim, _fptr(b), _i64(b.shape),
                                           _i64(b_str), b.ndim, _fptr(c), None, None)
        if rc:
            raise OracleError(rc, _ORACLE_ERR.get(rc, "error"))
        return c

    def matmul_2d_threads(self, a, b, threads=None):
        """Dense 2-D a @ b split by row blocks over host threads; bit-identical to matmul()."""
        from concurrent.futures import ThreadPoolExecutor
        M, K = a.shape
        N = b.shape[1]
        c = np.empty((M, N), dtype=np.float32)
        threads = threads or os.cpu_count() or 1
        a_s = [s // 4 for s in a.strides]
        b_s = [s // 4 for s in b.strides]
        fn = self.lib.oracle_matmul_rows_f32
        fn.restype = None

        def work(r):
            fn(_fptr(a), C.c_int64(a_s[0]), C.c_int64(a_s[1]), _fptr(b), C.c_int64(b_s[0]), C.c_int64(b_s[1]),
               _fptr(c), C.c_int64(M), C.c_int64(K), C.c_int64(N), C.c_int64(r[0]), C.c_int64(r[1]))
        step = max(1, (M + threads * 4 - 1) // (threads * 4))
        ranges = [(i, min(i + step, M)) for i in range(0, M, step)]
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(work, ranges))
        return c

    def matmul_f64(self, a, b, rows=None):
        """Double-accumulated product of selected rows (all rows when None) of dense 2-D a @ b."""
        from concurrent.futures import ThreadPoolExecutor
        M, K = a.shape
        N = b.shape[1]
        c = np.zeros((M, N), dtype=np.float64)
        a_s = [s // 4 for s in a.strides]
        b_s = [s // 4 for s in b.strides]
        fn = self.lib.oracle_matmul_rows_f64acc
        fn.restype = None
        rows = range(M) if rows is None else rows

        def work(r):
            fn(_fptr(a), C.c_int64(a_s[0]), C.c_int64(a_s[1]), _fptr(b), C.c_int64(b_s[0]), C.c_int64(b_s[1]),
               _fptr(c), C.c_int64(K), C.c_int64(N), C.c_int64(r), C.c_int64(r + 1))
        with ThreadPoolExecutor(os.cpu_count() or 1) as ex:
            list(ex.map(work, rows))
        return c

    def add_bias(self, y, bias):
        y = np.ascontiguousarray(y, dtype=np.float32).copy()
        cols = y.shape[-1]
        self.lib.oracle_add_bias_f32(_fptr(y), _fptr(np.ascontiguousarray(bias, dtype=np.float32)),
                                     C.c_int64(y.size // cols), C.c_int64(cols))
        return y

    def gelu(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        self.lib.oracle_gelu_f32(_fptr(x), _fptr(y), C.c_int64(x.size))
        return y

    def gelu_backward(self, x, dy):
        x = np.ascontiguousarray(x, dtype=np.float32)
        dy = np.ascontiguousarray(dy, dtype=np.float32)
        dx = np.empty_like(x)
        self.lib.oracle_gelu_backward_f32(_fptr(x), _fptr(dy), _fptr(dx), C.c_int64(x.size))
        return dx

    def softmax(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        cols = x.shape[-1]
        self.lib.oracle_softmax_rows_f32(_fptr(x), _fptr(y), C.c_int64(x.size // cols), C.c_int64(cols))
        return y

    def softmax_backward(self, s, dy):
        s = np.ascontiguousarray(s, dtype=np.float32)
        dy = np.ascontiguousarray(dy, dtype=np.float32)
        dx = np.empty_like(s)
        cols = s.shape[-1]
        self.lib.oracle_softmax_backward_rows_f32(_fptr(s), _fptr(dy), _fptr(dx), C.c_int64(s.size // cols),
                                                  C.c_int64(cols))
        return dx

    def colsum(self, x2d):
        x2d = np.ascontiguousarray(x2d, dtype=np.float32)
        out = np.empty(x2d.shape[1], dtype=np.float32)
        self.lib.oracle_colsum_f32(_fptr(x2d), C.c_int64(x2d.shape[0]), C.c_int64(x2d.shape[1]),
                                   C.c_int64(x2d.shape[1]), _fptr(out))
        return out

    def layernorm(self, x, gamma, beta, eps=1e-5):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        D = x.shape[-1]
        self.lib.oracle_layernorm_forward(_fptr(x), _fptr(np.ascontiguousarray(gamma, dtype=np.float32)),
                                          _fptr(np.ascontiguousarray(beta, dtype=np.float32)), _fptr(y),
                                          C.c_int64(x.size // D), C.c_int64(D), C.c_float(eps))
        return y

    def layernorm_backward(self, x, gamma, dy, eps=1e-5):
        """(dx, dgamma, dbeta)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        dy = np.ascontiguousarray(dy, dtype=np.float32)
        gamma = np.ascontiguousarray(gamma, dtype=np.float32)
        D = x.shape[-1]
        dx, dg, db, scratch = np.empty_like(x), np.empty(D, np.float32), np.empty(D, np.float32), np.empty(D, np.float32)
        self.lib.oracle_layernorm_backward(_fptr(x), _fptr(gamma), _fptr(dy), _fptr(dx), _fptr(dg), _fptr(db),
                                           _fptr(scratch), C.c_int64(x.size // D), C.c_int64(D), C.c_float(eps))
        return dx, dg, db

    def cross_entropy(self, logits, targets):
        """Mean loss over the rows of logits [..., V] with int64 targets [...]."""
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        targets = np.ascontiguousarray(targets, dtype=np.int64)
        V = logits.shape[-1]
        fn = self.lib.oracle_cross_entropy_forward
        fn.restype = C.c_float
        return np.float32(fn(_fptr(logits), targets.ctypes.data_as(C.c_void_p), C.c_int64(logits.size // V), C.c_int64(V)))

    def cross_entropy_backward(self, logits, targets, upstream=1.0):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        targets = np.ascontiguousarray(targets, dtype=np.int64)
        V = logits.shape[-1]
        grad = np.empty_like(logits)
        self.lib.oracle_cross_entropy_backward(_fptr(logits), targets.ctypes.data_as(C.c_void_p), C.c_float(upstream),
                                               _fptr(grad), C.c_int64(logits.size // V), C.c_int64(V))
        return grad

    def embedding(self, table, tokens, pos=None):
        """table[tokens] (+ pos[t] broadcast over the batch): tokens [B, T] -> [B, T, D]."""
        table = np.ascontiguousarray(table, dtype=np.float32)
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        vocab, D = table.shape
        T = tokens.shape[-1]
        out = np.empty(tokens.shape + (D,), dtype=np.float32)
        pos_c = None if pos is None else np.ascontiguousarray(pos, dtype=np.float32)
        fn = self.lib.oracle_embedding_forward
        fn.restype = C.c_int
        rc = fn(_fptr(table), tokens.ctypes.data_as(C.c_void_p), _fptr(pos_c) if pos_c is not None else None, _fptr(out),
                C.c_int64(tokens.size), C.c_int64(T), C.c_int64(D), C.c_int64(vocab))
        if rc:
            raise OracleError(rc, "Embedding index out of range")
        return out

    def embedding_backward(self, tokens, dout, vocab):
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        dout = np.ascontiguousarray(dout, dtype=np.float32)
        D = dout.shape[-1]
        dtable = np.empty((vocab, D), dtype=np.float32)
        self.lib.oracle_embedding_backward(tokens.ctypes.data_as(C.c_void_p), _fptr(dout), _fptr(dtable),
                                           C.c_int64(tokens.size), C.c_int64(D), C.c_int64(vocab))
        return dtable

    # Compositions that follow the reference call sequence.
    def linear(self, x, w, bias, gelu=False):
        """Linear::forward (+ Tensor::gelu): x . w^T through the transposed view, then the broadcast bias add."""
        pre = self.add_bias(self.matmul(x, w.T), bias)
        return (self.gelu(pre), pre) if gelu else (pre, pre)

    def scaled_dot(self, q, k, v):
        """ScaledDot::forward: S = q . k^T; S / sqrt(d); softmax; . v.  Returns (o, p)."""
        s = self.matmul(q, np.swapaxes(k, -1, -2))
        s = (s / np.float32(np.sqrt(np.float32(q.shape[-1])))).astype(np.float32)
        p = self.softmax(s)
        return self.matmul(p, v), p


class SeededRng:
    """std::mt19937 / std::mt19937_64 streams with the C++ standard distributions, as the reference's
    benchmarks and tests draw their inputs (seed 42, A first then B from the same generator)."""

    def __init__(self, seed=42):
        if not os.path.exists(ORACLE_PATH):
            build()
        self.lib = C.CDLL(ORACLE_PATH)
        self.lib.oracle_rng_create.restype = C.c_void_p
        self.h = C.c_void_p(self.lib.oracle_rng_create(C.c_uint64(seed)))

    def __del__(self):
        try:
            self.lib.oracle_rng_destroy(self.h)
        except Exception:
            pass

    def uniform(self, shape, lo=-1.0, hi=1.0):
        out = np.empty(shape, dtype=np.float32)
        self.lib.oracle_rng_uniform_f32(self.h, _fptr(out), C.c_int64(out.size), C.c_float(lo), C.c_float(hi))
        return out

    def normal(self, shape, mean=0.0, std=1.0):
        out = np.empty(shape, dtype=np.float32)
        self.lib.oracle_rng_normal_f32(self.h, _fptr(out), C.c_int64(out.size), C.c_float(mean), C.c_float(std))
        return out

    def tokens(self, shape, bound):
        out = np.empty(shape, dtype=np.int64)
        self.lib.oracle_rng_tokens_i64(self.h, _fptr(out), C.c_int64(out.size), C.c_int64(bound))
        return out


class RefView(C.Structure):
    _fields_ = [("ndim", C.c_int32), ("shape", C.c_int64 * 8), ("view_ndim", C.c_int32), ("view_shape", C.c_int64 * 8),
                ("t1", C.c_int32), ("t2", C.c_int32), ("t3", C.c_int32), ("t4", C.c_int32)]


def ref_view(shape, view=None, transpose=None, transpose2=None):
    v = RefView()
    v.ndim = len(shape)
    for i, s in enumerate(shape):
        v.shape[i] = s
    v.view_ndim = len(view) if view else 0
    for i, s in enumerate(view or ()):
        v.view_shape[i] = s
    v.t1, v.t2 = transpose if transpose else (-1, -1)
    v.t3, v.t4 = transpose2 if transpose2 else (-1, -1)
    return v


class Reference:
    """The reference's own CPU implementation behind ref_driver.cpp."""

    @staticmethod
    def available():
        return os.path.exists(REF_PATH)

    PATH = REF_PATH
    prefix = "ref_"       # ReferenceCuda switches to "ref_fused_" for the module-level calls

    def __init__(self):
        if not os.path.exists(self.PATH):
            raise RuntimeError("reference library not built (needs the reference sources): " + self.PATH)
        self.lib = C.CDLL(self.PATH)
        self.lib.ref_last_error.restype = C.c_char_p

    def _fn(self, name):
        return getattr(self.lib, self.prefix + name)

    def _check(self, rc):
        if rc:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def view_strides(self, view):
        shape, strides, nd = (C.c_int64 * 8)(), (C.c_int64 * 8)(), C.c_int32()
        self._check(self.lib.ref_view_strides(C.byref(view), shape, strides, C.byref(nd)))
        return tuple(shape[i] for i in range(nd.value)), tuple(strides[i] for i in range(nd.value))

    def matmul(self, a, va, b, vb, out_shape=None):
        """a, b: dense base arrays; va, vb: recipes (ref_view).  Raises RuntimeError with the reference's text.
        Without out_shape the product is evaluated twice (once to learn the result shape); timed callers pass it."""
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        if out_shape is None:
            shape, nd = (C.c_int64 * 8)(), C.c_int32()
            self._check(self.lib.ref_matmul(_fptr(a), C.byref(va), _fptr(b), C.byref(vb), None, shape, C.byref(nd)))
            out_shape = tuple(shape[i] for i in range(nd.value))
        out = np.empty(tuple(out_shape), dtype=np.float32)
        self._check(self.lib.ref_matmul(_fptr(a), C.byref(va), _fptr(b), C.byref(vb), _fptr(out), None, None))
        return out

    def matmul_i32(self, a, b):
        a = np.ascontiguousarray(a, dtype=np.int32)
        b = np.ascontiguousarray(b, dtype=np.int32)
        out = np.empty((a.shape[0], b.shape[1]), dtype=np.int32)
        self._check(self.lib.ref_matmul_i32(_fptr(a), _fptr(b), _fptr(out), C.c_int64(a.shape[0]),
                                            C.c_int64(a.shape[1]), C.c_int64(b.shape[1])))
        return out

    def linear(self, x, w, bias, gelu=False, dy=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        out_f, in_f = w.shape
        y = np.empty(x.shape[:-1] + (out_f,), dtype=np.float32)
        pre = np.empty_like(y)
        res = {"y": y, "preact": pre}
        if dy is not None:
            dy = np.ascontiguousarray(dy, dtype=np.float32)
            res.update(dx=np.empty_like(x), dw=np.empty_like(w), db=np.empty_like(bias))
        p = lambda k: _fptr(res[k]) if k in res else None
        self._check(self._fn("linear")(_fptr(x), _i64(x.shape), x.ndim, _fptr(w), _fptr(bias), C.c_int64(in_f),
                                        C.c_int64(out_f), int(gelu), _fptr(dy) if dy is not None else None,
                                        p("y"), p("preact"), p("dx"), p("dw"), p("db")))
        return res

    def layernorm(self, x, gamma, beta, eps=1e-5, dy=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        gamma, beta = (np.ascontiguousarray(t, dtype=np.float32) for t in (gamma, beta))
        D = x.shape[-1]
        res = {"y": np.empty_like(x)}
        if dy is not None:
            dy = np.ascontiguousarray(dy, dtype=np.float32)
            res.update(dx=np.empty_like(x), dgamma=np.empty_like(gamma), dbeta=np.empty_like(beta))
        p = lambda k: _fptr(res[k]) if k in res else None
        self._check(self.lib.ref_layernorm(_fptr(x), C.c_int64(x.size // D), C.c_int64(D), _fptr(gamma), _fptr(beta),
                                           C.c_float(eps), _fptr(dy) if dy is not None else None, p("y"), p("dx"),
                                           p("dgamma"), p("dbeta")))
        return res

    def cross_entropy(self, logits, targets, want_grad=True):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        targets = np.ascontiguousarray(targets, dtype=np.int64)
        B, T, V = logits.shape
        loss = C.c_float(0)
        grad = np.empty_like(logits) if want_grad else None
        self._check(self.lib.ref_cross_entropy(_fptr(logits), targets.ctypes.data_as(C.c_void_p), C.c_int64(B), C.c_int64(T),
                                               C.c_int64(V), C.byref(loss), _fptr(grad) if want_grad else None))
        return {"loss": np.float32(loss.value), "dlogits": grad}

    def embedding(self, table, tokens, dout=None):
        table = np.ascontiguousarray(table, dtype=np.float32)
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        vocab, D = table.shape
        B, T = tokens.shape
        res = {"out": np.empty((B, T, D), dtype=np.float32)}
        if dout is not None:
            dout = np.ascontiguousarray(dout, dtype=np.float32)
            res["dtable"] = np.empty_like(table)
        self._check(self.lib.ref_embedding(_fptr(table), C.c_int64(vocab), C.c_int64(D), tokens.ctypes.data_as(C.c_void_p),
                                           C.c_int64(B), C.c_int64(T), _fptr(dout) if dout is not None else None,
                                           _fptr(res["out"]), _fptr(res["dtable"]) if dout is not None else None))
        return res

    def ffn(self, x, w1, b1, w2, b2, dy=None):
        arrs = [np.ascontiguousarray(t, dtype=np.float32) for t in (x, w1, b1, w2, b2)]
        x, w1, b1, w2, b2 = arrs
        ff, embed = w1.shape
        res = {"y": np.empty_like(x)}
        if dy is not None:
            dy = np.ascontiguousarray(dy, dtype=np.float32)
            res.update(dx=np.empty_like(x), dw1=np.empty_like(w1), db1=np.empty_like(b1), dw2=np.empty_like(w2),
                       db2=np.empty_like(b2))
        p = lambda k: _fptr(res[k]) if k in res else None
        self._check(self._fn("ffn")(_fptr(x), _i64(x.shape), x.ndim, C.c_int64(embed), C.c_int64(ff), _fptr(w1),
                                     _fptr(b1), _fptr(w2), _fptr(b2), _fptr(dy) if dy is not None else None, p("y"),
                                     p("dx"), p("dw1"), p("db1"), p("dw2"), p("db2")))
        return res

    def scaled_dot(self, q, vq, k, vk, v, vv, out_shape, d_o=None):
        q, k, v = [np.ascontiguousarray(t, dtype=np.float32) for t in (q, k, v)]
        res = {"o": np.empty(out_shape, dtype=np.float32)}
        if d_o is not None:
            d_o = np.ascontiguousarray(d_o, dtype=np.float32)
            res.update(dq=np.empty_like(q), dk=np.empty_like(k), dv=np.empty_like(v))
        p = lambda n: _fptr(res[n]) if n in res else None
        self._check(self._fn("scaled_dot")(_fptr(q), C.byref(vq), _fptr(k), C.byref(vk), _fptr(v), C.byref(vv),
                                            _fptr(d_o) if d_o is not None else None, p("o"), p("dq"), p("dk"), p("dv")))
        return res

    def mha(self, x, params, H, dy=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        params = [np.ascontiguousarray(t, dtype=np.float32) for t in params]
        B, T, E = x.shape
        res = {"y": np.empty_like(x)}
        pp = (C.c_void_p * 8)(*[t.ctypes.data for t in params])
        dpp = None
        if dy is not None:
            dy = np.ascontiguousarray(dy, dtype=np.float32)
            res["dx"] = np.empty_like(x)
            res["dparams"] = [np.empty_like(t) for t in params]
            dpp = (C.c_void_p * 8)(*[t.ctypes.data for t in res["dparams"]])
        self._check(self._fn("mha")(_fptr(x), C.c_int64(B), C.c_int64(T), C.c_int64(E), C.c_int64(H), pp,
                                     _fptr(dy) if dy is not None else None, _fptr(res["y"]),
                                     _fptr(res["dx"]) if dy is not None else None, dpp))
        return res

    def gpt_param_layout(self, vocab, max_seq, E, H, Lyr, ff):
        n = C.c_int64()
        sizes, ranks = (C.c_int64 * 256)(), (C.c_int64 * 256)()
        self._check(self.lib.ref_gpt_param_count(C.c_int64(vocab), C.c_int64(max_seq), C.c_int64(E), C.c_int64(H),
                                                 C.c_int64(Lyr), C.c_int64(ff), C.byref(n), sizes, ranks))
        return [(sizes[i], ranks[i]) for i in range(n.value)]

    def gpt_step(self, vocab, max_seq, E, H, Lyr, ff, flat_params, tokens, targets, want_grads=True, want_logits=False):
        flat_params = np.ascontiguousarray(flat_params, dtype=np.float32)
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        targets = np.ascontiguousarray(targets, dtype=np.int64)
        batch, seq = tokens.shape
        loss = C.c_float()
        grads = np.empty_like(flat_params) if want_grads else None
        logits = np.empty((batch, seq, vocab), dtype=np.float32) if want_logits else None
        self._check(self.lib.ref_gpt_step(C.c_int64(vocab), C.c_int64(max_seq), C.c_int64(E), C.c_int64(H),
                                          C.c_int64(Lyr), C.c_int64(ff), C.c_int64(batch), C.c_int64(seq),
                                          _fptr(flat_params), _fptr(tokens), _fptr(targets), C.byref(loss),
                                          _fptr(logits) if want_logits else None,
                                          _fptr(grads) if want_grads else None))
        return loss.value, logits, grads


class ReferenceCuda(Reference):
    """The reference's CUDA path (sm_100a build with the b200 binding).  `backend` is the value of
    TENSOR_GEMM_BACKEND the reference reads on every matmul: None (cuBLAS FP32), "custom", or "b200";
    `precision` is TENSOR_GEMM_PRECISION for the b200 backend ("tf32" / "3xtf32").  With fused=True the
    module-level calls (linear, ffn, scaled_dot, mha) go through include/torchengine/te_b200_modules.h, i.e. the
    fused C-ABI calls with their own GradFn nodes inside the reference's autograd engine."""
    PATH = REF_CUDA_PATH

    @staticmethod
    def available():
        return os.path.exists(REF_CUDA_PATH)

    def __init__(self, backend=None, precision="tf32", fused=False):
        super().__init__()
        self.configure(backend, precision, fused)
        self._check(self.lib.ref_use_cuda(1))

    def configure(self, backend=None, precision="tf32", fused=False):
        if backend is None:
            os.environ.pop("TENSOR_GEMM_BACKEND", None)
        else:
            os.environ["TENSOR_GEMM_BACKEND"] = backend
        os.environ["TENSOR_GEMM_PRECISION"] = precision
        self.prefix = "ref_fused_" if fused else "ref_"
        return self

    def cublas_tf32(self, on):
        self._check(self.lib.ref_cuda_cublas_tf32(int(on)))

    def time_matmul(self, M, K, N, warmup=3, iters=10, want_result=False):
        """(ms per call, last product or None) of Tensor::matmul on mt19937(42) uniform(-1,1) operands."""
        ms = C.c_double()
        out = np.empty((M, N), dtype=np.float32) if want_result else None
        self._check(self.lib.ref_cuda_time_matmul(C.c_int64(M), C.c_int64(K), C.c_int64(N), C.c_int32(warmup),
                                                  C.c_int32(iters), C.byref(ms), _fptr(out) if want_result else None))
        return ms.value, out

    def gpt_bench(self, vocab, max_seq, E, H, Lyr, ff, flat_params, tokens, targets, warmup=1, steps=3):
        """(ms per forward+loss+backward step, last loss) of the reference's own GPT on the GPU."""
        flat_params = np.ascontiguousarray(flat_params, dtype=np.float32)
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        targets = np.ascontiguousarray(targets, dtype=np.int64)
        batch, seq = tokens.shape
        ms, loss = C.c_double(), C.c_float()
        self._check(self.lib.ref_cuda_gpt_bench(C.c_int64(vocab), C.c_int64(max_seq), C.c_int64(E), C.c_int64(H),
                                                C.c_int64(Lyr), C.c_int64(ff), C.c_int64(batch), C.c_int64(seq),
                                                _fptr(flat_params), _fptr(tokens), _fptr(targets), C.c_int32(warmup),
                                                C.c_int32(steps), C.byref(ms), C.byref(loss)))
        return ms.value, loss.value
