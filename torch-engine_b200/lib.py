"""ctypes binding of the C ABI declared in include/te_b200.h.

Loading fails loudly when libte_b200.so has not been built: there is no Python or CPU fallback.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libte_b200.so")

TE_OK = 0
TE_ERR_BAD_ARGUMENT, TE_ERR_UNSUPPORTED_LAYOUT, TE_ERR_SHAPE_NDIM, TE_ERR_SHAPE_INNER = 1, 2, 3, 4
TE_ERR_SHAPE_BROADCAST, TE_ERR_WORKSPACE, TE_ERR_CUDA, TE_ERR_DEVICE_TIMEOUT, TE_ERR_NO_DEVICE = 5, 6, 7, 8, 9
TE_ROW_MAJOR, TE_COL_MAJOR = 0, 1
TE_PREC_TF32, TE_PREC_3XTF32 = 0, 1
TE_EPI_NONE, TE_EPI_BIAS, TE_EPI_BIAS_GELU = 0, 1, 2
TE_SCALE_NONE, TE_SCALE_MUL, TE_SCALE_DIV = 0, 1, 2
TE_B200_STATIC_SCRATCH_BYTES = 64 << 20

c_float_p = C.POINTER(C.c_float)
c_i64_p = C.POINTER(C.c_int64)


class GemmDesc(C.Structure):
    """struct te_gemm_desc"""
    _fields_ = [
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
        ("a_major", C.c_int32), ("b_major", C.c_int32),
        ("batch_outer", C.c_int64), ("batch_inner", C.c_int64),
        ("a_stride_outer", C.c_int64), ("a_stride_inner", C.c_int64),
        ("b_stride_outer", C.c_int64), ("b_stride_inner", C.c_int64),
        ("c_stride_outer", C.c_int64), ("c_stride_inner", C.c_int64),
        ("alpha", C.c_float), ("scale_mode", C.c_int32), ("epilogue", C.c_int32),
        ("bias", C.c_void_p), ("preact_out", C.c_void_p), ("residual", C.c_void_p),
        ("precision", C.c_int32), ("reserved", C.c_int32),
    ]


class AttnDesc(C.Structure):
    """struct te_attn_desc"""
    _fields_ = [
        ("B", C.c_int64), ("H", C.c_int64), ("T", C.c_int64), ("d", C.c_int64),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("q_strides", C.c_int64 * 3), ("k_strides", C.c_int64 * 3), ("v_strides", C.c_int64 * 3),
        ("p_out", C.c_void_p), ("o", C.c_void_p), ("o_strides", C.c_int64 * 3),
        ("precision", C.c_int32), ("reserved", C.c_int32),
    ]


class AttnBwdDesc(C.Structure):
    """struct te_attn_bwd_desc"""
    _fields_ = [
        ("B", C.c_int64), ("H", C.c_int64), ("T", C.c_int64), ("d", C.c_int64),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("q_strides", C.c_int64 * 3), ("k_strides", C.c_int64 * 3), ("v_strides", C.c_int64 * 3),
        ("p", C.c_void_p), ("o", C.c_void_p), ("o_strides", C.c_int64 * 3),
        ("d_o", C.c_void_p), ("d_o_strides", C.c_int64 * 3),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("dq_strides", C.c_int64 * 3), ("dk_strides", C.c_int64 * 3), ("dv_strides", C.c_int64 * 3),
        ("precision", C.c_int32), ("reserved", C.c_int32),
    ]


class MhaDesc(C.Structure):
    """struct te_mha_desc"""
    _fields_ = [("B", C.c_int64), ("T", C.c_int64), ("E", C.c_int64), ("H", C.c_int64), ("x", C.c_void_p)] + \
               [(n, C.c_void_p) for n in ("wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo", "q", "k", "v", "p", "attn", "y",
                                          "residual")] + [("precision", C.c_int32), ("reserved", C.c_int32),
                                                         ("wqkv", C.c_void_p), ("ld_qkv", C.c_int64)]


class MhaBwdDesc(C.Structure):
    """struct te_mha_bwd_desc"""
    _fields_ = [("B", C.c_int64), ("T", C.c_int64), ("E", C.c_int64), ("H", C.c_int64)] + \
               [(n, C.c_void_p) for n in ("x", "wq", "wk", "wv", "wo", "q", "k", "v", "p", "attn", "dy", "dx", "dx_residual",
                                          "dwq", "dbq", "dwk", "dbk", "dwv", "dbv", "dwo", "dbo", "dq", "dk", "dv",
                                          "dattn")] + [("accumulate", C.c_int32), ("precision", C.c_int32),
                                                      ("wqkv", C.c_void_p), ("dwqkv", C.c_void_p), ("ld_qkv", C.c_int64)]


# name -> (restype, argtypes); every symbol include/te_b200.h declares
SIGNATURES = {
    "te_b200_init": (C.c_int, [C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]),
    "te_b200_destroy": (C.c_int, [C.c_void_p]),
    "te_b200_gemm_workspace_size": (C.c_int, [C.POINTER(GemmDesc), C.POINTER(C.c_size_t)]),
    "te_b200_launch_count": (C.c_int64, [C.c_void_p]),
    "te_b200_last_error": (C.c_char_p, []),
    "te_b200_status_string": (C.c_char_p, [C.c_int]),
    "te_b200_check_device_status": (C.c_int, [C.c_void_p]),
    "te_b200_gemm_f32": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p]),
    "te_b200_matmul_nd": (C.c_int, [C.c_void_p, C.c_void_p, c_i64_p, c_i64_p, C.c_int,
                                    C.c_void_p, c_i64_p, c_i64_p, C.c_int,
                                    C.c_void_p, c_i64_p, C.POINTER(C.c_int), C.c_int, C.c_void_p]),
    "te_b200_gemm_f32_host": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc)]),
    "te_b200_gemm_3xtf32_static": (C.c_int, [C.POINTER(GemmDesc), C.c_void_p, C.POINTER(C.c_int)]),
    "te_b200_softmax_rows_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "te_b200_softmax_backward_rows_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                                    C.c_int64, C.c_void_p]),
    "te_b200_gelu_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "te_b200_gelu_backward_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "te_b200_colsum_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "te_b200_linear_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "te_b200_linear_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "te_b200_linear_backward_gelu": (C.c_int, [C.c_void_p] + [C.c_void_p] * 7 + [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "te_b200_linear_backward_ex": (C.c_int, [C.c_void_p] + [C.c_void_p] * 9 + [C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "te_b200_mha_forward": (C.c_int, [C.c_void_p, C.POINTER(MhaDesc), C.c_void_p]),
    "te_b200_mha_backward": (C.c_int, [C.c_void_p, C.POINTER(MhaBwdDesc), C.c_void_p]),
    "te_b200_set_wait_limit_ns": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "te_b200_selftest_wait_timeout": (C.c_int, [C.c_void_p, C.c_void_p]),
    "te_b200_gemm_plan": (C.c_int, [C.POINTER(GemmDesc), C.c_int, C.c_size_t, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "te_b200_attention_forward": (C.c_int, [C.c_void_p, C.POINTER(AttnDesc), C.c_void_p]),
    "te_b200_attention_backward": (C.c_int, [C.c_void_p, C.POINTER(AttnBwdDesc), C.c_void_p]),
    "te_b200_layernorm_forward": (C.c_int, [C.c_void_p] + [C.c_void_p] * 4 + [C.c_int64, C.c_int64, C.c_float, C.c_void_p]),
    "te_b200_layernorm_backward": (C.c_int, [C.c_void_p] + [C.c_void_p] * 6 + [C.c_int64, C.c_int64, C.c_float, C.c_void_p]),
    "te_b200_layernorm_backward_ex": (C.c_int, [C.c_void_p] + [C.c_void_p] * 8 + [C.c_int64, C.c_int64, C.c_float, C.c_void_p]),
    "te_b200_embedding_forward": (C.c_int, [C.c_void_p] + [C.c_void_p] * 4 + [C.c_int64] * 4 + [C.c_void_p]),
    "te_b200_embedding_backward": (C.c_int, [C.c_void_p] + [C.c_void_p] * 3 + [C.c_int64] * 3 + [C.c_void_p]),
    "te_b200_cross_entropy": (C.c_int, [C.c_void_p] + [C.c_void_p] * 4 + [C.c_float, C.c_int64, C.c_int64, C.c_void_p]),
    "te_b200_comm_unique_id": (C.c_int, [C.c_void_p]),
    "te_b200_comm_init": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "te_b200_comm_destroy": (C.c_int, [C.c_void_p]),
    "te_b200_comm_rank": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "te_b200_all_gather_columns": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                              C.c_int64, C.c_void_p]),
    "te_b200_all_gather_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "te_b200_all_reduce_batch_mean": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "te_b200_gemm_f32_host_sharded": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc), C.c_int64]),
    "te_b200_shard_range": (C.c_int, [C.c_int64, C.c_int, C.c_int, C.c_int64, c_i64_p, c_i64_p]),
}

_lib = None


class BackendError(RuntimeError):
    """A non-zero status from the C ABI; `.status` holds the TE_ERR_* code."""

    def __init__(self, status, message):
        super().__init__(message)
        self.status = status


def load():
    """dlopens libte_b200.so and types every entry point.  Raises if the library is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libte_b200.so is not built (expected at %s); run `python torch-engine_b200/build.py`. "
            "This backend has no CPU or PyTorch fallback." % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status):
    """Converts a non-zero status into BackendError carrying the library's message."""
    if status != TE_OK:
        lib = load()
        msg = lib.te_b200_last_error().decode() or lib.te_b200_status_string(status).decode()
        raise BackendError(status, msg)


def status_string(status):
    return load().te_b200_status_string(status).decode()


def shard_range(total, world, rank, align=1):
    """(begin, count) of the units rank `rank` of `world` owns; see te_b200_shard_range."""
    b, n = C.c_int64(), C.c_int64()
    check(load().te_b200_shard_range(total, world, rank, align, C.byref(b), C.byref(n)))
    return b.value, n.value


def matmul_shape(a_shape, a_strides, b_shape, b_strides):
    """Result shape of an N-D matmul, validated exactly as Tensor::matmul does; needs no GPU."""
    na, nb = len(a_shape), len(b_shape)
    out = (C.c_int64 * 8)()
    nd = C.c_int()
    check(load().te_b200_matmul_nd(None, None, (C.c_int64 * max(na, 1))(*a_shape), (C.c_int64 * max(na, 1))(*a_strides), na,
                                   None, (C.c_int64 * max(nb, 1))(*b_shape), (C.c_int64 * max(nb, 1))(*b_strides), nb,
                                   None, out, C.byref(nd), TE_PREC_TF32, None))
    return tuple(out[i] for i in range(nd.value))
