"""B200 (sm_100a) FP32 matmul backend for TorchEngine: Python host side over the C-ABI library.

`lib`  - ctypes binding of include/te_b200.h (libte_b200.so, built in-tree by build.py).
`ops`  - tensor-level mirror of the reference operators on this path (matmul, Linear, ScaledDot ...),
         taking torch CUDA tensors only as device memory holders.
"""
from . import lib  # noqa: F401
from . import ops  # noqa: F401

__all__ = ["lib", "ops"]
