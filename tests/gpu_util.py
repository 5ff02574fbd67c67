"""Helpers for the GPU parity tests: error metrics and the tolerances of the two precision modes."""
import numpy as np

# max |C - Cref| / max |Cref| against the reference's FP32 result on the same inputs
TOL_REL = {"tf32": 2e-3, "3xtf32": 1e-5}


def rel_err(c, ref):
    ref = np.asarray(ref, dtype=np.float64)
    denom = np.abs(ref).max()
    if denom == 0:
        return float(np.abs(np.asarray(c, dtype=np.float64)).max())
    return float(np.abs(np.asarray(c, dtype=np.float64) - ref).max() / denom)


def assert_close(c, ref, precision, what=""):
    e = rel_err(c, ref)
    assert e <= TOL_REL[precision], f"{what}: relative error {e:.3e} > {TOL_REL[precision]:.0e} ({precision})"
    return e
