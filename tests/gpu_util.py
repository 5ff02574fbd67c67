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


def elementwise_rel_err(c, ref, floor=1e-2):
    """max |C - Cref| / |Cref| over the entries with |Cref| >= floor * rms(Cref): the stricter of the two readings of
    "relative error" for products of uniform(-1,1) operands, whose entries come arbitrarily close to zero."""
    ref = np.asarray(ref, dtype=np.float64)
    c = np.asarray(c, dtype=np.float64)
    rms = float(np.sqrt(np.mean(ref * ref)))
    mask = np.abs(ref) >= floor * rms
    if not mask.any():
        return 0.0
    return float((np.abs(c - ref)[mask] / np.abs(ref)[mask]).max())


def rel_err_floored(c, ref, floor):
    """rel_err with the scale floored: for gradients that are zero in exact arithmetic (the key-projection bias of an
    attention layer: softmax ignores a constant added to every key score) and hold only rounding noise in any
    implementation, the reference's included."""
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(np.asarray(c, dtype=np.float64) - ref).max() / max(float(np.abs(ref).max()), floor))
