"""Shared comparison helpers for the parity tests."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def rel_err(actual, ref):
    """max|actual-ref| / max|ref| over the finite entries of ref; non-finite entries
    (the -inf of impossible sentences / masked links) must match exactly."""
    actual = np.asarray(actual, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert actual.shape == ref.shape, (actual.shape, ref.shape)
    fin = np.isfinite(ref)
    assert np.array_equal(actual[~fin], ref[~fin], equal_nan=True), "non-finite pattern differs"
    if not fin.any():
        return 0.0
    scale = np.abs(ref[fin]).max()
    if scale == 0:
        scale = 1.0
    return float(np.abs(actual[fin] - ref[fin]).max() / scale)


def assert_rel(actual, ref, tol, what=""):
    e = rel_err(actual, ref)
    assert e <= tol, f"{what}: max|d|/max|ref| = {e:.3e} > {tol:.1e}"
    return e
