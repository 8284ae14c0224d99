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


def assert_rel_per_sentence(actual, ref, tol, what="", rtol_big=1e-3, big=1e-6):
    """The tolerance applied to every sentence (leading index) on its own scale, so that a
    sentence with small gradients cannot hide behind a large one; and, on top, every entry
    above `big` times its sentence's maximum must be right to `rtol_big` relative to itself
    (catches entries flushed or truncated by a path that rescales)."""
    actual = np.asarray(actual, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert actual.shape == ref.shape, (actual.shape, ref.shape)
    worst = 0.0
    for b in range(ref.shape[0]):
        e = rel_err(actual[b], ref[b])
        assert e <= tol, f"{what}, sentence {b}: max|d|/max|ref| = {e:.3e} > {tol:.1e}"
        worst = max(worst, e)
        r = ref[b]
        fin = np.isfinite(r)
        if fin.any():
            scale = np.abs(r[fin]).max()
            sel = fin & (np.abs(r) > big * scale)
            if sel.any():
                rel = np.abs(actual[b][sel] - r[sel]) / np.abs(r[sel])
                assert rel.max() <= rtol_big, (f"{what}, sentence {b}: an entry above {big:g} of the sentence "
                                               f"maximum is off by {rel.max():.3e} of itself")
    return worst


_PRECISION_BITS = {"float16": 11, "bfloat16": 8}


def plain_tol_16bit(dtype_name, tol=2e-3):
    """Tolerance of the plain max|d|/max|ref| rule for a gradient rounded once to a 16-bit format.
    Correct rounding alone moves an element by up to half a unit in the last place, 2^-p of a value
    just above a power of two (p significant bits): 2^-11 = 4.9e-4 in fp16, which fits inside the
    2e-3 budget, but 2^-8 = 3.9e-3 in bf16, which does not; for bf16 the plain rule can therefore
    only be held to that rounding bound (the budget itself is checked on the error beyond the
    half-ulp by assert_rel_quantized)."""
    return max(tol, 2.0 ** -_PRECISION_BITS[dtype_name] * 1.01)


def assert_rel_quantized(actual, ref, tol, dtype_name, what=""):
    """Like assert_rel for a result that was rounded ONCE to a 16-bit format: the part of
    each element's error that exceeds the format's own half-ulp must stay within
    tol * max|ref|.  (bf16 keeps 8 significant bits, so correct rounding alone is off by up
    to 2^-9..2^-8 of an element, more than the 2e-3 budget; fp16 keeps 11 bits.)"""
    actual = np.asarray(actual, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert actual.shape == ref.shape
    assert np.isfinite(actual).all() and np.isfinite(ref).all()
    bits = _PRECISION_BITS[dtype_name]
    mag = np.abs(ref)
    expo = np.floor(np.log2(np.where(mag > 0, mag, 1.0)))
    half_ulp = np.where(mag > 0, 2.0 ** (expo - bits), 0.0)
    if dtype_name == "float16":
        half_ulp = np.maximum(half_ulp, 2.0 ** -25)   # subnormal spacing
    excess = np.maximum(np.abs(actual - ref) - half_ulp, 0.0)
    scale = mag.max() if mag.max() > 0 else 1.0
    e = float(excess.max() / scale)
    assert e <= tol, f"{what}: error beyond the {dtype_name} half-ulp = {e:.3e} * max|ref| > {tol:.1e}"
    return e
