"""Shared test helpers: golden fixtures and seeded synthetic inputs."""

import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def full_rope(half_table: np.ndarray) -> np.ndarray:
    """(S, d/2) -> (S, d): both halves of the head share the rotary angle."""
    return np.concatenate((half_table, half_table), axis=-1)


# ---- evidence that a differing code is a rounding tie, not an error (reductions in another order move a float32 value
#      by a few ulp; a code may differ only where that value sits on a rounding boundary) ----

def assert_round_ties(x: np.ndarray, a: np.ndarray, b: np.ndarray, tol: float, what: str) -> dict:
    """x: float64 pre-rounding values (residual / scale); a, b: integer codes two implementations chose.  Wherever they
    differ, they must be the two neighbours of x and x must lie within `tol` of the half-way point between them."""
    x, a, b = np.asarray(x, np.float64), np.asarray(a, np.int64), np.asarray(b, np.int64)
    diff = a != b
    n = int(diff.sum())
    worst = 0.0
    if n:
        lo = np.minimum(a[diff], b[diff])
        assert np.all(np.abs(a[diff] - b[diff]) == 1), f"{what}: a code differs by more than one level"
        dist = np.abs(x[diff] - (lo + 0.5))
        worst = float(dist.max())
        assert worst < tol, f"{what}: a differing code is {worst:.3e} away from a rounding boundary (allowed {tol:.1e})"
    return {"differing": n, "of": int(diff.size), "worst_distance_to_tie": worst}


def assert_bucket_ties(y: np.ndarray, mids: np.ndarray, a: np.ndarray, b: np.ndarray, tol: float, what: str) -> dict:
    """y: float64 values that were bucketized against `mids`; a, b: the bucket indices two implementations chose."""
    y, a, b = np.asarray(y, np.float64), np.asarray(a, np.int64), np.asarray(b, np.int64)
    diff = a != b
    n = int(diff.sum())
    worst = 0.0
    if n:
        lo = np.minimum(a[diff], b[diff])
        assert np.all(np.abs(a[diff] - b[diff]) == 1), f"{what}: an index differs by more than one level"
        dist = np.abs(y[diff] - np.asarray(mids, np.float64)[lo])
        worst = float(dist.max())
        assert worst < tol, f"{what}: a differing index is {worst:.3e} away from a bucket boundary (allowed {tol:.1e})"
    return {"differing": n, "of": int(diff.size), "worst_distance_to_tie": worst}


def assert_fp16_rounding_ties(x64: np.ndarray, a16: np.ndarray, b16: np.ndarray, rel_tol: float, what: str) -> dict:
    """x64: float64 values before the fp16 rounding; a16, b16: the fp16 results of two implementations.  Wherever they
    differ they must be adjacent fp16 numbers and x64 must lie within rel_tol * |x| of the midpoint between them."""
    a16, b16 = np.asarray(a16, np.float16), np.asarray(b16, np.float16)
    diff = a16.view(np.uint16) != b16.view(np.uint16)
    n = int(diff.sum())
    worst, max_ulp = 0.0, 0
    if n:
        ua, ub = a16.view(np.uint16)[diff].astype(np.int64), b16.view(np.uint16)[diff].astype(np.int64)
        max_ulp = int(np.abs(ua - ub).max())  # same sign assumed below: adjacent bit patterns are adjacent numbers
        assert max_ulp == 1, f"{what}: fp16 values differ by {max_ulp} ulp"
        mid = (a16[diff].astype(np.float64) + b16[diff].astype(np.float64)) / 2
        rel = np.abs(np.asarray(x64, np.float64)[diff] - mid) / np.maximum(np.abs(mid), 1e-30)
        worst = float(rel.max())
        assert worst < rel_tol, f"{what}: a differing fp16 value is {worst:.3e} (relative) away from a rounding boundary"
    return {"differing": n, "of": int(diff.size), "max_ulp": max_ulp, "worst_rel_distance_to_tie": worst}
