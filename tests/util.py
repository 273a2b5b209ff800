"""Shared helpers for the parity tests."""
from __future__ import annotations

import numpy as np


def ulp_diff(a: np.ndarray, b: np.ndarray) -> int:
    """Largest distance in units in the last place between two float arrays of the same dtype
    (NaNs must coincide)."""
    a = np.atleast_1d(np.asarray(a))
    b = np.atleast_1d(np.asarray(b))
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    if a.size == 0:
        return 0
    nan_a, nan_b = np.isnan(a), np.isnan(b)
    assert np.array_equal(nan_a, nan_b), "NaN pattern differs"
    it = {2: np.int16, 4: np.int32, 8: np.int64}[a.dtype.itemsize]
    ia = a.view(it).astype(np.int64)
    ib = b.view(it).astype(np.int64)
    sign = np.int64(1) << (8 * a.dtype.itemsize - 1)
    ia = np.where(ia < 0, -(ia + sign) , ia)   # map to a monotone integer line
    ib = np.where(ib < 0, -(ib + sign), ib)
    d = np.abs(ia - ib)
    d[nan_a] = 0
    return int(d.max())


def to_np(t):
    return t.detach().cpu().numpy()


def rel_err(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    denom = np.maximum(np.abs(b), 1e-30)
    return float(np.max(np.abs(a - b) / denom)) if a.size else 0.0


def max_rel_to_scale(a, b):
    """max |a-b| / max|b| — the tolerance form used for reductions and matmul."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    if a.size == 0:
        return 0.0
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))
