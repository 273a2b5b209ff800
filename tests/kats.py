"""Loader for the known-answer fixtures in tests/golden/kats (made by tests/golden/extract_kats.py)."""
from __future__ import annotations

import glob
import json
import os

import numpy as np

KATS_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kats")

# Ops of the reference that are outside the operator path (CNN ops) or whose test relies on attribute
# forms of shape-only ops that this build does not take (Constant's value_floats / value_ints ...).
OUT_OF_SCOPE_OPS = {"Conv", "GlobalAveragePool", "MaxPool", "Constant"}


def _val(v):
    if v == "nan":
        return float("nan")
    if v == "inf":
        return float("inf")
    if v == "-inf":
        return float("-inf")
    return v


def array(dims, dtype, data):
    return np.array([_val(v) for v in data], dtype=np.dtype(dtype)).reshape(dims)


def load_cases():
    cases = []
    for path in sorted(glob.glob(os.path.join(KATS_DIR, "*.json"))):
        base = os.path.basename(path)
        if base.startswith("_") or base == "attention.json":
            continue
        for c in json.load(open(path)):
            if c["op"] in OUT_OF_SCOPE_OPS:
                continue
            c["id"] = f"{base[:-5]}::{c['name']}"
            cases.append(c)
    return cases


def attention():
    return json.load(open(os.path.join(KATS_DIR, "attention.json")))


def attr_value(a):
    if a["kind"] == "tensor":
        return array(a["dims"], a["dtype"] or "float32", a["value"])
    return a["value"]


def check(case, out_flat: np.ndarray):
    exp = case["expect"]
    want = np.array([_val(v) for v in exp["values"]], dtype=np.float64 if out_flat.dtype.kind == "f" else out_flat.dtype)
    assert out_flat.size == want.size, (case["id"], out_flat.shape, want.shape)
    if exp["kind"] == "eq":
        # the Rust literals are typed as the output dtype, so compare after rounding to it
        assert np.array_equal(out_flat, want.astype(out_flat.dtype), equal_nan=True), (case["id"], out_flat, want)
    else:
        assert np.all(np.abs(out_flat.astype(np.float64) - want.astype(np.float64)) <= exp["eps"] + 1e-12), (case["id"], out_flat, want)
