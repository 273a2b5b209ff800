"""Run reference call plans on the host build of the reference kernels.  TEST INFRASTRUCTURE ONLY.

`oracle/_ref/libref_cpu.so` is built by `oracle/Makefile` from the reference's own
cuda/src/ptx/*.cu sources (compiled as C++ behind oracle/ref_shim.h).  `run(plan)` forwards the
plan's positional arguments to the entry point through ref_driver.cpp:ref_launch, on `threads` host
threads (1 = the scalar port used as bit oracle; all cores = the timed CPU baseline).
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libref_cpu.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.ref_launch.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_uint64)]
        _lib.ref_launch.restype = ctypes.c_int
        _lib.ref_max_threads.restype = ctypes.c_int
    return _lib


def max_threads() -> int:
    return int(lib().ref_max_threads())


def run(plan, threads: int = 1):
    """Execute one plan; returns plan.out (filled in place)."""
    l = lib()
    fn = ctypes.cast(getattr(l, plan.symbol), ctypes.c_void_p).value
    vals = []
    keep = []
    for kind, v in plan.args:
        if kind in ("in", "out"):
            if v is None:
                vals.append(0)
            else:
                assert v.flags["C_CONTIGUOUS"]
                keep.append(v)
                # zero-sized arrays still need a valid (never dereferenced) pointer
                vals.append(v.ctypes.data if v.size else 0)
        elif kind == "u64":
            vals.append(int(v))
        elif kind == "i64":
            vals.append(int(v) & 0xFFFFFFFFFFFFFFFF)
        elif kind == "bool":
            vals.append(1 if v else 0)
        else:
            raise ValueError(kind)
    arr = (ctypes.c_uint64 * len(vals))(*vals)
    rc = l.ref_launch(fn, int(threads), len(vals), arr)
    if rc != 0:
        raise RuntimeError(f"ref_launch({plan.symbol}) failed: {rc}")
    return plan.out
