"""ctypes loader for librmlk_b200.so.

The library is the product; there is no fallback.  If it is missing or fails to load, importing
anything that needs it raises with the build command to run.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "librmlk_b200.so")
_lib = None


class LibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} not found: build it with `python -m rmlk_b200.build` (needs nvcc). "
                "rmlk_b200 has no CPU or PyTorch fallback.")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.rmlk_b200_last_error.restype = ctypes.c_char_p
        _lib.rmlk_b200_version.restype = ctypes.c_char_p
        _lib.rmlk_b200_dtype_size.restype = ctypes.c_size_t
        _lib.rmlk_b200_matmul_workspace_bytes.restype = ctypes.c_size_t
        _lib.rmlk_b200_matmul_tp_workspace_bytes.restype = ctypes.c_size_t
    return _lib


def last_error() -> str:
    return lib().rmlk_b200_last_error().decode()
