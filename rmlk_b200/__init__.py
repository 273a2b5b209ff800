"""rmlk_b200 — B200 (sm_100a) operator kernels for the rmlk runtime's op dispatch, behind a C ABI.

`rmlk_b200.kernels` binds the kernel launchers of include/rmlk_b200.h; `rmlk_b200.runtime` binds the
host-side op backends / executor of include/rmlk_b200_runtime.h and mirrors the reference's `OpTest`
harness.  Everything computes on the GPU through librmlk_b200.so; there is no CPU fallback.
"""
from . import dtypes  # noqa: F401
from ._lib import LIB_PATH, LibraryMissing, lib  # noqa: F401

__all__ = ["dtypes", "lib", "LIB_PATH", "LibraryMissing"]
