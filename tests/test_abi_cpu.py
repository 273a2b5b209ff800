"""The C-ABI library without a GPU: it loads, it exports every entry point the headers declare, and its pure host
functions (status mapping, Slice parameter normalisation, size queries) answer.  No kernel is launched here."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_entry_points():
    names = []
    for h in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        src = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names += re.findall(r"RMLK_API\s+[\w\s\*]+?\b(rmlk_\w+)\s*\(", src)
    return names


def test_library_exports_every_declared_entry_point():
    from rmlk_b200._lib import lib
    names = declared_entry_points()
    assert len(names) > 60 and len(set(names)) == len(names)
    missing = [n for n in names if not hasattr(lib(), n)]
    assert not missing, missing


def test_status_word_mapping():
    """1 / 2 are the Gather / ScatterND codes of the reference (ScatterNdError::KernelFailed, backend/scatter_nd.rs:198-203);
    5 is what a MatMul kernel stores when one of its bounded waits expires."""
    from rmlk_b200._lib import lib
    f = lib().rmlk_runtime_status_to_error
    f.restype = ctypes.c_int
    RMLK_OK, RMLK_ERR_TIMEOUT, RMLK_ERR_KERNEL_STATUS = 0, 5, 6
    assert f(0) == RMLK_OK
    assert f(1) == RMLK_ERR_KERNEL_STATUS and f(2) == RMLK_ERR_KERNEL_STATUS
    assert f(5) == RMLK_ERR_TIMEOUT


def test_host_only_queries():
    from rmlk_b200._lib import lib
    L = lib()
    L.rmlk_b200_dtype_size.restype = ctypes.c_size_t
    assert L.rmlk_b200_dtype_size(1) in (2, 4)          # a float type of the DataType enumeration
    L.rmlk_b200_matmul_static_scratch_bytes.restype = ctypes.c_size_t
    assert L.rmlk_b200_matmul_static_scratch_bytes() == 8 << 20
    L.rmlk_b200_version.restype = ctypes.c_char_p
    assert b"sm_100a" in L.rmlk_b200_version()
