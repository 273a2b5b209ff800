"""GPU: the allocation-free MatMul entry point (rmlk_b200_matmul_static) against rmlk_b200_matmul_ex.

Some callers of the library may not allocate device memory (a serving loop that must not stall the device, a
fixed memory budget, a plug-in that only receives buffers), so this entry point keeps the split-K scratch in
an array built into the library.  It must give what the regular entry point gives with a caller-provided
workspace, on repeated calls (the array keeps the previous call's contents), and must refuse shapes whose
scratch does not fit.  The file name sorts last so that a run that stops at the first failure has already
run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn, stream, m, n, k, a, w, out, extra):
    from rmlk_b200 import dtypes as dt
    return fn(ctypes.c_void_p(stream), dt.F32, ctypes.c_int64(1), ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(k),
              ctypes.c_void_p(a.data_ptr()), ctypes.c_int64(0), ctypes.c_void_p(w.data_ptr()), ctypes.c_int64(0),
              ctypes.c_void_p(out.data_ptr()), ctypes.c_int64(m * n), *extra)


@pytest.mark.parametrize("shape", [(1, 2048, 2048), (8, 512, 2048), (16, 2048, 8192), (64, 256, 8192), (128, 512, 4096)])
def test_static_scratch_matmul_matches_regular_entry_point(cuda, shape):
    from rmlk_b200 import kernels as K
    from rmlk_b200._lib import last_error, lib
    m, n, k = shape
    l = lib()
    l.rmlk_b200_matmul_static_scratch_bytes.restype = ctypes.c_size_t
    from rmlk_b200 import dtypes as dt
    need = K.matmul_workspace_bytes(1, m, n, k)
    assert need > 0, "case must exercise the split-K scratch"
    assert l.rmlk_b200_matmul_static_supported(dt.F32, ctypes.c_int64(1), ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(k)) == 1
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ws = torch.empty(need // 4, device="cuda")
    for trial in range(2):  # two calls in a row: the second one starts from the first one's leftovers
        a = torch.randn(m, k, device="cuda")
        w = torch.randn(k, n, device="cuda") * 0.05
        want = torch.empty(m, n, device="cuda")
        got = torch.full((m, n), float("nan"), device="cuda")
        rc = _call(l.rmlk_b200_matmul_ex, stream, m, n, k, a, w, want,
                   [ctypes.c_void_p(ws.data_ptr()), ctypes.c_size_t(need), ctypes.c_void_p(status.data_ptr())])
        assert rc == 0, last_error()
        rc = _call(l.rmlk_b200_matmul_static, stream, m, n, k, a, w, got, [ctypes.c_void_p(status.data_ptr())])
        assert rc == 0, last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) <= 1e-4 * scale, (shape, trial)   # the MatMul tolerance of the other tests
        ref = a.double() @ w.double()
        assert float((got.double() - ref).abs().max()) <= 1e-4 * float(ref.abs().max())


def test_static_scratch_matmul_rejects_oversized_shapes(cuda):
    from rmlk_b200 import kernels as K
    from rmlk_b200._lib import last_error, lib
    l = lib()
    l.rmlk_b200_matmul_static_scratch_bytes.restype = ctypes.c_size_t
    m, n, k = 256, 512, 8192   # eighteen K-splits of 512 KiB each: more than the 8 MiB array
    from rmlk_b200 import dtypes as dt
    assert K.matmul_workspace_bytes(1, m, n, k) > l.rmlk_b200_matmul_static_scratch_bytes()
    assert l.rmlk_b200_matmul_static_supported(dt.F32, ctypes.c_int64(1), ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(k)) == 0
    a = torch.randn(m, k, device="cuda")
    w = torch.randn(k, n, device="cuda")
    out = torch.zeros(m, n, device="cuda")
    rc = _call(l.rmlk_b200_matmul_static, torch.cuda.current_stream().cuda_stream, m, n, k, a, w, out, [ctypes.c_void_p(0)])
    assert rc == 1 and "scratch" in last_error()
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0, "nothing may be launched for a rejected shape"
