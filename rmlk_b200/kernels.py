"""Python bindings of the kernel launchers declared in include/rmlk_b200.h.

Thin mirror of the reference's launch wrappers (cuda/src/kernels/*.rs): arguments are device buffers
(torch CUDA tensors are used purely as memory handles) plus host-side shapes / strides, and every
call lands in librmlk_b200.so.  Outputs are allocated by the caller or, for convenience in tests, by
these helpers with `torch.empty` — the library itself never allocates.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import dtypes as dt
from ._lib import last_error, lib

BIN = {"add": 0, "sub": 1, "mul": 2, "div": 3, "equal": 4, "greater": 5}
UN = {"sqrt": 0, "neg": 1, "sin": 2, "cos": 3, "sigmoid": 4, "relu": 5}
SCATTER = {"none": 0, "add": 1, "mul": 2, "max": 3, "min": 4}


class RmlkError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"rmlk_b200 error {code}: {msg}")
        self.code = code
        self.msg = msg


def _check(rc: int):
    if rc != 0:
        raise RmlkError(rc, last_error())


def _i64(vals: Sequence[int]):
    return (ctypes.c_int64 * max(len(vals), 1))(*[int(v) for v in vals])


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*ts):
    for t in ts:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("rmlk_b200 kernels take contiguous CUDA tensors")


def dense_strides(shape):
    s = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        s[i] = s[i + 1] * shape[i + 1]
    return s


def broadcast_strides(shape, out_shape):
    """Element strides of a dense tensor of `shape` viewed as `out_shape` (0 on broadcast dims),
    right-aligned — reference runtime/src/utils/mod.rs:93-111."""
    st = dense_strides(shape)
    n = len(out_shape)
    r = [0] * n
    for i in range(n):
        j = i - (n - len(shape))
        if j >= 0 and shape[j] == out_shape[i] and shape[j] != 1:
            r[i] = st[j]
    return r


def _kshape(t):
    return [1] if t.dim() == 0 else list(t.shape)


def binary(op: str, a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(a, b, out)
    osh = list(torch.broadcast_shapes(tuple(_kshape(a)), tuple(_kshape(b))))
    odt = torch.bool if op in ("equal", "greater") else a.dtype
    if out is None:
        out = torch.empty(osh if (a.dim() or b.dim()) else [], dtype=odt, device=a.device)
    _check(lib().rmlk_b200_binary(_stream(), BIN[op], dt.from_torch(a.dtype), len(osh), _i64(osh),
                                  _i64(broadcast_strides(_kshape(a), osh)), _i64(broadcast_strides(_kshape(b), osh)),
                                  _ptr(a), _ptr(b), _ptr(out)))
    return out


def pow_(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(a, b, out)
    osh = list(torch.broadcast_shapes(tuple(_kshape(a)), tuple(_kshape(b))))
    if out is None:
        out = torch.empty(osh if (a.dim() or b.dim()) else [], dtype=a.dtype, device=a.device)
    _check(lib().rmlk_b200_pow(_stream(), dt.from_torch(a.dtype), dt.from_torch(b.dtype), len(osh), _i64(osh),
                               _i64(broadcast_strides(_kshape(a), osh)), _i64(broadcast_strides(_kshape(b), osh)),
                               _ptr(a), _ptr(b), _ptr(out)))
    return out


def unary(op: str, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(x, out)
    if out is None:
        out = torch.empty_like(x)
    _check(lib().rmlk_b200_unary(_stream(), UN[op], dt.from_torch(x.dtype), ctypes.c_size_t(x.numel()), _ptr(x), _ptr(out)))
    return out


def cast(x: torch.Tensor, to: torch.dtype, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(x, out)
    if out is None:
        out = torch.empty(x.shape, dtype=to, device=x.device)
    _check(lib().rmlk_b200_cast(_stream(), dt.from_torch(x.dtype), dt.from_torch(to), ctypes.c_size_t(x.numel()), _ptr(x), _ptr(out)))
    return out


def where(cond: torch.Tensor, x: torch.Tensor, y: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(cond, x, y, out)
    osh = list(torch.broadcast_shapes(tuple(_kshape(x)), tuple(_kshape(y)), tuple(_kshape(cond))))
    if out is None:
        out = torch.empty(osh if (x.dim() or y.dim() or cond.dim()) else [], dtype=x.dtype, device=x.device)
    _check(lib().rmlk_b200_where(_stream(), dt.from_torch(x.dtype), len(osh), _i64(osh),
                                 _i64(broadcast_strides(_kshape(x), osh)), _i64(broadcast_strides(_kshape(y), osh)),
                                 _i64(broadcast_strides(_kshape(cond), osh)), _ptr(x), _ptr(y), _ptr(cond), _ptr(out)))
    return out


def reduce_mean(x: torch.Tensor, axes: Sequence[int], keepdims: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(x, out)
    sh = _kshape(x)
    rank = len(sh)
    ax = sorted(a + rank if a < 0 else a for a in axes)
    osh = [1 if d in ax else sh[d] for d in range(rank)] if keepdims else [sh[d] for d in range(rank) if d not in ax]
    if out is None:
        out = torch.empty(osh, dtype=x.dtype, device=x.device)
    _check(lib().rmlk_b200_reduce_mean(_stream(), dt.from_torch(x.dtype), rank, _i64(sh), len(ax), _i64(ax), _ptr(x), _ptr(out)))
    return out


def softmax(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(x, out)
    if out is None:
        out = torch.empty_like(x)
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    _check(lib().rmlk_b200_softmax(_stream(), dt.from_torch(x.dtype), ctypes.c_int64(rows), ctypes.c_int64(cols), _ptr(x), _ptr(out)))
    return out


def gather(data: torch.Tensor, indices: torch.Tensor, axis: int = 0, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(data, indices, status)
    axis = axis + data.dim() if axis < 0 else axis
    sh = list(data.shape)
    outer = 1
    for d in sh[:axis]:
        outer *= d
    inner = 1
    for d in sh[axis + 1:]:
        inner *= d
    osh = sh[:axis] + list(indices.shape) + sh[axis + 1:]
    out = torch.empty(osh, dtype=data.dtype, device=data.device)
    _check(lib().rmlk_b200_gather(_stream(), data.element_size(), dt.from_torch(indices.dtype), ctypes.c_int64(outer),
                                  ctypes.c_int64(sh[axis]), ctypes.c_int64(inner), ctypes.c_int64(indices.numel()),
                                  _ptr(data), _ptr(indices), _ptr(out), _ptr(status)))
    return out


def scatter_nd(data: torch.Tensor, indices: torch.Tensor, updates: torch.Tensor, reduction: str = "none",
               status: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(data, indices, updates, status)
    k = indices.shape[-1] if indices.dim() > 1 else 1
    n_tuples = indices.numel() // k if k else 0
    out = torch.empty_like(data)
    _check(lib().rmlk_b200_scatter_nd(_stream(), SCATTER[reduction], dt.from_torch(data.dtype), data.dim(), _i64(list(data.shape)),
                                      ctypes.c_int64(n_tuples), k, _ptr(data), _ptr(indices), _ptr(updates), _ptr(out), _ptr(status)))
    return out


def slice_params(in_shape, starts, ends, axes=None, steps=None):
    rank = len(in_shape)
    os_, ost, osh = _i64([0] * rank), _i64([0] * rank), _i64([0] * rank)
    _check(lib().rmlk_b200_slice_params(rank, _i64(in_shape), len(starts), _i64(starts), _i64(ends),
                                        None if axes is None else _i64(axes), None if steps is None else _i64(steps), os_, ost, osh))
    return list(os_)[:rank], list(ost)[:rank], list(osh)[:rank]


def slice_(x: torch.Tensor, starts, ends, axes=None, steps=None) -> torch.Tensor:
    _require_cuda(x)
    st, sp, osh = slice_params(list(x.shape), starts, ends, axes, steps)
    out = torch.empty(osh, dtype=x.dtype, device=x.device)
    _check(lib().rmlk_b200_slice(_stream(), x.element_size(), x.dim(), _i64(list(x.shape)), _i64(osh), _i64(st), _i64(sp), _ptr(x), _ptr(out)))
    return out


def transpose(x: torch.Tensor, perm=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(x)
    if perm is None:
        perm = list(range(x.dim()))[::-1]
    if out is None:
        out = torch.empty([x.shape[p] for p in perm], dtype=x.dtype, device=x.device)
    _check(lib().rmlk_b200_transpose(_stream(), x.element_size(), x.dim(), _i64(list(x.shape)), _i64(perm), _ptr(x), _ptr(out)))
    return out


def concat(inputs: Sequence[torch.Tensor], axis: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(*inputs)
    rank = inputs[0].dim()
    axis = axis + rank if axis < 0 else axis
    sh = list(inputs[0].shape)
    outer = 1
    for d in sh[:axis]:
        outer *= d
    inner = 1
    for d in sh[axis + 1:]:
        inner *= d
    dims = [t.shape[axis] for t in inputs]
    osh = sh[:axis] + [sum(dims)] + sh[axis + 1:]
    if out is None:
        out = torch.empty(osh, dtype=inputs[0].dtype, device=inputs[0].device)
    ptrs = (ctypes.c_void_p * len(inputs))(*[t.data_ptr() for t in inputs])
    _check(lib().rmlk_b200_concat(_stream(), inputs[0].element_size(), len(inputs), ctypes.c_int64(outer), ctypes.c_int64(inner),
                                  _i64(dims), ptrs, _ptr(out)))
    return out


def expand(x: torch.Tensor, shape, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(x)
    osh = list(torch.broadcast_shapes(tuple(x.shape), tuple(int(v) for v in shape)))
    if out is None:
        out = torch.empty(osh, dtype=x.dtype, device=x.device)
    ish = _kshape(x)
    _check(lib().rmlk_b200_expand(_stream(), x.element_size(), len(ish), _i64(ish), len(osh), _i64(osh), _ptr(x), _ptr(out)))
    return out


def trilu(x: torch.Tensor, k: int = 0, upper: bool = True) -> torch.Tensor:
    _require_cuda(x)
    if x.dim() == 0:
        b, r, c = 1, 1, 1
    elif x.dim() == 1:
        b, r, c = 1, 1, x.shape[0]
    else:
        r, c = x.shape[-2], x.shape[-1]
        b = x.numel() // (r * c) if r * c else 0
    out = torch.empty_like(x)
    _check(lib().rmlk_b200_trilu(_stream(), x.element_size(), ctypes.c_int64(b), ctypes.c_int64(r), ctypes.c_int64(c), int(bool(upper)),
                                 ctypes.c_int64(int(k)), _ptr(x), _ptr(out)))
    return out


def range_(start, delta, n: int, dtype: torch.dtype, device="cuda") -> torch.Tensor:
    import numpy as np
    npdt = dt.to_numpy(dt.from_torch(dtype))
    s = np.array([start], dtype=npdt)
    d = np.array([delta], dtype=npdt)
    out = torch.empty([n], dtype=dtype, device=device)
    _check(lib().rmlk_b200_range(_stream(), dt.from_torch(dtype), ctypes.c_int64(n), ctypes.c_void_p(s.ctypes.data),
                                 ctypes.c_void_p(d.ctypes.data), _ptr(out)))
    return out


def fill(value, n: int, dtype: torch.dtype, device="cuda") -> torch.Tensor:
    import numpy as np
    v = np.array([value], dtype=dt.to_numpy(dt.from_torch(dtype)))
    out = torch.empty([n], dtype=dtype, device=device)
    _check(lib().rmlk_b200_fill(_stream(), out.element_size(), ctypes.c_int64(n), ctypes.c_void_p(v.ctypes.data), _ptr(out)))
    return out


def matmul_workspace_bytes(batch: int, m: int, n: int, k: int) -> int:
    return int(lib().rmlk_b200_matmul_workspace_bytes(dt.F32, ctypes.c_int64(batch), ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(k)))


def matmul(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a: [..., m, k], b: [..., k, n] with equal batch products or one of them unbatched (rank 2)."""
    _require_cuda(a, b, out, workspace)
    m, k = a.shape[-2], a.shape[-1]
    n = b.shape[-1]
    ba = a.numel() // (m * k) if m * k else 1
    bb = b.numel() // (k * n) if k * n else 1
    batch = max(ba, bb)
    lead = list(a.shape[:-2]) if ba >= bb else list(b.shape[:-2])
    if out is None:
        out = torch.empty(lead + [m, n], dtype=a.dtype, device=a.device)
    _check(lib().rmlk_b200_matmul(_stream(), dt.from_torch(a.dtype), ctypes.c_int64(batch), ctypes.c_int64(m), ctypes.c_int64(n),
                                  ctypes.c_int64(k), _ptr(a), ctypes.c_int64(m * k if ba > 1 else 0), _ptr(b),
                                  ctypes.c_int64(k * n if bb > 1 else 0), _ptr(out), ctypes.c_int64(m * n), _ptr(workspace),
                                  ctypes.c_size_t(0 if workspace is None else workspace.numel() * workspace.element_size())))
    return out


def matmul_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a: [batch..., m, k], b: [batch..., n, k] (row-major [n, k]) -> a x b^T: [batch..., m, n]."""
    _require_cuda(a, b, out)
    m, k = a.shape[-2], a.shape[-1]
    n = b.shape[-2]
    batch = a.numel() // (m * k) if m * k else 1
    if out is None:
        out = torch.empty(list(a.shape[:-2]) + [m, n], dtype=a.dtype, device=a.device)
    _check(lib().rmlk_b200_matmul_nt(_stream(), dt.from_torch(a.dtype), ctypes.c_int64(batch), ctypes.c_int64(m), ctypes.c_int64(n),
                                     ctypes.c_int64(k), _ptr(a), ctypes.c_int64(m * k), _ptr(b), ctypes.c_int64(n * k), _ptr(out),
                                     ctypes.c_int64(m * n)))
    return out


def matmul_parts(a: torch.Tensor, b: torch.Tensor):
    """a [m, k] x b [k, n] with the split-K partial sums left to the caller: returns (c, slabs, parts).  parts == 1: `c`
    holds the product; parts > 1: `slabs[:parts]` ([parts, m, n]) are to be added in order and `c` was not written."""
    _require_cuda(a, b)
    m, k = a.shape
    n = b.shape[1]
    need = lib().rmlk_b200_matmul_workspace_bytes(dt.from_torch(a.dtype), ctypes.c_int64(1), ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(k))
    ws = torch.empty(max(need // 4, 1), dtype=torch.float32, device=a.device)
    c = torch.empty(m, n, dtype=a.dtype, device=a.device)
    parts = ctypes.c_int(0)
    _check(lib().rmlk_b200_matmul_parts(_stream(), dt.from_torch(a.dtype), ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(k), _ptr(a), _ptr(b),
                                        _ptr(c), _ptr(ws), ctypes.c_size_t(need), None, ctypes.c_int(0), ctypes.byref(parts)))
    slabs = ws[:parts.value * m * n].view(parts.value, m, n) if parts.value > 1 else None
    return c, slabs, parts.value


def sum_parts(slabs: torch.Tensor) -> torch.Tensor:
    """0.f + slabs[0] + slabs[1] + ... (the split-K reduction of matmul)."""
    _require_cuda(slabs)
    out = torch.empty(list(slabs.shape[1:]), dtype=slabs.dtype, device=slabs.device)
    _check(lib().rmlk_b200_sum_parts(_stream(), dt.from_torch(slabs.dtype), ctypes.c_int(slabs.shape[0]), ctypes.c_int64(out.numel()), _ptr(slabs),
                                     _ptr(out)))
    return out


def strided_copy(base: torch.Tensor, shape: Sequence[int], strides: Sequence[int]) -> torch.Tensor:
    """Dense copy of the view of `base` (a contiguous buffer) with the given shape and element strides."""
    _require_cuda(base)
    out = torch.empty(list(shape), dtype=base.dtype, device=base.device)
    _check(lib().rmlk_b200_strided_copy(_stream(), base.element_size(), len(shape), _i64(list(shape)), _i64(list(strides)), _ptr(base), _ptr(out)))
    return out


def strided_copy_to(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """dst[...] = src[...] for two views of equal shape with arbitrary strides (views of CUDA buffers; no overlap)."""
    assert src.is_cuda and dst.is_cuda and src.shape == dst.shape and src.dtype == dst.dtype
    _check(lib().rmlk_b200_strided_copy_to(_stream(), src.element_size(), src.dim(), _i64(list(src.shape)), _i64(list(src.stride())),
                                           _i64(list(dst.stride())), ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(dst.data_ptr())))
    return dst


# ---- op chains as one launch (f32) ------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, exponent: float = 2.0) -> torch.Tensor:
    """Pow(x, exponent) -> ReduceMean(-1, keepdims) -> Add(eps) -> Sqrt -> Div(x, .) -> Mul(., weight)."""
    _require_cuda(x, weight)
    out = torch.empty_like(x)
    cols = x.shape[-1]
    _check(lib().rmlk_b200_rmsnorm(_stream(), dt.from_torch(x.dtype), ctypes.c_int64(x.numel() // cols if cols else 0), ctypes.c_int64(cols),
                                   _ptr(x), ctypes.c_float(exponent), ctypes.c_float(eps), _ptr(weight), _ptr(out)))
    return out


def add_rmsnorm(a: torch.Tensor, b: torch.Tensor, weight: torch.Tensor, eps: float, exponent: float = 2.0, parts: int = 1):
    """(a + b, rmsnorm(a + b)) in one launch; with parts > 1, b is [parts, *a.shape] split-K slabs added in order first."""
    _require_cuda(a, b, weight)
    total = torch.empty_like(a)
    out = torch.empty_like(a)
    cols = a.shape[-1]
    rows = a.numel() // cols if cols else 0
    _check(lib().rmlk_b200_add_rmsnorm(_stream(), dt.from_torch(a.dtype), ctypes.c_int64(rows), ctypes.c_int64(cols), _ptr(a), _ptr(b),
                                       ctypes.c_int(parts), ctypes.c_int64(a.numel()), ctypes.c_float(exponent), ctypes.c_float(eps), _ptr(weight),
                                       _ptr(total), _ptr(out)))
    return total, out


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x * cos + rotate_half(x) * sin for x [d0, d1, d2, D] (any strides) and cos / sin broadcastable to it.  `out` may
    be a strided view of a larger buffer (a slot of a cache): the result is written there."""
    _require_cuda(cos, sin)
    assert x.dim() == 4 and x.is_cuda   # x may be a permuted (non-contiguous) view: its strides are passed on
    if out is not None:
        assert out.is_cuda and out.shape == x.shape and out.dtype == x.dtype
        cs = cos.expand(x.shape).stride() if cos.dim() == 4 else cos.reshape([1] * (4 - cos.dim()) + list(cos.shape)).expand(x.shape).stride()
        ss = sin.expand(x.shape).stride() if sin.dim() == 4 else sin.reshape([1] * (4 - sin.dim()) + list(sin.shape)).expand(x.shape).stride()
        _check(lib().rmlk_b200_rope_to(_stream(), dt.from_torch(x.dtype), _i64(list(x.shape)), _i64(list(x.stride())), _i64(list(cs)), _i64(list(ss)),
                                       ctypes.c_void_p(x.data_ptr()), _ptr(cos), _ptr(sin), ctypes.c_void_p(out.data_ptr()), _i64(list(out.stride()))))
        return out
    out = torch.empty(list(x.shape), dtype=x.dtype, device=x.device)
    cs = cos.expand(x.shape).stride() if cos.dim() == 4 else cos.reshape([1] * (4 - cos.dim()) + list(cos.shape)).expand(x.shape).stride()
    ss = sin.expand(x.shape).stride() if sin.dim() == 4 else sin.reshape([1] * (4 - sin.dim()) + list(sin.shape)).expand(x.shape).stride()
    _check(lib().rmlk_b200_rope(_stream(), dt.from_torch(x.dtype), _i64(list(x.shape)), _i64(list(x.stride())), _i64(list(cs)), _i64(list(ss)),
                                _ptr(x), _ptr(cos), _ptr(sin), _ptr(out)))
    return out


def rope_tables(a: torch.Tensor, b: torch.Tensor):
    """cos, sin of Concat(f, f) with f = a[..., None] * b: a [rows] positions (f32), b [half] inverse frequencies -> two
    [rows, 2 half] tables in one launch."""
    _require_cuda(a, b)
    rows, half = a.numel(), b.numel()
    cos = torch.empty(rows, 2 * half, dtype=torch.float32, device=a.device)
    sin = torch.empty_like(cos)
    _check(lib().rmlk_b200_rope_tables(_stream(), dt.from_torch(a.dtype), ctypes.c_int64(rows), ctypes.c_int64(half), _ptr(a), _ptr(b), _ptr(cos),
                                       _ptr(sin)))
    return cos, sin


class _BatchJob(ctypes.Structure):
    """rmlk_batch_job of include/rmlk_b200.h."""
    _fields_ = [("kind", ctypes.c_int), ("rank", ctypes.c_int), ("in_parts", ctypes.c_int), ("reserved", ctypes.c_int),
                ("in_part_stride", ctypes.c_int64), ("shape", ctypes.c_int64 * 5), ("in_strides", ctypes.c_int64 * 5),
                ("out_strides", ctypes.c_int64 * 5), ("cos_strides", ctypes.c_int64 * 4), ("sin_strides", ctypes.c_int64 * 4),
                ("inp", ctypes.c_void_p), ("cosv", ctypes.c_void_p), ("sinv", ctypes.c_void_p), ("out", ctypes.c_void_p)]


def rope_copy_batch(jobs) -> None:
    """Several placements as one launch.  jobs: up to 4 tuples, ("rope", x, cos, sin, out) or ("copy", src, dst), all fp32 CUDA
    views (any strides; cos / sin broadcastable to x; out / dst may be slots of larger buffers).  A source given as
    (slabs, parts) - a view [parts, *shape] whose first stride is the distance between slabs - is read as the sum of the
    slabs in order."""
    arr = (_BatchJob * len(jobs))()
    keep = []
    for j, job in zip(arr, jobs):
        kind, src = job[0], job[1]
        parts = 0
        if isinstance(src, tuple):
            src, parts = src
            assert src.shape[0] == parts
            j.in_part_stride = src.stride(0)
            src = src[0]
        dst = job[-1]
        assert src.is_cuda and dst.is_cuda and src.dtype == torch.float32 and dst.dtype == torch.float32 and src.shape == dst.shape
        j.kind = 0 if kind == "rope" else 1
        j.rank = src.dim()
        j.in_parts = parts
        for d in range(src.dim()):
            j.shape[d], j.in_strides[d], j.out_strides[d] = src.shape[d], src.stride(d), dst.stride(d)
        if kind == "rope":
            assert src.dim() == 4
            for name, t in (("cos_strides", job[2]), ("sin_strides", job[3])):
                st = (t if t.dim() == 4 else t.reshape([1] * (4 - t.dim()) + list(t.shape))).expand(src.shape).stride()
                for d in range(4):
                    getattr(j, name)[d] = st[d]
            j.cosv, j.sinv = job[2].data_ptr(), job[3].data_ptr()
        j.inp, j.out = src.data_ptr(), dst.data_ptr()
        keep.append((src, dst))
    _check(lib().rmlk_b200_rope_copy_batch(_stream(), len(jobs), arr))


def gqa_decode_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask: Optional[torch.Tensor] = None,
                         split: bool = False, workspace: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [B, KV, G, D] (G <= 4 query heads per KV head, one token each); k, v [B, KV, T, D] views whose [T, D] blocks are
    dense (the batch / head dims may step over spare room); mask [B, 1 or KV*G, 1, T] or None -> [B, KV, G, D]."""
    _require_cuda(q, mask)
    B, KV, G, D = q.shape
    T = k.shape[2]
    assert k.is_cuda and v.is_cuda and k.shape == v.shape == (B, KV, T, D) and q.is_contiguous()
    assert k.stride(3) == 1 and k.stride(2) == D and v.stride(3) == 1 and v.stride(2) == D
    assert k.stride(0) == KV * k.stride(1) and v.stride(0) == KV * v.stride(1)
    if out is None:
        out = torch.empty_like(q)
    assert out.shape == q.shape and out.is_contiguous() and out.dtype == q.dtype
    mb = mh = 0
    if mask is not None:
        assert mask.dim() == 4 and mask.shape[0] == B and mask.shape[2] == 1 and mask.shape[3] == T and mask.stride(3) == 1
        mb, mh = mask.stride(0), (mask.stride(1) if mask.shape[1] > 1 else 0)
    args = (_stream(), dt.from_torch(q.dtype), ctypes.c_int64(B * KV), ctypes.c_int64(G), ctypes.c_int64(D),
            ctypes.c_int64(T), ctypes.c_int64(KV), _ptr(q), ctypes.c_void_p(k.data_ptr()), ctypes.c_int64(k.stride(1)),
            ctypes.c_void_p(v.data_ptr()), ctypes.c_int64(v.stride(1)), ctypes.c_float(scale),
            ctypes.c_void_p(0 if mask is None else mask.data_ptr()), ctypes.c_int64(mb), ctypes.c_int64(mh), _ptr(out))
    if workspace is not None:   # caller-owned workspace (zero-filled once): nothing allocated, nothing waited for
        _check(lib().rmlk_b200_gqa_decode_attention_ws(*args, _ptr(workspace), ctypes.c_size_t(workspace.numel() * workspace.element_size())))
    elif split:   # keys of a problem over several CTAs, merged through a zero-initialised workspace
        fn = lib().rmlk_b200_gqa_decode_attention_workspace_bytes
        fn.restype = ctypes.c_size_t
        need = fn(ctypes.c_int64(B * KV), ctypes.c_int64(G), ctypes.c_int64(D), ctypes.c_int64(T))
        ws = torch.zeros(max(need // 4, 4), dtype=torch.float32, device=q.device)
        _check(lib().rmlk_b200_gqa_decode_attention_ws(*args, _ptr(ws), ctypes.c_size_t(need)))
        assert need == 0 or int(ws.view(torch.int32)[: B * KV * 4].abs().sum()) == 0   # arrival counters are left at zero
    else:
        _check(lib().rmlk_b200_gqa_decode_attention(*args))
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """(gate * sigmoid(gate)) * up."""
    _require_cuda(gate, up)
    out = torch.empty_like(gate)
    _check(lib().rmlk_b200_swiglu(_stream(), dt.from_torch(gate.dtype), ctypes.c_int64(gate.numel()), _ptr(gate), _ptr(up), _ptr(out)))
    return out


def scale_mask_softmax(scores: torch.Tensor, scale: float, mask: torch.Tensor) -> torch.Tensor:
    """softmax(scores * scale + mask, -1) for scores [d0, d1, d2, T] and a mask broadcastable over d0..d2 with dense rows."""
    _require_cuda(scores, mask)
    assert scores.dim() == 4 and mask.shape[-1] == scores.shape[-1]
    out = torch.empty_like(scores)
    m4 = mask.reshape([1] * (4 - mask.dim()) + list(mask.shape)).expand(scores.shape)
    _check(lib().rmlk_b200_scale_mask_softmax(_stream(), dt.from_torch(scores.dtype), _i64(list(scores.shape[:3])), ctypes.c_int64(scores.shape[3]),
                                              _i64(list(m4.stride()[:3])), ctypes.c_float(scale), _ptr(scores), _ptr(mask), _ptr(out)))
    return out
