"""Call plans for the reference's kernel entry points.  TEST INFRASTRUCTURE ONLY.

A *plan* describes one launch of one reference `extern "C" __global__` entry point exactly as the
reference's launch wrappers (cuda/src/kernels/*.rs) and op backends
(runtime/src/providers/cuda/backend/*.rs) would issue it: the symbol name, the positional argument
list (with the `info` / `perm` / `axes` side buffers the backends build on the host) and the element
count that sizes the grid.  `oracle/ref_cpu.py` executes plans on the host build of the reference
kernels, `oracle/ref_gpu.py` on the PTX build of the same sources.

Argument encoding: ("in", ndarray) read-only buffer, ("out", ndarray) buffer read back after the
launch, ("u64", int) a size_t, ("i64", int) an int64_t, ("bool", bool).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

TAG = {
    np.dtype(np.float16): "f16", np.dtype(np.float32): "f32", np.dtype(np.float64): "f64",
    np.dtype(np.int8): "i8", np.dtype(np.uint8): "u8", np.dtype(np.int16): "i16", np.dtype(np.uint16): "u16",
    np.dtype(np.int32): "i32", np.dtype(np.uint32): "u32", np.dtype(np.int64): "i64", np.dtype(np.uint64): "u64",
    np.dtype(np.bool_): "bool",
}


@dataclass
class Plan:
    module: str          # reference file stem under cuda/src/ptx (also the PTX module name)
    symbol: str
    args: list
    n: int               # element count that sizes the launch (grid = ceil(n/128))
    out: np.ndarray = field(default=None)


def _c(a):
    return np.ascontiguousarray(a)


def _strides(shape):
    """runtime/src/utils/mod.rs:41-54 (compute_stride), in elements."""
    s = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        s[i] = s[i + 1] * shape[i + 1]
    return s


def _kshape(a):
    """Scalars are presented to kernels as shape [1], stride [1]
    (runtime/src/providers/cuda/utils.rs:5-18)."""
    return ([1], [1]) if a.ndim == 0 else (list(a.shape), _strides(a.shape))


def _bstride(shape, stride, out_shape):
    """compute_broadcast_stride_from_output_shape, runtime/src/utils/mod.rs:93-111."""
    n = len(out_shape)
    r = [0] * n
    for i in range(n):
        j = i - (n - len(shape))
        if j >= 0 and shape[j] == out_shape[i] and shape[j] != 1:
            r[i] = stride[j]
    return r


def _info(*blocks):
    return np.array([v for b in blocks for v in b], dtype=np.uint64)


def binary(symbol_stem: str, a, b, out_dtype, module=None) -> Plan:
    """backend/binary.rs:18-131 → kernels/binary.rs:58-100; info = [dims | a_strides | b_strides]."""
    a, b = _c(a), _c(b)
    ash, ast = _kshape(a)
    bsh, bst = _kshape(b)
    nd = max(len(ash), len(bsh))
    osh = list(np.broadcast_shapes(tuple(ash), tuple(bsh)))
    out = np.empty(osh, dtype=out_dtype)
    info = _info(osh, _bstride(ash, ast, osh), _bstride(bsh, bst, osh))
    return Plan(module or symbol_stem.split("_")[0], symbol_stem,
                [("u64", out.size), ("u64", nd), ("in", info), ("in", a), ("in", b), ("out", out)], out.size, out)


def arith(op: str, a, b) -> Plan:
    out_dt = np.bool_ if op in ("equal", "greater") else a.dtype
    return binary(f"{op}_fwd_{TAG[a.dtype]}", a, b, out_dt, module=op)


def pow_(a, b) -> Plan:
    return binary(f"pow_fwd_{TAG[a.dtype]}_{TAG[b.dtype]}", a, b, a.dtype, module="pow")


def unary(op: str, x) -> Plan:
    """kernels/unary.rs:10-42."""
    x = _c(x)
    out = np.empty_like(x)
    return Plan(op, f"{op}_fwd_{TAG[x.dtype]}", [("u64", x.size), ("in", x), ("out", out)], x.size, out)


def cast(x, to) -> Plan:
    """kernels/unary.rs:47-80."""
    x = _c(x)
    out = np.empty(x.shape, dtype=to)
    return Plan("cast", f"cast_fwd_{TAG[x.dtype]}_to_{TAG[np.dtype(to)]}",
                [("u64", x.size), ("in", x), ("out", out)], x.size, out)


def where(cond, x, y) -> Plan:
    """backend/whereop.rs:43-264 → kernels/whereop.rs:57-101; info = [dims | x | y | cond strides]."""
    cond, x, y = _c(cond), _c(x), _c(y)
    xs, xst = _kshape(x)
    ys, yst = _kshape(y)
    cs, cst = _kshape(cond)
    osh = list(np.broadcast_shapes(tuple(xs), tuple(ys), tuple(cs)))
    out = np.empty(osh, dtype=x.dtype)
    info = _info(osh, _bstride(xs, xst, osh), _bstride(ys, yst, osh), _bstride(cs, cst, osh))
    return Plan("where", f"where_fwd_{TAG[x.dtype]}",
                [("u64", out.size), ("u64", len(osh)), ("in", info), ("in", x), ("in", y), ("in", cond), ("out", out)],
                out.size, out)


def reduce_mean(x, axes, keepdims=True) -> Plan:
    """backend/reduce_mean.rs:139-209 → kernels/reduce_mean.rs:40-93; i32/i64 use the u32/u64 entry
    points (kernels/reduce_mean.rs:25-26)."""
    x = _c(x)
    sh, st = _kshape(x)
    rank = len(sh)
    axes = sorted(a + rank if a < 0 else a for a in axes)
    red = 1
    for a in axes:
        red *= sh[a]
    osh = [1 if d in axes else sh[d] for d in range(rank)] if keepdims else [sh[d] for d in range(rank) if d not in axes]
    out = np.empty(osh, dtype=x.dtype)
    tag = {"i32": "u32", "i64": "u64"}.get(TAG[x.dtype], TAG[x.dtype])
    return Plan("reduce_mean", f"reduce_mean_fwd_{tag}",
                [("in", np.array(axes, dtype=np.uint64)), ("u64", len(axes)), ("u64", rank), ("in", _info(sh, st)),
                 ("in", x), ("u64", red), ("u64", out.size), ("out", out)], out.size, out)


def expand(x, shape) -> Plan:
    """backend/expand.rs:49-216 → kernels/expand.rs:35-76."""
    x = _c(x)
    ish, ist = _kshape(x)
    osh = list(np.broadcast_shapes(tuple(x.shape), tuple(int(v) for v in shape)))
    out = np.empty(osh, dtype=x.dtype)
    return Plan("expand", f"expand_fwd_{TAG[x.dtype]}",
                [("u64", out.size), ("u64", len(ish)), ("u64", len(osh)), ("in", _info(ish, ist, osh, _strides(osh))),
                 ("in", x), ("out", out)], out.size, out)


def transpose(x, perm) -> Plan:
    """backend/transpose.rs:44-131 → kernels/transpose.rs:38-80; info = [dst dims | src strides |
    dst strides]."""
    x = _c(x)
    osh = [x.shape[p] for p in perm]
    out = np.empty(osh, dtype=x.dtype)
    info = _info(osh, _strides(x.shape), _strides(osh))
    return Plan("transpose", f"transpose_fwd_{TAG[x.dtype]}",
                [("u64", x.size), ("u64", x.ndim), ("in", info), ("in", np.array(perm, dtype=np.uint64)), ("in", x),
                 ("out", out)], x.size, out)


def slice_(x, starts, ends, axes, steps, out_shape, index_dtype=np.int64) -> Plan:
    """backend/slice.rs:49-203 → kernels/slice.rs:61-122.  `out_shape` comes from the backend's host
    helper (restated in oracle.ops.slice_params); the kernel re-derives starts/ends/steps from the
    device arrays.  A null axes/steps pointer means "absent"."""
    x = _c(x)
    out = np.zeros(out_shape, dtype=x.dtype)
    idt = np.dtype(index_dtype)
    info = _info(x.shape, _strides(x.shape), out_shape, _strides(x.shape))  # backend/slice.rs:110 quirk
    args = [("u64", out.size), ("u64", 0 if axes is None else len(axes)), ("u64", x.ndim), ("in", info), ("in", x),
            ("in", np.array(starts, dtype=idt)), ("in", np.array(ends, dtype=idt)),
            ("in", None if axes is None else np.array(axes, dtype=idt)),
            ("in", None if steps is None else np.array(steps, dtype=idt)), ("out", out)]
    return Plan("slice", f"slice_fwd_{TAG[x.dtype]}_with_index_{TAG[idt]}", args, out.size, out)


def scatter_nd(data, indices, updates, reduction="none"):
    """backend/scatter_nd.rs:78-210 → kernels/scatter_nd.rs:91-174.  Returns (plan, error_array)."""
    data, indices, updates = _c(data), _c(indices.astype(np.int64)), _c(updates)
    out = data.copy()
    err = np.zeros(1, dtype=np.int32)
    n_tuples = int(np.prod(indices.shape)) if indices.ndim == 1 else int(np.prod(indices.shape[:-1]))
    info = _info(data.shape, _strides(data.shape), indices.shape, _strides(indices.shape), updates.shape,
                 _strides(updates.shape))
    stem = "scatter_nd" if reduction == "none" else f"scatter_nd_{reduction}"
    p = Plan("scatter_nd", f"{stem}_fwd_{TAG[data.dtype]}",
             [("u64", n_tuples), ("u64", data.size), ("u64", data.ndim), ("u64", indices.ndim), ("u64", updates.ndim),
              ("in", info), ("in", indices), ("in", updates), ("out", out), ("out", err)], n_tuples, out)
    return p, err


def trilu(x, k=0, upper=True) -> Plan:
    """backend/trilu.rs:71-146 → kernels/trilu.rs:36-78.  The output buffer is pre-zeroed here because
    the kernel skips masked elements (trilu_op_macros.cuh:39-41)."""
    x = _c(x)
    if x.ndim == 0:
        sh3, st3 = [1, 1, 1], [1, 1, 1]
    elif x.ndim == 1:
        sh3, st3 = [1, 1, x.shape[0]], [x.shape[0], x.shape[0], 1]
    else:
        r, c = x.shape[-2], x.shape[-1]
        sh3, st3 = [int(np.prod(x.shape[:-2])), r, c], [r * c, c, 1]
    out = np.zeros_like(x)
    return Plan("trilu", f"trilu_fwd_{TAG[x.dtype]}",
                [("u64", x.size), ("u64", 3), ("bool", bool(upper)), ("i64", int(k)), ("in", _info(sh3, st3)), ("in", x),
                 ("out", out)], x.size, out)
