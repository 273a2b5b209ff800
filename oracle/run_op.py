"""Op-level front end of the numpy oracle.  TEST INFRASTRUCTURE ONLY.

`run(op, inputs, attrs)` evaluates one ONNX-style op node the way the reference's op backend would
(optional inputs, attribute defaults, dtype rejections — runtime/src/providers/cuda/backend/<op>.rs), on
top of the element-level restatements in oracle/ops.py.  Used to pin the oracle against the
reference's known-answer tests and as the CPU executor of the timed baseline (oracle/graph_cpu.py).
"""
from __future__ import annotations

import numpy as np

from . import ops as O

ONNX_DTYPE = {1: np.float32, 2: np.uint8, 3: np.int8, 4: np.uint16, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_,
              10: np.float16, 11: np.float64, 12: np.uint32, 13: np.uint64}


class Unsupported(TypeError):
    def __init__(self, dtype, what):
        super().__init__(f"unsupported data type: {np.dtype(dtype).name} ({what})")


def _need(dtype, allowed, what):
    if np.dtype(dtype) not in [np.dtype(a) for a in allowed]:
        raise Unsupported(dtype, what)


# (src, dst) pairs dispatched by the reference's Cast backend (backend/cast.rs:30-67); others are rejected.
_F = ("float16", "float32", "float64")
CAST_PAIRS = {(s, d) for s in _F for d in _F + ("int32", "uint32", "int64", "uint64") if s != d}
CAST_PAIRS |= {(s, d) for s in ("int32", "uint32", "int64", "uint64") for d in _F}
CAST_PAIRS |= {("int32", "int64"), ("uint32", "uint64"), ("int64", "int32"), ("uint64", "uint32"), ("bool", "float32")}

ARITH = (np.float16, np.float32, np.float64, np.int32, np.int64)
FLOATS = (np.float16, np.float32, np.float64)
COPYABLE = (np.float16, np.float32, np.float64, np.int32, np.uint32, np.int64, np.uint64)


def run(op: str, inputs, attrs=None) -> np.ndarray:
    a = attrs or {}
    x = inputs
    if op in ("Add", "Sub", "Mul", "Div", "Equal", "Greater"):
        _need(x[0].dtype, ARITH, op)
        if x[0].dtype != x[1].dtype:
            raise ValueError("operand data types differ")
        return O.binary(op.lower(), x[0], x[1])
    if op == "Pow":
        _need(x[0].dtype, ARITH, "pow base")
        return O.pow_(x[0], x[1])
    if op in ("Sqrt", "Sin", "Cos", "Sigmoid"):
        _need(x[0].dtype, FLOATS, op)
        return O.unary(op.lower(), x[0])
    if op in ("Neg", "Relu"):
        _need(x[0].dtype, ARITH, op)
        return O.unary(op.lower(), x[0])
    if op == "Cast":
        if "to" not in a:
            raise ValueError("missing `to` cast attribute")
        to = np.dtype(ONNX_DTYPE[int(a["to"])])
        if (x[0].dtype.name, to.name) not in CAST_PAIRS:
            raise TypeError(f"unsupported cast: {x[0].dtype.name} -> {to.name}")
        return O.cast(x[0], to)
    if op == "Where":
        _need(x[1].dtype, ARITH, "where")
        if x[0].dtype != np.bool_:
            raise ValueError("where: condition must be a bool tensor")
        return O.where(x[0], x[1], x[2])
    if op == "ReduceMean":
        _need(x[0].dtype, ARITH, "reduce_mean")
        axes = None
        if len(x) > 1 and x[1] is not None:
            if x[1].size:
                axes = [int(v) for v in x[1].reshape(-1)]
            elif x[1].ndim == 0:
                raise ValueError("ScalarAxisNotAllowed")
            else:
                axes = []
        elif "axes" in a:
            axes = list(a["axes"])
        return O.reduce_mean(x[0], axes, bool(a.get("keepdims", 1)), bool(a.get("noop_with_empty_axes", 0)))
    if op == "Softmax":
        _need(x[0].dtype, (np.float32,), "softmax")
        return O.softmax(x[0], int(a.get("axis", -1)))
    if op == "Gemm":
        _need(x[0].dtype, (np.float16, np.float32), "gemm")
        return O.gemm(x[0], x[1], x[2] if len(x) > 2 else None, float(a.get("alpha", 1.0)), float(a.get("beta", 1.0)),
                      bool(a.get("transA", 0)), bool(a.get("transB", 0)))
    if op == "MatMul":
        _need(x[0].dtype, (np.float32,), "matmul")
        return O.matmul(x[0], x[1])
    if op == "Gather":
        _need(x[0].dtype, COPYABLE, "gather")
        _need(x[1].dtype, (np.int32, np.int64), "gather indices")
        return O.gather(x[0], x[1], int(a.get("axis", 0)))
    if op == "ScatterND":
        _need(x[0].dtype, ARITH, "scatter_nd")
        _need(x[1].dtype, (np.int64,), "scatter_nd indices")
        red = str(a.get("reduction", "none")).lower()
        return O.scatter_nd(x[0], x[1], x[2], red)
    if op == "Slice":
        _need(x[0].dtype, ARITH, "slice")
        axes = None if len(x) < 4 or x[3] is None else [int(v) for v in x[3].reshape(-1)]
        steps = None if len(x) < 5 or x[4] is None else [int(v) for v in x[4].reshape(-1)]
        return O.slice_(x[0], [int(v) for v in x[1].reshape(-1)], [int(v) for v in x[2].reshape(-1)], axes, steps)
    if op == "Transpose":
        _need(x[0].dtype, ARITH, "transpose")
        return O.transpose(x[0], list(a["perm"]) if "perm" in a else None)
    if op == "Concat":
        _need(x[0].dtype, COPYABLE, "concat")
        if "axis" not in a:
            raise ValueError("`axis` is missing")
        return O.concat([t for t in x if t is not None], int(a["axis"]))
    if op == "Expand":
        _need(x[0].dtype, COPYABLE, "expand")
        return O.expand(x[0], [int(v) for v in x[1].reshape(-1)])
    if op == "Trilu":
        _need(x[0].dtype, COPYABLE, "trilu")
        k = 0
        if len(x) > 1 and x[1] is not None:
            if x[1].ndim != 0:
                raise ValueError("InvalidKTensor")
            k = int(x[1])
        return O.trilu(x[0], k, bool(a.get("upper", 1)))
    if op == "Range":
        _need(x[0].dtype, ARITH, "range")
        return O.range_(x[0].reshape(()).item(), x[1].reshape(()).item(), x[2].reshape(()).item(), x[0].dtype)
    if op == "Reshape":
        return O.reshape(x[0], [int(v) for v in x[1].reshape(-1)], bool(a.get("allowzero", 0)))
    if op == "Unsqueeze":
        axes = [int(v) for v in x[1].reshape(-1)] if len(x) > 1 and x[1] is not None else list(a["axes"])
        return O.unsqueeze(x[0], axes)
    if op == "Flatten":
        ax = int(a.get("axis", 1))
        ax = ax + x[0].ndim if ax < 0 else ax
        return x[0].reshape(int(np.prod(x[0].shape[:ax], dtype=np.int64)), -1).copy()
    if op == "Shape":
        # backend/shape.rs:30-80: optional start / end attributes, negative values count from the back
        rank = x[0].ndim
        start, end = int(a.get("start", 0)), int(a.get("end", rank))
        start = min(max(start + rank if start < 0 else start, 0), rank)
        end = min(max(end + rank if end < 0 else end, 0), rank)
        return np.array(x[0].shape[start:end], dtype=np.int64)
    if op == "ConstantOfShape":
        v = a.get("value")
        v = np.zeros(1, np.float32) if v is None else np.asarray(v)
        return np.full([int(d) for d in x[0].reshape(-1)], v.reshape(-1)[0], dtype=v.dtype)
    if op == "Constant":
        return np.asarray(a["value"]).copy()
    raise NotImplementedError(op)
