"""CPU restatement (numpy) of the reference's operator semantics.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py`` may
import this module; the product package never does.  Each function restates what the reference's
op backend plus kernel computes and cites the reference file:line it follows (paths are relative to
the reference project's root).

Pinning: every function here is checked in ``tests/test_oracle.py`` against

* the reference's own kernel sources compiled as host C++ (``oracle/_ref/libref_cpu.so``, driven by
  ``oracle/ref_cpu.py``) for the eleven hand-written kernel families, and
* the known-answer vectors transcribed from the reference's unit tests and its checked-in
  ORT-CPU goldens (``tests/golden/*.json``, produced by ``tests/golden/extract_kats.py``).

MatMul, Softmax, Sigmoid and Relu have no source in the reference (they call cuBLAS / cuDNN, neither
of which has a CPU build); for those the restatement is the published definition of the op and the
pins are the reference's known-answer tests and the attention golden only.
"""
from __future__ import annotations

import numpy as np

# ---------------------------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------------------------


def normalize_index(index: int, size: int) -> int:
    """runtime/src/utils/mod.rs:159-182 — negative indices wrap once; result must be <= size."""
    n = size + index if index < 0 else index
    if n < 0 or n > size:
        raise ValueError(f"axis out of bound {index}")
    return n


def broadcast_shape(a, b):
    """runtime/src/utils/mod.rs:114-143 (compute_broadcast_output_shape)."""
    nd = max(len(a), len(b))
    a = (1,) * (nd - len(a)) + tuple(a)
    b = (1,) * (nd - len(b)) + tuple(b)
    out = []
    for x, y in zip(a, b):
        if x != y and x != 1 and y != 1:
            raise ValueError(f"incompatible tensor shapes: {a} {b}")
        out.append(max(x, y))
    return tuple(out)


_FLOATS = (np.float16, np.float32, np.float64)


def _trunc_div(a, b):
    """C integer division (truncation toward zero), as `x / y` in cuda/src/ptx/div.cu:10-12."""
    q = np.abs(a) // np.abs(b)
    return (q * np.sign(a) * np.sign(b)).astype(a.dtype)


# ---------------------------------------------------------------------------------------------
# broadcast elementwise family
# ---------------------------------------------------------------------------------------------


def binary(op: str, a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """LONG_BINARY_OP_WITH_TYPES, cuda/src/ptx/headers/binary_op_macros.cuh:14-42 with the functors
    of add.cu:17-25, sub.cu:4-12, mul.cu:17-25, div.cu:4-12, equal.cu:4-12, greater.cu:4-12.
    Output shape: runtime/src/providers/cuda/backend/binary.rs:133-162 (NumPy broadcasting)."""
    broadcast_shape(a.shape, b.shape)
    with np.errstate(all="ignore"):
        if op == "add":
            return (a + b).astype(a.dtype)
        if op == "sub":
            return (a - b).astype(a.dtype)
        if op == "mul":
            return (a * b).astype(a.dtype)
        if op == "div":
            if a.dtype.type in _FLOATS:
                return (a / b).astype(a.dtype)
            return _trunc_div(*np.broadcast_arrays(a, b))
        if op == "equal":
            return a == b
        if op == "greater":
            return a > b
    raise ValueError(op)


def pow_(base: np.ndarray, exp: np.ndarray) -> np.ndarray:
    """cuda/src/ptx/pow.cu:6-65.  f16/f32 bases: powf(x, (float)y); f64: pow(x, (double)y);
    integer bases: (T)llround(pow((double)x, (double)y)).  Output dtype = base dtype
    (backend/pow.rs:95-117)."""
    broadcast_shape(base.shape, exp.shape)
    with np.errstate(all="ignore"):
        if base.dtype in (np.float16, np.float32):
            r = np.power(base.astype(np.float32), exp.astype(np.float32), dtype=np.float32)
            return r.astype(base.dtype)
        if base.dtype == np.float64:
            return np.power(base, exp.astype(np.float64))
        r = np.power(base.astype(np.float64), exp.astype(np.float64))
        # llround: half away from zero
        r = np.where(r >= 0, np.floor(r + 0.5), np.ceil(r - 0.5))
        return r.astype(np.int64).astype(base.dtype)


def unary(op: str, x: np.ndarray) -> np.ndarray:
    """UNARY_OP, cuda/src/ptx/headers/unary_op_macro.cuh:1-11 with sqrt.cu:5-9, neg.cu:4-12
    (x * -1), sin.cu:5-9, cos.cu:5-9 (f16 goes through float).  Sigmoid / Relu are
    cudnnActivationForward in the reference (cuda/src/kernels/activation.rs:6-39); restated by
    definition: 1/(1+exp(-x)) as in the reference's own check (cuda/src/kernels/sigmoid.rs:37-39)
    and max(x, 0)."""
    with np.errstate(all="ignore"):
        if op == "neg":
            return (x * x.dtype.type(-1)).astype(x.dtype)
        if op == "relu":
            return np.where(x > 0, x, x.dtype.type(0)).astype(x.dtype)
        w = x.astype(np.float32) if x.dtype == np.float16 else x
        if op == "sqrt":
            r = np.sqrt(w)
        elif op == "sin":
            r = np.sin(w)
        elif op == "cos":
            r = np.cos(w)
        elif op == "sigmoid":
            one = w.dtype.type(1)
            r = one / (one + np.exp(-w))
        else:
            raise ValueError(op)
        return r.astype(x.dtype)


def cast(x: np.ndarray, to) -> np.ndarray:
    """CAST_OP, cuda/src/ptx/headers/cast_op_macro.cuh:1-11 and cast.cu:6-124: static_cast, via
    float for f16, `x == 0 ? false : true` to bool.  Float→int of out-of-range / NaN values is
    undefined on the host, so callers keep such inputs out of CPU comparisons."""
    to = np.dtype(to)
    if to == np.bool_:
        return x != 0
    if to == np.float16 and x.dtype != np.float16:
        # cast.cu goes through float: __float2half(static_cast<float>(x))
        with np.errstate(all="ignore"):
            return x.astype(np.float32).astype(np.float16)
    with np.errstate(all="ignore"):
        if x.dtype.type in _FLOATS and to.kind in "iu":
            return np.trunc(x.astype(np.float64) if x.dtype != np.float32 else x).astype(to)
        return x.astype(to)


def where(cond: np.ndarray, x: np.ndarray, y: np.ndarray) -> np.ndarray:
    """LONG_TERNARY_OP_WITH_TYPES, cuda/src/ptx/headers/ternary_op_macro.cuh:1-34, where.cu:4-12
    (`z ? x : y`); 3-way broadcast per backend/whereop.rs:197-264; dtype from x."""
    s = broadcast_shape(broadcast_shape(x.shape, y.shape), cond.shape)
    return np.where(np.broadcast_to(cond, s), np.broadcast_to(x, s), np.broadcast_to(y, s)).astype(x.dtype)


# ---------------------------------------------------------------------------------------------
# reductions
# ---------------------------------------------------------------------------------------------


def reduce_mean(x: np.ndarray, axes=None, keepdims: bool = True, noop_with_empty_axes: bool = False) -> np.ndarray:
    """REDUCE_MEAN_OP_THREAD_PER_OUTPUT, cuda/src/ptx/headers/aggregation_op_macros.cuh:1-49:
    sequential accumulation in double (uint64_t for the integer variants, reduce_mean.cu:8-9), one
    division in double, cast back.  Axes handling per backend/reduce_mean.rs:72-168: `None` means
    all axes; an empty list means all axes unless noop_with_empty_axes, in which case the input is
    copied."""
    rank = max(x.ndim, 1)
    xs = x.reshape((1,)) if x.ndim == 0 else x
    if axes is not None and len(axes) == 0:
        if noop_with_empty_axes:
            return x.copy()
        axes = None
    if axes is None:
        axes = list(range(rank))
    axes = [normalize_index(int(a), rank) for a in axes]
    if len(set(axes)) != len(axes):
        raise ValueError("DuplicateAxis")
    if any(a >= rank for a in axes):
        raise ValueError("AxisOutOfBounds")
    count = 1
    for a in axes:
        count *= xs.shape[a]
    if xs.dtype.kind in "iu":
        acc = xs.astype(np.uint64).sum(axis=tuple(axes), keepdims=keepdims, dtype=np.uint64)
        div = acc.astype(np.float64) / np.float64(count)
        udt = np.uint32 if xs.dtype.itemsize == 4 else np.uint64
        out = np.trunc(div).astype(udt).view(xs.dtype) if div.ndim else np.array(np.trunc(div)).astype(udt).view(xs.dtype)
    else:
        acc = xs.astype(np.float64).sum(axis=tuple(axes), keepdims=keepdims, dtype=np.float64)
        out = (acc / np.float64(count)).astype(xs.dtype)
    out = np.asarray(out)
    if x.ndim == 0:
        return out.reshape(())
    return out


def softmax(x: np.ndarray, axis: int = -1) -> np.ndarray:
    """cudnnSoftmaxForward(MODE_CHANNEL) over the last axis after flattening to [N, C, 1, 1]
    (backend/softmax.rs:31-158; only axis −1, or 1 for rank 4).  Restated by definition, evaluated in
    double so that it is the value both cuDNN's FAST and ACCURATE algorithms approximate; the
    reference's own host formula is exp(x - max)/sum (backend/softmax.rs:301-305)."""
    if not (axis == -1 or (axis == 1 and x.ndim == 4)):
        raise ValueError(f"unsupported inputs axis `{axis}` and rank `{x.ndim}")
    w = x.astype(np.float64)
    w = w - w.max(axis=axis, keepdims=True)
    e = np.exp(w)
    return (e / e.sum(axis=axis, keepdims=True)).astype(x.dtype)


# ---------------------------------------------------------------------------------------------
# MatMul
# ---------------------------------------------------------------------------------------------


def matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """backend/matmul.rs:234-356 shape rules (rank-1 promotion, batch = product of the leading dims,
    batch broadcast only when one side's batch is 1) over cublasGemmStridedBatchedEx with fp32
    accumulate (cuda/src/kernels/gemm.rs:206-231).  Evaluated in double, cast back.  The flat
    element order equals the reference's; the shape follows NumPy (the reference collapses leading
    batch dims to [1,..,1,b,m,n], matmul.rs:321-333, same buffer)."""
    if a.ndim == 0 or b.ndim == 0:
        raise ValueError("ZeroRank")
    ka = a.shape[-1]
    kb = b.shape[0] if b.ndim == 1 else b.shape[-2]
    if ka != kb:
        raise ValueError("IncompatibleDimForMul")
    ba = int(np.prod(a.shape[:-2])) if a.ndim > 2 else 1
    bb = int(np.prod(b.shape[:-2])) if b.ndim > 2 else 1
    if ba != bb and ba != 1 and bb != 1:
        raise ValueError("IncompatibleDimForBroadcast")
    am = a.reshape(ba, -1, ka) if a.ndim >= 2 else a.reshape(1, 1, ka)
    bm = b.reshape(bb, kb, -1) if b.ndim >= 2 else b.reshape(1, kb, 1)
    r = np.matmul(am.astype(np.float64), bm.astype(np.float64)).astype(a.dtype)
    lead = a.shape[:-2] if ba >= bb and a.ndim > 2 else (b.shape[:-2] if b.ndim > 2 else ())
    if a.ndim == 1 and b.ndim == 1:
        return r.reshape(())
    if a.ndim == 1:
        return r.reshape(tuple(lead) + (bm.shape[2],))
    if b.ndim == 1:
        return r.reshape(tuple(lead) + (am.shape[1],))
    return r.reshape(tuple(lead) + (am.shape[1], bm.shape[2]))


def gemm(a: np.ndarray, b: np.ndarray, c=None, alpha: float = 1.0, beta: float = 1.0, trans_a: bool = False, trans_b: bool = False) -> np.ndarray:
    """ONNX Gemm as the reference's backend computes it (runtime/src/providers/cuda/backend/gemm.rs:149-216): rank-2 A and B, a
    logical transpose per flag (cuda/src/kernels/gemm.rs:21-72), alpha inside the GEMM, then y += beta * C with C broadcast
    to [M, N] (a vector of N entries is a row, one of M entries a column, backend/gemm.rs:225-227).  Evaluated in double.
    (The reference's 2-D bias strides, backend/gemm.rs:228-238, use the extents themselves as strides; the ONNX broadcast
    is restated here.)"""
    if a.ndim != 2 or b.ndim != 2:
        raise ValueError("expected inputs with rank 2")
    am = a.T if trans_a else a
    bm = b.T if trans_b else b
    if am.shape[1] != bm.shape[0]:
        raise ValueError("IncompatibleDimForMul")
    m, n = am.shape[0], bm.shape[1]
    y = np.float64(alpha) * np.matmul(am.astype(np.float64), bm.astype(np.float64))
    if c is not None:
        cc = np.asarray(c, dtype=np.float64)
        if cc.ndim == 1 and cc.shape[0] == n:
            cc = cc.reshape(1, n)
        elif cc.ndim == 1 and cc.shape[0] == m:
            cc = cc.reshape(m, 1)
        elif cc.ndim == 2 and cc.shape[0] in (m, 1) and cc.shape[1] in (n, 1):
            pass
        elif cc.size == 1:
            cc = cc.reshape(1, 1)
        else:
            raise ValueError("invalid tensor shape")
        y = y + np.float64(beta) * cc
    return y.astype(a.dtype)


# ---------------------------------------------------------------------------------------------
# indexing / layout
# ---------------------------------------------------------------------------------------------


def gather(data: np.ndarray, indices: np.ndarray, axis: int = 0) -> np.ndarray:
    """backend/gather.rs:98-258: output shape data[:axis] ++ indices.shape ++ data[axis+1:], negative
    indices wrap (normalize_index).  (The reference's host loop uses a product of strides as the
    per-batch offset, gather.rs:218, which is only right for axis <= 1; the ONNX definition is
    restated.)"""
    if data.ndim == 0:
        raise ValueError("scalar input data not allowed")
    axis = normalize_index(axis, data.ndim)
    idx = np.asarray(indices).astype(np.int64)
    if ((idx < -data.shape[axis]) | (idx >= data.shape[axis])).any():
        raise IndexError("gather index out of range")
    idx = np.where(idx < 0, idx + data.shape[axis], idx)
    return np.take(data, idx, axis=axis)


def concat(inputs, axis: int) -> np.ndarray:
    """backend/concat.rs:28-198: same rank, equal non-axis dims, scalars rejected."""
    if inputs[0].ndim == 0:
        raise ValueError("ScalarsAreNotAllowed")
    axis = normalize_index(axis, inputs[0].ndim)
    for t in inputs[1:]:
        if t.ndim != inputs[0].ndim:
            raise ValueError("ShapeMismatch")
        for d in range(t.ndim):
            if d != axis and t.shape[d] != inputs[0].shape[d]:
                raise ValueError("DimensionMismatch")
    return np.concatenate(inputs, axis=axis)


def expand(x: np.ndarray, shape) -> np.ndarray:
    """LONG_EXPAND_OP, cuda/src/ptx/headers/expand_op_macros.cuh:1-31; output shape is the two-way
    broadcast of the input shape and the requested shape (backend/expand.rs:128-175)."""
    s = broadcast_shape(x.shape, tuple(int(v) for v in shape))
    return np.broadcast_to(x, s).copy()


def transpose(x: np.ndarray, perm=None) -> np.ndarray:
    """LONG_TRANSPOSE_OP, cuda/src/ptx/headers/transpose_op_macros.cuh:1-25; perm default is the
    reversed axis list (backend/transpose.rs:134-178)."""
    if perm is None:
        perm = list(range(x.ndim))[::-1]
    if len(perm) != x.ndim:
        raise ValueError("InvalidPermLength")
    if any(p < 0 or p >= x.ndim for p in perm):
        raise ValueError("PermIndexOutOfBounds")
    return np.transpose(x, perm).copy(order="C")


def slice_params(in_shape, starts, ends, axes=None, steps=None):
    """Normalised (start, step, out_dim) per input axis.  Clamping follows
    backend/slice.rs:358-464 (compute_output_shape_helper) and the identical in-kernel logic of
    cuda/src/ptx/headers/slice_op_macros.cuh:24-75."""
    rank = len(in_shape)
    if axes is None:
        axes = list(range(len(starts)))
    if steps is not None and len(steps) != len(axes):
        raise ValueError("StepsAndAxesLengthMismatch")
    st = [0] * rank
    sp = [1] * rank
    od = list(in_shape)
    for k, raw_axis in enumerate(axes):
        axis = raw_axis + rank if raw_axis < 0 else raw_axis
        if axis < 0 or axis >= rank:
            raise ValueError("AxisOutOfRange")
        step = int(steps[k]) if steps is not None else 1
        if step == 0:
            raise ValueError("ZeroStep")
        dim = in_shape[axis]
        start = int(starts[k])
        if start < 0:
            start += dim
        if start < 0:
            start = 0
        if step > 0 and start > dim:
            start = dim
        elif step < 0 and start >= dim:
            start = dim - 1
        end = int(ends[k])
        if end < 0:
            end += dim
        if end < -1:
            end = -1
        if step > 0 and end > dim:
            end = dim
        elif step < 0 and end >= dim:
            end = dim - 1
        if (step < 0 and start < end) or (step > 0 and start >= end):
            n = 0
        elif step > 0:
            n = -((start - end) // step)
        else:
            n = -((end - start) // (-step))
        st[axis], sp[axis], od[axis] = start, step, n
    return st, sp, od


def slice_(x: np.ndarray, starts, ends, axes=None, steps=None) -> np.ndarray:
    """SLICE_OP, cuda/src/ptx/headers/slice_op_macros.cuh:1-96: out[idx] = in[start + step*idx]."""
    st, sp, od = slice_params(x.shape, starts, ends, axes, steps)
    index = tuple(st[d] + sp[d] * np.arange(od[d]) for d in range(x.ndim))
    return x[np.ix_(*index)].copy() if x.ndim else x.copy()


_SCATTER = {
    "none": lambda upd, out: upd,
    "add": lambda upd, out: upd + out,
    "mul": lambda upd, out: upd * out,
    "max": lambda upd, out: np.where(upd > out, upd, out),
    "min": lambda upd, out: np.where(upd < out, upd, out),
}


def scatter_nd(data: np.ndarray, indices: np.ndarray, updates: np.ndarray, reduction: str = "none") -> np.ndarray:
    """LONG_SCATTER_ND_OP, cuda/src/ptx/headers/scatter_op_macros.cuh:19-93 and scatter_nd.cu:4-32:
    output starts as a copy of data (backend/scatter_nd.rs:128-129); negative indices wrap; an index
    outside [0, dim) is error 1.  Tuples are applied in order here; the reference leaves duplicate
    targets unspecified (scatter_op_macros.cuh:16-17), so tests keep 'none' targets unique."""
    if data.ndim == 0 or indices.ndim == 0 or updates.ndim == 0:
        raise ValueError("ScalarInputsAreNotAllowed")
    out = data.copy()
    k = indices.shape[-1] if indices.ndim > 1 else 1
    idx = indices.reshape(-1, k).astype(np.int64)
    slice_shape = data.shape[k:]
    upd = updates.reshape((idx.shape[0],) + tuple(slice_shape))
    f = _SCATTER[reduction]
    for t in range(idx.shape[0]):
        tup = []
        for i in range(k):
            v = int(idx[t, i])
            if v < 0:
                v += data.shape[i]
            if v < 0 or v >= data.shape[i]:
                raise IndexError("scatter_nd kernel failed: code 1")
            tup.append(v)
        tup = tuple(tup)
        out[tup] = f(upd[t], out[tup]).astype(data.dtype)
    return out


def trilu(x: np.ndarray, k: int = 0, upper: bool = True) -> np.ndarray:
    """LONG_TRILU_OP, cuda/src/ptx/headers/trilu_op_macros.cuh:1-43 on the [batch, R, C] view of
    runtime/src/utils/mod.rs:226-239.  Elements outside the kept triangle are zero (ONNX; the
    reference kernel leaves them unwritten, trilu_op_macros.cuh:39-41, and every reference test
    expects zeros, backend/trilu.rs:181-277).  A lower triangle with k + row + 1 < 0 keeps nothing
    (ONNX); the reference's size_t `end` wraps there."""
    if x.ndim == 0:
        v = x.reshape(1, 1, 1)
    elif x.ndim == 1:
        v = x.reshape(1, 1, -1)
    else:
        v = x.reshape((-1,) + x.shape[-2:])
    r = np.arange(v.shape[1])[:, None]
    c = np.arange(v.shape[2])[None, :]
    keep = (c >= r + k) if upper else (c <= r + k)
    return np.where(keep[None], v, v.dtype.type(0)).reshape(x.shape)


def range_count(start, limit, delta, dtype) -> int:
    """backend/range.rs:136-192: truncating integer division for ints, ceil for floats."""
    dt = np.dtype(dtype)
    if dt.kind in "iu":
        q = abs(int(limit) - int(start)) // abs(int(delta))
        if (int(limit) - int(start) < 0) != (int(delta) < 0):
            q = -q
        return max(q, 0)
    t = dt.type
    c = np.ceil((t(limit) - t(start)) / t(delta))
    if c < 0:
        raise ValueError("ConversionError")
    return int(c)


def range_(start, limit, delta, dtype) -> np.ndarray:
    """backend/range.rs:195-205: out[i] = start + (T)i * delta evaluated in T (two roundings)."""
    dt = np.dtype(dtype)
    n = range_count(start, limit, delta, dt)
    i = np.arange(n).astype(dt)
    with np.errstate(all="ignore"):
        return (dt.type(start) + (i * dt.type(delta)).astype(dt)).astype(dt)


# ---------------------------------------------------------------------------------------------
# shape-only ops (the reference copies the payload; semantics only)
# ---------------------------------------------------------------------------------------------


def reshape(x: np.ndarray, shape, allowzero: bool = False) -> np.ndarray:
    """backend/reshape.rs:95-160: 0 copies the input dim (unless allowzero), -1 is inferred."""
    tgt = []
    neg = None
    for i, d in enumerate(int(v) for v in shape):
        if d == -1:
            if neg is not None:
                raise ValueError("ZeroDimAndNegDimWhenAllowZero")
            neg = i
            tgt.append(1)
        elif d == 0 and not allowzero:
            tgt.append(x.shape[i])
        else:
            tgt.append(d)
    if neg is not None:
        p = int(np.prod(tgt))
        if p == 0 or x.size % p:
            raise ValueError("UnableToHoldSameNumberOfElements")
        tgt[neg] = x.size // p
    return x.reshape(tgt).copy()


def unsqueeze(x: np.ndarray, axes) -> np.ndarray:
    """backend/unsqueeze.rs:85-130."""
    rank = x.ndim + len(axes)
    norm = sorted(normalize_index(int(a), rank) for a in axes)
    if len(set(norm)) != len(norm):
        raise ValueError("DuplicateAxes")
    out = x
    for a in norm:
        out = np.expand_dims(out, a)
    return out.copy()
