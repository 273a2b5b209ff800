"""CPU interpreter for op graphs.  TEST INFRASTRUCTURE ONLY.

Walks a `rmlk_b200.graphspec.GraphSpec` node by node, in order — the same sequential loop as the
reference's executor (runtime/src/core/instance.rs:100-112) — evaluating each op with the numpy oracle
(oracle/run_op.py).  It is the checker for multi-op graphs (a decoder layer, a whole decoder) and the timed
CPU baseline of bench.py: numpy's BLAS uses the host's cores for MatMul, everything else is vectorised
numpy.

A `fast` mode swaps the float64 MatMul / Softmax / ReduceMean restatements for float32 numpy calls; it is
only for timing (the CPU baseline) and for full-size runs where float64 would take minutes, never for
parity checks.
"""
from __future__ import annotations

import numpy as np

from . import run_op


def _fast_op(op, inputs, attrs):
    x = inputs
    if op == "MatMul":
        return np.matmul(x[0], x[1])
    if op == "Softmax":
        m = x[0].max(axis=-1, keepdims=True)
        e = np.exp(x[0] - m)
        return e / e.sum(axis=-1, keepdims=True)
    if op == "ReduceMean" and "axes" in attrs and len(x) == 1:
        return x[0].mean(axis=tuple(attrs["axes"]), keepdims=bool(attrs.get("keepdims", 1)), dtype=np.float64).astype(x[0].dtype)
    return None


def run_graph(spec, feeds: dict, fast: bool = False, weights: dict = None) -> dict:
    """Evaluate `spec` on host arrays.  `weights` supplies host copies for initializers that the spec
    holds on the device.  Returns {output name: ndarray}."""
    env = dict(spec.constants)
    if weights:
        env.update(weights)
    for name, dtype, _dims in spec.inputs:
        if name not in feeds:
            raise KeyError(f"graph input `{name}` was not fed")
        env[name] = np.asarray(feeds[name], dtype=dtype)
    last_use = {}
    for i, node in enumerate(spec.nodes):
        for n in node.inputs:
            if n:
                last_use[n] = i
    keep = set(spec.outputs) | set(spec.constants) | set(weights or ())
    for i, node in enumerate(spec.nodes):
        ins = [env[n] if n else None for n in node.inputs]
        out = _fast_op(node.op, ins, node.attrs) if fast else None
        if out is None:
            out = run_op.run(node.op, ins, node.attrs)
        env[node.outputs[0]] = out
        for n in node.inputs:  # free intermediates after their last use (the full-size graphs are large)
            if n and last_use.get(n) == i and n not in keep and n not in feeds:
                env.pop(n, None)
    return {n: env[n] for n in spec.outputs}
