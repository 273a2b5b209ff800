"""A neutral, pure-Python description of an op graph (values, initializers, op nodes in execution order).

The reference gets its graphs from ONNX files through rmlk_schema's importer
(schema/src/onnx_import/transform.rs:175-246), which is outside the operator path; here graphs are written
down directly with the same vocabulary — ONNX op names, ONNX attribute names, inputs by value name with ""
for an omitted optional input — and lowered onto the runtime with `to_runtime`.  Being plain data, the
same description can also be walked by a CPU interpreter in the test infrastructure.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np


@dataclass
class NodeSpec:
    op: str
    inputs: List[Optional[str]]
    outputs: List[str]
    attrs: Dict[str, object] = field(default_factory=dict)


@dataclass
class GraphSpec:
    inputs: List[tuple] = field(default_factory=list)              # (name, numpy dtype, dims with 0 = dynamic)
    constants: Dict[str, np.ndarray] = field(default_factory=dict)  # initializers held on the host
    device_constants: Dict[str, object] = field(default_factory=dict)  # initializers already on the device (torch tensors)
    nodes: List[NodeSpec] = field(default_factory=list)
    outputs: List[str] = field(default_factory=list)
    _n: int = 0

    # -- construction ----------------------------------------------------------------------------
    def input(self, name: str, dtype, dims: Sequence[int]) -> str:
        self.inputs.append((name, np.dtype(dtype), list(dims)))
        return name

    def const(self, name: str, array) -> str:
        self.constants[name] = np.require(array, requirements="C")
        return name

    def const_device(self, name: str, tensor) -> str:
        self.device_constants[name] = tensor
        return name

    def op(self, op: str, inputs: Sequence[Optional[str]], out: Optional[str] = None, **attrs) -> str:
        if out is None:
            self._n += 1
            out = f"{op.lower()}_{self._n}"
        self.nodes.append(NodeSpec(op, list(inputs), [out], dict(attrs)))
        return out

    def output(self, name: str) -> str:
        self.outputs.append(name)
        return name

    # -- lowering --------------------------------------------------------------------------------
    def to_runtime(self):
        """Build a rmlk_b200.runtime.GraphBuilder holding this graph."""
        from . import dtypes as dt
        from .runtime import AttributeType, GraphBuilder, Op
        g = GraphBuilder()
        for name, dtype, dims in self.inputs:
            g.input(name, dtype, dims)
        for name, a in self.constants.items():
            g.constant(name, a)
        for name, t in self.device_constants.items():
            g.constant_device(name, dt.from_torch(t.dtype), list(t.shape), t.data_ptr())
        declared = set(n for n, _, _ in self.inputs) | set(self.constants) | set(self.device_constants)
        for node in self.nodes:
            for o in node.outputs:
                if o not in declared:
                    g.value(o, dt.UNDEFINED, [])
                    declared.add(o)
            h = g.op(Op[node.op], [i or None for i in node.inputs], node.outputs)
            for k, v in node.attrs.items():
                h.attr(k, AttributeType.Tensor(v) if isinstance(v, np.ndarray) else v)
        for name in self.outputs:
            g.output(name)
        return g
