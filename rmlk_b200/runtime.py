"""Python face of the host runtime (include/rmlk_b200_runtime.h).

Mirrors the reference's public surface for the operator path so that tests read like the reference's:

    reference (Rust)                                         here
    -------------------------------------------------------  -----------------------------------------
    rmlk_schema::GraphBuilder (schema/src/builder.rs)        GraphBuilder
    rmlk_runtime::Builder::from_graph(g).build()             ModelInstance(graph)
    ModelInstance::run(HashMap<String, Value>)               ModelInstance.run({name: ndarray})
    rmlk_schema::Op, AttributeType                           Op, AttributeType
    runtime/src/testing.rs: OpTest                           OpTest

All computation happens in librmlk_b200.so on the GPU; numpy arrays are only the host-side containers
for inputs and outputs (the reference uses Vec<T>).
"""
from __future__ import annotations

import ctypes
import enum
from typing import Dict, Optional, Sequence

import numpy as np

from . import dtypes as dt
from ._lib import last_error, lib


class InferenceError(RuntimeError):
    """Counterpart of rmlk_runtime's InferenceError (runtime/src/core/error.rs:12-14)."""

    def __init__(self, code: int, msg: str):
        super().__init__(msg)
        self.code = code


def _check(rc: int):
    if rc != 0:
        raise InferenceError(rc, last_error())


class Op(enum.IntEnum):
    """rmlk_schema::Op discriminants (schema/src/op.rs:11-51)."""
    NoOp = 0
    Add = 1
    Cast = 2
    Concat = 3
    Conv = 4
    Const = 5
    ConstantOfShape = 6
    Div = 7
    Expand = 8
    Equal = 9
    Flatten = 10
    Gather = 11
    Gemm = 12
    GlobalAveragePool = 13
    MaxPool = 14
    Mul = 15
    MatMul = 16
    Pow = 17
    Range = 18
    Relu = 19
    ReduceMean = 20
    Reshape = 21
    ScatterND = 22
    Shape = 23
    Sigmoid = 24
    Slice = 25
    Softmax = 26
    Sqrt = 27
    Sub = 28
    Transpose = 29
    Trilu = 30
    Unsqueeze = 31
    Where = 32
    Constant = 33
    Greater = 34
    Neg = 35
    Sin = 36
    Cos = 37


class AttributeType:
    """Tagged attribute values, as rmlk_schema::AttributeType."""

    class Int(int):
        pass

    class Ints(list):
        pass

    class Float(float):
        pass

    class String(str):
        pass

    class Tensor:
        def __init__(self, array):
            self.array = np.require(array, requirements="C")


def _i64(vals: Sequence[int]):
    return (ctypes.c_int64 * max(len(vals), 1))(*[int(v) for v in vals])


def _setup(l):
    if getattr(l, "_rt_ready", False):
        return l
    l.rmlk_graph_create.restype = ctypes.c_void_p
    l.rmlk_graph_destroy.argtypes = [ctypes.c_void_p]
    l.rmlk_instance_create.restype = ctypes.c_void_p
    l.rmlk_instance_create.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t]
    l.rmlk_instance_destroy.argtypes = [ctypes.c_void_p]
    l.rmlk_instance_last_launches.restype = ctypes.c_int64
    l.rmlk_instance_last_launches.argtypes = [ctypes.c_void_p]
    l.rmlk_instance_last_syncs.restype = ctypes.c_int64
    l.rmlk_instance_last_syncs.argtypes = [ctypes.c_void_p]
    for fn in (l.rmlk_instance_fused_chains, l.rmlk_instance_fused_runs, l.rmlk_instance_fused_fallbacks):
        fn.restype = ctypes.c_int64
        fn.argtypes = [ctypes.c_void_p]
    l.rmlk_instance_arena_peak.restype = ctypes.c_size_t
    l.rmlk_instance_arena_peak.argtypes = [ctypes.c_void_p]
    l.rmlk_graph_input.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    l.rmlk_graph_value.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    l.rmlk_graph_constant.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                      ctypes.c_void_p, ctypes.c_size_t]
    l.rmlk_graph_constant_device.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    l.rmlk_graph_op.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    l.rmlk_graph_attr_int.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int64]
    l.rmlk_graph_attr_ints.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_void_p]
    l.rmlk_graph_attr_float.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_float]
    l.rmlk_graph_attr_string.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_char_p]
    l.rmlk_graph_attr_tensor.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    l.rmlk_graph_output.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
    l.rmlk_instance_set_input.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                          ctypes.c_void_p, ctypes.c_int]
    l.rmlk_instance_bind.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_char_p]
    l.rmlk_instance_run.argtypes = [ctypes.c_void_p]
    l.rmlk_instance_synchronize.argtypes = [ctypes.c_void_p]
    l.rmlk_instance_value_info.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_void_p]
    l.rmlk_instance_read.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t]
    l._rt_ready = True
    return l


def _rt():
    return _setup(lib())


class OpHandle:
    """Returned by GraphBuilder.op so attributes can be chained, like the reference's OpBuilder."""

    def __init__(self, g: "GraphBuilder", node: int):
        self._g = g
        self._node = node

    def attr(self, name: str, value) -> "OpHandle":
        l, h, n = _rt(), self._g._h, self._node
        key = name.encode()
        if isinstance(value, AttributeType.Tensor):
            a = value.array
            _check(l.rmlk_graph_attr_tensor(h, n, key, dt.from_numpy(a.dtype), a.ndim, _i64(a.shape), a.ctypes.data, a.nbytes))
        elif isinstance(value, (AttributeType.Ints, list, tuple)):
            _check(l.rmlk_graph_attr_ints(h, n, key, len(value), _i64(list(value))))
        elif isinstance(value, (AttributeType.String, str)):
            _check(l.rmlk_graph_attr_string(h, n, key, str(value).encode()))
        elif isinstance(value, (AttributeType.Float, float)):
            _check(l.rmlk_graph_attr_float(h, n, key, float(value)))
        elif isinstance(value, (AttributeType.Int, int, np.integer)):
            _check(l.rmlk_graph_attr_int(h, n, key, int(value)))
        else:
            raise TypeError(f"unsupported attribute value {value!r}")
        return self


class GraphBuilder:
    """rmlk_schema::GraphBuilder (schema/src/builder.rs:122-226)."""

    def __init__(self):
        self._h = _rt().rmlk_graph_create()
        if not self._h:
            raise MemoryError("rmlk_graph_create failed")
        self.inputs: Dict[str, tuple] = {}
        self.outputs = []

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _rt().rmlk_graph_destroy(h)
            except Exception:
                pass
            self._h = None

    def input(self, name: str, dtype, dims: Sequence[int]):
        code = dtype if isinstance(dtype, int) else dt.from_numpy(dtype)
        _check(_rt().rmlk_graph_input(self._h, name.encode(), code, len(dims), _i64(dims)))
        self.inputs[name] = (code, list(dims))
        return self

    def value(self, name: str, dtype, dims: Sequence[int]):
        code = dtype if isinstance(dtype, int) else dt.from_numpy(dtype)
        _check(_rt().rmlk_graph_value(self._h, name.encode(), code, len(dims), _i64(dims)))
        return self

    def constant(self, name: str, array):
        a = np.require(array, requirements="C")
        _check(_rt().rmlk_graph_constant(self._h, name.encode(), dt.from_numpy(a.dtype), a.ndim, _i64(a.shape), a.ctypes.data, a.nbytes))
        return self

    def constant_device(self, name: str, dtype: int, dims: Sequence[int], device_ptr: int):
        """An initializer already resident in device memory; used in place (the caller keeps it alive)."""
        _check(_rt().rmlk_graph_constant_device(self._h, name.encode(), dtype, len(dims), _i64(dims), ctypes.c_void_p(device_ptr)))
        return self

    def op(self, op: Op, inputs: Sequence[Optional[str]], outputs: Sequence[str]) -> OpHandle:
        ins = (ctypes.c_char_p * max(len(inputs), 1))(*[(s or "").encode() for s in inputs])
        outs = (ctypes.c_char_p * max(len(outputs), 1))(*[s.encode() for s in outputs])
        node = _rt().rmlk_graph_op(self._h, int(op), len(inputs), ins, len(outputs), outs)
        if node < 0:
            raise InferenceError(-node, last_error())
        return OpHandle(self, node)

    def output(self, name: str):
        _check(_rt().rmlk_graph_output(self._h, name.encode()))
        self.outputs.append(name)
        return self


class ModelInstance:
    """Builder::from_graph(graph).build() + ModelInstance (runtime/src/core/instance.rs:89-221)."""

    def __init__(self, graph: GraphBuilder, device: int = 0, stream: Optional[int] = None, arena_bytes: int = 0):
        self._graph_inputs = dict(graph.inputs)
        self._outputs = list(graph.outputs)
        self._h = _rt().rmlk_instance_create(graph._h, device, ctypes.c_void_p(stream or 0), arena_bytes)
        if not self._h:
            raise InferenceError(1, last_error())
        self._keep = []

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _rt().rmlk_instance_destroy(h)
            except Exception:
                pass
            self._h = None

    close = __del__

    # -- feeding ---------------------------------------------------------------------------------
    def set_input(self, name: str, array: np.ndarray):
        """Host input: copied H2D on the instance's stream (load_inputs, instance.rs:33-56)."""
        a = np.require(array, requirements="C")
        self._keep.append(a)
        _check(_rt().rmlk_instance_set_input(self._h, name.encode(), dt.from_numpy(a.dtype), a.ndim, _i64(a.shape), a.ctypes.data, 0))

    def set_input_ptr(self, name: str, dtype: int, dims: Sequence[int], ptr: int, on_device: bool):
        """Raw pointer input: pinned host memory (on_device=False) or a device buffer used in place."""
        _check(_rt().rmlk_instance_set_input(self._h, name.encode(), dtype, len(dims), _i64(dims), ctypes.c_void_p(ptr), 1 if on_device else 0))

    def bind(self, output: str, input_: str):
        """Carry `output` of one run into `input_` of the next on the device (no host round trip)."""
        _check(_rt().rmlk_instance_bind(self._h, output.encode(), input_.encode()))

    # -- running ---------------------------------------------------------------------------------
    def launch(self):
        """Enqueue one forward pass (the op loop of instance.rs:100-112); does not wait."""
        _check(_rt().rmlk_instance_run(self._h))
        self._keep.clear()

    def synchronize(self):
        _check(_rt().rmlk_instance_synchronize(self._h))

    def value_info(self, name: str):
        d = ctypes.c_int()
        r = ctypes.c_int()
        dims = (ctypes.c_int64 * 8)()
        p = ctypes.c_void_p()
        _check(_rt().rmlk_instance_value_info(self._h, name.encode(), ctypes.byref(d), ctypes.byref(r), dims, ctypes.byref(p)))
        return d.value, list(dims)[: r.value], p.value or 0

    def read(self, name: str) -> np.ndarray:
        d, shape, _ = self.value_info(name)
        out = np.empty(shape, dtype=dt.to_numpy(d))
        _check(_rt().rmlk_instance_read(self._h, name.encode(), out.ctypes.data, out.nbytes))
        return out

    def stream_output(self, name: str, ptr: int, nbytes: int):
        """Every following run delivers graph output `name` to the (pinned) host memory at `ptr`; see wait_outputs."""
        _check(_rt().rmlk_instance_stream_output(self._h, name.encode(), ctypes.c_void_p(ptr), ctypes.c_size_t(nbytes)))

    def wait_outputs(self):
        """Returns when the outputs registered with stream_output hold the values of the last run."""
        _check(_rt().rmlk_instance_wait_outputs(self._h))

    def read_into(self, name: str, ptr: int, nbytes: int):
        _check(_rt().rmlk_instance_read(self._h, name.encode(), ctypes.c_void_p(ptr), nbytes))

    def run(self, inputs: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
        """ModelInstance::run: feed host inputs, execute, return every graph output on the host."""
        for k, v in inputs.items():
            self.set_input(k, v)
        self.launch()
        return {name: self.read(name) for name in self._outputs}

    @property
    def last_launches(self) -> int:
        return int(_rt().rmlk_instance_last_launches(self._h))

    @property
    def last_syncs(self) -> int:
        return int(_rt().rmlk_instance_last_syncs(self._h))

    @property
    def fused(self) -> tuple:
        """(chains recognised in the graph, fused launches so far, fallbacks to single ops so far)."""
        r = _rt()
        return (int(r.rmlk_instance_fused_chains(self._h)), int(r.rmlk_instance_fused_runs(self._h)), int(r.rmlk_instance_fused_fallbacks(self._h)))

    @property
    def arena_peak(self) -> int:
        return int(_rt().rmlk_instance_arena_peak(self._h))


class OpTest:
    """Single-op test helper, the counterpart of runtime/src/testing.rs:25-195.

    Feeds are wired to the op in declaration order; the graph output is named ``y``.

        out = OpTest(Op.Add).input([2, 2], [1., 2., 3., 4.], np.float32) \\
                            .input([2, 2], [1., 2., 3., 4.], np.float32).run(np.float32)
    """

    def __init__(self, op: Op):
        self.op = op
        self.feeds = []
        self.attrs = []
        self.output_dims = None

    def input(self, dims, data, dtype=None) -> "OpTest":
        a = np.asarray(data, dtype=dtype).reshape(list(dims))
        self.feeds.append(("input", f"in{len(self.feeds)}", a))
        return self

    def constant(self, dims, data, dtype=None) -> "OpTest":
        a = np.asarray(data, dtype=dtype).reshape(list(dims))
        n = sum(1 for f in self.feeds if f[0] == "constant")
        self.feeds.append(("constant", f"const{n}", a))
        return self

    def skip_input(self) -> "OpTest":
        """An omitted optional input (empty name in ONNX)."""
        self.feeds.append(("skip", "", None))
        return self

    def attr(self, name: str, value) -> "OpTest":
        self.attrs.append((name, value))
        return self

    def output(self, dims) -> "OpTest":
        self.output_dims = list(dims)
        return self

    def _execute(self, out_dtype):
        g = GraphBuilder()
        names = []
        feeds = {}
        first_dims = None
        for kind, name, a in self.feeds:
            if kind == "input":
                g.input(name, a.dtype, a.shape)
                feeds[name] = a
            elif kind == "constant":
                g.constant(name, a)
            names.append(name if kind != "skip" else None)
            if first_dims is None and a is not None:
                first_dims = list(a.shape)
        dims = self.output_dims if self.output_dims is not None else first_dims
        if dims is None:
            raise ValueError("OpTest needs .output([...]) when there are no feeds")
        g.value("y", np.dtype(out_dtype), dims)
        h = g.op(self.op, names, ["y"])
        for k, v in self.attrs:
            h.attr(k, v)
        g.output("y")
        inst = ModelInstance(g)
        try:
            out = inst.run(feeds)["y"]
            self.launches = inst.last_launches
            self.syncs = inst.last_syncs
            return out
        finally:
            inst.close()

    def run(self, out_dtype) -> np.ndarray:
        """Run the op; returns the flat output (the reference returns Vec<T>) with `.result_shape` kept."""
        out = self._execute(out_dtype)
        if out.dtype != np.dtype(out_dtype):
            raise InferenceError(1, f"output dtype {out.dtype} does not match the requested {np.dtype(out_dtype)}")
        self.result_shape = list(out.shape)
        return out.reshape(-1)

    def run_err(self) -> InferenceError:
        try:
            self._execute(np.bool_)
        except InferenceError as e:
            return e
        raise AssertionError("expected op to fail, but it succeeded")
