"""CPU tests: pin the numpy oracle (oracle/ops.py, oracle/run_op.py).

1. Against the reference's own known-answer tests (tests/golden/kats/*.json, extracted from the
   reference's op-backend test modules) and its ORT-CPU attention golden.
2. Against the reference's own kernel sources compiled for the host (oracle/_ref/libref_cpu.so), on
   seeded random inputs, for the eleven hand-written kernel families.
"""
import numpy as np
import pytest

from oracle import ops as O
from oracle import ref_calls as RC
from oracle import ref_cpu, run_op
from tests import kats
from tests.util import ulp_diff

CASES = kats.load_cases()


@pytest.mark.parametrize("case", CASES, ids=[c["id"] for c in CASES])
def test_oracle_matches_reference_kat(case):
    inputs = [kats.array(f["dims"], f["dtype"], f["data"]) for f in case["feeds"]]
    attrs = {k: kats.attr_value(v) for k, v in case["attrs"].items()}
    if case["expect"]["kind"] == "error":
        with pytest.raises(Exception) as ei:
            run_op.run(case["op"], inputs, attrs)
        assert case["expect"]["contains"].lower() in str(ei.value).lower(), (case["id"], str(ei.value))
        return
    out = run_op.run(case["op"], inputs, attrs)
    assert out.dtype == np.dtype(case["run"]), case["id"]
    if case["output"] is not None:
        assert list(out.shape) == case["output"], (case["id"], out.shape)
    kats.check(case, out.reshape(-1))


def test_oracle_attention_golden():
    """Transpose -> MatMul -> Div -> Trilu(lower) -> Softmax -> MatMul on [1,2,4] (reference
    runtime/tests/graphs/attention.rs:9-56), compared with the checked-in ORT-CPU output at 1e-5."""
    g = kats.attention()
    q, k, v = (np.array(g[n], dtype=np.float32).reshape(1, 2, 4) for n in ("q", "k", "v"))
    kt = O.transpose(k, [0, 2, 1])
    s = O.matmul(q, kt)
    s = O.binary("div", s, np.array(2.0, dtype=np.float32))
    s = O.trilu(s, 0, upper=False)
    p = O.softmax(s, -1)
    out = O.matmul(p, v)
    assert np.max(np.abs(out.reshape(-1) - np.array(g["out"], dtype=np.float32))) <= 1e-5


needs_ref = pytest.mark.skipif(not ref_cpu.available(), reason="oracle/_ref not built (run `make -C oracle`)")


def _rand(shape, dtype, seed):
    r = np.random.default_rng(seed)
    if np.dtype(dtype).kind == "f":
        return r.uniform(-4, 4, size=shape).astype(dtype)
    if np.dtype(dtype).kind == "b":
        return r.random(size=shape) > 0.5
    return r.integers(-40, 41, size=shape).astype(dtype)


@needs_ref
@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32, np.int64])
def test_oracle_vs_reference_kernels_elementwise(dtype):
    shapes = [((2, 4, 1), (4, 3)), ((1, 8, 16), ()), ((5, 7), (7,)), ((3, 1, 5), (1, 4, 1))]
    for i, (sa, sb) in enumerate(shapes):
        a, b = _rand(sa, dtype, i), _rand(sb, dtype, 10 + i)
        if np.dtype(dtype).kind == "i":
            b = np.where(b == 0, 1, b).astype(dtype)
        for op in ["add", "sub", "mul", "div", "equal", "greater"]:
            assert np.array_equal(ref_cpu.run(RC.arith(op, a, b)).reshape(-1), O.binary(op, a, b).reshape(-1)), (op, dtype)
        c = _rand(np.broadcast_shapes(sa, sb), np.bool_, 20 + i)
        assert np.array_equal(ref_cpu.run(RC.where(c, a, b)).reshape(-1), O.where(c, a, b).reshape(-1))
    x = _rand((1000,), dtype, 5)
    assert np.array_equal(ref_cpu.run(RC.unary("neg", x)), O.unary("neg", x))
    if np.dtype(dtype).kind == "f":
        xp = np.abs(x)
        assert np.array_equal(ref_cpu.run(RC.unary("sqrt", xp)), O.unary("sqrt", xp))
        for op in ("sin", "cos"):
            assert ulp_diff(ref_cpu.run(RC.unary(op, x)), O.unary(op, x)) <= 2
        e = np.array(2.0, dtype=dtype)
        assert ulp_diff(ref_cpu.run(RC.pow_(xp, e)).reshape(-1), O.pow_(xp, e).reshape(-1)) <= 2
    else:
        e = np.array(3, dtype=dtype)
        small = (x % 7).astype(dtype)
        assert np.array_equal(ref_cpu.run(RC.pow_(small, e)).reshape(-1), O.pow_(small, e).reshape(-1))
    for dst in [np.float32, np.float64, np.int32, np.int64, np.bool_, np.float16]:
        if np.dtype(dst) == np.dtype(dtype):
            continue
        assert np.array_equal(ref_cpu.run(RC.cast(x, dst)), O.cast(x, dst)), (dtype, dst)


@needs_ref
def test_oracle_vs_reference_kernels_layout_and_reduce():
    x = _rand((3, 5, 7), np.float32, 1)
    for axes in ([0], [1], [2], [0, 2], [1, 2], [0, 1, 2]):
        for keep in (True, False):
            r = ref_cpu.run(RC.reduce_mean(x, axes, keep))
            assert np.array_equal(r.reshape(-1), O.reduce_mean(x, axes, keep).reshape(-1)), axes
    xi = np.random.default_rng(2).integers(0, 1000, (4, 6)).astype(np.int64)
    assert np.array_equal(ref_cpu.run(RC.reduce_mean(xi, [1], True)).reshape(-1), O.reduce_mean(xi, [1], True).reshape(-1))
    import itertools
    for perm in itertools.permutations(range(3)):
        assert np.array_equal(ref_cpu.run(RC.transpose(x, list(perm))), O.transpose(x, list(perm)))
    for st, en, ax, sp in [([1, -1], [3, -6], [1, 2], [1, -2]), ([0], [100], [2], [3]), ([-1], [-(2 ** 63)], [0], [-1]), ([2], [2], [1], None)]:
        want = O.slice_(x, st, en, ax, sp)
        if want.size:
            assert np.array_equal(ref_cpu.run(RC.slice_(x, st, en, ax, sp, list(want.shape))), want)
    for k in (-1, 0, 1, 3):
        for up in (True, False):
            assert np.array_equal(ref_cpu.run(RC.trilu(x, k, up)), O.trilu(x, k, up))
    assert np.array_equal(ref_cpu.run(RC.expand(x[:, :1, :], [2, 3, 5, 7])), O.expand(x[:, :1, :], [2, 3, 5, 7]))
    d = _rand((6, 5, 4), np.float32, 3)
    idx = np.array([[0, 1], [2, 2], [5, 4], [-1, 0]])
    u = _rand((4, 4), np.float32, 4)
    for red in ("none", "add", "mul", "max", "min"):
        p, err = RC.scatter_nd(d, idx, u, red)
        assert np.array_equal(ref_cpu.run(p), O.scatter_nd(d, idx, u, red)) and err[0] == 0
    p, err = RC.scatter_nd(d, np.array([[6, 0]]), u[:1], "none")
    ref_cpu.run(p)
    assert err[0] == 1
    with pytest.raises(IndexError):
        O.scatter_nd(d, np.array([[6, 0]]), u[:1], "none")


def test_slice_params_edge_cases():
    """ONNX clamping incl. INT_MIN / INT_MAX sentinels (reference cuda/src/kernels/slice.rs:200-700)."""
    big, small = 2 ** 63 - 1, -(2 ** 63)
    x = np.arange(10)
    for st, en, sp, want in [(0, big, 1, x), (-1, small, -1, x[::-1]), (5, big, 2, x[5::2]), (-3, big, 1, x[-3:]), (100, big, 1, x[:0]),
                             (8, 2, -3, x[8:2:-3]), (0, 0, 1, x[:0]), (-100, 3, 1, x[:3]), (big, small, -1, x[::-1]), (3, -100, -1, x[3::-1])]:
        assert np.array_equal(O.slice_(x, [st], [en], [0], [sp]), want), (st, en, sp)


def test_range_and_matmul_shapes():
    assert np.array_equal(O.range_(0, 5, 1, np.int64), np.arange(5))
    assert np.array_equal(O.range_(10, 4, -2, np.int64), np.array([10, 8, 6]))
    assert O.range_(0, 7, 2, np.int64).tolist() == [0, 2, 4]      # truncating count, reference backend/range.rs:140-152
    assert O.range_(0.0, 1.0, 0.3, np.float32).size == 4
    a = np.ones((2, 3, 4), np.float32)
    assert O.matmul(a, np.ones((4, 5), np.float32)).shape == (2, 3, 5)
    assert O.matmul(np.ones(4, np.float32), np.ones(4, np.float32)).shape == ()
    assert O.matmul(np.ones((1, 2, 3), np.float32), np.ones((2, 3, 2), np.float32)).shape == (2, 2, 2)
    with pytest.raises(ValueError):
        O.matmul(np.ones((2, 3, 4), np.float32), np.ones((3, 4, 5), np.float32))
