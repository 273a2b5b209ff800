"""GPU: the symbol-compatible kernels (rmlk_b200/tier1) under the reference's own launch contract.

Every case builds the launch exactly as the reference's wrappers and backends would (oracle/ref_calls.py: symbol
name, positional arguments, `info` buffers, grid = ceil(n / 128) x 128 threads) and runs it twice: on the PTX made
from the reference's sources and on the PTX made from rmlk_b200/tier1.  Results must be bit-identical (the
arithmetic is the same CUDA expression per dtype), and agree with the numpy restatement where the reference's
behaviour is deliberately not copied (Trilu's unwritten elements, ScatterND's `in + 0 * out`).
"""
import itertools
import os

import numpy as np
import pytest

from oracle import ops as O
from oracle import ref_calls as RC
from oracle import ref_gpu

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
T1 = os.path.join(ROOT, "rmlk_b200", "tier1", "ptx")


@pytest.fixture(scope="module", autouse=True)
def _need(cuda):
    if not os.path.isdir(T1):
        pytest.fail("rmlk_b200/tier1/ptx is missing: run `python -m rmlk_b200.build`")
    if not ref_gpu.available():
        pytest.skip("reference PTX build (oracle/_ref/ptx) not present")


def rng(seed):
    return np.random.default_rng(seed)


def rand(shape, dtype, seed=0):
    dtype = np.dtype(dtype)
    if dtype.kind == "f":
        return rng(seed).uniform(-4, 4, size=shape).astype(dtype)
    if dtype.kind == "b":
        return rng(seed).random(size=shape) > 0.5
    return rng(seed).integers(-40, 41, size=shape).astype(dtype)


def both(make_plan):
    """Runs the plan on the reference PTX and on the tier-1 PTX (fresh buffers each time)."""
    ref = ref_gpu.run(make_plan()).copy()
    mine = ref_gpu.run(make_plan(), ptx_dir=T1).copy()
    return mine, ref


SHAPES = [((2, 2), (2, 2)), ((), ()), ((), (2, 2)), ((2, 4, 1), (4, 3)), ((1, 64, 2048), ()), ((1, 64, 2048), (1, 64, 1)),
          ((1, 64, 2048), (2048,)), ((3, 1, 5), (1, 4, 1)), ((1031,), (1031,)), ((4096,), (4096,)), ((2, 1, 3, 1, 2, 1, 3, 2), (1, 2, 1, 3, 1, 2, 1, 2))]


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "equal", "greater"])
@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32, np.int64, np.float16])
def test_binary(op, dtype):
    for i, (sa, sb) in enumerate(SHAPES):
        a, b = rand(sa, dtype, i), rand(sb, dtype, 100 + i)
        if np.dtype(dtype).kind == "i" and op == "div":
            b = np.where(b == 0, 1, b).astype(dtype)
        mine, ref = both(lambda: RC.arith(op, a, b))
        assert mine.tobytes() == ref.tobytes(), (op, dtype, sa, sb)


def test_pow_unary_cast_where():
    for bt, et in [(np.float32, np.float32), (np.float32, np.int64), (np.int64, np.int32), (np.float64, np.float64), (np.float16, np.float32),
                   (np.int32, np.float32), (np.float32, np.uint8), (np.int64, np.float16)]:
        a = rng(1).uniform(0.1, 3, size=(5, 64)).astype(bt) if np.dtype(bt).kind == "f" else rng(1).integers(-5, 6, size=(5, 64)).astype(bt)
        e = rng(2).integers(0, 4, size=(64,)).astype(et)
        mine, ref = both(lambda: RC.pow_(a, e))
        assert mine.tobytes() == ref.tobytes(), (bt, et)
        mine, ref = both(lambda: RC.pow_(a, np.array(2, dtype=et)))
        assert mine.tobytes() == ref.tobytes(), (bt, et, "scalar")
    for op, dts in [("sqrt", "fdh"), ("neg", "fdhil"), ("sin", "fdh"), ("cos", "fdh")]:
        for c in dts:
            dt = {"f": np.float32, "d": np.float64, "h": np.float16, "i": np.int32, "l": np.int64}[c]
            for n in (1, 3, 1031, 1 << 14):
                x = np.abs(rand((n,), dt, n)) if op == "sqrt" else rand((n,), dt, n)
                mine, ref = both(lambda: RC.unary(op, x))
                assert mine.tobytes() == ref.tobytes(), (op, dt, n)
    types = [np.float16, np.float32, np.float64, np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64, np.uint64, np.bool_]
    import json
    pairs = {n for n, _ in json.load(open(os.path.join(ROOT, "tests", "golden", "tier1_entry_points.json")))["cast"]}
    done = 0
    for s, d in itertools.product(types, types):
        if f"cast_fwd_{RC.TAG[np.dtype(s)]}_to_{RC.TAG[np.dtype(d)]}" not in pairs:
            continue
        x = rand((1000,), s, 5)
        if np.dtype(s).kind == "f":
            x[:6] = [0.0, -0.0, 1e30, -1e30, np.nan, np.inf] if s != np.float16 else [0.0, -0.0, 6e4, -6e4, np.nan, np.inf]
        mine, ref = both(lambda: RC.cast(x, d))
        assert mine.tobytes() == ref.tobytes(), (s, d)
        done += 1
    assert done == 100
    for dt in (np.float32, np.int64, np.float16):
        for sx, sy, sc in [((4, 5), (4, 5), (4, 5)), ((4, 5), (), (4, 5)), ((1, 1, 7, 9), (), (3, 1, 7, 9)), ((6,), (6,), ())]:
            x, y, c = rand(sx, dt, 1), rand(sy, dt, 2), rand(sc, np.bool_, 3)
            mine, ref = both(lambda: RC.where(c, x, y))
            assert mine.tobytes() == ref.tobytes(), (dt, sx, sy, sc)


def test_layout_ops():
    for dt in (np.float32, np.int64, np.float16):
        x = rand((3, 5, 6, 7), dt, 4)
        for perm in [(0, 2, 1, 3), (0, 1, 3, 2), (3, 2, 1, 0), (1, 0, 3, 2), (0, 1, 2, 3)]:
            mine, ref = both(lambda: RC.transpose(x, list(perm)))
            assert mine.tobytes() == ref.tobytes(), (dt, perm)
        for sh, tgt in [((3, 1), [3, 4]), ((1,), [2, 3]), ((), [2, 2]), ((1, 8, 1, 5, 16), [1, 8, 4, 5, 16]), ((3, 4), [2, 3, 4])]:
            e = rand(sh, dt, 3)
            mine, ref = both(lambda: RC.expand(e, tgt))
            assert mine.tobytes() == ref.tobytes(), (dt, sh, tgt)
        for sh, st, en, ax, sp in [((20, 10, 5), [0, 0], [3, 10], [0, 1], [1, 1]), ((20, 10, 5), [0, 0, 3], [20, 10, 4], None, None),
                                   ((20, 10, 5), [20, 10, 4], [0, 0, 1], [0, 1, 2], [-1, -3, -2]), ((20, 10, 5), [1], [1000], [1], [1]),
                                   ((1, 4, 9, 16), [8], [16], [3], None), ((10,), [-3], [2 ** 31 - 1], [0], [1]), ((8, 6), [-1], [-(2 ** 31)], [0], [-1])]:
            s = rand(sh, dt, 9)
            want = O.slice_(s, st, en, ax, sp)
            if want.size == 0:
                continue
            for idt in (np.int64, np.int32):
                mine, ref = both(lambda: RC.slice_(s, st, en, ax, sp, list(want.shape), idt))
                assert mine.tobytes() == ref.tobytes(), (dt, sh, st, en, ax, sp, idt)
                assert np.array_equal(mine, want)
        for sh, k, upper in [((4, 4), 0, True), ((3, 5), 1, True), ((5, 3), -1, False), ((2, 3, 4, 4), 2, False), ((7, 12), -2, True), ((6,), 0, True)]:
            t = rand(sh, dt, 8)
            mine, ref = both(lambda: RC.trilu(t, k, upper))
            assert np.array_equal(mine, O.trilu(t, k, upper)), (dt, sh, k, upper)
            assert mine.tobytes() == ref.tobytes(), (dt, sh, k, upper)   # the plan pre-zeroes the output for the reference


def test_reduce_mean_and_scatter_nd():
    for dt in (np.float32, np.float64, np.float16, np.int32, np.int64):
        for sh, axes, keep in [((1, 64, 2048), [-1], True), ((3, 4, 5), [0, 2], True), ((3, 4, 5), [1], False), ((2, 3, 4, 5), [0, 1, 2, 3], True),
                               ((7, 1, 9), [1], True), ((130, 33), [0], False)]:
            x = rand(sh, dt, 6) if np.dtype(dt).kind == "f" else rng(6).integers(0, 50, size=sh).astype(dt)
            mine, ref = both(lambda: RC.reduce_mean(x, axes, keep))
            assert mine.tobytes() == ref.tobytes(), (dt, sh, axes)
    for dt in (np.float32, np.int64, np.float16, np.float64, np.int32):
        data = rand((8, 6, 4), dt, 1)
        cases = [(np.array([[0], [3], [-1]]), rand((3, 6, 4), dt, 2)), (np.array([[1, 2], [7, 0]]), rand((2, 4), dt, 3)),
                 (np.array([[[0, 0, 0]], [[7, 5, 3]]]), rand((2, 1), dt, 4))]
        for idx, upd in cases:
            for red in ("none", "add", "mul", "max", "min"):
                def run(ptx_dir):
                    plan, err = RC.scatter_nd(data, idx, upd, red)
                    out = ref_gpu.run(plan, ptx_dir=ptx_dir).copy()
                    return out, int(err[0])
                (mine, e1), (ref, e0) = run(T1), run(None)
                assert e0 == 0 and e1 == 0
                assert mine.tobytes() == ref.tobytes(), (dt, idx.shape, red)
        plan, err = RC.scatter_nd(data, np.array([[9]]), rand((1, 6, 4), dt, 5))   # index out of range -> error code 1
        ref_gpu.run(plan, ptx_dir=T1)
        assert int(err[0]) == 1
