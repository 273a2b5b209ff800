"""GPU parity tests of the kernel launchers (include/rmlk_b200.h) called through the C ABI.

Each case runs the CUDA kernel on seeded inputs and compares with
  * the numpy restatement (oracle/ops.py), and, for the reference's hand-written kernel families,
  * the reference's own kernels: compiled for the host (oracle/ref_cpu.py) and, where the PTX build is
    present, launched on the same GPU with the reference's launch contract (oracle/ref_gpu.py).

Bars (the path's stated tolerances): bit-exact for indexing, integer, compare ops and fp32
Add/Sub/Mul/Div/Neg/Sqrt; <= 2 ulp for Pow/Sin/Cos/Sigmoid; rel 1e-5 for ReduceMean/Softmax;
rel 1e-4 for MatMul.
"""
import numpy as np
import pytest
import torch

from oracle import ops as O
from oracle import ref_calls as RC
from oracle import ref_cpu, ref_gpu
from tests.util import max_rel_to_scale, to_np, ulp_diff

pytestmark = pytest.mark.gpu

K = None


@pytest.fixture(scope="module", autouse=True)
def _k(cuda):
    global K
    from rmlk_b200 import kernels
    K = kernels
    return kernels


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rng(seed=0):
    return np.random.default_rng(seed)


def rand(shape, dtype, seed=0, lo=-4.0, hi=4.0):
    r = rng(seed)
    dtype = np.dtype(dtype)
    if dtype.kind == "f":
        return r.uniform(lo, hi, size=shape).astype(dtype)
    if dtype.kind == "b":
        return r.random(size=shape) > 0.5
    return r.integers(int(lo * 10), int(hi * 10) + 1, size=shape).astype(dtype)


def ref_gpu_run(plan):
    if not ref_gpu.available():
        return None
    return ref_gpu.run(plan)


BCAST_SHAPES = [
    ((2, 2), (2, 2)),
    ((), ()),
    ((), (2, 2)),
    ((2, 2), (1,)),
    ((2, 4, 1), (4, 3)),
    ((2, 4, 3), (3,)),
    ((1, 64, 2048), ()),
    ((1, 64, 2048), (1, 64, 1)),
    ((1, 64, 2048), (2048,)),
    ((1, 32, 7, 64), (1, 1, 7, 64)),
    ((2, 3, 5, 7), (2, 1, 5, 1)),
    ((3, 1, 5), (1, 4, 1)),
    ((1031,), (1031,)),
    ((5, 1030), (1030,)),
    ((2, 1, 3, 1, 2, 1, 3, 2), (1, 2, 1, 3, 1, 2, 1, 2)),
]


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "equal", "greater"])
@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32, np.int64, np.float16])
def test_binary_bit_exact(op, dtype):
    for i, (sa, sb) in enumerate(BCAST_SHAPES):
        a = rand(sa, dtype, seed=i)
        b = rand(sb, dtype, seed=100 + i)
        if np.dtype(dtype).kind == "i" and op == "div":
            b = np.where(b == 0, 1, b).astype(dtype)
        if op == "equal" and sa == sb and len(sa):  # make some elements equal
            b = np.where(rng(i).random(sa) > 0.5, a, b).astype(dtype)
        got = to_np(K.binary(op, dev(a), dev(b)))
        plan = RC.arith(op, a, b)
        want_cpu = ref_cpu.run(plan).reshape(got.shape)
        if dtype == np.float16 and op == "div":
            assert ulp_diff(got, want_cpu) <= 1, (op, sa, sb)  # host f16 division rounds twice
        else:
            assert np.array_equal(got, want_cpu, equal_nan=True), (op, dtype, sa, sb)
        want_np = O.binary(op, a, b).reshape(got.shape)
        if dtype != np.float16:
            assert np.array_equal(got, want_np, equal_nan=True), (op, dtype, sa, sb)
        g = ref_gpu_run(RC.arith(op, a, b))
        if g is not None:
            assert np.array_equal(got, g.reshape(got.shape), equal_nan=True), ("ref-gpu", op, dtype, sa, sb)


def test_binary_specials_f32():
    a = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, 3.4e38, 1.0], dtype=np.float32)
    b = np.array([0.0, 0.0, np.inf, np.inf, 1.0, 1e-45, 3.4e38, 3.0], dtype=np.float32)
    for op in ["add", "sub", "mul", "div", "equal", "greater"]:
        got = to_np(K.binary(op, dev(a), dev(b)))
        with np.errstate(all="ignore"):
            want = O.binary(op, a, b)
        assert np.array_equal(got, want, equal_nan=True), op
        g = ref_gpu_run(RC.arith(op, a, b))
        if g is not None:
            assert got.tobytes() == g.tobytes(), op


POW_PAIRS = [(np.float32, np.float32), (np.float32, np.int32), (np.float32, np.int64), (np.int32, np.int32),
             (np.int32, np.int64), (np.int32, np.float32), (np.int64, np.int32), (np.int64, np.int64),
             (np.int64, np.float32), (np.float64, np.float64), (np.float16, np.float32), (np.float32, np.uint8),
             (np.float64, np.int16), (np.int64, np.uint16), (np.float32, np.float16)]


@pytest.mark.parametrize("bt,et", POW_PAIRS)
def test_pow(bt, et):
    for i, (sa, sb) in enumerate([((64, 33), ()), ((1, 64, 2048), ()), ((5, 7), (7,)), ((3, 1), (1, 4))]):
        if np.dtype(bt).kind == "f":
            a = rng(i).uniform(0.1, 3.0, size=sa).astype(bt)
        else:
            a = rng(i).integers(-5, 6, size=sa).astype(bt)
        if np.dtype(et).kind == "f":
            b = rng(50 + i).uniform(-2.0, 3.0, size=sb).astype(et) if np.dtype(bt).kind == "f" else \
                rng(50 + i).integers(0, 4, size=sb).astype(et)
        else:
            b = rng(50 + i).integers(0, 4, size=sb).astype(et)
        if sb == ():
            b = np.array(2, dtype=et)
        got = to_np(K.pow_(dev(a), dev(b)))
        want = O.pow_(a, b).reshape(got.shape)
        cpu = ref_cpu.run(RC.pow_(a, b)).reshape(got.shape)
        if np.dtype(bt).kind == "f":
            assert ulp_diff(got, want) <= 2, (bt, et, sa)
            assert ulp_diff(got, cpu) <= 2, (bt, et, sa)
        else:
            assert np.array_equal(got, want)
            assert np.array_equal(got, cpu)
        g = ref_gpu_run(RC.pow_(a, b))
        if g is not None:
            assert np.array_equal(got, g.reshape(got.shape), equal_nan=True), ("ref-gpu", bt, et, sa)


@pytest.mark.parametrize("op", ["sqrt", "neg", "sin", "cos"])
@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.float16])
def test_unary(op, dtype):
    for n in [1, 3, 64, 1031, 1 << 16]:
        x = rand((n,), dtype, seed=n, lo=0.0 if op == "sqrt" else -20.0, hi=20.0)
        got = to_np(K.unary(op, dev(x)))
        want = O.unary(op, x)
        cpu = ref_cpu.run(RC.unary(op, x))
        if op in ("sqrt", "neg"):
            assert np.array_equal(got, want), (op, dtype, n)
            assert np.array_equal(got, cpu), (op, dtype, n)
        else:
            assert ulp_diff(got, want) <= 2, (op, dtype, n)
            assert ulp_diff(got, cpu) <= 2, (op, dtype, n)
        g = ref_gpu_run(RC.unary(op, x))
        if g is not None:
            assert np.array_equal(got, g), ("ref-gpu", op, dtype, n)


def test_neg_ints_sigmoid_relu():
    for dtype in [np.int32, np.int64]:
        x = rand((1000,), dtype, seed=1)
        assert np.array_equal(to_np(K.unary("neg", dev(x))), ref_cpu.run(RC.unary("neg", x)))
        assert np.array_equal(to_np(K.unary("relu", dev(x))), O.unary("relu", x))
    for dtype in [np.float32, np.float64, np.float16]:
        x = rand((4099,), dtype, seed=2, lo=-12, hi=12)
        got = to_np(K.unary("sigmoid", dev(x)))
        # distance to the correctly rounded value (computed in double); f16 rounds the f32 result once more
        truth = (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(dtype)
        assert ulp_diff(got, truth) <= 2, dtype
        assert np.array_equal(to_np(K.unary("relu", dev(x))), O.unary("relu", x))
    # the reference's own known-answer bar for sigmoid: |y - 1/(1+e^-x)| <= 1e-6 (cuda/src/kernels/sigmoid.rs:37-39)
    x = np.array([-6.0, -1.0, 0.0, 1.0, 6.0], dtype=np.float32)
    got = to_np(K.unary("sigmoid", dev(x)))
    assert np.max(np.abs(got - 1.0 / (1.0 + np.exp(-x.astype(np.float64))))) <= 1e-6
    xn = np.array([np.nan, -1.0, 2.0], dtype=np.float32)
    assert np.array_equal(to_np(K.unary("relu", dev(xn))), np.array([0.0, 0.0, 2.0], dtype=np.float32))


CAST_TYPES = [np.float16, np.float32, np.float64, np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64,
              np.uint64, np.bool_]


def _in_reference_cast_set(s, d):
    s, d = np.dtype(s), np.dtype(d)
    if s == d:
        return False
    if s.kind == "b" or d.kind == "b":
        return True
    if s.kind == "f" or d.kind == "f":
        return True
    return s.kind == d.kind  # signed<->signed, unsigned<->unsigned only


@pytest.mark.parametrize("src", CAST_TYPES)
def test_cast_all_pairs(src):
    n = 1031
    for dst in CAST_TYPES:
        if np.dtype(src).kind == "f":
            lo, hi = (0.0, 100.0) if np.dtype(dst).kind in "ub" else (-100.0, 100.0)
            x = rng(3).uniform(lo, hi, size=n).astype(src)
            x[::7] = 0
        elif np.dtype(src).kind == "b":
            x = rng(3).random(n) > 0.5
        else:
            info = np.iinfo(src)
            lo = 0 if np.dtype(dst).kind in "ub" else max(info.min, -100)
            x = rng(3).integers(lo, min(info.max, 100) + 1, size=n).astype(src)
        got = to_np(K.cast(dev(x), torch.from_numpy(np.zeros(1, dtype=dst)).dtype))
        want = O.cast(x, dst)
        assert got.dtype == np.dtype(dst)
        assert np.array_equal(got, want), (src, dst)
        if _in_reference_cast_set(src, dst):
            assert np.array_equal(got, ref_cpu.run(RC.cast(x, dst))), ("ref-cpu", src, dst)
            g = ref_gpu_run(RC.cast(x, dst))
            if g is not None:
                assert np.array_equal(got, g), ("ref-gpu", src, dst)


def test_cast_specials_match_reference_gpu():
    """Out-of-range / NaN float->int is defined on the GPU only: compare with the reference's kernels on
    the same device (cuda/src/kernels/cast.rs:1386-1414 tests inf/NaN there too)."""
    if not ref_gpu.available():
        pytest.skip("reference PTX not built")
    x = np.array([np.nan, np.inf, -np.inf, 3e38, -3e38, 1e10, -1e10, 0.5, -0.5], dtype=np.float32)
    for dst in [np.int32, np.int64, np.uint32, np.uint64, np.float16, np.bool_, np.int8]:
        got = to_np(K.cast(dev(x), torch.from_numpy(np.zeros(1, dtype=dst)).dtype))
        g = ref_gpu.run(RC.cast(x, dst))
        assert got.tobytes() == g.tobytes(), dst


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32, np.int64, np.float16])
def test_where(dtype):
    shapes = [((2, 2), (2, 2), (2, 2)), ((), (), ()), ((4, 1), (1, 5), (4, 5)), ((1, 1, 7, 12), (1, 32, 7, 12), ()),
              ((3, 5, 8), (8,), (3, 1, 1)), ((1031,), (1031,), (1031,)), ((6, 16), (), (6, 16))]
    for i, (sc, sx, sy) in enumerate(shapes):
        c = rand(sc, np.bool_, seed=i)
        x = rand(sx, dtype, seed=10 + i)
        y = rand(sy, dtype, seed=20 + i)
        got = to_np(K.where(dev(c), dev(x), dev(y)))
        want = O.where(c, x, y).reshape(got.shape)
        assert np.array_equal(got, want), (dtype, sc, sx, sy)
        assert np.array_equal(got, ref_cpu.run(RC.where(c, x, y)).reshape(got.shape))
        g = ref_gpu_run(RC.where(c, x, y))
        if g is not None:
            assert np.array_equal(got, g.reshape(got.shape))


RM_CASES = [((1, 64, 2048), [2]), ((1, 64, 2048), [-1]), ((3, 5, 7), [0]), ((3, 5, 7), [1]), ((3, 5, 7), [2]),
            ((3, 5, 7), [0, 1]), ((3, 5, 7), [1, 2]), ((3, 5, 7), [0, 2]), ((3, 5, 7), [0, 1, 2]), ((4, 6, 8, 10), [1, 3]),
            ((4, 6, 8, 10), [0, 2]), ((300, 260), [1]), ((300, 260), [0]), ((2, 5000), [1]), ((5000, 2), [0]),
            ((7,), [0]), ((1, 1, 1), [1]), ((2, 3, 1, 4), [2]), ((33, 1024), [1]), ((2048, 64), [1])]


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.float16, np.int32, np.int64])
def test_reduce_mean(dtype):
    for i, (sh, axes) in enumerate(RM_CASES):
        if np.dtype(dtype).kind == "i":
            x = rng(i).integers(0, 1000, size=sh).astype(dtype)
        else:
            x = rand(sh, dtype, seed=i)
        for keep in (True, False):
            got = to_np(K.reduce_mean(dev(x), axes, keep))
            want = O.reduce_mean(x, axes, keep)
            cpu = ref_cpu.run(RC.reduce_mean(x, axes, keep))
            assert got.shape == tuple(want.shape), (sh, axes, keep)
            if np.dtype(dtype).kind == "i":
                assert np.array_equal(got, want), (dtype, sh, axes)
                assert np.array_equal(got, cpu.reshape(got.shape))
            else:
                tol = 1e-5 if dtype != np.float16 else 2e-3
                assert max_rel_to_scale(got, want) <= tol, (dtype, sh, axes)
                assert max_rel_to_scale(got, cpu.reshape(got.shape)) <= tol
                if dtype == np.float32:  # both are double-accumulated: at most one rounding apart
                    assert ulp_diff(got, cpu.reshape(got.shape)) <= 1, (sh, axes)


@pytest.mark.parametrize("shape", [(1, 4), (2, 3), (1, 32, 7, 12), (64, 128), (3, 4096), (5, 641), (2, 8, 1, 640), (7, 1000),
                                    (2, 2052), (4, 8192), (1, 20000), (2048, 513), (1, 1)])
def test_softmax(shape):
    x = rand(shape, np.float32, seed=shape[-1], lo=-6, hi=6)
    got = to_np(K.softmax(dev(x)))
    want = O.softmax(x)
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-30)) <= 1e-5
    assert np.allclose(got.sum(-1), 1.0, atol=1e-5)
    # the reference's masked-row case (backend/softmax.rs:259-275): -10000 logits go to exactly 0
    xm = x.copy()
    xm[..., shape[-1] // 2:] = -10000.0
    gm = to_np(K.softmax(dev(xm)))
    assert np.all(gm[..., shape[-1] // 2:] == 0.0) or shape[-1] == 1
    assert np.max(np.abs(gm - O.softmax(xm))) <= 1e-5
    for dtype, tol in [(np.float64, 1e-12), (np.float16, 2e-3)]:
        xd = x.astype(dtype)
        gd = to_np(K.softmax(dev(xd)))
        assert np.max(np.abs(gd.astype(np.float64) - O.softmax(xd.astype(np.float64)))) <= tol


MM_CASES = [(1, 1, 8192, 2048), (1, 8, 8192, 2048), (1, 16, 512, 2048), (1, 64, 2048, 2048), (1, 128, 1024, 256), (1, 1, 64, 64),
            (1, 3, 5, 7), (1, 2, 2, 2), (1, 17, 33, 65), (1, 70, 130, 50), (1, 129, 257, 100), (32, 1, 641, 64), (32, 1, 64, 641),
            (8, 128, 128, 64), (8, 128, 64, 128), (3, 5, 30, 9), (1, 1, 2048, 8192), (1, 200, 300, 4), (1, 4, 100, 1), (2, 16, 31, 1000),
            # many problems with a short K (one thread per column quad, no reduction)
            (2048, 1, 520, 64), (600, 2, 512, 128), (300, 4, 1024, 256), (300, 3, 1024, 252), (2048, 1, 160, 4),
            (2048, 1, 523, 64), (700, 2, 517, 128), (400, 4, 1001, 40), (400, 3, 1001, 252),
            # many problems with a narrow right operand (one CTA per problem, whole rows of B per load)
            (512, 4, 64, 523), (300, 1, 32, 100), (200, 3, 128, 77), (160, 2, 20, 1500), (150, 4, 4, 9)]


@pytest.mark.parametrize("case", MM_CASES)
def test_matmul(case):
    batch, m, n, k = case
    a = rng(1).normal(0, 1.0, size=(batch, m, k)).astype(np.float32)
    b = rng(2).normal(0, 1.0, size=(batch, k, n)).astype(np.float32)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    got = to_np(K.matmul(dev(a), dev(b)))
    assert max_rel_to_scale(got, want) <= 1e-4, case
    # with split-K scratch (same answer up to fp32 reassociation)
    ws_bytes = K.matmul_workspace_bytes(batch, m, n, k)
    if ws_bytes:
        ws = torch.empty(ws_bytes // 4, dtype=torch.float32, device="cuda")
        got2 = to_np(K.matmul(dev(a), dev(b), workspace=ws))
        assert max_rel_to_scale(got2, want) <= 1e-4, case
        got3 = to_np(K.matmul(dev(a), dev(b), workspace=ws))
        assert got2.tobytes() == got3.tobytes(), "split-K must be deterministic"
    # broadcast B over the batch (reference materialises copies, backend/matmul.rs:48-86)
    if batch > 1:
        got_b = to_np(K.matmul(dev(a), dev(b[0])))
        want_b = np.matmul(a.astype(np.float64), b[0].astype(np.float64))
        assert max_rel_to_scale(got_b, want_b) <= 1e-4


def test_matmul_small_integers_exact():
    """Integer-valued operands as in the reference's op tests (backend/matmul.rs:378-590): exact."""
    a = np.arange(1, 7, dtype=np.float32).reshape(2, 3)
    b = np.arange(7, 19, dtype=np.float32).reshape(3, 4)
    assert np.array_equal(to_np(K.matmul(dev(a), dev(b))), a @ b)
    a4 = np.ones((1, 24, 6, 6), dtype=np.float32)
    b4 = np.full((1, 24, 6, 128), 13.0, dtype=np.float32)
    assert np.all(to_np(K.matmul(dev(a4), dev(b4))) == 78.0)


@pytest.mark.parametrize("case", [(1, 64, 2048, 512), (1, 3, 5, 7), (1, 70, 130, 50), (3, 17, 33, 65), (8, 128, 64, 128), (2, 1, 100, 1), (1, 5, 9, 0)])
def test_matmul_f16(case):
    """f16 MatMul (cuBLAS with CUBLAS_COMPUTE_16F in the reference, cuda/src/params.rs:24-31): fp32 accumulation and one
    rounding to f16 here, so the result is the correctly rounded f16 of the exact product up to one f16 ulp."""
    batch, m, n, k = case
    a = rng(5).normal(0, 1.0, size=(batch, m, k)).astype(np.float16)
    b = rng(6).normal(0, 1.0, size=(batch, k, n)).astype(np.float16)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    got = to_np(K.matmul(dev(a), dev(b)))
    assert got.dtype == np.float16 and got.shape == want.shape
    err = np.abs(got.astype(np.float64) - want)
    assert np.all(err <= np.maximum(np.abs(want), 2.0 ** -14) * 2.0 ** -10 + 1e-6 * np.sqrt(max(k, 1))), case
    if batch > 1:   # right operand shared by the batch
        got_b = to_np(K.matmul(dev(a), dev(b[0])))
        want_b = np.matmul(a.astype(np.float64), b[0].astype(np.float64))
        assert np.all(np.abs(got_b.astype(np.float64) - want_b) <= np.maximum(np.abs(want_b), 2.0 ** -14) * 2.0 ** -10 + 1e-6 * np.sqrt(k))
    # integer-valued operands: exact
    ai = rng(7).integers(-4, 5, size=(batch, m, max(k, 1))).astype(np.float16)
    bi = rng(8).integers(-4, 5, size=(batch, max(k, 1), n)).astype(np.float16)
    assert np.array_equal(to_np(K.matmul(dev(ai), dev(bi))).astype(np.float64), np.matmul(ai.astype(np.float64), bi.astype(np.float64)))


@pytest.mark.parametrize("dtype", [np.float32, np.int64, np.float16, np.uint8])
def test_gather(dtype):
    cases = [((3, 4), [0, 2], 0), ((3, 4), [-3, -1], 0), ((3, 4), [1, 3], 1), ((2, 3, 4), [[1, 2], [0, -1]], 1),
             ((1000, 2048), list(rng(1).integers(0, 1000, 77)), 0), ((5, 6, 7), [2, 2, 0], 2), ((50, 3), [[0, 49]], 0),
             ((4, 1030), [3, 0], 0)]
    for sh, idx, axis in cases:
        x = rand(sh, dtype, seed=5) if np.dtype(dtype).kind != "u" else rng(5).integers(0, 255, sh).astype(dtype)
        for it in (np.int64, np.int32):
            ix = np.array(idx, dtype=it)
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            got = to_np(K.gather(dev(x), dev(ix), axis, status))
            assert np.array_equal(got, O.gather(x, ix, axis)), (sh, axis)
            assert int(status.item()) == 0
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    K.gather(dev(rand((3, 4), dtype, 1) if np.dtype(dtype).kind != "u" else np.zeros((3, 4), dtype)), dev(np.array([0, 3], dtype=np.int64)), 0, status)
    assert int(status.item()) == 1  # out-of-range index is reported, not dereferenced


@pytest.mark.parametrize("dtype", [np.float32, np.int64, np.float64, np.int32, np.float16])
def test_scatter_nd(dtype):
    d = rand((6, 5, 4), dtype, seed=1)
    cases = [(np.array([[0], [3], [5]]), (3, 5, 4)), (np.array([[0, 1], [2, 2], [5, 4], [-1, 0]]), (4, 4)),
             (np.array([[1, 2, 3], [0, 0, 0]]), (2,)), (np.array([[[1], [2]], [[4], [-6]]]), (2, 2, 5, 4))]
    for idx, ush in cases:
        u = rand(ush, dtype, seed=7)
        for red in ["none", "add", "mul", "max", "min"]:
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            got = to_np(K.scatter_nd(dev(d), dev(idx.astype(np.int64)), dev(u), red, status))
            want = O.scatter_nd(d, idx, u, red)
            if dtype == np.float16 and red in ("add", "mul"):
                assert ulp_diff(got, want) <= 1
            else:
                assert np.array_equal(got, want), (dtype, red, idx.shape)
            plan, err = RC.scatter_nd(d, idx, u, red)
            cpu = ref_cpu.run(plan)
            if not (dtype == np.float16 and red in ("add", "mul")):
                assert np.array_equal(got, cpu), ("ref-cpu", dtype, red)
            assert int(status.item()) == 0 and int(err[0]) == 0
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    K.scatter_nd(dev(d), dev(np.array([[6]], dtype=np.int64)), dev(rand((1, 5, 4), dtype, 3)), "none", status)
    assert int(status.item()) == 1  # reference error code 1: index outside [0, dim)


SLICE_CASES = [
    ((3, 5, 7), [1, -1], [3, -6], [1, 2], [1, -2]),
    ((1, 24, 27, 128), [0], [64], [3], None),
    ((1, 24, 27, 128), [64], [128], [-1], [1]),
    ((1, 32, 5, 64), [32], [2 ** 63 - 1], [3], [1]),
    ((20,), [0], [20], None, [3]),
    ((20,), [-1], [-(2 ** 63)], [0], [-1]),
    ((20, 10), [5, 0], [1, 10], [0, 1], [-2, 3]),
    ((4, 6), [10], [20], [0], None),
    ((4, 6), [2, 1], [2, 5], None, None),
    ((6, 8, 10), [1, 2, 3], [5, 7, 9], [0, 1, 2], [2, 2, 2]),
    ((2, 3, 4, 5), [0], [1], [1], None),
    ((8, 1024), [0], [512], [1], None),
    ((8, 1024), [2], [1024], [1], [2]),
]


@pytest.mark.parametrize("dtype", [np.float32, np.int64, np.float16])
def test_slice(dtype):
    for sh, st, en, ax, sp in SLICE_CASES:
        x = rand(sh, dtype, seed=9)
        got = to_np(K.slice_(dev(x), st, en, ax, sp))
        want = O.slice_(x, st, en, ax, sp)
        assert got.shape == want.shape, (sh, st, en, ax, sp)
        assert np.array_equal(got, want), (sh, st, en, ax, sp)
        if want.size:
            cpu = ref_cpu.run(RC.slice_(x, st, en, ax, sp, list(want.shape)))
            assert np.array_equal(got, cpu), ("ref-cpu", sh, st, en, ax, sp)


@pytest.mark.parametrize("dtype", [np.float32, np.int64, np.float16, np.uint8])
def test_transpose_all_4d_perms(dtype):
    import itertools
    x = rand((3, 5, 34, 66), dtype, seed=4) if np.dtype(dtype).kind != "u" else rng(4).integers(0, 255, (3, 5, 34, 66)).astype(dtype)
    for perm in itertools.permutations(range(4)):
        got = to_np(K.transpose(dev(x), list(perm)))
        assert np.array_equal(got, O.transpose(x, list(perm))), perm
    if dtype in (np.float32, np.int64, np.float16):
        for perm in [(0, 2, 1, 3), (0, 1, 3, 2), (3, 2, 1, 0)]:
            cpu = ref_cpu.run(RC.transpose(x, list(perm)))
            assert np.array_equal(to_np(K.transpose(dev(x), list(perm))), cpu)


def test_transpose_other_ranks():
    # shapes whose extents are multiples of 4 take the 64 x 64 tile kernel with 16-byte accesses
    for sh, perm in [((3, 5, 36, 68), [0, 1, 3, 2]), ((3, 5, 36, 68), [3, 2, 1, 0]), ((3, 8, 36, 68), [3, 0, 2, 1]), ((2, 100, 260), [0, 2, 1]),
                     ((4, 4, 4, 4), [3, 1, 2, 0]), ((1000, 520), [1, 0]), ((64, 64), [1, 0]), ((2, 8, 520, 64), [0, 1, 3, 2]),
                     ((3, 4, 200, 12), [2, 3, 0, 1]),
                     # only one side 16-byte aligned (rows of odd length on the other)
                     ((2, 8, 523, 64), [0, 1, 3, 2]), ((2, 8, 64, 523), [0, 1, 3, 2]), ((130, 257), [1, 0]), ((3, 77, 68), [0, 2, 1]),((7,), [0]), ((5, 9), [1, 0]), ((5, 9), None), ((2, 3, 4), [2, 0, 1]), ((1, 1, 5), [2, 1, 0]),
                     ((2, 3, 4, 5, 6), [4, 2, 0, 3, 1]), ((1, 128, 32, 64), [0, 2, 1, 3]), ((1, 8, 640, 64), [0, 1, 3, 2]),
                     ((2, 2, 2, 2, 2, 2, 2, 2), [7, 6, 5, 4, 3, 2, 1, 0]), ((100, 1), [1, 0])]:
        x = rand(sh, np.float32, seed=6)
        assert np.array_equal(to_np(K.transpose(dev(x), perm)), O.transpose(x, perm)), (sh, perm)


@pytest.mark.parametrize("dtype", [np.float32, np.int64, np.float16])
def test_concat(dtype):
    cases = [([(2, 3), (2, 3)], 0), ([(2, 3), (2, 5)], 1), ([(1, 8, 0, 64), (1, 8, 5, 64)], 2), ([(1, 8, 7, 64), (1, 8, 1, 64)], 2),
             ([(2, 3, 32), (2, 3, 32)], -1), ([(3,), (4,), (5,)], 0), ([(2, 1, 3), (2, 2, 3), (2, 3, 3)], 1),
             ([(4, 5)] * 20, 1), ([(1, 2, 3, 1), (1, 2, 3, 1)], 3), ([(64, 8, 512, 64), (64, 8, 1, 64)], 2)]
    for shapes, axis in cases:
        xs = [rand(s, dtype, seed=i) for i, s in enumerate(shapes)]
        got = to_np(K.concat([dev(x) for x in xs], axis))
        assert np.array_equal(got, O.concat(xs, axis)), (shapes, axis)


@pytest.mark.parametrize("dtype", [np.float32, np.int64, np.float16])
def test_expand(dtype):
    cases = [((3, 1), [3, 4]), ((1,), [2, 3]), ((), [2, 2]), ((1, 8, 1, 5, 64), [1, 8, 4, 5, 64]), ((2, 1, 6), [1, 1, 1]),
             ((3, 4), [2, 3, 4]), ((1, 1, 7, 12), [1, 32, 7, 12]), ((5,), [5]), ((1, 3), [4, 1, 1]),
             # one broadcast block between dense parts: the load-once / store-R-times kernel
             ((16, 8, 1, 37, 64), [16, 8, 4, 37, 64]), ((3, 1, 1, 8), [3, 5, 2, 8]), ((3, 1, 2, 1, 8), [3, 5, 2, 2, 8])]
    for sh, tgt in cases:
        x = rand(sh, dtype, seed=3)
        got = to_np(K.expand(dev(x), tgt))
        want = O.expand(x, tgt)
        assert np.array_equal(got, want), (sh, tgt)
        assert np.array_equal(got, ref_cpu.run(RC.expand(x, tgt)).reshape(got.shape))


@pytest.mark.parametrize("dtype", [np.float32, np.int64, np.float16, np.float64])
def test_trilu(dtype):
    for sh in [(4, 4), (3, 5), (5, 3), (2, 3, 4, 4), (1, 1, 7, 12), (6,), (128, 640), (2, 33, 33)]:
        x = rand(sh, dtype, seed=8)
        x = np.where(x == 0, 1, x).astype(dtype)
        for k in [0, 1, -1, 2, -2, 100, -100, 6]:
            for upper in (True, False):
                got = to_np(K.trilu(dev(x), k, upper))
                want = O.trilu(x, k, upper)
                assert np.array_equal(got, want), (sh, k, upper)
                if upper or k >= -1:  # the reference's lower-triangle `end` wraps when k + row + 1 < 0
                    assert np.array_equal(got, ref_cpu.run(RC.trilu(x, k, upper))), ("ref-cpu", sh, k, upper)


def test_range_and_fill():
    for dtype, start, delta, n in [(torch.int64, 0, 1, 640), (torch.int64, 5, -2, 7), (torch.int32, 3, 3, 100),
                                   (torch.float32, 0.0, 2.0, 32), (torch.float32, 0.1, 0.3, 1000), (torch.float64, -1.5, 0.7, 333),
                                   (torch.float16, 0.0, 0.5, 40)]:
        got = to_np(K.range_(start, delta, n, dtype))
        npdt = got.dtype
        want = O.range_(start, npdt.type(start) + npdt.type(delta) * npdt.type(n), delta, npdt)[:n]
        i = np.arange(n).astype(npdt)
        want = (npdt.type(start) + (i * npdt.type(delta)).astype(npdt)).astype(npdt)
        assert np.array_equal(got, want), (dtype, start, delta)
    for dtype, v in [(torch.float32, 1.5), (torch.int64, -7), (torch.bool, True), (torch.float16, 0.25)]:
        got = K.fill(v, 1031, dtype)
        assert bool((got == v).all())


def test_large_elementwise_and_copy_roundtrip():
    """Full-size property checks: 2^26-element add is linear; slice/concat and transpose round-trip."""
    n = 1 << 26
    a = torch.randn(n, device="cuda")
    b = torch.randn(n, device="cuda")
    s = K.binary("add", a, b)
    assert torch.equal(s, a + b)
    d = K.binary("sub", s, b)
    assert torch.allclose(d, a, atol=1e-5)
    x = torch.randn(64, 8, 513, 64, device="cuda")
    left = K.slice_(x, [0], [512], [2], None)
    right = K.slice_(x, [512], [513], [2], None)
    assert torch.equal(K.concat([left, right], 2), x)
    t = K.transpose(x, [0, 1, 3, 2])
    assert torch.equal(K.transpose(t, [0, 1, 3, 2]), x)
    assert torch.equal(t, x.permute(0, 1, 3, 2).contiguous())


TC_CASES = [(64, 8192, 2048), (64, 2048, 2048), (64, 512, 2048), (64, 2048, 8192), (17, 128, 32), (33, 256, 64), (100, 384, 96), (128, 1024, 256),
            (200, 256, 512), (300, 128, 2048), (64, 128256, 2048), (4096, 8192, 2048), (65, 128, 4096),
            # K split 7, 5 and 3 ways inside a thread-block cluster (rows of the tile not divisible by the split)
            (64, 2688, 2048), (64, 3712, 2048), (64, 6272, 2048), (17, 2688, 2048), (128, 2688, 1024),
            # merged q|k|v and gate|up projections of the 1B shape; the 8B shape (hidden 4096, FFN 14336) at decode and prefill M
            (64, 3072, 2048), (64, 16384, 2048), (64, 14336, 4096), (64, 4096, 14336), (4096, 14336, 4096), (4096, 4096, 14336)]


@pytest.mark.parametrize("case", TC_CASES)
def test_matmul_tensor_core_3xtf32(case):
    """Shapes that take the tcgen05 path (M > 16, N % 128 == 0, K % 32 == 0): fp32-level accuracy from the
    3xTF32 split (far inside the rel 1e-4 bar), with and without the split-K scratch, deterministic, and
    the bounded-wait status word stays clear."""
    m, n, k = case
    a = torch.randn(m, k, device="cuda") * 0.5
    w = torch.randn(k, n, device="cuda") * 0.02
    # reference in double on the GPU for the large cases (torch used as a checker only), numpy for small ones
    want = (a.double() @ w.double())
    scale = float(want.abs().max())
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    import ctypes
    from rmlk_b200 import dtypes as dt
    from rmlk_b200._lib import lib

    def run(ws):
        out = torch.empty(m, n, device="cuda")
        rc = lib().rmlk_b200_matmul_ex(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), dt.F32, ctypes.c_int64(1), ctypes.c_int64(m),
                                       ctypes.c_int64(n), ctypes.c_int64(k), ctypes.c_void_p(a.data_ptr()), ctypes.c_int64(0),
                                       ctypes.c_void_p(w.data_ptr()), ctypes.c_int64(0), ctypes.c_void_p(out.data_ptr()), ctypes.c_int64(m * n),
                                       ctypes.c_void_p(ws.data_ptr() if ws is not None else 0),
                                       ctypes.c_size_t(ws.numel() * 4 if ws is not None else 0), ctypes.c_void_p(status.data_ptr()))
        assert rc == 0
        return out

    got = run(None)
    assert int(status.item()) == 0, "a bounded wait expired"
    err = float((got.double() - want).abs().max()) / scale
    # The bar is 1e-4.  The tensor core adds into its fp32 accumulator with truncation, so the error grows with the number
    # of k-steps accumulated in one tile: about 1e-5 at K = 2048, 4e-5 at 8192, 7e-5 at 14336 (cuBLAS fp32: 5e-6 there).
    tol = 5e-5 if k <= 8192 else 1e-4
    assert err <= tol, (case, err)
    wsb = K.matmul_workspace_bytes(1, m, n, k)
    if wsb:
        ws = torch.empty(wsb // 4, device="cuda")
        g2 = run(ws)
        g3 = run(ws)
        assert int(status.item()) == 0
        assert float((g2.double() - want).abs().max()) / scale <= tol
        assert torch.equal(g2, g3)
    # exact on small integers: hi/lo split must not lose anything when the products are exactly representable
    ai = torch.randint(-8, 9, (m, k), device="cuda").float()
    wi = torch.randint(-8, 9, (k, n), device="cuda").float()
    a, w = ai, wi
    assert torch.equal(run(None), (ai.double() @ wi.double()).float())


NT_CASES = [(512, 4, 523, 64), (7, 1, 100, 64), (5, 2, 33, 16), (3, 3, 70, 128), (9, 8, 45, 32), (4, 4, 31, 4), (2, 4, 1000, 20),
            # shapes outside the warp-per-32-rows kernel: K not a multiple of 4, K > 128, M > 8
            (3, 2, 50, 30), (2, 3, 40, 300), (2, 20, 35, 64)]


@pytest.mark.parametrize("m", [1, 8, 16])
@pytest.mark.parametrize("kn", [(4096, 14336), (14336, 4096), (2048, 8192), (2048, 128256)])
def test_matmul_decode_rows_on_8b_and_1b_shapes(m, kn):
    """The memory-bound small-M MatMul (M <= 16) on the sweep's shapes: [M, 4096] x [4096, 14336] and [M, 14336] x
    [14336, 4096] (8B shape), [M, 2048] x [2048, 8192] and the 1B lm_head; operands N(0, 0.02) as in the sweep, against
    float64 on the same device; with and without split-K scratch; deterministic."""
    k, n = kn
    g = torch.Generator(device="cuda")
    g.manual_seed(100 + m)
    a = torch.randn(m, k, device="cuda", generator=g) * 0.02
    w = torch.randn(k, n, device="cuda", generator=g) * 0.02
    want = a.double() @ w.double()
    scale = float(want.abs().max())
    got = K.matmul(a, w)
    assert float((got.double() - want).abs().max()) <= 1e-4 * scale
    wsb = K.matmul_workspace_bytes(1, m, n, k)
    if wsb:
        ws = torch.empty(wsb // 4, device="cuda")
        g2 = K.matmul(a, w, workspace=ws)
        assert float((g2.double() - want).abs().max()) <= 1e-4 * scale
        assert torch.equal(g2, K.matmul(a, w, workspace=ws))


@pytest.mark.parametrize("case", NT_CASES)
def test_matmul_nt(case):
    """A x B^T with B stored [n, k]: equals MatMul(A, Transpose(B)) of the reference path within the MatMul bar."""
    batch, m, n, k = case
    a = rng(11).normal(0, 1.0, size=(batch, m, k)).astype(np.float32)
    b = rng(12).normal(0, 1.0, size=(batch, n, k)).astype(np.float32)
    want = np.matmul(a.astype(np.float64), np.swapaxes(b, 1, 2).astype(np.float64))
    got = to_np(K.matmul_nt(dev(a), dev(b)))
    assert got.shape == want.shape
    assert max_rel_to_scale(got, want) <= 1e-4, case
    # same numbers as the two-op path (Transpose copy, then MatMul) up to fp32 reassociation
    two_op = to_np(K.matmul(dev(a), K.transpose(dev(b), [0, 2, 1])))
    assert max_rel_to_scale(got, two_op.astype(np.float64)) <= 1e-5


def test_strided_copy_views():
    """Dense copy of strided / broadcast / permuted views of one buffer, against numpy's as_strided."""
    from numpy.lib.stride_tricks import as_strided
    base = rand((6 * 8 * 10 * 12,), np.float32, seed=13)
    cases = [((6, 8, 10, 12), (960, 120, 12, 1)),            # identity
             ((6, 8, 4, 10, 12), (960, 120, 0, 12, 1)),      # repeat a middle dim
             ((6, 12, 10, 8), (960, 1, 12, 120)),            # permuted, inner dim moves
             ((6, 8, 4, 12, 10), (960, 120, 0, 1, 12)),      # repeat + inner transpose
             ((3, 6, 8), (0, 960, 120)),                     # leading broadcast, strided inner
             ((5,), (0,)), ((), ()), ((6, 0, 3), (960, 1, 1))]
    for shape, strides in cases:
        got = to_np(K.strided_copy(dev(base), shape, strides))
        want = as_strided(base, shape=shape, strides=[4 * s for s in strides]) if len(shape) else base[:1].reshape(())
        assert got.shape == tuple(shape)
        assert np.array_equal(got, want), (shape, strides)
    b64 = rand((4 * 6 * 8,), np.int64, seed=14)
    got = to_np(K.strided_copy(dev(b64), (8, 4, 6), (1, 48, 8)))
    assert np.array_equal(got, np.ascontiguousarray(as_strided(b64, shape=(8, 4, 6), strides=(8, 384, 64))))


def test_strided_copy_to_places_views_inside_a_larger_buffer():
    """View -> view copy in one launch (new rows of a KV cache going into their slot): against torch's own copy_."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(21)
    # rows [B, KV, S, D] that exist as a permuted block of columns of a wider matrix, into [B, KV, cap, D] at row T
    for (B, KV, S, D, cap, T, wide, col0) in [(64, 8, 1, 64, 700, 523, 3072, 2560), (3, 2, 5, 16, 40, 7, 200, 33), (2, 4, 1, 6, 9, 8, 31, 3),
                                              (1, 1, 1, 64, 64, 63, 64, 0)]:
        src_buf = torch.randn(B * S, wide, device="cuda", generator=g)
        src = src_buf[:, col0:col0 + KV * D].view(B, S, KV, D).permute(0, 2, 1, 3)
        for dtype in (torch.float32, torch.int64, torch.float16):
            sb = (src_buf * 100).to(dtype)
            sv = sb[:, col0:col0 + KV * D].view(B, S, KV, D).permute(0, 2, 1, 3)
            cache = torch.zeros(B, KV, cap, D, device="cuda", dtype=dtype)
            want = cache.clone()
            want[:, :, T:T + S, :].copy_(sv)
            K.strided_copy_to(sv, cache[:, :, T:T + S, :])
            assert torch.equal(cache, want), (B, KV, S, D, dtype)
    # broadcast source, scalar, inner-dim transposes on both sides
    a = torch.randn(7, device="cuda", generator=g)
    out = torch.zeros(5, 7, 3, device="cuda")
    K.strided_copy_to(a.view(1, 7, 1).expand(5, 7, 3), out)
    assert torch.equal(out, a.view(1, 7, 1).expand(5, 7, 3).contiguous())
    m = torch.randn(33, 65, device="cuda", generator=g)
    outT = torch.zeros(65, 40, device="cuda")
    K.strided_copy_to(m.t(), outT[:, 2:35])
    assert torch.equal(outT[:, 2:35], m.t()) and float(outT[:, :2].abs().sum()) == 0.0 and float(outT[:, 35:].abs().sum()) == 0.0
    s0 = torch.tensor(3.5, device="cuda")
    d0 = torch.zeros((), device="cuda")
    K.strided_copy_to(s0, d0)
    assert float(d0) == 3.5


def test_rope_writes_into_a_cache_slot():
    """The rotary kernel with a placed output: same bits as the dense result, nothing outside the slot touched."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(22)
    for (B, KV, S, D, cap, T) in [(64, 8, 1, 64, 600, 523), (2, 3, 4, 16, 20, 5), (1, 1, 1, 2, 3, 2)]:
        xb = torch.randn(B, S, KV, D, device="cuda", generator=g)
        x = xb.permute(0, 2, 1, 3)
        cos, sin = torch.randn(B, 1, S, D, device="cuda", generator=g), torch.randn(B, 1, S, D, device="cuda", generator=g)
        want = K.rope(x, cos, sin)
        cache = torch.full((B, KV, cap, D), 7.0, device="cuda")
        K.rope(x, cos, sin, out=cache[:, :, T:T + S, :])
        assert torch.equal(cache[:, :, T:T + S, :], want)
        assert float((cache[:, :, :T, :] - 7.0).abs().sum()) == 0.0 and float((cache[:, :, T + S:, :] - 7.0).abs().sum()) == 0.0
