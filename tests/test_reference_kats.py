"""GPU: the reference's own op tests, replayed through this build's production entry point.

Every case of tests/golden/kats/*.json (extracted from the `OpTest`-style test modules of the reference's
runtime/src/providers/cuda/backend/*.rs) is rebuilt as a one-op graph and run through
GraphBuilder -> ModelInstance.run, i.e. through librmlk_b200.so's host runtime and CUDA kernels, with the
reference's expected values, tolerances and error expectations.  A few reference tests that compute
their expectation in host code are restated by hand at the end.
"""
import numpy as np
import pytest

from tests import kats

pytestmark = pytest.mark.gpu

CASES = kats.load_cases()


@pytest.fixture(scope="module")
def rt(cuda):
    from rmlk_b200 import runtime
    return runtime


def build(rt, case):
    t = rt.OpTest(rt.Op[case["op"]])
    for f in case["feeds"]:
        a = kats.array(f["dims"], f["dtype"], f["data"])
        (t.input if f["kind"] == "input" else t.constant)(f["dims"], a)
    for k, v in case["attrs"].items():
        val = kats.attr_value(v)
        t.attr(k, rt.AttributeType.Tensor(val) if v["kind"] == "tensor" else val)
    if case["output"] is not None:
        t.output(case["output"])
    return t


@pytest.mark.parametrize("case", CASES, ids=[c["id"] for c in CASES])
def test_reference_kat(rt, case):
    t = build(rt, case)
    if case["expect"]["kind"] == "error":
        err = t.run_err()
        assert case["expect"]["contains"].lower() in str(err).lower(), (case["id"], str(err))
        return
    out = t.run(np.dtype(case["run"]))
    if case["output"] is not None:
        assert t.result_shape == case["output"], (case["id"], t.result_shape)
    kats.check(case, out)
    assert t.syncs == 0, "small operands must be served from host mirrors, not D2H reads"


def test_attention_golden(rt):
    """runtime/tests/graphs/attention.rs:9-56: Transpose -> MatMul -> Div -> Trilu(lower) -> Softmax -> MatMul on
    [1,2,4], against the reference's checked-in ORT-CPU output at abs 1e-5."""
    g = kats.attention()
    q, k, v = (np.array(g[n], dtype=np.float32).reshape(1, 2, 4) for n in ("q", "k", "v"))
    b = rt.GraphBuilder()
    for n in ("q", "k", "v"):
        b.input(n, np.float32, [1, 2, 4])
    b.constant("scale", np.array(2.0, dtype=np.float32))
    for n, d in [("kt", [1, 4, 2]), ("scores", [1, 2, 2]), ("scaled", [1, 2, 2]), ("masked", [1, 2, 2]), ("probs", [1, 2, 2]), ("out", [1, 2, 4])]:
        b.value(n, np.float32, d)
    b.op(rt.Op.Transpose, ["k"], ["kt"]).attr("perm", [0, 2, 1])
    b.op(rt.Op.MatMul, ["q", "kt"], ["scores"])
    b.op(rt.Op.Div, ["scores", "scale"], ["scaled"])
    b.op(rt.Op.Trilu, ["scaled"], ["masked"]).attr("upper", 0)
    b.op(rt.Op.Softmax, ["masked"], ["probs"]).attr("axis", -1)
    b.op(rt.Op.MatMul, ["probs", "v"], ["out"])
    b.output("out")
    inst = rt.ModelInstance(b)
    out = inst.run({"q": q, "k": k, "v": v})["out"]
    assert out.shape == (1, 2, 4)
    assert np.max(np.abs(out.reshape(-1) - np.array(g["out"], dtype=np.float32))) <= 1e-5
    assert inst.last_launches == 6 and inst.last_syncs == 0


def test_add_chained_and_broadcast(rt):
    """backend/add.rs:132-232 (with_constant, broadcast_with_constant, broadcast_diff_len_shapes,
    three_inputs_chained) — two Adds in one graph instead of two OpTests."""
    b = rt.GraphBuilder()
    b.input("a", np.float32, [2, 4, 1]).input("b", np.float32, [4, 3])
    b.constant("c", np.array([100.0, 200.0, 300.0], dtype=np.float32))
    b.value("ab", np.float32, [2, 4, 3]).value("y", np.float32, [2, 4, 3])
    b.op(rt.Op.Add, ["a", "b"], ["ab"])
    b.op(rt.Op.Add, ["ab", "c"], ["y"])
    b.output("y")
    a = np.array([10, 20, 30, 40, 50, 60, 70, 80], dtype=np.float32).reshape(2, 4, 1)
    bb = np.array([1.1, 2.1, 3.1, 4.1, 5.1, 6.1, 7.1, 8.1, 9.1, 10.1, 11.1, 12.1], dtype=np.float32).reshape(4, 3)
    y = rt.ModelInstance(b).run({"a": a, "b": bb})["y"]
    want = np.array([111.1, 212.1, 313.1, 124.1, 225.1, 326.1, 137.1, 238.1, 339.1, 150.1, 251.1, 352.1, 151.1, 252.1, 353.1, 164.1,
                     265.1, 366.1, 177.1, 278.1, 379.1, 190.1, 291.1, 392.1], dtype=np.float32)
    assert np.allclose(y.reshape(-1), want, atol=1.2e-7 * 400)
    assert np.array_equal(y, (a + bb) + np.array([100.0, 200.0, 300.0], dtype=np.float32))


def test_softmax_large_and_masked(rt):
    """backend/softmax.rs:259-314: a 4096-wide row against the host formula, and -10000 masking."""
    x = ((np.arange(4096) % 79).astype(np.float32) * np.float32(0.01) - np.float32(3.0)).astype(np.float32)
    e = np.exp(x - x.max())
    want = e / e.sum()
    out = rt.OpTest(rt.Op.Softmax).input([1, 1, 1, 4096], x).attr("axis", -1).output([1, 1, 1, 4096]).run(np.float32)
    assert np.max(np.abs(out - want)) <= 1e-5
    xm = np.array([0.0, 0.5, -10000.0, -10000.0], dtype=np.float32)
    om = rt.OpTest(rt.Op.Softmax).input([1, 4], xm).run(np.float32)
    assert np.max(np.abs(om - np.array([0.37754068, 0.62245935, 0.0, 0.0], dtype=np.float32))) <= 1e-5


def test_matmul_vs_host_triple_loop(rt):
    """backend/matmul.rs:563-590 (batched_2d_vs_reference): [1, n_mid, k] x [k, n] against a host loop."""
    n_mid, k, n = 5, 7, 3
    a = ((np.arange(n_mid * k) % 11) - 5).astype(np.float32) * np.float32(0.25)
    b = ((np.arange(k * n) % 7) - 3).astype(np.float32) * np.float32(0.5)
    want = (a.reshape(n_mid, k).astype(np.float64) @ b.reshape(k, n).astype(np.float64)).astype(np.float32)
    out = rt.OpTest(rt.Op.MatMul).input([1, n_mid, k], a).input([k, n], b).output([1, n_mid, n]).run(np.float32)
    assert np.allclose(out, want.reshape(-1), rtol=1e-5, atol=1e-5)
    o4 = rt.OpTest(rt.Op.MatMul).input([1, 24, 6, 6], np.ones(24 * 36, np.float32)).input([1, 24, 6, 128], np.full(24 * 6 * 128, 13.0, np.float32)) \
        .output([1, 24, 6, 128])
    r4 = o4.run(np.float32)
    assert o4.result_shape == [1, 24, 6, 128] and np.all(r4 == 78.0)
    # f16 (backend/matmul.rs:227 dispatches Float16 to the same cuBLAS call): these values are exact in half precision
    ah, bh = a.astype(np.float16), b.astype(np.float16)
    wh = (ah.reshape(n_mid, k).astype(np.float64) @ bh.reshape(k, n).astype(np.float64)).astype(np.float16)
    outh = rt.OpTest(rt.Op.MatMul).input([1, n_mid, k], ah).input([k, n], bh).output([1, n_mid, n]).run(np.float16)
    assert outh.dtype == np.float16 and np.array_equal(outh, wh.reshape(-1))


def test_unary_basic(rt):
    """backend/{sqrt,sin,cos}.rs `basic`: compared with the host math at the reference's 1e-6 bar."""
    x = np.array([0.0, 0.5, 1.0, 2.0, 5.0, 100.0], dtype=np.float32)
    assert np.allclose(rt.OpTest(rt.Op.Sqrt).input([6], x).run(np.float32), np.sqrt(x), atol=1e-6)
    assert np.allclose(rt.OpTest(rt.Op.Sin).input([6], x).run(np.float32), np.sin(x), atol=1e-6)
    assert np.allclose(rt.OpTest(rt.Op.Cos).input([6], x).run(np.float32), np.cos(x), atol=1e-6)


def test_slice_large_rotate_half_shape(rt):
    """backend/slice.rs:767-788 (cuda_large): [1, 24, 27, 128] -> [..., 64:128], the rotate_half slice."""
    x = np.arange(24 * 27 * 128, dtype=np.float32).reshape(1, 24, 27, 128)
    t = rt.OpTest(rt.Op.Slice).input([1, 24, 27, 128], x).input([1], np.array([64], np.int64)).input([1], np.array([128], np.int64)) \
        .input([1], np.array([3], np.int64)).output([1, 24, 27, 64])
    out = t.run(np.float32)
    assert t.result_shape == [1, 24, 27, 64]
    assert np.array_equal(out, x[..., 64:].reshape(-1))


def test_unsqueeze_and_shape_are_views(rt):
    """backend/unsqueeze.rs:160-240: axes at start / mid / end / negative / multiple, any order."""
    data = np.zeros((3, 4, 5), dtype=np.float32)
    for axes, want in [([0], [1, 3, 4, 5]), ([1], [3, 1, 4, 5]), ([3], [3, 4, 5, 1]), ([-1], [3, 4, 5, 1]), ([0, 4], [1, 3, 4, 5, 1]),
                       ([4, 0], [1, 3, 4, 5, 1]), ([-2], [3, 4, 1, 5])]:
        t = rt.OpTest(rt.Op.Unsqueeze).input([3, 4, 5], data).input([len(axes)], np.array(axes, np.int64)).output(want)
        t.run(np.float32)
        assert t.result_shape == want, (axes, t.result_shape)
        assert t.launches == 0, "Unsqueeze must not copy"
    err = rt.OpTest(rt.Op.Unsqueeze).input([3], np.zeros(3, np.float32)).input([2], np.array([0, 0], np.int64)).output([1, 1, 3]).run_err()
    assert "duplicate" in str(err).lower()


def test_dynamic_shape_chain_needs_no_device_wait(rt):
    """Shape -> Gather -> Unsqueeze -> Concat -> Reshape, the int64 shape arithmetic of exported graphs,
    runs without a single D2H wait (the reference syncs in reshape.rs:102-103, gather.rs:38-42, ...)."""
    b = rt.GraphBuilder()
    b.input("x", np.float32, [0, 0, 8])
    b.constant("i0", np.array(0, np.int64)).constant("i1", np.array(1, np.int64)).constant("ax0", np.array([0], np.int64))
    b.constant("tail", np.array([2, 4], np.int64))
    for n, dt_, d in [("shp", np.int64, [3]), ("d0", np.int64, []), ("d1", np.int64, []), ("d0u", np.int64, [1]), ("d1u", np.int64, [1]),
                      ("tgt", np.int64, [4]), ("y", np.float32, [0, 0, 2, 4])]:
        b.value(n, dt_, d)
    b.op(rt.Op.Shape, ["x"], ["shp"])
    b.op(rt.Op.Gather, ["shp", "i0"], ["d0"])
    b.op(rt.Op.Gather, ["shp", "i1"], ["d1"])
    b.op(rt.Op.Unsqueeze, ["d0", "ax0"], ["d0u"])
    b.op(rt.Op.Unsqueeze, ["d1", "ax0"], ["d1u"])
    b.op(rt.Op.Concat, ["d0u", "d1u", "tail"], ["tgt"]).attr("axis", 0)
    b.op(rt.Op.Reshape, ["x", "tgt"], ["y"])
    b.output("y").output("tgt")
    inst = rt.ModelInstance(b)
    for shape in [(2, 3, 8), (5, 1, 8)]:
        x = np.random.default_rng(0).standard_normal(shape).astype(np.float32)
        out = inst.run({"x": x})
        assert out["y"].shape == shape[:2] + (2, 4) and np.array_equal(out["y"].reshape(-1), x.reshape(-1))
        assert out["tgt"].tolist() == [shape[0], shape[1], 2, 4]
        assert inst.last_syncs == 0


def test_carried_output_stays_on_device(rt):
    """KV-cache style: `present = Concat(past, new)` bound to `past` of the next run, no host round trip."""
    b = rt.GraphBuilder()
    b.input("past", np.float32, [1, 2, 0, 4]).input("new", np.float32, [1, 2, 1, 4])
    b.value("present", np.float32, [1, 2, 0, 4])
    b.op(rt.Op.Concat, ["past", "new"], ["present"]).attr("axis", 2)
    b.output("present")
    inst = rt.ModelInstance(b)
    inst.bind("present", "past")
    hist = []
    for step in range(5):
        new = np.full((1, 2, 1, 4), float(step), dtype=np.float32)
        feeds = {"new": new}
        if step == 0:
            feeds["past"] = np.zeros((1, 2, 0, 4), dtype=np.float32)   # empty past on the first step, as the reference harness feeds it
        hist.append(new)
        out = inst.run(feeds)["present"]
        assert np.array_equal(out, np.concatenate(hist, axis=2))


def test_errors_match_reference_behaviour(rt):
    err = rt.OpTest(rt.Op.Add).input([2, 3], np.zeros(6, np.float32)).input([3, 2], np.zeros(6, np.float32)).output([2, 3]).run_err()
    assert "incompatible" in str(err).lower()
    err = rt.OpTest(rt.Op.Gather).input([3], np.zeros(3, np.float32)).input([1], np.array([3], np.int64)).output([1]).run_err()
    assert "out of bound" in str(err).lower()
    # ScatterND with an index outside the data: reported through the device status word
    # (reference ScatterNdError::KernelFailed { code: 1 }, backend/scatter_nd.rs:198-203)
    err = rt.OpTest(rt.Op.ScatterND).input([4], np.zeros(4, np.float32)).input([1, 1], np.array([[7]], np.int64)) \
        .input([1], np.ones(1, np.float32)).output([4]).run_err()
    assert "kernel failed" in str(err).lower()
    err = rt.OpTest(rt.Op.MatMul).input([2, 3], np.zeros(6, np.float32)).input([2, 3], np.zeros(6, np.float32)).output([2, 3]).run_err()
    assert "IncompatibleDimForMul" in str(err)
    err = rt.OpTest(rt.Op.Softmax).input([2, 3], np.zeros(6, np.float32)).attr("axis", 0).run_err()
    assert "unsupported input" in str(err).lower()


def test_gemm_alpha_beta_bias_and_transposes(rt):
    """ONNX Gemm beyond the reference's two op tests (backend/gemm.rs:262-290): Y = alpha * op(A) * op(B) + beta * C with the
    bias shapes its backend accepts (backend/gemm.rs:219-240: a vector of N entries, a vector of M entries, [M, N] with
    ones), both transposes and non-default alpha / beta, against the oracle's float64 restatement at the MatMul bar."""
    from oracle import run_op
    r = np.random.default_rng(21)
    M, K, N = 5, 7, 12
    for ta in (0, 1):
        for tb in (0, 1):
            a = r.standard_normal((K, M) if ta else (M, K), dtype=np.float32)
            b = r.standard_normal((N, K) if tb else (K, N), dtype=np.float32)
            for cshape in (None, (N,), (M,), (M, N), (1, N), (M, 1), (1,)):
                for alpha, beta in ((1.0, 1.0), (0.5, 2.0)):
                    t = rt.OpTest(rt.Op.Gemm).input(list(a.shape), a).input(list(b.shape), b)
                    ins = [a, b]
                    if cshape is not None:
                        c = r.standard_normal(cshape, dtype=np.float32)
                        t.input(list(cshape), c)
                        ins.append(c)
                    attrs = {"transA": ta, "transB": tb, "alpha": alpha, "beta": beta}
                    for k, v in attrs.items():
                        t.attr(k, v)
                    got = t.output([M, N]).run(np.float32)
                    want = run_op.run("Gemm", ins, attrs)
                    assert t.result_shape == [M, N]
                    assert np.max(np.abs(got.reshape(M, N) - want)) <= 1e-4 * np.max(np.abs(want)), (ta, tb, cshape, alpha, beta)
    # a shape the tensor-core MatMul takes, with a row bias (the classifier head of a CNN in the reference's own use)
    a = r.standard_normal((64, 512), dtype=np.float32)
    b = r.standard_normal((512, 1024), dtype=np.float32) * np.float32(0.05)
    c = r.standard_normal((1024,), dtype=np.float32)
    got = rt.OpTest(rt.Op.Gemm).input([64, 512], a).input([512, 1024], b).input([1024], c).output([64, 1024]).run(np.float32).reshape(64, 1024)
    want = run_op.run("Gemm", [a, b, c], {})
    assert np.max(np.abs(got - want)) <= 1e-4 * np.max(np.abs(want))
    # f16: fp32 arithmetic, one rounding per stage
    ah, bh, ch = a[:8, :64].astype(np.float16), b[:64, :32].astype(np.float16), c[:32].astype(np.float16)
    goth = rt.OpTest(rt.Op.Gemm).input([8, 64], ah).input([64, 32], bh).input([32], ch).output([8, 32]).run(np.float16).reshape(8, 32)
    wanth = run_op.run("Gemm", [ah, bh, ch], {}).astype(np.float64)
    assert np.max(np.abs(goth.astype(np.float64) - wanth)) <= 4e-3 * max(1.0, np.max(np.abs(wanth)))
    # rank-3 operands are rejected, as in backend/gemm.rs:196-204
    err = rt.OpTest(rt.Op.Gemm).input([1, 2, 2], np.ones(4, np.float32)).input([2, 2], np.ones(4, np.float32)).output([2, 2]).run_err()
    assert "rank 2" in str(err)
