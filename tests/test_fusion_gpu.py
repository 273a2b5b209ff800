"""Op chains that run as one launch: RMSNorm, rotary embedding, SwiGLU gate, scale + mask + softmax.

The reference runs every node of these chains through its own backend.  The fused kernels must give what the chain
of single-op kernels gives: bit-identical where the chain has no reduction (rotary, SwiGLU), within the
ReduceMean / Softmax bar (rel 1e-5) where the row sums may associate differently.  The runtime substitutes a fused
kernel only when it recognises the whole chain and the run's tensors fit; otherwise the single ops run.
"""
import os

import numpy as np
import pytest
import torch

from oracle import graph_cpu
from rmlk_b200.graphspec import GraphSpec

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K(cuda):
    from rmlk_b200 import kernels
    return kernels


def test_fused_kernels_equal_the_single_op_chain(K):
    g = torch.Generator(device="cuda").manual_seed(3)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    # RMSNorm
    for rows, cols in [(64, 2048), (3, 7), (1, 4097), (130, 64), (64, 4096), (600, 2048), (600, 4096), (9, 1028)]:
        x, w = r(rows, cols) * 3, r(cols)
        two, eps = torch.tensor(2.0, device="cuda"), torch.tensor(1e-5, device="cuda")
        var = K.reduce_mean(K.pow_(x, two), [-1], True)
        want = K.binary("mul", K.binary("div", x, K.unary("sqrt", K.binary("add", var, eps))), w)
        got = K.rmsnorm(x, w, 1e-5)
        assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max()), (rows, cols)
        ref = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double()
        assert float((got.double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    # residual Add in front of RMSNorm, with the second operand whole or as split-K slabs: the same bits as
    # (split-K sum ->) Add -> the RMSNorm kernel
    # (few rows take wide CTAs with one pack per thread and up to 16 / 8 slab loads at once; many rows the 256-thread form)
    for rows, cols, parts in [(64, 2048, 1), (64, 2048, 9), (3, 7, 1), (3, 7, 4), (2, 4097, 11), (130, 64, 2), (5, 4096, 8), (5, 4096, 11),
                              (64, 2048, 17), (600, 2048, 9), (600, 4096, 3), (64, 1536, 6), (7, 3072, 2)]:
        a, w = r(rows, cols) * 3, r(cols)
        slabs = r(parts, rows, cols)
        b = K.sum_parts(slabs) if parts > 1 else slabs[0]
        if parts > 1:
            ref = torch.zeros(rows, cols, device="cuda")
            for k in range(parts):
                ref = ref + slabs[k]
            assert torch.equal(b, ref)
        want_sum = K.binary("add", a, b)
        want = K.rmsnorm(want_sum, w, 1e-5)
        got_sum, got = K.add_rmsnorm(a, slabs if parts > 1 else b, w, 1e-5, parts=parts)
        assert torch.equal(got_sum, want_sum), (rows, cols, parts)
        assert torch.equal(got, want), (rows, cols, parts)
    # MatMul that leaves its split-K slabs to the caller: their sum is the MatMul's own result
    for (m, k, n) in [(64, 2048, 2048), (64, 8192, 2048), (64, 2048, 8192), (8, 512, 256)]:
        a, b = r(m, k), r(k, n) * 0.05
        c, slabs, parts = K.matmul_parts(a, b)
        want = K.matmul(a, b, workspace=torch.empty(16 << 20, device="cuda"))   # with scratch: the same K split as above
        got = K.sum_parts(slabs) if parts > 1 else c
        assert torch.equal(got, want), (m, k, n, parts)
        # (64, 8192, 2048): 16 tiles on 148 SMs.  The one-tile-per-CTA kernel splits K through the workspace and leaves the
        # slabs (parts > 4); the persistent kernel shares tiles between CTAs and adds the partial tiles itself (parts == 1).
        assert parts >= 1
    # SwiGLU: no reduction, so the same bits as Sigmoid -> Mul -> Mul
    for n in [(64, 8192), (5, 7), (1,), (4099,)]:
        a, b = r(*n) * 4, r(*n)
        want = K.binary("mul", K.binary("mul", a, K.unary("sigmoid", a)), b)
        assert torch.equal(K.swiglu(a, b), want), n
    # rotary embedding: same bits as Mul, Slice x2, Neg, Concat, Mul, Add; x given as a permuted view too
    for (B, H, S, D) in [(4, 8, 1, 64), (2, 3, 5, 16), (1, 1, 7, 2), (3, 4, 2, 128)]:
        xb = r(B, S, H, D)
        cos, sin = r(B, 1, S, D), r(B, 1, S, D)
        for x in (xb.permute(0, 2, 1, 3), xb.permute(0, 2, 1, 3).contiguous()):
            xc = x.contiguous()
            lo = K.slice_(xc, [0], [D // 2], [3], None)
            hi = K.slice_(xc, [D // 2], [D], [3], None)
            rot = K.concat([K.unary("neg", hi), lo], -1)
            want = K.binary("add", K.binary("mul", xc, cos), K.binary("mul", rot, sin))
            assert torch.equal(K.rope(x, cos, sin), want), (B, H, S, D)
    # scale + mask + softmax
    for (B, H, S, T) in [(4, 8, 1, 523), (2, 3, 5, 33), (1, 2, 3, 1030), (2, 2, 2, 2048), (3, 1, 4, 7)]:
        s = r(B, H, S, T) * 5
        mask = torch.where(torch.rand(B, 1, S, T, device="cuda", generator=g) > 0.8, torch.tensor(float(np.finfo(np.float32).min), device="cuda"),
                           torch.tensor(0.0, device="cuda"))
        mask[..., 0] = 0.0
        scale = 0.125
        want = K.softmax(K.binary("add", K.binary("mul", s, torch.tensor(scale, device="cuda")), mask))
        got = K.scale_mask_softmax(s, scale, mask)
        assert float((got - want).abs().max()) <= 1e-6, (B, H, S, T)
        assert float((got.sum(-1) - 1).abs().max()) <= 1e-5


def i64(*v):
    return np.array(v, dtype=np.int64)


def block_graph(hidden, heads, D, exact_names=True):
    """RMSNorm -> projections -> rotary on q -> scores with scale and mask -> softmax; SwiGLU on the side."""
    g = GraphSpec()
    g.input("x", np.float32, [0, 0, hidden])
    g.input("cos", np.float32, [0, 1, 0, D])
    g.input("sin", np.float32, [0, 1, 0, D])
    g.input("mask", np.float32, [0, 1, 0, 0])
    g.input("k", np.float32, [0, heads, 0, D])
    rng = np.random.default_rng(0)
    g.const("w_norm", rng.standard_normal(hidden).astype(np.float32))
    g.const("wq", (rng.standard_normal((hidden, heads * D)) * 0.1).astype(np.float32))
    g.const("wg", (rng.standard_normal((hidden, 3 * hidden)) * 0.1).astype(np.float32))
    g.const("wu", (rng.standard_normal((hidden, 3 * hidden)) * 0.1).astype(np.float32))
    g.const("two", np.array(2.0, np.float32))
    g.const("eps", np.array(1e-5, np.float32))
    g.const("scale", np.array(1.0 / np.sqrt(D), np.float32))
    g.const("shape_q", i64(0, 0, heads, D))
    g.const("z", i64(0)); g.const("h", i64(D // 2)); g.const("d", i64(D)); g.const("ax", i64(3))
    x2 = g.op("Pow", ["x", "two"])
    var = g.op("ReduceMean", [x2], axes=[-1], keepdims=1)
    sd = g.op("Sqrt", [g.op("Add", [var, "eps"])])
    hn = g.op("Mul", [g.op("Div", ["x", sd]), "w_norm"], "normed")
    q = g.op("Transpose", [g.op("Reshape", [g.op("MatMul", [hn, "wq"]), "shape_q"])], perm=[0, 2, 1, 3])
    xc = g.op("Mul", [q, "cos"])
    lo = g.op("Slice", [q, "z", "h", "ax"])
    hi = g.op("Slice", [q, "h", "d", "ax"])
    rot = g.op("Concat", [g.op("Neg", [hi]), lo], axis=-1)
    qr = g.op("Add", [xc, g.op("Mul", [rot, "sin"])], "q_rot")
    sc = g.op("MatMul", [qr, g.op("Transpose", ["k"], perm=[0, 1, 3, 2])])
    pr = g.op("Softmax", [g.op("Add", [g.op("Mul", [sc, "scale"]), "mask"])], "probs", axis=-1)
    ga, up = g.op("MatMul", [hn, "wg"]), g.op("MatMul", [hn, "wu"])
    g.op("Mul", [g.op("Mul", [ga, g.op("Sigmoid", [ga])]), up], "gated")
    for o in ("normed", "q_rot", "probs", "gated"):
        g.output(o)
    return g


@pytest.mark.parametrize("B,S,T", [(3, 1, 37), (2, 5, 5), (1, 4, 20)])
def test_runtime_recognises_the_chains(cuda, B, S, T):
    from rmlk_b200.runtime import ModelInstance
    hidden, heads, D = 64, 4, 16
    spec = block_graph(hidden, heads, D)
    rng = np.random.default_rng(1)
    feeds = {"x": rng.standard_normal((B, S, hidden), dtype=np.float32), "cos": rng.standard_normal((B, 1, S, D), dtype=np.float32),
             "sin": rng.standard_normal((B, 1, S, D), dtype=np.float32), "k": rng.standard_normal((B, heads, T, D), dtype=np.float32),
             "mask": np.where(rng.random((B, 1, S, T)) > 0.7, np.finfo(np.float32).min, 0.0).astype(np.float32)}
    feeds["mask"][..., 0] = 0.0
    want = graph_cpu.run_graph(spec, feeds)

    def run(no_fusion):
        if no_fusion:
            os.environ["RMLK_B200_NO_FUSION"] = "1"
        try:
            inst = ModelInstance(spec.to_runtime())
        finally:
            os.environ.pop("RMLK_B200_NO_FUSION", None)
        for k, v in feeds.items():
            inst.set_input(k, v)
        inst.launch()
        return {o: inst.read(o) for o in spec.outputs}, inst.fused, inst.last_launches

    fused, counts, n_fused = run(False)
    plain, counts0, n_plain = run(True)
    assert counts == (4, 4, 0), counts          # RMSNorm, rotary, softmax and SwiGLU chains, all ran fused
    assert counts0 == (0, 0, 0)
    # launches saved: 5 + 6 + 2 + 2 by the chains, and the fused rotary / SwiGLU kernels read their inputs as views
    # (q permuted, gate / up as column blocks of one merged MatMul) where the single ops first copy them out
    assert n_plain - n_fused >= 5 + 6 + 2 + 2, (n_fused, n_plain)
    for o in spec.outputs:
        scale = np.max(np.abs(want[o]))
        assert np.max(np.abs(fused[o] - want[o])) <= 1e-4 * scale, o
        assert np.max(np.abs(fused[o] - plain[o])) <= 2e-6 * scale, o


def test_chain_falls_back_when_tensors_do_not_fit(cuda):
    """Same node pattern as RMSNorm, but the last Mul broadcasts the result up ([1, cols] * [rows, cols]): the fused
    kernel does not cover that, so the single ops run and the result is still right."""
    from rmlk_b200.runtime import ModelInstance
    g = GraphSpec()
    g.input("x", np.float32, [1, 0])
    g.input("w", np.float32, [0, 0])
    g.const("two", np.array(2.0, np.float32))
    g.const("eps", np.array(1e-5, np.float32))
    var = g.op("ReduceMean", [g.op("Pow", ["x", "two"])], axes=[-1], keepdims=1)
    g.op("Mul", [g.op("Div", ["x", g.op("Sqrt", [g.op("Add", [var, "eps"])])]), "w"], "y")
    g.output("y")
    rng = np.random.default_rng(2)
    feeds = {"x": rng.standard_normal((1, 40), dtype=np.float32), "w": rng.standard_normal((6, 40), dtype=np.float32)}
    inst = ModelInstance(g.to_runtime())
    for k, v in feeds.items():
        inst.set_input(k, v)
    inst.launch()
    got = inst.read("y")
    want = graph_cpu.run_graph(g, feeds)["y"]
    assert inst.fused == (1, 0, 1)
    assert got.shape == want.shape == (6, 40)
    assert np.max(np.abs(got - want)) <= 1e-5 * np.max(np.abs(want))
    # a value of the chain that is also a graph output keeps the chain from being matched at all
    g2 = GraphSpec()
    g2.input("x", np.float32, [0, 0])
    g2.const("w", rng.standard_normal(40).astype(np.float32))
    g2.const("two", np.array(2.0, np.float32))
    g2.const("eps", np.array(1e-5, np.float32))
    var = g2.op("ReduceMean", [g2.op("Pow", ["x", "two"])], "var", axes=[-1], keepdims=1)
    g2.op("Mul", [g2.op("Div", ["x", g2.op("Sqrt", [g2.op("Add", [var, "eps"])])]), "w"], "y")
    g2.output("y")
    g2.output("var")
    inst2 = ModelInstance(g2.to_runtime())
    inst2.set_input("x", feeds["x"])
    inst2.launch()
    assert inst2.fused == (0, 0, 0)
    w2 = graph_cpu.run_graph(g2, {"x": feeds["x"]})
    assert np.max(np.abs(inst2.read("y") - w2["y"])) <= 1e-5 * np.max(np.abs(w2["y"]))
    assert np.max(np.abs(inst2.read("var") - w2["var"])) <= 1e-5 * np.max(np.abs(w2["var"]))


def test_matmuls_sharing_their_left_operand_run_as_one(cuda):
    """q / k / v style projections of one activation against constant weights: one MatMul on the concatenated
    weights, outputs handed out as column blocks.  Same numbers as separate MatMuls; a differently shaped input in
    a later run, an output that leaves the graph and RMLK_B200_NO_MATMUL_MERGE=1 all fall back to single MatMuls."""
    from rmlk_b200.runtime import ModelInstance
    rng = np.random.default_rng(21)
    K_, Ns = 96, (64, 32, 128)
    g = GraphSpec()
    g.input("x", np.float32, [0, 0, K_])
    for i, n in enumerate(Ns):
        g.const(f"w{i}", (rng.standard_normal((K_, n)) * 0.2).astype(np.float32))
    g.const("w_out", (rng.standard_normal((K_, 8)) * 0.2).astype(np.float32))
    g.const("sh", i64(0, 0, 4, -1))
    ys = [g.op("MatMul", ["x", f"w{i}"], f"y{i}") for i in range(3)]
    g.op("MatMul", ["x", "w_out"], "direct")                                     # a graph output: stays a MatMul of its own
    g.op("Relu", [ys[0]], "r0")                                                   # dense consumer of a column block
    g.op("Transpose", [g.op("Reshape", [ys[1], "sh"])], "t1", perm=[0, 2, 1, 3])   # view chain on a column block
    g.op("Neg", ["t1"], "n1")
    g.op("Add", [ys[2], ys[2]], "a2")
    for o in ("direct", "r0", "n1", "a2"):
        g.output(o)

    def run(feeds, merge=True):
        if not merge:
            os.environ["RMLK_B200_NO_MATMUL_MERGE"] = "1"
        try:
            inst = ModelInstance(g.to_runtime())
        finally:
            os.environ.pop("RMLK_B200_NO_MATMUL_MERGE", None)
        outs = []
        for f in feeds:
            inst.set_input("x", f)
            inst.launch()
            outs.append(({o: inst.read(o) for o in g.outputs}, inst.last_launches))
        return outs

    feeds = [rng.standard_normal((2, 5, K_), dtype=np.float32), rng.standard_normal((1, 1, K_), dtype=np.float32),
             rng.standard_normal((3, 64, K_), dtype=np.float32)]
    merged, single = run(feeds), run(feeds, merge=False)
    for f, (got, n_m), (ref, n_s) in zip(feeds, merged, single):
        want = graph_cpu.run_graph(g, {"x": f})
        assert n_m <= n_s + 1, (n_m, n_s)   # three MatMuls became one; dense consumers of a column block copy it out first
        for o in g.outputs:
            assert got[o].shape == want[o].shape, o
            scale = np.max(np.abs(want[o]))
            assert np.max(np.abs(got[o] - want[o])) <= 1e-4 * scale, o
            assert np.max(np.abs(got[o] - ref[o])) <= 1e-5 * scale, o


def residual_graph(hidden, ffn, broadcast_add=False):
    """x -> MatMul -> residual Add -> RMSNorm -> MatMul -> residual Add (reads the first sum again) -> RMSNorm."""
    g = GraphSpec()
    g.input("x", np.float32, [0, hidden])
    g.input("y", np.float32, [0, ffn])
    rng = np.random.default_rng(5)
    g.const("w1", (rng.standard_normal((ffn, hidden)) * 0.05).astype(np.float32))
    g.const("w2", (rng.standard_normal((hidden, hidden)) * 0.05).astype(np.float32))
    g.const("n1", rng.standard_normal(hidden).astype(np.float32))
    g.const("n2", rng.standard_normal(hidden).astype(np.float32))
    g.const("two", np.array(2.0, np.float32))
    g.const("eps", np.array(1e-5, np.float32))
    if broadcast_add:
        g.input("x1", np.float32, [1, hidden])

    def norm(x, w, name):
        var = g.op("ReduceMean", [g.op("Pow", [x, "two"])], axes=[-1], keepdims=1)
        return g.op("Mul", [g.op("Div", [x, g.op("Sqrt", [g.op("Add", [var, "eps"])])]), w], name)

    r1 = g.op("Add", ["x1" if broadcast_add else "x", g.op("MatMul", ["y", "w1"])], "res1")
    h1 = norm(r1, "n1", "h1")
    r2 = g.op("Add", [g.op("MatMul", [h1, "w2"]), r1], "res2")
    norm(r2, "n2", "h2")
    g.output("h2")
    return g


@pytest.mark.parametrize("rows,hidden,ffn", [(64, 2048, 8192), (24, 256, 512), (3, 40, 72)])
def test_residual_add_joins_the_rmsnorm_chain(cuda, rows, hidden, ffn):
    """The Add that feeds an RMSNorm chain (and later readers) runs inside the chain's kernel, and a MatMul read only by
    that Add hands over its split-K slabs unreduced.  Same bits as with the Add and the split-K sum as launches of
    their own."""
    from rmlk_b200.runtime import ModelInstance
    spec = residual_graph(hidden, ffn)
    rng = np.random.default_rng(6)
    feeds = {"x": rng.standard_normal((rows, hidden), dtype=np.float32), "y": rng.standard_normal((rows, ffn), dtype=np.float32)}

    def run(env):
        os.environ.update(env)
        try:
            inst = ModelInstance(spec.to_runtime())
        finally:
            for k in env:
                os.environ.pop(k, None)
        for k, v in feeds.items():
            inst.set_input(k, v)
        inst.launch()
        first = inst.read("h2")
        inst.set_input("x", feeds["x"])
        inst.set_input("y", feeds["y"])
        inst.launch()                       # a second run reuses the slab buffer
        assert np.array_equal(inst.read("h2"), first)
        return first, inst.fused, inst.last_launches

    joined, counts, n_joined = run({})
    apart, counts0, n_apart = run({"RMLK_B200_NO_ADD_NORM": "1"})
    assert counts[0] == 2 and counts[2] == 0 and counts0[0] == 2
    assert np.array_equal(joined, apart)
    # two Adds fewer; on the large shape both MatMuls split K through the workspace: two reductions fewer as well
    assert n_apart - n_joined == (4 if rows == 64 else 2), (n_joined, n_apart)
    want = graph_cpu.run_graph(spec, feeds)["h2"]
    assert np.max(np.abs(joined - want)) <= 1e-4 * np.max(np.abs(want))


def test_residual_add_that_broadcasts_falls_back(cuda):
    """An Add in front of the chain whose operands differ in shape is outside the fused kernel: the members run one
    by one, and the MatMul's slabs are summed on the way."""
    from rmlk_b200.runtime import ModelInstance
    spec = residual_graph(2048, 8192, broadcast_add=True)
    rng = np.random.default_rng(7)
    feeds = {"x": rng.standard_normal((64, 2048), dtype=np.float32), "y": rng.standard_normal((64, 8192), dtype=np.float32),
             "x1": rng.standard_normal((1, 2048), dtype=np.float32)}
    inst = ModelInstance(spec.to_runtime())
    for k, v in feeds.items():
        inst.set_input(k, v)
    inst.launch()
    got = inst.read("h2")
    assert inst.fused[2] == 1 and inst.fused[1] == 1     # first chain fell back, second ran fused
    want = graph_cpu.run_graph(spec, feeds)["h2"]
    assert np.max(np.abs(got - want)) <= 1e-4 * np.max(np.abs(want))


def test_decode_attention_kernel(K):
    """One launch for scores -> scale -> mask -> softmax -> context over a cache with spare room, against the fp64
    result and against the single kernels it stands for."""
    g = torch.Generator(device="cuda").manual_seed(41)
    for (B, KV, G, T, D, cap) in [(64, 8, 4, 523, 64, 700), (3, 2, 4, 37, 16, 37), (2, 3, 2, 130, 32, 200), (2, 2, 1, 65, 128, 70),
                                  (1, 1, 3, 1, 64, 4), (2, 2, 4, 2500, 64, 2500)]:
        q = torch.randn(B, KV, G, D, device="cuda", generator=g)
        kbuf = torch.randn(B, KV, cap, D, device="cuda", generator=g)
        vbuf = torch.randn(B, KV, cap, D, device="cuda", generator=g)
        k, v = kbuf[:, :, :T, :], vbuf[:, :, :T, :]
        mask = torch.where(torch.rand(B, 1, 1, T, device="cuda", generator=g) > 0.8, torch.tensor(float(np.finfo(np.float32).min), device="cuda"),
                           torch.tensor(0.0, device="cuda"))
        mask[..., 0] = 0.0
        scale = 1.0 / np.sqrt(D)
        got = K.gqa_decode_attention(q, k, v, scale, mask)
        s64 = torch.einsum("bkgd,bktd->bkgt", q.double(), k.double()) * scale + mask.double().view(B, 1, 1, T)
        ref = torch.einsum("bkgt,bktd->bkgd", torch.softmax(s64, -1), v.double())
        assert float((got.double() - ref).abs().max()) <= 1e-5 * max(1.0, float(ref.abs().max())), (B, KV, G, T, D)
        # the single kernels: A x B^T per KV head, fused scale + mask + softmax, then P x V
        sc = K.matmul_nt(q.reshape(B * KV, G, D), k.contiguous().reshape(B * KV, T, D)).reshape(B, KV * G, 1, T)
        pr = K.scale_mask_softmax(sc, scale, mask) if T <= 2048 else torch.softmax(sc * scale + mask, -1)
        want = K.matmul(pr.reshape(B * KV, G, T), v.contiguous().reshape(B * KV, T, D)).reshape(B, KV, G, D)
        assert float((got - want).abs().max()) <= 1e-5 * max(1.0, float(want.abs().max())), (B, KV, G, T, D)
        got_split = K.gqa_decode_attention(q, k, v, scale, mask, split=True)   # keys of a problem over several CTAs
        assert float((got_split.double() - ref).abs().max()) <= 1e-5 * max(1.0, float(ref.abs().max())), (B, KV, G, T, D)
        assert torch.equal(got_split, K.gqa_decode_attention(q, k, v, scale, mask, split=True))   # merged in a fixed order
        nomask = K.gqa_decode_attention(q, k, v, scale, None)
        ref2 = torch.einsum("bkgt,bktd->bkgd", torch.softmax(torch.einsum("bkgd,bktd->bkgt", q.double(), k.double()) * scale, -1), v.double())
        assert float((nomask.double() - ref2).abs().max()) <= 1e-5 * max(1.0, float(ref2.abs().max()))


def attention_graph(KV, G, D):
    g = GraphSpec()
    g.input("q", np.float32, [0, KV * G, 0, D])
    g.input("new_k", np.float32, [0, KV, 0, D])
    g.input("new_v", np.float32, [0, KV, 0, D])
    g.input("past_k", np.float32, [0, KV, 0, D])
    g.input("past_v", np.float32, [0, KV, 0, D])
    g.input("mask", np.float32, [0, 1, 0, 0])
    g.const("scale", np.array(1.0 / np.sqrt(D), np.float32))
    g.const("ax2", i64(2))
    g.const("rep", i64(1, 1, G, 1, 1))
    g.const("heads", i64(0, KV * G, -1, D))
    g.op("Concat", ["past_k", "new_k"], "present_k", axis=2)
    g.op("Concat", ["past_v", "new_v"], "present_v", axis=2)

    def heads(c):
        return g.op("Reshape", [g.op("Expand", [g.op("Unsqueeze", [c, "ax2"]), "rep"]), "heads"])

    sc = g.op("MatMul", ["q", g.op("Transpose", [heads("present_k")], perm=[0, 1, 3, 2])])
    pr = g.op("Softmax", [g.op("Add", [g.op("Mul", [sc, "scale"]), "mask"])], axis=-1)
    g.op("MatMul", [pr, heads("present_v")], "ctx")
    for o in ("ctx", "present_k", "present_v"):
        g.output(o)
    return g


def test_rope_tables_equal_mul_concat_cos_sin(K, cuda):
    """rmlk_b200_rope_tables: the same bits as Mul -> Concat -> Cos / Sin, as a kernel and inside the runtime (where the four
    nodes of an exported rotary embedding become one launch; RMLK_B200_NO_FUSION=1 keeps them apart)."""
    from rmlk_b200.runtime import ModelInstance
    g0 = torch.Generator(device="cuda").manual_seed(2)
    pos = torch.randint(0, 4096, (37,), device="cuda", generator=g0).float()
    inv = (1.0 / (10000.0 ** (torch.arange(0, 64, 2, device="cuda").float() / 64.0))).contiguous()
    f = K.binary("mul", pos[:, None].contiguous(), inv)
    emb = torch.cat([f, f], dim=-1).contiguous()
    cos, sin = K.rope_tables(pos, inv)
    assert torch.equal(cos, K.unary("cos", emb)) and torch.equal(sin, K.unary("sin", emb))

    g = GraphSpec()
    g.input("pos", np.int64, [0, 0])
    g.const("inv", inv.cpu().numpy())
    g.const("ax2", np.array([2], np.int64)); g.const("ax1", np.array([1], np.int64))
    pf = g.op("Unsqueeze", [g.op("Cast", ["pos"], to=1), "ax2"])
    fr = g.op("Mul", [pf, "inv"])
    emb_v = g.op("Concat", [fr, fr], axis=-1)
    cos_v, sin_v = g.op("Cos", [emb_v]), g.op("Sin", [emb_v])   # (both tables are made before anything reads them, as exported)
    g.op("Unsqueeze", [cos_v, "ax1"], "cos4")
    g.op("Unsqueeze", [sin_v, "ax1"], "sin4")
    g.output("cos4"); g.output("sin4")

    def drive(env):
        os.environ.update(env)
        try:
            inst = ModelInstance(g.to_runtime())
        finally:
            for key in env:
                os.environ.pop(key, None)
        return inst

    fused, apart = drive({}), drive({"RMLK_B200_NO_FUSION": "1"})
    rng = np.random.default_rng(4)
    for shape in ((3, 1), (2, 17), (64, 1)):
        p = rng.integers(0, 5000, size=shape)
        outs = []
        for m in (fused, apart):
            m.set_input("pos", p)
            m.launch()
            outs.append((m.read("cos4"), m.read("sin4"), m.last_launches))
        assert outs[0][0].shape == (shape[0], 1, shape[1], 64)
        assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1]), shape
        assert outs[1][2] - outs[0][2] >= 2, (outs[0][2], outs[1][2])   # Mul, Concat, Cos, Sin -> one launch
        want = graph_cpu.run_graph(g, {"pos": p})
        assert np.max(np.abs(outs[0][0] - want["cos4"])) <= 2e-6 and np.max(np.abs(outs[0][1] - want["sin4"])) <= 2e-6


def test_mask_chain_is_one_launch(cuda):
    """The causal + padding mask of an exported decoder (ConstantOfShape, Trilu, Equal, Where, Cast, Equal, Where with two
    Unsqueeze views) runs as one launch; RMLK_B200_NO_FUSION=1 runs the seven ops.  Same bits, for decode and prefill shapes,
    with padded positions."""
    from rmlk_b200.runtime import ModelInstance
    g = GraphSpec()
    g.input("attention_mask", np.int64, [0, 0])
    g.input("ids", np.int64, [0, 0])
    g.input("past", np.float32, [0, 2, 0, 4])
    i64 = lambda *v: np.array(v, np.int64)  # noqa: E731
    g.const("i1", np.array(1, np.int64)); g.const("i2", np.array(2, np.int64))
    g.const("ax0", i64(0)); g.const("ax01", i64(0, 1)); g.const("ax12", i64(1, 2))
    g.const("one_f", np.array(1.0, np.float32)); g.const("zero_f", np.array(0.0, np.float32))
    g.const("min_f", np.array(np.finfo(np.float32).min, np.float32))
    s_len = g.op("Gather", [g.op("Shape", ["ids"]), "i1"], axis=0)
    p_len = g.op("Gather", [g.op("Shape", ["past"]), "i2"], axis=0)
    t_len = g.op("Add", [p_len, s_len])
    st = g.op("Concat", [g.op("Unsqueeze", [s_len, "ax0"]), g.op("Unsqueeze", [t_len, "ax0"])], axis=0)
    ones = g.op("ConstantOfShape", [st], value=np.array([1.0], np.float32))
    tri = g.op("Trilu", [ones, g.op("Add", [p_len, "i1"])], upper=1)
    causal = g.op("Where", [g.op("Equal", [tri, "one_f"]), "min_f", "zero_f"])
    causal4 = g.op("Unsqueeze", [causal, "ax01"])
    padded = g.op("Equal", [g.op("Cast", ["attention_mask"], to=1), "zero_f"])
    padded4 = g.op("Unsqueeze", [padded, "ax12"])
    g.op("Where", [padded4, "min_f", causal4], "mask")
    g.output("mask")

    def drive(env):
        os.environ.update(env)
        try:
            inst = ModelInstance(g.to_runtime())
        finally:
            for key in env:
                os.environ.pop(key, None)
        return inst

    fused, apart = drive({}), drive({"RMLK_B200_NO_FUSION": "1"})
    rng = np.random.default_rng(8)
    for B, P, S in ((3, 0, 5), (3, 5, 1), (64, 512, 1), (2, 7, 4)):
        am = (rng.random((B, P + S)) > 0.2).astype(np.int64)
        am[:, -1] = 1
        feeds = {"attention_mask": am, "ids": np.zeros((B, S), np.int64), "past": np.zeros((B, 2, P, 4), np.float32)}
        outs = []
        for m in (fused, apart):
            for key, val in feeds.items():
                m.set_input(key, val)
            m.launch()
            outs.append((m.read("mask"), m.last_launches))
        assert outs[0][0].shape == (B, 1, S, P + S)
        assert np.array_equal(outs[0][0], outs[1][0]), (B, P, S)
        assert outs[1][1] - outs[0][1] == 6, (outs[0][1], outs[1][1])
        want = graph_cpu.run_graph(g, feeds)["mask"]
        assert np.array_equal(outs[0][0], want)


def test_results_of_initializer_only_nodes_are_kept(cuda):
    """Range -> Cast -> Div -> Pow -> Div over constants (the inverse frequencies of a rotary embedding) runs in the first
    run only; later runs hand out the kept result and launch five kernels fewer.  A Transpose of an initializer stays a view
    (never launched, never copied).  RMLK_B200_NO_FOLD=1 recomputes everything; same bits either way."""
    from rmlk_b200.runtime import ModelInstance
    D = 64
    g = GraphSpec()
    g.input("pos", np.float32, [0, 1])
    g.input("x", np.float32, [0, D // 2])
    g.const("i0", np.array(0, np.int64)); g.const("hd", np.array(D, np.int64)); g.const("i2", np.array(2, np.int64))
    g.const("hd_f", np.array(float(D), np.float32)); g.const("theta", np.array(10000.0, np.float32)); g.const("one_f", np.array(1.0, np.float32))
    g.const("w", np.arange(D // 2 * 8, dtype=np.float32).reshape(8, D // 2) / 7.0)
    r = g.op("Range", ["i0", "hd", "i2"])
    inv = g.op("Div", ["one_f", g.op("Pow", ["theta", g.op("Div", [g.op("Cast", [r], to=1), "hd_f"])])])
    g.op("Mul", ["pos", inv], "freqs")
    g.op("MatMul", ["x", g.op("Transpose", ["w"], perm=[1, 0])], "xw")
    g.output("freqs")
    g.output("xw")

    def drive(env):
        os.environ.update(env)
        try:
            inst = ModelInstance(g.to_runtime())
        finally:
            for key in env:
                os.environ.pop(key, None)
        return inst

    kept, plain = drive({}), drive({"RMLK_B200_NO_FOLD": "1"})
    rng = np.random.default_rng(9)
    counts = {id(kept): [], id(plain): []}
    for step in range(3):
        feeds = {"pos": rng.standard_normal((5 + step, 1), dtype=np.float32), "x": rng.standard_normal((5 + step, D // 2), dtype=np.float32)}
        outs = []
        for m in (kept, plain):
            for key, val in feeds.items():
                m.set_input(key, val)
            m.launch()
            outs.append((m.read("freqs"), m.read("xw")))
            counts[id(m)].append(m.last_launches)
        assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1]), step
        want = graph_cpu.run_graph(g, feeds)
        assert np.max(np.abs(outs[0][0] - want["freqs"])) <= 1e-5 * np.max(np.abs(want["freqs"]))
        assert np.max(np.abs(outs[0][1] - want["xw"])) <= 1e-4 * np.max(np.abs(want["xw"]))
    a, b = counts[id(kept)], counts[id(plain)]
    assert b[0] == b[1] == b[2] and a[0] >= b[0] and a[1] == a[2] == b[1] - 5, (a, b)


def test_unsummed_projection_is_summed_when_something_else_reads_it(cuda):
    """A decode-sized merged q|k|v product leaves its split-K slabs unsummed for the collected rotary job, which adds them
    up as it reads.  Here the key and value blocks of the same product are also read by ordinary ops (a Mul and a Neg)
    while that job is still collected: the job goes out first, then the slabs are summed for the other readers.  Same bits
    as with collecting switched off, on a second run too."""
    from rmlk_b200.runtime import ModelInstance
    B, H, KV, D, hidden = 64, 32, 8, 64, 2048
    g = GraphSpec()
    g.input("x", np.float32, [B, 0, hidden])
    g.input("cos", np.float32, [B, 1, 0, D])
    g.input("sin", np.float32, [B, 1, 0, D])
    rng = np.random.default_rng(51)
    g.const("wq", (rng.standard_normal((hidden, H * D)) * 0.03).astype(np.float32))
    g.const("wk", (rng.standard_normal((hidden, KV * D)) * 0.03).astype(np.float32))
    g.const("wv", (rng.standard_normal((hidden, KV * D)) * 0.03).astype(np.float32))
    i64 = lambda *v: np.array(v, np.int64)  # noqa: E731
    g.const("shape_q", i64(0, 0, H, D)); g.const("shape_kv", i64(0, 0, KV, D))
    g.const("z", i64(0)); g.const("h", i64(D // 2)); g.const("d", i64(D)); g.const("ax", i64(3))
    g.const("two", np.array(2.0, np.float32))
    q4 = g.op("Transpose", [g.op("Reshape", [g.op("MatMul", ["x", "wq"]), "shape_q"])], perm=[0, 2, 1, 3])
    k = g.op("MatMul", ["x", "wk"])
    v = g.op("MatMul", ["x", "wv"])
    lo = g.op("Slice", [q4, "z", "h", "ax"])
    hi = g.op("Slice", [q4, "h", "d", "ax"])
    rot = g.op("Concat", [g.op("Neg", [hi]), lo], axis=-1)
    g.op("Add", [g.op("Mul", [q4, "cos"]), g.op("Mul", [rot, "sin"])], "qr")
    g.op("Mul", [k, "two"], "k2")
    g.op("Neg", [v], "vn")
    for o in ("qr", "k2", "vn"):
        g.output(o)

    def drive(env):
        os.environ.update(env)
        try:
            inst = ModelInstance(g.to_runtime())
        finally:
            for key in env:
                os.environ.pop(key, None)
        return inst

    collected, plain = drive({}), drive({"RMLK_B200_NO_BATCH": "1"})
    for step in range(2):
        feeds = {"x": rng.standard_normal((B, 1, hidden), dtype=np.float32), "cos": rng.standard_normal((B, 1, 1, D), dtype=np.float32),
                 "sin": rng.standard_normal((B, 1, 1, D), dtype=np.float32)}
        outs = []
        for m in (collected, plain):
            for key, val in feeds.items():
                m.set_input(key, val)
            m.launch()
            outs.append({o: m.read(o) for o in ("qr", "k2", "vn")})
        for o in ("qr", "k2", "vn"):
            assert np.array_equal(outs[0][o], outs[1][o]), (step, o)
        want = graph_cpu.run_graph(g, feeds)
        for o in ("qr", "k2", "vn"):
            assert np.max(np.abs(outs[0][o] - want[o])) <= 1e-4 * np.max(np.abs(want[o])), (step, o)


@pytest.mark.parametrize("D", [64, 12, 128])
def test_rope_copy_batch_equals_the_single_launches(K, D):
    """rmlk_b200_rope_copy_batch: rotated queries (dense), rotated keys and new values placed into cache slots, as one
    launch - bit for bit what rmlk_b200_rope / rope_to / strided_copy_to give one by one; also with the source left as
    split-K slabs (summed in slab order, as rmlk_b200_sum_parts would).  Head sizes that are multiples of 8 take the
    16-byte form of the kernel, 12 the element-wise one."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(5)
    B, H, KV, T0, cap = 3, 8, 2, 37, 64
    qkv = torch.randn(B, (H + 2 * KV) * D, device="cuda", generator=g)
    q = qkv[:, : H * D].view(B, 1, H, D).permute(0, 2, 1, 3)                   # [B, H, 1, D] views of the merged product
    k = qkv[:, H * D: (H + KV) * D].view(B, 1, KV, D).permute(0, 2, 1, 3)
    v = qkv[:, (H + KV) * D:].view(B, 1, KV, D).permute(0, 2, 1, 3)
    cos = torch.randn(B, 1, 1, D, device="cuda", generator=g)
    sin = torch.randn(B, 1, 1, D, device="cuda", generator=g)
    kc1, vc1 = torch.zeros(B, KV, cap, D, device="cuda"), torch.zeros(B, KV, cap, D, device="cuda")
    kc2, vc2 = torch.zeros_like(kc1), torch.zeros_like(vc1)
    want_q = K.rope(q, cos, sin)
    K.rope(k, cos, sin, out=kc1[:, :, T0: T0 + 1])
    K.strided_copy_to(v, vc1[:, :, T0: T0 + 1])
    got_q = torch.empty(B, H, 1, D, device="cuda")
    K.rope_copy_batch([("rope", q, cos, sin, got_q), ("rope", k, cos, sin, kc2[:, :, T0: T0 + 1]), ("copy", v, vc2[:, :, T0: T0 + 1])])
    assert torch.equal(got_q, want_q) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    # the same with the product still in 5 split-K slabs
    parts = 5
    slabs = torch.randn(parts, B, (H + 2 * KV) * D, device="cuda", generator=g)
    total = torch.zeros(B, (H + 2 * KV) * D, device="cuda")
    for p in range(parts):
        total += slabs[p]
    tq = total[:, : H * D].view(B, 1, H, D).permute(0, 2, 1, 3)
    tv = total[:, (H + KV) * D:].view(B, 1, KV, D).permute(0, 2, 1, 3)
    sq = slabs[:, :, : H * D].view(parts, B, 1, H, D).permute(0, 1, 3, 2, 4)
    sv = slabs[:, :, (H + KV) * D:].view(parts, B, 1, KV, D).permute(0, 1, 3, 2, 4)
    want_q = K.rope(tq, cos, sin)
    vc3, vc4 = torch.zeros_like(vc1), torch.zeros_like(vc1)
    K.strided_copy_to(tv, vc3[:, :, 5:6])
    got_q = torch.empty(B, H, 1, D, device="cuda")
    arr = [("rope", _slab_source(sq), cos, sin, got_q), ("copy", _slab_source(sv), vc4[:, :, 5:6])]
    K.rope_copy_batch(arr)
    assert torch.equal(got_q, want_q) and torch.equal(vc3, vc4)
    with pytest.raises(Exception):
        K.rope_copy_batch([("copy", v, vc2[:, :, 0:1])] * 5)   # more than RMLK_BATCH_MAX_JOBS


class _slab_source(tuple):
    """(view of slab 0, parts) with the slab stride taken from the slabs tensor: what rope_copy_batch reads as a sum."""
    def __new__(cls, slabs):
        return super().__new__(cls, (slabs, slabs.shape[0]))


@pytest.mark.parametrize("KV,G,D", [(2, 4, 64), (3, 2, 16), (2, 1, 128), (2, 8, 32), (1, 4, 20)])
def test_runtime_runs_decode_attention_as_one_launch(cuda, KV, G, D):
    """The five attention nodes of a decode step run as one kernel over the carried caches (RMLK_B200_ATTENTION=0 keeps the
    single kernels); a multi-token step, more than four query heads per KV head or an unsupported head size run the single
    kernels anyway.  Same numbers either way."""
    from rmlk_b200.runtime import ModelInstance
    spec = attention_graph(KV, G, D)
    B = 3

    def drive(env):
        os.environ.update(env)
        try:
            inst = ModelInstance(spec.to_runtime())
            inst.bind("present_k", "past_k")
            inst.bind("present_v", "past_v")
        finally:
            for k in env:
                os.environ.pop(k, None)
        return inst

    one, apart = drive({}), drive({"RMLK_B200_ATTENTION": "0"})
    r = np.random.default_rng(43)
    T = 0
    cache_k = np.zeros((B, KV, 0, D), np.float32)
    cache_v = np.zeros((B, KV, 0, D), np.float32)
    for step in range(70):
        S = 6 if step == 0 else 1
        T += S
        feeds = {"q": r.standard_normal((B, KV * G, S, D), dtype=np.float32), "new_k": r.standard_normal((B, KV, S, D), dtype=np.float32),
                 "new_v": r.standard_normal((B, KV, S, D), dtype=np.float32),
                 "mask": np.where(r.random((B, 1, S, T)) > 0.8, np.finfo(np.float32).min, 0.0).astype(np.float32)}
        feeds["mask"][..., 0] = 0.0
        for m in (one, apart):
            for k, v in feeds.items():
                m.set_input(k, v)
            if step == 0:
                m.set_input("past_k", cache_k)
                m.set_input("past_v", cache_v)
            m.launch()
        cache_k = np.concatenate([cache_k, feeds["new_k"]], axis=2)
        cache_v = np.concatenate([cache_v, feeds["new_v"]], axis=2)
        a, b = one.read("ctx"), apart.read("ctx")
        assert np.max(np.abs(a - b)) <= 1e-5 * max(1.0, np.max(np.abs(b))), step
        if step in (0, 1, 33, 69):
            s64 = np.einsum("bhsd,bhtd->bhst", feeds["q"].astype(np.float64), np.repeat(cache_k, G, axis=1).astype(np.float64)) / np.sqrt(D) + feeds["mask"]
            e = np.exp(s64 - s64.max(-1, keepdims=True))
            want = np.einsum("bhst,bhtd->bhsd", e / e.sum(-1, keepdims=True), np.repeat(cache_v, G, axis=1).astype(np.float64))
            assert np.max(np.abs(a - want)) <= 1e-4 * max(1.0, np.max(np.abs(want))), step
            assert np.array_equal(one.read("present_k"), cache_k)
    fits = G <= 4 and D in (16, 32, 64, 128)
    # decode steps: 2 appends + (1 | 3) attention launches
    # (the single kernels may take a launch more for a split-K sum, depending on the shape)
    saved = apart.last_launches - one.last_launches
    assert (saved >= 2) if fits else (saved == 0), (one.last_launches, apart.last_launches)


def test_one_launch_attention_when_the_batch_changes_between_runs(cuda):
    """The split-keys attention kernel keeps arrival counters at the head of its workspace and partial sums behind them;
    where the partial sums start depends on the number of problems.  An instance that runs 64 requests, then 8, then 64
    again re-uses the workspace with a different layout each time: results must still equal the single kernels' and the
    float64 definition (stale partial sums where counters are expected would leave the output unwritten)."""
    from rmlk_b200.runtime import ModelInstance
    KV, G, D, T0 = 2, 4, 64, 300   # 301+ keys: three splits of 128 keys per problem
    spec = attention_graph(KV, G, D)
    os.environ["RMLK_B200_ATTENTION"] = "split"
    try:
        one = ModelInstance(spec.to_runtime())
    finally:
        os.environ.pop("RMLK_B200_ATTENTION", None)
    os.environ["RMLK_B200_ATTENTION"] = "0"
    try:
        apart = ModelInstance(spec.to_runtime())
    finally:
        os.environ.pop("RMLK_B200_ATTENTION", None)
    for m in (one, apart):
        m.bind("present_k", "past_k")
        m.bind("present_v", "past_v")
    r = np.random.default_rng(77)
    for B in (64, 8, 64, 2, 64):
        cache_k = r.standard_normal((B, KV, T0, D), dtype=np.float32)
        cache_v = r.standard_normal((B, KV, T0, D), dtype=np.float32)
        for step in range(2):
            T = cache_k.shape[2] + 1
            feeds = {"q": r.standard_normal((B, KV * G, 1, D), dtype=np.float32), "new_k": r.standard_normal((B, KV, 1, D), dtype=np.float32),
                     "new_v": r.standard_normal((B, KV, 1, D), dtype=np.float32),
                     "mask": np.where(r.random((B, 1, 1, T)) > 0.8, np.finfo(np.float32).min, 0.0).astype(np.float32)}
            feeds["mask"][..., 0] = 0.0
            for m in (one, apart):
                for k, v in feeds.items():
                    m.set_input(k, v)
                if step == 0:
                    m.set_input("past_k", cache_k)
                    m.set_input("past_v", cache_v)
                m.launch()
            cache_k = np.concatenate([cache_k, feeds["new_k"]], axis=2)
            cache_v = np.concatenate([cache_v, feeds["new_v"]], axis=2)
            a, b = one.read("ctx"), apart.read("ctx")
            assert np.max(np.abs(a - b)) <= 1e-5 * max(1.0, np.max(np.abs(b))), (B, step)
            s64 = np.einsum("bhsd,bhtd->bhst", feeds["q"].astype(np.float64), np.repeat(cache_k, G, axis=1).astype(np.float64)) / np.sqrt(D) + feeds["mask"]
            e = np.exp(s64 - s64.max(-1, keepdims=True))
            want = np.einsum("bhst,bhtd->bhsd", e / e.sum(-1, keepdims=True), np.repeat(cache_v, G, axis=1).astype(np.float64))
            assert np.max(np.abs(a - want)) <= 1e-4 * max(1.0, np.max(np.abs(want))), (B, step)
        assert apart.last_launches - one.last_launches == 2, "the one-launch path ran"
