"""Per-op throughput sweep: achieved HBM GB/s (or TFLOP/s) of every kernel launcher on the shapes of the
indexing / layout sweep, the MatMul sweep and the Llama-3.2-1B-shaped decode step.

    python -m rmlk_b200.opbench [--json out.json] [--only substring]

Each case is launched through the C ABI (rmlk_b200.kernels), 20 launches captured into a CUDA graph and the
graph replayed, so the figure is device time per launch without host launch overhead.  Inputs rotate over a
ring of buffers larger than L2 (126 MB) so that reads come from HBM.  "bytes" is the op's algorithmic traffic:
actual operand bytes read once plus output bytes written once.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import kernels as K

L2_BYTES = 126 << 20


def peak_gbs():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def time_graph(fn_of_i, n=20, replays=3):
    """fn_of_i(i) enqueues launch i on the current stream."""
    for i in range(3):
        fn_of_i(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for i in range(n):
                fn_of_i(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (n * replays)


def ring(make, nbytes_each):
    n = max(2, min(8, L2_BYTES * 2 // max(nbytes_each, 1) + 1))
    return [make() for _ in range(n)]


def nbytes(*ts):
    return sum(t.numel() * t.element_size() for t in ts)


def cases():
    f32, i64 = torch.float32, torch.int64
    dev = "cuda"
    rnd = lambda *s: torch.randn(*s, device=dev)  # noqa: E731
    B, T = 64, 520

    def binary(name, sa, sb, op="add"):
        def build():
            a = ring(lambda: rnd(*sa), 4 * int(torch.tensor(sa).prod()))
            b = ring(lambda: rnd(*sb) if sb else torch.randn((), device=dev), 4 * int(torch.tensor(sb).prod()) if sb else 4)
            out = K.binary(op, a[0], b[0])
            return (lambda i: K.binary(op, a[i % len(a)], b[i % len(b)], out=out)), nbytes(a[0], b[0], out), 0
        return name, build

    def unary(name, shape, op):
        def build():
            a = ring(lambda: rnd(*shape), 4 * int(torch.tensor(shape).prod()))
            out = torch.empty_like(a[0])
            return (lambda i: K.unary(op, a[i % len(a)], out=out)), nbytes(a[0], out), 0
        return name, build

    def generic(name, make_inputs, call, extra_bytes=0, flops=0):
        def build():
            r = ring(make_inputs, nbytes(*[t for t in make_inputs() if torch.is_tensor(t)]))
            out = call(*r[0])
            b = nbytes(*[t for t in r[0] if torch.is_tensor(t)]) + nbytes(out) + extra_bytes
            return (lambda i: call(*r[i % len(r)])), b, flops
        return name, build

    def matmul(name, m, k, n):
        def build():
            w = ring(lambda: rnd(k, n) * 0.02, 4 * k * n)
            x = rnd(m, k)
            out = torch.empty(m, n, device=dev)
            wsb = K.matmul_workspace_bytes(1, m, n, k)
            ws = torch.empty(max(wsb // 4, 1), device=dev) if wsb else None
            return (lambda i: K.matmul(x, w[i % len(w)], out=out, workspace=ws)), 4 * (m * k + k * n + m * n), 2 * m * n * k
        return name, build

    def bmm(name, batch, m, k, n):
        def build():
            b = ring(lambda: rnd(batch, k, n), 4 * batch * k * n)
            a = rnd(batch, m, k)
            out = torch.empty(batch, m, n, device=dev)
            return (lambda i: K.matmul(a, b[i % len(b)], out=out)), 4 * batch * (m * k + k * n + m * n), 2 * batch * m * n * k
        return name, build

    idx_rows = 32768
    attn_ws = torch.zeros(1 << 20, device=dev)   # 4 MB, zero-filled once: arrival counters + partial results
    cs = [
        binary("add f32 same-shape 64M", (1 << 26,), (1 << 26,)),
        binary("mul f32 [32768,8192]*[32768,8192] (SwiGLU)", (32768, 8192), (32768, 8192), "mul"),
        binary("add f32 [32768,2048]+[2048] (bias row)", (32768, 2048), (2048,)),
        binary("div f32 [32768,2048]/[32768,1] (RMSNorm)", (32768, 2048), (32768, 1), "div"),
        binary("mul f32 [64,32,1,520]*scalar (decode scores)", (B, 32, 1, T), ()),
        binary("add f32 [64,32,128,640]+[64,1,128,640] (mask)", (B, 32, 128, 640), (B, 1, 128, 640)),
        binary("mul f32 [64,32,512,64]*[64,1,512,64] (RoPE)", (B, 32, 512, 64), (B, 1, 512, 64), "mul"),
        binary("greater f32->bool 64M", (1 << 26,), (1 << 26,), "greater"),
        unary("sigmoid f32 [32768,8192]", (32768, 8192), "sigmoid"),
        unary("neg f32 64M", (1 << 26,), "neg"),
        unary("sin f32 64M", (1 << 26,), "sin"),
        generic("cast i64->f32 64M", lambda: (torch.randint(0, 1000, (1 << 26,), device=dev),), lambda x: K.cast(x, f32)),
        generic("pow f32^2.0 [32768,2048]", lambda: (rnd(32768, 2048), torch.tensor(2.0, device=dev)), lambda x, e: K.pow_(x, e)),
        generic("where f32 [64,32,128,640] cond [64,1,128,640] y scalar",
                lambda: (torch.rand(B, 1, 128, 640, device=dev) > 0.5, rnd(B, 32, 128, 640), torch.tensor(0.0, device=dev)),
                lambda c, x, y: K.where(c, x, y)),
        generic("reduce_mean f32 [32768,2048] last axis", lambda: (rnd(32768, 2048),), lambda x: K.reduce_mean(x, [-1], True)),
        generic("reduce_mean f32 [64,2048] last axis (decode)", lambda: (rnd(64, 2048),), lambda x: K.reduce_mean(x, [-1], True)),
        generic("softmax f32 [64,32,128,640]", lambda: (rnd(B, 32, 128, 640),), lambda x: K.softmax(x)),
        generic("softmax f32 [2048,520] (decode)", lambda: (rnd(2048, T),), lambda x: K.softmax(x)),
        generic("softmax f32 [16384,4096]", lambda: (rnd(16384, 4096),), lambda x: K.softmax(x)),
        generic("gather f32 [128256,2048] 32768 rows i64", lambda: (rnd(128256, 2048), torch.randint(0, 128256, (idx_rows,), device=dev)),
                lambda d, ix: K.gather(d, ix, 0), extra_bytes=-4 * 128256 * 2048 + 4 * idx_rows * 2048),
        generic("concat f32 KV append [64,8,519,64]+[64,8,1,64] axis 2", lambda: (rnd(B, 8, T - 1, 64), rnd(B, 8, 1, 64)),
                lambda a, b: K.concat([a, b], 2)),
        generic("concat f32 [64,32,512,32]x2 axis -1 (rotate_half)", lambda: (rnd(B, 32, 512, 32), rnd(B, 32, 512, 32)),
                lambda a, b: K.concat([a, b], -1)),
        generic("slice f32 [64,32,512,64] -> [...,32:64]", lambda: (rnd(B, 32, 512, 64),), lambda x: K.slice_(x, [32], [64], [3], None),
                extra_bytes=-4 * B * 32 * 512 * 32),
        generic("slice i64 [2^27] step 2", lambda: (torch.randint(0, 9, (1 << 27,), device=dev),), lambda x: K.slice_(x, [0], [1 << 27], [0], [2]),
                extra_bytes=-8 * (1 << 26)),
        generic("transpose f32 [64,512,32,64] perm 0,2,1,3", lambda: (rnd(B, 512, 32, 64),), lambda x: K.transpose(x, [0, 2, 1, 3])),
        generic("transpose f32 [64,32,520,64] perm 0,1,3,2 (K^T)", lambda: (rnd(B, 32, T, 64),), lambda x: K.transpose(x, [0, 1, 3, 2])),
        generic("transpose f32 [8192,8192] perm 1,0", lambda: (rnd(8192, 8192),), lambda x: K.transpose(x, [1, 0])),
        generic("transpose i64 [64,64,64,64] perm 3,2,1,0", lambda: (torch.randint(0, 9, (64, 64, 64, 64), device=dev),),
                lambda x: K.transpose(x, [3, 2, 1, 0])),
        generic("expand f32 [64,8,1,520,64] -> [64,8,4,520,64] (GQA)", lambda: (rnd(B, 8, 1, T, 64),), lambda x: K.expand(x, [1, 1, 4, 1, 1])),
        generic("trilu f32 [16,4096,4096] upper k=1", lambda: (rnd(16, 4096, 4096),), lambda x: K.trilu(x, 1, True),
                extra_bytes=-4 * 16 * 4096 * 4096 // 2),
        generic("scatter_nd f32 data [65536,1024] 32768 rows", lambda: (rnd(65536, 1024), torch.randperm(65536, device=dev)[:32768].reshape(-1, 1),
                                                                        rnd(32768, 1024)), lambda d, ix, u: K.scatter_nd(d, ix, u),
                extra_bytes=-8 * 32768 + 8 * 32768 + 4 * 32768 * 1024),
        generic("range i64 64M", lambda: (), lambda: K.range_(0, 1, 1 << 26, i64)),
        matmul("matmul GEMV M=1 K=2048 N=8192", 1, 2048, 8192),
        matmul("matmul M=8 K=2048 N=8192", 8, 2048, 8192),
        matmul("matmul M=64 K=2048 N=8192", 64, 2048, 8192),
        matmul("matmul M=64 K=2048 N=16384 (gate|up merged)", 64, 2048, 16384),
        matmul("matmul M=64 K=2048 N=3072 (q|k|v merged)", 64, 2048, 3072),
        matmul("matmul M=64 K=8192 N=2048", 64, 8192, 2048),
        matmul("matmul M=64 K=2048 N=2048", 64, 2048, 2048),
        matmul("matmul M=64 K=2048 N=128256 (lm_head)", 64, 2048, 128256),
        matmul("matmul prefill M=4096 K=2048 N=8192", 4096, 2048, 8192),
        bmm("matmul batched 2048x[1,64]x[64,520] (decode scores)", 2048, 1, 64, T),
        bmm("matmul batched 2048x[1,520]x[520,64] (decode context)", 2048, 1, T, 64),
        bmm("matmul batched 256x[512,64]x[64,512] (prefill scores)", 256, 512, 64, 512),
        # grouped-query attention read from the KV cache in place: 4 query heads per KV head are 4 rows of one problem
        generic("matmul_nt 512x[4,64]x[523,64]^T (decode scores, cache in place)", lambda: (rnd(512, 4, 64), rnd(512, 523, 64)),
                lambda q, k: K.matmul_nt(q, k), flops=2 * 512 * 4 * 64 * 523),
        generic("matmul 512x[4,523]x[523,64] (decode context, cache in place)", lambda: (rnd(512, 4, 523), rnd(512, 523, 64)),
                lambda p, v: K.matmul(p, v), flops=2 * 512 * 4 * 64 * 523),
        # the same attention as one launch (scores, scale, mask-free softmax, context): one CTA per problem, and keys split over CTAs
        generic("gqa_decode_attention 512x[4,64] over [523,64] K and V, one CTA per problem",
                lambda: (rnd(64, 8, 4, 64), rnd(64, 8, 523, 64), rnd(64, 8, 523, 64)),
                lambda q, k, v: K.gqa_decode_attention(q, k, v, 0.125), flops=4 * 512 * 4 * 64 * 523),
        generic("gqa_decode_attention 512x[4,64] over [523,64] K and V, keys split over CTAs",
                lambda: (rnd(64, 8, 4, 64), rnd(64, 8, 523, 64), rnd(64, 8, 523, 64)),
                lambda q, k, v: K.gqa_decode_attention(q, k, v, 0.125, workspace=attn_ws), flops=4 * 512 * 4 * 64 * 523),
    ]
    return cs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    peak, kind = peak_gbs()
    rows = []
    for name, build in cases():
        if args.only and args.only not in name:
            continue
        fn, b, flops = build()
        ms = time_graph(fn)
        gbs = b / ms / 1e6
        row = {"op": name, "us": ms * 1e3, "bytes": b, "GB/s": gbs, "frac_of_%s_peak" % kind: gbs / peak}
        if flops:
            row["TFLOP/s"] = flops / ms / 1e9
        rows.append(row)
        print(f"{name:62s} {ms * 1e3:9.1f} us {gbs:8.0f} GB/s {gbs / peak * 100:5.1f}% of {kind} {peak:.0f}" +
              (f"  {row['TFLOP/s']:.1f} TFLOP/s" if flops else ""), flush=True)
        del fn
        torch.cuda.empty_cache()
    if args.json:
        json.dump({"peak_gbs": peak, "peak_kind": kind, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
