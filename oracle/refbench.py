"""The reference's own implementations timed on this machine, beside this library's.  TEST INFRASTRUCTURE ONLY.

    python -m oracle.refbench [--json out.json] [--only kernels|cpu|cublas|cudnn]

Four groups, all on the same operands as the library's launchers (rmlk_b200.kernels):

  kernels  the reference's hand-written kernels (oracle/_ref/ptx, the reference's .cu files compiled unchanged)
           launched on this GPU with the reference's contract (grid ceil(n/128) x 128 threads), the symbol-compatible
           kernels of rmlk_b200/tier1 under the same contract, and the library launcher.
  cpu      the same reference kernels compiled for the host (oracle/_ref/libref_cpu.so) on all host threads.
  cublas   the reference's MatMul is cublasGemmStridedBatchedEx with CUDA_R_32F operands and CUBLAS_COMPUTE_32F
           (cuda/src/kernels/gemm.rs:206-231, cuda/src/params.rs:10-22): timed here as torch.matmul with TF32 off, which
           issues cuBLAS fp32 GEMMs in that compute mode; also the numerical distance between the two results, and
           the TF32 tensor-core peak of this GPU (torch.matmul with TF32 allowed, 8192^3), the denominator for the
           3xTF32 prefill GEMM (three MMAs per algorithmic product: peak / 3).
  cudnn    cudnnSoftmaxForward(CUDNN_SOFTMAX_FAST, CUDNN_SOFTMAX_MODE_CHANNEL) on [rows, cols, 1, 1]
           (cuda/src/kernels/softmax.rs:26-34, backend/softmax.rs:90-99) and cudnnActivationForward sigmoid / relu with
           CUDNN_NOT_PROPAGATE_NAN (cuda/src/kernels/activation.rs:28-36, sigmoid.rs:25-27, relu.rs:25-27), called
           through ctypes with the reference's enums: time per call and the distance to this library's results.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import time

import numpy as np
import torch

from oracle import ref_calls as RC
from oracle import ref_cpu, ref_gpu
from rmlk_b200 import kernels as K
from rmlk_b200.opbench import ring, time_graph

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
T1 = os.path.join(ROOT, "rmlk_b200", "tier1", "ptx")


def kernel_cases():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((16384, 2048), dtype=np.float32)
    col = x[:, :1].copy()
    x4 = x.reshape(64, 128, 64, 64)
    e_in = x[:8192].reshape(64, 8, 1, 512, 64)[:, :, :, :256].copy()
    return [
        ("add f32 [16384,2048] same shape", lambda: RC.arith("add", x, x), lambda a: K.binary("add", a[0], a[0]), [x], 3 * x.nbytes),
        ("add f32 [16384,2048] + [2048]", lambda: RC.arith("add", x, x[0]), lambda a: K.binary("add", a[0], a[1]), [x, x[0].copy()], 2 * x.nbytes),
        ("div f32 [16384,2048] / [16384,1]", lambda: RC.arith("div", x, col), lambda a: K.binary("div", a[0], a[1]), [x, col], 2 * x.nbytes),
        ("sin f32 32M", lambda: RC.unary("sin", x), lambda a: K.unary("sin", a[0]), [x], 2 * x.nbytes),
        ("cast f32->i64 32M", lambda: RC.cast(x, np.int64), lambda a: K.cast(a[0], torch.int64), [x], 3 * x.nbytes),
        ("reduce_mean f32 [16384,2048] last axis", lambda: RC.reduce_mean(x, [-1]), lambda a: K.reduce_mean(a[0], [-1], True), [x], x.nbytes),
        ("transpose f32 [64,128,64,64] perm 0,2,1,3", lambda: RC.transpose(x4, [0, 2, 1, 3]), lambda a: K.transpose(a[0].view(64, 128, 64, 64), [0, 2, 1, 3]), [x], 2 * x.nbytes),
        ("transpose f32 [64,128,64,64] perm 0,1,3,2", lambda: RC.transpose(x4, [0, 1, 3, 2]), lambda a: K.transpose(a[0].view(64, 128, 64, 64), [0, 1, 3, 2]), [x], 2 * x.nbytes),
        ("expand f32 [64,8,1,256,64] -> x4", lambda: RC.expand(e_in, [64, 8, 4, 256, 64]), lambda a: K.expand(a[0], [64, 8, 4, 256, 64]), [e_in], 5 * e_in.nbytes),
        ("slice f32 [64,128,64,64] -> [...,32:64]", lambda: RC.slice_(x4, [32], [64], [3], [1], [64, 128, 64, 32]), lambda a: K.slice_(a[0].view(64, 128, 64, 64), [32], [64], [3], None), [x], x.nbytes),
        ("trilu f32 [8,2048,2048] upper k=1", lambda: RC.trilu(x.reshape(8, 2048, 2048), 1, True), lambda a: K.trilu(a[0].view(8, 2048, 2048), 1, True), [x], 3 * x.nbytes // 2),
        ("where f32 [16384,2048], y scalar", lambda: RC.where(x > 0, x, np.float32(0)), lambda a: K.where(a[1], a[0], a[2]), [x, x > 0, np.zeros((), np.float32)], 2 * x.nbytes + x.size),
    ]


def run_kernels(rows, with_gpu=True, with_cpu=True):
    threads = ref_cpu.max_threads() if ref_cpu.available() else 0
    print(f"{'case':46s} {'reference PTX':>14s} {'tier-1 PTX':>13s} {'library':>12s} {'reference on ' + str(threads) + ' host threads':>30s}   (us per launch, GB/s)")
    for name, plan, lib_fn, host_args, nbytes in kernel_cases():
        row = {"case": name, "bytes": nbytes}
        gb = lambda ms: nbytes / ms / 1e6  # noqa: E731
        try:
            p = plan()
        except Exception as e:  # a plan this oracle cannot build is left out of the table, not guessed
            print(f"{name:46s} plan not available: {e}")
            continue
        if with_gpu and ref_gpu.available():
            _, ms_ref = ref_gpu.run(p, time_iters=10)
            _, ms_t1 = ref_gpu.run(plan(), time_iters=10, ptx_dir=T1)
            dev = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in host_args]
            ms_lib = time_graph(lambda i: lib_fn(dev))
            row.update(ref_ptx_us=ms_ref * 1e3, tier1_us=ms_t1 * 1e3, library_us=ms_lib * 1e3, library_gbs=gb(ms_lib), ref_ptx_gbs=gb(ms_ref))
        if with_cpu and ref_cpu.available():
            ref_cpu.run(plan(), threads=threads)   # warm-up: page faults, thread pool
            t0 = time.perf_counter()
            reps = 3
            for _ in range(reps):
                ref_cpu.run(p, threads=threads)
            ms_cpu = (time.perf_counter() - t0) * 1e3 / reps
            row.update(ref_cpu_us=ms_cpu * 1e3, ref_cpu_gbs=gb(ms_cpu), cpu_threads=threads)
        rows.append(row)
        f = lambda k, g: f"{row[k]:9.1f} {row[g]:5.0f}" if k in row else f"{'-':>15s}"  # noqa: E731
        t1 = f"{row['tier1_us']:9.1f}" if "tier1_us" in row else "-"
        print(f"{name:46s} {f('ref_ptx_us', 'ref_ptx_gbs')} {t1:>13s} {f('library_us', 'library_gbs')} {f('ref_cpu_us', 'ref_cpu_gbs'):>30s}", flush=True)


MATMUL_SHAPES = [(1, 2048, 8192), (8, 2048, 8192), (64, 2048, 8192), (64, 2048, 16384), (64, 2048, 3072), (64, 8192, 2048), (64, 2048, 2048),
                 (64, 2048, 128256), (4096, 2048, 8192), (1, 4096, 14336), (8, 4096, 14336), (64, 4096, 14336), (4096, 4096, 14336),
                 (1, 14336, 4096), (8, 14336, 4096), (64, 14336, 4096), (4096, 14336, 4096)]


def run_cublas(rows):
    torch.backends.cuda.matmul.allow_tf32 = True
    a = torch.randn(8192, 8192, device="cuda")
    b = torch.randn(8192, 8192, device="cuda")
    c = torch.empty(8192, 8192, device="cuda")
    ms = min(time_graph(lambda i: torch.matmul(a, b, out=c), n=4, replays=2) for _ in range(3))
    tf32_peak = 2 * 8192 ** 3 / ms / 1e9
    print(f"TF32 tensor-core peak (cuBLAS, 8192^3, burst): {tf32_peak:.0f} TFLOP/s; a 3xTF32 GEMM can reach a third: {tf32_peak / 3:.0f} TFLOP/s algorithmic")
    rows.append({"case": "tf32_peak_tflops", "value": tf32_peak, "three_pass_ceiling": tf32_peak / 3})
    del a, b, c
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    print(f"{'MatMul [M,K]x[K,N]':34s} {'library us':>11s} {'cuBLAS fp32 us':>15s} {'library/cuBLAS':>15s} {'max |ours - cuBLAS| / scale':>28s} {'ours vs f64':>12s} {'cuBLAS vs f64':>14s}")
    for m, k, n in MATMUL_SHAPES:
        w = ring(lambda: torch.randn(k, n, device="cuda") * 0.02, 4 * k * n)
        x = torch.randn(m, k, device="cuda") * 0.02
        y = torch.empty(m, n, device="cuda")
        yb = torch.empty(m, n, device="cuda")
        wsb = K.matmul_workspace_bytes(1, m, n, k)
        ws = torch.empty(max(wsb // 4, 1), device="cuda") if wsb else None
        ms_lib = time_graph(lambda i: K.matmul(x, w[i % len(w)], out=y, workspace=ws))
        ms_blas = time_graph(lambda i: torch.matmul(x, w[i % len(w)], out=yb))
        K.matmul(x, w[0], out=y, workspace=ws)
        torch.matmul(x, w[0], out=yb)
        want = x.double() @ w[0].double()
        scale = float(want.abs().max())
        d = float((y - yb).abs().max()) / scale
        e_ours = float((y.double() - want).abs().max()) / scale
        e_blas = float((yb.double() - want).abs().max()) / scale
        rows.append({"case": f"matmul {m}x{k}x{n}", "library_us": ms_lib * 1e3, "cublas_fp32_us": ms_blas * 1e3, "ours_vs_cublas_rel": d,
                     "ours_vs_f64_rel": e_ours, "cublas_vs_f64_rel": e_blas, "library_tflops": 2 * m * n * k / ms_lib / 1e9,
                     "cublas_tflops": 2 * m * n * k / ms_blas / 1e9})
        print(f"[{m},{k}]x[{k},{n}]".ljust(34) + f" {ms_lib * 1e3:11.1f} {ms_blas * 1e3:15.1f} {ms_lib / ms_blas:15.2f} {d:28.2e} {e_ours:12.2e} {e_blas:14.2e}", flush=True)
        del w, x, y, yb, ws, want
        torch.cuda.empty_cache()


class Cudnn:
    """The few legacy cuDNN entry points the reference calls, through ctypes (no torch ops involved)."""
    FLOAT, SOFTMAX_FAST, SOFTMAX_MODE_CHANNEL, SIGMOID, RELU, NOT_PROPAGATE_NAN = 0, 0, 1, 0, 1, 0

    def __init__(self):
        self.l = ctypes.CDLL("libcudnn.so.9")
        self.h = ctypes.c_void_p()
        self.ok(self.l.cudnnCreate(ctypes.byref(self.h)), "cudnnCreate")
        self.ok(self.l.cudnnSetStream(self.h, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "cudnnSetStream")

    @staticmethod
    def ok(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed with status {rc}")

    def tensor(self, shape):
        """cudarc's create_nd_tensor: cudnnSetTensorNdDescriptor with dense strides."""
        d = ctypes.c_void_p()
        self.ok(self.l.cudnnCreateTensorDescriptor(ctypes.byref(d)), "cudnnCreateTensorDescriptor")
        n = len(shape)
        strides = [1] * n
        for i in range(n - 2, -1, -1):
            strides[i] = strides[i + 1] * shape[i + 1]
        self.ok(self.l.cudnnSetTensorNdDescriptor(d, self.FLOAT, n, (ctypes.c_int * n)(*shape), (ctypes.c_int * n)(*strides)), "cudnnSetTensorNdDescriptor")
        return d

    def set_stream(self):
        self.ok(self.l.cudnnSetStream(self.h, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "cudnnSetStream")

    def softmax(self, desc, x, y):
        one, zero = ctypes.c_float(1.0), ctypes.c_float(0.0)
        self.set_stream()
        self.ok(self.l.cudnnSoftmaxForward(self.h, self.SOFTMAX_FAST, self.SOFTMAX_MODE_CHANNEL, ctypes.byref(one), desc, ctypes.c_void_p(x.data_ptr()),
                                           ctypes.byref(zero), desc, ctypes.c_void_p(y.data_ptr())), "cudnnSoftmaxForward")

    def activation_desc(self, mode):
        a = ctypes.c_void_p()
        self.ok(self.l.cudnnCreateActivationDescriptor(ctypes.byref(a)), "cudnnCreateActivationDescriptor")
        self.ok(self.l.cudnnSetActivationDescriptor(a, mode, self.NOT_PROPAGATE_NAN, ctypes.c_double(0.0)), "cudnnSetActivationDescriptor")
        return a

    def activation(self, act, desc, x, y):
        one, zero = ctypes.c_float(1.0), ctypes.c_float(0.0)
        self.set_stream()
        self.ok(self.l.cudnnActivationForward(self.h, act, ctypes.byref(one), desc, ctypes.c_void_p(x.data_ptr()), ctypes.byref(zero), desc,
                                              ctypes.c_void_p(y.data_ptr())), "cudnnActivationForward")


def ulp_distance(a: torch.Tensor, b: torch.Tensor) -> int:
    ia = a.contiguous().view(torch.int32).to(torch.int64)
    ib = b.contiguous().view(torch.int32).to(torch.int64)
    ia = torch.where(ia < 0, -(ia + (1 << 31)), ia)
    ib = torch.where(ib < 0, -(ib + (1 << 31)), ib)
    return int((ia - ib).abs().max())


def run_cudnn(rows):
    cd = Cudnn()
    print(f"{'op':44s} {'library us':>11s} {'cuDNN us':>10s} {'library/cuDNN':>14s}   distance between the two results")
    for r, c in [(2048, 520), (64 * 32 * 128, 640), (16384, 4096)]:
        xs = ring(lambda: torch.randn(r, c, device="cuda"), 4 * r * c)
        y, yc = torch.empty(r, c, device="cuda"), torch.empty(r, c, device="cuda")
        desc = cd.tensor([r, c, 1, 1])
        ms_lib = time_graph(lambda i: K.softmax(xs[i % len(xs)], out=y))
        ms_dnn = time_graph(lambda i: cd.softmax(desc, xs[i % len(xs)], yc))
        K.softmax(xs[0], out=y)
        cd.softmax(desc, xs[0], yc)
        torch.cuda.synchronize()
        want = torch.softmax(xs[0].double(), -1)
        rel = float(((y - yc).abs() / yc.abs().clamp_min(1e-30)).max())
        row = {"case": f"softmax [{r},{c}]", "library_us": ms_lib * 1e3, "cudnn_us": ms_dnn * 1e3, "max_rel_ours_vs_cudnn": rel,
               "max_rel_ours_vs_f64": float(((y.double() - want).abs() / want).max()), "max_rel_cudnn_vs_f64": float(((yc.double() - want).abs() / want).max())}
        rows.append(row)
        print(f"softmax f32 [{r},{c}] last axis".ljust(44) + f" {ms_lib * 1e3:11.1f} {ms_dnn * 1e3:10.1f} {ms_lib / ms_dnn:14.2f}   max rel {rel:.2e} "
              f"(ours vs f64 {row['max_rel_ours_vs_f64']:.2e}, cuDNN vs f64 {row['max_rel_cudnn_vs_f64']:.2e})", flush=True)
        del xs, y, yc
    for name, mode in (("sigmoid", Cudnn.SIGMOID), ("relu", Cudnn.RELU)):
        shape = (1, 32768, 8192)            # rank 3 -> [1, 1, 32768, 8192] as the backend pads it (backend/activation.rs:127-155)
        xs = ring(lambda: torch.randn(shape, device="cuda") * 4, 4 * 32768 * 8192)
        y, yc = torch.empty(shape, device="cuda"), torch.empty(shape, device="cuda")
        desc = cd.tensor([1, 1, 32768, 8192])
        act = cd.activation_desc(mode)
        ms_lib = time_graph(lambda i: K.unary(name, xs[i % len(xs)], out=y))
        ms_dnn = time_graph(lambda i: cd.activation(act, desc, xs[i % len(xs)], yc))
        K.unary(name, xs[0], out=y)
        cd.activation(act, desc, xs[0], yc)
        torch.cuda.synchronize()
        ulp = ulp_distance(y, yc)
        want = torch.sigmoid(xs[0].double()).float() if name == "sigmoid" else torch.relu(xs[0])
        row = {"case": f"{name} [1,32768,8192]", "library_us": ms_lib * 1e3, "cudnn_us": ms_dnn * 1e3, "max_ulp_ours_vs_cudnn": ulp,
               "max_ulp_ours_vs_rounded_f64": ulp_distance(y, want), "max_ulp_cudnn_vs_rounded_f64": ulp_distance(yc, want)}
        rows.append(row)
        print(f"{name} f32 [1,32768,8192]".ljust(44) + f" {ms_lib * 1e3:11.1f} {ms_dnn * 1e3:10.1f} {ms_lib / ms_dnn:14.2f}   max {ulp} ulp "
              f"(ours vs correctly rounded {row['max_ulp_ours_vs_rounded_f64']} ulp, cuDNN {row['max_ulp_cudnn_vs_rounded_f64']} ulp)", flush=True)
        del xs, y, yc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", default=None, choices=["kernels", "cpu", "cublas", "cudnn"])
    args = ap.parse_args()
    out = {"kernels": [], "cublas": [], "cudnn": []}
    if args.only in (None, "kernels", "cpu"):
        run_kernels(out["kernels"], with_gpu=args.only != "cpu", with_cpu=args.only != "kernels")
    if args.only in (None, "cublas"):
        run_cublas(out["cublas"])
    if args.only in (None, "cudnn"):
        run_cudnn(out["cudnn"])
    if args.json:
        json.dump(out, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
