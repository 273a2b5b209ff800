"""Device time of the symbol-compatible kernels (rmlk_b200/tier1) beside the reference's own kernels on the same GPU,
both driven through the reference's launch contract (grid = ceil(n / 128) x 128 threads), and beside the library's
own launchers (include/rmlk_b200.h) on the same operands.

    python tests/tier1_vs_reference_timing.py

Not collected by pytest.  Uses oracle/ref_calls.py to build the launches, so it lives with the tests.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import ref_calls as RC  # noqa: E402
from oracle import ref_gpu  # noqa: E402
from rmlk_b200 import kernels as K  # noqa: E402
from rmlk_b200.opbench import time_graph  # noqa: E402

T1 = os.path.join(ROOT, "rmlk_b200", "tier1", "ptx")


def main():
    rng = np.random.default_rng(0)
    f = lambda *s: rng.standard_normal(s, dtype=np.float32)  # noqa: E731
    x = f(16384, 2048)
    cases = [
        ("add f32 [16384,2048] same shape", lambda: RC.arith("add", x, x), lambda a: K.binary("add", a[0], a[0]), [x], 3 * x.nbytes),
        ("add f32 [16384,2048] + [2048]", lambda: RC.arith("add", x, x[0]), lambda a: K.binary("add", a[0], a[1]), [x, x[0].copy()], 2 * x.nbytes),
        ("div f32 [16384,2048] / [16384,1]", lambda: RC.arith("div", x, x[:, :1].copy()), lambda a: K.binary("div", a[0], a[1]), [x, x[:, :1].copy()], 2 * x.nbytes),
        ("sin f32 32M", lambda: RC.unary("sin", x), lambda a: K.unary("sin", a[0]), [x], 2 * x.nbytes),
        ("cast f32->i64 32M", lambda: RC.cast(x, np.int64), lambda a: K.cast(a[0], torch.int64), [x], 3 * x.nbytes),
        ("reduce_mean f32 [16384,2048] last axis", lambda: RC.reduce_mean(x, [-1]), lambda a: K.reduce_mean(a[0], [-1], True), [x], x.nbytes),
        ("transpose f32 [64,128,64,64] perm 0,2,1,3", lambda: RC.transpose(x.reshape(64, 128, 64, 64), [0, 2, 1, 3]),
         lambda a: K.transpose(a[0].view(64, 128, 64, 64), [0, 2, 1, 3]), [x], 2 * x.nbytes),
        ("transpose f32 [64,128,64,64] perm 0,1,3,2", lambda: RC.transpose(x.reshape(64, 128, 64, 64), [0, 1, 3, 2]),
         lambda a: K.transpose(a[0].view(64, 128, 64, 64), [0, 1, 3, 2]), [x], 2 * x.nbytes),
        ("expand f32 [64,8,1,512,64] -> x4", lambda: RC.expand(x[:8192].reshape(64, 8, 1, 512, 64)[:, :, :, :256].copy(), [64, 8, 4, 256, 64]),
         lambda a: K.expand(a[0], [64, 8, 4, 256, 64]), [x[:8192].reshape(64, 8, 1, 512, 64)[:, :, :, :256].copy()], 5 * x.nbytes // 8),
    ]
    print(f"{'case':48s} {'reference PTX':>14s} {'tier-1 PTX':>12s} {'library':>10s}   (us per launch; GB/s of algorithmic bytes)")
    for name, plan, lib, host_args, nbytes in cases:
        _, ms_ref = ref_gpu.run(plan(), time_iters=10)
        _, ms_t1 = ref_gpu.run(plan(), time_iters=10, ptx_dir=T1)
        dev = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in host_args]
        ms_lib = time_graph(lambda i: lib(dev))
        gb = lambda ms: nbytes / ms / 1e6  # noqa: E731
        print(f"{name:48s} {ms_ref * 1e3:8.1f} {gb(ms_ref):5.0f} {ms_t1 * 1e3:7.1f} {gb(ms_t1):5.0f} {ms_lib * 1e3:6.1f} {gb(ms_lib):5.0f}", flush=True)


if __name__ == "__main__":
    main()
