"""Run reference call plans on the PTX build of the reference kernels.  TEST INFRASTRUCTURE ONLY.

`oracle/_ref/ptx/<op>.ptx` is what `nvcc -arch=sm_100a -ptx` makes of the reference's own
cuda/src/ptx/<op>.cu — the artefact the reference's cuda/build.rs embeds.  `run(plan)` loads the
module through the CUDA driver API and launches the entry point with the reference's contract:
grid = ceil(n/128) blocks of 128 threads, no shared memory (cuda/src/kernels/binary.rs:78-97 and the
identical `launch_config` in every other wrapper).  Needs a GPU; imported only by `-m gpu` tests and
by bench.py's optional "reference kernels on this GPU" report.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PTX_DIR = os.path.join(_HERE, "_ref", "ptx")
_modules = {}
_ctx_ready = False


def available() -> bool:
    return os.path.isdir(PTX_DIR)


def _drv():
    from cuda.bindings import driver
    return driver


def _chk(res):
    err = res[0]
    if int(err) != 0:
        raise RuntimeError(f"CUDA driver error {err}")
    return res[1:] if len(res) > 2 else (res[1] if len(res) == 2 else None)


def _init():
    """Use the primary context (shared with torch / the runtime API) of device 0."""
    global _ctx_ready
    if _ctx_ready:
        return
    d = _drv()
    _chk(d.cuInit(0))
    dev = _chk(d.cuDeviceGet(0))
    ctx = _chk(d.cuDevicePrimaryCtxRetain(dev))
    _chk(d.cuCtxSetCurrent(ctx))
    _ctx_ready = True


def _function(module: str, symbol: str, ptx_dir: str):
    d = _drv()
    _init()
    key = (ptx_dir, module)
    if key not in _modules:
        with open(os.path.join(ptx_dir, module + ".ptx"), "rb") as f:
            ptx = f.read() + b"\0"
        _modules[key] = _chk(d.cuModuleLoadData(ptx))
    return _chk(d.cuModuleGetFunction(_modules[key], symbol.encode()))


def run(plan, time_iters: int = 0, ptx_dir: str = None):
    """Execute one plan on the GPU; returns plan.out.  With time_iters > 0 also returns the mean
    launch time in milliseconds (CUDA events on the default stream).  `ptx_dir` selects another set of
    PTX modules with the same entry points (the symbol-compatible kernels of rmlk_b200/tier1) to be driven
    through the same launch contract."""
    d = _drv()
    fn = _function(plan.module, plan.symbol, ptx_dir or PTX_DIR)
    dev_bufs = []
    holders = []
    ptr_vals = []
    for kind, v in plan.args:
        if kind in ("in", "out"):
            if v is None:
                p = 0
            else:
                nbytes = max(int(v.nbytes), 16)
                p = int(_chk(d.cuMemAlloc(nbytes)))
                if v.nbytes:
                    _chk(d.cuMemcpyHtoD(p, v.ctypes.data, v.nbytes))
                dev_bufs.append((kind, v, p))
            c = ctypes.c_uint64(p)
        elif kind == "u64":
            c = ctypes.c_uint64(int(v))
        elif kind == "i64":
            c = ctypes.c_int64(int(v))
        elif kind == "bool":
            c = ctypes.c_uint8(1 if v else 0)
        else:
            raise ValueError(kind)
        holders.append(c)
        ptr_vals.append(ctypes.addressof(c))
    params = (ctypes.c_void_p * len(ptr_vals))(*ptr_vals)
    grid = max((int(plan.n) + 127) // 128, 1)

    def launch():
        _chk(d.cuLaunchKernel(fn, grid, 1, 1, 128, 1, 1, 0, 0, ctypes.addressof(params), 0))

    launch()
    _chk(d.cuCtxSynchronize())
    ms = None
    if time_iters > 0:
        e0 = _chk(d.cuEventCreate(0))
        e1 = _chk(d.cuEventCreate(0))
        _chk(d.cuEventRecord(e0, 0))
        for _ in range(time_iters):
            launch()
        _chk(d.cuEventRecord(e1, 0))
        _chk(d.cuEventSynchronize(e1))
        ms = float(_chk(d.cuEventElapsedTime(e0, e1))) / time_iters
    for kind, v, p in dev_bufs:
        if kind == "out" and v.nbytes and time_iters == 0:
            _chk(d.cuMemcpyDtoH(v.ctypes.data, p, v.nbytes))
        _chk(d.cuMemFree(p))
    return (plan.out, ms) if time_iters > 0 else plan.out
