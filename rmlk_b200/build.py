"""In-tree build of librmlk_b200.so with nvcc for sm_100a.

`python -m rmlk_b200.build` (or `build()` from `__graft_entry__`) compiles every `csrc/*.cu` and
`csrc/runtime/*.cpp` to an object under `csrc/build/` (git-ignored) and links
`rmlk_b200/librmlk_b200.so` next to this file.  Objects are rebuilt only when a source or header is
newer.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "librmlk_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC = os.environ.get("RMLK_NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-I", INCLUDE, "-I", CSRC,
]


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "runtime", "*.cpp")))


def _headers():
    return (glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "runtime", "*.h")) +
            glob.glob(os.path.join(INCLUDE, "*.h")))


def _obj_path(src: str) -> str:
    rel = os.path.relpath(src, CSRC).replace(os.sep, "_")
    return os.path.join(OBJ, rel + ".o")


def _compile(src: str, verbose: bool) -> str:
    obj = _obj_path(src)
    cmd = [NVCC] + NVCC_FLAGS + (["-x", "cu"] if src.endswith(".cpp") else []) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr.strip():
        print(r.stderr, file=sys.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    srcs = _sources()
    hdr_mtime = max((os.path.getmtime(h) for h in _headers()), default=0.0)
    todo = []
    for s in srcs:
        o = _obj_path(s)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_mtime):
            todo.append(s)
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
            list(ex.map(lambda s: _compile(s, verbose), todo))
    objs = [_obj_path(s) for s in srcs]
    if todo or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


TIER1 = os.path.join(HERE, "tier1")
TIER1_PTX = os.path.join(TIER1, "ptx")


def build_tier1(force: bool = False) -> str:
    """PTX of the symbol-compatible kernels (rmlk_b200/tier1/*.cu), one module per reference module, built the
    way the reference's cuda/build.rs builds its own files: plain nvcc, compute capability 10.0, include
    path = the headers directory, no extra flags."""
    os.makedirs(TIER1_PTX, exist_ok=True)
    hdr = max(os.path.getmtime(h) for h in glob.glob(os.path.join(TIER1, "headers", "*.cuh")))
    todo = []
    for src in sorted(glob.glob(os.path.join(TIER1, "*.cu"))):
        out = os.path.join(TIER1_PTX, os.path.basename(src)[:-3] + ".ptx")
        if force or not os.path.exists(out) or os.path.getmtime(out) < max(os.path.getmtime(src), hdr):
            todo.append((src, out))

    def one(job):
        src, out = job
        r = subprocess.run([NVCC, "-ptx", "-arch=sm_100", "-I", os.path.join(TIER1, "headers"), src, "-o", out], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc -ptx failed for {src}:\n{r.stdout}\n{r.stderr}")

    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
            list(ex.map(one, todo))
    return TIER1_PTX


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_tier1(force="--force" in sys.argv))
