"""Streaming ceiling of a [K, N] fp32 weight matrix on this GPU, by access pattern (no arithmetic).

`python -m rmlk_b200.streambench K N [reps]` compiles `csrc/tools/stream_probe.cu` with nvcc (into `csrc/build/`) and
runs it: plain 128-bit loads, then TMA loads into a ring of shared-memory stages as the tensor-core MatMul issues them
(row-major boxes of 32 or 128 columns, tile-major contiguous blocks, 1-D bulk copies, 256-column tiles), one CTA per
(tile, K split) or 148 CTAs over a balanced range of k-blocks.  The figures are what a weight-streaming kernel on
this shape can reach at best; `profiles/` quotes them beside the MatMul's own numbers.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "tools", "stream_probe.cu")
OUT = os.path.join(HERE, "csrc", "build", "stream_probe")
NVCC = os.environ.get("RMLK_NVCC", "/usr/local/cuda/bin/nvcc")


def build() -> str:
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    if not os.path.exists(OUT) or os.path.getmtime(OUT) < os.path.getmtime(SRC):
        subprocess.run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-o", OUT, SRC, "-lcuda"], check=True)
    return OUT


def main(argv):
    exe = build()
    return subprocess.run([exe] + argv).returncode


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
