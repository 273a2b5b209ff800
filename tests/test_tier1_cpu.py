"""The symbol-compatible kernels (rmlk_b200/tier1) export exactly the reference's entry points.

tests/golden/tier1_entry_points.json lists every `extern "C" __global__` of the reference's 19 PTX modules
(cuda/src/ptx/*.cu) with its parameter types.  The PTX built from rmlk_b200/tier1/*.cu with plain `nvcc -ptx`
must define the same modules, the same names and the same parameter lists, or the reference's launch
wrappers (cuda/src/kernels/*.rs) could not drive it unmodified.
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.golden.extract_entry_points import entry_points  # noqa: E402


def test_tier1_ptx_matches_the_reference_interface():
    from rmlk_b200 import build
    ptx_dir = build.build_tier1()
    want = json.load(open(os.path.join(ROOT, "tests", "golden", "tier1_entry_points.json")))
    got = entry_points(ptx_dir)
    assert sorted(got) == sorted(want), "one PTX module per reference module"
    total = 0
    for module, entries in want.items():
        mine = {name: params for name, params in got[module]}
        for name, params in entries:
            assert name in mine, f"{module}: entry point {name} is missing"
            assert mine[name] == params, f"{module}.{name}: parameter list {mine[name]} != {params}"
            total += 1
        assert len(mine) == len(entries), f"{module}: extra entry points {sorted(set(mine) - {n for n, _ in entries})}"
    assert total == 266


def test_tier1_sources_need_no_special_flags():
    """Built the way the reference's build script builds its own files: no sm_100a-only code, no extra nvcc flags."""
    src_dir = os.path.join(ROOT, "rmlk_b200", "tier1")
    for f in os.listdir(src_dir):
        if f.endswith(".cu"):
            text = open(os.path.join(src_dir, f)).read()
            for token in ("tcgen05", "cp.async.bulk", "__cluster_dims__", "asm volatile"):
                assert token not in text, (f, token)
