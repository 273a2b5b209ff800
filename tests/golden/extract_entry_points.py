"""Writes tests/golden/tier1_entry_points.json: every entry point of the reference's PTX modules with its
parameter types, in order.

    make -C oracle REF=<reference checkout>        # builds oracle/_ref/ptx/*.ptx from the reference's own sources
    python tests/golden/extract_entry_points.py

The list is the interface that the symbol-compatible kernels (rmlk_b200/tier1) must reproduce: the reference's
launch wrappers look kernels up by these names (cuda/src/kernels/*.rs `load_kernel`) and pass arguments
positionally.
"""
import glob
import json
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def entry_points(ptx_dir):
    out = {}
    for f in sorted(glob.glob(os.path.join(ptx_dir, "*.ptx"))):
        s = open(f).read()
        ents = re.findall(r"\.visible \.entry (\w+)\(\s*(.*?)\)\s*(?:\.maxntid[^\n]*\n)?\{", s, re.S)
        out[os.path.basename(f)[:-4]] = sorted([name, re.findall(r"\.param (?:\.align \d+ )?\.(\w+) ", params)] for name, params in ents)
    return out


if __name__ == "__main__":
    eps = entry_points(os.path.join(ROOT, "oracle", "_ref", "ptx"))
    json.dump(eps, open(os.path.join(HERE, "tier1_entry_points.json"), "w"), indent=0, sort_keys=True)
    print(sum(len(v) for v in eps.values()), "entry points in", len(eps), "modules")
