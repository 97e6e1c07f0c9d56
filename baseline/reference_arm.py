"""`bench.py --impl reference`: the reference's own runtime on the same metric and config.

The arm expects the unmodified reference installed under baseline/_ref (pip --target).  The reference is a script
tree without packaging metadata, so that install produces nothing; the arm then reports why in one line.
"""
from __future__ import annotations

import os

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def run(args) -> dict:
    if not os.path.isdir(os.path.join(REF, "runtime")):
        return {"impl": "reference", "unavailable": "reference not installed under baseline/_ref: the source tree has "
                "no setup.py / pyproject.toml, so pip cannot build or install it, and its runtime needs apex, "
                "torch._six and JIT-built sm_70/sm_80 extensions that cannot be supplied unmodified"}
    return {"impl": "reference", "unavailable": "baseline/_ref holds a reference tree, but its runtime imports apex and "
            "torch._six and JIT-builds sm_70/sm_80 extensions: it cannot run unmodified in this image"}
