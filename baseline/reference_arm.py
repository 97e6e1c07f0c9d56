"""`bench.py --impl reference`: the reference's own runtime on the same metric and config.

The reference tree is installed (copied, unmodified) under baseline/_ref by baseline/install_reference.py.
When that directory is absent, or the reference cannot run in this image, the arm reports why in one line.
"""
from __future__ import annotations

import os

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def run(args) -> dict:
    if not os.path.isdir(os.path.join(REF, "runtime")):
        return {"impl": "reference", "unavailable": "reference not installed under baseline/_ref: the source tree has "
                "no setup.py / pyproject.toml, so `pip install /root/reference` cannot build it"}
    try:
        from . import reference_runner
    except Exception as e:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"reference runner failed to import: {e}"}
    return reference_runner.run(args)
