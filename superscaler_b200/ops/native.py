"""Loader of the native sm_100a extension (``superscaler_b200/_C*.so``).

The extension is built ahead of time by ``python -m superscaler_b200.build`` and lives inside the
package directory.  On a machine with a GPU a missing or unloadable extension is an error: the
CUDA path never falls back to eager PyTorch silently.  On a CPU-only machine ``available()`` is
False and the pure-PyTorch reference implementations in ``ops.reference`` serve the tests.
"""
from __future__ import annotations

import glob
import importlib.util
import os

import torch

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_mod = None
_err = None


def _load():
    global _mod, _err
    if _mod is not None or _err is not None:
        return
    cands = sorted(glob.glob(os.path.join(_PKG_DIR, "_C*.so")))
    if not cands:
        _err = FileNotFoundError(
            f"native extension not built: no _C*.so in {_PKG_DIR}; run `python -m superscaler_b200.build`")
        return
    try:
        spec = importlib.util.spec_from_file_location("superscaler_b200._C", cands[0])
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mod = mod
    except Exception as e:  # noqa: BLE001 - reported verbatim by ext()
        _err = e


def available() -> bool:
    """True when the extension is importable AND a CUDA device is present."""
    _load()
    return _mod is not None and torch.cuda.is_available()


def ext():
    """The extension module; raises when it cannot be loaded."""
    _load()
    if _mod is None:
        raise RuntimeError(f"superscaler_b200 native extension unavailable: {_err}")
    return _mod


def check_status() -> int:
    """Reads the per-device kernel status word (synchronises).  0 = every bounded wait completed."""
    st = ext().status()
    code = int(st.item())
    return code


def raise_on_error() -> None:
    code = check_status()
    if code != 0:
        ext().status().zero_()
        raise RuntimeError(f"a superscaler_b200 kernel reported status {code} (1 = barrier wait ran out, "
                           "2 = peer wait ran out, 3 = bad argument)")
