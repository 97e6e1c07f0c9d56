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


# kernels launched by one call of each binding (for launch accounting in benchmarks)
KERNELS_PER_CALL = {"gemm": 1, "layernorm_fwd": 1, "layernorm_bwd": 2, "colsum": 1, "elementwise": 1,
                    "cast_f32_to_bf16": 1, "softmax_fwd": 1, "softmax_bwd": 1, "sumsq": 2, "adam_step": 1,
                    "sgd_step": 1, "embedding_fwd": 1, "embedding_bwd": 1, "ce_stats": 1, "ce_finalize": 1,
                    "attn_fwd": 1, "attn_bwd": 3, "im2col": 1, "col2im": 1, "subsample": 1, "bn_fwd": 3, "bn_bwd": 3, "bn_apply": 1,
                    "maxpool_fwd": 1, "maxpool_bwd": 1, "avgpool": 1, "allreduce_scale_f32": 1,
                    "reduce_scatter_scale_sumsq_f32": 1, "allgather_b16": 1}
launch_counter = {"kernels": 0, "calls": 0}


class _Counting:
    """Proxy over the extension module that counts kernel launches issued through it."""

    def __init__(self, mod):
        self._mod = mod
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._mod, name)
            n = KERNELS_PER_CALL.get(name, 0)
            if n == 0:
                fn = raw
            else:
                def fn(*a, _raw=raw, _n=n):
                    launch_counter["kernels"] += _n
                    launch_counter["calls"] += 1
                    return _raw(*a)
            self._cache[name] = fn
        return fn


_proxy = None


def ext():
    """The extension module (behind a launch-counting proxy); raises when it cannot be loaded."""
    global _proxy
    _load()
    if _mod is None:
        raise RuntimeError(f"superscaler_b200 native extension unavailable: {_err}")
    if _proxy is None:
        _proxy = _Counting(_mod)
    return _proxy


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
