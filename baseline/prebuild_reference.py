"""Copies the unmodified reference tree to baseline/_ref and pre-builds the reference's own CUDA extensions.

The reference JIT-builds four extensions at start-up (runtime/megatron/fused_kernels/__init__.py:30-95) into
fused_kernels/build/ through torch.utils.cpp_extension.load.  Running that same loader here, with the device
capability of a B200 reported to torch's extension builder, leaves the objects, the ninja file and the shared objects
in that directory, so that a later start on a GPU box finds them up to date instead of compiling for minutes.
Nothing under baseline/_ref is edited; the build directory is the reference's own output directory.
"""
from __future__ import annotations

import os
import shutil
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SOURCE = os.environ.get("SSB_REFERENCE_SOURCE", os.path.join(os.sep, "root", "reference"))


def copy_tree() -> bool:
    if os.path.isfile(os.path.join(REF, "runtime", "pretrain_gpt.py")):
        return True
    if not os.path.isdir(os.path.join(SOURCE, "runtime")):
        return False
    os.makedirs(REF, exist_ok=True)
    for part in ("runtime", "search", "profiler"):
        dst = os.path.join(REF, part)
        if not os.path.isdir(dst):
            shutil.copytree(os.path.join(SOURCE, part), dst)
    return True


def prebuild_extensions(verbose: bool = False) -> None:
    import torch
    from baseline import reference_arm as ra
    ra._install_shims()
    if not torch.cuda.is_available():
        # what torch's builder would see on the GPU box: one visible device of compute capability 10.0
        torch.cuda.device_count = lambda: 1
        torch.cuda.get_device_capability = lambda *_: (10, 0)
    with open(ra.PREBUILT_MARK, "w") as f:
        f.write(ra.RUNTIME)
    from megatron import fused_kernels
    fused_kernels.load(types.SimpleNamespace(rank=0 if verbose else 1, masked_softmax_fusion=True))
    import subprocess
    subprocess.run(["make", "-C", os.path.join(ra.runtime_dir(), "megatron", "data")], check=True,
                   stdout=None if verbose else subprocess.DEVNULL)


def main(verbose: bool = False) -> None:
    if copy_tree():
        prebuild_extensions(verbose)


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(HERE))
    main(verbose="-v" in sys.argv)
