"""Ahead-of-time build of the native extension ``superscaler_b200/_C*.so``.

``python -m superscaler_b200.build`` compiles every ``csrc/*.cu`` with
``nvcc -gencode arch=compute_100a,code=sm_100a`` (cross-compiles without a GPU), compiles the
bindings with the host compiler and links one shared object IN the package directory, so the
built library travels with the source tree.  Objects are cached under ``csrc/build/`` and only
rebuilt when a source or header is newer.

The reference JIT-builds its four extensions for sm_70/sm_80 at start-up on rank 0
(runtime/megatron/fused_kernels/__init__.py:30-95); here the build is explicit and ahead of time.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "build"
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
TARGET = PKG / f"_C{EXT_SUFFIX}"
HOST_SRC = PKG / "csrc_host"                      # host-only helpers (no CUDA, no torch): loadable on CPU boxes
HOST_MODULES = {"dataset_helpers.cpp": "_data_helpers", "search_native.cpp": "_search_native"}
HOST_TARGET = PKG / f"_data_helpers{EXT_SUFFIX}"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _torch_paths():
    import torch
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths()
    lib = ce.library_paths()
    return inc, lib, bool(torch._C._GLIBCXX_USE_CXX11_ABI)


def _newer(src_files, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in src_files)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build(verbose: bool = False, force: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    cu_files = sorted(CSRC.glob("*.cu"))
    cpp_files = sorted(CSRC.glob("*.cpp"))
    inc, lib, cxx11 = _torch_paths()
    py_inc = sysconfig.get_paths()["include"]
    jobs = []
    objs = []
    for cu in cu_files:
        o = OBJ / (cu.stem + ".o")
        objs.append(o)
        if force or _newer([cu] + headers, o):
            cmd = [NVCC, *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-cudart", "shared",
                   "-c", str(cu), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    for cpp in cpp_files:
        o = OBJ / (cpp.stem + ".o")
        objs.append(o)
        if force or _newer([cpp] + headers, o):
            cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
                   f"-D_GLIBCXX_USE_CXX11_ABI={int(cxx11)}", "-I/usr/local/cuda/include", f"-I{py_inc}"]
            cmd += [f"-I{i}" for i in inc]
            cmd += ["-c", str(cpp), "-o", str(o)]
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(_run, jobs):
                if verbose and out.strip():
                    print(out)
    if force or jobs or _newer(objs, TARGET):
        link = ["g++", "-shared", "-o", str(TARGET), *map(str, objs)]
        for l in lib:
            link += [f"-L{l}", f"-Wl,-rpath,{l}"]
        link += ["-L/usr/local/cuda/lib64", "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda",
                 "-ltorch_cuda", "-lcudart"]
        _run(link)
    build_host_helpers(force)
    return TARGET


def build_host_helpers(force: bool = False) -> Path:
    """Host-only helpers, one pybind11 module per source file, compiled with the host compiler only: the dataset
    index builders and the inner loops of the search's cost model.  Floating-point contraction is off so that the
    native cost model rounds exactly like its Python definition."""
    import pybind11
    py_inc = sysconfig.get_paths()["include"]
    for src_name, module in HOST_MODULES.items():
        src = HOST_SRC / src_name
        target = PKG / f"{module}{EXT_SUFFIX}"
        if force or _newer([src], target):
            _run(["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fPIC", "-shared", f"-I{py_inc}",
                  f"-I{pybind11.get_include()}", str(src), "-o", str(target)])
    return HOST_TARGET


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(path)
