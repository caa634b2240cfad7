"""Builds the CUDA library of the token sampler in-tree with nvcc for sm_100a.

    python -m executorch_b200.build          # or: from executorch_b200.build import build

Output: executorch_b200/lib/libetb200_sampler.so (C ABI declared in include/etb200_sampler.h).
nvcc cross-compiles without a GPU, so this also serves as the "does it build" check.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libetb200_sampler.so")

SOURCES = ["sampler_kernels.cu", "c_api.cu", "static_scratch.cu"]
HEADERS = sorted(f for f in os.listdir(CSRC) if f.endswith(".cuh")) + [
    os.path.join("..", "..", "include", "etb200_sampler.h")]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the sampler has no non-CUDA build")
    return exe


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    os.makedirs(LIBDIR, exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB


PYBIND = os.path.join(LIBDIR, "_sampler_pybind" + (__import__("sysconfig").get_config_var("EXT_SUFFIX") or ".so"))


def build_pybind(force: bool = False) -> str:
    """Builds the pybind11 module over the C++ Sampler class (g++; links the CUDA library)."""
    import sysconfig

    import pybind11

    src = os.path.join(CSRC, "pybind.cpp")
    hpp = os.path.join(PKG, "..", "include", "etb200_sampler.hpp")
    if (not force and os.path.exists(PYBIND)
            and os.path.getmtime(PYBIND) > max(os.path.getmtime(src), os.path.getmtime(hpp), os.path.getmtime(LIB))):
        return PYBIND
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden",
           "-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], src,
           "-L" + LIBDIR, "-letb200_sampler", "-Wl,-rpath,$ORIGIN", "-o", PYBIND]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    return PYBIND


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_pybind(force="--force" in sys.argv))
