"""Builds libvsparse_b200.so (CUDA kernels + C ABI + host builder) and the C++ benchmark drivers in-tree.

    python -m vectorsparse_b200.build            # library + drivers
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libvsparse_b200.so")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build vectorsparse_b200")
    return exe


def _sources():
    c = os.path.join(HERE, "csrc")
    return [os.path.join(c, "vsparse_abi.cu"), os.path.join(c, "host_build.cpp")]


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _all_deps():
    deps = [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    c = os.path.join(HERE, "csrc")
    deps += [os.path.join(c, f) for f in os.listdir(c)]
    return deps


def build_library(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale(LIB, _all_deps()):
        return LIB
    cmd = [_nvcc(), *ARCH, "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(HERE, "csrc"), "-o", LIB, *_sources()]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    subprocess.run(cmd, check=True)
    return LIB


def build_drivers(force: bool = False):
    """spmm_benchmark / sddmm_benchmark: same positional command line as the reference drivers; compat_check: every
    overload of include/vsparse_compat.h against a host product."""
    out = []
    d = os.path.join(HERE, "drivers")
    for name in ("spmm_benchmark", "sddmm_benchmark", "compat_check"):
        src = os.path.join(d, name + ".cpp")
        exe = os.path.join(d, name)
        deps = [src, os.path.join(d, "driver_common.h"), os.path.join(ROOT, "include", "vsparse_compat.h"), LIB]
        if force or _stale(exe, deps):
            subprocess.run([_nvcc(), *ARCH, "-O2", "-std=c++17", "-x", "cu", "-I", os.path.join(ROOT, "include"), "-o", exe, src,
                            "-L", HERE, "-lvsparse_b200", "-Xlinker", "-rpath," + HERE], check=True)
        out.append(exe)
    return out


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    build_drivers(force="--force" in sys.argv)
    print(LIB)
