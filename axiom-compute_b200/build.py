"""Builds libaxc_cuda.so (sm_100a only) in-tree with nvcc.

The shared library is the product: hand-written CUDA kernels plus the runtime layer behind
the C ABI of ``include/axc_cuda.h``.  ``python -m`` is not needed; call ``build_library()``
or run this file.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libaxc_cuda.so")
SOURCES = ["axc_runtime.cu", "q4_stream.cu", "q4k_matvec.cu", "q4_0_matvec.cu", "q4k_prefill.cu", "axc_static.cu"]
HEADERS = ["axc_device.cuh", "axc_kernels.h", os.path.join("..", "..", "include", "axc_cuda.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-O2,-Wall",
    "--shared", "-cudart", "static",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libaxc_cuda.so cannot be built")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    """Compile every CUDA source for sm_100a into ``libaxc_cuda.so``; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS]
    if ptxas_info:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB_PATH] + [os.path.join(CSRC, s) for s in SOURCES]
    env = dict(os.environ)
    # nvcc's host compiler must be the system g++ (some shells export CC/CXX to wrappers).
    env.pop("CC", None)
    env.pop("CXX", None)
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if verbose or res.returncode != 0 or ptxas_info:
        sys.stderr.write(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libaxc_cuda.so:\n" + res.stdout[-4000:])
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force=True, verbose=True, ptxas_info="-v" in sys.argv))
