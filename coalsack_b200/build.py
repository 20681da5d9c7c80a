"""Build recipe of the CUDA library (``libcsk_moe.so``), in-tree.

nvcc cross-compiles for sm_100a without a GPU present.  The library links only
the CUDA runtime and driver; it does not depend on PyTorch.
"""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcsk_moe.so")
SOURCES = ["csk_moe.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "csk_moe.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False, extra_flags=()) -> str:
    """Compile csrc/*.cu into libcsk_moe.so if it is missing or older than its sources."""
    if not force and not _stale():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, *extra_flags, "-I", os.path.join(ROOT, "include"), "-I", CSRC,
           "-o", LIB, *[os.path.join(CSRC, s) for s in SOURCES], "-lcuda"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        print(" ".join(cmd))
        print(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError("nvcc failed building libcsk_moe.so")
    return LIB


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
