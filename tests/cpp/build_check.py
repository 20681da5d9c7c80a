"""Builds tests/cpp/_build/shim_check: coalsack's own headers with the GPU
operator bindings (coalsack_b200/host) placed ahead of them on the include path.
Needs the reference checkout; where it is absent a prebuilt binary is kept."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_build", "shim_check")


def build(ref: str | None = None, verbose: bool = False) -> str | None:
    if ref is None:
        import oracle
        ref = oracle.reference_root()
    if not ref or not os.path.exists(os.path.join(ref, "include", "coalsack", "nn", "nn_nodes.h")):
        return OUT if os.path.exists(OUT) else None
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = ["g++", "-std=c++20", "-O1",
           "-I", os.path.join(ROOT, "coalsack_b200", "host"), "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(ROOT, "oracle", "cereal_shim"), "-I", os.path.join(ROOT, "oracle", "spdlog_shim"),
           "-I", os.path.join(ref, "include"),
           os.path.join(HERE, "shim_check.cpp"), "-o", OUT, "-L", os.path.join(ROOT, "coalsack_b200"), "-lcsk_moe",
           "-Wl,-rpath,$ORIGIN/../../../coalsack_b200", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        print(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError("building the C++ binding check failed")
    return OUT


if __name__ == "__main__":
    print(build(verbose=True))
