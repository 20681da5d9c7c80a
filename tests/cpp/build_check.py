"""Builds tests/cpp/_build/shim_check: coalsack's own headers with the GPU
operator bindings (coalsack_b200/host) placed ahead of them on the include path.
Needs the reference checkout; where it is absent a prebuilt binary is kept."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_build", "shim_check")


GRAPH_OUT = os.path.join(HERE, "_build", "graph_check")
DENSE_OUT = os.path.join(HERE, "_build", "dense_check")
EXPERT_F16_OUT = os.path.join(HERE, "_build", "expert_f16_check")


def _compile(src, out, ref, extra_inc=(), verbose=False):
    cmd = ["g++", "-std=c++20", "-O1"]
    for inc in extra_inc:
        cmd += ["-I", inc]
    cmd += ["-I", os.path.join(ROOT, "coalsack_b200", "host"), "-I", os.path.join(ROOT, "include"),
            "-I", os.path.join(ROOT, "oracle", "cereal_shim"), "-I", os.path.join(ROOT, "oracle", "spdlog_shim"),
            "-I", os.path.join(ref, "include"),
            src, "-o", out, "-L", os.path.join(ROOT, "coalsack_b200"), "-lcsk_moe",
            "-Wl,-rpath,$ORIGIN/../../../coalsack_b200", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        print(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError(f"building {os.path.basename(out)} failed")
    return out


def build(ref: str | None = None, verbose: bool = False) -> str | None:
    """shim_check (the three operator bindings driven by hand) and graph_check (the MoE sub-graph built by
    coalsack's own graph_builder, with an in-memory weight provider from tests/cpp/stub)."""
    if ref is None:
        import oracle
        ref = oracle.reference_root()
    if not ref or not os.path.exists(os.path.join(ref, "include", "coalsack", "nn", "nn_nodes.h")):
        return OUT if os.path.exists(OUT) else None
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    _compile(os.path.join(HERE, "shim_check.cpp"), OUT, ref, verbose=verbose)
    _compile(os.path.join(HERE, "graph_check.cpp"), GRAPH_OUT, ref, extra_inc=[os.path.join(HERE, "stub")], verbose=verbose)
    _compile(os.path.join(HERE, "dense_check.cpp"), DENSE_OUT, ref, verbose=verbose)
    _compile(os.path.join(HERE, "expert_f16_check.cpp"), EXPERT_F16_OUT, ref, verbose=verbose)
    return OUT


if __name__ == "__main__":
    print(build(verbose=True))
