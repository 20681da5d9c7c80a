"""The C++ operator bindings (coalsack_b200/host) inside coalsack's own headers:
they compile against the reference tree in place of its CPU operators (CPU
check), and a program that drives moe_router_node -> E x expert_mlp_node (through
process() with result_messages) -> expert_merge_node on the GPU reproduces the
CPU checker (GPU check, run from the prebuilt binary)."""
import os
import subprocess

import numpy as np
import pytest

from tests import cases
from tests.cpp import build_check



def test_bindings_compile_against_reference_headers():
    import oracle
    REF = oracle.reference_root()
    if not REF:
        pytest.skip("no reference checkout here")
    from coalsack_b200.build import build_library
    build_library()
    exe = build_check.build(REF)
    assert exe and os.path.exists(exe)
    syms = subprocess.run(["nm", "-D", exe], capture_output=True, text=True).stdout
    for s in ("csk_moe_route", "csk_moe_expert_forward", "csk_moe_merge", "csk_moe_load_expert_mxfp4"):
        assert s in syms, f"{s}: the reference's CPU operator was compiled instead of the GPU binding"


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["tiny_a", "tiny_b"])
def test_graph_nodes_on_gpu_match_checker(gpu_lib, golden, tag, tmp_path):
    exe = build_check.OUT
    if not os.path.exists(exe):
        pytest.skip("tests/cpp/_build/shim_check was not built (needs the reference checkout at build time)")
    sh, h, Wg, rb, ex, wbf = cases.tiny_case(tag)
    assert not wbf
    inp, outp = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(inp, "wb") as f:
        f.write(np.array([sh.num_experts, sh.top_k, sh.hidden, sh.ffn, sh.tokens, sh.act, int(sh.has_bias)],
                         np.int32).tobytes())
        f.write(h.tobytes())
        f.write(Wg.tobytes())
        f.write((rb if rb is not None else np.zeros(sh.num_experts, np.float32)).tobytes())
        for e in range(sh.num_experts):
            for n in ("w_up", "w_gate", "w_down"):
                f.write(ex[n][e].tobytes())
            if sh.has_bias:
                for n in ("b_up", "b_gate", "b_down"):
                    f.write(ex[n][e].tobytes())
    r = subprocess.run([exe, str(inp), str(outp)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = np.fromfile(outp, np.float32)
    T, k, H = sh.tokens, sh.top_k, sh.hidden
    ro = raw[:T * k * 2].reshape(T, k, 2)
    out = raw[T * k * 2:].reshape(T, H)
    if rb is None:
        # the program always passes a bias tensor; zeros leave the logits unchanged
        pass
    assert np.array_equal(ro[..., 0], golden[f"{tag}_router"][..., 0])
    mx, mr = cases.err_stats(out, golden[f"{tag}_out"])
    assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (mx, mr)
