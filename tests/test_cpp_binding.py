"""The C++ operator bindings (coalsack_b200/host) inside coalsack's own headers:
they compile against the reference tree in place of its CPU operators (CPU
check); a program that drives moe_router_node -> E x expert_mlp_node (through
process() with result_messages) -> expert_merge_node on the GPU reproduces the
CPU checker; and the MoE sub-graph built by coalsack's own graph_builder
(router, weight fetch, E expert nodes, merge, with their sync nodes) does so in
the strict one-call-per-expert mode and in the fused one-call-per-layer mode
(GPU checks, run from the prebuilt binaries)."""
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
    assert os.path.exists(build_check.GRAPH_OUT)
    syms = subprocess.run(["nm", "-D", build_check.GRAPH_OUT], capture_output=True, text=True).stdout
    for s in ("csk_moe_route", "csk_moe_forward", "csk_moe_expert_forward", "csk_moe_load_expert_mxfp4", "csk_moe_set_activation"):
        assert s in syms, f"{s}: graph_check does not reach the GPU bindings"
    assert os.path.exists(build_check.DENSE_OUT)
    syms = subprocess.run(["nm", "-D", build_check.DENSE_OUT], capture_output=True, text=True).stdout
    for s in ("csk_moe_load_expert_f16", "csk_moe_load_expert_f32", "csk_moe_dense_forward"):
        assert s in syms, f"{s}: dense_check does not reach the GPU binding"
    assert os.path.exists(build_check.EXPERT_F16_OUT)
    syms = subprocess.run(["nm", "-D", build_check.EXPERT_F16_OUT], capture_output=True, text=True).stdout
    for s in ("csk_moe_load_expert_f16", "csk_moe_expert_forward", "csk_moe_merge"):
        assert s in syms, f"{s}: expert_f16_check does not reach the GPU binding"


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


def _write_layer(path, sh, h, Wg, rb, ex):
    with open(path, "wb") as f:
        f.write(np.array([sh.num_experts, sh.top_k, sh.hidden, sh.ffn, h.shape[0], sh.act, int(sh.has_bias)],
                         np.int32).tobytes())
        f.write(np.ascontiguousarray(h, np.float32).tobytes())
        f.write(Wg.tobytes())
        f.write((rb if rb is not None else np.zeros(sh.num_experts, np.float32)).tobytes())
        for e in range(sh.num_experts):
            for n in ("w_up", "w_gate", "w_down"):
                f.write(ex[n][e].tobytes())
            if sh.has_bias:
                for n in ("b_up", "b_gate", "b_down"):
                    f.write(ex[n][e].tobytes())


def _run_graph(inp, outp, mode, frames, T, k, H):
    exe = build_check.GRAPH_OUT
    r = subprocess.run([exe, str(inp), str(outp), mode, str(frames)], capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = np.fromfile(outp, np.float32)
    info = dict(kv.split("=") for kv in r.stdout.split("graph_check ok:")[1].split())
    return raw[:T * k * 2].reshape(T, k, 2), raw[T * k * 2:].reshape(T, H), info


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["tiny_a", "tiny_b", "tiny_d"])
def test_graph_builder_subgraph_strict_and_fused(gpu_lib, golden, tag, tmp_path):
    """coalsack's graph_builder wires router -> fetch -> experts -> merge; both modes reproduce the reference's
    output for the layer, and in fused mode the second frame pulls no weights from the provider any more."""
    if not os.path.exists(build_check.GRAPH_OUT):
        pytest.skip("tests/cpp/_build/graph_check was not built (needs the reference checkout at build time)")
    sh, h, Wg, rb, ex, wbf = cases.tiny_case(tag)
    assert not wbf
    inp = tmp_path / "in.bin"
    _write_layer(inp, sh, h, Wg, rb, ex)
    T, k, H = sh.tokens, sh.top_k, sh.hidden
    for mode in ("strict", "fused"):
        ro, out, info = _run_graph(inp, tmp_path / f"out_{mode}.bin", mode, 2, T, k, H)
        assert np.array_equal(ro[..., 0], golden[f"{tag}_router"][..., 0]), mode
        mx, mr = cases.err_stats(out, golden[f"{tag}_out"])
        assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (tag, mode, mx, mr)
        if mode == "fused":
            # one probe of the first selected expert's shape; no expert is fetched again
            assert int(info["provider_gets_last_frame"]) <= 1, info


@pytest.mark.gpu
def test_graph_fused_mode_at_the_20b_shape(gpu_lib, port, tmp_path):
    """The 32-expert 2880 x 2880 layer with 32 tokens through the graph in fused mode: parity with the checker,
    and the time of a frame next to one csk_moe_forward call on the same batch."""
    import time
    from coalsack_b200 import MoeLayer, synth
    if not os.path.exists(build_check.GRAPH_OUT):
        pytest.skip("tests/cpp/_build/graph_check was not built (needs the reference checkout at build time)")
    sh = synth.C0
    h, Wg, rb, ex = cases.layer_inputs(sh)
    inp = tmp_path / "c0.bin"
    _write_layer(inp, sh, h, Wg, rb, ex)
    T, k, H = sh.tokens, sh.top_k, sh.hidden
    ro, out, info = _run_graph(inp, tmp_path / "c0_out.bin", "fused", 4, T, k, H)
    want_ro = port.router(h, Wg, rb, k)
    assert np.array_equal(ro[..., 0], want_ro[..., 0])
    want, _ = port.moe_layer(h, Wg, rb, ex, k, sh.act, nthreads=16, router_out=ro)
    mx, mr = cases.err_stats(out, want)
    assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (mx, mr)
    lay = MoeLayer.from_shape(sh, max_tokens=64)
    lay.set_router(Wg, rb)
    lay.load_experts(ex)
    for _ in range(3):
        lay.forward(h)
    t0 = time.perf_counter()
    for _ in range(10):
        lay.forward(h)
    direct_ms = (time.perf_counter() - t0) * 100.0
    lay.close()
    graph_ms = float(info["last_frame_ms"])
    print(f"fused graph frame {graph_ms:.3f} ms vs csk_moe_forward {direct_ms:.3f} ms ({graph_ms / direct_ms:.2f}x)")
    # the graph adds the router node's own call, E + 3 message hops and the fetch node's residency check
    assert graph_ms < 4.0 * direct_ms + 0.5


@pytest.mark.gpu
@pytest.mark.parametrize("bias,f32", [(True, False), (False, False), (True, True)])
def test_dense_ffn_node_binding(gpu_lib, port, bias, f32, tmp_path):
    """coalsack's dense_ffn_node type with the GPU binding behind it (FLOAT16 weights, and FLOAT32 ones, which the
    device rounds to fp16): output against the restatement, the weights uploaded once and again after an in-place
    refill, the reference's error text."""
    exe = build_check.DENSE_OUT
    if not os.path.exists(exe):
        pytest.skip("tests/cpp/_build/dense_check was not built (needs the reference checkout at build time)")
    make = cases.dense_ffn_case_f32 if f32 else cases.dense_ffn_case
    hidden, gw, uw, dw, bg, bu, bd = make(H=256, F=192, T=37, bias=bias, seed=83)
    inp, outp = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(inp, "wb") as f:
        f.write(np.array([256, 192, 37, int(bias) | (2 if f32 else 0)], np.int32).tobytes())
        for a in (hidden, gw, uw, dw) + ((bg, bu, bd) if bias else ()):
            f.write(np.ascontiguousarray(a).tobytes())
    r = subprocess.run([exe, str(inp), str(outp)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = np.fromfile(outp, np.float32).reshape(2, 37, 256)
    for got, gate in ((raw[0], gw), (raw[1], -gw)):
        want = port.dense_ffn(hidden, gate, uw, dw, bg, bu, bd)
        mx, mr = cases.err_stats(got, want)
        assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (mx, mr)


@pytest.mark.gpu
@pytest.mark.parametrize("bias", [True, False])
def test_expert_node_binding_with_fp16_weights(gpu_lib, port, bias, tmp_path):
    """coalsack's expert node fed FLOAT16 weight tensors (expert_mlp_node.h:269-389: what the provider makes
    of Q4_K / Q6_K / F16 expert slices) with the GPU binding behind it: E expert nodes through process(), the
    merge node, against the restatement; an expert nobody selected answers with the {0}-shaped tensor."""
    exe = build_check.EXPERT_F16_OUT
    if not os.path.exists(exe):
        pytest.skip("tests/cpp/_build/expert_f16_check was not built (needs the reference checkout at build time)")
    E, k, H, F, T = 7, 2, 256, 192, 45
    rng = np.random.default_rng(97)
    hidden = rng.standard_normal((T, H)).astype(np.float32)
    ro = np.zeros((T, k, 2), np.float32)
    for t in range(T):
        ro[t, :, 0] = rng.choice(E - 1, size=k, replace=False)   # expert E-1 is never selected
        w = np.exp(rng.standard_normal(k)).astype(np.float32)
        ro[t, :, 1] = w / w.sum()
    experts = [cases.dense_ffn_case(H=H, F=F, T=1, bias=True, seed=300 + e)[1:] for e in range(E)]
    inp, outp = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(inp, "wb") as f:
        f.write(np.array([E, k, H, F, T, 1, int(bias)], np.int32).tobytes())
        f.write(hidden.tobytes())
        f.write(ro.tobytes())
        for gw, uw, dw, bg, bu, bd in experts:
            for a in (uw, gw, dw) + ((bu, bg, bd) if bias else ()):
                f.write(np.ascontiguousarray(a).tobytes())
    r = subprocess.run([exe, str(inp), str(outp)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "placeholders=1" in r.stdout, r.stdout
    got = np.fromfile(outp, np.float32).reshape(T, H)
    dense = [port.dense_ffn(hidden, gw, uw, dw, *((bg, bu, bd) if bias else (None, None, None)))
             for gw, uw, dw, bg, bu, bd in experts]
    want = np.zeros((T, H), np.float32)
    for t in range(T):
        for j in range(k):
            want[t] = want[t] + np.float32(ro[t, j, 1]) * dense[int(ro[t, j, 0])][t]
    mx, mr = cases.err_stats(got, want)
    assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (mx, mr)


@pytest.mark.gpu
def test_graph_builder_subgraph_with_fp16_experts(gpu_lib, port, tmp_path):
    """The MoE sub-graph wired by coalsack's graph_builder with a provider that serves FLOAT16 expert tensors (what
    it makes of Q4_K / Q6_K / F16 models): strict and fused mode against the restatement; fused mode keeps the
    experts resident (no provider traffic in the second frame beyond the shape probe)."""
    if not os.path.exists(build_check.GRAPH_OUT):
        pytest.skip("tests/cpp/_build/graph_check was not built (needs the reference checkout at build time)")
    E, k, H, F, T = 6, 2, 256, 192, 33
    rng = np.random.default_rng(141)
    hidden = rng.standard_normal((T, H)).astype(np.float32)
    Wg = (rng.standard_normal((E, H)) * 0.3).astype(np.float32)
    rb = (rng.standard_normal(E) * 0.1).astype(np.float32)
    experts = [cases.dense_ffn_case(H=H, F=F, T=1, bias=True, seed=700 + e)[1:] for e in range(E)]
    inp = tmp_path / "in.bin"
    with open(inp, "wb") as f:
        f.write(np.array([E, k, H, F, T, 1, 1], np.int32).tobytes())
        f.write(hidden.tobytes())
        f.write(Wg.tobytes())
        f.write(rb.tobytes())
        for gw, uw, dw, bg, bu, bd in experts:
            for a in (uw, gw, dw, bu, bg, bd):
                f.write(np.ascontiguousarray(a).tobytes())
    want_ro = port.router(hidden, Wg, rb, k)
    dense = [port.dense_ffn(hidden, *experts[e]) for e in range(E)]
    want = np.zeros((T, H), np.float32)
    for t in range(T):
        for j in range(k):
            want[t] = want[t] + np.float32(want_ro[t, j, 1]) * dense[int(want_ro[t, j, 0])][t]
    for mode in ("strict", "fused"):
        outp = tmp_path / f"out_{mode}.bin"
        r = subprocess.run([build_check.GRAPH_OUT, str(inp), str(outp), mode, "2", "f16"], capture_output=True, text=True,
                           timeout=180)
        assert r.returncode == 0, r.stdout + r.stderr
        raw = np.fromfile(outp, np.float32)
        ro, out = raw[:T * k * 2].reshape(T, k, 2), raw[T * k * 2:].reshape(T, H)
        assert np.array_equal(ro[..., 0], want_ro[..., 0]), mode
        mx, mr = cases.err_stats(out, want)
        assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (mode, mx, mr)
        if mode == "fused":
            info = dict(kv.split("=") for kv in r.stdout.split("graph_check ok:")[1].split())
            assert int(info["provider_gets_last_frame"]) <= 1, info
