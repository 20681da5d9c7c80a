"""Parity of the CUDA path, through the C ABI, with the CPU checker: golden
vectors of the unmodified reference, the plain-C restatement on the same seeded
inputs, and the reference itself where its compiled wrapper travelled along."""
import numpy as np
import pytest

from coalsack_b200 import (CskError, MoeLayer, PATH_STREAM, PATH_TILE, PATH_TILE_PAIR, expert_merge_node, expert_mlp_node,
                           moe_router_node, synth)
from tests import cases

pytestmark = pytest.mark.gpu


def make_layer(sh, Wg, rb, ex, wbf=False, max_tokens=None, sigmoid=False, **kw):
    lay = MoeLayer.from_shape(sh, max_tokens=max_tokens or sh.tokens, weight_before_ffn=wbf,
                              sigmoid_gating=sigmoid, **kw)
    lay.set_router(Wg, rb)
    lay.load_experts(ex)
    return lay


def assert_close(got, want, what=""):
    mx, mr = cases.err_stats(got, want)
    assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, f"{what}: max/rms={mx:.3e} meanrel={mr:.3e}"
    return mx, mr


def same_experts(a, b):
    return np.array_equal(a[..., 0], b[..., 0])


# ---- weight repack ----------------------------------------------------------
@pytest.mark.parametrize("tag", ["tiny_a", "tiny_b", "tiny_d"])
def test_repack_is_lossless(gpu_lib, tag):
    sh, h, Wg, rb, ex, wbf = cases.tiny_case(tag)
    lay = make_layer(sh, Wg, rb, ex)
    for e in range(sh.num_experts):
        for which, name in enumerate(("w_up", "w_gate", "w_down")):
            assert np.array_equal(lay.unpack_expert(e, which), ex[name][e]), (e, name)          # streaming layout
            assert np.array_equal(lay.unpack_expert(e, which + 3), ex[name][e]), (e, name, "T")  # tensor-core layout
    lay.close()


def test_repack_is_lossless_full_size(gpu_lib):
    sh = synth.C0.with_(num_experts=2, top_k=2)
    ex = synth.all_experts(sh)
    lay = MoeLayer.from_shape(sh, max_tokens=8)
    lay.load_experts(ex)
    for e in range(2):
        for which, name in enumerate(("w_up", "w_gate", "w_down")):
            assert np.array_equal(lay.unpack_expert(e, which), ex[name][e])
            assert np.array_equal(lay.unpack_expert(e, which + 3), ex[name][e])
    lay.close()


# ---- router -------------------------------------------------------------------
def test_router_topk_selection(gpu_lib, golden):
    # the reference's own exact-index test (test/test_moe_router.cpp:82-138)
    hid, gw, gb, k = cases.topk_selection_case()
    node = moe_router_node()
    node.set_config(6, k)
    out = node.compute_test(hid.reshape(1, 1, 4), gw, gb)
    assert out.shape == (1, 1, 3, 2)
    assert list(out[0, 0, :, 0].astype(int)) == [5, 4, 3]
    assert np.allclose(out[..., 1], golden["topk_selection"][..., 1].reshape(1, 1, 3), atol=1e-6)


def test_router_basic_properties(gpu_lib):
    # the reference's Basic / WeightNormalization tests (test/test_moe_router.cpp:24-79, 206-251)
    rng = np.random.default_rng(42)
    hid = rng.uniform(-1, 1, (1, 2, 4)).astype(np.float32)
    gw = rng.uniform(-1, 1, (8, 4)).astype(np.float32)
    node = moe_router_node()
    node.set_config(8, 2)
    out = node.compute_test(hid, gw, np.zeros(8, np.float32))
    assert out.shape == (1, 2, 2, 2)
    assert np.all(out[..., 0] >= 0) and np.all(out[..., 0] < 8) and np.all(out[..., 1] > 0)
    assert np.allclose(out[..., 1].sum(-1), 1.0, atol=1e-5)


def test_router_golden_bit_exact_indices(gpu_lib, golden, port):
    hid, gw, rb = cases.router16_case()
    node = moe_router_node()
    node.set_config(32, 4)
    for key, bias in (("router16", rb), ("router16_nobias", None)):
        out = node.compute_test(hid.reshape(2, 8, 128), gw, bias).reshape(16, 4, 2)
        assert same_experts(out, golden[key])
        assert np.allclose(out[..., 1], golden[key][..., 1], atol=1e-6)
    node.set_sigmoid_gating(True)
    out = node.compute_test(hid.reshape(2, 8, 128), gw, rb).reshape(16, 4, 2)
    assert same_experts(out, golden["router16_sigmoid"])
    assert np.allclose(out[..., 1], golden["router16_sigmoid"][..., 1], atol=1e-6)


def test_router_logits_bit_exact_vs_restatement(gpu_lib, port):
    """Indices for every token of a 128-expert, H=2880 router over 512 tokens."""
    sh = synth.C2.with_(tokens=512)
    hid, Wg, rb = synth.hidden_states(sh), synth.router_weight(sh), synth.router_bias(sh)
    lay = MoeLayer(sh.num_experts, sh.top_k, sh.hidden, 32, has_bias=False, max_tokens=512)
    lay.set_router(Wg, rb)
    got = lay.route(hid)
    want = port.router(hid, Wg, rb, sh.top_k)
    assert same_experts(got, want)
    assert np.allclose(got[..., 1], want[..., 1], atol=2e-6)
    lay.close()


def test_router_errors(gpu_lib):
    node = moe_router_node()
    node.set_config(8, 2)
    with pytest.raises(RuntimeError, match="must be 3D"):
        node.compute_test(np.zeros((2, 4), np.float32), np.zeros((8, 4), np.float32))
    with pytest.raises(RuntimeError, match="shape mismatch"):
        node.compute_test(np.zeros((1, 2, 4), np.float32), np.zeros((7, 4), np.float32))
    with pytest.raises(RuntimeError, match="gate_bias must have"):
        node.compute_test(np.zeros((1, 2, 4), np.float32), np.zeros((8, 4), np.float32), np.zeros(3, np.float32))


# ---- expert MLP -----------------------------------------------------------------
def test_expert_single_token_vs_reference_call(gpu_lib, port):
    """expert_mlp_node::compute_test_mxfp4: one token through one expert."""
    for H, F, act, bias in ((64, 64, 0, True), (96, 160, 1, False), (2880, 2880, 0, True), (2048, 768, 1, False)):
        sh = synth.tiny(seed=31, E=1, k=1, H=H, F=F, T=1, has_bias=bias, act=act)
        x = synth.hidden_states(sh)[0]
        w = synth.expert_weights(sh, 0)
        node = expert_mlp_node(0)
        node.set_activation_type(act)
        got = node.compute_test_mxfp4(x, w["w_up"], w["w_gate"], w["w_down"], w["b_up"], w["b_gate"],
                                      w["b_down"], H, F)
        want = port.expert_token(x, w["w_up"], w["w_gate"], w["w_down"], w["b_up"], w["b_gate"],
                                 w["b_down"], H, F, act)
        assert_close(got, want, f"H={H} F={F}")


def test_modified_swiglu_point(gpu_lib):
    """The reference's only value check of the activation (test/test_expert_mlp.cpp:118-200):
    gate = 1.0 and up = 1.5 on every feature."""
    H = F = 64
    # one non-zero weight per row: code 2 (value 1.0 at scale 2^0 -> e = 127) for gate, 3 (1.5) for up
    def rows(code):
        m = np.zeros((F, H // 32, 17), np.uint8)
        m[:, :, 0] = 127
        m[:, 0, 1] = code
        return m.reshape(-1)
    w_down = np.zeros((H, F // 32, 17), np.uint8)
    w_down[:, :, 0] = 127
    for o in range(H):
        j = o % 32
        w_down[o, o // 32, 1 + (j & 15)] = 2 if j < 16 else (2 << 4)   # identity matrix
    x = np.zeros(H, np.float32)
    x[0] = 1.0
    node = expert_mlp_node(0)
    got = node.compute_test_mxfp4(x, rows(3), rows(2), w_down.reshape(-1), None, None, None, H, F)
    g, u = 1.0, 1.5
    want = g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)
    # the reference checks this point to 1e-3 on its fp16-weight path; the activation is stored
    # as fp16 here (2.1 * 2^-11 = 1.0e-3 of rounding), hence 2e-3
    assert np.allclose(got, want, atol=2e-3)


@pytest.mark.parametrize("tag", list(cases.TINY_CASES))
def test_tiny_layers(gpu_lib, golden, tag):
    sh, h, Wg, rb, ex, wbf = cases.tiny_case(tag)
    lay = make_layer(sh, Wg, rb, ex, wbf)
    out, ro = lay.forward(h)
    assert same_experts(ro, golden[f"{tag}_router"])
    assert np.allclose(ro[..., 1], golden[f"{tag}_router"][..., 1], atol=2e-6)
    assert_close(out, golden[f"{tag}_out"], tag)
    # per-expert nodes: dense output with zero rows, or the empty tensor
    nodes = []
    for e in range(sh.num_experts):
        o = lay.expert_forward(e, h, golden[f"{tag}_router"])
        assert (o is not None) == bool(golden[f"{tag}_selected"][e])
        if o is not None:
            picked = (golden[f"{tag}_router"][:, :, 0].astype(int) == e).any(axis=1)
            assert np.all(o[~picked] == 0.0)
            if picked.sum() > 1:
                assert_close(o[picked], golden[f"{tag}_nodes"][e][picked], f"{tag} expert {e}")
        nodes.append(o)
    # merge of reference node outputs: pure fp32 multiply-adds in router order -> bit-exact
    ref_nodes = [golden[f"{tag}_nodes"][e] if golden[f"{tag}_selected"][e] else None
                 for e in range(sh.num_experts)]
    merged = lay.merge(golden[f"{tag}_router"], ref_nodes)
    assert np.array_equal(merged, golden[f"{tag}_merge"])
    lay.close()


def test_tiny_layer_given_router_output(gpu_lib, golden):
    sh, h, Wg, rb, ex, wbf = cases.tiny_case("tiny_a")
    lay = make_layer(sh, Wg, rb, ex, wbf)
    out, ro = lay.forward(h, router_out=golden["tiny_a_router"])
    assert np.array_equal(ro, golden["tiny_a_router"])
    assert_close(out, golden["tiny_a_out"])
    lay.close()


def test_exponent_range(gpu_lib, port):
    """Scale exponents far outside the benchmark's [118,124]: dequantisation stays exact."""
    sh = synth.tiny(seed=41, E=4, k=2, H=128, F=128, T=6, has_bias=False)
    h, Wg, rb, ex = cases.layer_inputs(sh, router_scale=50.0, exp_lo=70, exp_hi=120)
    for e in range(4):
        ex["w_down"][e] = synth.mxfp4_matrix(sh.seed, synth._T_WDOWN, e, 128, 128, 120, 200)
    lay = make_layer(sh, Wg, rb, ex)
    lay.set_path(PATH_STREAM)
    out, ro = lay.forward(h)
    want, _ = port.moe_layer(h, Wg, rb, ex, 2, sh.act, router_out=ro)
    assert np.all(np.isfinite(want)) and np.any(want != 0)
    assert_close(out, want, "wide exponents")
    lay.close()


def test_c0_t1_and_t32(gpu_lib, golden, port):
    sh = synth.C0
    h, Wg, rb, ex = cases.layer_inputs(sh, 32)
    lay = make_layer(sh, Wg, rb, ex, max_tokens=32)
    out1, ro1 = lay.forward(h[:1])
    assert same_experts(ro1, golden["c0_t1_router"])
    assert_close(out1, golden["c0_t1_out"], "c0 T=1")
    out32, ro32 = lay.forward(h)
    assert same_experts(ro32, golden["c0_t32_router"])
    assert_close(out32[:4], golden["c0_t32_out_first4"], "c0 T=32 first rows")
    rms = golden["c0_t32_out_rms"]
    assert np.max(np.abs(out32.astype(np.float64).sum(1) - golden["c0_t32_out_rowsum"])) < 0.5 * rms
    # whole output against the restatement run here
    want, _ = port.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, nthreads=8, router_out=ro32)
    mx, mr = assert_close(out32, want, "c0 T=32")
    rows, distinct, wbytes = lay.counters()
    assert rows.sum() == 32 * 4 and distinct == (rows > 0).sum()
    assert wbytes == distinct * (sh.mxfp4_bytes_per_expert + sh.bias_bytes_per_expert)
    lay.close()


def test_c4_shape(gpu_lib, golden):
    sh, h, Wg, rb, ex = cases.c4x8_case()
    lay = make_layer(sh, Wg, rb, ex)
    out, ro = lay.forward(h)
    assert same_experts(ro, golden["c4x8_router"])
    assert_close(out, golden["c4x8_out"], "qwen-shaped")
    lay.close()


def test_many_rows_one_expert_and_ragged(gpu_lib, port):
    """Skewed routing: one expert takes most rows, some take none (row tiles of several heights)."""
    sh = synth.tiny(seed=51, E=8, k=2, H=192, F=224, T=300, has_bias=True)
    h, Wg, rb, ex = cases.layer_inputs(sh, router_scale=40.0)
    rb = rb.copy()
    rb[0] += 60.0     # expert 0 nearly always wins a slot
    rb[5:] -= 50.0    # experts 5..7 never selected
    lay = make_layer(sh, Wg, rb, ex, max_tokens=300)
    out, ro = lay.forward(h)
    want_ro = port.router(h, Wg, rb, 2)
    assert same_experts(ro, want_ro)
    rows, distinct, _ = lay.counters()
    assert rows[0] > 250 and rows[5:].sum() == 0 and rows.sum() == 600
    want, _ = port.moe_layer(h, Wg, rb, ex, 2, sh.act, nthreads=8, router_out=ro)
    assert_close(out, want, "skewed")
    for path in (PATH_STREAM, PATH_TILE, PATH_TILE_PAIR):
        lay.set_path(path)
        out2, _ = lay.forward(h, router_out=ro)
        assert_close(out2, want, f"skewed path {path}")
    lay.close()


# ---- error behaviour ---------------------------------------------------------------
def test_errors_are_values_not_crashes(gpu_lib):
    sh, h, Wg, rb, ex, wbf = cases.tiny_case("tiny_a")
    lay = MoeLayer.from_shape(sh, max_tokens=4)
    with pytest.raises(CskError, match="router weights were never set"):
        lay.forward(h)
    lay.set_router(Wg, rb)
    with pytest.raises(CskError, match="not loaded"):
        lay.forward(h)                      # experts missing
    assert lay._lib.csk_moe_expert_resident(lay._h, 0) == 0
    lay.load_experts(ex)
    with pytest.raises(CskError, match="max_tokens"):
        lay.forward(np.zeros((5, sh.hidden), np.float32))
    bad = np.zeros((3, 2, 2), np.float32)
    bad[0, 0, 0] = 99
    with pytest.raises(CskError, match="out of range"):
        lay.forward(h, router_out=bad)
    with pytest.raises(CskError):
        lay.load_expert(17, ex["w_up"][0], ex["w_gate"][0], ex["w_down"][0])
    out, _ = lay.forward(h)                 # the handle is still usable after every error
    assert np.all(np.isfinite(out))
    lay.close()


def test_merge_node_errors(gpu_lib):
    node = expert_merge_node()
    node.set_config(2, 1)
    ro = np.array([[[[0.0, 1.0]]]], np.float32)
    with pytest.raises(RuntimeError, match="expected 3 inputs"):
        node.compute_test([ro, np.zeros((1, 1, 32), np.float32)])
    with pytest.raises(RuntimeError, match="no non-empty"):
        node.compute_test([ro, np.zeros((0,), np.float32), np.zeros((0,), np.float32)])
    ro_bad = np.array([[[[5.0, 1.0]]]], np.float32)
    with pytest.raises(RuntimeError, match="out of range"):
        node.compute_test([ro_bad, np.zeros((1, 1, 32), np.float32), np.zeros((1, 1, 32), np.float32)])
    y = np.arange(32, dtype=np.float32).reshape(1, 1, 32)
    ro2 = np.array([[[[1.0, 0.25]]]], np.float32)
    out = node.compute_test([ro2, np.zeros((0,), np.float32), y])
    assert np.array_equal(out, 0.25 * y)


def test_expert_node_empty_and_dense(gpu_lib, golden):
    sh, h, Wg, rb, ex, wbf = cases.tiny_case("tiny_b")
    ro = golden["tiny_b_router"]
    sel = golden["tiny_b_selected"]
    e_empty = int(np.argmin(sel)) if not sel.all() else None
    e_dense = int(np.argmax(sel))
    node = expert_mlp_node(e_dense)
    node.set_activation_type(expert_mlp_node.activation_type.STANDARD_SWIGLU)
    out = node.compute_with_mxfp4(h.reshape(1, *h.shape), *cases.expert_args(ex, e_dense),
                                  ro.reshape(1, *ro.shape), sh.ffn)
    assert out.shape == (1, sh.tokens, sh.hidden)
    picked = (ro[:, :, 0].astype(int) == e_dense).any(axis=1)
    assert np.all(out[0][~picked] == 0)
    assert_close(out[0][picked], golden["tiny_b_nodes"][e_dense][picked])
    if e_empty is not None:
        node = expert_mlp_node(e_empty)
        out = node.compute_with_mxfp4(h.reshape(1, *h.shape), *cases.expert_args(ex, e_empty),
                                      ro.reshape(1, *ro.shape), sh.ffn)
        assert out.shape == (0,)
    with pytest.raises(RuntimeError, match="must be 3D"):
        node.compute_with_mxfp4(h, *cases.expert_args(ex, 0), ro.reshape(1, *ro.shape), sh.ffn)


# ---- the tensor-core (tcgen05) kernel, forced --------------------------------------
TILE_KERNELS = [pytest.param(PATH_TILE, id="one_cta"), pytest.param(PATH_TILE_PAIR, id="cta_pair")]


@pytest.mark.parametrize("tile", TILE_KERNELS)
@pytest.mark.parametrize("tag", list(cases.TINY_CASES))
def test_tile_path_tiny_layers(gpu_lib, golden, tag, tile):
    sh, h, Wg, rb, ex, wbf = cases.tiny_case(tag)
    lay = make_layer(sh, Wg, rb, ex, wbf)
    lay.set_path(tile)
    out, ro = lay.forward(h)
    assert lay.timings()["path"] == PATH_TILE
    assert same_experts(ro, golden[f"{tag}_router"])
    assert_close(out, golden[f"{tag}_out"], tag)
    for e in range(sh.num_experts):
        o = lay.expert_forward(e, h, golden[f"{tag}_router"])
        assert (o is not None) == bool(golden[f"{tag}_selected"][e])
        if o is not None:
            picked = (golden[f"{tag}_router"][:, :, 0].astype(int) == e).any(axis=1)
            assert np.all(o[~picked] == 0.0)
            if picked.sum() > 1:
                assert_close(o[picked], golden[f"{tag}_nodes"][e][picked], f"{tag} expert {e}")
    lay.close()


@pytest.mark.parametrize("tile", TILE_KERNELS)
def test_tile_path_c0(gpu_lib, golden, port, tile):
    sh = synth.C0
    h, Wg, rb, ex = cases.layer_inputs(sh, 32)
    lay = make_layer(sh, Wg, rb, ex, max_tokens=32)
    lay.set_path(tile)
    out1, ro1 = lay.forward(h[:1])
    assert_close(out1, golden["c0_t1_out"], "c0 T=1 tile")
    out32, ro32 = lay.forward(h)
    assert same_experts(ro32, golden["c0_t32_router"])
    assert_close(out32[:4], golden["c0_t32_out_first4"], "c0 T=32 tile")
    want, _ = port.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, nthreads=8, router_out=ro32)
    assert_close(out32, want, "c0 T=32 tile, all rows")
    lay.close()


def test_tile_path_wide_exponents(gpu_lib, port):
    """Scale exponents spread over 37 binades inside one matrix stay exact in the fp16 tile.
    (Gate/up scales are kept small so the pre-activations stay near the clamp range: with
    weights in the thousands a 16-bit input row alone moves pre-activations by whole units.)"""
    sh = synth.tiny(seed=43, E=4, k=2, H=128, F=128, T=200, has_bias=False)
    h, Wg, rb, ex = cases.layer_inputs(sh, router_scale=50.0, exp_lo=84, exp_hi=120)
    for e in range(4):
        ex["w_down"][e] = synth.mxfp4_matrix(sh.seed, synth._T_WDOWN, e, 128, 128, 100, 136)
    lay = make_layer(sh, Wg, rb, ex, max_tokens=200)
    want = None
    for path in (PATH_TILE, PATH_TILE_PAIR, PATH_STREAM):
        lay.set_path(path)
        out, ro = lay.forward(h)
        if want is None:
            want, _ = port.moe_layer(h, Wg, rb, ex, 2, sh.act, nthreads=8, router_out=ro)
        assert_close(out, want, f"wide exponents, path {path}")
    lay.close()


def test_edge_scale_bytes(gpu_lib, port):
    """Scale bytes 0, 1, 2 (the reference reads 0 and 1 as fp32 subnormals, gguf_dequant.h:419-433) on
    blocks with arbitrary codes, and 254 / 255 on blocks of zero codes (zero under any scale; with
    non-zero codes the reference's own fp32 weights overflow there), scattered over every matrix of
    every expert: both kernels must match the checker, and the repack must return the bytes unchanged."""
    sh = synth.tiny(seed=47, E=4, k=2, H=128, F=192, T=150, has_bias=True)
    h, Wg, rb, ex = cases.layer_inputs(sh, router_scale=50.0)
    rng = np.random.default_rng(470)
    for name in ("w_up", "w_gate", "w_down"):
        for e in range(sh.num_experts):
            blocks = ex[name][e].reshape(-1, 17).copy()
            pick = rng.choice(blocks.shape[0], size=blocks.shape[0] // 8, replace=False)
            for i, b in enumerate(pick):
                kind = i % 5
                blocks[b, 0] = (0, 1, 2, 254, 255)[kind]
                if kind >= 3:
                    blocks[b, 1:] = 0
            ex[name][e] = blocks.reshape(-1)
    lay = make_layer(sh, Wg, rb, ex, max_tokens=sh.tokens)
    for which, name in enumerate(("w_up", "w_gate", "w_down", "w_up", "w_gate", "w_down")):
        want_blocks = ex[name][1].reshape(-1, 17).copy()
        if which < 3:
            want_blocks[want_blocks[:, 0] == 255, 0] = 254   # the streaming layout stores 255 as what it is read as
        assert np.array_equal(lay.unpack_expert(1, which), want_blocks.reshape(-1)), which
    want = None
    for path in (PATH_STREAM, PATH_TILE, PATH_TILE_PAIR):
        lay.set_path(path)
        out, ro = lay.forward(h)
        if want is None:
            want, _ = port.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, nthreads=8, router_out=ro)
            assert np.all(np.isfinite(want)) and np.any(want != 0)
        assert np.all(np.isfinite(out)), path
        assert_close(out, want, f"edge scale bytes, path {path}")
    lay.close()


@pytest.mark.parametrize("tile", TILE_KERNELS)
def test_bounded_wait_runs_out_and_the_handle_recovers(gpu_lib, port, tile):
    """The failure path of the tensor-core kernel, made to happen without any fault: the wait budget is
    cut to 0.1 ms and the next launch's copy role is told to issue nothing, so the MMA, dequantiser and
    epilogue roles all wait on barriers that nothing arms, give up, tear down (tensor memory freed) and
    the call returns CSK_ERR_DEVICE.  The same handle then computes the layer correctly."""
    sh = synth.tiny(seed=49, E=4, k=2, H=128, F=128, T=96, has_bias=True)
    h, Wg, rb, ex = cases.layer_inputs(sh, router_scale=50.0)
    lay = make_layer(sh, Wg, rb, ex, max_tokens=sh.tokens)
    lay.set_path(tile)
    good, ro = lay.forward(h)
    try:
        lay.debug_set(lay.DEBUG_WAIT_BUDGET, 200_000)
        lay.debug_set(lay.DEBUG_STALL_TILE_PRODUCER, 1)
        with pytest.raises(CskError) as err:
            lay.forward(h)
        assert err.value.code == -3 and "wait ran out" in str(err.value)
    finally:
        lay.debug_set(lay.DEBUG_WAIT_BUDGET, 2_000_000_000)
    again, ro2 = lay.forward(h)
    assert np.array_equal(ro, ro2) and np.array_equal(good, again)
    want, _ = port.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, nthreads=8, router_out=ro)
    assert_close(again, want, "after the aborted call")
    lay.close()


@pytest.mark.parametrize("shape", ["tiny", "c0"])
def test_block_with_norm_and_residual(gpu_lib, port, shape):
    """x -> rmsnorm -> router -> experts -> merge -> + x as one call: the normed rows equal the reference's
    bit for bit (so the routing does), the result equals x + the checker's layer output on those rows."""
    if shape == "tiny":
        sh = synth.tiny(seed=51, E=8, k=2, H=256, F=192, T=70, has_bias=True)
        h, Wg, rb, ex = cases.layer_inputs(sh, router_scale=30.0)
    else:
        sh = synth.C0
        h, Wg, rb, ex = cases.layer_inputs(sh)
    g = np.random.default_rng(510)
    x = (h * g.uniform(0.2, 5.0, size=(h.shape[0], 1))).astype(np.float32)     # rows of different scale
    nw = (1.0 + 0.1 * g.standard_normal(sh.hidden)).astype(np.float32)
    lay = make_layer(sh, Wg, rb, ex, max_tokens=x.shape[0])
    lay.set_ffn_norm(nw, 1e-5)
    for path in (PATH_STREAM, PATH_TILE):
        lay.set_path(path)
        out, ro = lay.block_forward(x)
        n = port.rmsnorm(x, nw, 1e-5)
        want_ro = port.router(n, Wg, rb, sh.top_k)
        assert np.array_equal(ro[..., 0], want_ro[..., 0]), "routing after the fused norm differs"
        want, _ = port.moe_layer(n, Wg, rb, ex, sh.top_k, sh.act, nthreads=16, router_out=ro)
        assert_close(out.astype(np.float64) - x, want, f"block, path {path}")
        # and the norm alone, through a layer whose router sees it: same rows as the plain entry point on n
        out2, ro2 = lay.forward(n)
        assert np.array_equal(ro2[..., 0], ro[..., 0])
        assert np.array_equal((x + out2).astype(np.float32), out)
    lay.close()


def test_block_with_shared_expert(gpu_lib, port):
    """The Llama-4 style block (llm_engine.cpp:714-777): x -> rmsnorm -> [routed experts -> merge] + [shared dense FFN]
    -> + x in one call.  Routing bit-exact after the fused norm; the result equals x + (layer + dense FFN) of the
    checker on the normed rows; with the bit-exact pieces it equals the sum of the separate entry points bit for bit."""
    sh = synth.tiny(seed=57, E=8, k=2, H=256, F=192, T=150, has_bias=True)
    h, Wg, rb, ex = cases.layer_inputs(sh, router_scale=30.0)
    g = np.random.default_rng(570)
    x_all = (h * g.uniform(0.2, 5.0, size=(h.shape[0], 1))).astype(np.float32)
    nw = (1.0 + 0.1 * g.standard_normal(sh.hidden)).astype(np.float32)
    _, gw, uw, dw, bg, bu, bd = cases.dense_ffn_case(H=256, F=320, T=1, bias=True, seed=571)
    lay = make_layer(sh, Wg, rb, ex, max_tokens=x_all.shape[0])
    lay.set_ffn_norm(nw, 1e-5)
    shared = MoeLayer(1, 1, 256, 320, activation=synth.STANDARD_SWIGLU, has_bias=True, max_tokens=x_all.shape[0],
                      weights_f16=True)
    shared.load_expert_f16(0, uw, gw, dw, bu, bg, bd)
    for T in (150, 5):      # the tensor-core kernel; the streaming kernel with its captured launch sequence
        x = x_all[:T]
        for rep in range(2):
            out, ro = lay.block_forward(x, shared=shared)
        n = port.rmsnorm(x, nw, 1e-5)
        want_ro = port.router(n, Wg, rb, sh.top_k)
        assert np.array_equal(ro[..., 0], want_ro[..., 0]), "routing after the fused norm differs"
        moe, _ = port.moe_layer(n, Wg, rb, ex, sh.top_k, sh.act, nthreads=16, router_out=ro)
        dense = port.dense_ffn(n, gw, uw, dw, bg, bu, bd)
        assert_close(out.astype(np.float64) - x, moe.astype(np.float64) + dense, f"block with shared expert, T={T}")
        # the same from the separate entry points, added in the reference's order: x + (merge + shared)
        out_moe, ro2 = lay.forward(n)
        out_sh = shared.dense_forward(n)
        assert np.array_equal(ro2[..., 0], ro[..., 0])
        assert np.array_equal((x + (out_moe + out_sh)).astype(np.float32), out)
    with pytest.raises(CskError, match="shared expert must be another layer"):
        lay.block_forward(x_all[:4], shared=lay)
    empty = MoeLayer(1, 1, 256, 320, activation=synth.STANDARD_SWIGLU, has_bias=False, max_tokens=8, weights_f16=True)
    with pytest.raises(CskError, match="not loaded"):
        lay.block_forward(x_all[:4], shared=empty)
    empty.close()
    shared.close()
    lay.close()


def test_bulk_load_and_weight_image(gpu_lib, port, tmp_path):
    """The model's [E, rows, cols] expert tensors loaded as slabs give the same layer as expert-by-expert
    loading, bit for bit; the repacked image written to a file and read into a fresh handle does too."""
    sh = synth.tiny(seed=53, E=6, k=2, H=128, F=160, T=40, has_bias=True)
    h, Wg, rb, ex = cases.layer_inputs(sh, router_scale=40.0)
    one = make_layer(sh, Wg, rb, ex, max_tokens=sh.tokens)
    want, want_ro = one.forward(h)
    slab = {n: np.stack(ex[n]) for n in ex}
    bulk = MoeLayer.from_shape(sh, max_tokens=sh.tokens)
    bulk.set_router(Wg, rb)
    bulk.load_experts_bulk(0, slab["w_up"][:4], slab["w_gate"][:4], slab["w_down"][:4], slab["b_up"][:4],
                           slab["b_gate"][:4], slab["b_down"][:4])
    assert bulk.expert_resident(3) and not bulk.expert_resident(4)
    bulk.load_experts_bulk(4, slab["w_up"][4:], slab["w_gate"][4:], slab["w_down"][4:], slab["b_up"][4:],
                           slab["b_gate"][4:], slab["b_down"][4:])
    for which in range(6):
        assert np.array_equal(bulk.unpack_expert(5, which), one.unpack_expert(5, which))
    got, ro = bulk.forward(h)
    assert np.array_equal(ro, want_ro) and np.array_equal(got, want)
    img = tmp_path / "layer.img"
    bulk.save_image(img)
    fresh = MoeLayer.from_shape(sh, max_tokens=sh.tokens)
    fresh.set_router(Wg, rb)
    fresh.load_image(img)
    got2, _ = fresh.forward(h)
    assert np.array_equal(got2, want)
    other = MoeLayer.from_shape(sh.with_(ffn=192), max_tokens=8)
    with pytest.raises(CskError):
        other.load_image(img)
    for lay in (one, bulk, fresh, other):
        lay.close()
