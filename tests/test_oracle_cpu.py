"""The CPU checker itself: the plain-C restatement against the golden vectors
the unmodified reference produced, against the reference's own known-answer
tests, and (where the reference is compiled) against the reference directly."""
import numpy as np
import pytest

from coalsack_b200 import synth
from tests import cases


def test_e8m0_known_answers(port, golden):
    # reference test/test_gguf_dequant.cpp:266-280
    assert port.e8m0(127) == 0.5 and port.e8m0(128) == 1.0 and port.e8m0(129) == 2.0
    got = np.array([port.e8m0(x) for x in range(256)], np.float32)
    assert np.array_equal(got.view(np.uint32), golden["e8m0_all"].view(np.uint32))


def test_dequant_zero_block(port):
    # reference test/test_gguf_dequant.cpp:244-263
    blk = np.zeros(17, np.uint8)
    blk[0] = 128
    assert np.all(port.dequant(blk) == 0.0)


def test_dequant_golden(port, golden):
    got = port.dequant(cases.codec_blocks())
    assert np.array_equal(got.view(np.uint32), golden["codec_values"].view(np.uint32))
    # block 0 has scale 1 and every code once in the low nibbles: doubled E2M1 values
    assert list(got[:16]) == [0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12]


def test_router_topk_selection(port, golden):
    # reference test/test_moe_router.cpp:82-138: experts 5, 4, 3 in that order
    hid, gw, gb, k = cases.topk_selection_case()
    out = port.router(hid, gw, gb, k)
    assert list(out[0, :, 0].astype(int)) == [5, 4, 3]
    assert np.array_equal(out, golden["topk_selection"])


def test_router_golden(port, golden):
    hid, gw, rb = cases.router16_case()
    assert cases.crc(hid, gw, rb) == golden["router16_crc"], "synthetic generator drifted"
    for key, kw in (("router16", {}), ("router16_sigmoid", {"sigmoid": True})):
        out = port.router(hid, gw, rb, 4, **kw)
        assert np.array_equal(out, golden[key])
    out = port.router(hid, gw, None, 4)
    assert np.array_equal(out, golden["router16_nobias"])
    # reference test/test_moe_router.cpp:77,199: weights positive, summing to 1
    w = golden["router16"][..., 1]
    assert np.all(w > 0) and np.allclose(w.sum(-1), 1.0, atol=1e-5)


@pytest.mark.parametrize("tag", list(cases.TINY_CASES))
def test_tiny_layers_golden(port, golden, tag):
    sh, h, Wg, rb, ex, wbf = cases.tiny_case(tag)
    assert cases.inputs_crc(h, Wg, rb, ex) == golden[f"{tag}_crc"], "synthetic generator drifted"
    out, ro = port.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, weight_before_ffn=wbf)
    assert np.array_equal(ro, golden[f"{tag}_router"])
    assert np.array_equal(out, golden[f"{tag}_out"])
    nodes = []
    for e in range(sh.num_experts):
        o = port.expert_node(e, h, *cases.expert_args(ex, e), ro, sh.ffn, sh.act, wbf)
        assert (o is not None) == bool(golden[f"{tag}_selected"][e])
        if o is not None:
            assert np.array_equal(o, golden[f"{tag}_nodes"][e])
            # rows of tokens that did not pick the expert are exactly zero
            picked = (ro[:, :, 0].astype(int) == e).any(axis=1)
            assert np.all(o[~picked] == 0.0)
        nodes.append(o)
    merged = port.merge(ro, nodes, sh.hidden, wbf)
    assert np.array_equal(merged, golden[f"{tag}_merge"])
    # merging the per-expert node outputs equals the fused layer evaluation
    assert np.array_equal(merged, out)


def test_c0_golden(port, golden):
    sh = synth.C0
    h, Wg, rb, ex = cases.layer_inputs(sh, 32)
    assert cases.inputs_crc(h, Wg, rb, ex) == golden["c0_crc"], "synthetic generator drifted"
    out1, ro1 = port.moe_layer(h[:1], Wg, rb, ex, sh.top_k, sh.act, nthreads=4)
    assert np.array_equal(ro1, golden["c0_t1_router"])
    assert np.array_equal(out1, golden["c0_t1_out"])
    out4, ro4 = port.moe_layer(h[:4], Wg, rb, ex, sh.top_k, sh.act, nthreads=4)
    assert np.array_equal(ro4, golden["c0_t32_router"][:4])
    assert np.array_equal(out4, golden["c0_t32_out_first4"])


def test_c4_golden(port, golden):
    sh, h, Wg, rb, ex = cases.c4x8_case()
    assert cases.inputs_crc(h, Wg, rb, ex) == golden["c4x8_crc"], "synthetic generator drifted"
    out, ro = port.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, nthreads=4)
    assert np.array_equal(ro, golden["c4x8_router"])
    assert np.array_equal(out, golden["c4x8_out"])
    assert np.allclose(ro[..., 1].sum(-1), 1.0, atol=1e-5)


def test_merge_errors(port):
    ro = np.array([[[7.0, 1.0]]], np.float32)
    with pytest.raises(RuntimeError):
        port.merge(ro, [np.zeros((1, 32), np.float32)] * 2, 32)       # expert id out of range
    with pytest.raises(RuntimeError):
        port.merge(np.array([[[0.0, 1.0]]], np.float32), [None, None], 32)  # all inputs empty


def test_port_equals_reference_on_fresh_inputs(port, ref):
    """Bit-for-bit agreement with the compiled reference on inputs that are not in the fixtures."""
    sh = synth.tiny(seed=97, E=8, k=3, H=160, F=224, T=7, has_bias=True, act=synth.STANDARD_SWIGLU)
    h, Wg, rb, ex = cases.layer_inputs(sh, router_scale=30.0, exp_lo=90, exp_hi=150)
    a, ra = port.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act)
    b, rb_ = ref.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act)
    assert np.array_equal(ra, rb_) and np.array_equal(a, b)
    for x in (0, 1, 2, 254, 255):
        assert port.e8m0(x) == ref.e8m0(x)


def test_rmsnorm_golden_and_reference(port, golden):
    """The restated RMSNorm equals the reference's node output bit for bit (fixture), and the reference
    itself on fresh inputs where its compiled wrapper is present."""
    x, w = cases.rmsnorm_case()
    assert cases.crc(x, w) == golden["rmsnorm_crc"]
    assert np.array_equal(port.rmsnorm(x, w, 1e-5), golden["rmsnorm_out"])
    import oracle
    if oracle.have_ref():
        g = np.random.default_rng(7)
        x2 = g.standard_normal((9, 2880)).astype(np.float32)
        w2 = g.standard_normal(2880).astype(np.float32)
        assert np.array_equal(port.rmsnorm(x2, w2, 1e-6), oracle.ref().rmsnorm(x2, w2, 1e-6))


@pytest.mark.parametrize("tag,bias", [("dense_b", True), ("dense_nb", False)])
def test_dense_ffn_golden_and_reference(port, golden, tag, bias):
    """The restated dense FFN (dense_ffn_node, fp16 weights) equals the reference's node output bit for bit
    on the fixture, and the compiled reference itself on fresh inputs where its wrapper is present."""
    hidden, gw, uw, dw, bg, bu, bd = cases.dense_ffn_case(bias=bias)
    assert cases.crc(hidden, gw.view(np.uint16), uw.view(np.uint16), dw.view(np.uint16)) == golden[tag + "_crc"]
    assert np.array_equal(port.dense_ffn(hidden, gw, uw, dw, bg, bu, bd), golden[tag + "_out"])
    import oracle
    if oracle.have_ref():
        args = cases.dense_ffn_case(H=2880, F=96, T=3, bias=bias, seed=78)
        assert np.array_equal(port.dense_ffn(*args), oracle.ref().dense_ffn(*args))


def test_dense_ffn_fp32_weights_golden_and_reference(port, golden):
    """dense_ffn_node's FLOAT32-weight path (dense_ffn_node.h:121-149): restatement against the fixture and,
    where present, the compiled reference, bit for bit."""
    args = cases.dense_ffn_case_f32()
    assert cases.crc(*args[:4]) == golden["dense32_crc"]
    assert np.array_equal(port.dense_ffn(*args), golden["dense32_out"])
    import oracle
    if oracle.have_ref():
        args = cases.dense_ffn_case_f32(H=2880, F=96, T=3, bias=False, seed=178)
        assert np.array_equal(port.dense_ffn(*args), oracle.ref().dense_ffn(*args))


@pytest.mark.parametrize("name,t", [("q4k", cases.Q4_K), ("q6k", cases.Q6_K)])
def test_kquant_to_fp16_golden_and_reference(port, golden, name, t):
    """Q4_K / Q6_K expert slices to fp16 (moe_weight_provider.cpp:17-33): the restatement equals the fixture the
    reference produced bit for bit, ordinary and arbitrary headers; the compiled reference on fresh blocks;
    and, in the F16C rounding, an independent numpy statement of the layout rounded by numpy."""
    for kind, wild in (("", False), ("_wild", True)):
        blocks = cases.kquant_blocks(t, 48, 61 + t, wild)
        assert cases.crc(blocks) == golden[f"{name}{kind}_crc"]
        got = port.dequant_kquant(t, blocks, 48 * 256)
        assert np.array_equal(got.view(np.uint16), golden[f"{name}{kind}_f16"])
    import oracle
    if oracle.have_ref():
        for wild in (False, True):
            blocks = cases.kquant_blocks(t, 2048, 7, wild)
            assert np.array_equal(port.dequant_kquant(t, blocks, 2048 * 256).view(np.uint16),
                                  oracle.ref().dequant_kquant(t, blocks, 2048 * 256).view(np.uint16))
    blocks = cases.kquant_blocks(t, 1024, 9, True)
    with np.errstate(all="ignore"):
        want = cases.kquant_values_f32(t, blocks).astype(np.float16)
    got = port.dequant_kquant(t, blocks, 1024 * 256, nearest=True)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got.view(np.uint16)[~nan], want.view(np.uint16)[~nan])


def test_kquant_known_answers(port):
    """The known answers of the reference's own decoder tests (test/test_gguf_dequant.cpp:683-760: with d = 1,
    dmin = 0 and sub-block scales 1, 2, 4, 8 value 2 is 1 * (low nibble of byte 2) = 2 and value 32 is
    2 * (high nibble of byte 0) = 2; :396-445, 521-552: every value finite), and the truncating conversion:
    0.1 * 63 * 15 - 0.05 * 21 with fp16 headers."""
    b = np.zeros(144, np.uint8)
    b[0:2] = np.array([1.0], np.float16).view(np.uint8)
    b[4:8] = [1, 2, 4, 8]
    i = np.arange(128)
    b[16:] = (((i + 1) % 16) << 4) | (i % 16)
    v = port.dequant_kquant(cases.Q4_K, b, 256).astype(np.float32)
    assert v[2] == 2.0 and v[32] == 2.0 and v[0] == 0.0 and v[1] == 1.0
    assert np.array_equal(v[:32], (i[:32] % 16).astype(np.float32))
    assert np.array_equal(v[32:64], 2.0 * ((i[:32] + 1) % 16))
    b = np.zeros(144, np.uint8)
    b[0:2] = np.array([0.1], np.float16).view(np.uint8)
    b[2:4] = np.array([0.05], np.float16).view(np.uint8)
    b[4:16] = [0x3F, 0x80, 0xC5, 0x2A, 0x15, 0xF0, 0x88, 0x1F, 0xAA, 0x55, 0xCC, 0x33]
    val = ((i // 32) * 3 + (i % 32)) % 16
    b[16:] = val | ((15 - val) << 4)
    v = port.dequant_kquant(cases.Q4_K, b, 256)
    assert np.all(np.isfinite(v))
    d, dmin = np.float32(np.float16(0.1)), np.float32(np.float16(0.05))
    want = np.float32(np.float32(d * np.float32(63)) * np.float32(15)) - np.float32(dmin * np.float32(21))
    bits = np.array([want], np.float32).view(np.uint32)[0]
    trunc = np.uint16(((bits >> 16) & 0x8000) | ((((bits >> 23) & 0xFF) - 112) << 10) | ((bits >> 13) & 0x3FF))
    assert v.view(np.uint16)[15] == trunc        # value 15: low nibble 15 of byte 15, sub-block 0 (scale 63, min 21)
    b = np.zeros(210, np.uint8)
    b[0:128] = (np.arange(128) * 13) % 256
    b[128:192] = (np.arange(64) * 31) % 256
    b[192:208] = (((np.arange(16) * 11) % 128) - 64).astype(np.int8).view(np.uint8)
    b[208:210] = np.array([0.07], np.float16).view(np.uint8)
    v = port.dequant_kquant(cases.Q6_K, b, 256)
    assert np.all(np.isfinite(v))
    with np.errstate(all="ignore"):
        near = cases.kquant_values_f32(cases.Q6_K, b).astype(np.float16).astype(np.float32)
    assert np.all(np.abs(v.astype(np.float32) - near) <= np.abs(near) * 2.0 ** -10 + 1e-7)
    with pytest.raises(AssertionError):
        port.dequant_kquant(cases.Q4_K, np.zeros(144, np.uint8), 255)
