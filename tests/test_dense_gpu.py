"""The shared expert's dense FFN (dense_ffn_node.h:28-219) and fp16 expert weights on the tensor-core kernel,
against the CPU restatement of the reference (pinned bit for bit against the compiled reference on CPU)."""
from __future__ import annotations

import numpy as np
import pytest

from coalsack_b200 import CskError, MoeLayer, PATH_STREAM, PATH_TILE_PAIR, dense_ffn_node, synth
from tests import cases

pytestmark = pytest.mark.gpu


def assert_close(got, want, what):
    mx, mr = cases.err_stats(got, want)
    assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (what, mx, mr)


@pytest.mark.parametrize("tag,bias", [("dense_b", True), ("dense_nb", False)])
def test_dense_ffn_golden(gpu_lib, golden, tag, bias):
    hidden, gw, uw, dw, bg, bu, bd = cases.dense_ffn_case(bias=bias)
    node = dense_ffn_node()
    inputs = [hidden[None], gw, uw, dw] + ([bg, bu, bd] if bias else [])
    out = node.compute(inputs)
    assert out.shape == (1,) + hidden.shape and out.dtype == np.float32
    assert_close(out[0], golden[tag + "_out"], tag)
    # one row at a time gives the same rows (a row's value does not depend on its batch)
    one = node.compute([hidden[None, :1]] + inputs[1:])
    assert np.array_equal(one[0, 0], out[0, 0])
    node.close()


def test_dense_ffn_gptoss_shape_and_determinism(gpu_lib, port):
    """2880 x 2880, 8192 rows (43 row tiles of one weight set): a seeded sample of rows against the
    restatement, and thirty repeats equal bit for bit (a ring whose stages alternate between the two
    dequantiser groups once let a late copy be mistaken for the one before it: found by this check)."""
    H = F = 2880
    T = 8192
    hidden, gw, uw, dw, bg, bu, bd = cases.dense_ffn_case(H=H, F=F, T=T, bias=True, seed=79)
    node = dense_ffn_node()
    inputs = [hidden[None], gw, uw, dw, bg, bu, bd]
    first = node.compute(inputs)
    pick = np.sort(np.random.default_rng(5).choice(T, size=48, replace=False))
    want = port.dense_ffn(hidden[pick], gw, uw, dw, bg, bu, bd)
    assert_close(first[0][pick], want, "dense 2880x2880")
    assert np.all(np.isfinite(first))
    for rep in range(30):
        again = node.compute(inputs)
        assert np.array_equal(first, again), f"repeat {rep} differs in {int((first != again).any(axis=2).sum())} rows"
    node.close()


def test_dense_ffn_ragged_sizes(gpu_lib, port):
    """Sizes that are multiples of 32 but not of the tile sizes (64 columns, 128/256 weight rows), odd row counts."""
    for H, F, T in ((96, 160, 1), (160, 96, 193), (352, 288, 385)):
        hidden, gw, uw, dw, bg, bu, bd = cases.dense_ffn_case(H=H, F=F, T=T, bias=True, seed=80 + T)
        node = dense_ffn_node()
        out = node.compute([hidden[None], gw, uw, dw, bg, bu, bd])
        assert_close(out[0], port.dense_ffn(hidden, gw, uw, dw, bg, bu, bd), (H, F, T))
        node.close()


def test_dense_ffn_fp32_weights(gpu_lib, golden, port):
    """FLOAT32 weights (the reference's scalar path): rounded to fp16 on the device, inside the stated tolerance of
    the reference's fp32 arithmetic; a weight beyond the fp16 range is refused."""
    args = cases.dense_ffn_case_f32()
    hidden = args[0]
    node = dense_ffn_node()
    out = node.compute([hidden[None]] + list(args[1:]))
    assert_close(out[0], golden["dense32_out"], "dense fp32 weights")
    node.close()
    hidden, gw, uw, dw, _, _, _ = cases.dense_ffn_case_f32(H=352, F=288, T=200, bias=False, seed=179)
    node = dense_ffn_node()
    out = node.compute([hidden[None], gw, uw, dw])
    assert_close(out[0], port.dense_ffn(hidden, gw, uw, dw), "dense fp32 weights, no bias")
    node.close()
    big = gw.copy()
    big[3, 5] = 1.0e5
    node = dense_ffn_node()
    with pytest.raises(CskError, match="beyond the fp16 range"):
        node.compute([hidden[None], big, uw, dw])
    node.close()
    with pytest.raises(RuntimeError, match="all be FLOAT16 or all FLOAT32"):
        dense_ffn_node().compute([hidden[None], gw, uw.astype(np.float16), dw])


def test_dense_ffn_errors(gpu_lib):
    hidden, gw, uw, dw, bg, bu, bd = cases.dense_ffn_case()
    node = dense_ffn_node()
    with pytest.raises(RuntimeError, match="expected 4 or 7 inputs"):
        node.compute([hidden[None], gw, uw])
    with pytest.raises(RuntimeError, match="hidden_states must be 3D"):
        node.compute([hidden, gw, uw, dw])
    with pytest.raises(RuntimeError, match="weight tensors must be 2D"):
        node.compute([hidden[None], gw.reshape(-1), uw, dw])
    with pytest.raises(RuntimeError, match="down_w shape mismatch"):
        node.compute([hidden[None], gw, uw, dw.T.copy()])
    with pytest.raises(RuntimeError, match="gate_w/up_w shape mismatch"):
        node.compute([hidden[None], gw, uw[:-32], dw])
    with pytest.raises(RuntimeError, match="FLOAT16"):
        node.compute([hidden[None], gw.astype(np.float64), uw.astype(np.float64), dw.astype(np.float64)])
    # the two weight formats do not mix, and fp16 layers have the one-CTA tensor-core kernel only
    lay = MoeLayer(1, 1, 256, 192, activation=1, has_bias=False, max_tokens=16, weights_f16=True)
    with pytest.raises(CskError, match="fp16 weights"):
        lay.load_expert(0, np.zeros(256 * 192 // 32 * 17, np.uint8), np.zeros(256 * 192 // 32 * 17, np.uint8),
                        np.zeros(256 * 192 // 32 * 17, np.uint8))
    for path in (PATH_STREAM, PATH_TILE_PAIR):
        with pytest.raises(CskError, match="fp16 weights"):
            lay.set_path(path)
    with pytest.raises(CskError, match="not loaded"):
        lay.dense_forward(hidden)
    lay.close()
    mx = MoeLayer(4, 2, 256, 192, max_tokens=16)
    with pytest.raises(CskError, match="MXFP4 weights"):
        mx.load_expert_f16(0, uw, gw, dw)
    with pytest.raises(CskError, match="num_experts = top_k = 1"):
        mx.dense_forward(hidden)
    mx.close()


def test_moe_layer_with_fp16_experts(gpu_lib, port):
    """Routed experts with fp16 weights (the reference dequantises Q4_K / Q6_K expert slices to fp16,
    expert_mlp_node.h:533-647): router by the library, each selected expert's rows by the dense
    restatement, merged in router order."""
    E, k, H, F, T = 6, 2, 256, 192, 150
    rng = np.random.default_rng(91)
    hidden = rng.standard_normal((T, H)).astype(np.float32)
    Wg = (rng.standard_normal((E, H)) * 0.3).astype(np.float32)
    experts = [cases.dense_ffn_case(H=H, F=F, T=1, bias=True, seed=200 + e)[1:] for e in range(E)]
    lay = MoeLayer(E, k, H, F, activation=synth.STANDARD_SWIGLU, has_bias=True, max_tokens=T, weights_f16=True)
    lay.set_router(Wg, None)
    for e, (gw, uw, dw, bg, bu, bd) in enumerate(experts):
        lay.load_expert_f16(e, uw, gw, dw, bu, bg, bd)
    out, ro = lay.forward(hidden)
    want_ro = port.router(hidden, Wg, None, k)
    assert np.array_equal(ro[..., 0], want_ro[..., 0])
    dense = [port.dense_ffn(hidden, *experts[e]) for e in range(E)]
    want = np.zeros((T, H), np.float32)
    for t in range(T):
        for j in range(k):
            e, w = int(ro[t, j, 0]), np.float32(ro[t, j, 1])
            want[t] = want[t] + w * dense[e][t]
    assert_close(out, want, "fp16 experts")
    rows, distinct, _ = lay.counters()
    assert rows.sum() == T * k
    lay.close()
