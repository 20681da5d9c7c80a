"""Q4_K / Q6_K expert slices decoded on the device (the weight provider's host conversion,
src/llm/moe_weight_provider.cpp:17-33, 134-159): fp16 bit patterns against the fixture the reference produced
and against the CPU restatement, and a layer loaded from raw blocks against the same layer loaded from the
restatement's fp16 values."""
from __future__ import annotations

import numpy as np
import pytest

from coalsack_b200 import (CskError, GGML_F16, GGML_Q4_K, GGML_Q6_K, MoeLayer, dequant_ggml_f16, synth)
from tests import cases

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,t", [("q4k", GGML_Q4_K), ("q6k", GGML_Q6_K)])
def test_kquant_decode_bit_exact(gpu_lib, golden, port, name, t):
    for kind, wild in (("", False), ("_wild", True)):
        blocks = cases.kquant_blocks(t, 48, 61 + t, wild)
        assert cases.crc(blocks) == golden[f"{name}{kind}_crc"]
        got = dequant_ggml_f16(t, blocks, 48 * 256)
        assert np.array_equal(got.view(np.uint16), golden[f"{name}{kind}_f16"]), (name, kind)
    # a slice of the 2880 x 2880 expert (32400 super-blocks), both roundings, arbitrary headers in a second pass
    nb = 2880 * 2880 // 256
    for wild in (False, True):
        blocks = cases.kquant_blocks(t, nb, 11, wild)
        for nearest in (False, True):
            got = dequant_ggml_f16(t, blocks, nb * 256, nearest=nearest)
            want = port.dequant_kquant(t, blocks, nb * 256, nearest=nearest)
            if nearest:
                # NaN payloads are not part of the contract in this rounding
                nan = np.isnan(want)
                assert np.array_equal(np.isnan(got), nan)
                assert np.array_equal(got.view(np.uint16)[~nan], want.view(np.uint16)[~nan]), (name, wild)
            else:
                assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), (name, wild)


def test_kquant_decode_errors(gpu_lib):
    with pytest.raises(CskError, match="multiple of 256"):
        dequant_ggml_f16(GGML_Q4_K, np.zeros(144, np.uint8), 255)
    with pytest.raises(CskError, match="not handled"):
        dequant_ggml_f16(13, np.zeros(176, np.uint8), 256)
    with pytest.raises(RuntimeError, match="expected 288 bytes"):
        dequant_ggml_f16(GGML_Q4_K, np.zeros(144, np.uint8), 512)


def test_layer_loaded_from_kquant_blocks(gpu_lib, port):
    """Experts whose up/gate slices are Q4_K and whose down slice is Q6_K (one expert keeps an F16 down slice):
    the layer's output equals, bit for bit, that of a layer given the fp16 values the restatement decodes."""
    E, k, H, F, T = 5, 2, 256, 192, 70
    rng = np.random.default_rng(123)
    hidden = rng.standard_normal((T, H)).astype(np.float32)
    Wg = (rng.standard_normal((E, H)) * 0.3).astype(np.float32)
    nb = H * F // 256
    raw, vals, biases = [], [], []
    for e in range(E):
        up = cases.kquant_blocks(GGML_Q4_K, nb, 400 + e, scale=0.0005)
        gate = cases.kquant_blocks(GGML_Q4_K, nb, 500 + e, scale=0.0005)
        if e == 3:
            down_t, down = GGML_F16, (rng.standard_normal((H, F)) * 0.05).astype(np.float16)
            down_v = down
        else:
            down_t, down = GGML_Q6_K, cases.kquant_blocks(GGML_Q6_K, nb, 600 + e, scale=0.00005)
            down_v = port.dequant_kquant(GGML_Q6_K, down, H * F).reshape(H, F)
        raw.append(((GGML_Q4_K, up), (GGML_Q4_K, gate), (down_t, down)))
        vals.append((port.dequant_kquant(GGML_Q4_K, up, H * F).reshape(F, H),
                     port.dequant_kquant(GGML_Q4_K, gate, H * F).reshape(F, H), down_v))
        biases.append([(rng.standard_normal(n) * 0.01).astype(np.float32) for n in (F, F, H)])
    outs = []
    for mode in ("blocks", "values"):
        lay = MoeLayer(E, k, H, F, activation=synth.STANDARD_SWIGLU, has_bias=True, max_tokens=T, weights_f16=True)
        lay.set_router(Wg, None)
        for e in range(E):
            if mode == "blocks":
                lay.load_expert_ggml(e, *raw[e], *biases[e])
            else:
                lay.load_expert_f16(e, *vals[e], *biases[e])
        out, ro = lay.forward(hidden)
        outs.append(out)
        lay.close()
    assert np.all(np.isfinite(outs[0])) and np.abs(outs[0]).max() > 0
    assert np.array_equal(outs[0], outs[1])
    # and the values path itself against the CPU restatement of the expert math
    want_ro = port.router(hidden, Wg, None, k)
    dense = [port.dense_ffn(hidden, vals[e][1], vals[e][0], vals[e][2], biases[e][1], biases[e][0], biases[e][2])
             for e in range(E)]
    want = np.zeros((T, H), np.float32)
    for t in range(T):
        for j in range(k):
            want[t] = want[t] + np.float32(want_ro[t, j, 1]) * dense[int(want_ro[t, j, 0])][t]
    mx, mr = cases.err_stats(outs[0], want)
    assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (mx, mr)
    # state errors
    mxl = MoeLayer(4, 2, 256, 192, max_tokens=16)
    with pytest.raises(CskError, match="CSK_WEIGHTS_F16"):
        mxl.load_expert_ggml(0, *raw[0], *[None] * 3)
    mxl.close()
