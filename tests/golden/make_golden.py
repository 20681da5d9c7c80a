"""Generates tests/golden/moe_golden.npz by running the UNMODIFIED reference
(oracle/_ref/libcsk_ref.so, built from the reference checkout by
oracle/Makefile) on seeded inputs.  Run from the repository root:

    make -C oracle && python tests/golden/make_golden.py

Inputs are not stored: they are regenerated from coalsack_b200.synth seeds; a
checksum of every input buffer is stored so that a drift of the generator is
caught instead of silently comparing different problems.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from coalsack_b200 import synth  # noqa: E402
from tests import cases  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "moe_golden.npz")


def main():
    r = oracle.ref()
    g = {}

    # codec (the reference's tests: test/test_gguf_dequant.cpp:244-280)
    g["e8m0_all"] = np.array([r.e8m0(x) for x in range(256)], np.float32)
    g["codec_values"] = r.dequant(cases.codec_blocks())

    # router known answer (test/test_moe_router.cpp:82-138): experts 5, 4, 3
    hid, gw, gb, k = cases.topk_selection_case()
    g["topk_selection"] = r.router(hid, gw, gb, k)

    # router at the size of the reference's 32-expert test (test/test_moe_router.cpp:141-203)
    hid, gw, rb = cases.router16_case()
    g["router16_crc"] = cases.crc(hid, gw, rb)
    g["router16"] = r.router(hid, gw, rb, 4)
    g["router16_sigmoid"] = r.router(hid, gw, rb, 4, sigmoid=True)
    g["router16_nobias"] = r.router(hid, gw, None, 4)

    for tag in cases.TINY_CASES:
        sh, h, Wg, rb, ex, wbf = cases.tiny_case(tag)
        g[f"{tag}_crc"] = cases.inputs_crc(h, Wg, rb, ex)
        out, ro = r.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, weight_before_ffn=wbf)
        g[f"{tag}_router"] = ro
        g[f"{tag}_out"] = out
        node_outs = [r.expert_node(e, h, *cases.expert_args(ex, e), ro, sh.ffn, sh.act, wbf)
                     for e in range(sh.num_experts)]
        g[f"{tag}_selected"] = np.array([o is not None for o in node_outs])
        g[f"{tag}_nodes"] = np.stack([o if o is not None else np.zeros_like(h) for o in node_outs])
        g[f"{tag}_merge"] = r.merge(ro, node_outs, sh.hidden, wbf)

    # gpt-oss-20b shaped layer (benchmark configuration 0): T = 1 and T = 32
    sh = synth.C0
    h, Wg, rb, ex = cases.layer_inputs(sh, 32)
    g["c0_crc"] = cases.inputs_crc(h, Wg, rb, ex)
    out1, ro1 = r.moe_layer(h[:1], Wg, rb, ex, sh.top_k, sh.act, nthreads=4)
    g["c0_t1_router"], g["c0_t1_out"] = ro1, out1
    out32, ro32 = r.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, nthreads=8)
    g["c0_t32_router"] = ro32
    g["c0_t32_out_first4"] = out32[:4]
    g["c0_t32_out_rms"] = np.float64(np.sqrt(np.mean(out32.astype(np.float64) ** 2)))
    g["c0_t32_out_rowsum"] = out32.astype(np.float64).sum(axis=1)

    # Qwen3-30B-A3B shaped experts (benchmark configuration 4), 8 of the 128
    # experts: top-8 routing with softmax over the selected, plain SwiGLU, no biases
    sh, h, Wg, rb, ex = cases.c4x8_case()
    g["c4x8_crc"] = cases.inputs_crc(h, Wg, rb, ex)
    out, ro = r.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, nthreads=4)
    g["c4x8_router"], g["c4x8_out"] = ro, out

    # the RMSNorm in front of the router (rmsnorm_node::compute_test, eps as graph_builder sets it)
    x, w = cases.rmsnorm_case()
    g["rmsnorm_out"] = r.rmsnorm(x, w, 1e-5)
    g["rmsnorm_crc"] = cases.crc(x, w)

    # the shared expert's dense FFN (dense_ffn_node::compute), fp16 weights, with and without biases
    for tag, bias in (("dense_b", True), ("dense_nb", False)):
        hidden, gw, uw, dw, bg, bu, bd = cases.dense_ffn_case(bias=bias)
        g[tag + "_out"] = r.dense_ffn(hidden, gw, uw, dw, bg, bu, bd)
        g[tag + "_crc"] = cases.crc(hidden, gw.view(np.uint16), uw.view(np.uint16), dw.view(np.uint16))

    # the same node with FLOAT32 weights (its scalar path)
    args = cases.dense_ffn_case_f32()
    g["dense32_out"] = r.dense_ffn(*args)
    g["dense32_crc"] = cases.crc(*args[:4])

    # Q4_K / Q6_K expert slices to fp16 as the weight provider makes them (src/llm/moe_weight_provider.cpp:17-33):
    # ordinary headers, and headers of any bit pattern (subnormal, infinite, NaN)
    for name, t in (("q4k", cases.Q4_K), ("q6k", cases.Q6_K)):
        for kind, wild in (("", False), ("_wild", True)):
            blocks = cases.kquant_blocks(t, 48, 61 + t, wild)
            g[f"{name}{kind}_f16"] = r.dequant_kquant(t, blocks, 48 * 256).view(np.uint16)
            g[f"{name}{kind}_crc"] = cases.crc(blocks)

    np.savez_compressed(OUT, **g)
    print(f"wrote {OUT}: {os.path.getsize(OUT) / 1024:.1f} KiB, {len(g)} arrays")


if __name__ == "__main__":
    main()
