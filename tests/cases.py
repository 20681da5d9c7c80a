"""Seeded problem instances shared by the golden-vector generator and the tests."""
from __future__ import annotations

import zlib

import numpy as np

from coalsack_b200 import synth


def crc(*arrays) -> np.uint32:
    c = 0
    for a in arrays:
        if a is not None:
            c = zlib.crc32(np.ascontiguousarray(a).tobytes(), c)
    return np.uint32(c)


def layer_inputs(shape, tokens=None, router_scale=1.0, exp_lo=118, exp_hi=124):
    """(hidden, Wg, router bias, experts) of a layer shape.  ``router_scale``
    widens the logit spread of small layers so that top-k gaps are not tiny."""
    h = synth.hidden_states(shape, tokens)
    Wg = synth.router_weight(shape) * np.float32(router_scale)
    rb = synth.router_bias(shape)
    ex = synth.all_experts(shape)
    if (exp_lo, exp_hi) != (118, 124):
        for e in range(shape.num_experts):
            ex["w_up"][e] = synth.mxfp4_matrix(shape.seed, synth._T_WUP, e, shape.ffn, shape.hidden, exp_lo, exp_hi)
            ex["w_gate"][e] = synth.mxfp4_matrix(shape.seed, synth._T_WGATE, e, shape.ffn, shape.hidden, exp_lo, exp_hi)
            ex["w_down"][e] = synth.mxfp4_matrix(shape.seed, synth._T_WDOWN, e, shape.hidden, shape.ffn, exp_lo, exp_hi)
    return h, Wg, rb, ex


def inputs_crc(h, Wg, rb, ex) -> np.uint32:
    parts = [h, Wg, rb]
    for name in ("w_up", "w_gate", "w_down", "b_up", "b_gate", "b_down"):
        if ex.get(name) is not None:
            parts += list(ex[name])
    return crc(*parts)


def expert_args(ex, e):
    """(w_up, w_gate, w_down, b_up, b_gate, b_down) of expert e."""
    b = [ex[n][e] if ex.get(n) is not None else None for n in ("b_up", "b_gate", "b_down")]
    return (ex["w_up"][e], ex["w_gate"][e], ex["w_down"][e], *b)


# tag -> (synth.tiny kwargs, weight_before_ffn, router scale, (exp_lo, exp_hi))
TINY_CASES = {
    "tiny_a": (dict(seed=11, E=4, k=2, H=64, F=64, T=3, has_bias=True, act=synth.MODIFIED_SWIGLU),
               False, 50.0, (118, 124)),
    "tiny_b": (dict(seed=12, E=8, k=2, H=96, F=160, T=9, has_bias=False, act=synth.STANDARD_SWIGLU),
               False, 50.0, (118, 124)),
    "tiny_c": (dict(seed=13, E=6, k=3, H=128, F=96, T=5, has_bias=True, act=synth.MODIFIED_SWIGLU),
               True, 50.0, (118, 124)),
    "tiny_d": (dict(seed=14, E=16, k=4, H=256, F=320, T=40, has_bias=True, act=synth.MODIFIED_SWIGLU),
               False, 20.0, (112, 130)),
}


def tiny_case(tag):
    """(shape, hidden, Wg, router bias, experts, weight_before_ffn)."""
    kw, wbf, rscale, (lo, hi) = TINY_CASES[tag]
    sh = synth.tiny(**kw)
    h, Wg, rb, ex = layer_inputs(sh, router_scale=rscale, exp_lo=lo, exp_hi=hi)
    return sh, h, Wg, rb, ex, wbf


def router16_case():
    """Router inputs at the size of the reference's own 32-expert / top-4 router test."""
    sh = synth.LayerShape("router_gptoss_scale", 32, 4, 128, 32, True, "normal", 0, 21, 16)
    return synth.hidden_states(sh), synth.router_weight(sh) * np.float32(10), synth.router_bias(sh)


def topk_selection_case():
    """The reference's TopKSelection test: hidden = 1, gate row e = e / H."""
    H, E, k = 4, 6, 3
    hid = np.ones((1, H), np.float32)
    gw = np.repeat((np.arange(E, dtype=np.float32) / np.float32(H))[:, None], H, axis=1)
    return hid, np.ascontiguousarray(gw, np.float32), np.zeros(E, np.float32), k


def c4x8_case():
    sh = synth.C4.with_(num_experts=8, tokens=4)
    return (sh, *layer_inputs(sh, router_scale=10.0))


def codec_blocks():
    blk = np.zeros(17 * 3, np.uint8)
    blk[0], blk[17], blk[34] = 128, 119, 0
    blk[1:17] = np.arange(16) | (np.arange(16)[::-1] << 4)
    blk[18:34] = (np.arange(16) * 17) & 0xFF
    blk[35:51] = 0xF1
    return blk


def err_stats(got, ref):
    """(max-abs error / output RMS, mean|err| / mean|ref|) -- the two parity statistics."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    rms = np.sqrt(np.mean(ref ** 2))
    return float(np.max(np.abs(got - ref)) / rms), float(np.mean(np.abs(got - ref)) / np.mean(np.abs(ref)))


MAX_ABS_OVER_RMS = 2e-2   # parity tolerance: max-abs error <= 2e-2 x output RMS
MEAN_REL = 5e-3           # parity tolerance: mean|err| / mean|ref| <= 5e-3


def rmsnorm_case():
    """Input [6, 320] (scaled so that rows differ in magnitude) and weight [320] of the RMSNorm fixture."""
    g = np.random.default_rng(2024)
    x = (g.standard_normal((6, 320)) * np.array([0.1, 1.0, 3.0, 10.0, 0.01, 1.0])[:, None]).astype(np.float32)
    w = (1.0 + 0.1 * g.standard_normal(320)).astype(np.float32)
    return x, w


def dense_ffn_case(H=256, F=192, T=9, bias=True, seed=77):
    """Inputs of the shared expert's dense FFN fixture: hidden [T,H] fp32, gate/up [F,H] and down [H,F]
    float16 (N(0, 0.05), with a few subnormal and large entries), fp32 biases or None."""
    g = np.random.default_rng(seed)
    hidden = g.standard_normal((T, H)).astype(np.float32)
    gate_w = (g.standard_normal((F, H)) * 0.05).astype(np.float16)
    up_w = (g.standard_normal((F, H)) * 0.05).astype(np.float16)
    down_w = (g.standard_normal((H, F)) * 0.05).astype(np.float16)
    gate_w[0, :4] = np.array([6e-8, -3e-6, 1.5, -2.0], dtype=np.float16)   # subnormals and large values
    b = [(g.standard_normal(n) * 0.01).astype(np.float32) for n in (F, F, H)] if bias else [None, None, None]
    return hidden, gate_w, up_w, down_w, b[0], b[1], b[2]


def dense_ffn_case_f32(H=256, F=192, T=9, bias=True, seed=177):
    """The same with FLOAT32 weights (dense_ffn_node's scalar path): N(0, 0.05) values that are NOT fp16 numbers."""
    g = np.random.default_rng(seed)
    hidden = g.standard_normal((T, H)).astype(np.float32)
    w = [(g.standard_normal(s) * 0.05).astype(np.float32) for s in ((F, H), (F, H), (H, F))]
    b = [(g.standard_normal(n) * 0.01).astype(np.float32) for n in (F, F, H)] if bias else [None, None, None]
    return hidden, w[0], w[1], w[2], b[0], b[1], b[2]


Q4_K, Q6_K = 12, 14                      # ggml_type values
KQUANT_BLOCK_BYTES = {Q4_K: 144, Q6_K: 210}


def kquant_blocks(ggml_type, nblocks, seed, wild=False, scale=0.01):
    """Seeded Q4_K (fp16 d, fp16 dmin, 12 scale bytes, 128 nibble bytes) or Q6_K (128 low-nibble bytes, 64
    high-bit bytes, 16 int8 scales, fp16 d) super-blocks, every code and scale byte uniform; the fp16 headers
    N(0, scale), or with ``wild`` any 16-bit pattern (subnormals, infinities, NaNs)."""
    g = np.random.default_rng(seed)
    per = KQUANT_BLOCK_BYTES[ggml_type]
    b = g.integers(0, 256, size=(nblocks, per), dtype=np.uint8)
    nh = 2 if ggml_type == Q4_K else 1
    if wild:
        hdr = g.integers(0, 65536, size=(nblocks, nh)).astype(np.uint16)
    else:
        hdr = (g.standard_normal((nblocks, nh)) * scale).astype(np.float16).view(np.uint16)
    off = 0 if ggml_type == Q4_K else 208
    b[:, off:off + 2 * nh] = hdr.view(np.uint8).reshape(nblocks, 2 * nh)
    return b


def kquant_values_f32(ggml_type, blocks):
    """The fp32 values of Q4_K / Q6_K super-blocks, written with numpy array arithmetic (float32 products and
    differences, each rounded once): an independent statement of the layout, gguf_dequant.h:147-261."""
    b = np.asarray(blocks, np.uint8).reshape(-1, KQUANT_BLOCK_BYTES[ggml_type])
    nb = b.shape[0]
    out = np.empty((nb, 256), np.float32)
    with np.errstate(all="ignore"):
        if ggml_type == Q4_K:
            d = b[:, 0:2].copy().view(np.float16).astype(np.float32)           # [nb,1]
            dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)
            sc = b[:, 4:16].astype(np.int32)
            q = b[:, 16:144].reshape(nb, 4, 32)
            for j in range(8):
                if j < 4:
                    s, m = sc[:, j] & 0x3F, sc[:, j + 4] & 0x3F
                else:
                    s = (sc[:, j + 4] & 0x0F) | ((sc[:, j - 4] >> 6) << 4)
                    m = (sc[:, j + 4] >> 4) | ((sc[:, j] >> 6) << 4)
                ds = d * s[:, None].astype(np.float32)
                ms = dmin * m[:, None].astype(np.float32)
                v = (q[:, j // 2] >> 4) if (j & 1) else (q[:, j // 2] & 0x0F)
                out[:, j * 32:(j + 1) * 32] = ds * v.astype(np.float32) - ms
        else:
            d = b[:, 208:210].copy().view(np.float16).astype(np.float32)
            sc = b[:, 192:208].copy().view(np.int8).astype(np.float32)
            for half in range(2):
                ql = b[:, half * 64:half * 64 + 64].astype(np.int32)
                qh = b[:, 128 + half * 32:128 + half * 32 + 32].astype(np.int32)
                for i in range(4):
                    lo = ql[:, 32 * (i & 1):32 * (i & 1) + 32]
                    nib = (lo & 0x0F) if i < 2 else (lo >> 4)
                    qv = (nib | (((qh >> (2 * i)) & 3) << 4)) - 32
                    scale = np.repeat(sc[:, half * 8 + 2 * i:half * 8 + 2 * i + 2], 16, axis=1)   # l/16 + 2i
                    out[:, half * 128 + 32 * i:half * 128 + 32 * i + 32] = (d * scale) * qv.astype(np.float32)
    return out.reshape(-1)
