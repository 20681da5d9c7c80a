"""Seeded synthetic MoE layers with the shapes and value distributions of the
benchmark configurations (no checkpoint or dataset is read).

Every tensor is drawn from its own counter-based stream (Philox keyed by
``(seed, tensor id, index)``), so any rank can generate exactly the experts it
owns and the CPU checker and the CUDA path see bit-identical buffers.

Expert matrices are generated directly in the MXFP4 wire format the reference
holds in ``dynamic_mx_tensor`` (include/coalsack/tensor/dynamic_mx_tensor.h:19-44):
row-major rows of ``cols/32`` blocks, each block one E8M0 scale byte followed by
16 bytes of packed E2M1 codes.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace

import numpy as np

MODIFIED_SWIGLU = 0  # expert_mlp_node::activation_type::MODIFIED_SWIGLU
STANDARD_SWIGLU = 1  # expert_mlp_node::activation_type::STANDARD_SWIGLU

_T_HIDDEN, _T_WG, _T_RBIAS, _T_WUP, _T_WGATE, _T_WDOWN, _T_BUP, _T_BGATE, _T_BDOWN = range(9)


@dataclass(frozen=True)
class LayerShape:
    name: str
    num_experts: int
    top_k: int
    hidden: int
    ffn: int
    has_bias: bool = True
    router_bias: str = "normal"  # "normal" | "zipf" | "none"
    act: int = MODIFIED_SWIGLU
    seed: int = 0
    tokens: int = 1

    def with_(self, **kw) -> "LayerShape":
        return replace(self, **kw)

    @property
    def mxfp4_bytes_per_expert(self) -> int:
        return 3 * self.hidden * self.ffn // 32 * 17

    @property
    def bias_bytes_per_expert(self) -> int:
        return (2 * self.ffn + self.hidden) * 4 if self.has_bias else 0


# The benchmark configurations (gpt-oss-20b / gpt-oss-120b / Qwen3-30B-A3B shaped layers).
C0 = LayerShape("c0_gptoss20b_cpu", 32, 4, 2880, 2880, True, "normal", MODIFIED_SWIGLU, 0, 32)
C1 = LayerShape("c1_gptoss20b_prefill4096_zipf", 32, 4, 2880, 2880, True, "zipf", MODIFIED_SWIGLU, 1, 4096)
C2 = LayerShape("c2_gptoss120b_prefill8192", 128, 4, 2880, 2880, True, "normal", MODIFIED_SWIGLU, 2, 8192)
C3 = LayerShape("c3_gptoss120b_decode", 128, 4, 2880, 2880, True, "normal", MODIFIED_SWIGLU, 3, 1)
C4 = LayerShape("c4_qwen3_30b_a3b_prefill2048", 128, 8, 2048, 768, False, "none", STANDARD_SWIGLU, 4, 2048)
CONFIGS = {"c0": C0, "c1": C1, "c2": C2, "c3": C3, "c4": C4}


def _rng(seed: int, tensor_id: int, index: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed, (tensor_id << 40) | index]))


def hidden_states(shape: LayerShape, tokens: int | None = None, rep: int = 0) -> np.ndarray:
    """[T,H] fp32 ~ N(0,1); ``rep`` selects a fresh batch of the decode sweep."""
    T = shape.tokens if tokens is None else tokens
    return _rng(shape.seed, _T_HIDDEN, rep).standard_normal((T, shape.hidden), dtype=np.float32)


def router_weight(shape: LayerShape) -> np.ndarray:
    w = _rng(shape.seed, _T_WG).standard_normal((shape.num_experts, shape.hidden), dtype=np.float32)
    return w * np.float32(0.02)


def router_bias(shape: LayerShape) -> np.ndarray | None:
    E = shape.num_experts
    if shape.router_bias == "none":
        return None
    if shape.router_bias == "zipf":
        return (0.5 * np.log(1.0 / (np.arange(E) + 1.0))).astype(np.float32)
    return _rng(shape.seed, _T_RBIAS).standard_normal(E, dtype=np.float32) * np.float32(0.01)


def mxfp4_matrix(seed: int, tensor_id: int, expert: int, rows: int, cols: int,
                 exp_lo: int = 118, exp_hi: int = 124) -> np.ndarray:
    """[rows*cols/32*17] uint8: codes uniform over all 16 nibbles, E8M0 scale
    exponent uniform over the integers [exp_lo, exp_hi]."""
    g = _rng(seed, tensor_id, expert)
    nblk = rows * cols // 32
    out = np.empty((nblk, 17), np.uint8)
    out[:, 0] = g.integers(exp_lo, exp_hi + 1, size=nblk, dtype=np.uint8)
    out[:, 1:] = g.integers(0, 256, size=(nblk, 16), dtype=np.uint8)
    return out.reshape(-1)


def expert_weights(shape: LayerShape, expert: int) -> dict:
    """One expert: ``w_up``/``w_gate`` [F,H] and ``w_down`` [H,F] as MXFP4 bytes,
    ``b_up``/``b_gate`` [F], ``b_down`` [H] fp32 ~ N(0, 0.01) or None."""
    H, F, s = shape.hidden, shape.ffn, shape.seed
    d = {
        "w_up": mxfp4_matrix(s, _T_WUP, expert, F, H),
        "w_gate": mxfp4_matrix(s, _T_WGATE, expert, F, H),
        "w_down": mxfp4_matrix(s, _T_WDOWN, expert, H, F),
        "b_up": None, "b_gate": None, "b_down": None,
    }
    if shape.has_bias:
        d["b_up"] = _rng(s, _T_BUP, expert).standard_normal(F, dtype=np.float32) * np.float32(0.01)
        d["b_gate"] = _rng(s, _T_BGATE, expert).standard_normal(F, dtype=np.float32) * np.float32(0.01)
        d["b_down"] = _rng(s, _T_BDOWN, expert).standard_normal(H, dtype=np.float32) * np.float32(0.01)
    return d


def all_experts(shape: LayerShape, experts=None) -> dict:
    """Lists over experts of the fields of :func:`expert_weights`."""
    ids = range(shape.num_experts) if experts is None else experts
    per = [expert_weights(shape, e) for e in ids]
    out = {k: [p[k] for p in per] for k in ("w_up", "w_gate", "w_down")}
    for k in ("b_up", "b_gate", "b_down"):
        out[k] = [p[k] for p in per] if shape.has_bias else None
    return out


def tiny(seed: int = 11, E: int = 4, k: int = 2, H: int = 64, F: int = 64, T: int = 3,
         has_bias: bool = True, act: int = MODIFIED_SWIGLU, exp_lo: int = 118,
         exp_hi: int = 124) -> LayerShape:
    """A small layer for unit tests (same generator, arbitrary sizes)."""
    return LayerShape(f"tiny_e{E}k{k}h{H}f{F}", E, k, H, F, has_bias,
                      "normal" if has_bias else "none", act, seed, T)
