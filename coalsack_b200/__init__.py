"""B200-native mixture-of-experts hot path behind coalsack's MoE operator API.

The compute lives in ``libcsk_moe.so`` (hand-written sm_100a CUDA behind the C
ABI of ``include/csk_moe.h``); this package is the thin host side.
"""
from .moe import (CskError, GGML_F16, GGML_Q4_K, GGML_Q6_K, MoeLayer, PATH_AUTO, PATH_STREAM, PATH_TILE,  # noqa: F401
                  PATH_TILE_PAIR, dense_ffn_node, dequant_ggml_f16, expert_merge_node, expert_mlp_node, moe_router_node)
from . import synth  # noqa: F401
