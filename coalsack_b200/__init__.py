"""B200-native mixture-of-experts hot path behind coalsack's MoE operator API.

The compute lives in ``libcsk_moe.so`` (hand-written sm_100a CUDA behind the C
ABI of ``include/csk_moe.h``); this package is the thin host side.
"""
from .moe import (CskError, MoeLayer, PATH_AUTO, PATH_STREAM, PATH_TILE, PATH_TILE_PAIR, dense_ffn_node,  # noqa: F401
                  expert_merge_node, expert_mlp_node, moe_router_node)
from . import synth  # noqa: F401
