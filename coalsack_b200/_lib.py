"""ctypes binding of ``libcsk_moe.so`` (the C ABI declared in include/csk_moe.h).

There is no CPU fallback: if the library cannot be loaded the import fails.
"""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB

_i32, _i64, _vp = C.c_int32, C.c_int64, C.c_void_p
_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)


class Config(C.Structure):
    """csk_moe_config"""
    _fields_ = [(n, _i32) for n in (
        "num_experts", "top_k", "hidden", "ffn", "activation", "has_bias", "sigmoid_gating",
        "weight_before_ffn", "device", "expert_begin", "expert_count", "weight_format")] + [("max_tokens", _i64)]


class Timings(C.Structure):
    """csk_moe_timings"""
    _fields_ = [(n, C.c_float) for n in ("route_ms", "permute_ms", "gate_up_ms", "down_ms", "combine_ms",
                                         "total_ms")] + [("path", _i32), ("launches", _i32)]


# every symbol include/csk_moe.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "csk_moe_create": (C.c_int, [C.POINTER(Config), C.POINTER(_vp)]),
    "csk_moe_destroy": (C.c_int, [_vp]),
    "csk_moe_last_error": (C.c_char_p, [_vp]),
    "csk_moe_device_ok": (C.c_int, [C.c_int]),
    "csk_moe_set_router": (C.c_int, [_vp, _vp, _vp]),
    "csk_moe_load_expert_mxfp4": (C.c_int, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "csk_moe_load_expert_f16": (C.c_int, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "csk_moe_load_expert_f32": (C.c_int, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "csk_moe_load_expert_ggml": (C.c_int, [_vp, _i32, _i32, _vp, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _i32]),
    "csk_moe_dequant_ggml_f16": (C.c_int, [_i32, _i32, _vp, _i64, _vp, _i32]),
    "csk_moe_dense_forward": (C.c_int, [_vp, _vp, _i64, _vp]),
    "csk_moe_dense_forward_dev": (C.c_int, [_vp, _vp, _i64, _vp, _vp]),
    "csk_moe_load_experts_mxfp4": (C.c_int, [_vp, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "csk_moe_save_image": (C.c_int, [_vp, C.c_char_p]),
    "csk_moe_load_image": (C.c_int, [_vp, C.c_char_p]),
    "csk_moe_unpack_expert_mxfp4": (C.c_int, [_vp, _i32, _i32, _vp]),
    "csk_moe_expert_resident": (C.c_int, [_vp, _i32]),
    "csk_moe_route": (C.c_int, [_vp, _vp, _i64, _vp]),
    "csk_moe_forward": (C.c_int, [_vp, _vp, _i64, _vp, _vp, _vp]),
    "csk_moe_expert_forward": (C.c_int, [_vp, _i32, _vp, _i64, _vp, _vp, C.POINTER(_i32)]),
    "csk_moe_merge": (C.c_int, [_vp, _vp, _i64, _vp, _vp]),
    "csk_moe_route_dev": (C.c_int, [_vp, _vp, _i64, _vp, _vp]),
    "csk_moe_forward_dev": (C.c_int, [_vp, _vp, _i64, _vp, _vp, _vp, _vp]),
    "csk_moe_sync": (C.c_int, [_vp]),
    "csk_moe_set_ffn_norm": (C.c_int, [_vp, _vp, C.c_float]),
    "csk_moe_block_forward": (C.c_int, [_vp, _vp, _i64, _vp, _vp]),
    "csk_moe_block_forward_dev": (C.c_int, [_vp, _vp, _i64, _vp, _vp, _vp]),
    "csk_moe_block_forward_shared": (C.c_int, [_vp, _vp, _vp, _i64, _vp, _vp]),
    "csk_moe_block_forward_shared_dev": (C.c_int, [_vp, _vp, _vp, _i64, _vp, _vp, _vp]),
    "csk_moe_route_static": (C.c_int, [_vp, _i64, _i32, _vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "csk_moe_route_static_status": (C.c_int, []),
    "csk_moe_debug_set": (C.c_int, [_vp, _i32, _i64]),
    "csk_moe_ep_dispatch_dev": (C.c_int, [_vp, _vp, _i64, _vp, _vp, _vp, _vp]),
    "csk_moe_ep_experts_dev": (C.c_int, [_vp, _vp, _vp, _i32, _i64, _vp, _vp]),
    "csk_moe_ep_combine_dev": (C.c_int, [_vp, _vp, _i64, _vp, _vp, _vp]),
    "csk_moe_ep_row_pitch": (C.c_int, [_vp]),
    "csk_moe_ep_set_slot_map": (C.c_int, [_vp, _i32, _vp, _vp]),
    "csk_moe_ep_p2p_export": (C.c_int, [_vp, _vp]),
    "csk_moe_ep_p2p_import": (C.c_int, [_vp, _i32, _i32, _vp]),
    "csk_moe_ep_p2p_local_ptrs": (C.c_int, [_vp, _vp, _vp, _vp]),
    "csk_moe_ep_p2p_import_ptrs": (C.c_int, [_vp, _i32, _i32, _vp, _vp, _vp]),
    "csk_moe_ep_p2p_sync_dev": (C.c_int, [_vp, _i32, _vp, _vp, _vp]),
    "csk_moe_ep_p2p_counts_dev": (C.c_int, [_vp, _vp, _i64, _vp, _vp, _vp]),
    "csk_moe_ep_p2p_scatter_dev": (C.c_int, [_vp, _vp, _i64, _vp, _vp]),
    "csk_moe_ep_p2p_experts_dev": (C.c_int, [_vp, _vp, _i64, _vp]),
    "csk_moe_ep_p2p_combine_dev": (C.c_int, [_vp, _i64, _vp, _vp, _vp]),
    "csk_moe_set_path": (C.c_int, [_vp, _i32]),
    "csk_moe_set_activation": (C.c_int, [_vp, _i32, _i32]),
    "csk_moe_set_router_mode": (C.c_int, [_vp, _i32]),
    "csk_moe_get_router_stats": (C.c_int, [_vp, _vp, _vp]),
    "csk_moe_enable_timing": (C.c_int, [_vp, _i32]),
    "csk_moe_get_timings": (C.c_int, [_vp, C.POINTER(Timings)]),
    "csk_moe_get_counters": (C.c_int, [_vp, _vp, _vp, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load the library and bind every declared symbol (raises if one is missing)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            raise ImportError(
                f"{LIB} is missing: build it with `python -m coalsack_b200.build` "
                "(there is no CPU fallback for the MoE path)")
        lib = C.CDLL(LIB)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
