"""Host-side mirror, in Python, of the reference's operator interface for the
MoE path, over the C ABI of ``libcsk_moe.so``.

``MoeLayer`` wraps one ``csk_moe_layer`` handle.  The node classes keep the
names, setters, argument meaning and error behaviour of the reference's
operators so tests written against the reference read the same here:

    moe_router_node    include/coalsack/nn/nn_ops/moe_router_node.h:22-124
    expert_mlp_node    include/coalsack/nn/nn_ops/expert_mlp_node.h:25-148, 392-530
    expert_merge_node  include/coalsack/nn/nn_ops/expert_merge_node.h:9-134

Every computation runs on the GPU; nothing here falls back to the CPU.
"""
from __future__ import annotations

import ctypes as C
import enum

import numpy as np

from . import _lib
from ._lib import Config, Timings

PATH_AUTO, PATH_STREAM, PATH_TILE, PATH_TILE_PAIR = 0, 1, 2, 3
GGML_F16, GGML_Q4_K, GGML_Q6_K = 1, 12, 14     # ggml_type values (gguf_types.h:24-39)


class CskError(RuntimeError):
    """A non-zero status from the C ABI (the C++ node shim throws std::runtime_error)."""

    def __init__(self, code: int, msg: str):
        super().__init__(msg)
        self.code = code


def _np_f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def dequant_ggml_f16(ggml_type, blocks, n_elements, nearest=False, device=0):
    """Q4_K / Q6_K super-blocks (uint8) to ``n_elements`` float16 values on the device: what
    moe_weight_provider.cpp:17-33 does on the host (``nearest``: the reference's F16C build of fp32_to_fp16)."""
    lib = _lib.load()
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    per = {GGML_Q4_K: 144, GGML_Q6_K: 210}.get(ggml_type)
    if per is not None and n_elements % 256 == 0 and blocks.size != n_elements // 256 * per:
        raise RuntimeError(f"ggml type {ggml_type}: expected {n_elements // 256 * per} bytes, got {blocks.size}")
    out = np.empty(max(int(n_elements), 0), np.uint16)
    rc = lib.csk_moe_dequant_ggml_f16(device, int(ggml_type), _p(blocks), int(n_elements), _p(out), int(bool(nearest)))
    if rc != 0:
        raise CskError(rc, lib.csk_moe_last_error(None).decode())
    return out.view(np.float16)


def _np_u8(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.uint8)


def _p(a):
    """void* of a numpy array, a torch tensor, an int address or None."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    if isinstance(a, int):
        return a
    return a.data_ptr()


class MoeLayer:
    """One MoE layer resident on one GPU (a ``csk_moe_layer`` handle)."""

    def __init__(self, num_experts, top_k, hidden, ffn, activation=0, has_bias=True,
                 sigmoid_gating=False, weight_before_ffn=False, device=0, expert_begin=0,
                 expert_count=0, max_tokens=1024, weights_f16=False):
        self._lib = _lib.load()
        self.cfg = Config(num_experts, top_k, hidden, ffn, int(activation), int(has_bias),
                          int(sigmoid_gating), int(weight_before_ffn), device, expert_begin,
                          expert_count, 1 if weights_f16 else 0, max_tokens)
        self.weights_f16 = bool(weights_f16)
        self.E, self.k, self.H, self.F = num_experts, top_k, hidden, ffn
        self.E_router = num_experts  # experts the router scores (fewer than E under an expert-parallel slot map)
        self.max_tokens = max_tokens
        self._h = C.c_void_p()
        rc = self._lib.csk_moe_create(C.byref(self.cfg), C.byref(self._h))
        if rc:
            raise CskError(rc, self._lib.csk_moe_last_error(None).decode())

    @classmethod
    def from_shape(cls, shape, device=0, max_tokens=None, expert_begin=0, expert_count=0, **kw):
        return cls(shape.num_experts, shape.top_k, shape.hidden, shape.ffn, shape.act, shape.has_bias,
                   device=device, expert_begin=expert_begin, expert_count=expert_count,
                   max_tokens=max_tokens or shape.tokens, **kw)

    # -- plumbing -----------------------------------------------------------
    def _check(self, rc):
        if rc:
            raise CskError(rc, self._lib.csk_moe_last_error(self._h).decode())

    def close(self):
        if self._h:
            self._lib.csk_moe_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- weights ------------------------------------------------------------
    def set_router(self, gate_w, gate_bias=None):
        gate_w, gate_bias = _np_f32(gate_w), _np_f32(gate_bias)
        if gate_w.shape != (self.E_router, self.H):
            raise RuntimeError(f"moe_router: gate_weights shape mismatch, expected [{self.E_router}, {self.H}], "
                               f"got [{gate_w.shape[0]}, {gate_w.shape[1]}]")
        self._check(self._lib.csk_moe_set_router(self._h, _p(gate_w), _p(gate_bias)))

    def load_expert(self, expert_id, w_up, w_gate, w_down, b_up=None, b_gate=None, b_down=None):
        nbytes = self.H * self.F // 32 * 17
        arrs = [_np_u8(w_up).reshape(-1), _np_u8(w_gate).reshape(-1), _np_u8(w_down).reshape(-1)]
        for a in arrs:
            if a.size != nbytes:
                raise RuntimeError("expert_mlp: weight dimension mismatch")
        b = [_np_f32(b_up), _np_f32(b_gate), _np_f32(b_down)]
        self._check(self._lib.csk_moe_load_expert_mxfp4(self._h, expert_id, *map(_p, arrs), *map(_p, b)))

    def load_expert_f16(self, expert_id, w_up, w_gate, w_down, b_up=None, b_gate=None, b_down=None):
        """fp16 weights: w_up, w_gate [F,H], w_down [H,F] (numpy float16 or the uint16 bit patterns)."""
        arrs = []
        for a, shape in ((w_up, (self.F, self.H)), (w_gate, (self.F, self.H)), (w_down, (self.H, self.F))):
            a = np.asarray(a)
            a = np.ascontiguousarray(a.view(np.uint16) if a.dtype == np.float16 else a.astype(np.uint16, copy=False))
            if a.size != shape[0] * shape[1]:
                raise RuntimeError("dense_ffn: weight dimension mismatch")
            arrs.append(a.reshape(-1))
        b = [_np_f32(b_up), _np_f32(b_gate), _np_f32(b_down)]
        self._check(self._lib.csk_moe_load_expert_f16(self._h, expert_id, *map(_p, arrs), *map(_p, b)))

    def load_expert_f32(self, expert_id, w_up, w_gate, w_down, b_up=None, b_gate=None, b_down=None):
        """fp32 weight matrices, rounded to fp16 on the device (refused when a weight exceeds the fp16 range)."""
        arrs = []
        for a, shape in ((w_up, (self.F, self.H)), (w_gate, (self.F, self.H)), (w_down, (self.H, self.F))):
            a = _np_f32(a)
            if a.size != shape[0] * shape[1]:
                raise RuntimeError("dense_ffn: weight dimension mismatch")
            arrs.append(a.reshape(-1))
        b = [_np_f32(b_up), _np_f32(b_gate), _np_f32(b_down)]
        self._check(self._lib.csk_moe_load_expert_f32(self._h, expert_id, *map(_p, arrs), *map(_p, b)))

    def load_expert_ggml(self, expert_id, w_up, w_gate, w_down, b_up=None, b_gate=None, b_down=None, nearest=False):
        """Expert slices as the GGUF file holds them: each of w_up, w_gate, w_down is ``(ggml_type, array)`` with
        ggml_type GGML_F16 (float16 / uint16 values), GGML_Q4_K or GGML_Q6_K (uint8 super-blocks); decoded on
        the device to the fp16 values the reference's weight provider would make (``nearest``: its F16C build)."""
        types, arrs = [], []
        for t, a in (w_up, w_gate, w_down):
            a = np.asarray(a)
            if t == GGML_F16:
                a = a.view(np.uint16) if a.dtype == np.float16 else a.astype(np.uint16, copy=False)
                want = self.H * self.F
            elif t in (GGML_Q4_K, GGML_Q6_K):
                a = a.astype(np.uint8, copy=False)
                want = self.H * self.F // 256 * (144 if t == GGML_Q4_K else 210)
            else:
                raise RuntimeError(f"ggml type {t} is not handled")
            a = np.ascontiguousarray(a).reshape(-1)
            if a.size != want:
                raise RuntimeError(f"ggml type {t}: expected {want} elements, got {a.size}")
            types.append(int(t))
            arrs.append(a)
        b = [_np_f32(b_up), _np_f32(b_gate), _np_f32(b_down)]
        self._check(self._lib.csk_moe_load_expert_ggml(self._h, expert_id, types[0], _p(arrs[0]), types[1], _p(arrs[1]),
                                                       types[2], _p(arrs[2]), *map(_p, b), int(bool(nearest))))

    def dense_forward(self, hidden):
        """The dense FFN (a layer with one expert and top-1): every row through the weight set."""
        hidden = _np_f32(hidden)
        T = hidden.size // self.H
        out = np.empty((T, self.H), dtype=np.float32)
        self._check(self._lib.csk_moe_dense_forward(self._h, _p(hidden), T, _p(out)))
        return out.reshape(hidden.shape)

    def dense_forward_dev(self, d_hidden, T, d_out, stream=None):
        self._check(self._lib.csk_moe_dense_forward_dev(self._h, _p(d_hidden), T, _p(d_out), stream))

    def load_experts(self, experts: dict, ids=None):
        """``experts``: lists as made by ``synth.all_experts`` (index i <-> ids[i])."""
        ids = list(range(self.E)) if ids is None else list(ids)
        for i, e in enumerate(ids):
            b = [experts[n][i] if experts.get(n) is not None else None for n in ("b_up", "b_gate", "b_down")]
            self.load_expert(e, experts["w_up"][i], experts["w_gate"][i], experts["w_down"][i], *b)

    def load_experts_bulk(self, first_expert, w_up, w_gate, w_down, b_up=None, b_gate=None, b_down=None):
        """Slabs [count, rows*cols/32*17] of MXFP4 blocks (and [count, n] fp32 biases) for experts
        first_expert .. first_expert + count - 1."""
        nbytes = self.H * self.F // 32 * 17
        slabs = [_np_u8(a).reshape(-1, nbytes) for a in (w_up, w_gate, w_down)]
        count = slabs[0].shape[0]
        if any(a.shape[0] != count for a in slabs):
            raise RuntimeError("expert_mlp: weight dimension mismatch")
        b = [None if a is None else _np_f32(a).reshape(count, -1) for a in (b_up, b_gate, b_down)]
        self._check(self._lib.csk_moe_load_experts_mxfp4(self._h, first_expert, count, *map(_p, slabs), *map(_p, b)))

    def save_image(self, path):
        self._check(self._lib.csk_moe_save_image(self._h, str(path).encode()))

    def load_image(self, path):
        self._check(self._lib.csk_moe_load_image(self._h, str(path).encode()))

    def unpack_expert(self, expert_id, which):
        out = np.empty(self.H * self.F // 32 * 17, np.uint8)
        self._check(self._lib.csk_moe_unpack_expert_mxfp4(self._h, expert_id, which, _p(out)))
        return out

    def expert_resident(self, expert_id) -> bool:
        return bool(self._lib.csk_moe_expert_resident(self._h, expert_id))

    # -- host-buffer calls ----------------------------------------------------
    def route(self, hidden):
        hidden = _np_f32(hidden).reshape(-1, self.H)
        T = hidden.shape[0]
        out = np.empty((T, self.k, 2), np.float32)
        self._check(self._lib.csk_moe_route(self._h, _p(hidden), T, _p(out)))
        return out

    def forward(self, hidden, router_out=None, out=None, router_out_buf=None):
        """(out[T,H], router_out[T,k,2]).  ``hidden``/``out`` may be pinned torch tensors."""
        if isinstance(hidden, np.ndarray) or not hasattr(hidden, "data_ptr"):
            hidden = _np_f32(hidden).reshape(-1, self.H)
        T = hidden.shape[0]
        if out is None:
            out = np.empty((T, self.H), np.float32)
        r_in = _np_f32(router_out)
        r_out = router_out_buf if router_out_buf is not None else np.empty((T, self.k, 2), np.float32)
        self._check(self._lib.csk_moe_forward(self._h, _p(hidden), T, _p(r_in), _p(r_out), _p(out)))
        return out, r_out

    def set_ffn_norm(self, weight, eps=1e-5):
        """Weight [H] and epsilon of the RMSNorm in front of the router (rmsnorm_node)."""
        w = _np_f32(weight).reshape(-1)
        if w.shape[0] != self.H:
            raise RuntimeError("rmsnorm: weight shape must be [hidden_dim]")
        self._check(self._lib.csk_moe_set_ffn_norm(self._h, _p(w), float(eps)))

    def block_forward(self, x, shared=None):
        """(x + moe(n) [+ shared(n)], router_out) with n = rmsnorm(x) * weight: the layer with its norm and residual,
        and optionally the shared expert's dense FFN (``shared``: a dense MoeLayer, one expert, top-1, fp16 format)."""
        x = _np_f32(x).reshape(-1, self.H)
        T = x.shape[0]
        out = np.empty((T, self.H), np.float32)
        ro = np.empty((T, self.k, 2), np.float32)
        if shared is None:
            self._check(self._lib.csk_moe_block_forward(self._h, _p(x), T, _p(ro), _p(out)))
        else:
            self._check(self._lib.csk_moe_block_forward_shared(self._h, shared._h, _p(x), T, _p(ro), _p(out)))
        return out, ro

    def block_forward_dev(self, d_x, T, d_router_out, d_out, stream=None, shared=None):
        self._check(self._lib.csk_moe_block_forward_shared_dev(self._h, shared._h if shared is not None else None,
                                                               _p(d_x), T, _p(d_router_out), _p(d_out), stream))

    def expert_forward(self, expert_id, hidden, router_out):
        """Dense [T,H] output of one expert node, or None for the {0}-shaped empty tensor."""
        hidden = _np_f32(hidden).reshape(-1, self.H)
        router_out = _np_f32(router_out)
        T = hidden.shape[0]
        out = np.empty((T, self.H), np.float32)
        sel = C.c_int32(0)
        self._check(self._lib.csk_moe_expert_forward(self._h, expert_id, _p(hidden), T, _p(router_out),
                                                     _p(out), C.byref(sel)))
        return out if sel.value else None

    def merge(self, router_out, expert_outs):
        router_out = _np_f32(router_out)
        T = router_out.shape[0]
        keep = [None if a is None else _np_f32(a) for a in expert_outs]
        ptrs = (C.c_void_p * self.E)(*[None if a is None else a.ctypes.data for a in keep])
        out = np.empty((T, self.H), np.float32)
        self._check(self._lib.csk_moe_merge(self._h, _p(router_out), T, ptrs, _p(out)))
        return out

    # -- device-buffer calls (torch CUDA tensors or raw addresses) -------------
    def route_dev(self, d_hidden, T, d_router_out, stream=None):
        self._check(self._lib.csk_moe_route_dev(self._h, _p(d_hidden), T, _p(d_router_out), stream))

    def forward_dev(self, d_hidden, T, d_out, d_router_in=None, d_router_out=None, stream=None):
        self._check(self._lib.csk_moe_forward_dev(self._h, _p(d_hidden), T, _p(d_router_in),
                                                  _p(d_router_out), _p(d_out), stream))

    def sync(self):
        """Wait for the last device-buffer call and raise what its kernels reported."""
        self._check(self._lib.csk_moe_sync(self._h))

    def ep_row_pitch(self) -> int:
        return self._lib.csk_moe_ep_row_pitch(self._h)

    def ep_dispatch_dev(self, d_hidden, T, d_send, d_counts, d_router_in=None, stream=None):
        self._check(self._lib.csk_moe_ep_dispatch_dev(self._h, _p(d_hidden), T, _p(d_router_in), _p(d_send),
                                                      _p(d_counts), stream))

    def ep_experts_dev(self, d_recv, d_recv_counts, n_src, total_rows, d_ret, stream=None):
        self._check(self._lib.csk_moe_ep_experts_dev(self._h, _p(d_recv), _p(d_recv_counts), n_src,
                                                     total_rows, _p(d_ret), stream))

    def ep_combine_dev(self, d_back, T, d_out, d_router_out=None, stream=None):
        self._check(self._lib.csk_moe_ep_combine_dev(self._h, _p(d_back), T, _p(d_out), _p(d_router_out),
                                                     stream))

    def ep_set_slot_map(self, primary_slot, replica_slot=None):
        """Router over len(primary_slot) logical experts; dispatch groups expert e under slot
        primary_slot[e] (odd tokens under replica_slot[e] where that is >= 0).  None removes the map."""
        if primary_slot is None:
            self._check(self._lib.csk_moe_ep_set_slot_map(self._h, 0, None, None))
            self.E_router = self.E
            return
        p = np.ascontiguousarray(primary_slot, dtype=np.int32)
        r = None if replica_slot is None else np.ascontiguousarray(replica_slot, dtype=np.int32)
        if r is not None and r.shape != p.shape:
            raise ValueError("replica_slot must have the shape of primary_slot")
        self._check(self._lib.csk_moe_ep_set_slot_map(self._h, int(p.shape[0]), _p(p), _p(r)))
        self.E_router = int(p.shape[0])

    # -- expert parallelism over peer memory ---------------------------------------
    IPC_BYTES = 3 * 72

    def ep_p2p_export(self) -> bytes:
        buf = (C.c_uint8 * self.IPC_BYTES)()
        self._check(self._lib.csk_moe_ep_p2p_export(self._h, buf))
        return bytes(buf)

    def ep_p2p_import(self, rank, world, all_handles: bytes):
        if len(all_handles) != world * self.IPC_BYTES:
            raise ValueError(f"all_handles must hold world * {self.IPC_BYTES} bytes")
        buf = (C.c_uint8 * len(all_handles)).from_buffer_copy(all_handles)
        self._check(self._lib.csk_moe_ep_p2p_import(self._h, rank, world, buf))

    def ep_p2p_local_ptrs(self):
        p = [C.c_void_p() for _ in range(3)]
        self._check(self._lib.csk_moe_ep_p2p_local_ptrs(self._h, C.byref(p[0]), C.byref(p[1]), C.byref(p[2])))
        return tuple(x.value for x in p)

    def ep_p2p_import_ptrs(self, rank, world, x16, info, back):
        arr = lambda v: (C.c_void_p * world)(*v)
        self._check(self._lib.csk_moe_ep_p2p_import_ptrs(self._h, rank, world, arr(x16), arr(info), arr(back)))

    def ep_p2p_sync_dev(self, which, d_counts=None, d_all_counts=None, stream=None):
        self._check(self._lib.csk_moe_ep_p2p_sync_dev(self._h, which, _p(d_counts), _p(d_all_counts), stream))

    def ep_p2p_counts_dev(self, d_hidden, T, d_counts, d_router_in=None, stream=None):
        self._check(self._lib.csk_moe_ep_p2p_counts_dev(self._h, _p(d_hidden), T, _p(d_router_in), _p(d_counts), stream))

    def ep_p2p_scatter_dev(self, d_hidden, T, d_all_counts, stream=None):
        self._check(self._lib.csk_moe_ep_p2p_scatter_dev(self._h, _p(d_hidden), T, _p(d_all_counts), stream))

    def ep_p2p_experts_dev(self, d_all_counts, rows_hint, stream=None):
        self._check(self._lib.csk_moe_ep_p2p_experts_dev(self._h, _p(d_all_counts), rows_hint, stream))

    def ep_p2p_combine_dev(self, T, d_out, d_router_out=None, stream=None):
        self._check(self._lib.csk_moe_ep_p2p_combine_dev(self._h, T, _p(d_out), _p(d_router_out), stream))

    # -- knobs / observability ---------------------------------------------------
    def set_path(self, path):
        self._check(self._lib.csk_moe_set_path(self._h, path))

    ROUTER_AUTO, ROUTER_CHAIN, ROUTER_CERTIFIED = 0, 1, 2

    def set_router_mode(self, mode):
        self._check(self._lib.csk_moe_set_router_mode(self._h, int(mode)))

    def router_stats(self):
        """(tokens routed in certified mode, tokens of those recomputed by the chain)."""
        a, b = C.c_int64(0), C.c_int64(0)
        self._check(self._lib.csk_moe_get_router_stats(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    DEBUG_WAIT_BUDGET, DEBUG_STALL_TILE_PRODUCER = 0, 1

    def debug_set(self, key, value):
        """Test hooks of the failure path (csk_moe_debug_set)."""
        self._check(self._lib.csk_moe_debug_set(self._h, int(key), int(value)))

    def enable_timing(self, on=True):
        self._check(self._lib.csk_moe_enable_timing(self._h, int(on)))

    def timings(self) -> dict:
        t = Timings()
        self._check(self._lib.csk_moe_get_timings(self._h, C.byref(t)))
        return {n: getattr(t, n) for n, _ in Timings._fields_}

    def counters(self):
        rows = np.zeros(self.E, np.int64)
        d, b = C.c_int64(0), C.c_int64(0)
        self._check(self._lib.csk_moe_get_counters(self._h, _p(rows), C.byref(d), C.byref(b)))
        return rows, d.value, b.value


# ---------------------------------------------------------------------------
# Operator classes with the reference's names and setters
# ---------------------------------------------------------------------------
class moe_router_node:
    """moe_router_node (moe_router_node.h:22-124): ``set_config``, ``set_sigmoid_gating``,
    ``compute_test(hidden_states[B,S,H], gate_weights[E,H][, gate_bias[E]]) -> [B,S,k,2]``."""

    def __init__(self, device=0):
        self.num_experts_, self.top_k_, self.use_sigmoid_gating_ = 0, 0, False
        self.device = device
        self._layer = None
        self._key = None

    def set_config(self, num_experts, top_k):
        self.num_experts_, self.top_k_ = int(num_experts), int(top_k)

    def set_sigmoid_gating(self, v):
        self.use_sigmoid_gating_ = bool(v)

    def compute_test(self, hidden_states, gate_weights, gate_bias=None):
        hidden_states, gate_weights = np.asarray(hidden_states), np.asarray(gate_weights)
        if hidden_states.ndim != 3:
            raise RuntimeError("moe_router: hidden_states must be 3D [batch, seq_len, hidden_dim], got "
                               f"{hidden_states.ndim}D")
        if gate_weights.ndim != 2:
            raise RuntimeError("moe_router: gate_weights must be 2D [num_experts, hidden_dim], got "
                               f"{gate_weights.ndim}D")
        if gate_bias is not None and np.asarray(gate_bias).ndim != 1:
            raise RuntimeError(f"moe_router: gate_bias must be 1D [num_experts], got {np.asarray(gate_bias).ndim}D")
        B, S, H = hidden_states.shape
        if gate_weights.shape != (self.num_experts_, H):
            raise RuntimeError(f"moe_router: gate_weights shape mismatch, expected [{self.num_experts_}, {H}], "
                               f"got [{gate_weights.shape[0]}, {gate_weights.shape[1]}]")
        if gate_bias is not None and np.asarray(gate_bias).shape[0] != self.num_experts_:
            raise RuntimeError(f"moe_router: gate_bias must have num_experts={self.num_experts_} elements, "
                               f"got {np.asarray(gate_bias).shape[0]}")
        if hidden_states.dtype != np.float32:
            raise RuntimeError("moe_router: only float32 supported on the GPU path")
        T = B * S
        Hp = (H + 31) // 32 * 32  # the layer handle wants H % 32 == 0; zero columns add exact zeros
        key = (self.num_experts_, self.top_k_, Hp, self.use_sigmoid_gating_, T)
        if self._key != key:
            if self._layer is not None:
                self._layer.close()
            self._layer = MoeLayer(self.num_experts_, self.top_k_, Hp, 32, has_bias=False,
                                   sigmoid_gating=self.use_sigmoid_gating_, device=self.device,
                                   max_tokens=max(T, 1))
            self._key = key
        h2 = hidden_states.reshape(T, H)
        if Hp != H:
            h2 = np.concatenate([h2, np.zeros((T, Hp - H), np.float32)], axis=1)
            gate_weights = np.concatenate([gate_weights, np.zeros((self.num_experts_, Hp - H), np.float32)], axis=1)
        self._layer.set_router(gate_weights, gate_bias)
        return self._layer.route(h2).reshape(B, S, self.top_k_, 2)


class expert_mlp_node:
    """expert_mlp_node (expert_mlp_node.h:25-148), MXFP4 weight path."""

    class activation_type(enum.IntEnum):
        MODIFIED_SWIGLU = 0
        STANDARD_SWIGLU = 1

    def __init__(self, expert_id=0, device=0):
        self.expert_id_ = int(expert_id)
        self.activation_type_ = expert_mlp_node.activation_type.MODIFIED_SWIGLU
        self.weight_before_ffn_ = False
        self.device = device
        self._layer = None
        self._key = None

    def get_expert_id(self):
        return self.expert_id_

    def get_proc_name(self):
        return "expert_mlp"

    def set_activation_type(self, t):
        self.activation_type_ = expert_mlp_node.activation_type(t)

    def get_activation_type(self):
        return self.activation_type_

    def set_weight_before_ffn(self, v):
        self.weight_before_ffn_ = bool(v)

    def _get_layer(self, H, F, has_bias, k, T, n_ids=1):
        E = max(self.expert_id_ + 1, k, n_ids)  # the layer's id space must cover every id the router names
        key = (H, F, has_bias, k, int(self.activation_type_), self.weight_before_ffn_, self.expert_id_, E)
        if self._key != key or self._layer.max_tokens < T:
            if self._layer is not None:
                self._layer.close()
            # a one-expert layer whose only resident expert carries this node's id
            self._layer = MoeLayer(E, k, H, F,
                                   int(self.activation_type_), has_bias,
                                   weight_before_ffn=self.weight_before_ffn_, device=self.device,
                                   expert_begin=self.expert_id_, expert_count=1, max_tokens=max(T, 64))
            self._key = key
        return self._layer

    def compute_test_mxfp4(self, hidden_vec, w_up, w_gate, w_down, b_up, b_gate, b_down, hidden_dim,
                           expert_ffn_dim):
        """One token through this expert (expert_mlp_node.h:63-70)."""
        if hidden_dim % 2 or expert_ffn_dim % 2:
            raise RuntimeError("compute_token_mxfp4: dimensions must be even")
        lay = self._get_layer(hidden_dim, expert_ffn_dim, b_up is not None, 1, 1)
        lay.load_expert(self.expert_id_, w_up, w_gate, w_down, b_up, b_gate, b_down)
        r = np.array([[[self.expert_id_, 1.0]]], np.float32)
        out = lay.expert_forward(self.expert_id_, np.asarray(hidden_vec, np.float32).reshape(1, -1), r)
        return out[0]

    def compute_with_mxfp4(self, hidden_states, w_up, w_gate, w_down, b_up, b_gate, b_down, router_output,
                           expert_ffn_dim):
        """The node's MXFP4 branch (expert_mlp_node.h:392-485): dense [B,S,H] output with
        zero rows for tokens that did not select this expert, or a {0}-shaped tensor."""
        hidden_states, router_output = np.asarray(hidden_states), np.asarray(router_output)
        if hidden_states.ndim != 3:
            raise RuntimeError("expert_mlp: hidden_states must be 3D")
        if router_output.ndim != 4 or router_output.shape[3] != 2:
            raise RuntimeError("expert_mlp: router_output must be 4D [batch, seq_len, top_k, 2]")
        B, S, H = hidden_states.shape
        F = int(expert_ffn_dim)
        if not np.any(router_output[..., 0].astype(np.int32) == self.expert_id_):
            return np.zeros((0,), np.float32)
        if H % 32:
            raise RuntimeError(f"expert_mlp: hidden_dim must be a multiple of 32 for MXFP4, got {H}")
        if F % 32:
            raise RuntimeError(f"expert_mlp: expert_ffn_dim must be a multiple of 32 for MXFP4, got {F}")
        k = router_output.shape[2]
        lay = self._get_layer(H, F, b_up is not None, k, B * S, int(router_output[..., 0].max()) + 1)
        lay.load_expert(self.expert_id_, w_up, w_gate, w_down, b_up, b_gate, b_down)
        out = lay.expert_forward(self.expert_id_, hidden_states.reshape(B * S, H),
                                 router_output.reshape(B * S, k, 2))
        return out.reshape(B, S, H)


class dense_ffn_node:
    """dense_ffn_node (dense_ffn_node.h:28-219): the shared expert's dense gated FFN with standard
    SwiGLU; fp16 or fp32 weights (the latter rounded to fp16 on the device: the tensor-core kernel's
    operands), fp32 hidden states and biases.  ``compute(inputs)`` takes the reference's 4 or 7 inputs:
    hidden [B,S,H], gate_w [F,H], up_w [F,H], down_w [H,F] (all float16 or all float32)
    [, gate_b [F], up_b [F], down_b [H]]."""

    def __init__(self, device=0):
        self.device = device
        self._layer = None
        self._key = None

    def compute(self, inputs):
        if len(inputs) not in (4, 7):
            raise RuntimeError("dense_ffn: expected 4 or 7 inputs (hidden, gate_w, up_w, down_w[, gate_b, up_b, "
                               f"down_b]), got {len(inputs)}")
        hidden, gate_w, up_w, down_w = inputs[:4]
        hidden = np.asarray(hidden)
        if hidden.ndim != 3:
            raise RuntimeError(f"dense_ffn: hidden_states must be 3D [B, S, D], got {hidden.ndim}D")
        if any(np.asarray(w).ndim != 2 for w in (gate_w, up_w, down_w)):
            raise RuntimeError("dense_ffn: weight tensors must be 2D")
        wdt = np.asarray(gate_w).dtype
        if wdt not in (np.float16, np.float32) or any(np.asarray(w).dtype != wdt for w in (up_w, down_w)):
            raise RuntimeError("dense_ffn: weight tensors must all be FLOAT16 or all FLOAT32")
        if hidden.dtype != np.float32:
            raise RuntimeError("dense_ffn: hidden_states must be FLOAT32")
        B, S, H = hidden.shape
        F = gate_w.shape[0]
        if gate_w.shape[1] != H or up_w.shape != (F, H):
            raise RuntimeError("dense_ffn: gate_w/up_w shape mismatch")
        if down_w.shape != (H, F):
            raise RuntimeError(f"dense_ffn: down_w shape mismatch, expected [{H}, {F}], got "
                               f"[{down_w.shape[0]}, {down_w.shape[1]}]")
        has_bias = len(inputs) == 7
        key = (H, F, has_bias, id(gate_w), id(up_w), id(down_w))
        T = B * S
        if self._layer is None or self._key != key or self._layer.max_tokens < T:
            if self._layer is not None:
                self._layer.close()
            self._layer = MoeLayer(1, 1, H, F, activation=1, has_bias=has_bias, device=self.device,
                                   max_tokens=max(T, 64), weights_f16=True)
            b = inputs[4:7] if has_bias else (None, None, None)
            # the reference's input order is gate, up, down; biases gate, up, down
            load = self._layer.load_expert_f16 if wdt == np.float16 else self._layer.load_expert_f32
            load(0, up_w, gate_w, down_w, b[1] if has_bias else None, b[0] if has_bias else None,
                 b[2] if has_bias else None)
            self._key = key
        return self._layer.dense_forward(hidden.reshape(T, H)).reshape(B, S, H)

    def close(self):
        if self._layer is not None:
            self._layer.close()
            self._layer = None


class expert_merge_node:
    """expert_merge_node (expert_merge_node.h:9-134)."""

    def __init__(self, device=0):
        self.num_experts_, self.top_k_, self.weight_before_ffn_ = 0, 0, False
        self.device = device

    def set_config(self, num_experts, top_k):
        self.num_experts_, self.top_k_ = int(num_experts), int(top_k)

    def set_weight_before_ffn(self, v):
        self.weight_before_ffn_ = bool(v)

    def compute_test(self, inputs):
        if len(inputs) != self.num_experts_ + 1:
            raise RuntimeError(f"expert_merge: expected {self.num_experts_ + 1} inputs, got {len(inputs)}")
        router = np.asarray(inputs[0])
        if router.ndim != 4 or router.shape[2] != self.top_k_ or router.shape[3] != 2:
            raise RuntimeError(f"expert_merge: router output must have shape [batch, seq_len, {self.top_k_}, 2]")
        B, S = router.shape[:2]
        dense = [a for a in inputs[1:] if np.asarray(a).ndim == 3 and np.asarray(a).shape[0] > 0]
        if not dense:
            raise RuntimeError("expert_merge: no non-empty expert outputs found")
        H = np.asarray(dense[0]).shape[2]
        for a in dense:
            if np.asarray(a).shape != (B, S, H):
                raise RuntimeError("expert_merge: all non-empty expert outputs must have same shape")
        if router.dtype != np.float32:
            raise RuntimeError("expert_merge: only float32 supported")
        Hp = (H + 31) // 32 * 32
        lay = MoeLayer(self.num_experts_, self.top_k_, Hp, 32, has_bias=False,
                       weight_before_ffn=self.weight_before_ffn_, device=self.device, max_tokens=B * S)
        outs = []
        for a in inputs[1:]:
            a = np.asarray(a)
            if a.ndim == 3 and a.shape[0] > 0:
                a = a.reshape(B * S, H).astype(np.float32)
                if Hp != H:
                    a = np.concatenate([a, np.zeros((B * S, Hp - H), np.float32)], axis=1)
                outs.append(a)
            else:
                outs.append(None)
        try:
            out = lay.merge(router.reshape(B * S, self.top_k_, 2), outs)
        finally:
            lay.close()
        return out[:, :H].reshape(B, S, H)
