"""TEST INFRASTRUCTURE ONLY: ctypes bindings of the two CPU checkers.

``port`` is the plain-C restatement (``moe_oracle.c``); ``ref`` is the
unmodified reference compiled behind a C wrapper (``ref_wrapper.cpp``), present
only where ``oracle/_ref/libcsk_ref.so`` was built.  Nothing under the product
package may import this module; tests, the smoke check and the benchmark's CPU
arm do.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import threading

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(_HERE, "libcsk_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libcsk_ref.so")

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)


def reference_root():
    """Root of a reference checkout, or None: $COALSACK_REF, else a directory named
    ``reference`` beside this repository."""
    cands = [os.environ.get("COALSACK_REF"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "include", "coalsack", "nn", "nn_ops", "expert_mlp_node.h")):
            return c
    return None


def build(verbose: bool = False) -> None:
    """Run oracle/Makefile (the C restatement always; the reference wrapper
    when a reference checkout is present)."""
    ref = reference_root()
    r = subprocess.run(["make", "-C", _HERE] + ([f"REF={ref}"] if ref else []), capture_output=True, text=True)
    if verbose or r.returncode:
        print(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError("oracle build failed")


def _fp(a):
    return None if a is None else a.ctypes.data_as(_f32p)


def _bp(a):
    return None if a is None else a.ctypes.data_as(_u8p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.uint8)


def _ptr_array(arrs, ctype):
    """C array of pointers to the given numpy arrays (None -> NULL array)."""
    if arrs is None:
        return None, None
    keep = [np.ascontiguousarray(a) for a in arrs]
    arr = (C.c_void_p * len(keep))(*[a.ctypes.data for a in keep])
    return arr, keep


class _Lib:
    """Common surface of both checkers; ``prefix`` is ``orc_`` or ``ref_``."""

    def __init__(self, path: str, prefix: str):
        self.lib = C.CDLL(path)
        self.prefix = prefix
        self.is_ref = prefix == "ref_"
        L = self.lib
        self._e8m0 = getattr(L, "orc_e8m0_half" if not self.is_ref else "ref_e8m0_to_fp32_half")
        self._e8m0.restype = C.c_float
        self._e8m0.argtypes = [C.c_uint8]
        self._deq = getattr(L, "orc_dequant_mxfp4" if not self.is_ref else "ref_dequantize_block_mxfp4")
        self._deq.restype = None
        self._deq.argtypes = [_u8p, _f32p, C.c_int64]
        self._router = getattr(L, prefix + "router")
        self._router.restype = C.c_int
        self._router.argtypes = [_f32p, C.c_int64, C.c_int64, _f32p, _f32p, C.c_int64, C.c_int64,
                                 C.c_int, _f32p] + ([] if self.is_ref else [_f32p])
        self._tok = getattr(L, prefix + "expert_token_mxfp4")
        self._tok.restype = C.c_int
        self._tok.argtypes = [_f32p, _u8p, _u8p, _u8p, _f32p, _f32p, _f32p, _f32p, C.c_int64,
                              C.c_int64, C.c_int]
        self._node = getattr(L, prefix + "expert_node_mxfp4")
        self._node.restype = C.c_int
        self._node.argtypes = [C.c_int, _f32p, C.c_int64, C.c_int64, C.c_int64, _u8p, _u8p, _u8p,
                               _f32p, _f32p, _f32p, _f32p, C.c_int64, C.c_int, C.c_int, _f32p]
        self._merge = getattr(L, prefix + "merge")
        self._merge.restype = C.c_int
        self._merge.argtypes = [_f32p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                C.c_int, _f32p]
        self._rms = getattr(L, prefix + "rmsnorm")
        self._rms.restype = C.c_int
        self._rms.argtypes = [_f32p, _f32p, C.c_float, _f32p, C.c_int64, C.c_int64]
        self._dense = getattr(L, prefix + "dense_ffn_f16")
        self._dense.restype = C.c_int
        self._dense.argtypes = [_f32p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                C.c_void_p, C.c_void_p, C.c_void_p, _f32p]
        self._dense32 = getattr(L, prefix + "dense_ffn_f32")
        self._dense32.restype = C.c_int
        self._dense32.argtypes = [_f32p, C.c_int64, C.c_int64, C.c_int64, _f32p, _f32p, _f32p,
                                  C.c_void_p, C.c_void_p, C.c_void_p, _f32p]
        if self.is_ref:
            self._kq = L.ref_dequant_kquant_f16
            self._kq.restype = C.c_int
            self._kq.argtypes = [C.c_int, _u8p, C.c_int64, C.c_void_p]
        else:
            self._kq4, self._kq6 = L.orc_dequant_q4k_f16, L.orc_dequant_q6k_f16
            for fn in (self._kq4, self._kq6):
                fn.restype = C.c_int
                fn.argtypes = [_u8p, C.c_int64, C.c_void_p, C.c_int]
        self._layer = getattr(L, prefix + "moe_layer")
        self._layer.restype = C.c_int
        if self.is_ref:
            L.ref_last_error.restype = C.c_char_p
            self._layer.argtypes = [_f32p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                    _f32p, _f32p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                    C.c_int, _f32p, _f32p]
        else:
            self._layer.argtypes = [_f32p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                    C.c_int64, _f32p, _f32p, C.c_int, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                    C.c_int, C.c_int, _f32p, _f32p]

    def _err(self, rc, what):
        msg = self.lib.ref_last_error().decode() if self.is_ref else f"code {rc}"
        raise RuntimeError(f"{what}: {msg}")

    # --- codec -----------------------------------------------------------
    def e8m0(self, x: int) -> float:
        return float(self._e8m0(x))

    def dequant(self, blocks: np.ndarray) -> np.ndarray:
        blocks = _u8(blocks).reshape(-1)
        n = blocks.size // 17 * 32
        out = np.empty(n, np.float32)
        self._deq(_bp(blocks), _fp(out), n)
        return out

    # --- router ----------------------------------------------------------
    def router(self, hidden, Wg, bias, k, sigmoid=False):
        hidden, Wg, bias = _f32(hidden), _f32(Wg), _f32(bias)
        T, H = hidden.shape
        E = Wg.shape[0]
        out = np.empty((T, k, 2), np.float32)
        args = [_fp(hidden), T, H, _fp(Wg), _fp(bias), E, k, int(sigmoid), _fp(out)]
        if not self.is_ref:
            args.append(None)
        rc = self._router(*args)
        if rc:
            self._err(rc, "router")
        return out

    def router_logits(self, hidden, Wg, bias, k):
        """(router_out, logits[T,E]) -- restatement only."""
        assert not self.is_ref
        hidden, Wg, bias = _f32(hidden), _f32(Wg), _f32(bias)
        T, H = hidden.shape
        E = Wg.shape[0]
        out = np.empty((T, k, 2), np.float32)
        lg = np.empty((T, E), np.float32)
        rc = self._router(_fp(hidden), T, H, _fp(Wg), _fp(bias), E, k, 0, _fp(out), _fp(lg))
        if rc:
            self._err(rc, "router")
        return out, lg

    def rmsnorm(self, x, w, eps=1e-5):
        """RMSNorm over the last dimension of x [T,H] with weight [H]."""
        x, w = _f32(x), _f32(w)
        out = np.empty_like(x)
        rc = self._rms(_fp(x), _fp(w), float(eps), _fp(out), x.shape[0], x.shape[1])
        if rc:
            self._err(rc, "rmsnorm")
        return out

    def dense_ffn(self, hidden, gate_w, up_w, down_w, gate_b=None, up_b=None, down_b=None):
        """dense_ffn_node: hidden [T,H] fp32; gate_w, up_w [F,H], down_w [H,F] all float16 or all float32;
        biases fp32 or None."""
        hidden = _f32(hidden)
        T, H = hidden.shape
        if np.asarray(gate_w).dtype == np.float32:
            w = [_f32(a) for a in (gate_w, up_w, down_w)]
            F = w[0].shape[0]
            b = [None if a is None else _f32(a) for a in (gate_b, up_b, down_b)]
            out = np.empty((T, H), dtype=np.float32)
            rc = self._dense32(_fp(hidden), T, H, F, *[_fp(a) for a in w],
                               *[None if a is None else a.ctypes.data for a in b], _fp(out))
            if rc:
                self._err(rc, "dense_ffn")
            return out
        w = [np.ascontiguousarray(np.asarray(a).view(np.uint16) if np.asarray(a).dtype == np.float16 else a,
                                  dtype=np.uint16) for a in (gate_w, up_w, down_w)]
        F = w[0].shape[0]
        b = [None if a is None else _f32(a) for a in (gate_b, up_b, down_b)]
        out = np.empty((T, H), dtype=np.float32)
        rc = self._dense(_fp(hidden), T, H, F, *[a.ctypes.data for a in w],
                         *[None if a is None else a.ctypes.data for a in b], _fp(out))
        if rc:
            self._err(rc, "dense_ffn")
        return out

    # --- expert ----------------------------------------------------------
    def dequant_kquant(self, ggml_type: int, blocks: np.ndarray, n: int, nearest: bool = False) -> np.ndarray:
        """Q4_K (12) or Q6_K (14) super-blocks to the fp16 values the weight provider makes of them
        (moe_weight_provider.cpp:17-33); n values, a multiple of 256.  ``nearest`` (restatement only): the
        reference's F16C build of fp32_to_fp16 instead of the portable one its build flags select."""
        if ggml_type not in (12, 14):
            raise ValueError("ggml_type must be 12 (Q4_K) or 14 (Q6_K)")
        blocks = _u8(blocks).reshape(-1)
        assert n % 256 == 0 and blocks.size == n // 256 * (144 if ggml_type == 12 else 210)
        out = np.empty(n, np.uint16)
        if self.is_ref:
            if nearest:
                raise ValueError("the compiled reference is the portable build")
            rc = self._kq(ggml_type, _bp(blocks), n, out.ctypes.data)
        else:
            rc = (self._kq4 if ggml_type == 12 else self._kq6)(_bp(blocks), n, out.ctypes.data, int(nearest))
        if rc:
            self._err(rc, "dequant_kquant")
        return out.view(np.float16)

    def expert_token(self, x, w_up, w_gate, w_down, b_up, b_gate, b_down, H, F, act):
        x = _f32(x)
        out = np.empty(H, np.float32)
        w_up, w_gate, w_down = _u8(w_up), _u8(w_gate), _u8(w_down)
        b_up, b_gate, b_down = _f32(b_up), _f32(b_gate), _f32(b_down)
        rc = self._tok(_fp(x), _bp(w_up), _bp(w_gate), _bp(w_down), _fp(b_up), _fp(b_gate),
                       _fp(b_down), _fp(out), H, F, act)
        if rc:
            self._err(rc, "expert_token")
        return out

    def expert_node(self, expert_id, hidden, w_up, w_gate, w_down, b_up, b_gate, b_down,
                    router_out, F, act, weight_before_ffn=False):
        """Dense [T,H] node output, or None for the {0}-shaped empty tensor."""
        hidden, router_out = _f32(hidden), _f32(router_out)
        T, H = hidden.shape
        k = router_out.shape[1]
        w_up, w_gate, w_down = _u8(w_up), _u8(w_gate), _u8(w_down)
        b_up, b_gate, b_down = _f32(b_up), _f32(b_gate), _f32(b_down)
        out = np.empty((T, H), np.float32)
        rc = self._node(expert_id, _fp(hidden), T, H, F, _bp(w_up), _bp(w_gate), _bp(w_down),
                        _fp(b_up), _fp(b_gate), _fp(b_down), _fp(router_out), k, act,
                        int(weight_before_ffn), _fp(out))
        if rc < 0:
            self._err(rc, "expert_node")
        return out if rc == 1 else None

    # --- merge -----------------------------------------------------------
    def merge(self, router_out, expert_outs, H, weight_before_ffn=False):
        router_out = _f32(router_out)
        T, k = router_out.shape[:2]
        E = len(expert_outs)
        keep = [None if a is None else _f32(a) for a in expert_outs]
        ptrs = (C.c_void_p * E)(*[None if a is None else a.ctypes.data for a in keep])
        out = np.empty((T, H), np.float32)
        rc = self._merge(_fp(router_out), T, k, E, H, ptrs, int(weight_before_ffn), _fp(out))
        if rc:
            self._err(rc, "merge")
        return out

    # --- whole layer -----------------------------------------------------
    def moe_layer(self, hidden, Wg, router_bias, experts, k, act, sigmoid=False,
                  weight_before_ffn=False, nthreads=1, router_out=None):
        """experts: dict with lists 'w_up','w_gate','w_down' ([E] uint8 arrays of
        17-byte blocks) and optionally 'b_up','b_gate','b_down' ([E] fp32).
        Returns (out[T,H], router_out[T,k,2])."""
        hidden, Wg, router_bias = _f32(hidden), _f32(Wg), _f32(router_bias)
        T, H = hidden.shape
        E = Wg.shape[0]
        F = experts["w_up"][0].size // 17 * 32 // H
        pu, k1 = _ptr_array(experts["w_up"], _u8p)
        pg, k2 = _ptr_array(experts["w_gate"], _u8p)
        pd, k3 = _ptr_array(experts["w_down"], _u8p)
        has_b = experts.get("b_up") is not None
        bu, k4 = _ptr_array([_f32(b) for b in experts["b_up"]] if has_b else None, _f32p)
        bg, k5 = _ptr_array([_f32(b) for b in experts["b_gate"]] if has_b else None, _f32p)
        bd, k6 = _ptr_array([_f32(b) for b in experts["b_down"]] if has_b else None, _f32p)
        compute_router = router_out is None
        r = np.empty((T, k, 2), np.float32) if compute_router else _f32(router_out).copy()
        out = np.empty((T, H), np.float32)
        if self.is_ref:
            rc = self._layer(_fp(hidden), T, H, F, E, k, _fp(Wg), _fp(router_bias), int(sigmoid),
                             pu, pg, pd, bu, bg, bd, act, int(weight_before_ffn), nthreads,
                             int(compute_router), _fp(r), _fp(out))
            if rc:
                self._err(rc, "moe_layer")
        else:
            # the restatement is single-threaded C; fan token ranges out here
            nthreads = max(1, min(nthreads, T))
            bounds = np.linspace(0, T, nthreads + 1).astype(np.int64)
            rcs = [0] * nthreads

            def run(i):
                rcs[i] = self._layer(_fp(hidden), int(bounds[i]), int(bounds[i + 1]), H, F, E, k,
                                     _fp(Wg), _fp(router_bias), int(sigmoid), pu, pg, pd, bu, bg,
                                     bd, act, int(weight_before_ffn), int(compute_router), _fp(r),
                                     _fp(out))

            ths = [threading.Thread(target=run, args=(i,)) for i in range(1, nthreads)]
            for th in ths:
                th.start()
            run(0)
            for th in ths:
                th.join()
            if any(rcs):
                self._err(max(rcs, key=abs), "moe_layer")
        return out, r


_port = None
_ref = None


def port() -> _Lib:
    global _port
    if _port is None:
        if not os.path.exists(PORT_SO):
            build()
        _port = _Lib(PORT_SO, "orc_")
    return _port


def have_ref() -> bool:
    return os.path.exists(REF_SO)


def ref() -> _Lib:
    global _ref
    if _ref is None:
        if not have_ref():
            raise RuntimeError("oracle/_ref/libcsk_ref.so is not built (needs the reference checkout)")
        _ref = _Lib(REF_SO, "ref_")
    return _ref
