"""The allocation-free routing entry point (csk_moe_route_static) against the
handle-based one (csk_moe_route_dev), through the C ABI.

It exists for hosts that cannot call cudaMalloc at this point: the GPU's memory
already belongs to someone else's pool, or the calling thread must not wait on
the allocator.  Its scratch is a fixed array inside the library, shared by all
calls, so the check runs two different batches back to back: the second must
not see anything of the first.  Collected last on purpose (file name), and it
passes alone in a fresh process as well as after every other test.
"""
import ctypes as C

import numpy as np
import pytest

from coalsack_b200 import MoeLayer, _lib, synth

pytestmark = pytest.mark.gpu


def _route_both(lib, layer, hidden_np, Wg_d, rb_d, E, k, torch):
    T, H = hidden_np.shape
    h_d = torch.from_numpy(hidden_np).cuda()
    want = torch.empty((T, k, 2), dtype=torch.float32, device="cuda")
    got = torch.full((T, k, 2), -1.0, dtype=torch.float32, device="cuda")
    layer.route_dev(h_d, T, want)
    rc = lib.csk_moe_route_static(h_d.data_ptr(), T, H, Wg_d.data_ptr(), rb_d.data_ptr() if rb_d is not None else None,
                                  E, k, 0, got.data_ptr(), None)
    assert rc == 0, lib.csk_moe_last_error(None).decode()
    torch.cuda.synchronize()
    return got.cpu().numpy(), want.cpu().numpy()


def test_route_static_matches_handle_router_twice(gpu_lib):
    import torch
    torch.cuda.set_device(0)
    lib = _lib.load()
    sh = synth.C2.with_(tokens=192)
    E, k, H = sh.num_experts, sh.top_k, sh.hidden
    Wg, rb = synth.router_weight(sh), synth.router_bias(sh)
    layer = MoeLayer(E, k, H, 32, has_bias=False, max_tokens=192)
    layer.set_router(Wg, rb)
    Wg_d, rb_d = torch.from_numpy(Wg).cuda(), torch.from_numpy(rb).cuda()
    # two calls in a row on different batches (prefill-sized tiling, then decode-sized)
    for rep, T in ((0, 192), (1, 7)):
        hidden = synth.hidden_states(sh, T, rep=rep)
        got, want = _route_both(lib, layer, hidden, Wg_d, rb_d, E, k, torch)
        assert np.array_equal(got[..., 0], want[..., 0]), f"call {rep}: expert ids differ"
        assert np.allclose(got[..., 1], want[..., 1], atol=2e-6), f"call {rep}: routing weights differ"
    layer.close()


def test_route_static_rejects_oversize(gpu_lib):
    import torch
    lib = _lib.load()
    x = torch.zeros(64, device="cuda")
    p = x.data_ptr()
    # 4096 tokens x 128 experts is twice the built-in scratch
    assert lib.csk_moe_route_static(p, 4096, 64, p, None, 128, 4, 0, p, None) == -4
    assert b"exceeds the built-in scratch" in lib.csk_moe_last_error(None)
    assert lib.csk_moe_route_static(p, 8, 48, p, None, 8, 2, 0, p, None) == -1
    assert lib.csk_moe_route_static(None, 8, 64, p, None, 8, 2, 0, p, None) == -1
