"""The allocation-free routing entry point (csk_moe_route_static), through the C
ABI, against the CPU restatement of the reference router and against the
handle-based entry point (csk_moe_route_dev).

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


def _route_static(lib, hidden_np, Wg_d, rb_d, E, k, torch):
    T, H = hidden_np.shape
    h_d = torch.from_numpy(hidden_np).cuda()
    got = torch.full((T, k, 2), -1.0, dtype=torch.float32, device="cuda")
    rc = lib.csk_moe_route_static(h_d.data_ptr(), T, H, Wg_d.data_ptr(), rb_d.data_ptr() if rb_d is not None else None,
                                  E, k, 0, got.data_ptr(), None)
    assert rc == 0, lib.csk_moe_last_error(None).decode()
    torch.cuda.synchronize()
    assert lib.csk_moe_route_static_status() == 0, lib.csk_moe_last_error(None).decode()
    return got.cpu().numpy(), h_d


def test_route_static_matches_checker_and_handle_router_twice(gpu_lib, port):
    import torch
    torch.cuda.set_device(0)
    lib = _lib.load()
    sh = synth.C2.with_(tokens=192)
    E, k, H = sh.num_experts, sh.top_k, sh.hidden
    Wg, rb = synth.router_weight(sh), synth.router_bias(sh)
    layer = MoeLayer(E, k, H, 32, has_bias=False, max_tokens=192)
    layer.set_router(Wg, rb)
    Wg_d, rb_d = torch.from_numpy(Wg).cuda(), torch.from_numpy(rb).cuda()
    # two calls in a row on different batches (prefill-sized tiling, then decode-sized): the second must see
    # nothing of the first in the shared scratch
    for rep, T in ((0, 192), (1, 7)):
        hidden = synth.hidden_states(sh, T, rep=rep)
        got, h_d = _route_static(lib, hidden, Wg_d, rb_d, E, k, torch)
        want = port.router(hidden, Wg, rb, k)                     # the CPU restatement of the reference router
        assert np.array_equal(got[..., 0], want[..., 0]), f"call {rep}: expert ids differ from the checker"
        assert np.allclose(got[..., 1], want[..., 1], atol=2e-6), f"call {rep}: routing weights differ"
        via_handle = torch.empty((T, k, 2), dtype=torch.float32, device="cuda")
        layer.route_dev(h_d, T, via_handle)
        torch.cuda.synchronize()
        assert np.array_equal(got[..., 0], via_handle.cpu().numpy()[..., 0]), f"call {rep}: differs from csk_moe_route_dev"
    layer.close()


def test_route_static_allocates_nothing(gpu_lib):
    """After the first (address-resolving) call, further calls leave the device's free memory unchanged."""
    import torch
    torch.cuda.set_device(0)
    lib = _lib.load()
    sh = synth.C2.with_(tokens=64)
    E, k, H = sh.num_experts, sh.top_k, sh.hidden
    Wg_d = torch.from_numpy(synth.router_weight(sh)).cuda()
    h_d = torch.from_numpy(synth.hidden_states(sh, 64)).cuda()
    out = torch.empty((64, k, 2), dtype=torch.float32, device="cuda")
    call = lambda: lib.csk_moe_route_static(h_d.data_ptr(), 64, H, Wg_d.data_ptr(), None, E, k, 0, out.data_ptr(), None)
    assert call() == 0
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0


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
