"""The certified fast router against the CPU restatement of the reference's sequential-chain router:
expert indices must be identical for every token, whichever of the two passes (fast logits accepted by
their error bounds, or the chain for the tokens they cannot separate) produced them."""
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

from coalsack_b200 import MoeLayer, synth

pytestmark = pytest.mark.gpu


def _router_layer(E, k, H, Wg, rb, max_tokens, sigmoid=False):
    """A router-only layer with the certified pass switched on for every batch size (the default mode
    keeps it for batches of up to four tokens)."""
    lay = MoeLayer(E, k, H, 32, has_bias=False, sigmoid_gating=sigmoid, max_tokens=max_tokens)
    lay.set_router(Wg, rb)
    lay.set_router_mode(lay.ROUTER_CERTIFIED)
    return lay


def _cpu_router(port, h, Wg, rb, k, threads=16):
    parts = np.array_split(np.arange(h.shape[0]), threads)
    with ThreadPoolExecutor(threads) as ex:
        outs = list(ex.map(lambda idx: port.router(h[idx], Wg, rb, k) if len(idx) else np.zeros((0, k, 2), np.float32), parts))
    return np.concatenate(outs)


def test_certified_router_49152_tokens_of_the_120b_shape(gpu_lib, port):
    """49 152 tokens on the 128-expert router, routed in decode-sized batches of 1 to 128 tokens through
    the certified pass: indices bit-exact, routing weights within 2e-6, and only a few percent of
    the tokens needed the chain.  Then one 8192-token batch in each of the three modes."""
    import torch
    sh = synth.C2
    E, k, H = sh.num_experts, sh.top_k, sh.hidden
    Wg, rb = synth.router_weight(sh), synth.router_bias(sh)
    lay = _router_layer(E, k, H, Wg, rb, 8192)
    sizes = [128, 64, 32, 16, 8, 4, 2, 1, 100, 29]
    for rep in range(6):
        h = synth.hidden_states(sh, 8192, rep=rep)
        h_d = torch.from_numpy(h).cuda()
        ro_d = torch.empty((8192, k, 2), dtype=torch.float32, device="cuda")
        pos, i = 0, 0
        while pos < 8192:
            n = min(sizes[i % len(sizes)] if rep == 0 else 128, 8192 - pos)
            lay.route_dev(h_d[pos:pos + n], n, ro_d[pos:pos + n])
            pos += n
            i += 1
        torch.cuda.synchronize()
        lay.sync()
        got = ro_d.cpu().numpy()
        want = _cpu_router(port, h, Wg, rb, k)
        assert np.array_equal(got[..., 0], want[..., 0]), f"batch {rep}: expert indices differ"
        assert np.allclose(got[..., 1], want[..., 1], atol=2e-6)
    routed, chained = lay.router_stats()
    assert routed == 6 * 8192
    assert 0 < chained < 0.08 * routed, (routed, chained)
    print(f"certified router: {chained} of {routed} tokens recomputed by the chain ({100.0 * chained / routed:.2f} %)")
    for mode in (lay.ROUTER_CERTIFIED, lay.ROUTER_CHAIN, lay.ROUTER_AUTO):   # a prefill-sized batch in every mode
        lay.set_router_mode(mode)
        h = synth.hidden_states(sh, 8192, rep=7)
        got = lay.route(h)
        want = _cpu_router(port, h, Wg, rb, k)
        assert np.array_equal(got[..., 0], want[..., 0]) and np.allclose(got[..., 1], want[..., 1], atol=2e-6)
    lay.set_router_mode(lay.ROUTER_CHAIN)
    h = synth.hidden_states(sh, 64, rep=8)
    assert np.array_equal(lay.route(h)[..., 0], port.router(h, Wg, rb, k)[..., 0])
    lay.close()


@pytest.mark.parametrize("T", [1, 3, 8, 37, 64, 128, 700])
def test_certified_router_small_batches(gpu_lib, port, T):
    """Decode-sized and ragged batches, sigmoid gating included, on the C4 router (no bias, top-8)."""
    sh = synth.C4
    E, k, H = sh.num_experts, sh.top_k, sh.hidden
    Wg = synth.router_weight(sh)
    for sigmoid in (False, True):
        lay = _router_layer(E, k, H, Wg, None, 1024, sigmoid=sigmoid)
        for rep in range(3):
            h = synth.hidden_states(sh, T, rep=10 * T + rep)
            got = lay.route(h)
            want = port.router(h, Wg, None, k, sigmoid)
            assert np.array_equal(got[..., 0], want[..., 0]), (T, rep, sigmoid)
            assert np.allclose(got[..., 1], want[..., 1], atol=2e-6)
        lay.close()


def test_near_ties_take_the_chain_and_still_match(gpu_lib, port):
    """Gate rows in near-duplicate pairs (a tenth of the elements moved by parts in 2^-14, so the twins'
    logits differ by about 1e-5): for most tokens two of the best logits are closer than any error bound,
    the selection cannot be certified and the chain decides.  Tokens whose CPU logits tie exactly among the
    k+1 best are left out (the reference's order is unspecified there, moe_router_node.h:175-177)."""
    rng = np.random.default_rng(5)
    E, k, H, T = 64, 4, 1024, 128
    base = (rng.standard_normal((E // 2, H)) * 0.05).astype(np.float32)
    twin = base.copy()
    move = rng.random((E // 2, H)) < 0.1
    twin[move] *= np.float32(1.0 + 2.0 ** -14)
    Wg = np.ascontiguousarray(np.stack([base, twin], axis=1).reshape(E, H))
    rb = (rng.standard_normal(E) * 0.01).astype(np.float32)
    rb[1::2] = rb[0::2]
    h = rng.standard_normal((T, H)).astype(np.float32)
    lay = _router_layer(E, k, H, Wg, rb, T)
    got = lay.route(h)
    routed, chained = lay.router_stats()
    assert routed == T and chained > T // 2, (routed, chained)
    want, logits = port.router_logits(h, Wg, rb, k)
    top = -np.sort(-logits, axis=1)[:, :k + 1]
    clean = np.all(top[:, :-1] != top[:, 1:], axis=1)
    assert clean.sum() > T // 2
    assert np.array_equal(got[clean][..., 0], want[clean][..., 0])
    lay.close()
