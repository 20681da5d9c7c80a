"""The expert-parallel stages of the C ABI (dispatch / experts / combine) on ONE
GPU: N ranks are N handles in one process and the two all-to-all exchanges are
plain slice copies, run one after the other (nothing here waits on another
kernel).  Result must match the single-device layer and the CPU checker."""
import numpy as np
import pytest

from coalsack_b200 import MoeLayer, PATH_STREAM, PATH_TILE, synth
from tests import cases

pytestmark = pytest.mark.gpu


def run_emulated_ep(torch, sh, N, tokens, Wg, rb, ex, path, slot_map=None):
    E, k, H = sh.num_experts, sh.top_k, sh.hidden
    eloc = E // N
    dev = torch.device("cuda", 0)
    layers, hs = [], []
    for r in range(N):
        lay = MoeLayer.from_shape(sh, max_tokens=max(sum(tokens), 1), expert_begin=r * eloc, expert_count=eloc)
        if slot_map is not None:
            lay.ep_set_slot_map(*slot_map)
        lay.set_router(Wg, rb)
        lay.load_experts({n: (None if ex.get(n) is None else ex[n][r * eloc:(r + 1) * eloc])
                          for n in ("w_up", "w_gate", "w_down", "b_up", "b_gate", "b_down")},
                         ids=range(r * eloc, (r + 1) * eloc))
        lay.set_path(path)
        layers.append(lay)
        hs.append(torch.from_numpy(synth.hidden_states(sh, tokens[r], rep=r)).to(dev))
    pitch = layers[0].ep_row_pitch()
    send = [torch.zeros((tokens[r] * k, pitch), dtype=torch.float16, device=dev) for r in range(N)]
    counts = [torch.zeros(E, dtype=torch.int32, device=dev) for _ in range(N)]
    for r in range(N):
        layers[r].ep_dispatch_dev(hs[r], tokens[r], send[r], counts[r])
    torch.cuda.synchronize()
    cn = np.stack([c.cpu().numpy() for c in counts])             # [src, expert]
    offs = np.concatenate([np.zeros((N, 1), np.int64), np.cumsum(cn, axis=1)], axis=1)
    outs = []
    rets = []
    for d in range(N):                                            # destination rank d receives from every src
        segs = [send[s][offs[s, d * eloc]:offs[s, (d + 1) * eloc]] for s in range(N)]
        recv = torch.cat(segs) if segs else send[0][:0]
        rc = torch.from_numpy(np.ascontiguousarray(cn[:, d * eloc:(d + 1) * eloc]).astype(np.int32)).to(dev)
        total = recv.shape[0]
        ret = torch.zeros((max(total, 1), H), dtype=torch.float32, device=dev)
        if total:
            layers[d].ep_experts_dev(recv.contiguous(), rc, N, total, ret)
            layers[d].sync()
        rets.append((ret, [s.shape[0] for s in segs]))
    for s in range(N):                                            # rows travel back in the order they were sent
        parts = []
        for d in range(N):
            ret, lens = rets[d]
            start = sum(lens[:s])
            parts.append(ret[start:start + lens[s]])
        back = torch.cat(parts).contiguous()
        assert back.shape[0] == tokens[s] * k
        out = torch.empty((tokens[s], H), dtype=torch.float32, device=dev)
        ro = torch.empty((tokens[s], k, 2), dtype=torch.float32, device=dev)
        layers[s].ep_combine_dev(back, tokens[s], out, ro)
        torch.cuda.synchronize()
        outs.append((out.cpu().numpy(), ro.cpu().numpy(), hs[s].cpu().numpy()))
    for lay in layers:
        lay.close()
    return outs


@pytest.mark.parametrize("path", [PATH_STREAM, PATH_TILE])
@pytest.mark.parametrize("N,tokens", [(2, (37, 64)), (4, (3, 0 + 1, 50, 9))])
def test_emulated_ep_matches_checker(gpu_lib, port, path, N, tokens):
    import torch
    sh = synth.tiny(seed=81, E=8, k=3, H=192, F=160, T=1, has_bias=True)
    _, Wg, rb, ex = cases.layer_inputs(sh, router_scale=40.0)
    for out, ro, h in run_emulated_ep(torch, sh, N, tokens, Wg, rb, ex, path):
        want, want_ro = port.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, nthreads=4)
        assert np.array_equal(ro[..., 0], want_ro[..., 0])
        mx, mr = cases.err_stats(out, want)
        assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (path, N, mx, mr)


@pytest.mark.parametrize("path", [PATH_STREAM, PATH_TILE])
def test_emulated_ep_with_replicated_experts(gpu_lib, port, path):
    """Two ranks, five slots each for eight experts: the planner gives the heaviest experts a
    second copy; odd tokens go there.  Output and routing (logical ids) must match the checker."""
    import torch
    from coalsack_b200.ep import plan_placement
    sh = synth.tiny(seed=83, E=8, k=3, H=192, F=160, T=1, has_bias=True)
    _, Wg, rb, ex = cases.layer_inputs(sh, router_scale=40.0)
    load = np.array([900, 100, 90, 80, 70, 60, 50, 40])
    pl = plan_placement(load, 2, extra_slots=1)
    assert (pl.replica_of >= 0).any() and pl.n_slots == 10
    copies = set(int(s) for s in pl.replica_of if s >= 0)
    primary = -np.ones(8, dtype=np.int32)
    replica = -np.ones(8, dtype=np.int32)
    for p, e in enumerate(pl.slots):
        if e >= 0 and p not in copies:
            primary[e], replica[e] = p, pl.replica_of[p]
    src = np.where(pl.slots >= 0, pl.slots, 0)           # empty slots carry some expert's weights, never routed
    exp = {n: (None if ex.get(n) is None else [ex[n][e] for e in src]) for n in ex}
    shp = sh.with_(num_experts=pl.n_slots)
    tokens = (37, 64)
    for out, ro, h in run_emulated_ep(torch, shp, 2, tokens, Wg, rb, exp, path, slot_map=(primary, replica)):
        want, want_ro = port.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, nthreads=4)
        assert np.array_equal(ro[..., 0], want_ro[..., 0])
        mx, mr = cases.err_stats(out, want)
        assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (path, mx, mr)


def run_emulated_p2p(torch, sh, N, tokens, Wg, rb, ex, path, slot_map=None):
    """N ranks as N handles on one GPU; the peers' buffers are exchanged as raw pointers and the
    stages run in lockstep (all ranks' scatter, then all ranks' experts, ...), so no kernel ever
    waits for another."""
    E, k, H = sh.num_experts, sh.top_k, sh.hidden
    eloc = E // N
    dev = torch.device("cuda", 0)
    cap = max(sum(tokens), 1)
    layers, hs = [], []
    for r in range(N):
        lay = MoeLayer.from_shape(sh, max_tokens=cap, expert_begin=r * eloc, expert_count=eloc)
        if slot_map is not None:
            lay.ep_set_slot_map(*slot_map)
        lay.set_router(Wg, rb)
        lay.load_experts({n: (None if ex.get(n) is None else ex[n][r * eloc:(r + 1) * eloc])
                          for n in ("w_up", "w_gate", "w_down", "b_up", "b_gate", "b_down")},
                         ids=range(r * eloc, (r + 1) * eloc))
        lay.set_path(path)
        layers.append(lay)
        hs.append(torch.from_numpy(synth.hidden_states(sh, tokens[r], rep=r)).to(dev))
    ptrs = [lay.ep_p2p_local_ptrs() for lay in layers]
    for r, lay in enumerate(layers):
        lay.ep_p2p_import_ptrs(r, N, [p[0] for p in ptrs], [p[1] for p in ptrs], [p[2] for p in ptrs])
    counts = [torch.zeros(E, dtype=torch.int32, device=dev) for _ in range(N)]
    for r in range(N):
        if tokens[r]:
            layers[r].ep_p2p_counts_dev(hs[r], tokens[r], counts[r])
    torch.cuda.synchronize()
    all_counts = torch.cat(counts).contiguous()
    for r in range(N):
        if tokens[r]:
            layers[r].ep_p2p_scatter_dev(hs[r], tokens[r], all_counts)
    torch.cuda.synchronize()
    for r in range(N):
        layers[r].ep_p2p_experts_dev(all_counts, max(1, sum(tokens) * k // N))
        layers[r].sync()
    outs = []
    for r in range(N):
        if not tokens[r]:
            continue
        out = torch.empty((tokens[r], H), dtype=torch.float32, device=dev)
        ro = torch.empty((tokens[r], k, 2), dtype=torch.float32, device=dev)
        layers[r].ep_p2p_combine_dev(tokens[r], out, ro)
        torch.cuda.synchronize()
        outs.append((out.cpu().numpy(), ro.cpu().numpy(), hs[r].cpu().numpy()))
    for lay in layers:
        lay.close()
    return outs


@pytest.mark.parametrize("path", [PATH_STREAM, PATH_TILE])
@pytest.mark.parametrize("N,tokens", [(2, (37, 64)), (4, (3, 1, 50, 9)), (2, (0, 40))])
def test_emulated_p2p_matches_checker(gpu_lib, port, path, N, tokens):
    import torch
    sh = synth.tiny(seed=85, E=8, k=3, H=192, F=160, T=1, has_bias=True)
    _, Wg, rb, ex = cases.layer_inputs(sh, router_scale=40.0)
    for out, ro, h in run_emulated_p2p(torch, sh, N, tokens, Wg, rb, ex, path):
        want, want_ro = port.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, nthreads=4)
        assert np.array_equal(ro[..., 0], want_ro[..., 0])
        mx, mr = cases.err_stats(out, want)
        assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (path, N, mx, mr)


@pytest.mark.parametrize("base", ["c2", "c4"])
def test_emulated_p2p_128_experts_16_per_rank_with_slot_map(gpu_lib, port, base):
    """The 128-expert shapes over eight emulated ranks, sixteen slots each, placed by the planner from a
    calibration batch (so logical expert ids and slots differ), peer-memory step, tensor-core and
    streaming kernels, against the checker."""
    import torch
    from coalsack_b200.ep import calibration_load, plan_placement
    N, per_rank = 8, 24
    sh = synth.CONFIGS[base].with_(tokens=per_rank)
    Wg, rb = synth.router_weight(sh), synth.router_bias(sh)
    load = sum(calibration_load(sh, synth.hidden_states(sh, per_rank, rep=r)) for r in range(N))
    pl = plan_placement(load, N, extra_slots=0)
    assert pl.n_slots == 128 and not np.array_equal(pl.slots, np.arange(128))
    ex = synth.all_experts(sh)
    exp = {n: (None if ex.get(n) is None else [ex[n][e] for e in pl.slots]) for n in ex}   # slot order
    tokens = (per_rank,) * N
    for path in (PATH_TILE, PATH_STREAM):
        for out, ro, h in run_emulated_p2p(torch, sh, N, tokens, Wg, rb, exp, path, slot_map=pl.slot_map(128)):
            want, want_ro = port.moe_layer(h, Wg, rb, ex, sh.top_k, sh.act, nthreads=16)
            assert np.array_equal(ro[..., 0], want_ro[..., 0])
            mx, mr = cases.err_stats(out, want)
            assert mx <= cases.MAX_ABS_OVER_RMS and mr <= cases.MEAN_REL, (base, path, mx, mr)


def test_emulated_p2p_overflow_is_a_status_not_a_fault(gpu_lib):
    """Every token of both ranks routes to rank 0's experts, which therefore receives twice the rows its
    buffers hold (max_tokens * top_k).  Senders skip the rows that do not fit, the row plan is flagged,
    the receive side derives no output pointers from it, and csk_moe_sync reports CSK_ERR_NOMEM on every
    rank.  Canary rows after each rank's used part of the output stay untouched."""
    import torch
    from coalsack_b200 import CskError
    sh = synth.tiny(seed=87, E=8, k=2, H=192, F=160, T=1, has_bias=True)
    _, Wg, rb, ex = cases.layer_inputs(sh, router_scale=1.0)
    rb = np.where(np.arange(8) < 4, 50.0, -50.0).astype(np.float32)   # experts 0..3 (rank 0) always win
    N, T = 2, 40
    dev = torch.device("cuda", 0)
    layers, hs = [], []
    for r in range(N):
        lay = MoeLayer.from_shape(sh, max_tokens=T, expert_begin=4 * r, expert_count=4)
        lay.set_router(Wg, rb)
        lay.load_experts({n: ex[n][4 * r:4 * r + 4] for n in ex}, ids=range(4 * r, 4 * r + 4))
        layers.append(lay)
        hs.append(torch.from_numpy(synth.hidden_states(sh, T, rep=r)).to(dev))
    ptrs = [lay.ep_p2p_local_ptrs() for lay in layers]
    for r, lay in enumerate(layers):
        lay.ep_p2p_import_ptrs(r, N, [p[0] for p in ptrs], [p[1] for p in ptrs], [p[2] for p in ptrs])
    counts = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(N)]
    for r in range(N):
        layers[r].ep_p2p_counts_dev(hs[r], T, counts[r])
    torch.cuda.synchronize()
    all_counts = torch.cat(counts).contiguous()
    assert int(all_counts.view(N, 8)[:, :4].sum()) == N * T * sh.top_k > T * sh.top_k
    for r in range(N):
        layers[r].ep_p2p_scatter_dev(hs[r], T, all_counts)
    torch.cuda.synchronize()
    codes = []
    for r in range(N):
        layers[r].ep_p2p_experts_dev(all_counts, T * sh.top_k)
        with pytest.raises(CskError) as err:
            layers[r].sync()
        codes.append(err.value.code)
    torch.cuda.synchronize()
    assert codes == [-4, -4]
    for lay in layers:
        lay.close()
