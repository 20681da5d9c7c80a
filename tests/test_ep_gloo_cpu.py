"""Expert parallelism over two gloo ranks on the CPU: the collective plumbing of
EpLayer (count gather, variable-split all-to-all both ways, ordering of rows)
with the reference restatement as compute backend must reproduce the
single-process layer bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from coalsack_b200 import synth
from coalsack_b200.ep import EpLayer, strided_placement
from tests import cases


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tokens, ok):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from tests.ep_cpu_backend import OracleBackend
        sh = synth.tiny(seed=71, E=8, k=3, H=64, F=96, T=tokens[rank], has_bias=True)
        h_all, Wg, rb, ex = cases.layer_inputs(sh, router_scale=40.0)
        h = synth.hidden_states(sh, tokens[rank], rep=rank)
        backend = OracleBackend(sh, rank, world, Wg, rb, ex)
        ep = EpLayer(backend, world)
        out = torch.empty((tokens[rank], sh.hidden), dtype=torch.float32)
        for _ in range(2):  # twice: buffers are reused across steps
            received = ep.forward(torch.from_numpy(h), tokens[rank], out)
        want, want_ro = oracle.port().moe_layer(h, Wg, rb, ex, sh.top_k, sh.act)
        assert np.array_equal(backend.router_out, want_ro)
        assert np.array_equal(out.numpy(), want), f"rank {rank}: output differs"
        # every row went to the rank that owns its expert
        tot = torch.tensor([received], dtype=torch.int64)
        dist.all_reduce(tot)
        assert int(tot) == sum(tokens) * sh.top_k
        ok[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens", [(5, 9), (1, 0 + 4)])
def test_ep_two_ranks_gloo(port, tokens):
    ok = mp.get_context("spawn").Array("i", [0, 0])
    mp.spawn(_worker, args=(2, _free_port(), tokens, ok), nprocs=2, join=True)
    assert list(ok) == [1, 1]


def test_strided_placement_is_a_permutation():
    for E, N in ((32, 8), (128, 8), (32, 2), (8, 1)):
        p = strided_placement(E, N)
        assert sorted(p.tolist()) == list(range(E))
        per = E // N
        for r in range(N):
            assert all(int(e) % N == r for e in p[r * per:(r + 1) * per])


def test_balanced_placement_spreads_a_skewed_load():
    from coalsack_b200.ep import balanced_placement
    rng = np.random.default_rng(7)
    for E, N in ((32, 8), (128, 8), (32, 2), (8, 1)):
        load = (1000.0 / np.sqrt(np.arange(E) + 1.0) + rng.integers(0, 20, E)).round()
        p = balanced_placement(load, N)
        assert sorted(p.tolist()) == list(range(E))
        per = E // N
        worst = max(load[p[r * per:(r + 1) * per]].sum() for r in range(N))
        strided = strided_placement(E, N)
        worst_strided = max(load[strided[r * per:(r + 1) * per]].sum() for r in range(N))
        assert worst <= worst_strided
        # no rank can do better than the mean, nor than the single heaviest expert plus the lightest others
        assert worst >= load.sum() / N - 1e-9


def test_plan_placement_with_second_copies():
    from coalsack_b200.ep import plan_placement
    load = np.array([900, 100, 90, 80, 70, 60, 50, 40], dtype=np.float64)
    pl = plan_placement(load, 2, extra_slots=1)
    assert pl.n_slots == 10 and pl.per_rank == 5
    primary, replica = pl.slot_map(8)
    assert sorted(set(primary.tolist())) == sorted(primary.tolist())          # distinct slots
    assert replica[0] >= 0, "the expert with 60 % of the rows gets a second copy"
    for e in range(8):
        assert pl.slots[primary[e]] == e
        if replica[e] >= 0:
            assert pl.slots[replica[e]] == e
            assert primary[e] // pl.per_rank != replica[e] // pl.per_rank    # the copies sit on different ranks
    # the busiest rank with the split (each copy serves half the rows) beats the best whole-expert packing
    def rank_load(p):
        l = np.zeros(2)
        for slot, e in enumerate(p.slots):
            if e >= 0:
                shared = replica[e] >= 0 if p is pl else False
                l[slot // p.per_rank] += load[e] / (2 if shared else 1)
        return l.max()
    assert rank_load(pl) < rank_load(plan_placement(load, 2, extra_slots=0))
