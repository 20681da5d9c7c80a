"""A CPU stand-in for the three compute stages of expert parallelism, built on
the plain-C restatement of the reference, so the collective plumbing of
``coalsack_b200.ep.EpLayer`` can run over gloo without a GPU.  Test code only."""
from __future__ import annotations

import numpy as np
import torch

import oracle


class OracleBackend:
    def __init__(self, shape, rank, world, Wg, rb, experts):
        self.sh = shape
        self.eloc = shape.num_experts // world
        self.e0 = rank * self.eloc
        self.Wg, self.rb, self.ex = Wg, rb, experts
        self.H, self.k = shape.hidden, shape.top_k
        self.p = oracle.port()

    def new_rows(self, n):
        return torch.empty((n, self.H), dtype=torch.float32)

    new_out_rows = new_rows

    def new_counts(self, n):
        return torch.empty(n, dtype=torch.int32)

    def dispatch(self, hidden, T, send, counts):
        h = hidden.numpy()[:T]
        self.router_out = self.p.router(h, self.Wg, self.rb, self.k)
        ids = self.router_out[..., 0].astype(np.int64).reshape(-1)
        order = np.argsort(ids, kind="stable")           # grouped by global expert id
        self.row_of_pair = np.empty(T * self.k, np.int64)
        self.row_of_pair[order] = np.arange(T * self.k)
        send.numpy()[:] = h[order // self.k]
        counts.numpy()[:] = np.bincount(ids, minlength=self.sh.num_experts).astype(np.int32)

    def experts(self, recv, recv_counts, n_src, total_rows, ret):
        rc = recv_counts.numpy().reshape(n_src, self.eloc)
        x, y = recv.numpy(), ret.numpy()
        r = 0
        for s in range(n_src):
            for e in range(self.eloc):
                g = self.e0 + e
                b = [self.ex[n][g] if self.ex.get(n) is not None else None for n in ("b_up", "b_gate", "b_down")]
                for _ in range(int(rc[s, e])):
                    y[r] = self.p.expert_token(x[r], self.ex["w_up"][g], self.ex["w_gate"][g], self.ex["w_down"][g],
                                               *b, self.H, self.sh.ffn, self.sh.act)
                    r += 1
        assert r == total_rows

    def combine(self, back, T, out):
        y, o = back.numpy(), out.numpy()
        o[:T] = 0
        for t in range(T):
            for j in range(self.k):
                w = np.float32(self.router_out[t, j, 1])
                o[t] = o[t] + w * y[self.row_of_pair[t * self.k + j]]
