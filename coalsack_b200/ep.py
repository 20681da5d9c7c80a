"""Expert parallelism for the MoE layer: one process per GPU, experts sharded,
tokens data-parallel, two all-to-all exchanges per step.

The reference runs every expert of a layer serially on one host thread
(src/llm/llm_engine.cpp:737-747); sharding experts across GPUs is new here.  Rank
r holds experts [r*E/N, (r+1)*E/N) and its own batch of tokens.  A step is

    dispatch   route the local tokens, group their (token, expert) rows by
               destination rank then expert                      (compute backend)
    gather     all ranks' per-expert row counts                  (all_gather)
    exchange   rows to the ranks that own their experts          (all_to_all, variable splits)
    experts    gated MLP of the resident experts over the rows   (compute backend)
    exchange   output rows back to the ranks that own the tokens (all_to_all)
    combine    weighted sum over the k slots in router order     (compute backend)

The collective plumbing is backend-agnostic (NCCL on GPUs; the same code runs on
gloo with a CPU compute backend in the tests).  The compute backend on GPUs is
``GpuBackend`` over the C ABI's ``csk_moe_ep_*`` entry points.
"""
from __future__ import annotations

import numpy as np

from . import synth


def strided_placement(E: int, world: int) -> np.ndarray:
    """physical slot -> logical expert so that rank r holds the logical experts
    r, r+N, r+2N, ...  (spreads a load that falls off with the expert index)."""
    per = E // world
    return np.array([(p % per) * world + p // per for p in range(E)], dtype=np.int64)


class GpuBackend:
    """The three compute stages on one GPU (torch CUDA tensors in and out)."""

    def __init__(self, shape, rank, world, device_index, max_tokens, placement=None):
        import torch
        from .moe import MoeLayer
        self.torch = torch
        self.sh = shape
        E = shape.num_experts
        assert E % world == 0, "experts must divide evenly over the ranks"
        self.eloc = E // world
        self.e0 = rank * self.eloc
        self.dev = torch.device("cuda", device_index)
        self.place = np.arange(E) if placement is None else np.asarray(placement)
        # under expert parallelism a rank can receive more rows than it sends; size for the worst
        # case the benchmark configurations produce (all rows of every rank landing here is 8x)
        self.layer = MoeLayer.from_shape(shape, device=device_index, max_tokens=max_tokens,
                                         expert_begin=self.e0, expert_count=self.eloc)
        self.pitch = self.layer.ep_row_pitch()
        self.row_dtype = torch.float16
        self.H, self.k = shape.hidden, shape.top_k

    def load_synthetic(self):
        sh = self.sh
        Wg, rb = synth.router_weight(sh), synth.router_bias(sh)
        self.layer.set_router(Wg[self.place], None if rb is None else rb[self.place])
        for p in range(self.e0, self.e0 + self.eloc):
            w = synth.expert_weights(sh, int(self.place[p]))
            self.layer.load_expert(p, w["w_up"], w["w_gate"], w["w_down"], w["b_up"], w["b_gate"], w["b_down"])

    def stream(self):
        return self.torch.cuda.current_stream(self.dev).cuda_stream

    def new_rows(self, n):
        return self.torch.empty((n, self.pitch), dtype=self.row_dtype, device=self.dev)

    def new_out_rows(self, n):
        return self.torch.empty((n, self.H), dtype=self.torch.float32, device=self.dev)

    def new_counts(self, n):
        return self.torch.empty(n, dtype=self.torch.int32, device=self.dev)

    def dispatch(self, hidden, T, send, counts):
        self.layer.ep_dispatch_dev(hidden, T, send, counts, stream=self.stream())

    def experts(self, recv, recv_counts, n_src, total_rows, ret):
        if total_rows:
            self.layer.ep_experts_dev(recv, recv_counts, n_src, total_rows, ret, stream=self.stream())

    def combine(self, back, T, out):
        self.layer.ep_combine_dev(back, T, out, stream=self.stream())


class EpLayer:
    """The step above over any ``torch.distributed`` process group."""

    def __init__(self, backend, world, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.b = backend
        self.world = world
        self.group = group
        self.eloc = backend.eloc
        self._bufs = {}

    def _buf(self, name, maker, n):
        cur = self._bufs.get(name)
        if cur is None or cur.shape[0] < n:
            cur = maker(max(n, 1))
            self._bufs[name] = cur
        return cur[:n]

    def forward(self, hidden, T, out):
        b, dist, N = self.b, self.dist, self.world
        rows = T * b.k
        E = N * self.eloc
        send = self._buf("send", b.new_rows, rows)
        counts = self._buf("counts", b.new_counts, E)
        b.dispatch(hidden, T, send, counts)
        # every rank's counts: one small collective, one host read
        all_counts = self._buf("all_counts", b.new_counts, N * E)
        dist.all_gather_into_tensor(all_counts, counts, group=self.group)
        ac = all_counts.cpu().numpy().reshape(N, E)  # [source rank, global expert]
        me = dist.get_rank(self.group)
        send_splits = ac[me].reshape(N, self.eloc).sum(1).tolist()                    # rows to each destination
        recv_mat = ac[:, me * self.eloc:(me + 1) * self.eloc]                       # [source rank, local expert]
        recv_splits = recv_mat.sum(1).tolist()
        total = int(sum(recv_splits))
        recv = self._buf("recv", b.new_rows, total)
        dist.all_to_all_single(recv, send, output_split_sizes=recv_splits, input_split_sizes=send_splits,
                               group=self.group)
        recv_counts = self._buf("recv_counts", b.new_counts, N * self.eloc)
        recv_counts.copy_(all_counts.view(N, E)[:, me * self.eloc:(me + 1) * self.eloc].reshape(-1))
        ret = self._buf("ret", b.new_out_rows, total)
        b.experts(recv, recv_counts, N, total, ret)
        back = self._buf("back", b.new_out_rows, rows)
        dist.all_to_all_single(back, ret, output_split_sizes=send_splits, input_split_sizes=recv_splits,
                               group=self.group)
        b.combine(back, T, out)
        return total


class EpBench:
    """bench.py's N > 1 runner: weak scaling, T tokens per rank."""

    def __init__(self, sh, rank, world, local):
        import torch
        self.torch = torch
        self.sh, self.rank, self.world = sh, rank, world
        self.dev = torch.device("cuda", local)
        place = strided_placement(sh.num_experts, world) if sh.router_bias == "zipf" else None
        # a rank may receive more rows than it sends when routing is uneven: leave 3x head-room
        self.backend = GpuBackend(sh, rank, world, local, max_tokens=3 * sh.tokens, placement=place)
        self.backend.load_synthetic()
        self.ep = EpLayer(self.backend, world)
        h = synth.hidden_states(sh, rep=rank)
        self.h_host = torch.from_numpy(h).pin_memory()
        self.out_host = torch.empty_like(self.h_host).pin_memory()
        self.d_hidden = self.h_host.to(self.dev)
        self.d_out = torch.empty_like(self.d_hidden)
        self.torch_stream = torch.cuda.current_stream(self.dev)
        self.T = sh.tokens

    def step_dev(self):
        self.ep.forward(self.d_hidden, self.T, self.d_out)

    def sync(self):
        self.torch.cuda.synchronize()

    def stage_times(self, steps):
        """Device time of the two expert contractions on this rank (events inside the library)
        plus whole-stage times from torch events around dispatch / exchange / experts / combine."""
        lay = self.backend.layer
        lay.enable_timing(True)
        acc = {"gate_up_ms": 0.0, "down_ms": 0.0}
        n = max(3, min(steps, 10))
        rows = 0
        for _ in range(n):
            rows = self.ep.forward(self.d_hidden, self.T, self.d_out)
            self.torch.cuda.synchronize()
            t = lay.timings()
            acc["gate_up_ms"] += t["gate_up_ms"]
            acc["down_ms"] += t["down_ms"]
            path = t["path"]
        lay.enable_timing(False)
        out = {k: v / n for k, v in acc.items()}
        out.update(route_ms=0.0, permute_ms=0.0, combine_ms=0.0, total_ms=out["gate_up_ms"] + out["down_ms"],
                   path={1: "stream", 2: "tile"}.get(int(path), "?"), launches=14, rows_received=int(rows))
        out["gate_up_kernel"] = "k_stream<gated>" if out["path"] == "stream" else "k_tile<gated>"
        return out

    def time_e2e(self, steps, warmup):
        import time
        torch = self.torch
        for _ in range(warmup):
            self.d_hidden.copy_(self.h_host, non_blocking=True)
            self.step_dev()
            self.out_host.copy_(self.d_out, non_blocking=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.d_hidden.copy_(self.h_host, non_blocking=True)
            self.step_dev()
            self.out_host.copy_(self.d_out, non_blocking=True)
            torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3 / steps
