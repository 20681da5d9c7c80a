"""Expert parallelism for the MoE layer: one process per GPU, expert slots sharded,
tokens data-parallel.

The reference runs every expert of a layer serially on one host thread
(src/llm/llm_engine.cpp:737-747); sharding experts across GPUs is new here.  Every
rank holds E/N expert slots (plus a spare when an expert is worth a second copy) and
its own batch of tokens.  Two host loops drive the same kernels:

``P2pEpLayer`` (default on GPUs): rows travel as peer stores issued by the kernels
themselves over NVLink --

    counts     route the local tokens, map experts to slots, count rows per slot
    gather     all ranks' counts                                  (all_gather, 4*E bytes)
    scatter    every row straight into the owning rank's row buffer, at its final
               expert-grouped position
    barrier
    experts    gated MLP of the resident experts; the down projection's epilogue
               stores every output row straight into the token owner's buffer
    barrier
    combine    weighted sum over the k slots in router order

``EpLayer``: the same step with two all-to-all exchanges (dispatch -> gather of counts
-> all_to_all of rows -> experts -> all_to_all of output rows -> combine).  Its
collective plumbing is backend-agnostic: the same code runs on gloo with a CPU compute
backend in the tests.

Placement (`plan_placement`) comes from the load of one calibration batch.
"""
from __future__ import annotations

import numpy as np

from . import synth


def strided_placement(E: int, world: int) -> np.ndarray:
    """physical slot -> logical expert so that rank r holds the logical experts
    r, r+N, r+2N, ...  (spreads a load that falls off with the expert index)."""
    per = E // world
    return np.array([(p % per) * world + p // per for p in range(E)], dtype=np.int64)


def _lpt(items, world, cap):
    """items: (load, expert, copy).  Longest-processing-time packing into `world` bins of
    `cap` slots, the two copies of an expert never in one bin."""
    bins = [[] for _ in range(world)]
    tot = np.zeros(world)
    for it in sorted(items, key=lambda x: (-x[0], x[1], x[2])):
        ok = [i for i in range(world) if len(bins[i]) < cap and all(o[1] != it[1] for o in bins[i])]
        r = min(ok, key=lambda i: (tot[i], i))
        bins[r].append(it)
        tot[r] += it[0]
    return bins, float(tot.max())


class Placement:
    """slots[p] = logical expert held by physical slot p (-1: empty); replica_of[p] = slot
    of the second copy of the expert whose first copy is slot p, else -1."""

    def __init__(self, slots, replica_of, world):
        self.slots = np.asarray(slots, dtype=np.int64)
        self.replica_of = np.asarray(replica_of, dtype=np.int32)
        self.world = world
        self.per_rank = len(self.slots) // world

    @property
    def n_slots(self):
        return len(self.slots)

    def slot_map(self, E: int):
        """(primary_slot[e], replica_slot[e]) of every logical expert, as csk_moe_ep_set_slot_map takes them."""
        primary = -np.ones(E, dtype=np.int32)
        replica = -np.ones(E, dtype=np.int32)
        copies = set(int(s) for s in self.replica_of if s >= 0)
        for p, e in enumerate(self.slots):
            if e >= 0 and p not in copies:
                primary[e] = p
                replica[e] = self.replica_of[p]
        assert (primary >= 0).all(), "every expert needs a slot"
        return primary, replica


def plan_placement(load, world: int, extra_slots: int = 0) -> Placement:
    """Placement of E experts on `world` ranks from a measured load per expert (rows it
    received in a calibration batch).  E/world (+ extra_slots) slots per rank; the heaviest
    experts get a second copy on another rank while that lowers the most loaded rank (each
    copy then serves every other token).  Deterministic: every rank computes the same plan."""
    load = np.asarray(load, dtype=np.float64)
    E = load.shape[0]
    cap = E // world + extra_slots
    items = [(load[e], e, 0) for e in range(E)]
    bins, worst = _lpt(items, world, cap)
    free = world * extra_slots
    split = set()
    while free > 0:
        cand = [e for e in np.argsort(-load, kind="stable") if int(e) not in split]
        if not cand:
            break
        e = int(cand[0])
        trial = [it for it in items if it[1] != e] + [(load[e] / 2, e, 0), (load[e] / 2, e, 1)]
        tb, tw = _lpt(trial, world, cap)
        if tw >= worst:
            break
        items, bins, worst = trial, tb, tw
        split.add(e)
        free -= 1
    slots = -np.ones(world * cap, dtype=np.int64)
    where = {}
    for r, b in enumerate(bins):
        for j, it in enumerate(sorted(b, key=lambda x: (x[1], x[2]))):
            slots[r * cap + j] = it[1]
            where[(it[1], it[2])] = r * cap + j
    replica_of = -np.ones(world * cap, dtype=np.int32)
    for e in split:
        replica_of[where[(e, 0)]] = where[(e, 1)]
    return Placement(slots, replica_of, world)


def placement_max_load(place: Placement, load) -> float:
    """Rows the busiest rank receives under `place` for the per-expert `load` (an expert with a
    second copy sends half of its rows to each)."""
    load = np.asarray(load, dtype=np.float64)
    copies = {int(s): p for p, s in enumerate(place.replica_of) if s >= 0}   # copy slot -> primary slot
    split = set(int(place.slots[p]) for p in copies.values())
    per_rank = np.zeros(place.world)
    for p, e in enumerate(place.slots):
        if e >= 0:
            per_rank[p // place.per_rank] += load[e] / (2.0 if int(e) in split else 1.0)
    return float(per_rank.max())


def best_placement(load, world: int) -> Placement:
    """The plan with one spare slot per rank when that lowers the busiest rank's load (uneven
    expert counts per rank already help a skewed load, with or without second copies), else the
    plan without spare slots."""
    tight = plan_placement(load, world, extra_slots=0)
    spare = plan_placement(load, world, extra_slots=1)
    return spare if placement_max_load(spare, load) < placement_max_load(tight, load) * 0.999 else tight


def balanced_placement(load, world: int) -> np.ndarray:
    """physical slot -> logical expert, E/world experts per rank, no replicas."""
    return plan_placement(load, world, 0).slots


def calibration_load(shape, hidden: np.ndarray) -> np.ndarray:
    """Rows per expert that `hidden` [T,H] would route (host arithmetic, ordinary matmul:
    good enough to size a placement, not used for results)."""
    Wg, rb = synth.router_weight(shape), synth.router_bias(shape)
    logits = hidden.astype(np.float32) @ Wg.T
    if rb is not None:
        logits = logits + rb
    top = np.argpartition(-logits, shape.top_k - 1, axis=1)[:, :shape.top_k]
    return np.bincount(top.ravel(), minlength=shape.num_experts).astype(np.int64)


class GpuBackend:
    """The three compute stages on one GPU (torch CUDA tensors in and out)."""

    def __init__(self, shape, rank, world, device_index, max_tokens, placement=None):
        import torch
        from .moe import MoeLayer
        self.torch = torch
        self.sh = shape
        E = shape.num_experts
        if placement is None:
            assert E % world == 0, "experts must divide evenly over the ranks"
            placement = Placement(np.arange(E), -np.ones(E, dtype=np.int32), world)
        elif not isinstance(placement, Placement):
            placement = Placement(np.asarray(placement), -np.ones(len(placement), dtype=np.int32), world)
        self.placement = placement
        self.eloc = placement.per_rank
        self.e0 = rank * self.eloc
        self.dev = torch.device("cuda", device_index)
        # the layer sees physical slots as its experts
        self.layer = MoeLayer.from_shape(shape.with_(num_experts=placement.n_slots), device=device_index,
                                         max_tokens=max_tokens, expert_begin=self.e0, expert_count=self.eloc)
        self.pitch = self.layer.ep_row_pitch()
        self.row_dtype = torch.float16
        self.H, self.k = shape.hidden, shape.top_k

    def slot_map(self):
        return self.placement.slot_map(self.sh.num_experts)

    def load_synthetic(self):
        sh = self.sh
        self.layer.ep_set_slot_map(*self.slot_map())
        self.layer.set_router(synth.router_weight(sh), synth.router_bias(sh))
        for p in range(self.e0, self.e0 + self.eloc):
            e = int(self.placement.slots[p])
            if e < 0:
                continue
            w = synth.expert_weights(sh, e)
            self.layer.load_expert(p, w["w_up"], w["w_gate"], w["w_down"], w["b_up"], w["b_gate"], w["b_down"])

    def stream(self):
        """Handle of torch's current stream, which the process group's collectives order themselves with.
        It must not be the legacy default stream: the C ABI reads a null stream as "the layer's own
        stream", and kernels there would race with the collectives."""
        h = self.torch.cuda.current_stream(self.dev).cuda_stream
        if not h:
            raise RuntimeError("run the expert-parallel step inside `with torch.cuda.stream(s)` for a "
                               "non-default stream s (a null stream handle means the layer's own stream)")
        return h

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


class P2pEpLayer:
    """The same step with the rows moved by the kernels themselves over NVLink peer memory:
    dispatch stores each row into the owning rank's row buffer at its final position, the down
    projection's epilogue stores each output row into the token owner's return buffer.  The
    process group is left with an all-gather of 4*E bytes per rank and two barriers; nothing in
    the step waits on the host.  GPU backend only (`GpuBackend`)."""

    def __init__(self, backend, world, group=None):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.b, self.world, self.group = backend, world, group
        lay = backend.layer
        rank = dist.get_rank(group)
        # exchange the CUDA IPC handles of the three buffers every peer writes into
        mine = torch.frombuffer(bytearray(lay.ep_p2p_export()), dtype=torch.uint8).to(backend.dev)
        allh = torch.empty(world * mine.numel(), dtype=torch.uint8, device=backend.dev)
        dist.all_gather_into_tensor(allh, mine, group=group)
        lay.ep_p2p_import(rank, world, bytes(allh.cpu().numpy().tobytes()))
        E = lay.E
        self.counts = torch.zeros(E, dtype=torch.int32, device=backend.dev)
        self.all_counts = torch.zeros(world * E, dtype=torch.int32, device=backend.dev)
        self.token = torch.zeros(1, dtype=torch.int32, device=backend.dev)
        # the gather of the counts and the two barriers: flags in peer memory written by a kernel of
        # the library (default), or the process group's collectives (CSK_EP_FLAGS=0)
        import os
        self.flags = os.environ.get("CSK_EP_FLAGS", "1") != "0"
        dist.barrier(group=group)  # every rank has imported before anyone signals

    def _barrier(self, which):
        # stream-ordered: every rank's kernels before it have finished (their peer stores are done)
        if self.flags:
            self.b.layer.ep_p2p_sync_dev(which, stream=self.b.stream())
        else:
            self.dist.all_reduce(self.token, group=self.group)

    def forward(self, hidden, T, out, mark=None):
        """One step.  `mark(name)`, when given, is called after each stage is enqueued (the bench
        records an event there to break the step's time down)."""
        mark = mark or (lambda name: None)
        lay, st = self.b.layer, self.b.stream()
        if T:
            lay.ep_p2p_counts_dev(hidden, T, self.counts, stream=st)
        else:
            self.counts.zero_()  # a rank without tokens still serves its experts
        mark("route_count")
        if self.flags:
            lay.ep_p2p_sync_dev(0, self.counts, self.all_counts, stream=st)
        else:
            self.dist.all_gather_into_tensor(self.all_counts, self.counts, group=self.group)
        mark("gather_counts")
        if T:
            lay.ep_p2p_scatter_dev(hidden, T, self.all_counts, stream=st)
        mark("scatter")
        self._barrier(1)
        mark("barrier_rows")
        lay.ep_p2p_experts_dev(self.all_counts, max(T, 1) * self.b.k, stream=st)
        mark("experts")
        self._barrier(2)
        mark("barrier_out")
        if T:
            lay.ep_p2p_combine_dev(T, out, stream=st)
        mark("combine")
        return T * self.b.k


class EpBench:
    """bench.py's N > 1 runner: T tokens per rank (the bench divides a fixed total by the ranks for
    strong scaling, or keeps the per-rank count for weak scaling)."""

    def __init__(self, sh, rank, world, local):
        import torch
        self.torch = torch
        self.sh, self.rank, self.world = sh, rank, world
        self.dev = torch.device("cuda", local)
        # expert placement from the load of one calibration batch (every rank's own tokens, summed)
        h = synth.hidden_states(sh, rep=rank)
        load = torch.from_numpy(calibration_load(sh, h)).to(self.dev)
        import torch.distributed as dist
        dist.all_reduce(load)
        load = load.cpu().numpy()
        place = best_placement(load, world)
        # a rank may receive more rows than it sends when routing is uneven: leave 3x head-room
        self.backend = GpuBackend(sh, rank, world, local, max_tokens=3 * sh.tokens, placement=place)
        self.backend.load_synthetic()
        # rows move over peer memory unless CSK_EP_NCCL=1 asks for the all-to-all version
        import os
        self.p2p = os.environ.get("CSK_EP_NCCL", "0") != "1"
        if self.p2p:
            try:
                self.ep = P2pEpLayer(self.backend, world)
            except Exception as exc:  # no peer access between these GPUs: the all-to-all step still works
                import sys
                print(f"[rank {rank}] peer-memory step unavailable ({exc}); using the all-to-all step", file=sys.stderr)
                self.p2p = False
            # every rank must take the same step
            agree = torch.tensor([1 if self.p2p else 0], device=self.dev)
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
            self.p2p = bool(agree.item())
        if not self.p2p:
            self.ep = EpLayer(self.backend, world)
        self.exchange = ("rows stored into peer memory by the dispatch and down-projection kernels (NVLink); counts and "
                         + ("barriers by flags in peer memory" if getattr(self.ep, "flags", False) else "barriers by NCCL")
                         if self.p2p else "all-to-all collectives (NCCL)")

        self.place = place
        self.load = load
        self.h_host = torch.from_numpy(h).pin_memory()
        self.out_host = torch.empty_like(self.h_host).pin_memory()
        self.d_hidden = self.h_host.to(self.dev)
        self.d_out = torch.empty_like(self.d_hidden)
        self.torch_stream = torch.cuda.Stream(device=self.dev)
        self.T = sh.tokens
        self._graph, self._graph_ok = None, os.environ.get("CSK_EP_GRAPH", "1") != "0"

    def step_dev(self):
        """One step on the bench's stream.  The peer-memory step with flag barriers is a fixed sequence of
        kernel launches (no host reads, barrier generations kept on the device), so it is captured into a
        CUDA graph on first use and replayed: sixteen short kernels leave the host's launch path."""
        torch = self.torch
        if self._graph is None and self._graph_ok and self.p2p and getattr(self.ep, "flags", False):
            try:
                with torch.cuda.stream(self.torch_stream):
                    self.ep.forward(self.d_hidden, self.T, self.d_out)   # warm: nothing is created lazily in capture
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.torch_stream, capture_error_mode="thread_local"):
                    self.ep.forward(self.d_hidden, self.T, self.d_out)
                self._graph = g
                self.exchange += "; the step replayed as one CUDA graph"
            except Exception as exc:  # capture refused: keep launching the stages one by one
                import sys
                print(f"[rank {self.rank}] step not captured ({exc}); launching eagerly", file=sys.stderr)
                self._graph_ok = False
                torch.cuda.synchronize()
            # every rank must run the same way (a rank replaying against ranks launching eagerly is still
            # the same kernel sequence, but keep the runs uniform)
            import torch.distributed as dist
            agree = torch.tensor([1 if self._graph is not None else 0], device=self.dev)
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
            if not bool(agree.item()):
                self._graph, self._graph_ok = None, False
                self.exchange = self.exchange.replace("; the step replayed as one CUDA graph", "")
        with torch.cuda.stream(self.torch_stream):
            if self._graph is not None:
                self._graph.replay()
            else:
                self.ep.forward(self.d_hidden, self.T, self.d_out)

    def sync(self):
        self.torch.cuda.synchronize()

    def stage_times(self, steps):
        """Device time of the two expert contractions on this rank (events inside the library) and,
        for the peer-memory step, of every stage of the step (events between the stages on the
        step's stream), each as the maximum over the ranks; plus the rows every rank received."""
        import torch.distributed as dist
        torch = self.torch
        lay = self.backend.layer
        lay.enable_timing(True)
        acc = {"gate_up_ms": 0.0, "down_ms": 0.0}
        names, stage_acc = [], {}
        n = max(3, min(steps, 10))
        rows = 0
        for _ in range(n):
            evs = []

            def mark(name):
                e = torch.cuda.Event(enable_timing=True)
                e.record(self.torch_stream)
                evs.append((name, e))

            with torch.cuda.stream(self.torch_stream):
                mark("start")
                if self.p2p:
                    rows = self.ep.forward(self.d_hidden, self.T, self.d_out, mark=mark)
                else:
                    rows = self.ep.forward(self.d_hidden, self.T, self.d_out)
                    mark("step")
            torch.cuda.synchronize()
            for (_, a), (name, b) in zip(evs[:-1], evs[1:]):
                stage_acc[name] = stage_acc.get(name, 0.0) + a.elapsed_time(b)
                if name not in names:
                    names.append(name)
            if self.p2p:  # rows this rank's experts actually received
                b = self.backend
                rows = int(self.ep.all_counts.view(self.world, -1)[:, b.e0:b.e0 + b.eloc].sum().item())
            t = lay.timings()
            acc["gate_up_ms"] += t["gate_up_ms"]
            acc["down_ms"] += t["down_ms"]
            path = t["path"]
        lay.enable_timing(False)
        out = {k: v / n for k, v in acc.items()}
        # every stage as the slowest rank saw it, and the rows each rank's experts received
        vec = torch.tensor([stage_acc[x] / n for x in names] + [float(rows)], device=self.dev, dtype=torch.float64)
        gathered = [torch.empty_like(vec) for _ in range(self.world)]
        dist.all_gather(gathered, vec)
        g = torch.stack(gathered).cpu().numpy()
        # A stage that computes counts as the slowest rank saw it (max).  A stage that only waits for the
        # other ranks (the gather of the counts, the two barriers) absorbs whatever skew the ranks arrived
        # with, so its own cost is what the LAST rank to arrive saw (min).
        waits = ("gather_counts", "barrier_rows", "barrier_out")
        stage_max = {x + "_ms": float(g[:, i].min() if x in waits else g[:, i].max()) for i, x in enumerate(names)}
        rows_all = [int(r) for r in g[:, -1]]
        limiting = max(stage_max, key=stage_max.get) if stage_max else None
        out.update(route_ms=0.0, permute_ms=0.0, combine_ms=0.0, total_ms=out["gate_up_ms"] + out["down_ms"],
                   path={1: "stream", 2: "tile"}.get(int(path), "?"), launches=14, rows_received=int(rows))
        out["gate_up_kernel"] = "k_stream<gated>" if out["path"] == "stream" else "k_tile<gated>"
        out["ep"] = {"stages_ms_max_over_ranks": stage_max,
                     "stages_note": "max over ranks; the gather of the counts and the two barriers as the last "
                                    "rank to arrive saw them (min over ranks)",
                     "limiting_stage": limiting,
                     "rows_received_per_rank": rows_all,
                     "rows_max_over_mean": float(max(rows_all) / max(1.0, np.mean(rows_all))),
                     "slots": int(self.place.n_slots), "second_copies": int((self.place.replica_of >= 0).sum()),
                     "planned_max_over_mean": float(placement_max_load(self.place, self.load) /
                                                    max(1.0, float(np.sum(self.load)) / self.world))}
        return out

    def time_e2e(self, steps, warmup):
        import time
        torch = self.torch
        for _ in range(warmup):
            with torch.cuda.stream(self.torch_stream):
                self.d_hidden.copy_(self.h_host, non_blocking=True)
                self.step_dev()
                self.out_host.copy_(self.d_out, non_blocking=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            with torch.cuda.stream(self.torch_stream):
                self.d_hidden.copy_(self.h_host, non_blocking=True)
                self.step_dev()
                self.out_host.copy_(self.d_out, non_blocking=True)
            torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3 / steps
