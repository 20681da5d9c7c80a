#!/usr/bin/env python
"""Benchmark of the MoE layer on B200: tokens/s of one layer pass over one
batch of synthetic tokens, with the roofline of its dominant kernel, a decode
sweep, and the reference's CPU implementation timed beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

A step is one pass of router -> dispatch -> grouped MXFP4 gated MLP -> combine
over one batch.  The default workload is the gpt-oss-120b-shaped layer (128
experts, top-4, 2880 x 2880, 8192 tokens).  ``value`` is measured with the batch
already resident in HBM (CUDA events on the stream the kernels run on, max over
ranks); ``e2e`` goes through the host-buffer entry point ``csk_moe_forward`` with
pinned host buffers, so it includes the host->device and device->host copies.
``decode`` (one GPU) is the same layer at 1..256 tokens per step, 100 fresh
batches each, in microseconds per step and per token against the HBM roofline.
``dense_ffn`` (one GPU) is the shared expert's dense FFN (fp16 weights of the layer's
size) on the same token count, in TFLOP/s against the measured bf16 peak.

N > 1 (launched by torchrun, one rank per GPU): expert parallelism.  Each rank
holds E/N expert slots and T/N of the batch's tokens (strong scaling: the batch
is the same 8192 tokens at every N; ``--scaling weak`` gives every rank the whole
token count instead).  Rows travel between ranks as peer-memory stores issued by
the dispatch and down-projection kernels (NVLink); ``CSK_EP_NCCL=1`` selects the
variant with NCCL all-to-all collectives.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from coalsack_b200 import synth  # noqa: E402

METRIC = "moe_layer_prefill_tokens_per_s"
UNIT = "tokens/s"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel, from an ncu capture
# (--metrics dram__bytes_read.sum,dram__bytes_write.sum) of this program on the same workload, single GPU.
# Key = (workload name, tokens, kernel).  Other workloads report null.
MEASURED_TRAFFIC = {
    ("c2_gptoss120b_prefill8192", 8192, "k_tile<gated>"): 1599.2e6,   # 1417.8 MB read + 181.4 MB written
    ("c3_gptoss120b_decode", 64, "k_stream<gated>"): 954.3e6,        # 949.0 MB read + 5.3 MB written
}


def measured_traffic(sh, kernel, world):
    return MEASURED_TRAFFIC.get((sh.name, sh.tokens, kernel)) if world == 1 else None


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            self.th = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.th.join(timeout=2)
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load are the faster half (idle samples sit at a low clock)
        sm.sort()
        return {"sm_mhz": float(np.median(sm[len(sm) // 2:])), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def workload_shape(name, tokens=None):
    sh = synth.CONFIGS[name]
    return sh.with_(tokens=tokens) if tokens else sh


def algorithmic_flops(sh, T):
    """T*k*6*H*F for the experts (the reference bench's own convention,
    test/bench_expert_mlp_mxfp4.cpp:148) + T*2*E*H for the router."""
    return T * sh.top_k * 6.0 * sh.hidden * sh.ffn + T * 2.0 * sh.num_experts * sh.hidden


# ---------------------------------------------------------------------------
# reference arm: the reference's own CPU code on the host cores
# ---------------------------------------------------------------------------
def time_reference(sh, steps, warmup, budget_s=12.0):
    """tokens/s of the reference's CPU implementation (oracle/_ref when it was
    compiled, else the plain-C restatement) with every host thread, each step a
    bounded sample of the workload's tokens."""
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    lib = oracle.ref() if kind == "reference" else oracle.port()
    cores = os.cpu_count() or 1
    Wg, rb = synth.router_weight(sh), synth.router_bias(sh)
    # experts actually hit by the sample are generated lazily: the sample is small
    n0 = max(cores, 16)
    h0 = synth.hidden_states(sh, min(sh.tokens, 2048)) if sh.tokens >= n0 else synth.hidden_states(sh, n0)
    ro = oracle.port().router(h0, Wg, rb, sh.top_k)
    need = sorted(set(ro[..., 0].astype(int).ravel().tolist()))
    dummy = np.zeros(17 * sh.hidden * sh.ffn // 32, np.uint8)
    cache = {e: synth.expert_weights(sh, e) for e in need}
    ex = {k: [cache[e][k] if e in cache else dummy for e in range(sh.num_experts)] for k in ("w_up", "w_gate", "w_down")}
    for k in ("b_up", "b_gate", "b_down"):
        ex[k] = ([cache[e][k] if e in cache else np.zeros(1, np.float32) for e in range(sh.num_experts)]
                 if sh.has_bias else None)
    # size the sample: one probe, then scale to the time budget
    t0 = time.perf_counter()
    lib.moe_layer(h0[:n0], Wg, rb, ex, sh.top_k, sh.act, nthreads=cores)
    per_tok = (time.perf_counter() - t0) / n0
    n = int(min(h0.shape[0], max(n0, budget_s / max(per_tok, 1e-9) / max(steps + warmup, 1))))
    for _ in range(warmup):
        lib.moe_layer(h0[:n], Wg, rb, ex, sh.top_k, sh.act, nthreads=cores)
    t0 = time.perf_counter()
    for _ in range(steps):
        lib.moe_layer(h0[:n], Wg, rb, ex, sh.top_k, sh.act, nthreads=cores)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return {"value": n / dt, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"{n} of the workload's tokens per step, router + {sh.top_k} expert calls per token + merge, "
                      f"{cores} host threads over tokens; tokens/s extrapolates linearly in tokens"}, dt * 1e3


def per_rank_shape(args, world):
    """The workload one rank sees: under strong scaling the batch's tokens are split over the ranks."""
    sh = workload_shape(args.workload, args.tokens)
    total = sh.tokens if args.scaling == "strong" else sh.tokens * world
    if args.scaling == "strong":
        if sh.tokens % world:
            raise SystemExit(f"{sh.tokens} tokens do not split evenly over {world} ranks")
        sh = sh.with_(tokens=sh.tokens // world)
    return sh, total


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sh, total = per_rank_shape(args, args.gpus)
    cb, ms = time_reference(sh.with_(tokens=total), args.steps, args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_of(sh, total, args), "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def config_of(sh, total, args):
    return {"workload": f"{sh.name}: E={sh.num_experts} top-{sh.top_k} H={sh.hidden} F={sh.ffn} MXFP4, "
                        f"T={total} tokens in total, router bias {sh.router_bias}, seed {sh.seed}",
            "tokens_total": total, "experts": sh.num_experts, "top_k": sh.top_k, "hidden": sh.hidden,
            "ffn": sh.ffn, "parallelism": "single GPU" if args.gpus == 1 else f"expert-parallel x{args.gpus}",
            "l2": "weights + grouped activations per step exceed the 126 MB L2 (no flush needed)"}


# ---------------------------------------------------------------------------
# decode sweep (one GPU): the same layer at a few tokens per step
# ---------------------------------------------------------------------------
DECODE_BATCHES = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def dense_ffn_point(sh, peaks, torch, stream, steps=10):
    """The shared expert's dense FFN (fp16 weights, the layer's H and F) on the workload's token count:
    device time per call, flops = 6*T*H*F, against the measured bf16 peak."""
    from coalsack_b200 import MoeLayer
    T, H, F = sh.tokens, sh.hidden, sh.ffn
    g = np.random.Generator(np.random.Philox(key=[sh.seed, 77]))
    w = [(g.standard_normal(s, dtype=np.float32) * 0.03).astype(np.float16) for s in ((F, H), (F, H), (H, F))]
    lay = MoeLayer(1, 1, H, F, activation=synth.STANDARD_SWIGLU, has_bias=False, max_tokens=T, weights_f16=True)
    lay.load_expert_f16(0, w[0], w[1], w[2])
    d_h = torch.from_numpy(synth.hidden_states(sh)).cuda()
    d_o = torch.empty_like(d_h)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        for _ in range(3):
            lay.dense_forward_dev(d_h, T, d_o, stream=stream.cuda_stream)
        ev0.record(stream)
        for _ in range(steps):
            lay.dense_forward_dev(d_h, T, d_o, stream=stream.cuda_stream)
        ev1.record(stream)
    torch.cuda.synchronize()
    lay.sync()
    ms = ev0.elapsed_time(ev1) / steps
    lay.close()
    tf = 6.0 * T * H * F / (ms * 1e-3) / 1e12
    return {"workload": f"dense_ffn_node: fp16 weights {H}x{F}, {T} tokens, standard SwiGLU, no biases",
            "ms_per_call": ms, "tokens_per_s": T / (ms * 1e-3), "tflops": tf, "frac": tf / peaks["tflops"],
            "peak": peaks["tflops"], "peak_source": peaks["source"] + " (burst bf16 cuBLAS)"}


def decode_sweep(layer, sh, peaks, torch, stream, reps=100, nbuf=16):
    """Microseconds per step and per token for batches of 1..256 tokens on the resident layer: `reps`
    batches of fresh N(0,1) activations each (the decode workload's seed), timed back to back in segments
    of `nbuf` steps over `nbuf` device buffers that are refilled (untimed) between segments, so that no
    step repeats an earlier step's activations or expert set.  Algorithmic bytes per step =
    U * (MXFP4 bytes + bias bytes of one expert) + router weights and bias + T*H*4 in + T*H*4 out, with
    U = distinct experts the router actually selected for that batch."""
    d3 = synth.C3
    H, E, k = sh.hidden, sh.num_experts, sh.top_k
    per_expert = sh.mxfp4_bytes_per_expert + sh.bias_bytes_per_expert
    dev = torch.device("cuda", torch.cuda.current_device())
    rows = []
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for T in DECODE_BATCHES:
        bufs = [torch.empty((T, H), dtype=torch.float32, device=dev) for _ in range(nbuf)]
        outs = [torch.empty((T, H), dtype=torch.float32, device=dev) for _ in range(nbuf)]
        ro = torch.empty((T, k, 2), dtype=torch.float32, device=dev)

        def fill(first, n):
            for i in range(n):
                bufs[i].copy_(torch.from_numpy(synth.hidden_states(d3, T, rep=first + i)))
            torch.cuda.synchronize()

        def run(n):
            for i in range(n):
                layer.forward_dev(bufs[i], T, outs[i], stream=stream.cuda_stream)

        fill(reps, nbuf)  # warm-up on batches the timed repetitions do not use (captures the launch sequences)
        with torch.cuda.stream(stream):
            run(nbuf)
            run(nbuf)
        torch.cuda.synchronize()
        total_ms, distinct = 0.0, []
        for first in range(0, reps, nbuf):
            n = min(nbuf, reps - first)
            fill(first, n)
            with torch.cuda.stream(stream):
                ev0.record(stream)
                run(n)
                ev1.record(stream)
            torch.cuda.synchronize()
            total_ms += ev0.elapsed_time(ev1)
            for i in range(n):  # untimed: which experts each batch selected
                layer.route_dev(bufs[i], T, ro, stream=stream.cuda_stream)
                torch.cuda.synchronize()
                distinct.append(len(set(ro[..., 0].reshape(-1).to(torch.int64).tolist())))
        layer.sync()
        us = total_ms * 1e3 / reps
        u = float(np.mean(distinct))
        byts = u * per_expert + E * H * 4 + (E * 4 if sh.router_bias != "none" else 0) + 2 * T * H * 4
        gbs = byts / (us * 1e-6) / 1e9
        rows.append({"tokens": T, "us_per_step": us, "us_per_token": us / T, "distinct_experts": u,
                     "bytes_per_step": byts, "gbs": gbs, "frac": gbs / peaks["hbm_gbs"]})
    return {"workload": f"{d3.name}: the resident layer, fresh N(0,1) activations per repetition (seed {d3.seed})",
            "reps": reps, "bound": "hbm", "peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"] + " (copy bandwidth)",
            "batches": rows}


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def run_ours(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    sh, total = per_rank_shape(args, world)
    T, H, k, E = sh.tokens, sh.hidden, sh.top_k, sh.num_experts

    if world > 1:
        from coalsack_b200 import ep
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        runner = ep.EpBench(sh, rank, world, local)
    else:
        runner = SingleGpu(sh, local, args.path)

    sampler = ClockSampler(local)
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        runner.step_dev()
    runner.sync()

    # ---- device-resident timing ------------------------------------------------
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream = runner.torch_stream
    with torch.cuda.stream(stream):
        ev0.record(stream)
        for _ in range(args.steps):
            runner.step_dev()
        ev1.record(stream)
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # the timed region of a small workload is shorter than nvidia-smi's sampling period: keep the same
    # steps running (untimed, every rank: the steps are collective under expert parallelism) until the sampler
    # has seen the GPU under this load for about half a second
    extra = 0
    if ms < 600.0:  # ms is the same on every rank (max over ranks)
        n_extra = int(min(2000, max(0.0, 600.0 - ms) / max(ms / args.steps, 1e-3)))
        for i in range(n_extra):
            runner.step_dev()
            if i % 64 == 63:
                runner.sync()
        extra = n_extra
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = f"timed region + {extra} more identical steps (untimed)"
    runner.sync()
    ms_per_step = ms / args.steps
    value = total / (ms_per_step * 1e-3)

    # ---- per-kernel timing for the roofline (separate pass, timers on) -------------
    stage = runner.stage_times(args.steps)

    # ---- end to end through the host-buffer entry point -----------------------------
    e2e_ms = None
    if not args.skip_e2e:
        e2e_ms = runner.time_e2e(args.steps, warmup)
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    rows = stage.get("rows_received", T * k)   # under expert parallelism: rows this rank's experts processed
    gu_ms = stage["gate_up_ms"]
    if stage["path"] == "tile":
        # dense contraction: algorithmic FLOP of the gate and up projections, 2 * rows * 2F * H
        gu_flops = rows * 4.0 * H * sh.ffn
        achieved = gu_flops / (gu_ms * 1e-3) / 1e12 if gu_ms > 0 else 0.0
        roofline = {"bound": "tensor", "kernel": stage["gate_up_kernel"], "achieved": achieved, "peak": peaks["tflops"],
                    "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
                    "peak_source": peaks["source"] + " (burst bf16 cuBLAS)"}
    else:
        # weight streaming: algorithmic bytes = the packed gate/up records of every expert that received rows
        # (544 bytes per 16 features x 64 columns, gate and up), read once per 8- or 16-row tile
        recs = -(-sh.ffn // 16) * -(-H // 64) * 2
        gu_bytes = stage.get("row_tiles", 0) * recs * 544.0
        achieved = gu_bytes / (gu_ms * 1e-3) / 1e9 if gu_ms > 0 else 0.0
        roofline = {"bound": "hbm", "kernel": stage["gate_up_kernel"], "achieved": achieved, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                    "peak_source": peaks["source"] + " (copy bandwidth)"}
    roofline.update({"traffic": measured_traffic(sh, stage["gate_up_kernel"], world), "ms_per_launch": gu_ms,
                     "rows_per_launch": int(rows),
                     "layer_tflops": algorithmic_flops(sh, total) / (ms_per_step * 1e-3) / 1e12,
                     "stages_ms": {n: stage[n] for n in stage if n.endswith("_ms")}})
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f16 operands (MXFP4 weights dequantised exactly), f32 accumulate; f32 router",
            "data": "synthetic", "config": config_of(sh, total, args), "clocks": clocks,
            "gpu_launches": int(stage["launches"]) * args.steps, "path": stage["path"], "roofline": roofline}
    if e2e_ms is not None:
        line["e2e"] = {"value": total / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": T * H * 4 * world,
                       "d2h_bytes_per_step": (T * H * 4 + (T * k * 2 * 4 if world == 1 else 0)) * world}
    if world > 1:
        line["config"]["tokens_per_gpu"] = T
        line["config"]["exchange"] = runner.exchange
        line["expert_parallel"] = stage.get("ep", {})
    if world == 1 and not args.skip_decode and sh.name == synth.C2.name:
        line["decode"] = decode_sweep(runner.layer, sh, peaks, torch, runner.torch_stream)
        line["dense_ffn"] = dense_ffn_point(sh, peaks, torch, runner.torch_stream)
    if world == 1 and not args.skip_cpu:
        line["cpu_baseline"], _ = time_reference(sh, 2, 1)
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


class SingleGpu:
    """The layer on one GPU: weights resident, one batch in HBM (``step_dev``)
    or in pinned host memory (``time_e2e``)."""

    def __init__(self, sh, local, path="auto"):
        import torch
        from coalsack_b200 import MoeLayer, moe
        self.torch = torch
        self.sh = sh
        dev = torch.device("cuda", local)
        self.layer = MoeLayer.from_shape(sh, device=local, max_tokens=sh.tokens)
        self.layer.set_router(synth.router_weight(sh), synth.router_bias(sh))
        for e in range(sh.num_experts):
            w = synth.expert_weights(sh, e)
            self.layer.load_expert(e, w["w_up"], w["w_gate"], w["w_down"], w["b_up"], w["b_gate"], w["b_down"])
        self.layer.set_path({"auto": moe.PATH_AUTO, "stream": moe.PATH_STREAM, "tile": moe.PATH_TILE,
                             "tile_pair": moe.PATH_TILE_PAIR}[path])
        h = synth.hidden_states(sh)
        self.h_host = torch.from_numpy(h).pin_memory()
        self.out_host = torch.empty_like(self.h_host).pin_memory()
        self.ro_host = torch.empty((sh.tokens, sh.top_k, 2), dtype=torch.float32).pin_memory()
        self.d_hidden = self.h_host.to(dev)
        self.d_out = torch.empty_like(self.d_hidden)
        self.torch_stream = torch.cuda.Stream(device=dev)
        self.T = sh.tokens

    def step_dev(self):
        self.layer.forward_dev(self.d_hidden, self.T, self.d_out, stream=self.torch_stream.cuda_stream)

    def sync(self):
        self.torch.cuda.synchronize()
        self.layer.sync()

    def stage_times(self, steps):
        self.layer.enable_timing(True)
        acc = None
        n = max(3, min(steps, 20))
        for _ in range(n):
            self.step_dev()
            self.layer.sync()
            t = self.layer.timings()
            acc = t if acc is None else {k: acc[k] + t[k] for k in t}
        self.layer.enable_timing(False)
        out = {k: acc[k] / n for k in acc}
        out["path"] = {1: "stream", 2: "tile"}.get(int(round(out["path"])), "?")
        rows_per_expert, _, _ = self.layer.counters()
        tr = 16 if self.T * self.sh.top_k > 8 * self.sh.num_experts else 8
        out["row_tiles"] = int(sum(-(-int(r) // tr) for r in rows_per_expert))
        out["gate_up_kernel"] = "k_stream<gated>" if out["path"] == "stream" else "k_tile<gated>"
        return out

    def time_e2e(self, steps, warmup):
        for _ in range(warmup):
            self.layer.forward(self.h_host, out=self.out_host, router_out_buf=self.ro_host)
        t0 = time.perf_counter()
        for _ in range(steps):
            self.layer.forward(self.h_host, out=self.out_host, router_out_buf=self.ro_host)
        return (time.perf_counter() - t0) * 1e3 / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(synth.CONFIGS))
    ap.add_argument("--tokens", type=int, default=None, help="override the workload's token count")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: split the workload's tokens over the ranks (strong) or give every rank all of them (weak)")
    ap.add_argument("--path", default="auto", choices=["auto", "stream", "tile", "tile_pair"],
                    help="force one expert kernel (N=1 profiling runs); auto picks by rows per expert")
    ap.add_argument("--skip-cpu", action="store_true", help="leave out the cpu_baseline leg (profiling runs)")
    ap.add_argument("--skip-decode", action="store_true", help="leave out the decode sweep (profiling runs)")
    ap.add_argument("--skip-e2e", action="store_true", help="leave out the host-buffer leg (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
