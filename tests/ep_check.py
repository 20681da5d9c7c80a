"""Multi-GPU self-check of the expert-parallel steps, run under torchrun:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        tests/ep_check.py [--tokens T] [--workload c2] [--steps S] [--nccl]

Every rank compares, step after step, the output of the expert-parallel layer for its own
tokens with the output of the single-GPU layer (all experts resident) for the same tokens.
The two use the same kernels on the same rows, so the results must be identical; the check
allows 1e-3 of the largest output magnitude and reports the number of tokens beyond it.
Exit code 1 if any rank saw a bad token.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    import torch
    import torch.distributed as dist

    from coalsack_b200 import MoeLayer, ep, synth

    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=512, help="tokens per rank")
    ap.add_argument("--workload", default="c1")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--nccl", action="store_true", help="check the all-to-all step instead of the peer-memory step")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    sh = synth.CONFIGS[args.workload].with_(tokens=args.tokens)

    lay = MoeLayer.from_shape(sh, device=local, max_tokens=args.tokens)
    lay.set_router(synth.router_weight(sh), synth.router_bias(sh))
    for e in range(sh.num_experts):
        w = synth.expert_weights(sh, e)
        lay.load_expert(e, w["w_up"], w["w_gate"], w["w_down"], w["b_up"], w["b_gate"], w["b_down"])
    want, _ = lay.forward(synth.hidden_states(sh, rep=rank))
    lay.close()

    os.environ["CSK_EP_NCCL"] = "1" if args.nccl else "0"
    b = ep.EpBench(sh, rank, world, local)
    bad_total = 0
    per_step = []
    for _ in range(args.steps):
        b.step_dev()
        b.sync()
        got = b.d_out.cpu().numpy()
        diff = np.abs(got - want).max(axis=1)
        bad = int((diff > 1e-3 * np.abs(want).max()).sum())
        per_step.append(bad)
        bad_total += bad
        b.d_out.zero_()
    pl = b.backend.placement
    print(f"rank {rank}/{world} {'all-to-all' if args.nccl else 'peer-memory'} step, {args.workload}, "
          f"{args.tokens} tokens per rank, {pl.n_slots} slots, {int((pl.replica_of >= 0).sum())} second copies: "
          f"bad tokens per step {per_step}", flush=True)
    t = torch.tensor([bad_total], device=dev)
    dist.all_reduce(t)
    dist.barrier()
    dist.destroy_process_group()
    return 1 if int(t.item()) else 0


if __name__ == "__main__":
    sys.exit(main())
