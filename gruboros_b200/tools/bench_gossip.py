"""Gossip data-plane benchmark: time of the fused NVLink transfer + merge for a population of 1B-parameter members.

Launch with torchrun, one rank per GPU.  Every rank builds the model and its Schedule-Free state in symmetric
buffers; then R tournament rounds run (random pairs, rank-dependent fitness so every pair has a loser).  The loser's
single kernel reads the winner's parameters, z and second moments through IPC-mapped peer pointers and merges them
into its own (clonal copy, or recombination with optimizer interpolation).  Reported per merge method: median
device time of that kernel over the rounds this rank lost, bytes read over NVLink, and the fraction of the measured
peer-copy bandwidth (770 GB/s per direction).  The reference moves the same state through D2H, torch.save, TCP,
torch.load and H2D (gossip/evolutionary_node.py:591-725).

    python -m torch.distributed.run --nproc-per-node 2 -m gruboros_b200.tools.bench_gossip [--model 1b] [--rounds 6]
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import tempfile

import torch
import torch.distributed as dist

from ..models.minlm import minLM
from ..optim.schedulefree import AdamWScheduleFree
from ..ops import _lib as L
from ..parallel.gossip import EvolutionaryTrainingNode

MODELS = {"1b": dict(num_tokens=256, dim=2048, depth=20), "100m": dict(num_tokens=256, dim=512, depth=32)}
NVLINK_GBS = 770.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1b", choices=list(MODELS))
    ap.add_argument("--rounds", type=int, default=6)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    host = dist.new_group(backend="gloo")
    out_dir = tempfile.mkdtemp()
    results = {}
    torch.manual_seed(rank)
    model = minLM(**MODELS[a.model]).to(dev)
    opt = AdamWScheduleFree(model.parameters(), lr=1e-3, betas=(0.9, 0.995))
    opt.train()
    node = EvolutionaryTrainingNode(f"node_{rank}", model, opt, rank, local, world, output_dir=out_dir,
                                    gossip_temp_dir=os.path.join(out_dir, "tmp"), transport="nvlink", gossip_every=1,
                                    merge_method="clonal", host_group=host, bootstrap_nodes=[])
    for method, opt_mode in (("clonal", "interpolate"), ("recombination", "interpolate"), ("recombination", "reset")):
        node.merge_method, node.optimizer_recombination, node.recombination_alpha = method, opt_mode, 0.3
        times, nbytes = [], 0
        for r in range(a.rounds):
            # fitness rotates so that every rank loses in some rounds
            with node.fitness_lock:
                node.fitness_tracker.ema_loss = 1.0 + ((rank + r) % world)
            node.current_step = r
            node._nvlink_round()
            t = getattr(node, "last_transfer", None)
            if t is not None:
                times.append(t["ms"]); nbytes = t["bytes"]
                node.last_transfer = None
        torch.cuda.synchronize()
        L.check_device_status()
        if times:
            ms = statistics.median(times)
            results[f"{method}/{opt_mode}"] = {"ms": ms, "GB": nbytes / 1e9, "GBs": nbytes / 1e6 / ms,
                                               "frac_of_measured_nvlink_770": nbytes / 1e6 / ms / NVLINK_GBS, "losses": len(times)}
    gathered = [None] * world
    dist.all_gather_object(gathered, results)
    if rank == 0:
        print(json.dumps({"model": a.model, "world": world, "params": sum(p.numel() for p in model.parameters()),
                          "per_rank": gathered}, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
