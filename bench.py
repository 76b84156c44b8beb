#!/usr/bin/env python
"""Headline benchmark: training throughput (bytes/s == tokens/s) of the ~1B-parameter minLM.

Config (the one the baseline names): dim 2048, depth 20, expansion 1.5, ff_mult 4, vocab 256, bf16 compute;
sequences of 4096 bytes trained as two TBPTT chunks of 2048 with hidden-state carry, micro-batch 8 per GPU,
Schedule-Free AdamW step after every chunk; synthetic Zipf(1.1) bytes; data parallel over N GPUs (weak scaling).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one 4096-byte sequence per batch row = 2 x (forward, backward, optimizer step).
For N > 1 launch with torchrun (one rank per GPU).  Rank 0 prints ONE JSON line.

Two timed regions, K steps each, both bracketed by barrier + synchronize and timed with CUDA events (max over ranks):
  value : inputs already on the device, no host round trip inside the region;
  e2e   : every step copies its input bytes from pinned host memory and reads the step's loss back.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

MODELS = {
    "1b": dict(num_tokens=256, dim=2048, depth=20, ff_mult=4, expansion=1.5),
    "3b": dict(num_tokens=256, dim=3072, depth=26, ff_mult=4, expansion=1.5),
    "tiny": dict(num_tokens=256, dim=256, depth=2, ff_mult=4, expansion=1.5),
}
METRIC = "train bytes/sec (1B minLM, device-timed, max over ranks)"


def metric_name(model: str) -> str:
    return METRIC.replace("1B", model.upper())


def shared_config(args, world: int) -> dict:
    """The part of the printed ``config`` that names the workload.  Both arms print exactly this (what differs
    between the implementations goes under ``impl_notes``), so a reader can check that they ran the same thing."""
    cfg = MODELS[args.model]
    return {"model": f"minLM {args.model} dim{cfg['dim']} depth{cfg['depth']} exp{cfg['expansion']} ff{cfg['ff_mult']} "
                     f"vocab{cfg['num_tokens']}",
            "global_batch": args.batch * world, "micro_batch": args.batch, "seq_len": args.seq, "chunk": args.chunk,
            "optimizer": "Schedule-Free AdamW lr 1e-3 betas (0.9, 0.995) wd 1e-4, step after every chunk",
            "parallelism": f"{args.parallel}{world}",
            "l2": "per-step working set (weights + activations, > 20 GB) far exceeds the 126 MB L2"}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", choices=list(MODELS), default="1b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--parallel", choices=["dp", "fsdp", "gossip"], default="dp",
                    help="multi-GPU mode: dp (headline config), fsdp (3B config: --model 3b --batch 4 --seq 8192) or "
                         "gossip (a population of independent replicas, tournament every --gossip_every chunk-steps)")
    ap.add_argument("--gossip_every", type=int, default=50, help="gossip: chunk-steps between tournament rounds")
    ap.add_argument("--gossip_rate", type=float, default=0.02,
                    help="gossip, reference arm: per-step mixing probability of the reference's protocol (0.02 = every 50 steps)")
    return ap.parse_args()


def zipf_bytes(n_seq, batch, seq, seed):
    """Pinned uint8 [n_seq, batch, seq] of i.i.d. Zipf(s=1.1) bytes over 0..255."""
    import torch
    g = torch.Generator().manual_seed(seed)
    w = 1.0 / torch.arange(1, 257, dtype=torch.float64) ** 1.1
    x = torch.multinomial(w / w.sum(), n_seq * batch * seq, replacement=True, generator=g)
    x = x.to(torch.uint8).view(n_seq, batch, seq)
    return x.pin_memory() if torch.cuda.is_available() else x


class ClockSampler:
    """Samples SM clock and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc, self.index = None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [s.strip() for s in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    return rank, world, local


def timed(run_step, steps, barrier, world, torch, dist, finish=None):
    """K steps between barrier+synchronize, CUDA-event time, max over ranks.  Returns milliseconds.
    ``finish`` (optional) runs inside the timed region after the last step (e.g. collecting read-backs in flight)."""
    barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        run_step(i)
    if finish is not None:
        finish()
    b.record()
    torch.cuda.synchronize()
    barrier()
    ms = torch.tensor([a.elapsed_time(b)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def gossip_main(args, rank, world, local):
    """Population benchmark (gossip configuration): every rank trains its own replica on its own data; every
    --gossip_every chunk-steps random pairs compare fitness over the host and each loser pulls the winner's weights
    and optimizer state over NVLink, fused with the merge (recombination, alpha = softmax of -loss, optimizer
    interpolation).  value = bytes trained per second by the whole population, rounds included."""
    import statistics as st
    import tempfile
    import torch
    import torch.distributed as dist
    from gruboros_b200.models.minlm import minLM
    from gruboros_b200.optim.schedulefree import AdamWScheduleFree
    from gruboros_b200.parallel.gossip import EvolutionaryTrainingNode
    from gruboros_b200.runtime.metrics import AsyncScalarReader
    from gruboros_b200.runtime.trainer import Trainer
    from gruboros_b200.ops import kernels, _lib

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    host_group = dist.new_group(backend="gloo") if world > 1 else None
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)
    torch.manual_seed(42)
    model = minLM(**MODELS[args.model]).to(dev)
    opt = AdamWScheduleFree(model.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
    opt.train()
    out_dir = tempfile.mkdtemp(prefix="grb_gossip_bench_")
    node = EvolutionaryTrainingNode(f"node_{rank}", model, opt, rank, local, world, output_dir=out_dir,
                                    gossip_temp_dir=os.path.join(out_dir, "tmp"), transport="nvlink" if world > 1 else "tcp",
                                    gossip_every=args.gossip_every if world > 1 else 0, merge_method="recombination",
                                    recombination_alpha=0.3, optimizer_recombination="interpolate", alpha_mode="softmax",
                                    host_group=host_group, bootstrap_nodes=[], listen=False)
    node.start_gossip_protocol()
    trainer = Trainer(model, opt, chunk_size=args.chunk, grad_accum=1)
    W, Kst = args.warmup, args.steps
    n_chunks = args.seq // args.chunk
    host = zipf_bytes(W + Kst, args.batch, args.seq, seed=1234 + rank)
    stage = torch.empty(args.batch, args.seq, dtype=torch.uint8, device=dev)
    reader = AsyncScalarReader()
    state = {"chunk_step": 0, "last": None, "transfers": []}

    def feed(pairs):
        for s, v in pairs:
            node.update_fitness(v, s)
            state["last"] = v

    def step(i):
        stage.copy_(host[i], non_blocking=True)                       # H2D from pinned memory
        trainer.reset_hidden()
        for c in range(n_chunks):
            node.apply_pending_update()
            loss = trainer.step_chunk(stage[:, c * args.chunk:(c + 1) * args.chunk])
            s = state["chunk_step"]
            reader.push(s, loss)                                      # D2H read of the chunk's loss, picked up when it lands
            if node.gossip_every and (s + 1) % node.gossip_every == 0:
                feed(reader.drain())                                  # a round compares up-to-date fitness values
            else:
                feed(reader.ready())
            node.current_step = s
            node.check_for_updates()                                  # runs the tournament round when one is due
            t = getattr(node, "last_transfer", None)
            if t is not None:
                state["transfers"].append(t)
                node.last_transfer = None
            state["chunk_step"] = s + 1

    for i in range(W):
        step(i)
    torch.cuda.synchronize()
    _lib.check_device_status()
    state["transfers"].clear()
    rounds0 = node.rounds
    sampler = ClockSampler(local)
    sampler.start()
    n0 = kernels.LAUNCHES
    ms = timed(lambda i: step(W + i), Kst, barrier, world, torch, dist, finish=lambda: feed(reader.drain()))
    launches = kernels.LAUNCHES - n0
    clocks = sampler.stop()
    _lib.check_device_status()
    node.stop_gossip_protocol()
    mine = {"rank": rank, "transfers": state["transfers"], "status": node.get_status()}
    gathered = [mine]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, mine, group=host_group)
    if rank == 0:
        tr = [t for g in gathered for t in g["transfers"]]
        bytes_per_step = args.batch * args.seq * world
        value = bytes_per_step * Kst / (ms / 1e3)
        print(json.dumps({
            "metric": "train bytes/sec (gossip population of 1B minLM replicas, device-timed, max over ranks)".replace("1B", args.model.upper()),
            "value": value, "unit": "bytes/s", "n_gpus": world, "steps": Kst, "warmup": W, "ms_per_step": ms / Kst,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic Zipf(1.1) bytes, random-init weights", "impl": "ours",
            "config": dict(shared_config(args, world), parallelism=f"gossip{world}"),
            "gossip": {"every_chunk_steps": args.gossip_every, "rounds_in_timed_region": node.rounds - rounds0,
                       "merges": len(tr), "transfer_merge_ms_median": st.median(t["ms"] for t in tr) if tr else None,
                       "bytes_per_merge": tr[0]["bytes"] if tr else None,
                       "GBs_median": st.median(t["bytes"] / 1e6 / t["ms"] for t in tr) if tr else None,
                       "merge": "recombination, alpha = softmax(-loss), optimizer state (z, v) interpolated",
                       "mixes_won": sum(g["status"]["won_mixes"] for g in gathered),
                       "mixes_lost": sum(g["status"]["lost_mixes"] for g in gathered),
                       "failed_mixes": sum(g["status"]["failed_mixes"] for g in gathered)},
            "clocks": clocks,
            "e2e": {"value": value, "unit": "bytes/s", "ms_per_step": ms / Kst, "h2d_bytes_per_step": args.batch * args.seq,
                    "d2h_bytes_per_step": 4 * n_chunks, "last_loss": state["last"],
                    "note": "the timed region itself is end to end: pinned-host input copy and loss read-back every step"},
            "gpu_launches": launches}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    args = parse()
    rank, world, local = dist_env()
    if args.impl == "reference":
        if args.parallel == "gossip":
            from baseline import reference_gossip
            return reference_gossip.main(args, rank, world, local)
        from baseline import reference_bench
        return reference_bench.main(args, rank, world, local)
    if args.parallel == "gossip":
        return gossip_main(args, rank, world, local)

    import torch
    import torch.distributed as dist
    from gruboros_b200.models.minlm import minLM
    from gruboros_b200.optim.schedulefree import AdamWScheduleFree
    from gruboros_b200.runtime.trainer import Trainer
    from gruboros_b200.ops import kernels, _lib

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)

    torch.manual_seed(42)                      # same initial weights on every rank (reference train.py:313-317)
    cfg = MODELS[args.model]
    model = minLM(**cfg).to(dev)
    parallel = None
    if world > 1:
        if args.parallel == "fsdp":
            from gruboros_b200.parallel.fsdp import FullyShardedDataParallel
            parallel = FullyShardedDataParallel(model, rank=rank, world=world, device=dev)
        else:
            from gruboros_b200.parallel.dp import DataParallel
            parallel = DataParallel(model, rank=rank, world=world, device=dev)
    opt = AdamWScheduleFree(model.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
    if parallel is not None:
        parallel.bind_optimizer(opt)
    opt.train()
    trainer = Trainer(model, opt, chunk_size=args.chunk, grad_accum=1, parallel=parallel)

    W, Kst = args.warmup, args.steps
    host = zipf_bytes(W + 2 * Kst, args.batch, args.seq, seed=1234 + rank)
    dev_data = host.to(dev)

    for i in range(W):
        trainer.train_sequence(dev_data[i])
    torch.cuda.synchronize()
    _lib.check_device_status()

    sampler = ClockSampler(local)
    sampler.start()
    n0 = kernels.LAUNCHES
    ms = timed(lambda i: trainer.train_sequence(dev_data[W + i]), Kst, barrier, world, torch, dist)
    launches = kernels.LAUNCHES - n0

    # end to end through the public API: every step's input bytes come from pinned host memory and every step's loss
    # is read back to the host - the way train.py does it: the copy of step i's loss is started behind step i and
    # picked up when it has landed (runtime.metrics.AsyncScalarReader), so the host never idles the GPU; all reads
    # are complete before the region's closing event
    from gruboros_b200.runtime.metrics import AsyncScalarReader
    stages = [torch.empty(args.batch, args.seq, dtype=torch.uint8, device=dev) for _ in range(2)]
    reader = AsyncScalarReader()
    last = {"n": 0}

    def collect(pairs):
        for _, v in pairs:
            last["loss"] = v
            last["n"] += 1

    def e2e_step(i):
        stage = stages[i % 2]
        stage.copy_(host[W + Kst + i], non_blocking=True)            # H2D from pinned memory
        losses = trainer.train_sequence(stage)
        reader.push(i, torch.stack(losses).mean())                    # D2H read of the step's result
        collect(reader.ready())

    ms_e2e = timed(e2e_step, Kst, barrier, world, torch, dist, finish=lambda: collect(reader.drain()))
    assert last["n"] == Kst, "every step's loss must have been read inside the timed region"
    clocks = sampler.stop()
    _lib.check_device_status()

    free_b, total_b = torch.cuda.mem_get_info(dev)      # includes the peer-mapped buffers, which torch does not track
    mem = torch.tensor([float(total_b - free_b)], device=dev)
    if world > 1:
        dist.all_reduce(mem, op=dist.ReduceOp.MAX)
    max_mem = float(mem.item())
    bytes_per_step = args.batch * args.seq * world
    value = bytes_per_step * Kst / (ms / 1e3)
    e2e = bytes_per_step * Kst / (ms_e2e / 1e3)
    if rank == 0:
        print(json.dumps({
            "metric": metric_name(args.model), "value": value, "unit": "bytes/s", "n_gpus": world, "steps": Kst, "warmup": W,
            "ms_per_step": ms / Kst, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic Zipf(1.1) bytes, random-init weights", "impl": "ours",
            "config": shared_config(args, world),
            "impl_notes": {"optimizer_in_backward": bool(trainer.optimizer_steps and trainer.last_folded),
                           "precision": "bf16 GEMM operands and saved activations, fp32 residual stream / masters / optimizer state",
                           "device_memory_in_use_gb": round(max_mem / 2 ** 30, 2),
                           **({"sharded_bytes_per_rank": parallel.persistent_bytes()} if hasattr(parallel, "persistent_bytes") else {})},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "bytes/s", "ms_per_step": ms_e2e / Kst, "h2d_bytes_per_step": args.batch * args.seq,
                    "d2h_bytes_per_step": 4, "last_loss": last.get("loss")},
            "gpu_launches": launches,
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
