"""Reference arm of bench.py: the unmodified reference model (baseline/_ref/mingru) trained through its own public
API with stock PyTorch (cuBLAS + ATen, NCCL via DDP for N > 1), on the same metric, config and data as our arm.

What the harness adds, because the reference's train.py has none of it: bf16 autocast around the forward (the
baseline definition), DistributedDataParallel for N > 1 (the reference has no data-parallel mode) and a pure
PyTorch stand-in for the missing ``schedulefree`` package.  The loop itself follows train.py:772-818: per chunk
forward with hidden carry, backward, detach, optimizer step, zero_grad.
"""
from __future__ import annotations

import json
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main(args, rank, world, local):
    if not (REF / "mingru" / "minLM.py").exists():
        return unavailable("baseline/_ref is empty: the reference has no setup.py/pyproject.toml and was not installed")
    for k in [k for k in sys.modules if k == "mingru" or k.startswith("mingru.")]:
        del sys.modules[k]
    sys.path.insert(0, str(REF))
    import torch
    import torch.distributed as dist
    from mingru.minLM import minLM           # the reference's module
    import mingru
    assert str(REF) in str(Path(mingru.__file__).resolve()), "reference arm must import the reference model"
    from baseline.schedulefree_shim import AdamWScheduleFree
    import bench

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.set_float32_matmul_precision("high")          # train.py:294

    torch.manual_seed(42)
    cfg = dict(bench.MODELS[args.model])
    model = minLM(**cfg).to(dev)
    opt = AdamWScheduleFree(model.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
    opt.train()
    net = model
    mode = "single"
    if world > 1 and getattr(args, "parallel", "dp") == "fsdp":
        # the reference has no sharded mode either: torch FSDP2 (one unit per minGRU / feed-forward block, bf16 parameters on the wire and in
        # the matmuls, fp32 gradient reduction) is the stock-PyTorch baseline for the sharded configuration
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
        for layer in model.layers:            # a layer is a bare ModuleList (no forward): shard its two blocks
            fully_shard(layer[2], mp_policy=mp)       # minGRU
            fully_shard(layer[4], mp_policy=mp)       # FeedForward
        fully_shard(model, mp_policy=mp)
        mode = f"fsdp2x{world}"
    elif world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        net = DDP(model, device_ids=[local], gradient_as_bucket_view=True)
        mode = f"ddp{world}"
    if mode.startswith("fsdp"):           # optimizer over the sharded (DTensor) parameters
        opt = AdamWScheduleFree(model.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
        opt.train()

    W, Kst = args.warmup, args.steps
    host = bench.zipf_bytes(W + 2 * Kst, args.batch, args.seq, seed=1234 + rank)
    dev_data = host.to(dev)
    state = {"micro": args.batch}

    def train_sequence(tokens):
        """tokens uint8 [B, seq]; TBPTT over chunks; micro-batches of state['micro'] rows accumulate to one step."""
        B = tokens.shape[0]
        micro = state["micro"]
        n_chunks = tokens.shape[1] // args.chunk
        hiddens = [None] * (B // micro)
        losses = []
        for c in range(n_chunks):
            tot = 0.0
            for mi in range(B // micro):
                ck = tokens[mi * micro:(mi + 1) * micro, c * args.chunk:(c + 1) * args.chunk].long()
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    loss, nh = net(ck, return_loss=True, return_prev_hiddens=True, prev_hiddens=hiddens[mi])
                (loss * (micro / B)).backward()
                hiddens[mi] = [h.detach() for h in nh]
                tot = tot + loss.detach() * (micro / B)
            opt.step()
            opt.zero_grad()
            losses.append(tot)
        return losses

    # warm-up; on out-of-memory halve the micro-batch (same bytes per optimizer step through accumulation)
    i = 0
    while i < W:
        try:
            train_sequence(dev_data[i])
            i += 1
        except torch.cuda.OutOfMemoryError:
            opt.zero_grad(set_to_none=True)
            torch.cuda.empty_cache()
            if state["micro"] == 1:
                return unavailable("reference model does not fit one sequence per micro-batch on this GPU")
            state["micro"] //= 2
            i = 0
    torch.cuda.synchronize()

    sampler = bench.ClockSampler(local)
    sampler.start()
    ms = bench.timed(lambda i: train_sequence(dev_data[W + i]), Kst, barrier, world, torch, dist)
    stage = torch.empty(args.batch, args.seq, dtype=torch.uint8, device=dev)
    last = {}

    def e2e_step(i):
        stage.copy_(host[W + Kst + i], non_blocking=True)
        losses = train_sequence(stage)
        last["loss"] = float(torch.stack(losses).mean().item())

    ms_e2e = bench.timed(e2e_step, Kst, barrier, world, torch, dist)
    clocks = sampler.stop()
    bytes_per_step = args.batch * args.seq * world
    if rank == 0:
        print(json.dumps({
            "metric": bench.metric_name(args.model), "value": bytes_per_step * Kst / (ms / 1e3), "unit": "bytes/s", "n_gpus": world,
            "steps": Kst, "warmup": W, "ms_per_step": ms / Kst, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic Zipf(1.1) bytes, random-init weights",
            "impl": "reference",
            "config": dict(bench.shared_config(args, world), micro_batch=state["micro"]),
            "impl_notes": {"model_class": "reference mingru.minLM (unmodified)", "precision": "bf16 autocast, fp32 parameters",
                           "optimizer_impl": "pure-PyTorch foreach stand-in for the schedulefree package",
                           "wrapper": mode, "max_memory_allocated_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 2)},
            "clocks": clocks,
            "e2e": {"value": bytes_per_step * Kst / (ms_e2e / 1e3), "unit": "bytes/s", "ms_per_step": ms_e2e / Kst,
                    "h2d_bytes_per_step": args.batch * args.seq, "d2h_bytes_per_step": 4, "last_loss": last.get("loss")},
            "gpu_launches": 0,
        }))
    if world > 1:
        dist.destroy_process_group()
    return 0
