"""Worker for the multi-GPU FSDP test (torchrun, one rank per GPU): trains a small model fully sharded with NaN
poisoning of stale weight ranges and compares with a single replica trained by rank 0 on the whole batch."""
import copy
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from gruboros_b200.models.minlm import minLM
from gruboros_b200.optim.schedulefree import AdamWScheduleFree
from gruboros_b200.ops import _lib as L
from gruboros_b200.parallel.fsdp import FullyShardedDataParallel
from gruboros_b200.runtime.trainer import Trainer
from tests.test_model_cpu import randomize, zipf_bytes


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    base = minLM(num_tokens=256, dim=256, depth=3)
    randomize(base, 5)
    model = copy.deepcopy(base).to(dev)
    before = torch.cuda.memory_allocated(dev)
    fs = FullyShardedDataParallel(model, rank=rank, world=world, device=dev, debug_poison=True)
    opt = AdamWScheduleFree(model.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
    fs.bind_optimizer(opt)
    opt.train()
    trainer = Trainer(model, opt, chunk_size=129, grad_accum=1, parallel=fs)
    Bper = 2
    x = zipf_bytes(world * Bper, 4 * 129, seed=9).to(dev)
    losses = trainer.train_sequence(x[rank * Bper:(rank + 1) * Bper])
    torch.cuda.synchronize()
    L.check_device_status()
    mean_loss = torch.stack(losses).clone()
    dist.all_reduce(mean_loss)
    mean_loss /= world
    fs.gather_params()
    torch.cuda.synchronize()
    # ZeRO-3 memory: per-rank parameters + gradients + optimizer state are 1/world of the unsharded total, and no
    # rank holds a full weight matrix at rest
    pb = fs.persistent_bytes()
    assert pb["sharded_params_grads_state"] * world == pb["unsharded_equivalent"], pb
    got = torch.cat([p.detach().reshape(-1) for p in model.parameters()]).clone()      # full model, gathered above
    assert got.numel() == sum(p.numel() for p in base.parameters())
    fs.release_params()
    assert all(p.numel() == 0 for p in fs.big.params)
    out = {"rank": rank, "loss": mean_loss.tolist(), "gathered_MB": fs.gathered_bytes / 1e6, "bytes": pb}
    if rank == 0:
        single = copy.deepcopy(base).to(dev)
        osingle = AdamWScheduleFree(single.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
        osingle.train()
        ls = torch.stack(Trainer(single, osingle, chunk_size=129).train_sequence(x))
        sflat = single.fused_engine().flat
        want = torch.cat([p.detach().reshape(-1) for p in single.parameters()])
        d = (got - want).abs()
        out.update(single_loss=ls.tolist(), loss_max_diff=(ls - mean_loss).abs().max().item(),
                   param_mean_diff=d.mean().item(), param_max_diff=d.max().item())
        out["ok"] = bool(out["loss_max_diff"] < 3e-3 and out["param_mean_diff"] < 1e-4 and out["param_max_diff"] < 1e-2
                         and all(v == v for v in out["loss"]))
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0 and not out["ok"]:
        sys.exit(1)


if __name__ == "__main__":
    main()
