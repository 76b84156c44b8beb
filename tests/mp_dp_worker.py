"""Worker for the multi-GPU data-parallel test (launched by torchrun, one rank per GPU).

Every rank builds the same model and the same global batch, trains on its slice through DataParallel
(reduce-scatter fused into wgrad over NVLink peer memory), and rank 0 also trains a single replica on the
whole batch.  Prints one JSON line with the comparison."""
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
from gruboros_b200.parallel.dp import DataParallel
from gruboros_b200.runtime.trainer import Trainer
from tests.test_model_cpu import randomize, zipf_bytes


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    base = minLM(num_tokens=256, dim=256, depth=2)
    randomize(base, 5)
    model = copy.deepcopy(base).to(dev)
    fold = os.environ.get("DP_FOLD", "1") == "1"
    # ownership of the flat space: dealt round-robin in chunks (default) or one contiguous shard per rank
    nvls = os.environ.get("DP_NVLS", "0") == "1"
    if nvls:
        from gruboros_b200.parallel import nvls as nv
        ok_here = torch.tensor([int(nv.supported(local))], device=dev)
        dist.all_reduce(ok_here, op=dist.ReduceOp.MIN)
        if not int(ok_here.item()):
            if rank == 0:
                print(json.dumps({"ok": True, "skipped": "the driver reports no NVSwitch multicast support"}), flush=True)
            dist.barrier(); dist.destroy_process_group()
            return
    dp = DataParallel(model, rank=rank, world=world, device=dev, interleave=os.environ.get("DP_INTERLEAVE", "1") == "1",
                      nvls=nvls)
    opt = AdamWScheduleFree(model.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
    dp.bind_optimizer(opt)
    opt.train()
    trainer = Trainer(model, opt, chunk_size=129, grad_accum=1, parallel=dp)
    # DP_FOLD=1: the sharded optimizer runs per layer inside backward (cross-rank flags); 0: after backward
    trainer.fold_parallel = fold
    Bper = 2
    x = zipf_bytes(world * Bper, 3 * 129, seed=9).to(dev)
    mine = x[rank * Bper:(rank + 1) * Bper]
    losses = trainer.train_sequence(mine)
    torch.cuda.synchronize()
    L.check_device_status()
    mean_loss = torch.stack(losses).clone()
    dist.all_reduce(mean_loss)
    mean_loss /= world
    # checkpoint path: every rank pulls the shards it does not own
    dp.gather_params()
    z, v = dp.gather_optimizer_state()
    torch.cuda.synchronize()
    L.check_device_status()
    # every rank's bf16 weight mirror holds the same values (published by the owners: peer stores or one multimem store)
    mirror = dp.flat.w16.float().double()
    sums = torch.stack([mirror.sum(), (mirror * mirror).sum()])
    allsums = [torch.zeros_like(sums) for _ in range(world)]
    dist.all_gather(allsums, sums)
    mirrors_equal = all(torch.equal(a, allsums[0]) for a in allsums)
    out = {"rank": rank, "loss": mean_loss.tolist(), "folded": trainer.last_folded, "interleave": dp.interleave,
           "steps": trainer.optimizer_steps, "mirrors_equal": mirrors_equal, "nvls": dp.mc16 is not None}
    if rank == 0:
        single = copy.deepcopy(base).to(dev)
        osingle = AdamWScheduleFree(single.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
        osingle.train()
        ts = Trainer(single, osingle, chunk_size=129, grad_accum=1)
        ls = torch.stack(ts.train_sequence(x))
        sflat = single.fused_engine().flat
        n = sflat.numel
        d = (dp.flat.data[:n] - sflat.data).abs()
        dz = (z[:n] - sflat.sf_z).abs()
        out.update(single_loss=ls.tolist(), param_max_diff=d.max().item(), param_mean_diff=d.mean().item(),
                   z_mean_diff=dz.mean().item(), loss_max_diff=(ls - mean_loss).abs().max().item())
        ok = (out["loss_max_diff"] < 2e-3 and out["param_mean_diff"] < 1e-4 and out["param_max_diff"] < 1e-2
              and mirrors_equal)
        out["ok"] = bool(ok)
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0 and not out["ok"]:
        sys.exit(1)


if __name__ == "__main__":
    main()
