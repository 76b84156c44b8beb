"""Worker for the multi-GPU gossip test (torchrun, one rank per GPU): every rank trains its own replica on its own
data; every 2 optimizer steps a tournament round runs over NVLink peer memory (clonal merge).  After a round the
loser must hold exactly the winner's parameters and Schedule-Free state."""
import json
import os
import sys
import tempfile
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from gruboros_b200.models.minlm import minLM
from gruboros_b200.optim.schedulefree import AdamWScheduleFree
from gruboros_b200.ops import _lib as L
from gruboros_b200.parallel.gossip import EvolutionaryTrainingNode, pair_ranks
from tests.test_model_cpu import randomize, zipf_bytes


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    host = dist.new_group(backend="gloo")
    torch.manual_seed(0)
    model = minLM(num_tokens=256, dim=256, depth=2)
    randomize(model, 5 + rank)
    model = model.to(dev)
    opt = AdamWScheduleFree(model.parameters(), lr=1e-3, betas=(0.9, 0.995))
    opt.train()
    out_dir = os.environ.get("GOSSIP_TEST_DIR") or tempfile.mkdtemp()
    node = EvolutionaryTrainingNode(f"node_{rank}", model, opt, rank, local, world, output_dir=out_dir,
                                    gossip_temp_dir=os.path.join(out_dir, "tmp"), transport="nvlink", gossip_every=2,
                                    merge_method="clonal", host_group=host, bootstrap_nodes=[])
    node.start_gossip_protocol()
    x = zipf_bytes(2, 4 * 65, seed=100 + rank).to(dev)
    applied_any = False
    for step in range(4):
        node.apply_pending_update()
        loss = model(x[:, step * 65:(step + 1) * 65], return_loss=True)
        loss.backward()
        opt.step(); opt.zero_grad()
        node.update_fitness(loss.item() + rank, step)       # rank 0 always has the best fitness
        node.check_for_updates()
        a, _ = node._last_round_result
        applied_any |= a
        if (step + 1) % 2 == 0:
            # right after a round: compare checksums of each pair
            flat = node.flat
            sums = torch.stack([flat.data.double().sum(), flat.sf_z.double().sum(), flat.sf_v.double().sum()])
            allsums = [torch.zeros_like(sums) for _ in range(world)]
            dist.all_gather(allsums, sums)
            pairs = pair_ranks(world, node.rounds)
            for p, q in pairs:
                if rank in (p, q):
                    assert torch.equal(allsums[p], allsums[q]), (step, p, q, allsums[p], allsums[q])
    torch.cuda.synchronize()
    L.check_device_status()
    st = node.get_status()
    node.stop_gossip_protocol()
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "won": st["won_mixes"], "lost": st["lost_mixes"], "failed": st["failed_mixes"],
                                      "transfer": getattr(node, "last_transfer", None)})
    if rank == 0:
        ok = sum(g["won"] for g in gathered) == sum(g["lost"] for g in gathered) > 0 and all(g["failed"] == 0 for g in gathered)
        print(json.dumps({"ok": bool(ok), "status": gathered}), flush=True)
        if not ok:
            sys.exit(1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
