"""Fully sharded data parallel path with the ranks emulated on ONE GPU (run one after another on one stream).
bf16 weights are sharded at rest; non-owned ranges are poisoned with NaN whenever they go stale, so a finite loss
that matches a single replica proves that every weight a kernel read had been all-gathered first."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

from gruboros_b200.models.minlm import minLM
from gruboros_b200.optim.schedulefree import AdamWScheduleFree
from gruboros_b200.ops import kernels as K
from gruboros_b200.parallel.comm import LocalTransport, PeerGroup
from gruboros_b200.parallel.fsdp import FullyShardedDataParallel
from tests.test_model_cpu import randomize, zipf_bytes


@pytest.mark.parametrize("interleave", [True, False])
@pytest.mark.parametrize("world,reshard,mode", [(2, False, "auto"), (4, True, "auto"), (2, True, "2cta")])
def test_emulated_fsdp_matches_single_replica(world, reshard, mode, interleave):
    """interleave: gradients / optimizer state dealt in chunks over the ranks (the bf16 weights stay in one
    contiguous shard per rank) or everything in the contiguous shard."""
    old_mode, K.GEMM_MODE = K.GEMM_MODE, mode
    try:
        torch.manual_seed(0)
        base = minLM(num_tokens=256, dim=128, depth=3)
        randomize(base, 5)
        dev = torch.device("cuda", 0)
        single = copy.deepcopy(base).to(dev)
        osingle = AdamWScheduleFree(single.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
        osingle.train()
        hub = LocalTransport(world)
        models = [copy.deepcopy(base).to(dev) for _ in range(world)]
        fs = [FullyShardedDataParallel(m, rank=r, world=world, device=dev, group=PeerGroup(r, world, dev, hub.for_rank(r)),
                                       reshard_after_forward=reshard, debug_poison=True, interleave=interleave)
              for r, m in enumerate(models)]
        for f in fs:
            f.connect()
        opts = []
        for m, f in zip(models, fs):
            o = AdamWScheduleFree(m.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
            f.bind_optimizer(o)
            o.train()
            opts.append(o)
        Bper, chunk = 2, 65
        x = zipf_bytes(world * Bper, 4 * chunk, seed=9).to(dev)
        hid_s, hid = None, [None] * world
        for c in range(4):
            ck = x[:, c * chunk:(c + 1) * chunk]
            ls, hid_s = single.fused_engine().train_step(ck, hid_s)
            osingle.step(); osingle.zero_grad()
            losses = []
            for r, m in enumerate(models):
                l, hid[r] = m.fused_engine().train_step(ck[r * Bper:(r + 1) * Bper], hid[r])
                losses.append(l)
            for f in fs:
                f.push_vector_grads()
            for f in fs:
                f.group.signal_only()
            for f in fs:
                f.group.wait_only()
            for o in opts:
                o.step(); o.zero_grad()
            for f in fs:
                f.bcast_vector_params()
            for f in fs:
                f.group.signal_only()
            for f in fs:
                f.group.wait_only()
            for f in fs:
                f._drop_all()
            mean = torch.stack(losses).mean().item()
            assert mean == mean and abs(mean - ls.item()) < 2e-3, (c, mean, ls.item())
        torch.cuda.synchronize()
        from gruboros_b200.ops import _lib as L
        L.check_device_status()
        assert all(f.gathered_bytes > 0 for f in fs)
        # each rank's owned bf16 range equals the single replica's
        sflat = single.fused_engine().flat
        for f in fs:
            lo, hi = f.begin, min(f.begin + f.shard, sflat.numel)
            d = (f.flat.w16[lo:hi].float() - sflat.w16[lo:hi].float()).abs()
            assert d.max().item() < 1e-2 and (d > 1e-3).float().mean().item() < 2e-2
    finally:
        K.GEMM_MODE = old_mode
