"""Fully sharded (ZeRO-3) path with the ranks emulated on ONE GPU (run one after another on one stream).
Every rank keeps only its packed share of masters, gradients, optimizer state and bf16 weights; a layer's weights
exist in full only inside one of two workspace slots, which are poisoned with NaN whenever they go stale - so a
finite loss that matches a single replica proves that every weight a kernel read had been all-gathered first."""
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


def _build(world, dim, depth):
    torch.manual_seed(0)
    base = minLM(num_tokens=256, dim=dim, depth=depth)
    randomize(base, 5)
    dev = torch.device("cuda", 0)
    single = copy.deepcopy(base).to(dev)
    hub = LocalTransport(world)
    models = [copy.deepcopy(base).to(dev) for _ in range(world)]
    fs = [FullyShardedDataParallel(m, rank=r, world=world, device=dev, group=PeerGroup(r, world, dev, hub.for_rank(r)),
                                   debug_poison=True) for r, m in enumerate(models)]
    for f in fs:
        f.connect()
    return base, single, models, fs, dev


@pytest.mark.parametrize("world,mode", [(2, "auto"), (4, "auto"), (2, "2cta")])
def test_emulated_fsdp_matches_single_replica(world, mode):
    old_mode, K.GEMM_MODE = K.GEMM_MODE, mode
    try:
        base, single, models, fs, dev = _build(world, 128, 3)
        osingle = AdamWScheduleFree(single.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
        osingle.train()
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
            # all signals are queued before any wait, so the waits find their flags already set
            for f in fs:
                f.push_vector_grads()
            for f in fs:
                f.group.signal_only()
            for f in fs:
                f.group.wait_only()
            for o in opts:
                o.step(); o.zero_grad()
            for f in fs:
                f.bcast_small_params()
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
        # every rank's packed masters equal the single replica's values of the chunks it owns, and the small
        # replicated space is identical on all ranks
        sflat = single.fused_engine().flat
        names = {n: i for i, n in enumerate(sflat.names)}
        chunk_el = 1 << fs[0].CHUNK_SHIFT
        full = torch.zeros(fs[0].big.numel, device=dev)
        for j, n in enumerate(fs[0].big.names):
            fs[0].big.view(full, j).copy_(sflat.view(sflat.data, names[n]))
        for f in fs:
            want = full.view(-1, world, chunk_el)[:, f.rank].reshape(-1)
            d = (f.y - want).abs()
            assert d.max().item() < 1e-2 and d.mean().item() < 1e-4, (f.rank, d.max().item(), d.mean().item())
            assert torch.equal(f.w16, f.y.bfloat16())
            assert torch.equal(f.small.data, fs[0].small.data)
        for j, n in enumerate(fs[0].small.names):
            d = (fs[1].small.view(fs[1].small.data, j) - sflat.view(sflat.data, names[n])).abs().max().item()
            assert d < 1e-2, (n, d)
    finally:
        K.GEMM_MODE = old_mode


def test_sharded_memory_and_checkpoint_round_trip():
    """Per-rank persistent bytes are 1/world of the unsharded total (+ the small replicated space); gathering
    gives back the full reference-layout state_dict and optimizer state, which load into fresh shards."""
    world = 4
    base, single, models, fs, dev = _build(world, 128, 2)
    for f in fs:
        b = f.persistent_bytes()
        assert b["sharded_params_grads_state"] * world == b["unsharded_equivalent"]
        assert b["replicated_small"] < 0.2 * b["unsharded_equivalent"]
        assert all(p.numel() == 0 for p in f.big.params)          # no full matrix anywhere at rest
    opts = []
    for m, f in zip(models, fs):
        o = AdamWScheduleFree(m.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
        f.bind_optimizer(o); o.train(); opts.append(o)
    for f in fs:        # LocalTransport ranks run one after another: barriers are signal-all-then-wait-all
        f.group.device_barrier = lambda: None
    fs[1].gather_params()
    sd = models[1].state_dict()
    ref = base.state_dict()
    assert list(sd) == list(ref)
    for k in ref:
        assert torch.equal(sd[k].cpu(), ref[k]), k
    osd = fs[1].optimizer_state_dict()
    assert set(osd["state"][0]) == {"z", "exp_avg_sq"} and len(osd["state"]) == len(ref)
    for i, (k, v) in enumerate(ref.items()):
        assert torch.equal(osd["state"][i]["z"], v), k
    fs[1].release_params()
    assert all(p.numel() == 0 for p in fs[1].big.params)
    # perturb, then restore from the saved optimizer state
    fs[2].z.add_(1.0); fs[2].v.add_(1.0)
    fs[2].load_optimizer_state_dict(osd)
    want = fs[2].y
    assert torch.equal(fs[2].z, want) and float(fs[2].v.abs().max()) == 0.0
