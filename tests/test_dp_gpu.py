"""Data-parallel path (reduce-scatter fused into wgrad, sharded optimizer, fused weight all-gather) with several
ranks emulated on ONE GPU: the ranks live in one process and run one after another on one stream, so no kernel
ever waits for another launch.  The result must match one replica trained on the concatenated batch."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

from gruboros_b200.models.minlm import minLM
from gruboros_b200.optim.schedulefree import AdamWScheduleFree
from gruboros_b200.parallel.comm import LocalTransport, PeerGroup
from gruboros_b200.parallel.dp import DataParallel
from tests.test_model_cpu import randomize, zipf_bytes


@pytest.mark.parametrize("interleave", [True, False])
@pytest.mark.parametrize("world", [2, 4])
def test_emulated_ranks_match_single_replica(world, interleave):
    """interleave: ownership dealt round-robin in 256 KB chunks (default) or one contiguous shard per rank."""
    torch.manual_seed(0)
    base = minLM(num_tokens=256, dim=128, depth=2)
    randomize(base, 5)
    dev = torch.device("cuda", 0)
    single = copy.deepcopy(base).to(dev)
    osingle = AdamWScheduleFree(single.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
    osingle.train()
    hub = LocalTransport(world)
    models = [copy.deepcopy(base).to(dev) for _ in range(world)]
    dps = [DataParallel(m, rank=r, world=world, device=dev, group=PeerGroup(r, world, dev, hub.for_rank(r)),
                        interleave=interleave) for r, m in enumerate(models)]

    def full(dp, t):                       # a single-replica flat tensor padded to the data-parallel flat length
        out = torch.zeros(dp.flat.numel, device=dev, dtype=t.dtype)
        out[:t.numel()] = t
        return out

    for dp in dps:
        dp.connect()
    opts = []
    for m, dp in zip(models, dps):
        o = AdamWScheduleFree(m.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
        dp.bind_optimizer(o)
        o.train()
        opts.append(o)
    Bper, chunk = 2, 65
    x = zipf_bytes(world * Bper, 3 * chunk, seed=9).to(dev)
    hid_s, hid = None, [None] * world
    for c in range(3):
        ck = x[:, c * chunk:(c + 1) * chunk]
        ls, hid_s = single.fused_engine().train_step(ck, hid_s)
        saved_single_grad = single.fused_engine().flat.grad.clone()
        osingle.step(); osingle.zero_grad()
        losses = []
        for r, m in enumerate(models):
            l, hid[r] = m.fused_engine().train_step(ck[r * Bper:(r + 1) * Bper], hid[r])
            losses.append(l)
        # all signals are queued before any wait, so the waits find their flags already set
        for dp in dps:
            dp.push_vector_grads()
        for dp in dps:
            dp.group.signal_only()
        for dp in dps:
            dp.group.wait_only()
        if c == 0:
            # the reduce-scatter result: the owner's range holds the sum over ranks of the local gradients
            sg = single.fused_engine().flat.grad
            for dp in dps:
                mine = dp.owned(dp.flat.grad) / world
                ref = dp.owned(full(dp, saved_single_grad))
                err = (mine - ref).abs().max().item()
                assert err < 2e-3 * ref.abs().max().item() + 1e-7, (dp.rank, err, ref.abs().max().item())
        for o in opts:
            o.step(); o.zero_grad()
        for dp in dps:
            dp.bcast_vector_params()
        for dp in dps:
            dp.group.signal_only()
        for dp in dps:
            dp.group.wait_only()
        assert abs(torch.stack(losses).mean().item() - ls.item()) < 1e-3
    torch.cuda.synchronize()
    from gruboros_b200.ops import _lib as L
    L.check_device_status()
    # every rank's bf16 weights equal the single replica's; fp32 values match inside the owned range
    sflat = single.fused_engine().flat
    n = sflat.numel
    # Adam-normalised updates amplify rounding noise of near-zero gradient elements, so parameters are compared
    # statistically: after three steps of size <= 1e-3 almost all elements agree closely
    for dp in dps:
        d16 = (dp.flat.w16[:n].float() - sflat.w16.float()).abs()
        assert d16.max().item() < 1e-2 and (d16 > 1e-3).float().mean().item() < 2e-2
        d32 = (dp.owned(dp.flat.data) - dp.owned(full(dp, sflat.data))).abs()
        assert d32.max().item() < 1e-2 and d32.mean().item() < 1e-4, (d32.max().item(), d32.mean().item())
        for p, o in zip(dp.flat.params, dp.flat.offsets):
            if p.dim() < 2 or p is dp.flat.params[0]:     # 1-D parameters and the embedding are fp32 on every rank
                assert (dp.flat.data[o:o + p.numel()] - sflat.data[o:o + p.numel()]).abs().max().item() < 5e-3
    # checkpoint path: after the gathers every rank holds every owner's fp32 parameters and optimizer state
    # (run rank by rank; the barriers inside find their flags set because every rank signals before any waits)
    for dp in dps:
        dp.group.device_barrier = lambda: None
    zs = []
    for dp in dps:
        dp.gather_params()
        zs.append(dp.gather_optimizer_state())
    torch.cuda.synchronize()
    for dp, (z, v) in zip(dps, zs):
        d = (dp.flat.data[:n] - sflat.data).abs()
        assert d.max().item() < 1e-2 and d.mean().item() < 1e-4
        dz = (z[:n] - sflat.sf_z).abs()
        assert dz.mean().item() < 1e-4, dz.mean().item()
        assert torch.equal(z, zs[0][0]) and torch.equal(v, zs[0][1])
    # optimizer state in the per-parameter layout: equals what the single replica's optimizer would save, and loading
    # it back restores every rank's share exactly
    ssd = osingle.state_dict()["state"]
    for dp in dps:
        sd = dp.optimizer_state_dict()
        assert len(sd["state"]) == len(dp.flat.params) and sd["param_groups"][0]["k"] == 3
        for i, p in enumerate(dp.flat.params):
            assert sd["state"][i]["z"].shape == p.shape
            # (Adam-normalised steps of near-zero gradient elements differ in sign between the runs: up to
            # 3 steps x lr per element, so small parameters are compared loosely; a wrong mapping would be off by
            # the parameters' own magnitude)
            dzi = (sd["state"][i]["z"] - ssd[i]["z"].cpu()).abs()
            assert dzi.mean().item() < 2e-3 and dzi.max().item() < 1e-2, (i, dzi.mean().item(), dzi.max().item())
            off = dp.flat.offsets[i]
            assert torch.equal(sd["state"][i]["z"].reshape(-1), zs[0][0][off:off + p.numel()].cpu())
            assert torch.equal(sd["state"][i]["exp_avg_sq"].reshape(-1), zs[0][1][off:off + p.numel()].cpu())
        z_before, v_before = dp.z.clone(), dp.v.clone()
        dp.z.zero_(); dp.v.fill_(7.0)
        dp.load_optimizer_state_dict(sd)
        assert torch.equal(dp.z, z_before) and torch.equal(dp.v, v_before)
        dp.reset_optimizer_state()
        assert torch.equal(dp.z, dp.owned(dp.flat.data).reshape(-1)) and float(dp.v.abs().max()) == 0.0
        dp.z.copy_(z_before); dp.v.copy_(v_before)        # the other ranks' state dicts gather this rank's share


def test_device_barrier_times_out_without_peer():
    """A flag that nobody sets: the bounded wait gives up, sets the status word, and the context stays usable."""
    dev = torch.device("cuda", 0)
    hub = LocalTransport(2)
    g0 = PeerGroup(0, 2, dev, hub.for_rank(0))
    g1 = PeerGroup(1, 2, dev, hub.for_rank(1))
    g0.finish_local_connect(); g1.finish_local_connect()
    g0.signal_only()                      # rank 1 never signals
    g0.wait_only(timeout_ns=50_000_000)   # 50 ms
    torch.cuda.synchronize()
    from gruboros_b200.ops import _lib as L
    with pytest.raises(RuntimeError):
        L.check_device_status(dev)
    assert torch.ones(4, device=dev).sum().item() == 4.0
