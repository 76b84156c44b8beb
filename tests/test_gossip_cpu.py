"""Gossip protocol logic on CPU: tournaments over the TCP transport between nodes living in one process,
merge math, counters, failure handling (host-side only), fitness EMA, ranking, rejuvenation."""
import math
import os
import socket
import time

import pytest
import torch

from gruboros_b200.models.minlm import minLM
from gruboros_b200.optim.schedulefree import AdamWScheduleFree
from gruboros_b200.parallel.gossip import (EvolutionaryTrainingNode, FilesystemCoordinator, FitnessTracker, NetworkUtils,
                                           blend_alpha, pair_ranks)
from gruboros_b200.runtime.checkpoint import build_checkpoint, save_checkpoint_atomic, CheckpointManager


def free_base_port(n=2):
    socks = []
    try:
        while True:
            s = socket.socket(); s.bind(("127.0.0.1", 0)); base = s.getsockname()[1]; s.close()
            ok = True
            for i in range(n):
                t = socket.socket()
                try:
                    t.bind(("127.0.0.1", base + i)); socks.append(t)
                except OSError:
                    ok = False
                    break
            for t in socks:
                t.close()
            socks.clear()
            if ok:
                return base
    finally:
        for t in socks:
            t.close()


def tiny(seed):
    torch.manual_seed(seed)
    m = minLM(num_tokens=256, dim=32, depth=1)
    with torch.no_grad():
        for p in m.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    o = AdamWScheduleFree(m.parameters(), lr=1e-3, betas=(0.9, 0.995))
    o.train()
    x = torch.randint(0, 256, (2, 17))
    m(x, return_loss=True).backward()
    o.step(); o.zero_grad()
    return m, o


def make_nodes(tmp_path, monkeypatch, **kw):
    base = free_base_port(2)
    monkeypatch.setenv("GOSSIP_BASE_PORT", str(base))
    monkeypatch.setenv("GOSSIP_STARTUP_DELAY", "0.1")
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    nodes = []
    for r in range(2):
        m, o = tiny(r)
        peers = [f"localhost:{base + q}" for q in range(2) if q != r]
        n = EvolutionaryTrainingNode(f"node_{r}", m, o, global_rank=r, local_rank=r, world_size=2, mixing_probability=1.0,
                                     output_dir=str(tmp_path), gossip_temp_dir=str(tmp_path / "tmp"), transport="tcp",
                                     bootstrap_nodes=peers, **kw)
        nodes.append(n)
    return nodes


def wait_for(cond, timeout=20.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        if cond():
            return True
        time.sleep(0.05)
    return False


def test_fitness_tracker_ema():
    f = FitnessTracker(decay_factor=0.9)
    assert math.isinf(f.get_fitness())
    f.update(2.0); f.update(1.0)
    assert abs(f.get_fitness() - (0.1 * 1.0 + 0.9 * 2.0)) < 1e-12
    f.inherit_fitness(0.5)
    assert f.get_fitness() == 0.5


def test_pairing_is_a_matching_and_shared():
    for world in (2, 5, 8):
        for rnd in range(5):
            pairs = pair_ranks(world, rnd)
            flat = [r for p in pairs for r in p]
            assert len(flat) == len(set(flat)) == world - world % 2
            assert pairs == pair_ranks(world, rnd)
    assert pair_ranks(8, 1) != pair_ranks(8, 2)
    assert blend_alpha("fixed", 0.3, 5.0, 1.0) == 0.3
    assert abs(blend_alpha("softmax", 0.3, 2.0, 2.0) - 0.5) < 1e-12
    assert blend_alpha("softmax", 0.3, 5.0, 1.0) > 0.9


@pytest.mark.parametrize("method,opt_mode", [("clonal", "interpolate"), ("recombination", "interpolate"), ("recombination", "reset")])
def test_tcp_tournament_winner_flows_to_loser(tmp_path, monkeypatch, method, opt_mode):
    nodes = make_nodes(tmp_path, monkeypatch, merge_method=method, recombination_alpha=0.25, optimizer_recombination=opt_mode)
    good, bad = nodes
    good.update_fitness(1.0, 0); bad.update_fitness(3.0, 0)       # node 0 is fitter
    before_bad = {k: v.clone() for k, v in bad.model.state_dict().items()}
    good_sd = {k: v.clone() for k, v in good.model.state_dict().items()}
    z_bad = bad.optimizer.state[next(bad.model.parameters())]["z"].clone()
    z_good = good.optimizer.state[next(good.model.parameters())]["z"].clone()
    for n in nodes:
        n.start_gossip_protocol()
    try:
        assert wait_for(lambda: bad.mixes_lost >= 1 and not bad.incoming_updates.empty(), 30)
        bad.mixing_probability = good.mixing_probability = 0.0
        bad.check_for_updates()
        applied, needs_reset = bad.apply_pending_update()
        assert applied and needs_reset == (method == "recombination" and opt_mode == "reset")
        p_name = "token_emb.weight"
        if method == "clonal":
            torch.testing.assert_close(bad.model.state_dict()[p_name], good_sd[p_name])
            assert bad.get_current_fitness() == pytest.approx(1.0)
        else:
            want = before_bad[p_name] * 0.75 + good_sd[p_name] * 0.25
            torch.testing.assert_close(bad.model.state_dict()[p_name], want)
            assert bad.get_current_fitness() == pytest.approx(3.0)        # fitness is not inherited
            z_now = bad.optimizer.state[next(bad.model.parameters())]["z"]
            if opt_mode == "interpolate":
                torch.testing.assert_close(z_now, z_bad * 0.75 + z_good * 0.25)
            else:
                torch.testing.assert_close(z_now, z_bad)
        st_good, st_bad = good.get_status(), bad.get_status()
        assert st_good["won_mixes"] >= 1 and st_bad["lost_mixes"] >= 1
        assert st_bad["successful_mixes"] == 1
        assert st_good["failed_mixes"] >= 0 and st_bad["failed_mixes"] >= 0
        log = open(bad.logger.log_file).read()
        assert "WEIGHT_RECEIVE_COMPLETE" in log and log.splitlines()[0].split("\t")[4] == "event_type"
    finally:
        for n in nodes:
            n.stop_gossip_protocol()


def test_compat_mode_reproduces_reference_noop_interpolation(tmp_path, monkeypatch):
    nodes = make_nodes(tmp_path, monkeypatch, merge_method="recombination", recombination_alpha=0.5,
                       optimizer_recombination="interpolate", compat=True)
    good, bad = nodes
    winner = good._snapshot()
    z_before = bad.optimizer.state[next(bad.model.parameters())]["z"].clone()
    bad._merge_state_dicts(winner["model_state_dict"], winner["optimizer_state_dict"], 1.0)
    torch.testing.assert_close(bad.optimizer.state[next(bad.model.parameters())]["z"], z_before)


def test_dead_peer_is_a_failed_mix_not_an_error(tmp_path, monkeypatch):
    nodes = make_nodes(tmp_path, monkeypatch)
    alive = nodes[0]
    alive.listen = True
    alive.update_fitness(2.0, 0)
    alive.start_gossip_protocol()                 # node 1 never starts: connection refused
    try:
        for s in range(1, 4):
            alive.update_fitness(2.0, s)
        assert wait_for(lambda: "MIX_ATTEMPT_FAILED" in open(alive.logger.log_file).read(), 20)
        st = alive.get_status()
        assert st["failed_mixes"] >= 1
        assert st["won_mixes"] == 0 and st["lost_mixes"] == 0
        assert "MIX_ATTEMPT_FAILED" in open(alive.logger.log_file).read()
    finally:
        alive.stop_gossip_protocol()


def test_truncated_payload_is_rejected(tmp_path, monkeypatch):
    nodes = make_nodes(tmp_path, monkeypatch)
    a, b = socket.socketpair()
    try:
        a.sendall((1000).to_bytes(8, "big") + b"x" * 10)
        a.close()
        assert nodes[0]._receive_weights_from_peer(b, "cid", "peer") is None
        assert "WEIGHT_RECEIVE_ERROR" in open(nodes[0].logger.log_file).read()
    finally:
        b.close()


def test_filesystem_coordinator_ranking(tmp_path):
    cs = [FilesystemCoordinator(r, 3, str(tmp_path)) for r in range(3)]
    for c, fit in zip(cs, (2.0, 1.0, 3.0)):
        c.set_fitness_provider(lambda fit=fit: fit)
        assert c.publish()
    stale = os.path.join(cs[0].fitness_dir, "rank_0009.json")
    open(stale, "w").write('{"rank": 9, "fitness": 0.1, "timestamp": 0}')
    ranks = cs[0].rank_population()
    assert ranks == {1: 0.0, 0: 0.5, 2: 1.0}
    for c in cs:
        c.refresh()
    assert [c.get_my_percentile() for c in cs] == [0.5, 0.0, 1.0]


def test_rejuvenation_prefers_better_then_older_elite(tmp_path):
    m, o = tiny(0)
    node = EvolutionaryTrainingNode("n", m, o, 0, 0, 1, output_dir=str(tmp_path), gossip_temp_dir=str(tmp_path / "t"),
                                    transport="tcp", bootstrap_nodes=[])
    node.update_fitness(2.0, 0)
    donor, od = tiny(7)
    cfg = dict(num_tokens=256, dim=32, depth=1)
    for step, loss in ((10, 1.5000), (50, 1.4990), (20, 2.5)):
        save_checkpoint_atomic(build_checkpoint(step, donor, od, loss, cfg), str(tmp_path), step, 0, loss)
    CheckpointManager(str(tmp_path), keep_elite_n=5).run_once()
    before = m.token_emb.weight.detach().clone()
    ok, reset = node.attempt_rejuvenation(m, alpha=0.5, tiebreaker_threshold=0.005)
    assert ok and reset
    torch.testing.assert_close(m.token_emb.weight.detach(), 0.5 * before + 0.5 * donor.token_emb.weight.detach())
    assert node.get_current_fitness() == pytest.approx(1.4990)      # marginally better and more steps wins the tie
    assert "S:50" in open(node.logger.log_file).read()


def test_network_utils_conventions(monkeypatch, tmp_path):
    monkeypatch.delenv("GOSSIP_BASE_PORT", raising=False)
    assert NetworkUtils.get_gossip_port(3) == 29504
    monkeypatch.chdir(tmp_path)
    monkeypatch.delenv("SLURM_JOB_NODELIST", raising=False)
    monkeypatch.setenv("SLURM_JOB_ID", "77")
    monkeypatch.setenv("RANKS_PER_NODE", "2")
    (tmp_path / "hostfile-job77.txt").write_text("nodeA slots=2\nnodeB slots=2\n")
    peers = NetworkUtils.get_bootstrap_nodes(0, 0)
    assert peers == ["nodeA:29501", "nodeA:29502", "nodeB:29501", "nodeB:29502"]


def test_hybrid_transport_chooses_per_pair(tmp_path, monkeypatch):
    """``hybrid``: NVLink rounds among the ranks of a box, the TCP protocol with everybody else.  On CPU the box of
    one rank has no NVLink partner, so the node falls back to TCP for every pair and still completes a tournament."""
    # membership and per-pair choice with peer memory stubbed out (no GPU needed for the bookkeeping)
    class Stub(EvolutionaryTrainingNode):
        def _setup_nvlink(self):
            self.stubbed = True

    m, o = tiny(0)
    n = Stub("node_5", m, o, global_rank=5, local_rank=1, world_size=8, output_dir=str(tmp_path), transport="hybrid",
             box_size=4, gossip_temp_dir=str(tmp_path / "tmp"), bootstrap_nodes=[], listen=False)
    assert n.stubbed and n.nv_members == [4, 5, 6, 7] and n.nv_rank == 1 and n.uses_nvlink and n.uses_tcp
    assert [n.transport_for(r) for r in (4, 6, 7)] == ["nvlink"] * 3
    assert [n.transport_for(r) for r in (0, 3, 5)] == ["tcp"] * 3
    peers = EvolutionaryTrainingNode.cross_box_peers(["nodeA:29501", "nodeA:29502", "nodeB:29501", "localhost:29503"], "nodeA")
    assert peers == ["nodeB:29501"]
    # a box of one rank: pure TCP behaviour, end to end
    base = free_base_port(2)
    monkeypatch.setenv("GOSSIP_BASE_PORT", str(base))
    monkeypatch.setenv("GOSSIP_STARTUP_DELAY", "0.1")
    nodes = []
    for r in range(2):
        mm, oo = tiny(r)
        nodes.append(EvolutionaryTrainingNode(f"node_{r}", mm, oo, global_rank=r, local_rank=r, world_size=2,
                                              mixing_probability=1.0, output_dir=str(tmp_path), transport="hybrid", box_size=1,
                                              gossip_temp_dir=str(tmp_path / "tmp"), merge_method="clonal",
                                              bootstrap_nodes=[f"localhost:{base + q}" for q in range(2) if q != r]))
    good, bad = nodes
    assert not good.uses_nvlink and good.transport_for(1) == "tcp"
    good.update_fitness(1.0, 0); bad.update_fitness(3.0, 0)
    want = good.model.state_dict()["token_emb.weight"].clone()
    for nd in nodes:
        nd.start_gossip_protocol()
    try:
        assert wait_for(lambda: bad.mixes_lost >= 1 and not bad.incoming_updates.empty(), 30)
        bad.mixing_probability = good.mixing_probability = 0.0
        bad.check_for_updates()
        applied, _ = bad.apply_pending_update()
        assert applied
        torch.testing.assert_close(bad.model.state_dict()["token_emb.weight"], want)
    finally:
        for nd in nodes:
            nd.stop_gossip_protocol()
