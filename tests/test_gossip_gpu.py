"""NVLink gossip data plane with the ranks emulated on ONE GPU (one process, one stream, phases interleaved so
that no kernel ever waits on a later launch): the loser's fused transfer+merge kernel against host-computed
merges, for clonal / recombination (fixed and softmax alpha) / optimizer interpolation and reset."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

from gruboros_b200.models.minlm import minLM
from gruboros_b200.optim.schedulefree import AdamWScheduleFree
from gruboros_b200.parallel.comm import LocalTransport, PeerGroup
from gruboros_b200.parallel.gossip import EvolutionaryTrainingNode, blend_alpha, pair_ranks
from tests.test_model_cpu import randomize, zipf_bytes


def build(world, tmp_path, **kw):
    dev = torch.device("cuda", 0)
    hub = LocalTransport(world)
    nodes = []
    for r in range(world):
        torch.manual_seed(r)
        m = minLM(num_tokens=256, dim=128, depth=2)
        randomize(m, 10 + r)
        m = m.to(dev)
        o = AdamWScheduleFree(m.parameters(), lr=1e-3, betas=(0.9, 0.995))
        o.train()
        n = EvolutionaryTrainingNode(f"node_{r}", m, o, r, r, world, output_dir=str(tmp_path), gossip_temp_dir=str(tmp_path / "t"),
                                     transport="nvlink", gossip_every=1, peer_group=PeerGroup(r, world, dev, hub.for_rank(r)),
                                     bootstrap_nodes=[], **kw)
        nodes.append(n)
    for n in nodes:
        n.finish_nvlink_connect()
    x = zipf_bytes(2, 65, seed=3).to(dev)
    for r, n in enumerate(nodes):                       # one training step each so that z, v are non-trivial
        loss = n.model(x, return_loss=True)
        loss.backward()
        n.optimizer.step(); n.optimizer.zero_grad()
        n.update_fitness(1.0 + r, 0)                    # rank 0 is the fittest
    return nodes


def run_round(nodes):
    board = [{"rank": n.global_rank, "fitness": n.get_current_fitness(), "k": n.optimizer.param_groups[0]["k"] + 10 * n.global_rank,
              "weight_sum": n.optimizer.param_groups[0]["weight_sum"], "lr_max": n.optimizer.param_groups[0]["lr_max"]} for n in nodes]
    ctxs = [n._round_begin(board) for n in nodes]
    for n, c in zip(nodes, ctxs):
        n._round_transfer(c)
    return [n._round_end(c) for n, c in zip(nodes, ctxs)], board


@pytest.mark.parametrize("method,opt_mode,alpha_mode", [("clonal", "interpolate", "fixed"), ("recombination", "interpolate", "fixed"),
                                                        ("recombination", "interpolate", "softmax"), ("recombination", "reset", "fixed")])
def test_fused_transfer_merge_matches_host_merge(tmp_path, method, opt_mode, alpha_mode):
    nodes = build(2, tmp_path, merge_method=method, recombination_alpha=0.3, optimizer_recombination=opt_mode, alpha_mode=alpha_mode)
    win, lose = nodes
    snap = lambda n: (n.flat.data.clone(), n.flat.sf_z.clone(), n.flat.sf_v.clone())
    wy, wz, wv = snap(win)
    ly, lz, lv = snap(lose)
    results, board = run_round(nodes)
    assert results[0] == (False, False)
    assert results[1] == (True, method == "recombination" and opt_mode == "reset")
    y, z, v = snap(lose)
    if method == "clonal":
        assert torch.equal(y, wy) and torch.equal(z, wz) and torch.equal(v, wv)
        assert lose.get_current_fitness() == pytest.approx(1.0)
        assert lose.optimizer.param_groups[0]["k"] == board[0]["k"]
    else:
        a = blend_alpha(alpha_mode, 0.3, 2.0, 1.0)
        torch.testing.assert_close(y, ly + a * (wy - ly), rtol=1e-6, atol=1e-6)
        if opt_mode == "interpolate":
            torch.testing.assert_close(z, lz + a * (wz - lz), rtol=1e-6, atol=1e-6)
            torch.testing.assert_close(v, lv + a * (wv - lv), rtol=1e-6, atol=1e-7)
        else:
            assert torch.equal(z, lz) and torch.equal(v, lv)
        assert lose.get_current_fitness() == pytest.approx(2.0)
    assert torch.equal(lose.flat.w16, lose.flat.data.bfloat16())          # bf16 mirror rewritten in the same pass
    wy2, _, _ = snap(win)
    assert torch.equal(wy2, wy)                                            # the winner is untouched
    assert win.get_status()["won_mixes"] == 1 and lose.get_status()["lost_mixes"] == 1 and lose.successful_mixes == 1
    assert "NVLink peer read fused with merge" in open(lose.logger.log_file).read()
    # the merged model still trains through the fused engine
    x = zipf_bytes(2, 65, seed=4).cuda()
    assert torch.isfinite(lose.model(x, return_loss=True))


def test_four_rank_round_pairs_everyone(tmp_path):
    nodes = build(4, tmp_path, merge_method="clonal")
    before = [n.flat.data.clone() for n in nodes]
    results, _ = run_round(nodes)
    pairs = pair_ranks(4, 1)
    for a, b in pairs:
        w, l = (a, b) if a < b else (b, a)             # fitness = 1 + rank
        assert torch.equal(nodes[l].flat.data, before[w])
        assert torch.equal(nodes[w].flat.data, before[w])
        assert results[l][0] and not results[w][0]
