"""Optimizer, TBPTT integration against the reference, data, checkpoints, sizing - all on CPU."""
import json
import math
import os
import time

import numpy as np
import pytest
import torch

from baseline.schedulefree_shim import AdamWScheduleFree as ShimSF
from gruboros_b200.models.minlm import minLM
from gruboros_b200.optim.schedulefree import AdamWScheduleFree
from gruboros_b200.runtime.checkpoint import (CheckpointManager, CkptEntry, build_checkpoint, checkpoint_name,
                                              load_checkpoint, plan_retention, save_checkpoint_atomic)
from gruboros_b200.runtime.data import ContinuousIIDDataset, SequenceLoader, ZipfBytes
from gruboros_b200.runtime.trainer import Trainer
from gruboros_b200.utils.locks import file_lock
from gruboros_b200.utils.sizes import (calculate_model_size, parse_size_with_suffix, resolve_model_config,
                                       solve_for_depth, solve_for_dimension)
from tests.refload import load_reference_mingru
from tests.test_model_cpu import zipf_bytes

REF = load_reference_mingru()


def test_schedulefree_matches_upstream_algorithm_for_100_steps():
    torch.manual_seed(0)
    w0 = torch.randn(37, 11)
    a, b = torch.nn.Parameter(w0.clone()), torch.nn.Parameter(w0.clone())
    kw = dict(lr=3e-3, betas=(0.9, 0.995), weight_decay=1e-2, warmup_steps=10)
    oa, ob = AdamWScheduleFree([a], **kw), ShimSF([b], **kw)
    oa.train(); ob.train()
    for i in range(100):
        g = torch.randn(37, 11, generator=torch.Generator().manual_seed(i))
        a.grad, b.grad = g.clone(), g.clone()
        oa.step(); ob.step()
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    sa, sb = oa.state_dict(), ob.state_dict()
    assert set(sa["state"][0]) == set(sb["state"][0]) == {"z", "exp_avg_sq"}
    ga, gb = sa["param_groups"][0], sb["param_groups"][0]
    for k in ("k", "lr_max", "weight_sum", "train_mode", "scheduled_lr", "warmup_steps", "r", "weight_lr_power"):
        assert ga[k] == pytest.approx(gb[k]), k
    # eval / train swap and state_dict interchange
    oa.eval(); ob.eval()
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    oa.train()
    c = torch.nn.Parameter(a.detach().clone())
    oc = AdamWScheduleFree([c], **kw)
    oc.load_state_dict(sb)                      # optimizer state written by the other implementation loads
    assert oc.param_groups[0]["k"] == 100
    with pytest.raises(RuntimeError):
        oa.eval(); oa.step()


@pytest.mark.skipif(REF is None, reason="reference tree not present")
def test_config1_tbptt_loss_curve_matches_reference():
    """D512 x 6, batch 2, seq 512 as two chunks of 256 with carry, Zipf(1.1) bytes, 20 Schedule-Free AdamW steps
    (lr 1e-3), fp32 on CPU: our framework vs the reference model + stand-in optimizer."""
    _, ref_l = REF
    cfg = dict(num_tokens=256, dim=512, depth=6, ff_mult=4, expansion=1.5)
    torch.manual_seed(42)
    ours = minLM(**cfg)
    ref = ref_l.minLM(**cfg)
    ref.load_state_dict(ours.state_dict())
    oo = AdamWScheduleFree(ours.parameters(), lr=1e-3); oo.train()
    orf = ShimSF(ref.parameters(), lr=1e-3); orf.train()
    trainer = Trainer(ours, oo, chunk_size=256)
    data = zipf_bytes(10 * 2, 512, seed=11).view(10, 2, 512)
    lo, lr = [], []
    t0 = time.time()
    for seq in data:
        lo += [l.item() for l in trainer.train_sequence(seq)]
    t_ours = time.time() - t0
    t0 = time.time()
    for seq in data:
        hid = None
        for c in range(2):
            loss, hid = ref(seq[:, c * 256:(c + 1) * 256], return_loss=True, return_prev_hiddens=True, prev_hiddens=hid)
            loss.backward()
            hid = [h.detach() for h in hid]
            orf.step(); orf.zero_grad()
            lr.append(loss.item())
    t_ref = time.time() - t0
    assert len(lo) == len(lr) == 20
    assert abs(lo[0] - math.log(256)) < 0.01
    assert max(abs(a - b) for a, b in zip(lo, lr)) < 2e-3, (lo, lr)
    assert lo[-1] < lo[0] - 0.5                                  # it learns the Zipf marginal
    print(f"config-1 CPU: ours {t_ours / 20:.3f} s/step, reference {t_ref / 20:.3f} s/step, final loss {lo[-1]:.4f}")


def test_sizes():
    assert parse_size_with_suffix("2k") == 2048 and parse_size_with_suffix("100m") == 100 * 2 ** 20
    assert parse_size_with_suffix("1g") == 2 ** 30 and parse_size_with_suffix("1.5k") == 1536 and parse_size_with_suffix(7) == 7
    c = resolve_model_config("1g")
    assert (c["dim"], c["depth"]) == (1024, 82)
    c = resolve_model_config("100m")
    assert (c["dim"], c["depth"]) == (512, 32)
    assert resolve_model_config("1g", dim="1024", expansion=3.0, ff_mult=1.5)["depth"] == 85
    assert resolve_model_config("1g", dim="2k", depth=20)["dim"] == 2048
    d = solve_for_dimension(1e9, 20)
    assert d % 64 == 0 and abs(calculate_model_size(dict(dim=d, depth=20, num_tokens=256, ff_mult=4, expansion=1.5)) / 1e9 - 1) < 0.1
    assert solve_for_depth(1e9, 2048) == 19 or solve_for_depth(1e9, 2048) == 20


def test_dataset_and_loader(tmp_path):
    path = tmp_path / "corpus.bin"
    raw = np.arange(10000, dtype=np.uint32).astype(np.uint8)
    raw.tofile(path)
    ds = ContinuousIIDDataset(str(path), chunk_size=64, context_chunks=4, seed=5, samples_per_epoch=8, verbose=False)
    x = ds[0]
    assert x.dtype == torch.long and x.shape == (256,)
    assert torch.equal((x[1:] - x[:-1]) % 256, torch.ones(255, dtype=torch.long))      # one contiguous span
    ds2 = ContinuousIIDDataset(str(path), chunk_size=64, context_chunks=4, seed=5, samples_per_epoch=8, verbose=False)
    assert torch.equal(ds2[0], x)                                                        # seeded
    z = ZipfBytes(4096, s=1.1, seed=1)
    b = z.sample_bytes()
    counts = np.bincount(b, minlength=256)
    assert counts[0] > counts[5] > counts[100] and b.dtype == np.uint8
    loader = SequenceLoader(ZipfBytes(128, seed=2), batch_size=3)
    batch = next(loader)
    assert batch.shape == (3, 128) and batch.dtype == torch.uint8
    loader.close()
    assert not loader.thread.is_alive()          # close() waits for the worker: nothing of it runs at process exit


def test_checkpoint_roundtrip_and_retention(tmp_path):
    torch.manual_seed(0)
    cfg = dict(num_tokens=256, dim=32, depth=1)
    m = minLM(**cfg)
    o = AdamWScheduleFree(m.parameters(), lr=1e-3); o.train()
    m(torch.randint(0, 256, (2, 9)), return_loss=True).backward(); o.step()
    losses = [3.0, 2.0, 2.5, 1.5, 4.0, 3.5]
    for i, l in enumerate(losses):
        assert save_checkpoint_atomic(build_checkpoint(i, m, o, l, cfg), str(tmp_path), i, 0, l)
        os.utime(tmp_path / checkpoint_name(0, i, l), (1000 + i, 1000 + i))
    (tmp_path / "checkpoint_rank_0000_step_000099_loss_9.0000.pt.tmp").write_bytes(b"x")
    os.utime(tmp_path / "checkpoint_rank_0000_step_000099_loss_9.0000.pt.tmp", (1, 1))
    mgr = CheckpointManager(str(tmp_path), keep_last_n=2, keep_elite_n=2)
    mgr.run_once()
    assert os.readlink(tmp_path / "latest.pt") == checkpoint_name(0, 5, 3.5)
    assert os.readlink(tmp_path / "best.pt") == checkpoint_name(0, 3, 1.5)
    assert os.readlink(tmp_path / "elite_02.pt") == checkpoint_name(0, 1, 2.0)
    left = sorted(p.name for p in tmp_path.glob("checkpoint_*.pt"))
    assert left == sorted(checkpoint_name(0, i, losses[i]) for i in (1, 3, 4, 5))
    assert not list(tmp_path.glob("*.tmp"))
    ck = load_checkpoint(str(tmp_path))
    assert set(ck) == {"step", "model_state_dict", "optimizer_state_dict", "ema_fitness", "model_config"}
    assert all(v.dtype == torch.float32 for v in ck["model_state_dict"].values())
    m2 = minLM(**ck["model_config"]); m2.load_state_dict(ck["model_state_dict"])
    o2 = AdamWScheduleFree(m2.parameters(), lr=1e-3); o2.load_state_dict(ck["optimizer_state_dict"])
    assert o2.param_groups[0]["k"] == 1
    # the pure policy: archived files survive
    es = [CkptEntry(f"/x/{i}", 0, i, l, 1000 + i) for i, l in enumerate(losses)]
    _, _, _, rem = plan_retention(es, 2, 2, archived={"/x/0"})
    assert sorted(e.step for e in rem) == [2]


def test_file_lock_times_out(tmp_path):
    lock = str(tmp_path / "l.lock")
    with file_lock(lock, timeout=1):
        with pytest.raises(TimeoutError):
            with file_lock(lock, timeout=0.05):
                pass
    with file_lock(lock, timeout=0.05):
        pass


def test_train_cli_runs_and_resumes(tmp_path):
    from gruboros_b200.runtime.train_main import main
    out = str(tmp_path / "run")
    base = ["--synthetic", "zipf:1.1", "--dim", "64", "--depth", "1", "--chunk_size", "32", "--context_chunks", "2",
            "--batch_size", "2", "--log_every", "2", "--final_checkpoint", "--save_every", "0"]
    argv = base + ["--train_steps", "6", "--output", out]
    assert main(argv) == 0
    rows = open(os.path.join(out, "metrics", "training_metrics_rank_000.tsv")).read().strip().splitlines()
    assert rows[0].split("\t")[:4] == ["rank", "step", "time_elapsed_s", "train_loss"] and len(rows) == 7
    assert json.load(open(os.path.join(out, "config.json")))["dim"] == 64
    assert os.path.islink(os.path.join(out, "latest.pt"))
    assert main(base + ["--train_steps", "8", "--resume", out]) == 0
    rows = open(os.path.join(out, "metrics", "training_metrics_rank_000.tsv")).read().strip().splitlines()
    assert [r.split("\t")[1] for r in rows[1:]] == ["6", "7"]


def test_data_parallel_modes_refuse_cpu():
    from gruboros_b200.runtime.train_main import require_cuda_for
    require_cuda_for("gossip", "cpu")
    require_cuda_for("none", "cpu")
    require_cuda_for("dp", "cuda:0")
    for mode in ("dp", "fsdp"):
        with pytest.raises(SystemExit):
            require_cuda_for(mode, "cpu")


def test_checkpoint_written_by_the_reference_stack_loads_generates_and_resumes(tmp_path):
    """A checkpoint as the reference's train.py writes it (its model's state_dict, its optimizer's state_dict, the
    same keys and file name) is picked up by load_model / generate and by --resume."""
    from gruboros_b200.runtime.generation import generate, load_model
    from gruboros_b200.runtime.train_main import main
    _, ref_l = REF
    cfg = dict(num_tokens=256, dim=64, depth=1, ff_mult=4, expansion=1.5)
    torch.manual_seed(3)
    ref = ref_l.minLM(**cfg)
    opt = ShimSF(ref.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4); opt.train()
    x = zipf_bytes(2, 33, seed=5)
    for _ in range(2):
        ref(x, return_loss=True).backward(); opt.step(); opt.zero_grad()
    out = tmp_path / "run"
    out.mkdir()
    name = checkpoint_name(0, 2, 5.5)
    torch.save({"step": 2, "model_state_dict": ref.state_dict(), "optimizer_state_dict": opt.state_dict(),
                "ema_fitness": 5.5, "model_config": cfg}, out / name)
    os.symlink(name, out / "latest.pt")
    model, got_cfg = load_model(str(out), device="cpu")
    assert got_cfg == cfg
    with torch.no_grad():
        assert torch.allclose(model(x[:, :16]), ref(x[:, :16]), atol=1e-5)
    toks = generate(model, x[:1, :8], 5, temperature=0.0, device="cpu", stream=False)
    assert toks.shape == (1, 5)
    argv = ["--synthetic", "zipf:1.1", "--chunk_size", "32", "--context_chunks", "2", "--batch_size", "2", "--log_every", "1",
            "--save_every", "0", "--train_steps", "4", "--resume", str(out)]
    assert main(argv) == 0
    rows = (out / "metrics" / "training_metrics_rank_000.tsv").read_text().strip().splitlines()
    assert [r.split("\t")[1] for r in rows[1:]] == ["2", "3"]           # continues from the saved step


def test_async_scalar_reader_orders_and_drains():
    """Losses pushed as device scalars come back oldest first; ready() never blocks, drain() returns the rest."""
    from gruboros_b200.runtime.metrics import AsyncScalarReader
    r = AsyncScalarReader(slots=4)
    for i in range(10):
        r.push(i, torch.tensor(float(i) * 0.5))
    got = r.ready() + r.drain()
    assert [t for t, _ in got] == list(range(10)) and [v for _, v in got] == [i * 0.5 for i in range(10)]
    assert len(r) == 0 and r.drain() == []
