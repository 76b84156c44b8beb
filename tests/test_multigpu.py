"""Multi-GPU tests: each spawns `torchrun` with one rank per GPU and checks the worker's verdict.
Skipped on machines with fewer than two GPUs (the multi-rank logic is then covered by the single-GPU
emulation in test_dp_gpu.py and by the CPU tests of the gossip protocol)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def run_workers(script, nproc, port, extra_env=None, timeout=600):
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / script)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=str(ROOT))
    return res


NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0


def ranks(n):
    """Parametrisation over rank counts: 2, 4 and 8, each skipped unless that many GPUs are present."""
    return pytest.param(n, marks=pytest.mark.skipif(NGPU < n, reason=f"needs {n} GPUs"))


def verdict(res):
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    return json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])


@pytest.mark.parametrize("nproc", [ranks(2), ranks(4), ranks(8)])
@pytest.mark.parametrize("fold,interleave", [("1", "1"), ("0", "1"), ("1", "0")])
def test_data_parallel_matches_single_replica(nproc, fold, interleave):
    """fold=1: sharded optimizer folded into backward behind per-layer cross-rank flags; fold=0: after backward.
    interleave=1: ownership dealt round-robin in 256 KB chunks (default); 0: one contiguous shard per rank."""
    res = run_workers("mp_dp_worker.py", nproc, 29611 + int(fold) + 2 * int(interleave) + 10 * nproc,
                      extra_env={"DP_FOLD": fold, "DP_INTERLEAVE": interleave, "NCCL_NVLS_ENABLE": "0"})
    out = verdict(res)
    assert out["ok"] and out["folded"] == (fold == "1") and out["steps"] == 3, out
    assert out["interleave"] == (interleave == "1"), out


@pytest.mark.parametrize("nproc", [ranks(2), ranks(4), ranks(8)])
def test_data_parallel_with_multicast_weight_mirror(nproc):
    """GRB_NVLS path: the bf16 mirrors are bound to one NVSwitch multicast object and owners publish new weights with
    one multimem store.  Skips itself (inside the worker) where the driver reports no multicast support."""
    res = run_workers("mp_dp_worker.py", nproc, 29911 + nproc, extra_env={"DP_FOLD": "0", "DP_NVLS": "1", "NCCL_NVLS_ENABLE": "0"})
    out = verdict(res)
    assert out["ok"], out
    if "skipped" not in out:
        assert out["nvls"] and out["mirrors_equal"], out


@pytest.mark.parametrize("nproc", [ranks(2), ranks(4), ranks(8)])
def test_fsdp_matches_single_replica(nproc):
    res = run_workers("mp_fsdp_worker.py", nproc, 29721 + nproc)
    out = verdict(res)
    assert out["ok"] and out["gathered_MB"] > 0, out


@pytest.mark.parametrize("nproc", [ranks(2), ranks(4), ranks(8)])
def test_gossip_nvlink(nproc, tmp_path):
    res = run_workers("mp_gossip_worker.py", nproc, 29831 + nproc,
                      extra_env={"GOSSIP_TEST_DIR": str(tmp_path), "NCCL_NVLS_ENABLE": "0"})
    out = verdict(res)
    assert out["ok"], out


@pytest.mark.parametrize("mode", ["dp", "fsdp"])
@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
def test_train_cli_parallel_modes_save_and_resume(mode, tmp_path):
    """train.py --parallel dp / fsdp on two ranks: trains, writes a reference-layout checkpoint gathered from the
    shards, and a second launch resumes from it (every rank takes its share of parameters and optimizer state)."""
    out = tmp_path / "run"
    base = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1"]
    args = ["train.py", "--synthetic", "zipf:1.1", "--dim", "256", "--depth", "2", "--chunk_size", "129", "--context_chunks", "2",
            "--batch_size", "2", "--log_every", "2", "--save_every", "0", "--parallel", mode, "--final_checkpoint", "--progress", "off"]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r1 = subprocess.run(base + ["--master-port", "29951" if mode == "dp" else "29953"] + args + ["--train_steps", "4", "--output", str(out)],
                        capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r1.returncode == 0, r1.stdout[-2000:] + r1.stderr[-3000:]
    ck = torch.load(out / "latest.pt", map_location="cpu", weights_only=False)
    sd = ck["model_state_dict"]
    assert sd["layers.0.2.to_hidden_and_gate.weight"].shape == (768, 256) and ck["step"] == 4
    assert set(ck["optimizer_state_dict"]["state"][1]) == {"z", "exp_avg_sq"}
    assert all(torch.isfinite(v).all() for v in sd.values())
    r2 = subprocess.run(base + ["--master-port", "29952" if mode == "dp" else "29954"] + args + ["--train_steps", "8", "--resume", str(out)],
                        capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r2.returncode == 0, r2.stdout[-2000:] + r2.stderr[-3000:]
    rows = (out / "metrics" / "training_metrics_rank_000.tsv").read_text().strip().splitlines()
    assert [r.split("\t")[1] for r in rows[1:]] == ["4", "5", "6", "7"]
    losses = [float(r.split("\t")[3]) for r in rows[1:]]
    assert all(l == l and l < 6.0 for l in losses), losses
