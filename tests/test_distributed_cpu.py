"""Multi-process training on CPU: two `train.py` ranks (gloo rendezvous) forming a gossip population over the TCP
transport on localhost.  Checks that both ranks train, tournaments happen, weights flow and metrics / event logs
are written in the reference's formats."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.timeout(300)
def test_two_rank_population_trains_and_mixes(tmp_path):
    out = tmp_path / "run"
    port, gossip_base = free_port(), free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", LOCAL_WORLD_SIZE="2",
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), GOSSIP_BASE_PORT=str(gossip_base),
                   GOSSIP_STARTUP_DELAY="0.2", CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2",
                   PYTHONPATH=str(ROOT))
        cmd = [sys.executable, str(ROOT / "train.py"), "--synthetic", "zipf:1.1", "--dim", "64", "--depth", "1",
               "--chunk_size", "32", "--context_chunks", "2", "--batch_size", "2", "--train_steps", "150",
               "--output", str(out), "--log_every", "5", "--save_every", "0", "--gossip_mixing_rate", "0.3",
               "--gossip_merge_method", "recombination", "--gossip_recombination_alpha", "0.3",
               "--gossip_temp_dir", str(tmp_path / "gtmp"), "--filesystem-coordinator"]
        procs.append(subprocess.Popen(cmd, env=env, cwd=str(tmp_path), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=280)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(o[-1500:] for o in outs)
    for rank in range(2):
        rows = (out / "metrics" / f"training_metrics_rank_{rank:03d}.tsv").read_text().strip().splitlines()
        assert len(rows) == 151
        last = dict(zip(rows[0].split("\t"), rows[-1].split("\t")))
        assert float(last["train_loss"]) < 5.3
    logs = list((out / "gossip").glob("*.tsv"))
    assert len(logs) == 2
    text = "".join(l.read_text() for l in logs)
    assert "MIX_ATTEMPT_START" in text and "SERVER_STARTED" in text
    won = sum(int(dict(zip(r[0].split("\t"), r[-1].split("\t")))["won_mixes"]) for r in
              [(out / "metrics" / f"training_metrics_rank_{k:03d}.tsv").read_text().strip().splitlines() for k in range(2)])
    assert won >= 1, text[-2000:]
    assert "WEIGHT_RECEIVE_COMPLETE" in text and "WEIGHT_SEND_COMPLETE" in text
