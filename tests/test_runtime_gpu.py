"""train.py's driver on a GPU: the fused path through the command line, resume, and what happens when a bounded
device-side wait reports a timeout (a stalled or departed peer): training stops and no checkpoint is written."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

BASE = ["--synthetic", "zipf:1.1", "--dim", "128", "--depth", "2", "--chunk_size", "65", "--context_chunks", "2",
        "--batch_size", "2", "--log_every", "2", "--save_every", "0", "--cuda"]


def test_train_cli_fused_runs_and_resumes_on_gpu(tmp_path):
    from gruboros_b200.ops import kernels as K
    from gruboros_b200.runtime.train_main import main
    out = str(tmp_path / "run")
    n0 = K.LAUNCHES
    assert main(BASE + ["--train_steps", "4", "--output", out, "--final_checkpoint"]) == 0
    assert K.LAUNCHES - n0 > 100, "the fused kernels did not run"
    assert os.path.islink(os.path.join(out, "latest.pt"))
    # resume: the optimizer state is loaded before the first fused step builds the flat buffers
    assert main(BASE + ["--train_steps", "8", "--resume", out, "--final_checkpoint"]) == 0
    rows = open(os.path.join(out, "metrics", "training_metrics_rank_000.tsv")).read().strip().splitlines()
    assert [r.split("\t")[1] for r in rows[1:]] == ["4", "5", "6", "7"]
    losses = [float(r.split("\t")[3]) for r in rows[1:]]
    assert all(l == l and l < 6.0 for l in losses)


def test_device_timeout_status_stops_training_and_blocks_checkpoints(tmp_path, monkeypatch):
    """A wait that ran out leaves a status word; the driver reads it where it synchronises anyway (loss read-back,
    checkpoint) and refuses to go on.  The word is set by hand here - no kernel is made to wait."""
    from gruboros_b200.ops import _lib as L
    from gruboros_b200.runtime import train_main
    from gruboros_b200.runtime.trainer import Trainer
    real = Trainer.step_chunk
    calls = {"n": 0}

    def step_chunk(self, chunk):
        calls["n"] += 1
        loss = real(self, chunk)
        if calls["n"] == 3:
            L.err_flag(chunk.device).fill_(21)        # what a bounded wait writes when it gives up
        return loss

    monkeypatch.setattr(Trainer, "step_chunk", step_chunk)
    out = str(tmp_path / "run")
    with pytest.raises(RuntimeError, match="timed out"):
        train_main.main(BASE + ["--train_steps", "12", "--output", out, "--final_checkpoint"])
    assert calls["n"] <= 4
    assert not [f for f in os.listdir(out) if f.endswith(".pt")], "a checkpoint was written after the timeout"
    assert int(L.err_flag(torch.device("cuda", torch.cuda.current_device())).item()) == 0    # reported once, then cleared


def test_async_scalar_reader_on_device():
    """Pinned-host read-back of device scalars without a stream stall: more pushes than slots, values and order kept."""
    from gruboros_b200.runtime.metrics import AsyncScalarReader
    r = AsyncScalarReader(slots=4)
    vals = torch.arange(12, device="cuda", dtype=torch.float32) * 0.25
    got = []
    for i in range(12):
        r.push(i, vals[i])
        got += r.ready()
    got += r.drain()
    assert [t for t, _ in got] == list(range(12))
    assert [v for _, v in got] == [i * 0.25 for i in range(12)]
