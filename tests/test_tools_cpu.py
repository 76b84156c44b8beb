"""Offline tools: parquet extraction, metrics merge, loss-curve fit."""
import numpy as np
import pandas as pd
import pytest

from gruboros_b200.tools import combine_metrics, extract_text, fit_loss_curve


def test_extract_text_writes_nul_delimited_utf8(tmp_path):
    pa = pytest.importorskip("pyarrow")
    import pyarrow.parquet as pq
    docs = ["hello world", "x", "héllo ünicode", None, "a longer document here"]
    pq.write_table(pa.table({"text": docs, "other": list(range(5))}), tmp_path / "a.parquet")
    out = tmp_path / "corpus.bin"
    assert extract_text.main([str(tmp_path), "-o", str(out), "--min-length", "2"]) == 0
    parts = out.read_bytes().split(b"\0")
    assert parts[-1] == b"" and [p.decode() for p in parts[:-1]] == ["hello world", "héllo ünicode", "a longer document here"]
    assert extract_text.main([str(tmp_path / "none")]) == 1


def make_run(root, name, ranks=2, steps=30):
    d = root / name / "metrics"
    d.mkdir(parents=True)
    (root / name / "config.json").write_text('{"dim": 64, "depth": 2, "ff_mult": 4.0, "expansion": 1.5}')
    cols = ["rank", "step", "time_elapsed_s", "train_loss", "ema_loss", "total_tokens_processed", "tokens_per_sec",
            "learning_rate", "initiated_mixes", "received_mixes", "won_mixes", "lost_mixes", "failed_mixes"]
    for r in range(ranks):
        t = np.arange(steps)
        loss = 2.0 * np.exp(-0.1 * t) + 3.0 + 0.01 * r
        df = pd.DataFrame({c: 0 for c in cols}, index=t)
        df["rank"], df["step"], df["train_loss"], df["ema_loss"], df["tokens_per_sec"] = r, t, loss, loss, 100.0
        df.to_csv(d / f"training_metrics_rank_{r:03d}.tsv", sep="\t", index=False)
    return root / name


def test_combine_metrics_and_fit(tmp_path, capsys):
    run = make_run(tmp_path, "runA")
    out, summ = tmp_path / "all.tsv", tmp_path / "sum.tsv"
    assert combine_metrics.main([str(run), "-o", str(out), "--summary", str(summ)]) == 0
    df = pd.read_csv(out, sep="\t")
    assert len(df) == 60 and set(df["run"]) == {"runA"} and df["dim"].iloc[0] == 64
    s = pd.read_csv(summ, sep="\t")
    assert len(s) == 30 and s["ranks"].iloc[0] == 2 and s["tokens_per_sec"].iloc[0] == 200.0
    assert abs(s["best_ema"].iloc[0] - 5.0) < 1e-9
    assert fit_loss_curve.main([str(run), "--column", "train_loss"]) == 0
    text = capsys.readouterr().out
    assert "exponential" in text
    fits = fit_loss_curve.fit(np.arange(30), 2.0 * np.exp(-0.1 * (np.arange(30) + 1.0)) + 3.0)
    a, b, c = fits["exponential"][0]
    assert abs(a - 2.0) < 1e-3 and abs(b - 0.1) < 1e-4 and abs(c - 3.0) < 1e-3


def test_read_last_line(tmp_path):
    from gruboros_b200.utils.files import read_last_line
    p = tmp_path / "m.tsv"
    assert read_last_line(str(p)) == ""
    p.write_text("step\tloss\n1\t5.5\n2\t5.1\n\n")
    assert read_last_line(str(p)) == "2\t5.1"
    p.write_text("x" * 100000 + "\nlast line")
    assert read_last_line(str(p)) == "last line"
