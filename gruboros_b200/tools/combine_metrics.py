"""Merge the per-rank metrics TSVs of one or more runs into a single table.

The reference ships a combiner for an older file layout (combine_metrics.py:1-149 expects ``model_summary.txt`` and
``training_metrics.tsv``, which its current train.py no longer writes).  This one reads what training actually
produces: ``<run>/metrics/training_metrics_rank_NNN.tsv`` and ``<run>/config.json``; every row gets the run name
and the model configuration as extra columns, plus a population summary (best / mean / worst EMA loss per step).

    python -m gruboros_b200.tools.combine_metrics RUN_DIR... -o combined.tsv [--summary summary.tsv]
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import sys

import pandas as pd


def load_run(run_dir: str) -> pd.DataFrame:
    files = sorted(glob.glob(os.path.join(run_dir, "metrics", "training_metrics_rank_*.tsv")))
    if not files:
        return pd.DataFrame()
    df = pd.concat([pd.read_csv(f, sep="\t", na_values=["NA"]) for f in files], ignore_index=True)
    df.insert(0, "run", os.path.basename(os.path.normpath(run_dir)))
    cfg_path = os.path.join(run_dir, "config.json")
    if os.path.exists(cfg_path):
        with open(cfg_path) as f:
            cfg = json.load(f)
        for k in ("dim", "depth", "ff_mult", "expansion"):
            if k in cfg:
                df[k] = cfg[k]
    return df


def population_summary(df: pd.DataFrame) -> pd.DataFrame:
    g = df.groupby(["run", "step"])
    return g.agg(ranks=("rank", "nunique"), best_ema=("ema_loss", "min"), mean_ema=("ema_loss", "mean"),
                 worst_ema=("ema_loss", "max"), mean_loss=("train_loss", "mean"),
                 tokens_per_sec=("tokens_per_sec", "sum")).reset_index()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("runs", nargs="+")
    ap.add_argument("--output", "-o", required=True)
    ap.add_argument("--summary", default=None)
    a = ap.parse_args(argv)
    frames = [d for d in map(load_run, a.runs) if not d.empty]
    if not frames:
        print("no metrics found", file=sys.stderr)
        return 1
    df = pd.concat(frames, ignore_index=True)
    df.to_csv(a.output, sep="\t", index=False)
    if a.summary:
        population_summary(df).to_csv(a.summary, sep="\t", index=False)
    print(f"{len(df)} rows from {len(frames)} runs -> {a.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
