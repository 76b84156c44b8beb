"""Fit the training loss curve of a run with an exponential and a power law and extrapolate.

Plays the role of the reference's plot_train.R (exp / power-law fits of the loss curve), but works on the columns
training actually writes (``train_loss`` / ``ema_loss`` per step; the R script needs a ``val_loss`` column that
train.py never produced) and prints a table instead of drawing:

    loss(t) = a * exp(-b t) + c          loss(t) = a * t^(-b) + c

    python -m gruboros_b200.tools.fit_loss_curve RUN_DIR_OR_TSV [--column ema_loss] [--horizon 2.0]
"""
from __future__ import annotations

import argparse
import glob
import os
import sys

import numpy as np
import pandas as pd
from scipy.optimize import curve_fit


def exp_law(t, a, b, c):
    return a * np.exp(-b * t) + c


def power_law(t, a, b, c):
    return a * np.power(t, -b) + c


def fit(steps: np.ndarray, loss: np.ndarray):
    """Returns {name: (params, rmse)} for the fits that converged."""
    t = steps.astype(np.float64) + 1.0
    out = {}
    span = max(loss.max() - loss.min(), 1e-6)
    for name, fn, p0 in (("exponential", exp_law, (span, 1.0 / max(t.max(), 1.0), loss.min())),
                         ("power_law", power_law, (span, 0.5, loss.min() * 0.9))):
        try:
            p, _ = curve_fit(fn, t, loss, p0=p0, maxfev=20000)
            out[name] = (p, float(np.sqrt(np.mean((fn(t, *p) - loss) ** 2))))
        except (RuntimeError, ValueError):
            continue
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("path")
    ap.add_argument("--column", default="ema_loss")
    ap.add_argument("--horizon", type=float, default=2.0, help="extrapolate to this multiple of the last step")
    a = ap.parse_args(argv)
    files = [a.path] if os.path.isfile(a.path) else sorted(glob.glob(os.path.join(a.path, "metrics", "*.tsv")))
    if not files:
        print("no metrics file found", file=sys.stderr)
        return 1
    df = pd.concat([pd.read_csv(f, sep="\t", na_values=["NA"]) for f in files])
    curve = df.groupby("step")[a.column].mean().dropna()
    fits = fit(curve.index.to_numpy(), curve.to_numpy())
    target = (curve.index.max() + 1) * a.horizon
    print(f"{len(curve)} steps, last {a.column} = {curve.iloc[-1]:.4f}")
    for name, (p, rmse) in fits.items():
        fn = exp_law if name == "exponential" else power_law
        print(f"{name:12s} a={p[0]:.4g} b={p[1]:.4g} c={p[2]:.4g}  rmse={rmse:.4g}  "
              f"predicted at step {int(target)}: {fn(target, *p):.4f}  asymptote: {p[2]:.4f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
