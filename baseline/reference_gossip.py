"""Reference arm of the gossip configuration: the UNMODIFIED reference ``train.py`` (baseline/_ref/train.py), a
population of one full replica per rank exchanging weights over its own TCP protocol.

What this harness supplies, and nothing else: the missing ``schedulefree`` package (baseline/schedulefree_shim.py,
registered under that name), a ``hostfile-job*.txt`` for the reference's peer discovery
(gossip/network_utils.py:34-121), a synthetic Zipf(1.1) byte file for ``--data``, and the ``gossip/`` and
``metrics/`` directories that the reference expects its launch script to have created.  The reference trains in
fp32 with TF32 matmuls (train.py:294; it contains no autocast).  Afterwards rank 0 reads the reference's own logs:
the per-rank gossip TSVs (``WEIGHT_SEND_COMPLETE`` / ``WEIGHT_RECEIVE_COMPLETE`` events with their transfer times,
gossip/evolutionary_node.py:641-650,696-709) and the metrics TSV (tokens per second).

Launched by ``bench.py --impl reference --parallel gossip`` under torchrun, one rank per GPU.
"""
from __future__ import annotations

import csv
import glob
import json
import os
import runpy
import socket
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def _zipf_file(path: Path, nbytes: int) -> None:
    import torch
    g = torch.Generator().manual_seed(1234)
    w = 1.0 / torch.arange(1, 257, dtype=torch.float64) ** 1.1
    x = torch.multinomial(w / w.sum(), nbytes, replacement=True, generator=g).to(torch.uint8)
    path.write_bytes(x.numpy().tobytes())


def main(args, rank, world, local):
    if not (REF / "train.py").exists():
        return unavailable("baseline/_ref/train.py is missing: the reference was not installed")
    import bench
    cfg = bench.MODELS[args.model]
    run = Path(os.environ.get("GRB_REF_GOSSIP_DIR", f"/tmp/ref_gossip_{os.environ.get('MASTER_PORT', '0')}"))
    out = run / "out"
    if rank == 0:
        for d in (out / "gossip", out / "metrics", run / "tmp"):
            d.mkdir(parents=True, exist_ok=True)
        _zipf_file(run / "data.bin", 64 * 1024 * 1024)
        host = socket.gethostname().split(".")[0]
        try:
            socket.gethostbyname(host)
        except OSError:
            host = "localhost"      # then a rank also lists itself as a peer; a self-mix still runs the whole data path
        (run / "hostfile-job0.txt").write_text(f"{host} slots={world}\n")
        (run / "ready").write_text("1")
    else:
        for _ in range(600):
            if (run / "ready").exists():
                break
            time.sleep(0.1)
    os.chdir(run)                                   # the reference globs hostfile-job*.txt in the working directory
    os.environ["RANKS_PER_NODE"] = str(world)
    os.environ.pop("SLURM_JOB_NODELIST", None)
    os.environ["SLURM_JOB_ID"] = "0"
    sys.path.insert(0, str(REF))
    from baseline import schedulefree_shim
    sys.modules["schedulefree"] = schedulefree_shim
    steps = args.steps * (args.seq // args.chunk)    # the reference counts chunk-steps
    sys.argv = [str(REF / "train.py"), "--cuda", "--data", str(run / "data.bin"), "--output", str(out),
                "--train_steps", str(steps), "--dim", str(cfg["dim"]), "--depth", str(cfg["depth"]),
                "--expansion_factor", str(cfg["expansion"]), "--ff_mult", str(cfg["ff_mult"]),
                "--chunk_size", str(args.chunk), "--context_chunks", str(args.seq // args.chunk),
                "--batch_size", str(args.batch), "--lr", "1e-3", "--sf_beta2", "0.995", "--weight_decay", "1e-4",
                "--save_every", "1000000", "--gossip_mixing_rate", str(args.gossip_rate),
                "--gossip_merge_method", "recombination", "--gossip_recombination_alpha", "0.3",
                "--gossip_optimizer_recombination", "interpolate", "--gossip_temp_dir", str(run / "tmp")]
    t0 = time.time()
    try:
        runpy.run_path(str(REF / "train.py"), run_name="__main__")
    except SystemExit as e:
        if e.code not in (0, None):
            return unavailable(f"reference train.py exited with {e.code}")
    wall = time.time() - t0
    # transfers still in flight when training ends run in daemon threads: give them a bounded time to log
    deadline = time.time() + float(os.environ.get("GRB_REF_GOSSIP_DRAIN_S", "90"))
    while time.time() < deadline and list((run / "tmp").glob("gossip_payload_*")):
        time.sleep(1.0)
    (run / f"done_{rank}").write_text("1")
    if rank != 0:
        return 0
    for _ in range(1200):
        if all((run / f"done_{r}").exists() for r in range(world)):
            break
        time.sleep(0.1)
    events, kinds, fail_msgs = [], {}, []
    for f in glob.glob(str(out / "gossip" / "*.tsv")):
        with open(f) as fh:
            for row in csv.DictReader(fh, delimiter="\t"):
                kinds[row.get("event_type")] = kinds.get(row.get("event_type"), 0) + 1
                if "FAILED" in (row.get("event_type") or "") or "ERROR" in (row.get("event_type") or ""):
                    fail_msgs.append((row.get("message") or "")[:160])
                if row.get("event_type") in ("WEIGHT_SEND_COMPLETE", "WEIGHT_RECEIVE_COMPLETE"):
                    try:
                        events.append((row["event_type"], float(row["data_size_mb"]), float(row["transfer_time_ms"])))
                    except (KeyError, ValueError):
                        pass
    rates = []
    for f in glob.glob(str(out / "metrics" / "training_metrics_rank_*.tsv")):
        rows = list(csv.DictReader(open(f), delimiter="\t"))
        if rows:
            rates.append(float(rows[-1]["tokens_per_sec"]))
    recv = sorted(t for k, _, t in events if k == "WEIGHT_RECEIVE_COMPLETE")
    send = sorted(t for k, _, t in events if k == "WEIGHT_SEND_COMPLETE")
    res = {"metric": f"train bytes/sec (gossip population of {args.model.upper()} minLM replicas, wall clock of the reference's own log)",
           "value": sum(rates), "unit": "bytes/s", "n_gpus": world, "steps": args.steps, "warmup": 0, "impl": "reference",
           "higher_is_better": True, "dtype": "fp32 parameters, TF32 matmuls (the reference's train.py has no autocast)",
           "data": "synthetic Zipf(1.1) bytes, random-init weights",
           "config": dict(bench.shared_config(args, world), parallelism=f"gossip{world}"),
           "gossip": {"mixing_rate": args.gossip_rate, "transfers_received": len(recv), "transfers_sent": len(send),
                      "receive_ms_median": recv[len(recv) // 2] if recv else None,
                      "send_ms_median": send[len(send) // 2] if send else None,
                      "payload_mb": events[0][1] if events else None, "event_counts": kinds, "first_failures": fail_msgs[:3],
                      "note": "times are the reference's own WEIGHT_*_COMPLETE log fields (socket transfer only: the "
                              "torch.save / torch.load / host-device copies and the merge around it are not logged)"},
           "wall_s": wall}
    if not events:
        res["unavailable"] = "no weight transfer completed within the run (see gossip TSVs); throughput is still reported"
    print(json.dumps(res))
    return 0
