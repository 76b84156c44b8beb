"""Checkpoint files and their retention.

File format and naming are the reference's (train.py:241-258, 703-714): ``torch.save`` of
``{'step', 'model_state_dict', 'optimizer_state_dict', 'ema_fitness', 'model_config'}`` to
``checkpoint_rank_{rank:04d}_step_{step:06d}_loss_{ema:.4f}.pt`` through a ``.tmp`` file and an atomic rename.
Tensors are written as fp32 under the reference's parameter names whatever the internal storage is (flat
buffers, bf16 mirrors, sharded optimizer state), so checkpoints move freely between the two code bases.

``CheckpointManager`` is the rank-0 background thread of train.py:30-239: it keeps ``latest.pt`` / ``best.pt`` /
``elite_NN.pt`` / ``archive_NNN.pt`` symlinks current, prunes files that are neither recent, elite nor archived,
and removes stale ``.tmp`` files.  The policy itself is the pure function ``plan_retention``.
"""
from __future__ import annotations

import atexit
import contextlib
import glob
import os
import random
import re
import threading
import time
from dataclasses import dataclass

import torch

CKPT_RE = re.compile(r"checkpoint_rank_(\d+)_step_(\d+)_loss_([\d.inf]+)\.pt$")


def checkpoint_name(rank: int, step: int, ema_fitness: float) -> str:
    return f"checkpoint_rank_{rank:04d}_step_{step:06d}_loss_{ema_fitness:.4f}.pt"


def build_checkpoint(step, model, optimizer, ema_fitness, model_config) -> dict:
    """Reference-layout checkpoint dict; tensors are detached fp32 clones on the CPU."""
    model_sd = {k: v.detach().to("cpu", torch.float32).clone() if v.is_floating_point() else v.detach().cpu().clone()
                for k, v in model.state_dict().items()}
    opt_sd = optimizer.state_dict()
    opt_sd = {"state": {i: {k: (t.detach().cpu().clone() if torch.is_tensor(t) else t) for k, t in st.items()}
                        for i, st in opt_sd["state"].items()},
              "param_groups": opt_sd["param_groups"]}
    return {"step": step, "model_state_dict": model_sd, "optimizer_state_dict": opt_sd,
            "ema_fitness": ema_fitness, "model_config": model_config}


def save_checkpoint_atomic(checkpoint_data: dict, checkpoint_dir: str, step: int, global_rank: int, ema_fitness: float) -> bool:
    final = os.path.join(checkpoint_dir, checkpoint_name(global_rank, step, ema_fitness))
    tmp = final + ".tmp"
    try:
        torch.save(checkpoint_data, tmp)
        os.rename(tmp, final)
        return True
    except Exception as exc:  # a failed save must never stop training
        with contextlib.suppress(OSError):
            if os.path.exists(tmp):
                os.remove(tmp)
        print(f"Rank {global_rank}: checkpoint save failed: {exc}")
        return False


def load_checkpoint(path: str, map_location="cpu") -> dict:
    """Load a checkpoint file or, given a directory, its ``latest.pt``."""
    if os.path.isdir(path):
        path = os.path.join(path, "latest.pt")
    return torch.load(path, map_location=map_location, weights_only=False)


@dataclass(frozen=True)
class CkptEntry:
    path: str
    rank: int
    step: int
    loss: float
    mtime: float


def parse_checkpoint(path: str):
    m = CKPT_RE.search(os.path.basename(path))
    if m is None:
        return None
    try:
        return CkptEntry(path, int(m.group(1)), int(m.group(2)), float(m.group(3)), os.path.getmtime(path))
    except (FileNotFoundError, ValueError):
        return None


def plan_retention(entries, keep_last_n: int, keep_elite_n: int, archived: set = frozenset()):
    """Pure retention policy.  Returns (latest, best, elites, removable): newest by mtime, lowest loss, the
    `keep_elite_n` lowest-loss entries in order, and the entries that are neither elite, among the
    `keep_last_n` most recent, nor already archived."""
    if not entries:
        return None, None, [], []
    latest = max(entries, key=lambda e: e.mtime)
    by_loss = sorted(entries, key=lambda e: e.loss)
    elites = by_loss[:keep_elite_n]
    recent = sorted(entries, key=lambda e: e.mtime, reverse=True)[:keep_last_n]
    keep = {os.path.realpath(e.path) for e in elites} | {os.path.realpath(e.path) for e in recent} | set(archived)
    removable = [e for e in entries if os.path.realpath(e.path) not in keep]
    if len(entries) <= keep_last_n and len(entries) <= keep_elite_n:
        removable = []
    return latest, by_loss[0], elites, removable


class CheckpointManager:
    def __init__(self, checkpoint_dir, check_interval=10, keep_last_n=5, keep_elite_n=10, global_rank=0, archive_rate=0.0):
        self.checkpoint_dir, self.check_interval = checkpoint_dir, check_interval
        self.keep_last_n, self.keep_elite_n = keep_last_n, keep_elite_n
        self.global_rank, self.archive_rate = global_rank, archive_rate
        self.archive_counter = 0
        self.active = global_rank == 0
        self.running = False
        self.thread = None
        self._stop = threading.Event()
        self._rng = random.Random(0xC0FFEE)

    # ---- thread control
    def start(self):
        if not self.active or self.running:
            return
        self.running = True
        self._stop.clear()
        self.thread = threading.Thread(target=self._loop, daemon=True, name="checkpoint-manager")
        self.thread.start()
        atexit.register(self.stop)

    def stop(self):
        if not self.active or not self.running:
            return
        self.running = False
        self._stop.set()
        if self.thread is not None and self.thread.is_alive():
            self.thread.join(timeout=5)

    def _loop(self):
        while self.running and not self._stop.is_set():
            try:
                self.run_once()
            except Exception as exc:
                print(f"Rank 0: checkpoint manager error: {exc}")
            if self._stop.wait(self.check_interval):
                break

    # ---- one maintenance cycle (also callable synchronously, e.g. from tests or at exit)
    def run_once(self):
        paths = glob.glob(os.path.join(self.checkpoint_dir, "checkpoint_rank_*_step_*_loss_*.pt"))
        entries = [e for e in map(parse_checkpoint, paths) if e is not None]
        if entries:
            archived = {os.path.realpath(s) for s in glob.glob(os.path.join(self.checkpoint_dir, "archive_*.pt"))
                        if os.path.islink(s)}
            latest, best, elites, removable = plan_retention(entries, self.keep_last_n, self.keep_elite_n, archived)
            self._symlink(latest.path, "latest.pt")
            self._symlink(best.path, "best.pt")
            for i, e in enumerate(elites, 1):
                self._symlink(e.path, f"elite_{i:02d}.pt")
            for i in range(len(elites) + 1, self.keep_elite_n + 20):
                link = os.path.join(self.checkpoint_dir, f"elite_{i:02d}.pt")
                if os.path.islink(link):
                    os.remove(link)
            for e in removable:
                try:
                    if self.archive_rate > 0 and self._rng.random() < self.archive_rate:
                        self.archive_counter += 1
                        self._symlink(e.path, f"archive_{self.archive_counter:03d}.pt")
                    else:
                        os.remove(e.path)
                except OSError:
                    continue
        self._remove_stale_tmp()

    def _symlink(self, target_path: str, link_name: str):
        target = os.path.basename(target_path)
        link = os.path.join(self.checkpoint_dir, link_name)
        if os.path.islink(link) and os.readlink(link) == target:
            return
        tmp = link + ".tmp"
        if os.path.lexists(tmp):
            os.remove(tmp)
        os.symlink(target, tmp)
        os.rename(tmp, link)

    def _remove_stale_tmp(self, max_age_s: float = 600.0):
        cutoff = time.time() - max_age_s
        for tmp in glob.glob(os.path.join(self.checkpoint_dir, "checkpoint_*.pt.tmp")):
            try:
                if os.path.getmtime(tmp) < cutoff:
                    os.remove(tmp)
            except OSError:
                continue
