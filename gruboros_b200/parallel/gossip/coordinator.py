"""Population-wide fitness ranking through a shared directory.

Protocol of the reference (gossip/filesystem_coordinator.py:8-133): every rank periodically writes
`fitness/rank_NNNN.json` ({rank, fitness, timestamp}, atomic rename); rank 0 reads all files younger than
`max_age` seconds, sorts by fitness and writes `global_ranking.json` mapping rank -> percentile (0.0 best,
1.0 worst, 0.5 for a population of one); every rank re-reads that file when it changes.  The three actions are
plain methods (`publish`, `rank_population`, `refresh`) so they can be driven without the thread.
"""
from __future__ import annotations

import glob
import json
import math
import os
import threading
import time


class FilesystemCoordinator:
    def __init__(self, global_rank, world_size, output_dir, interval=10.0, publish_every=15.0, max_age=300.0,
                 initial_delay=5.0):
        self.global_rank, self.world_size = global_rank, world_size
        self.is_coordinator = global_rank == 0
        self.fitness_dir = os.path.join(output_dir, "fitness")
        self.fitness_file = os.path.join(self.fitness_dir, f"rank_{global_rank:04d}.json")
        self.ranking_file = os.path.join(output_dir, "global_ranking.json")
        os.makedirs(self.fitness_dir, exist_ok=True)
        self.interval, self.publish_every, self.max_age, self.initial_delay = interval, publish_every, max_age, initial_delay
        self.running = False
        self.thread = None
        self._wake = threading.Event()
        self.last_fitness_update = 0.0
        self.last_ranking_read = 0.0
        self.population_rankings: dict = {}
        self.get_fitness = lambda: None

    def set_fitness_provider(self, fn) -> None:
        self.get_fitness = fn

    def get_my_percentile(self):
        return self.population_rankings.get(str(self.global_rank))

    # -- actions
    @staticmethod
    def _atomic_json(path, obj):
        tmp = path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(obj, f)
        os.rename(tmp, path)

    def publish(self) -> bool:
        fitness = self.get_fitness()
        if fitness is None or math.isinf(fitness) or math.isnan(fitness):
            return False
        self._atomic_json(self.fitness_file, {"rank": self.global_rank, "fitness": fitness, "timestamp": time.time()})
        self.last_fitness_update = time.time()
        return True

    def rank_population(self) -> dict:
        now, entries = time.time(), []
        for path in glob.glob(os.path.join(self.fitness_dir, "rank_*.json")):
            try:
                with open(path) as f:
                    d = json.load(f)
                if now - d["timestamp"] < self.max_age:
                    entries.append((d["rank"], d["fitness"]))
            except (OSError, ValueError, KeyError):
                continue
        if not entries:
            return {}
        entries.sort(key=lambda e: e[1])
        n = len(entries)
        rankings = {rank: (i / (n - 1) if n > 1 else 0.5) for i, (rank, _) in enumerate(entries)}
        self._atomic_json(self.ranking_file, {"timestamp": now, "rankings": rankings})
        return rankings

    def refresh(self) -> None:
        try:
            mtime = os.path.getmtime(self.ranking_file)
            if mtime <= self.last_ranking_read:
                return
            with open(self.ranking_file) as f:
                d = json.load(f)
            if time.time() - d["timestamp"] < self.max_age:
                self.population_rankings = d["rankings"]
                self.last_ranking_read = mtime
        except (OSError, ValueError, KeyError):
            pass

    # -- thread
    def start(self):
        self.running = True
        self._wake.clear()
        self.thread = threading.Thread(target=self._run, daemon=True, name="fs-coordinator")
        self.thread.start()

    def stop(self):
        self.running = False
        self._wake.set()
        if self.thread is not None:
            self.thread.join(timeout=5)

    def _run(self):
        if self._wake.wait(self.initial_delay):
            return
        while self.running:
            try:
                if time.time() - self.last_fitness_update > self.publish_every:
                    self.publish()
                if self.is_coordinator:
                    self.rank_population()
                self.refresh()
            except Exception as exc:
                print(f"[Rank {self.global_rank}] FilesystemCoordinator error: {exc}", flush=True)
            if self._wake.wait(self.interval):
                break
