"""Training data: byte sequences for TBPTT.

``ContinuousIIDDataset`` is the reference's sampler (train.py:387-419): the corpus is one memory-mapped
uint8 file; every item is ONE contiguous span of ``chunk_size * context_chunks`` bytes starting at a position
drawn from ``random.Random(seed)``, so consecutive chunks of an item continue the same text.
``ZipfBytes`` is the synthetic stand-in (i.i.d. Zipf(s) bytes) used by benchmarks and tests.
``SequenceLoader`` batches items into pinned uint8 host buffers on a background thread and hands them to the
GPU with an asynchronous copy - the role torch's DataLoader worker process plays in the reference
(train.py:665-670) without the per-item int64 conversion and inter-process queue.
"""
from __future__ import annotations

import queue
import random
import threading

import numpy as np
import torch


class ContinuousIIDDataset(torch.utils.data.Dataset):
    def __init__(self, filepath, chunk_size, context_chunks=1, seed=42, samples_per_epoch=10000, batch_size=1,
                 global_rank=0, dtype=torch.long, verbose=True):
        super().__init__()
        self.filepath, self.chunk_size, self.context_chunks = filepath, chunk_size, context_chunks
        self.total_seq_len = chunk_size * context_chunks
        self.seed, self.samples_per_epoch, self.dtype = seed, samples_per_epoch, dtype
        self.mmap = np.memmap(filepath, dtype=np.uint8, mode="r")
        if len(self.mmap) < self.total_seq_len:
            raise ValueError(f"{filepath} has {len(self.mmap)} bytes, fewer than one sequence ({self.total_seq_len})")
        self.max_start = len(self.mmap) - self.total_seq_len
        self.rng = random.Random(seed)
        if verbose and global_rank == 0:
            print(f"ContinuousIIDDataset: {filepath} ({len(self.mmap):,} bytes); sequences of {self.total_seq_len} "
                  f"bytes = {context_chunks} chunks of {chunk_size}; {samples_per_epoch // max(1, batch_size)} batches per epoch")

    def __len__(self):
        return self.samples_per_epoch

    def sample_bytes(self) -> np.ndarray:
        pos = int(self.rng.random() * self.max_start)
        return self.mmap[pos:pos + self.total_seq_len]

    def __getitem__(self, idx):
        t = torch.from_numpy(np.array(self.sample_bytes(), dtype=np.uint8))
        return t if self.dtype == torch.uint8 else t.to(self.dtype)


class ZipfBytes:
    """Infinite source of i.i.d. bytes with P(rank r) ~ 1 / r^s over the 256 byte values (seeded)."""

    def __init__(self, total_seq_len: int, s: float = 1.1, seed: int = 42):
        self.total_seq_len = total_seq_len
        w = 1.0 / np.arange(1, 257, dtype=np.float64) ** s
        self.cdf = np.cumsum(w / w.sum())
        self.rng = np.random.default_rng(seed)

    def sample_bytes(self) -> np.ndarray:
        u = self.rng.random(self.total_seq_len)
        return np.minimum(np.searchsorted(self.cdf, u), 255).astype(np.uint8)


class SequenceLoader:
    """Iterator of [batch, total_seq_len] uint8 batches.  ``device=None`` yields pinned (if CUDA exists) host
    tensors; with a CUDA device the batch is copied asynchronously and the device tensor is yielded."""

    def __init__(self, source, batch_size: int, device=None, prefetch: int = 4):
        self.source, self.batch_size, self.device = source, batch_size, device
        self.q: queue.Queue = queue.Queue(maxsize=max(1, prefetch))
        self._stop = threading.Event()
        self._pin = torch.cuda.is_available()
        self.thread = threading.Thread(target=self._work, daemon=True, name="sequence-loader")
        self.thread.start()

    def _work(self):
        n = self.source.total_seq_len
        while not self._stop.is_set():
            buf = torch.empty(self.batch_size, n, dtype=torch.uint8, pin_memory=self._pin)
            arr = buf.numpy()
            for b in range(self.batch_size):
                arr[b] = self.source.sample_bytes()
            while not self._stop.is_set():
                try:
                    self.q.put(buf, timeout=0.2)
                    break
                except queue.Full:
                    continue

    def __iter__(self):
        return self

    def __next__(self):
        host = self.q.get()
        if self.device is None:
            return host
        return host.to(self.device, non_blocking=True)

    def close(self):
        """Stops the worker and waits for it: the thread allocates pinned host memory (a CUDA call), and a process
        that exits while such a call is in flight on another thread can abort in the runtime's teardown."""
        self._stop.set()
        if self.thread.is_alive() and threading.current_thread() is not self.thread:
            self.thread.join(timeout=5.0)
