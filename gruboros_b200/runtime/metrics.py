"""Per-rank training metrics in the reference's TSV schema (train.py:676-688, 742-764).

One row per chunk-step: rank, step, time_elapsed_s, train_loss, ema_loss, total_tokens_processed,
tokens_per_sec, learning_rate, initiated_mixes, received_mixes, won_mixes, lost_mixes, failed_mixes
[, skipped_due_to_lock].  Rows are buffered and flushed every `flush_every` steps (the reference reopens the
file on every step).  ``tokens_per_sec`` is the reference's cumulative wall-clock figure; the extra
``DeviceTimer`` measures the same quantity on the GPU with CUDA events, without a host sync per step.
"""
from __future__ import annotations

import os
import time

import torch

BASE_COLUMNS = ["rank", "step", "time_elapsed_s", "train_loss", "ema_loss", "total_tokens_processed",
                "tokens_per_sec", "learning_rate", "initiated_mixes", "received_mixes", "won_mixes", "lost_mixes",
                "failed_mixes"]


class MetricsLogger:
    def __init__(self, output_dir: str, global_rank: int, batch_size: int, chunk_size: int, with_lock_column=False,
                 flush_every: int = 20):
        self.dir = os.path.join(output_dir, "metrics")
        os.makedirs(self.dir, exist_ok=True)
        self.path = os.path.join(self.dir, f"training_metrics_rank_{global_rank:03d}.tsv")
        self.columns = BASE_COLUMNS + (["skipped_due_to_lock"] if with_lock_column else [])
        self.rank, self.batch_size, self.chunk_size = global_rank, batch_size, chunk_size
        self.flush_every = max(1, flush_every)
        self.start = time.time()
        self.total_tokens = 0
        self._rows = []
        with open(self.path, "w") as f:
            f.write("\t".join(self.columns) + "\n")

    def log(self, step: int, train_loss: float, ema_loss, lr: float, mix_status: dict):
        elapsed = time.time() - self.start
        self.total_tokens = (step + 1) * self.batch_size * self.chunk_size
        rate = self.total_tokens / elapsed if elapsed > 0 else 0.0
        row = [self.rank, step, f"{elapsed:.2f}", f"{train_loss:.6f}",
               f"{ema_loss:.6f}" if ema_loss is not None else "NA", self.total_tokens, f"{rate:.2f}", f"{lr:.8f}",
               mix_status.get("initiated_mixes", 0), mix_status.get("received_mixes", 0),
               mix_status.get("won_mixes", 0), mix_status.get("lost_mixes", 0), mix_status.get("failed_mixes", 0)]
        if len(self.columns) > len(BASE_COLUMNS):
            row.append(mix_status.get("skipped_due_to_lock", 0))
        self._rows.append("\t".join(str(v) for v in row))
        if len(self._rows) >= self.flush_every:
            self.flush()
        return rate

    def flush(self):
        if self._rows:
            with open(self.path, "a") as f:
                f.write("\n".join(self._rows) + "\n")
            self._rows.clear()

    def close(self):
        self.flush()


class DeviceTimer:
    """Throughput measured on the device: CUDA events around spans of steps, read back without stalling the
    stream (an event pair is only queried once it has completed)."""

    def __init__(self, bytes_per_step: int, enabled: bool = True):
        self.bytes_per_step = bytes_per_step
        self.enabled = enabled and torch.cuda.is_available()
        self._open = None
        self._pending = []
        self.total_ms = 0.0
        self.total_steps = 0

    def begin(self):
        if self.enabled and self._open is None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._open = (ev, 0)

    def step(self, n: int = 1, close_every: int = 50):
        if not self.enabled or self._open is None:
            return
        ev, count = self._open
        count += n
        if count >= close_every:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self._pending.append((ev, end, count))
            self._open = None
            self.begin()
        else:
            self._open = (ev, count)
        self._drain()

    def _drain(self):
        keep = []
        for a, b, n in self._pending:
            if b.query():
                self.total_ms += a.elapsed_time(b)
                self.total_steps += n
            else:
                keep.append((a, b, n))
        self._pending = keep

    def bytes_per_sec(self):
        self._drain()
        return self.bytes_per_step * self.total_steps / (self.total_ms / 1e3) if self.total_ms > 0 else None


class AsyncScalarReader:
    """Device scalars (losses) read back to the host without stalling the stream.

    ``push(tag, t)`` starts a non-blocking copy of the 0-dim tensor ``t`` into pinned host memory and records an
    event behind it; ``ready()`` returns the (tag, value) pairs whose copies have completed, oldest first, and
    ``drain()`` waits for the rest.  The reference reads ``loss.item()`` after every chunk (train.py:799), which
    idles the GPU while the host catches up; here the next chunk is already queued when a value arrives.  Works on
    CPU tensors too (values are then available immediately)."""

    def __init__(self, slots: int = 64):
        self._slots = slots
        self._host = None
        self._free = list(range(slots))
        self._inflight = []          # (tag, slot, event)

    def push(self, tag, t: torch.Tensor) -> None:
        if not t.is_cuda:
            self._inflight.append((tag, float(t), None))
            return
        if self._host is None:
            self._host = torch.empty(self._slots, dtype=torch.float32).pin_memory()
        if not self._free:
            self._wait_oldest()
        slot = self._free.pop()
        self._host[slot:slot + 1].copy_(t.detach().reshape(1).float(), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._inflight.append((tag, slot, ev))

    def _take(self, n: int):
        out = []
        for tag, slot, ev in self._inflight[:n]:
            if ev is None:
                out.append((tag, slot))
            else:
                out.append((tag, float(self._host[slot])))
                self._free.append(slot)
        del self._inflight[:n]
        return out

    def _wait_oldest(self):
        tag, slot, ev = self._inflight[0]
        if ev is not None:
            ev.synchronize()
        self._done_cache = getattr(self, "_done_cache", []) + self._take(1)

    def ready(self):
        """Completed reads, oldest first (never blocks)."""
        out = getattr(self, "_done_cache", [])
        self._done_cache = []
        n = 0
        for tag, slot, ev in self._inflight:
            if ev is not None and not ev.query():
                break
            n += 1
        return out + self._take(n)

    def drain(self):
        """All outstanding reads (blocks until the last copy has landed)."""
        if self._inflight and self._inflight[-1][2] is not None:
            self._inflight[-1][2].synchronize()
        out = getattr(self, "_done_cache", [])
        self._done_cache = []
        return out + self._take(len(self._inflight))

    def __len__(self):
        return len(self._inflight)
