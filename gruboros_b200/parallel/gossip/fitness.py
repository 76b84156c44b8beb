"""Fitness of a population member = exponential moving average of its training loss (lower is better).

Same definition as the reference (gossip/fitness_tracker.py:4-40): ema <- (1-decay) * loss + decay * ema,
first sample initialises it, `inf` before any sample; a clonally overwritten member inherits the winner's value.
"""
from __future__ import annotations

import math


class FitnessTracker:
    def __init__(self, decay_factor: float = 0.95):
        self.alpha = 1.0 - decay_factor
        self.ema_loss: float | None = None
        self.step_count = 0

    def update(self, loss_value: float) -> None:
        loss_value = float(loss_value)
        if self.ema_loss is None:
            self.ema_loss = loss_value
        else:
            self.ema_loss += self.alpha * (loss_value - self.ema_loss)
        self.step_count += 1

    def get_fitness(self) -> float:
        return self.ema_loss if self.ema_loss is not None else math.inf

    get_recent_loss = get_fitness

    def inherit_fitness(self, source_ema_loss: float) -> None:
        self.ema_loss = float(source_ema_loss)
