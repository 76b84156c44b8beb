"""TBPTT training loop core: chunks with hidden-state carry, gradient accumulation, optimizer step.

This is the loop of the reference's ``train.py:772-818`` as a reusable object: every call to
``step_chunk`` consumes one ``chunk_size``-byte chunk (inputs = first chunk_size-1 bytes, labels =
last chunk_size-1), carries the detached per-layer hidden state to the next chunk of the same
sequence, and steps the optimizer every ``grad_accum`` chunks.  On a B200 the chunk runs through
the fused engine (no autograd graph); elsewhere through the module path with autograd.
"""
from __future__ import annotations

import os

import torch


class Trainer:
    def __init__(self, model, optimizer, *, chunk_size: int, grad_accum: int = 1, parallel=None):
        """parallel: optional gradient synchroniser with ``pre_backward()``/``reduce_gradients()`` hooks
        (``gruboros_b200.parallel.dp.DataParallel``); None trains a single replica."""
        self.model, self.optimizer = model, optimizer
        self.chunk_size, self.grad_accum = chunk_size, max(1, grad_accum)
        self.parallel = parallel
        # no accumulation: update each layer while backward continues (GRB_FOLD=0 steps after backward instead)
        self.overlap_optimizer = os.environ.get("GRB_FOLD", "1") == "1"
        self.fold_parallel = os.environ.get("GRB_DP_FOLD", "0") == "1"   # same under data parallelism (per-layer rank flags)
        self.hidden = None
        self.chunks_done = 0
        self.optimizer_steps = 0
        self.last_folded = False          # whether the last optimizer step ran inside backward

    def reset_hidden(self) -> None:
        self.hidden = None

    def _fused(self, chunk) -> bool:
        return chunk.is_cuda and getattr(self.model, "_fusable", False) and getattr(self.model, "use_fused", False)

    def step_chunk(self, chunk: torch.Tensor):
        """One chunk: forward, backward (scaled by 1/grad_accum), optimizer step at accumulation boundaries.
        Returns the (unscaled) loss as a 0-dim tensor on the chunk's device - no host sync."""
        scale = 1.0 / self.grad_accum
        stepped = False
        if self._fused(chunk):
            engine = self.model.fused_engine()
            if self.parallel is not None:
                self.parallel.pre_backward(engine)
            engine.ensure_flat(chunk.device)
            stepper = None
            if self.overlap_optimizer and self.grad_accum == 1:
                if self.parallel is None:
                    if hasattr(self.optimizer, "overlappable") and self.optimizer.overlappable(engine.flat):
                        from ..models.engine import _LocalStepper
                        stepper = _LocalStepper(self.optimizer, engine.flat)
                elif self.fold_parallel and hasattr(self.parallel, "fold_stepper"):
                    stepper = self.parallel.fold_stepper()      # data parallel: per-layer flags + sharded update
            loss, hidden = engine.train_step(chunk, self.hidden, loss_scale=scale, stepper=stepper)
            stepped = stepper is not None
            self.last_folded = stepped
        else:
            loss, hidden = self.model(chunk, return_loss=True, return_prev_hiddens=True, prev_hiddens=self.hidden)
            (loss * scale).backward()
            loss = loss.detach()
        self.hidden = [h.detach() for h in hidden]
        self.chunks_done += 1
        if stepped:
            self.optimizer_steps += 1
        elif self.chunks_done % self.grad_accum == 0:
            if self.parallel is not None:
                self.parallel.reduce_gradients()
            self.optimizer.step()
            self.optimizer.zero_grad()
            if self.parallel is not None:
                self.parallel.post_step()
            self.optimizer_steps += 1
        return loss

    def train_sequence(self, tokens: torch.Tensor):
        """tokens: [B, n * chunk_size] bytes of contiguous text.  Runs the n chunks in order with carry and
        returns their losses (list of 0-dim tensors).  The hidden state is reset at the start."""
        self.reset_hidden()
        n = tokens.shape[1] // self.chunk_size
        return [self.step_chunk(tokens[:, i * self.chunk_size:(i + 1) * self.chunk_size]) for i in range(n)]
