"""Byte-level minGRU language model.

Constructor, forward signature and ``state_dict`` layout match the reference
(mingru/minLM.py:43-206): ``layers.{i}`` is the ModuleList
``[conv|None, RMSNorm, minGRU, RMSNorm, FeedForward, Dropout|None]`` so checkpoint
keys are ``layers.{i}.1.weight``, ``layers.{i}.2.to_hidden_and_gate.weight`` ...

Two execution paths share the parameters:

* the module path below (plain PyTorch, any device, autograd) - used on CPU,
  for the optional conv / dropout variants and as the numerical oracle;
* the fused path (``gruboros_b200.models.engine.FusedEngine``): on a B200 a whole
  forward (and backward) pass runs as a fixed sequence of hand-written sm_100a
  kernels over preallocated buffers.  ``forward`` selects it automatically for
  CUDA inputs; ``loss.backward()`` keeps working through a custom autograd node.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from .mingru import minGRU


def FeedForward(dim: int, mult: float = 4) -> nn.Sequential:
    """Linear -> exact GELU -> Linear, both with bias (reference mingru/minLM.py:17-23)."""
    inner = int(dim * mult)
    return nn.Sequential(nn.Linear(dim, inner), nn.GELU(), nn.Linear(inner, dim))


class CausalDepthWiseConv1d(nn.Module):
    """Optional left-padded depthwise + pointwise convolution (reference mingru/minLM.py:27-39)."""

    def __init__(self, dim: int, kernel_size: int):
        super().__init__()
        self.kernel_size = kernel_size
        self.net = nn.Sequential(
            nn.Conv1d(dim, dim, kernel_size=kernel_size, groups=dim),
            nn.Conv1d(dim, dim, kernel_size=1),
        )

    def forward(self, x):
        y = F.pad(x.transpose(1, 2), (self.kernel_size - 1, 0))
        return self.net(y).transpose(1, 2)


class minLM(nn.Module):
    def __init__(self, *, num_tokens, dim, depth, ff_mult=4, expansion=1.5, conv_kernel_size=3, use_lstm=None,
                 enable_conv=False, dropout=0.0):
        super().__init__()
        self.num_tokens, self.dim, self.depth = num_tokens, dim, depth
        self.ff_mult, self.expansion = ff_mult, expansion
        self.token_emb = nn.Embedding(num_tokens, dim)
        self.layers = nn.ModuleList([
            nn.ModuleList([
                CausalDepthWiseConv1d(dim, conv_kernel_size) if enable_conv else None,
                nn.RMSNorm(dim),
                minGRU(dim, expansion_factor=expansion),
                nn.RMSNorm(dim),
                FeedForward(dim, mult=ff_mult),
                nn.Dropout(dropout) if dropout > 0.0 else None,
            ]) for _ in range(depth)
        ])
        self.norm = nn.RMSNorm(dim)
        self.to_logits = nn.Linear(dim, num_tokens, bias=False)
        self.can_cache = not enable_conv
        self._fusable = (not enable_conv) and not (dropout > 0.0) and expansion != 1.0
        self._engine = None
        self.use_fused = True            # set False to force the module path on CUDA
        self._initialize_weights()

    # ------------------------------------------------------------------ init
    def _initialize_weights(self):
        """Every residual branch starts as the identity: output projections are zero, input-facing
        matrices are N(0, (0.02/sqrt(dim))^2) (reference mingru/minLM.py:157-206)."""
        std = 0.02 / math.sqrt(self.dim)
        nn.init.normal_(self.token_emb.weight, mean=0.0, std=std)
        nn.init.normal_(self.to_logits.weight, mean=0.0, std=std)
        for layer in self.layers:
            rnn, ff = layer[2], layer[4]
            nn.init.normal_(rnn.to_hidden_and_gate.weight, mean=0.0, std=std)
            if isinstance(rnn.to_out, nn.Linear):
                nn.init.zeros_(rnn.to_out.weight)
            nn.init.normal_(ff[0].weight, mean=0.0, std=std)
            nn.init.zeros_(ff[2].weight)
            nn.init.zeros_(ff[2].bias)

    # --------------------------------------------------------------- engine
    def fused_engine(self):
        """The sm_100a execution engine bound to this module's parameters (created on first use)."""
        if self._engine is None:
            from .engine import FusedEngine
            self._engine = FusedEngine(self)
        return self._engine

    def _use_fused(self, x: torch.Tensor) -> bool:
        return self.use_fused and self._fusable and x.is_cuda

    # -------------------------------------------------------------- forward
    def forward(self, x, return_loss=False, return_prev_hiddens=False, prev_hiddens=None):
        if self._use_fused(x):
            return self.fused_engine().module_forward(x, return_loss, return_prev_hiddens, prev_hiddens)
        return self._module_forward(x, return_loss, return_prev_hiddens, prev_hiddens)

    def _module_forward(self, x, return_loss=False, return_prev_hiddens=False, prev_hiddens=None):
        if return_loss:
            x, labels = x[:, :-1], x[:, 1:]
        x = self.token_emb(x.long())
        if prev_hiddens is not None and not return_loss:
            x = x[:, -1:]                      # decode: only the newest token is fed
        carried = iter(prev_hiddens if prev_hiddens is not None else [])
        next_prev_hiddens = []
        for conv, norm, rnn, ff_norm, ff, dropout in self.layers:
            if conv is not None:
                assert prev_hiddens is None, "caching not supported for conv version"
                x = conv(x) + x
            out, nxt = rnn(norm(x), next(carried, None), return_next_prev_hidden=True)
            x = out + x
            next_prev_hiddens.append(nxt)
            x = ff(ff_norm(x)) + x
            if dropout is not None:
                x = dropout(x)
        logits = self.to_logits(self.norm(x))
        if not return_loss:
            return (logits, next_prev_hiddens) if return_prev_hiddens else logits
        loss = F.cross_entropy(logits.transpose(1, 2), labels.long())
        return (loss, next_prev_hiddens) if return_prev_hiddens else loss
