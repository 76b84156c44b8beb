"""minGRU layer (Feng et al., "Were RNNs All We Needed?", arXiv:2410.01201).

Module API and parameter names match the reference (mingru/minGRU.py:33-76):
``minGRU(dim, expansion_factor=1., proj_out=None)`` with ``to_hidden_and_gate``
(hidden rows first, gate rows second) and ``to_out``;
``forward(x, prev_hidden=None, return_next_prev_hidden=False)``.

This file is the framework-level (any device, autograd) implementation.  On a
B200 the training hot path does not go through it: ``minLM`` hands whole
forward/backward passes to ``gruboros_b200.models.engine``, which runs the
hand-written sm_100a kernels.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn


def g(x: torch.Tensor) -> torch.Tensor:
    """Positive candidate activation: x + 0.5 for x >= 0, sigmoid(x) below (reference mingru/minGRU.py:24-25)."""
    return torch.where(x >= 0, x + 0.5, torch.sigmoid(x))


def log_g(x: torch.Tensor) -> torch.Tensor:
    """log(g(x)) evaluated without leaving log space (reference mingru/minGRU.py:27-28)."""
    return torch.where(x >= 0, torch.log(F.relu(x) + 0.5), F.logsigmoid(x))


def heinsen_associative_scan_log(log_coeffs: torch.Tensor, log_values: torch.Tensor) -> torch.Tensor:
    """h_t = a_t h_{t-1} + b_t for all t at once, given log a and log b (Heinsen 2023; reference mingru/minGRU.py:16-20)."""
    prefix = torch.cumsum(log_coeffs, dim=1)
    return torch.exp(prefix + torch.logcumsumexp(log_values - prefix, dim=1))


def mingru_scan(hidden: torch.Tensor, gate: torch.Tensor, prev_hidden: torch.Tensor | None) -> torch.Tensor:
    """All hidden states of h_t = (1 - z_t) h_{t-1} + z_t g(u_t), z = sigmoid(gate), u = hidden pre-activation.

    ``prev_hidden`` is [B, 1, C] (strictly positive, as every state this recurrence produces is) or None.
    """
    log_keep = F.logsigmoid(-gate)                       # log(1 - z)
    log_in = F.logsigmoid(gate) + log_g(hidden)          # log(z g(u))
    if prev_hidden is not None:
        log_in = torch.cat((torch.log(prev_hidden), log_in), dim=1)
        log_keep = F.pad(log_keep, (0, 0, 1, 0))
    return heinsen_associative_scan_log(log_keep, log_in)[:, -hidden.shape[1]:]


class minGRU(nn.Module):
    def __init__(self, dim: int, expansion_factor: float = 1.0, proj_out: bool | None = None):
        super().__init__()
        dim_inner = int(dim * expansion_factor)
        if proj_out is None:
            proj_out = expansion_factor != 1.0
        self.dim_inner = dim_inner
        self.to_hidden_and_gate = nn.Linear(dim, dim_inner * 2, bias=False)
        self.to_out = nn.Linear(dim_inner, dim, bias=False) if proj_out else nn.Identity()

    def forward(self, x, prev_hidden=None, return_next_prev_hidden=False):
        hidden, gate = self.to_hidden_and_gate(x).chunk(2, dim=-1)
        if x.shape[1] == 1:
            # one recurrent step (decode)
            cand, z = g(hidden), torch.sigmoid(gate)
            out = torch.lerp(prev_hidden, cand, z) if prev_hidden is not None else cand * z
        else:
            out = mingru_scan(hidden, gate, prev_hidden)
        next_prev_hidden = out[:, -1:]
        out = self.to_out(out)
        return (out, next_prev_hidden) if return_next_prev_hidden else out
