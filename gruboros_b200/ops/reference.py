"""Plain-PyTorch restatements of every fused op, used on CPU and as the numerical
reference for the CUDA kernels.  They follow the reference model's math
(mingru/minGRU.py:16-28,43-76; mingru/minLM.py:17-23) but in linear space.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def g_act(x: torch.Tensor) -> torch.Tensor:
    """g(x) = x + 0.5 for x >= 0, sigmoid(x) otherwise (mingru/minGRU.py:24-25)."""
    return torch.where(x >= 0, x + 0.5, torch.sigmoid(x))


def scan_ref(k: torch.Tensor, u: torch.Tensor, h0: torch.Tensor | None = None):
    """h_t = (1 - sigmoid(k_t)) h_{t-1} + sigmoid(k_t) g(u_t) over dim 1.  Returns (h [B,T,C], h_T [B,C])."""
    z = torch.sigmoid(k)
    b = z * g_act(u)
    a = 1 - z
    h = torch.zeros_like(k[:, 0]) if h0 is None else h0
    out = []
    for t in range(k.shape[1]):
        h = a[:, t] * h + b[:, t]
        out.append(h)
    return torch.stack(out, 1), h


def scan_chunked(k: torch.Tensor, u: torch.Tensor, h0: torch.Tensor | None = None, chunk: int = 64):
    """Same recurrence evaluated chunk-parallel (closed form inside a chunk, carry across chunks).

    Inside a chunk: with A_t = prod_{s<=t} a_s, h_t = A_t (h_in + sum_{s<=t} b_s / A_s); the ratio is kept stable
    by working with log A (all a in (0,1)) as the reference's Heinsen form does, but only over `chunk` steps.
    """
    B, T, Cc = k.shape
    z = torch.sigmoid(k)
    log_a = F.logsigmoid(-k)
    b = z * g_act(u)
    h = torch.zeros(B, Cc, dtype=k.dtype, device=k.device) if h0 is None else h0
    outs = []
    for s in range(0, T, chunk):
        la = log_a[:, s:s + chunk].cumsum(1)                        # log A_t
        # h_t = exp(la_t) * h_in + sum_{s<=t} exp(la_t - la_s) b_s ; compute via logcumsumexp on log b - la
        logb = torch.log(b[:, s:s + chunk].clamp_min(1e-38))
        acc = torch.logcumsumexp(logb - la, dim=1)
        hc = torch.exp(la) * h.unsqueeze(1) + torch.exp(la + acc)
        outs.append(hc)
        h = hc[:, -1]
    return torch.cat(outs, 1), h


def rmsnorm_ref(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def sfadamw_ref(y, z, v, g, *, lr, beta1, beta2, bias2, eps, wd, ckp1):
    """One Schedule-Free AdamW parameter update (facebookresearch/schedule_free AdamWScheduleFree.step)."""
    v = beta2 * v + (1 - beta2) * g * g
    gh = g / ((v / bias2).sqrt() + eps) + wd * y
    y = torch.lerp(y, z, ckp1) + lr * (beta1 * (1 - ckp1) - 1) * gh
    z = z - lr * gh
    return y, z, v
