"""Flat parameter storage.

All parameters of a model live in ONE fp32 buffer (and their gradients in one more, plus a
bf16 mirror for the tensor cores); ``nn.Parameter.data`` / ``.grad`` become views into it.
That gives the fused optimizer, the data-parallel reduce-scatter and the gossip merge a single
contiguous range to stream over, while ``state_dict()`` keeps the per-tensor reference layout.
"""
from __future__ import annotations

import weakref

import torch
from torch import nn

ALIGN = 64  # elements: 256 B in fp32, 128 B in bf16 (TMA wants 16-byte aligned bases)

_REGISTRY: "weakref.WeakValueDictionary[int, FlatParams]" = weakref.WeakValueDictionary()


def lookup(param: torch.Tensor):
    """The FlatParams that owns ``param`` (None if it is an ordinary tensor)."""
    ref = getattr(param, "_grb_flat", None)
    return ref() if ref is not None else None


class FlatParams:
    def __init__(self, module: nn.Module, device=None, pad_to: int = 1, allocator=None, select=None,
                 layout_only: bool = False, mirror: bool = True):
        """allocator(name, numel, dtype) -> zero-filled tensor; lets the buffers come from a symmetric (peer-mapped) heap.
        select(name, param) -> bool restricts the flat space to a subset of the module's parameters.
        layout_only: compute names / offsets / numel but allocate nothing and leave the parameters alone (fully
        sharded training keeps only each rank's share of such a space).  mirror=False: no bf16 mirror."""
        params = [(n, p) for n, p in module.named_parameters() if select is None or select(n, p)]
        if not params:
            raise ValueError("module has no parameters")
        device = torch.device(device) if device is not None else params[0][1].device
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.numel = (off + pad_to * ALIGN - 1) // (pad_to * ALIGN) * (pad_to * ALIGN)
        self.device = device
        self.allocator = allocator      # None: ordinary torch allocations
        self.shapes = [tuple(p.shape) for p in self.params]
        if layout_only:
            self.data = self.grad = self.w16 = None
            self.w16_version = -1
            return
        if allocator is None:
            allocator = lambda name, numel, dtype: torch.zeros(numel, dtype=dtype, device=device)
        self.data = allocator("data", self.numel, torch.float32)
        self.grad = allocator("grad", self.numel, torch.float32)
        self.w16 = allocator("w16", self.numel, torch.bfloat16) if device.type == "cuda" and mirror else None
        self.w16_version = -1
        for p, o in zip(self.params, self.offsets):
            view = self.data[o:o + p.numel()].view(p.shape)
            view.copy_(p.data.to(device=device, dtype=torch.float32))
            p.data = view
            p.grad = None
            p._grb_flat = weakref.ref(self)
        self.attach_grads()
        _REGISTRY[id(self)] = self

    # -- views ---------------------------------------------------------------
    def view(self, buf: torch.Tensor, i: int) -> torch.Tensor:
        shape, o = self.shapes[i], self.offsets[i]
        n = 1
        for d in shape:
            n *= d
        return buf[o:o + n].view(shape)

    def index_of(self, param) -> int:
        for i, p in enumerate(self.params):
            if p is param:
                return i
        raise KeyError("parameter not in this flat buffer")

    def attach_grads(self) -> None:
        """Make every ``p.grad`` a view of the flat gradient buffer (cheap; safe to repeat)."""
        for i, p in enumerate(self.params):
            if p.grad is None or p.grad.data_ptr() != self.grad.data_ptr() + 4 * self.offsets[i]:
                p.grad = self.view(self.grad, i)

    def reclaim_discarded_grads(self) -> None:
        """Zero the flat gradient range of every parameter whose ``.grad`` is None.

        The fused backward ACCUMULATES into the flat buffer.  ``module.zero_grad()`` and torch optimizers'
        ``zero_grad(set_to_none=True)`` (the default) only drop the ``p.grad`` views; without this the next backward
        would add to the previous step's gradients.  Called at the start of every fused backward."""
        dropped = [i for i, p in enumerate(self.params) if p.grad is None]
        if not dropped:
            return
        if len(dropped) == len(self.params):
            self.grad.zero_()
        else:
            for i in dropped:
                self.view(self.grad, i).zero_()

    def intact(self) -> bool:
        """False if something (``module.to()``, ``load_state_dict(assign=True)``) re-pointed a parameter."""
        base = self.data.data_ptr()
        return all(p.data_ptr() == base + 4 * o for p, o in zip(self.params, self.offsets))

    def version(self) -> int:
        return sum(p._version for p in self.params)
