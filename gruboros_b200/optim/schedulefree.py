"""Schedule-Free AdamW (Defazio et al., "The Road Less Scheduled", 2024).

Drop-in for ``schedulefree.AdamWScheduleFree`` as the reference uses it (train.py:19,635-642,808):
same constructor, ``train()`` / ``eval()`` mode switch, ``step()``, and the same ``state_dict()``
layout (per-parameter ``z`` and ``exp_avg_sq``; group keys ``k, lr_max, weight_sum, train_mode,
scheduled_lr, warmup_steps, r, weight_lr_power``), so optimizer checkpoints are interchangeable.

Update per step k (0-based) for parameter y with gradient g:
    lr_t  = lr * min(1, (k+1)/warmup);  lr_max = max(lr_max, lr_t)
    w     = (k+1)^r * lr_max^weight_lr_power;  weight_sum += w;  c = w / weight_sum
    v     = beta2 v + (1-beta2) g^2
    gh    = g / (sqrt(v / (1-beta2^(k+1))) + eps) + weight_decay * y
    y     = lerp(y, z, c) + lr_t (beta1 (1-c) - 1) gh
    z     = z - lr_t gh
The model holds y while training; ``eval()`` swaps in the averaged iterate x = lerp(y, z, 1-1/beta1).

On a B200, parameters that live in a ``FlatParams`` buffer are updated by ONE fused kernel
(``csrc/optim.cu``) that also rewrites the bf16 weight mirror and clears the gradients; any other
parameter takes the plain PyTorch path below.
"""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer

from ..utils.flat import lookup


class AdamWScheduleFree(Optimizer):
    def __init__(self, params, lr=0.0025, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, warmup_steps=0, r=0.0,
                 weight_lr_power=2.0, foreach=None, fused=None):
        defaults = dict(lr=lr, betas=betas, eps=eps, r=r, k=0, warmup_steps=warmup_steps, train_mode=False,
                        weight_sum=0.0, lr_max=-1.0, scheduled_lr=0.0, weight_lr_power=weight_lr_power,
                        weight_decay=weight_decay, foreach=foreach)
        super().__init__(params, defaults)
        self.use_fused = fused if fused is not None else True
        self.grad_scale = 1.0        # multiplies gradients inside the step (e.g. 1/world_size)
        self.fused_launches = 0
        self.shard = None            # set by DataParallel.bind_optimizer: sharded fused step

    # ------------------------------------------------------------ mode swap
    @torch.no_grad()
    def eval(self):
        for group in self.param_groups:
            if group["train_mode"]:
                beta1 = group["betas"][0]
                for p in group["params"]:
                    state = self.state[p]
                    if "z" in state:
                        p.lerp_(state["z"].to(p.device), 1 - 1 / beta1)   # y -> x
                group["train_mode"] = False

    @torch.no_grad()
    def train(self):
        for group in self.param_groups:
            if not group["train_mode"]:
                beta1 = group["betas"][0]
                for p in group["params"]:
                    state = self.state[p]
                    if "z" in state:
                        p.lerp_(state["z"].to(p.device), 1 - beta1)       # x -> y
                group["train_mode"] = True

    # ----------------------------------------------------------------- state
    def _init_state(self, group, skip=()):
        """z = copy of the parameter, exp_avg_sq = 0.  Parameters that are consecutive views of one flat buffer
        get consecutive views of one flat z and one flat exp_avg_sq, which is what the fused kernel streams."""
        pending = [p for p in group["params"] if "z" not in self.state[p] and id(p) not in skip]
        if not pending:
            return
        owners = {}
        for p in pending:
            owner = lookup(p)
            if owner is not None and p.is_cuda:
                owners.setdefault(id(owner), (owner, []))[1].append(p)
            else:
                st = self.state[p]
                st["z"] = torch.clone(p, memory_format=torch.preserve_format).detach()
                st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        for owner, plist in owners.values():
            zflat, vflat = self._flat_state_buffers(owner)
            zflat.copy_(owner.data)
            vflat.zero_()
            for p in plist:
                i = owner.index_of(p)
                st = self.state[p]
                st["z"] = owner.view(zflat, i)
                st["exp_avg_sq"] = owner.view(vflat, i)

    @staticmethod
    def _flat_state_buffers(owner):
        """Flat z / exp_avg_sq buffers of a FlatParams (created once; from its allocator when it has one, so
        that peer-mapped parameter storage gets peer-mapped optimizer state)."""
        if not hasattr(owner, "sf_z"):
            if owner.allocator is not None:
                owner.sf_z = owner.allocator("sf_z", owner.numel, torch.float32)
                owner.sf_v = owner.allocator("sf_v", owner.numel, torch.float32)
            else:
                owner.sf_z = torch.empty_like(owner.data)
                owner.sf_v = torch.empty_like(owner.data)
        return owner.sf_z, owner.sf_v

    @torch.no_grad()
    def ensure_state(self):
        """Create the optimizer state now instead of lazily at the first step."""
        for group in self.param_groups:
            self._init_state(group)

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        # loaded tensors are fresh allocations: fold them back into flat buffers where possible
        for group in self.param_groups:
            self._adopt_flat_state(group)

    @torch.no_grad()
    def _adopt_flat_state(self, group) -> None:
        """Move per-parameter state tensors that are NOT views of their owner's flat z / exp_avg_sq buffers into
        those buffers (creating them if needed).  That is the case after ``load_state_dict`` (fresh allocations),
        and also when the state was loaded before the parameters were moved into a ``FlatParams`` buffer - the
        fused kernels stream over the flat buffers, so they must hold the loaded values before the first step."""
        if group["params"]:
            # every step calls this: when the first parameter's state already is a view of the flat buffers (the
            # state is created and adopted for all parameters of a buffer together) there is nothing to do
            p0 = group["params"][0]
            owner0, st0 = lookup(p0), self.state.get(p0, {})
            if owner0 is None or (hasattr(owner0, "sf_z") and "z" in st0 and
                                  st0["z"].data_ptr() == owner0.sf_z.data_ptr() + 4 * owner0.offsets[owner0.index_of(p0)]):
                return
        owners = {}
        for p in group["params"]:
            owner = lookup(p)
            st = self.state.get(p, {})
            if owner is None or not p.is_cuda or "z" not in st:
                continue
            i = owner.index_of(p)
            if hasattr(owner, "sf_z") and st["z"].data_ptr() == owner.sf_z.data_ptr() + 4 * owner.offsets[i] \
                    and st["exp_avg_sq"].data_ptr() == owner.sf_v.data_ptr() + 4 * owner.offsets[i]:
                continue
            owners.setdefault(id(owner), (owner, []))[1].append((p, i))
        for owner, plist in owners.values():
            fresh = not hasattr(owner, "sf_z")
            zflat, vflat = self._flat_state_buffers(owner)
            if fresh:
                zflat.copy_(owner.data)
                vflat.zero_()
            for p, i in plist:
                st = self.state[p]
                owner.view(zflat, i).copy_(st["z"])
                owner.view(vflat, i).copy_(st["exp_avg_sq"])
                st["z"], st["exp_avg_sq"] = owner.view(zflat, i), owner.view(vflat, i)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            if not group["train_mode"]:
                raise RuntimeError("Optimizer was not in train mode when step is called. Call .train() first.")
            beta1, beta2 = group["betas"]
            k = group["k"]
            hp = self._advance(group)
            lr, bias2, ckp1 = hp["lr"], hp["bias2"], hp["ckp1"]

            done = set()
            shard = getattr(self, "shard", None)
            if shard is not None:
                # data parallel: this rank updates only the element range it owns (state lives in `shard`)
                shard.sharded_step(hp, self.grad_scale)
                done = {id(p) for p in shard.flat.params}
                self.fused_launches += 1
            self._init_state(group, skip=done)
            if shard is None:
                self._adopt_flat_state(group)
            if self.use_fused and shard is None:
                done = self._fused_group_step(group, hp)
            for p in group["params"]:
                if p.grad is None or id(p) in done:
                    continue
                g = p.grad if self.grad_scale == 1.0 else p.grad * self.grad_scale
                st = self.state[p]
                z, v = st["z"], st["exp_avg_sq"]
                v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
                gh = g / (v.div(bias2).sqrt_().add_(group["eps"]))
                gh.add_(p, alpha=group["weight_decay"])
                p.lerp_(z, ckp1)
                p.add_(gh, alpha=lr * (beta1 * (1 - ckp1) - 1))
                z.sub_(gh, alpha=lr)
            group["k"] = k + 1
        return loss

    @staticmethod
    def _advance(group) -> dict:
        """Per-step scalars of one parameter group (learning-rate warm-up, bias correction, averaging weight c);
        updates the group's bookkeeping except the step counter k."""
        beta1, beta2 = group["betas"]
        k = group["k"]
        warmup = group["warmup_steps"]
        sched = min(1.0, (k + 1) / warmup) if warmup > 0 and k < warmup else 1.0
        bias2 = 1 - beta2 ** (k + 1)
        lr = group["lr"] * sched
        group["scheduled_lr"] = lr
        lr_max = group["lr_max"] = max(lr, group["lr_max"])
        weight = ((k + 1) ** group["r"]) * (lr_max ** group["weight_lr_power"])
        weight_sum = group["weight_sum"] = group["weight_sum"] + weight
        ckp1 = weight / weight_sum if weight_sum != 0 else 0.0
        return dict(lr=lr, beta1=beta1, beta2=beta2, bias2=bias2, eps=group["eps"], wd=group["weight_decay"], ckp1=ckp1)

    # -------------------------------------------------- range-wise step (overlapped with backward)
    def overlappable(self, owner) -> bool:
        """True if one fused kernel per flat range can replace step(): a single group that holds exactly the
        parameters of `owner` (a FlatParams), fused path enabled, no sharding."""
        return (self.use_fused and self.shard is None and len(self.param_groups) == 1 and owner is not None
                and len(self.param_groups[0]["params"]) == len(owner.params) and owner.intact()
                and all(lookup(p) is owner for p in self.param_groups[0]["params"][:1]))

    @torch.no_grad()
    def begin_ranged_step(self, owner) -> dict:
        group = self.param_groups[0]
        if not group["train_mode"]:
            raise RuntimeError("Optimizer was not in train mode when step is called. Call .train() first.")
        self._init_state(group)
        self._adopt_flat_state(group)
        return self._advance(group)

    @torch.no_grad()
    def step_range(self, owner, lo: int, hi: int, hp: dict) -> None:
        """Schedule-Free AdamW on flat elements [lo, hi) of `owner` (multiples of 4), on the current stream."""
        from ..ops import kernels as K
        K.sfadamw_step(owner.data[lo:hi], owner.sf_z[lo:hi], owner.sf_v[lo:hi], owner.grad[lo:hi], owner.w16[lo:hi],
                       gscale=self.grad_scale, zero_grad=True, **hp)

    def end_ranged_step(self, owner) -> None:
        self.param_groups[0]["k"] += 1
        owner.w16_version = owner.version() + owner.data._version
        owner._grad_clean = True
        self.fused_launches += 1

    def _fused_group_step(self, group, hp) -> set:
        """Run the fused kernel over every flat buffer that this group covers completely."""
        from ..ops import kernels as K
        done = set()
        owners = {}
        for p in group["params"]:
            owner = lookup(p)
            if owner is not None and p.is_cuda and hasattr(owner, "sf_z"):
                owners.setdefault(id(owner), (owner, []))[1].append(p)
        for owner, plist in owners.values():
            if len(plist) != len(owner.params) or not owner.intact():
                continue
            if any(self.state[p]["z"].data_ptr() != owner.sf_z.data_ptr() + 4 * owner.offsets[owner.index_of(p)]
                   for p in plist[:1]):
                continue
            K.sfadamw_step(owner.data, owner.sf_z, owner.sf_v, owner.grad, owner.w16, gscale=self.grad_scale,
                           zero_grad=True, **hp)
            owner.w16_version = owner.version() + owner.data._version
            owner._grad_clean = True
            self.fused_launches += 1
            done.update(id(p) for p in plist)
        return done

    def zero_grad(self, set_to_none: bool = True):
        """Gradients that are views of a flat buffer are zeroed in place (the fused step already cleared them);
        others follow ``set_to_none``."""
        flats = {}
        for group in self.param_groups:
            for p in group["params"]:
                owner = lookup(p)
                if owner is not None:
                    flats[id(owner)] = owner
                elif p.grad is not None:
                    if set_to_none:
                        p.grad = None
                    else:
                        p.grad.zero_()
        for owner in flats.values():
            if not getattr(owner, "_grad_clean", False):
                owner.grad.zero_()
            owner._grad_clean = False
