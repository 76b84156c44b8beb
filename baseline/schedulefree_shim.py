"""Stand-in for the third-party ``schedulefree`` package, which the reference imports (train.py:19) but which is
not installable offline.  Pure PyTorch ``_foreach`` implementation of AdamWScheduleFree, following the upstream
algorithm (facebookresearch/schedule_free, AdamWScheduleFree.step) so that the reference's training loop runs
unmodified.  Used only by the baseline harness, never by the framework.
"""
import math

import torch


class AdamWScheduleFree(torch.optim.Optimizer):
    def __init__(self, params, lr=0.0025, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, warmup_steps=0, r=0.0,
                 weight_lr_power=2.0, foreach=True):
        defaults = dict(lr=lr, betas=betas, eps=eps, r=r, k=0, warmup_steps=warmup_steps, train_mode=False,
                        weight_sum=0.0, lr_max=-1.0, scheduled_lr=0.0, weight_lr_power=weight_lr_power,
                        weight_decay=weight_decay, foreach=foreach)
        super().__init__(params, defaults)

    @torch.no_grad()
    def eval(self):
        for group in self.param_groups:
            if group["train_mode"]:
                beta1, _ = group["betas"]
                for p in group["params"]:
                    state = self.state[p]
                    if "z" in state:
                        p.lerp_(end=state["z"], weight=1 - 1 / beta1)
                group["train_mode"] = False

    @torch.no_grad()
    def train(self):
        for group in self.param_groups:
            if not group["train_mode"]:
                beta1, _ = group["betas"]
                for p in group["params"]:
                    state = self.state[p]
                    if "z" in state:
                        p.lerp_(end=state["z"], weight=1 - beta1)
                group["train_mode"] = True

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            if not group["train_mode"]:
                raise Exception("Optimizer was not in train mode when step is called.")
            eps, beta1, beta2 = group["eps"], *group["betas"]
            decay, k, warmup_steps = group["weight_decay"], group["k"], group["warmup_steps"]
            sched = (k + 1) / warmup_steps if k < warmup_steps else 1.0
            bias_correction2 = 1 - beta2 ** (k + 1)
            lr = group["lr"] * sched
            group["scheduled_lr"] = lr
            lr_max = group["lr_max"] = max(lr, group["lr_max"])
            weight = ((k + 1) ** group["r"]) * (lr_max ** group["weight_lr_power"])
            weight_sum = group["weight_sum"] = group["weight_sum"] + weight
            ckp1 = weight / weight_sum if weight_sum else 0.0
            active = [p for p in group["params"] if p.grad is not None]
            for p in active:
                if "z" not in self.state[p]:
                    self.state[p]["z"] = torch.clone(p, memory_format=torch.preserve_format)
                    self.state[p]["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            if active:
                y = active
                grad = [p.grad for p in active]
                z = [self.state[p]["z"] for p in active]
                exp_avg_sq = [self.state[p]["exp_avg_sq"] for p in active]
                torch._foreach_mul_(exp_avg_sq, beta2)
                torch._foreach_addcmul_(exp_avg_sq, grad, grad, value=1 - beta2)
                denom = torch._foreach_div(exp_avg_sq, bias_correction2)
                torch._foreach_sqrt_(denom)
                torch._foreach_add_(denom, eps)
                torch._foreach_div_(grad, denom)
                torch._foreach_add_(grad, y, alpha=decay)
                torch._foreach_lerp_(y, z, weight=ckp1)
                torch._foreach_add_(y, grad, alpha=lr * (beta1 * (1 - ckp1) - 1))
                torch._foreach_sub_(z, grad, alpha=lr)
            group["k"] = k + 1
        return loss
