"""Fully sharded data parallelism (ZeRO-3 style) over NVLink peer memory.

Builds on ``DataParallel`` (gradient reduce-scatter fused into the wgrad epilogues, optimizer state and updates
sharded over the ranks, ownership dealt in chunks).  In addition the bf16 compute weights are sharded AT REST: after an optimizer
step a rank holds up-to-date bf16 values only for the range it owns.  Before a layer runs, the ranges of that
layer owned by other ranks are all-gathered into the local mirror by plain peer loads - and that all-gather is
fused into a GEMM: the CTA-pair tcgen05 kernel carries two extra warps per CTA that stream the NEXT unit's
remote shards over NVLink while the tensor cores work on the current gate GEMM (``EpiArgs::copy_*``), so the
transfer costs no launch of its own and hides under the math.  Only the first unit of a pass is fetched by a
stand-alone copy kernel.  Units are the layers in execution order plus the head (final norm + logits).

``reshard_after_forward=True`` drops the gathered weights after the forward pass (they are gathered again,
in reverse order, during backward - the ZeRO-3 memory behaviour); the default keeps them until the optimizer
step, which a 180 GB B200 can afford.  ``debug_poison`` overwrites every dropped range with NaN so a test
proves that nothing stale is ever read.

The reference has no sharded mode at all (train.py:644-648: one full replica per rank); this is the capability
its 3B configuration needs.
"""
from __future__ import annotations

import torch

from ..ops import _lib as L
from ..ops import kernels as K
from .comm import _lib, ptr_array
from .dp import DataParallel


class FullyShardedDataParallel(DataParallel):
    def __init__(self, model, *, rank, world, device, group=None, reshard_after_forward=False, debug_poison=False,
                 interleave=None):
        self.reshard_after_forward = reshard_after_forward
        self.debug_poison = debug_poison
        self.resident: set[int] = set()
        self.units: list[tuple[int, int]] = []
        self.gathered_bytes = 0
        # bf16 weights: one contiguous shard per rank (the all-gather copies contiguous ranges of one holder);
        # gradients, fp32 masters and optimizer state: dealt in chunks like the data-parallel mode unless
        # GRB_DP_INTERLEAVE=0, so that a layer's gradient tiles do not all converge on the rank that holds the layer
        super().__init__(model, rank=rank, world=world, device=device, group=group, interleave=interleave)

    # ------------------------------------------------------------------ wiring
    def connect(self) -> None:
        super().connect()
        f = self.flat
        index = {n: i for i, n in enumerate(f.names)}
        end = lambda i: f.offsets[i] + (f.params[i].numel() + 63) // 64 * 64
        depth = self.engine.depth
        self.units = []
        for li in range(depth):
            lo = f.offsets[index[f"layers.{li}.1.weight"]]
            hi = end(index[f"layers.{li}.4.2.bias"])
            self.units.append((lo, hi))
        self.units.append((f.offsets[index["norm.weight"]], end(index["to_logits.weight"])))     # head = unit `depth`
        self.resident = set(range(len(self.units)))      # the initial cast made every rank's mirror complete
        self.engine.param_gather = self

    def segments(self, unit: int):
        """Peer-load segments (src, dst, bytes) that complete unit `unit` of the local bf16 mirror."""
        lo, hi = self.units[unit]
        base = self.flat.w16.data_ptr()
        segs = []
        for r in range(self.world):
            if r == self.rank:
                continue
            a, b = max(lo, r * self.shard), min(hi, (r + 1) * self.shard)
            if b > a:
                segs.append((self.w16_ptrs[r] + 2 * a, base + 2 * a, 2 * (b - a)))
        return segs

    # ------------------------------------------------------------- engine hooks
    def _order(self, direction: str):
        n = len(self.units)
        return list(range(n)) if direction == "fwd" else list(range(n - 1, -1, -1))

    def begin_pass(self, direction: str) -> None:
        """Make the first unit of the pass resident with a stand-alone gather."""
        if direction == "bwd" and self.reshard_after_forward:
            self._drop_all()
        first = self._order(direction)[0]
        if first not in self.resident:
            segs = self.segments(first)
            K.copy_segments(segs)
            self.gathered_bytes += sum(s[2] for s in segs)
            self.resident.add(first)

    def prefetch(self, direction: str, unit: int):
        """Side-copy segments for the unit that runs after `unit` (None when it is already resident)."""
        order = self._order(direction)
        pos = order.index(unit)
        if pos + 1 >= len(order):
            return None
        nxt = order[pos + 1]
        if nxt in self.resident:
            return None
        self.resident.add(nxt)
        segs = self.segments(nxt)
        self.gathered_bytes += sum(s[2] for s in segs)
        return segs or None

    def _drop_all(self) -> None:
        self.resident.clear()
        if self.debug_poison:
            w = self.flat.w16
            if self.begin > 0:
                w[:self.begin].fill_(float("nan"))
            if self.begin + self.shard < w.numel():
                w[self.begin + self.shard:].fill_(float("nan"))

    # ------------------------------------------------------------- step hooks
    def fold_stepper(self):
        return None     # the sharded mirror is re-gathered layer by layer during backward: the update stays after it

    def _holder_shard(self) -> int:
        return self.shard

    def sharded_step(self, hp: dict, grad_scale: float) -> None:
        """Fused Schedule-Free AdamW on the owned elements; each new bf16 weight goes only to the rank that holds
        its range (sharded at rest) - with contiguous ownership that is this rank itself."""
        if self.interleave:
            return super().sharded_step(hp, grad_scale)
        f = self.flat
        L.check(_lib().grb_sfadamw_shard_step(f.data.data_ptr(), self.z.data_ptr(), self.v.data_ptr(), f.grad.data_ptr(),
                                              ptr_array([f.w16.data_ptr()]), 1, self.begin, self.shard,
                                              hp["lr"], hp["beta1"], hp["beta2"], hp["bias2"], hp["eps"], hp["wd"],
                                              hp["ckp1"], grad_scale, 1, L.stream()), "grb_sfadamw_shard_step")
        K._count()
        f.w16_version = f.version() + f.data._version
        f._grad_clean = True

    def post_step(self) -> None:
        super().post_step()
        self._drop_all()        # every non-owned range of the mirror is stale now
