"""Fully sharded data parallelism (ZeRO-3) over NVLink peer memory.

Nothing of a weight matrix is replicated at rest.  The flat space of all weight matrices is dealt round-robin in
256 KB chunks over the ranks (``csrc/owner.cuh``), and every rank keeps ONLY its own chunks, packed: fp32 masters,
fp32 gradients, Schedule-Free z and second moments, and the bf16 compute copy - 18 bytes per parameter divided by
the world size.  What a step adds on top is transient:

  forward / backward  a layer's bf16 weights are all-gathered into one of two workspace slots right before the layer
             runs, and that all-gather is fused into a GEMM: the CTA-pair tcgen05 kernel's two copy warps per CTA
             stream the NEXT layer's chunks out of the peers' packed shards (plain peer loads over NVLink) while the
             tensor cores work on the current layer's gate GEMM (forward) or FF2 dgrad (backward).  Only the first
             layer of a pass is fetched by a stand-alone kernel.  Two slots alternate, so at most two layers of
             gathered weights exist at any time (weights are always re-gathered in backward).
  gradients  every wgrad GEMM's epilogue adds its tile into the OWNER's packed gradient shard
             (``red.global.add.f32`` on a peer pointer at the element's position inside that shard) - the
             reduce-scatter is part of the GEMM, and no rank ever holds a full-size gradient.
  optimizer  one fused Schedule-Free AdamW pass over the rank's packed arrays writes masters, state and the bf16
             shard; nothing is broadcast.

The 1-D parameters (norm weights, biases) and the embedding table are read in fp32 by the kernels and are tiny
(< 0.1 % of a model): they stay replicated in a small second flat space.  Rank 0 owns that space: the other ranks
add their gradients into rank 0's buffer, rank 0 steps them and copies the new values to every rank, so the
replicas stay bitwise equal.

Checkpoints keep the reference's per-parameter layout: ``gather_params`` materialises the full fp32 parameters
from the shards for ``state_dict()`` (and ``release_params`` drops them again), ``optimizer_state_dict`` rebuilds
the per-parameter optimizer state.

The reference has no sharded mode at all (train.py:644-648: one full replica per rank); this is the capability
its 3B configuration needs.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _lib as L
from ..ops import kernels as K
from ..utils.flat import FlatParams
from .comm import PeerGroup, _lib, ptr_array


def _is_matrix(name: str, p) -> bool:
    return p.dim() >= 2 and name != "token_emb.weight"


class _AllParams:
    """What the optimizer asks of a parameter store: the parameters it covers."""

    def __init__(self, params):
        self.params = params


class FullyShardedDataParallel:
    CHUNK_SHIFT = 16          # 2^16 elements per ownership chunk (256 KB of fp32, 128 KB of bf16)

    def __init__(self, model, *, rank: int, world: int, device, group: PeerGroup | None = None, debug_poison: bool = False):
        """debug_poison fills a workspace slot with NaN whenever its contents go stale, so a finite loss proves that
        every weight a kernel read had been gathered first."""
        self.model, self.rank, self.world = model, rank, world
        self.device = torch.device(device)
        self.group = group if group is not None else PeerGroup(rank, world, self.device)
        self.debug_poison = debug_poison
        self.engine = engine = model.fused_engine()
        chunk = 1 << self.CHUNK_SHIFT
        g = self.group

        def sym(name, numel, dtype):
            item = torch.empty(0, dtype=dtype).element_size()
            return g.alloc(name, numel * item).tensor(dtype, numel)

        big_names = {n for n, p in model.named_parameters() if _is_matrix(n, p)}
        # ---- the big space: layout only; each rank stores its chunks packed
        self.big = FlatParams(model, self.device, pad_to=world * chunk // 64, select=_is_matrix, layout_only=True)
        self.shard = self.big.numel // world
        self.own = -self.CHUNK_SHIFT
        self.y = sym("z3_y", self.shard, torch.float32)
        self.g = sym("z3_g", self.shard, torch.float32)
        self.z = sym("z3_z", self.shard, torch.float32)
        self.v = sym("z3_v", self.shard, torch.float32)
        self.w16 = sym("z3_w16", self.shard, torch.bfloat16)
        # one transient full-size fp32 copy to cut this rank's chunks out of the freshly initialised parameters
        full = torch.zeros(self.big.numel, dtype=torch.float32, device=self.device)
        for p, o in zip(self.big.params, self.big.offsets):
            full[o:o + p.numel()].copy_(p.data.reshape(-1).to(self.device, torch.float32))
        self.y.copy_(full.view(-1, world, chunk)[:, rank].reshape(-1))
        del full
        self.z.copy_(self.y)
        K.cast_f32_bf16(self.y, self.w16)
        for p in self.big.params:              # the matrices now live only in the shards
            p.data = torch.empty(0, dtype=p.dtype, device=self.device)
            p.grad = None
        # ---- the small space: replicated fp32, rank 0 owns it
        self.small = FlatParams(model, self.device, select=lambda n, p: n not in big_names, mirror=False,
                                allocator=lambda name, numel, dtype: sym(f"z3_small_{name}", numel, dtype))
        self.small_z = sym("z3_small_z", self.small.numel, torch.float32)      # used on rank 0; symmetric so that a
        self.small_v = sym("z3_small_v", self.small.numel, torch.float32)      # checkpointing rank could pull them
        self.small_z.copy_(self.small.data)
        vec = [(o, p.numel()) for p, o in zip(self.small.params, self.small.offsets) if p.dim() < 2]
        self.vec_ranges = torch.tensor(vec, dtype=torch.int64, device=self.device).reshape(-1, 2)
        allr = [(o, p.numel()) for p, o in zip(self.small.params, self.small.offsets)]
        self.all_ranges = torch.tensor(allr, dtype=torch.int64, device=self.device).reshape(-1, 2)
        # ---- routing: engine index i (position in named_parameters order) -> (space, index in that space)
        self.names = [n for n, _ in model.named_parameters()]
        big_ix = {n: j for j, n in enumerate(self.big.names)}
        small_ix = {n: j for j, n in enumerate(self.small.names)}
        self.route = [("big", big_ix[n]) if n in big_ix else ("small", small_ix[n]) for n in self.names]
        self.flat = _AllParams(list(model.parameters()))
        # ---- units (layers in execution order, then the head) and the two workspace slots
        depth = engine.depth
        self.units = []
        for li in range(depth):
            js = [big_ix[f"layers.{li}.2.to_hidden_and_gate.weight"], big_ix[f"layers.{li}.4.2.weight"]]
            self.units.append((self.big.offsets[js[0]], self._end(js[1])))
        jl = big_ix["to_logits.weight"]
        self.units.append((self.big.offsets[jl], self._end(jl)))
        self.unit_of = {}
        for j, o in enumerate(self.big.offsets):
            for u, (lo, hi) in enumerate(self.units):
                if lo <= o < hi:
                    self.unit_of[j] = u
        cap = max(hi - lo for lo, hi in self.units)
        self.ws = [torch.empty(cap, dtype=torch.bfloat16, device=self.device) for _ in range(2)]
        self.slot_unit = [None, None]
        self.gathered_bytes = 0
        self.optimizer = None
        self._connected = False
        if not hasattr(self.group.transport, "hub"):
            self.connect()

    def _end(self, j: int) -> int:
        n = 1
        for d in self.big.shapes[j]:
            n *= d
        return self.big.offsets[j] + (n + 63) // 64 * 64

    # ------------------------------------------------------------------ wiring
    def connect(self) -> None:
        """Resolve the peers' buffer addresses (called once every rank has allocated its buffers)."""
        if hasattr(self.group.transport, "hub"):
            self.group.finish_local_connect()
        g = self.group
        self.g_ptrs = g.ptrs("z3_g")
        self.w16_ptrs = g.ptrs("z3_w16")
        self.small_grad_ptrs = g.ptrs("z3_small_grad")
        self.small_data_ptrs = g.ptrs("z3_small_data")
        eng = self.engine
        eng.store = self
        eng.param_gather = self
        eng.grad_sink = (self.g_ptrs, self.own)        # marks the engine data parallel (split-K choice)
        eng.ensure_flat(self.device)
        self._connected = True
        g.transport.host_barrier()

    def bind_optimizer(self, optimizer) -> None:
        from ..optim.schedulefree import AdamWScheduleFree
        if not isinstance(optimizer, AdamWScheduleFree):
            raise TypeError(f"sharded training needs AdamWScheduleFree (its fused step over the packed shards); "
                            f"got {type(optimizer).__name__}")
        self.optimizer = optimizer
        optimizer.shard = self
        optimizer.grad_scale = 1.0 / self.world

    # ------------------------------------------------- parameter store (engine side)
    def param(self, i: int) -> torch.Tensor:
        space, j = self.route[i]
        if space != "small":
            raise RuntimeError(f"{self.names[i]} is sharded: it has no replicated fp32 copy")
        return self.small.view(self.small.data, j)

    def grad(self, i: int) -> torch.Tensor:
        space, j = self.route[i]
        if space != "small":
            raise RuntimeError(f"{self.names[i]} is sharded: its gradient only exists in the owners' shards")
        return self.small.view(self.small.grad, j)

    def weight(self, i: int) -> torch.Tensor:
        """bf16 view of weight matrix i inside the workspace slot that holds its unit (gathered on the stream already)."""
        space, j = self.route[i]
        if space != "big":
            raise RuntimeError(f"{self.names[i]} is not a sharded weight matrix")
        u = self.unit_of[j]
        if self.slot_unit[u % 2] != u:
            raise RuntimeError(f"weights of unit {u} are not resident (slots hold {self.slot_unit})")
        off = self.big.offsets[j] - self.units[u][0]
        n = 1
        for d in self.big.shapes[j]:
            n *= d
        return self.ws[u % 2][off:off + n].view(self.big.shapes[j])

    def scatter(self, i: int):
        """Where the gradient of matrix i goes: (peer pointers, ownership descriptor, flat offset, packed)."""
        space, j = self.route[i]
        if space == "big":
            return (self.g_ptrs, self.own, self.big.offsets[j], True, self.shard)
        # the embedding table: rank 0 owns the whole small space (contiguous ownership of small.numel elements)
        return (self.small_grad_ptrs, self.small.numel, self.small.offsets[j], False, self.small.numel)

    # ------------------------------------------------------------- weight gathers
    def _gather_args(self, unit: int):
        lo, hi = self.units[unit]
        return (self.w16_ptrs, self.CHUNK_SHIFT, lo, hi, self.ws[unit % 2].data_ptr(), self.shard, self.ws[unit % 2].numel())

    def _order(self, direction: str):
        n = len(self.units)
        return list(range(n)) if direction == "fwd" else list(range(n - 1, -1, -1))

    def _claim(self, unit: int) -> bool:
        """Mark `unit` as the content of its slot; False if it already is."""
        if self.slot_unit[unit % 2] == unit:
            return False
        if self.debug_poison:
            self.ws[unit % 2].fill_(float("nan"))
        self.slot_unit[unit % 2] = unit
        lo, hi = self.units[unit]
        self.gathered_bytes += 2 * (hi - lo)
        return True

    def begin_pass(self, direction: str) -> None:
        """Make the first unit of the pass resident with a stand-alone gather."""
        first = self._order(direction)[0]
        if self._claim(first):
            K.gather_chunks(*self._gather_args(first))

    def prefetch(self, direction: str, unit: int) -> dict:
        """Keyword arguments for the GEMM that should gather the unit running after `unit` ({} when resident)."""
        order = self._order(direction)
        pos = order.index(unit)
        if pos + 1 >= len(order):
            return {}
        nxt = order[pos + 1]
        if not self._claim(nxt):
            return {}
        return {"gather": self._gather_args(nxt)}

    def _drop_all(self) -> None:
        self.slot_unit = [None, None]
        if self.debug_poison:
            for w in self.ws:
                w.fill_(float("nan"))

    # ------------------------------------------------------------- step hooks
    def pre_backward(self, engine) -> None:
        pass

    def fold_stepper(self):
        return None     # weights are re-gathered layer by layer during backward: the update stays after it

    def push_vector_grads(self) -> None:
        """Add the locally accumulated gradients of the 1-D parameters into rank 0's buffer (and clear them here)."""
        n = self.vec_ranges.shape[0]
        L.check(_lib().grb_push_add_ranges(self.small.grad.data_ptr(), ptr_array(self.small_grad_ptrs), self.world, self.rank,
                                           self.vec_ranges.data_ptr(), n, self.small.numel, L.stream()), "grb_push_add_ranges")
        K._count()

    def reduce_gradients(self) -> None:
        self.push_vector_grads()
        self.group.device_barrier()
        K._count(2)

    def sharded_step(self, hp: dict, grad_scale: float) -> None:
        """Fused Schedule-Free AdamW over this rank's packed shard (masters, state, bf16 copy, gradient clear), and on
        rank 0 over the small replicated space."""
        K.sfadamw_step(self.y, self.z, self.v, self.g, self.w16, gscale=grad_scale, zero_grad=True, **hp)
        if self.rank == 0:
            K.sfadamw_step(self.small.data, self.small_z, self.small_v, self.small.grad, None, gscale=grad_scale,
                           zero_grad=True, **hp)
        self.small._grad_clean = True

    def bcast_small_params(self) -> None:
        """Rank 0 copies the new values of the small space to every rank."""
        n = self.all_ranges.shape[0]
        L.check(_lib().grb_bcast_ranges(self.small.data.data_ptr(), ptr_array(self.small_data_ptrs), self.world, self.rank,
                                        self.all_ranges.data_ptr(), n, self.small.numel, L.stream()), "grb_bcast_ranges")
        K._count()

    def bcast_vector_params(self) -> None:
        self.bcast_small_params()

    def post_step(self) -> None:
        self.bcast_small_params()
        self.group.device_barrier()
        K._count(2)
        self._drop_all()        # every gathered weight is stale now

    # ------------------------------------------------------------ memory report
    def persistent_bytes(self) -> dict:
        """Bytes this rank holds between steps, by kind, and the transient workspace."""
        sh = self.shard
        return {"sharded_params_grads_state": sh * (4 + 4 + 4 + 4 + 2), "replicated_small": self.small.numel * 16,
                "gather_workspace": sum(w.numel() * 2 for w in self.ws),
                "unsharded_equivalent": self.big.numel * 18}

    # ------------------------------------------------------- checkpoint support
    def _gather_packed(self, name: str) -> torch.Tensor:
        """Full fp32 flat tensor of the big space rebuilt from every rank's packed buffer `name`."""
        out = torch.empty(self.big.numel, dtype=torch.float32, device=self.device)
        L.check(L.lib().grb_gather_interleaved(out.data_ptr(), ptr_array(self.group.ptrs(name)), self.world, self.rank,
                                               self.CHUNK_SHIFT, self.big.numel, 1, 0, L.stream()), "grb_gather_interleaved")
        K._count()
        return out

    def gather_params(self, materialize: bool = True) -> None:
        """Collective.  Give the sharded parameters full fp32 values again (views of one temporary buffer) so that
        ``state_dict()`` / generation see the whole model; ``release_params`` frees it.  Ranks that only take part
        pass materialize=False."""
        self.group.device_barrier()
        if materialize:
            full = self._gather_packed("z3_y")
            for j, p in enumerate(self.big.params):
                p.data = self.big.view(full, j)
        self.group.device_barrier()

    def release_params(self) -> None:
        for p in self.big.params:
            p.data = torch.empty(0, dtype=p.dtype, device=self.device)

    def reset_optimizer_state(self) -> None:
        self.z.copy_(self.y)
        self.v.zero_()
        self.small_z.copy_(self.small.data)
        self.small_v.zero_()

    def optimizer_state_dict(self, materialize: bool = True):
        """Collective.  The optimizer state in the reference's per-parameter layout (``state[i] = {z, exp_avg_sq}``,
        CPU fp32 tensors shaped like parameter i, in named_parameters order), rebuilt from the shards."""
        self.group.device_barrier()
        out = None
        if materialize:
            z, v = self._gather_packed("z3_z"), self._gather_packed("z3_v")
            sz, sv = self.small_z, self.small_v
            if self.rank != 0:      # rank 0 keeps the small space's state: read it through its symmetric buffers
                sz, sv = torch.empty_like(self.small_z), torch.empty_like(self.small_v)
                K.merge([(sz, self.group.ptrs("z3_small_z")[0], 1.0), (sv, self.group.ptrs("z3_small_v")[0], 1.0)], None,
                        self.small.numel)
            state = {}
            for i, (space, j) in enumerate(self.route):
                fl, zz, vv = (self.big, z, v) if space == "big" else (self.small, sz, sv)
                state[i] = {"z": fl.view(zz, j).cpu().clone(), "exp_avg_sq": fl.view(vv, j).cpu().clone()}
            groups = self.optimizer.state_dict()["param_groups"] if self.optimizer is not None else []
            out = {"state": state, "param_groups": groups}
        self.group.device_barrier()
        return out

    def load_optimizer_state_dict(self, sd: dict) -> None:
        """Take this rank's share of a per-parameter optimizer state; parameters without saved state start fresh."""
        chunk = 1 << self.CHUNK_SHIFT
        for key, packed in (("z", self.z), ("exp_avg_sq", self.v)):
            full = torch.zeros(self.big.numel, dtype=torch.float32, device=self.device)
            if key == "z":      # default: z = parameter
                L.check(L.lib().grb_gather_interleaved(full.data_ptr(), ptr_array(self.group.ptrs("z3_y")), self.world, self.rank,
                                                       self.CHUNK_SHIFT, self.big.numel, 1, 0, L.stream()), "grb_gather_interleaved")
            for i, (space, j) in enumerate(self.route):
                st = sd.get("state", {}).get(i)
                if space == "big" and st and key in st:
                    self.big.view(full, j).copy_(st[key].to(self.device, torch.float32))
            packed.copy_(full.view(-1, self.world, chunk)[:, self.rank].reshape(-1))
            del full
        for i, (space, j) in enumerate(self.route):
            st = sd.get("state", {}).get(i)
            if space == "small" and st and "z" in st:
                self.small.view(self.small_z, j).copy_(st["z"].to(self.device, torch.float32))
                self.small.view(self.small_v, j).copy_(st["exp_avg_sq"].to(self.device, torch.float32))
        if self.optimizer is not None and sd.get("param_groups"):
            self.optimizer.load_state_dict({"state": {}, "param_groups": sd["param_groups"]})
        self.group.transport.host_barrier()
