"""Data parallelism over NVLink peer memory, with the gradient reduce-scatter fused into backward.

The reference has no data-parallel mode (every rank trains its own replica, train.py:644-648); this is the
data-parallel training the 1B benchmark config asks for.  Layout: the flat parameter space is cut into
`world` equal element ranges; rank r OWNS range r - it keeps the Schedule-Free state (z, v) only for that
range and is the only rank that updates it (ZeRO-1 style).

  ownership  by default the flat space is dealt round-robin in 256 KB chunks rather than cut into `world` contiguous
             shards, so that every weight matrix is spread over all owners: all ranks work on the same layer at the
             same time, and with contiguous shards their gradient tiles would all converge on the one rank that
             holds that matrix ((world - 1) x the matrix through one NVLink ingress per GEMM).
  backward   every wgrad GEMM's epilogue adds its tile straight into the OWNER's flat gradient buffer
             (red.global.add.f32 on a peer pointer, tile by tile while later tiles still compute) - there
             is no separate collective.  Vector gradients (norm weights, biases) accumulate locally and are
             pushed by one small kernel.
  barrier    flag exchange in peer memory (stream ordered, bounded wait).
  optimizer  each rank runs the fused Schedule-Free AdamW kernel on its range and stores the new bf16
             weights into EVERY rank's mirror (the parameter all-gather fused into the update); fp32 values
             of the vector parameters are copied to the peers the same way.
  barrier    then the next forward may start.

With one optimizer step per chunk the update is folded into backward as well (``fold_stepper``): when a rank has
launched the last gradient kernel of a layer it raises that layer's flag on every peer; the owners of the layer's
range wait (side stream, bounded) for all ranks' flags and update + republish just that range while the remaining
layers' backward still runs; one barrier at the end replaces the two above.

No NCCL call is made on this path; torch.distributed is only the host side channel that carries the IPC
handles at start-up.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from ..ops import _lib as L
from ..ops import kernels as K
from ..utils.flat import FlatParams
from .comm import PeerGroup, _lib, ptr_array


class DataParallel:
    # elements per ownership chunk when the flat space is dealt round-robin (2^16 fp32 = 256 KB = 32 rows of a
    # 2048-wide matrix: every 256-row gradient tile fans out to all owners)
    CHUNK_SHIFT = 16

    def __init__(self, model, *, rank: int, world: int, device, group: PeerGroup | None = None,
                 interleave: bool | None = None, nvls: bool | None = None):
        """interleave: deal ownership of the flat space round-robin in chunks (default; GRB_DP_INTERLEAVE=0 turns it
        off) instead of one contiguous shard per rank - see ``csrc/owner.cuh`` for why; the sharded-weights subclass
        needs contiguous shards."""
        if interleave is None:
            interleave = os.environ.get("GRB_DP_INTERLEAVE", "1") == "1"
        self.model, self.rank, self.world = model, rank, world
        self.interleave = bool(interleave) and world > 1
        self.device = torch.device(device)
        self.group = group if group is not None else PeerGroup(rank, world, self.device)
        engine = model.fused_engine()
        self.engine = engine

        # GRB_NVLS=1: the bf16 weight mirrors of all ranks are bound to one NVSwitch multicast object, and an owner
        # publishes a new weight with ONE multimem store instead of one store per rank (parallel/nvls.py)
        self.mc16 = None
        self._mc_buf = None
        want_nvls = nvls if nvls is not None else os.environ.get("GRB_NVLS", "0") == "1"

        def allocator(name, numel, dtype):
            item = torch.empty(0, dtype=dtype).element_size()
            if name == "w16" and want_nvls and world > 1 and not hasattr(self.group.transport, "hub"):
                from .nvls import MulticastBuffer
                self._mc_buf = MulticastBuffer("flat_w16", numel * item, rank, world, self.device,
                                               self.group.transport.host_barrier)
                self.mc16 = self._mc_buf.mc_ptr
                return self._mc_buf.tensor(dtype, numel)
            return self.group.alloc(f"flat_{name}", numel * item).tensor(dtype, numel)

        # equal shares: a multiple of 1024 elements each, or of whole chunks when ownership is dealt round-robin
        chunk = 1 << self.CHUNK_SHIFT
        pad = world * chunk // 64 if self.interleave else world * 16
        self.flat = FlatParams(model, self.device, pad_to=pad, allocator=allocator)
        engine.ensure_flat(self.device)
        assert engine.flat is self.flat
        self.shard = self.flat.numel // world                     # elements owned by each rank
        self.begin = rank * self.shard                            # (contiguous ownership only)
        self.own = -self.CHUNK_SHIFT if self.interleave else self.shard     # descriptor the kernels take (owner.cuh)
        # optimizer state of the owned elements (symmetric, so a checkpointing rank can pull the other ranks')
        self.z = self.group.alloc("sf_z", self.shard * 4).tensor(torch.float32, self.shard)
        self.v = self.group.alloc("sf_v", self.shard * 4).tensor(torch.float32, self.shard)
        if self.interleave:
            self.z.copy_(self.flat.data.view(-1, world, chunk)[:, rank].reshape(-1))
        else:
            self.z.copy_(self.flat.data[self.begin:self.begin + self.shard])
        # ranges of 1-D parameters (accumulated locally, exchanged by the small push kernels)
        vec = [(o, p.numel()) for p, o in zip(self.flat.params, self.flat.offsets) if p.dim() < 2]
        self.vec_ranges = torch.tensor(vec, dtype=torch.int64, device=self.device).reshape(-1, 2)
        # parameters the kernels read in fp32 (1-D parameters and the embedding table): owners republish them
        # after every update; the embedding's gradient still arrives through the scatter epilogue
        f32 = vec + [(o, p.numel()) for n, p, o in zip(self.flat.names, self.flat.params, self.flat.offsets)
                     if p.dim() == 2 and n == "token_emb.weight"]
        self.f32_ranges = torch.tensor(f32, dtype=torch.int64, device=self.device).reshape(-1, 2)
        # per-layer completion flags for the folded step: [unit][rank] int64, value = number of the step
        self.MAX_UNITS = 128
        self.unit_flags = self.group.alloc("unit_flags", self.MAX_UNITS * 8 * 8)
        self.unit_flags.tensor(torch.int64, self.MAX_UNITS * 8).zero_()
        self._fold_step = 0
        self._unit_cache = None
        self.optimizer = None
        self._connected = False
        if not hasattr(self.group.transport, "hub"):
            self.connect()

    # ------------------------------------------------------------------ wiring
    def connect(self) -> None:
        """Resolve the peers' buffer addresses (called once every rank has allocated its buffers)."""
        if hasattr(self.group.transport, "hub"):
            self.group.finish_local_connect()
        g = self.group
        self.grad_ptrs = g.ptrs("flat_grad")
        self.data_ptrs = g.ptrs("flat_data")
        # with a multicast mirror there are no per-peer pointers to it: every write goes through the multicast address
        self.w16_ptrs = g.ptrs("flat_w16") if self.mc16 is None else [self.flat.w16.data_ptr()] * self.world
        self.engine.grad_sink = (self.grad_ptrs, self.own)
        K.cast_f32_bf16(self.flat.data, self.flat.w16)
        self.flat.w16_version = self.flat.version() + self.flat.data._version
        self._connected = True
        g.transport.host_barrier()

    def bind_optimizer(self, optimizer) -> None:
        """Switch `optimizer` (AdamWScheduleFree) to the sharded fused step for this model's parameters."""
        from ..optim.schedulefree import AdamWScheduleFree
        if not isinstance(optimizer, AdamWScheduleFree):
            # any other optimizer would step on local gradients that hold only this rank's owned chunks (summed over
            # ranks, unscaled) and zeros elsewhere, and the ranks would silently diverge
            raise TypeError(f"data-parallel / sharded training needs AdamWScheduleFree (its sharded fused step); "
                            f"got {type(optimizer).__name__}")
        self.optimizer = optimizer
        optimizer.shard = self
        optimizer.grad_scale = 1.0 / self.world

    @staticmethod
    def owner_of(idx: int, own: int, world: int) -> int:
        """Host restatement of ``grb_owner`` (csrc/owner.cuh)."""
        return idx // own if own > 0 else (idx >> (-own)) % world

    @staticmethod
    def local_index(idx: int, own: int, world: int) -> int:
        """Host restatement of ``grb_local_index``: where an owned element sits in its owner's compact state."""
        if own > 0:
            return idx % own
        sh = -own
        return (((idx >> sh) // world) << sh) + (idx & ((1 << sh) - 1))

    def owned(self, t: torch.Tensor) -> torch.Tensor:
        """The elements this rank owns of a full-length flat tensor (a view; [chunks, chunk] when interleaved)."""
        if self.interleave:
            return t[:self.flat.numel].view(-1, self.world, 1 << self.CHUNK_SHIFT)[:, self.rank]
        return t[self.begin:self.begin + self.shard]

    # ------------------------------------------------------------- step hooks
    def pre_backward(self, engine) -> None:
        pass    # the engine already carries the scatter sink

    def push_vector_grads(self) -> None:
        """Add the locally accumulated gradients of 1-D parameters into their owners' buffers."""
        n = self.vec_ranges.shape[0]
        L.check(_lib().grb_push_add_ranges(self.flat.grad.data_ptr(), ptr_array(self.grad_ptrs), self.world, self.rank,
                                           self.vec_ranges.data_ptr(), n, self.own, L.stream()), "grb_push_add_ranges")
        K._count()

    def reduce_gradients(self) -> None:
        """Finish the reduce-scatter: push vector gradients to their owners, then the cross-GPU barrier."""
        self.push_vector_grads()
        self.group.device_barrier()
        K._count(2)

    def _holder_shard(self) -> int:
        """0: every rank keeps a full bf16 mirror (the update is broadcast); the sharded-weights subclass returns the
        size of the contiguous bf16 shard each rank holds at rest."""
        return 0

    def sharded_step(self, hp: dict, grad_scale: float) -> None:
        """Fused Schedule-Free AdamW on the owned elements; new bf16 weights go to every rank's mirror."""
        f = self.flat
        if self.interleave:
            L.check(_lib().grb_sfadamw_interleaved_step(f.data.data_ptr(), self.z.data_ptr(), self.v.data_ptr(),
                                                        f.grad.data_ptr(), ptr_array(self.w16_ptrs), self.world, self.rank,
                                                        self.CHUNK_SHIFT, self.shard, hp["lr"], hp["beta1"], hp["beta2"],
                                                        hp["bias2"], hp["eps"], hp["wd"], hp["ckp1"], grad_scale, 1,
                                                        self._holder_shard(), self.mc16, L.stream()), "grb_sfadamw_interleaved_step")
            K._count()
            f.w16_version = f.version() + f.data._version
            f._grad_clean = True
            return
        L.check(_lib().grb_sfadamw_shard_step(f.data.data_ptr(), self.z.data_ptr(), self.v.data_ptr(), f.grad.data_ptr(),
                                              ptr_array(self.w16_ptrs), self.world, self.begin, self.shard,
                                              hp["lr"], hp["beta1"], hp["beta2"], hp["bias2"], hp["eps"], hp["wd"],
                                              hp["ckp1"], grad_scale, 1, self.mc16, L.stream()), "grb_sfadamw_shard_step")
        K._count()
        f.w16_version = f.version() + f.data._version
        f._grad_clean = True

    def bcast_vector_params(self) -> None:
        """Owners copy the parameters that kernels read in fp32 (1-D parameters, embedding table) to their peers."""
        n = self.f32_ranges.shape[0]
        L.check(_lib().grb_bcast_ranges(self.flat.data.data_ptr(), ptr_array(self.data_ptrs), self.world, self.rank,
                                        self.f32_ranges.data_ptr(), n, self.own, L.stream()), "grb_bcast_ranges")
        K._count()

    def post_step(self) -> None:
        """After the optimizer: publish vector parameters, then barrier so the next forward sees every update."""
        self.bcast_vector_params()
        self.group.device_barrier()
        K._count(2)

    # ------------------------------------------------ optimizer folded into backward
    def fold_stepper(self):
        """Stepper for ``FusedEngine.train_step``: per-layer cross-rank completion flags, then the sharded update of
        that layer on a side stream.  None when no optimizer is bound."""
        ok = self.optimizer is not None and self._connected and len(self.optimizer.param_groups) == 1
        return _FoldStepper(self) if ok else None

    def _unit_tables(self, units):
        """Per unit: its vector-gradient ranges, its fp32-published ranges and the part of it this rank owns."""
        if self._unit_cache is not None and self._unit_cache[0] == units:
            return self._unit_cache[1]
        if len(units) > self.MAX_UNITS:
            raise ValueError("too many parameter units for the per-layer flags")
        vec, f32 = self.vec_ranges.tolist(), self.f32_ranges.tolist()
        mine_lo, mine_hi = self.begin, self.begin + self.shard
        flag_ptrs = self.group.ptrs("unit_flags")
        tabs = []
        for j, (lo, hi) in enumerate(units):
            pick = lambda rs: torch.tensor([r for r in rs if lo <= r[0] < hi], dtype=torch.int64, device=self.device).reshape(-1, 2)
            if self.interleave:
                a, b = lo, hi          # chunks dealt round-robin: the kernel walks this rank's chunks inside [lo, hi)
            else:
                a, b = max(lo, mine_lo), min(hi, mine_hi)
            tabs.append(dict(vec=pick(vec), f32=pick(f32), own=(a, b) if b > a else None,
                             signal=ptr_array([p + j * 64 for p in flag_ptrs]), wait=self.unit_flags.ptr + j * 64))
        self._unit_cache = (list(units), tabs)
        return tabs

    # ------------------------------------------------------- checkpoint support
    def release_params(self) -> None:
        """Counterpart of ``gather_params`` for storage that drops the gathered values again (nothing to do here:
        every rank keeps full fp32 parameters)."""

    def gather_params(self, materialize: bool = True) -> None:
        """Pull the up-to-date fp32 values of the ranges other ranks own (before state_dict / generation)."""
        self.group.device_barrier()
        if self.interleave:
            L.check(_lib().grb_gather_interleaved(self.flat.data.data_ptr(), ptr_array(self.data_ptrs), self.world, self.rank,
                                                  self.CHUNK_SHIFT, self.flat.numel, 0, 1, L.stream()), "grb_gather_interleaved")
        for r in range(self.world):
            if r == self.rank or self.interleave:
                continue
            lo = r * self.shard
            dst = self.flat.data[lo:lo + self.shard]
            K.merge([(dst, self.data_ptrs[r] + 4 * lo, 1.0)], None, self.shard)
        self.group.device_barrier()
        self.flat.w16_version = self.flat.version() + self.flat.data._version

    def reset_optimizer_state(self) -> None:
        """z <- the current parameters, second moments <- 0, for the owned elements (a fresh optimizer)."""
        self.z.copy_(self.owned(self.flat.data).reshape(-1))
        self.v.zero_()

    def optimizer_state_dict(self, materialize: bool = True):
        """Collective.  The optimizer state in the reference's per-parameter layout (``state[i] = {z, exp_avg_sq}``,
        CPU fp32 tensors shaped like parameter i, plus the bound optimizer's ``param_groups``), rebuilt from every
        owner's share - what a single-replica run of the same optimizer would save.  Ranks that only take part in
        the gather pass ``materialize=False`` and get None (no host copies)."""
        z, v = self.gather_optimizer_state()
        if not materialize:
            return None
        state = {}
        for i, (p, off) in enumerate(zip(self.flat.params, self.flat.offsets)):
            n = p.numel()
            state[i] = {"z": z[off:off + n].view(p.shape).cpu().clone(), "exp_avg_sq": v[off:off + n].view(p.shape).cpu().clone()}
        groups = self.optimizer.state_dict()["param_groups"] if self.optimizer is not None else []
        return {"state": state, "param_groups": groups}

    def load_optimizer_state_dict(self, sd: dict) -> None:
        """Take this rank's share of a per-parameter optimizer state (as written by ``optimizer_state_dict`` or by a
        single-replica run); parameters without saved state start fresh (z = parameter, second moment 0)."""
        z = self.flat.data.clone()
        v = torch.zeros_like(z)
        for i, (p, off) in enumerate(zip(self.flat.params, self.flat.offsets)):
            st = sd.get("state", {}).get(i)
            if st and "z" in st:
                n = p.numel()
                z[off:off + n].copy_(st["z"].reshape(-1).to(z.device, torch.float32))
                v[off:off + n].copy_(st["exp_avg_sq"].reshape(-1).to(z.device, torch.float32))
        self.z.copy_(self.owned(z).reshape(-1))
        self.v.copy_(self.owned(v).reshape(-1))
        if self.optimizer is not None and sd.get("param_groups"):
            self.optimizer.load_state_dict({"state": {}, "param_groups": sd["param_groups"]})

    def gather_optimizer_state(self):
        """Full flat z and exp_avg_sq on this rank (for a reference-layout optimizer state_dict)."""
        self.group.device_barrier()
        z = torch.empty(self.flat.numel, dtype=torch.float32, device=self.device)
        v = torch.empty_like(z)
        zp, vp = self.group.ptrs("sf_z"), self.group.ptrs("sf_v")
        if self.interleave:
            for dst, src in ((z, zp), (v, vp)):
                L.check(_lib().grb_gather_interleaved(dst.data_ptr(), ptr_array(src), self.world, self.rank, self.CHUNK_SHIFT,
                                                      self.flat.numel, 1, 0, L.stream()), "grb_gather_interleaved")
        for r in range(self.world if not self.interleave else 0):
            lo = r * self.shard
            K.merge([(z[lo:lo + self.shard], zp[r], 1.0), (v[lo:lo + self.shard], vp[r], 1.0)], None, self.shard)
        self.group.device_barrier()
        return z, v


class _FoldStepper:
    """See ``DataParallel.fold_stepper``."""

    def __init__(self, dp: DataParallel):
        self.dp = dp

    def begin(self, units):
        dp = self.dp
        self.tabs = dp._unit_tables(units)
        group = dp.optimizer.param_groups[0]
        if not group["train_mode"]:
            raise RuntimeError("Optimizer was not in train mode when step is called. Call .train() first.")
        self.hp = dp.optimizer._advance(group)       # the state of the owned range lives in dp.z / dp.v
        dp._fold_step += 1

    def unit_done(self, j, main, side):
        dp, t, lib = self.dp, self.tabs[j], _lib()
        f, hp = dp.flat, self.hp
        # main stream: vector gradients of this unit to their owners, then "rank has finished unit j"
        if t["vec"].shape[0]:
            L.check(lib.grb_push_add_ranges(f.grad.data_ptr(), ptr_array(dp.grad_ptrs), dp.world, dp.rank, t["vec"].data_ptr(),
                                            t["vec"].shape[0], dp.own, L.stream()), "grb_push_add_ranges")
        L.check(lib.grb_comm_signal(t["signal"], dp.world, dp.rank, dp._fold_step, L.stream()), "grb_comm_signal")
        K._count(2)
        if t["own"] is None:
            return
        lo, hi = t["own"]
        ev = torch.cuda.Event()
        ev.record(main)
        with torch.cuda.stream(side):
            side.wait_event(ev)
            st = L.stream()
            L.check(lib.grb_comm_wait(t["wait"], dp.world, dp._fold_step, dp.group.timeout_ns,
                                      L.err_flag(dp.device).data_ptr(), st), "grb_comm_wait")
            if dp.interleave:
                L.check(lib.grb_sfadamw_interleaved_range_step(
                    f.data.data_ptr(), dp.z.data_ptr(), dp.v.data_ptr(), f.grad.data_ptr(), ptr_array(dp.w16_ptrs), dp.world,
                    dp.rank, dp.CHUNK_SHIFT, lo, hi, hp["lr"], hp["beta1"], hp["beta2"], hp["bias2"], hp["eps"], hp["wd"],
                    hp["ckp1"], dp.optimizer.grad_scale, 1, dp._holder_shard(), dp.mc16, st), "grb_sfadamw_interleaved_range_step")
            else:
                off = lo - dp.begin
                L.check(lib.grb_sfadamw_shard_step(f.data.data_ptr(), dp.z[off:].data_ptr(), dp.v[off:].data_ptr(), f.grad.data_ptr(),
                                                   ptr_array(dp.w16_ptrs), dp.world, lo, hi - lo, hp["lr"], hp["beta1"],
                                                   hp["beta2"], hp["bias2"], hp["eps"], hp["wd"], hp["ckp1"],
                                                   dp.optimizer.grad_scale, 1, dp.mc16, st), "grb_sfadamw_shard_step")
            if t["f32"].shape[0]:
                L.check(lib.grb_bcast_ranges(f.data.data_ptr(), ptr_array(dp.data_ptrs), dp.world, dp.rank, t["f32"].data_ptr(),
                                             t["f32"].shape[0], dp.own, st), "grb_bcast_ranges")
            K._count(3)

    def end(self, main, side):
        dp = self.dp
        main.wait_stream(side)
        dp.optimizer.end_ranged_step(dp.flat)
        dp.group.device_barrier()          # every rank's updates and republished weights are in place
        K._count(2)
