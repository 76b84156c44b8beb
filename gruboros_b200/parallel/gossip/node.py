"""Evolutionary gossip: a population of independently trained replicas that hold pairwise fitness
tournaments; the winner's weights (and optimizer state) flow to the loser and are merged there.

Public surface and semantics follow the reference's ``EvolutionaryTrainingNode``
(gossip/evolutionary_node.py:56-858): ``start_gossip_protocol``, ``update_fitness``, ``check_for_updates``,
``apply_pending_update`` -> (applied, needs_optimizer_reset), ``request_mix``, ``get_current_fitness``,
``get_status`` (initiated / received / won / lost / failed / successful mixes), ``stop_gossip_protocol``,
``attempt_rejuvenation``, ``.coordinator``, ``.node_lock_path``, ``.optimizer``; merge methods ``clonal`` and
``recombination`` with optimizer ``interpolate`` / ``reset``; the same TSV event log.

Two transports:

``nvlink``  (ranks of one NVSwitch domain; the B200 data plane)  Tournaments are synchronous rounds every
            ``gossip_every`` optimizer steps.  Only scalars cross the host: each rank's EMA loss and optimizer
            counters (one small all-gather).  Pairs come from a shared-seed shuffle, so no negotiation is
            needed.  The loser then launches ONE kernel that reads the winner's parameters, Schedule-Free z and
            second moments straight from the winner's memory (CUDA-IPC mapped peer pointers over NVLink) and
            blends them into its own buffers in the same pass, rewriting its bf16 weight mirror.  Peer-memory
            flag barriers (bounded waits) fence the read against the winner's next update.
``tcp``     (anything else: multi-node populations, CPU runs)  The reference's wire protocol: initiator
            connects to ``host:29501+local_rank``, sends ``EMA_LOSS:<ema>:CID:<id>``, the server answers
            ``SENDING_WEIGHTS`` / ``SEND_ME_WEIGHTS`` (server wins iff its EMA loss is strictly lower), the winner
            streams an 8-byte big-endian length plus a ``torch.save`` blob, the loser queues it and the main
            thread merges it at the next step boundary.  Snapshots are taken under ``training_lock`` so a
            sender never reads a half-updated model (the reference reads it unsynchronised).

``hybrid``  (several boxes)  Both at once, chosen per pair: ranks of the same box (``box_size`` consecutive global
            ranks, default ``LOCAL_WORLD_SIZE``) hold NVLink rounds among themselves, and the TCP protocol runs
            with the ranks of every other box (``transport_for(peer_rank)`` says which).  A rank whose box has no
            other member behaves like a ``tcp`` node.

Deviations from the reference, on purpose: optimizer interpolation really interpolates (the reference's is a
silent no-op because it compares integer state keys with Parameter keys) and includes Schedule-Free ``z``;
``alpha_mode='softmax'`` weights the blend by softmax(-loss) over the pair; ``compat=True`` restores the
reference's behaviour for parity tests.
"""
from __future__ import annotations

import glob
import io
import math
import os
import queue
import random
import re
import socket
import struct
import tempfile
import threading
import time
import uuid
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import torch

from ...utils.flat import lookup
from ...utils.locks import file_lock
from .coordinator import FilesystemCoordinator
from .fitness import FitnessTracker
from .logger import GossipLogger
from .network import NetworkUtils


@dataclass
class WeightUpdate:
    state_dict: dict
    optimizer_state_dict: Optional[dict]
    source_node: str
    source_ema_loss: float
    correlation_id: str


def pair_ranks(world: int, round_index: int, seed: int = 42) -> list[tuple[int, int]]:
    """Random perfect matching of the ranks for one tournament round; identical on every rank."""
    order = list(range(world))
    random.Random(seed * 1_000_003 + round_index).shuffle(order)
    return [(order[i], order[i + 1]) for i in range(0, world - 1, 2)]


def blend_alpha(mode: str, fixed_alpha: float, loser_loss: float, winner_loss: float) -> float:
    """Weight of the WINNER in the blend: fixed, or softmax(-loss) over the pair = sigmoid(loser - winner)."""
    if mode == "softmax":
        d = loser_loss - winner_loss
        if math.isinf(d) or math.isnan(d):
            return 1.0 if loser_loss > winner_loss else 0.5
        return 1.0 / (1.0 + math.exp(-d))
    return fixed_alpha


class EvolutionaryTrainingNode:
    def __init__(self, node_id, model, optimizer, global_rank, local_rank, world_size, data_parallel_rank=0,
                 tp_size=1, mixing_probability=0.01, output_dir=None, merge_method="clonal", recombination_alpha=0.5,
                 optimizer_recombination="reset", gossip_temp_dir=None, fitness_decay_factor=0.95,
                 use_node_local_lock=False, use_filesystem_coordinator=False, save_callback=None,
                 transport="tcp", gossip_every=0, alpha_mode="fixed", compat=False, peer_group=None,
                 host_group=None, pairing_seed=42, bootstrap_nodes=None, listen=True, box_size=None):
        self.node_id, self.model, self.optimizer = node_id, model, optimizer
        self.global_rank, self.local_rank, self.world_size = global_rank, local_rank, world_size
        self.data_parallel_rank, self.tp_size = data_parallel_rank, tp_size
        self.mixing_probability = mixing_probability
        self.merge_method, self.recombination_alpha = merge_method, recombination_alpha
        self.optimizer_recombination = optimizer_recombination
        self.use_node_local_lock, self.use_filesystem_coordinator = use_node_local_lock, use_filesystem_coordinator
        self.output_dir, self.save_callback = output_dir, save_callback
        self.transport, self.gossip_every = transport, int(gossip_every)
        self.alpha_mode, self.compat, self.pairing_seed = alpha_mode, compat, pairing_seed
        self.peer_group, self.host_group = peer_group, host_group
        self.listen = listen
        # the ranks that hold NVLink rounds together: everybody ("nvlink"), or this rank's box ("hybrid")
        if transport == "hybrid":
            bs = int(box_size or os.environ.get("LOCAL_WORLD_SIZE") or os.environ.get("RANKS_PER_NODE") or world_size)
            self.box_size = max(1, min(bs, world_size))
            first = (global_rank // self.box_size) * self.box_size
            self.nv_members = list(range(first, min(first + self.box_size, world_size)))
        else:
            self.box_size = world_size
            self.nv_members = list(range(world_size))
        self.nv_rank = self.nv_members.index(global_rank)
        self.uses_nvlink = transport == "nvlink" or (transport == "hybrid" and len(self.nv_members) > 1)
        self.uses_tcp = transport == "tcp" or transport == "hybrid"

        self.coordinator = None
        if use_filesystem_coordinator:
            self.coordinator = FilesystemCoordinator(global_rank, world_size, output_dir)
            self.coordinator.set_fitness_provider(self.get_current_fitness)
        self.mixing_rng = random.Random(42 + global_rank * 1000)
        self.incoming_updates: queue.Queue = queue.Queue()
        self.step_notifications: queue.Queue = queue.Queue(maxsize=1024)
        self.fitness_tracker = FitnessTracker(decay_factor=fitness_decay_factor)
        self.fitness_lock = threading.Lock()
        self.training_lock = threading.RLock()      # held by the training loop while it mutates the model
        self.pending_update: WeightUpdate | None = None
        self._last_round_result = (False, False)
        self.logger = GossipLogger(node_id, global_rank, local_rank, data_parallel_rank, output_dir)
        self.gossip_temp_dir = (gossip_temp_dir or os.environ.get("LUSTRE_SCRATCH") or os.environ.get("SCRATCH")
                                or tempfile.gettempdir())
        os.makedirs(self.gossip_temp_dir, exist_ok=True)
        self.gossip_port = NetworkUtils.get_gossip_port(local_rank)
        self.bootstrap_nodes = (list(bootstrap_nodes) if bootstrap_nodes is not None
                                else NetworkUtils.get_bootstrap_nodes(global_rank, local_rank))
        if transport == "hybrid" and bootstrap_nodes is None:
            # peers of this box are reached over NVLink: the TCP peer list keeps only the other hosts
            self.bootstrap_nodes = self.cross_box_peers(self.bootstrap_nodes, NetworkUtils.get_local_node_address())
        self.peer_list: dict = {}
        self.gossip_running = False
        self.gossip_thread = self.server_thread = None
        self.mixing_attempts = self.successful_mixes = self.current_step = 0
        self.outbound_mixes_attempted = self.inbound_mixes_attempted = 0
        self.mixes_won = self.mixes_lost = 0
        self.rounds = 0
        self._counter_lock = threading.Lock()
        if use_node_local_lock:
            self.node_lock_path = os.path.join(self.gossip_temp_dir, "gossip.node.lock")
            self.mixes_skipped_locked = 0
            if local_rank == 0:
                Path(self.node_lock_path).touch()
                self.logger.log_event("NODE_LOCK_INIT", message=f"Initialized lock file at {self.node_lock_path}")
            self.logger.log_event("NODE_LOCK_ENABLED", message=f"Lock file: {self.node_lock_path}")
        if self.uses_nvlink:
            self._setup_nvlink()
        self.logger.log_event("NODE_STARTUP", message=f"transport={transport}, mixing_prob={mixing_probability}, "
                                                      f"gossip_every={gossip_every}, merge={merge_method}")

    # ------------------------------------------------------------------ per-pair transport
    def transport_for(self, peer_rank: int) -> str:
        """Which data plane a tournament with global rank `peer_rank` uses: the fused NVLink pull inside this rank's
        box (when the node has peer memory set up), the TCP protocol otherwise."""
        return "nvlink" if self.uses_nvlink and peer_rank in self.nv_members and peer_rank != self.global_rank else "tcp"

    @staticmethod
    def cross_box_peers(addresses, my_host):
        """The ``host:port`` peers that are not on `my_host` (those are this box's ranks, served over NVLink)."""
        mine = {my_host, "localhost", "127.0.0.1"} if my_host else {"localhost", "127.0.0.1"}
        try:
            mine.add(socket.gethostname())
            mine.add(socket.gethostname().split(".")[0])
        except OSError:
            pass
        return [a for a in addresses if a.rsplit(":", 1)[0] not in mine]

    # ------------------------------------------------------------------ fitness / status
    def update_fitness(self, loss_value, step: int) -> None:
        with self.fitness_lock:
            self.fitness_tracker.update(float(loss_value))
        self.current_step = step
        if self.uses_tcp:
            try:
                self.step_notifications.put_nowait(step)
            except queue.Full:
                pass

    def get_current_fitness(self) -> float:
        with self.fitness_lock:
            return self.fitness_tracker.get_fitness()

    def request_mix(self) -> None:
        """Kept for API compatibility: mixing is driven by the worker thread (tcp) or by rounds (nvlink)."""

    def get_status(self) -> dict:
        out, inn, won, lost = self.outbound_mixes_attempted, self.inbound_mixes_attempted, self.mixes_won, self.mixes_lost
        status = {"node_id": self.node_id, "fitness": self.get_current_fitness(), "peer_count": len(self.peer_list),
                  "successful_mixes": self.successful_mixes, "current_step": self.current_step,
                  "initiated_mixes": out, "received_mixes": inn, "won_mixes": won, "lost_mixes": lost,
                  "failed_mixes": (out + inn) - (won + lost)}
        if self.use_node_local_lock:
            status["skipped_due_to_lock"] = self.mixes_skipped_locked
        return status

    def _bump(self, name: str, n: int = 1) -> None:
        with self._counter_lock:
            setattr(self, name, getattr(self, name) + n)

    # ------------------------------------------------------------------ thread control
    def start_gossip_protocol(self) -> None:
        if self.coordinator is not None:
            self.coordinator.start()
        self.gossip_running = True
        if self.uses_tcp:
            self.gossip_thread = threading.Thread(target=self._gossip_worker, daemon=True, name="gossip-worker")
            self.gossip_thread.start()
            if self.listen:
                self.server_thread = threading.Thread(target=self._server_loop, daemon=True, name="gossip-server")
                self.server_thread.start()
        self.logger.log_event("GOSSIP_PROTOCOL_STARTED", message=f"transport={self.transport}")

    def stop_gossip_protocol(self) -> None:
        if self.coordinator is not None:
            self.coordinator.stop()
        self.gossip_running = False
        for t in (self.gossip_thread, self.server_thread):
            if t is not None:
                t.join(timeout=5)
        self.logger.log_event("GOSSIP_PROTOCOL_STOPPED", message="Gossip protocol stopped.")

    # ------------------------------------------------------------------ main-thread hooks
    def check_for_updates(self):
        """Called right after an optimizer step.  tcp: pop one received update and stage it for the next step
        boundary.  nvlink: run a tournament round if this step closes a gossip interval."""
        if self.uses_nvlink:
            if self.gossip_every > 0 and (self.current_step + 1) % self.gossip_every == 0:
                self._last_round_result = self._nvlink_round()
            if not self.uses_tcp:
                return None
        try:
            update = self.incoming_updates.get_nowait()
        except queue.Empty:
            return None
        self.pending_update = update
        return update

    def apply_pending_update(self) -> tuple[bool, bool]:
        """Top of a training step: merge a staged update.  Returns (applied, needs_optimizer_reset)."""
        applied, needs_reset = False, False
        if self.uses_nvlink:
            (applied, needs_reset), self._last_round_result = self._last_round_result, (False, False)
            if not self.uses_tcp:
                return applied, needs_reset
        if self.pending_update is None:
            return applied, needs_reset
        upd, self.pending_update = self.pending_update, None
        with self.training_lock:
            needs_reset = self._merge_state_dicts(upd.state_dict, upd.optimizer_state_dict, upd.source_ema_loss) or needs_reset
        self.successful_mixes += 1
        return True, needs_reset

    # ------------------------------------------------------------------ merge (host tensors / generic path)
    def _merge_state_dicts(self, winner_model: dict, winner_opt: Optional[dict], winner_loss: float) -> bool:
        needs_reset = False
        if self.merge_method == "recombination":
            alpha = blend_alpha(self.alpha_mode, self.recombination_alpha, self.get_current_fitness(), winner_loss)
            with torch.no_grad():
                for name, p in self.model.named_parameters():
                    if name in winner_model and p.dtype.is_floating_point:
                        p.lerp_(winner_model[name].to(p.device, p.dtype), alpha)
                if self.optimizer_recombination == "interpolate" and winner_opt and not self.compat:
                    self._interpolate_optimizer(winner_opt, alpha)
                elif self.optimizer_recombination == "reset":
                    needs_reset = True
        else:
            self.model.load_state_dict(winner_model)
            if winner_opt:
                self.optimizer.load_state_dict(winner_opt)
            with self.fitness_lock:
                self.fitness_tracker.inherit_fitness(winner_loss)
        return needs_reset

    def _interpolate_optimizer(self, winner_opt: dict, alpha: float) -> None:
        """state[k] <- (1-alpha) state[k] + alpha winner[k] for every tensor state both sides have (Schedule-Free
        z and exp_avg_sq, or AdamW's exp_avg / exp_avg_sq).  Winner states are keyed by parameter index."""
        params = [p for g in self.optimizer.param_groups for p in g["params"]]
        for idx, wstate in winner_opt.get("state", {}).items():
            i = int(idx)
            if i >= len(params):
                continue
            mine = self.optimizer.state.get(params[i])
            if not mine:
                continue
            for key, wt in wstate.items():
                if torch.is_tensor(wt) and key in mine and torch.is_tensor(mine[key]) and mine[key].dtype.is_floating_point \
                        and mine[key].shape == wt.shape:
                    mine[key].lerp_(wt.to(mine[key].device, mine[key].dtype), alpha)

    # ------------------------------------------------------------------ nvlink transport
    def _setup_nvlink(self) -> None:
        """Parameters, gradients, bf16 mirror and optimizer state move into symmetric (IPC-mapped) buffers."""
        from ...utils.flat import FlatParams
        from ..comm import PeerGroup
        dev = next(self.model.parameters()).device
        if dev.type != "cuda":
            raise RuntimeError("the nvlink gossip transport needs the model on a CUDA device")
        if self.peer_group is None:
            if len(self.nv_members) == self.world_size:
                self.peer_group = PeerGroup(self.global_rank, self.world_size, dev)
            else:
                # hybrid: peer memory only among this box's ranks; handles travel over a process group of the box
                from ..comm import TorchDistTransport
                if self.host_group is None:
                    self.host_group = self._box_process_group()
                self.peer_group = PeerGroup(self.nv_rank, len(self.nv_members), dev,
                                            TorchDistTransport(self.nv_rank, len(self.nv_members), self.host_group))
        g = self.peer_group

        def allocator(name, numel, dtype):
            item = torch.empty(0, dtype=dtype).element_size()
            return g.alloc(f"gossip_{name}", numel * item).tensor(dtype, numel)

        saved_opt = self.optimizer.state_dict() if len(self.optimizer.state) else None
        flat = FlatParams(self.model, dev, allocator=allocator)
        flat.allocator = allocator
        self.flat = flat
        engine = self.model.fused_engine() if hasattr(self.model, "fused_engine") else None
        if engine is not None:
            engine.ensure_flat(dev)
        if saved_opt is not None:
            self.optimizer.load_state_dict(saved_opt)
        if hasattr(self.optimizer, "ensure_state"):
            self.optimizer.ensure_state()
        if hasattr(g.transport, "hub"):
            return      # single-process emulation: caller runs finish_nvlink_connect() once all ranks exist
        self.finish_nvlink_connect()

    def finish_nvlink_connect(self) -> None:
        g = self.peer_group
        if hasattr(g.transport, "hub"):
            g.finish_local_connect()
        self._y_ptrs = g.ptrs("gossip_data")
        self._z_ptrs = g.ptrs("gossip_sf_z") if "gossip_sf_z" in g._ptrs else None
        self._v_ptrs = g.ptrs("gossip_sf_v") if "gossip_sf_v" in g._ptrs else None

    def _box_process_group(self):
        """gloo group of this rank's box (collective over ALL ranks: every box's group is created in the same order)."""
        import torch.distributed as dist
        mine = None
        for first in range(0, self.world_size, self.box_size):
            ranks = list(range(first, min(first + self.box_size, self.world_size)))
            grp = dist.new_group(ranks=ranks, backend="gloo")
            if self.global_rank in ranks:
                mine = grp
        return mine

    def _host_allgather(self, payload):
        import torch.distributed as dist
        out = [None] * len(self.nv_members)
        dist.all_gather_object(out, payload, group=self.host_group)
        return out

    def _nvlink_round(self, board=None) -> tuple[bool, bool]:
        """One synchronous tournament round = begin (scalars, pairing, first barrier signal), transfer (wait, the
        loser's fused pull, second signal), end (wait, status).  The three phases are separate methods so that a
        single-process emulation can interleave several ranks without any kernel waiting on a later launch."""
        ctx = self._round_begin(board)
        if ctx is None:
            return False, False
        self._round_transfer(ctx)
        return self._round_end(ctx)

    def _round_begin(self, board=None):
        self.rounds += 1
        step, cid = self.current_step, f"r{self.rounds:07d}"
        group0 = self.optimizer.param_groups[0]
        mine = {"rank": self.global_rank, "fitness": self.get_current_fitness(),
                "k": group0.get("k", 0), "weight_sum": group0.get("weight_sum", 0.0), "lr_max": group0.get("lr_max", -1.0)}
        try:
            board = board if board is not None else self._host_allgather(mine)
        except Exception as exc:                      # a dead or late peer: the round is abandoned, training goes on
            self._bump("outbound_mixes_attempted")
            self.logger.log_event("MIX_ATTEMPT_FAILED", step=step, correlation_id=cid, message=f"fitness exchange: {exc}")
            return None
        # pairs are drawn among the ranks that share peer memory (positions in nv_members; the whole world unless hybrid)
        pairs = pair_ranks(len(self.nv_members), self.rounds, self.pairing_seed + self.nv_members[0])
        partner = next((b if a == self.nv_rank else a for a, b in pairs if self.nv_rank in (a, b)), None)
        ctx = {"board": board, "partner": partner, "cid": cid, "step": step, "applied": False, "needs_reset": False,
               "won": False}
        self.peer_group.signal_only()                 # my last update is complete (stream ordered)
        return ctx

    def _round_transfer(self, ctx) -> None:
        from ...ops import kernels as K
        g, partner, board, cid, step = self.peer_group, ctx["partner"], ctx["board"], ctx["cid"], ctx["step"]
        g.wait_only()                                 # ... and so is everybody else's
        if partner is not None:
            me_fit, pa_fit = board[self.nv_rank]["fitness"], board[partner]["fitness"]
            i_win = (me_fit, self.nv_rank) < (pa_fit, partner)
            initiator = min(self.nv_rank, partner) == self.nv_rank
            self._bump("outbound_mixes_attempted" if initiator else "inbound_mixes_attempted")
            self.logger.log_event("MIX_ATTEMPT_START" if initiator else "INCOMING_FITNESS_COMPARISON", step=step,
                                  fitness=me_fit, correlation_id=cid, peer_addr=f"rank{self.nv_members[partner]}",
                                  message=f"peer_fitness={pa_fit:.4f}")
            if math.isinf(me_fit) and math.isinf(pa_fit):
                pass                                  # nobody has a fitness yet: counted as a failed mix
            elif i_win:
                self._bump("mixes_won")
                ctx["won"] = True
            else:
                self._bump("mixes_lost")
                ctx["needs_reset"] = self._nvlink_pull(partner, board[partner], me_fit, pa_fit, cid, K)
                ctx["applied"] = True
        g.signal_only()                               # done reading my partner's memory

    def _round_end(self, ctx) -> tuple[bool, bool]:
        from ...ops import _lib as L
        g = self.peer_group
        g.wait_only()                                 # losers are done reading before winners train on
        torch.cuda.current_stream().synchronize()
        try:
            L.check_device_status(g.device)
        except RuntimeError as exc:
            self.logger.log_event("MIX_ATTEMPT_FAILED", step=ctx["step"], correlation_id=ctx["cid"], message=str(exc))
            if ctx["applied"]:
                self._bump("mixes_lost", -1)
            if ctx["won"]:
                self._bump("mixes_won", -1)
            return False, False
        self._flush_transfer_log()
        if ctx["applied"]:
            self.successful_mixes += 1
        elif ctx["won"] and self.save_callback:
            try:
                self.save_callback(ctx["step"], self.get_current_fitness(), opportunistic=True)
            except Exception as exc:
                self.logger.log_event("OPPORTUNISTIC_SAVE_FAILED", message=str(exc))
        return ctx["applied"], ctx["needs_reset"]

    def _nvlink_pull(self, winner: int, winner_info: dict, my_loss: float, winner_loss: float, cid: str, K) -> bool:
        """The fused transfer + merge: one kernel reads the winner's buffers over NVLink and blends into ours."""
        flat = self.flat
        n = flat.numel
        opt_flat = hasattr(flat, "sf_z") and self._z_ptrs is not None
        needs_reset = False
        if self.merge_method == "clonal":
            a_y = a_z = a_v = 1.0
        else:
            a_y = blend_alpha(self.alpha_mode, self.recombination_alpha, my_loss, winner_loss)
            interp = self.optimizer_recombination == "interpolate" and not self.compat
            a_z = a_v = a_y if interp else 0.0
            needs_reset = self.optimizer_recombination == "reset"
        pairs = [(flat.data, self._y_ptrs[winner], a_y)]
        if opt_flat and (a_z or a_v):
            pairs += [(flat.sf_z, self._z_ptrs[winner], a_z), (flat.sf_v, self._v_ptrs[winner], a_v)]
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        K.merge(pairs, flat.w16, n)
        t1.record()
        flat.w16_version = flat.version() + flat.data._version
        if self.merge_method == "clonal":
            for grp in self.optimizer.param_groups:
                for key in ("k", "weight_sum", "lr_max"):
                    if key in grp and key in winner_info:
                        grp[key] = winner_info[key]
            with self.fitness_lock:
                self.fitness_tracker.inherit_fitness(winner_loss)
        nbytes = 4 * n * len(pairs)
        self._pending_transfer_log = (t0, t1, nbytes, winner, winner_loss, cid)
        return needs_reset

    def _flush_transfer_log(self) -> None:
        pend, self._pending_transfer_log = getattr(self, "_pending_transfer_log", None), None
        if pend is None:
            return
        t0, t1, nbytes, winner, winner_loss, cid = pend
        t1.synchronize()
        ms = t0.elapsed_time(t1)
        self.logger.log_event("WEIGHT_RECEIVE_COMPLETE", step=self.current_step, correlation_id=cid,
                              peer_addr=f"rank{winner}", data_size_bytes=nbytes, transfer_time_ms=ms, fitness=winner_loss,
                              message=f"NVLink peer read fused with merge: {nbytes / 1e9 / max(ms, 1e-6) * 1e3:.1f} GB/s")
        self.last_transfer = {"bytes": nbytes, "ms": ms}

    # ------------------------------------------------------------------ tcp transport
    def _gossip_worker(self) -> None:
        time.sleep(float(os.environ.get("GOSSIP_STARTUP_DELAY", "2")))
        for addr in self.bootstrap_nodes:
            self.peer_list[addr] = {}
        self.logger.log_event("PEER_DISCOVERY", message=f"Found {len(self.peer_list)} peers: {list(self.peer_list)[:16]}")
        while self.gossip_running:
            try:
                try:
                    step = self.step_notifications.get(timeout=0.5)
                except queue.Empty:
                    continue
                self.current_step = step
                if self.mixing_rng.random() >= self.mixing_probability:
                    continue
                if self.use_node_local_lock:
                    try:
                        with file_lock(self.node_lock_path, timeout=0.05):
                            self.logger.log_event("MIX_DECISION_LOCKED", step=step, fitness=self.get_current_fitness(),
                                                  message="Acquired node lock, proceeding with mix.")
                            self._try_mix_with_peer()
                    except TimeoutError:
                        self.mixes_skipped_locked += 1
                        self.logger.log_event("MIX_ATTEMPT_SKIPPED", step=step, message="Node lock was busy, skipping mix attempt.")
                else:
                    self.logger.log_event("MIX_DECISION", step=step, fitness=self.get_current_fitness(),
                                          message="Attempting mix (locking disabled).")
                    self._try_mix_with_peer()
            except Exception as exc:
                self.logger.log_event("GOSSIP_WORKER_ERROR", message=str(exc))
                time.sleep(0.5)

    def _server_loop(self) -> None:
        srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.settimeout(0.5)
        try:
            NetworkUtils.optimize_socket(srv)
            srv.bind(("0.0.0.0", self.gossip_port))
            srv.listen(8)
            self.logger.log_event("SERVER_STARTED", message=f"Listening on {self.logger.node_identity}")
            while self.gossip_running:
                try:
                    conn, addr = srv.accept()
                except socket.timeout:
                    continue
                except OSError as exc:
                    if self.gossip_running:
                        self.logger.log_event("SERVER_ERROR", message=str(exc))
                        time.sleep(0.5)
                    continue
                threading.Thread(target=self._handle_incoming_request, args=(conn, addr), daemon=True).start()
        except OSError as exc:
            self.logger.log_event("SERVER_ERROR", message=str(exc))
        finally:
            srv.close()

    def _handle_incoming_request(self, conn, addr) -> None:
        peer, cid = f"{addr[0]}:{addr[1]}", None
        self._bump("inbound_mixes_attempted")
        try:
            NetworkUtils.optimize_socket(conn)
            conn.settimeout(5.0)
            msg = conn.recv(1024).decode()
            if not msg.startswith("EMA_LOSS:"):
                return
            parts = msg.split(":")
            peer_fitness = float(parts[1])
            cid = parts[3] if len(parts) >= 4 and parts[2] == "CID" else self.logger.generate_correlation_id()
            ours = self.get_current_fitness()
            self.logger.log_event("INCOMING_FITNESS_COMPARISON", step=self.current_step, fitness=ours,
                                  correlation_id=cid, peer_addr=peer, message=f"peer_fitness={peer_fitness:.4f}")
            conn.settimeout(120.0)
            if ours < peer_fitness:
                conn.send(b"SENDING_WEIGHTS")
                self._send_our_weights_to_peer(conn, cid)
                self._bump("mixes_won")
                self._opportunistic_save(ours)
            else:
                conn.send(b"SEND_ME_WEIGHTS")
                upd = self._receive_weights_from_peer(conn, cid, peer)
                if upd is not None:
                    self._bump("mixes_lost")
                    self.incoming_updates.put(upd)
                    self.logger.log_event("WEIGHT_UPDATE_QUEUED", step=self.current_step, correlation_id=cid,
                                          peer_addr=peer, fitness=upd.source_ema_loss)
        except Exception as exc:
            self.logger.log_event("INCOMING_REQUEST_ERROR", step=self.current_step, correlation_id=cid, peer_addr=peer,
                                  message=str(exc))
        finally:
            conn.close()

    def _try_mix_with_peer(self) -> None:
        me = self.logger.node_identity
        others = [p for p in self.peer_list if p != me]
        if not others:
            return
        self._bump("outbound_mixes_attempted")
        cid = self.logger.generate_correlation_id()
        peer = self.mixing_rng.choice(others)
        self.logger.log_event("MIX_ATTEMPT_START", step=self.current_step, correlation_id=cid, peer_addr=peer,
                              fitness=self.get_current_fitness())
        host, port = peer.rsplit(":", 1)
        sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        try:
            NetworkUtils.optimize_socket(sock)
            sock.settimeout(3.0)
            sock.connect((host, int(port)))
            ours = self.get_current_fitness()
            sock.send(f"EMA_LOSS:{ours:.6f}:CID:{cid}".encode())
            sock.settimeout(2.0)
            reply = sock.recv(1024)
            sock.settimeout(120.0)
            if reply == b"SENDING_WEIGHTS":
                upd = self._receive_weights_from_peer(sock, cid, peer)
                if upd is not None:
                    self._bump("mixes_lost")
                    self.incoming_updates.put(upd)
            elif reply == b"SEND_ME_WEIGHTS":
                self._send_our_weights_to_peer(sock, cid)
                self._bump("mixes_won")
                self._opportunistic_save(ours)
            else:
                raise ConnectionError(f"unexpected handshake reply {reply!r}")
            self.mixing_attempts += 1
        except Exception as exc:
            self.logger.log_event("MIX_ATTEMPT_FAILED", step=self.current_step, correlation_id=cid, peer_addr=peer,
                                  message=str(exc))
        finally:
            sock.close()

    def _opportunistic_save(self, fitness: float) -> None:
        if self.save_callback:
            try:
                self.save_callback(self.current_step, fitness, opportunistic=True)
            except Exception as exc:
                self.logger.log_event("OPPORTUNISTIC_SAVE_FAILED", message=str(exc))

    def _snapshot(self) -> dict:
        """CPU copy of model + optimizer state taken while the training loop is between steps."""
        with self.training_lock:
            model_sd = {k: v.detach().cpu().clone() for k, v in self.model.state_dict().items()}
            osd = self.optimizer.state_dict()
            opt_sd = {"state": {i: {k: (t.detach().cpu().clone() if torch.is_tensor(t) else t) for k, t in st.items()}
                                for i, st in osd["state"].items()}, "param_groups": osd["param_groups"]}
        return {"model_state_dict": model_sd, "optimizer_state_dict": opt_sd}

    def _send_our_weights_to_peer(self, sock, cid: str) -> None:
        t0 = time.time()
        path = os.path.join(self.gossip_temp_dir, f"gossip_payload_{uuid.uuid4()}.pt")
        try:
            payload = self._snapshot()
            ours = self.get_current_fitness()
            payload.update(ema_loss=ours, correlation_id=cid)
            torch.save(payload, path)
            size = os.path.getsize(path)
            sock.sendall(struct.pack("!Q", size))
            with open(path, "rb") as f:
                while True:
                    chunk = f.read(4 << 20)
                    if not chunk:
                        break
                    sock.sendall(chunk)
            ms = (time.time() - t0) * 1e3
            self.logger.log_event("WEIGHT_SEND_COMPLETE", step=self.current_step, correlation_id=cid, data_size_bytes=size,
                                  transfer_time_ms=ms, fitness=ours, message=f"Throughput: {size / 1e6 / max(ms / 1e3, 1e-9):.2f} MB/s")
        except Exception as exc:
            self.logger.log_event("WEIGHT_SEND_ERROR", step=self.current_step, correlation_id=cid, message=str(exc))
            raise
        finally:
            self._remove_temp(path)

    def _receive_weights_from_peer(self, sock, cid: str, peer: str):
        t0 = time.time()
        path = os.path.join(self.gossip_temp_dir, f"gossip_payload_{uuid.uuid4()}.pt")
        try:
            head = b""
            while len(head) < 8:
                chunk = sock.recv(8 - len(head))
                if not chunk:
                    raise ConnectionError("connection closed before the payload length arrived")
                head += chunk
            size = struct.unpack("!Q", head)[0]
            got = 0
            with open(path, "wb") as f:
                while got < size:
                    chunk = sock.recv(min(4 << 20, size - got))
                    if not chunk:
                        raise ConnectionError("connection broke while receiving the weight payload")
                    f.write(chunk)
                    got += len(chunk)
            data = torch.load(path, map_location="cpu", weights_only=False)
            ms = (time.time() - t0) * 1e3
            loss = data.get("ema_loss", math.inf)
            self.logger.log_event("WEIGHT_RECEIVE_COMPLETE", step=self.current_step, correlation_id=cid, data_size_bytes=size,
                                  transfer_time_ms=ms, fitness=loss, message=f"Throughput: {size / 1e6 / max(ms / 1e3, 1e-9):.2f} MB/s")
            return WeightUpdate(data.get("model_state_dict"), data.get("optimizer_state_dict"), peer, loss, cid)
        except Exception as exc:
            self.logger.log_event("WEIGHT_RECEIVE_ERROR", step=self.current_step, correlation_id=cid, message=str(exc))
            return None
        finally:
            self._remove_temp(path)

    def _remove_temp(self, path: str) -> None:
        try:
            if os.path.exists(path):
                os.remove(path)
        except OSError as exc:
            self.logger.log_event("TEMP_FILE_CLEANUP_ERROR", message=f"Failed to remove {path}: {exc}")

    # ------------------------------------------------------------------ rejuvenation
    def attempt_rejuvenation(self, model, alpha: float, tiebreaker_threshold: float = 0.005) -> tuple[bool, bool]:
        """Blend a strictly better elite checkpoint into `model`.  Among the ``elite_*.pt`` links, a candidate
        replaces the current choice if it is better by more than `tiebreaker_threshold` (relative), or marginally
        better and trained for more steps.  Returns (rejuvenated, needs_optimizer_reset)."""
        mine = self.get_current_fitness()
        if math.isinf(mine) or not self.output_dir:
            return False, False
        best_fit, best_step, chosen = mine, -1, None
        for link in glob.glob(os.path.join(self.output_dir, "elite_*.pt")):
            try:
                target = os.path.basename(os.readlink(link))
                lm, sm = re.search(r"loss_([\d.inf]+)\.pt", target), re.search(r"step_(\d+)", target)
                if not lm or not sm:
                    continue
                fit, stp = float(lm.group(1)), int(sm.group(1))
            except (OSError, ValueError):
                continue
            if fit >= mine:
                continue
            if fit < best_fit * (1.0 - tiebreaker_threshold) or (fit < best_fit and stp > best_step):
                best_fit, best_step, chosen = fit, stp, link
        if chosen is None:
            self.logger.log_event("REJUVENATION_SKIPPED", step=self.current_step, fitness=mine,
                                  message=f"No elite model found with fitness < {mine:.4f}")
            return False, False
        try:
            ckpt = torch.load(chosen, map_location="cpu", weights_only=False)
            elite = ckpt["model_state_dict"]
            with self.training_lock, torch.no_grad():
                for name, p in model.named_parameters():
                    if name in elite:
                        p.lerp_(elite[name].to(p.device, p.dtype), alpha)
            if "ema_fitness" in ckpt:
                with self.fitness_lock:
                    self.fitness_tracker.inherit_fitness(ckpt["ema_fitness"])
            self.logger.log_event("REJUVENATION_SUCCESS", step=self.current_step, fitness=ckpt.get("ema_fitness"),
                                  message=f"Blended with {os.path.basename(chosen)} (L:{best_fit:.4f} S:{best_step})")
            return True, True
        except Exception as exc:
            self.logger.log_event("REJUVENATION_FAILED", step=self.current_step, message=str(exc))
            return False, False
