"""``train.py`` driver: distributed set-up, model / optimizer construction or resume, data, gossip or
data-parallel wiring, the TBPTT loop with metrics and probabilistic checkpointing.

Behaviour follows the reference's ``main()`` (train.py:497-858): ranks from RANK/LOCAL_RANK/WORLD_SIZE (or the
SLURM equivalents); identical initial weights on every rank (torch seed 42) with per-rank data and mixing RNG
(python seed 42+rank); one loop iteration = one chunk; hidden state carried across the ``context_chunks`` chunks
of a sequence and reset with each new sequence; optimizer step every ``grad_accum`` chunks; gossip hooks around
the step; one metrics row per chunk-step; checkpoint with probability 1/(save_every*world) per step (x5 for
tournament winners, scaled by fitness percentile when asked).  Differences: output directories are created here;
losses are read back every ``--log_every`` steps instead of every step (rows still carry per-step values);
``--final_checkpoint`` adds a save at exit; ``--parallel dp`` trains one model data-parallel instead of a population.
"""
from __future__ import annotations

import datetime
import json
import os
import random
import time
from datetime import timedelta

import numpy as np
import torch
import torch.distributed as dist

from ..models.minlm import minLM
from ..optim.schedulefree import AdamWScheduleFree
from ..parallel.gossip import EvolutionaryTrainingNode
from ..utils.locks import file_lock
from ..utils.sizes import get_parameter_count_str, parse_size_with_suffix, resolve_model_config
from ..utils.files import read_last_line
from .checkpoint import CheckpointManager, build_checkpoint, load_checkpoint, save_checkpoint_atomic
from .data import ContinuousIIDDataset, SequenceLoader, ZipfBytes
from .flags import get_args
from .metrics import DeviceTimer, MetricsLogger
from .trainer import Trainer
from ..ops import _lib as L

SEED = 42


def dist_env():
    e = os.environ
    return (int(e.get("RANK", e.get("SLURM_PROCID", "0"))), int(e.get("LOCAL_RANK", e.get("SLURM_LOCALID", "0"))),
            int(e.get("WORLD_SIZE", e.get("SLURM_NPROCS", "1"))))


def pick_device(local_rank: int):
    if torch.cuda.is_available():
        idx = 0 if torch.cuda.device_count() == 1 else local_rank
        dev = torch.device("cuda", idx)
        torch.cuda.set_device(dev)
        return dev
    return torch.device("cpu")


def make_optimizer(args, model):
    if args.schedulefree:
        return AdamWScheduleFree(model.parameters(), lr=args.lr, betas=(args.sf_beta, args.sf_beta2), weight_decay=args.weight_decay)
    return torch.optim.AdamW(model.parameters(), lr=args.lr, betas=(args.sf_beta, args.sf_beta2), weight_decay=args.weight_decay)


def require_cuda_for(mode: str, device) -> None:
    """Data-parallel and sharded training run over NVLink peer memory; without CUDA devices the ranks would silently
    train unrelated replicas, so refuse instead (a CPU population is what ``--parallel gossip`` over TCP is for)."""
    if mode in ("dp", "fsdp") and torch.device(device).type != "cuda":
        raise SystemExit(f"--parallel {mode} needs one CUDA device per rank; on CPU use --parallel gossip")


def main(argv=None):
    args = get_args(argv)
    rank, local_rank, world = dist_env()
    device = pick_device(local_rank)
    own_group = world > 1 and not dist.is_initialized()
    if own_group:
        # host control plane only (rendezvous, IPC-handle and fitness-scalar exchange): gloo, like the reference
        dist.init_process_group(backend="gloo", timeout=timedelta(seconds=7200))
    random.seed(SEED + rank)
    np.random.seed(SEED)
    torch.manual_seed(SEED)

    train_steps = int(parse_size_with_suffix(args.train_steps))
    chunk_size = int(parse_size_with_suffix(args.chunk_size))
    batch_size = int(parse_size_with_suffix(args.batch_size))
    batches_per_epoch = int(parse_size_with_suffix(args.batches_per_epoch))

    out_dir = args.output or datetime.datetime.now().strftime("%Y%m%d_%H%M%S")
    if args.resume:
        out_dir = os.path.dirname(args.resume) if os.path.isfile(args.resume) else args.resume
    if rank == 0:
        for sub in ("", "metrics", "gossip", "fitness"):
            os.makedirs(os.path.join(out_dir, sub), exist_ok=True)
    if world > 1:
        dist.barrier()

    manager = CheckpointManager(out_dir, keep_last_n=args.keep_checkpoints, keep_elite_n=args.keep_elite,
                                global_rank=rank, archive_rate=args.archive_rate)
    manager.start()

    model_config, ckpt, step0 = None, None, 0
    if args.resume:
        path = args.resume if os.path.isfile(args.resume) else os.path.join(args.resume, "latest.pt")
        if os.path.exists(path):
            ckpt = load_checkpoint(path)
            model_config, step0 = ckpt.get("model_config"), ckpt.get("step", 0)
            if rank == 0:
                print(f"Loading checkpoint from {path} (step {step0})")
                last = read_last_line(os.path.join(out_dir, "metrics", f"training_metrics_rank_{rank:03d}.tsv"))
                if last:
                    print(f"Last metrics row of the run being resumed: {last}")
    if model_config is None:
        model_config = resolve_model_config(args.params, args.dim, args.depth, args.expansion_factor, args.ff_mult)
    if rank == 0:
        print(f"Model size: {get_parameter_count_str(model_config)} parameters\nConfiguration: {model_config}")
        with open(os.path.join(out_dir, "config.json"), "w") as f:
            json.dump(model_config, f, indent=2)

    model = minLM(**model_config).to(device)
    model.use_fused = args.fused
    if ckpt is not None:
        # before any wrapper takes the parameters over (the sharded mode keeps only this rank's share of them)
        model.load_state_dict(ckpt["model_state_dict"])
    mode = args.parallel if world > 1 else ("none" if args.parallel in ("dp", "fsdp") else args.parallel)
    parallel = None
    require_cuda_for(mode, device)
    if mode in ("dp", "fsdp") and not args.schedulefree:
        raise SystemExit(f"--parallel {mode} shards the Schedule-Free AdamW step over the ranks; it cannot be combined "
                         "with --no-schedulefree")
    if mode in ("dp", "fsdp") and device.type == "cuda":
        if mode == "fsdp":
            from ..parallel.fsdp import FullyShardedDataParallel as Par
        else:
            from ..parallel.dp import DataParallel as Par
        parallel = Par(model, rank=rank, world=world, device=device)
    optimizer = make_optimizer(args, model)
    if ckpt is not None and parallel is None:
        optimizer.load_state_dict(ckpt["optimizer_state_dict"])
    if parallel is not None:
        parallel.bind_optimizer(optimizer)
        if ckpt is not None:        # every rank takes its share of the saved per-parameter state
            parallel.load_optimizer_state_dict(ckpt["optimizer_state_dict"])
    if args.schedulefree:
        optimizer.train()

    total_len = chunk_size * args.context_chunks
    if args.synthetic:
        kind, _, s = args.synthetic.partition(":")
        if kind != "zipf":
            raise SystemExit(f"unknown synthetic source {args.synthetic!r}")
        source = ZipfBytes(total_len, s=float(s or 1.1), seed=SEED + rank)
    else:
        source = ContinuousIIDDataset(args.data, chunk_size, args.context_chunks, seed=SEED + rank,
                                      samples_per_epoch=batches_per_epoch * batch_size, batch_size=batch_size,
                                      global_rank=rank, dtype=torch.uint8)
    loader = SequenceLoader(source, batch_size, device=device if device.type == "cuda" else None)

    metrics = MetricsLogger(out_dir, rank, batch_size, chunk_size, with_lock_column=args.use_gossip_lock, flush_every=args.log_every)
    timer = DeviceTimer(batch_size * chunk_size, enabled=device.type == "cuda")

    pop = world if mode == "gossip" else 1
    base_p = (1.0 / (args.save_every * pop)) if args.save_every > 0 else 0.0
    save_probability = base_p * (4.5 if args.use_gossip_lock else 1.0)
    saver_rank = mode == "gossip" or rank == 0

    def device_ok() -> bool:
        """False (after reporting) if a bounded device-side wait gave up since the last check: gradients or weights
        of the steps since then are incomplete, so nothing derived from them may be saved or trained on."""
        if device.type != "cuda":
            return True
        try:
            L.check_device_status(device)
            return True
        except RuntimeError as e:
            print(f"[rank {rank}] {e}", flush=True)
            return False

    def save_now(step, fitness):
        if not device_ok():
            raise RuntimeError("refusing to write a checkpoint: a device-side wait timed out (a peer stalled or left)")
        opt_sd = None
        if parallel is not None:
            parallel.gather_params(materialize=saver_rank)
            opt_sd = parallel.optimizer_state_dict(materialize=saver_rank)     # collective; reference layout
        data = build_checkpoint(step, model, optimizer, fitness, model_config) if saver_rank else None
        if data is not None and opt_sd is not None:
            data["optimizer_state_dict"] = opt_sd
        ok = save_checkpoint_atomic(data, out_dir, step, rank, fitness) if saver_rank else False
        if parallel is not None:
            parallel.release_params()
        return ok

    def save_callback(step, fitness, opportunistic=False):
        p = save_probability * (5.0 if opportunistic else 1.0)
        if parallel is None and random.random() < p:
            return save_now(step, fitness)
        return False

    transport = args.gossip_transport
    if transport == "auto":
        # one box: NVLink rounds; several boxes with several GPUs each: NVLink inside a box and TCP across ("hybrid")
        local_world = int(os.environ.get("LOCAL_WORLD_SIZE", world))
        if mode == "gossip" and world > 1 and device.type == "cuda" and local_world == world:
            transport = "nvlink"
        elif mode == "gossip" and world > 1 and device.type == "cuda" and 1 < local_world < world:
            transport = "hybrid"
        else:
            transport = "tcp"
    gossip_every = args.gossip_every or (max(1, round(1.0 / args.gossip_mixing_rate)) if args.gossip_mixing_rate > 0 else 0)
    node = EvolutionaryTrainingNode(
        node_id=f"node_{rank}", model=model, optimizer=optimizer, global_rank=rank, local_rank=local_rank,
        world_size=world, data_parallel_rank=rank, tp_size=1,
        mixing_probability=args.gossip_mixing_rate if mode == "gossip" else 0.0, output_dir=out_dir,
        merge_method=args.gossip_merge_method, recombination_alpha=args.gossip_recombination_alpha,
        optimizer_recombination=args.gossip_optimizer_recombination, gossip_temp_dir=args.gossip_temp_dir,
        fitness_decay_factor=args.gossip_fitness_decay, use_node_local_lock=args.use_gossip_lock,
        use_filesystem_coordinator=args.filesystem_coordinator, save_callback=save_callback,
        transport=transport if mode == "gossip" else "tcp", gossip_every=gossip_every if mode == "gossip" else 0,
        alpha_mode=args.gossip_alpha_mode, compat=args.gossip_compat, listen=(mode == "gossip" and world > 1))
    node.start_gossip_protocol()
    if rank == 0:
        print(f"parallel={mode} gossip_transport={node.transport} device={device} chunk={chunk_size} x{args.context_chunks} "
              f"batch={batch_size} grad_accum={args.grad_accum}")

    trainer = Trainer(model, optimizer, chunk_size=chunk_size, grad_accum=args.grad_accum, parallel=parallel)
    step = step0
    pending = []          # (step, loss tensor) not yet read back
    long_batch = None
    last_loss = float("nan")
    timer.begin()
    t_start = time.time()
    bar = None
    if rank == 0 and args.progress != "off":       # the reference's tqdm bar (train.py:825-830)
        try:
            import sys
            from tqdm import tqdm
            if args.progress == "on" or sys.stderr.isatty():
                bar = tqdm(total=train_steps, initial=step0, desc="Training", dynamic_ncols=True)
        except ImportError:
            bar = None
    try:
        while step < train_steps:
            with node.training_lock:
                applied, needs_reset = node.apply_pending_update()
                if needs_reset:
                    optimizer = make_optimizer(args, model)
                    if parallel is not None:
                        parallel.bind_optimizer(optimizer)
                    if args.schedulefree:
                        optimizer.train()
                    node.optimizer = trainer.optimizer = optimizer
                    optimizer.zero_grad()
                if args.rejuvenation and node.coordinator is not None and random.random() < args.rejuvenation_probability:
                    pct = node.coordinator.get_my_percentile()
                    if pct is not None and pct >= args.rejuvenation_threshold:
                        node.attempt_rejuvenation(model, args.gossip_recombination_alpha, args.rejuvenation_tiebreaker_threshold)
                if step % args.context_chunks == 0:
                    long_batch = next(loader)
                    trainer.reset_hidden()
                c = step % args.context_chunks
                chunk = long_batch[:, c * chunk_size:(c + 1) * chunk_size]
                loss = trainer.step_chunk(chunk)
            pending.append((step, loss))
            timer.step()
            boundary = (step + 1) % args.grad_accum == 0
            sync_now = len(pending) >= args.log_every or (boundary and mode == "gossip" and node.uses_nvlink
                                                          and node.gossip_every and (step + 1) % node.gossip_every == 0)
            if sync_now or step + 1 >= train_steps:
                vals = torch.stack([l for _, l in pending]).float().cpu().tolist()
                if not device_ok():      # the host is synchronised here anyway
                    raise RuntimeError("training aborted: a device-side wait timed out (a peer stalled or left); "
                                       "resume from the last checkpoint")
                for (s, _), v in zip(pending, vals):
                    node.update_fitness(v, s)
                    metrics.log(s, v, node.get_current_fitness(), optimizer.param_groups[0]["lr"], node.get_status())
                last_loss = vals[-1]
                pending.clear()
            if boundary:
                with node.training_lock:
                    node.current_step = step
                    node.check_for_updates()
                node.request_mix()
            fitness = node.get_current_fitness()
            if step > 0 and save_probability > 0 and parallel is None:
                p = save_probability
                if args.fitness_weighted_checkpointing and node.coordinator is not None:
                    pct = node.coordinator.get_my_percentile()
                    if pct is not None:
                        p *= 1.0 + (args.elite_checkpoint_multiplier - 1.0) * (1.0 - pct)
                if random.random() < p:
                    if args.use_gossip_lock:
                        try:
                            with file_lock(node.node_lock_path, timeout=0.01):
                                save_now(step, fitness)
                        except TimeoutError:
                            pass
                    else:
                        save_now(step, fitness)
            elif parallel is not None and args.save_every > 0 and step > 0 and step % args.save_every == 0:
                save_now(step, fitness)
            if rank == 0 and (step % max(1, args.log_every) == 0 or step + 1 == train_steps):
                rate = timer.bytes_per_sec()
                shown = f"{last_loss:.4f}" if last_loss == last_loss else "(pending)"
                if bar is not None:
                    bar.set_postfix(loss=shown, ema=f"{fitness:.4f}", mixes=node.successful_mixes,
                                    kBps=f"{rate / 1e3:.1f}" if rate else "-")
                else:
                    print(f"step {step} loss {shown} ema {fitness:.4f} mixes {node.successful_mixes}"
                          + (f" device {rate / 1e3:.1f} kB/s" if rate else ""), flush=True)
            if bar is not None:
                bar.update(1)
            step += 1
        if args.final_checkpoint:
            save_now(step, node.get_current_fitness())
    finally:
        if bar is not None:
            bar.close()
        metrics.close()
        node.stop_gossip_protocol()
        loader.close()
        manager.run_once() if manager.active else None
        manager.stop()
    if rank == 0:
        print(f"\nTraining complete: {step - step0} steps in {time.time() - t_start:.1f}s.")
    if world > 1 and dist.is_initialized():
        dist.barrier()
        if own_group:
            # joins the process group's helper threads; a rank that exits with them running can abort in their
            # destructors once its peers have closed their sockets
            dist.destroy_process_group()
    return 0
