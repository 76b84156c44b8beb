"""Command-line flags of ``train.py``.

Every flag of the reference CLI is accepted with the same name and default (train.py:436-495); the flags after
the "B200 additions" comment are new.  ``--cuda`` / ``--rocm`` stay accepted for launch-script compatibility but
are optional: the device is picked from what is present, and there is a single (CUDA, sm_100a) kernel path.
"""
from __future__ import annotations

import argparse


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Evolutionary / data-parallel training of a byte-level minGRU language model")
    a = p.add_argument
    a("--local_rank", type=int, default=-1, help="local rank from launcher")
    a("--train_steps", type=str, default="100k", help="number of training steps (chunk-steps)")
    a("--data", type=str, default=None, help="path to the training corpus (raw bytes); or use --synthetic")
    a("--output", type=str, default=None, help="directory for checkpoints, metrics and logs")
    a("--resume", type=str, default=None, help="checkpoint file or directory to resume from")
    a("--save_every", type=int, default=2000, help="target average interval (steps) between checkpoints across the population")
    a("--batches_per_epoch", type=str, default="100")
    a("--params", type=str, default="100m", help="target parameter count (e.g. 15m, 1g)")
    a("--dim", type=str, default=None)
    a("--depth", type=int, default=None)
    a("--expansion_factor", type=float, default=1.5)
    a("--ff_mult", type=float, default=4.0)
    a("--chunk_size", type=str, default="2k", help="bytes per TBPTT chunk")
    a("--context_chunks", type=int, default=1, help="consecutive chunks that carry hidden state")
    a("--batch_size", type=str, default="4", help="sequences per GPU")
    a("--lr", type=float, default=1e-3)
    a("--weight_decay", type=float, default=0.01)
    a("--grad_accum", type=int, default=1)
    a("--keep_checkpoints", type=int, default=3)
    a("--keep_elite", type=int, default=10)
    a("--archive_rate", type=float, default=0.0)
    a("--no-schedulefree", dest="schedulefree", action="store_false", default=True)
    a("--sf_beta", type=float, default=0.9)
    a("--sf_beta2", type=float, default=0.999)
    a("--gossip_merge_method", type=str, default="recombination", choices=["clonal", "recombination"])
    a("--gossip_recombination_alpha", type=float, default=0.5)
    a("--gossip_optimizer_recombination", type=str, default="interpolate", choices=["reset", "interpolate"])
    a("--gossip_mixing_rate", type=float, default=0.01)
    a("--gossip_temp_dir", type=str, default=None)
    a("--gossip_fitness_decay", type=float, default=0.995)
    a("--gossip-node-local-lock", dest="use_gossip_lock", action="store_true", default=False)
    a("--filesystem-coordinator", action="store_true")
    a("--rejuvenation-probability", type=float, default=0.001)
    a("--rejuvenation-threshold", type=float, default=0.75)
    a("--fitness-weighted-checkpointing", action="store_true")
    a("--elite-checkpoint-multiplier", type=float, default=4.0)
    a("--rejuvenation-tiebreaker-threshold", type=float, default=0.005)
    g = p.add_mutually_exclusive_group(required=False)
    g.add_argument("--cuda", action="store_true")
    g.add_argument("--rocm", action="store_true")
    # ---- B200 additions
    a("--parallel", choices=["gossip", "dp", "fsdp", "none"], default="gossip",
      help="gossip: independent replicas with tournaments (the reference's mode); dp: data parallel with the "
           "gradient reduce-scatter fused into backward; fsdp: parameters sharded too")
    a("--gossip_transport", choices=["auto", "nvlink", "tcp", "hybrid"], default="auto",
      help="nvlink: in-box peer-memory transfer fused with the merge; tcp: the reference's socket protocol")
    a("--gossip_every", type=int, default=0, help="nvlink transport: tournament round every N optimizer steps "
                                                   "(0: derive from --gossip_mixing_rate as round(1/rate))")
    a("--gossip_alpha_mode", choices=["fixed", "softmax"], default="fixed",
      help="recombination weight of the winner: --gossip_recombination_alpha, or softmax(-loss) over the pair")
    a("--gossip_compat", action="store_true", help="reproduce the reference's optimizer-interpolation no-op")
    a("--rejuvenation", action="store_true", help="enable elite-checkpoint rejuvenation (flags above)")
    a("--synthetic", type=str, default=None, help="synthetic data instead of --data, e.g. zipf:1.1")
    a("--final_checkpoint", action="store_true", help="always write a checkpoint when training ends")
    a("--progress", choices=["auto", "on", "off"], default="auto",
      help="tqdm progress bar on rank 0 like the reference's (auto: only when stderr is a terminal; otherwise one line per --log_every steps)")
    a("--no-fused", dest="fused", action="store_false", default=True, help="force the plain PyTorch module path")
    a("--log_every", type=int, default=20, help="flush metrics / read losses back every N steps")
    return p


def get_args(argv=None):
    args = build_parser().parse_args(argv)
    if args.data is None and args.synthetic is None:
        raise SystemExit("train.py: one of --data or --synthetic is required")
    return args
