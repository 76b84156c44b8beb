#!/bin/bash
# Single-node 8 x B200 launch: one rank per GPU with torchrun (the reference's train.cuda.sh used the DeepSpeed
# launcher for the same purpose).  The production recipe of the reference is kept: dim 1024, expansion 3.0,
# ff_mult 1.5, ~1G parameters, lr 1e-3, betas (0.9, 0.995), wd 1e-4, chunk 2048 x 8 chunks, batch 1, accum 8.
#
#   launch/train.b200.sh DATA_FILE [OUTPUT_DIR] [extra train.py flags...]
#   PARALLEL=dp launch/train.b200.sh ...      # data parallel instead of the evolutionary population
set -euo pipefail
DATA=${1:?usage: train.b200.sh DATA_FILE [OUTPUT_DIR] [flags]}
OUT=${2:-runs/$(date +%Y%m%d_%H%M%S)}
shift $(( $# > 1 ? 2 : 1 ))
NGPU=${NGPU:-$(nvidia-smi -L | wc -l)}
PARALLEL=${PARALLEL:-gossip}
mkdir -p "$OUT"
export RANKS_PER_NODE=$NGPU MASTER_ADDR=${MASTER_ADDR:-127.0.0.1} MASTER_PORT=${MASTER_PORT:-29500}
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" \
  --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" \
  "$(dirname "$0")/../train.py" \
  --data "$DATA" --output "$OUT" --parallel "$PARALLEL" \
  --train_steps 100k --save_every 500 --keep_checkpoints 5 --keep_elite 10 \
  --dim 1024 --expansion_factor 3.0 --ff_mult 1.5 --params 1g \
  --chunk_size 2048 --context_chunks 8 --batch_size 1 --grad_accum 8 \
  --lr 1e-3 --sf_beta 0.9 --sf_beta2 0.995 --weight_decay 1e-4 \
  --gossip_merge_method recombination --gossip_recombination_alpha 0.3 \
  --gossip_optimizer_recombination interpolate --gossip_mixing_rate 0.002 --gossip_fitness_decay 0.995 \
  --filesystem-coordinator --fitness-weighted-checkpointing "$@"
