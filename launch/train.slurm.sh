#!/bin/bash
#SBATCH --job-name=gruboros-b200
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=8
#SBATCH --gpus-per-node=8
#SBATCH --time=24:00:00
# Multi-node population: one task per GPU via srun (train.py reads SLURM_PROCID / SLURM_LOCALID / SLURM_NPROCS).
# Within a node tournaments use NVLink peer memory when all ranks share one NVSwitch domain; across nodes the TCP
# transport is used (peers come from SLURM_JOB_NODELIST).  A rank that dies does not take the job down
# (--no-kill, death log), as in the reference's Frontier script.
set -uo pipefail
DATA=${DATA:?set DATA to the corpus file}
OUT=${OUT:-runs/$SLURM_JOB_ID}
mkdir -p "$OUT"
export RANKS_PER_NODE=8
export MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n1) MASTER_PORT=29500
srun --no-kill --kill-on-bad-exit=0 bash -c "
  python $(dirname "$0")/../train.py --data $DATA --output $OUT --parallel gossip --gossip_transport tcp \
    --params 1g --dim 1024 --expansion_factor 3.0 --ff_mult 1.5 --chunk_size 2048 --context_chunks 8 \
    --batch_size 1 --grad_accum 8 --lr 1e-3 --sf_beta2 0.995 --weight_decay 1e-4 \
    --gossip_recombination_alpha 0.3 --gossip_mixing_rate 0.002 --filesystem-coordinator ${EXTRA:-} \
  || { echo \"\$(date) rank \$SLURM_PROCID on \$(hostname) exited with \$?\" >> $OUT/deaths.log; sleep infinity; }"
