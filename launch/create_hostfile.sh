#!/bin/bash
# Writes hostfile-job<ID>.txt ("host slots=8" per node) from the SLURM node list; the TCP gossip transport reads it
# for peer discovery when scontrol is not available on the compute nodes.
set -euo pipefail
ID=${SLURM_JOB_ID:-local}
OUT=hostfile-job${ID}.txt
if [ -n "${SLURM_JOB_NODELIST:-}" ]; then
  scontrol show hostnames "$SLURM_JOB_NODELIST" | awk -v s="${RANKS_PER_NODE:-8}" '{print $1" slots="s}' > "$OUT"
else
  echo "localhost slots=${RANKS_PER_NODE:-8}" > "$OUT"
fi
echo "wrote $OUT"; cat "$OUT"
