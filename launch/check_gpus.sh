#!/bin/bash
# Environment dump before a run: GPUs, NVLink topology, distributed variables (reading only; changes nothing).
echo "host: $(hostname)"
nvidia-smi --query-gpu=index,name,memory.total,clocks.max.sm --format=csv
nvidia-smi topo -m 2>/dev/null | head -20
for v in RANK LOCAL_RANK WORLD_SIZE LOCAL_WORLD_SIZE RANKS_PER_NODE MASTER_ADDR MASTER_PORT SLURM_JOB_NODELIST SLURM_PROCID CUDA_VISIBLE_DEVICES; do
  echo "$v=${!v:-<unset>}"
done
python - <<'PY'
import torch
print("torch", torch.__version__, "cuda", torch.version.cuda, "devices", torch.cuda.device_count())
from gruboros_b200.ops import _lib
print("kernel library:", _lib.LIB_PATH, "built" if _lib.available() else "MISSING (python -m gruboros_b200.build)")
PY
