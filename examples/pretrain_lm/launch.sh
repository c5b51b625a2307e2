#!/bin/bash
# Start one pre-training example on every GPU of this node (and of the other nodes of a SLURM step).
#
#   bash examples/pretrain_lm/launch.sh qwen3-30b-a3b
#   srun -W 0 examples/pretrain_lm/launch.sh gpt-oss-120b      # multi-node
set -euo pipefail
[ $# -eq 1 ] || { echo "usage: $0 <example directory name>" >&2; exit 2; }

export OMP_NUM_THREADS=${OMP_NUM_THREADS:-8} PYTHONUNBUFFERED=1
NODES=${SLURM_NNODES:-1}
NODE=${SLURM_NODEID:-0}
HEAD=${SLURM_LAUNCH_NODE_IPADDR:-127.0.0.1}

LOG=logging/pretrain_lm/$1_node$NODE.log
mkdir -p "$(dirname "$LOG")"
python -m torch.distributed.run --nnodes="$NODES" --node-rank="$NODE" --nproc-per-node=gpu \
    --rdzv-backend=c10d --rdzv-endpoint="$HEAD:15213" \
    "examples/pretrain_lm/$1/script.py" 2>&1 | tee "$LOG"
