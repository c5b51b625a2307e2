#!/bin/bash
# bash benchmarks/pretraining/launch.sh <model> <cluster/mesh>     (srun -W 0 ... for several nodes)
set -euo pipefail
[ $# -ge 2 ] || { python benchmarks/pretraining/run.py --list; exit 2; }
export OMP_NUM_THREADS=${OMP_NUM_THREADS:-8} PYTHONUNBUFFERED=1
LOG=logging/benchmarks/$1/$(echo "$2" | tr / _)_node${SLURM_NODEID:-0}.log
mkdir -p "$(dirname "$LOG")"
python -m torch.distributed.run --nnodes="${SLURM_NNODES:-1}" --node-rank="${SLURM_NODEID:-0}" --nproc-per-node=gpu \
    --rdzv-backend=c10d --rdzv-endpoint="${SLURM_LAUNCH_NODE_IPADDR:-127.0.0.1}:15213" \
    benchmarks/pretraining/run.py "$1" "$2" 2>&1 | tee "$LOG"
