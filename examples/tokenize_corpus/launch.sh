#!/bin/bash
# Run one corpus tokenization example:  bash examples/tokenize_corpus/launch.sh <example directory name> [extra args]
set -euo pipefail
[ $# -ge 1 ] || { echo "usage: $0 <example directory name> [args]" >&2; exit 2; }
export PYTHONUNBUFFERED=1
NAME=$1; shift
LOG=logging/tokenize_corpus/${NAME}_node${SLURM_NODEID:-0}.log
mkdir -p "$(dirname "$LOG")"
python "examples/tokenize_corpus/$NAME/script.py" "$@" 2>&1 | tee "$LOG"
