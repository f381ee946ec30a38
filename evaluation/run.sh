#!/bin/bash
# Launch evaluation/eval.py on N GPUs of this node (reference: evaluation/run.sh, which builds an mpirun line per socket).
#   evaluation/run.sh <gpus> <eval.py arguments...>
set -e
n=${1:?usage: run.sh <gpus> <eval.py arguments...>}; shift
cd "$(dirname "$0")/.."
if [ "$n" -le 1 ]; then exec python evaluation/eval.py "$@"; fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$n" --master-addr 127.0.0.1 \
     --master-port "${MASTER_PORT:-29577}" evaluation/eval.py "$@"
