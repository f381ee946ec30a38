#!/bin/bash
# Multi-node launch of benchmarks/benchmark.py (reference: benchmark/run_benchmark_dist.sh, which builds an mpirun line
# over several hosts).  Run the same command on every node; ranks of one node use that node's GPUs.
#   NNODES=2 NODE_RANK=0 MASTER_ADDR=10.0.0.1 benchmarks/run_benchmark_dist.sh -m llama-2-70b -d bf16 -bs 16 -in 2048 -out 128
# Options after the environment are those of run_benchmark.sh / benchmark.py.  Tensor parallelism runs inside a node
# (NVLink); with XFT_PIPELINE_STAGE=<NNODES> the nodes become pipeline stages connected by NCCL send / recv.
set -e
cd "$(dirname "$0")/.."
NNODES=${NNODES:-1}
NODE_RANK=${NODE_RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-29555}
GPUS=${GPUS_PER_NODE:-$(python -c "import torch; print(max(torch.cuda.device_count(), 1))")}
model="llama-2-7b"; args=()
while [ $# -gt 0 ]; do
  case "$1" in
    -m|--model_name) model="$2"; shift 2 ;;
    *) args+=("$1"); shift ;;
  esac
done
if [ "$NNODES" -gt 1 ] && [ -z "$XFT_PIPELINE_STAGE" ]; then export XFT_PIPELINE_STAGE=$NNODES; fi
echo "nodes=$NNODES node_rank=$NODE_RANK gpus/node=$GPUS pipeline stages=${XFT_PIPELINE_STAGE:-1} model=$model"
if [ -d "$model" ]; then margs=(--model_path "$model"); else margs=(--model_name "$model"); export XFT_FAKE_MODEL=${XFT_FAKE_MODEL:-2}; fi
exec python -m torch.distributed.run --nnodes="$NNODES" --node-rank="$NODE_RANK" --nproc-per-node="$GPUS" \
  --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" benchmarks/benchmark.py "${margs[@]}" "${args[@]}"
