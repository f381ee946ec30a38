#!/bin/bash
# Front end of benchmarks/benchmark.py (reference: benchmark/run_benchmark.sh, which derives an mpirun line from the
# NUMA topology; here the topology is "how many B200s does this node have" and the launcher is torchrun).
#
#   run_benchmark.sh -m <model name or converted dir> [-d bf16] [-kvd fp16] [-bs 1] [-in 32] [-out 32] [-i 3] [-w 1]
#                    [-g <gpus>|auto] [-tp <tokenizer dir>] [--fake]
set -e
HERE=$(cd "$(dirname "$0")" && pwd)
MODEL="" DTYPE=bf16 KVD=fp16 BS=1 IN=32 OUT=32 ITER=3 WARM=1 GPUS=1 TOK="" FAKE=0
while [ $# -gt 0 ]; do
  case "$1" in
    -m|--model_name) MODEL=$2; shift 2;;
    -d|--dtype) DTYPE=$2; shift 2;;
    -kvd|--kv_cache_dtype) KVD=$2; shift 2;;
    -bs|--batch_size) BS=$2; shift 2;;
    -in|--input_tokens) IN=$2; shift 2;;
    -out|--output_tokens) OUT=$2; shift 2;;
    -i|--iter) ITER=$2; shift 2;;
    -w|--warmup) WARM=$2; shift 2;;
    -g|--gpus|-s|--sockets) GPUS=$2; shift 2;;
    -tp|--token_path) TOK=$2; shift 2;;
    --fake) FAKE=1; shift;;
    -h|--help) sed -n 2,8p "$0"; exit 0;;
    *) echo "unknown flag $1" >&2; exit 2;;
  esac
done
[ -n "$MODEL" ] || { echo "need -m <model>" >&2; exit 2; }
if [ "$GPUS" = auto ]; then GPUS=$(nvidia-smi -L 2>/dev/null | wc -l); [ "$GPUS" -ge 1 ] || GPUS=1; fi
ARGS=(--dtype "$DTYPE" --kv_cache_dtype "$KVD" --batch_size "$BS" --input_tokens "$IN" --output_tokens "$OUT" --iteration "$ITER" --warmup "$WARM")
if [ -d "$MODEL" ]; then ARGS+=(--model_path "$MODEL"); else ARGS+=(--model_name "$MODEL"); FAKE=1; fi
[ -n "$TOK" ] && ARGS+=(--token_path "$TOK")
[ "$FAKE" = 1 ] && export XFT_FAKE_MODEL=${XFT_FAKE_MODEL:-2}
echo "benchmark: model=$MODEL dtype=$DTYPE kv=$KVD bs=$BS in=$IN out=$OUT gpus=$GPUS fake=$FAKE"
if [ "$GPUS" -gt 1 ]; then
  exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 \
       --master-port "${MASTER_PORT:-29533}" "$HERE/benchmark.py" "${ARGS[@]}"
else
  exec python "$HERE/benchmark.py" "${ARGS[@]}"
fi
