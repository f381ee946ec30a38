#!/bin/bash
# Front end of benchmarks/benchmark.py (reference: benchmark/run_benchmark.sh, which derives an mpirun line from the
# NUMA topology; here the topology is "how many B200s does this node have" and the launcher is torchrun).
#
#   run_benchmark.sh -m <model name or converted dir> [-d bf16] [-kvd fp16] [-bs 1] [-in 32] [-out 32] [-i 3] [-w 1]
#                    [-g <gpus>|auto] [-tp <tokenizer dir>] [--fake]
#   the reference's other options are taken too: -mp <converted dir> (with -m as the name), -s <sockets> = GPUs,
#   -sid <ids> = CUDA_VISIBLE_DEVICES, -c <csv file>, -p <prompt file>, -splen / -sc (sonnet prompts)
set -e
HERE=$(cd "$(dirname "$0")" && pwd)
MODEL="" MPATH="" DTYPE=bf16 KVD=fp16 BS=1 IN=32 OUT=32 ITER=3 WARM=1 GPUS=1 TOK="" FAKE=0 CSV="" PROMPTS="" SPLEN="" SCOUNT=""
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
    -mp|--model_path) MPATH=$2; shift 2;;
    -sid|--sockets_id) export CUDA_VISIBLE_DEVICES=$2; shift 2;;
    -c|--csv) CSV=$2; shift 2;;
    -p|--prompt_path) PROMPTS=$2; shift 2;;
    -splen|--sonnet_prefix_len) SPLEN=$2; shift 2;;
    -sc|--sonnet_count) SCOUNT=$2; shift 2;;
    --fake) FAKE=1; shift;;
    -h|--help) sed -n 2,10p "$0"; exit 0;;
    *) echo "unknown flag $1" >&2; exit 2;;
  esac
done
[ -n "$MPATH" ] && MODEL=$MPATH
[ -n "$MODEL" ] || { echo "need -m <model>" >&2; exit 2; }
if [ "$GPUS" = auto ]; then GPUS=$(nvidia-smi -L 2>/dev/null | wc -l); [ "$GPUS" -ge 1 ] || GPUS=1; fi
ARGS=(--dtype "$DTYPE" --kv_cache_dtype "$KVD" --batch_size "$BS" --input_tokens "$IN" --output_tokens "$OUT" --iteration "$ITER" --warmup "$WARM")
if [ -d "$MODEL" ]; then ARGS+=(--model_path "$MODEL"); else ARGS+=(--model_name "$MODEL"); FAKE=1; fi
[ -n "$TOK" ] && ARGS+=(--token_path "$TOK")
[ -n "$CSV" ] && ARGS+=(--csv "$CSV")
[ -n "$PROMPTS" ] && ARGS+=(--prompt_path "$PROMPTS")
[ -n "$SPLEN" ] && ARGS+=(--sonnet_prefix_len "$SPLEN")
[ -n "$SCOUNT" ] && ARGS+=(--sonnet_count "$SCOUNT")
[ "$FAKE" = 1 ] && export XFT_FAKE_MODEL=${XFT_FAKE_MODEL:-2}
echo "benchmark: model=$MODEL dtype=$DTYPE kv=$KVD bs=$BS in=$IN out=$OUT gpus=$GPUS fake=$FAKE"
if [ "$GPUS" -gt 1 ]; then
  exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 \
       --master-port "${MASTER_PORT:-29533}" "$HERE/benchmark.py" "${ARGS[@]}"
else
  exec python "$HERE/benchmark.py" "${ARGS[@]}"
fi
