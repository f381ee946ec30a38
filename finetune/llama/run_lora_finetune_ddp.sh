#!/bin/bash
# Data-parallel LoRA fine-tuning, one process per GPU.  usage: run_lora_finetune_ddp.sh <gpus> <hf model dir> <data.json> [out dir]
set -e
HERE=$(cd "$(dirname "$0")" && pwd)
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$1" --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29577}" \
    "$HERE/finetune.py" --base_model "$2" --data_path "$3" --output_dir "${4:-./lora-alpaca}" \
    --bf16 --batch_size 128 --micro_batch_size 8 --num_epochs 3 --learning_rate 3e-4 --cutoff_len 512 --merge
