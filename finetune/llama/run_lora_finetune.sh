#!/bin/bash
# LoRA fine-tuning on one GPU (or the CPU with --cpu).  usage: run_lora_finetune.sh <hf model dir> <data.json> [out dir]
set -e
HERE=$(cd "$(dirname "$0")" && pwd)
python "$HERE/finetune.py" --base_model "$1" --data_path "$2" --output_dir "${3:-./lora-alpaca}" \
    --bf16 --batch_size 128 --micro_batch_size 16 --num_epochs 3 --learning_rate 3e-4 --cutoff_len 512 \
    --lora_r 8 --lora_alpha 16 --lora_dropout 0.05 --lora_target_modules q_proj v_proj --merge
