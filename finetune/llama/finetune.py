#!/usr/bin/env python
"""LoRA fine-tuning of a Llama-family HuggingFace checkpoint, independent of the inference engine (the reference
ships the same kind of recipe on HF + PEFT for CPUs: finetune/llama/training/finetune.py).  This one needs only
PyTorch and transformers: the low-rank adapters are a small module of this file, data is Alpaca-style JSON or
pre-tokenised JSONL, and one process per GPU trains under DistributedDataParallel when launched with torchrun.

    python finetune/llama/finetune.py --base_model /path/to/hf-llama --data_path alpaca.json --output_dir lora-out \
        --bf16 --num_epochs 3 --merge
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 finetune/llama/finetune.py ...     # data parallel

Outputs: `adapter_model.pt` + `adapter_config.json` (A/B matrices per wrapped projection) and, with --merge, a full
HF checkpoint under `<output_dir>/merged` that `xfastertransformer_b200.LlamaConvert` turns into an engine model.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import random
import time
from typing import Dict, List, Optional

import torch
import torch.nn as nn

PROMPT_INPUT = ("Below is an instruction that describes a task, paired with an input that provides further context. "
                "Write a response that appropriately completes the request.\n\n### Instruction:\n{instruction}\n\n"
                "### Input:\n{input}\n\n### Response:\n")
PROMPT_NO_INPUT = ("Below is an instruction that describes a task. Write a response that appropriately completes the "
                   "request.\n\n### Instruction:\n{instruction}\n\n### Response:\n")


class LoRALinear(nn.Module):
    """y = W x + (alpha / r) * B (A dropout(x));  W frozen, A ~ kaiming-uniform, B = 0 (so training starts at W)."""

    def __init__(self, base: nn.Linear, r: int, alpha: float, dropout: float):
        super().__init__()
        self.base = base
        for p in self.base.parameters():
            p.requires_grad_(False)
        self.r, self.scaling = r, alpha / r
        self.lora_A = nn.Parameter(torch.empty(r, base.in_features, dtype=torch.float32))
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, r, dtype=torch.float32))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.drop = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    def forward(self, x):
        y = self.base(x)
        z = self.drop(x).to(self.lora_A.dtype) @ self.lora_A.t() @ self.lora_B.t()
        return y + (self.scaling * z).to(y.dtype)

    @torch.no_grad()
    def merge(self) -> nn.Linear:
        self.base.weight += (self.scaling * (self.lora_B @ self.lora_A)).to(self.base.weight.dtype)
        return self.base


def add_lora(model: nn.Module, targets: List[str], r: int, alpha: float, dropout: float) -> List[str]:
    wrapped = []
    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            if isinstance(child, nn.Linear) and child_name in targets:
                setattr(mod, child_name, LoRALinear(child, r, alpha, dropout))
                wrapped.append(f"{name}.{child_name}" if name else child_name)
    for n, p in model.named_parameters():
        if "lora_" not in n:
            p.requires_grad_(False)
    return wrapped


def adapter_state(model: nn.Module) -> Dict[str, torch.Tensor]:
    return {n: p.detach().cpu() for n, p in model.named_parameters() if "lora_" in n}


def merge_lora(model: nn.Module) -> None:
    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            if isinstance(child, LoRALinear):
                setattr(mod, child_name, child.merge())


# ----------------------------------------------------------------------------------------------- data
def load_records(path: str) -> List[dict]:
    with open(path) as f:
        text = f.read().strip()
    if text.startswith("["):
        return json.loads(text)
    return [json.loads(line) for line in text.splitlines() if line.strip()]


def tokenize_record(rec: dict, tok, cutoff: int, train_on_inputs: bool) -> Dict[str, List[int]]:
    if "input_ids" in rec:                                  # pre-tokenised
        ids = list(rec["input_ids"])[:cutoff]
        labels = list(rec.get("labels", ids))[:cutoff]
        return {"input_ids": ids, "labels": labels}
    prompt = (PROMPT_INPUT if rec.get("input") else PROMPT_NO_INPUT).format(**{"input": "", **rec})
    full = prompt + rec.get("output", "")
    ids = tok(full, truncation=True, max_length=cutoff, add_special_tokens=True)["input_ids"]
    if len(ids) < cutoff and tok.eos_token_id is not None and (not ids or ids[-1] != tok.eos_token_id):
        ids = ids + [tok.eos_token_id]
    labels = list(ids)
    if not train_on_inputs:
        n_prompt = len(tok(prompt, truncation=True, max_length=cutoff, add_special_tokens=True)["input_ids"])
        labels[:n_prompt] = [-100] * min(n_prompt, len(labels))
    return {"input_ids": ids, "labels": labels}


def collate(batch: List[Dict[str, List[int]]], pad_id: int):
    n = max(len(b["input_ids"]) for b in batch)
    ids = torch.full((len(batch), n), pad_id, dtype=torch.long)
    labels = torch.full((len(batch), n), -100, dtype=torch.long)
    mask = torch.zeros(len(batch), n, dtype=torch.long)
    for i, b in enumerate(batch):
        m = len(b["input_ids"])
        ids[i, :m] = torch.tensor(b["input_ids"])
        labels[i, :m] = torch.tensor(b["labels"])
        mask[i, :m] = 1
    return ids, labels, mask


# ----------------------------------------------------------------------------------------------- training
def train(args) -> Dict[str, float]:
    import transformers
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and not args.cpu
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if use_cuda else "gloo")
    random.seed(args.seed)
    torch.manual_seed(args.seed)

    dtype = torch.bfloat16 if args.bf16 else torch.float32
    model = transformers.AutoModelForCausalLM.from_pretrained(args.base_model, torch_dtype=dtype)
    tok = None
    try:
        tok = transformers.AutoTokenizer.from_pretrained(args.base_model)
    except Exception:
        pass                                                # pre-tokenised data needs none
    wrapped = add_lora(model, args.lora_target_modules, args.lora_r, args.lora_alpha, args.lora_dropout)
    if not wrapped:
        raise SystemExit(f"no nn.Linear named {args.lora_target_modules} in the model")
    model.to(device)
    if args.gradient_checkpointing:
        model.gradient_checkpointing_enable()
        model.enable_input_require_grads()
    n_train = sum(p.numel() for p in model.parameters() if p.requires_grad)
    n_all = sum(p.numel() for p in model.parameters())
    if rank == 0:
        print(f"LoRA on {len(wrapped)} projections: {n_train:,} trainable of {n_all:,} parameters "
              f"({100.0 * n_train / n_all:.3f}%)", flush=True)

    records = load_records(args.data_path)
    data = [tokenize_record(r, tok, args.cutoff_len, args.train_on_inputs) for r in records]
    data = [d for d in data if any(l != -100 for l in d["labels"][1:])]
    if args.val_set_size > 0:
        random.shuffle(data)
        val, data = data[:args.val_set_size], data[args.val_set_size:]
    else:
        val = []
    pad_id = (tok.pad_token_id if tok is not None and tok.pad_token_id is not None else 0)
    ddp = model
    if world > 1:
        ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local] if use_cuda else None)
    opt = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=args.learning_rate, weight_decay=0.0)
    micro = args.micro_batch_size
    accum = max(1, args.batch_size // (micro * world))
    steps_per_epoch = max(1, len(data) // (micro * world * accum))
    total = args.max_steps if args.max_steps > 0 else steps_per_epoch * args.num_epochs
    warm = min(args.warmup_steps, max(total - 1, 0))
    sched = torch.optim.lr_scheduler.LambdaLR(
        opt, lambda s: (s + 1) / (warm + 1) if s < warm else max(0.0, (total - s) / max(1, total - warm)))

    def loss_of(batch):
        ids, labels, mask = (t.to(device) for t in collate(batch, pad_id))
        with torch.autocast(device.type, dtype=torch.bfloat16, enabled=args.bf16):
            out = ddp(input_ids=ids, attention_mask=mask, labels=labels)
        return out.loss

    step, first, last, t0 = 0, None, None, time.time()
    model.train()
    while step < total:
        order = list(range(len(data)))
        random.shuffle(order)
        order = order[rank::world]
        for i in range(0, len(order) - micro * accum + 1, micro * accum):
            opt.zero_grad(set_to_none=True)
            tot = 0.0
            for a in range(accum):
                batch = [data[j] for j in order[i + a * micro:i + (a + 1) * micro]]
                loss = loss_of(batch) / accum
                loss.backward()
                tot += loss.item()
            torch.nn.utils.clip_grad_norm_([p for p in model.parameters() if p.requires_grad], 1.0)
            opt.step()
            sched.step()
            step += 1
            first = tot if first is None else first
            last = tot
            if rank == 0 and (step % args.logging_steps == 0 or step == total):
                print(f"step {step}/{total} loss {tot:.4f} lr {sched.get_last_lr()[0]:.2e} "
                      f"{(time.time() - t0) / step:.2f} s/step", flush=True)
            if step >= total:
                break
    result = {"first_loss": first, "last_loss": last, "steps": step}
    if val:
        model.eval()
        with torch.no_grad():
            vl = [loss_of(val[i:i + micro]).item() for i in range(0, len(val), micro)]
        result["val_loss"] = sum(vl) / len(vl)
    if rank == 0:
        os.makedirs(args.output_dir, exist_ok=True)
        torch.save(adapter_state(model), os.path.join(args.output_dir, "adapter_model.pt"))
        with open(os.path.join(args.output_dir, "adapter_config.json"), "w") as f:
            json.dump({"r": args.lora_r, "lora_alpha": args.lora_alpha, "lora_dropout": args.lora_dropout,
                       "target_modules": args.lora_target_modules, "base_model": args.base_model, "wrapped": wrapped,
                       **result}, f, indent=1)
        if args.merge:
            merge_lora(model)
            model.save_pretrained(os.path.join(args.output_dir, "merged"), safe_serialization=True)
            if tok is not None:
                tok.save_pretrained(os.path.join(args.output_dir, "merged"))
        print(json.dumps(result), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    return result


def parse(argv: Optional[List[str]] = None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--base_model", required=True)
    ap.add_argument("--data_path", required=True)
    ap.add_argument("--output_dir", default="./lora-alpaca")
    ap.add_argument("--bf16", action="store_true")
    ap.add_argument("--cpu", action="store_true", help="train on the CPU even if a GPU is present")
    ap.add_argument("--batch_size", type=int, default=128)
    ap.add_argument("--micro_batch_size", type=int, default=16)
    ap.add_argument("--num_epochs", type=int, default=3)
    ap.add_argument("--max_steps", type=int, default=-1)
    ap.add_argument("--learning_rate", type=float, default=3e-4)
    ap.add_argument("--warmup_steps", type=int, default=100)
    ap.add_argument("--cutoff_len", type=int, default=256)
    ap.add_argument("--val_set_size", type=int, default=0)
    ap.add_argument("--logging_steps", type=int, default=10)
    ap.add_argument("--lora_r", type=int, default=8)
    ap.add_argument("--lora_alpha", type=float, default=16)
    ap.add_argument("--lora_dropout", type=float, default=0.05)
    ap.add_argument("--lora_target_modules", nargs="+", default=["q_proj", "v_proj"])
    ap.add_argument("--train_on_inputs", action="store_true")
    ap.add_argument("--gradient_checkpointing", action="store_true")
    ap.add_argument("--merge", action="store_true", help="also write the merged HF checkpoint")
    ap.add_argument("--seed", type=int, default=42)
    return ap.parse_args(argv)


if __name__ == "__main__":
    train(parse())
