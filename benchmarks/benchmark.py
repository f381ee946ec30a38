#!/usr/bin/env python
"""Latency / throughput benchmark with the reference's protocol and metric definitions
(``benchmark/benchmark.py:252-391``): warm-up generations, then per iteration ``set_input`` -> timed ``forward()``
loop -> ``finalize()``; first-token latency = first forward, next-token latency = each later forward, throughput =
1000 / mean(next_token_ms) * batch_size.  Fake weights (``XFT_FAKE_MODEL``) need only a config.ini.

    python benchmarks/benchmark.py --model_path <dir> --dtype bf16 --batch_size 1 --input_tokens 1024 \
        --output_tokens 128 --iteration 3 --warmup 1 [--csv out.csv] [--fake 2]
Multi-GPU: launch with torchrun; followers mirror rank 0 (they run the same calls with ignored arguments).
"""
import argparse
import csv
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_path", "-m", default="")
    ap.add_argument("--model_name", default="", help="a preset of tools/synthetic.py (e.g. llama-2-7b): config only, fake weights")
    ap.add_argument("--token_path", "-tp", default="", help="HF tokenizer dir: prompts come from prompt.json instead of random ids")
    ap.add_argument("--dtype", "-d", default="bf16")
    ap.add_argument("--kv_cache_dtype", "-kvd", default="fp16")
    ap.add_argument("--batch_size", "-bs", type=int, default=1)
    ap.add_argument("--input_tokens", "-in", type=int, default=32)
    ap.add_argument("--output_tokens", "-out", type=int, default=32)
    ap.add_argument("--iteration", "-i", type=int, default=3)
    ap.add_argument("--warmup", "-w", type=int, default=1)
    ap.add_argument("--beam_width", type=int, default=1)
    ap.add_argument("--csv", default="")
    ap.add_argument("--fake", type=int, default=0, help="XFT_FAKE_MODEL value (1 zeros, 2 random)")
    a = ap.parse_args()
    if not a.model_path and not a.model_name:
        ap.error("one of --model_path / --model_name is required")
    if a.model_name and not a.model_path:
        import tempfile
        from xfastertransformer_b200.tools.synthetic import config_only, preset
        a.model_path = os.path.join(tempfile.gettempdir(), f"xft_bench_{a.model_name}_{os.environ.get('RANK', '0')}")
        config_only(a.model_path, preset(a.model_name))
        a.fake = a.fake or 2
    if a.fake:
        os.environ["XFT_FAKE_MODEL"] = str(a.fake)
    import torch

    import xfastertransformer_b200 as xft
    model = xft.AutoModel.from_pretrained(a.model_path, dtype=a.dtype, kv_cache_dtype=a.kv_cache_dtype)
    cuda = model.model.ctx.device.type == "cuda"
    vocab = model.model.cfg.vocab_size
    ids = torch.randint(5, max(vocab - 1, 6), (a.batch_size, a.input_tokens), generator=torch.Generator().manual_seed(1))
    if a.token_path:
        # real text: the prompt.json entry of that length, or the filler sentence repeated, cut to the token count
        import json
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.token_path)
        prompts = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "prompt.json")))
        text = prompts.get(str(a.input_tokens)) or prompts["long_unit"] * (a.input_tokens // 8 + 1)
        t = tok(text, add_special_tokens=True)["input_ids"]
        while len(t) < a.input_tokens:
            t = t + t
        ids = torch.tensor([t[:a.input_tokens]] * a.batch_size)
    max_len = a.input_tokens + a.output_tokens

    def sync():
        if cuda:
            torch.cuda.synchronize()

    for _ in range(a.warmup):
        model.generate(ids, max_length=max_len, num_beams=a.beam_width, eos_token_id=-2, pad_token_id=0)
    first, nxt, total = [], [], []
    for _ in range(a.iteration):
        model.set_input(ids, max_length=max_len, num_beams=a.beam_width, eos_token_id=-2, pad_token_id=0)
        sync()
        t_all = time.perf_counter()
        step = 0
        while not model.is_done():
            t0 = time.perf_counter()
            model.forward()
            sync()
            ms = (time.perf_counter() - t0) * 1e3
            (first if step == 0 else nxt).append(ms)
            step += 1
        total.append((time.perf_counter() - t_all) * 1e3)
        model.finalize()
    if model.rank != 0:
        return
    p90 = sorted(nxt)[int(0.9 * (len(nxt) - 1))] if nxt else 0.0
    res = {"model": os.path.basename(a.model_path.rstrip("/")), "dtype": a.dtype, "kv_cache_dtype": a.kv_cache_dtype,
           "batch_size": a.batch_size, "input_tokens": a.input_tokens, "output_tokens": a.output_tokens,
           "infer_avg_ms": round(statistics.mean(total), 3), "first_token_avg_ms": round(statistics.mean(first), 3),
           "next_token_max_ms": round(max(nxt), 3) if nxt else 0, "next_token_min_ms": round(min(nxt), 3) if nxt else 0,
           "next_token_p90_ms": round(p90, 3), "next_token_avg_ms": round(statistics.mean(nxt), 3) if nxt else 0,
           "throughput_tokens_per_s": round(1000.0 / statistics.mean(nxt) * a.batch_size, 2) if nxt else 0}
    print("=" * 60)
    for k, v in res.items():
        print(f"{k:>26}: {v}")
    if a.csv:
        new = not os.path.exists(a.csv)
        with open(a.csv, "a", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(res))
            if new:
                w.writeheader()
            w.writerow(res)


if __name__ == "__main__":
    main()
