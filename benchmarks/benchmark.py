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


def build_prompt_ids(tok, a, path, json):
    """[batch, input_tokens] token ids from the reference's prompt sources (benchmark/benchmark.py:204-270)."""
    import torch

    def fit(t):
        while len(t) < a.input_tokens:
            t = t + t
        return t[:a.input_tokens]

    if a.input_prompt:
        return torch.tensor([fit(tok(a.input_prompt, add_special_tokens=True)["input_ids"])] * a.batch_size)
    if path.endswith(".sonnet"):
        # prompts that share their first --sonnet_prefix_len tokens (prefix sharing / prefix cache runs): the prefix is
        # the head of the poem, the rest of each prompt is a different run of lines
        lines = [l for l in open(path, encoding="utf-8").read().splitlines() if l.strip()]
        prefix, k = [], 0
        while len(prefix) < a.sonnet_prefix_len and k < len(lines):
            prefix += tok(lines[k] + "\n", add_special_tokens=(k == 0))["input_ids"]
            k += 1
        prefix = prefix[:min(a.sonnet_prefix_len, a.input_tokens)]
        rows = []
        for r in range(max(1, a.sonnet_count)):
            tail, j = [], (k + 7 * r) % max(len(lines), 1)
            while len(prefix) + len(tail) < a.input_tokens:
                tail += tok(lines[j % len(lines)] + "\n", add_special_tokens=False)["input_ids"]
                j += 1
            rows.append((prefix + tail)[:a.input_tokens])
        return torch.tensor(rows)
    if path.endswith(".txt"):
        pool = [l for l in open(path, encoding="utf-8").read().splitlines() if l.strip()]
        return torch.tensor([fit(tok(pool[i % len(pool)], add_special_tokens=True)["input_ids"]) for i in range(a.batch_size)])
    if not path.endswith(".json"):
        raise ValueError("prompt files are .json, .txt or .sonnet")
    prompts = json.load(open(path))
    text = prompts.get(str(a.input_tokens)) or prompts.get("long_unit", "It is a truth universally acknowledged. ") * (a.input_tokens // 8 + 1)
    return torch.tensor([fit(tok(text, add_special_tokens=True)["input_ids"])] * a.batch_size)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_path", "-m", default="")
    ap.add_argument("--model_name", default="", help="a preset of tools/synthetic.py (e.g. llama-2-7b): config only, fake weights")
    ap.add_argument("--token_path", "-tp", default="", help="HF tokenizer dir: prompts come from prompt.json instead of random ids")
    ap.add_argument("--dtype", "-d", default="bf16")
    ap.add_argument("--kv_cache_dtype", "-kvd", default="fp16")
    ap.add_argument("--batch_size", "-bs", type=int, default=1)
    ap.add_argument("--input_tokens", "--token_in", "-in", dest="input_tokens", type=int, default=32)
    ap.add_argument("--output_tokens", "--token_out", "-out", dest="output_tokens", type=int, default=32)
    # the reference's prompt options (benchmark/benchmark.py:76-91); they need --token_path
    ap.add_argument("--input_prompt", default=None, help="prompt text instead of an entry of the prompt file")
    ap.add_argument("--prompt_path", default="", help=".json (token count -> text; default: the bundled prompt.json), .txt (one prompt "
                    "per line), or .sonnet (poem lines: --sonnet_count prompts that share a prefix of --sonnet_prefix_len tokens)")
    ap.add_argument("--padding", default="True", help="accepted for the reference's command lines; prompts of one batch have one length here")
    ap.add_argument("--sonnet_prefix_len", type=int, default=200)
    ap.add_argument("--sonnet_count", type=int, default=20)
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
        # real text: the prompt given, an entry of the prompt file of that length, or the filler sentence repeated — cut to
        # the token count
        import json
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.token_path)
        path = a.prompt_path or os.path.join(os.path.dirname(os.path.abspath(__file__)), "prompt.json")
        ids = build_prompt_ids(tok, a, path, json)
        a.batch_size, a.input_tokens = ids.shape
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
