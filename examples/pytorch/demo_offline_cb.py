#!/usr/bin/env python
"""Client-side continuous-batching scheduler (reference: ``examples/pytorch/demo_offline_cb.py:239-305``): admit
waiting prompts (one prefill call), decode all running sequences together (up to ``--max_batch``), retire a
sequence on eos / length and free its KV blocks, until the queue is empty.  Greedy selection on the returned logits.

    python examples/pytorch/demo_offline_cb.py -m <model dir> [--num_prompts 16] [--max_batch 64] [--output_len 32]
    python examples/pytorch/demo_offline_cb.py -m <model dir> -t <HF tokenizer dir> [-i prompts.txt] [-s]

With `-t` the prompts are text (the reference's options: `-i` a file with one prompt per line, else built-in prompts; `-s`
prints the answers in the order of the prompts instead of the order in which they finish); without it, random token ids.
"""
import argparse
import os
import random
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


BUILTIN_PROMPTS = [
    "Once upon a time, there existed a little girl who liked to have adventures.",
    "The capital of France is",
    "Explain in one sentence why the sky is blue.",
    "Write a haiku about the sea.",
    "List three prime numbers.",
    "What is the boiling point of water at sea level?",
]


def run(model, prompts, max_batch=64, output_len=32, eos=-1, prefill_per_step=4, finished=None):
    waiting = list(enumerate(prompts))
    running = {}            # seq_id -> dict(req, last, n)
    results = {}
    steps = 0
    while waiting or running:
        if waiting and len(running) < max_batch:
            take = waiting[:min(prefill_per_step, max_batch - len(running))]
            del waiting[:len(take)]
            sids = model.set_input_cb([p for _, p in take], None, [len(p) + output_len + 1 for _, p in take])
            logits = model.forward_cb()
            for (req, p), sid, row in zip(take, sids.tolist(), logits):
                running[sid] = dict(req=req, out=[int(row.argmax())])
        else:
            sids = list(running)
            model.set_input_cb([running[s]["out"][-1] for s in sids], sids, None)
            logits = model.forward_cb()
            for s, row in zip(sids, logits):
                running[s]["out"].append(int(row.argmax()))
        steps += 1
        done = [s for s, r in running.items() if len(r["out"]) >= output_len or r["out"][-1] == eos]
        if done:
            model.free_seqs(done)
            for s in done:
                r = running.pop(s)
                results[r["req"]] = r["out"]
                if finished is not None:
                    finished(r["req"], r["out"])
    return [results[i] for i in range(len(prompts))], steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model_path", required=True)
    ap.add_argument("-d", "--dtype", default="bf16")
    ap.add_argument("--kv_cache_dtype", default="fp16")
    ap.add_argument("-t", "--token_path", default="", help="Hugging Face tokenizer directory: text prompts instead of random ids")
    ap.add_argument("-i", "--input_file", default="", help="one prompt per line (with -t); default: built-in prompts")
    ap.add_argument("-s", "--sort_results", action="store_true", help="print the answers in the order of the prompts")
    ap.add_argument("--num_prompts", type=int, default=16)
    ap.add_argument("--max_batch", type=int, default=64)
    ap.add_argument("--output_len", type=int, default=32)
    a = ap.parse_args()
    import xfastertransformer_b200 as xft
    model = xft.AutoModel.from_pretrained(a.model_path, dtype=a.dtype, kv_cache_dtype=a.kv_cache_dtype)
    if model.rank != 0:                  # several GPUs (torchrun): the other ranks execute rank 0's calls
        model.follow()
        return
    tok, texts, eos = None, None, -1
    if a.token_path:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.token_path)
        texts = [l.strip() for l in open(a.input_file, encoding="utf-8") if l.strip()] if a.input_file else BUILTIN_PROMPTS
        prompts = [tok(t, add_special_tokens=True)["input_ids"] for t in texts]
        eos = tok.eos_token_id if tok.eos_token_id is not None else -1
    else:
        rng = random.Random(0)
        v = model.model.cfg.vocab_size
        prompts = [[rng.randrange(5, v) for _ in range(rng.randint(8, 64))] for _ in range(a.num_prompts)]

    def show(req, out):
        print(f"[{req}] {texts[req]!r} -> {tok.decode(out, skip_special_tokens=True)!r}", flush=True)

    t0 = time.perf_counter()
    outs, steps = run(model, prompts, a.max_batch, a.output_len, eos=eos, finished=show if tok and not a.sort_results else None)
    dt = time.perf_counter() - t0
    if tok and a.sort_results:
        for req, out in enumerate(outs):
            show(req, out)
    n = sum(len(o) for o in outs)
    print(f"{len(prompts)} requests, {n} tokens, {steps} engine steps, {n / dt:.1f} tokens/s")
    model.model.exit_slaves()


if __name__ == "__main__":
    main()
