#!/usr/bin/env python
"""Interactive / one-shot generation demo (reference: ``examples/pytorch/demo.py``).  Works on token ids, or on text
when a HuggingFace tokenizer directory is given.

    python examples/pytorch/demo.py -m <xft model dir> [-t <tokenizer dir>] [-d bf16] [--input "..."] [--ids "1 2 3"]
        [--output_len 64] [--do_sample] [--streaming]
Followers (rank != 0 under torchrun) loop on ``generate()``.
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


class IdStreamer:
    """Minimal streamer protocol (put / end), like transformers' BaseStreamer."""

    def __init__(self, tok=None):
        self.tok, self.first = tok, True

    def put(self, value):
        if self.first:
            self.first = False
            return
        ids = value.flatten().tolist()
        print(self.tok.decode(ids) if self.tok else " ".join(map(str, ids)), end=" ", flush=True)

    def end(self):
        print()


def boolean_string(v):
    """The reference's demos take `--flag True` / `--flag False` (examples/pytorch/demo.py:52-58); a bare `--flag` means True."""
    if isinstance(v, bool):
        return v
    if v.lower() not in ("true", "false"):
        raise argparse.ArgumentTypeError("expected True or False")
    return v.lower() == "true"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model_path", required=True)
    ap.add_argument("-t", "--token_path", default="")
    ap.add_argument("-d", "--dtype", default="bf16")
    ap.add_argument("--kv_cache_dtype", default="fp16")
    ap.add_argument("--input", default="Once upon a time, there existed a little girl who liked to have adventures.")
    ap.add_argument("--ids", default="")
    ap.add_argument("-o", "--output_len", type=int, default=64)
    ap.add_argument("--num_beams", type=int, default=1)
    ap.add_argument("--do_sample", nargs="?", const=True, default=False, type=boolean_string)
    ap.add_argument("--padding", nargs="?", const=True, default=False, type=boolean_string,
                    help="accepted for the reference's command lines: one prompt needs no padding")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top_k", type=int, default=50)
    ap.add_argument("--top_p", type=float, default=1.0)
    ap.add_argument("--rep_penalty", type=float, default=1.0)
    ap.add_argument("--streaming", nargs="?", const=True, default=False, type=boolean_string)
    ap.add_argument("--chat", nargs="?", const=True, default=False, type=boolean_string, help="read prompts from stdin in a loop")
    a = ap.parse_args()
    import torch

    import xfastertransformer_b200 as xft
    model = xft.AutoModel.from_pretrained(a.model_path, dtype=a.dtype, kv_cache_dtype=a.kv_cache_dtype)
    if model.rank != 0:
        while True:
            model.generate()
    tok = None
    if a.token_path:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.token_path, trust_remote_code=False)
    while True:
        if a.ids or tok is None:
            ids = torch.tensor([[int(t) for t in (a.ids or "1 2 3 4 5 6 7 8").split()]])
        else:
            text = input("\nPlease enter the prompt: ") if a.chat else a.input
            ids = tok(text, return_tensors="pt").input_ids
        t0 = time.perf_counter()
        out = model.generate(ids, max_length=ids.shape[1] + a.output_len, num_beams=a.num_beams, do_sample=a.do_sample,
                             temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, repetition_penalty=a.rep_penalty,
                             streamer=IdStreamer(tok) if a.streaming and a.num_beams == 1 else None)
        dt = time.perf_counter() - t0
        gen = out[0, ids.shape[1]:].tolist()
        print(tok.decode(gen) if tok else gen)
        print(f"[{len(gen)} tokens in {dt * 1e3:.1f} ms]")
        if not a.chat:
            break
    model.model.exit_slaves()


if __name__ == "__main__":
    main()
