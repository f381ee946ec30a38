#!/usr/bin/env python
"""Prefix-sharing A/B (reference: ``examples/pytorch/prefix_sharing.py:113-170``): the same prompts with and without
a shared cached prefix must give identical tokens, and the first-token time drops.

    python examples/pytorch/prefix_sharing.py -m <model dir> [--prefix_len 512] [--tail_len 32]
    python examples/pytorch/prefix_sharing.py -m <model dir> -t <HF tokenizer dir> [--input "..."] [--prefix_len 10] [--output_len 100]

With `-t` the prompt is text, as in the reference: its first `--prefix_len` tokens become the shared prefix (here cut down
to whole 64-token KV blocks; the tokens in between are computed with the rest of the prompt), and the answer is printed.
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model_path", required=True)
    ap.add_argument("-d", "--dtype", default="bf16")
    # the reference's options (examples/pytorch/prefix_sharing.py:55-63)
    ap.add_argument("-t", "--token_path", default="")
    ap.add_argument("--input", default="Once upon a time, there existed a little girl who liked to have adventures. " * 12)
    ap.add_argument("--padding", default="False", help="accepted; one prompt needs no padding")
    ap.add_argument("--streaming", default="False", help="accepted; the answer is printed when it is complete")
    ap.add_argument("--num_beams", type=int, default=1)
    ap.add_argument("--output_len", type=int, default=16)
    ap.add_argument("--prefix_len", type=int, default=512)
    ap.add_argument("--tail_len", type=int, default=32)
    ap.add_argument("--batch", type=int, default=4)
    a = ap.parse_args()
    import torch

    import xfastertransformer_b200 as xft
    model = xft.AutoModel.from_pretrained(a.model_path, dtype=a.dtype)
    tok = None
    if a.token_path:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.token_path)
        ids = tok(a.input, return_tensors="pt").input_ids
        prefix = ids[:, :min(a.prefix_len, ids.shape[1] - 1)]
    else:
        g = torch.Generator().manual_seed(0)
        v = model.model.cfg.vocab_size
        prefix = torch.randint(5, v, (1, a.prefix_len), generator=g)
        ids = torch.cat([prefix.expand(a.batch, -1), torch.randint(5, v, (a.batch, a.tail_len), generator=g)], 1)

    def timed():
        model.set_input(ids, max_length=ids.shape[1] + a.output_len, num_beams=a.num_beams)
        t0 = time.perf_counter()
        model.forward()
        first = (time.perf_counter() - t0) * 1e3
        while not model.is_done():
            model.forward()
        return model.finalize(), first

    base, t_base = timed()
    model.prefix_sharing(prefix)
    shared, t_shared = timed()
    model.disable_prefix_sharing()
    print(f"identical: {torch.equal(base, shared)}; first token {t_base:.1f} ms -> {t_shared:.1f} ms with the shared prefix")
    if tok is not None:
        print(tok.decode(shared[0, ids.shape[1]:].tolist(), skip_special_tokens=True))


if __name__ == "__main__":
    main()
