#!/usr/bin/env python
"""Prefix-sharing A/B (reference: ``examples/pytorch/prefix_sharing.py:113-170``): the same prompts with and without
a shared cached prefix must give identical tokens, and the first-token time drops.

    python examples/pytorch/prefix_sharing.py -m <model dir> [--prefix_len 512] [--tail_len 32]
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
    ap.add_argument("--prefix_len", type=int, default=512)
    ap.add_argument("--tail_len", type=int, default=32)
    ap.add_argument("--batch", type=int, default=4)
    a = ap.parse_args()
    import torch

    import xfastertransformer_b200 as xft
    model = xft.AutoModel.from_pretrained(a.model_path, dtype=a.dtype)
    g = torch.Generator().manual_seed(0)
    v = model.model.cfg.vocab_size
    prefix = torch.randint(5, v, (1, a.prefix_len), generator=g)
    ids = torch.cat([prefix.expand(a.batch, -1), torch.randint(5, v, (a.batch, a.tail_len), generator=g)], 1)

    def timed():
        model.set_input(ids, max_length=ids.shape[1] + 16)
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


if __name__ == "__main__":
    main()
