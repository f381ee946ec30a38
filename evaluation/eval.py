#!/usr/bin/env python
"""Accuracy evaluation hook (reference: ``evaluation/eval.cpp:31-139`` + ``eval.py`` / ``eval_models.py`` — a pybind
module returning all-position logits to lm-evaluation-harness).  Here ``AutoModel.__call__`` already returns
``[batch, seq, vocab]`` logits, so the adapter is Python only:

* `XFTEvalModel` — the ``loglikelihood`` primitive the harness needs (sum of target log-probs + greedy match);
* `perplexity(model, ids)` — token-level perplexity of a tensor of ids;
* with ``lm_eval`` installed: ``python evaluation/eval.py -m <dir> -t <tokenizer> --tasks lambada_openai``.
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class XFTEvalModel:
    def __init__(self, model, max_length=2048):
        self.model, self.max_length = model, max_length

    @torch.no_grad()
    def loglikelihood_tokens(self, context, continuation):
        """(sum log p(continuation | context), continuation is the greedy choice)."""
        ids = (list(context) + list(continuation))[-self.max_length:]
        n = len(continuation)
        logits = self.model(torch.tensor([ids]))[0]                  # [seq, vocab]
        lp = torch.log_softmax(logits[-n - 1:-1].float(), -1)
        tgt = torch.tensor(ids[-n:])
        ll = lp.gather(1, tgt[:, None]).sum().item()
        return ll, bool((lp.argmax(-1) == tgt).all())


@torch.no_grad()
def perplexity(model, ids: torch.Tensor, window: int = 1024) -> float:
    nll, cnt = 0.0, 0
    for s in range(0, ids.numel() - 1, window):
        chunk = ids[s:s + window + 1]
        if chunk.numel() < 2:
            break
        logits = model(chunk[None, :-1])[0]
        lp = torch.log_softmax(logits.float(), -1)
        nll -= lp.gather(1, chunk[1:, None]).sum().item()
        cnt += chunk.numel() - 1
    return math.exp(nll / max(cnt, 1))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model_path", required=True)
    ap.add_argument("-t", "--token_path", default="")
    ap.add_argument("-d", "--dtype", default="bf16")
    ap.add_argument("--tasks", default="")
    ap.add_argument("--ids_file", default="", help="text file of whitespace-separated token ids for perplexity")
    a = ap.parse_args()
    import xfastertransformer_b200 as xft
    model = xft.AutoModel.from_pretrained(a.model_path, dtype=a.dtype)
    if a.ids_file:
        ids = torch.tensor([int(t) for t in open(a.ids_file).read().split()])
        print(f"perplexity: {perplexity(model, ids):.4f}")
    if a.tasks:
        try:
            import lm_eval  # noqa: F401
        except ImportError:
            sys.exit("lm-evaluation-harness is not installed; use --ids_file or the XFTEvalModel class directly")
        from transformers import AutoTokenizer
        from lm_eval import simple_evaluate
        from lm_eval.api.model import LM

        tok = AutoTokenizer.from_pretrained(a.token_path)
        ev = XFTEvalModel(model)

        class Adapter(LM):
            def loglikelihood(self, requests):
                return [ev.loglikelihood_tokens(tok.encode(r.args[0]), tok.encode(r.args[1], add_special_tokens=False)) for r in requests]

            def loglikelihood_rolling(self, requests):
                return [(-math.log(perplexity(model, torch.tensor(tok.encode(r.args[0])))),) for r in requests]

            def generate_until(self, requests):
                outs = []
                for r in requests:
                    ids = torch.tensor([tok.encode(r.args[0])])
                    o = model.generate(ids, max_length=ids.shape[1] + 64)
                    outs.append(tok.decode(o[0, ids.shape[1]:].tolist()))
                return outs

        print(simple_evaluate(model=Adapter(), tasks=a.tasks.split(","))["results"])


if __name__ == "__main__":
    main()
