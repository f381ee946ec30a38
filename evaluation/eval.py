#!/usr/bin/env python
"""Accuracy evaluation hook (reference: ``evaluation/eval.cpp:31-139`` + ``eval.py`` / ``eval_models.py`` — a pybind
module returning all-position logits to lm-evaluation-harness).  Here ``AutoModel.__call__`` already returns all-position
logits, so the adapter is Python only:

* `XFTEvalModel` — the primitives the harness needs: ``loglikelihood_tokens`` (sum of target log-probs + greedy match),
  the same for a batch of requests in one forward (``loglikelihood_batch``), ``rolling_loglikelihood`` (total
  log-likelihood of a long text in windows) and ``generate_until`` (greedy, cut at stop strings);
* `perplexity(model, ids)` — token-level perplexity of a tensor of ids;
* with ``lm_eval`` installed: ``python evaluation/eval.py -m <dir> -t <tokenizer> --tasks lambada_openai``
  (several GPUs: the same under torchrun; rank 0 evaluates, the other ranks follow).
"""
import argparse
import math
import os
import sys
from typing import List, Sequence, Tuple

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class XFTEvalModel:
    def __init__(self, model, max_length: int = 2048, batch_size: int = 8):
        self.model, self.max_length, self.batch_size = model, max_length, batch_size

    @staticmethod
    def _score(logits: torch.Tensor, ids: Sequence[int], n: int) -> Tuple[float, bool]:
        """logits [len(ids), vocab] of one sequence; the last n tokens are the continuation."""
        lp = torch.log_softmax(logits[-n - 1:-1].float(), -1)
        tgt = torch.tensor(list(ids[-n:]), device=lp.device)
        return lp.gather(1, tgt[:, None]).sum().item(), bool((lp.argmax(-1) == tgt).all())

    @torch.no_grad()
    def loglikelihood_tokens(self, context, continuation) -> Tuple[float, bool]:
        """(sum log p(continuation | context), continuation is the greedy choice).  The context is cut from the left
        when the pair is longer than max_length, as the harness does."""
        ids = (list(context) + list(continuation))[-self.max_length:]
        n = min(len(continuation), len(ids) - 1)
        return self._score(self.model(torch.tensor([ids]))[0], ids, n)

    @torch.no_grad()
    def loglikelihood_batch(self, pairs: Sequence[Tuple[Sequence[int], Sequence[int]]]) -> List[Tuple[float, bool]]:
        """Several (context, continuation) pairs per forward: prompts of different length run as one ragged batch."""
        out: List[Tuple[float, bool]] = [None] * len(pairs)
        order = sorted(range(len(pairs)), key=lambda i: -(len(pairs[i][0]) + len(pairs[i][1])))
        for s in range(0, len(order), self.batch_size):
            idxs = order[s:s + self.batch_size]
            seqs = [(list(pairs[i][0]) + list(pairs[i][1]))[-self.max_length:] for i in idxs]
            logits = self.model(seqs)
            if logits.dim() == 3:                                   # equal lengths: [batch, seq, vocab]
                rows = [logits[j] for j in range(len(seqs))]
            else:                                                   # ragged: rows of all sequences, concatenated
                offs = [0]
                for q in seqs:
                    offs.append(offs[-1] + len(q))
                rows = [logits[offs[j]:offs[j + 1]] for j in range(len(seqs))]
            for j, i in enumerate(idxs):
                out[i] = self._score(rows[j], seqs[j], min(len(pairs[i][1]), len(seqs[j]) - 1))
        return out

    @torch.no_grad()
    def rolling_loglikelihood(self, ids: Sequence[int], prefix_token: int = None) -> float:
        """Total log-likelihood of `ids` in disjoint windows of max_length tokens, each window conditioned on the token
        before it (the first on `prefix_token`, if given)."""
        ids = list(ids)
        total, prev = 0.0, prefix_token
        for s in range(0, len(ids), self.max_length):
            win = ids[s:s + self.max_length]
            ctx = [prev] if prev is not None else []
            if not ctx and len(win) < 2:
                break
            seq = ctx + win
            n = len(win) if ctx else len(win) - 1
            total += self._score(self.model(torch.tensor([seq]))[0], seq, n)[0]
            prev = win[-1]
        return total

    @torch.no_grad()
    def generate_until(self, ids: Sequence[int], decode, until: Sequence[str] = (), max_gen_toks: int = 64,
                       eos_token_id: int = -1) -> str:
        """Greedy continuation of `ids`, cut at the first stop string; `decode` maps token ids to text."""
        room = max(self.max_length - max_gen_toks, 1)
        ids = list(ids)[-room:]
        o = self.model.generate(torch.tensor([ids]), max_length=len(ids) + max_gen_toks, eos_token_id=eos_token_id)
        text = decode([t for t in o[0, len(ids):].tolist() if t != eos_token_id])
        cut = min((text.find(u) for u in until if u and u in text), default=-1)
        return text[:cut] if cut >= 0 else text


@torch.no_grad()
def perplexity(model, ids: torch.Tensor, window: int = 1024) -> float:
    nll, cnt = 0.0, 0
    for s in range(0, ids.numel() - 1, window):
        chunk = ids[s:s + window + 1]
        if chunk.numel() < 2:
            break
        logits = model(chunk[None, :-1])[0]
        lp = torch.log_softmax(logits.float(), -1)
        nll -= lp.gather(1, chunk[1:, None].to(lp.device)).sum().item()
        cnt += chunk.numel() - 1
    return math.exp(nll / max(cnt, 1))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model_path", required=True)
    ap.add_argument("-t", "--token_path", default="")
    ap.add_argument("-d", "--dtype", default="bf16")
    ap.add_argument("--tasks", default="")
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--max_length", type=int, default=2048)
    ap.add_argument("--limit", type=float, default=None, help="lm-eval: examples per task (or a fraction)")
    ap.add_argument("--ids_file", default="", help="text file of whitespace-separated token ids for perplexity")
    a = ap.parse_args()
    import xfastertransformer_b200 as xft
    model = xft.AutoModel.from_pretrained(a.model_path, dtype=a.dtype)
    if model.rank != 0:
        model.follow()                    # executes rank 0's forward / generate calls until shutdown
        return
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

        tok = AutoTokenizer.from_pretrained(a.token_path, trust_remote_code=True)
        ev = XFTEvalModel(model, a.max_length, a.batch_size)
        eos = tok.eos_token_id if tok.eos_token_id is not None else -1

        class Adapter(LM):
            def loglikelihood(self, requests):
                pairs = []
                for r in requests:
                    ctx = tok.encode(r.args[0]) if r.args[0] else [eos]
                    pairs.append((ctx, tok.encode(r.args[1], add_special_tokens=False)))
                return ev.loglikelihood_batch(pairs)

            def loglikelihood_rolling(self, requests):
                return [(ev.rolling_loglikelihood(tok.encode(r.args[0], add_special_tokens=False), eos),) for r in requests]

            def generate_until(self, requests):
                outs = []
                for r in requests:
                    kw = r.args[1] if len(r.args) > 1 and isinstance(r.args[1], dict) else {}
                    until = kw.get("until", [])
                    until = [until] if isinstance(until, str) else list(until)
                    outs.append(ev.generate_until(tok.encode(r.args[0]), lambda t: tok.decode(t, skip_special_tokens=True),
                                                  until, int(kw.get("max_gen_toks", 64)), eos))
                return outs

        print(simple_evaluate(model=Adapter(), tasks=a.tasks.split(","), limit=a.limit)["results"])


if __name__ == "__main__":
    main()
