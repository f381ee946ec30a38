"""Token selection: greedy, top-k/top-p sampling, beam search, logits processors.

Reference: ``src/searchers/greedy_search.cpp``, ``sampling.cpp:22-154``, ``sample_search.cpp:118-268``,
``beam_search.cpp:27-564``, ``search_utils.cpp:28-172``.  All functions take this rank's vocab slice
of the logits and finish with identical results on every TP rank:

* greedy — local (max, first index) per row, gather of the (value, id) pairs, strictly-greater
  wins so the lowest rank / lowest id wins ties (``sampling.cpp:103-127``);
* sampling / beams — the slices are gathered into full rows (batch x vocab floats), then every rank
  runs the same deterministic selection with a shared counter-based seed (the reference
  broadcasts rank 0's draw instead, ``sample_search.cpp:249``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..parallel.dist import DistContext
from .sequence import SamplingMeta


def gather_logits(local: torch.Tensor, ctx: DistContext, sizes: Optional[List[int]]) -> torch.Tensor:
    """Vocab-split slices -> full rows (Model::forward allgatherv + reorder, models.cpp:797-826)."""
    return ctx.all_gather_cat(local, sizes, dim=-1)


def greedy_select(local: torch.Tensor, vocab_offset: int, ctx: DistContext) -> torch.Tensor:
    """-> int64 [rows] global token ids."""
    v, i = ops.argmax_rows(local)
    if ctx.tp_size == 1:
        return i.long()
    pair = torch.stack([v.float(), (i + vocab_offset).float()], dim=-1)       # ids exact below 2^24
    peer = getattr(ctx, "peer", None)
    if peer is not None and pair.is_cuda and pair.numel() <= peer.slot:
        allp = peer.all_gather(pair.contiguous())                              # peer-memory kernel, graph-safe
    else:
        allp = ctx.all_gather_cat(pair.unsqueeze(0), None, dim=0)              # [tp, rows, 2]
    vals, ids = allp[..., 0], allp[..., 1]
    best = torch.argmax(vals, dim=0)           # first (lowest rank) maximum
    return ids.gather(0, best[None])[0].long()


def apply_repetition_penalty(local: torch.Tensor, token_lists: Sequence[Sequence[int]], penalty: float,
                             vocab_offset: int) -> torch.Tensor:
    if local.is_cuda:
        from ..ops import native_sample
        if not (local.dtype == torch.float32 and local.stride(-1) == 1):
            local = local.float().contiguous()
        return native_sample.repetition_penalty(local, token_lists, penalty, vocab_offset)
    from ..ops import reference as R
    return R.repetition_penalty(local, token_lists, penalty, vocab_offset)


class Philox:
    """Counter-based uniform stream: (seed, step, row) -> u in [0,1).  Every rank draws the
    same numbers; explicit seeding replaces the reference's std::random_device reseed per step."""

    def __init__(self, seed: Optional[int]):
        import os
        self.seed = int.from_bytes(os.urandom(4), "little") if seed is None else int(seed)
        self.step = 0

    def uniform(self, rows: int) -> torch.Tensor:
        g = torch.Generator()
        g.manual_seed((self.seed * 1000003 + self.step) & 0x7FFFFFFFFFFFFFFF)
        self.step += 1
        return torch.rand(rows, generator=g)


def sample_select(full_logits: torch.Tensor, cfg: SamplingMeta, rng: Philox) -> torch.Tensor:
    u = rng.uniform(full_logits.shape[0])
    return ops.sample_top_k_top_p(full_logits, cfg.top_k, cfg.top_p, cfg.temperature, u).long()


def match_stop_words(tokens: Sequence[int], stop_words: Sequence[Sequence[int]]) -> bool:
    """True if the generated tail equals any stop-word list (search_utils.cpp:28-101)."""
    n = len(tokens)
    for w in stop_words:
        m = len(w)
        if m and m <= n and list(tokens[n - m:]) == list(w):
            return True
    return False


# ------------------------------------------------------------------------------------------
# beam search (HF semantics, as ported by the reference: beam_search.cpp:87-345)
# ------------------------------------------------------------------------------------------
class BeamHypotheses:
    def __init__(self, num_beams: int, length_penalty: float, early_stopping: bool):
        self.num_beams, self.length_penalty, self.early_stopping = num_beams, length_penalty, early_stopping
        self.beams: List[Tuple[float, List[int]]] = []
        self.worst = 1e9

    def add(self, hyp: List[int], sum_logprobs: float, length: int) -> None:
        score = sum_logprobs / (max(length, 1) ** self.length_penalty)
        if len(self.beams) < self.num_beams or score > self.worst:
            self.beams.append((score, hyp))
            if len(self.beams) > self.num_beams:
                self.beams.sort(key=lambda x: x[0])
                del self.beams[0]
                self.worst = self.beams[0][0]
            else:
                self.worst = min(score, self.worst)

    def is_done(self, best_sum_logprobs: float, cur_len: int) -> bool:
        if len(self.beams) < self.num_beams:
            return False
        if self.early_stopping:
            return True
        return self.worst >= best_sum_logprobs / (max(cur_len, 1) ** self.length_penalty)


BEAM_TOPK_MAX = 64          # widest per-beam candidate list of `ops.beam_topk`


class BeamSearchScorer:
    """Per-request beam bookkeeping.  `process` consumes the top 2*num_beams candidates of each
    request and returns the next (scores, tokens, source-beam indices)."""

    def __init__(self, batch: int, cfg: SamplingMeta, prompt_len=0):
        """`prompt_len`: one length or one per request.  Hypotheses are ranked by sum of log-probabilities divided by
        length ** length_penalty where, as in the reference (src/searchers/beam_search.cpp:87-112,137-194: the hypothesis
        is the whole row of input ids), the length is prompt + tokens generated before the closing one."""
        self.bs, self.nb = batch, cfg.num_beams
        self.cfg = cfg
        self.prompt_lens = [int(prompt_len)] * batch if isinstance(prompt_len, int) else [int(x) for x in prompt_len]
        assert len(self.prompt_lens) == batch
        self.hyps = [BeamHypotheses(cfg.num_beams, cfg.length_penalty, cfg.early_stopping) for _ in range(batch)]
        self.done = [False] * batch
        self.beam_scores = torch.zeros(batch, cfg.num_beams)
        self.beam_scores[:, 1:] = -1e9
        self.seqs: List[List[int]] = [[] for _ in range(batch * cfg.num_beams)]   # generated tokens per beam

    @property
    def is_done(self) -> bool:
        return all(self.done)

    def process(self, logprobs: torch.Tensor):
        """logprobs: [bs*nb, vocab] log-softmax of the current step (host tensor)."""
        bs, nb = self.bs, self.nb
        V = logprobs.shape[-1]
        scores = logprobs + self.beam_scores.view(-1, 1)
        scores = scores.view(bs, nb * V)
        top_s, top_i = torch.topk(scores, 2 * nb, dim=1)
        return self._advance(top_s, top_i // V, top_i % V)

    def process_topk(self, logp: torch.Tensor, idx: torch.Tensor):
        """Same step from each beam's own k >= min(2*nb, vocab) best continuations (`ops.beam_topk`): logp, idx
        [bs*nb, k], sorted by value.  The best 2*nb of a request's nb*vocab candidates can take at most 2*nb from one
        beam, so merging the per-beam lists loses nothing; only k values per beam cross to the host instead of the
        vocabulary."""
        bs, nb = self.bs, self.nb
        k = logp.shape[-1]
        scores = (logp.float().cpu() + self.beam_scores.view(-1, 1)).reshape(bs, nb * k)
        top_s, top_i = torch.topk(scores, min(2 * nb, nb * k), dim=1)
        tok = idx.cpu().long().reshape(bs, nb * k).gather(1, top_i)
        return self._advance(top_s, top_i // k, tok)

    def _advance(self, top_s: torch.Tensor, src_beam: torch.Tensor, tok: torch.Tensor):
        """top_s, src_beam, tok: [bs, <= 2*nb] candidates of every request, best first."""
        bs, nb = self.bs, self.nb
        eos, pad = self.cfg.eos_token_id, self.cfg.pad_token_id
        gen = len(self.seqs[0])                        # tokens every open beam has generated so far
        next_tokens = torch.full((bs, nb), pad if pad >= 0 else 0, dtype=torch.long)
        next_src = torch.zeros(bs, nb, dtype=torch.long)
        next_scores = torch.zeros(bs, nb)
        for b in range(bs):
            if self.done[b]:
                next_src[b] = torch.arange(nb)
                next_scores[b] = self.beam_scores[b]
                continue
            k = 0
            cur_len = self.prompt_lens[b] + gen
            for rank in range(top_s.shape[1]):
                t, s, sb = int(tok[b, rank]), float(top_s[b, rank]), int(src_beam[b, rank])
                if t == eos and eos >= 0:
                    if rank >= nb:
                        continue
                    self.hyps[b].add(self.seqs[b * nb + sb] + [t], s, cur_len)
                else:
                    next_tokens[b, k], next_src[b, k], next_scores[b, k] = t, sb, s
                    k += 1
                if k == nb:
                    break
            self.done[b] = self.done[b] or self.hyps[b].is_done(float(top_s[b].max()), cur_len)
        # commit
        new_seqs = []
        for b in range(bs):
            for j in range(nb):
                new_seqs.append(self.seqs[b * nb + int(next_src[b, j])] + [int(next_tokens[b, j])])
        self.seqs = new_seqs
        self.beam_scores = next_scores
        flat_src = (next_src + torch.arange(bs)[:, None] * nb).view(-1)
        return next_tokens.view(-1), flat_src

    def finalize(self, prompts: List[List[int]], max_length: int) -> List[List[int]]:
        bs, nb = self.bs, self.nb
        nret = max(1, min(self.cfg.num_return_sequences, nb))
        out = []
        for b in range(bs):
            if not self.done[b] or len(self.hyps[b].beams) < nret:
                for j in range(nb):
                    self.hyps[b].add(self.seqs[b * nb + j], float(self.beam_scores[b, j]),
                                     self.prompt_lens[b] + len(self.seqs[b * nb + j]))
            best = sorted(self.hyps[b].beams, key=lambda x: x[0], reverse=True)[:nret]
            for _, h in best:
                out.append(prompts[b] + h)
        pad = self.cfg.pad_token_id if self.cfg.pad_token_id >= 0 else max(self.cfg.eos_token_id, 0)
        width = min(max(len(o) for o in out), max_length)
        return [o[:width] + [pad] * (width - len(o[:width])) for o in out]
