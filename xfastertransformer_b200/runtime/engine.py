"""Generation driver — the reference's ``xft::Model`` (``include/models.h:25-128``,
``src/models/models.cpp``) re-designed around a paged cache and a single control message.

API parity (same names and meaning as the torch custom class of the reference,
``src/pytorch/auto_model.h:23-360``): ``set_input / config / input / forward(=generate step) /
is_done / finalize / set_input_cb / forward_cb / free_seqs / set_prefix / unset_prefix``.

Multi-rank protocol: rank 0 drives; every state-changing call ships ONE self-describing message
``(opcode, payload)``; follower ranks call the same API (arguments ignored) or simply loop on
``generate()`` and execute whatever arrives — they never have to guess which code path rank 0
took (the reference's followers must, ``models.cpp:202-253`` vs ``:706-717``).  Forward steps
carry no message: all ranks run the same deterministic step.  A shutdown opcode replaces the
poison values of ``models.cpp:80-96``.

Differences by design: greedy, sampling and beam search all run on the continuous-batching path
(the reference's CB ``generate()`` throws for sampling/beams, ``models.cpp:868-884``); prefix
sharing works on this path too via shared cache blocks.
"""
from __future__ import annotations

import sys
import time
from typing import List, Optional, Sequence

import torch

from .. import ops
from ..config import KV_DTYPES, ModelConfig, split_hybrid_dtype
from ..models.decoder import Batch, Decoder
from ..parallel.dist import CommError, DistContext
from ..utils import log, trace
from ..utils.flags import Env
from ..utils.trace import TimeLine
from ..utils.watchdog import StepTimeout, StepWatchdog  # noqa: F401  (StepTimeout is re-exported)
from . import sampler as S
from .kv_cache import PagedKVCache
from .sequence import SamplingMeta, SequenceMeta, SequencePool

OP_SET_INPUT, OP_CONFIG, OP_INPUT, OP_SET_INPUT_CB, OP_FREE_SEQS, OP_SET_PREFIX, OP_UNSET_PREFIX, OP_SHUTDOWN, \
    OP_FINALIZE, OP_LOGITS_ALL = range(10)


def _to_lists(ids) -> List[List[int]]:
    if ids is None:
        return []
    if isinstance(ids, torch.Tensor):
        if ids.dim() == 1:
            ids = ids.unsqueeze(0)
        return [[int(t) for t in row] for row in ids.tolist()]
    if ids and isinstance(ids[0], int):
        return [list(ids)]
    return [list(r) for r in ids]


class Model:
    def __init__(self, path: str, dtype: str = "bf16", kv_cache_dtype: str = "fp16",
                 ctx: Optional[DistContext] = None):
        if kv_cache_dtype not in KV_DTYPES:
            raise ValueError(f"don't support KV cache data type: {kv_cache_dtype}.")
        self.ctx = ctx or DistContext.get()
        self.cfg = ModelConfig.from_ini(path)
        self.env = Env.get()
        d_prefill, d_decode = split_hybrid_dtype(dtype)
        if self.cfg.model_type == "deepseek_moe" and d_prefill not in ("bf16", "fp8_e4m3"):
            raise ValueError("deepseek_moe supports bf16 and fp8_e4m3 only")      # model_factory.h:105-114
        if d_prefill == "fp8_e4m3" and self.cfg.model_type != "deepseek_moe":
            raise ValueError("fp8_e4m3 is supported for deepseek_moe only")
        with TimeLine("Model.load"):
            self.decoder = Decoder(self.cfg, self.ctx, path, d_decode)
            # hybrid A_B: model A serves the first token, B the next ones; they share embedding,
            # head, KV cache and buffers (src/models/hybrid_model.h:23-105)
            self.prefill_decoder = self.decoder if d_prefill == d_decode else \
                Decoder(self.cfg, self.ctx, path, d_prefill, embed_from=self.decoder)
        geo = self.decoder.kv_geometry()
        self.cache = PagedKVCache(len(self.decoder.layers), geo["kv_heads"], geo["k_dim"], geo["v_dim"],
                                  kv_cache_dtype, self.ctx.device, self.env.kv_block_size,
                                  self.decoder.act_dtype, geo["latent"])
        if self.env.prefix_cache and self.ctx.dp_size == 1:
            # data-parallel attention keeps each sequence's cache on one rank only, while all ranks must agree on how
            # many tokens a prompt still has to run: automatic reuse stays off there
            from .kv_cache import PrefixIndex
            self.cache.prefix_index = PrefixIndex(self.cache)
        self.pool = SequencePool()
        self.sampling = SamplingMeta()
        self._greedy_cfg = SamplingMeta()
        self._cb_greedy = False
        self.working: List[SequenceMeta] = []          # sequences of the current request (batch API)
        self.cb_active: List[SequenceMeta] = []        # sequences of the last set_input_cb
        self.rng = S.Philox(None)
        self.scorer: Optional[S.BeamSearchScorer] = None
        self.prefix_seq: Optional[SequenceMeta] = None
        self._prompts: List[List[int]] = []
        self._closed = False
        self.vocab_sizes = [self._vocab_size_of(r) for r in range(self.ctx.tp_size)]
        self.runner = None
        if self.ctx.device.type == "cuda" and self.ctx.tp_size > 1 and self.env.fused_comm and self.ctx.peer is None \
                and self.ctx.tp_size <= 8:
            from ..parallel.fused_comm import PeerComm
            self.ctx.peer = PeerComm(self.ctx, n_max=self.cfg.hidden_size)
        if self.ctx.device.type == "cuda" and self.ctx.dp_size > 1 and self.env.moe_fused_a2a and self.decoder.has_moe \
                and self.ctx.epcomm is None and self.ctx.dp_size <= 8:
            from ..parallel.fused_comm import EpComm
            self.ctx.epcomm = EpComm(self.ctx, self.cfg.hidden_size, self.cfg.num_experts_per_tok)
        if self.ctx.device.type == "cuda":
            from .cuda_runner import CudaRunner
            self.runner = CudaRunner(self)
        if self.env.kv_cache_gb > 0:
            # size the KV pools once: pools that never grow never move, so captured decode graphs stay valid
            per = max(self.cache.bytes_per_block(), 1)
            self.cache.ensure_blocks(max(int(self.env.kv_cache_gb * (1 << 30)) // per, 1))
        self.step_times_ms: List[float] = []
        self.spec_steps = self.spec_emitted = self.spec_accepted = 0      # n-gram speculative decoding counters
        # XFT_STEP_TIMEOUT_S > 0: a monitor thread reports a step that runs over (log + stack dump) and the step raises
        # StepTimeout when it returns
        self.watchdog = StepWatchdog(self.env.step_timeout_s)

    # ------------------------------------------------------------------------------------
    def _vocab_size_of(self, r: int) -> int:
        from ..parallel.partition import vocab_range
        a, b = vocab_range(self.cfg.vocab_size, self.ctx.tp_size, r)
        return b - a

    @property
    def rank(self) -> int:
        return self.ctx.rank

    def get_rank(self) -> int:
        return self.ctx.rank

    # ------------------------------------------------------------------------------------
    # control plane
    # ------------------------------------------------------------------------------------
    def _sync(self, op: int, payload):
        """Rank 0 sends (op, payload); followers receive and return what rank 0 sent."""
        if self.ctx.world == 1:
            return op, payload
        msg = self.ctx.ctrl_broadcast((op, payload) if self.ctx.is_master else None)
        return msg

    def _dispatch(self, op: int, payload):
        if op == OP_SET_INPUT:
            return self._do_set_input(*payload)
        if op == OP_CONFIG:
            return self._do_config(payload)
        if op == OP_INPUT:
            return self._do_input(payload)
        if op == OP_SET_INPUT_CB:
            return self._do_set_input_cb(*payload)
        if op == OP_FREE_SEQS:
            return self._do_free_seqs(payload)
        if op == OP_SET_PREFIX:
            return self._do_set_prefix(payload)
        if op == OP_UNSET_PREFIX:
            return self._do_unset_prefix()
        if op == OP_LOGITS_ALL:
            return self._do_logits_all(payload)
        if op == OP_SHUTDOWN:
            self._closed = True
            if not self.ctx.is_master:
                log.info(f"rank {self.ctx.rank}: shutdown received")
                sys.exit(0)
            return None
        raise RuntimeError(f"unknown control opcode {op}")

    def _call(self, op: int, payload):
        op, payload = self._sync(op, payload)
        return self._dispatch(op, payload)

    def exit_slaves(self) -> None:
        """Tell follower ranks to leave their serving loop (models.cpp:80-96)."""
        if self.ctx.world > 1 and self.ctx.is_master and not self._closed:
            try:
                self._sync(OP_SHUTDOWN, None)
            except CommError:
                pass
        self._closed = True

    # ------------------------------------------------------------------------------------
    # batch API (set_input / config+input / forward / is_done / finalize)
    # ------------------------------------------------------------------------------------
    def set_input(self, input_ids=None, max_length=20, num_beams=1, num_return_sequences=1, length_penalty=1.0,
                  early_stopping=False, eos_token_id=-1, pad_token_id=-1, do_sample=False, temperature=1.0,
                  top_k=50, top_p=1.0, repetition_penalty=1.0, stop_words_ids=None, seed=None, **kw):
        cfg = SamplingMeta(max_length, num_beams, num_return_sequences, length_penalty, early_stopping, eos_token_id,
                           pad_token_id, do_sample, temperature, top_k, top_p, repetition_penalty,
                           stop_words_ids or [], seed)
        return self._call(OP_SET_INPUT, (_to_lists(input_ids), cfg))

    def config(self, max_length=20, num_beams=1, num_return_sequences=1, length_penalty=1.0, early_stopping=False,
               eos_token_id=-1, pad_token_id=-1, do_sample=False, temperature=1.0, top_k=50, top_p=1.0,
               repetition_penalty=1.0, stop_words_ids=None, seed=None, **kw):
        cfg = SamplingMeta(max_length, num_beams, num_return_sequences, length_penalty, early_stopping, eos_token_id,
                           pad_token_id, do_sample, temperature, top_k, top_p, repetition_penalty,
                           stop_words_ids or [], seed)
        return self._call(OP_CONFIG, cfg)

    def input(self, input_ids=None):
        return self._call(OP_INPUT, _to_lists(input_ids))

    def _do_config(self, cfg: SamplingMeta):
        if cfg.eos_token_id == -1:
            cfg.eos_token_id = self.cfg.end_id
        if cfg.pad_token_id == -1:
            cfg.pad_token_id = cfg.eos_token_id
        cfg.clean_stop_words()
        self.sampling = cfg
        self.rng = S.Philox(cfg.seed if cfg.seed is not None else
                            (int(time.time()) if self.ctx.world == 1 else 1234))

    def _do_input(self, prompts: List[List[int]]):
        self._release_working()
        cfg = self.sampling
        if not prompts:
            raise ValueError("input_ids is empty")
        self._prompts = prompts
        nb = max(cfg.num_beams, 1)
        dp, me = self.ctx.dp_size, self.ctx.dp_rank          # data-parallel attention: a rank caches only its own requests
        seqs = []
        for g, p in enumerate(prompts):
            if len(p) >= cfg.max_length:
                log.warning(f"prompt {g}: length {len(p)} >= max_length {cfg.max_length}")
            s = self.pool.new(p, max(cfg.max_length, len(p) + 1), group=g, owner=g % self.ctx.dp_size)
            self.cache.add_sequence(s.seq_id)
            self._attach_prefix(s)                # before the reservation: adopted blocks must not be evicted for it
            seqs.append(s)
        total_blocks = sum(self.cache.blocks_for(max(cfg.max_length, len(p)) + 1)
                           for g, p in enumerate(prompts) if g % dp == me) * nb
        self.cache.reserve(total_blocks)
        self.working = seqs
        self.scorer = None
        self._beam_pending = nb > 1

    def _do_set_input(self, prompts, cfg):
        self._do_config(cfg)
        self._do_input(prompts)

    def _attach_prefix(self, s: SequenceMeta) -> None:
        """Share the cached prefix blocks if the prompt starts with the prefix (prefix sharing,
        src/models/common_decoder.h:337-353,695-771)."""
        pre = self.prefix_seq
        if pre is None:
            idx = self.cache.prefix_index
            if idx is not None and s.past_len == 0 and len(s.pending) == len(s.prompt):
                blocks = idx.lookup(s.prompt)
                if blocks:
                    n = self.cache.adopt(s.seq_id, blocks)
                    s.past_len = s.prefix_len = n
                    s.pending = s.prompt[n:]
            return
        n = len(pre.prompt)
        if len(s.prompt) > n and s.prompt[:n] == pre.prompt:
            self.cache.fork(pre.seq_id, s.seq_id)
            s.past_len = n
            s.prefix_len = n
            s.pending = s.prompt[n:]

    def is_done(self) -> bool:
        if self.scorer is not None:
            return self.scorer.is_done or all(s.done for s in self.working)
        return all(s.done for s in self.working) if self.working else True

    def forward(self) -> torch.Tensor:
        """One generation step for the current request: returns the next token per sequence
        (``Model::generate``, models.cpp:834-902).  Finished rows keep emitting eos."""
        cfg = self.sampling
        seqs = self.working
        if not seqs:
            raise RuntimeError("forward() before set_input()/input()")
        t0 = time.perf_counter()
        with self.watchdog.scope("forward"):
            if cfg.num_beams > 1:
                out = self._beam_step()
            else:
                active = [x for x in seqs if not x.done]
                if not active:
                    out = torch.full((len(seqs),), cfg.eos_token_id, dtype=torch.int64)
                elif self._spec_ok(active, cfg) and self._spec_step(active, cfg):
                    out = torch.tensor([s.generated[-1] if s.generated else cfg.eos_token_id for s in seqs],
                                       dtype=torch.int64)
                elif self.runner is not None and self.runner.can_run(active, cfg):
                    toks = self.runner.step(active, cfg)
                    out = self._commit(seqs, toks, cfg)
                else:
                    local = self._run(active)
                    toks = self._select(local, active, cfg).tolist()
                    out = self._commit(seqs, toks, cfg)
        self.step_times_ms.append((time.perf_counter() - t0) * 1e3)
        return out

    # -- n-gram speculative decoding (greedy only) -----------------------------------------------
    def _spec_ok(self, seqs: Sequence[SequenceMeta], cfg: SamplingMeta) -> bool:
        return (self.env.spec_ngram > 0 and not cfg.do_sample and cfg.num_beams == 1 and cfg.repetition_penalty == 1.0
                and self.ctx.pp_size == 1 and self.ctx.dp_size == 1 and self.decoder.spec.rope != "2d"
                and all(len(s.pending) == 1 and s.past_len > 0 for s in seqs))

    @staticmethod
    def _ngram_draft(tokens: List[int], k: int, window: int = 1024) -> List[int]:
        """Up to k tokens that followed the most recent earlier occurrence of the current suffix (3, 2 or 1 tokens)."""
        n_tok = len(tokens)
        lo = max(0, n_tok - window)
        for n in (3, 2, 1):
            if n_tok <= n:
                continue
            pat = tokens[-n:]
            for i in range(n_tok - n - 1, lo - 1, -1):
                if tokens[i:i + n] == pat:
                    return tokens[i + n:i + n + k]
        return []

    def _draft_for(self, s: SequenceMeta, k: int) -> List[int]:
        """`_ngram_draft` for a live sequence, in time independent of its length: the sequence carries a table from
        every 1-, 2- and 3-gram that has a successor to the position of that successor (latest occurrence wins), which
        is extended by the few tokens that arrived since the last step."""
        toks = s.all_tokens()
        n_tok = len(toks)
        table = s.__dict__.setdefault("_ngrams", {})
        upto = s.__dict__.get("_ngrams_upto", 0)
        for j in range(upto, n_tok - 1):                     # n-grams ending at j have the successor toks[j + 1]
            for n in (1, 2, 3):
                if j + 1 >= n:
                    table[tuple(toks[j - n + 1:j + 1])] = j + 1
        s.__dict__["_ngrams_upto"] = max(upto, n_tok - 1)
        for n in (3, 2, 1):
            if n_tok > n:
                pos = table.get(tuple(toks[-n:]))
                if pos is not None:
                    return toks[pos:pos + k]
        return []

    def _spec_step(self, seqs: Sequence[SequenceMeta], cfg: SamplingMeta) -> bool:
        """One decode step that may emit several tokens per sequence.  Each sequence proposes draft tokens from its own
        history; one forward scores the pending token and the drafts; the longest draft prefix that greedy decoding
        would have produced itself is kept, plus the token after it, and the cache positions of rejected drafts are
        dropped.  The result is exactly plain greedy decoding (a decode step is bound by the weight stream, so a few
        extra rows are nearly free).  Returns False when no sequence had a draft: the caller runs a normal step."""
        k = self.env.spec_ngram
        drafts = []
        for s in seqs:
            room = s.max_len - s.total_len - 1               # tokens that may still follow the one after the draft
            drafts.append(self._draft_for(s, min(k, room)) if room > 0 else [])
        if not any(drafts):
            return False
        for s, e in zip(seqs, self._spec_score(seqs, drafts)):
            for t in e:
                s.step_forward(t)
                self.spec_emitted += 1
                if t == cfg.eos_token_id or s.total_len >= s.max_len or \
                        (cfg.stop_words and S.match_stop_words(s.generated, cfg.stop_words)):
                    s.done = True
                    break
            self.cache.truncate(s.seq_id, s.past_len)        # positions of rejected drafts are written again later
        self.spec_steps += 1
        return True

    def _spec_score(self, seqs: Sequence[SequenceMeta], drafts: List[List[int]]) -> List[List[int]]:
        """One forward over every sequence's pending token followed by its drafts.  Returns per sequence the tokens
        greedy decoding emits from here: the drafts it would have chosen itself, then its own next token.  The
        sequences come back as they went in (same past length, the one pending token); the cache holds the draft
        positions too, and the caller truncates it to what it keeps."""
        starts = [s.past_len for s in seqs]
        lasts = [s.pending[0] for s in seqs]
        for s, d in zip(seqs, drafts):
            s.pending = s.pending + d
        local = self._run(seqs, logits_all=True)             # one row per pending token, sequence after sequence
        preds = S.greedy_select(local, self.decoder.v0, self.ctx).cpu().tolist()
        out, row = [], 0
        for s, d, p0, last in zip(seqs, drafts, starts, lasts):
            p = preds[row:row + 1 + len(d)]
            row += 1 + len(d)
            acc = 0
            while acc < len(d) and int(p[acc]) == d[acc]:
                acc += 1
            s.past_len, s.pending = p0, [last]
            self.spec_accepted += acc
            out.append(d[:acc] + [int(p[acc])])
        return out

    def _select(self, local: torch.Tensor, seqs: Sequence[SequenceMeta], cfg: SamplingMeta) -> torch.Tensor:
        d = self.decoder
        if cfg.repetition_penalty != 1.0:
            local = S.apply_repetition_penalty(local, [s.all_tokens() for s in seqs], cfg.repetition_penalty, d.v0)
        if not cfg.do_sample:
            return S.greedy_select(local, d.v0, self.ctx).cpu()
        full = S.gather_logits(local, self.ctx, self.vocab_sizes)
        return S.sample_select(full, cfg, self.rng).cpu()

    def _commit(self, seqs, toks: List[int], cfg: SamplingMeta) -> torch.Tensor:
        """`toks` holds one token per not-yet-done sequence, in order."""
        out = []
        it = iter(toks)
        for s in seqs:
            if s.done:
                out.append(cfg.eos_token_id)
                continue
            t = int(next(it))
            s.step_forward(t)
            # stopCheck (sampling.cpp:134-154): eos, or total_len + 1 >= max_len
            if t == cfg.eos_token_id or s.total_len >= s.max_len or \
                    (cfg.stop_words and S.match_stop_words(s.generated, cfg.stop_words)):
                s.done = True
            out.append(t)
        return torch.tensor(out, dtype=torch.int64)

    # -- beams ------------------------------------------------------------------------------
    def _beam_step(self) -> torch.Tensor:
        cfg = self.sampling
        nb = cfg.num_beams
        if self._beam_pending:
            # prefill once per request, then fork each into num_beams cache-sharing sequences
            reqs = self.working
            local = self._run(reqs)
            full = S.gather_logits(local, self.ctx, self.vocab_sizes).float()
            for s in reqs:
                s.past_len += len(s.pending)
                s.pending = []
            beams = []
            for s in reqs:
                beams.append(s)
                for _ in range(nb - 1):
                    c = self.pool.new(s.prompt, s.max_len, group=s.group, owner=s.owner)      # beams stay with their request
                    c.past_len, c.pending = s.past_len, []
                    self.cache.fork(s.seq_id, c.seq_id)
                    beams.append(c)
            self.working = beams
            self.scorer = S.BeamSearchScorer(len(reqs), cfg, [len(s.prompt) for s in reqs])
            full = full.repeat_interleave(nb, 0)
            self._beam_pending = False
        else:
            local = self._run(self.working)
            full = S.gather_logits(local, self.ctx, self.vocab_sizes).float()
        if cfg.repetition_penalty != 1.0:
            full = S.apply_repetition_penalty(full, [s.prompt + g for s, g in zip(self.working, self.scorer.seqs)],
                                              cfg.repetition_penalty, 0)
        # The vocabulary stays where the logits are: each beam's log-softmax and its 2 x beams best continuations are
        # found there, and only those pairs reach the scorer on the host.
        k = min(2 * nb, full.shape[-1])
        if k <= S.BEAM_TOPK_MAX:
            toks, src = self.scorer.process_topk(*ops.beam_topk(full, k))
        else:
            toks, src = self.scorer.process(torch.log_softmax(full.cpu(), -1))
        ids = [s.seq_id for s in self.working]
        self.cache.reorder(ids, src.tolist())                 # beam reorder = block-table permutation
        old_gen = [list(s.generated) for s in self.working]
        for i, s in enumerate(self.working):
            s.generated = old_gen[int(src[i])] + [int(toks[i])]
            s.past_len = self.cache.lens[s.seq_id]
            s.pending = [int(toks[i])]
            if s.total_len >= s.max_len:
                s.done = True
        return toks

    def finalize(self) -> torch.Tensor:
        """prompt+generated of every sequence, padded to a rectangle (models.cpp:734-758)."""
        cfg = self.sampling
        if self.scorer is not None:
            rows = self.scorer.finalize(self._prompts, cfg.max_length)
        else:
            rows = [s.all_tokens() for s in self.working]
            w = max(len(r) for r in rows) if rows else 0
            pad = cfg.pad_token_id if cfg.pad_token_id >= 0 else cfg.eos_token_id
            rows = [r + [pad] * (w - len(r)) for r in rows]
        self._release_working()
        if trace.enabled():
            trace.dump()
        return torch.tensor(rows, dtype=torch.int64)

    def _release_working(self) -> None:
        for s in self.working:
            self.cache.free_sequence(s.seq_id)
            self.pool.remove(s.seq_id)
        self.working = []
        self.scorer = None
        if self.runner is not None:
            self.runner.reset()

    # ------------------------------------------------------------------------------------
    # continuous-batching API
    # ------------------------------------------------------------------------------------
    def set_input_cb(self, input_ids=None, seq_lens=None, seq_ids=None, max_length=None, greedy: bool = False,
                     append: bool = False, hold: bool = False, extend: bool = False) -> torch.Tensor:
        """Prefill: ``input_ids`` = flattened prompts + ``seq_lens``; decode: ``input_ids`` [bs,1] +
        ``seq_ids``.  Returns the sequence ids (models.cpp:586-674).  ``greedy=True`` announces that the step will be
        run with ``forward_cb_greedy`` (followers need to know which forward follows).

        Mixed steps (new prompts and running sequences in ONE forward, so decoding does not pause while prompts are
        prefilled): call once with the prompts and ``hold=True`` (followers do not run a forward yet), then once with
        the next tokens and ``append=True``; the logits rows come back in that order.

        Chunked prefill (``extend=True``, with ``seq_ids`` and ``seq_lens``): the tokens continue the PROMPTS of known
        sequences that have not generated anything yet, so a long prompt can be fed in pieces between the decode steps
        of the other sequences.  Create the sequence with its first piece and the ``max_length`` of the whole request;
        the logits of every piece but the last are of no use to the caller."""
        def tl(x):
            if x is None:
                return None
            if isinstance(x, torch.Tensor):
                return [int(v) for v in x.flatten().tolist()]
            if isinstance(x, int):
                return [x]
            return [int(v) for v in (sum(x, []) if x and isinstance(x[0], (list, tuple)) else x)]
        ids = tl(input_ids)
        if seq_lens is None and seq_ids is None and isinstance(input_ids, torch.Tensor) and input_ids.dim() == 2:
            seq_lens = [input_ids.shape[1]] * input_ids.shape[0]
        if seq_lens is None and seq_ids is None and isinstance(input_ids, (list, tuple)) and input_ids and \
                isinstance(input_ids[0], (list, tuple)):
            seq_lens = [len(r) for r in input_ids]
        return self._call(OP_SET_INPUT_CB, (ids, tl(seq_lens), tl(seq_ids), tl(max_length), bool(greedy), bool(append),
                                            bool(hold), bool(extend)))

    def _do_set_input_cb(self, ids, seq_lens, seq_ids, max_len, greedy: bool = False, append: bool = False,
                         hold: bool = False, extend: bool = False) -> torch.Tensor:
        active = []
        self._cb_greedy = bool(greedy)
        self._cb_hold = bool(hold)
        if not seq_ids:                                   # new prompts
            if not seq_lens or sum(seq_lens) != len(ids):
                raise ValueError("set_input_cb: seq_lens do not add up to the number of input ids")
            mls = max_len or [self.cfg.max_pos_seq_len or 2048]
            if len(mls) == 1:
                mls = mls * len(seq_lens)
            off = 0
            for n, m in zip(seq_lens, mls):
                s = self.pool.new(ids[off:off + n], max(m, n + 1))
                s.owner = s.seq_id % self.ctx.dp_size
                off += n
                active.append(s)
            for s in active:
                self.cache.add_sequence(s.seq_id)
                self._attach_prefix(s)            # before the reservation: adopted blocks must not be evicted for it
            # data-parallel attention: a rank caches only the sequences it owns
            self.cache.reserve(sum(self.cache.blocks_for(s.max_len + 1) - len(self.cache.tables[s.seq_id])
                                   for s in active if s.owner == self.ctx.dp_rank))
        elif extend:                                      # further prompt pieces of known sequences
            if not seq_lens or len(seq_lens) != len(seq_ids) or sum(seq_lens) != len(ids):
                raise ValueError("set_input_cb(extend=True): one piece per sequence id, seq_lens adding up to the ids")
            off = 0
            for sid, n in zip(seq_ids, seq_lens):
                s = self.pool.get(sid)
                if s.pending or s.generated:
                    raise RuntimeError(f"sequence {sid}: a prompt grows only between forwards and before generation")
                if len(s.prompt) + n >= s.max_len:
                    raise ValueError(f"sequence {sid}: prompt of {len(s.prompt) + n} tokens exceeds its max_length {s.max_len}")
                piece = ids[off:off + n]
                off += n
                s.prompt = s.prompt + piece
                s.pending = list(piece)
                active.append(s)
        else:                                             # next tokens of known sequences
            if len(ids) != len(seq_ids):
                raise ValueError("set_input_cb: one next token per sequence id expected")
            for sid, t in zip(seq_ids, ids):
                s = self.pool.get(sid)
                if s.pending and s.past_len == 0 and not s.generated:
                    raise RuntimeError(f"sequence {sid} has not been prefilled")
                s.step_forward(int(t))
                active.append(s)
        self.cb_active = (self.cb_active + active) if append else active
        return torch.tensor([s.seq_id for s in active], dtype=torch.int64)

    def forward_cb(self) -> torch.Tensor:
        """fp32 logits [bs, vocab] of the sequences of the last set_input_cb (models.cpp:760-830)."""
        seqs = self.cb_active
        if not seqs:
            raise RuntimeError("forward_cb() before set_input_cb()")
        with self.watchdog.scope("forward_cb"):
            local = self._run(seqs)
            for s in seqs:                      # inputs are now in the cache
                s.past_len += len(s.pending)
                s.pending = []
            return S.gather_logits(local, self.ctx, self.vocab_sizes).float()

    def forward_cb_greedy(self) -> torch.Tensor:
        """Greedy next token [bs] of the sequences of the last ``set_input_cb(..., greedy=True)``, chosen on the device:
        no logits leave the GPU, and a pure decode step replays the captured CUDA graph (one H2D copy, one replay,
        one D2H copy of the tokens).  Extension of the reference's API for serving schedulers."""
        seqs = self.cb_active
        if not seqs:
            raise RuntimeError("forward_cb_greedy() before set_input_cb()")
        if self.ctx.world > 1 and not getattr(self, "_cb_greedy", False):
            raise RuntimeError("forward_cb_greedy() needs set_input_cb(..., greedy=True) on more than one rank")
        cfg = self._greedy_cfg
        if self._spec_ok(seqs, cfg):
            # XFT_SPEC_NGRAM: a decode step may emit several tokens per sequence.  The accepted drafts become part of
            # the sequence here; the caller reads all emitted tokens from `cb_emitted` and feeds back only the last.
            k = self.env.spec_ngram
            drafts = [self._draft_for(s, max(min(k, s.max_len - s.total_len - 1), 0)) for s in seqs]
            if any(drafts):
                with self.watchdog.scope("forward_cb_greedy"):
                    emitted = self._spec_score(seqs, drafts)
                for s, e in zip(seqs, emitted):
                    for t in e[:-1]:
                        s.step_forward(t)
                    s.past_len += len(s.pending)
                    s.pending = []
                    self.cache.truncate(s.seq_id, s.past_len)
                    self.spec_emitted += len(e)
                self.spec_steps += 1
                self.cb_emitted = emitted
                return torch.tensor([e[-1] for e in emitted], dtype=torch.int64)
        with self.watchdog.scope("forward_cb_greedy"):
            if self.runner is not None and self.runner.can_run(seqs, cfg) and self.runner.worth_capturing(seqs):
                toks = self.runner.step(seqs, cfg)
            else:
                local = self._run(seqs)
                toks = S.greedy_select(local, self.decoder.v0, self.ctx).cpu().tolist()
        for s in seqs:
            s.past_len += len(s.pending)
            s.pending = []
        self.cb_emitted = [[int(t)] for t in toks]
        return torch.tensor([int(t) for t in toks], dtype=torch.int64)

    def follow(self) -> None:
        """Follower ranks: execute rank 0's control messages until shutdown, whatever API rank 0 uses.  Forward steps
        carry no message, so the follower runs the ones that rank 0 is bound to run: after ``set_input`` / ``input``
        the decode loop of ``generate`` (``forward`` until ``is_done``), after every ``set_input_cb`` exactly one
        ``forward_cb`` (a serving scheduler does the same) unless the message said hold; all-position logits run
        inside their own message.  The reference's followers sit in ``while True: model.generate()``, which covers the
        first case only (serving/grpc_launcher/server.py:144-152)."""
        if self.ctx.world == 1 or self.ctx.is_master:
            return
        while not self._closed:
            op, payload = self._sync(0, None)
            self._dispatch(op, payload)
            if op in (OP_SET_INPUT, OP_INPUT):
                while not self.is_done():
                    self.forward()
                self.finalize()
            elif op == OP_SET_INPUT_CB and not getattr(self, "_cb_hold", False):
                if getattr(self, "_cb_greedy", False):
                    self.forward_cb_greedy()
                else:
                    self.forward_cb()

    def follow_cb(self) -> None:
        """Follower loop of a continuous-batching server (same loop as `follow`)."""
        self.follow()

    def free_seqs(self, seq_ids=None) -> bool:
        if isinstance(seq_ids, torch.Tensor):
            seq_ids = seq_ids.tolist()
        return self._call(OP_FREE_SEQS, list(seq_ids or []))

    def _do_free_seqs(self, seq_ids) -> bool:
        for sid in seq_ids:
            if sid in self.pool:
                self.cache.free_sequence(sid)
                self.pool.remove(sid)
        self.cb_active = [s for s in self.cb_active if s.seq_id in self.pool]
        if trace.enabled():
            trace.dump()
        return True

    # ------------------------------------------------------------------------------------
    # prefix sharing
    # ------------------------------------------------------------------------------------
    def set_prefix(self, input_ids=None):
        return self._call(OP_SET_PREFIX, _to_lists(input_ids))

    def unset_prefix(self):
        return self._call(OP_UNSET_PREFIX, None)

    def _do_set_prefix(self, prompts):
        self._do_unset_prefix()
        if not prompts or not prompts[0]:
            return
        ids = prompts[0]
        # keep whole blocks only, so sharers never write into a shared block
        n = (len(ids) // self.cache.block) * self.cache.block
        if n == 0:
            return
        if self.ctx.dp_size > 1:
            raise RuntimeError("prefix sharing is not available with XFT_ATTENTION_DP=1 (a prefix lives on one rank)")
        s = self.pool.new(ids[:n], n + 1)
        self.cache.add_sequence(s.seq_id, n)
        self._run([s])
        s.past_len, s.pending = n, []
        self.prefix_seq = s

    def _do_unset_prefix(self):
        if self.prefix_seq is not None:
            self.cache.free_sequence(self.prefix_seq.seq_id)
            self.pool.remove(self.prefix_seq.seq_id)
            self.prefix_seq = None

    # ------------------------------------------------------------------------------------
    # the step
    # ------------------------------------------------------------------------------------
    def make_batch(self, seqs: Sequence[SequenceMeta], logits_all: bool = False) -> Batch:
        dev = self.ctx.device
        ids, pos, slots, cu, kvl, rows = [], [], [], [0], [], []
        for s in seqs:
            n = len(s.pending)
            if n == 0:
                raise RuntimeError(f"sequence {s.seq_id} has no pending input")
            # the cache may already hold this sequence's positions (beam fork) — append after them
            start = s.past_len
            have = self.cache.lens[s.seq_id]
            if have > start:
                self.cache.truncate(s.seq_id, start)
            sl = self.cache.append_slots(s.seq_id, n)
            ids.extend(s.pending)
            pos.extend(range(start, start + n))
            slots.extend(sl)
            cu.append(cu[-1] + n)
            kvl.append(start + n)
            rows.extend(range(cu[-2], cu[-1]) if logits_all else [cu[-1] - 1])
        decode = all(cu[i + 1] - cu[i] == 1 for i in range(len(seqs)))
        bt = self.cache.block_table([s.seq_id for s in seqs])
        i32 = lambda x: torch.tensor(x, dtype=torch.int32).to(dev, non_blocking=True)
        b = Batch(ids=i32(ids), positions=i32(pos), slots=i32(slots), cu_q=cu, kv_lens=kvl, block_table=bt.to(dev),
                  logit_rows=None if (logits_all or decode) else i32(rows).long() if dev.type == "cpu" else i32(rows),
                  is_decode=decode, max_q=max(cu[i + 1] - cu[i] for i in range(len(seqs))), max_kv=max(kvl))
        b.cu_q_dev, b.kv_lens_dev = i32(cu), i32(kvl)
        if self.decoder.spec.rope == "2d":
            self._chatglm_positions(b, seqs)
        return b

    def _chatglm_positions(self, b: Batch, seqs) -> None:
        """ChatGLM-1 2-D positions: position = index up to the [gMASK]/[MASK] slot then frozen;
        block position = 0 in the context, 1,2,... from bos on (src/models/chatglm.cpp:118-206).
        Both mask tokens are honoured (the reference only ever detects gMASK, chatglm.cpp:139)."""
        GMASK, MASK, BOS = 130001, 130000, 130004
        p1, p2, pl = [], [], []
        for s in seqs:
            prompt = s.prompt
            ctx_len = prompt.index(BOS) if BOS in prompt else len(prompt) - 1
            mask_pos = prompt.index(GMASK) if GMASK in prompt else (prompt.index(MASK) if MASK in prompt else ctx_len)
            for p in range(s.past_len, s.past_len + len(s.pending)):
                if p < ctx_len:
                    p1.append(p)
                    p2.append(0)
                else:
                    p1.append(mask_pos)
                    p2.append(p - ctx_len + 1)
            pl.append(ctx_len)
        dev = self.ctx.device
        b.positions = torch.tensor(p1, dtype=torch.int32, device=dev)
        b.positions2 = torch.tensor(p2, dtype=torch.int32, device=dev)
        b.prefix_lm_lens = pl

    def _groups(self, seqs: Sequence[SequenceMeta]) -> List[List[SequenceMeta]]:
        """How one call is cut into forward passes.  Prefill of many long prompts runs in groups of at most
        XFT_MAX_BATCH_TOKENS tokens so the activation footprint stays bounded (each group is a self-contained ragged
        batch).  With pipeline stages, XFT_MAX_REQUEST_NUM > 1 additionally cuts a batch into that many micro-batches
        so the stages work on different micro-batches at the same time (the reference's in-flight request limit,
        src/utils/environment.h:233; src/models/common_decoder.h:384-391)."""
        cap = self.env.max_batch_tokens
        groups = [list(seqs)]
        if len(seqs) > 1 and sum(len(s.pending) for s in seqs) > cap and any(len(s.pending) > 1 for s in seqs):
            groups, cur, n = [], [], 0
            for s in seqs:
                if cur and n + len(s.pending) > cap:
                    groups.append(cur)
                    cur, n = [], 0
                cur.append(s)
                n += len(s.pending)
            groups.append(cur)
        m = self.env.max_request_num
        if self.ctx.pp_size > 1 and m > 1 and len(groups) == 1 and len(seqs) > 1:
            per = (len(seqs) + min(m, len(seqs)) - 1) // min(m, len(seqs))
            groups = [list(seqs[i:i + per]) for i in range(0, len(seqs), per)]
        return groups

    def _run(self, seqs: Sequence[SequenceMeta], logits_all: bool = False) -> torch.Tensor:
        """Run the decoder over the pending inputs of `seqs`; returns this rank's logits slice."""
        if self.ctx.dp_size > 1:
            return self._dp_forward(seqs, logits_all)
        groups = self._groups(seqs)
        if self.ctx.pp_size > 1:
            return self._pp_forward(groups, logits_all)
        if self.env.prefill_overlap and self.ctx.tp_size > 1 and len(seqs) > 1 and all(len(s.pending) > 1 for s in seqs):
            return self._run_overlapped(seqs, groups, logits_all)
        if len(groups) > 1:
            return torch.cat([self._run(g, logits_all) for g in groups], dim=0)
        b = self.make_batch(seqs, logits_all)
        dec = self.decoder if b.is_decode else self.prefill_decoder
        name = "Next Token" if b.is_decode else "1st Token"
        with TimeLine(name), torch.no_grad():
            out = dec.forward(b, self.cache)
        self._remember_prefixes(seqs)
        return out

    def _run_overlapped(self, seqs, groups, logits_all: bool) -> torch.Tensor:
        """Tensor-parallel prefill with XFT_PREFILL_OVERLAP=1: the groups are taken two at a time and interleaved block
        by block (Decoder.forward_pair), so the all-reduce of one group travels while the other one computes.  A single
        group is cut in two halves of about the same number of tokens first."""
        if len(groups) == 1:
            total, acc, cut = sum(len(s.pending) for s in seqs), 0, 1
            for i, s in enumerate(seqs[:-1]):
                acc += len(s.pending)
                cut = i + 1
                if acc * 2 >= total:
                    break
            groups = [list(seqs[:cut]), list(seqs[cut:])]
        outs = []
        dec = self.prefill_decoder
        with torch.no_grad():
            for i in range(0, len(groups) - 1, 2):
                b0, b1 = self.make_batch(groups[i], logits_all), self.make_batch(groups[i + 1], logits_all)
                with TimeLine("1st Token"):
                    o0, o1 = dec.forward_pair(b0, b1, self.cache)
                self._remember_prefixes(groups[i])
                self._remember_prefixes(groups[i + 1])
                outs += [o0, o1]
            if len(groups) % 2:
                b = self.make_batch(groups[-1], logits_all)
                with TimeLine("1st Token"):
                    outs.append(dec.forward(b, self.cache))
                self._remember_prefixes(groups[-1])
        return torch.cat(outs, dim=0)

    def _remember_prefixes(self, seqs: Sequence[SequenceMeta]) -> None:
        """Automatic prefix reuse: the full blocks a prefill has just written become available to later prompts."""
        idx = self.cache.prefix_index
        if idx is None:
            return
        for s in seqs:
            if len(s.pending) > 1 and s.seq_id in self.cache.tables:
                n = s.past_len + len(s.pending)               # tokens of this sequence now in the cache
                idx.insert(s.all_tokens()[:n], self.cache.tables[s.seq_id])

    def _dp_forward(self, seqs: Sequence[SequenceMeta], logits_all: bool) -> torch.Tensor:
        """Data-parallel attention (XFT_ATTENTION_DP=1): every rank runs the decoder on the sequences it owns; inside
        the MoE layers tokens visit the ranks that own their experts (Decoder._moe_dp).  All ranks know all sequences,
        so each one can tell how many passes the busiest rank needs and joins the expert exchange of every pass, with
        or without tokens of its own.  The logits rows are then gathered so that every rank returns the same
        [rows, vocab] tensor, in the order of `seqs`, and steps its sequences identically."""
        ctx = self.ctx
        mine = [s for s in seqs if s.owner == ctx.dp_rank]
        per_rank = [self._groups([s for s in seqs if s.owner == r]) if any(s.owner == r for s in seqs) else []
                    for r in range(ctx.dp_size)]
        n_pass = max(len(g) for g in per_rank)
        my_groups = per_rank[ctx.dp_rank]
        outs = []
        with torch.no_grad():
            for i in range(n_pass):
                ctx.dp_max_tokens = max(sum(len(s.pending) for s in g[i]) if i < len(g) else 0 for g in per_rank)
                if i < len(my_groups):
                    b = self.make_batch(my_groups[i], logits_all)
                    dec = self.decoder if b.is_decode else self.prefill_decoder
                    with TimeLine("Next Token" if b.is_decode else "1st Token"):
                        outs.append(dec.forward(b, self.cache).float())
                else:
                    self.decoder.forward_idle()
        rows_of = (lambda s: len(s.pending)) if logits_all else (lambda s: 1)
        counts = [sum(rows_of(s) for s in seqs if s.owner == r) for r in range(ctx.dp_size)]
        vocab = self.decoder.v1 - self.decoder.v0
        local = torch.cat(outs, dim=0) if outs else torch.zeros(0, vocab, dtype=torch.float32, device=ctx.device)
        assert local.shape[0] == counts[ctx.dp_rank], (local.shape, counts, len(mine))
        parts = ctx.all_gather_rows(local, counts)
        offs = [0] * ctx.dp_size
        rows = []
        for s in seqs:                              # back to the caller's order
            n = rows_of(s)
            rows.append(parts[s.owner][offs[s.owner]:offs[s.owner] + n])
            offs[s.owner] += n
        return torch.cat(rows, dim=0)

    def _pp_forward(self, groups: List[List[SequenceMeta]], logits_all: bool) -> torch.Tensor:
        """Pipeline stages over p2p send / recv of the hidden state (C8).  Every group is one micro-batch: a stage
        posts the receives of all micro-batches up front, runs them in order and sends each result on without
        waiting, so stage s works on micro-batch m while stage s + 1 works on m - 1.  The last stage's logits are
        then shared with the other stages so that every rank selects the same token and steps its sequences (the
        reference returns tokens to stage 0 only, C9)."""
        import torch.distributed as dist
        ctx = self.ctx
        batches = [self.make_batch(g, logits_all) for g in groups]
        decs = [self.decoder if b.is_decode else self.prefill_decoder for b in batches]
        first, last = decs[0].first_stage, decs[0].last_stage
        recvs = []
        if not first:
            for b, dec in zip(batches, decs):
                h = torch.empty(b.ids.shape[0], self.cfg.hidden_size, dtype=dec.act_dtype, device=ctx.device)
                recvs.append((ctx.recv(h, ctx.rank - ctx.tp_size), h))
        outs, sends = [], []
        with torch.no_grad():
            for i, (b, dec) in enumerate(zip(batches, decs)):
                hidden = None
                if not first:
                    recvs[i][0].wait()
                    hidden = recvs[i][1]
                with TimeLine("Next Token" if b.is_decode else "1st Token"):
                    out = dec.forward(b, self.cache, hidden)
                if not last:
                    sends.append((ctx.send(out, ctx.rank + ctx.tp_size), out))     # the tensor stays alive until wait()
                outs.append(out)
        for h, _ in sends:
            h.wait()
        for g in groups:
            self._remember_prefixes(g)
        self.pp_microbatches = getattr(self, "pp_microbatches", 0) + len(batches)
        # same tp_rank column across stages
        src = (ctx.pp_size - 1) * ctx.tp_size + ctx.tp_rank
        grp = self._pp_column_group()
        res = []
        for b, dec, out in zip(batches, decs, outs):
            rows = b.num_seqs if b.logit_rows is not None or b.is_decode else b.ids.shape[0]
            logits = out if last else torch.empty(rows, dec.v1 - dec.v0, dtype=torch.float32, device=ctx.device)
            dist.broadcast(logits, src, group=grp)
            res.append(logits)
        return res[0] if len(res) == 1 else torch.cat(res, dim=0)

    def _pp_column_group(self):
        if not hasattr(self, "_pp_groups"):
            import torch.distributed as dist
            self._pp_groups = {}
            for t in range(self.ctx.tp_size):
                g = dist.new_group([s * self.ctx.tp_size + t for s in range(self.ctx.pp_size)])
                self._pp_groups[t] = g
        return self._pp_groups[self.ctx.tp_rank]

    # ------------------------------------------------------------------------------------
    def forward_logits_all(self, input_ids) -> torch.Tensor:
        """All-position logits of a batch of prompts (evaluation hook; evaluation/eval.cpp:70-139)."""
        return self._call(OP_LOGITS_ALL, _to_lists(input_ids))

    def _do_logits_all(self, prompts) -> torch.Tensor:
        seqs = []
        self.cache.reserve(sum(self.cache.blocks_for(len(p) + 1) for p in prompts))
        for p in prompts:
            s = self.pool.new(p, len(p) + 1)
            s.owner = s.seq_id % self.ctx.dp_size
            self.cache.add_sequence(s.seq_id)
            seqs.append(s)
        local = self._run(seqs, logits_all=True)
        full = S.gather_logits(local, self.ctx, self.vocab_sizes).float()
        for s in seqs:
            self.cache.free_sequence(s.seq_id)
            self.pool.remove(s.seq_id)
        if all(len(p) == len(prompts[0]) for p in prompts):
            return full.view(len(prompts), len(prompts[0]), -1)
        return full

    def __del__(self):
        try:
            self.exit_slaves()
        except Exception:
            pass
