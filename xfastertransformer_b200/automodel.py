"""Python ``AutoModel`` — same surface as the reference's
(``src/xfastertransformer/automodel.py:19-264``): ``from_pretrained(path, dtype, kv_cache_dtype)``,
``generate / forward / set_input / config / input / is_done / finalize / set_input_cb /
forward_cb / free_seqs / prefix_sharing / disable_prefix_sharing / rank``.

On rank 0 the arguments drive the run; on follower ranks they are ignored and the call executes
whatever rank 0 broadcast, so ``while True: model.generate()`` is a complete follower loop
(reference README.md:300-328).
"""
from __future__ import annotations

from typing import List, Optional, Union

import torch

from .config import KV_DTYPES, WEIGHT_DTYPES
from .runtime.engine import Model


class AutoModel:
    def __init__(self, path, dtype: str = "fp16", kv_cache_dtype: str = "fp16"):
        if dtype not in WEIGHT_DTYPES:
            raise Exception(f"{self.__class__.__name__} don't support {dtype}.")
        if kv_cache_dtype not in KV_DTYPES:
            raise Exception(f"{self.__class__.__name__} don't support KV cache data type: {kv_cache_dtype}.")
        self.model = Model(path, dtype, kv_cache_dtype)

    @classmethod
    def from_pretrained(cls, path, dtype: str = "fp16", kv_cache_dtype: str = "fp16"):
        return cls(path, dtype, kv_cache_dtype)

    def __call__(self, inputs, **kwargs):
        """All-position logits [bs, seq, vocab] (torch binding ``forward``, auto_model.h:160-190)."""
        return self.model.forward_logits_all(inputs)

    @property
    def rank(self):
        return self.model.get_rank()

    # -- continuous batching ------------------------------------------------------------
    def set_input_cb(self, input_ids: Optional[Union[List[int], List[List[int]], torch.Tensor]] = None,
                     seq_ids: Optional[Union[List[int], torch.Tensor]] = None,
                     max_length: Optional[Union[int, List[int], torch.Tensor]] = None, greedy: bool = False,
                     append: bool = False, hold: bool = False, extend: bool = False):
        """``append`` / ``hold`` build one forward out of new prompts and running sequences, ``extend`` feeds further
        pieces of the prompts of known sequences (chunked prefill; ``input_ids`` = one list per sequence id); see
        ``runtime.engine.Model.set_input_cb``.  All three are extensions of the reference's call."""
        seq_lens = None
        if extend:
            if seq_ids is None or not isinstance(input_ids, list) or not input_ids or not isinstance(input_ids[0], list):
                raise ValueError("extend=True takes seq_ids and one list of tokens per sequence")
            seq_lens = [len(r) for r in input_ids]
            input_ids = [t for r in input_ids for t in r]
            return self.model.set_input_cb(input_ids, seq_lens, seq_ids, max_length, greedy, append, hold, True)
        if isinstance(input_ids, list):
            if seq_ids is None:
                if input_ids and isinstance(input_ids[0], list):
                    seq_lens = [len(r) for r in input_ids]
                    input_ids = [t for r in input_ids for t in r]
                else:
                    raise ValueError("For prompts, input_ids should not be List[int].")
            elif input_ids and isinstance(input_ids[0], list):
                input_ids = [t for r in input_ids for t in r]
        return self.model.set_input_cb(input_ids, seq_lens, seq_ids, max_length, greedy, append, hold)

    def follow(self):
        """Follower ranks: run rank 0's calls (generate, continuous batching, all-position logits) until shutdown."""
        return self.model.follow()

    def follow_cb(self):
        """Follower ranks of a continuous-batching server: mirror rank 0 until it shuts down."""
        return self.model.follow_cb()

    def forward_cb(self):
        return self.model.forward_cb()

    def forward_cb_greedy(self):
        """Greedy next tokens of the last ``set_input_cb(..., greedy=True)``, selected on the device (decode steps
        replay the CUDA graph).  Not in the reference's API."""
        return self.model.forward_cb_greedy()

    def free_seqs(self, seq_ids: Optional[Union[List[int], torch.Tensor]] = None):
        return self.model.free_seqs(seq_ids)

    # -- batch generation -----------------------------------------------------------------
    def finalize(self):
        return self.model.finalize()

    def is_done(self):
        return self.model.is_done()

    def config(self, max_length=20, num_beams=1, num_return_sequences=1, length_penalty=1.0, early_stopping=False,
               eos_token_id=-1, pad_token_id=-1, do_sample=False, temperature=1.0, top_k=50, top_p=1.0,
               repetition_penalty=1.0, stop_words_ids: Union[List[List[int]], None] = None, **kwargs):
        self.model.config(max_length, num_beams, num_return_sequences, length_penalty, early_stopping, eos_token_id,
                          pad_token_id, do_sample, temperature, top_k, top_p, repetition_penalty, stop_words_ids,
                          **kwargs)

    def input(self, input_ids=None):
        self.model.input(input_ids)

    def set_input(self, input_ids=None, max_length=20, num_beams=1, num_return_sequences=1, length_penalty=1.0,
                  early_stopping=False, eos_token_id=-1, pad_token_id=-1, do_sample=False, temperature=1.0,
                  top_k=50, top_p=1.0, repetition_penalty=1.0, stop_words_ids: Union[List[List[int]], None] = None,
                  **kwargs):
        self.model.set_input(input_ids, max_length, num_beams, num_return_sequences, length_penalty, early_stopping,
                             eos_token_id, pad_token_id, do_sample, temperature, top_k, top_p, repetition_penalty,
                             stop_words_ids, **kwargs)

    def forward(self):
        return self.model.forward()

    def prefix_sharing(self, input_ids=None, truncate_tail=0):
        if input_ids is not None and truncate_tail > 0:
            input_ids = input_ids[:, :-truncate_tail]
        self.model.set_prefix(input_ids)

    def disable_prefix_sharing(self):
        self.model.unset_prefix()

    @torch.no_grad()
    def generate(self, input_ids=None, max_length=20, num_beams=1, num_return_sequences=1, length_penalty=1.0,
                 early_stopping=False, eos_token_id=-1, pad_token_id=-1, do_sample=False, temperature=1.0, top_k=50,
                 top_p=1.0, repetition_penalty=1.0, stop_words_ids: Union[List[List[int]], None] = None,
                 streamer=None, **kwargs):
        if streamer is not None:
            if num_beams > 1:
                raise ValueError("`streamer` cannot be used with beam search (yet!). Make sure that `num_beams` is set to 1.")
            if input_ids is not None and input_ids.size(0) != 1:
                raise ValueError("`streamer` cannot be used with batch size != 1 (yet!).")
            if input_ids is not None:
                streamer.put(input_ids.cpu())
        # One control message whatever the mode; greedy, sampling and beams share the paged path.
        self.set_input(input_ids, max_length, num_beams, num_return_sequences, length_penalty, early_stopping,
                       eos_token_id, pad_token_id, do_sample, temperature, top_k, top_p, repetition_penalty,
                       stop_words_ids, **kwargs)
        sent = 0
        while not self.is_done():
            next_tokens = self.forward()
            if streamer is not None and input_ids is not None:
                # everything the step produced: one token, or several when drafts were accepted (XFT_SPEC_NGRAM)
                gen = self.model.working[0].generated if self.model.working else []
                new = gen[sent:] if len(gen) > sent else next_tokens.flatten().tolist()[:1]
                sent = max(len(gen), sent + len(new))
                streamer.put(torch.tensor(new, dtype=torch.int64))
        if streamer is not None and input_ids is not None:
            streamer.end()
        return self.finalize()
