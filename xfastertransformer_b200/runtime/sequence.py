"""Per-request state (reference ``src/common/sequence.h:47-407``, ``src/searchers/sampling_params.h``).

`SequenceMeta` tracks prompt, generated tokens, how many tokens are already in the KV cache
(`past_len`) and the pending input of the next forward; `SequenceIDManager` hands out ids
0..10239 with wrap-around exactly like the reference so that follower ranks, which run the
same allocator, stay in lock-step without the ids being transmitted.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

MAX_SEQ_ID = 10240


class SequenceIDManager:
    def __init__(self):
        self._next = 0

    def create(self, in_use) -> int:
        for _ in range(MAX_SEQ_ID):
            sid = self._next
            self._next = (self._next + 1) % MAX_SEQ_ID
            if sid not in in_use:
                return sid
        raise RuntimeError("no free sequence id")


@dataclass
class SamplingMeta:
    """SearcherConfig (include/abstract_searcher.h:20-67) + stop words + seed."""
    max_length: int = 20
    num_beams: int = 1
    num_return_sequences: int = 1
    length_penalty: float = 1.0
    early_stopping: bool = False
    eos_token_id: int = -1
    pad_token_id: int = -1
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int = 50
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    stop_words: List[List[int]] = field(default_factory=list)
    seed: Optional[int] = None

    def clean_stop_words(self) -> None:
        """Drop empty lists, lists with ids <= 0 and a lone eos (sampling_params.h:30-41)."""
        out = []
        for w in self.stop_words or []:
            if not w or any(t <= 0 for t in w):
                continue
            if len(w) == 1 and w[0] == self.eos_token_id:
                continue
            out.append(list(w))
        self.stop_words = out


@dataclass
class SequenceMeta:
    seq_id: int
    prompt: List[int]
    max_len: int
    generated: List[int] = field(default_factory=list)
    past_len: int = 0                 # tokens whose K/V are in the cache
    pending: List[int] = field(default_factory=list)   # tokens the next forward consumes
    done: bool = False
    group: int = -1                   # request index for beams
    prefix_len: int = 0               # tokens inherited from a shared prefix
    owner: int = 0                    # data-parallel attention: the rank that holds this sequence's KV cache

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.generated)

    def step_forward(self, token: int) -> None:
        """Account for a finished forward and queue `token` as the next input
        (SequenceMeta::stepForward, sequence.h:104-113)."""
        self.past_len += len(self.pending)
        self.generated.append(token)
        self.pending = [token]

    def all_tokens(self) -> List[int]:
        return self.prompt + self.generated


class SequencePool:
    def __init__(self):
        self.seqs: Dict[int, SequenceMeta] = {}
        self.ids = SequenceIDManager()

    def new(self, prompt: List[int], max_len: int, group: int = -1, seq_id: Optional[int] = None,
            owner: int = 0) -> SequenceMeta:
        sid = self.ids.create(self.seqs) if seq_id is None else seq_id
        s = SequenceMeta(sid, list(prompt), max_len, pending=list(prompt), group=group, owner=owner)
        self.seqs[sid] = s
        return s

    def get(self, sid: int) -> SequenceMeta:
        if sid not in self.seqs:
            raise KeyError(f"unknown sequence id {sid}")
        return self.seqs[sid]

    def remove(self, sid: int) -> None:
        self.seqs.pop(sid, None)

    def __contains__(self, sid: int) -> bool:
        return sid in self.seqs
