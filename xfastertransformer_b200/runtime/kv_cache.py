"""Paged KV cache: block allocator with reference counts + per-layer block pools.

The reference keeps one contiguous ``[maxSeq, 1, kvHeads, headSize]`` tensor per sequence and
layer, reserved for ``maxLen`` tokens up front and recycled through a free list
(``src/common/kvcache_mgr.h:78-129,196-249``, ``src/common/kvcache_tensor.h:64-336``); beam
reorder and prefix sharing physically copy rows (``kvcache_tensor.h:146-289``,
``src/models/kvcache_manager.cpp:57-106``).  Here the cache is paged in 64-token blocks:

* pool per layer: ``K, V : [num_blocks, kv_heads, block, head_dim]`` (bf16/fp16, or int8 with a
  parallel fp32 scale ``[num_blocks, kv_heads, block]`` — one scale per token·head exactly like
  the reference's int8 cache, ``kvcache_tensor.h:100-104``); MLA models keep a single latent pool
  ``[num_blocks, 1, block, kv_lora+rope]``.
* a sequence is a list of block ids; blocks are reference-counted so a shared prefix or a beam
  fork is a table copy, and beam reorder is a permutation of tables (no data moves unless the
  partially filled tail block must be split — copy-on-write).

When built, the native allocator (``csrc/core/paged_kv.cc``) backs `BlockAllocator`; the Python
implementation below is the same algorithm and the fallback.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch


class BlockAllocator:
    def __init__(self, num_blocks: int):
        self.num_blocks = num_blocks
        self.free: List[int] = list(range(num_blocks - 1, -1, -1))
        self.ref = [0] * num_blocks

    def grow(self, new_total: int) -> None:
        self.free = list(range(new_total - 1, self.num_blocks - 1, -1)) + self.free
        self.ref.extend([0] * (new_total - self.num_blocks))
        self.num_blocks = new_total

    @property
    def num_free(self) -> int:
        return len(self.free)

    def alloc(self) -> int:
        if not self.free:
            raise MemoryError("KV cache exhausted")
        b = self.free.pop()
        self.ref[b] = 1
        return b

    def share(self, b: int) -> int:
        self.ref[b] += 1
        return b

    def release(self, b: int) -> None:
        self.ref[b] -= 1
        if self.ref[b] == 0:
            self.free.append(b)
        elif self.ref[b] < 0:
            raise RuntimeError(f"double free of KV block {b}")


class PrefixIndex:
    """Automatic prefix reuse: full token blocks that a prefill has written are remembered under a hash chain of their
    tokens (the digest of block j covers blocks 0..j), so a later prompt that starts with the same tokens adopts those
    blocks instead of recomputing them.  The index holds one reference per remembered block; blocks are immutable once
    full (a sequence only ever writes into its own tail block), so sharing them is safe.  Least recently used entries
    whose block nobody else holds are dropped when the allocator runs short.  (The reference only has the explicit,
    single-prefix ``setPrefix`` API: src/models/common_decoder.h:337-353.)"""

    def __init__(self, cache: "PagedKVCache"):
        from collections import OrderedDict
        self.cache = cache
        self.entries: "OrderedDict[bytes, int]" = OrderedDict()       # chain digest -> block id
        self.lookups = self.hit_blocks = self.evicted = 0

    def _digests(self, tokens: Sequence[int], n_blocks: int) -> List[bytes]:
        import hashlib
        import struct
        b = self.cache.block
        out, prev = [], b""
        for j in range(n_blocks):
            chunk = tokens[j * b:(j + 1) * b]
            prev = hashlib.blake2b(prev + struct.pack(f"<{b}i", *chunk), digest_size=16).digest()
            out.append(prev)
        return out

    def lookup(self, tokens: Sequence[int]) -> List[int]:
        """Blocks holding the longest remembered prefix of `tokens`, leaving at least one token to run."""
        self.lookups += 1
        n = (len(tokens) - 1) // self.cache.block
        hit: List[bytes] = []
        for d in self._digests(tokens, n):
            if d not in self.entries:
                break
            hit.append(d)
        for d in reversed(hit):                   # a parent ends up more recent than its children: evicted after them
            self.entries.move_to_end(d)
        self.hit_blocks += len(hit)
        return [self.entries[d] for d in hit]

    def insert(self, tokens: Sequence[int], table: Sequence[int]) -> int:
        """Remember the full blocks of `tokens` (already written to `table`); returns how many were new."""
        n = min(len(tokens) // self.cache.block, len(table))
        new = 0
        for j, d in enumerate(self._digests(tokens, n)):
            if d in self.entries:
                self.entries.move_to_end(d)
                continue
            self.entries[d] = self.cache.alloc.share(table[j])
            new += 1
        return new

    def evict(self, want: int) -> int:
        """Drop up to `want` least recently used entries whose block only the index still holds."""
        freed = 0
        for d in list(self.entries):
            if freed >= want:
                break
            b = self.entries[d]
            if self.cache.alloc.ref[b] == 1:
                del self.entries[d]
                self.cache.alloc.release(b)
                freed += 1
        self.evicted += freed
        return freed

    def clear(self) -> None:
        for b in self.entries.values():
            self.cache.alloc.release(b)
        self.entries.clear()


class PagedKVCache:
    def __init__(self, num_layers: int, kv_heads: int, k_dim: int, v_dim: int, dtype: str, device: torch.device,
                 block_size: int = 64, act_dtype: torch.dtype = torch.bfloat16, latent: bool = False):
        self.L, self.H, self.kd, self.vd = num_layers, kv_heads, k_dim, v_dim
        self.block = block_size
        self.device = device
        self.latent = latent                     # MLA: single pool, no V
        self.int8 = dtype == "int8"
        if self.int8:
            self.dtype = torch.int8
        elif dtype == "fp16" and act_dtype == torch.float16:
            self.dtype = torch.float16
        else:
            # the engine's activations are bf16; an "fp16" request keeps a 16-bit cache in the
            # activation type so the attention kernels read it without conversion
            self.dtype = act_dtype if act_dtype in (torch.bfloat16, torch.float16) else \
                (torch.bfloat16 if dtype == "bf16" else torch.float32 if device.type == "cpu" else torch.float16)
        self.alloc = BlockAllocator(0)
        self.k: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        self.ks: List[Optional[torch.Tensor]] = []
        self.vs: List[Optional[torch.Tensor]] = []
        self.tables: Dict[int, List[int]] = {}
        self.lens: Dict[int, int] = {}
        self.version = 0                         # bumped when pools are reallocated
        self.prefix_index: Optional[PrefixIndex] = None      # set by the engine when automatic prefix reuse is on

    # -- capacity -------------------------------------------------------------------
    def bytes_per_block(self) -> int:
        e = torch.empty((), dtype=self.dtype).element_size()
        per = self.H * self.block * self.kd * e + (0 if self.latent else self.H * self.block * self.vd * e)
        if self.int8:
            per += 2 * self.H * self.block * 4
        return per * self.L

    def ensure_blocks(self, total: int) -> None:
        """Grow pools to hold `total` blocks (existing contents preserved)."""
        if total <= self.alloc.num_blocks:
            return
        old = self.alloc.num_blocks
        mk = lambda d, dt=None: torch.zeros(total, self.H, self.block, d, dtype=dt or self.dtype, device=self.device)
        nk, nv, nks, nvs = [], [], [], []
        for l in range(self.L):
            k = mk(self.kd)
            v = None if self.latent else mk(self.vd)
            if old:
                k[:old] = self.k[l]
                if v is not None:
                    v[:old] = self.v[l]
            nk.append(k)
            nv.append(v)
            if self.int8:
                s1 = torch.zeros(total, self.H, self.block, dtype=torch.float32, device=self.device)
                s2 = torch.zeros_like(s1)
                if old:
                    s1[:old] = self.ks[l]
                    s2[:old] = self.vs[l]
                nks.append(s1)
                nvs.append(s2)
            else:
                nks.append(None)
                nvs.append(None)
            if old:
                self.k[l] = None
                self.v[l] = None
        self.k, self.v, self.ks, self.vs = nk, nv, nks, nvs
        self.alloc.grow(total)
        self.version += 1

    def blocks_for(self, n_tokens: int) -> int:
        return (n_tokens + self.block - 1) // self.block

    def reserve(self, extra_blocks: int) -> None:
        """Make sure `extra_blocks` free blocks exist (grows geometrically)."""
        if self.alloc.num_free >= extra_blocks:
            return
        if self.prefix_index is not None and self.alloc.num_blocks > 0:
            # remembered prefixes give way before the pools grow (growing moves the pools and invalidates graphs)
            self.prefix_index.evict(extra_blocks - self.alloc.num_free)
            if self.alloc.num_free >= extra_blocks:
                return
        need = self.alloc.num_blocks - self.alloc.num_free + extra_blocks
        self.ensure_blocks(max(need, int(self.alloc.num_blocks * 1.5)))

    # -- sequences ------------------------------------------------------------------
    def add_sequence(self, seq_id: int, max_len: int = 0) -> None:
        if seq_id in self.tables:
            raise KeyError(f"sequence {seq_id} already in the cache")
        self.tables[seq_id] = []
        self.lens[seq_id] = 0
        if max_len:
            self.reserve(self.blocks_for(max_len))

    def free_sequence(self, seq_id: int) -> None:
        for b in self.tables.pop(seq_id, []):
            self.alloc.release(b)
        self.lens.pop(seq_id, None)

    def adopt(self, seq_id: int, blocks: Sequence[int]) -> int:
        """Start a fresh sequence on shared, full blocks (automatic prefix reuse); returns the tokens they hold."""
        assert not self.tables[seq_id], "adopt() is for a sequence that holds nothing yet"
        self.tables[seq_id] = [self.alloc.share(b) for b in blocks]
        self.lens[seq_id] = len(blocks) * self.block
        return self.lens[seq_id]

    def fork(self, src: int, dst: int) -> None:
        """dst shares all of src's blocks (prefix sharing, beam expansion)."""
        if dst in self.tables:
            self.free_sequence(dst)
        self.tables[dst] = [self.alloc.share(b) for b in self.tables[src]]
        self.lens[dst] = self.lens[src]

    def append_slots(self, seq_id: int, n_new: int) -> List[int]:
        """Reserve `n_new` token positions at the end of the sequence; returns flat slot ids
        (block*block_size+offset).  A shared, partially filled tail block is copied first."""
        tab = self.tables[seq_id]
        cur = self.lens[seq_id]
        slots = []
        off = cur % self.block
        if off and tab and self.alloc.ref[tab[-1]] > 1:
            self.reserve(1)
            nb = self.alloc.alloc()
            self._copy_block(tab[-1], nb)
            self.alloc.release(tab[-1])
            tab[-1] = nb
        need = self.blocks_for(cur + n_new) - len(tab)
        if need > 0:
            self.reserve(need)
            tab.extend(self.alloc.alloc() for _ in range(need))
        for p in range(cur, cur + n_new):
            slots.append(tab[p // self.block] * self.block + p % self.block)
        self.lens[seq_id] = cur + n_new
        return slots

    def truncate(self, seq_id: int, new_len: int) -> None:
        tab = self.tables[seq_id]
        keep = self.blocks_for(new_len)
        for b in tab[keep:]:
            self.alloc.release(b)
        del tab[keep:]
        self.lens[seq_id] = new_len

    def reorder(self, seq_ids: Sequence[int], src_index: Sequence[int]) -> None:
        """Beam reorder: sequence seq_ids[i] continues from old seq_ids[src_index[i]]
        (KVCacheTensor::reorder, kvcache_tensor.h:146-260) — a permutation of block tables."""
        old_tabs = {s: self.tables[s] for s in seq_ids}
        old_lens = {s: self.lens[s] for s in seq_ids}
        new = {}
        for i, s in enumerate(seq_ids):
            src = seq_ids[src_index[i]]
            new[s] = [self.alloc.share(b) for b in old_tabs[src]]
        for s in seq_ids:
            for b in old_tabs[s]:
                self.alloc.release(b)
        for i, s in enumerate(seq_ids):
            self.tables[s] = new[s]
            self.lens[s] = old_lens[seq_ids[src_index[i]]]

    def _copy_block(self, src: int, dst: int) -> None:
        for l in range(self.L):
            self.k[l][dst].copy_(self.k[l][src])
            if self.v[l] is not None:
                self.v[l][dst].copy_(self.v[l][src])
            if self.int8:
                self.ks[l][dst].copy_(self.ks[l][src])
                self.vs[l][dst].copy_(self.vs[l][src])

    def block_table(self, seq_ids: Sequence[int], width: Optional[int] = None) -> torch.Tensor:
        """int32 [len(seq_ids), width] on the host (unused entries 0)."""
        w = max([len(self.tables[s]) for s in seq_ids] + [1]) if width is None else width
        # one conversion for the whole table: this runs once per decode step on the host
        rows = []
        for s in seq_ids:
            tab = self.tables[s]
            if len(tab) > w:
                raise ValueError(f"sequence {s} holds {len(tab)} blocks, more than the table width {w}")
            rows.append(tab + [0] * (w - len(tab)))
        return torch.tensor(rows, dtype=torch.int32).view(len(seq_ids), w)
