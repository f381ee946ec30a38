"""Decode fast path on the GPU: one CUDA graph per (batch size, table width), replayed per step.

The reference runs every step through its OpenMP layer loop (``src/models/common_decoder.h:591-693``).
On B200 a decode step of a large model is a few hundred short kernels, so launch overhead would
dominate: the whole step — embedding, all layers (GEMMs with fused epilogues, RoPE + cache append,
flash-decode, the TP reductions), final norm, lm_head, arg-max and the cross-rank (value, id)
merge — is captured once and replayed.  Per step the host only

  1. appends one cache slot per sequence (block allocator, host side),
  2. fills ONE pinned int32 staging buffer [ids | positions | slots | kv_lens | block_table],
  3. issues one H2D copy, one graph launch, one D2H copy of the chosen tokens, and waits.

Greedy decoding with no repetition penalty takes this path; anything else (sampling, beams,
penalties, prefill, pipeline stages) runs the eager path in `engine.Model`.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..models.decoder import Batch
from ..utils import trace
from . import sampler as S


class _Graph:
    __slots__ = ("graph", "B", "W", "host", "dev", "tok_dev", "tok_host", "batch", "version", "nsplit", "kernels")


class CudaRunner:
    def __init__(self, model):
        self.m = model
        self.dev = model.ctx.device
        self.graphs: Dict[tuple, _Graph] = {}
        self.enabled = model.env.cuda_graph
        self.stream = torch.cuda.Stream(device=self.dev)
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.graph_launches = 0
        self.kernel_launches = 0          # kernels of this library launched through replayed graphs / eager steps
        self.timing = False               # record a CUDA-event pair around each step's launch
        self.step_events = []
        self._scratch_block = None
        if self.enabled:
            # taken now, while the pools are empty: a block taken after a request reserved its blocks would leave that
            # request one block short and make the pools grow (and move) in the middle of its decode
            self._scratch()

    def reset(self) -> None:
        pass

    def can_run(self, seqs: Sequence, cfg) -> bool:
        if not self.enabled or cfg.do_sample or cfg.num_beams > 1 or cfg.repetition_penalty != 1.0:
            return False
        if self.m.ctx.pp_size > 1 or self.m.decoder.spec.rope == "2d" or trace.enabled() or self.m.env.debug_dir:
            return False
        if self.m.env.verbose >= 1:          # per-GEMM timing lines need real launches with a synchronise around each
            return False
        if self.m.ctx.dp_size > 1:
            # data-parallel attention: every rank replays a graph over ITS sequences.  The MoE token exchange must then
            # be the peer-memory kernels (no host-side count exchange inside a captured step), and every rank's local
            # batch must fit them.
            ctx = self.m.ctx
            if self.m.decoder.has_moe:
                if ctx.epcomm is None:
                    return False
                per_rank = [sum(1 for s in seqs if s.owner == r) for r in range(ctx.dp_size)]
                if max(self.bucket(n) if n else 0 for n in per_rank) > ctx.epcomm.max_tokens:
                    return False
        if self.m.ctx.tp_size > 1:
            # every cross-rank sum of a captured step must be a peer-memory kernel (fused into the GEMM for bf16
            # weights, the one-shot all-reduce for the experts' partial sums and for weight types the fused kernel does
            # not take), which holds at most `slot` values; without it the step would put a NCCL collective inside the
            # captured graph
            peer = getattr(self.m.ctx, "peer", None)
            rows = self.bucket(len(seqs))
            if peer is None or rows * self.m.cfg.hidden_size > peer.slot:
                return False
        return all(len(s.pending) == 1 and s.past_len > 0 for s in seqs)

    @staticmethod
    def bucket(n: int) -> int:
        """Batch sizes are padded up to a bucket so that a serving loop whose batch shrinks and grows by one sequence at
        a time replays a handful of graphs: powers of two up to 8, multiples of 4 up to 16, of 8 up to 64, of 16 up to
        128, of 32 beyond (padding never exceeds half of the real rows above 8)."""
        if n <= 8:
            b = 1
            while b < n:
                b *= 2
            return b
        step = 4 if n <= 16 else 8 if n <= 64 else 16 if n <= 128 else 32
        return (n + step - 1) // step * step

    def _key(self, seqs: Sequence):
        W = max(self.m.cache.blocks_for(s.max_len + 1) for s in seqs)
        W = (W + 7) // 8 * 8
        fw = getattr(self, "fixed_width", None)      # serving: one block-table width for every request length
        if fw is not None and W <= fw:
            W = fw
        return self.bucket(len(seqs)), W

    def _scratch(self) -> int:
        """One KV block owned by the runner: padding rows of a bucketed batch write their key/value there and attend
        to it (a context of one token), so they touch no live sequence."""
        if getattr(self, "_scratch_block", None) is None:
            self.m.cache.reserve(1)
            self._scratch_block = self.m.cache.alloc.alloc()
        return self._scratch_block

    def worth_capturing(self, seqs: Sequence) -> bool:
        """For callers whose batch composition changes from step to step (serving): a shape is captured only when
        it is requested twice in a row or already has a graph; a shape seen once runs eagerly."""
        key = self._key(seqs)
        hit = key in self.graphs or key == getattr(self, "_last_key", None)
        self._last_key = key
        if len(self.graphs) > 64 and key not in self.graphs:      # bound the memory held by captured shapes
            self.graphs.pop(next(iter(self.graphs)))
        return hit

    # ------------------------------------------------------------------------------------
    def _layout(self, B: int, W: int):
        o_ids, o_pos, o_slot, o_kv = 0, B, 2 * B, 3 * B
        o_cu = 4 * B
        o_bt = 5 * B + 1
        # keep the block table 16-byte aligned
        o_bt = (o_bt + 3) // 4 * 4
        return o_ids, o_pos, o_slot, o_kv, o_cu, o_bt, o_bt + B * W

    def _build(self, B: int, W: int, max_kv_hint: int) -> _Graph:
        m = self.m
        g = _Graph()
        g.B, g.W = B, W
        o_ids, o_pos, o_slot, o_kv, o_cu, o_bt, total = self._layout(B, W)
        g.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        g.dev = torch.zeros(total, dtype=torch.int32, device=self.dev)
        g.tok_dev = torch.zeros(B, dtype=torch.int64, device=self.dev)
        g.tok_host = torch.zeros(B, dtype=torch.int64).pin_memory()
        g.host[o_cu:o_cu + B + 1] = torch.arange(B + 1, dtype=torch.int32)
        d = g.dev
        dec = m.decoder
        from ..ops import native as N
        g.nsplit, _ = N.plan_attn_splits(B, max(dec.hkv, 1), dec.group, dec.D, max_kv_hint, m.cache.int8)
        b = Batch(ids=d[o_ids:o_ids + B], positions=d[o_pos:o_pos + B], slots=d[o_slot:o_slot + B],
                  cu_q=list(range(B + 1)), kv_lens=[max_kv_hint] * B, block_table=d[o_bt:o_bt + B * W].view(B, W),
                  logit_rows=None, is_decode=True, max_q=1, max_kv=max_kv_hint)
        b.cu_q_dev = d[o_cu:o_cu + B + 1]
        b.kv_lens_dev = d[o_kv:o_kv + B]
        b.meta["nsplit"] = g.nsplit
        g.batch = b
        g.version = m.cache.version
        g.graph = None
        return g

    def _step_body(self, g: _Graph) -> None:
        m = self.m
        local = m.decoder.forward(g.batch, m.cache)
        toks = S.greedy_select(local, m.decoder.v0, m.ctx)
        g.tok_dev.copy_(toks)

    def _reserve_slots(self, seqs) -> List[int]:
        """Cache positions of this step's tokens.  Runs before the graph is chosen: appending may grow the pools, which
        moves them and invalidates every captured graph."""
        cache = self.m.cache
        slots = []
        for s in seqs:
            start = s.past_len
            if cache.lens[s.seq_id] > start:
                cache.truncate(s.seq_id, start)
            slots.append(cache.append_slots(s.seq_id, 1)[0])
        return slots

    def _fill(self, g: _Graph, seqs, slots: List[int]) -> None:
        m = self.m
        B, W = g.B, g.W
        o_ids, o_pos, o_slot, o_kv, o_cu, o_bt, total = self._layout(B, W)
        h = g.host
        cache = m.cache
        slots = list(slots)
        ids = [s.pending[0] for s in seqs]
        pos = [s.past_len for s in seqs]
        kvl = [s.past_len + 1 for s in seqs]
        pad = B - len(seqs)
        if pad:                                        # padding rows of the bucket: one token in the scratch block
            sb = self._scratch()
            ids += [0] * pad
            pos += [0] * pad
            slots += [sb * cache.block] * pad
            kvl += [1] * pad
        # ids | positions | slots | kv lengths are adjacent in the staging buffer: one conversion, one copy
        assert (o_ids, o_pos, o_slot, o_kv) == (0, B, 2 * B, 3 * B)
        h[0:4 * B] = torch.tensor(ids + pos + slots + kvl, dtype=torch.int32)
        bt = cache.block_table([s.seq_id for s in seqs], W)
        n = len(seqs)
        h[o_bt:o_bt + n * W] = bt.view(-1)
        if pad:
            h[o_bt + n * W:o_bt + B * W] = self._scratch()

    def step(self, seqs: Sequence, cfg) -> List[int]:
        if self.m.ctx.dp_size > 1:
            return self._step_dp(seqs, cfg)
        return self._step_local(seqs, cfg)

    def _step_dp(self, seqs: Sequence, cfg) -> List[int]:
        """Data-parallel attention: this rank decodes the sequences it owns (a graph per local batch bucket; a rank
        without sequences replays a graph that only serves its experts), then the chosen tokens are exchanged on the
        host so that every rank steps all sequences."""
        import torch.distributed as dist
        ctx = self.m.ctx
        local = [s for s in seqs if s.owner == ctx.dp_rank]
        per_rank = [sum(1 for s in seqs if s.owner == r) for r in range(ctx.dp_size)]
        ctx.dp_max_tokens = max(self.bucket(n) if n else 0 for n in per_rank)
        toks = self._step_local(local, cfg) if local else self._step_idle()
        # one fixed-size gather of token ids (rows padded with -1): no pickling, one round on the control group
        n = max(max(per_rank), 1)
        mine = torch.full((n,), -1, dtype=torch.int64)
        if toks:
            mine[:len(toks)] = torch.tensor([int(t) for t in toks], dtype=torch.int64)
        allt = torch.empty(ctx.world * n, dtype=torch.int64)
        dist.all_gather_into_tensor(allt, mine, group=ctx.ctrl_group)
        rows = allt.view(ctx.world, n).tolist()
        its = [iter(r) for r in rows]
        return [next(its[s.owner]) for s in seqs]

    def _step_idle(self) -> List[int]:
        """No sequence of this step lives here: run (and capture once) the expert exchange of every MoE layer."""
        if not self.m.decoder.has_moe:
            return []                              # dense model: nothing to serve
        g = self.graphs.get("idle")
        st = self.stream
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st), torch.no_grad():
            if g is None:
                self.m.decoder.forward_idle()
                st.synchronize()
                g = _Graph()
                g.version = -1
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=st):
                    self.m.decoder.forward_idle()
                g.graph = graph
                self.graphs["idle"] = g
            else:
                g.graph.replay()
                self.graph_launches += 1
        st.synchronize()
        return []

    def _step_local(self, seqs: Sequence, cfg) -> List[int]:
        m = self.m
        n_real = len(seqs)
        self._scratch()                                # both may grow the pools: before the version check below
        slots = self._reserve_slots(seqs)
        key = self._key(seqs)
        B, W = key
        g = self.graphs.get(key)
        if g is not None and g.version != m.cache.version:
            g = None                                   # cache pools were reallocated: pointers changed
        if g is None:
            g = self._build(B, W, max(s.max_len for s in seqs))
            self.graphs[key] = g
        self._fill(g, seqs, slots)
        st = self.stream
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st), torch.no_grad():
            g.dev.copy_(g.host, non_blocking=True)
            if g.graph is None:
                # eager run (allocates workspaces, JIT-free), then capture
                self._step_body(g)
                st.synchronize()
                from ..ops import native as N
                ws = N.Workspace.get(self.dev)
                n0 = ws.launches
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=st):
                    self._step_body(g)
                g.graph = graph
                g.kernels = ws.launches - n0
                self.kernel_launches += g.kernels
                # the eager run already produced this step's tokens and wrote its K/V; replaying the
                # captured step would redo identical work — harmless, but skip it
            else:
                if self.timing:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(st)
                g.graph.replay()
                if self.timing:
                    e1.record(st)
                    self.step_events.append((e0, e1))
                self.graph_launches += 1
                self.kernel_launches += g.kernels
            g.tok_host.copy_(g.tok_dev, non_blocking=True)
        st.synchronize()
        self.h2d_bytes += g.host.numel() * 4
        self.d2h_bytes += g.tok_host.numel() * 8
        return g.tok_host.tolist()[:n_real]
