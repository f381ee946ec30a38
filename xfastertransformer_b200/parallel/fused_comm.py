"""Peer-memory communication for the tensor-parallel group: symmetric buffers over CUDA IPC and
the kernels that use them (fused GEMM + one-shot all-reduce, stand-alone one-shot all-reduce).

The reference reduces the partial o_proj / down_proj outputs with a separate collective after the
GEMM (``src/layers/decoder_block.h:122-134`` -> ``Messenger::reduceAdd`` -> oneCCL or the
shared-memory chain of ``src/utils/shm_ccl.cpp:82-145``).  Here, at decode sizes, the GEMM's epilogue
pushes each finished output tile straight into every peer's receive slot over NVLink, waits (bounded) for
the peers' words and sums them in rank order — one kernel, no separate
collective, bit-identical results on all ranks.  Larger token counts fall back to NCCL.

Buffer per rank (allocated once, mapped by every peer): recv [2 parities][world][T_CAP x N_MAX] 8-byte
words, each {fp32 value, epoch}.  The epoch next to a value tells the reader it has arrived, so the
latency of the collective is one NVLink store propagation: no fence, flag or barrier in between.  A
device-side epoch counter (bumped by the last CTA of every launch) selects the parity, so CUDA-graph
replays stay in step without host involvement.

Also here, both opt-in: the plumbing of the fused prefill GEMM + reduce-scatter + all-gather kernel
(``PeerComm.gemm_ar_bulk``, csrc/kernels/gemm_prefill_sm100.cu) and `EpComm`, the expert-parallel token exchange of
data-parallel attention (csrc/kernels/ep_comm.cu).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import native as N


class CommParams(C.Structure):
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("recv", C.c_void_p * 8), ("epoch", C.c_void_p),
                ("done", C.c_void_p), ("slot_stride", C.c_longlong), ("parity_stride", C.c_longlong),
                ("wait_cycles", C.c_longlong), ("two_shot", C.c_int), ("result", C.c_void_p * 8)]


class ArParams(C.Structure):
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("recv", C.c_void_p * 8), ("epoch", C.c_void_p),
                ("done", C.c_void_p), ("cap", C.c_longlong), ("wait_cycles", C.c_longlong), ("status", C.c_void_p)]


class _RawCuda:
    """__cuda_array_interface__ holder: lets torch view a range of the symmetric buffer without copying."""

    def __init__(self, ptr: int, shape, owner):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<i2", "data": (ptr, False), "version": 3,
                                         "strides": None}
        self._owner = owner


def _view_bf16(ptr: int, rows: int, cols: int, device, owner) -> torch.Tensor:
    return torch.as_tensor(_RawCuda(ptr, (rows, cols), owner), device=device).view(torch.bfloat16)


def _symmetric_alloc(ctx, lib, nbytes: int, first: int, world: int, rank: int):
    """Allocate `nbytes` (zeroed) on this GPU and map the same allocation of the other `world - 1` ranks of the group
    that starts at global rank `first` (CUDA IPC).  Returns (own base address, base address per group rank, the peer
    mappings to close later).  Collective over ctx.ctrl_group."""
    base = C.c_void_p()
    N._check(lib.xft_comm_alloc(C.c_size_t(nbytes), C.byref(base)), "comm_alloc")
    hb = lib.xft_comm_handle_bytes()
    h = (C.c_char * hb)()
    N._check(lib.xft_comm_ipc_handle(C.c_void_p(base.value), h), "ipc_handle")
    allh: List = [None] * ctx.world
    dist.all_gather_object(allh, (ctx.rank, bytes(h)), group=ctx.ctrl_group)
    peer_base: List[int] = []
    opened: List[int] = []
    for r in range(world):
        if r == rank:
            peer_base.append(base.value)
            continue
        grank, hbytes = allh[first + r]
        p = C.c_void_p()
        buf = (C.c_char * hb).from_buffer_copy(hbytes)
        N._check(lib.xft_comm_ipc_open(buf, C.byref(p)), f"ipc_open(rank {grank})")
        peer_base.append(p.value)
        opened.append(p.value)
    return base.value, peer_base, opened


class BulkArParams(C.Structure):
    """Mirror of the struct of the same name in csrc/kernels/gemm_prefill_sm100.cu."""
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("part", C.c_void_p * 8), ("flag_part", C.c_void_p * 8),
                ("out", C.c_void_p * 8), ("flag_res", C.c_void_p * 8), ("epoch", C.c_void_p), ("done", C.c_void_p),
                ("part_stride", C.c_longlong), ("wait_cycles", C.c_longlong)]


class PeerComm:
    T_CAP = 64
    MAX_TILES = 1024

    def __init__(self, ctx, n_max: int, wait_ms: float = 2000.0):
        self.ctx = ctx
        self.world, self.rank = ctx.tp_size, ctx.tp_rank
        if not (2 <= self.world <= 8):
            raise ValueError("PeerComm supports 2..8 ranks")
        lib = N.lib()
        for fn in ("xft_comm_alloc", "xft_comm_free", "xft_comm_ipc_handle", "xft_comm_ipc_open", "xft_comm_ipc_close",
                   "xft_comm_handle_bytes", "xft_gemm_bf16_ar", "xft_allreduce_oneshot", "xft_gemm_bf16_prefill"):
            getattr(lib, fn).restype = C.c_int
        self.lib = lib
        self.slot = self.T_CAP * n_max                           # {value, epoch} words per source slot
        self.recv_bytes = 2 * self.world * self.slot * 8
        nbytes = self.recv_bytes + 2 * self.slot * 8           # + result area of the two-shot mode
        # Optional area of the fused prefill GEMM + all-reduce (XFT_PREFILL_FUSED_AR=1): partial sums from every rank
        # for the token blocks this rank owns, two output buffers that the owners of the other blocks write into
        # (consecutive launches alternate between them, so a launch never overwrites the residual it reads), flags.
        self.bulk = None
        self.bulk_tokens = int(os.environ.get("XFT_MAX_BATCH_TOKENS", "8192")) \
            if os.environ.get("XFT_PREFILL_FUSED_AR", "0") == "1" else 0
        if self.bulk_tokens > 0:
            pe, nfp, nfr = C.c_longlong(), C.c_longlong(), C.c_longlong()
            lib.xft_prefill_ar_sizes(self.bulk_tokens, n_max, self.world, C.byref(pe), C.byref(nfp), C.byref(nfr))
            al = lambda v: (v + 255) // 256 * 256
            self._b_part_stride = pe.value
            self._b_off_part = al(nbytes)
            self._b_off_out = [al(self._b_off_part + self.world * pe.value * 2)]
            self._b_off_out.append(al(self._b_off_out[0] + self.bulk_tokens * n_max * 2))
            self._b_off_fp = al(self._b_off_out[1] + self.bulk_tokens * n_max * 2)
            self._b_off_fr = al(self._b_off_fp + nfp.value * 4)
            nbytes = al(self._b_off_fr + nfr.value * 4)
        self.nbytes = nbytes
        self.base, self.peer_base, self._opened = _symmetric_alloc(ctx, lib, nbytes, ctx.pp_rank * ctx.tp_size,
                                                                   self.world, self.rank)
        self.counters = torch.zeros(4, dtype=torch.int32, device=ctx.device)   # [epoch, done]
        clock_khz = 1_900_000
        self.wait_cycles = int(wait_ms * clock_khz)
        self.gp = CommParams()
        self.ap = ArParams()
        for prm in (self.gp, self.ap):
            prm.world, prm.rank = self.world, self.rank
            for r in range(self.world):
                prm.recv[r] = self.peer_base[r]
            prm.epoch = self.counters.data_ptr()
            prm.done = self.counters.data_ptr() + 4
            prm.wait_cycles = self.wait_cycles
        for r in range(self.world):
            self.gp.result[r] = self.peer_base[r] + self.recv_bytes
        # Reduce-scatter + all-gather inside the epilogue (two-shot) trades one more NVLink hop for less traffic: it
        # pays off from 4 ranks on and more than 16 tokens; up to 16 tokens the one-shot push wins at every world
        # size measured (8 ranks, 70B decode: 10.3 vs 11.1 ms per step).  XFT_AR_TWO_SHOT=0/1 overrides.
        ts = os.environ.get("XFT_AR_TWO_SHOT")
        self._two_shot_env = int(ts) if ts is not None else None
        self.gp.two_shot = 0
        self.gp.slot_stride = self.slot
        self.gp.parity_stride = self.world * self.slot
        self.ap.cap = self.slot
        self.ap.status = N.Workspace.get(ctx.device).status.data_ptr()
        self.fused_calls = 0
        if self.bulk_tokens > 0:
            self.bulk_counters = torch.zeros(4, dtype=torch.int32, device=ctx.device)   # [epoch, done]
            self.bulk = []
            for which in range(2):
                bp = BulkArParams()
                bp.world, bp.rank = self.world, self.rank
                for r in range(self.world):
                    b = self.peer_base[r]
                    bp.part[r] = b + self._b_off_part
                    bp.out[r] = b + self._b_off_out[which]
                    bp.flag_part[r] = b + self._b_off_fp
                    bp.flag_res[r] = b + self._b_off_fr
                bp.epoch = self.bulk_counters.data_ptr()
                bp.done = self.bulk_counters.data_ptr() + 4
                bp.part_stride = self._b_part_stride
                bp.wait_cycles = self.wait_cycles
                self.bulk.append(bp)
            self._bulk_next = 0
            self._bulk_orders = {}
            self.n_max = n_max
            self.bulk_calls = 0
        dist.barrier(group=ctx.ctrl_group)

    # ------------------------------------------------------------------------------------
    def can_fuse(self, T: int, n: int, kind: str) -> bool:
        return kind == "bf16" and T <= self.T_CAP and T * n <= self.slot and (n + 127) // 128 <= self.MAX_TILES

    def gemm_ar(self, x, W, bias=None, act=None, residual=None, res_scale=1.0, out_dtype=None):
        """Y = act(sum over ranks of x_r @ W_r^T + bias) + res_scale*residual, on every rank."""
        x2, ldx = N._rows2d(x)
        T, K = x2.shape
        n = W.out_features
        fp32 = out_dtype == torch.float32
        out = torch.empty(T, n, dtype=torch.float32 if fp32 else torch.bfloat16, device=x.device)
        r2, ldr = (None, 0)
        if residual is not None:
            r2 = residual.reshape(-1, residual.shape[-1])
            ldr = r2.stride(0)
        ws = N.Workspace.get(x.device)
        self.gp.two_shot = self._two_shot_env if self._two_shot_env is not None else int(self.world >= 4 and T > 16)
        if N._ENV().gemm_streamk:
            # balanced weight-stream kernel: finished tiles are pushed to the peers and every CTA reduces its share of
            # the whole output (one-shot up to 16 tokens, reduce-scatter + all-gather above)
            if self._two_shot_env is None:
                # from 4 ranks on the owners reduce and hand the result out (two-shot): the one-shot form makes the
                # finishing CTAs store every word world times, which costs more than the extra NVLink hop at any size
                self.gp.two_shot = int(self.world >= 4)
            if fp32:
                self.gp.two_shot = 0
            N._gemm_sk(x2, ldx, W.w, out, T, n, K, False, 0, bias, r2, ldr, res_scale, act, None, None, self.gp, None)
            self.fused_calls += 1
            return out.view(*x.shape[:-1], n)
        if fp32:
            # the two-shot form hands the finished values to the other ranks as bf16 pairs, which would leave the
            # owner with fp32 and everyone else with rounded values: fp32 outputs always take the one-shot form
            self.gp.two_shot = 0
        rc = self.lib.xft_gemm_bf16_ar(N._p(x2), ldx, N._p(W.w), W.w.stride(0), N._p(out), out.stride(0), int(fp32), T, n,
                                       K, N._p(bias), N._p(r2), ldr, C.c_float(res_scale), N._ACT[act], N._p(ws.ws),
                                       C.c_size_t(ws.ws_bytes), N._p(ws.counters), ws.n_counters, N._p(ws.status),
                                       C.byref(self.gp), self.T_CAP, self.MAX_TILES, N._stream())
        N._check(rc, "gemm_bf16_ar")
        ws.launches += 1
        self.fused_calls += 1
        return out.view(*x.shape[:-1], n)

    # ------------------------------------------------------------------------------------
    def can_fuse_bulk(self, T: int, n: int, K: int, kind: str) -> bool:
        """Must give the same answer on every rank (a rank that took the unfused path would leave the others waiting),
        so it looks only at what all ranks share: token count, output width, weight type.  A slice whose K is not a
        multiple of 8 is rejected by the kernel's entry point with an error on that rank."""
        return self.bulk is not None and kind == "bf16" and self.T_CAP < T <= self.bulk_tokens and n <= self.n_max

    def _bulk_order(self, T: int, device) -> torch.Tensor:
        from .partition import block_visit_order
        bn = 256 if T > 128 else 128
        nb = (T + bn - 1) // bn
        t = self._bulk_orders.get(nb)
        if t is None:
            t = torch.tensor(block_visit_order(nb, self.world, self.rank), dtype=torch.int32, device=device)
            self._bulk_orders[nb] = t
        return t

    def gemm_ar_bulk(self, x, W, bias=None, act=None, residual=None, res_scale=1.0):
        """Prefill sizes: Y = act(sum over ranks of x_r @ W_r^T + bias) + res_scale * residual on every rank, as one
        persistent kernel that reduce-scatters its tiles into the owners' memory and all-gathers the finished tiles
        (csrc/kernels/gemm_prefill_sm100.cu).  The result is a view of one of two symmetric buffers and stays valid
        until the second next call."""
        x2, ldx = N._rows2d(x)
        T, K = x2.shape
        n = W.out_features
        which = self._bulk_next
        span = self.bulk_tokens * self.n_max * 2

        def inside(t, w):
            lo = self.base + self._b_off_out[w]
            return t is not None and lo <= t.data_ptr() < lo + span
        if inside(residual, which) or inside(x, which):
            which ^= 1                 # never write the buffer this call still reads
            if inside(residual, which) or inside(x, which):
                return None            # both in use: the caller takes the unfused path
        self._bulk_next = which ^ 1
        bp = self.bulk[which]
        out_ptr = self.base + self._b_off_out[which]
        r2, ldr = (None, 0)
        if residual is not None:
            r2 = residual.reshape(-1, residual.shape[-1])
            ldr = r2.stride(0)
        ws = N.Workspace.get(x.device)
        order = self._bulk_order(T, x.device)
        rc = self.lib.xft_gemm_bf16_prefill(N._p(x2), ldx, N._p(W.w), W.w.shape[0], W.w.stride(0), C.c_void_p(out_ptr), n,
                                            T, n, K, N._p(bias), N._p(r2), ldr, C.c_float(res_scale), N._ACT[act],
                                            N._p(order), N._p(ws.status), C.byref(bp), 0, N._stream())
        N._check(rc, "gemm_bf16_prefill(all-reduce)")
        ws.launches += 1
        self.bulk_calls += 1
        out = _view_bf16(out_ptr, T, n, x.device, self)
        return out.view(*x.shape[:-1], n)

    def _collective(self, t: torch.Tensor, out: torch.Tensor, add_f32, gather: int) -> torch.Tensor:
        n = t.numel()
        nblocks = max(1, min(296, (n + 1023) // 1024))
        rc = self.lib.xft_allreduce_oneshot(N._p(t), N._p(out), N._p(add_f32), C.c_longlong(n),
                                            0 if t.dtype == torch.float32 else 1, C.byref(self.ap), nblocks, gather,
                                            N._stream())
        N._check(rc, "allreduce_oneshot")
        N.Workspace.get(t.device).launches += 1
        return out

    def all_reduce(self, t: torch.Tensor, add_f32: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Out-of-place one-shot sum of a small fp32/bf16 tensor (numel <= slot capacity)."""
        assert t.is_contiguous() and t.numel() <= self.slot and t.dtype in (torch.float32, torch.bfloat16)
        return self._collective(t, torch.empty_like(t), add_f32, 0)

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[world, *t.shape] of a small fp32/bf16 tensor, through the same kernel."""
        assert t.is_contiguous() and t.numel() <= self.slot and t.dtype in (torch.float32, torch.bfloat16)
        out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        return self._collective(t, out, None, 1)

    def close(self) -> None:
        for p in self._opened:
            self.lib.xft_comm_ipc_close(C.c_void_p(p))
        self._opened = []
        if self.base:
            self.lib.xft_comm_free(C.c_void_p(self.base))
            self.base = 0


class EpParams(C.Structure):
    """Mirror of the struct of the same name in csrc/kernels/ep_comm.cu."""
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("rx_tok", C.c_void_p * 8), ("rx_meta", C.c_void_p * 8),
                ("rx_cnt", C.c_void_p * 8), ("ret", C.c_void_p * 8), ("ret_flag", C.c_void_p * 8), ("epoch", C.c_void_p),
                ("done", C.c_void_p), ("cap", C.c_int), ("pairs_cap", C.c_int), ("H", C.c_int),
                ("wait_cycles", C.c_longlong), ("status", C.c_void_p)]


class EpComm:
    """Expert-parallel token exchange over peer memory for data-parallel attention (decode sizes): dispatch, receive,
    return and combine kernels of csrc/kernels/ep_comm.cu around the grouped expert GEMMs.  One symmetric buffer per
    rank, mapped by every peer through CUDA IPC: a receive area of `cap` rows per source rank, a return area of
    `max_tokens * top_k` rows, count / flag words.  Nothing here synchronises with the host."""

    def __init__(self, ctx, hidden: int, top_k: int, max_tokens: int = 64, wait_ms: float = 2000.0):
        self.ctx = ctx
        self.world, self.rank = ctx.dp_size, ctx.dp_rank
        if not (2 <= self.world <= 8):
            raise ValueError("EpComm supports 2..8 ranks")
        lib = N.lib()
        for fn in ("xft_comm_alloc", "xft_comm_free", "xft_comm_ipc_handle", "xft_comm_ipc_open", "xft_comm_ipc_close",
                   "xft_comm_handle_bytes", "xft_ep_dispatch", "xft_ep_receive", "xft_ep_return", "xft_ep_combine"):
            getattr(lib, fn).restype = C.c_int
        self.lib = lib
        self.H, self.k, self.max_tokens = hidden, top_k, max_tokens
        self.cap = max_tokens * top_k                  # worst case: every pair of one source goes to one rank
        self.pairs_cap = max_tokens * top_k
        al = lambda v: (v + 255) // 256 * 256
        self.off_tok = 0
        self.off_meta = al(self.world * self.cap * hidden * 2)
        self.off_cnt = al(self.off_meta + self.world * self.cap * 2 * 4)
        self.off_ret = al(self.off_cnt + self.world * 8)
        self.off_flag = al(self.off_ret + self.pairs_cap * hidden * 2)
        self.nbytes = al(self.off_flag + self.world * 8)
        self.base, self.peer_base, self._opened = _symmetric_alloc(ctx, lib, self.nbytes, 0, self.world, self.rank)
        dev = ctx.device
        self.counters = torch.zeros(8, dtype=torch.int32, device=dev)          # [epoch, done x 3]
        self.prm = EpParams()
        q = self.prm
        q.world, q.rank, q.cap, q.pairs_cap, q.H = self.world, self.rank, self.cap, self.pairs_cap, hidden
        for r in range(self.world):
            b = self.peer_base[r]
            q.rx_tok[r], q.rx_meta[r], q.rx_cnt[r] = b + self.off_tok, b + self.off_meta, b + self.off_cnt
            q.ret[r], q.ret_flag[r] = b + self.off_ret, b + self.off_flag
        q.epoch = self.counters.data_ptr()
        q.done = self.counters.data_ptr() + 4
        q.wait_cycles = int(wait_ms * 1_900_000)
        q.status = N.Workspace.get(dev).status.data_ptr()
        rows = self.world * self.cap
        self.dest = torch.empty(self.pairs_cap, dtype=torch.int32, device=dev)
        self.slot = torch.empty(self.pairs_cap, dtype=torch.int32, device=dev)
        self.cnt = torch.zeros(8, dtype=torch.int32, device=dev)
        self.rx_idx = torch.empty(rows, 1, dtype=torch.int32, device=dev)
        self.rx_cnt = torch.zeros(8, dtype=torch.int32, device=dev)
        self.ones = torch.ones(rows, 1, dtype=torch.float32, device=dev)
        self.rx_view = _view_bf16(self.base + self.off_tok, rows, hidden, dev, self)
        self.exchanges = 0
        dist.barrier(group=ctx.ctrl_group)

    def fits(self, T: int, k: int) -> bool:
        return T <= self.max_tokens and k == self.k

    def exchange(self, h, idx, w, num_experts, run_experts, add_f32=None, residual=None):
        """h [T, H] bf16 (T may be 0), idx / w [T, k]; run_experts(rows bf16 [R, H], expert ids int32 [R, 1], ones) ->
        fp32 [R, H].  Returns sum_k w * expert(h) + add_f32 + residual as bf16 [T, H]."""
        T = h.shape[0]
        k = self.k
        ws = N.Workspace.get(h.device)
        st = N._stream()
        x2, ldx = (h, self.H) if T == 0 else N._rows2d(h)
        idx32 = idx if idx is None or idx.dtype == torch.int32 else idx.int()
        N._check(self.lib.xft_ep_dispatch(N._p(x2 if T else None), ldx, N._p(idx32), T, k, num_experts, N._p(self.dest),
                                          N._p(self.slot), N._p(self.cnt), C.byref(self.prm), st), "ep_dispatch")
        N._check(self.lib.xft_ep_receive(N._p(self.rx_idx), N._p(self.rx_cnt), C.byref(self.prm), st), "ep_receive")
        y = run_experts(self.rx_view, self.rx_idx, self.ones)
        N._check(self.lib.xft_ep_return(N._p(y), N._p(self.rx_cnt), C.byref(self.prm), st), "ep_return")
        out = torch.empty(T, self.H, dtype=torch.bfloat16, device=h.device)
        r2, ldr = (None, 0)
        if residual is not None and T:
            r2, ldr = N._rows2d(residual)
        wf = None if w is None else w.float().contiguous()
        N._check(self.lib.xft_ep_combine(N._p(wf), N._p(self.dest), T, k, N._p(add_f32), N._p(r2), ldr, N._p(out),
                                         C.byref(self.prm), st), "ep_combine")
        ws.launches += 5
        self.exchanges += 1
        return out

    def close(self) -> None:
        for p in self._opened:
            self.lib.xft_comm_ipc_close(C.c_void_p(p))
        self._opened = []
        if self.base:
            self.lib.xft_comm_free(C.c_void_p(self.base))
            self.base = 0
