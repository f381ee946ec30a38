"""DeepSeek MLA on the GPU: absorb GEMMs as grouped tcgen05 GEMMs (one group per head) around the latent-cache
attention kernel (csrc/kernels/mla.cu).  The absorbed form is used for prefill and decode alike."""
from __future__ import annotations

import ctypes as C
from typing import Dict

import torch

from . import native as N

_ready = False
_tables: Dict[tuple, tuple] = {}


def _lib():
    global _ready
    lib = N.lib()
    if not _ready:
        lib.xft_mla_attention.restype = C.c_int
        lib.xft_gemm_bf16_grouped.restype = C.c_int
        _ready = True
    return lib


def _head_tiles(H: int, T: int, dev):
    """Static tile table of a per-head grouped GEMM: rows of head h are [h*T, (h+1)*T)."""
    bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128
    key = (H, T, bn, dev.index)
    if key not in _tables:
        rows = []
        for h in range(H):
            for j in range(0, T, bn):
                rows.append([h, h * T + j, min(bn, T - j), 0])
        tiles = torch.tensor(rows, dtype=torch.int32, device=dev)
        meta = torch.tensor([len(rows), H * T], dtype=torch.int32, device=dev)
        _tables[key] = (tiles, meta, len(rows), bn)
    return _tables[key]


def _per_head_gemm(x_ht, w_stacked, H, T, n_out, k_in):
    """x_ht [H*T, k_in] bf16 (rows grouped by head) x per-head weights [H*n_out, k_in] -> [H*T, n_out] bf16."""
    tiles, meta, nt, bn = _head_tiles(H, T, x_ht.device)
    out = torch.empty(H * T, n_out, dtype=torch.bfloat16, device=x_ht.device)
    ws = N.Workspace.get(x_ht.device)
    rc = _lib().xft_gemm_bf16_grouped(N._p(x_ht), k_in, H * T, N._p(w_stacked), H * n_out, k_in, N._p(out), n_out, 0,
                                      n_out, k_in, 0, 0, n_out, N._p(tiles), N._p(meta), nt, bn, N._p(None), 0,
                                      N._p(ws.status), N._stream())
    N._check(rc, "per-head grouped gemm")
    ws.launches += 1
    return out


def mla_attention(q_nope, q_rope, latent_cache, block_table, cu_q, kv_lens, w_uk, w_uv, scale, absorbed=True, meta=None):
    T, Hl, nope = q_nope.shape
    L = w_uk.shape[2]
    vd = w_uv.shape[1]
    rope = q_rope.shape[2]
    assert L == 512 and rope == 64, "MLA kernel is specialised for kv_lora_rank 512 + rope 64"
    dev = q_nope.device
    ws = N.Workspace.get(dev)
    # W_uk^T stacked per head: [Hl*L, nope] (linear weight [out=L, in=nope])
    # cached on the tensor itself (an id()-keyed table would hand a dead tensor's copy to a new tensor that reuses
    # its address)
    wk = getattr(w_uk, "_xft_wk_t", None)
    if wk is None or wk.shape != (Hl * L, nope):
        wk = w_uk.transpose(1, 2).contiguous().view(Hl * L, nope)
        w_uk._xft_wk_t = wk
    wv = w_uv.reshape(Hl * vd, L)
    q_ht = q_nope.transpose(0, 1).contiguous().view(Hl * T, nope)
    q_abs = _per_head_gemm(q_ht, wk, Hl, T, L, nope)                 # [Hl*T, L]
    if meta is not None and getattr(meta, "cu_q_dev", None) is not None:
        cu_dev, kv_dev, max_kv, B = meta.cu_q_dev, meta.kv_lens_dev, meta.max_kv, len(kv_lens)
        decode = meta.is_decode
    else:
        cu_dev = torch.tensor(list(cu_q), dtype=torch.int32, device=dev)
        kv_dev = torch.tensor(list(kv_lens), dtype=torch.int32, device=dev)
        max_kv, B = max(kv_lens), len(kv_lens)
        decode = all(cu_q[i + 1] - cu_q[i] == 1 for i in range(B))
    o_lat = torch.empty(Hl * T, L, dtype=torch.bfloat16, device=dev)
    nb, _, bs, W = latent_cache.shape
    chunks = (Hl + 15) // 16
    nsplit, po, pm = 1, None, None
    if decode:
        ntiles = (max_kv + 31) // 32
        ctas = T * chunks
        nsplit = max(1, min(296 // max(ctas, 1), ntiles // 8 if ntiles >= 16 else 1, 16))
        if nsplit > 1 and ctas <= ws.attn_counters.numel():
            po, pm = ws.attn_partials(ctas * nsplit * 16 * L, ctas * nsplit * 32)
        else:
            nsplit = 1
    q_rope = q_rope.contiguous()
    rc = _lib().xft_mla_attention(N._p(q_abs), C.c_longlong(T * L), C.c_longlong(L), N._p(q_rope), C.c_longlong(rope),
                                  C.c_longlong(Hl * rope), N._p(o_lat), C.c_longlong(T * L), C.c_longlong(L),
                                  N._p(latent_cache), N._p(block_table), block_table.stride(0), N._p(cu_dev),
                                  N._p(kv_dev), B, T, Hl, bs, nb, C.c_float(scale), nsplit, N._p(po), N._p(pm),
                                  N._p(ws.attn_counters), N._p(ws.status), N._stream())
    N._check(rc, "mla_attention")
    ws.launches += 1
    o = _per_head_gemm(o_lat, wv, Hl, T, vd, L)                      # [Hl*T, vd]
    return o.view(Hl, T, vd).transpose(0, 1).contiguous()
