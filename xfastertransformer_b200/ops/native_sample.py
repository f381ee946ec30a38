"""Bindings of the sampling kernels (csrc/kernels/sample.cu)."""
from __future__ import annotations

import ctypes as C

import torch

from . import native as N


def sample_top_k_top_p(logits, top_k, top_p, temperature, uniform):
    l2 = logits.reshape(-1, logits.shape[-1])
    if l2.dtype != torch.float32 or l2.stride(1) != 1:
        l2 = l2.float().contiguous()
    rows, V = l2.shape
    u = uniform.to(device=l2.device, dtype=torch.float32).contiguous()
    out = torch.empty(rows, dtype=torch.int32, device=l2.device)
    lib = N.lib()
    lib.xft_sample_topk_topp.restype = C.c_int
    N._check(lib.xft_sample_topk_topp(N._p(l2), l2.stride(0), rows, V, int(top_k), C.c_float(top_p),
                                      C.c_float(temperature), N._p(u), N._p(out), N._stream()), "sample_topk_topp")
    N.Workspace.get(l2.device).launches += 1
    return out.long()


BEAM_TOPK_MAX = 64


def beam_topk(logits, k):
    """Per row of fp32 logits [rows, V]: (log-softmax values [rows, k] fp32, token ids [rows, k] int64) of the k best
    entries, best first, lower id first among equals.  k <= BEAM_TOPK_MAX."""
    l2 = logits.reshape(-1, logits.shape[-1])
    if l2.dtype != torch.float32 or l2.stride(1) != 1:
        l2 = l2.float().contiguous()
    rows, V = l2.shape
    k = int(k)
    if not 1 <= k <= min(V, BEAM_TOPK_MAX):
        raise ValueError(f"beam_topk: k = {k} outside [1, min(vocab, {BEAM_TOPK_MAX})]")
    vals = torch.empty(rows, k, dtype=torch.float32, device=l2.device)
    idx = torch.empty(rows, k, dtype=torch.int32, device=l2.device)
    lib = N.lib()
    lib.xft_beam_topk.restype = C.c_int
    N._check(lib.xft_beam_topk(N._p(l2), l2.stride(0), rows, V, k, N._p(vals), N._p(idx), N._stream()), "beam_topk")
    N.Workspace.get(l2.device).launches += 1
    return vals, idx.long()


def repetition_penalty(logits, token_lists, penalty, vocab_offset=0):
    """In place on fp32 logits [rows, V]; `token_lists`: per-row iterable of token ids."""
    rows, V = logits.shape
    m = max((len(t) for t in token_lists), default=0)
    if m == 0 or penalty == 1.0:
        return logits
    tk = torch.full((rows, m), -1, dtype=torch.int32)
    for r, t in enumerate(token_lists):
        if len(t):
            tk[r, :len(t)] = torch.as_tensor(list(t), dtype=torch.int32)
    tk = tk.to(logits.device)
    lib = N.lib()
    lib.xft_repetition_penalty.restype = C.c_int
    N._check(lib.xft_repetition_penalty(N._p(logits), logits.stride(0), rows, V, N._p(tk), m, C.c_float(penalty),
                                        vocab_offset, N._stream()), "repetition_penalty")
    N.Workspace.get(logits.device).launches += 1
    return logits
