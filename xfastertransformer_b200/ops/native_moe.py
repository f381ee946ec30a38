"""Bindings of the MoE kernels (csrc/kernels/moe.cu) and the grouped tcgen05 GEMM: router, device-side dispatch
plan, row gather, grouped gate‖up(+act) and down GEMMs over rows sorted by expert, weighted combine.  Nothing
synchronises with the host, so the whole MoE layer is capturable in the decode CUDA graph."""
from __future__ import annotations

import ctypes as C
import torch

from . import native as N
from . import reference as R

_KIND = {"mixtral": 0, "softmax_topk": 1, "deepseek": 2}
_ready = False


def _lib():
    global _ready
    lib = N.lib()
    if not _ready:
        for fn in ("xft_moe_route", "xft_moe_plan", "xft_moe_gather", "xft_moe_combine", "xft_gemm_bf16_grouped",
                   "xft_qgemm_grouped"):
            getattr(lib, fn).restype = C.c_int
        _ready = True
    return lib


def route(logits, kind, top_k, bias=None, n_group=1, topk_group=1, routed_scaling=1.0, norm_topk=True,
          scoring="sigmoid"):
    l2 = logits.reshape(-1, logits.shape[-1])
    assert l2.dtype == torch.float32 and l2.stride(1) == 1
    T, E = l2.shape
    idx = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    rc = _lib().xft_moe_route(N._p(l2), l2.stride(0), T, E, top_k, _KIND[kind], N._p(bias), n_group, topk_group,
                              C.c_float(routed_scaling), int(bool(norm_topk)), int(scoring == "sigmoid"), N._p(idx),
                              N._p(w), N._stream())
    N._check(rc, "moe_route")
    N.Workspace.get(logits.device).launches += 1
    return idx, w


def pack_experts(experts) -> dict:
    """Stack the local experts' weights: gate‖up [E*2I, H] and down [E*H, I] (bf16; other kinds are expanded
    once here).  The per-expert LinearWeights are re-pointed at views of the stacks so nothing is held twice."""
    # the pack lives in the first expert's weight object (an id()-keyed table would hand a dead list's pack to a
    # new list that happens to reuse its address)
    gu0, dn0 = experts[0]
    pk = gu0.cache.get("moe_pack")
    if pk is not None and pk["E"] == len(experts) and pk["last"] is experts[-1][0]:
        return pk
    if all(g.kind == "fp8" and d.kind == "fp8" for g, d in experts) and _fp8_packable(gu0, dn0):
        return _pack_fp8(experts)
    I, H = dn0.in_features, dn0.out_features
    E = len(experts)
    dev = gu0.w.device
    gu = torch.empty(E * 2 * I, H, dtype=torch.bfloat16, device=dev)
    dn = torch.empty(E * H, I, dtype=torch.bfloat16, device=dev)
    for e, (g, d) in enumerate(experts):
        gv, dv = gu[e * 2 * I:(e + 1) * 2 * I], dn[e * H:(e + 1) * H]
        gv.copy_(g.w if g.kind == "bf16" else R.dequant_weight(g))
        dv.copy_(d.w if d.kind == "bf16" else R.dequant_weight(d))
        if g.kind == "bf16":
            g.w = gv
        if d.kind == "bf16":
            d.w = dv
    pk = dict(gu=gu, dn=dn, I=I, H=H, E=E, last=experts[-1][0])
    gu0.cache["moe_pack"] = pk
    return pk


def _fp8_packable(gu: "object", dn: "object") -> bool:
    I, H = dn.in_features, dn.out_features
    return gu.block == 128 and dn.block == 128 and I % 128 == 0 and H % 128 == 0


def _pack_fp8(experts) -> dict:
    """fp8 experts stay fp8 on the device: the e4m3 matrices and their 128x128 block scales are stacked and the
    grouped fp8 GEMM expands tiles to bf16 in shared memory on the way to the tensor core."""
    gu0, dn0 = experts[0]
    I, H = dn0.in_features, dn0.out_features
    E = len(experts)
    dev = gu0.w.device
    gu = torch.empty(E * 2 * I, H, dtype=torch.uint8, device=dev)
    dn = torch.empty(E * H, I, dtype=torch.uint8, device=dev)
    gus = torch.empty(E * (2 * I // 128), gu0.scale.shape[1], dtype=torch.float32, device=dev)
    dns = torch.empty(E * (H // 128), dn0.scale.shape[1], dtype=torch.float32, device=dev)
    for e, (g, d) in enumerate(experts):
        gv, dv = gu[e * 2 * I:(e + 1) * 2 * I], dn[e * H:(e + 1) * H]
        gv.copy_(g.w.view(torch.uint8))
        dv.copy_(d.w.view(torch.uint8))
        gus[e * (2 * I // 128):(e + 1) * (2 * I // 128)].copy_(g.scale)
        dns[e * (H // 128):(e + 1) * (H // 128)].copy_(d.scale)
        g.w = gv.view(torch.float8_e4m3fn)               # re-point at the stack: nothing is held twice
        d.w = dv.view(torch.float8_e4m3fn)
    pk = dict(gu=gu, dn=dn, gus=gus, dns=dns, I=I, H=H, E=E, fp8=True, last=experts[-1][0])
    gu0.cache["moe_pack"] = pk
    return pk


def moe_experts(x, idx, w, experts, act="silu", expert_offset=0, packed=None, expected_pairs=None):
    """sum_k w[t,k] * down_e(act(gate_e x) * up_e x) over the local experts -> fp32 [T, H].  `expected_pairs`: about how
    many (token, expert) pairs are real when most rows of `idx` are padding (-1), e.g. the receive area of the expert
    exchange; it only picks the token tile of the grouped GEMMs."""
    pk = packed or pack_experts(experts)
    x2, ldx = N._rows2d(x)
    T, H = x2.shape
    k = idx.shape[1]
    E, I = pk["E"], pk["I"]
    dev = x.device
    ws = N.Workspace.get(dev)
    lib = _lib()
    avg = max(1, ((T * k if expected_pairs is None else min(int(expected_pairs), T * k)) + E - 1) // E)
    bn = 16 if avg <= 16 else 32 if avg <= 32 else 64 if avg <= 64 else 128
    max_rows = T * k
    max_tiles = (max_rows + bn - 1) // bn + E
    idx32 = idx if idx.dtype == torch.int32 else idx.int()
    pos = torch.empty(T * k, dtype=torch.int32, device=dev)
    src = torch.empty(max_rows, dtype=torch.int32, device=dev)
    row_w = torch.empty(max_rows, dtype=torch.float32, device=dev)
    tiles = torch.empty(max_tiles, 4, dtype=torch.int32, device=dev)
    meta = torch.empty(2, dtype=torch.int32, device=dev)
    N._check(lib.xft_moe_plan(N._p(idx32), N._p(w.contiguous()), T, k, expert_offset, expert_offset + E, bn, N._p(pos),
                              N._p(src), N._p(row_w), N._p(tiles), N._p(meta), max_tiles, max_rows, N._stream()),
             "moe_plan")
    xs = torch.empty(max_rows, H, dtype=torch.bfloat16, device=dev)
    N._check(lib.xft_moe_gather(N._p(x2), ldx, N._p(src), N._p(meta), N._p(xs), max_rows, H, N._stream()), "moe_gather")
    h1 = torch.empty(max_rows, I, dtype=torch.bfloat16, device=dev)
    if pk.get("fp8"):
        ys = torch.empty(max_rows, H, dtype=torch.float32, device=dev)
        N._check(lib.xft_qgemm_grouped(N._p(xs), H, max_rows, N._p(pk["gu"]), E * 2 * I, H, N._p(h1), I, 0, I, H, 1, I, 2 * I,
                                       N._p(pk["gus"]), pk["gus"].shape[1], N._p(tiles), N._p(meta), max_tiles, min(bn, 128),
                                       N._p(None), N._ACT[act], N._p(ws.status), N._stream()), "grouped fp8 gate_up")
        N._check(lib.xft_qgemm_grouped(N._p(h1), I, max_rows, N._p(pk["dn"]), E * H, I, N._p(ys), H, 1, H, I, 0, 0, H,
                                       N._p(pk["dns"]), pk["dns"].shape[1], N._p(tiles), N._p(meta), max_tiles, min(bn, 128),
                                       N._p(row_w), 0, N._p(ws.status), N._stream()), "grouped fp8 down")
        out = torch.empty(T, H, dtype=torch.float32, device=dev)
        N._check(lib.xft_moe_combine(N._p(ys), N._p(pos), k, N._p(None), N._p(None), 0, N._p(None), N._p(out), T, H,
                                     N._stream()), "moe_combine")
        ws.launches += 5
        return out
    N._check(lib.xft_gemm_bf16_grouped(N._p(xs), H, max_rows, N._p(pk["gu"]), E * 2 * I, H, N._p(h1), I, 0, I, H, 1, I,
                                       2 * I, N._p(tiles), N._p(meta), max_tiles, bn, N._p(None), N._ACT[act],
                                       N._p(ws.status), N._stream()), "grouped gate_up")
    ys = torch.empty(max_rows, H, dtype=torch.float32, device=dev)
    N._check(lib.xft_gemm_bf16_grouped(N._p(h1), I, max_rows, N._p(pk["dn"]), E * H, I, N._p(ys), H, 1, H, I, 0, 0, H,
                                       N._p(tiles), N._p(meta), max_tiles, bn, N._p(row_w), 0, N._p(ws.status),
                                       N._stream()), "grouped down")
    out = torch.empty(T, H, dtype=torch.float32, device=dev)
    N._check(lib.xft_moe_combine(N._p(ys), N._p(pos), k, N._p(None), N._p(None), 0, N._p(None), N._p(out), T, H,
                                 N._stream()), "moe_combine")
    ws.launches += 5
    return out
