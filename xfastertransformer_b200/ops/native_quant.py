"""Bindings of the quantised GEMM kernels (csrc/kernels/quant_gemm_sm100.cu): weight-only int8 / uint4 / nf4 /
fp8-e4m3 dequant-GEMM and W8A8 (dynamic int8 activations x int8 weights on the int8 tensor path)."""
from __future__ import annotations

import ctypes as C

import torch

from . import native as N

_QT = {"int8": 0, "int4": 1, "nf4": 2, "fp8": 3, "int4f": 4}
_ready = False


def _lib():
    global _ready
    lib = N.lib()
    if not _ready:
        for fn in ("xft_qgemm", "xft_quant_act", "xft_row_sum", "xft_w8a8_gemm"):
            getattr(lib, fn).restype = C.c_int
        _ready = True
    return lib


def _row_sums(x2, ldx):
    T, K = x2.shape
    out = torch.empty(T, dtype=torch.float32, device=x2.device)
    N._check(_lib().xft_row_sum(N._p(x2), ldx, N._p(out), T, K, N._stream()), "row_sum")
    N.Workspace.get(x2.device).launches += 1
    return out


def _int4_fast(W, w):
    """uint4 weights in the kernel's fast layout (cached on the weight): within every 32-bit word the eight codes
    e0..e7 move from nibble order [e0 e1 ... e7] to [e0 e2 e4 e6 | e1 e3 e5 e7], which lets the kernel build a bf16
    pair with one shift and one logic op; and the zero point absorbs the constant 128 the kernel adds to each code."""
    c = W.cache.get("int4f")
    if c is None:
        w32 = w.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        out = torch.zeros_like(w32)
        for i in range(4):
            out |= ((w32 >> (8 * i)) & 0xF) << (4 * i)                 # e_{2i}   -> nibble i
            out |= ((w32 >> (8 * i + 4)) & 0xF) << (16 + 4 * i)        # e_{2i+1} -> nibble i + 4
        out = torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)
        wf = out.view(torch.uint8).view(w.shape[0], -1)
        zero = (W.zero if W.zero is not None else torch.zeros_like(W.scale)) - 128.0 * W.scale
        c = (wf, zero.contiguous())
        W.cache["int4f"] = c
    return c


def _qgemm(x, W, n_out, gated, bias, act, residual, res_scale, out_dtype):
    x2, ldx = N._rows2d(x)
    T, K = x2.shape
    if K % 8:
        raise N.KernelError(f"quantised GEMM needs K % 8 == 0 (got {K})")
    fp32 = out_dtype == torch.float32
    out = torch.empty(T, n_out, dtype=torch.float32 if fp32 else torch.bfloat16, device=x.device)
    ws = N.Workspace.get(x.device)
    zero = W.zero if (W.zero is not None and W.kind != "nf4") else None
    xsum = _row_sums(x2, ldx) if zero is not None else None
    r2, ldr = (None, 0)
    if residual is not None:
        r2 = residual.reshape(-1, residual.shape[-1])
        ldr = r2.stride(0)
    w = W.w if W.w.dtype != torch.float8_e4m3fn else W.w.view(torch.uint8)
    if (w.stride(0) * w.element_size()) % 16:
        # TMA rows must start on 16-byte boundaries: keep a copy whose row pitch is padded (zero codes past K
        # multiply zero-filled activations, so they add nothing)
        wp = W.cache.get("w_pitch16")
        if wp is None:
            cols = w.shape[1]
            pad = (-cols * w.element_size()) % 16 // w.element_size()
            wp = torch.nn.functional.pad(w, (0, pad)).contiguous()[:, :cols]
            W.cache["w_pitch16"] = wp
        w = wp
    scale_ld = W.scale.shape[1] if W.kind == "fp8" else 0
    kind = W.kind
    if kind == "int4":
        cols = w.shape[1]
        full = w if w.is_contiguous() else torch.as_strided(w, (w.shape[0], w.stride(0)), (w.stride(0), 1))
        wq, zero = _int4_fast(W, full)
        w = wq[:, :cols]
        kind = "int4f"
        if xsum is None:
            xsum = _row_sums(x2, ldx)
    rc = _lib().xft_qgemm(N._p(x2), ldx, N._p(w), w.shape[0], w.stride(0) * w.element_size(), _QT[kind], N._p(out),
                          out.stride(0), int(fp32), T, n_out, K, int(gated), n_out if gated else 0, N._p(W.scale),
                          N._p(zero), N._p(xsum), scale_ld, N._p(bias), N._p(r2), ldr, C.c_float(res_scale),
                          N._ACT[act], N._p(ws.ws), C.c_size_t(ws.ws_bytes), N._p(ws.counters), ws.n_counters,
                          N._p(ws.status), N._stream())
    N._check(rc, f"qgemm[{W.kind}]")
    ws.launches += 1
    return out


_QMODE = {"int8": 0, "w8a8": 0, "int4": 1, "nf4": 2}
_SRC_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def quantize_rows(w, kind):
    """Quantise-at-load on the device: dense w [out, in] (fp32 / fp16 / bf16, on the GPU) -> (codes, scale[out],
    zero[out], wsum[out] or None) in the layouts of `ops.reference.quantize_{int8,uint4,nf4}_per_channel`: int8 codes
    [out, in], or two 4-bit codes per byte [out, in / 2].  `wsum` (sum of the codes per row) only for kind "w8a8"."""
    if w.dim() != 2 or w.stride(1) != 1 or w.dtype not in _SRC_DT:
        w = w.contiguous() if w.dtype in _SRC_DT else w.float().contiguous()
    rows, K = w.shape
    mode = _QMODE[kind]
    if mode and K % 2:
        raise ValueError("4-bit weights need an even input dimension")
    q = torch.empty(rows, K if mode == 0 else K // 2, dtype=torch.int8 if mode == 0 else torch.uint8, device=w.device)
    sz = torch.empty(3, rows, dtype=torch.float32, device=w.device)
    wsum = sz[2] if kind == "w8a8" else None
    fn = _lib().xft_quantize_rows
    fn.restype = C.c_int
    N._check(fn(N._p(w), _SRC_DT[w.dtype], C.c_longlong(w.stride(0)), rows, K, mode, N._p(q), C.c_longlong(q.stride(0)),
                N._p(sz[0]), N._p(sz[1]), N._p(wsum), N._stream()), "quantize_rows")
    N.Workspace.get(w.device).launches += 1
    return q, sz[0], sz[1], wsum


def quant_act(x2, ldx):
    """bf16 [T,K] -> (int8 [T,K], scale[T], zero[T], qsum[T]) per-row dynamic asymmetric."""
    T, K = x2.shape
    q = torch.empty(T, K, dtype=torch.int8, device=x2.device)
    s = torch.empty(3, T, dtype=torch.float32, device=x2.device)
    N._check(_lib().xft_quant_act(N._p(x2), ldx, N._p(q), K, N._p(s[0]), N._p(s[1]), N._p(s[2]), T, K, N._stream()),
             "quant_act")
    N.Workspace.get(x2.device).launches += 1
    return q, s[0], s[1], s[2]


def _w8a8(x, W, rows, bias, act, residual, res_scale, out_dtype, row0=0):
    x2, ldx = N._rows2d(x)
    T, K = x2.shape
    q, sa, za, qs = quant_act(x2, ldx)
    fp32 = out_dtype == torch.float32
    out = torch.empty(T, rows, dtype=torch.float32 if fp32 else torch.bfloat16, device=x.device)
    ws = N.Workspace.get(x.device)
    r2, ldr = (None, 0)
    if residual is not None:
        r2 = residual.reshape(-1, residual.shape[-1])
        ldr = r2.stride(0)
    w = W.w[row0:row0 + rows]
    sl = slice(row0, row0 + rows)
    rc = _lib().xft_w8a8_gemm(N._p(q), K, N._p(w), W.w.stride(0), N._p(out), out.stride(0), int(fp32), T, rows, K,
                              N._p(sa), N._p(za), N._p(qs), N._p(W.scale[sl]), N._p(W.zero[sl]), N._p(W.wsum[sl]),
                              N._p(bias), N._p(r2), ldr, C.c_float(res_scale), N._ACT[act], N._p(ws.ws),
                              C.c_size_t(ws.ws_bytes), N._p(ws.counters), ws.n_counters, N._p(ws.status), N._stream())
    N._check(rc, "w8a8_gemm")
    ws.launches += 1
    return out


def linear(x, W, bias=None, act=None, residual=None, res_scale=1.0, out_dtype=None):
    if W.kind == "w8a8":
        return _w8a8(x, W, W.out_features, bias, act, residual, res_scale, out_dtype)
    if W.kind in _QT:
        return _qgemm(x, W, W.out_features, False, bias, act, residual, res_scale, out_dtype)
    raise N.KernelError(f"no sm_100a GEMM for weight kind {W.kind}")


def linear_gated(x, W, act="silu", bias=None):
    I = W.out_features // 2
    if W.kind == "w8a8":
        # one int8 GEMM over both halves (activations are quantised once), then act(gate)*up
        gu = _w8a8(x, W, 2 * I, bias, None, None, 1.0, None)
        return N.gated_act(gu, act)
    if W.kind == "fp8" and I % 128:
        gu = _qgemm(x, W, 2 * I, False, bias, None, None, 1.0, None)
        return N.gated_act(gu, act)
    return _qgemm(x, W, I, True, bias, act, None, 1.0, None)
