"""ctypes bindings to the hand-written sm_100a kernels (``lib/libxft_b200_kernels.so``).

Tensors are passed as raw device pointers plus the current CUDA stream, so every call is
capturable in a CUDA graph and costs no framework dispatch.  Nothing here falls back to a
PyTorch implementation: a missing library or an unsupported variant raises.

A `Workspace` per device owns the scratch the kernels need (split-K partial tiles and tile
counters, split-KV partials, the status word the bounded waits report into); it is allocated
once, so steady-state steps allocate only their outputs.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional

import torch

_LIB = None
_ACT = {None: 0, "none": 0, "relu": 1, "silu": 2, "gelu": 3, "gelu_tanh": 3, "gelu_new": 3, "gelu_pytorch_tanh": 3,
        "swiglu": 2}

STATUS_TEXT = {0: "ok", 1: "producer timed out waiting for a free stage", 2: "MMA warp timed out waiting for TMA data",
               3: "epilogue timed out waiting for the accumulator", 4: "timed out waiting for a peer flag",
               5: "index out of range (access skipped)", 6: "a CTA timed out waiting for the other CTAs of its grid"}


class KernelError(RuntimeError):
    pass


def _ENV():
    from ..utils.flags import Env
    return Env.get()


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libxft_b200_kernels.so")


def lib():
    global _LIB
    if _LIB is None:
        p = lib_path()
        if not os.path.exists(p):
            raise KernelError(f"{p} is missing: run `python csrc/build.py` (or __graft_entry__.build())")
        _LIB = C.CDLL(p)
        for fn in ("xft_gemm_bf16", "xft_embedding", "xft_rmsnorm", "xft_layernorm", "xft_gated_act",
                   "xft_qkv_rope_cache", "xft_rope", "xft_latent_write", "xft_argmax", "xft_paged_attention"):
            getattr(_LIB, fn).restype = C.c_int
        # XFT_PDL=0: plain stream order instead of programmatic dependent launch between the kernels
        _LIB.xft_set_pdl(int(os.environ.get("XFT_PDL", "1") != "0"))
    return _LIB


def _p(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


class Workspace:
    _by_dev: Dict[int, "Workspace"] = {}

    def __init__(self, device: torch.device):
        self.device = device
        self.ws_bytes = 96 << 20
        self.ws = torch.empty(self.ws_bytes // 4, dtype=torch.float32, device=device)
        self.n_counters = 8192
        self.counters = torch.zeros(self.n_counters, dtype=torch.int32, device=device)
        self.attn_counters = torch.zeros(16384, dtype=torch.int32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.part_o = None
        self.part_ml = None
        self.launches = 0

    @classmethod
    def get(cls, device: torch.device) -> "Workspace":
        idx = device.index if device.index is not None else torch.cuda.current_device()
        if idx not in cls._by_dev:
            cls._by_dev[idx] = cls(torch.device("cuda", idx))
        return cls._by_dev[idx]

    PART_O_FLOATS = 16 << 20          # split-KV partial outputs: fixed size, so captured graphs never see it move

    def attn_partials(self, n_o: int, n_ml: int):
        """Scratch of the split-KV decode.  Allocated once at a fixed size: a CUDA graph captured earlier keeps
        pointing at it, so it must never be reallocated; callers clamp their split count to its capacity."""
        if self.part_o is None:
            self.part_o = torch.empty(self.PART_O_FLOATS, dtype=torch.float32, device=self.device)
            self.part_ml = torch.empty(self.PART_O_FLOATS // 32, dtype=torch.float32, device=self.device)
        if n_o > self.part_o.numel() or n_ml > self.part_ml.numel():
            raise KernelError(f"split-KV scratch too small for {n_o} partial outputs")
        return self.part_o, self.part_ml

    def check_status(self) -> None:
        """Read the status word (synchronises).  Raises if any kernel reported a time-out or a
        bad index; the context stays usable."""
        s = int(self.status[0].item())
        if s != 0:
            self.status.zero_()
            raise KernelError(f"kernel status {s}: {STATUS_TEXT.get(s, '?')}")


def launches(device=None) -> int:
    d = device or torch.device("cuda", torch.cuda.current_device())
    return Workspace.get(d).launches


# ------------------------------------------------------------------------------------------
def _rows2d(x: torch.Tensor):
    """[T, K] view with unit inner stride -> (tensor, ld)."""
    if x.dim() != 2:
        x = x.reshape(-1, x.shape[-1])
    if x.stride(1) != 1 or (x.stride(0) * x.element_size()) % 16 or x.data_ptr() % 16:
        x = x.contiguous()
    return x, x.stride(0) if x.shape[0] > 1 else max(x.stride(0), x.shape[1])


def embedding(ids, table, scale, out_dtype, pos_table=None, positions=None, pos_offset=0):
    T, H = ids.numel(), table.shape[1]
    out = torch.empty(T, H, dtype=torch.bfloat16, device=table.device)
    ws = Workspace.get(table.device)
    ids32 = ids if ids.dtype == torch.int32 else ids.int()
    pos32 = None if positions is None else (positions if positions.dtype == torch.int32 else positions.int())
    rc = lib().xft_embedding(_p(ids32), _p(table), _p(out), T, H, table.shape[0], C.c_float(scale), _p(pos_table),
                             _p(pos32), pos_offset, 0 if pos_table is None else pos_table.shape[0], _p(ws.status),
                             _stream())
    _check(rc, "embedding")
    ws.launches += 1
    return out if out_dtype == torch.bfloat16 else out.to(out_dtype)


def rmsnorm(x, w, eps, residual=None):
    x2, ldx = _rows2d(x)
    T, H = x2.shape
    y = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    h = None
    r2, ldr = (None, 0)
    if residual is not None:
        r2, ldr = _rows2d(residual)
        h = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    rc = lib().xft_rmsnorm(_p(x2), ldx, _p(r2), ldr, _p(w), _p(y), H, _p(h), T, H, C.c_float(eps), _stream())
    _check(rc, "rmsnorm")
    Workspace.get(x.device).launches += 1
    y = y.view(*x.shape[:-1], H)
    return (y, h.view_as(y)) if residual is not None else y


def layernorm(x, w, b, eps):
    x2, ldx = _rows2d(x)
    T, H = x2.shape
    y = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    rc = lib().xft_layernorm(_p(x2), ldx, _p(w), _p(b), _p(y), H, T, H, C.c_float(eps), _stream())
    _check(rc, "layernorm")
    Workspace.get(x.device).launches += 1
    return y.view(*x.shape[:-1], H)


def gemm_bf16(x, w, N, gated=False, dual_off=0, bias=None, act=None, residual=None, res_scale=1.0, out_dtype=None,
              out=None, row_scale=None, force_splits=0):
    """Y[T,N] = epi(X[T,K] · W[rows,K]^T) on tcgen05.  `w`: bf16 [rows, K] (rows = N, or 2 blocks for gated)."""
    x2, ldx = _rows2d(x)
    T, K = x2.shape
    assert w.dtype == torch.bfloat16 and w.stride(1) == 1 and w.shape[1] == K, (w.dtype, w.shape, K)
    assert x2.dtype == torch.bfloat16
    if K % 8:
        raise KernelError(f"K={K} must be a multiple of 8 (16-byte TMA rows)")
    fp32 = out_dtype == torch.float32
    if out is None:
        out = torch.empty(T, N, dtype=torch.float32 if fp32 else torch.bfloat16, device=x.device)
    r2, ldr = (None, 0)
    if residual is not None:
        r2 = residual.reshape(-1, residual.shape[-1])
        assert r2.stride(1) == 1 and r2.dtype == torch.bfloat16
        ldr = r2.stride(0)
    ws = Workspace.get(x.device)
    if T <= SK_MAX_TOKENS and force_splits == 0 and _sk_choice(T, N, K, gated):
        _gemm_sk(x2, ldx, w, out, T, N, K, gated, dual_off, bias, r2, ldr, res_scale, act, row_scale, None, None, None)
        return out
    # measured on B200 (benchmarks/bench_gemm.py --shapes prefill): the token-major kernel wins wherever the epilogue
    # weighs (reductions up to 8192, ungated); long reductions and the gated form stay on the tile-per-CTA kernel, whose
    # paired 256 x 256 tiles read fewer operand bytes per FLOP
    if _ENV().gemm_prefill_tm and T > 128 and not fp32 and row_scale is None and out.stride(1) == 1 \
            and out.dtype == torch.bfloat16 and (K <= 8192 and not gated or _ENV().gemm_prefill_tm_all):
        # prompt sizes: persistent token-major kernel (tokens are the MMA rows, so bias / residual / output move as
        # 16-byte vectors along a token's features; two TMEM accumulators overlap the epilogue with the next tile)
        L = lib()
        L.xft_gemm_bf16_prefill_tm.restype = C.c_int
        rc = L.xft_gemm_bf16_prefill_tm(_p(x2), ldx, _p(w), w.shape[0], w.stride(0), _p(out), out.stride(0), T, N, K,
                                        int(gated), dual_off, _p(bias), _p(r2), ldr, C.c_float(res_scale), _ACT[act],
                                        _p(ws.status), 0, _stream())
        _check(rc, "gemm_bf16_prefill_tm")
        ws.launches += 1
        return out
    if _ENV().gemm_persistent and T > 128 and gated and not fp32 and row_scale is None and out.stride(1) == 1 \
            and residual is None:
        # gated form of the persistent kernel: four 128-column accumulators, act(gate) * up on the way out
        rc = lib().xft_gemm_bf16_prefill_gated(_p(x2), ldx, _p(w), w.shape[0], w.stride(0), _p(out), out.stride(0), T, N, K,
                                               dual_off, _p(bias), _ACT[act], _p(ws.status), 0, _stream())
        _check(rc, "gemm_bf16_prefill_gated")
        ws.launches += 1
        return out
    if _ENV().gemm_persistent and T > 128 and not gated and not fp32 and row_scale is None and out.stride(1) == 1:
        # persistent tile loop with two TMEM accumulators (csrc/kernels/gemm_prefill_sm100.cu), opt-in
        rc = lib().xft_gemm_bf16_prefill(_p(x2), ldx, _p(w), w.shape[0], w.stride(0), _p(out), out.stride(0), T, N, K,
                                         _p(bias), _p(r2), ldr, C.c_float(res_scale), _ACT[act], _p(None),
                                         _p(ws.status), _p(None), 0, _stream())
        _check(rc, "gemm_bf16_prefill")
        ws.launches += 1
        return out
    rc = lib().xft_gemm_bf16(_p(x2), ldx, _p(w), w.shape[0], w.stride(0), _p(out), out.stride(0), int(fp32), T, N, K,
                             int(gated), dual_off, _p(bias), _p(r2), ldr, C.c_float(res_scale), _ACT[act],
                             _p(row_scale), _p(ws.ws), C.c_size_t(ws.ws_bytes), _p(ws.counters), ws.n_counters,
                             _p(ws.status), force_splits, _stream())
    _check(rc, "gemm_bf16")
    ws.launches += 1
    return out


SK_MAX_TOKENS = 64


class SkQkv(C.Structure):
    """Mirror of the struct of the same name in csrc/kernels/gemm_decode_sm100.cu."""
    _fields_ = [("q_out", C.c_void_p), ("hq", C.c_int), ("hkv", C.c_int), ("positions", C.c_void_p),
                ("table", C.c_void_p), ("rot", C.c_int), ("style", C.c_int), ("rot_off", C.c_int), ("max_pos", C.c_int),
                ("q_scale", C.c_void_p), ("kc", C.c_void_p), ("vc", C.c_void_p), ("bs", C.c_int),
                ("nslots", C.c_longlong), ("slots", C.c_void_p)]


_sk_choices: Dict[tuple, int] = {}


def _sk_choice(T, N, K, gated) -> int:
    """Which kernel runs this decode-size product: 0 = the tile-per-CTA kernel (gemm_sm100.cu), otherwise the kernel of
    gemm_decode_sm100.cu (1 = balanced stream, s >= 2 = clusters of s CTAs per tile); see xft_gemm_sk_choice."""
    if not _ENV().gemm_streamk:
        return 0
    key = (pick_bn(T), N, K, bool(gated))
    c = _sk_choices.get(key)
    if c is None:
        c = _sk_choices[key] = int(lib().xft_gemm_sk_choice(T, N, K, int(gated), 0))
    return c


def pick_bn(T: int) -> int:
    return 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128 if T <= 128 else 256


def _gemm_sk(x2, ldx, w, out, T, N, K, gated, dual_off, bias, r2, ldr, res_scale, act, row_scale, rms_eps, comm, qkv):
    """One launch of the decode-size weight-stream GEMM (T <= 64)."""
    ws = Workspace.get(x2.device)
    L = lib()
    L.xft_gemm_sk.restype = C.c_int
    eps = C.byref(C.c_float(rms_eps)) if rms_eps is not None else None
    rc = L.xft_gemm_sk(_p(x2), ldx, _p(w), w.shape[0], w.stride(0), _p(out), out.stride(0) if out is not None else 0,
                       int(out is not None and out.dtype == torch.float32), T, N, K, int(gated), dual_off, _p(bias),
                       _p(r2), ldr, C.c_float(res_scale), _ACT[act], _p(row_scale), eps, _p(ws.ws),
                       C.c_size_t(ws.ws_bytes), _p(ws.counters), ws.n_counters, _p(ws.status),
                       C.byref(comm) if comm is not None else None, C.byref(qkv) if qkv is not None else None, _stream())
    _check(rc, "gemm_sk")
    ws.launches += 1


def can_fuse_qkv_rope(W, T, D, kc, ks, q_norm_w, k_norm_w, style) -> bool:
    """The QKV product can end in RoPE + paged cache append (one kernel instead of two): bf16 weights, head_dim 128,
    a bf16 cache, no per-head q/k norm, at most SK_MAX_TOKENS rows."""
    e = _ENV()
    return (e.gemm_streamk and e.fuse_qkv_rope and W.kind == "bf16" and T <= SK_MAX_TOKENS and D == 128 and ks is None
            and kc.dtype == torch.bfloat16 and q_norm_w is None and k_norm_w is None and style in ("half", "interleaved"))


def qkv_linear_rope_cache(x, W, bias, rms_eps, hq, hkv, positions, table, rot_dim, style, kc, vc, slots, q_scale=None,
                          rot_offset=0):
    """q = RoPE(split(x W^T + b)) and K / V appended to the paged cache, as ONE kernel: the QKV product's epilogue
    rotates each finished head and stores it where the attention kernel reads it.  `rms_eps` set: `x` is the
    un-normalised hidden state and W carries the norm's gain (see fold_norm_gain)."""
    x2, ldx = _rows2d(x)
    T, K = x2.shape
    N = (hq + 2 * hkv) * 128
    assert W.w.shape[0] == N and W.w.shape[1] == K and x2.dtype == torch.bfloat16
    q = torch.empty(T, hq, 128, dtype=torch.bfloat16, device=x.device)
    nb, _, bs, _ = kc.shape
    qp = SkQkv()
    qp.q_out, qp.hq, qp.hkv = q.data_ptr(), hq, hkv
    qp.positions = positions.data_ptr()
    qp.table = table.data_ptr() if table is not None else None
    qp.rot = rot_dim if table is not None else 0
    qp.style = 0 if style == "half" else 1
    qp.rot_off = rot_offset
    qp.max_pos = table.shape[0] if table is not None else 0
    qp.q_scale = q_scale.data_ptr() if q_scale is not None else None
    qp.kc, qp.vc, qp.bs, qp.nslots = kc.data_ptr(), vc.data_ptr(), bs, nb * bs
    qp.slots = slots.data_ptr()
    _gemm_sk(x2, ldx, W.w, None, T, N, K, False, 0, bias, None, 0, 1.0, None, None, rms_eps, None, qp)
    return q


RMS_FUSE_MAX_TOKENS = 64
_ones_cache: Dict[tuple, torch.Tensor] = {}


def _ones(n: int, device) -> torch.Tensor:
    key = (n, str(device))
    if key not in _ones_cache:
        _ones_cache[key] = torch.ones(n, dtype=torch.float32, device=device)
    return _ones_cache[key]


def linear_rms(x, W, eps, bias=None, act=None, gated=False, out_dtype=None):
    """RMSNorm(x) @ W^T where W already carries the norm's gain in its columns (see fold_norm_gain).  Up to
    RMS_FUSE_MAX_TOKENS rows this is ONE kernel: the GEMM computes each token's 1/rms beside its main loop and
    scales the accumulator.  Larger batches (prefill) run the gain-free norm kernel, then the GEMM."""
    assert W.kind == "bf16"
    x2, ldx = _rows2d(x)
    T, K = x2.shape
    N = W.out_features // 2 if gated else W.out_features
    if T > RMS_FUSE_MAX_TOKENS:
        h = rmsnorm(x, _ones(K, x.device), eps)
        return linear_gated(h, W, act, bias) if gated else linear(h, W, bias, act, out_dtype=out_dtype)
    w = W.w
    assert w.dtype == torch.bfloat16 and w.stride(1) == 1 and w.shape[1] == K and x2.dtype == torch.bfloat16
    fp32 = out_dtype == torch.float32
    out = torch.empty(T, N, dtype=torch.float32 if fp32 else torch.bfloat16, device=x.device)
    if _sk_choice(T, N, K, gated):
        _gemm_sk(x2, ldx, w, out, T, N, K, gated, N if gated else 0, bias, None, 0, 1.0, act, None, eps, None, None)
        return out.view(*x.shape[:-1], N)
    ws = Workspace.get(x.device)
    rc = lib().xft_gemm_bf16_rms(_p(x2), ldx, _p(w), w.shape[0], w.stride(0), _p(out), out.stride(0), int(fp32), T, N, K,
                                 int(gated), N if gated else 0, _p(bias), _ACT[act], C.c_float(eps), _p(ws.ws),
                                 C.c_size_t(ws.ws_bytes), _p(ws.counters), ws.n_counters, _p(ws.status), _stream())
    _check(rc, "gemm_bf16_rms")
    ws.launches += 1
    return out.view(*x.shape[:-1], N)


def linear(x, W, bias=None, act=None, residual=None, res_scale=1.0, out_dtype=None):
    lead = x.shape[:-1]
    if W.kind == "bf16":
        y = gemm_bf16(x, W.w, W.out_features, bias=bias, act=act, residual=residual, res_scale=res_scale,
                      out_dtype=out_dtype)
    else:
        from . import native_quant
        y = native_quant.linear(x, W, bias, act, residual, res_scale, out_dtype)
    return y.view(*lead, W.out_features)


def linear_gated(x, W, act="silu", bias=None):
    lead = x.shape[:-1]
    I = W.out_features // 2
    if W.kind == "bf16":
        y = gemm_bf16(x, W.w, I, gated=True, dual_off=I, bias=bias, act=act)
    else:
        from . import native_quant
        y = native_quant.linear_gated(x, W, act, bias)
    return y.view(*lead, I)


def gated_act(gu, act="silu"):
    gu2 = gu.reshape(-1, gu.shape[-1]).contiguous()
    T, I2 = gu2.shape
    out = torch.empty(T, I2 // 2, dtype=torch.bfloat16, device=gu.device)
    _check(lib().xft_gated_act(_p(gu2), _p(out), T, I2 // 2, _ACT[act], _stream()), "gated_act")
    Workspace.get(gu.device).launches += 1
    return out.view(*gu.shape[:-1], I2 // 2)


# ------------------------------------------------------------------------------------------
def qkv_rope_cache(qkv, hq, hkv, d, positions, table, rot_dim, style, kc, vc, ks, vs, slots,
                   q_scale=None, q_norm_w=None, k_norm_w=None, eps=1e-6, rot_offset=0):
    qkv2, ldq = _rows2d(qkv)
    T = qkv2.shape[0]
    q = torch.empty(T, hq, d, dtype=torch.bfloat16, device=qkv.device)
    ws = Workspace.get(qkv.device)
    nb, _, bs, _ = kc.shape
    rc = lib().xft_qkv_rope_cache(_p(qkv2), ldq, T, hq, hkv, d, _p(positions), _p(table),
                                  rot_dim if table is not None else 0, 0 if style == "half" else 1, rot_offset,
                                  0 if table is None else table.shape[0], _p(q_scale), _p(q_norm_w), _p(k_norm_w),
                                  C.c_float(eps), _p(q), _p(kc), _p(vc), _p(ks), _p(vs), int(ks is not None), bs,
                                  C.c_longlong(nb * bs), _p(slots), _p(ws.status), _stream())
    _check(rc, "qkv_rope_cache")
    ws.launches += 1
    return q


def qkv_rope2d_cache(qkv, hq, hkv, d, positions, positions2, table, kc, vc, ks, vs, slots):
    """ChatGLM-1: split, rotate the two halves of every q / k head by their own position stream, append k / v."""
    qkv2, ldq = _rows2d(qkv)
    T = qkv2.shape[0]
    q = torch.empty(T, hq, d, dtype=torch.bfloat16, device=qkv.device)
    ws = Workspace.get(qkv.device)
    nb, _, bs, _ = kc.shape
    fn = lib().xft_qkv_rope2d_cache
    fn.restype = C.c_int
    _check(fn(_p(qkv2), ldq, T, hq, hkv, d, _p(positions), _p(positions2), _p(table), d // 2, table.shape[0], _p(q),
              _p(kc), _p(vc), _p(ks), _p(vs), int(ks is not None), bs, C.c_longlong(nb * bs), _p(slots), _p(ws.status),
              _stream()), "qkv_rope2d_cache")
    ws.launches += 1
    return q


def rope_apply(q, k, positions, table, rot_dim, style="half", rot_offset=0, q_scale=None):
    ws = Workspace.get(q.device)
    st = 0 if style == "half" else 1
    q = q.contiguous().clone() if not q.is_contiguous() else q.clone()
    T, nh, D = q.shape
    _check(lib().xft_rope(_p(q), T, nh, D, _p(positions), _p(table), rot_dim, st, rot_offset, table.shape[0],
                          _p(q_scale), _p(ws.status), _stream()), "rope")
    ws.launches += 1
    if k is not None:
        k = k.contiguous().clone()
        _check(lib().xft_rope(_p(k), T, k.shape[1], k.shape[2], _p(positions), _p(table), rot_dim, st, rot_offset,
                              table.shape[0], C.c_void_p(0), _p(ws.status), _stream()), "rope")
        ws.launches += 1
    return q, k


def latent_cache_write(latent, cache, slots):
    l2, ld = _rows2d(latent)
    ws = Workspace.get(latent.device)
    nb, _, bs, W = cache.shape
    _check(lib().xft_latent_write(_p(l2), ld, _p(cache), W, _p(slots), C.c_longlong(nb * bs), l2.shape[0],
                                  _p(ws.status), _stream()), "latent_write")
    ws.launches += 1


def mla_prep(q, kv, Hl, nope, rope, kvl, positions, table, kv_norm_w, eps, cache, slots):
    """q [T, Hl*(nope+rope)], kv [T, kvl+rope] (row views allowed) -> (q_nope [T,Hl,nope], q_rope [T,Hl,rope]); the
    normalised compressed KV and the rotated shared key part land in the latent cache at `slots`.  q_nope is a
    [T,Hl,nope] VIEW of head-major storage [Hl,T,nope]: the absorb GEMM reads its rows grouped by head, so
    `q_nope.transpose(0, 1)` is contiguous and costs no copy."""
    def rows(x):
        if x.stride(1) != 1 or x.stride(0) % 2 or x.data_ptr() % 4:
            x = x.contiguous()
        return x, x.stride(0)
    q2, ldq = rows(q)
    kv2, ldkv = rows(kv)
    T = q2.shape[0]
    q_nope = torch.empty(Hl, T, nope, dtype=torch.bfloat16, device=q.device)
    q_rope = torch.empty(T, Hl, rope, dtype=torch.bfloat16, device=q.device)
    ws = Workspace.get(q.device)
    nb, _, bs, W = cache.shape
    if W != kvl + rope or cache.dtype != torch.bfloat16:
        raise ValueError("mla_prep: latent cache must be bf16 rows of kv_lora_rank + rope")
    fn = lib().xft_mla_prep
    fn.restype = C.c_int
    _check(fn(_p(q2), ldq, _p(kv2), ldkv, T, Hl, nope, rope, kvl, _p(positions), _p(table), table.shape[0],
              _p(kv_norm_w), C.c_float(eps), _p(q_nope), _p(q_rope), _p(cache), C.c_longlong(nb * bs), _p(slots),
              _p(ws.status), 1, _stream()), "mla_prep")
    ws.launches += 1
    return q_nope.transpose(0, 1), q_rope


def plan_attn_splits(B, hkv, group, D, max_kv, int8=False):
    """Split-KV factor of a decode launch and the tile count it was planned on: fill the resident CTA slots (two
    CTAs per SM for the TMA-ring kernel of bf16 caches, three for the cp.async kernel of int8 caches) while leaving
    every slice at least eight tiles."""
    tma = not int8 and _ENV().attn_tma
    kt = 64 if tma else {64: 64, 128: 32, 256: 16}[D]
    slots = (296 if D <= 128 else 148) if tma else 444
    ntiles = (max_kv + kt - 1) // kt
    ctas = B * max(hkv, 1) * ((group + 15) // 16)
    nsplit = max(1, min(slots // max(ctas, 1), ntiles // 8 if ntiles >= 16 else 1, 32))
    if _ENV().attn_splits > 0:
        nsplit = max(1, min(_ENV().attn_splits, ntiles, 32))
    return nsplit, ntiles


def paged_attention(q, kc, vc, block_table, cu_q, kv_lens, scale, ks=None, vs=None, slopes=None, causal=True,
                    prefix_lm_lens=None, group=None, q_off=0, meta=None):
    assert causal
    T, hq, D = q.shape
    nb, hkv, bs, _ = kc.shape
    dev = q.device
    ws = Workspace.get(dev)
    B = len(kv_lens)
    if meta is not None and getattr(meta, "cu_q_dev", None) is not None:
        cu_dev, kv_dev = meta.cu_q_dev, meta.kv_lens_dev
        decode, max_q, max_kv = meta.is_decode, meta.max_q, meta.max_kv
    else:
        cu_dev = torch.tensor(list(cu_q), dtype=torch.int32, device=dev)
        kv_dev = torch.tensor(list(kv_lens), dtype=torch.int32, device=dev)
        max_q = max(cu_q[i + 1] - cu_q[i] for i in range(B))
        max_kv = max(kv_lens)
        decode = max_q == 1 and all(cu_q[i + 1] - cu_q[i] == 1 for i in range(B))
    pl = None
    if prefix_lm_lens is not None:
        pl = torch.tensor(list(prefix_lm_lens), dtype=torch.int32, device=dev)
    g = group or max(hq // hkv, 1)
    out = torch.empty_like(q)
    nsplit, po, pm = 1, None, None
    if decode:
        nsplit, ntiles = plan_attn_splits(B, hkv, g, D, max_kv, ks is not None)
        if meta is not None and getattr(meta, "meta", None) is not None and "nsplit" in meta.meta:
            nsplit = meta.meta["nsplit"]
        if B * hkv * ((g + 15) // 16) > ws.attn_counters.numel():
            nsplit = 1
        # the partial buffers have a fixed capacity (D >= 64, so the (m, l) buffer of 1/32 the size always suffices)
        nsplit = max(1, min(nsplit, ws.PART_O_FLOATS // max(B * hq * D, 1)))
        if nsplit > 1:
            po, pm = ws.attn_partials(B * hq * nsplit * D, B * hq * nsplit * 2)
    q = q.contiguous()
    if (not decode and D == 128 and bs == 64 and ks is None and slopes is None and pl is None and kc.dtype == torch.bfloat16
            and max_q >= _ENV().attn_tc_min_q):
        # prompt phase on the tcgen05 tensor cores (csrc/kernels/attention_prefill_sm100.cu)
        L = lib()
        L.xft_attn_prefill_tc.restype = C.c_int
        rc = L.xft_attn_prefill_tc(_p(q), _p(out), _p(kc), _p(vc), _p(block_table), block_table.stride(0), _p(cu_dev),
                                   _p(kv_dev), B, T, max_q, hq, hkv, g, q_off, bs, nb, C.c_float(scale), _p(ws.status),
                                   _stream())
        _check(rc, "attn_prefill_tc")
        ws.launches += 1
        return out
    rc = lib().xft_paged_attention(_p(q), _p(out), _p(kc), _p(vc), _p(ks), _p(vs), _p(block_table),
                                   block_table.stride(0), _p(cu_dev), _p(kv_dev), B, max_q, hq, hkv, g, q_off, D, bs,
                                   nb, C.c_float(scale), _p(slopes), _p(pl), (1 if _ENV().attn_tma else 2) if decode else 0, nsplit, _p(po), _p(pm),
                                   _p(ws.attn_counters), _p(ws.status), _stream())
    _check(rc, "paged_attention")
    ws.launches += 1
    return out


def mla_attention(q_nope, q_rope, latent_cache, block_table, cu_q, kv_lens, w_uk, w_uv, scale, absorbed=True,
                  meta=None):
    from . import native_mla
    return native_mla.mla_attention(q_nope, q_rope, latent_cache, block_table, cu_q, kv_lens, w_uk, w_uv, scale,
                                    absorbed, meta)


def route(logits, kind, top_k, bias=None, n_group=1, topk_group=1, routed_scaling=1.0, norm_topk=True,
          scoring="sigmoid"):
    from . import native_moe
    return native_moe.route(logits, kind, top_k, bias, n_group, topk_group, routed_scaling, norm_topk, scoring)


def moe_experts(x, idx, w, experts, act="silu", expert_offset=0, packed=None, expected_pairs=None):
    from . import native_moe
    return native_moe.moe_experts(x, idx, w, experts, act, expert_offset, packed, expected_pairs)


# ------------------------------------------------------------------------------------------
def argmax_rows(logits):
    l2 = logits.reshape(-1, logits.shape[-1])
    assert l2.dtype == torch.float32 and l2.stride(1) == 1
    rows, V = l2.shape
    vals = torch.empty(rows, dtype=torch.float32, device=logits.device)
    idx = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(lib().xft_argmax(_p(l2), l2.stride(0), rows, V, _p(vals), _p(idx), _stream()), "argmax")
    Workspace.get(logits.device).launches += 1
    return vals, idx


def sample_top_k_top_p(logits, top_k, top_p, temperature, uniform):
    from . import native_sample
    return native_sample.sample_top_k_top_p(logits, top_k, top_p, temperature, uniform)
