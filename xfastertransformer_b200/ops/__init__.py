"""Op entry points.  Device switch only: CPU tensors run `ops.reference` (pure PyTorch),
CUDA tensors run the hand-written sm_100a kernels of `ops.native` (libxft_b200_kernels.so).

There is no silent fallback on a GPU: if the kernel library is missing or an op has no
kernel for the requested variant, the call raises.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import reference as R

_native = None


def _nat():
    global _native
    if _native is None:
        import importlib
        _native = importlib.import_module(__name__ + ".native")
    return _native


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


# -- embedding / norms ----------------------------------------------------------------------
def embedding(ids, table, scale=1.0, out_dtype=torch.float32, pos_table=None, positions=None, pos_offset=0):
    if _cuda(table):
        return _nat().embedding(ids, table, scale, out_dtype, pos_table, positions, pos_offset)
    return R.embedding(ids, table, scale, out_dtype, pos_table, positions, pos_offset)


def rmsnorm(x, w, eps, residual=None):
    if _cuda(x):
        return _nat().rmsnorm(x, w, eps, residual)
    return R.rmsnorm(x, w, eps, residual)


def layernorm(x, w, b, eps):
    if _cuda(x):
        return _nat().layernorm(x, w, b, eps)
    return R.layernorm(x, w, b, eps)


# -- GEMMs ---------------------------------------------------------------------------------
def _verbose() -> bool:
    from ..utils.flags import Env
    return Env.get().verbose >= 1


def _timed(kernel: str, x, W, fn):
    """XFT_VERBOSE >= 1: run one GEMM-shaped op between two time stamps (device-synchronised on a GPU) and print the
    reference's per-call line ``xft_verbose,exec,<dev>,api,<kernel>,m<M>n<N>k<K>,<ms>`` (src/utils/verbose.h:24-83).
    The decode graph runner steps aside while this is on, so every call is a real launch."""
    import time
    from ..utils import log
    cuda = _cuda(x)
    if cuda:
        torch.cuda.synchronize(x.device)
    t0 = time.perf_counter()
    y = fn()
    if cuda:
        torch.cuda.synchronize(x.device)
    ms = (time.perf_counter() - t0) * 1e3
    log.verbose_line("gpu" if cuda else "cpu", kernel, x.numel() // x.shape[-1], W.out_features, x.shape[-1], ms)
    return y


def linear(x, W, bias=None, act=None, residual=None, res_scale=1.0, out_dtype=None):
    if _verbose():
        name = "gemm" + ("_bias" if bias is not None else "") + (f"_{act}" if act else "") + \
            ("_residual" if residual is not None else "")
        impl = _nat().linear if _cuda(x) else R.linear
        return _timed(name, x, W, lambda: impl(x, W, bias, act, residual, res_scale, out_dtype))
    if _cuda(x):
        return _nat().linear(x, W, bias, act, residual, res_scale, out_dtype)
    return R.linear(x, W, bias, act, residual, res_scale, out_dtype)


def _linear_rms(x, W, eps, bias, act, gated, out_dtype):
    if _cuda(x):
        return _nat().linear_rms(x, W, eps, bias, act, gated, out_dtype)
    h = R.rmsnorm(x, torch.ones(x.shape[-1], dtype=torch.float32), eps)
    return R.linear_gated(h, W, act, bias) if gated else R.linear(h, W, bias, act, None, 1.0, out_dtype)


def linear_rms(x, W, eps, bias=None, act=None, gated=False, out_dtype=None):
    """RMSNorm(x) @ W^T for a weight whose columns already carry the norm's gain (loader.fold_norm_gain)."""
    if _verbose():
        return _timed("rmsnorm_gemm" + ("_gated" if gated else ""), x, W,
                      lambda: _linear_rms(x, W, eps, bias, act, gated, out_dtype))
    return _linear_rms(x, W, eps, bias, act, gated, out_dtype)


def linear_gated(x, W, act="silu", bias=None):
    if _verbose():
        impl = _nat().linear_gated if _cuda(x) else R.linear_gated
        return _timed(f"gemm_gated_{act}", x, W, lambda: impl(x, W, act, bias))
    if _cuda(x):
        return _nat().linear_gated(x, W, act, bias)
    return R.linear_gated(x, W, act, bias)


def gated_act(gu, act="silu"):
    if _cuda(gu):
        return _nat().gated_act(gu, act)
    return R.gated_act(gu, act)


# -- attention -----------------------------------------------------------------------------
def qkv_rope_cache(qkv, hq, hkv, d, positions, table, rot_dim, style, kc, vc, ks, vs, slots,
                   q_scale=None, q_norm_w=None, k_norm_w=None, eps=1e-6, rot_offset=0):
    """Split packed qkv [T,(hq+2hkv)*d], optional per-head q/k RMSNorm (Qwen3), RoPE on q and k,
    append k/v to the paged cache at `slots` (int8-quantising when scales are given); returns
    q [T,hq,d].  One kernel on the GPU (reference: QKPO + storeKVCache,
    src/layers/attention.h:560-640, src/kernels/attention_kernels.h:45-69)."""
    if _cuda(qkv):
        return _nat().qkv_rope_cache(qkv, hq, hkv, d, positions, table, rot_dim, style, kc, vc, ks, vs, slots,
                                       q_scale, q_norm_w, k_norm_w, eps, rot_offset)
    T = qkv.shape[0]
    q = qkv[:, : hq * d].reshape(T, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].reshape(T, hkv, d)
    v = qkv[:, (hq + hkv) * d:].reshape(T, hkv, d)
    if q_norm_w is not None:
        q = R.rmsnorm(q, q_norm_w, eps)
        k = R.rmsnorm(k, k_norm_w, eps)
    if table is not None and rot_dim > 0:
        q, k = R.rope_apply(q, k, positions, table, rot_dim, style, rot_offset, q_scale)
    elif q_scale is not None:
        q = (q.float() * q_scale[:, None, None]).to(q.dtype)
    R.kv_cache_write(k, v, kc, vc, slots, ks, vs)
    return q.contiguous()


def qkv_rope2d_cache(qkv, hq, hkv, d, positions, positions2, table, kc, vc, ks, vs, slots):
    """ChatGLM-1's two-stream rotary with the cache append: the first half of every q / k head turns by `positions`,
    the second half by `positions2` (block positions), both from one table [max_pos, d/2]; k / v go to the paged cache
    at `slots`; returns q [T,hq,d].  One kernel on the GPU (reference: src/layers/rope_2d.cpp,
    src/models/chatglm.cpp:118-206)."""
    if _cuda(qkv):
        return _nat().qkv_rope2d_cache(qkv, hq, hkv, d, positions, positions2, table, kc, vc, ks, vs, slots)
    T = qkv.shape[0]
    q = qkv[:, : hq * d].reshape(T, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].reshape(T, hkv, d)
    v = qkv[:, (hq + hkv) * d:].reshape(T, hkv, d)
    half = d // 2
    q, k = R.rope_apply(q, k, positions, table, half, "half", 0)
    q, k = R.rope_apply(q, k, positions2, table, half, "half", half)
    R.kv_cache_write(k, v, kc, vc, slots, ks, vs)
    return q.contiguous()


def can_fuse_qkv_rope(W, T, D, kc, ks, q_norm_w, k_norm_w, style) -> bool:
    """True when the QKV product, RoPE and the cache append can run as one kernel (GPU, decode sizes)."""
    return _cuda(kc) and _nat().can_fuse_qkv_rope(W, T, D, kc, ks, q_norm_w, k_norm_w, style)


def qkv_linear_rope_cache(x, W, bias, rms_eps, hq, hkv, positions, table, rot_dim, style, kc, vc, slots, q_scale=None):
    """QKV product with split + RoPE + paged cache append as its epilogue; returns q [T, hq, D].  GPU only: callers
    ask can_fuse_qkv_rope first and otherwise run linear / linear_rms followed by qkv_rope_cache."""
    return _nat().qkv_linear_rope_cache(x, W, bias, rms_eps, hq, hkv, positions, table, rot_dim, style, kc, vc, slots,
                                        q_scale)


def paged_attention(q, kc, vc, block_table, cu_q, kv_lens, scale, ks=None, vs=None, slopes=None,
                    causal=True, prefix_lm_lens=None, group=None, q_off=0, meta=None):
    if _cuda(q):
        return _nat().paged_attention(q, kc, vc, block_table, cu_q, kv_lens, scale, ks, vs, slopes,
                                        causal, prefix_lm_lens, group, q_off, meta)
    return R.paged_attention(q, kc, vc, block_table, cu_q, kv_lens, scale, ks, vs, slopes, causal,
                             prefix_lm_lens, group, q_off)


def mla_attention(q_nope, q_rope, latent_cache, block_table, cu_q, kv_lens, w_uk, w_uv, scale, absorbed=True,
                  meta=None):
    if _cuda(q_nope):
        return _nat().mla_attention(q_nope, q_rope, latent_cache, block_table, cu_q, kv_lens, w_uk, w_uv,
                                      scale, absorbed, meta)
    return R.mla_attention(q_nope, q_rope, latent_cache, block_table, cu_q, kv_lens, w_uk, w_uv, scale, absorbed)


def rope_apply(q, k, positions, table, rot_dim, style="half", rot_offset=0, q_scale=None):
    if _cuda(q):
        return _nat().rope_apply(q, k, positions, table, rot_dim, style, rot_offset, q_scale)
    return R.rope_apply(q, k, positions, table, rot_dim, style, rot_offset, q_scale)


def latent_cache_write(latent, cache, slots):
    """latent [T, kv_lora+rope] -> cache [nb,1,block,kv_lora+rope] at `slots`."""
    if _cuda(latent):
        return _nat().latent_cache_write(latent, cache, slots)
    blk = cache.shape[2]
    cache[(slots // blk).long(), 0, (slots % blk).long()] = latent.to(cache.dtype)


def mla_prep(q, kv, Hl, nope, rope, kvl, positions, table, kv_norm_w, eps, cache, slots):
    """What sits between the MLA projections and the MLA attention: split every query head of q [T, Hl*(nope+rope)]
    into its no-position part and its rotated part (interleaved pairs), RMS-normalise the compressed KV kv[:, :kvl],
    rotate the shared key part kv[:, kvl:], and append (normalised KV ‖ rotated key) to the latent cache at `slots`.
    Returns (q_nope [T,Hl,nope], q_rope [T,Hl,rope]).  One kernel on the GPU."""
    if _cuda(q) and cache.dtype == torch.bfloat16:
        return _nat().mla_prep(q, kv, Hl, nope, rope, kvl, positions, table, kv_norm_w, eps, cache, slots)
    T = q.shape[0]
    q3 = q.reshape(T, Hl, nope + rope)
    ckv = R.rmsnorm(kv[:, :kvl], kv_norm_w, eps)
    q_rope, kr = R.rope_apply(q3[..., nope:], kv[:, kvl:].reshape(T, 1, rope), positions, table, rope, "interleaved", 0)
    latent_cache_write(torch.cat([ckv, kr.reshape(T, rope)], dim=-1), cache, slots)
    return q3[..., :nope].contiguous(), q_rope.contiguous()


# -- MoE -----------------------------------------------------------------------------------
def route(logits, kind, top_k, bias=None, n_group=1, topk_group=1, routed_scaling=1.0, norm_topk=True,
          scoring="sigmoid"):
    if _cuda(logits):
        return _nat().route(logits, kind, top_k, bias, n_group, topk_group, routed_scaling, norm_topk, scoring)
    if kind == "mixtral":
        return R.route_mixtral(logits, top_k)
    if kind == "softmax_topk":
        return R.route_softmax_topk(logits, top_k, norm_topk)
    if kind == "deepseek":
        return R.route_deepseek(logits, bias, top_k, n_group, topk_group, routed_scaling, norm_topk, scoring)
    raise ValueError(kind)


def moe_experts(x, idx, w, experts, act="silu", expert_offset=0, packed=None, expected_pairs=None):
    if _cuda(x):
        return _nat().moe_experts(x, idx, w, experts, act, expert_offset, packed, expected_pairs)
    return R.moe_experts(x, idx, w, experts, act, expert_offset)


# -- sampling ------------------------------------------------------------------------------
def argmax_rows(logits):
    if _cuda(logits):
        return _nat().argmax_rows(logits)
    return R.argmax_rows(logits)


def beam_topk(logits, k):
    """(log-softmax values, token ids) of each row's k best entries, best first."""
    if _cuda(logits):
        from . import native_sample
        return native_sample.beam_topk(logits, k)
    return R.beam_topk(logits, k)


def sample_top_k_top_p(logits, top_k, top_p, temperature, uniform):
    if _cuda(logits):
        return _nat().sample_top_k_top_p(logits, top_k, top_p, temperature, uniform)
    return R.sample_top_k_top_p(logits, top_k, top_p, temperature, uniform)
