"""Pure-PyTorch implementation of every op of the engine.

Two jobs: (1) it *is* the CPU execution path (tiny-Llama config under gloo), and (2) it is
the fp32 oracle each sm_100a kernel is tested against.  It is never used on a GPU hot path.
Everything accumulates in fp32 and rounds once at the end, which is what the CUDA kernels do
(TMEM accumulators are fp32).

Op semantics mirror the reference kernels listed per function.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

# NF4 code book (QLoRA); reference: src/common/normal_float4x2.h
NF4_CODE = torch.tensor([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
    0.7229568362236023, 1.0], dtype=torch.float32)


# ----------------------------------------------------------------------------------------
# embedding / norms
# ----------------------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0,
              out_dtype: torch.dtype = torch.float32,
              pos_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None,
              pos_offset: int = 0) -> torch.Tensor:
    """Row gather (+sqrt(hidden) scale for Gemma, + learned positions for OPT).
    Reference: src/kernels/token_embedding_kernels.cpp:24-54, token_embedding_gemma.h:46-72,
    opt_embedding.h:52-81."""
    x = table[ids.long()].float()
    if scale != 1.0:
        x = x * scale
    if pos_table is not None:
        x = x + pos_table[positions.long() + pos_offset].float()
    return x.to(out_dtype)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None):
    """y = x * rsqrt(mean(x^2)+eps) * w  (src/kernels/rmsnorm_kernels.cpp:27-84).
    With `residual`, first h = x + residual and (y, h) is returned."""
    xf = x.float()
    if residual is not None:
        xf = xf + residual.float()
        h = xf.to(x.dtype)
        xf = h.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    y = (xf * torch.rsqrt(var + eps) * w.float()).to(x.dtype)
    return (y, h) if residual is not None else y


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float):
    """(x-mean)*rstd*gamma+beta  (src/kernels/layernorm_kernels.cpp:27-80)."""
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = (xf - mu).pow(2).mean(-1, keepdim=True)
    y = (xf - mu) * torch.rsqrt(var + eps) * w.float()
    if b is not None:
        y = y + b.float()
    return y.to(x.dtype)


# ----------------------------------------------------------------------------------------
# quantisation helpers (load time) and dequantisation (oracle)
# ----------------------------------------------------------------------------------------
def quantize_int8_per_channel(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """w[out,in] -> (q int8 [out,in], scale[out], zero[out]) with w ~= q*scale+zero
    (asymmetric, per output channel; reference matmul_helper.h:205-262)."""
    wf = w.float()
    mx = wf.amax(1)
    mn = wf.amin(1)
    scale = ((mx - mn) / 255.0).clamp_min(1e-10)
    zero = (mx + mn) / 2.0 + 0.5 * scale
    q = torch.round((wf - zero[:, None]) / scale[:, None]).clamp_(-128, 127).to(torch.int8)
    return q, scale, zero


def quantize_uint4_per_channel(w: torch.Tensor):
    """w[out,in] -> (packed uint8 [out, in/2], scale[out], zero[out]); low nibble = even index
    (src/common/uint4x2.h:45-49), w ~= q*scale + zero, q in [0,15]."""
    wf = w.float()
    mx = wf.amax(1)
    mn = wf.amin(1)
    scale = ((mx - mn) / 15.0).clamp_min(1e-10)
    zero = mn
    q = torch.round((wf - zero[:, None]) / scale[:, None]).clamp_(0, 15).to(torch.uint8)
    return pack_nibbles(q), scale, zero


def quantize_nf4_per_channel(w: torch.Tensor):
    """w[out,in] -> (packed codes, scale[out]=absmax, zero[out]=0); w ~= NF4[q]*scale."""
    wf = w.float()
    scale = wf.abs().amax(1).clamp_min(1e-10)
    xn = wf / scale[:, None]
    code = NF4_CODE.to(wf.device)
    q = (xn[..., None] - code).abs().argmin(-1).to(torch.uint8)
    return pack_nibbles(q), scale, torch.zeros_like(scale)


def pack_nibbles(q: torch.Tensor) -> torch.Tensor:
    assert q.shape[-1] % 2 == 0
    return (q[..., 0::2] | (q[..., 1::2] << 4)).contiguous()


def unpack_nibbles(p: torch.Tensor) -> torch.Tensor:
    lo = p & 0xF
    hi = (p >> 4) & 0xF
    return torch.stack([lo, hi], dim=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)


def quantize_fp8_block(w: torch.Tensor, block: int = 128):
    """w[out,in] -> (e4m3 [out,in], scale_inv fp32 [ceil(out/b), ceil(in/b)]) with
    w ~= fp8 * scale_inv[block]  (DeepSeek-V3 weight_scale_inv convention)."""
    o, i = w.shape
    ob, ib = (o + block - 1) // block, (i + block - 1) // block
    wp = torch.zeros(ob * block, ib * block, dtype=torch.float32, device=w.device)
    wp[:o, :i] = w.float()
    blk = wp.view(ob, block, ib, block)
    amax = blk.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale_inv = amax / 448.0
    q = (blk / scale_inv[:, None, :, None]).view(ob * block, ib * block)[:o, :i]
    return q.to(torch.float8_e4m3fn), scale_inv


def dequant_weight(W) -> torch.Tensor:
    """LinearWeight -> fp32 [out,in]."""
    k = W.kind
    if k in ("bf16", "fp16", "fp32"):
        return W.w.float()
    if k in ("int8", "w8a8"):
        return W.w.float() * W.scale[:, None] + W.zero[:, None]
    if k == "int4":
        return unpack_nibbles(W.w).float() * W.scale[:, None] + W.zero[:, None]
    if k == "nf4":
        return NF4_CODE.to(W.w.device)[unpack_nibbles(W.w).long()] * W.scale[:, None] + W.zero[:, None]
    if k == "fp8":
        o, i = W.w.shape
        b = W.block
        s = W.scale.repeat_interleave(b, 0)[:o].repeat_interleave(b, 1)[:, :i]
        return W.w.float() * s
    raise ValueError(k)


def quantize_act_w8a8(x: torch.Tensor):
    """Per-row dynamic asymmetric int8 (matmul_helper.h:2813-2855): zero=(min+max)/2,
    scale=max|x-zero|/127 -> (q int8, scale[rows], zero[rows])."""
    xf = x.float()
    mx = xf.amax(-1)
    mn = xf.amin(-1)
    zero = (mx + mn) / 2
    scale = ((xf - zero[..., None]).abs().amax(-1) / 127.0).clamp_min(1e-10)
    q = torch.round((xf - zero[..., None]) / scale[..., None]).clamp_(-127, 127).to(torch.int8)
    return q, scale, zero


# ----------------------------------------------------------------------------------------
# GEMM with fused epilogues
# ----------------------------------------------------------------------------------------
def _act(y: torch.Tensor, act: Optional[str]) -> torch.Tensor:
    if act is None or act == "none":
        return y
    if act == "relu":
        return F.relu(y)
    if act == "silu":
        return F.silu(y)
    if act in ("gelu", "gelu_tanh", "gelu_new", "gelu_pytorch_tanh"):
        return F.gelu(y, approximate="tanh")
    if act == "gelu_erf":
        return F.gelu(y)
    raise ValueError(act)


def linear(x: torch.Tensor, W, bias: Optional[torch.Tensor] = None, act: Optional[str] = None,
           residual: Optional[torch.Tensor] = None, res_scale: float = 1.0,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = act(x @ W^T + bias) + res_scale*residual.  Covers MMHelper::compute,
    compute_bias, compute_biasadd_relu, compute_silu, compute_gelu, compute_residential,
    compute_resext (src/utils/matmul_helper.h:565-1705).  `W` is a LinearWeight ([out,in])."""
    out_dtype = out_dtype or x.dtype
    if W.kind == "w8a8":
        q, sa, za = quantize_act_w8a8(x)
        xf = q.float() * sa[..., None] + za[..., None]
    else:
        xf = x.float()
    y = xf @ dequant_weight(W).t()
    if bias is not None:
        y = y + bias.float()
    y = _act(y, act)
    if residual is not None:
        y = y + res_scale * residual.float()
    return y.to(out_dtype)


def gated_act(gu: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """cat(gate, up)[..., 2I] -> act(gate) * up  (siluSum/geluSum, decoder_util.h:495-607)."""
    i = gu.shape[-1] // 2
    g, u = gu[..., :i].float(), gu[..., i:].float()
    return (_act(g, act) * u).to(gu.dtype)


def linear_gated(x: torch.Tensor, W, act: str = "silu", bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T) with W = cat(gate, up) on the out dim; the intermediate is
    kept in fp32 (the fused kernel applies the activation on the TMEM accumulators)."""
    xf = x.float()
    if W.kind == "w8a8":
        q, sa, za = quantize_act_w8a8(x)
        xf = q.float() * sa[..., None] + za[..., None]
    y = xf @ dequant_weight(W).t()
    if bias is not None:
        y = y + bias.float()
    i = y.shape[-1] // 2
    return (_act(y[..., :i], act) * y[..., i:]).to(x.dtype)


# ----------------------------------------------------------------------------------------
# RoPE tables and application
# ----------------------------------------------------------------------------------------
def _yarn_find_dim(num_rot: float, dim: int, base: float, max_pos: int) -> float:
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def yarn_mscale(scale: float = 1.0, mscale: float = 1.0) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def rope_inv_freq(rot_dim: int, theta: float, scaling_type: str = "", factor: float = 1.0,
                  original_max_pos: int = 2048, beta_fast: float = 32, beta_slow: float = 1) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    if scaling_type == "linear" and factor != 1.0:
        inv = inv / factor
    elif scaling_type == "yarn" and factor != 1.0:
        low = max(math.floor(_yarn_find_dim(beta_fast, rot_dim, theta, original_max_pos)), 0)
        high = min(math.ceil(_yarn_find_dim(beta_slow, rot_dim, theta, original_max_pos)), rot_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(rot_dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        mask = 1.0 - ramp                      # 1 -> extrapolate (keep), 0 -> interpolate
        inv = inv / factor * (1 - mask) + inv * mask
    return inv.float()


def rope_table(max_pos: int, rot_dim: int, theta: float = 10000.0, scaling_type: str = "",
               factor: float = 1.0, original_max_pos: int = 2048, beta_fast: float = 32,
               beta_slow: float = 1, mscale: float = 1.0, mscale_all_dim: float = 0.0,
               table_scale: Optional[float] = None) -> torch.Tensor:
    """-> fp32 [max_pos, rot_dim] = cat(cos, sin) of pos*inv_freq (rot_dim/2 each).

    YaRN multiplies the table by yarn_mscale(factor, mscale)/yarn_mscale(factor, mscale_all_dim)
    (rotary_embedding_deepseekv2.cpp:62-85; yarn_scaled_rotary_embedding.cpp:26-84 uses
    0.1*ln(factor)+1)."""
    inv = rope_inv_freq(rot_dim, theta, scaling_type, factor, original_max_pos, beta_fast, beta_slow)
    t = torch.arange(max_pos, dtype=torch.float32)
    fr = torch.outer(t, inv)
    s = 1.0
    if table_scale is not None:
        s = table_scale
    elif scaling_type == "yarn" and factor > 1.0:
        s = yarn_mscale(factor, mscale) / (yarn_mscale(factor, mscale_all_dim) if mscale_all_dim else 1.0)
    return torch.cat([fr.cos() * s, fr.sin() * s], dim=-1)


def telechat_ntk_alpha(true_seq_len: int) -> float:
    """TeleChat's NTK factor for a context of `true_seq_len` tokens: 2^ceil(log2(len / 4096) + 1) - 1, at least 1; the
    rotary base becomes theta * alpha^(dim / (dim - 2)) (src/layers/rotary_embedding_telechat.cpp:29-35)."""
    ctx = math.log(true_seq_len / 4096.0) / math.log(2.0) + 1
    return max(2.0 ** math.ceil(ctx) - 1, 1.0)


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, style: str) -> torch.Tensor:
    """x [T,H,rot] fp32; cos/sin [T,rot/2]."""
    c, s = cos[:, None, :], sin[:, None, :]
    if style == "half":            # pairs (i, i+rot/2)  (llama / neox)
        h = x.shape[-1] // 2
        x1, x2 = x[..., :h], x[..., h:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    if style == "interleaved":     # pairs (2i, 2i+1)  (chatglm2 / gpt-j / deepseek storage)
        x1, x2 = x[..., 0::2], x[..., 1::2]
        o = torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
        return o.flatten(-2)
    raise ValueError(style)


def rope_apply(q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor, table: torch.Tensor,
               rot_dim: int, style: str = "half", rot_offset: int = 0,
               q_scale: Optional[torch.Tensor] = None):
    """Rotate dims [rot_offset, rot_offset+rot_dim) of every head of q [T,Hq,D] and k [T,Hk,D].
    `q_scale` [T] is Qwen's log-n query scaling.  Reference:
    src/kernels/rotary_embedding_kernels.cpp:57-199 (llama), :201-361 (chatglm2), :363-528 (qwen),
    :676-797 (deepseek-v2)."""
    cs = table[positions.long()]
    half = rot_dim // 2
    cos, sin = cs[:, :half], cs[:, half:]

    def one(x):
        xf = x.float()
        rot = _rotate(xf[..., rot_offset:rot_offset + rot_dim], cos, sin, style)
        out = torch.cat([xf[..., :rot_offset], rot, xf[..., rot_offset + rot_dim:]], dim=-1)
        return out

    qo = one(q)
    if q_scale is not None:
        qo = qo * q_scale[:, None, None].float()
    qo = qo.to(q.dtype)
    ko = one(k).to(k.dtype) if k is not None else None
    return qo, ko


def alibi_slopes(n_heads: int) -> torch.Tensor:
    """ALiBi slopes (src/layers/alibi_embedding.cpp): powers of 2^(-8/n) with the usual
    interleave for non-power-of-two head counts."""
    def pow2(n):
        start = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]
    if math.log2(n_heads).is_integer():
        s = pow2(n_heads)
    else:
        c = 2 ** math.floor(math.log2(n_heads))
        s = pow2(c) + pow2(2 * c)[0::2][: n_heads - c]
    return torch.tensor(s, dtype=torch.float32)


# ----------------------------------------------------------------------------------------
# paged KV cache write + attention
# ----------------------------------------------------------------------------------------
def quantize_kv_int8(x: torch.Tensor):
    """[T,H,D] -> int8 + fp32 scale [T,H]; symmetric absmax/127, round-nearest
    (src/utils/quantize_util.h:22-51)."""
    xf = x.float()
    scale = xf.abs().amax(-1) / 127.0
    q = torch.round(xf / scale.clamp_min(1e-20)[..., None]).clamp_(-127, 127).to(torch.int8)
    return q, scale


def kv_cache_write(k: torch.Tensor, v: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor,
                   slots: torch.Tensor, ks: Optional[torch.Tensor] = None, vs: Optional[torch.Tensor] = None):
    """Write new keys/values of T tokens into a paged cache.

    kc/vc: [num_blocks, Hkv, block, D] (int8 if `ks`/`vs` [num_blocks, Hkv, block] given);
    slots[T] = block_id*block + offset.  (storeKVCache, attention_kernels.h:45-69)."""
    blk = kc.shape[2]
    b = (slots // blk).long()
    o = (slots % blk).long()
    if ks is not None:
        qk, sk = quantize_kv_int8(k)
        qv, sv = quantize_kv_int8(v)
        kc[b, :, o, :] = qk
        vc[b, :, o, :] = qv
        ks[b, :, o] = sk
        vs[b, :, o] = sv
    else:
        kc[b, :, o, :] = k.to(kc.dtype)
        vc[b, :, o, :] = v.to(vc.dtype)


def _gather_kv(cache: torch.Tensor, scale: Optional[torch.Tensor], blocks: torch.Tensor, n: int) -> torch.Tensor:
    """-> fp32 [Hkv, n, D] of one sequence."""
    blk = cache.shape[2]
    nb = (n + blk - 1) // blk
    x = cache[blocks[:nb].long()]                      # [nb,H,blk,D]
    x = x.permute(1, 0, 2, 3).reshape(cache.shape[1], nb * blk, cache.shape[3])[:, :n].float()
    if scale is not None:
        s = scale[blocks[:nb].long()].permute(1, 0, 2).reshape(cache.shape[1], nb * blk)[:, :n]
        x = x * s[..., None]
    return x


def paged_attention(q: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, block_table: torch.Tensor,
                    cu_q: Sequence[int], kv_lens: Sequence[int], scale: float,
                    ks: Optional[torch.Tensor] = None, vs: Optional[torch.Tensor] = None,
                    slopes: Optional[torch.Tensor] = None, causal: bool = True,
                    prefix_lm_lens: Optional[Sequence[int]] = None, group: Optional[int] = None,
                    q_off: int = 0) -> torch.Tensor:
    """Ragged-batch attention over a paged cache that already holds the new tokens.

    q [T,Hq,D]; sequence b owns query rows cu_q[b]:cu_q[b+1]; its keys are cache positions
    0..kv_lens[b]-1; query row i sits at position kv_len - q_len + i and sees keys <= it.
    One definition covers prefill (q_len = kv_len), decode (q_len = 1) and chunked/prefix
    prefill, i.e. selfAttention / crossAttnByHead / crossAttnShardedHead / flash / paged
    crossAttention of the reference (src/kernels/attention_kernels.h, attention_kernels.cpp).
    `prefix_lm_lens[b]`: keys below it are visible to every query (ChatGLM-1 prefix mask).
    Local query head i reads local kv head (i + q_off) // group; the defaults (group = Hq/Hkv,
    q_off = 0) are plain GQA, other values appear with uneven TP head ranges
    (split_util.h:61-99: the kv range is the covering range of the q range).
    """
    T, Hq, D = q.shape
    Hkv = kc.shape[1]
    g = group or max(Hq // Hkv, 1)
    hmap = ((torch.arange(Hq, device=q.device) + q_off) // g).clamp_max(Hkv - 1)
    out = torch.empty(T, Hq, vc.shape[3], dtype=torch.float32, device=q.device)
    for b in range(len(kv_lens)):
        q0, q1 = int(cu_q[b]), int(cu_q[b + 1])
        n = int(kv_lens[b])
        ql = q1 - q0
        if ql == 0:
            continue
        K = _gather_kv(kc, ks, block_table[b], n)       # [Hkv,n,D]
        V = _gather_kv(vc, vs, block_table[b], n)
        Q = q[q0:q1].float().permute(1, 0, 2)           # [Hq,ql,D]
        Kx = K[hmap]
        Vx = V[hmap]
        s = torch.matmul(Q, Kx.transpose(1, 2)) * scale  # [Hq,ql,n]
        qpos = torch.arange(n - ql, n, device=q.device)
        kpos = torch.arange(n, device=q.device)
        if slopes is not None:
            # bias = slope * (k - q): zero on the diagonal, negative to the left
            s = s + slopes.to(q.device)[:, None, None] * (kpos[None, None, :] - qpos[None, :, None]).float()
        if causal:
            mask = kpos[None, :] > qpos[:, None]
            if prefix_lm_lens is not None:
                mask = mask & (kpos[None, :] >= int(prefix_lm_lens[b]))
            s = s.masked_fill(mask[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[q0:q1] = torch.matmul(p, Vx).permute(1, 0, 2)
    return out.to(q.dtype)


# ----------------------------------------------------------------------------------------
# MLA (DeepSeek) — latent cache [num_blocks, 1, block, kv_lora + rope]
# ----------------------------------------------------------------------------------------
def mla_attention(q_nope: torch.Tensor, q_rope: torch.Tensor, latent_cache: torch.Tensor,
                  block_table: torch.Tensor, cu_q, kv_lens, w_uk: torch.Tensor, w_uv: torch.Tensor,
                  scale: float, absorbed: bool = True) -> torch.Tensor:
    """DeepSeek MLA over the latent cache (c_kv[kv_lora] ‖ k_rope[rope] per token).

    q_nope [T,H,nope], q_rope [T,H,rope]; w_uk [H,nope,kv_lora], w_uv [H,v,kv_lora].
    absorbed:   S = (q_nope·W_uk)·c_kvᵀ + q_rope·k_ropeᵀ ; O = (softmax(S)·c_kv)·W_uvᵀ
    otherwise:  K_nope = c_kv·W_ukᵀ, V = c_kv·W_uvᵀ are materialised (prefill form).
    Reference: crossAttnByHead_DS (attention_kernels.h:1132-1281), selfAttention_MLA (:569-766).
    """
    T, H, nope = q_nope.shape
    L = w_uk.shape[2]
    vd = w_uv.shape[1]
    out = torch.empty(T, H, vd, dtype=torch.float32, device=q_nope.device)
    for b in range(len(kv_lens)):
        q0, q1 = int(cu_q[b]), int(cu_q[b + 1])
        n, ql = int(kv_lens[b]), q1 - q0
        if ql == 0:
            continue
        lat = _gather_kv(latent_cache, None, block_table[b], n)[0]   # [n, L+rope]
        ckv, kr = lat[:, :L], lat[:, L:]
        qn = q_nope[q0:q1].float().permute(1, 0, 2)                  # [H,ql,nope]
        qr = q_rope[q0:q1].float().permute(1, 0, 2)                  # [H,ql,rope]
        if absorbed:
            qa = torch.matmul(qn, w_uk.float())                      # [H,ql,L]
            s = torch.matmul(qa, ckv.t()) + torch.matmul(qr, kr.t())
        else:
            kn = torch.einsum("nl,hdl->hnd", ckv, w_uk.float())      # [H,n,nope]
            s = torch.matmul(qn, kn.transpose(1, 2)) + torch.matmul(qr, kr.t())
        s = s * scale
        qpos = torch.arange(n - ql, n, device=s.device)
        kpos = torch.arange(n, device=s.device)
        s = s.masked_fill((kpos[None, :] > qpos[:, None])[None], float("-inf"))
        p = torch.softmax(s, -1)
        if absorbed:
            o = torch.matmul(torch.matmul(p, ckv), w_uv.float().transpose(1, 2))   # [H,ql,v]
        else:
            v = torch.einsum("nl,hdl->hnd", ckv, w_uv.float())
            o = torch.matmul(p, v)
        out[q0:q1] = o.permute(1, 0, 2)
    return out.to(q_nope.dtype)


# ----------------------------------------------------------------------------------------
# MoE routing
# ----------------------------------------------------------------------------------------
def route_mixtral(logits: torch.Tensor, top_k: int = 2):
    """top-k on raw logits, then softmax over the selected logits only
    (src/layers/mlp_mixtral.h:223-281)."""
    v, idx = torch.topk(logits.float(), top_k, dim=-1)
    return idx, torch.softmax(v, dim=-1)


def route_softmax_topk(logits: torch.Tensor, top_k: int, renorm: bool = True):
    """full softmax -> top-k -> renormalise (src/layers/moe_qwen3.h:283-315)."""
    p = torch.softmax(logits.float(), -1)
    v, idx = torch.topk(p, top_k, dim=-1)
    if renorm:
        v = v / v.sum(-1, keepdim=True)
    return idx, v


def route_deepseek(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, n_group: int,
                   topk_group: int, routed_scaling: float, norm_topk: bool = True,
                   scoring: str = "sigmoid"):
    """DeepSeek-V3 ``noaux_tc`` (src/layers/moe_deepseek.h:226-283,402-536): sigmoid scores;
    selection uses score+bias: group score = sum of its top-2, keep `topk_group` groups, take
    top-k experts inside them; weights are the *unbiased* scores, normalised
    (÷(sum+1e-20)) and multiplied by `routed_scaling`."""
    x = logits.float()
    scores = torch.sigmoid(x) if scoring == "sigmoid" else torch.softmax(x, -1)
    T, E = scores.shape
    sel = scores + (bias.float() if bias is not None else 0.0)
    if n_group > 1:
        grp = sel.view(T, n_group, E // n_group)
        gscore = grp.topk(2, dim=-1)[0].sum(-1)
        gidx = gscore.topk(topk_group, dim=-1)[1]
        gmask = torch.zeros(T, n_group, device=x.device, dtype=torch.bool).scatter_(1, gidx, True)
        sel = sel.masked_fill(~gmask[:, :, None].expand(T, n_group, E // n_group).reshape(T, E), float("-inf"))
    idx = sel.topk(top_k, dim=-1)[1]
    w = scores.gather(1, idx)
    if norm_topk:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return idx, w * routed_scaling


def moe_experts(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, experts, act: str = "silu",
                expert_offset: int = 0) -> torch.Tensor:
    """sum_k w[t,k] * down_e(act(gate_e x) * up_e x) over the experts in `experts`
    (list of (gate_up LinearWeight, down LinearWeight), global id = expert_offset+i).
    Experts with no token are skipped (gather -> MLP -> weighted scatter-add:
    moe_deepseek.h:380-398, mlp_mixtral.h:204-219).  Returns fp32 [T, hidden]."""
    T = x.shape[0]
    out = None
    for i, (gu, dn) in enumerate(experts):
        e = expert_offset + i
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = linear_gated(x[tok], gu, act)
        y = linear(h, dn, out_dtype=torch.float32)
        if out is None:
            out = torch.zeros(T, y.shape[-1], dtype=torch.float32, device=x.device)
        out.index_add_(0, tok, y * w[tok, slot].float()[:, None])
    if out is None:
        out = torch.zeros(T, experts[0][1].out_features, dtype=torch.float32, device=x.device)
    return out


# ----------------------------------------------------------------------------------------
# samplers / logits processors
# ----------------------------------------------------------------------------------------
def argmax_rows(logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(max value, first index of the max) per row — first max wins ties (sampling.cpp:22-131)."""
    v, i = torch.max(logits.float(), dim=-1)
    return v, i


def repetition_penalty(logits: torch.Tensor, token_lists, penalty: float, vocab_offset: int = 0):
    """l<0 ? l*p : l/p on unique prompt+generated ids that fall into this rank's vocab slice
    (src/searchers/search_utils.cpp:104-172)."""
    if penalty == 1.0:
        return logits
    n = logits.shape[-1]
    for r, toks in enumerate(token_lists):
        ids = torch.unique(torch.as_tensor(list(toks), dtype=torch.long, device=logits.device)) - vocab_offset
        ids = ids[(ids >= 0) & (ids < n)]
        if ids.numel() == 0:
            continue
        l = logits[r, ids]
        logits[r, ids] = torch.where(l < 0, l * penalty, l / penalty)
    return logits


def sample_top_k_top_p(logits: torch.Tensor, top_k: int, top_p: float, temperature: float,
                       uniform: torch.Tensor) -> torch.Tensor:
    """top-k -> /T -> top-p prefix (never fewer than 2 kept) -> softmax -> inverse CDF with one
    uniform draw per row (src/searchers/sample_search.cpp:118-268).  top_k is clamped to [1, min(V, 1024)], the
    candidate capacity of the device kernel, so both implementations keep the same set."""
    k = max(1, min(top_k, logits.shape[-1], 1024))
    v, idx = torch.topk(logits.float(), k, dim=-1)
    v = v / max(temperature, 1e-6)
    p = torch.softmax(v, -1)
    if top_p < 1.0 and k > 1:
        c = torch.cumsum(p, -1)
        keep = (c - p) < top_p
        keep[:, : min(2, k)] = True
        v = v.masked_fill(~keep, float("-inf"))
        p = torch.softmax(v, -1)
    c = torch.cumsum(p, -1)
    u = uniform.to(c.device).float().clamp(0, 1 - 1e-7)[:, None]
    choice = (c <= u).sum(-1).clamp_max(k - 1)
    return idx.gather(1, choice[:, None]).squeeze(1)


def log_softmax(logits: torch.Tensor) -> torch.Tensor:
    return torch.log_softmax(logits.float(), dim=-1)


def beam_topk(logits: torch.Tensor, k: int):
    """Per row: the k best log-softmax values and their token ids, best first, lower id first among equals (the part
    of a beam-search step that touches the whole vocabulary, src/searchers/beam_search.cpp:356-540)."""
    lp = torch.log_softmax(logits.float().reshape(-1, logits.shape[-1]), dim=-1)
    order = torch.sort(lp, dim=-1, descending=True, stable=True).indices[:, :k]
    return lp.gather(1, order), order
