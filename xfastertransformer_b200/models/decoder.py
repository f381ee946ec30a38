"""The generic, config-driven decoder.

One class runs every family of the reference (``src/models/common_decoder.h:152-1013`` plus the
16 per-family subclasses, ``src/layers/decoder_block.h``, ``src/layers/attention.h``,
``attn_deepseek.h``, ``mlp_llama.h``, ``mlp_standard.h``, ``mlp_chatglm2.h``, ``mlp_mixtral.h``,
``moe_qwen3.h``, ``moe_deepseek.h``, ``dist_linear.h``).  The family differences are the fields
of `FamilySpec`; weight and KV-cache dtypes are data as well (`LinearWeight.kind`,
`PagedKVCache.dtype`) instead of template parameters.

Tensor parallelism follows the reference algebra: column-sliced QKV / gate‖up, row-sliced
o_proj / down, residual (+bias) folded in on TP rank 0 only, then a sum over ranks
(``attention.h:446-478``, ``mlp_llama.h:243-244``, ``decoder_block.h:122-134``).  On GPUs the
row-parallel GEMM and that sum are one fused kernel (`parallel.fused_comm`).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..ops import reference as R
from ..parallel import partition as P
from ..parallel.dist import DistContext
from ..runtime.kv_cache import PagedKVCache
from ..runtime.loader import LinearWeight, WeightSource, cat_linear, make_linear
from ..utils.flags import Env
from ..utils import debugger
from ..utils.progress import ProgressBar
from ..utils.trace import TimeLine
from .registry import FamilySpec, family_for

WEIGHT_KIND = {"bf16": "bf16", "fp16": "fp16", "int8": "int8", "w8a8": "w8a8", "int4": "int4", "nf4": "nf4",
               "fp8_e4m3": "fp8", "fp32": "fp32"}


@dataclass
class Batch:
    """One forward's worth of ragged sequences (all-prefill or all-decode, like the reference:
    ``common_decoder.h:592``).  Tensors live on the model device; lists stay on the host."""
    ids: torch.Tensor                 # [T] int32
    positions: torch.Tensor           # [T] int32
    slots: torch.Tensor               # [T] int32 (paged cache slot of each new token)
    cu_q: List[int]                   # [B+1]
    kv_lens: List[int]                # [B] keys visible after this step's append
    block_table: torch.Tensor         # [B, W] int32
    logit_rows: Optional[torch.Tensor] = None   # rows of the flattened batch that need logits
    cu_q_dev: Optional[torch.Tensor] = None
    kv_lens_dev: Optional[torch.Tensor] = None
    is_decode: bool = False
    positions2: Optional[torch.Tensor] = None   # ChatGLM-1 block positions
    prefix_lm_lens: Optional[List[int]] = None
    max_q: int = 0
    max_kv: int = 0
    meta: dict = field(default_factory=dict)    # kernel-side scheduling scratch (native)

    @property
    def num_seqs(self) -> int:
        return len(self.kv_lens)


class Layer:
    """Plain attribute bag for one layer's weights."""
    pass


class Decoder:
    def __init__(self, cfg: ModelConfig, ctx: DistContext, path: str, weight_dtype: str,
                 act_dtype: Optional[torch.dtype] = None, embed_from: Optional["Decoder"] = None):
        self.cfg = cfg
        self.ctx = ctx
        self.spec: FamilySpec = family_for(cfg)
        self.device = ctx.device
        self.kind = WEIGHT_KIND[weight_dtype]
        if self.device.type == "cuda" and self.kind in ("fp16", "fp32"):
            # activations on B200 are bf16 end to end; 16-bit float weights are kept in bf16 so
            # both tcgen05 operands share a type
            self.kind = "bf16"
        if self.kind == "fp8" and cfg.weight_data_type != "fp8_e4m3" and not Env.get().fake_model:
            pass  # a bf16 DeepSeek checkpoint quantised to fp8 at load
        self.act_dtype = act_dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.tp, self.tpr = ctx.tp_size, ctx.tp_rank
        self.src = WeightSource(path, cfg.weight_data_type, self.device)
        # DeepSeek checkpoints keep embedding, lm_head, norms and the router in bf16 whatever the projection type
        # (deepseek_moe_convert.py:117-180)
        self.aux_dtype = "bf16" if cfg.model_type == "deepseek_moe" else None
        self.l0, self.l1 = P.pp_layer_range(cfg.num_layer, ctx.pp_size, ctx.pp_rank)
        self.first_stage = ctx.pp_rank == 0
        self.last_stage = ctx.pp_rank == ctx.pp_size - 1
        c = cfg
        (self.qs, self.qe), (self.ks, self.ke) = P.head_range(c.head_num, c.kv_head_num, self.tp, self.tpr)
        self.hq, self.hkv = self.qe - self.qs, self.ke - self.ks
        self.group = max(c.head_num // max(c.kv_head_num, 1), 1)
        self.q_off = self.qs - self.ks * self.group
        self.D = c.size_per_head
        self.eps = c.layernorm_eps
        self.scale = c.attn_scale
        self._build_rope()
        self.slopes = None
        if self.spec.alibi:
            self.slopes = R.alibi_slopes(c.head_num)[self.qs:self.qe].to(self.device)
        # weights
        with TimeLine("Decoder.loadWeights"):
            self._load_embedding(embed_from)
            self.layers: List[Layer] = [self._load_layer(i)
                                        for i in ProgressBar.wrap(range(self.l0, self.l1), "Loading layers")]
            self._load_head(embed_from)
            self._fold_norms()
        self.has_moe = any(L.mlp_kind not in ("llama", "gpt") for L in self.layers)
        self.pairs_run = 0          # forward_pair calls
        self._overlap = False       # True while forward_pair interleaves two batches (all-reduces are started, not awaited)
        self._work = None

    # ------------------------------------------------------------------------------------
    # rotary tables
    # ------------------------------------------------------------------------------------
    def _build_rope(self) -> None:
        c, s = self.cfg, self.spec
        self.rope_table = None
        self.rot_dim = 0
        self.rope_style = s.rope
        if s.rope == "none":
            return
        max_pos = max(c.max_pos_seq_len, c.model_max_length, 2048)
        r = c.rope
        if s.attention == "mla":
            self.rot_dim = c.qk_rope_head_dim
            max_pos = min(max_pos, 163840)
            tab = R.rope_table(max_pos, self.rot_dim, r.theta, r.scaling_type, r.scaling_factor, r.original_max_pos,
                               r.beta_fast, r.beta_slow, r.mscale, r.mscale_all_dim)
        elif s.rope == "2d":
            self.rot_dim = self.D // 2          # each half of the head rotates with its own position stream
            self.rope_style = "half"
            tab = R.rope_table(max_pos, self.rot_dim, r.theta)
        else:
            self.rot_dim = int(self.D * s.rot_frac)
            theta = r.theta
            if c.model_type in ("chatglm2", "chatglm3", "chatglm4") and r.scaling_factor != 1.0 and not r.scaling_type:
                theta = theta * r.scaling_factor      # rope_ratio of long-context GLM checkpoints
                tab = R.rope_table(max_pos, self.rot_dim, theta)
            elif c.model_type == "yarn_llama" or r.scaling_type == "yarn":
                # reference: LlamaYaRNScaledRotaryEmbedding (yarn_scaled_rotary_embedding.cpp:26-84):
                # table scale 0.1*ln(factor)+1
                tab = R.rope_table(max_pos, self.rot_dim, theta, "yarn", r.scaling_factor, r.original_max_pos,
                                   r.beta_fast, r.beta_slow, table_scale=R.yarn_mscale(r.scaling_factor, 1.0))
            else:
                tab = R.rope_table(max_pos, self.rot_dim, theta, r.scaling_type, r.scaling_factor)
        self.rope_table = tab.to(self.device)
        self.max_rope_pos = max_pos
        self._ntk_tables: Dict[int, torch.Tensor] = {}

    def _qwen_rope(self, max_kv: int):
        """Qwen-1: dynamic-NTK base for contexts beyond seq_length and log-n query scaling
        (src/layers/rotary_embedding_qwen.cpp:33-135)."""
        c = self.cfg
        seq_len = c.seq_length if c.seq_length > 0 else 8192
        table = self.rope_table
        if c.use_dynamic_ntk and max_kv > seq_len:
            ctx_v = math.log(max_kv / seq_len, 2) + 1
            alpha = max(2 ** math.ceil(ctx_v) - 1, 1)
            if alpha not in self._ntk_tables:
                base = c.rope.theta * alpha ** (self.rot_dim / (self.rot_dim - 2))
                self._ntk_tables[alpha] = R.rope_table(self.max_rope_pos, self.rot_dim, base).to(self.device)
            table = self._ntk_tables[alpha]
        return table, seq_len

    def _telechat_rope(self, max_kv: int, max_q: int):
        """TeleChat: NTK-scaled base computed from max(context length, training length) — so even short contexts use
        the base of the training length — and, when the table for a base is first built during a pass whose input is
        longer than the training length, cos / sin scaled by 0.1 ln(input / training) + 1
        (src/layers/rotary_embedding_telechat.cpp:29-35,68-117, rotary_embedding_telechat.h:26-75).  Tables are kept
        per base, as the reference keeps them."""
        c = self.cfg
        train = c.max_pos_seq_len if c.max_pos_seq_len > 0 else 2048
        alpha = R.telechat_ntk_alpha(max(max_kv, train))
        if alpha not in self._ntk_tables:
            mscale = 0.1 * math.log(max_q / train) + 1.0 if max_q > train else 1.0
            base = c.rope.theta * alpha ** (self.rot_dim / (self.rot_dim - 2))
            self._ntk_tables[alpha] = R.rope_table(self.max_rope_pos, self.rot_dim, base, table_scale=mscale).to(self.device)
        return self._ntk_tables[alpha]

    # ------------------------------------------------------------------------------------
    # weight loading
    # ------------------------------------------------------------------------------------
    def _vec(self, name, n, rng=None, ones=False):
        return self.src.vector(name, n, dtype=self.aux_dtype, out_dtype=torch.float32, rng=rng, fake_ones=ones)

    def _opt_vec(self, name, n, rng=None, default_present=False):
        if self.src.fake:
            return self._vec(name, n, rng) if default_present else None
        return self._vec(name, n, rng) if self.src.exists(name) else None

    def _load_embedding(self, share: Optional["Decoder"]) -> None:
        c = self.cfg
        if share is not None:
            self.wte, self.wpe = share.wte, share.wpe
            return
        self.wte = self.wpe = None
        if self.first_stage:
            edt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            self.wte = self.src.matrix("model.wte.bin", (c.vocab_size, c.hidden_size), dtype=self.aux_dtype).to(edt)
            if self.spec.embedding == "opt":
                npos = c.max_pos_seq_len + 2
                self.wpe = self.src.matrix("model.wpe.bin", (npos, c.hidden_size)).to(edt)

    def _load_head(self, share: Optional["Decoder"]) -> None:
        c = self.cfg
        self.final_w = self.final_b = self.lm_head = None
        self.v0, self.v1 = P.vocab_range(c.vocab_size, self.tp, self.tpr)
        if not self.last_stage:
            return
        if share is not None:
            self.final_w, self.final_b, self.lm_head = share.final_w, share.final_b, share.lm_head
            return
        self.final_w = self._vec("model.final_layernorm.weight.bin", c.hidden_size, ones=True)
        if self.spec.norm == "layer":
            self.final_b = self._opt_vec("model.final_layernorm.bias.bin", c.hidden_size, default_present=True)
        hk = "bf16" if self.device.type == "cuda" else "fp32"   # DistLinear keeps 16-bit weights (dist_linear.h:38-64)
        self.lm_head = self.src.linear("model.lm_head.weight.bin", c.hidden_size, c.vocab_size, hk,
                                       out_rng=(self.v0, self.v1), transposed_on_disk=True, dtype=self.aux_dtype)

    def _lin(self, name, in_f, out_f, in_rng=None, out_rng=None, out_ranges=None, kind=None) -> LinearWeight:
        """A projection by base name: fp file ``<name>.weight.0.bin`` or GPTQ ``<name>.qweight.0.bin``."""
        c = self.cfg
        kind = kind or self.kind
        if c.quant_qweight_data_type in ("int8", "uint4") and not self.src.fake:
            return self.src.gptq_linear(name, in_f, out_f, c.quant_qweight_data_type, kind, in_rng, out_rng, out_ranges)
        return self.src.linear(name + ".weight.0.bin", in_f, out_f, kind, in_rng, out_rng, out_ranges)

    def _load_layer(self, i: int) -> Layer:
        c, s = self.cfg, self.spec
        L = Layer()
        L.idx = i
        p = f"model.layers.{i}."
        H = c.hidden_size
        L.attn_norm_w = self._vec(p + "input_layernorm.weight.bin", H, ones=True)
        L.attn_norm_b = self._opt_vec(p + "input_layernorm.bias.bin", H, default_present=s.norm == "layer") \
            if s.norm == "layer" else None
        if s.attention == "mla":
            self._load_mla(L, p)
        else:
            D = self.D
            qsz, kvsz = c.head_num * D, c.kv_head_num * D
            ranges = [(self.qs * D, self.qe * D), (qsz + self.ks * D, qsz + self.ke * D),
                      (qsz + kvsz + self.ks * D, qsz + kvsz + self.ke * D)]
            L.qkv = self._lin(p + "attention.query_key_value", H, qsz + 2 * kvsz, out_ranges=ranges)
            bname = p + "attention.query_key_value.bias.0.bin"
            L.qkv_b = None
            if (self.src.fake and s.qkv_bias) or self.src.exists(bname):
                if self.src.fake:
                    L.qkv_b = self._vec(bname, sum(e - b for b, e in ranges))
                else:
                    L.qkv_b = torch.cat([self._vec(bname, qsz + 2 * kvsz, rng=r) for r in ranges])
            L.o = self._lin(p + "attention.dense", qsz, H, in_rng=(self.qs * D, self.qe * D))
            L.o_b = self._opt_vec(p + "attention.dense.bias.bin", H, default_present=s.dense_bias)
            L.q_norm = L.k_norm = None
            if c.do_qk_norm:
                L.q_norm = self._vec(p + "attention.q_norm.weight.bin", D, ones=True)
                L.k_norm = self._vec(p + "attention.k_norm.weight.bin", D, ones=True)
        L.mlp_norm_w = self._vec(p + "post_attention_layernorm.weight.bin", H, ones=True)
        L.mlp_norm_b = self._opt_vec(p + "post_attention_layernorm.bias.bin", H, default_present=s.norm == "layer") \
            if s.norm == "layer" else None
        kind = s.mlp
        if kind == "deepseek":
            kind = "llama_ds" if i < c.first_k_dense_replace else "deepseek"
        L.mlp_kind = kind
        getattr(self, "_load_mlp_" + kind)(L, p, i)
        return L

    # -- dense MLPs -----------------------------------------------------------------------
    def _ffn_range(self, inter: int, gran: int = 1, split_idx: Optional[int] = None):
        idx = self.tpr if split_idx is None else split_idx
        if gran > 1 and inter % gran == 0:
            return P.task_range_gran(inter, gran, self.tp, idx)
        return P.task_range(inter, self.tp, idx)

    def _load_mlp_llama(self, L, p, i):
        c = self.cfg
        H, I = c.hidden_size, c.inter_size
        r = self._ffn_range(I)
        g = self._lin(p + "mlp.gate_proj", H, I, out_rng=r)
        u = self._lin(p + "mlp.up_proj", H, I, out_rng=r)
        L.gate_up = cat_linear([g, u])
        L.down = self._lin(p + "mlp.down_proj", I, H, in_rng=r)
        L.act = "gelu" if c.activation_type.startswith("gelu") else c.activation_type

    def _load_mlp_chatglm2(self, L, p, i):
        """HF ``dense_h_to_4h`` holds gate‖up on the out dim (src/layers/mlp_chatglm2.h:27-128)."""
        c = self.cfg
        H, I = c.hidden_size, c.inter_size
        r = self._ffn_range(I)
        L.gate_up = self._lin(p + "mlp.dense_h_to_4h", H, 2 * I, out_ranges=[r, (I + r[0], I + r[1])])
        L.down = self._lin(p + "mlp.dense_4h_to_h", I, H, in_rng=r)
        L.act = "silu"
        L.mlp_kind = "llama"

    def _load_mlp_gpt(self, L, p, i):
        c = self.cfg
        H, I = c.hidden_size, c.inter_size
        r = self._ffn_range(I)
        L.fc1 = self._lin(p + "mlp.dense_h_to_4h", H, I, out_rng=r)
        L.fc1_b = self._opt_vec(p + "mlp.dense_h_to_4h.bias.0.bin", I, rng=r, default_present=True)
        L.fc2 = self._lin(p + "mlp.dense_4h_to_h", I, H, in_rng=r)
        L.fc2_b = self._opt_vec(p + "mlp.dense_4h_to_h.bias.bin", H, default_present=True)
        L.act = "relu" if c.activation_type == "relu" else "gelu"

    # -- MoE ------------------------------------------------------------------------------
    def _expert(self, names, H, I, layer, e) -> tuple:
        """(gate‖up, down) of one expert; EP keeps whole experts, TP slices the intermediate
        dim with the reference's rotation (mlp_llama.h:70-79)."""
        env = Env.get()
        if self.ctx.ep_size > 1:
            r = (0, I)
        else:
            gran = 128 if self.kind == "fp8" else 1
            r = self._ffn_range(I, gran, P.moe_slice_index(self.tpr, self.tp, layer, e, env.moe_split_balance_dim))
        g = self._named_lin(names[0], H, I, out_rng=r)
        u = self._named_lin(names[1], H, I, out_rng=r)
        d = self._named_lin(names[2], I, H, in_rng=r)
        return cat_linear([g, u]), d

    def _named_lin(self, fname, in_f, out_f, in_rng=None, out_rng=None):
        if self.cfg.model_type == "deepseek_moe":
            return self.src.fp8_linear(fname, in_f, out_f, in_rng, out_rng, kind=self.kind)
        return self.src.linear(fname, in_f, out_f, self.kind, in_rng, out_rng)

    def _local_experts(self, E: int):
        if self.ctx.ep_size > 1:
            return P.expert_range(E, self.ctx.ep_size, self.ctx.ep_rank)
        return 0, E

    def _load_mlp_mixtral(self, L, p, i):
        c = self.cfg
        H, I, E = c.hidden_size, c.inter_size, c.sparse_experts
        L.router = self.src.linear(p + "moe.gate.weight.bin", H, E, "fp32" if self.device.type == "cpu" else "bf16")
        L.e0, L.e1 = self._local_experts(E)
        L.experts = [self._expert([p + f"moe.sparse_experts.{e}.w{j}.0.bin" for j in (1, 2, 3)], H, I, i, e)
                     for e in range(L.e0, L.e1)]
        L.act = c.activation_type if c.activation_type != "swiglu" else "silu"
        L.top_k = c.num_experts_per_tok or 2
        L.route_kind = "mixtral"

    def _load_mlp_qwen3_moe(self, L, p, i):
        c = self.cfg
        H, E = c.hidden_size, c.sparse_experts
        I = c.moe_intermediate_size or c.inter_size
        L.router = self.src.linear(p + "mlp.gate.weight.0.bin", H, E, "fp32" if self.device.type == "cpu" else "bf16")
        L.e0, L.e1 = self._local_experts(E)
        L.experts = [self._expert([p + f"mlp.experts.{e}.{n}_proj.weight.0.bin" for n in ("gate", "up", "down")],
                                  H, I, i, e) for e in range(L.e0, L.e1)]
        L.act = "silu"
        L.top_k = c.num_experts_per_tok or 8
        L.route_kind = "softmax_topk"

    def _load_mlp_llama_ds(self, L, p, i):
        c = self.cfg
        H, I = c.hidden_size, c.inter_size
        r = self._ffn_range(I, 128)
        g = self.src.fp8_linear(p + "mlp.gate_proj", H, I, out_rng=r, kind=self.kind)
        u = self.src.fp8_linear(p + "mlp.up_proj", H, I, out_rng=r, kind=self.kind)
        L.gate_up = cat_linear([g, u])
        L.down = self.src.fp8_linear(p + "mlp.down_proj", I, H, in_rng=r, kind=self.kind)
        L.act = "silu"
        L.mlp_kind = "llama"

    def _load_mlp_deepseek(self, L, p, i):
        c = self.cfg
        H, E, I = c.hidden_size, c.sparse_experts, c.moe_intermediate_size
        rk = "fp32" if self.device.type == "cpu" else "bf16"
        if self.src.fake:
            L.router = self.src.linear(p + "mlp.gate.weight.bin", H, E, rk)
            L.router_bias = self.src.vector(p + "mlp.gate.e_score_correction_bias.bin", E) \
                if c.topk_method == "noaux_tc" else None
        else:
            w = self.src.matrix(p + "mlp.gate.weight.bin", (H, E), dtype="bf16")
            L.router = make_linear(w.t().contiguous(), rk)
            bn = p + "mlp.gate.e_score_correction_bias.bin"
            L.router_bias = self.src.vector(bn, E, dtype="bf16") if self.src.exists(bn) else None
        L.shared = None
        if c.dense_experts > 0:
            SI = c.dense_experts * I
            r = self._ffn_range(SI, 128)
            g = self.src.fp8_linear(p + "mlp.shared_experts.gate_proj", H, SI, out_rng=r, kind=self.kind)
            u = self.src.fp8_linear(p + "mlp.shared_experts.up_proj", H, SI, out_rng=r, kind=self.kind)
            d = self.src.fp8_linear(p + "mlp.shared_experts.down_proj", SI, H, in_rng=r, kind=self.kind)
            L.shared = (cat_linear([g, u]), d)
        L.e0, L.e1 = self._local_experts(E)
        L.experts = [self._expert([p + f"mlp.experts.{e}.{n}_proj" for n in ("gate", "up", "down")], H, I, i, e)
                     for e in range(L.e0, L.e1)]
        L.act = "silu"
        L.top_k = c.num_experts_per_tok
        L.route_kind = "deepseek"

    # -- MLA ------------------------------------------------------------------------------
    def _load_mla(self, L, p):
        c = self.cfg
        H = c.hidden_size
        nope, rope, vd, kvl, ql = c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim, c.kv_lora_rank, c.q_lora_rank
        qk = nope + rope
        hs, he = self.qs, self.qe
        kv_a = self.src.fp8_linear(p + "self_attn.kv_a_proj_with_mqa", H, kvl + rope, kind=self.kind)
        if ql > 0:
            q_a = self.src.fp8_linear(p + "self_attn.q_a_proj", H, ql, kind=self.kind)
            L.qkv_a = cat_linear([q_a, kv_a])             # merged down-projection (attn_deepseek.h:78-117)
            L.q_a_norm = self.src.vector(p + "self_attn.q_a_layernorm.weight.bin", ql, dtype="bf16", fake_ones=True)
            L.q_b = self.src.fp8_linear(p + "self_attn.q_b_proj", ql, c.head_num * qk,
                                        out_rng=(hs * qk, he * qk), kind=self.kind)
        else:
            q = self.src.fp8_linear(p + "self_attn.q_a_proj", H, c.head_num * qk, out_rng=(hs * qk, he * qk),
                                    kind=self.kind)
            L.qkv_a = cat_linear([q, kv_a]) if (he - hs) * qk % 128 == 0 or self.kind != "fp8" else None
            L.q_direct, L.kv_a = q, kv_a
            L.q_a_norm = L.q_b = None
        L.kv_a_norm = self.src.vector(p + "self_attn.kv_a_layernorm.weight.bin", kvl, dtype="bf16", fake_ones=True)
        # kv_b [kv_lora, heads*(nope+v)] -> per-head W_uk [nope,kv_lora], W_uv [v,kv_lora], kept dense
        # in the activation type (absorbed decode multiplies them per head; attn_deepseek.h:408-433)
        kvb = self.src.fp8_linear(p + "self_attn.kv_b_proj", kvl, c.head_num * (nope + vd),
                                  out_rng=(hs * (nope + vd), he * (nope + vd)), kind=self.kind)
        dense = R.dequant_weight(kvb).view(he - hs, nope + vd, kvl)
        adt = self.act_dtype
        L.w_uk = dense[:, :nope].contiguous().to(adt)
        L.w_uv = dense[:, nope:].contiguous().to(adt)
        L.o = self.src.fp8_linear(p + "attention.dense", c.head_num * vd, H, in_rng=(hs * vd, he * vd), kind=self.kind)
        L.o_b = None

    def _fold_norms(self) -> None:
        """On a GPU, multiply the RMSNorm gain into the columns of the bf16 projection that consumes the
        normalised state (QKV, gate|up, lm_head).  What is left of the norm is one factor per token,
        rsqrt(mean(x^2) + eps), which the GEMM computes itself at decode sizes (ops.linear_rms): two launches
        per layer disappear from the decode step.  The reference keeps the norm as its own kernel
        (src/layers/attention.h, src/layers/mlp_llama.h call norm.forward before the first GEMM)."""
        s = self.spec
        self.head_fold = False
        for L in self.layers:
            L.attn_fold = L.mlp_fold = False
        if self.device.type != "cuda" or s.norm != "rms" or s.resid_from_norm or not Env.get().fuse_norm:
            return

        def fold(W: LinearWeight, g: torch.Tensor) -> bool:
            if W is None or W.kind != "bf16" or W.w.dtype != torch.bfloat16:
                return False
            if not W.cache.get("norm_folded"):
                gf = g.to(W.w.device, torch.float32)[None, :]
                for r in range(0, W.w.shape[0], 8192):
                    W.w[r:r + 8192] = (W.w[r:r + 8192].float() * gf).to(torch.bfloat16)
                W.cache["norm_folded"] = True
            return True

        for L in self.layers:
            if s.attention != "mla" and L.attn_norm_b is None:
                L.attn_fold = fold(L.qkv, L.attn_norm_w)
            if L.mlp_kind == "llama" and L.mlp_norm_b is None:
                L.mlp_fold = fold(L.gate_up, L.mlp_norm_w)
        if self.last_stage and self.lm_head is not None and self.final_b is None:
            self.head_fold = fold(self.lm_head, self.final_w)

    # ------------------------------------------------------------------------------------
    # forward
    # ------------------------------------------------------------------------------------
    def _norm(self, x, w, b):
        if self.spec.norm == "rms":
            return ops.rmsnorm(x, w, self.eps)
        return ops.layernorm(x, w, b, self.eps)

    def _row_parallel(self, h, W, bias, residual, res_scale=1.0):
        """Row-parallel GEMM + sum over TP ranks.  With peer memory (B200, decode sizes) this is ONE
        kernel: the GEMM epilogue all-reduces its tiles over NVLink and adds bias/residual after the
        sum.  Otherwise: partial GEMM with residual/bias on rank 0 only, then a collective."""
        peer = getattr(self.ctx, "peer", None)
        if self.tp > 1 and peer is not None and h.is_cuda:
            T = h.numel() // h.shape[-1]
            if peer.can_fuse(T, W.out_features, W.kind):
                return peer.gemm_ar(h, W, bias, None, residual, res_scale)
            if peer.can_fuse_bulk(T, W.out_features, h.shape[-1], W.kind):      # prefill sizes, opt-in
                y = peer.gemm_ar_bulk(h, W, bias, None, residual, res_scale)
                if y is not None:
                    return y
        lead = self.tpr == 0
        y = ops.linear(h, W, bias if lead else None, None, residual if lead else None, res_scale)
        if self.tp > 1:
            if self._overlap:
                # interleaved prefill: the sum is started here and waited for by the driver of the two interleaved
                # batches, after it has enqueued the other batch's next block (Decoder.forward_pair)
                self._work = self.ctx.all_reduce_async(y)
            elif peer is not None and y.is_cuda and y.numel() <= peer.slot and \
                    y.dtype in (torch.float32, torch.bfloat16):
                # decode sizes with a weight type (or a token count) the fused kernel does not take: the partial
                # products are summed by the peer-memory one-shot kernel, which a CUDA graph can hold (a NCCL call
                # cannot safely sit in one).  The decision depends on the shape only, so every rank takes it alike.
                y = peer.all_reduce(y.contiguous())
            else:
                y = self.ctx.all_reduce(y)
        return y

    def embed(self, b: Batch) -> torch.Tensor:
        c, s = self.cfg, self.spec
        with TimeLine("Decoder.embedding"):
            scale = math.sqrt(c.hidden_size) if s.embedding == "gemma" else 1.0
            if s.embedding == "opt":
                return ops.embedding(b.ids, self.wte, scale, self.act_dtype, self.wpe, b.positions, 2)
            return ops.embedding(b.ids, self.wte, scale, self.act_dtype)

    def _attention(self, L: Layer, x, b: Batch, cache: PagedKVCache, li: int):
        c, s = self.cfg, self.spec
        h = None
        if not L.attn_fold:
            with TimeLine("Attention.norm"):
                h = self._norm(x, L.attn_norm_w, L.attn_norm_b)
        if s.attention == "mla":
            a = self._mla(L, h, b, cache, li)
        else:
            table, q_scale, positions = self.rope_table, None, b.positions
            if s.logn_ntk and table is not None:
                table, seq_len = self._qwen_rope(b.max_kv)
                if c.use_logn_attn and b.max_kv > seq_len:
                    q_scale = torch.clamp(torch.log(b.positions.float() + 1) / math.log(seq_len), min=1.0)
            if s.telechat_ntk and table is not None:
                table = self._telechat_rope(b.max_kv, b.max_q)
            xin = x if L.attn_fold else h
            fused_qkv = (xin.is_cuda and s.rope != "2d" and
                         ops.can_fuse_qkv_rope(L.qkv, xin.numel() // xin.shape[-1], self.D, cache.k[li], cache.ks[li],
                                               L.q_norm, L.k_norm, self.rope_style))
            if fused_qkv:
                # decode sizes: RoPE and the cache append are the epilogue of the QKV product (one kernel)
                with TimeLine("QKV.linear+QKPO"):
                    q = ops.qkv_linear_rope_cache(xin, L.qkv, L.qkv_b, self.eps if L.attn_fold else None, self.hq,
                                                  self.hkv, positions, table, self.rot_dim, self.rope_style,
                                                  cache.k[li], cache.v[li], b.slots, q_scale)
            else:
                with TimeLine("QKV.linear"):
                    qkv = ops.linear_rms(x, L.qkv, self.eps, L.qkv_b) if L.attn_fold else ops.linear(h, L.qkv, L.qkv_b)
            with TimeLine("QKPO"):
                if fused_qkv:
                    pass
                elif s.rope == "2d":
                    q = self._rope2d_cache(L, qkv, b, cache, li)
                else:
                    q = ops.qkv_rope_cache(qkv, self.hq, self.hkv, self.D, positions, table, self.rot_dim,
                                           self.rope_style, cache.k[li], cache.v[li], cache.ks[li], cache.vs[li],
                                           b.slots, q_scale, L.q_norm, L.k_norm, self.eps)
            with TimeLine("MHA"):
                a = ops.paged_attention(q, cache.k[li], cache.v[li], b.block_table, b.cu_q, b.kv_lens, self.scale,
                                        cache.ks[li], cache.vs[li], self.slopes, True,
                                        b.prefix_lm_lens if s.prefix_lm else None, self.group, self.q_off, b)
            a = a.reshape(a.shape[0], -1)
        with TimeLine("Output"):
            if s.resid_from_norm:
                alpha = math.sqrt(2 * c.num_layer)
                return self._row_parallel(a, L.o, L.o_b, h, alpha)
            return self._row_parallel(a, L.o, L.o_b, x)

    def _rope2d_cache(self, L, qkv, b: Batch, cache, li):
        """ChatGLM-1: first half of each head rotates with the position stream, second half with
        the block-position stream (src/layers/rope_2d.cpp, src/models/chatglm.cpp:118-206)."""
        return ops.qkv_rope2d_cache(qkv, self.hq, self.hkv, self.D, b.positions, b.positions2, self.rope_table,
                                    cache.k[li], cache.v[li], cache.ks[li], cache.vs[li], b.slots)

    def _mla(self, L: Layer, h, b: Batch, cache: PagedKVCache, li: int):
        c = self.cfg
        nope, rope, vd, kvl, ql = c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim, c.kv_lora_rank, c.q_lora_rank
        T = h.shape[0]
        Hl = self.hq
        if ql > 0:
            qa_kv = ops.linear(h, L.qkv_a)                       # [T, ql + kvl + rope]
            qa = ops.rmsnorm(qa_kv[:, :ql], L.q_a_norm, self.eps)
            q = ops.linear(qa, L.q_b)
            kv = qa_kv[:, ql:]
        elif L.qkv_a is not None:
            both = ops.linear(h, L.qkv_a)
            q, kv = both[:, : Hl * (nope + rope)], both[:, Hl * (nope + rope):]
        else:
            q, kv = ops.linear(h, L.q_direct), ops.linear(h, L.kv_a)
        q_nope, q_rope = ops.mla_prep(q, kv, Hl, nope, rope, kvl, b.positions, self.rope_table, L.kv_a_norm, self.eps,
                                      cache.k[li], b.slots)
        a = ops.mla_attention(q_nope, q_rope, cache.k[li], b.block_table, b.cu_q, b.kv_lens, L.w_uk, L.w_uv,
                              self.scale, absorbed=b.is_decode, meta=b)
        return a.reshape(T, Hl * vd)

    def _mlp(self, L: Layer, x, b: Batch):
        s = self.spec
        k = L.mlp_kind
        if L.mlp_fold:
            with TimeLine("LlamaMLP"):
                g = ops.linear_rms(x, L.gate_up, self.eps, None, L.act, gated=True)
                return self._row_parallel(g, L.down, None, x, 1.0)
        with TimeLine("MLP.norm"):
            h = self._norm(x, L.mlp_norm_w, L.mlp_norm_b)
        resid, rs = (h, math.sqrt(2 * self.cfg.num_layer)) if s.resid_from_norm else (x, 1.0)
        if k == "llama":
            with TimeLine("LlamaMLP"):
                g = ops.linear_gated(h, L.gate_up, L.act)
                return self._row_parallel(g, L.down, None, resid, rs)
        if k == "gpt":
            with TimeLine("MLP"):
                g = ops.linear(h, L.fc1, L.fc1_b, L.act)
                return self._row_parallel(g, L.fc2, L.fc2_b, resid, rs)
        with TimeLine("MoE"):
            return self._moe(L, h, x)

    def _route(self, L: Layer, h):
        c = self.cfg
        logits = ops.linear(h, L.router, out_dtype=torch.float32)
        if L.route_kind == "deepseek":
            return ops.route(logits, "deepseek", L.top_k, L.router_bias, max(c.n_group, 1), max(c.topk_group, 1),
                             c.routed_scaling_factor, c.norm_topk_prob, c.scoring_func or "sigmoid")
        if L.route_kind == "softmax_topk":
            return ops.route(logits, "softmax_topk", L.top_k, norm_topk=c.norm_topk_prob or True)
        return ops.route(logits, "mixtral", L.top_k)

    def _moe_dp(self, L: Layer, h, x):
        """MoE block with data-parallel attention (XFT_ATTENTION_DP=1): this rank holds only ITS sequences' tokens.
        Dispatch: every (token, expert) pair travels to the rank that owns the expert (all-to-all, rows grouped by
        destination).  The owners run their experts on what they received.  Combine: the expert outputs travel back
        the same way and are summed with the routing weights at the token's home rank.  `h` may have no rows (a rank
        without work in this step still serves its experts to the others); then `x` is unused."""
        ctx, c = self.ctx, self.cfg
        T, H = h.shape[0], c.hidden_size
        E, k = c.sparse_experts, L.top_k
        dev = h.device
        ep = getattr(ctx, "epcomm", None)
        if ep is not None and h.is_cuda and ep.fits(ctx.dp_max_tokens, k):
            # decode sizes, opt-in (XFT_MOE_FUSED_A2A=1): the rows cross NVLink as stores from the dispatch / return
            # kernels, no host-side count exchange (csrc/kernels/ep_comm.cu).  dp_max_tokens is the largest local
            # token count over the ranks in this pass, so all ranks take the same branch.
            idx, w = self._route(L, h) if T > 0 else (None, None)
            shared = None
            if T > 0 and getattr(L, "shared", None) is not None:
                shared = ops.linear(ops.linear_gated(h, L.shared[0], L.act), L.shared[1], out_dtype=torch.float32)
            # the receive area has room for the worst case; about dp_max_tokens * k of its rows are real on average
            run = lambda rows, ids, ones: ops.moe_experts(rows, ids, ones, L.experts, L.act, L.e0, getattr(L, "packed", None),
                                                          expected_pairs=max(ctx.dp_max_tokens, 1) * k)
            return ep.exchange(h, idx, w, E, run, shared, x)
        if T > 0:
            idx, w = self._route(L, h)
            flat_e = idx.reshape(-1).long()
            flat_t = torch.arange(T, device=dev).repeat_interleave(k)
            if not hasattr(self, "_expert_owner"):
                self._expert_owner = torch.tensor([P.expert_owner(e, E, ctx.ep_size) for e in range(E)], device=dev)
            dest = self._expert_owner[flat_e]
            order = torch.argsort(dest, stable=True)
            send_counts = torch.bincount(dest, minlength=ctx.ep_size).tolist()
            send_tok = h[flat_t[order]]
            send_e = flat_e[order].int()
        else:
            send_counts = [0] * ctx.ep_size
            send_tok = h.new_zeros(0, H)
            send_e = torch.zeros(0, dtype=torch.int32, device=dev)
        recv_tok, recv_counts = ctx.all_to_all(send_tok, send_counts)
        recv_e = ctx.all_to_all_known(torch.empty(sum(recv_counts), dtype=torch.int32, device=dev), send_e, recv_counts,
                                      send_counts)
        R = recv_tok.shape[0]
        if R > 0:
            ones = torch.ones(R, 1, dtype=torch.float32, device=dev)
            y = ops.moe_experts(recv_tok, recv_e.view(R, 1), ones, L.experts, L.act, L.e0, getattr(L, "packed", None))
        else:
            y = torch.zeros(0, H, dtype=torch.float32, device=dev)
        back = ctx.all_to_all_known(torch.empty(sum(send_counts), H, dtype=torch.float32, device=dev), y, send_counts,
                                    recv_counts)
        if T == 0:
            return h
        out = torch.zeros(T, H, dtype=torch.float32, device=dev)
        out.index_add_(0, flat_t[order], back * w.reshape(-1)[order].float()[:, None])
        if getattr(L, "shared", None) is not None:
            g = ops.linear_gated(h, L.shared[0], L.act)
            out = out + ops.linear(g, L.shared[1], out_dtype=torch.float32)
        return (out + x.float()).to(x.dtype)

    def forward_idle(self) -> None:
        """Data-parallel attention: a rank with no sequence in this pass still takes part in the dispatch / combine
        of every MoE layer (its experts may be needed by the others)."""
        empty = torch.zeros(0, self.cfg.hidden_size, dtype=self.act_dtype, device=self.device)
        for L in self.layers:
            if L.mlp_kind not in ("llama", "gpt"):
                self._moe_dp(L, empty, None)

    def _moe(self, L: Layer, h, x):
        if self.ctx.dp_size > 1:
            return self._moe_dp(L, h, x)
        c = self.cfg
        logits = ops.linear(h, L.router, out_dtype=torch.float32)
        if L.route_kind == "deepseek":
            idx, w = ops.route(logits, "deepseek", L.top_k, L.router_bias, max(c.n_group, 1), max(c.topk_group, 1),
                               c.routed_scaling_factor, c.norm_topk_prob, c.scoring_func or "sigmoid")
        elif L.route_kind == "softmax_topk":
            idx, w = ops.route(logits, "softmax_topk", L.top_k, norm_topk=c.norm_topk_prob or True)
        else:
            idx, w = ops.route(logits, "mixtral", L.top_k)
        out = ops.moe_experts(h, idx, w, L.experts, L.act, L.e0, getattr(L, "packed", None))   # fp32 partial
        if getattr(L, "shared", None) is not None:
            g = ops.linear_gated(h, L.shared[0], L.act)
            out = out + ops.linear(g, L.shared[1], out_dtype=torch.float32)
        if self.tpr == 0:
            out = out + x.float()
        if self.tp > 1:
            peer = getattr(self.ctx, "peer", None)
            if peer is not None and out.is_cuda and out.numel() <= peer.slot:
                # decode sizes: the peer-memory one-shot kernel sums the fp32 partials (it can be captured in a CUDA
                # graph, which a NCCL call cannot safely be)
                return peer.all_reduce(out.contiguous()).to(x.dtype)
            y = out.to(x.dtype)
            if self._overlap:                 # interleaved prefill: started here, awaited by forward_pair's driver
                self._work = self.ctx.all_reduce_async(y)
                return y
            return self.ctx.all_reduce(y)
        return out.to(x.dtype)

    def forward_layers(self, x: torch.Tensor, b: Batch, cache: PagedKVCache) -> torch.Tensor:
        dbg = debugger.enabled()
        step = debugger.next_step() if dbg else 0
        if dbg:
            debugger.dump("embedding", x, self.ctx.rank, step)
        for li, L in enumerate(self.layers):
            with TimeLine("Decoder.forwardAttention"):
                x = self._attention(L, x, b, cache, li)
            if dbg:
                debugger.dump(f"layer{self.l0 + li}_attn_out", x, self.ctx.rank, step)
            with TimeLine("Decoder.forwardFFN"):
                x = self._mlp(L, x, b)
            if dbg:
                debugger.dump(f"layer{self.l0 + li}_ffn_out", x, self.ctx.rank, step)
        return x

    def _layers_interleaved(self, x: torch.Tensor, b: Batch, cache: PagedKVCache):
        """forward_layers as a generator: after every block whose row-parallel sum was only started, it hands the
        pending handle to the driver and continues when asked to."""
        for li, L in enumerate(self.layers):
            x = self._attention(L, x, b, cache, li)
            w, self._work = self._work, None
            yield w
            x = self._mlp(L, x, b)
            w, self._work = self._work, None
            yield w
        return x

    def forward_pair(self, b0: Batch, b1: Batch, cache: PagedKVCache):
        """Prefill of two batches with the tensor-parallel sums of one overlapping the compute of the other
        (XFT_PREFILL_OVERLAP=1).  The reference waits for every all-reduce before it goes on
        (src/layers/decoder_block.h:122-134); here batch A starts the sum of its block and, while NVLink carries it,
        batch B's next block runs on the SMs, and so on alternately.  Results are those of two forward() calls."""
        assert self.first_stage and self.last_stage and self.ctx.dp_size == 1
        xs = [self.embed(b0), self.embed(b1)]
        bs = [b0, b1]
        self.pairs_run += 1
        self._overlap = True
        try:
            gens = [self._layers_interleaved(xs[i], bs[i], cache) for i in range(2)]
            pending = [None, None]
            alive = [True, True]
            while any(alive):
                for i in range(2):
                    if not alive[i]:
                        continue
                    if pending[i] is not None:
                        pending[i].wait()
                        pending[i] = None
                    try:
                        pending[i] = next(gens[i])
                    except StopIteration as e:
                        xs[i] = e.value
                        alive[i] = False
        finally:
            self._overlap = False
            self._work = None
        return self.head(xs[0], b0), self.head(xs[1], b1)

    def head(self, x: torch.Tensor, b: Batch) -> torch.Tensor:
        """Final norm on the rows that need logits + vocab-split lm_head -> fp32 [rows, vocab/tp]."""
        if b.logit_rows is not None:
            x = x.index_select(0, b.logit_rows)
        if self.head_fold:
            with TimeLine("DistLinear.forward"):
                return ops.linear_rms(x, self.lm_head, self.eps, out_dtype=torch.float32)
        x = self._norm(x, self.final_w, self.final_b)
        with TimeLine("DistLinear.forward"):
            return ops.linear(x, self.lm_head, out_dtype=torch.float32)

    def forward(self, b: Batch, cache: PagedKVCache, hidden: Optional[torch.Tensor] = None) -> torch.Tensor:
        """First stage embeds `b.ids`; later stages take `hidden`.  Returns local logits on the
        last stage, the hidden state otherwise."""
        with TimeLine("Decoder.forward"):
            x = self.embed(b) if self.first_stage else hidden
            x = self.forward_layers(x, b, cache)
            if self.last_stage:
                return self.head(x, b)
            return x

    # -- sizes ------------------------------------------------------------------------------
    def kv_geometry(self):
        c = self.cfg
        if self.spec.attention == "mla":
            return dict(kv_heads=1, k_dim=c.kv_lora_rank + c.qk_rope_head_dim, v_dim=0, latent=True)
        return dict(kv_heads=self.hkv, k_dim=self.D, v_dim=self.D, latent=False)

    def weight_bytes(self) -> int:
        n = 0
        for L in self.layers:
            for v in vars(L).values():
                if isinstance(v, LinearWeight):
                    n += v.nbytes
                elif isinstance(v, (list, tuple)):
                    for e in v:
                        if isinstance(e, tuple):
                            n += sum(w.nbytes for w in e if isinstance(w, LinearWeight))
        if self.lm_head is not None:
            n += self.lm_head.nbytes
        return n
