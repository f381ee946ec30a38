"""Model configuration: ``config.ini`` parsing and dtype-string handling.

The checkpoint directory contract is the reference's: one ``config.ini`` whose single
section name selects the model family, plus raw ``.bin`` tensors.  The keys and their
defaults follow ``src/models/common_decoder.h:167-270`` of the reference; the dtype
vocabulary follows ``include/dtype.h:18-36`` and
``src/xfastertransformer/automodel.py:19-47``.

Unlike the reference, where every (family, weight type, kv type) triple is a C++ template
instantiation, here all of this is *data*: one `ModelConfig` drives one generic decoder.
"""
from __future__ import annotations

import configparser
import math
import os
from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

# dtype strings accepted by AutoModel (reference automodel.py:20-37)
WEIGHT_DTYPES = (
    "fp16", "bf16", "int8", "w8a8", "int4", "nf4",
    "bf16_fp16", "bf16_int8", "bf16_w8a8", "bf16_int4", "bf16_nf4",
    "w8a8_int8", "w8a8_int4", "w8a8_nf4", "fp8_e4m3",
)
KV_DTYPES = ("fp16", "bf16", "int8")

# config.ini section names registered by the reference (model_factory.h / models.cpp:1022)
MODEL_TYPES = (
    "llama", "yarn_llama", "gemma", "qwen", "qwen2", "qwen3", "qwen3_moe", "mixtral",
    "deepseek_moe", "baichuan", "chatglm", "chatglm2", "chatglm3", "chatglm4", "gpt",
    "telechat",
)


def split_hybrid_dtype(dtype: str) -> Tuple[str, str]:
    """``"bf16_int8"`` -> (prefill dtype, decode dtype); plain names map to themselves.

    ``fp8_e4m3`` contains an underscore but is a single type (reference
    ``hybrid_model.h:46-83`` registers only the pairs listed in `WEIGHT_DTYPES`).
    """
    if dtype not in WEIGHT_DTYPES:
        raise ValueError(f"AutoModel don't support {dtype}.")
    if dtype == "fp8_e4m3" or "_" not in dtype:
        return dtype, dtype
    a, b = dtype.split("_", 1)
    return a, b


def _to_bool(v) -> bool:
    if isinstance(v, bool):
        return v
    s = str(v).strip().lower()
    if s in ("1", "true", "yes", "on"):
        return True
    if s in ("0", "false", "no", "off", ""):
        return False
    return bool(float(s))


@dataclass
class RopeConfig:
    theta: float = 10000.0
    scaling_type: str = ""            # "", "linear", "yarn", "dynamic"
    scaling_factor: float = 1.0
    original_max_pos: int = 2048
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 1.0


@dataclass
class ModelConfig:
    model_type: str = "llama"
    head_num: int = 0
    kv_head_num: int = 0
    size_per_head: int = 0
    hidden_size: int = 0
    inter_size: int = 0
    num_layer: int = 0
    vocab_size: int = 0
    max_pos_seq_len: int = 0
    model_max_length: int = 0
    seq_length: int = -1              # Qwen-1 training length for log-n / NTK
    use_logn_attn: bool = True
    use_dynamic_ntk: bool = True
    layernorm_eps: float = 1e-6
    activation_type: str = "silu"
    start_id: int = 0
    end_id: int = 0
    pad_id: int = -1
    weight_data_type: str = "fp16"    # storage type of the .bin files
    quant_qweight_data_type: str = ""
    quant_scales_data_type: str = ""
    quant_zeros_data_type: str = ""
    quant_groupsize: int = -1
    rope: RopeConfig = field(default_factory=RopeConfig)
    # MoE
    sparse_experts: int = 8
    dense_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = False
    first_k_dense_replace: int = 0
    topk_group: int = 0
    n_group: int = 0
    topk_method: str = ""
    scoring_func: str = ""
    routed_scaling_factor: float = 1.0
    # MLA
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # Qwen3
    do_qk_norm: bool = False
    # raw key/value pairs (for family-specific look-ups, like DecoderContext::GetAttr)
    raw: Dict[str, str] = field(default_factory=dict)

    # ---- derived ----------------------------------------------------------------------
    @property
    def is_mla(self) -> bool:
        return self.qk_nope_head_dim > 0 and self.qk_rope_head_dim > 0

    @property
    def q_size(self) -> int:
        return self.head_num * self.size_per_head

    @property
    def kv_size(self) -> int:
        return self.kv_head_num * self.size_per_head

    @property
    def attn_scale(self) -> float:
        """Softmax scale.  MLA: 1/sqrt(nope+rope) * mscale^2 where the reference hard-wires
        the YaRN factor 40 (``common_decoder.h:272-274``); here the factor comes from the
        config so other factors work too (identical for DeepSeek-V3/R1, factor 40)."""
        if self.is_mla:
            base = 1.0 / math.sqrt(self.qk_nope_head_dim + self.qk_rope_head_dim)
            if self.rope.scaling_type == "yarn" and self.rope.scaling_factor > 1:
                m = 0.1 * self.rope.mscale_all_dim * math.log(self.rope.scaling_factor) + 1.0
                return base * m * m
            return base
        return 1.0 / math.sqrt(self.size_per_head)

    def get(self, key: str, default=None):
        return self.raw.get(key, default)

    # ---- io ---------------------------------------------------------------------------
    @classmethod
    def from_ini(cls, path: str) -> "ModelConfig":
        ini = path if path.endswith(".ini") else os.path.join(path, "config.ini")
        if not os.path.exists(ini):
            raise FileNotFoundError(f"config.ini not found under {path}")
        cp = configparser.ConfigParser()
        cp.read(ini)
        secs = cp.sections()
        if not secs:
            raise ValueError(f"{ini} has no section")
        sec = secs[0]
        if sec not in MODEL_TYPES:
            raise ValueError(f"unsupported model type [{sec}] in {ini}")
        kv = {k: v for k, v in cp[sec].items()}

        def gi(k, d=0):
            return int(float(kv[k])) if k in kv and kv[k] != "" else d

        def gf(k, d=0.0):
            return float(kv[k]) if k in kv and kv[k] != "" else d

        def gs(k, d=""):
            return kv.get(k, d)

        def gb(k, d=False):
            return _to_bool(kv[k]) if k in kv else d

        head_num = gi("head_num")
        size_per_head = gi("size_per_head")
        max_pos = gi("max_pos_seq_len", 0)
        # The reference reads only `layernorm_eps` (default 1e-6) and ignores the
        # `rms_norm_eps` some converters write; honour both, in that order.
        eps = gf("layernorm_eps", gf("rms_norm_eps", 1e-6))
        c = cls(
            model_type=sec,
            head_num=head_num,
            kv_head_num=gi("kv_head_num", head_num),
            size_per_head=size_per_head,
            hidden_size=gi("hidden_size", head_num * size_per_head),
            inter_size=gi("inter_size"),
            num_layer=gi("num_layer"),
            vocab_size=gi("vocab_size"),
            max_pos_seq_len=max_pos,
            model_max_length=gi("model_max_length", max_pos),
            seq_length=gi("seq_length", -1),
            use_logn_attn=gb("use_logn_attn", True),
            use_dynamic_ntk=gb("use_dynamic_ntk", True),
            layernorm_eps=eps,
            activation_type=gs("activation_type", "silu").lower(),
            start_id=gi("start_id", 0),
            end_id=gi("end_id", gi("start_id", 0)),
            pad_id=gi("pad_id", -1),
            weight_data_type=gs("weight_data_type", "fp16").lower(),
            quant_qweight_data_type=gs("quant_qweight_data_type", ""),
            quant_scales_data_type=gs("quant_scales_data_type", ""),
            quant_zeros_data_type=gs("quant_zeros_data_type", ""),
            quant_groupsize=gi("quant_groupsize", -1),
            rope=RopeConfig(
                theta=gf("rope_theta", 10000.0),
                scaling_type=gs("rope_scaling_type", gs("rope_type", "")).lower(),
                scaling_factor=gf("rope_scaling_factor", gf("scaling_factor", 1.0)),
                original_max_pos=gi("rope_scaling_original_max_position_embeddings", 2048),
                beta_fast=gf("rope_scaling_beta_fast", 32),
                beta_slow=gf("rope_scaling_beta_slow", 1),
                mscale=gf("rope_scaling_mscale", 1.0),
                mscale_all_dim=gf("rope_scaling_mscale_all_dim", 1.0),
            ),
            sparse_experts=gi("sparse_experts", 8),
            dense_experts=gi("dense_experts", 0),
            num_experts_per_tok=gi("num_experts_per_tok", 0),
            moe_intermediate_size=gi("moe_intermediate_size", 0),
            norm_topk_prob=gb("norm_topk_prob", False),
            first_k_dense_replace=gi("first_k_dense_replace", 0),
            topk_group=gi("topk_group", 0),
            n_group=gi("n_group", 0),
            topk_method=gs("topk_method", ""),
            scoring_func=gs("scoring_func", ""),
            routed_scaling_factor=gf("routed_scaling_factor", 1.0),
            q_lora_rank=gi("q_lora_rank", 0),
            kv_lora_rank=gi("kv_lora_rank", 0),
            qk_nope_head_dim=gi("qk_nope_head_dim", 0),
            qk_rope_head_dim=gi("qk_rope_head_dim", 0),
            v_head_dim=gi("v_head_dim", 0),
            do_qk_norm=gb("do_qk_norm", False),
            raw=kv,
        )
        if c.quant_qweight_data_type in ("int8", "uint4"):
            if c.quant_scales_data_type != "fp32" or c.quant_zeros_data_type != "fp32":
                raise ValueError("quantised checkpoints need fp32 scales and zeros")
            if c.quant_groupsize != -1:
                raise ValueError("Quantization with groupsize is not supported.")
        if c.model_type == "mixtral" and c.num_experts_per_tok == 0:
            c.num_experts_per_tok = 2
        if c.is_mla and c.v_head_dim == 0:
            c.v_head_dim = c.size_per_head
        return c

    def to_ini(self, path: str, extra: Optional[Dict[str, str]] = None) -> None:
        """Write a config.ini the way the converters do (one section = model type)."""
        cp = configparser.ConfigParser()
        d: Dict[str, str] = dict(self.raw)
        d.update({
            "head_num": str(self.head_num),
            "kv_head_num": str(self.kv_head_num),
            "size_per_head": str(self.size_per_head),
            "hidden_size": str(self.hidden_size),
            "inter_size": str(self.inter_size),
            "num_layer": str(self.num_layer),
            "vocab_size": str(self.vocab_size),
            "max_pos_seq_len": str(self.max_pos_seq_len),
            "layernorm_eps": repr(self.layernorm_eps),
            "activation_type": self.activation_type,
            "start_id": str(self.start_id),
            "end_id": str(self.end_id),
            "weight_data_type": self.weight_data_type,
            "rope_theta": repr(self.rope.theta),
        })
        if self.rope.scaling_type:
            d.update({
                "rope_scaling_type": self.rope.scaling_type,
                "rope_scaling_factor": repr(self.rope.scaling_factor),
                "rope_scaling_original_max_position_embeddings": str(self.rope.original_max_pos),
                "rope_scaling_beta_fast": repr(self.rope.beta_fast),
                "rope_scaling_beta_slow": repr(self.rope.beta_slow),
                "rope_scaling_mscale": repr(self.rope.mscale),
                "rope_scaling_mscale_all_dim": repr(self.rope.mscale_all_dim),
            })
        if self.model_type in ("mixtral", "qwen3_moe", "deepseek_moe"):
            d.update({
                "sparse_experts": str(self.sparse_experts),
                "dense_experts": str(self.dense_experts),
                "num_experts_per_tok": str(self.num_experts_per_tok),
                "moe_intermediate_size": str(self.moe_intermediate_size),
                "norm_topk_prob": str(self.norm_topk_prob),
            })
        if self.is_mla:
            d.update({
                "q_lora_rank": str(self.q_lora_rank),
                "kv_lora_rank": str(self.kv_lora_rank),
                "qk_nope_head_dim": str(self.qk_nope_head_dim),
                "qk_rope_head_dim": str(self.qk_rope_head_dim),
                "v_head_dim": str(self.v_head_dim),
                "first_k_dense_replace": str(self.first_k_dense_replace),
                "topk_group": str(self.topk_group),
                "n_group": str(self.n_group),
                "topk_method": self.topk_method,
                "scoring_func": self.scoring_func,
                "routed_scaling_factor": repr(self.routed_scaling_factor),
            })
        if self.do_qk_norm:
            d["do_qk_norm"] = "1"
        if self.model_type == "qwen":
            d.update({"seq_length": str(self.seq_length), "use_logn_attn": str(int(self.use_logn_attn)),
                      "use_dynamic_ntk": str(int(self.use_dynamic_ntk))})
        if extra:
            d.update(extra)
        cp[self.model_type] = d
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.ini"), "w") as f:
            cp.write(f)
