"""Family registry: ``config.ini`` section name -> `FamilySpec`.

The reference instantiates one C++ class per family through a string-keyed factory
(``src/models/model_factory.h:57-114``, table of families ``src/models/*.cpp``).  Here a family is
a row of data consumed by the one generic decoder (`models/decoder.py`).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Dict

from ..config import ModelConfig


@dataclass(frozen=True)
class FamilySpec:
    name: str
    norm: str = "rms"               # rms | layer
    rope: str = "half"              # half | interleaved | 2d | none
    rot_frac: float = 1.0           # rotary dims / head dim (chatglm2+: 0.5)
    qkv_bias: bool = False          # default when no file tells (fake weights)
    dense_bias: bool = False
    mlp: str = "llama"              # llama | gpt | chatglm2 | mixtral | qwen3_moe | deepseek
    embedding: str = "plain"        # plain | gemma | opt
    attention: str = "gqa"          # gqa | mla
    alibi: bool = False             # decided per config for baichuan
    logn_ntk: bool = False          # qwen-1 dynamic NTK + log-n scaling
    telechat_ntk: bool = False      # telechat: NTK base from max(context, training length) + mscale on long inputs
    resid_from_norm: bool = False   # chatglm-1: residual = alpha * normed input
    prefix_lm: bool = False         # chatglm-1 bidirectional prompt
    final_norm: bool = True
    embed_dtype: str = "same"


FAMILIES: Dict[str, FamilySpec] = {
    "llama": FamilySpec("llama"),
    "yarn_llama": FamilySpec("yarn_llama"),
    "gemma": FamilySpec("gemma", embedding="gemma"),
    "qwen": FamilySpec("qwen", qkv_bias=True, logn_ntk=True),
    "qwen2": FamilySpec("qwen2", qkv_bias=True),
    "qwen3": FamilySpec("qwen3"),
    "qwen3_moe": FamilySpec("qwen3_moe", mlp="qwen3_moe"),
    "mixtral": FamilySpec("mixtral", mlp="mixtral"),
    "deepseek_moe": FamilySpec("deepseek_moe", mlp="deepseek", attention="mla", rope="interleaved"),
    "baichuan": FamilySpec("baichuan"),
    "chatglm": FamilySpec("chatglm", norm="layer", rope="2d", qkv_bias=True, dense_bias=True, mlp="gpt",
                          resid_from_norm=True, prefix_lm=True),
    "chatglm2": FamilySpec("chatglm2", rope="interleaved", rot_frac=0.5, qkv_bias=True, mlp="chatglm2"),
    "chatglm3": FamilySpec("chatglm3", rope="interleaved", rot_frac=0.5, qkv_bias=True, mlp="chatglm2"),
    "chatglm4": FamilySpec("chatglm4", rope="interleaved", rot_frac=0.5, qkv_bias=True, mlp="chatglm2"),
    "gpt": FamilySpec("gpt", norm="layer", rope="none", qkv_bias=True, dense_bias=True, mlp="gpt", embedding="opt"),
    "telechat": FamilySpec("telechat", dense_bias=True, telechat_ntk=True),
}


def family_for(cfg: ModelConfig) -> FamilySpec:
    if cfg.model_type not in FAMILIES:
        raise ValueError(f"unsupported model type {cfg.model_type}")
    spec = FAMILIES[cfg.model_type]
    if cfg.model_type == "baichuan" and cfg.max_pos_seq_len <= 0:
        # Baichuan-13B has no rotary table: ALiBi (src/layers/attn_baichuan.h:33-47)
        spec = replace(spec, alibi=True, rope="none")
    return spec


def model_key(cfg: ModelConfig, weight_dtype: str, kv_dtype: str) -> str:
    """The reference's factory key ``"<type>-<weiT>-<kvT>"`` (models.cpp:1022-1033), kept for logs."""
    return f"{cfg.model_type}-{weight_dtype}-{kv_dtype}"
