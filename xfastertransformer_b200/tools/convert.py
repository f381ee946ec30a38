"""HuggingFace checkpoint -> converted model directory (config.ini + per-tensor .bin files).

Same output contract as the reference's converters (``src/xfastertransformer/tools/convert.py:108-170`` and the
per-family files: ``llama_convert.py``, ``qwen2_convert.py``, ``qwen3_convert.py``, ``mixtral_convert.py``,
``opt_convert.py``, ``chatglm*_convert.py``, ``baichuan*_convert.py``, ``telechat_convert.py``,
``deepseek_moe_convert.py``): one section in config.ini named after the model type, linear weights stored
transposed ``[in, out]``, q/k/v merged into ``attention.query_key_value.weight.0.bin``, the vestigial ``.0``
suffix on split-able tensors.

Unlike the reference, which instantiates each model through ``AutoModelForCausalLM`` (and therefore needs the
model's remote code for ChatGLM / Baichuan / Qwen-1 / TeleChat), this converter reads ``config.json`` and the
``*.safetensors`` / ``*.bin`` shards directly and maps parameter names, so it needs only the files.
"""
from __future__ import annotations

import configparser
import glob
import json
import os
from typing import Callable, Dict, Iterator, Optional

import torch

from ..runtime.loader import write_bin


class StateDict:
    """Lazy view over the tensors of a HF checkpoint directory (safetensors preferred, torch .bin otherwise)."""

    def __init__(self, path: str):
        self.path = path
        self._where: Dict[str, str] = {}
        self._open = {}
        st = sorted(glob.glob(os.path.join(path, "*.safetensors")))
        if st:
            from safetensors import safe_open
            for f in st:
                h = safe_open(f, framework="pt")
                self._open[f] = h
                for k in h.keys():
                    self._where[k] = f
            self.kind = "safetensors"
        else:
            bins = sorted(glob.glob(os.path.join(path, "pytorch_model*.bin")))
            if not bins:
                raise FileNotFoundError(f"no *.safetensors or pytorch_model*.bin under {path}")
            self._sd = {}
            for f in bins:
                self._sd.update(torch.load(f, map_location="cpu", weights_only=True))
            self._where = {k: "bin" for k in self._sd}
            self.kind = "bin"

    def __contains__(self, k: str) -> bool:
        return k in self._where

    def keys(self) -> Iterator[str]:
        return iter(self._where)

    def get(self, k: str) -> torch.Tensor:
        if k not in self._where:
            raise KeyError(f"{k} not in checkpoint {self.path}")
        if self.kind == "safetensors":
            return self._open[self._where[k]].get_tensor(k)
        return self._sd[k]


class BaseModelConvert:
    """``Convert().convert(input_dir, output_dir=None, dtype="fp16", processes=8)``."""

    SECTION = "llama"
    SUPPORTED_DTYPES = ("fp16", "bf16", "fp32")

    def __init__(self):
        self.default_dtype = "fp16"

    # -- public entry point (reference: BaseModelConvert.convert, convert.py:140-170) -------------------------
    def convert(self, input_dir: str, output_dir: Optional[str] = None, dtype: Optional[str] = None, processes: int = 8,
                from_quantized_model: Optional[str] = None) -> str:
        dtype = dtype or self.default_dtype
        if dtype not in self.SUPPORTED_DTYPES:
            raise ValueError(f"{type(self).__name__} supports {self.SUPPORTED_DTYPES}, got {dtype}")
        if output_dir is None:
            output_dir = input_dir.rstrip("/") + "-xft"
        os.makedirs(output_dir, exist_ok=True)
        with open(os.path.join(input_dir, "config.json")) as f:
            hf = json.load(f)
        sd = StateDict(input_dir)
        if from_quantized_model == "gptq" or "quantization_config" in hf and hf["quantization_config"].get("quant_method") == "gptq":
            return self.convert_gptq(hf, sd, output_dir)
        self.dtype = dtype
        self.out = output_dir
        ini = self.build_config(hf)
        ini["weight_data_type"] = dtype
        cp = configparser.ConfigParser()
        cp[self.SECTION] = {k: str(v) for k, v in ini.items()}
        with open(os.path.join(output_dir, "config.ini"), "w") as f:
            cp.write(f)
        self.write_weights(hf, sd)
        return output_dir

    # -- helpers ------------------------------------------------------------------------------------------------
    def save(self, name: str, t: torch.Tensor, dtype: Optional[str] = None) -> None:
        if not name.startswith("model."):
            name = "model." + name
        write_bin(os.path.join(self.out, name + ".bin"), t.float() if (dtype or self.dtype) != "bf16" else t, dtype or self.dtype)

    def save_linear(self, name: str, w_out_in: torch.Tensor, dtype: Optional[str] = None) -> None:
        """HF nn.Linear weight [out, in] -> file [in, out]."""
        self.save(name, w_out_in.t().contiguous(), dtype)

    def common_config(self, hf: dict) -> dict:
        heads = hf["num_attention_heads"]
        hidden = hf["hidden_size"]
        d = {
            "model_name": hf.get("_name_or_path", self.SECTION) or self.SECTION,
            "head_num": heads,
            "kv_head_num": hf.get("num_key_value_heads", heads),
            "hidden_size": hidden,
            "size_per_head": hf.get("head_dim") or hidden // heads,
            "inter_size": hf.get("intermediate_size", 4 * hidden),
            "max_pos_seq_len": hf.get("max_position_embeddings", 2048),
            "num_layer": hf["num_hidden_layers"],
            "layernorm_eps": hf.get("rms_norm_eps", hf.get("layer_norm_epsilon", hf.get("layernorm_epsilon", 1e-6))),
            "layernorm_type": "pre_layernorm",
            "activation_type": hf.get("hidden_act", hf.get("hidden_activation", "silu")) or "silu",
            "rope_theta": hf.get("rope_theta", 10000),
            "has_post_decoder_layernorm": 1,
            "vocab_size": hf["vocab_size"],
            "start_id": hf.get("bos_token_id", 0) if hf.get("bos_token_id") is not None else 0,
            "end_id": _first(hf.get("eos_token_id", 0)),
            "pad_id": hf.get("pad_token_id") if hf.get("pad_token_id") is not None else -1,
        }
        rs = hf.get("rope_scaling") or hf.get("rope_parameters") or None
        if isinstance(rs, dict) and (rs.get("type") or rs.get("rope_type")) not in (None, "default"):
            d["rope_scaling_type"] = rs.get("type") or rs.get("rope_type")
            d["rope_scaling_factor"] = rs.get("factor", 1.0)
            for k_src, k_dst in (("original_max_position_embeddings", "rope_scaling_original_max_position_embeddings"),
                                 ("beta_fast", "rope_scaling_beta_fast"), ("beta_slow", "rope_scaling_beta_slow"),
                                 ("mscale", "rope_scaling_mscale"), ("mscale_all_dim", "rope_scaling_mscale_all_dim")):
                if k_src in rs:
                    d[k_dst] = rs[k_src]
        if isinstance(rs, dict) and "rope_theta" in rs:
            d["rope_theta"] = rs["rope_theta"]
        return d

    def build_config(self, hf: dict) -> dict:
        return self.common_config(hf)

    def write_weights(self, hf: dict, sd: StateDict) -> None:
        raise NotImplementedError

    def convert_gptq(self, hf: dict, sd: StateDict, output_dir: str) -> str:
        raise NotImplementedError(f"{type(self).__name__} has no GPTQ path")

    # shared by the llama-style families
    def write_llama_style(self, hf: dict, sd: StateDict, prefix: str = "model.", norm_plus_one: bool = False,
                          qk_norm: bool = False, mlp: Optional[Callable[[int], None]] = None) -> None:
        L = hf["num_hidden_layers"]
        emb = sd.get(prefix + "embed_tokens.weight")
        self.save("wte", emb)
        nw = lambda t: (t.float() + 1.0) if norm_plus_one else t
        self.save("final_layernorm.weight", nw(sd.get(prefix + "norm.weight")))
        head = sd.get("lm_head.weight") if "lm_head.weight" in sd else emb       # tied embeddings
        self.save("lm_head.weight", head)
        for i in range(L):
            p = f"{prefix}layers.{i}."
            o = f"layers.{i}."
            q, k, v = (sd.get(p + f"self_attn.{n}_proj.weight") for n in "qkv")
            self.save_linear(o + "attention.query_key_value.weight.0", torch.cat([q, k, v], 0))
            if p + "self_attn.q_proj.bias" in sd:
                self.save(o + "attention.query_key_value.bias.0",
                          torch.cat([sd.get(p + f"self_attn.{n}_proj.bias") for n in "qkv"], 0))
            self.save_linear(o + "attention.dense.weight.0", sd.get(p + "self_attn.o_proj.weight"))
            if p + "self_attn.o_proj.bias" in sd:
                self.save(o + "attention.dense.bias", sd.get(p + "self_attn.o_proj.bias"))
            self.save(o + "input_layernorm.weight", nw(sd.get(p + "input_layernorm.weight")))
            self.save(o + "post_attention_layernorm.weight", nw(sd.get(p + "post_attention_layernorm.weight")))
            if qk_norm:
                self.save(o + "attention.q_norm.weight", sd.get(p + "self_attn.q_norm.weight"))
                self.save(o + "attention.k_norm.weight", sd.get(p + "self_attn.k_norm.weight"))
            if mlp is not None:
                mlp(i)
            else:
                for n in ("gate", "up", "down"):
                    self.save_linear(o + f"mlp.{n}_proj.weight.0", sd.get(p + f"mlp.{n}_proj.weight"))


def _first(v):
    if isinstance(v, (list, tuple)):
        return v[0] if v else 0
    return 0 if v is None else v
