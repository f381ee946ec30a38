"""Llama-family converters (Llama 1/2/3, Yi, DeepSeek-coder, Gemma, YaRN-Llama) — reference
``src/xfastertransformer/tools/llama_convert.py``, ``yarn_llama_convert.py``.  GPTQ checkpoints (AutoGPTQ int4/int8,
``llama_convert.py:235-434``) are unpacked to int8 / uint4x2 ``qweight`` + fp32 ``scales`` / ``zeros`` with
``zeros = -scale * (qzero + 1 [- 128])``."""
from __future__ import annotations

import configparser
import os

import numpy as np

from .convert import BaseModelConvert, StateDict


class LlamaConvert(BaseModelConvert):
    SECTION = "llama"

    def build_config(self, hf):
        d = self.common_config(hf)
        if d.get("rope_scaling_type") == "llama3":       # handled as plain RoPE with its own theta
            d.pop("rope_scaling_type")
        return d

    def write_weights(self, hf, sd):
        self.write_llama_style(hf, sd)

    # -- GPTQ ------------------------------------------------------------------------------------------------
    def convert_gptq(self, hf, sd: StateDict, output_dir: str) -> str:
        qc = hf.get("quantization_config", {})
        bits = int(qc.get("bits", 4))
        if bits not in (4, 8):
            raise ValueError("GPTQ conversion supports 4 and 8 bits")
        if int(qc.get("group_size", -1)) != -1:
            raise ValueError("Quantization with groupsize is not supported (per-channel only)")
        self.out, self.dtype = output_dir, "fp16"
        ini = self.build_config(hf)
        ini.update({"weight_data_type": "fp16", "quant_qweight_data_type": "int8" if bits == 8 else "uint4",
                    "quant_scales_data_type": "fp32", "quant_zeros_data_type": "fp32", "quant_groupsize": -1})
        cp = configparser.ConfigParser()
        cp[self.SECTION] = {k: str(v) for k, v in ini.items()}
        with open(os.path.join(output_dir, "config.ini"), "w") as f:
            cp.write(f)
        self.save("wte", sd.get("model.embed_tokens.weight"))
        self.save("final_layernorm.weight", sd.get("model.norm.weight"))
        self.save("lm_head.weight", sd.get("lm_head.weight") if "lm_head.weight" in sd else sd.get("model.embed_tokens.weight"))

        def unpack(name):
            """AutoGPTQ: qweight int32 [in/pack, out] packed along in; qzeros int32 [1, out/pack]; scales [1, out]."""
            pack = 32 // bits
            qw = sd.get(name + ".qweight").numpy().astype(np.uint32)
            shifts = (np.arange(pack, dtype=np.uint32) * bits)[None, :, None]
            q = ((qw[:, None, :] >> shifts) & ((1 << bits) - 1)).reshape(-1, qw.shape[1])          # [in, out]
            qz = sd.get(name + ".qzeros").numpy().astype(np.uint32)
            z = ((qz[:, :, None] >> (np.arange(pack, dtype=np.uint32) * bits)[None, None, :]) & ((1 << bits) - 1)).reshape(-1)
            s = sd.get(name + ".scales").float().numpy().reshape(-1)
            # AutoGPTQ stores zero - 1: add the 1 back modulo 2^bits (a true zero point of 0 is stored as all ones)
            z = (z + 1) & ((1 << bits) - 1)
            if bits == 8:
                qi = (q.astype(np.int32) - 128).astype(np.int8)
                zeros = -s * (z.astype(np.float32) - 128)
                return qi, s, zeros
            return q.astype(np.uint8), s, -s * z.astype(np.float32)

        def put(name, parts):
            qs, ss, zs = zip(*parts)
            q = np.concatenate(qs, axis=1)
            if bits == 4:
                q = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)     # low nibble = even column
            q.tofile(os.path.join(output_dir, f"model.{name}.qweight.0.bin"))
            np.concatenate(ss).astype(np.float32).tofile(os.path.join(output_dir, f"model.{name}.scales.0.bin"))
            np.concatenate(zs).astype(np.float32).tofile(os.path.join(output_dir, f"model.{name}.zeros.0.bin"))

        for i in range(hf["num_hidden_layers"]):
            p, o = f"model.layers.{i}.", f"layers.{i}."
            put(o + "attention.query_key_value", [unpack(p + f"self_attn.{n}_proj") for n in "qkv"])
            put(o + "attention.dense", [unpack(p + "self_attn.o_proj")])
            for n in ("gate", "up", "down"):
                put(o + f"mlp.{n}_proj", [unpack(p + f"mlp.{n}_proj")])
            self.save(o + "input_layernorm.weight", sd.get(p + "input_layernorm.weight"))
            self.save(o + "post_attention_layernorm.weight", sd.get(p + "post_attention_layernorm.weight"))
        return output_dir


class YiConvert(LlamaConvert):
    pass


class DeepSeekConvert(LlamaConvert):
    """DeepSeek-coder / DeepSeek-LLM dense models (Llama architecture)."""


class GemmaConvert(LlamaConvert):
    """Gemma stores RMSNorm weights as (w - 1): the converted files hold w + 1 so the engine's norm is plain
    (llama_convert.py:195-196); the section is ``gemma`` (embedding x sqrt(hidden), GELU gate)."""
    SECTION = "gemma"

    def build_config(self, hf):
        d = super().build_config(hf)
        d["activation_type"] = "gelu"
        return d

    def write_weights(self, hf, sd):
        self.write_llama_style(hf, sd, norm_plus_one=True)


class YaRNLlamaConvert(LlamaConvert):
    SECTION = "yarn_llama"

    def build_config(self, hf):
        d = self.common_config(hf)
        d.setdefault("rope_scaling_type", "yarn")
        return d
