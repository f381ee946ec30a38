"""Qwen converters — reference ``qwen_convert.py`` (Qwen-1: c_attn / w1 / w2 naming, dynamic NTK + log-n flags),
``qwen2_convert.py`` (Llama layout + QKV bias), ``qwen3_convert.py`` (per-head q/k norm; dense and MoE)."""
from __future__ import annotations


from .convert import BaseModelConvert
from .llama_convert import LlamaConvert


class Qwen2Convert(LlamaConvert):
    SECTION = "qwen2"


class Qwen3Convert(LlamaConvert):
    SECTION = "qwen3"

    def build_config(self, hf):
        d = super().build_config(hf)
        d["do_qk_norm"] = 1
        if hf.get("num_experts"):
            d.update({"sparse_experts": hf["num_experts"], "num_experts_per_tok": hf["num_experts_per_tok"],
                      "moe_intermediate_size": hf["moe_intermediate_size"], "inter_size": hf["moe_intermediate_size"],
                      "norm_topk_prob": int(bool(hf.get("norm_topk_prob", True)))})
        return d

    def convert(self, input_dir, output_dir=None, dtype=None, processes=8, from_quantized_model=None):
        import json, os
        with open(os.path.join(input_dir, "config.json")) as f:
            self.SECTION = "qwen3_moe" if json.load(f).get("num_experts") else "qwen3"
        return super().convert(input_dir, output_dir, dtype, processes, from_quantized_model)

    def write_weights(self, hf, sd):
        if not hf.get("num_experts"):
            return self.write_llama_style(hf, sd, qk_norm=True)

        def moe(i):
            p, o = f"model.layers.{i}.", f"layers.{i}."
            self.save_linear(o + "mlp.gate.weight.0", sd.get(p + "mlp.gate.weight"))
            for e in range(hf["num_experts"]):
                for n in ("gate", "up", "down"):
                    self.save_linear(o + f"mlp.experts.{e}.{n}_proj.weight.0", sd.get(p + f"mlp.experts.{e}.{n}_proj.weight"))
        self.write_llama_style(hf, sd, qk_norm=True, mlp=moe)


class QwenConvert(BaseModelConvert):
    """Qwen-1 (``transformer.h.N.attn.c_attn`` ...): MLP is c_proj(w1(x) * silu(w2(x))), i.e. gate = w2, up = w1."""
    SECTION = "qwen"

    def build_config(self, hf):
        heads = hf["num_attention_heads"]
        hidden = hf["hidden_size"]
        return {"model_name": hf.get("_name_or_path", "qwen"), "head_num": heads, "kv_head_num": heads,
                "size_per_head": hf.get("kv_channels", hidden // heads), "hidden_size": hidden,
                "inter_size": hf["intermediate_size"] // 2, "max_pos_seq_len": hf.get("max_position_embeddings", 8192),
                "seq_length": hf.get("seq_length", 8192), "num_layer": hf["num_hidden_layers"],
                "layernorm_eps": hf.get("layer_norm_epsilon", 1e-6), "layernorm_type": "pre_layernorm",
                "activation_type": "silu", "rope_theta": hf.get("rotary_emb_base", 10000),
                "use_logn_attn": int(bool(hf.get("use_logn_attn", True))),
                "use_dynamic_ntk": int(bool(hf.get("use_dynamic_ntk", True))), "has_post_decoder_layernorm": 1,
                "vocab_size": hf["vocab_size"], "start_id": 151643, "end_id": 151643}

    def write_weights(self, hf, sd):
        self.save("wte", sd.get("transformer.wte.weight"))
        self.save("final_layernorm.weight", sd.get("transformer.ln_f.weight"))
        self.save("lm_head.weight", sd.get("lm_head.weight"))
        for i in range(hf["num_hidden_layers"]):
            p, o = f"transformer.h.{i}.", f"layers.{i}."
            self.save_linear(o + "attention.query_key_value.weight.0", sd.get(p + "attn.c_attn.weight"))
            self.save(o + "attention.query_key_value.bias.0", sd.get(p + "attn.c_attn.bias"))
            self.save_linear(o + "attention.dense.weight.0", sd.get(p + "attn.c_proj.weight"))
            self.save(o + "input_layernorm.weight", sd.get(p + "ln_1.weight"))
            self.save(o + "post_attention_layernorm.weight", sd.get(p + "ln_2.weight"))
            self.save_linear(o + "mlp.gate_proj.weight.0", sd.get(p + "mlp.w2.weight"))
            self.save_linear(o + "mlp.up_proj.weight.0", sd.get(p + "mlp.w1.weight"))
            self.save_linear(o + "mlp.down_proj.weight.0", sd.get(p + "mlp.c_proj.weight"))
