"""OPT converter — reference ``opt_convert.py``: section ``gpt``; learned positions (``model.wpe.bin``, offset 2),
LayerNorm with bias, ReLU FFN as ``mlp.dense_h_to_4h`` / ``mlp.dense_4h_to_h``."""
from __future__ import annotations

import torch

from .convert import BaseModelConvert


class OPTConvert(BaseModelConvert):
    SECTION = "gpt"

    def build_config(self, hf):
        heads, hidden = hf["num_attention_heads"], hf["hidden_size"]
        return {"model_name": hf.get("_name_or_path", "opt"), "head_num": heads, "kv_head_num": heads,
                "size_per_head": hidden // heads, "hidden_size": hidden, "inter_size": hf["ffn_dim"],
                "max_pos_seq_len": hf["max_position_embeddings"], "num_layer": hf["num_hidden_layers"],
                "layernorm_eps": 1e-5, "layernorm_type": "pre_layernorm", "activation_type": hf.get("activation_function", "relu"),
                "has_post_decoder_layernorm": 1, "vocab_size": hf["vocab_size"], "start_id": hf.get("bos_token_id", 2),
                "end_id": hf.get("eos_token_id", 2)}

    def write_weights(self, hf, sd):
        pre = "model.decoder." if "model.decoder.embed_tokens.weight" in sd else "decoder."
        emb = sd.get(pre + "embed_tokens.weight")
        self.save("wte", emb)
        self.save("wpe", sd.get(pre + "embed_positions.weight"))
        self.save("final_layernorm.weight", sd.get(pre + "final_layer_norm.weight"))
        self.save("final_layernorm.bias", sd.get(pre + "final_layer_norm.bias"))
        self.save("lm_head.weight", sd.get("lm_head.weight") if "lm_head.weight" in sd else emb)
        for i in range(hf["num_hidden_layers"]):
            p, o = f"{pre}layers.{i}.", f"layers.{i}."
            self.save_linear(o + "attention.query_key_value.weight.0",
                             torch.cat([sd.get(p + f"self_attn.{n}_proj.weight") for n in "qkv"], 0))
            self.save(o + "attention.query_key_value.bias.0", torch.cat([sd.get(p + f"self_attn.{n}_proj.bias") for n in "qkv"], 0))
            self.save_linear(o + "attention.dense.weight.0", sd.get(p + "self_attn.out_proj.weight"))
            self.save(o + "attention.dense.bias", sd.get(p + "self_attn.out_proj.bias"))
            self.save(o + "input_layernorm.weight", sd.get(p + "self_attn_layer_norm.weight"))
            self.save(o + "input_layernorm.bias", sd.get(p + "self_attn_layer_norm.bias"))
            self.save(o + "post_attention_layernorm.weight", sd.get(p + "final_layer_norm.weight"))
            self.save(o + "post_attention_layernorm.bias", sd.get(p + "final_layer_norm.bias"))
            self.save_linear(o + "mlp.dense_h_to_4h.weight.0", sd.get(p + "fc1.weight"))
            self.save(o + "mlp.dense_h_to_4h.bias.0", sd.get(p + "fc1.bias"))
            self.save_linear(o + "mlp.dense_4h_to_h.weight.0", sd.get(p + "fc2.weight"))
            self.save(o + "mlp.dense_4h_to_h.bias", sd.get(p + "fc2.bias"))
