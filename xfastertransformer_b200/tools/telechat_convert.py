"""TeleChat converter — reference ``telechat_convert.py``: separate ``query`` and per-head interleaved
``key_value`` projections, biased ``dense`` / ``down_proj``."""
from __future__ import annotations

import torch

from .convert import BaseModelConvert


class TelechatConvert(BaseModelConvert):
    SECTION = "telechat"

    def build_config(self, hf):
        heads = hf.get("n_head", hf.get("num_attention_heads"))
        hidden = hf["hidden_size"]
        return {"model_name": hf.get("_name_or_path", "telechat"), "head_num": heads, "kv_head_num": heads,
                "size_per_head": hidden // heads, "hidden_size": hidden, "inter_size": hf["ffn_hidden_size"],
                "max_pos_seq_len": hf.get("seq_length", hf.get("training_seqlen", 8192)),
                "num_layer": hf.get("n_layer", hf.get("num_hidden_layers")),
                "layernorm_eps": hf.get("layer_norm_epsilon", 1e-5), "layernorm_type": "pre_layernorm",
                "activation_type": "silu", "has_post_decoder_layernorm": 1, "vocab_size": hf["vocab_size"],
                "start_id": hf.get("bos_token_id", 1), "end_id": hf.get("eos_token_id", 2)}

    def write_weights(self, hf, sd):
        heads = hf.get("n_head", hf.get("num_attention_heads"))
        d = hf["hidden_size"] // heads
        L = hf.get("n_layer", hf.get("num_hidden_layers"))
        self.save("wte", sd.get("transformer.word_embeddings.weight"))
        self.save("final_layernorm.weight", sd.get("transformer.ln_f.weight"))
        self.save("lm_head.weight", sd.get("lm_head.weight") if "lm_head.weight" in sd else sd.get("transformer.word_embeddings.weight"))
        for i in range(L):
            p, o = f"transformer.h.{i}.", f"layers.{i}."
            q = sd.get(p + "self_attention.query.weight")
            kv = sd.get(p + "self_attention.key_value.weight").view(heads, 2, d, -1)
            k, v = kv[:, 0].reshape(heads * d, -1), kv[:, 1].reshape(heads * d, -1)
            self.save_linear(o + "attention.query_key_value.weight.0", torch.cat([q, k, v], 0))
            self.save_linear(o + "attention.dense.weight.0", sd.get(p + "self_attention.dense.weight"))
            self.save(o + "attention.dense.bias", sd.get(p + "self_attention.dense.bias"))
            self.save(o + "input_layernorm.weight", sd.get(p + "input_layernorm.weight"))
            self.save(o + "post_attention_layernorm.weight", sd.get(p + "post_attention_layernorm.weight"))
            for n in ("gate", "up", "down"):
                self.save_linear(o + f"mlp.{n}_proj.weight.0", sd.get(p + f"mlp.{n}_proj.weight"))
            if p + "mlp.down_proj.bias" in sd:
                self.save(o + "mlp.down_proj.bias.0", sd.get(p + "mlp.down_proj.bias"))
