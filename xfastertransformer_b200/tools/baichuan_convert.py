"""Baichuan / Baichuan2 converters — reference ``baichuan_convert.py``, ``baichuan2_convert.py``: ``W_pack`` holds
q‖k‖v stacked on the out dimension; the 13B models have no rotary table (``max_pos_seq_len = 0`` selects ALiBi in
the engine); Baichuan2's ``NormHead`` lm_head rows are L2-normalised at conversion."""
from __future__ import annotations

import torch

from .convert import BaseModelConvert


class BaichuanConvert(BaseModelConvert):
    SECTION = "baichuan"
    NORM_HEAD = False

    def build_config(self, hf):
        d = self.common_config(hf)
        alibi = "max_position_embeddings" not in hf or hf.get("num_hidden_layers") == 40
        d["max_pos_seq_len"] = 0 if alibi else hf["max_position_embeddings"]
        d["model_max_length"] = hf.get("model_max_length", 4096)
        return d

    def write_weights(self, hf, sd):
        self.save("wte", sd.get("model.embed_tokens.weight"))
        self.save("final_layernorm.weight", sd.get("model.norm.weight"))
        head = sd.get("lm_head.weight").float()
        if self.NORM_HEAD:
            head = torch.nn.functional.normalize(head)
        self.save("lm_head.weight", head)
        for i in range(hf["num_hidden_layers"]):
            p, o = f"model.layers.{i}.", f"layers.{i}."
            self.save_linear(o + "attention.query_key_value.weight.0", sd.get(p + "self_attn.W_pack.weight"))
            self.save_linear(o + "attention.dense.weight.0", sd.get(p + "self_attn.o_proj.weight"))
            self.save(o + "input_layernorm.weight", sd.get(p + "input_layernorm.weight"))
            self.save(o + "post_attention_layernorm.weight", sd.get(p + "post_attention_layernorm.weight"))
            for n in ("gate", "up", "down"):
                self.save_linear(o + f"mlp.{n}_proj.weight.0", sd.get(p + f"mlp.{n}_proj.weight"))


class Baichuan2Convert(BaichuanConvert):
    NORM_HEAD = True
