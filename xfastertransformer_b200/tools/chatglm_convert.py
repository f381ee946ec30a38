"""ChatGLM converters — reference ``chatglm_convert.py`` (GLM-1: 2-D RoPE, LayerNorm, per-head interleaved
q/k/v), ``chatglm2_convert.py`` / ``chatglm3_convert.py`` / ``chatglm4_convert.py`` (multi-query groups, merged
SwiGLU ``dense_h_to_4h`` = gate‖up, half-dim interleaved RoPE, ``rope_ratio``)."""
from __future__ import annotations


from .convert import BaseModelConvert


class ChatGLM2Convert(BaseModelConvert):
    SECTION = "chatglm2"

    def build_config(self, hf):
        heads, hidden = hf["num_attention_heads"], hf["hidden_size"]
        kv = hf.get("multi_query_group_num", heads) if hf.get("multi_query_attention", False) else heads
        return {"model_name": hf.get("_name_or_path", self.SECTION), "head_num": heads, "kv_head_num": kv,
                "size_per_head": hf.get("kv_channels", hidden // heads), "hidden_size": hidden,
                "inter_size": hf["ffn_hidden_size"], "max_pos_seq_len": hf.get("seq_length", 32768),
                "num_layer": hf["num_layers"], "layernorm_eps": hf.get("layernorm_epsilon", 1e-5),
                "layernorm_type": "pre_layernorm", "activation_type": "swiglu", "has_post_decoder_layernorm": 1,
                "rope_scaling_factor": hf.get("rope_ratio", 1.0), "vocab_size": hf["padded_vocab_size"],
                "start_id": hf.get("bos_token_id", 1) or 1, "end_id": _eos(hf)}

    def write_weights(self, hf, sd):
        self.save("wte", sd.get("transformer.embedding.word_embeddings.weight"))
        self.save("final_layernorm.weight", sd.get("transformer.encoder.final_layernorm.weight"))
        self.save("lm_head.weight", sd.get("transformer.output_layer.weight"))
        for i in range(hf["num_layers"]):
            p, o = f"transformer.encoder.layers.{i}.", f"layers.{i}."
            self.save_linear(o + "attention.query_key_value.weight.0", sd.get(p + "self_attention.query_key_value.weight"))
            if p + "self_attention.query_key_value.bias" in sd:
                self.save(o + "attention.query_key_value.bias.0", sd.get(p + "self_attention.query_key_value.bias"))
            self.save_linear(o + "attention.dense.weight.0", sd.get(p + "self_attention.dense.weight"))
            self.save(o + "input_layernorm.weight", sd.get(p + "input_layernorm.weight"))
            self.save(o + "post_attention_layernorm.weight", sd.get(p + "post_attention_layernorm.weight"))
            self.save_linear(o + "mlp.dense_h_to_4h.weight.0", sd.get(p + "mlp.dense_h_to_4h.weight"))
            self.save_linear(o + "mlp.dense_4h_to_h.weight.0", sd.get(p + "mlp.dense_4h_to_h.weight"))


class ChatGLM3Convert(ChatGLM2Convert):
    SECTION = "chatglm3"


class ChatGLM4Convert(ChatGLM2Convert):
    SECTION = "chatglm4"


class ChatGLMConvert(BaseModelConvert):
    """ChatGLM-6B (v1).  Its fused QKV is laid out [head][q|k|v][dim]; the engine wants q‖k‖v."""
    SECTION = "chatglm"

    def build_config(self, hf):
        heads, hidden = hf["num_attention_heads"], hf["hidden_size"]
        return {"model_name": hf.get("_name_or_path", "chatglm"), "head_num": heads, "kv_head_num": heads,
                "size_per_head": hidden // heads, "hidden_size": hidden, "inter_size": hf.get("inner_hidden_size", 4 * hidden),
                "max_pos_seq_len": hf.get("max_sequence_length", 2048), "num_layer": hf["num_layers"],
                "layernorm_eps": hf.get("layernorm_epsilon", 1e-5), "layernorm_type": "pre_layernorm",
                "activation_type": "gelu", "has_post_decoder_layernorm": 1, "vocab_size": hf["vocab_size"],
                "start_id": hf.get("bos_token_id", 130004), "end_id": hf.get("eos_token_id", 130005)}

    def write_weights(self, hf, sd):
        heads = hf["num_attention_heads"]
        d = hf["hidden_size"] // heads
        self.save("wte", sd.get("transformer.word_embeddings.weight"))
        self.save("final_layernorm.weight", sd.get("transformer.final_layernorm.weight"))
        self.save("final_layernorm.bias", sd.get("transformer.final_layernorm.bias"))
        self.save("lm_head.weight", sd.get("lm_head.weight"))
        for i in range(hf["num_layers"]):
            p, o = f"transformer.layers.{i}.", f"layers.{i}."
            w = sd.get(p + "attention.query_key_value.weight").view(heads, 3, d, -1)
            b = sd.get(p + "attention.query_key_value.bias").view(heads, 3, d)
            self.save_linear(o + "attention.query_key_value.weight.0", w.permute(1, 0, 2, 3).reshape(3 * heads * d, -1))
            self.save(o + "attention.query_key_value.bias.0", b.permute(1, 0, 2).reshape(-1))
            self.save_linear(o + "attention.dense.weight.0", sd.get(p + "attention.dense.weight"))
            self.save(o + "attention.dense.bias", sd.get(p + "attention.dense.bias"))
            for n in ("input_layernorm", "post_attention_layernorm"):
                self.save(o + n + ".weight", sd.get(p + n + ".weight"))
                self.save(o + n + ".bias", sd.get(p + n + ".bias"))
            self.save_linear(o + "mlp.dense_h_to_4h.weight.0", sd.get(p + "mlp.dense_h_to_4h.weight"))
            self.save(o + "mlp.dense_h_to_4h.bias.0", sd.get(p + "mlp.dense_h_to_4h.bias"))
            self.save_linear(o + "mlp.dense_4h_to_h.weight.0", sd.get(p + "mlp.dense_4h_to_h.weight"))
            self.save(o + "mlp.dense_4h_to_h.bias", sd.get(p + "mlp.dense_4h_to_h.bias"))


def _eos(hf):
    e = hf.get("eos_token_id", 2)
    return e[0] if isinstance(e, (list, tuple)) else e
