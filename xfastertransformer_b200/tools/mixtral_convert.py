"""Mixtral converter — reference ``mixtral_convert.py:85-215``: router ``moe.gate.weight.bin`` [hidden, E]; experts
``moe.sparse_experts.<e>.w{1,2,3}.0.bin`` in (gate, up, down) order, i.e. HF w2/w3 swapped."""
from __future__ import annotations

from .llama_convert import LlamaConvert


class MixtralConvert(LlamaConvert):
    SECTION = "mixtral"

    def build_config(self, hf):
        d = super().build_config(hf)
        d.update({"sparse_experts": hf.get("num_local_experts", 8), "num_experts_per_tok": hf.get("num_experts_per_tok", 2)})
        return d

    def write_weights(self, hf, sd):
        def moe(i):
            p, o = f"model.layers.{i}.block_sparse_moe.", f"layers.{i}.moe."
            self.save_linear(o + "gate.weight", sd.get(p + "gate.weight"))
            for e in range(hf.get("num_local_experts", 8)):
                self.save_linear(o + f"sparse_experts.{e}.w1.0", sd.get(p + f"experts.{e}.w1.weight"))     # gate
                self.save_linear(o + f"sparse_experts.{e}.w2.0", sd.get(p + f"experts.{e}.w3.weight"))     # up
                self.save_linear(o + f"sparse_experts.{e}.w3.0", sd.get(p + f"experts.{e}.w2.weight"))     # down
        self.write_llama_style(hf, sd, mlp=moe)
