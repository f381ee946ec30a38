"""DeepSeek-V2 / V3 / R1 converters — reference ``deepseek_moe_convert.py:31-375``.  dtype ``bf16`` writes bf16
projections; ``fp8_e4m3`` keeps the checkpoint's native e4m3 weights (``weight_block_size == [128, 128]``) and
writes each ``weight_scale_inv`` as fp32 ``[ceil(in/128), ceil(out/128)]`` (transposed like the weight).  Embedding,
lm_head, all norms, the router weight and ``e_score_correction_bias`` are always bf16; no ``.0`` suffix."""
from __future__ import annotations

import torch

from ..ops import reference as R
from .convert import BaseModelConvert


class DeepSeekV2Convert(BaseModelConvert):
    SECTION = "deepseek_moe"
    SUPPORTED_DTYPES = ("bf16", "fp8_e4m3")

    def __init__(self):
        super().__init__()
        self.default_dtype = "bf16"

    def build_config(self, hf):
        d = self.common_config(hf)
        d.update({
            "size_per_head": hf.get("v_head_dim", 128), "attn_params_type": "MLAttnParams",
            "ffn_params_type": "DeepSeekFFNParams", "q_lora_rank": hf.get("q_lora_rank") or 0,
            "kv_lora_rank": hf["kv_lora_rank"], "qk_rope_head_dim": hf["qk_rope_head_dim"],
            "v_head_dim": hf["v_head_dim"], "qk_nope_head_dim": hf["qk_nope_head_dim"],
            "moe_intermediate_size": hf["moe_intermediate_size"], "first_k_dense_replace": hf.get("first_k_dense_replace", 0),
            "dense_experts": hf.get("n_shared_experts") or 0, "sparse_experts": hf["n_routed_experts"],
            "routed_scaling_factor": hf.get("routed_scaling_factor", 1.0), "topk_method": hf.get("topk_method", "greedy"),
            "n_group": hf.get("n_group") or 1, "topk_group": hf.get("topk_group") or 1,
            "num_experts_per_tok": hf["num_experts_per_tok"], "norm_topk_prob": bool(hf.get("norm_topk_prob", False)),
            "scoring_func": hf.get("scoring_func", "softmax"),
        })
        if self.dtype == "fp8_e4m3":
            q = hf.get("quantization_config", {})
            if q and list(q.get("weight_block_size", [128, 128])) != [128, 128]:
                raise ValueError("fp8 conversion expects weight_block_size == [128, 128]")
        return d

    def convert(self, input_dir, output_dir=None, dtype=None, processes=8, from_quantized_model=None):
        self.dtype = dtype or self.default_dtype
        return super().convert(input_dir, output_dir, dtype or self.default_dtype, processes, None)

    def _proj(self, name, src, sd):
        """One projection: fp8 (+scale) or bf16 [in, out]."""
        w = sd.get(src + ".weight")
        has_scale = (src + ".weight_scale_inv") in sd
        if self.dtype == "fp8_e4m3":
            if has_scale and w.dtype == torch.float8_e4m3fn:
                q, s = w, sd.get(src + ".weight_scale_inv").float()
            else:
                q, s = R.quantize_fp8_block(w.float())
            self.save(name + ".weight", q.view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn), "fp8_e4m3")
            self.save(name + ".weight_scale_inv", s.t().contiguous(), "fp32")
        else:
            if has_scale and w.dtype == torch.float8_e4m3fn:
                from ..runtime.loader import LinearWeight
                w = R.dequant_weight(LinearWeight("fp8", w, sd.get(src + ".weight_scale_inv").float(),
                                                  in_features=w.shape[1], out_features=w.shape[0]))
            self.save(name + ".weight", w.t().contiguous(), "bf16")

    def write_weights(self, hf, sd):
        bf = "bf16"
        self.save("wte", sd.get("model.embed_tokens.weight"), bf)
        self.save("final_layernorm.weight", sd.get("model.norm.weight"), bf)
        self.save("lm_head.weight", sd.get("lm_head.weight") if "lm_head.weight" in sd else sd.get("model.embed_tokens.weight"), bf)
        for i in range(hf["num_hidden_layers"]):
            p, o = f"model.layers.{i}.", f"layers.{i}."
            self.save(o + "input_layernorm.weight", sd.get(p + "input_layernorm.weight"), bf)
            self.save(o + "post_attention_layernorm.weight", sd.get(p + "post_attention_layernorm.weight"), bf)
            if hf.get("q_lora_rank"):
                self._proj(o + "self_attn.q_a_proj", p + "self_attn.q_a_proj", sd)
                self.save(o + "self_attn.q_a_layernorm.weight", sd.get(p + "self_attn.q_a_layernorm.weight"), bf)
                self._proj(o + "self_attn.q_b_proj", p + "self_attn.q_b_proj", sd)
            else:
                self._proj(o + "self_attn.q_a_proj", p + "self_attn.q_proj", sd)
            self._proj(o + "self_attn.kv_a_proj_with_mqa", p + "self_attn.kv_a_proj_with_mqa", sd)
            self.save(o + "self_attn.kv_a_layernorm.weight", sd.get(p + "self_attn.kv_a_layernorm.weight"), bf)
            self._proj(o + "self_attn.kv_b_proj", p + "self_attn.kv_b_proj", sd)
            self._proj(o + "attention.dense", p + "self_attn.o_proj", sd)
            if i < hf.get("first_k_dense_replace", 0):
                for n in ("gate", "up", "down"):
                    self._proj(o + f"mlp.{n}_proj", p + f"mlp.{n}_proj", sd)
                continue
            self.save(o + "mlp.gate.weight", sd.get(p + "mlp.gate.weight").t().contiguous(), bf)
            if p + "mlp.gate.e_score_correction_bias" in sd:
                self.save(o + "mlp.gate.e_score_correction_bias", sd.get(p + "mlp.gate.e_score_correction_bias"), bf)
            if hf.get("n_shared_experts"):
                for n in ("gate", "up", "down"):
                    self._proj(o + f"mlp.shared_experts.{n}_proj", p + f"mlp.shared_experts.{n}_proj", sd)
            for e in range(hf["n_routed_experts"]):
                for n in ("gate", "up", "down"):
                    self._proj(o + f"mlp.experts.{e}.{n}_proj", p + f"mlp.experts.{e}.{n}_proj", sd)


class DeepSeekV3Convert(DeepSeekV2Convert):
    pass


class DeepSeekR1Convert(DeepSeekV2Convert):
    pass
