"""Synthetic checkpoints in the converted-model layout (config.ini + .bin), for tests and
benchmarks: random N(0, std) weights of a named architecture, written exactly where the
converters of the reference put them (``src/xfastertransformer/tools/llama_convert.py:177-233``,
``mixtral_convert.py:196-215``, ``qwen3_convert.py:120-160``, ``deepseek_moe_convert.py:182-375``,
``opt_convert.py``, ``chatglm2_convert.py``).

`config_only(path, cfg)` writes just config.ini: together with ``XFT_FAKE_MODEL=2`` the engine
draws the weights on the device, which is how the large benchmark configs are built.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from ..config import ModelConfig, RopeConfig
from ..ops import reference as R
from ..runtime.loader import write_bin

PRESETS: Dict[str, dict] = {
    # BASELINE configs
    "tiny-llama": dict(model_type="llama", num_layer=2, hidden_size=256, head_num=4, kv_head_num=4, size_per_head=64,
                       inter_size=688, vocab_size=32000, max_pos_seq_len=2048, layernorm_eps=1e-6),
    "llama-2-7b": dict(model_type="llama", num_layer=32, hidden_size=4096, head_num=32, kv_head_num=32,
                       size_per_head=128, inter_size=11008, vocab_size=32000, max_pos_seq_len=4096),
    "llama-2-70b": dict(model_type="llama", num_layer=80, hidden_size=8192, head_num=64, kv_head_num=8,
                        size_per_head=128, inter_size=28672, vocab_size=32000, max_pos_seq_len=4096),
    # one tensor-parallel rank's share of Llama-2-70B at TP=8 (8 q heads + 1 kv head, FFN slice 3584, vocab slice
    # 4000) as a stand-alone model: isolates per-GPU kernel time from communication when profiling on one GPU
    "llama-2-70b-tp8-slice": dict(model_type="llama", num_layer=80, hidden_size=8192, head_num=8, kv_head_num=1,
                                  size_per_head=128, inter_size=3584, vocab_size=4000, max_pos_seq_len=4096),
    "mixtral-8x7b": dict(model_type="mixtral", num_layer=32, hidden_size=4096, head_num=32, kv_head_num=8,
                         size_per_head=128, inter_size=14336, vocab_size=32000, max_pos_seq_len=32768,
                         sparse_experts=8, num_experts_per_tok=2, rope=RopeConfig(theta=1e6)),
    "deepseek-v3": dict(model_type="deepseek_moe", num_layer=61, hidden_size=7168, head_num=128, kv_head_num=128,
                        size_per_head=128, inter_size=18432, vocab_size=129280, max_pos_seq_len=163840,
                        q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                        moe_intermediate_size=2048, first_k_dense_replace=3, dense_experts=1, sparse_experts=256,
                        routed_scaling_factor=2.5, topk_method="noaux_tc", n_group=8, topk_group=4,
                        num_experts_per_tok=8, norm_topk_prob=True, scoring_func="sigmoid",
                        weight_data_type="fp8_e4m3",
                        rope=RopeConfig(theta=10000, scaling_type="yarn", scaling_factor=40, original_max_pos=4096,
                                        beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0)),
}


def preset(name: str, **over) -> ModelConfig:
    if name not in PRESETS:
        from .model_zoo import ZOO          # public model architectures (examples/model_config)
        if name not in ZOO:
            raise KeyError(f"unknown model preset '{name}'; known: {sorted(set(PRESETS) | set(ZOO))}")
        d = dict(ZOO[name])
    else:
        d = dict(PRESETS[name])
    d.update(over)
    d.setdefault("activation_type", "silu")
    d.setdefault("weight_data_type", "bf16")
    d.setdefault("start_id", 1)
    d.setdefault("end_id", 2)
    return ModelConfig(**d)


def config_only(path: str, cfg: ModelConfig) -> str:
    cfg.to_ini(path)
    return path


def write_synthetic_checkpoint(path: str, cfg: ModelConfig, seed: int = 0, std: float = 0.02,
                               dtype: Optional[str] = None) -> str:
    """Write config.ini and every tensor.  Linear weights are drawn in HF orientation [out,in]
    in fp32, rounded to `dtype`, and stored transposed ([in,out]) like the converters do."""
    dtype = dtype or cfg.weight_data_type
    os.makedirs(path, exist_ok=True)
    cfg.weight_data_type = dtype
    cfg.to_ini(path)
    g = torch.Generator().manual_seed(seed)
    H, D = cfg.hidden_size, cfg.size_per_head
    mt = cfg.model_type

    def rnd(*shape, s=std):
        return torch.randn(*shape, generator=g) * s

    def put(name, t, dt=None):
        write_bin(os.path.join(path, name), t, dt or dtype)

    def put_lin(name, out_f, in_f, dt=None):
        """HF weight [out,in] -> file [in,out]."""
        put(name, rnd(out_f, in_f).t().contiguous(), dt)

    def put_fp8_lin(base, out_f, in_f):
        w = rnd(out_f, in_f)
        if dtype == "fp8_e4m3":
            q, s = R.quantize_fp8_block(w)              # [out,in], [out/128,in/128]
            put(base + ".weight.bin", q.view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn), "fp8_e4m3")
            put(base + ".weight_scale_inv.bin", s.t().contiguous(), "fp32")
        else:
            put(base + ".weight.bin", w.t().contiguous(), dtype)

    norm_dt = "bf16" if mt == "deepseek_moe" else dtype
    emb_dt = "bf16" if mt == "deepseek_moe" else dtype
    put("model.wte.bin", rnd(cfg.vocab_size, H), emb_dt)
    put("model.final_layernorm.weight.bin", 1.0 + rnd(H, s=0.05), norm_dt)
    put("model.lm_head.weight.bin", rnd(cfg.vocab_size, H), emb_dt)
    layer_norm = mt in ("gpt", "chatglm")
    if layer_norm:
        put("model.final_layernorm.bias.bin", rnd(H, s=0.05))
    if mt == "gpt":
        put("model.wpe.bin", rnd(cfg.max_pos_seq_len + 2, H))
    for i in range(cfg.num_layer):
        p = f"model.layers.{i}."
        put(p + "input_layernorm.weight.bin", 1.0 + rnd(H, s=0.05), norm_dt)
        put(p + "post_attention_layernorm.weight.bin", 1.0 + rnd(H, s=0.05), norm_dt)
        if layer_norm:
            put(p + "input_layernorm.bias.bin", rnd(H, s=0.05))
            put(p + "post_attention_layernorm.bias.bin", rnd(H, s=0.05))
        if mt == "deepseek_moe":
            nope, rope, vd = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
            kvl, ql, nh = cfg.kv_lora_rank, cfg.q_lora_rank, cfg.head_num
            if ql > 0:
                put_fp8_lin(p + "self_attn.q_a_proj", ql, H)
                put(p + "self_attn.q_a_layernorm.weight.bin", 1.0 + rnd(ql, s=0.05), "bf16")
                put_fp8_lin(p + "self_attn.q_b_proj", nh * (nope + rope), ql)
            else:
                put_fp8_lin(p + "self_attn.q_a_proj", nh * (nope + rope), H)
            put_fp8_lin(p + "self_attn.kv_a_proj_with_mqa", kvl + rope, H)
            put(p + "self_attn.kv_a_layernorm.weight.bin", 1.0 + rnd(kvl, s=0.05), "bf16")
            put_fp8_lin(p + "self_attn.kv_b_proj", nh * (nope + vd), kvl)
            put_fp8_lin(p + "attention.dense", H, nh * vd)
            if i < cfg.first_k_dense_replace:
                for n, (o, k) in dict(gate=(cfg.inter_size, H), up=(cfg.inter_size, H), down=(H, cfg.inter_size)).items():
                    put_fp8_lin(p + f"mlp.{n}_proj", o, k)
            else:
                E, I = cfg.sparse_experts, cfg.moe_intermediate_size
                put(p + "mlp.gate.weight.bin", rnd(E, H, s=0.5).t().contiguous(), "bf16")
                if cfg.topk_method == "noaux_tc":
                    put(p + "mlp.gate.e_score_correction_bias.bin", rnd(E, s=0.1), "bf16")
                SI = cfg.dense_experts * I
                if SI:
                    for n, (o, k) in dict(gate=(SI, H), up=(SI, H), down=(H, SI)).items():
                        put_fp8_lin(p + f"mlp.shared_experts.{n}_proj", o, k)
                for e in range(E):
                    for n, (o, k) in dict(gate=(I, H), up=(I, H), down=(H, I)).items():
                        put_fp8_lin(p + f"mlp.experts.{e}.{n}_proj", o, k)
            continue
        qsz, kvsz = cfg.head_num * D, cfg.kv_head_num * D
        put_lin(p + "attention.query_key_value.weight.0.bin", qsz + 2 * kvsz, H)
        put_lin(p + "attention.dense.weight.0.bin", H, qsz)
        if mt in ("qwen", "qwen2", "chatglm", "chatglm2", "chatglm3", "chatglm4", "gpt"):
            put(p + "attention.query_key_value.bias.0.bin", rnd(qsz + 2 * kvsz, s=0.05))
        if mt in ("gpt", "chatglm", "telechat"):
            put(p + "attention.dense.bias.bin", rnd(H, s=0.05))
        if cfg.do_qk_norm:
            put(p + "attention.q_norm.weight.bin", 1.0 + rnd(D, s=0.05))
            put(p + "attention.k_norm.weight.bin", 1.0 + rnd(D, s=0.05))
        I = cfg.inter_size
        if mt in ("gpt", "chatglm"):
            put_lin(p + "mlp.dense_h_to_4h.weight.0.bin", I, H)
            put(p + "mlp.dense_h_to_4h.bias.0.bin", rnd(I, s=0.05))
            put_lin(p + "mlp.dense_4h_to_h.weight.0.bin", H, I)
            put(p + "mlp.dense_4h_to_h.bias.bin", rnd(H, s=0.05))
        elif mt in ("chatglm2", "chatglm3", "chatglm4"):
            put_lin(p + "mlp.dense_h_to_4h.weight.0.bin", 2 * I, H)
            put_lin(p + "mlp.dense_4h_to_h.weight.0.bin", H, I)
        elif mt == "mixtral":
            E = cfg.sparse_experts
            put(p + "moe.gate.weight.bin", rnd(E, H, s=0.5).t().contiguous())
            for e in range(E):
                put_lin(p + f"moe.sparse_experts.{e}.w1.0.bin", I, H)     # gate
                put_lin(p + f"moe.sparse_experts.{e}.w2.0.bin", I, H)     # up
                put_lin(p + f"moe.sparse_experts.{e}.w3.0.bin", H, I)     # down
        elif mt == "qwen3_moe":
            E, MI = cfg.sparse_experts, cfg.moe_intermediate_size or I
            put(p + "mlp.gate.weight.0.bin", rnd(E, H, s=0.5).t().contiguous())
            for e in range(E):
                put_lin(p + f"mlp.experts.{e}.gate_proj.weight.0.bin", MI, H)
                put_lin(p + f"mlp.experts.{e}.up_proj.weight.0.bin", MI, H)
                put_lin(p + f"mlp.experts.{e}.down_proj.weight.0.bin", H, MI)
        else:
            put_lin(p + "mlp.gate_proj.weight.0.bin", I, H)
            put_lin(p + "mlp.up_proj.weight.0.bin", I, H)
            put_lin(p + "mlp.down_proj.weight.0.bin", H, I)
    return path
