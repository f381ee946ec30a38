"""Converters against HuggingFace: a random tiny HF model is saved, converted, loaded by the engine (CPU path),
and the engine's all-position logits must equal the HF model's — orientation, q/k/v merge, w2/w3 swap, norm
conventions and config keys are all exercised.  Plus a checkpoint round trip through the GPTQ layout."""
import os

import pytest
import torch

transformers = pytest.importorskip("transformers")

import xfastertransformer_b200 as xft


@pytest.fixture(autouse=True)
def _cpu(monkeypatch):
    monkeypatch.setenv("XFT_ENGINE", "CPU")


def _roundtrip(hf_model, conv, tmp_path, ids, tol=1.5e-2, dtype="fp32"):   # engine weights are bf16-rounded
    src = str(tmp_path / "hf")
    hf_model.save_pretrained(src, safe_serialization=True)
    out = conv().convert(src, str(tmp_path / "xft"), dtype=dtype)
    m = xft.AutoModel.from_pretrained(out, dtype="bf16")
    got = m(ids)
    with torch.no_grad():
        want = hf_model(ids).logits.float()
    assert torch.allclose(got, want, atol=tol, rtol=tol), (got - want).abs().max()
    return out


def test_llama_convert(tmp_path):
    from transformers import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=352, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=256, rms_norm_eps=1e-5, tie_word_embeddings=False)
    model = LlamaForCausalLM(cfg).eval()
    ids = torch.randint(0, 512, (2, 17))
    out = _roundtrip(model, xft.LlamaConvert, tmp_path, ids)
    from xfastertransformer_b200.config import ModelConfig
    c = ModelConfig.from_ini(out)
    assert (c.model_type, c.head_num, c.kv_head_num, c.inter_size, c.layernorm_eps) == ("llama", 4, 2, 352, 1e-5)


def test_qwen2_convert_with_bias(tmp_path):
    from transformers import Qwen2Config, Qwen2ForCausalLM
    torch.manual_seed(1)
    cfg = Qwen2Config(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=4, max_position_embeddings=256, tie_word_embeddings=True)
    model = Qwen2ForCausalLM(cfg).eval()
    _roundtrip(model, xft.Qwen2Convert, tmp_path, torch.randint(0, 512, (1, 23)))


def test_mixtral_convert_swaps_w2_w3(tmp_path):
    from transformers import MixtralConfig, MixtralForCausalLM
    torch.manual_seed(2)
    cfg = MixtralConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2, max_position_embeddings=256)
    model = MixtralForCausalLM(cfg).eval()
    _roundtrip(model, xft.MixtralConvert, tmp_path, torch.randint(0, 512, (2, 11)))


def test_opt_convert(tmp_path):
    from transformers import OPTConfig, OPTForCausalLM
    torch.manual_seed(3)
    cfg = OPTConfig(vocab_size=512, hidden_size=128, ffn_dim=256, num_hidden_layers=2, num_attention_heads=4,
                    max_position_embeddings=128, word_embed_proj_dim=128, do_layer_norm_before=True)
    model = OPTForCausalLM(cfg).eval()
    _roundtrip(model, xft.OPTConvert, tmp_path, torch.randint(3, 512, (2, 13)))


def test_gemma_convert(tmp_path):
    from transformers import GemmaConfig, GemmaForCausalLM
    torch.manual_seed(4)
    cfg = GemmaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=1, head_dim=32, max_position_embeddings=256)
    model = GemmaForCausalLM(cfg).eval()
    _roundtrip(model, xft.GemmaConvert, tmp_path, torch.randint(0, 512, (1, 19)))


def test_qwen3_convert(tmp_path):
    try:
        from transformers import Qwen3Config, Qwen3ForCausalLM
    except ImportError:
        pytest.skip("transformers without Qwen3")
    torch.manual_seed(5)
    cfg = Qwen3Config(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=48, max_position_embeddings=256, tie_word_embeddings=False)
    model = Qwen3ForCausalLM(cfg).eval()
    _roundtrip(model, xft.Qwen3Convert, tmp_path, torch.randint(0, 512, (2, 9)))


def test_gptq_layout_roundtrip(tmp_path):
    """Write a GPTQ-style converted directory by hand (int8 and uint4 qweight + scales + zeros) and load it."""
    from xfastertransformer_b200.config import ModelConfig
    from xfastertransformer_b200.ops import reference as R
    from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint
    import numpy as np
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from gptq_util import make_gptq_dir
    for qt in ("int8", "uint4"):
        cfg = preset("tiny-llama", vocab_size=512)
        dense = str(tmp_path / (qt + "_dense"))
        write_synthetic_checkpoint(dense, cfg, seed=0, dtype="fp32", std=0.08)
        base = xft.AutoModel.from_pretrained(dense, dtype="bf16")
        ids = torch.randint(0, 512, (1, 12))
        want = base(ids)
        d = make_gptq_dir(str(tmp_path / qt), cfg, qt, seed=0, std=0.08)
        m = xft.AutoModel.from_pretrained(d, dtype="int8" if qt == "int8" else "int4")
        got = m(ids)
        rel = (got - want).abs().max().item() / want.abs().max().item()
        assert rel < (0.1 if qt == "int8" else 0.6), rel


def test_reference_tool_module_names_resolve():
    """`xfastertransformer.tools` and the reference's per-family module names import the same converter classes."""
    import importlib
    import xfastertransformer as ref_name
    from xfastertransformer.tools import LlamaConvert, DeepSeekR1Convert
    assert LlamaConvert is ref_name.LlamaConvert is xft.LlamaConvert and DeepSeekR1Convert is xft.DeepSeekR1Convert
    for mod, cls in (("llama_convert", "LlamaConvert"), ("yarn_llama_convert", "YaRNLlamaConvert"),
                     ("qwen_convert", "QwenConvert"), ("qwen2_convert", "Qwen2Convert"), ("qwen3_convert", "Qwen3Convert"),
                     ("chatglm_convert", "ChatGLMConvert"), ("chatglm2_convert", "ChatGLM2Convert"),
                     ("chatglm3_convert", "ChatGLM3Convert"), ("chatglm4_convert", "ChatGLM4Convert"),
                     ("opt_convert", "OPTConvert"), ("baichuan_convert", "BaichuanConvert"),
                     ("baichuan2_convert", "Baichuan2Convert"), ("telechat_convert", "TelechatConvert"),
                     ("mixtral_convert", "MixtralConvert"), ("deepseek_moe_convert", "DeepSeekV3Convert"),
                     ("convert", "BaseModelConvert")):
        m = importlib.import_module(f"xfastertransformer.tools.{mod}")
        assert getattr(m, cls) is getattr(xft.tools, cls), (mod, cls)
    with pytest.raises(ImportError):
        importlib.import_module("xfastertransformer.tools.no_such_convert")


def test_converter_cli_picks_the_family(tmp_path, capsys):
    """python -m xfastertransformer_b200.tools: the converter follows from config.json; the converted model matches HF."""
    from transformers import Qwen2Config, Qwen2ForCausalLM
    from xfastertransformer_b200.tools.__main__ import main, pick_converter
    torch.manual_seed(5)
    cfg = Qwen2Config(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=256, tie_word_embeddings=False)
    model = Qwen2ForCausalLM(cfg).eval()
    src, out = str(tmp_path / "hf"), str(tmp_path / "xft")
    model.save_pretrained(src, safe_serialization=True)
    assert main(["-i", src, "-o", out, "-d", "fp32"]) == 0
    assert "Qwen2Convert: wrote" in capsys.readouterr().out
    ids = torch.randint(0, 512, (1, 15))
    got = xft.AutoModel.from_pretrained(out, dtype="bf16")(ids)
    with torch.no_grad():
        want = model(ids).logits.float()
    assert torch.allclose(got, want, atol=1.5e-2, rtol=1.5e-2)
    assert main(["--list"]) == 0 and "DeepSeekR1Convert" in capsys.readouterr().out
    pick = lambda **kw: pick_converter(kw)
    assert pick(model_type="llama") == "LlamaConvert" and pick(model_type="mixtral") == "MixtralConvert"
    assert pick(model_type="llama", rope_scaling={"type": "yarn", "factor": 4}) == "YaRNLlamaConvert"
    assert pick(model_type="deepseek_v3") == "DeepSeekV3Convert" and pick(model_type="qwen3_moe") == "Qwen3Convert"
    assert pick(model_type="chatglm", multi_query_attention=True, _name_or_path="THUDM/chatglm3-6b") == "ChatGLM3Convert"
    assert pick(model_type="chatglm", multi_query_attention=True, _name_or_path="THUDM/glm-4-9b") == "ChatGLM4Convert"
    assert pick(model_type="chatglm", num_layers=28) == "ChatGLMConvert"
    assert pick(architectures=["BaichuanForCausalLM"], vocab_size=125696) == "Baichuan2Convert"
    with pytest.raises(ValueError):
        pick(model_type="mamba")
    with pytest.raises(SystemExit):
        main(["-i", src, "--family", "NoSuchConvert"])


@pytest.mark.parametrize("bits", [4, 8])
def test_gptq_checkpoint_conversion_with_wrapped_zero_points(tmp_path, bits):
    """An AutoGPTQ-format Llama checkpoint written by hand (qweight packed along the input dimension, qzeros holding
    zero - 1, per-channel scales) goes through LlamaConvert and must reproduce the dense model built from the same
    dequantised weights.  Half of the channels use a true zero point of 0, which AutoGPTQ stores as all ones
    (2^bits - 1): the converter has to add the 1 back modulo 2^bits (reference tools/llama_convert.py:360-364)."""
    import json
    import numpy as np
    from safetensors.torch import save_file
    from transformers import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(bits)
    cfg = LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=128, tie_word_embeddings=False)
    model = LlamaForCausalLM(cfg).eval()
    sd = {k: v.detach().clone() for k, v in model.state_dict().items()}
    pack, qmax = 32 // bits, (1 << bits) - 1
    out = {}
    for name, w in list(sd.items()):
        if not (name.endswith("_proj.weight") and ".layers." in name):
            out[name] = w.contiguous()
            continue
        W = w.float().t().contiguous()                                   # [in, out]
        zero = torch.where(torch.arange(W.shape[1]) % 2 == 0, 0, (qmax + 1) // 2)   # true zero points: 0 or mid-range
        lo, hi = W.min(0).values, W.max(0).values
        # zero = 0 channels hold only non-negative levels: shift those channels so they are representable
        scale = torch.where(zero == 0, (hi - lo).clamp_min(1e-6) / qmax, torch.maximum(hi, -lo).clamp_min(1e-6) / ((qmax - 1) // 2))
        shift = torch.where(zero == 0, lo, torch.zeros_like(lo))
        q = torch.clamp(torch.round((W - shift) / scale) + zero, 0, qmax).to(torch.int64)
        deq = (q - zero).float() * scale                                  # what GPTQ inference computes
        sd[name] = deq.t().contiguous()                                   # the dense twin uses exactly these weights
        qw = q.view(W.shape[0] // pack, pack, W.shape[1])
        packed = sum((qw[:, j, :] << (bits * j)) for j in range(pack))
        zstore = ((zero - 1) & qmax).view(1, W.shape[1] // pack, pack)   # AutoGPTQ stores zero - 1 (0 -> all ones)
        zpacked = sum((zstore[:, :, j] << (bits * j)) for j in range(pack))
        to_i32 = lambda t: torch.from_numpy(t.numpy().astype(np.uint32).view(np.int32).copy())
        base = name[: -len(".weight")]
        out[base + ".qweight"], out[base + ".qzeros"] = to_i32(packed), to_i32(zpacked)
        out[base + ".scales"] = scale.view(1, -1).half()
        assert int(zstore.max()) == qmax                                 # the all-ones case is present
    src = tmp_path / "gptq"
    src.mkdir()
    save_file(out, str(src / "model.safetensors"))
    hf = cfg.to_dict()
    hf["quantization_config"] = {"quant_method": "gptq", "bits": bits, "group_size": -1}
    (src / "config.json").write_text(json.dumps(hf))
    dst = str(tmp_path / "xft")
    assert xft.LlamaConvert().convert(str(src), dst, from_quantized_model="gptq")
    got = xft.AutoModel.from_pretrained(dst, dtype="int4" if bits == 4 else "int8")(torch.randint(0, 256, (1, 9),
                                        generator=torch.Generator().manual_seed(1)))
    model.load_state_dict(sd)
    ids = torch.randint(0, 256, (1, 9), generator=torch.Generator().manual_seed(1))
    want = model(ids).logits.float()
    rel = (got - want).abs().max().item() / want.abs().max().item()
    assert rel < 3e-2, rel            # fp16 scales are the only rounding left; a wrong zero point is an O(1) error


def test_builtin_gptq_quantizer_beats_round_to_nearest_and_converts(tmp_path):
    """tools/quantization/quantize_gptq.py: (1) on a linear layer with correlated inputs the GPTQ update gives a smaller
    OUTPUT error than rounding to nearest on the same grid; (2) the AutoGPTQ-format directory it writes for a tiny Llama
    goes through LlamaConvert and the int4 engine reproduces the dequantised HF model."""
    import json
    from safetensors.torch import load_file
    from transformers import LlamaConfig, LlamaForCausalLM
    from xfastertransformer_b200.tools.quantization import quantize_gptq as Q
    g = torch.Generator().manual_seed(0)
    n, fin, fout = 512, 96, 64
    X = torch.randn(n, 24, generator=g) @ torch.randn(24, fin, generator=g) + 0.3 * torch.randn(n, fin, generator=g)
    W = torch.randn(fout, fin, generator=g) * 0.1
    H = 2.0 * X.t() @ X / n
    for bits in (4, 8):
        q, s, z = Q.gptq_quantize(W, H, bits)
        qr, sr, zr = Q.rtn_quantize(W, bits)
        deq = lambda q_, s_, z_: (q_ - z_[:, None]).float() * s_[:, None]
        e_gptq = (X @ (deq(q, s, z) - W).t()).pow(2).mean().item()
        e_rtn = (X @ (deq(qr, sr, zr) - W).t()).pow(2).mean().item()
        assert int(q.min()) >= 0 and int(q.max()) <= (1 << bits) - 1
        assert e_gptq < 0.8 * e_rtn, (bits, e_gptq, e_rtn)
    torch.manual_seed(1)
    cfg = LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=128, tie_word_embeddings=False)
    src = tmp_path / "hf"
    LlamaForCausalLM(cfg).eval().save_pretrained(str(src), safe_serialization=True)
    out = Q.quantize_checkpoint(str(src), str(tmp_path / "gptq"), bits=4, samples=4, seq_len=32)
    conf = json.load(open(os.path.join(out, "config.json")))
    assert conf["quantization_config"] == {"quant_method": "gptq", "bits": 4, "group_size": -1, "sym": False, "desc_act": False}
    sd = load_file(os.path.join(out, "model.safetensors"))
    qw = sd["model.layers.0.mlp.down_proj.qweight"]
    assert qw.dtype == torch.int32 and tuple(qw.shape) == (128 // 8, 64)
    # dense twin of the quantised checkpoint: unpack what was written
    model = LlamaForCausalLM(cfg).eval()
    ref = load_file(os.path.join(str(src), "model.safetensors"))
    for name in list(ref):
        base = name[: -len(".weight")]
        if base + ".qweight" in sd:
            qw, qz, sc = sd[base + ".qweight"], sd[base + ".qzeros"], sd[base + ".scales"].float()[0]
            shifts = torch.arange(8) * 4
            lv = ((qw[:, None, :] >> shifts[None, :, None]) & 15).reshape(-1, qw.shape[1])          # [in, out]
            zp = (((qz[:, :, None] >> shifts[None, None, :]) & 15).reshape(-1) + 1) & 15
            ref[name] = ((lv - zp[None, :]).float() * sc[None, :]).t().contiguous()
    model.load_state_dict(ref)
    dst = str(tmp_path / "xft")
    xft.LlamaConvert().convert(out, dst, from_quantized_model="gptq")
    ids = torch.randint(0, 256, (1, 9), generator=torch.Generator().manual_seed(2))
    got = xft.AutoModel.from_pretrained(dst, dtype="int4")(ids)
    want = model(ids).logits.float()
    assert (got - want).abs().max().item() / want.abs().max().item() < 3e-2


def test_builtin_awq_scale_search(tmp_path):
    """The activation-aware step of tools/quantization/quantize_gptq.py: (1) with a few loud input channels the searched
    scales cut the 4-bit output error of a layer; (2) folding the scales into a tiny Llama (norm gains, up_proj and
    v_proj rows) leaves its logits unchanged; (3) the AWQ + GPTQ checkpoint is an ordinary GPTQ directory whose dense
    twin stays closer to the original model than round-to-nearest does."""
    from safetensors.torch import load_file
    from transformers import LlamaConfig, LlamaForCausalLM
    from xfastertransformer_b200.tools.quantization import quantize_gptq as Q
    g = torch.Generator().manual_seed(3)
    n, fin, fout = 1024, 128, 96
    X = torch.randn(n, fin, generator=g)
    X[:, [3, 40, 77]] *= 25.0                               # loud channels: their weights matter most for the output
    W = torch.randn(fout, fin, generator=g) * 0.1
    H = 2.0 * X.t() @ X / n
    s, ratio, best, base = Q.awq_search_scale([W], H, X.abs().mean(0), 4)
    assert ratio > 0 and best < 0.7 * base, (ratio, best, base)
    assert s[[3, 40, 77]].min() > s.median()                # the loud channels are the ones enlarged
    qs, ss, zs = Q.rtn_quantize(W * s[None, :], 4)
    qr, sr, zr = Q.rtn_quantize(W, 4)
    deq = lambda q_, s_, z_: (q_ - z_[:, None]).float() * s_[:, None]
    e_awq = ((X / s) @ deq(qs, ss, zs).t() - X @ W.t()).pow(2).mean().item()
    e_rtn = (X @ deq(qr, sr, zr).t() - X @ W.t()).pow(2).mean().item()
    assert e_awq < 0.7 * e_rtn, (e_awq, e_rtn)

    torch.manual_seed(4)
    cfg = LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=4, max_position_embeddings=128, tie_word_embeddings=False)
    model = LlamaForCausalLM(cfg).eval()
    with torch.no_grad():
        for layer in model.model.layers:                    # loud channels in the normalised state
            layer.input_layernorm.weight[[5, 30]] *= 12.0
            layer.post_attention_layernorm.weight[[9]] *= 12.0
    src = tmp_path / "hf"
    model.save_pretrained(str(src), safe_serialization=True)
    ids = torch.randint(0, 256, (2, 24), generator=g)
    want = model(ids).logits.float()
    batches = [torch.randint(0, 256, (1, 32), generator=g) for _ in range(6)]
    twin = LlamaForCausalLM.from_pretrained(str(src), torch_dtype=torch.float32).eval()
    Q.apply_awq(twin, batches, bits=4)
    changed = (twin.model.layers[0].input_layernorm.weight - model.model.layers[0].input_layernorm.weight).abs().max().item()
    assert changed > 1e-3                                   # scales were found and folded in ...
    assert (twin(ids).logits.float() - want).abs().max().item() < 2e-3 * want.abs().max().item()      # ... same function

    def dense_twin(out_dir):
        sd = load_file(os.path.join(out_dir, "model.safetensors"))
        m = LlamaForCausalLM(cfg).eval()
        state = {}
        for name in m.state_dict():
            base = name[: -len(".weight")] if name.endswith(".weight") else name
            if base + ".qweight" in sd:
                qw, qz, sc = sd[base + ".qweight"], sd[base + ".qzeros"], sd[base + ".scales"].float()[0]
                shifts = torch.arange(8) * 4
                lv = ((qw[:, None, :] >> shifts[None, :, None]) & 15).reshape(-1, qw.shape[1])
                zp = (((qz[:, :, None] >> shifts[None, None, :]) & 15).reshape(-1) + 1) & 15
                state[name] = ((lv - zp[None, :]).float() * sc[None, :]).t().contiguous()
            else:
                state[name] = sd[name]
        m.load_state_dict(state)
        return m

    both = Q.quantize_checkpoint(str(src), str(tmp_path / "awq_gptq"), bits=4, samples=6, seq_len=32, awq=True)
    e_both = (dense_twin(both)(ids).logits.float() - want).abs().mean().item()
    rtn = LlamaForCausalLM.from_pretrained(str(src), torch_dtype=torch.float32).eval()
    with torch.no_grad():
        for name, mod in rtn.named_modules():
            if isinstance(mod, torch.nn.Linear) and ".layers." in name:
                q, sc, z = Q.rtn_quantize(mod.weight.data, 4)
                mod.weight.data = deq(q, sc, z)
    e_rtn_model = (rtn(ids).logits.float() - want).abs().mean().item()
    assert e_both < e_rtn_model, (e_both, e_rtn_model)
