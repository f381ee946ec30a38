"""Command line for the checkpoint converters:

    python -m xfastertransformer_b200.tools -i /hf/Llama-2-7b-hf -o /models/llama-2-7b-xft -d bf16
    python -m xfastertransformer_b200.tools -i /hf/Qwen2-7B-GPTQ -o /models/qwen2-7b-int4 --from_quantized_model gptq
    python -m xfastertransformer_b200.tools --list

The family is read from the Hugging Face ``config.json`` (``model_type`` / ``architectures``) unless ``--family`` names
a converter class.  The reference documents the equivalent one-liner
``python -c 'import xfastertransformer as xft; xft.LlamaConvert().convert("in", "out")'``, which works here too.
"""
import argparse
import json
import os
import sys

from . import _CONVERTERS, __getattr__ as _converter

# Hugging Face model_type -> converter class
BY_MODEL_TYPE = {
    "llama": "LlamaConvert", "mistral": "LlamaConvert", "yi": "YiConvert", "gemma": "GemmaConvert",
    "qwen": "QwenConvert", "qwen2": "Qwen2Convert", "qwen3": "Qwen3Convert", "qwen3_moe": "Qwen3Convert",
    "opt": "OPTConvert", "baichuan": "BaichuanConvert", "telechat": "TelechatConvert", "mixtral": "MixtralConvert",
    "deepseek_v2": "DeepSeekV2Convert", "deepseek_v3": "DeepSeekV3Convert",
}


def pick_converter(hf: dict) -> str:
    """Converter class name for a Hugging Face config."""
    mt = (hf.get("model_type") or "").lower()
    arch = " ".join(hf.get("architectures") or []).lower()
    if mt == "chatglm" or "chatglm" in arch:
        # ChatGLM generations share the model_type: v1 has no multi-query attention, v2 / v3 differ by the tokenizer
        # (same tensors), v4 ("glm-4") names its layers the same way with a larger rope ratio
        if not hf.get("multi_query_attention", False) and "num_layers" in hf and "ffn_hidden_size" not in hf:
            return "ChatGLMConvert"
        name = (hf.get("_name_or_path") or "").lower()
        if "glm-4" in name or "glm4" in name:
            return "ChatGLM4Convert"
        return "ChatGLM3Convert" if "chatglm3" in name else "ChatGLM2Convert"
    if mt == "baichuan" or "baichuan" in arch:
        return "Baichuan2Convert" if hf.get("vocab_size", 0) > 64000 or "baichuan2" in (hf.get("_name_or_path") or "").lower() \
            else "BaichuanConvert"
    if mt == "llama" and isinstance(hf.get("rope_scaling"), dict) and \
            (hf["rope_scaling"].get("type") or hf["rope_scaling"].get("rope_type")) == "yarn":
        return "YaRNLlamaConvert"
    if mt in BY_MODEL_TYPE:
        return BY_MODEL_TYPE[mt]
    raise ValueError(f"no converter for model_type '{mt}' (architectures: {arch or 'none'}); pass --family, "
                     f"one of {sorted(c for c in _CONVERTERS if c != 'BaseModelConvert')}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m xfastertransformer_b200.tools", description=__doc__.split("\n\n")[0])
    ap.add_argument("-i", "--input_dir", help="Hugging Face checkpoint directory")
    ap.add_argument("-o", "--output_dir", default=None, help="default: <input_dir>-xft")
    ap.add_argument("-d", "--dtype", default=None, help="fp16 | bf16 | fp32 (DeepSeek: fp8_e4m3 | bf16)")
    ap.add_argument("--family", default=None, help="converter class, e.g. LlamaConvert (default: from config.json)")
    ap.add_argument("--from_quantized_model", default=None, choices=[None, "gptq"])
    ap.add_argument("--processes", type=int, default=8)
    ap.add_argument("--list", action="store_true", help="list the converter classes and exit")
    a = ap.parse_args(argv)
    if a.list:
        print("\n".join(sorted(c for c in _CONVERTERS if c != "BaseModelConvert")))
        return 0
    if not a.input_dir:
        ap.error("-i/--input_dir is required")
    name = a.family
    if name is None:
        with open(os.path.join(a.input_dir, "config.json")) as f:
            name = pick_converter(json.load(f))
    if name not in _CONVERTERS:
        ap.error(f"unknown converter {name}")
    conv = _converter(name)()
    kw = {}
    if a.from_quantized_model:
        kw["from_quantized_model"] = a.from_quantized_model
    out = conv.convert(a.input_dir, a.output_dir, a.dtype, a.processes, **kw)
    print(f"{name}: wrote {out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
