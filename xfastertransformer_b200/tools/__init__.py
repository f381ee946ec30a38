"""Checkpoint converters and model tooling (reference: ``src/xfastertransformer/tools/__init__.py``, which exports one
``*Convert`` class per model family).  The classes are imported on first use; the reference's module names
(``llama_convert``, ``chatglm2_convert``, ``baichuan2_convert`` ...) resolve to the module that holds the class here."""
import importlib

_CONVERTERS = {
    "LlamaConvert": "llama_convert", "YiConvert": "llama_convert", "GemmaConvert": "llama_convert",
    "DeepSeekConvert": "llama_convert", "YaRNLlamaConvert": "llama_convert",
    "Qwen2Convert": "qwen_convert", "QwenConvert": "qwen_convert", "Qwen3Convert": "qwen_convert",
    "ChatGLMConvert": "chatglm_convert", "ChatGLM2Convert": "chatglm_convert", "ChatGLM3Convert": "chatglm_convert",
    "ChatGLM4Convert": "chatglm_convert", "OPTConvert": "opt_convert", "BaichuanConvert": "baichuan_convert",
    "Baichuan2Convert": "baichuan_convert", "TelechatConvert": "telechat_convert", "MixtralConvert": "mixtral_convert",
    "DeepSeekV2Convert": "deepseek_moe_convert", "DeepSeekV3Convert": "deepseek_moe_convert",
    "DeepSeekR1Convert": "deepseek_moe_convert", "BaseModelConvert": "convert",
}

# module names of the reference's tools package -> module of this package that holds the same classes
REFERENCE_MODULES = {
    "convert": "convert", "llama_convert": "llama_convert", "yarn_llama_convert": "llama_convert",
    "qwen_convert": "qwen_convert", "qwen2_convert": "qwen_convert", "qwen3_convert": "qwen_convert",
    "chatglm_convert": "chatglm_convert", "chatglm2_convert": "chatglm_convert", "chatglm3_convert": "chatglm_convert",
    "chatglm4_convert": "chatglm_convert", "opt_convert": "opt_convert", "baichuan_convert": "baichuan_convert",
    "baichuan2_convert": "baichuan_convert", "telechat_convert": "telechat_convert", "mixtral_convert": "mixtral_convert",
    "deepseek_moe_convert": "deepseek_moe_convert",
}


def __getattr__(name):
    if name in _CONVERTERS:
        return getattr(importlib.import_module(f"{__name__}.{_CONVERTERS[name]}"), name)
    if name in REFERENCE_MODULES and REFERENCE_MODULES[name] != name:
        return importlib.import_module(f"{__name__}.{REFERENCE_MODULES[name]}")
    raise AttributeError(f"module {__name__} has no attribute {name}")


__all__ = list(_CONVERTERS)
