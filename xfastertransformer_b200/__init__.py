"""xfastertransformer_b200 — a Blackwell-native LLM inference engine with the API of
intel/xFasterTransformer (package layout of the reference: ``src/xfastertransformer/__init__.py``).

Converters are imported lazily, as in the reference (``__init__.py:35-121``).
"""
from .automodel import AutoModel
from .env import get_env

__version__ = "0.3.0"

_CONVERTERS = {
    "LlamaConvert": "llama_convert", "YiConvert": "llama_convert", "GemmaConvert": "llama_convert",
    "DeepSeekConvert": "llama_convert", "YaRNLlamaConvert": "llama_convert",
    "Qwen2Convert": "qwen_convert", "QwenConvert": "qwen_convert", "Qwen3Convert": "qwen_convert",
    "ChatGLMConvert": "chatglm_convert", "ChatGLM2Convert": "chatglm_convert", "ChatGLM3Convert": "chatglm_convert",
    "ChatGLM4Convert": "chatglm_convert", "OPTConvert": "opt_convert", "BaichuanConvert": "baichuan_convert",
    "Baichuan2Convert": "baichuan_convert", "TelechatConvert": "telechat_convert", "MixtralConvert": "mixtral_convert",
    "DeepSeekV2Convert": "deepseek_moe_convert", "DeepSeekV3Convert": "deepseek_moe_convert",
    "DeepSeekR1Convert": "deepseek_moe_convert",
}


def __getattr__(name):
    if name in _CONVERTERS:
        import importlib
        mod = importlib.import_module(f".tools.{_CONVERTERS[name]}", __name__)
        return getattr(mod, name)
    raise AttributeError(f"module {__name__} has no attribute {name}")


__all__ = ["AutoModel", "get_env"] + list(_CONVERTERS)
