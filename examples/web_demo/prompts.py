"""Chat prompt formats per model family (the reference keeps one web demo per family because of these:
``examples/web_demo/{Llama2,Llama3,ChatGLM,ChatGLM2,ChatGLM3,Qwen,Qwen2,Baichuan2,Gemma,Yi}.py``).  Used when the tokenizer
has no ``chat_template`` of its own.  ``history`` is a list of (user, assistant) pairs; ``build_prompt`` returns text."""
from typing import List, Tuple

History = List[Tuple[str, str]]


def llama2(history: History, message: str, system: str = "") -> str:
    out, first = "", True
    for u, a in history + [(message, None)]:
        u = f"<<SYS>>\n{system}\n<</SYS>>\n\n{u}" if first and system else u
        first = False
        out += f"<s>[INST] {u.strip()} [/INST]" + (f" {a.strip()} </s>" if a is not None else "")
    return out


def llama3(history: History, message: str, system: str = "") -> str:
    def turn(role, text):
        return f"<|start_header_id|>{role}<|end_header_id|>\n\n{text.strip()}<|eot_id|>"
    out = "<|begin_of_text|>" + (turn("system", system) if system else "")
    for u, a in history:
        out += turn("user", u) + turn("assistant", a)
    return out + turn("user", message) + "<|start_header_id|>assistant<|end_header_id|>\n\n"


def chatml(history: History, message: str, system: str = "You are a helpful assistant.") -> str:
    """Qwen, Qwen2 / Qwen3, Yi-chat."""
    out = f"<|im_start|>system\n{system}<|im_end|>\n" if system else ""
    for u, a in history:
        out += f"<|im_start|>user\n{u}<|im_end|>\n<|im_start|>assistant\n{a}<|im_end|>\n"
    return out + f"<|im_start|>user\n{message}<|im_end|>\n<|im_start|>assistant\n"


def chatglm(history: History, message: str, system: str = "") -> str:
    """ChatGLM-6B (v1)."""
    if not history:
        return message
    out = ""
    for i, (u, a) in enumerate(history):
        out += f"[Round {i}]\n问：{u}\n答：{a}\n"
    return out + f"[Round {len(history)}]\n问：{message}\n答："


def chatglm2(history: History, message: str, system: str = "") -> str:
    out = ""
    for i, (u, a) in enumerate(history):
        out += f"[Round {i + 1}]\n\n问：{u}\n\n答：{a}\n\n"
    return out + f"[Round {len(history) + 1}]\n\n问：{message}\n\n答："


def chatglm3(history: History, message: str, system: str = "") -> str:
    out = f"<|system|>\n {system}" if system else ""
    for u, a in history:
        out += f"<|user|>\n {u}<|assistant|>\n {a}"
    return out + f"<|user|>\n {message}<|assistant|>"


def baichuan2(history: History, message: str, system: str = "") -> str:
    out = system
    for u, a in history:
        out += f"<reserved_106>{u}<reserved_107>{a}"
    return out + f"<reserved_106>{message}<reserved_107>"


def gemma(history: History, message: str, system: str = "") -> str:
    out = "<bos>"
    for u, a in history:
        out += f"<start_of_turn>user\n{u}<end_of_turn>\n<start_of_turn>model\n{a}<end_of_turn>\n"
    return out + f"<start_of_turn>user\n{message}<end_of_turn>\n<start_of_turn>model\n"


FORMATS = {"llama2": llama2, "llama3": llama3, "qwen": chatml, "qwen2": chatml, "qwen3": chatml, "yi": chatml,
           "chatglm": chatglm, "chatglm2": chatglm2, "chatglm3": chatglm3, "chatglm4": chatglm3, "baichuan2": baichuan2,
           "gemma": gemma}


def build_prompt(family: str, history: History, message: str, system: str = "") -> str:
    if family not in FORMATS:
        raise KeyError(f"unknown chat format '{family}'; known: {sorted(FORMATS)}")
    return FORMATS[family](history, message, system) if system else FORMATS[family](history, message)
