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


# Per-family settings of the chat demos (the reference's ten demo files differ in exactly these): page title, prompt
# format, the strings that end an assistant turn besides the tokenizer's EOS (looked up as single tokens), and how many
# past rounds are put back into the prompt.
FAMILIES = {
    "llama2": dict(title="Llama2", chat_format="llama2", stop=["</s>"], max_rounds=2),
    "llama3": dict(title="Llama3", chat_format="llama3", stop=["<|eot_id|>", "<|end_of_text|>"], max_rounds=8),
    "qwen": dict(title="Qwen", chat_format="qwen", stop=["<|im_end|>", "<|endoftext|>"], max_rounds=8),
    "qwen2": dict(title="Qwen2", chat_format="qwen2", stop=["<|im_end|>", "<|endoftext|>"], max_rounds=8),
    "yi": dict(title="Yi", chat_format="yi", stop=["<|im_end|>", "<|endoftext|>"], max_rounds=8),
    "chatglm": dict(title="ChatGLM", chat_format="chatglm", stop=["<eop>"], max_rounds=8),
    "chatglm2": dict(title="ChatGLM2", chat_format="chatglm2", stop=[], max_rounds=8),
    "chatglm3": dict(title="ChatGLM3", chat_format="chatglm3", stop=["<|user|>", "<|observation|>"], max_rounds=8),
    "chatglm4": dict(title="ChatGLM4", chat_format="chatglm4", stop=["<|user|>", "<|observation|>", "<|endoftext|>"], max_rounds=8),
    "baichuan2": dict(title="Baichuan2", chat_format="baichuan2", stop=[], max_rounds=8),
    "gemma": dict(title="Gemma", chat_format="gemma", stop=["<end_of_turn>"], max_rounds=8),
}


def stop_token_ids(tokenizer, family: str):
    """Ids of the family's end-of-turn strings that the tokenizer knows as ONE token (others are ignored), plus its EOS."""
    ids = []
    unk = getattr(tokenizer, "unk_token_id", None)
    for s in FAMILIES.get(family, {}).get("stop", []):
        try:
            t = tokenizer.convert_tokens_to_ids(s)
        except Exception:
            t = None
        if isinstance(t, int) and t >= 0 and t != unk and t not in ids:
            ids.append(t)
    eos = getattr(tokenizer, "eos_token_id", None)
    if isinstance(eos, int) and eos >= 0 and eos not in ids:
        ids.append(eos)
    return ids
