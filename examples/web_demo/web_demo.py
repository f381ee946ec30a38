#!/usr/bin/env python
"""Gradio chat demo (reference: ``examples/web_demo/*.py``).  The engine is config-driven, so the demo is one program;
the per-family launchers beside it (``Llama2.py``, ``Llama3.py``, ``Qwen.py``, ``Qwen2.py``, ``Yi.py``, ``ChatGLM.py`` …
``ChatGLM4.py``, ``Baichuan2.py``, ``Gemma.py`` — the reference's file names) start it with that family's prompt
format, end-of-turn tokens and history depth (``prompts.FAMILIES``).  Needs ``gradio`` and a HuggingFace tokenizer.

    python examples/web_demo/Llama2.py -m <xft model dir> -t <tokenizer dir> [-d bf16] [--kv_cache_dtype fp16] [--port 7860]
    python examples/web_demo/web_demo.py -m <xft model dir> -t <tokenizer dir> [--chat_format llama3]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main(family: str = ""):
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model_path", required=True)
    ap.add_argument("-t", "--token_path", required=True)
    ap.add_argument("-d", "--dtype", default="bf16")
    ap.add_argument("--kv_cache_dtype", default="fp16", choices=["fp16", "bf16", "int8"])
    ap.add_argument("--port", type=int, default=7860)
    ap.add_argument("--chat_format", default=family, help="prompt format when the tokenizer has no chat template: "
                    "llama2, llama3, qwen, qwen2, qwen3, yi, chatglm, chatglm2, chatglm3, chatglm4, baichuan2, gemma")
    a = ap.parse_args()
    try:
        import gradio as gr
    except ImportError:
        sys.exit("gradio is not installed in this environment: pip install gradio")
    from transformers import AutoTokenizer

    import xfastertransformer_b200 as xft
    tok = AutoTokenizer.from_pretrained(a.token_path)
    model = xft.AutoModel.from_pretrained(a.model_path, dtype=a.dtype, kv_cache_dtype=a.kv_cache_dtype)
    from prompts import FAMILIES, build_prompt, stop_token_ids       # examples/web_demo/prompts.py
    fam = FAMILIES.get(a.chat_format, {})
    stops = stop_token_ids(tok, a.chat_format)
    if model.rank != 0:
        while True:
            model.generate()

    def chat(message, history, max_new, temperature, top_p):
        history = list(history)[-fam.get("max_rounds", 8):]
        msgs = [{"role": r, "content": c} for u, b in history for r, c in (("user", u), ("assistant", b))]
        msgs.append({"role": "user", "content": message})
        try:
            if family:
                raise ValueError("a per-family launcher uses its own prompt format")
            ids = tok.apply_chat_template(msgs, add_generation_prompt=True, return_tensors="pt")
        except Exception:
            if a.chat_format:
                ids = tok(build_prompt(a.chat_format, list(history), message), return_tensors="pt",
                          add_special_tokens=False).input_ids
            else:
                ids = tok(message, return_tensors="pt").input_ids
        model.set_input(ids, max_length=ids.shape[1] + int(max_new), do_sample=temperature > 0, temperature=max(temperature, 1e-3),
                        top_p=top_p, eos_token_id=tok.eos_token_id or -1, stop_words_ids=[[t] for t in stops] or None)
        out = []
        while not model.is_done():
            t = int(model.forward()[0])
            if t in stops:
                break
            out.append(t)
            yield tok.decode(out, skip_special_tokens=True)
        model.finalize()

    gr.ChatInterface(chat, title="xFasterTransformer-B200 " + fam.get("title", "chat"), additional_inputs=[gr.Slider(16, 2048, 256, label="max new tokens"),
                                              gr.Slider(0, 2, 0.7, label="temperature"), gr.Slider(0, 1, 0.9, label="top-p")]
                     ).launch(server_name="0.0.0.0", server_port=a.port)


if __name__ == "__main__":
    main()
