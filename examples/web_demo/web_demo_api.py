#!/usr/bin/env python
"""Gradio chat front end for an OpenAI-compatible endpoint (reference: ``examples/web_demo/web_demo_api.py``): the
model runs in ``serving/openai_server.py`` (any number of GPUs), this process only renders the conversation and
streams the server's answer.

    python serving/openai_server.py --model_path <dir> --token_path <tokenizer dir> --port 8000 &
    python examples/web_demo/web_demo_api.py --url http://127.0.0.1:8000 [--port 7860]
"""
import argparse
import json
import sys
import urllib.request


def stream_chat(url, messages, max_tokens, temperature, top_p):
    body = json.dumps({"messages": messages, "max_tokens": max_tokens, "temperature": temperature, "top_p": top_p,
                       "stream": True}).encode()
    req = urllib.request.Request(url + "/v1/chat/completions", data=body, headers={"Content-Type": "application/json"})
    text = ""
    with urllib.request.urlopen(req, timeout=3600) as r:
        for raw in r:
            line = raw.decode().strip()
            if not line.startswith("data: {"):
                continue
            text += json.loads(line[6:])["choices"][0]["delta"].get("content", "")
            yield text


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--port", type=int, default=7860)
    a = ap.parse_args()
    try:
        import gradio as gr
    except ImportError:
        sys.exit("gradio is not installed in this environment: pip install gradio")

    def chat(message, history, max_new, temperature, top_p):
        msgs = [{"role": r, "content": c} for u, b in history for r, c in (("user", u), ("assistant", b))]
        msgs.append({"role": "user", "content": message})
        yield from stream_chat(a.url, msgs, int(max_new), float(temperature), float(top_p))

    gr.ChatInterface(chat, additional_inputs=[gr.Slider(16, 2048, 256, label="max new tokens"),
                                              gr.Slider(0.0, 2.0, 0.7, label="temperature"),
                                              gr.Slider(0.1, 1.0, 0.9, label="top-p")]).launch(server_port=a.port)


if __name__ == "__main__":
    main()
