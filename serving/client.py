#!/usr/bin/env python
"""Command-line client of the token-id server (reference: ``serving/grpc_launcher/client.py`` and ``client_stream.py``):
waits for the server's health check, tokenizes a prompt (a Hugging Face tokenizer directory, or token ids given directly),
calls ``predict`` or, with ``--stream``, ``predict_stream`` and prints the text (or ids) as it arrives.

    python serving/client.py --port 50051 -t /models/llama-2-7b-hf -i "Once upon a time" --max_length 128 --stream
    python serving/client.py --port 50051 --ids "1 15043 29892" --max_length 32
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from server import Client  # noqa: E402


def wait_healthy(client: Client, timeout_s: float = 30.0) -> bool:
    """Poll the health method until the server answers SERVING (the reference polls for 30 s as well)."""
    t0 = time.time()
    while time.time() - t0 < timeout_s:
        try:
            if client.health().get("status") == "SERVING":
                return True
        except Exception:
            pass
        time.sleep(0.2)
    return False


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=50051)
    ap.add_argument("-t", "--token_path", default="", help="Hugging Face tokenizer directory")
    ap.add_argument("-i", "--input", default="Once upon a time, there existed a little girl who liked to have adventures.")
    ap.add_argument("--ids", default="", help="prompt as token ids separated by spaces (no tokenizer needed)")
    ap.add_argument("--max_length", type=int, default=128)
    ap.add_argument("--num_beams", type=int, default=1)
    ap.add_argument("--do_sample", action="store_true")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top_k", type=int, default=50)
    ap.add_argument("--top_p", type=float, default=1.0)
    ap.add_argument("--repetition_penalty", type=float, default=1.0)
    ap.add_argument("--eos_token_id", type=int, default=-1)
    ap.add_argument("--stream", action="store_true")
    ap.add_argument("--health_timeout", type=float, default=30.0)
    a = ap.parse_args(argv)
    tok = None
    if a.ids:
        ids = [int(t) for t in a.ids.split()]
    else:
        if not a.token_path:
            ap.error("give --ids, or -t <tokenizer dir> with -i <text>")
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.token_path, trust_remote_code=True)
        ids = tok(a.input)["input_ids"]
        if a.eos_token_id < 0 and tok.eos_token_id is not None:
            a.eos_token_id = tok.eos_token_id
    client = Client(f"{a.host}:{a.port}")
    if not wait_healthy(client, a.health_timeout):
        print("server is not healthy", file=sys.stderr)
        return 1
    kw = dict(max_length=a.max_length, num_beams=a.num_beams, do_sample=a.do_sample, temperature=a.temperature,
              top_k=a.top_k, top_p=a.top_p, repetition_penalty=a.repetition_penalty, eos_token_id=a.eos_token_id)
    show = (lambda t: tok.decode(t, skip_special_tokens=True)) if tok else (lambda t: " ".join(map(str, t)))
    t0 = time.perf_counter()
    if a.stream:
        got, first = [], None
        for msg in client.predict_stream([ids], **kw):
            if first is None:
                first = time.perf_counter() - t0
            got += msg["Ids"]
            print(show(msg["Ids"]), end=" " if not tok else "", flush=True)
        print()
        dt = time.perf_counter() - t0
        n = max(len(got), 1)
        print(f"first token {1e3 * (first or 0):.1f} ms, {n} tokens, {1e3 * (dt - (first or 0)) / max(n - 1, 1):.1f} ms/token",
              file=sys.stderr)
    else:
        r = client.predict([ids], **kw)
        print(show(r["Ids"][len(ids):] if r["seq_len"] > len(ids) else r["Ids"]))
        print(f"{1e3 * (time.perf_counter() - t0):.1f} ms", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
