#!/usr/bin/env python
"""Serving benchmark against an OpenAI-compatible endpoint (serving/openai_server.py): the metrics of the reference's
vLLM-xFT guide (``serving/vllm-xft.md:133-150``) — request throughput, input / output token throughput, mean / median /
P99 time to first token (TTFT) and time per output token (TPOT).

    python benchmarks/benchmark_serving.py --url http://127.0.0.1:8000 --num_prompts 200 --request_rate 8 \
        --input_len 512 --output_len 128 [--vocab 32000]
Prompts are random token ids (the server accepts id lists), arrivals are Poisson at `--request_rate` (inf = all at once),
responses are streamed so the first-token time is observed at the client.
"""
import argparse
import json
import random
import statistics
import threading
import time
import urllib.request


def one_request(url, prompt, out_len, rec):
    body = json.dumps({"prompt": prompt, "max_tokens": out_len, "stream": True}).encode()
    req = urllib.request.Request(url + "/v1/completions", data=body, headers={"Content-Type": "application/json"})
    t0 = time.perf_counter()
    first, last, n = None, None, 0
    try:
        with urllib.request.urlopen(req, timeout=3600) as r:
            for raw in r:
                line = raw.decode().strip()
                if not line.startswith("data: {"):
                    continue
                now = time.perf_counter()
                first = first or now
                last = now
                n += 1
        rec.update(ok=True, ttft=(first or t0) - t0, latency=(last or t0) - t0, out=n,
                   tpot=((last - first) / (n - 1)) if n > 1 else 0.0)
    except Exception as e:
        rec.update(ok=False, error=str(e))


def pct(v, p):
    s = sorted(v)
    return s[min(len(s) - 1, int(p / 100.0 * len(s)))] if s else 0.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--num_prompts", type=int, default=100)
    ap.add_argument("--request_rate", type=float, default=float("inf"))
    ap.add_argument("--input_len", type=int, default=512)
    ap.add_argument("--output_len", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--shared_prefix_len", type=int, default=0,
                    help="the first N tokens are the same in every prompt (a system prompt): what automatic prefix reuse "
                         "(XFT_PREFIX_CACHE=1 on the server) saves")
    a = ap.parse_args()
    rng = random.Random(a.seed)
    shared = [rng.randrange(5, a.vocab) for _ in range(min(a.shared_prefix_len, a.input_len))]
    prompts = [shared + [rng.randrange(5, a.vocab) for _ in range(a.input_len - len(shared))] for _ in range(a.num_prompts)]
    recs = [dict(inp=len(p)) for p in prompts]
    threads = []
    t0 = time.perf_counter()
    for p, rec in zip(prompts, recs):
        th = threading.Thread(target=one_request, args=(a.url, p, a.output_len, rec))
        th.start()
        threads.append(th)
        if a.request_rate != float("inf"):
            time.sleep(rng.expovariate(a.request_rate))
    for th in threads:
        th.join()
    dt = time.perf_counter() - t0
    ok = [r for r in recs if r.get("ok")]
    ttft = [r["ttft"] * 1e3 for r in ok]
    tpot = [r["tpot"] * 1e3 for r in ok if r["out"] > 1]
    res = {
        "successful_requests": len(ok), "failed_requests": len(recs) - len(ok), "duration_s": round(dt, 3),
        "request_throughput_per_s": round(len(ok) / dt, 3),
        "input_token_throughput_per_s": round(sum(r["inp"] for r in ok) / dt, 1),
        "output_token_throughput_per_s": round(sum(r["out"] for r in ok) / dt, 1),
        "mean_ttft_ms": round(statistics.mean(ttft), 2) if ttft else 0, "median_ttft_ms": round(statistics.median(ttft), 2) if ttft else 0,
        "p99_ttft_ms": round(pct(ttft, 99), 2),
        "mean_tpot_ms": round(statistics.mean(tpot), 2) if tpot else 0, "median_tpot_ms": round(statistics.median(tpot), 2) if tpot else 0,
        "p99_tpot_ms": round(pct(tpot, 99), 2),
    }
    print(json.dumps(res, indent=1))
    return res


if __name__ == "__main__":
    main()
