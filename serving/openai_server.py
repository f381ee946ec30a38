#!/usr/bin/env python
"""OpenAI-compatible HTTP server with an in-process continuous-batching scheduler.

The reference reaches this surface through its vLLM fork (``serving/vllm-xft.md``: an OpenAI API server on rank 0, slave
entry points on the other ranks).  Here the scheduler is part of the repository: one thread owns the engine and drives
``set_input_cb`` / ``forward_cb`` / ``free_seqs`` — waiting prompts are admitted between decode steps, all running
sequences decode together, finished ones free their KV blocks — while HTTP handler threads only enqueue requests and
read their token streams.  Ranks other than 0 follow rank 0's control messages, as in ``serving/server.py``.

    python serving/openai_server.py --model_path <dir> [--token_path <hf tokenizer dir>] --port 8000
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 serving/openai_server.py --model_path <dir> ...

Endpoints: ``POST /v1/completions``, ``POST /v1/chat/completions`` (both with ``stream``), ``GET /v1/models``,
``GET /health``, ``GET /metrics`` (Prometheus text: requests, tokens, TTFT and per-token latency sums).  ``prompt`` may
be a string (needs a tokenizer) or a list of token ids (answered with ``token_ids`` next to ``text``).
"""
from __future__ import annotations

import argparse
import json
import os
import queue
import sys
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, List, Optional

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


MAX_BODY_BYTES = 16 << 20          # a request body larger than this is refused with 413


class Request:
    def __init__(self, prompt_ids: List[int], max_tokens: int, temperature: float, top_p: float, top_k: int,
                 stop_ids: List[int], seed: Optional[int], repetition_penalty: float = 1.0,
                 logprobs: Optional[int] = None, stop_fn=None):
        self.id = uuid.uuid4().hex[:24]
        self.prompt_ids = prompt_ids
        self.max_tokens = max(1, max_tokens)
        self.temperature, self.top_p, self.top_k = temperature, top_p, top_k
        self.stop_ids = set(stop_ids)
        self.seed = seed
        self.repetition_penalty = float(repetition_penalty)
        self.logprobs = logprobs                      # None, or how many alternatives to report per position (0 = chosen only)
        self.stop_fn = stop_fn                        # callable(generated ids) -> bool: a stop string has appeared
        self.cancelled = False                        # set by the handler when the client went away
        self.fed = 0                                  # chunked prefill: prompt tokens already given to the engine
        self.token_logprobs: List[float] = []
        self.top_logprobs: List[Dict[int, float]] = []
        self.out: "queue.Queue" = queue.Queue()       # ints, then None (or an Exception) at the end
        self.generated: List[int] = []
        self.finish_reason = "length"
        self.t_arrive = time.perf_counter()
        self.t_first: Optional[float] = None
        self.t_last: Optional[float] = None

    @property
    def greedy_on_device(self) -> bool:
        """True when the token can be picked on the device: arg-max, no penalty, no log-probabilities wanted."""
        return self.temperature <= 1e-5 and self.repetition_penalty == 1.0 and self.logprobs is None


class Scheduler(threading.Thread):
    """Continuous batching on one engine.  ``max_batch`` bounds the running set, ``prefill_per_step`` the prompts
    admitted between two decode steps (a long queue must not starve the running sequences)."""

    def __init__(self, model, max_batch: int = 64, prefill_per_step: int = 4, eos_id: int = -1):
        super().__init__(daemon=True)
        import torch
        self.torch = torch
        self.model = model
        self.max_batch, self.prefill_per_step, self.eos_id = max_batch, prefill_per_step, eos_id
        self.waiting: "queue.Queue[Request]" = queue.Queue()
        self.running: Dict[int, Request] = {}
        self.stop_flag = threading.Event()
        self.metrics = dict(requests=0, finished=0, prompt_tokens=0, generated_tokens=0, ttft_sum=0.0, tpot_sum=0.0,
                            tpot_count=0, steps=0, mixed_steps=0, errors=0, cancelled=0, prefill_chunks=0, rejected=0, spec_tokens=0)
        self.mixed_steps = False          # prefill new prompts in the same forward as the running sequences' decode
        self.max_queue = 0                # > 0: requests beyond this many waiting ones are refused with 429
        self.prefill_chunk = 0            # > 0: prompts longer than this are fed in pieces of this many tokens, one piece
        #                                   per scheduler turn, so a long prompt does not stall the running sequences
        self.prefilling: Dict[int, Request] = {}      # sequences whose prompt is still being fed (req.fed tokens so far)
        self.max_len = int(getattr(model.model.cfg, "max_pos_seq_len", 0) or 0)
        self.kv_fraction = 0.8            # share of the free device memory the warm-up gives to the KV pools

    def warmup(self, max_context: int = 0) -> int:
        """Capture the decode CUDA graphs of every batch bucket up to ``max_batch`` before the first request arrives
        (a capture costs an eager step plus the capture itself, which would otherwise land on live requests).  All
        graphs share one block-table width, sized for ``max_context`` tokens.  Returns the number of buckets run."""
        runner = getattr(self.model.model, "runner", None)
        if runner is None or not getattr(runner, "enabled", False):
            return 0
        cache = self.model.model.cache
        ctx = max_context or self.max_len or 4096
        runner.fixed_width = (cache.blocks_for(ctx + 1) + 7) // 8 * 8
        # Size the KV pools once, now: a pool that grows under load moves, and every captured graph would have to be
        # captured again.  kv_fraction of the free device memory, capped at what max_batch full contexts need.
        try:
            free, _ = self.torch.cuda.mem_get_info(self.model.model.ctx.device)
            want = min(int(self.kv_fraction * free) // max(cache.bytes_per_block(), 1),
                       self.max_batch * cache.blocks_for(ctx + 1) + 8)
            if want > cache.alloc.num_blocks:
                cache.ensure_blocks(want)
        except Exception:
            pass
        sizes = sorted({runner.bucket(n) for n in range(1, self.max_batch + 1)})
        for b in sizes:
            sids = self.model.set_input_cb([[1, 2, 3, 4]] * b, None, [16] * b, greedy=True)
            toks = self.model.forward_cb_greedy()
            for _ in range(3):                       # eager, capture, replay
                self.model.set_input_cb([[int(t)] for t in toks], sids, None, greedy=True)
                toks = self.model.forward_cb_greedy()
            self.model.free_seqs(sids)
        # one prompt-sized prefill as well: the first request should not pay for the first use of the prefill kernels
        n = max(8, min(512, ctx - 16))
        sids = self.model.set_input_cb([[1 + (i % 7) for i in range(n)]], None, [n + 8], greedy=True)
        self.model.forward_cb_greedy()
        self.model.free_seqs(sids)
        return len(sizes)

    # -- API for handler threads ------------------------------------------------------------
    def submit(self, req: Request) -> Request:
        self.metrics["requests"] += 1
        self.waiting.put(req)
        return req

    def shutdown(self):
        self.stop_flag.set()
        self.waiting.put(None)

    # -- token selection on the host (one row of fp32 logits) --------------------------------
    def _select(self, req: Request, row) -> int:
        torch = self.torch
        row = row.float()
        if req.repetition_penalty != 1.0:
            seen = torch.tensor(sorted(set(req.prompt_ids) | set(req.generated)), dtype=torch.long, device=row.device)
            seen = seen[seen < row.numel()]
            v = row[seen]
            row = row.clone()
            row[seen] = torch.where(v < 0, v * req.repetition_penalty, v / req.repetition_penalty)
        tok = self._pick(req, row)
        if req.logprobs is not None:
            lp = torch.log_softmax(row, -1)
            req.token_logprobs.append(float(lp[tok]))
            k = min(int(req.logprobs), 20)
            top = torch.topk(lp, k) if k > 0 else None
            req.top_logprobs.append({int(i): float(x) for x, i in zip(top.values, top.indices)} if top is not None else {})
        return tok

    def _pick(self, req: Request, row) -> int:
        torch = self.torch
        if req.temperature <= 1e-5:
            return int(row.argmax())
        logits = row / req.temperature
        if req.top_k > 0 and req.top_k < logits.numel():
            kth = torch.topk(logits, req.top_k).values[-1]
            logits = torch.where(logits < kth, torch.full_like(logits, float("-inf")), logits)
        probs = torch.softmax(logits, -1)
        if req.top_p < 1.0:
            sp, si = torch.sort(probs, descending=True)
            keep = (torch.cumsum(sp, 0) - sp) < req.top_p
            keep[0] = True
            mask = torch.zeros_like(probs, dtype=torch.bool)
            mask[si[keep]] = True
            probs = torch.where(mask, probs, torch.zeros_like(probs))
            probs = probs / probs.sum()
        g = None
        if req.seed is not None:
            g = torch.Generator(device=probs.device).manual_seed(req.seed + len(req.generated))
        return int(torch.multinomial(probs, 1, generator=g))

    def _forward(self, reqs: List[Request], greedy: bool) -> List[int]:
        """One engine step for `reqs` (already announced with set_input_cb).  All-greedy batches pick their tokens on
        the device (decode steps replay the CUDA graph); otherwise the logits come back and each request samples."""
        if greedy:
            return [int(t) for t in self.model.forward_cb_greedy()]
        logits = self.model.forward_cb()
        # a request whose prompt is still being fed has no token to pick yet
        return [self._select(r, row) if r.fed >= len(r.prompt_ids) else -1 for r, row in zip(reqs, logits)]

    def _emit(self, req: Request, tok: int) -> bool:
        """Record a token; returns True when the request is finished."""
        now = time.perf_counter()
        if req.t_first is None:
            req.t_first = now
            self.metrics["ttft_sum"] += now - req.t_arrive
        else:
            self.metrics["tpot_sum"] += now - req.t_last
            self.metrics["tpot_count"] += 1
        req.t_last = now
        req.generated.append(tok)
        self.metrics["generated_tokens"] += 1
        req.out.put(tok)
        if req.cancelled:                          # the client closed its stream: stop spending steps on it
            req.finish_reason = "cancelled"
            self.metrics["cancelled"] += 1
            return True
        if tok == self.eos_id or tok in req.stop_ids or (req.stop_fn is not None and req.stop_fn(req.generated)):
            req.finish_reason = "stop"
            return True
        return len(req.generated) >= req.max_tokens

    def _finish(self, sids: List[int]):
        if not sids:
            return
        self.model.free_seqs(sids)
        for s in sids:
            r = self.running.pop(s)
            self.metrics["finished"] += 1
            r.out.put(None)

    def _fail(self, reqs: List[Request], err: Exception):
        self.metrics["errors"] += len(reqs)
        for r in reqs:
            r.out.put(err)

    # -- the loop ---------------------------------------------------------------------------
    def run(self):
        while not self.stop_flag.is_set():
            admitted: List[Request] = []
            block = not self.running and not self.prefilling
            while len(self.running) + len(self.prefilling) + len(admitted) < self.max_batch and \
                    len(admitted) < self.prefill_per_step:
                try:
                    r = self.waiting.get(block=block and not admitted, timeout=0.2 if block else None)
                except queue.Empty:
                    break
                if r is None:
                    return
                admitted.append(r)
                block = False
            try:
                if admitted:
                    ok = []
                    for r in admitted:
                        total = len(r.prompt_ids) + r.max_tokens + 1
                        if not r.prompt_ids or (self.max_len and total > self.max_len):
                            self._fail([r], ValueError(f"prompt + max_tokens = {total - 1} tokens exceeds the model's "
                                                       f"{self.max_len} positions" if r.prompt_ids else "empty prompt"))
                        else:
                            ok.append(r)
                    long = [r for r in ok if self.prefill_chunk > 0 and len(r.prompt_ids) > self.prefill_chunk]
                    if long:
                        # chunked prefill: the first piece creates the sequence (sized for the whole request); the
                        # rest follows one piece per turn below
                        ok = [r for r in ok if r not in long]
                        c = self.prefill_chunk
                        sids = self.model.set_input_cb([r.prompt_ids[:c] for r in long], None,
                                                       [len(r.prompt_ids) + r.max_tokens + 1 for r in long], greedy=True)
                        for r, sid in zip(long, [int(x) for x in sids]):
                            r.fed = c
                            self.prefilling[sid] = r
                        self.model.forward_cb_greedy()
                        self.metrics["steps"] += 1
                        self.metrics["prefill_chunks"] += len(long)
                    for r in ok:
                        r.fed = len(r.prompt_ids)
                    if ok and self.mixed_steps and self.running:
                        # one forward for the new prompts AND the running sequences: decoding does not pause for prefill
                        sids_run = list(self.running)
                        reqs_run = [self.running[s] for s in sids_run]
                        greedy = all(r.greedy_on_device for r in ok + reqs_run)
                        sids_new = self.model.set_input_cb([r.prompt_ids for r in ok], None,
                                                           [len(r.prompt_ids) + r.max_tokens + 1 for r in ok], greedy=greedy,
                                                           hold=True)
                        self.model.set_input_cb([r.generated[-1] for r in reqs_run], sids_run, None, greedy=greedy, append=True)
                        picks = self._forward(ok + reqs_run, greedy)
                        done = []
                        for r, sid, tok in zip(ok, [int(s) for s in sids_new], picks[:len(ok)]):
                            self.running[sid] = r
                            self.metrics["prompt_tokens"] += len(r.prompt_ids)
                            if self._emit(r, tok):
                                done.append(sid)
                        done += [s for s, r, tok in zip(sids_run, reqs_run, picks[len(ok):]) if self._emit(r, tok)]
                        self._finish(done)
                        self.metrics["steps"] += 1
                        self.metrics["mixed_steps"] += 1
                        continue
                    if ok:
                        greedy = all(r.greedy_on_device for r in ok)
                        sids = self.model.set_input_cb([r.prompt_ids for r in ok], None,
                                                       [len(r.prompt_ids) + r.max_tokens + 1 for r in ok], greedy=greedy)
                        picks = self._forward(ok, greedy)
                        done = []
                        for r, sid, tok in zip(ok, [int(s) for s in sids], picks):
                            self.running[sid] = r
                            self.metrics["prompt_tokens"] += len(r.prompt_ids)
                            if self._emit(r, tok):
                                done.append(sid)
                        self._finish(done)
                        self.metrics["steps"] += 1
                if self.prefilling:
                    self._feed_prompts()
                if self.running:
                    sids = list(self.running)
                    reqs = [self.running[s] for s in sids]
                    greedy = all(r.greedy_on_device for r in reqs)
                    self.model.set_input_cb([r.generated[-1] for r in reqs], sids, None, greedy=greedy)
                    picks = self._forward(reqs, greedy)
                    # with XFT_SPEC_NGRAM the engine may have accepted draft tokens: every request then gets all the
                    # tokens of the step, in order, and stops at the first one that ends it
                    many = getattr(getattr(self.model, "model", None), "cb_emitted", None) if greedy else None
                    if not many or len(many) != len(reqs) or [m[-1] for m in many] != picks:
                        many = [[tok] for tok in picks]
                    done = []
                    for sid, r, toks in zip(sids, reqs, many):
                        self.metrics["spec_tokens"] += len(toks) - 1
                        if any(self._emit(r, t) for t in toks):
                            done.append(sid)
                    self._finish(done)
                    self.metrics["steps"] += 1
            except Exception as e:      # an engine error ends the affected requests, not the server
                known = list(self.running.values()) + list(self.prefilling.values())
                victims = known + [r for r in admitted if r not in known]
                try:
                    if self.running or self.prefilling:
                        self.model.free_seqs(list(self.running) + list(self.prefilling))
                except Exception:
                    pass
                self.running.clear()
                self.prefilling.clear()
                self._fail(victims, e)

    def _feed_prompts(self):
        """Chunked prefill: the next piece of up to ``prefill_per_step`` long prompts, in one forward.  A prompt whose
        last piece went in gets its first token from this forward and joins the running set."""
        c = self.prefill_chunk
        sids = list(self.prefilling)[:self.prefill_per_step]
        gone = [s for s in sids if self.prefilling[s].cancelled]
        if gone:                                        # the client left while its prompt was still being fed
            self.model.free_seqs(gone)
            for s in gone:
                r = self.prefilling.pop(s)
                self.metrics["cancelled"] += 1
                r.finish_reason = "cancelled"
                r.out.put(None)
            sids = [s for s in sids if s not in gone]
        if not sids:
            return
        reqs = [self.prefilling[s] for s in sids]
        pieces = [r.prompt_ids[r.fed:r.fed + c] for r in reqs]
        greedy = all(r.greedy_on_device for r in reqs)
        self.model.set_input_cb(pieces, sids, None, greedy=greedy, extend=True)
        for r, p in zip(reqs, pieces):
            r.fed += len(p)
        picks = self._forward(reqs, greedy)
        self.metrics["steps"] += 1
        self.metrics["prefill_chunks"] += len(sids)
        done = []
        for sid, r, tok in zip(sids, reqs, picks):
            if r.fed >= len(r.prompt_ids):
                del self.prefilling[sid]
                self.running[sid] = r
                self.metrics["prompt_tokens"] += len(r.prompt_ids)
                if self._emit(r, tok):
                    done.append(sid)
        self._finish(done)


class Tokenizer:
    """HF tokenizer when a path is given; otherwise only token-id prompts are accepted and text is the ids joined."""

    def __init__(self, path: str = ""):
        self.tok = None
        if path:
            from transformers import AutoTokenizer
            self.tok = AutoTokenizer.from_pretrained(path)

    def encode(self, prompt) -> List[int]:
        if isinstance(prompt, list):
            if prompt and isinstance(prompt[0], list):
                prompt = prompt[0]
            return [int(t) for t in prompt]
        if self.tok is None:
            raise ValueError("text prompts need --token_path; send a list of token ids instead")
        return self.tok(prompt, add_special_tokens=True)["input_ids"]

    def chat(self, messages) -> List[int]:
        if self.tok is not None and getattr(self.tok, "chat_template", None):
            return self.tok.apply_chat_template(messages, add_generation_prompt=True, tokenize=True)
        text = "".join(f"<|{m.get('role', 'user')}|>\n{m.get('content', '')}\n" for m in messages) + "<|assistant|>\n"
        return self.encode(text)

    def decode(self, ids: List[int]) -> str:
        if self.tok is None:
            return " ".join(str(i) for i in ids)
        return self.tok.decode(ids, skip_special_tokens=True)

    @property
    def eos(self) -> int:
        return self.tok.eos_token_id if self.tok is not None and self.tok.eos_token_id is not None else -1


def make_handler(sched: Scheduler, tok: Tokenizer, model_name: str):
    class H(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, *a):
            pass

        def _json(self, code: int, obj):
            body = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):
            if self.path == "/health":
                wd = getattr(getattr(sched.model, "model", sched.model), "watchdog", None)
                stuck = bool(wd is not None and wd.overdue)        # an engine step is past XFT_STEP_TIMEOUT_S right now
                return self._json(503 if stuck else 200,
                                  {"status": "stuck" if stuck else "ok", "running": len(sched.running),
                                   "waiting": sched.waiting.qsize(), "overdue_steps": wd.trips if wd is not None else 0})
            if self.path == "/v1/models":
                return self._json(200, {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "xft"}]})
            if self.path == "/metrics":
                m = sched.metrics
                lines = [f"xft_{k} {v}" for k, v in m.items()]
                lines.append(f"xft_running {len(sched.running)}")
                idx = getattr(getattr(getattr(sched.model, "model", None), "cache", None), "prefix_index", None)
                if idx is not None:               # automatic prefix reuse (XFT_PREFIX_CACHE=1)
                    lines += [f"xft_prefix_lookups {idx.lookups}", f"xft_prefix_hit_blocks {idx.hit_blocks}",
                              f"xft_prefix_cached_blocks {len(idx.entries)}", f"xft_prefix_evicted_blocks {idx.evicted}"]
                lines.append(f"xft_waiting {sched.waiting.qsize()}")
                body = ("\n".join(lines) + "\n").encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                return self.wfile.write(body)
            self._json(404, {"error": {"message": f"no route {self.path}"}})

        def _prompts(self, q, chat: bool) -> List[List[int]]:
            """One id list per prompt: a string, a list of strings, a list of ids or a list of id lists."""
            if chat:
                return [tok.chat(q.get("messages", []))]
            p = q.get("prompt", "")
            if isinstance(p, list) and p and isinstance(p[0], (str, list)):
                return [tok.encode(x) for x in p]
            return [tok.encode(p)]

        def do_POST(self):
            try:
                n_body = int(self.headers.get("Content-Length", 0))
                if n_body > MAX_BODY_BYTES:
                    return self._json(413, {"error": {"message": f"request body over {MAX_BODY_BYTES} bytes",
                                                      "type": "invalid_request_error"}})
                q = json.loads(self.rfile.read(n_body) or b"{}")
                chat = self.path == "/v1/chat/completions"
                if not chat and self.path != "/v1/completions":
                    return self._json(404, {"error": {"message": f"no route {self.path}"}})
                prompts = self._prompts(q, chat)
                n = max(1, int(q.get("n", 1)))
                stop_ids = [int(s) for s in q.get("stop_token_ids", [])]
                stops = q.get("stop") or []
                stops = [stops] if isinstance(stops, str) else [str(x) for x in stops if x]
                lp = q.get("logprobs")
                if chat:                  # chat API: logprobs is a flag, top_logprobs the count
                    lp = int(q.get("top_logprobs", 0)) if lp else None
                elif lp is not None and lp is not False:
                    lp = int(lp)
                else:
                    lp = None
                if q.get("stream") and (n > 1 or len(prompts) > 1):
                    raise ValueError("stream supports one prompt and n = 1")
                stop_fn = (lambda ids: any(x in tok.decode(ids) for x in stops)) if stops else None
                temp = float(q.get("temperature", 1.0 if q.get("do_sample") else 0.0))
                reqs = []
                for ids in prompts:
                    for k in range(n):
                        seed = q.get("seed")
                        reqs.append(Request(ids, int(q.get("max_tokens", 16)), temp, float(q.get("top_p", 1.0)),
                                            int(q.get("top_k", 0)), stop_ids, None if seed is None else int(seed) + 7919 * k,
                                            float(q.get("repetition_penalty", 1.0)), lp, stop_fn))
            except Exception as e:
                return self._json(400, {"error": {"message": str(e), "type": "invalid_request_error"}})
            if sched.max_queue > 0 and sched.waiting.qsize() + len(reqs) > sched.max_queue:
                sched.metrics["rejected"] += len(reqs)
                return self._json(429, {"error": {"message": f"{sched.waiting.qsize()} requests are already waiting",
                                                  "type": "server_overloaded"}})
            for r in reqs:
                sched.submit(r)
            created = int(time.time())
            kind = "chat.completion" if chat else "text_completion"

            def cut(text: str):
                """Text up to the first stop string, and whether one was found."""
                at = min((text.find(x) for x in stops if x in text), default=-1)
                return (text[:at], True) if at >= 0 else (text, False)

            if q.get("stream"):
                req = reqs[0]
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Connection", "close")
                self.end_headers()
                sent_text = ""
                while True:
                    t = req.out.get()
                    if t is None or isinstance(t, Exception):
                        break
                    if tok.tok:
                        full, hit = cut(tok.decode(req.generated))
                        text = full[len(sent_text):]
                        sent_text = full
                    else:
                        text, hit = str(t) + " ", False
                    if not text and not hit:
                        continue
                    delta = {"delta": {"content": text}} if chat else {"text": text, "token_ids": [t]}
                    chunk = {"id": req.id, "object": kind + ".chunk", "created": created, "model": model_name,
                             "choices": [dict(index=0, finish_reason=None, **delta)]}
                    try:
                        self.wfile.write(b"data: " + json.dumps(chunk).encode() + b"\n\n")
                        self.wfile.flush()
                    except (BrokenPipeError, ConnectionResetError, ConnectionAbortedError):
                        req.cancelled = True       # the scheduler drops the request at its next token
                        self.close_connection = True
                        return
                end = {"id": req.id, "object": kind + ".chunk", "created": created, "model": model_name,
                       "choices": [dict(index=0, finish_reason=req.finish_reason, **({"delta": {}} if chat else {"text": "", "token_ids": []}))]}
                self.wfile.write(b"data: " + json.dumps(end).encode() + b"\n\n")
                self.wfile.write(b"data: [DONE]\n\n")
                self.wfile.flush()
                self.close_connection = True
                return
            err = None
            for req in reqs:
                while True:
                    t = req.out.get()
                    if t is None:
                        break
                    if isinstance(t, Exception):
                        err = t
                        break
            if err is not None:
                return self._json(400 if isinstance(err, ValueError) else 500, {"error": {"message": str(err)}})
            choices = []
            for i, req in enumerate(reqs):
                text, hit = cut(tok.decode(req.generated))
                choice = {"index": i, "finish_reason": "stop" if hit else req.finish_reason}
                if req.logprobs is not None:
                    pieces = [tok.decode([t]) for t in req.generated]
                    if chat:
                        choice["logprobs"] = {"content": [
                            {"token": pc, "logprob": l, "top_logprobs": [{"token": tok.decode([j]), "logprob": x}
                                                                          for j, x in top.items()]}
                            for pc, l, top in zip(pieces, req.token_logprobs, req.top_logprobs)]}
                    else:
                        choice["logprobs"] = {"tokens": pieces, "token_logprobs": req.token_logprobs,
                                              "top_logprobs": [{tok.decode([j]): x for j, x in top.items()}
                                                               for top in req.top_logprobs]}
                if chat:
                    choice["message"] = {"role": "assistant", "content": text}
                else:
                    if q.get("echo"):
                        text = tok.decode(req.prompt_ids) + (" " if not tok.tok else "") + text
                    choice.update(text=text, token_ids=req.generated)
                choices.append(choice)
            n_prompt = sum(len(r.prompt_ids) for r in reqs)
            n_gen = sum(len(r.generated) for r in reqs)
            self._json(200, {"id": reqs[0].id, "object": kind, "created": created, "model": model_name, "choices": choices,
                             "usage": {"prompt_tokens": n_prompt, "completion_tokens": n_gen,
                                       "total_tokens": n_prompt + n_gen}})
    return H


def serve(model, port: int, token_path: str = "", max_batch: int = 64, prefill_per_step: int = 4, model_name: str = "xft",
          warmup: bool = False, max_context: int = 0, mixed_steps: bool = False, prefill_chunk: int = 0,
          max_queue: int = 0):
    """Start scheduler + HTTP server (threads); returns (httpd, scheduler, bound_port)."""
    tok = Tokenizer(token_path)
    sched = Scheduler(model, max_batch, prefill_per_step, eos_id=tok.eos)
    sched.mixed_steps = mixed_steps
    sched.prefill_chunk = max(0, int(prefill_chunk))
    sched.max_queue = max(0, int(max_queue))
    if warmup:
        sched.warmup(max_context)
    sched.start()
    httpd = ThreadingHTTPServer(("0.0.0.0", port), make_handler(sched, tok, model_name))
    httpd.daemon_threads = True
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    return httpd, sched, httpd.server_address[1]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_path", required=True)
    ap.add_argument("--token_path", default="")
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--kv_cache_dtype", default="fp16")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--max_batch", type=int, default=64)
    ap.add_argument("--prefill_per_step", type=int, default=4)
    ap.add_argument("--no_warmup", action="store_true", help="do not pre-capture the decode graphs of every batch bucket")
    ap.add_argument("--max_context", type=int, default=0, help="longest prompt + output the graphs are sized for")
    ap.add_argument("--max_queue", type=int, default=0, help="refuse requests with 429 beyond this many waiting ones (0 = no limit)")
    ap.add_argument("--prefill_chunk", type=int, default=0,
                    help="feed prompts longer than this many tokens in pieces, one per scheduler turn (0 = whole prompts)")
    ap.add_argument("--mixed_steps", action="store_true",
                    help="prefill new prompts in the same forward as the running sequences (lower time per output token "
                         "under load; the step runs eagerly instead of replaying the decode graph)")
    a = ap.parse_args()
    import xfastertransformer_b200 as xft
    model = xft.AutoModel.from_pretrained(a.model_path, dtype=a.dtype, kv_cache_dtype=a.kv_cache_dtype)
    if model.rank != 0:
        model.follow_cb()                # follower ranks mirror rank 0's engine calls until shutdown
        return
    httpd, sched, port = serve(model, a.port, a.token_path, a.max_batch, a.prefill_per_step,
                               os.path.basename(a.model_path.rstrip("/")), warmup=not a.no_warmup,
                               max_context=a.max_context, mixed_steps=a.mixed_steps, prefill_chunk=a.prefill_chunk,
                               max_queue=a.max_queue)
    print(f"OpenAI-compatible server on :{port}", flush=True)
    # SIGTERM / Ctrl-C: stop accepting, let the scheduler finish its turn, release the follower ranks
    import signal
    stop = threading.Event()
    for sig in (signal.SIGINT, signal.SIGTERM):
        signal.signal(sig, lambda *_: stop.set())
    stop.wait()
    httpd.shutdown()
    sched.shutdown()
    sched.join(timeout=30)
    model.model.exit_slaves()


if __name__ == "__main__":
    main()
