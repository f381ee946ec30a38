#!/usr/bin/env python
"""Token-id serving launcher (reference: ``serving/grpc_launcher/server.py:70-152``): rank 0 serves ``predict`` /
``predict_stream`` / ``health`` over gRPC; every other rank sits in ``model.follow()`` (the reference:
``while True: model.generate()``) and executes what rank 0 broadcasts.  Messages are JSON objects with the fields of ``xft.proto``.

    python serving/server.py --model_path <dir> --dtype bf16 --port 50051
    torchrun --nproc-per-node 8 ... serving/server.py --model_path <dir> --dtype bf16

`Client` is a matching minimal client.  Also usable without gRPC as an HTTP JSON endpoint (``--http``).
"""
import argparse
import json
import os
import sys
import threading
from concurrent import futures

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

SERVICE = "xft.XFastertransformerService"
_enc = lambda o: json.dumps(o).encode()
_dec = lambda b: json.loads(b.decode()) if b else {}


class Servicer:
    def __init__(self, model, defaults=None):
        self.model = model
        self.lock = threading.Lock()      # one generation at a time: the engine state is per request
        # generation settings of the launcher's command line (the reference fixes them there, server.py:67-73); a request
        # that carries a field overrides it
        self.defaults = dict(num_beams=1, do_sample=False, temperature=1.0, top_k=50, top_p=1.0, repetition_penalty=1.0,
                             output_len=None)
        self.defaults.update(defaults or {})

    def _kwargs(self, q):
        d = self.defaults
        max_length = q.get("max_length")
        if max_length is None:
            bs = int(q.get("batch_size", 1))
            max_length = len(q["Ids"]) // max(bs, 1) + d["output_len"] if d["output_len"] else 128
        kw = dict(max_length=max_length, num_beams=q.get("num_beams", d["num_beams"]), do_sample=q.get("do_sample", d["do_sample"]),
                  temperature=q.get("temperature", d["temperature"]), top_k=q.get("top_k", d["top_k"]), top_p=q.get("top_p", d["top_p"]),
                  repetition_penalty=q.get("repetition_penalty", d["repetition_penalty"]), eos_token_id=q.get("eos_token_id", -1),
                  pad_token_id=q.get("pad_token_id", -1))
        return kw

    def _ids(self, q):
        import torch
        bs = int(q.get("batch_size", 1))
        ids = torch.tensor(q["Ids"], dtype=torch.int64).view(bs, -1)
        return ids

    def predict(self, q, ctx=None):
        with self.lock:
            out = self.model.generate(self._ids(q), **self._kwargs(q))
        return {"Ids": out.flatten().tolist(), "batch_size": out.shape[0], "seq_len": out.shape[1]}

    def predict_stream(self, q, ctx=None):
        with self.lock:
            self.model.set_input(self._ids(q), **self._kwargs(q))
            try:
                sent = None
                while not self.model.is_done():
                    t = self.model.forward()
                    seqs = getattr(getattr(self.model, "model", None), "working", None)
                    if not seqs or len(seqs) != t.shape[0]:
                        yield {"Ids": t.flatten().tolist(), "batch_size": t.shape[0], "seq_len": 1}
                        continue
                    # a step may produce several tokens per sequence (XFT_SPEC_NGRAM): send them all; rows that got
                    # fewer are padded with -1 and `counts` says how many are real
                    sent = sent or [0] * len(seqs)
                    new = [s.generated[n:] for s, n in zip(seqs, sent)]
                    new = [r if r else [int(t[i])] for i, r in enumerate(new)]          # finished rows keep emitting eos
                    sent = [max(len(s.generated), n) for s, n in zip(seqs, sent)]
                    w = max(len(r) for r in new)
                    msg = {"Ids": [x for r in new for x in r + [-1] * (w - len(r))], "batch_size": len(new), "seq_len": w}
                    if w > 1:
                        msg["counts"] = [len(r) for r in new]
                    yield msg
            finally:
                # a client that left early must not leave the follower ranks ahead of rank 0: they run the request to
                # its end, so rank 0 does too
                while not self.model.is_done():
                    self.model.forward()
                self.model.finalize()

    def health(self, q=None, ctx=None):
        return {"status": "SERVING"}


def serve_grpc(model, port: int, workers: int = 4, defaults=None):
    import grpc
    sv = Servicer(model, defaults)
    handlers = {
        "predict": grpc.unary_unary_rpc_method_handler(sv.predict, request_deserializer=_dec, response_serializer=_enc),
        "predict_stream": grpc.unary_stream_rpc_method_handler(sv.predict_stream, request_deserializer=_dec,
                                                               response_serializer=_enc),
        "health": grpc.unary_unary_rpc_method_handler(sv.health, request_deserializer=_dec, response_serializer=_enc),
    }
    server = grpc.server(futures.ThreadPoolExecutor(max_workers=workers))
    server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(SERVICE, handlers),))
    bound = server.add_insecure_port(f"[::]:{port}")
    server.start()
    return server, bound


def serve_http(model, port: int, defaults=None):
    from http.server import BaseHTTPRequestHandler, HTTPServer
    sv = Servicer(model, defaults)

    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_GET(self):
            body = _enc(sv.health())
            self.send_response(200); self.send_header("Content-Type", "application/json"); self.end_headers(); self.wfile.write(body)

        def do_POST(self):
            n_body = int(self.headers.get("Content-Length", 0))
            if n_body > (16 << 20):
                self.send_response(413)
                self.end_headers()
                return
            raw = self.rfile.read(n_body)
            try:
                body, code = _enc(sv.predict(_dec(raw))), 200
            except Exception as e:      # report, keep serving
                body, code = _enc({"error": str(e)}), 400
            self.send_response(code); self.send_header("Content-Type", "application/json"); self.end_headers(); self.wfile.write(body)

    httpd = HTTPServer(("0.0.0.0", port), H)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    return httpd, httpd.server_address[1]


class Client:
    def __init__(self, target: str):
        import grpc
        self.ch = grpc.insecure_channel(target)
        mk = lambda n, stream=False: (self.ch.unary_stream if stream else self.ch.unary_unary)(
            f"/{SERVICE}/{n}", request_serializer=_enc, response_deserializer=_dec)
        self._predict, self._stream, self._health = mk("predict"), mk("predict_stream", True), mk("health")

    def predict(self, ids, **kw):
        bs = len(ids)
        return self._predict(dict(Ids=[t for r in ids for t in r], batch_size=bs, **kw))

    def predict_stream(self, ids, **kw):
        return self._stream(dict(Ids=[t for r in ids for t in r], batch_size=len(ids), **kw))

    def health(self):
        return self._health({})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model_path", required=True)
    ap.add_argument("-d", "--dtype", default="bf16")
    ap.add_argument("--kv_cache_dtype", default="fp16")
    ap.add_argument("--port", type=int, default=50051)
    ap.add_argument("--http", action="store_true")
    # the reference's launcher fixes the generation settings on its command line (serving/grpc_launcher/server.py:67-73);
    # here they are the defaults of requests that do not carry the field
    boolean = lambda v: str(v).lower() == "true"
    ap.add_argument("--num_beams", type=int, default=1)
    ap.add_argument("--output_len", type=int, default=None, help="tokens to generate beyond the prompt when a request has no max_length")
    ap.add_argument("--do_sample", type=boolean, default=False)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top_p", type=float, default=1.0)
    ap.add_argument("--top_k", type=int, default=50)
    ap.add_argument("--rep_penalty", type=float, default=1.0)
    a = ap.parse_args()
    defaults = dict(num_beams=a.num_beams, output_len=a.output_len, do_sample=a.do_sample, temperature=a.temperature, top_p=a.top_p,
                    top_k=a.top_k, repetition_penalty=a.rep_penalty)
    import xfastertransformer_b200 as xft
    model = xft.AutoModel.from_pretrained(a.model_path, dtype=a.dtype, kv_cache_dtype=a.kv_cache_dtype)
    if model.rank != 0:
        model.follow()                   # follower: execute whatever rank 0 calls (exits on shutdown)
        return
    if a.http:
        srv, port = serve_http(model, a.port, defaults)
        print(f"HTTP serving on :{port}", flush=True)
        threading.Event().wait()
    else:
        srv, port = serve_grpc(model, a.port, defaults=defaults)
        print(f"gRPC serving on :{port}", flush=True)
        srv.wait_for_termination()


if __name__ == "__main__":
    main()
