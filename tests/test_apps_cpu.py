"""Apps around the engine on the CPU path: serving launcher (gRPC + HTTP), offline continuous-batching scheduler,
evaluation adapter, benchmark CLI, timeline, MLServer runtime object."""
import json
import os
import subprocess
import sys
import urllib.request

import pytest
import torch

import xfastertransformer_b200 as xft
from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


@pytest.fixture(autouse=True)
def _cpu(monkeypatch):
    monkeypatch.setenv("XFT_ENGINE", "CPU")


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("tiny"))
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=800), seed=0, dtype="bf16", std=0.08)
    return d


def test_grpc_and_http_serving(tiny):
    from serving.server import Client, serve_grpc, serve_http
    model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    want = model.generate(torch.tensor([[5, 6, 7, 8], [9, 10, 11, 12]]), max_length=10)
    srv, port = serve_grpc(model, 0)
    try:
        c = Client(f"127.0.0.1:{port}")
        assert c.health()["status"] == "SERVING"
        r = c.predict([[5, 6, 7, 8], [9, 10, 11, 12]], max_length=10)
        assert torch.equal(torch.tensor(r["Ids"]).view(2, -1), want)
        steps = list(c.predict_stream([[5, 6, 7, 8]], max_length=10))
        assert [s["Ids"][0] for s in steps] == want[0, 4:].tolist()
    finally:
        srv.stop(0)
    httpd, hport = serve_http(model, 0)
    try:
        req = urllib.request.Request(f"http://127.0.0.1:{hport}/", data=json.dumps(
            {"Ids": [5, 6, 7, 8], "batch_size": 1, "max_length": 10}).encode(), method="POST")
        r = json.loads(urllib.request.urlopen(req, timeout=60).read())
        assert r["Ids"] == want[0].tolist()
    finally:
        httpd.shutdown()


def test_offline_cb_scheduler_matches_batch_generate(tiny):
    sys.path.insert(0, os.path.join(ROOT, "examples", "pytorch"))
    from demo_offline_cb import run
    model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    prompts = [[5, 6, 7], [9, 10, 11, 12, 13, 14], [20, 21], [30, 31, 32, 33], [40] * 9]
    outs, steps = run(model, prompts, max_batch=3, output_len=6, prefill_per_step=2)
    for p, o in zip(prompts, outs):
        want = model.generate(torch.tensor([p]), max_length=len(p) + 6)[0, len(p):].tolist()
        assert o == want
    assert model.model.cache.alloc.num_free == model.model.cache.alloc.num_blocks


def test_eval_adapter_and_perplexity(tiny):
    sys.path.insert(0, os.path.join(ROOT, "evaluation"))
    from eval import XFTEvalModel, perplexity
    model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    ids = torch.randint(0, 800, (40,), generator=torch.Generator().manual_seed(0))
    ppl = perplexity(model, ids, window=16)
    assert 1.0 < ppl < 5000
    ev = XFTEvalModel(model)
    greedy = model.generate(ids[None, :10], max_length=13)[0, 10:].tolist()
    ll, is_greedy = ev.loglikelihood_tokens(ids[:10].tolist(), greedy)
    assert is_greedy and ll < 0
    ll2, g2 = ev.loglikelihood_tokens(ids[:10].tolist(), [(greedy[0] + 1) % 800] + greedy[1:])
    assert ll2 < ll and not g2


def test_benchmark_cli_and_timeline(tiny, tmp_path):
    csvf = str(tmp_path / "b.csv")
    env = dict(os.environ, XFT_ENGINE="CPU", XFT_TIMELINE="1", XFT_TIMELINE_WHITELIST="Decoder.forward,1st Token,Next Token")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", "benchmark.py"), "-m", tiny, "-d", "bf16", "-bs", "2",
                        "-in", "16", "-out", "6", "-i", "2", "-w", "1", "--csv", csvf], env=env, capture_output=True,
                       text=True, timeout=600, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    assert "throughput_tokens_per_s" in r.stdout and "first_token_avg_ms" in r.stdout
    rows = open(csvf).read().strip().splitlines()
    assert len(rows) == 2 and rows[0].startswith("model,dtype")
    traces = [f for f in os.listdir(tmp_path) if f.startswith("timeline_") and f.endswith(".json")]
    assert traces, "finalize() must dump the chrome trace when XFT_TIMELINE=1"
    ev = json.load(open(os.path.join(tmp_path, traces[0])))["traceEvents"]
    names = {e["name"] for e in ev}
    assert names <= {"Decoder.forward", "1st Token", "Next Token"} and "Next Token" in names
    assert all(e["ph"] == "X" and e["dur"] >= 0 for e in ev)


def test_mlserver_runtime_object(tiny):
    from serving.mlserver_runtime import XFTRuntime
    rt = XFTRuntime(model_path=tiny, dtype="bf16", max_length=9)
    assert rt.load_sync()
    out = rt.predict_ids([[5, 6, 7, 8]])
    assert out.shape == (1, 9)
