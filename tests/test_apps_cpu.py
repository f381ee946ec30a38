"""Apps around the engine on the CPU path: serving launcher (gRPC + HTTP), offline continuous-batching scheduler,
evaluation adapter, benchmark CLI, timeline, MLServer runtime object."""
import json
import math
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


def _run_script(path, argv, capsys):
    """main() of an example script in this process (a new interpreter costs ten seconds of imports)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("script_" + os.path.basename(path).replace(".", "_"), path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    old = sys.argv
    sys.argv = [path] + list(argv)
    try:
        capsys.readouterr()
        mod.main()
    finally:
        sys.argv = old
    return capsys.readouterr().out


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
        # the command-line client (serving/client.py): health poll, unary and streaming calls on token ids
        import contextlib
        import io
        from serving import client as cli
        for extra in ([], ["--stream"]):
            buf = io.StringIO()
            with contextlib.redirect_stdout(buf):
                assert cli.main(["--port", str(port), "--ids", "5 6 7 8", "--max_length", "10", *extra]) == 0
            assert [int(t) for t in buf.getvalue().split()] == want[0, 4:].tolist()
    finally:
        srv.stop(0)
    from serving import client as cli
    assert cli.main(["--port", "1", "--ids", "5", "--health_timeout", "0.5"]) == 1      # nobody serves there
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
    # several requests per forward (ragged lengths) give the same numbers as one by one
    pairs = [(ids[:10].tolist(), greedy), (ids[:5].tolist(), ids[5:9].tolist()), (ids[3:20].tolist(), ids[20:22].tolist()),
             (ids[:10].tolist(), ids[10:13].tolist())]
    ev.batch_size = 3
    batch = ev.loglikelihood_batch(pairs)
    for (c, t), (bl, bg) in zip(pairs, batch):
        sl, sg = ev.loglikelihood_tokens(c, t)
        assert abs(sl - bl) < 1e-3 * max(1.0, abs(sl)) and sg == bg
    assert batch[0][1] and abs(batch[0][0] - ll) < 1e-3 * abs(ll)
    # rolling log-likelihood: windows add up to the sum over the text; consistent with the perplexity
    ev.max_length = 16
    total = ev.rolling_loglikelihood(ids.tolist())
    assert total < 0
    ev.max_length = 64
    whole = ev.rolling_loglikelihood(ids.tolist())
    assert abs(math.exp(-whole / (ids.numel() - 1)) - perplexity(model, ids, window=64)) < 1e-2 * perplexity(model, ids, window=64)
    # greedy generation cut at a stop string ("text" = ids joined by spaces)
    dec = lambda t: " ".join(map(str, t))
    full = ev.generate_until(ids[:10].tolist(), dec, [], 6)
    assert full.split() == [str(t) for t in model.generate(ids[None, :10], max_length=16)[0, 10:].tolist()]
    stop = " " + full.split()[2]
    assert ev.generate_until(ids[:10].tolist(), dec, [stop], 6) == " ".join(full.split()[:2])


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


def test_lora_finetune_reduces_loss_and_merges(tmp_path):
    """finetune/llama/finetune.py on a tiny random Llama (CPU, pre-tokenised data): loss falls, the adapter is saved,
    the merged checkpoint differs from the base only in the wrapped projections and converts to an engine model."""
    import importlib.util
    import json
    import transformers
    spec = importlib.util.spec_from_file_location("ft", os.path.join(ROOT, "finetune", "llama", "finetune.py"))
    ft = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ft)
    cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=64)
    torch.manual_seed(0)
    base = transformers.LlamaForCausalLM(cfg)
    bdir = str(tmp_path / "base")
    base.save_pretrained(bdir, safe_serialization=True)
    g = torch.Generator().manual_seed(0)
    pattern = torch.randint(3, 128, (12,), generator=g).tolist()
    with open(tmp_path / "data.jsonl", "w") as f:
        for i in range(32):
            ids = (pattern * 3)[i % 5:i % 5 + 24]
            f.write(json.dumps({"input_ids": ids}) + "\n")
    out = str(tmp_path / "out")
    args = ft.parse(["--base_model", bdir, "--data_path", str(tmp_path / "data.jsonl"), "--output_dir", out, "--cpu",
                     "--batch_size", "8", "--micro_batch_size", "8", "--max_steps", "30", "--learning_rate", "2e-2",
                     "--warmup_steps", "2", "--lora_r", "8", "--lora_dropout", "0", "--merge", "--logging_steps", "100",
                     "--lora_target_modules", "q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"])
    res = ft.train(args)
    assert res["last_loss"] < 0.9 * res["first_loss"], res      # frozen random embeddings bound what LoRA can reach
    ad = torch.load(os.path.join(out, "adapter_model.pt"))
    assert len(ad) == 7 * 2 * 2 and all(v.abs().sum() > 0 for k, v in ad.items() if "lora_B" in k)
    merged = transformers.LlamaForCausalLM.from_pretrained(os.path.join(out, "merged"))
    sd0, sd1 = base.state_dict(), merged.state_dict()
    changed = {k for k in sd0 if not torch.equal(sd0[k], sd1[k])}
    assert changed and all("_proj" in k for k in changed), changed
    from xfastertransformer_b200 import LlamaConvert
    conv = LlamaConvert().convert(os.path.join(out, "merged"), str(tmp_path / "xft"), dtype="fp32")
    assert os.path.exists(os.path.join(conv, "config.ini"))


def test_openai_server_continuous_batching(tmp_path):
    """serving/openai_server.py on the CPU engine with token-id prompts: concurrent /v1/completions requests are batched
    by the scheduler and return what a lone greedy generate() returns; streaming, /v1/models, /metrics, errors."""
    import importlib.util
    import threading
    spec = importlib.util.spec_from_file_location("oai", os.path.join(ROOT, "serving", "openai_server.py"))
    oai = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(oai)
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=500), seed=3, dtype="fp32", std=0.1)
    model = xft.AutoModel.from_pretrained(d, dtype="bf16")
    prompts = [[5, 9, 100, 42, 7], [11, 12, 13], [400, 3, 77, 8, 19, 21, 6], [50, 60]]
    want = [model.generate(torch.tensor([p]), max_length=len(p) + 6)[0, len(p):].tolist() for p in prompts]
    httpd, sched, port = oai.serve(model, 0, max_batch=8, prefill_per_step=2, model_name="tiny")
    base = f"http://127.0.0.1:{port}"

    def post(path, body):
        req = urllib.request.Request(base + path, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
        try:
            with urllib.request.urlopen(req, timeout=120) as r:
                return r.status, r.read()
        except urllib.error.HTTPError as e:
            return e.code, e.read()

    try:
        got = [None] * len(prompts)

        def one(i):
            code, body = post("/v1/completions", {"prompt": prompts[i], "max_tokens": 6})
            assert code == 200, body
            got[i] = json.loads(body)

        ths = [threading.Thread(target=one, args=(i,)) for i in range(len(prompts))]
        [t.start() for t in ths]
        [t.join() for t in ths]
        for i, r in enumerate(got):
            assert r["choices"][0]["token_ids"] == want[i], (i, r, want[i])
            assert r["usage"]["prompt_tokens"] == len(prompts[i]) and r["usage"]["completion_tokens"] == 6
        # streaming returns the same tokens as server-sent events
        code, body = post("/v1/completions", {"prompt": prompts[0], "max_tokens": 6, "stream": True})
        assert code == 200
        chunks = [json.loads(l[6:])["choices"][0] for l in body.decode().split("\n\n") if l.startswith("data: {")]
        toks = [c["token_ids"][0] for c in chunks if c["token_ids"]]
        assert toks == want[0] and body.decode().strip().endswith("[DONE]")
        assert chunks[-1]["finish_reason"] == "length" and all(c["finish_reason"] is None for c in chunks[:-1])
        # n choices, several prompts, echo, log-probabilities, repetition penalty, stop strings (ids joined by spaces
        # are the "text" when no tokenizer is loaded)
        code, body = post("/v1/completions", {"prompt": [prompts[0], prompts[1]], "max_tokens": 6, "n": 2, "logprobs": 3})
        r = json.loads(body)
        assert code == 200 and [c["index"] for c in r["choices"]] == [0, 1, 2, 3]
        assert [c["token_ids"] for c in r["choices"]] == [want[0], want[0], want[1], want[1]]      # greedy: n copies agree
        lp = r["choices"][0]["logprobs"]
        assert len(lp["token_logprobs"]) == 6 and all(x <= 0 for x in lp["token_logprobs"])
        assert all(len(t) == 3 and abs(max(t.values()) - l) < 1e-6 for t, l in zip(lp["top_logprobs"], lp["token_logprobs"]))
        assert r["usage"]["completion_tokens"] == 24
        stop_at = f" {want[0][2]} "
        code, body = post("/v1/completions", {"prompt": prompts[0], "max_tokens": 6, "stop": [stop_at.strip()], "echo": True})
        c = json.loads(body)["choices"][0]
        assert c["finish_reason"] == "stop" and c["token_ids"] == want[0][:3]
        assert c["text"].split() == [str(t) for t in prompts[0] + want[0][:2]]
        code, body = post("/v1/completions", {"prompt": prompts[0], "max_tokens": 6, "repetition_penalty": 50.0})
        pen = json.loads(body)["choices"][0]["token_ids"]
        assert code == 200 and len(set(pen)) == 6 and not set(pen) & set(prompts[0])     # a huge penalty forbids repeats
        assert post("/v1/completions", {"prompt": prompts[0], "n": 2, "stream": True})[0] == 400
        # malformed and oversized bodies are refused, the server keeps serving
        bad = urllib.request.Request(base + "/v1/completions", data=b"{not json", headers={"Content-Type": "application/json"})
        try:
            urllib.request.urlopen(bad, timeout=30)
            assert False, "malformed JSON must not be accepted"
        except urllib.error.HTTPError as e:
            assert e.code == 400
        import http.client
        conn = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
        conn.putrequest("POST", "/v1/completions")
        conn.putheader("Content-Length", str(oai.MAX_BODY_BYTES + 1))
        conn.endheaders()
        assert conn.getresponse().status == 413
        conn.close()
        assert post("/v1/completions", {"prompt": prompts[1], "max_tokens": 2})[0] == 200
        # text prompt without a tokenizer, and a prompt longer than the model: 400, server keeps serving
        assert post("/v1/completions", {"prompt": "hello"})[0] == 400
        assert post("/v1/completions", {"prompt": [1] * 40, "max_tokens": 100000})[0] == 400
        assert json.loads(urllib.request.urlopen(base + "/v1/models").read())["data"][0]["id"] == "tiny"
        m = urllib.request.urlopen(base + "/metrics").read().decode()
        assert "xft_finished 12" in m and "xft_generated_tokens 65" in m
        assert sched.metrics["steps"] < 12 * 7         # requests shared engine steps
        # nothing leaks: every sequence was freed and every KV block is back in the pool
        eng = model.model
        assert not sched.running and not eng.pool.seqs and not eng.cache.tables
        assert eng.cache.alloc.num_free == eng.cache.alloc.num_blocks
    finally:
        sched.shutdown()
        httpd.shutdown()


def test_benchmark_serving_client(tmp_path, capsys):
    """benchmarks/benchmark_serving.py against the in-process OpenAI server: all requests succeed, TTFT/TPOT reported."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("oai", os.path.join(ROOT, "serving", "openai_server.py"))
    oai = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(oai)
    spec = importlib.util.spec_from_file_location("bs", os.path.join(ROOT, "benchmarks", "benchmark_serving.py"))
    bs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bs)
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=500), seed=4, dtype="fp32", std=0.1)
    model = xft.AutoModel.from_pretrained(d, dtype="bf16")
    httpd, sched, port = oai.serve(model, 0, max_batch=8, prefill_per_step=4)
    try:
        old = sys.argv
        sys.argv = ["benchmark_serving.py", "--url", f"http://127.0.0.1:{port}", "--num_prompts", "6", "--input_len", "12",
                    "--output_len", "5", "--vocab", "500"]
        res = bs.main()
        sys.argv = old
        assert res["successful_requests"] == 6 and res["failed_requests"] == 0
        assert res["output_token_throughput_per_s"] > 0 and res["mean_ttft_ms"] > 0 and res["mean_tpot_ms"] > 0
    finally:
        sched.shutdown()
        httpd.shutdown()


def test_chat_prompt_formats():
    """examples/web_demo/prompts.py: the per-family chat formats."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("prompts", os.path.join(ROOT, "examples", "web_demo", "prompts.py"))
    P = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(P)
    h = [("hi", "hello")]
    assert P.build_prompt("llama2", h, "how are you?") == "<s>[INST] hi [/INST] hello </s><s>[INST] how are you? [/INST]"
    assert P.build_prompt("llama2", [], "q", "be brief").startswith("<s>[INST] <<SYS>>\nbe brief\n<</SYS>>\n\nq [/INST]")
    l3 = P.build_prompt("llama3", h, "x")
    assert l3.startswith("<|begin_of_text|><|start_header_id|>user<|end_header_id|>\n\nhi<|eot_id|>")
    assert l3.endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")
    q = P.build_prompt("qwen2", h, "x")
    assert q.count("<|im_start|>") == 5 and q.endswith("<|im_start|>assistant\n")
    assert P.build_prompt("chatglm2", h, "x") == "[Round 1]\n\n问：hi\n\n答：hello\n\n[Round 2]\n\n问：x\n\n答："
    assert P.build_prompt("chatglm", [], "x") == "x"
    assert P.build_prompt("chatglm3", h, "x").endswith("<|user|>\n x<|assistant|>")
    assert P.build_prompt("baichuan2", h, "x") == "<reserved_106>hi<reserved_107>hello<reserved_106>x<reserved_107>"
    assert P.build_prompt("gemma", [], "x") == "<bos><start_of_turn>user\nx<end_of_turn>\n<start_of_turn>model\n"
    with pytest.raises(KeyError):
        P.build_prompt("nope", [], "x")
    # per-family demo settings: every family of the reference's demo files has a launcher, a known prompt format, and its
    # end-of-turn strings resolve to token ids only when the tokenizer knows them as one token
    for fn, fam in (("Llama2", "llama2"), ("Llama3", "llama3"), ("Qwen", "qwen"), ("Qwen2", "qwen2"), ("Yi", "yi"),
                    ("ChatGLM", "chatglm"), ("ChatGLM2", "chatglm2"), ("ChatGLM3", "chatglm3"), ("ChatGLM4", "chatglm4"),
                    ("Baichuan2", "baichuan2"), ("Gemma", "gemma")):
        src = open(os.path.join(ROOT, "examples", "web_demo", fn + ".py")).read()
        assert f'main("{fam}")' in src
        assert P.FAMILIES[fam]["chat_format"] in P.FORMATS and P.FAMILIES[fam]["max_rounds"] >= 1

    class Tok:
        unk_token_id, eos_token_id = 0, 2

        def convert_tokens_to_ids(self, s):
            return {"<|eot_id|>": 9}.get(s, 0)
    assert P.stop_token_ids(Tok(), "llama3") == [9, 2] and P.stop_token_ids(Tok(), "gemma") == [2]


def test_bench_reference_arm_prints_unavailable_line():
    """`bench.py --impl reference` prints exactly one JSON line saying why the reference cannot run here and exits 0."""
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "4",
                        "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and d["unavailable"]


def test_bench_cli_contract_flags():
    """The driver's command line (`--gpus N --steps K --warmup W`) parses, and unknown models fail with a clear message."""
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--model", "--batch", "--input-len", "--dtype"):
        assert flag in r.stdout, flag


def test_openai_server_mixed_prefill_decode_steps(tmp_path):
    """--mixed_steps: prompts admitted while others decode share one forward with them; outputs stay those of a lone
    greedy generate()."""
    import importlib.util
    import threading
    spec = importlib.util.spec_from_file_location("oai", os.path.join(ROOT, "serving", "openai_server.py"))
    oai = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(oai)
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=500), seed=6, dtype="fp32", std=0.1)
    model = xft.AutoModel.from_pretrained(d, dtype="bf16")
    prompts = [[5, 9, 100, 42, 7], [11, 12, 13], [400, 3, 77, 8, 19, 21, 6], [50, 60], [7, 7, 7, 9]]
    want = [model.generate(torch.tensor([p]), max_length=len(p) + 8)[0, len(p):].tolist() for p in prompts]
    httpd, sched, port = oai.serve(model, 0, max_batch=8, prefill_per_step=1, model_name="tiny", mixed_steps=True)
    base = f"http://127.0.0.1:{port}"
    got = [None] * len(prompts)

    def one(i):
        req = urllib.request.Request(base + "/v1/completions", data=json.dumps({"prompt": prompts[i], "max_tokens": 8}).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            got[i] = json.loads(r.read())

    try:
        ths = [threading.Thread(target=one, args=(i,)) for i in range(len(prompts))]
        [t.start() for t in ths]
        [t.join() for t in ths]
        for i, r in enumerate(got):
            assert r["choices"][0]["token_ids"] == want[i], (i, r["choices"][0]["token_ids"], want[i])
        assert sched.metrics["mixed_steps"] >= 1
    finally:
        sched.shutdown()
        httpd.shutdown()


def test_openai_server_drops_a_request_whose_client_left(tmp_path):
    """A streaming client that closes its connection: the handler marks the request, the scheduler frees it at the next
    token instead of generating all max_tokens, and the engine is clean afterwards."""
    import importlib.util
    import socket
    import time
    spec = importlib.util.spec_from_file_location("oai", os.path.join(ROOT, "serving", "openai_server.py"))
    oai = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(oai)
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=500), seed=3, dtype="fp32", std=0.1)
    model = xft.AutoModel.from_pretrained(d, dtype="bf16")
    httpd, sched, port = oai.serve(model, 0, max_batch=4, model_name="tiny")
    try:
        body = json.dumps({"prompt": [5, 9, 100], "max_tokens": 1500, "stream": True}).encode()
        s = socket.create_connection(("127.0.0.1", port), timeout=30)
        s.sendall(b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: "
                  + str(len(body)).encode() + b"\r\n\r\n" + body)
        got = b""
        while got.count(b"data: ") < 3:                 # a few tokens arrive, then the client leaves
            got += s.recv(4096)
        s.setsockopt(socket.SOL_SOCKET, socket.SO_LINGER, b"\x01\x00\x00\x00\x00\x00\x00\x00")      # reset on close
        s.close()
        t0 = time.time()
        while sched.metrics["cancelled"] == 0 and time.time() - t0 < 60:
            time.sleep(0.05)
        assert sched.metrics["cancelled"] == 1 and sched.metrics["generated_tokens"] < 1500
        t0 = time.time()
        while sched.running and time.time() - t0 < 10:
            time.sleep(0.05)
        eng = model.model
        assert not sched.running and not eng.cache.tables and eng.cache.alloc.num_free == eng.cache.alloc.num_blocks
    finally:
        sched.shutdown()
        httpd.shutdown()


def test_openai_server_chunked_prefill(tmp_path):
    """--prefill_chunk: long prompts are fed in pieces between the decode steps of the running sequences; every request
    still returns what a lone greedy generate() returns, sampled requests included, and nothing leaks."""
    import importlib.util
    import threading
    spec = importlib.util.spec_from_file_location("oai", os.path.join(ROOT, "serving", "openai_server.py"))
    oai = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(oai)
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=500), seed=3, dtype="fp32", std=0.1)
    model = xft.AutoModel.from_pretrained(d, dtype="bf16")
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(5, 490, (n,), generator=g).tolist() for n in (50, 7, 33, 16, 70, 3)]
    want = [model.generate(torch.tensor([p]), max_length=len(p) + 5)[0, len(p):].tolist() for p in prompts]
    httpd, sched, port = oai.serve(model, 0, max_batch=8, prefill_per_step=2, model_name="tiny", prefill_chunk=16)
    base = f"http://127.0.0.1:{port}"

    def post(body):
        req = urllib.request.Request(base + "/v1/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            return json.loads(r.read())

    try:
        got = [None] * len(prompts)

        def one(i):
            got[i] = post({"prompt": prompts[i], "max_tokens": 5})

        ths = [threading.Thread(target=one, args=(i,)) for i in range(len(prompts))]
        [t.start() for t in ths]
        [t.join() for t in ths]
        for i, r in enumerate(got):
            assert r["choices"][0]["token_ids"] == want[i], (i, r["choices"][0]["token_ids"], want[i])
        # 50, 33 and 70 tokens at 16 per piece: 4 + 3 + 5 pieces
        assert sched.metrics["prefill_chunks"] == 12 and sched.metrics["prompt_tokens"] == sum(map(len, prompts))
        # a request that needs the logits (log-probabilities) through the chunked path
        r = post({"prompt": prompts[0], "max_tokens": 5, "logprobs": 1})
        assert r["choices"][0]["token_ids"] == want[0] and len(r["choices"][0]["logprobs"]["token_logprobs"]) == 5
        eng = model.model
        assert not sched.running and not sched.prefilling and not eng.cache.tables
        assert eng.cache.alloc.num_free == eng.cache.alloc.num_blocks
        # back-pressure: with a queue limit, a burst beyond it is refused with 429 and counted
        sched.max_queue = 1
        req = urllib.request.Request(base + "/v1/completions", data=json.dumps({"prompt": [prompts[1]] * 3, "max_tokens": 2}).encode(),
                                     headers={"Content-Type": "application/json"})
        try:
            urllib.request.urlopen(req, timeout=30)
            assert False, "three prompts must not fit a queue of one"
        except urllib.error.HTTPError as e:
            assert e.code == 429
        assert sched.metrics["rejected"] == 3 and post({"prompt": prompts[1], "max_tokens": 2})["choices"][0]["token_ids"] == want[1][:2]
    finally:
        sched.shutdown()
        httpd.shutdown()


@pytest.mark.parametrize("ranks", [1, 2])
def test_openai_server_process_serves_and_stops_on_sigterm(tiny, ranks):
    """serving/openai_server.py as a process (alone, and with a follower rank under torchrun): answers /health and a
    completion, then SIGTERM ends every rank cleanly."""
    import signal
    import socket
    import time
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, XFT_ENGINE="CPU", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    server = [os.path.join(ROOT, "serving", "openai_server.py"), "--model_path", tiny, "--no_warmup", "--port", str(port)]
    if ranks == 1:
        cmd = [sys.executable] + server
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}", "--master-addr",
               "127.0.0.1", "--master-port", "29691"] + server
    p = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, start_new_session=True)
    try:
        base = f"http://127.0.0.1:{port}"
        t0 = time.time()
        while True:
            try:
                if json.loads(urllib.request.urlopen(base + "/health", timeout=2).read())["status"] == "ok":
                    break
            except Exception:
                assert p.poll() is None and time.time() - t0 < 120, "server did not come up"
                time.sleep(0.3)
        req = urllib.request.Request(base + "/v1/completions", data=json.dumps({"prompt": [5, 6, 7, 8], "max_tokens": 4}).encode(),
                                     headers={"Content-Type": "application/json"})
        r = json.loads(urllib.request.urlopen(req, timeout=60).read())
        assert len(r["choices"][0]["token_ids"]) == 4
        if ranks == 1:
            p.send_signal(signal.SIGTERM)
        else:
            # torchrun forwards the signal to its workers; rank 0 then releases the follower
            os.killpg(os.getpgid(p.pid), signal.SIGTERM)
        out, _ = p.communicate(timeout=60)
        if ranks == 1:
            assert p.returncode == 0, out[-2000:]
    finally:
        if p.poll() is None:
            os.killpg(os.getpgid(p.pid), signal.SIGKILL)
            p.wait()


def test_server_warmup_walks_every_bucket_and_leaves_the_cache_clean(tiny):
    """Scheduler.warmup on a stand-in runner (the real one needs a GPU): one short session per batch bucket plus one
    prompt-sized prefill, every sequence freed again."""
    import importlib.util
    from xfastertransformer_b200.runtime.cuda_runner import CudaRunner
    spec = importlib.util.spec_from_file_location("oai", os.path.join(ROOT, "serving", "openai_server.py"))
    oai = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(oai)
    model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    eng = model.model

    class StandIn:
        enabled = True
        fixed_width = None
        bucket = staticmethod(CudaRunner.bucket)
        seen = []

        def can_run(self, seqs, cfg):
            self.seen.append(len(seqs))
            return False

        def reset(self):
            pass
    eng.runner = StandIn()
    sched = oai.Scheduler(model, max_batch=20, prefill_per_step=2)
    n = sched.warmup(max_context=300)
    assert n == len({CudaRunner.bucket(b) for b in range(1, 21)}) == 7
    assert eng.runner.fixed_width == (eng.cache.blocks_for(301) + 7) // 8 * 8
    assert sorted(set(eng.runner.seen)) == [1, 2, 4, 8, 12, 16, 24]
    assert not eng.cache.tables and not eng.pool.seqs and eng.cache.alloc.num_free == eng.cache.alloc.num_blocks


def test_grpc_stream_carries_every_token_under_speculative_decoding(tiny, monkeypatch):
    """predict_stream with XFT_SPEC_NGRAM on: steps that emit several tokens send them all (rows padded with -1, `counts`
    says how many are real); the concatenation equals generate()."""
    from serving.server import Servicer
    from xfastertransformer_b200.runtime.engine import Model
    from xfastertransformer_b200.utils.flags import Env
    plain = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    ids = torch.randint(5, 790, (2, 12), generator=torch.Generator().manual_seed(9))
    want = plain.generate(ids, max_length=12 + 20)
    rows = {tuple(r[:12].tolist()): r.tolist() for r in want}

    def oracle(self, s, k):                      # row 0 always gets two right drafts, row 1 none
        tokens = s.all_tokens()
        full = rows[tuple(tokens[:12])]
        return full[len(tokens):len(tokens) + 2] if full == rows[tuple(ids[0].tolist())] else []
    monkeypatch.setenv("XFT_SPEC_NGRAM", "4")
    Env.get().reload()
    try:
        model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
        monkeypatch.setattr(Model, "_draft_for", oracle)
        sv = Servicer(model)
        got = [[], []]
        widths = set()
        for msg in sv.predict_stream({"Ids": ids.flatten().tolist(), "batch_size": 2, "max_length": 32}):
            w = msg["seq_len"]
            widths.add(w)
            cnt = msg.get("counts", [w] * 2)
            for i in range(2):
                got[i] += msg["Ids"][i * w:i * w + cnt[i]]
        assert 3 in widths
        eos_free = lambda r: [t for t in r if t != -1]
        assert eos_free(got[0])[:20] == want[0, 12:].tolist() and eos_free(got[1])[:20] == want[1, 12:].tolist()
    finally:
        monkeypatch.delenv("XFT_SPEC_NGRAM")
        Env.get().reload()


def test_openai_server_emits_every_token_of_a_speculative_step(tmp_path, monkeypatch):
    """XFT_SPEC_NGRAM in the serving scheduler: a decode step that accepted drafts hands all its tokens to the request,
    in order; requests stop exactly where plain greedy decoding stops (max_tokens in the middle of an accepted run,
    a stop token inside it); the cache ends empty."""
    import importlib.util
    import threading
    from xfastertransformer_b200.runtime.engine import Model
    from xfastertransformer_b200.utils.flags import Env
    spec = importlib.util.spec_from_file_location("oai", os.path.join(ROOT, "serving", "openai_server.py"))
    oai = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(oai)
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=500), seed=5, dtype="fp32", std=0.1)
    model = xft.AutoModel.from_pretrained(d, dtype="bf16")
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(5, 490, (n,), generator=g).tolist() for n in (12, 5, 9)]
    full = {tuple(p): p + model.generate(torch.tensor([p]), max_length=len(p) + 14)[0, len(p):].tolist() for p in prompts}
    want = [full[tuple(p)][len(p):] for p in prompts]

    def oracle(self, s, k):                      # the true continuation, with every fourth draft position falsified
        toks = s.all_tokens()
        ref = full[tuple(toks[:len(s.prompt)])]
        dr = ref[len(toks):len(toks) + k]
        return [t if (len(toks) + i) % 4 else (t + 1) % 500 for i, t in enumerate(dr)]

    monkeypatch.setenv("XFT_SPEC_NGRAM", "3")
    Env.get().reload()
    monkeypatch.setattr(Model, "_draft_for", oracle)
    httpd, sched, port = oai.serve(model, 0, max_batch=8, model_name="tiny")
    base = f"http://127.0.0.1:{port}"

    def post(body):
        req = urllib.request.Request(base + "/v1/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            return json.loads(r.read())

    try:
        lens = [14, 7, 10]
        got = [None] * len(prompts)

        def one(i):
            got[i] = post({"prompt": prompts[i], "max_tokens": lens[i]})

        ths = [threading.Thread(target=one, args=(i,)) for i in range(len(prompts))]
        [t.start() for t in ths]
        [t.join() for t in ths]
        for i, r in enumerate(got):
            assert r["choices"][0]["token_ids"] == want[i][:lens[i]], (i, r["choices"][0]["token_ids"], want[i])
        eng = model.model
        assert sched.metrics["spec_tokens"] > 0 and eng.spec_accepted >= sched.metrics["spec_tokens"]
        # fewer engine steps than tokens: one prefill per request group, then decode steps that emit several tokens
        assert sched.metrics["steps"] < sum(lens)
        # a stop token inside an accepted run ends the request there
        stop_at = want[0][6]
        first = want[0].index(stop_at)
        r = post({"prompt": prompts[0], "max_tokens": 14, "stop_token_ids": [stop_at]})
        assert r["choices"][0]["token_ids"] == want[0][:first + 1], (r["choices"][0]["token_ids"], want[0], stop_at)
        assert not sched.running and not eng.cache.tables
        assert eng.cache.alloc.num_free == eng.cache.alloc.num_blocks
    finally:
        sched.shutdown()
        httpd.shutdown()
        monkeypatch.delenv("XFT_SPEC_NGRAM")
        Env.get().reload()


def test_benchmark_prompt_sources_of_the_reference(tiny, tmp_path):
    """benchmarks/benchmark.py takes the reference's flag names (--token_in / --token_out, --input_prompt, --prompt_path
    with .json / .txt / .sonnet files, --sonnet_prefix_len / --sonnet_count, --padding): prompts are cut or repeated to
    the token count; the sonnet prompts share their first --sonnet_prefix_len tokens and differ after them."""
    import argparse
    import importlib.util
    import json as json_mod
    spec = importlib.util.spec_from_file_location("bench_cli", os.path.join(ROOT, "benchmarks", "benchmark.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    class Tok:                                   # a word-level stand-in for a Hugging Face tokenizer
        def __call__(self, text, add_special_tokens=True):
            return {"input_ids": ([1] if add_special_tokens else []) + [3 + (hash(w) % 200) for w in text.split()]}

    a = argparse.Namespace(input_tokens=24, batch_size=3, input_prompt=None, sonnet_prefix_len=10, sonnet_count=4)
    poem = tmp_path / "poem.sonnet"
    poem.write_text("\n".join("line %d of the poem has a few words in it" % i for i in range(40)) + "\n")
    ids = mod.build_prompt_ids(Tok(), a, str(poem), json_mod)
    assert ids.shape == (4, 24)
    assert all(torch.equal(ids[r, :10], ids[0, :10]) for r in range(4)) and len({tuple(r.tolist()) for r in ids}) == 4
    txt = tmp_path / "p.txt"
    txt.write_text("first prompt here\nsecond one is a little longer than that\n")
    ids = mod.build_prompt_ids(Tok(), a, str(txt), json_mod)
    assert ids.shape == (3, 24) and not torch.equal(ids[0], ids[1]) and torch.equal(ids[0], ids[2])
    js = tmp_path / "p.json"
    js.write_text(json_mod.dumps({"24": "exact entry for twenty four tokens", "long_unit": "filler words "}))
    ids = mod.build_prompt_ids(Tok(), a, str(js), json_mod)
    assert ids.shape == (3, 24) and torch.equal(ids[0], ids[1])
    a.input_prompt = "an explicit prompt"
    assert mod.build_prompt_ids(Tok(), a, str(js), json_mod).shape == (3, 24)
    with pytest.raises(ValueError):
        a.input_prompt = None
        mod.build_prompt_ids(Tok(), a, str(tmp_path / "p.csv"), json_mod)
    # the reference's spelling of the length flags on the command line
    r = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", "benchmark.py"), "--model_path", tiny, "--dtype", "bf16",
                        "--batch_size", "1", "--token_in", "8", "--token_out", "3", "--iteration", "1", "--warmup", "0", "--padding", "False"],
                       env=dict(os.environ, XFT_ENGINE="CPU"), capture_output=True, text=True, timeout=600, cwd=str(tmp_path))
    assert r.returncode == 0 and "input_tokens: 8" in r.stdout.replace("  ", " ").replace("  ", " "), r.stdout[-800:] + r.stderr[-800:]


def test_demo_takes_the_reference_command_line(tiny, tmp_path, capsys):
    """examples/pytorch/demo.py with the reference's spelling of the boolean options (`--streaming False --chat False
    --do_sample True --padding False`, examples/pytorch/demo.py:61-74 there) and with bare flags."""
    demo = os.path.join(ROOT, "examples", "pytorch", "demo.py")
    for extra in (["--streaming", "False", "--chat", "False", "--do_sample", "True", "--top_k", "3", "--padding", "False", "-o", "4"],
                  ["--streaming", "--output_len", "4"]):
        out = _run_script(demo, ["-m", tiny, "-d", "bf16", "--ids", "5 6 7 8"] + extra, capsys)
        assert "[4 tokens in" in out, out[-800:]
    sys.path.insert(0, os.path.dirname(demo))
    import argparse
    from demo import boolean_string
    assert boolean_string("True") is True and boolean_string("false") is False and boolean_string(True) is True
    with pytest.raises(argparse.ArgumentTypeError):
        boolean_string("maybe")


def test_text_modes_of_the_example_scripts(tmp_path, capsys):
    """examples/pytorch/demo_offline_cb.py and prefix_sharing.py with the reference's text options (-t tokenizer, -i prompt
    file, -s sorted answers; --input / --prefix_len / --output_len): a small byte-level BPE tokenizer trained here stands
    in for a model's."""
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    from transformers import PreTrainedTokenizerFast
    from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    corpus = ["Once upon a time, there existed a little girl who liked to have adventures.", "The capital of France is Paris.",
              "Explain why the sky is blue. Write a haiku about the sea. List three prime numbers."] * 4
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=400, special_tokens=["<|endoftext|>"],
                                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    tdir = str(tmp_path / "tok")
    PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<|endoftext|>").save_pretrained(tdir)
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=512), seed=0, dtype="bf16", std=0.05)
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("The capital of France is\n\nWrite a haiku about the sea.\nList three prime numbers.\n")
    out = _run_script(os.path.join(ROOT, "examples", "pytorch", "demo_offline_cb.py"),
                      ["-m", d, "-t", tdir, "-i", str(prompts), "-s", "--output_len", "4", "--kv_cache_dtype", "fp16"], capsys)
    shown = [l for l in out.splitlines() if l.startswith("[")]
    assert [l[:3] for l in shown] == ["[0]", "[1]", "[2]"] and "'The capital of France is'" in shown[0]      # -s: in prompt order
    assert "3 requests" in out
    out = _run_script(os.path.join(ROOT, "examples", "pytorch", "prefix_sharing.py"),
                      ["-m", d, "-t", tdir, "--prefix_len", "70", "--output_len", "4", "--streaming", "False", "--padding", "False"], capsys)
    assert "identical: True" in out, out[-800:]


def test_launcher_defaults_from_the_command_line(tiny):
    """serving/server.py: the reference fixes the generation settings on the launcher's command line (--output_len,
    --num_beams, --do_sample, ...); here they are the defaults of requests that do not carry the field."""
    import xfastertransformer_b200 as xft
    from serving.server import Servicer
    model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    sv = Servicer(model, dict(output_len=3, num_beams=2))
    kw = sv._kwargs({"Ids": [5, 6, 7, 8, 9, 10], "batch_size": 2})
    assert kw["max_length"] == 3 + 3 and kw["num_beams"] == 2 and kw["top_k"] == 50
    kw = sv._kwargs({"Ids": [5, 6, 7], "max_length": 9, "num_beams": 1})
    assert kw["max_length"] == 9 and kw["num_beams"] == 1
    out = sv.predict({"Ids": [5, 6, 7, 8], "batch_size": 1, "num_beams": 1})
    assert out["seq_len"] == 4 + 3
    assert Servicer(model)._kwargs({"Ids": [1, 2]})["max_length"] == 128
