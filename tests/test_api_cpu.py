"""API behaviour on the CPU path: continuous-batching invariance, prefix sharing, sampling and beams through the
engine, max_length semantics, hybrid dtypes, quantised dtypes, int8 KV, model-family smoke matrix, fault handling."""
import os

import pytest
import torch

import xfastertransformer_b200 as xft
from xfastertransformer_b200.config import ModelConfig
from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint


@pytest.fixture(autouse=True)
def _cpu(monkeypatch):
    monkeypatch.setenv("XFT_ENGINE", "CPU")


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("tiny"))
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=1000), seed=0, dtype="bf16", std=0.08)
    return d


def _greedy_stream(model, prompt, n):
    """Decode one sequence alone through the CB API; returns its n tokens."""
    sid = model.set_input_cb([prompt], None, 128)
    toks = []
    logits = model.forward_cb()
    for _ in range(n):
        t = int(logits[0].argmax())
        toks.append(t)
        model.set_input_cb([t], sid, 128)
        logits = model.forward_cb()
    model.free_seqs(sid)
    return toks


def test_continuous_batching_invariance(tiny):
    """The reference's cb_check scenario (examples/cpp/cb_check.cpp:373-455): the same prompt submitted at three
    different moments, batched with the others at different depths, must emit identical streams."""
    m = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    prompt = [5, 17, 99, 200, 3, 42, 7]
    want = _greedy_stream(m, prompt, 8)
    streams = {0: [], 1: [], 2: []}
    ids = {}
    last = {}

    def prefill(k):
        sid = m.set_input_cb([prompt], None, 128)
        ids[k] = int(sid[0])
        lg = m.forward_cb()
        last[k] = int(lg[0].argmax())
        streams[k].append(last[k])

    def decode(keys):
        m.set_input_cb([last[k] for k in keys], [ids[k] for k in keys], 128)
        lg = m.forward_cb()
        for i, k in enumerate(keys):
            last[k] = int(lg[i].argmax())
            streams[k].append(last[k])

    prefill(0); decode([0]); decode([0])
    prefill(1); decode([0, 1])
    prefill(2); decode([0, 1, 2]); decode([0, 1, 2])
    m.free_seqs([ids[0]])
    while len(streams[2]) < 8:
        decode([1, 2])
    m.free_seqs([ids[1], ids[2]])
    for k in streams:
        n = min(len(streams[k]), 8)
        assert streams[k][:n] == want[:n], (k, streams[k], want)
    assert m.model.cache.alloc.num_free == m.model.cache.alloc.num_blocks, "all KV blocks returned"


def test_prefix_sharing_same_tokens(tiny):
    m = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    g = torch.Generator().manual_seed(4)
    prefix = torch.randint(0, 1000, (1, 64), generator=g)
    tail = torch.randint(0, 1000, (2, 9), generator=g)
    ids = torch.cat([prefix.expand(2, -1), tail], 1)
    base = m.generate(ids, max_length=85)
    m.prefix_sharing(prefix)
    shared = m.generate(ids, max_length=85)
    assert m.model.prefix_seq is not None
    m.disable_prefix_sharing()
    assert torch.equal(base, shared)


def test_max_length_counts_the_prompt_and_eos_stops(tiny):
    m = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    ids = torch.randint(0, 1000, (2, 10), generator=torch.Generator().manual_seed(5))
    out = m.generate(ids, max_length=14)
    assert out.shape == (2, 14)
    first = int(out[0, 10])
    out2 = m.generate(ids, max_length=20, eos_token_id=first, pad_token_id=0)
    assert out2.shape[1] <= 20 and int(out2[0, 10]) == first
    assert (out2[0, 11:] == first).all() or (out2[0, 11:] == 0).all()      # finished row is padded


def test_sampling_seeded_and_beams(tiny):
    m = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    ids = torch.randint(0, 1000, (2, 8), generator=torch.Generator().manual_seed(6))
    a = m.generate(ids, max_length=16, do_sample=True, top_k=20, top_p=0.9, temperature=0.8, seed=11)
    b = m.generate(ids, max_length=16, do_sample=True, top_k=20, top_p=0.9, temperature=0.8, seed=11)
    c = m.generate(ids, max_length=16, do_sample=True, top_k=20, top_p=0.9, temperature=0.8, seed=12)
    assert torch.equal(a, b) and not torch.equal(a, c)
    greedy = m.generate(ids, max_length=16)
    beams = m.generate(ids, max_length=16, num_beams=3)
    assert beams.shape == (2, 16) and torch.equal(beams[:, :8], ids)
    one = m.generate(ids, max_length=16, num_beams=1)
    assert torch.equal(one, greedy)
    rp = m.generate(ids, max_length=16, repetition_penalty=1.5)
    assert rp.shape == (2, 16)
    assert m.model.cache.alloc.num_free == m.model.cache.alloc.num_blocks


@pytest.mark.parametrize("dtype", ["fp16", "int8", "w8a8", "int4", "nf4", "bf16_int8", "w8a8_nf4"])
@pytest.mark.parametrize("kv", ["fp16", "int8"])
def test_dtype_matrix(tiny, dtype, kv):
    """The reference's CI matrix (ci/test_case:47-112) as a correctness check: quantised models track the bf16 one."""
    ids = torch.randint(0, 1000, (2, 12), generator=torch.Generator().manual_seed(7))
    base = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    want = base(ids)
    m = xft.AutoModel.from_pretrained(tiny, dtype=dtype, kv_cache_dtype=kv)
    got = m(ids)
    rel = (got - want).abs().max().item() / want.abs().max().item()
    assert rel < (0.6 if "4" in dtype else 0.2), rel
    assert m.generate(ids, max_length=16).shape == (2, 16)


FAMILIES = {
    "llama": {}, "yarn_llama": dict(), "gemma": dict(activation_type="gelu"), "qwen": dict(seq_length=64),
    "qwen2": {}, "qwen3": dict(do_qk_norm=True), "baichuan": {}, "chatglm2": dict(kv_head_num=2),
    "chatglm3": dict(kv_head_num=2), "chatglm4": dict(kv_head_num=2), "gpt": dict(activation_type="relu"),
    "telechat": {}, "chatglm": dict(activation_type="gelu"),
}


@pytest.mark.parametrize("mt", sorted(FAMILIES))
def test_family_smoke_and_decode_consistency(mt, tmp_path):
    """Every registered family loads a synthetic checkpoint, and incremental decoding reproduces the full-prefill
    logits (KV cache, RoPE variant, masks and positions agree between the two paths)."""
    kw = dict(model_type=mt, num_layer=2, hidden_size=128, head_num=4, kv_head_num=4, size_per_head=32, inter_size=256,
              vocab_size=512, max_pos_seq_len=256, activation_type="silu", weight_data_type="fp32", start_id=1, end_id=2)
    kw.update(FAMILIES[mt])
    cfg = ModelConfig(**kw)
    if mt == "yarn_llama":
        cfg.rope.scaling_type, cfg.rope.scaling_factor, cfg.rope.original_max_pos = "yarn", 4.0, 64
    d = str(tmp_path / mt)
    write_synthetic_checkpoint(d, cfg, seed=1, dtype="fp32", std=0.1)
    m = xft.AutoModel.from_pretrained(d, dtype="bf16")
    ids = torch.randint(5, 500, (1, 20), generator=torch.Generator().manual_seed(8))
    if mt == "chatglm":
        ids[0, -2], ids[0, -1] = 130001 % 512, 130004 % 512      # shape-only stand-ins (ids above vocab are illegal here)
    full = m(ids)[0]                                                # [20, vocab]
    sid = m.set_input_cb([ids[0, :12].tolist()], None, 64)
    lg = m.forward_cb()
    if mt != "chatglm":                                             # ChatGLM-1's prefix mask makes prompt logits context-dependent
        assert torch.allclose(lg[0], full[11], atol=2e-3, rtol=2e-3), (lg[0] - full[11]).abs().max()
        for t in range(12, 20):
            m.set_input_cb([int(ids[0, t])], sid, 64)
            lg = m.forward_cb()
            assert torch.allclose(lg[0], full[t], atol=2e-3, rtol=2e-3), (t, (lg[0] - full[t]).abs().max())
    m.free_seqs(sid)
    assert m.generate(ids, max_length=24).shape == (1, 24)


def test_baichuan_alibi_and_fake_model(tmp_path, monkeypatch):
    cfg = ModelConfig(model_type="baichuan", num_layer=2, hidden_size=128, head_num=4, kv_head_num=4, size_per_head=32,
                      inter_size=256, vocab_size=512, max_pos_seq_len=0, activation_type="silu", weight_data_type="bf16")
    d = str(tmp_path / "b13")
    cfg.to_ini(d)
    monkeypatch.setenv("XFT_FAKE_MODEL", "2")       # weights drawn in memory, config.ini only
    from xfastertransformer_b200.utils.flags import Env
    Env._inst = None
    m = xft.AutoModel.from_pretrained(d, dtype="bf16")
    assert m.model.decoder.spec.alibi and m.model.decoder.slopes is not None
    assert m.generate(torch.randint(0, 512, (2, 9)), max_length=12).shape == (2, 12)


def test_faults_are_errors_not_crashes(tiny, tmp_path):
    import shutil
    bad = str(tmp_path / "bad")
    shutil.copytree(tiny, bad)
    f = os.path.join(bad, "model.layers.0.mlp.down_proj.weight.0.bin")
    with open(f, "r+b") as fh:
        fh.truncate(os.path.getsize(f) // 2)                      # truncated tensor file
    with pytest.raises(ValueError, match="expected"):
        xft.AutoModel.from_pretrained(bad, dtype="bf16")
    with pytest.raises(Exception, match="don't support"):
        xft.AutoModel.from_pretrained(tiny, dtype="fp64")
    with pytest.raises(Exception, match="KV cache"):
        xft.AutoModel.from_pretrained(tiny, dtype="bf16", kv_cache_dtype="fp8")
    with pytest.raises(FileNotFoundError):
        xft.AutoModel.from_pretrained(str(tmp_path / "nowhere"), dtype="bf16")
    m = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    with pytest.raises(KeyError):
        m.set_input_cb([1], [9999], 32)                            # unknown sequence id
    with pytest.raises(RuntimeError):
        m.forward_cb()                                             # nothing scheduled


def test_model_zoo_configs_parse_and_split():
    """Every examples/model_config/<name>/config.ini parses, maps to a registered family, and its tensor-parallel
    layout is valid for 1, 2, 4 and 8 ranks; the files are what tools/model_zoo.py generates."""
    import glob
    from xfastertransformer_b200.config import ModelConfig
    from xfastertransformer_b200.models.registry import family_for
    from xfastertransformer_b200.parallel import partition as P
    from xfastertransformer_b200.tools.synthetic import preset
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "model_config")
    dirs = sorted(glob.glob(os.path.join(root, "*", "config.ini")))
    assert len(dirs) >= 40
    for ini in dirs:
        name = os.path.basename(os.path.dirname(ini))
        cfg = ModelConfig.from_ini(os.path.dirname(ini))
        spec = family_for(cfg)
        assert spec is not None, name
        assert cfg.head_num > 0 and cfg.hidden_size > 0 and cfg.num_layer > 0 and cfg.vocab_size > 0, name
        if name != "deepseek-r1":
            ref = preset(name)
            assert (ref.model_type, ref.num_layer, ref.hidden_size, ref.head_num, ref.kv_head_num, ref.inter_size) == \
                   (cfg.model_type, cfg.num_layer, cfg.hidden_size, cfg.head_num, cfg.kv_head_num, cfg.inter_size), name
        for tp in (1, 2, 4, 8):
            q_total = 0
            for r in range(tp):
                (q0, q1), (k0, k1) = P.head_range(cfg.head_num, cfg.kv_head_num, tp, r)
                assert q1 >= q0 and k1 > k0 or q1 == q0, (name, tp, r)
                q_total += q1 - q0
            assert q_total == cfg.head_num, (name, tp)
            inter = cfg.moe_intermediate_size or cfg.inter_size
            if cfg.model_type != "deepseek_moe":
                spans = [P.task_range(inter, tp, r) for r in range(tp)]
                assert spans[0][0] == 0 and spans[-1][1] == inter and all(a[1] == b[0] for a, b in zip(spans, spans[1:])), (name, tp)


def test_debug_dir_dumps_layer_outputs(tmp_path, monkeypatch):
    """XFT_DEBUG_DIR: every forward writes the hidden state after each attention / FFN block and a summary log."""
    import glob
    import torch
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint
    from xfastertransformer_b200.utils.flags import Env
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=300), seed=0, dtype="fp32", std=0.05)
    dbg = str(tmp_path / "dbg")
    monkeypatch.setenv("XFT_DEBUG_DIR", dbg)
    Env.get().reload()
    try:
        m = xft.AutoModel.from_pretrained(d, dtype="bf16")
        m.generate(torch.tensor([[5, 6, 7, 8]]), max_length=6)
    finally:
        monkeypatch.delenv("XFT_DEBUG_DIR")
        Env.get().reload()
    files = sorted(os.path.basename(f) for f in glob.glob(os.path.join(dbg, "*.pt")))
    assert any(f.endswith("_layer0_attn_out.pt") for f in files) and any(f.endswith("_layer1_ffn_out.pt") for f in files)
    t = torch.load(os.path.join(dbg, [f for f in files if f.endswith("_embedding.pt")][0]))
    assert t.shape == (4, 256) and torch.isfinite(t).all()
    log = open(os.path.join(dbg, "rank0.log")).read()
    assert "layer1_attn_out" in log and "absmax" in log


def test_mixed_prefill_and_decode_in_one_forward(tiny):
    """set_input_cb(hold=True) + set_input_cb(append=True): new prompts and running sequences share one forward and
    get the logits they get in separate forwards."""
    import torch
    import xfastertransformer_b200 as xft
    m = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    g = torch.Generator().manual_seed(3)
    p1 = torch.randint(5, 900, (2, 12), generator=g).tolist()
    p2 = torch.randint(5, 900, (1, 20), generator=g).tolist()
    # separate: prefill p1, decode one step, prefill p2
    s1 = m.set_input_cb(p1, None, 40)
    l1 = m.forward_cb()
    t1 = l1.argmax(-1).tolist()
    m.set_input_cb([[t] for t in t1], s1, None)
    want_dec = m.forward_cb().clone()
    s2 = m.set_input_cb(p2, None, 40)
    want_pre = m.forward_cb().clone()
    m.free_seqs(torch.cat([s1, s2]))
    # mixed: prefill p1, then ONE forward with p2's prefill and p1's decode step
    s1 = m.set_input_cb(p1, None, 40)
    m.forward_cb()
    s2 = m.set_input_cb(p2, None, 40, hold=True)
    m.set_input_cb([[t] for t in t1], s1, None, append=True)
    both = m.forward_cb()
    assert both.shape[0] == 3
    assert torch.allclose(both[:1], want_pre, atol=2e-3, rtol=2e-3)
    assert torch.allclose(both[1:], want_dec, atol=2e-3, rtol=2e-3)
    # the sequences keep going after a mixed step
    nxt = both.argmax(-1).tolist()
    m.set_input_cb([[nxt[1]], [nxt[2]], [nxt[0]]], torch.cat([s1, s2]), None)
    assert m.forward_cb().shape[0] == 3
    m.free_seqs(torch.cat([s1, s2]))


def test_step_watchdog_reports_an_overdue_step_and_the_step_raises(tiny, capfd):
    """XFT_STEP_TIMEOUT_S: a step that runs over the limit is reported by the monitor thread while it is still running
    (log line, stack dump, hook) and raises StepTimeout when it returns; steps within the limit are untouched and the
    engine stays usable afterwards."""
    import time
    from xfastertransformer_b200.utils.watchdog import StepTimeout, StepWatchdog
    seen = []
    wd = StepWatchdog(0.05, on_timeout=lambda what, late: seen.append((what, late)))
    with wd.scope("fast"):
        pass
    assert wd.trips == 0 and not seen
    t0 = time.monotonic()
    with pytest.raises(StepTimeout, match="slow step"):
        with wd.scope("slow step"):
            while not seen and time.monotonic() - t0 < 5:      # the hook fires while the step is still inside
                time.sleep(0.01)
            assert wd.overdue                  # what a health check sees while the step is stuck
    assert not wd.overdue
    assert wd.trips == 1 and seen[0][0] == "slow step" and seen[0][1] >= 0.05
    cap = capfd.readouterr()
    assert "step watchdog" in cap.out and "slow step" in cap.out            # the log line (the logger writes stdout)
    assert "most recent call first" in cap.err                              # faulthandler's dump of every thread
    with pytest.raises(KeyError):              # the step's own exception is not replaced by the time-out
        with wd.scope("raises"):
            time.sleep(0.12)
            raise KeyError("x")
    with wd.scope("fast again"):
        pass
    wd.close()
    off = StepWatchdog(0.0)
    with off.scope("never guarded"):
        time.sleep(0.01)
    assert off._thread is None

    # through the engine: a forward slowed down beyond the limit raises, the next one works
    model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    m = model.model
    m.watchdog = StepWatchdog(0.05, dump_stacks=False)
    ids = torch.tensor([[5, 6, 7, 8]])
    model.set_input(ids, max_length=12)
    real_run = m._run

    def slow_run(seqs, logits_all=False):
        time.sleep(0.15)
        return real_run(seqs, logits_all)
    m._run = slow_run
    with pytest.raises(StepTimeout):
        model.forward()
    m._run = real_run
    m.watchdog.close()
    m.watchdog = StepWatchdog(30.0)
    model.set_input(ids, max_length=12)
    assert model.forward().shape[0] == 1
    m.watchdog.close()


def test_xft_verbose_prints_one_line_per_gemm(tiny, monkeypatch, capfd):
    """XFT_VERBOSE=1: every GEMM-shaped op prints the reference's line xft_verbose,exec,<dev>,api,<kernel>,m..n..k..,<ms>."""
    import re
    from xfastertransformer_b200.utils.flags import Env
    monkeypatch.setenv("XFT_VERBOSE", "1")
    Env.get().reload()
    try:
        model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
        capfd.readouterr()
        model.generate(torch.tensor([[5, 6, 7, 8]]), max_length=6)
        out = capfd.readouterr().out
    finally:
        monkeypatch.delenv("XFT_VERBOSE")
        Env.get().reload()
    lines = [l for l in out.splitlines() if l.startswith("xft_verbose,exec,cpu,api,")]
    # per forward of the 2-layer model: (qkv, o_proj, gate-up, down) x 2 + lm_head = 9 GEMMs; prefill + 1 decode step
    assert len(lines) == 18, len(lines)
    assert all(re.fullmatch(r"xft_verbose,exec,cpu,api,[a-z_]+,m\d+n\d+k\d+,\d+\.\d+", l) for l in lines), lines[:3]
    assert any(",m4n" in l for l in lines) and any(",m1n" in l for l in lines)        # prefill rows, then one row
    assert sum("gated" in l for l in lines) == 4 and sum("n1000k256" in l for l in lines) == 2


def test_automatic_prefix_reuse_keeps_results_and_skips_work(tiny, monkeypatch):
    """XFT_PREFIX_CACHE=1: a prompt that starts with tokens an earlier prefill has cached adopts those KV blocks and
    runs only the rest; logits and generated tokens equal the engine without reuse."""
    from xfastertransformer_b200.utils.flags import Env
    g = torch.Generator().manual_seed(11)
    common = torch.randint(5, 900, (150,), generator=g).tolist()              # two full 64-token blocks + 22
    p1 = common + torch.randint(5, 900, (9,), generator=g).tolist()
    p2 = common + torch.randint(5, 900, (30,), generator=g).tolist()
    p3 = common[:100] + torch.randint(5, 900, (7,), generator=g).tolist()     # shares one full block only
    plain = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    want = {}
    for name, p in (("p1", p1), ("p2", p2), ("p3", p3)):
        sid = plain.set_input_cb([p], None, 256)
        want[name] = plain.forward_cb()
        plain.free_seqs(sid)
    want_gen = plain.generate(torch.tensor([p2]), max_length=len(p2) + 6)
    monkeypatch.setenv("XFT_PREFIX_CACHE", "1")
    Env.get().reload()
    try:
        m = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    finally:
        monkeypatch.delenv("XFT_PREFIX_CACHE")
        Env.get().reload()
    eng = m.model
    idx = eng.cache.prefix_index
    assert idx is not None
    ran = []
    real = eng.make_batch
    eng.make_batch = lambda seqs, la=False: (ran.append(sum(len(s.pending) for s in seqs)), real(seqs, la))[1]
    sid = m.set_input_cb([p1], None, 256)
    got1 = m.forward_cb()
    m.free_seqs(sid)
    assert ran[-1] == len(p1) and idx.hit_blocks == 0 and len(idx.entries) == 2
    sid = m.set_input_cb([p2, p3], None, 256)                  # both reuse blocks of p1, in one ragged prefill
    got23 = m.forward_cb()
    m.free_seqs(sid)
    assert ran[-1] == (len(p2) - 128) + (len(p3) - 64) and idx.hit_blocks == 3
    for got, name in ((got1[0], "p1"), (got23[0], "p2"), (got23[1], "p3")):
        assert torch.allclose(got, want[name][0], atol=2e-3, rtol=2e-3), name
    out = m.generate(torch.tensor([p2]), max_length=len(p2) + 6)            # batch API: prefill of 2 full blocks is skipped
    assert torch.equal(out, want_gen) and ran[-6] == len(p2) - 128
    # nothing leaks: the only blocks still held are the remembered ones
    assert not eng.cache.tables and eng.cache.alloc.num_blocks - eng.cache.alloc.num_free == len(idx.entries)


@pytest.mark.parametrize("prefix_cache", [0, 1])
def test_continuous_batching_random_schedules(tiny, monkeypatch, prefix_cache):
    """Randomised continuous-batching sessions: prompts arrive at random steps (sometimes several at once, sometimes in
    the same forward as the running sequences), sequences leave at random lengths, some prompts repeat a long common
    beginning.  Every sequence's tokens must equal its stand-alone greedy decode, whatever it shared a batch with, and
    the cache must be empty at the end (apart from remembered prefix blocks)."""
    import random
    from xfastertransformer_b200.utils.flags import Env
    monkeypatch.setenv("XFT_PREFIX_CACHE", str(prefix_cache))
    Env.get().reload()
    try:
        model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    finally:
        monkeypatch.delenv("XFT_PREFIX_CACHE")
        Env.get().reload()
    rng = random.Random(7 + prefix_cache)
    common = [rng.randrange(5, 900) for _ in range(70)]
    prompts = []
    for i in range(9):
        body = [rng.randrange(5, 900) for _ in range(rng.randint(1, 40))]
        prompts.append((common + body) if i % 3 == 0 else body)
    want_len = [rng.randint(1, 9) for _ in prompts]
    solo = [_greedy_stream(model, p, n) for p, n in zip(prompts, want_len)]
    arrive = sorted(rng.randint(0, 12) for _ in prompts)
    got = {i: [] for i in range(len(prompts))}
    sid_of, last = {}, {}
    step, nxt = 0, 0
    while nxt < len(prompts) or sid_of:
        new = []
        while nxt < len(prompts) and arrive[nxt] <= step:
            new.append(nxt)
            nxt += 1
        running = list(sid_of)
        if new and running and rng.random() < 0.5:
            # mixed step: the new prompts and the running sequences' next tokens in ONE forward
            sids = model.set_input_cb([prompts[i] for i in new], None, 256, hold=True)
            model.set_input_cb([last[i] for i in running], [sid_of[i] for i in running], None, append=True)
            logits = model.forward_cb()
            for i, s in zip(new, sids.tolist()):
                sid_of[i] = s
            order = new + running
        else:
            order = []
            if new:
                sids = model.set_input_cb([prompts[i] for i in new], None, 256)
                logits_new = model.forward_cb()
                for i, s in zip(new, sids.tolist()):
                    sid_of[i] = s
                order += new
            if running:
                model.set_input_cb([last[i] for i in running], [sid_of[i] for i in running], None)
                logits_run = model.forward_cb()
                order += running
            parts = ([logits_new] if new else []) + ([logits_run] if running else [])
            logits = torch.cat(parts, 0) if parts else None
        done = []
        for row, i in enumerate(order):
            t = int(logits[row].argmax())
            got[i].append(t)
            last[i] = t
            if len(got[i]) >= want_len[i]:
                done.append(i)
        if done:
            model.free_seqs([sid_of.pop(i) for i in done])
        step += 1
        assert step < 200
    for i in range(len(prompts)):
        assert got[i] == solo[i], (i, got[i], solo[i])
    eng = model.model
    held = len(eng.cache.prefix_index.entries) if eng.cache.prefix_index is not None else 0
    assert not eng.cache.tables and eng.cache.alloc.num_blocks - eng.cache.alloc.num_free == held
    if prefix_cache:
        assert eng.cache.prefix_index.hit_blocks >= 2          # the common beginning (one full block) was reused


def test_chunked_prefill_through_extend(tiny):
    """set_input_cb(extend=True): a prompt fed in pieces, with another sequence decoding in between (also in the same
    forward), ends with the logits of the one-shot prefill and continues with the same tokens."""
    model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    g = torch.Generator().manual_seed(21)
    long_p = torch.randint(5, 900, (150,), generator=g).tolist()
    other = torch.randint(5, 900, (12,), generator=g).tolist()
    sid = model.set_input_cb([long_p], None, 256)
    want = model.forward_cb()[0]
    model.free_seqs(sid)
    want_other = _greedy_stream(model, other, 6)
    so = model.set_input_cb([other], None, 64)
    lo = model.forward_cb()
    toks = [int(lo[0].argmax())]
    s1 = model.set_input_cb([long_p[:64]], None, [200])                       # first piece; max_length of the whole request
    model.forward_cb()
    model.set_input_cb([toks[-1]], so, None)                                   # the other sequence decodes in between
    toks.append(int(model.forward_cb()[0].argmax()))
    # second piece in the same forward as the other sequence's next token
    model.set_input_cb([long_p[64:130]], s1, None, extend=True, hold=True)
    model.set_input_cb([toks[-1]], so, None, append=True)
    both = model.forward_cb()
    toks.append(int(both[1].argmax()))
    model.set_input_cb([long_p[130:]], s1, None, extend=True)
    got = model.forward_cb()[0]
    assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), (got - want).abs().max()
    for _ in range(3):
        model.set_input_cb([toks[-1]], so, None)
        toks.append(int(model.forward_cb()[0].argmax()))
    assert toks == want_other
    # the sequence decodes on from here like any other
    t = int(got.argmax())
    model.set_input_cb([t], s1, None)
    nxt = model.forward_cb()
    sid = model.set_input_cb([long_p + [t]], None, 256)
    assert torch.allclose(nxt[0], model.forward_cb()[0], atol=2e-3, rtol=2e-3)
    model.free_seqs(sid)
    with pytest.raises(RuntimeError):
        model.set_input_cb([[1, 2]], s1, None, extend=True)                   # a prompt does not grow after generation started
    model.free_seqs(torch.cat([s1, so]))
    with pytest.raises(ValueError):
        s2 = model.set_input_cb([[1, 2, 3]], None, [6])
        model.forward_cb()
        model.set_input_cb([[4, 5, 6, 7]], s2, None, extend=True)             # beyond the sequence's max_length


def test_ngram_speculative_decoding_is_exact(tiny, monkeypatch):
    """XFT_SPEC_NGRAM=k: drafts are verified in one forward and the output equals plain greedy decoding token for
    token.  First with the real n-gram drafts (random text: few are accepted), then with drafts taken from the known
    continuation with every third token falsified: two accepted + one corrected token per step, rejected cache
    positions rewritten later, eos and max_length honoured inside a run of accepted tokens."""
    from xfastertransformer_b200.runtime.engine import Model
    from xfastertransformer_b200.utils.flags import Env
    g = torch.Generator().manual_seed(3)
    motif = torch.randint(5, 900, (6,), generator=g)
    ids = torch.stack([motif.repeat(5), torch.randint(5, 900, (30,), generator=g), torch.randint(5, 900, (30,), generator=g)])
    plain = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    want = plain.generate(ids, max_length=30 + 48)
    eos = int(want[0, 30 + 9])                                   # a token that does occur: row 0 stops on it
    want_eos = plain.generate(ids, max_length=30 + 48, eos_token_id=eos, pad_token_id=0)
    assert Model._ngram_draft([1, 2, 3, 9, 9, 1, 2, 3], 4) == [9, 9, 1, 2] and Model._ngram_draft([1, 2, 3], 4) == []
    assert Model._ngram_draft([5, 6, 7, 5], 2) == [6, 7] and Model._ngram_draft([4, 4, 4, 4], 3) == [4]
    monkeypatch.setenv("XFT_SPEC_NGRAM", "4")
    Env.get().reload()
    try:
        m = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
        eng = m.model
        assert torch.equal(m.generate(ids, max_length=30 + 48), want) and eng.spec_steps > 0
        # oracle drafts: the true continuation, the third draft token wrong
        rows = {tuple(r[:30].tolist()): r.tolist() for r in want}

        # the incremental table gives what the plain search gives, step by step over a growing sequence
        from xfastertransformer_b200.runtime.sequence import SequenceMeta
        import random
        rng = random.Random(0)
        seq = SequenceMeta(0, [rng.randrange(4) for _ in range(9)], 500)
        for _ in range(120):
            assert eng._draft_for(seq, 4) == Model._ngram_draft(seq.all_tokens(), 4, window=10 ** 6)
            seq.generated.append(rng.randrange(4))

        def oracle(self, s, k):
            tokens = s.all_tokens()
            full = rows[tuple(tokens[:30])]
            d = full[len(tokens):len(tokens) + k]
            if len(d) > 2:
                d[2] = (d[2] + 1) % 900
            return d
        monkeypatch.setattr(Model, "_draft_for", oracle)
        s0, e0, a0, f0 = eng.spec_steps, eng.spec_emitted, eng.spec_accepted, len(eng.step_times_ms)
        assert torch.equal(m.generate(ids, max_length=30 + 48), want)
        steps = eng.spec_steps - s0
        # two accepted drafts + the corrected token per sequence and step, except near max_length where the drafts shrink
        assert eng.spec_accepted - a0 >= 2 * 3 * (steps - 2) and eng.spec_emitted - e0 >= 3 * 42
        assert len(eng.step_times_ms) - f0 <= 20                    # instead of 48 forwards
        assert torch.equal(m.generate(ids, max_length=30 + 48, eos_token_id=eos, pad_token_id=0), want_eos)
        assert not eng.cache.tables and eng.cache.alloc.num_free == eng.cache.alloc.num_blocks

        class Streamer:                      # a streamer sees every token, also those accepted several at a time
            def __init__(self):
                self.chunks, self.ended = [], False

            def put(self, t):
                self.chunks.append(t.flatten().tolist())

            def end(self):
                self.ended = True
        st = Streamer()
        out1 = m.generate(ids[:1], max_length=30 + 48, streamer=st)
        assert st.ended and st.chunks[0] == ids[0].tolist() and sum(st.chunks[1:], []) == out1[0, 30:].tolist()
        assert max(len(c) for c in st.chunks[1:]) == 3
        # sampling and beams do not take the speculative path
        s1 = eng.spec_steps
        m.generate(ids[:1], max_length=40, num_beams=2)
        m.generate(ids[:1], max_length=40, do_sample=True, seed=1)
        assert eng.spec_steps == s1
    finally:
        monkeypatch.delenv("XFT_SPEC_NGRAM")
        Env.get().reload()


def test_telechat_long_prompt_matches_eager_ntk_oracle(tmp_path):
    """TeleChat's rotary table: the NTK base comes from max(context, training length) and a prompt longer than the
    training length also scales cos / sin by 0.1 ln(len / training) + 1
    (src/layers/rotary_embedding_telechat.cpp:29-35,68-117).  Checked against an independent eager model for a prompt
    inside the training length (base of the training length, no scale) and one beyond it (larger base, scaled table);
    plain RoPE would fail both."""
    import math
    from eager_llama import EagerLlama, _load
    train = 8192          # alpha = 3 inside the training length; a 9000-token prompt would be too slow on CPU, so the
    # "long" case shrinks the training length instead (alpha = 1, mscale > 1)
    for train, S in ((8192, 40), (32, 70)):
        cfg = ModelConfig(model_type="telechat", num_layer=2, hidden_size=128, head_num=4, kv_head_num=4,
                          size_per_head=32, inter_size=256, vocab_size=512, max_pos_seq_len=train,
                          activation_type="silu", weight_data_type="bf16", start_id=1, end_id=2)
        d = str(tmp_path / f"tc{train}")
        write_synthetic_checkpoint(d, cfg, seed=3, dtype="bf16", std=0.1)
        ids = torch.randint(5, 500, (1, S), generator=torch.Generator().manual_seed(S))
        got = xft.AutoModel.from_pretrained(d, dtype="bf16")(ids)[0]

        class EagerTeleChat(EagerLlama):
            def __init__(self, path):
                super().__init__(path)
                for i, l in enumerate(self.layers):
                    l["ob"] = _load(path, f"model.layers.{i}.attention.dense.bias.bin", (self.H,), "bf16")
                true_len = max(S, train)
                alpha = max(2.0 ** math.ceil(math.log2(true_len / 4096.0) + 1) - 1, 1.0)
                self.theta = self.theta * alpha ** (self.D / (self.D - 2))
                self.mscale = 0.1 * math.log(S / train) + 1.0 if S > train else 1.0

            def _rope(self, x, pos):
                D = self.D
                inv = 1.0 / (self.theta ** (torch.arange(0, D, 2).float() / D))
                f = torch.outer(pos.float(), inv)
                cos, sin = f.cos()[None, :, None, :] * self.mscale, f.sin()[None, :, None, :] * self.mscale
                x1, x2 = x[..., : D // 2], x[..., D // 2:]
                return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

        e = EagerTeleChat(d)
        # the o_proj bias: fold it into the residual stream by patching the product (x + a @ o + b)
        want = _eager_with_o_bias(e, ids)[0]
        err = (got - want).abs().max().item()
        assert err < 2e-3, (train, err)
        plain = EagerLlama(d)
        for l_p, l_e in zip(plain.layers, e.layers):
            l_p["ob"] = l_e["ob"]
        off = (got - _eager_with_o_bias(plain, ids)[0]).abs().max().item()
        assert off > 5 * max(err, 1e-2), (train, err, off)


def _eager_with_o_bias(e, ids):
    """EagerLlama.logits with a bias on the attention output projection (TeleChat)."""
    import math
    import torch.nn.functional as F
    B, S = ids.shape
    x = e.wte[ids]
    pos = torch.arange(S)
    mask = torch.full((S, S), float("-inf")).triu(1)
    g = e.nh // e.nkv
    for l in e.layers:
        h = e._norm(x, l["n1"])
        qkv = h @ l["qkv"]
        q = qkv[..., : e.nh * e.D].view(B, S, e.nh, e.D)
        k = qkv[..., e.nh * e.D:(e.nh + e.nkv) * e.D].view(B, S, e.nkv, e.D)
        v = qkv[..., (e.nh + e.nkv) * e.D:].view(B, S, e.nkv, e.D)
        q, k = e._rope(q, pos), e._rope(k, pos)
        k, v = k.repeat_interleave(g, 2), v.repeat_interleave(g, 2)
        s = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(e.D) + mask
        a = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v).reshape(B, S, -1)
        x = x + a @ l["o"] + l["ob"]
        h = e._norm(x, l["n2"])
        x = x + (F.silu(h @ l["g"]) * (h @ l["u"])) @ l["d"]
    return e._norm(x, e.fn) @ e.head.t()
