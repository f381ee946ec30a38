"""The native C++ API (xft::AutoModel in libxft_b200_core.so) through the example CLI, against the Python engine."""
import os
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("kv", ["fp16", "int8"])
def test_cpp_example_matches_python(kv, tmp_path):
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=2000), seed=0, dtype="bf16", std=0.08)
    prompt = [5, 17, 99, 200, 3, 42, 7, 1500, 23]
    m = xft.AutoModel.from_pretrained(d, dtype="bf16", kv_cache_dtype=kv)
    want = m.generate(torch.tensor([prompt, prompt]), max_length=len(prompt) + 12)[0, len(prompt):].tolist()
    exe = os.path.join(ROOT, "xfastertransformer_b200", "lib", "xft_example")
    r = subprocess.run([exe, "-m", d, "-i", " ".join(map(str, prompt)), "-b", "2", "-o", "12", "--kv_cache_dtype", kv,
                        "--no_stream"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    rows = [l for l in r.stdout.splitlines() if l.startswith("[")]
    got = [[int(t) for t in l.split("]")[1].split()] for l in rows]
    assert len(got) == 2 and got[0] == got[1]
    # same kernels, same order of operations: token streams agree (allow a late divergence from bf16 ties)
    agree = sum(a == b for a, b in zip(got[0], want))
    assert agree >= 10, (got[0], want)
    assert "first token" in r.stdout


def test_torch_custom_class_binding(tmp_path):
    """torch.classes.xfastertransformer.AutoModel (csrc/api/torch_binding.cc): generate(), continuous batching
    and logits agree with the Python engine on the same checkpoint."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint
    lib = os.path.join(ROOT, "xfastertransformer_b200", "lib", "libxft_b200_torch.so")
    if not os.path.exists(lib):
        pytest.skip("torch binding not built")
    torch.ops.load_library(lib)
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=2000), seed=1, dtype="bf16", std=0.08)
    prompt = torch.tensor([[5, 17, 99, 200, 3, 42, 7, 1500, 23]] * 2)
    P = prompt.shape[1]
    py = xft.AutoModel.from_pretrained(d, dtype="bf16")
    want = py.generate(prompt, max_length=P + 8)
    m = torch.classes.xfastertransformer.AutoModel(d, "bf16", "fp16")
    assert m.get_rank() == 0
    m.config(P + 8, None, None, None, None, None, None, None, None, None, None, None, None)
    m.input(prompt)
    steps = 0
    while not m.is_done():
        t = m.generate()
        assert t.numel() == 2
        steps += 1
    out = m.finalize()
    assert out.shape == (2, P + 8) and steps == 8
    agree = (out[0, P:] == want[0, P:]).sum().item()
    assert agree >= 6, (out[0].tolist(), want[0].tolist())
    # continuous batching: prefill two prompts, read logits
    ids = m.set_input_cb(prompt, None, None, torch.tensor([P + 4, P + 4]))
    assert ids.numel() == 2
    logits = m.forward_cb()
    assert logits.shape == (2, 2000) and torch.isfinite(logits).all()
    assert int(logits[0].argmax()) == int(want[0, P])
    assert m.free_seqs(ids)


def test_cb_check_cli(tmp_path):
    """examples/cpp/cb_check.cpp: sequences decoded alone and inside a staggered continuous batch agree."""
    from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint
    exe = os.path.join(ROOT, "xfastertransformer_b200", "lib", "xft_cb_check")
    if not os.path.exists(exe):
        pytest.skip("cb_check not built")
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=2000), seed=2, dtype="bf16", std=0.08)
    r = subprocess.run([exe, "-m", d, "-n", "5", "-o", "10", "--stride", "2", "--max_len", "90", "--tolerate", "1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "sequences identical" in r.stdout


def test_cpp_beam_search_matches_python(tmp_path):
    """Beam search in the C++ runtime (host scorer + block-table reorder) through the torch binding, against the Python
    engine's beam search on the same checkpoint."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint
    lib = os.path.join(ROOT, "xfastertransformer_b200", "lib", "libxft_b200_torch.so")
    if not os.path.exists(lib):
        pytest.skip("torch binding not built")
    torch.ops.load_library(lib)
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=300), seed=5, dtype="bf16", std=0.15)
    prompt = torch.tensor([[5, 17, 99, 200, 3, 42, 7], [9, 8, 250, 6, 5, 4, 3]])
    P, new = prompt.shape[1], 10
    py = xft.AutoModel.from_pretrained(d, dtype="bf16")
    want = py.generate(prompt, max_length=P + new, num_beams=3, eos_token_id=299, pad_token_id=0)
    m = torch.classes.xfastertransformer.AutoModel(d, "bf16", "fp16")
    m.config(P + new, 3, 1, None, None, 299, 0, None, None, None, None, None, None)
    m.input(prompt)
    steps = 0
    while not m.is_done():
        t = m.generate()
        assert t.numel() == 2 * 3
        steps += 1
        assert steps <= new
    out = m.finalize()
    assert out.shape[0] == 2 and out.shape[1] <= P + new
    assert torch.equal(out[:, :P], prompt)
    # Beams amplify last-bit differences between the two engines (a flipped near-tie changes the surviving
    # hypotheses), so compare what beam search optimises: the sequence log-probability under the fp32 oracle.
    import sys
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from eager_llama import EagerLlama
    ref = EagerLlama(d)

    def seq_logprob(row):
        row = row[:P + new]
        n = len(row)
        while n > P and row[n - 1] == 0:      # padding
            n -= 1
        ids = torch.tensor([row[:n]])
        lp = torch.log_softmax(ref.logits(ids[:, :-1])[0], -1)
        return sum(float(lp[t - 1, ids[0, t]]) for t in range(P, n)) / max(n - P, 1)

    for b in range(2):
        got_lp, want_lp = seq_logprob(out[b].tolist()), seq_logprob(want[b].tolist())
        assert got_lp >= want_lp - max(0.25, 0.1 * abs(want_lp)), (b, got_lp, want_lp, out[b].tolist(), want[b].tolist())


_CPP_FAMILIES = {
    "gemma": dict(activation_type="gelu"),
    "qwen": dict(seq_length=16),                       # prompt longer than the training length: NTK base + log-n scale
    "qwen3": dict(do_qk_norm=True, kv_head_num=2),
    "baichuan": dict(max_pos_seq_len=0),               # no rotary table: ALiBi
    "chatglm2": dict(kv_head_num=2),
    "chatglm4": dict(kv_head_num=1),
    "gpt": dict(activation_type="relu"),
    "telechat": {},
    "chatglm": dict(activation_type="gelu"),
    "mixtral": dict(sparse_experts=8, num_experts_per_tok=2),
    # every expert selected: the comparison with the fp32 oracle is then free of the discrete jumps a flipped near-tie
    # between the 4th and 5th expert would cause (the top-k selection itself is checked against its oracle in
    # tests/test_moe_gpu.py, and with Mixtral above)
    "qwen3_moe": dict(sparse_experts=4, num_experts_per_tok=4, moe_intermediate_size=256, do_qk_norm=True, kv_head_num=2),
}


def _cpu_oracle_logits(d, prompt, monkeypatch):
    """Last-position logits from the package's fp32 PyTorch path (XFT_ENGINE=CPU): none of the CUDA kernels."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.parallel.dist import DistContext
    from xfastertransformer_b200.utils.flags import Env
    monkeypatch.setenv("XFT_ENGINE", "CPU")
    Env._inst = None
    DistContext.reset()             # the process-wide context remembers its device
    try:
        m = xft.AutoModel.from_pretrained(d, dtype="bf16")
        assert m.model.ctx.device.type == "cpu"
        return m(prompt)[:, -1].float()
    finally:
        monkeypatch.delenv("XFT_ENGINE")
        Env._inst = None
        DistContext.reset()


@pytest.mark.parametrize("mt", sorted(_CPP_FAMILIES))
def test_cpp_engine_families_match_python(mt, tmp_path, monkeypatch):
    """Every family of the C++ engine (norm kind, biases, rotary variant, MLP layout or experts, position scheme) against the
    Python engine on the same synthetic checkpoint: last-prompt-token logits numerically, then greedy tokens.  Both GPU
    engines are also held against the fp32 PyTorch path of the package."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.config import ModelConfig
    from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint
    lib = os.path.join(ROOT, "xfastertransformer_b200", "lib", "libxft_b200_torch.so")
    if not os.path.exists(lib):
        pytest.skip("torch binding not built")
    torch.ops.load_library(lib)
    kw = dict(model_type=mt, num_layer=2, hidden_size=256, head_num=4, kv_head_num=4, size_per_head=64, inter_size=512,
              vocab_size=1000, max_pos_seq_len=512, activation_type="silu", weight_data_type="bf16", start_id=1, end_id=2)
    kw.update(_CPP_FAMILIES[mt])
    d = str(tmp_path / mt)
    write_synthetic_checkpoint(d, ModelConfig(**kw), seed=3, dtype="bf16", std=0.08)
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(5, 990, (2, 24), generator=g)
    P, new = prompt.shape[1], 8
    oracle = _cpu_oracle_logits(d, prompt, monkeypatch)
    py = xft.AutoModel.from_pretrained(d, dtype="bf16")
    assert py.model.ctx.device.type == "cuda"
    want_logits = py(prompt)[:, -1].float().cpu()
    tol = 0.08 * max(1.0, oracle.abs().max().item())
    assert (want_logits - oracle).abs().max().item() < tol, (mt, "python engine", (want_logits - oracle).abs().max().item())
    m = torch.classes.xfastertransformer.AutoModel(d, "bf16", "fp16")
    ids = m.set_input_cb(prompt, None, None, torch.tensor([P + 4, P + 4]))
    got_logits = m.forward_cb().float().cpu()
    assert m.free_seqs(ids)
    assert (got_logits - oracle).abs().max().item() < tol, (mt, "C++ engine", (got_logits - oracle).abs().max().item())
    err = (got_logits - want_logits).abs().max().item()
    assert err <= 0.06 * want_logits.abs().max().item() + 0.03, (mt, err, want_logits.abs().max().item())
    m.config(P + new, None, None, None, None, 100000, 0, None, None, None, None, None, None)
    m.input(prompt)
    while not m.is_done():
        m.generate()
    out = m.finalize()
    assert out.shape == (2, P + new)
    assert torch.equal(out[:, :P].cpu(), prompt)
    # teacher-forced check of the C++ decode path (cache, positions, tables of later steps): its tokens are fed to the
    # Python engine one step at a time, and each must be (near-)best under the Python logits of that step
    sid = py.set_input_cb(prompt.tolist(), None, P + new + 2)
    lg = py.forward_cb().float().cpu()
    for t in range(new):
        tok = out[:, P + t].cpu()
        best = lg.max(-1).values
        assert (lg.gather(1, tok[:, None])[:, 0] >= best - 0.05 * best.abs() - 0.1).all(), (mt, t, tok.tolist(), lg.argmax(-1).tolist())
        if t + 1 < new:
            py.set_input_cb(tok.tolist(), sid, P + new + 2)
            lg = py.forward_cb().float().cpu()
    py.free_seqs(sid)


@pytest.mark.parametrize("dtype", ["int8", "w8a8", "nf4", "int4", "bf16_int8", "w8a8_nf4"])
def test_cpp_engine_quantised_weights(dtype, tmp_path, monkeypatch):
    """Quantise-at-load in the C++ engine (per-channel int8 weight-only, int8 x int8, NF4, uint4, and hybrid types: one
    form for the prompt pass, another for decode steps): same codes as the Python engine with that dtype, so the logits
    agree closely; both track the fp32 oracle of the dense model within the quantisation error."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint
    lib = os.path.join(ROOT, "xfastertransformer_b200", "lib", "libxft_b200_torch.so")
    if not os.path.exists(lib):
        pytest.skip("torch binding not built")
    torch.ops.load_library(lib)
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=2000, kv_head_num=2), seed=6, dtype="bf16", std=0.08)
    prompt = torch.randint(5, 1990, (2, 20), generator=torch.Generator().manual_seed(2))
    P = prompt.shape[1]
    oracle = _cpu_oracle_logits(d, prompt, monkeypatch)
    py = xft.AutoModel.from_pretrained(d, dtype=dtype)
    want = py(prompt)[:, -1].float().cpu()
    m = torch.classes.xfastertransformer.AutoModel(d, dtype, "fp16")
    ids = m.set_input_cb(prompt, None, None, torch.tensor([P + 4, P + 4]))
    got = m.forward_cb().float().cpu()
    assert m.free_seqs(ids)
    top = oracle.abs().max().item()
    assert (got - want).abs().max().item() <= 0.03 * top + 0.02, (dtype, (got - want).abs().max().item(), top)
    first = dtype.split("_")[0]
    assert (got - oracle).abs().max().item() <= (0.9 if first in ("nf4", "int4") else 0.2) * top, (dtype, (got - oracle).abs().max().item())
    m.config(P + 6, None, None, None, None, 100000, 0, None, None, None, None, None, None)
    m.input(prompt)
    while not m.is_done():
        m.generate()
    out = m.finalize()
    assert out.shape == (2, P + 6)
    # decode steps (the second type of a hybrid): teacher-forced through the Python engine of the same dtype
    sid = py.set_input_cb(prompt.tolist(), None, P + 8)
    lg = py.forward_cb().float().cpu()
    for t in range(6):
        tok = out[:, P + t].cpu()
        best = lg.max(-1).values
        assert (lg.gather(1, tok[:, None])[:, 0] >= best - 0.05 * best.abs() - 0.1).all(), (dtype, t, tok.tolist(), lg.argmax(-1).tolist())
        if t + 1 < 6:
            py.set_input_cb(tok.tolist(), sid, P + 8)
            lg = py.forward_cb().float().cpu()
    py.free_seqs(sid)


@pytest.mark.parametrize("dtype,routing", [("bf16", "all"), ("fp8_e4m3", "all"), ("bf16", "grouped")])
def test_cpp_engine_deepseek(dtype, routing, tmp_path, monkeypatch):
    """DeepSeek in the C++ engine (latent attention with query compression, YaRN table, dense first layer, shared +
    routed experts, e4m3 checkpoints dequantised at load) against the Python engine and the fp32 PyTorch path.
    "all": every expert is selected, so the comparison has no discrete routing decisions in it and is tight on every row;
    "grouped": 4 of 16 experts out of the 2 best of 4 groups — a near-tie may pick another expert for some token and move
    that row's logits, so at least half of the rows must agree tightly (a wrong routing parameter would move all)."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.config import ModelConfig, RopeConfig
    from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint
    lib = os.path.join(ROOT, "xfastertransformer_b200", "lib", "libxft_b200_torch.so")
    if not os.path.exists(lib):
        pytest.skip("torch binding not built")
    torch.ops.load_library(lib)
    route = dict(sparse_experts=8, n_group=1, topk_group=1, num_experts_per_tok=8) if routing == "all" else \
        dict(sparse_experts=16, n_group=4, topk_group=2, num_experts_per_tok=4)
    cfg = ModelConfig(model_type="deepseek_moe", num_layer=3, hidden_size=512, head_num=8, kv_head_num=8, size_per_head=128,
                      inter_size=1024, vocab_size=1024, max_pos_seq_len=4096, q_lora_rank=256, kv_lora_rank=512,
                      qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, moe_intermediate_size=256,
                      first_k_dense_replace=1, dense_experts=1, routed_scaling_factor=2.5, topk_method="noaux_tc",
                      norm_topk_prob=True, scoring_func="sigmoid", activation_type="silu", weight_data_type=dtype,
                      start_id=0, end_id=1,
                      rope=RopeConfig(theta=10000, scaling_type="yarn", scaling_factor=40, original_max_pos=4096,
                                      beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0), **route)
    d = str(tmp_path / "ds")
    write_synthetic_checkpoint(d, cfg, seed=0, dtype=dtype, std=0.05)
    prompt = torch.randint(0, 1024, (4, 24), generator=torch.Generator().manual_seed(3))
    P, new = prompt.shape[1], 6
    oracle = _cpu_oracle_logits(d, prompt, monkeypatch)
    py = xft.AutoModel.from_pretrained(d, dtype="bf16", kv_cache_dtype="bf16")
    want = py(prompt)[:, -1].float().cpu()
    m = torch.classes.xfastertransformer.AutoModel(d, "bf16", "fp16")
    ids = m.set_input_cb(prompt, None, None, torch.tensor([P + 4] * 4))
    got = m.forward_cb().float().cpu()
    assert m.free_seqs(ids)
    top = max(1.0, oracle.abs().max().item())
    row_err = lambda a, b: (a - b).abs().amax(-1)
    need = 4 if routing == "all" else 2
    assert (row_err(got, oracle) < 0.1 * top).sum().item() >= need, (row_err(got, oracle).tolist(), top)
    assert (row_err(got, want) < 0.06 * top + 0.03).sum().item() >= need, (row_err(got, want).tolist(), top)
    # decode steps: latent cache append, split latent attention, block tables
    m.config(P + new, None, None, None, None, 100000, 0, None, None, None, None, None, None)
    m.input(prompt)
    while not m.is_done():
        m.generate()
    out = m.finalize()
    assert out.shape == (4, P + new) and torch.equal(out[:, :P].cpu(), prompt)
    if routing == "all":
        sid = py.set_input_cb(prompt.tolist(), None, P + new + 2)
        lg = py.forward_cb().float().cpu()
        for t in range(new):
            tok = out[:, P + t].cpu()
            best = lg.max(-1).values
            assert (lg.gather(1, tok[:, None])[:, 0] >= best - 0.05 * best.abs() - 0.1).all(), (t, tok.tolist(), lg.argmax(-1).tolist())
            if t + 1 < new:
                py.set_input_cb(tok.tolist(), sid, P + new + 2)
                lg = py.forward_cb().float().cpu()
        py.free_seqs(sid)


@pytest.mark.parametrize("case", ["llama-2", "llama-4", "llama-2-int8", "gpt-2", "chatglm2-2", "chatglm-2"])
def test_cpp_tensor_parallel_thread_ranks(case, tmp_path):
    """Tensor parallelism of the C++ engine on one GPU (examples/cpp/tp_check.cpp): N ranks as threads of one process,
    each loading its heads / FFN rows / lm_head rows, against the single-rank engine — logits of the prompt pass and of
    teacher-forced decode steps.  4 ranks over 2 KV heads share KV heads between ranks (query-head offset inside the
    group) and split FFN and vocabulary unevenly; gpt / chatglm carry biases that must enter once; int8 quantises the
    slices."""
    from xfastertransformer_b200.config import ModelConfig
    from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint
    exe = os.path.join(ROOT, "xfastertransformer_b200", "lib", "xft_tp_check")
    if not os.path.exists(exe):
        pytest.skip("tp_check not built")
    parts = case.split("-")
    fam, ranks, dtype = parts[0], parts[1], (parts[2] if len(parts) > 2 else "bf16")
    kw = dict(model_type=fam, num_layer=2, hidden_size=256, head_num=4, kv_head_num=2, size_per_head=64, inter_size=688,
              vocab_size=2000, max_pos_seq_len=512, activation_type="silu", weight_data_type="bf16", start_id=1, end_id=2)
    if fam in ("gpt", "chatglm"):
        kw.update(kv_head_num=4, activation_type="relu" if fam == "gpt" else "gelu")
    d = str(tmp_path / "m")
    write_synthetic_checkpoint(d, ModelConfig(**kw), seed=8, dtype="bf16", std=0.08)
    r = subprocess.run([exe, "-m", d, "-n", ranks, "-d", dtype, "-o", "4"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "tensor-parallel ranks agree" in r.stdout, r.stdout


@pytest.mark.parametrize("qt,dtype", [("int8", "int8"), ("uint4", "int4"), ("uint4", "bf16"), ("int8", "w8a8")])
def test_cpp_engine_gptq_checkpoint(qt, dtype, tmp_path):
    """GPTQ-converted checkpoints in the C++ engine: stored codes kept as they are when the weight type matches
    (int8 -> int8 / w8a8, uint4 -> int4), dequantised otherwise — against the Python engine on the same directory; and
    the same directory as two tensor-parallel thread ranks (slices of the code tensors) against one rank."""
    import sys
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.tools.synthetic import preset
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from gptq_util import make_gptq_dir
    lib = os.path.join(ROOT, "xfastertransformer_b200", "lib", "libxft_b200_torch.so")
    if not os.path.exists(lib):
        pytest.skip("torch binding not built")
    torch.ops.load_library(lib)
    d = make_gptq_dir(str(tmp_path / "g"), preset("tiny-llama", vocab_size=2000, kv_head_num=2), qt, seed=4)
    prompt = torch.randint(5, 1990, (2, 20), generator=torch.Generator().manual_seed(2))
    P = prompt.shape[1]
    py = xft.AutoModel.from_pretrained(d, dtype=dtype)
    want = py(prompt)[:, -1].float().cpu()
    m = torch.classes.xfastertransformer.AutoModel(d, dtype, "fp16")
    ids = m.set_input_cb(prompt, None, None, torch.tensor([P + 4, P + 4]))
    got = m.forward_cb().float().cpu()
    assert m.free_seqs(ids)
    top = max(1.0, want.abs().max().item())
    assert (got - want).abs().max().item() <= 0.03 * top + 0.02, (qt, dtype, (got - want).abs().max().item(), top)
    exe = os.path.join(ROOT, "xfastertransformer_b200", "lib", "xft_tp_check")
    if os.path.exists(exe) and qt == dtype.replace("int4", "uint4"):
        r = subprocess.run([exe, "-m", d, "-n", "2", "-d", dtype, "-o", "2"], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0 and "tensor-parallel ranks agree" in r.stdout, r.stdout + r.stderr
