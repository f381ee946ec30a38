"""The C++ engine's host side on a CPU box: csrc/tests/engine_hostcheck.cc drives xft::AutoModel through every request
shape over a host stand-in of the device library (csrc/tests/mock_device.cc) whose kernels touch exactly the memory the
real ones read and write and refuse what the real entry points refuse; AddressSanitizer + UndefinedBehaviorSanitizer +
exact-size buffers (XFT_ARENA_EXACT) then check buffer sizes, strides, slot / block arithmetic and the ranges of every
rank for every family, weight type and rank layout, and that ranks produce the same tokens.  With the stand-in's arithmetic
switched on (XFT_MOCK_MATH) the engine's logits are compared with the PyTorch path of the package: every family,
quantised and GPTQ checkpoints, tensor- and expert-parallel thread ranks, pipeline stages with micro-batches, real
process ranks over a stand-in NCCL, greedy and beam generation, the per-layer debug dumps; the example programs and the
cases of the GPU thread-rank tests run over it too."""
import os
import shutil
import subprocess
import sys

import struct

import numpy as np
import pytest
import torch

from xfastertransformer_b200.config import ModelConfig, RopeConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CORE = ["engine.cc", "comm.cc", "runtime.cc", "ini.cc", "beam.cc", "env.cc", "arena.cc", "rope_tables.cc", "gptq.cc"]
TOKENIZERS = ["tokenizer.cc", "bpe_tokenizer.cc"]            # only the cb_check program reads tokenizer files


@pytest.fixture(scope="module")
def hostcheck(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    out = tmp_path_factory.mktemp("hostcheck")
    exe = str(out / "engine_hostcheck")
    flags = ["-g", "-std=c++17", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer",
             "-I", os.path.join(ROOT, "csrc", "api"), "-I", os.path.join(ROOT, "csrc", "core"), "-I", "/usr/local/cuda/include"]
    srcs = [os.path.join(ROOT, "csrc", "tests", "engine_hostcheck.cc"), os.path.join(ROOT, "csrc", "tests", "mock_device.cc")] + \
           [os.path.join(ROOT, "csrc", "core", f) for f in CORE + TOKENIZERS]
    # one compiler process per source, side by side; the stand-in's arithmetic loops want -O2, the engine compiles faster at -O1
    jobs = []
    for src in srcs:
        obj = str(out / (os.path.basename(src) + ".o"))
        opt = "-O2" if src.endswith("mock_device.cc") else "-O1"
        jobs.append((obj, subprocess.Popen(["g++", opt] + flags + ["-c", src, "-o", obj], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for obj, job in jobs:
        log = job.communicate(timeout=900)[0]
        assert job.returncode == 0, log[-4000:]
    engine_objs = [o for o, _ in jobs[:len(jobs) - len(TOKENIZERS)]]
    tokenizer_objs = [o for o, _ in jobs[len(jobs) - len(TOKENIZERS):]]
    b = subprocess.run(["g++", "-fsanitize=address,undefined"] + engine_objs + ["-o", exe, "-ldl", "-lpthread"],
                       capture_output=True, text=True, timeout=900)
    assert b.returncode == 0, b.stderr[-4000:]
    # a stand-in NCCL for the runs with process ranks
    b = subprocess.run(["g++", "-O1", "-g", "-std=c++17", "-shared", "-fPIC", os.path.join(ROOT, "csrc", "tests", "fake_nccl.cc"), "-o",
                        str(out / "libfake_nccl.so"), "-lrt", "-lpthread"], capture_output=True, text=True, timeout=900)
    assert b.returncode == 0, b.stderr[-4000:]
    # the example programs over the same stand-in (everything but the harness's own main)
    for prog in ("tp_check", "cb_check"):
        b = subprocess.run(["g++", "-O1"] + flags + [os.path.join(ROOT, "examples", "cpp", prog + ".cpp")] + engine_objs[1:] +
                           (tokenizer_objs if prog == "cb_check" else []) +
                           ["-o", str(out / prog), "-ldl", "-lpthread"], capture_output=True, text=True, timeout=900)
        assert b.returncode == 0, b.stderr[-4000:]
    return exe


def _run(exe, d, dtype, kv, ranks, fake=True, stages=1, micro=1):
    env = dict(os.environ, XFT_ARENA_EXACT="1", ASAN_OPTIONS="detect_leaks=1", UBSAN_OPTIONS="print_stacktrace=1",
               XFT_PIPELINE_STAGE=str(stages), XFT_MAX_REQUEST_NUM=str(micro))
    if fake:
        env["XFT_FAKE_MODEL"] = "2"
    else:
        env.pop("XFT_FAKE_MODEL", None)
    r = subprocess.run([exe, d, dtype, kv, str(ranks)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "hostcheck ok" in r.stdout, (d, dtype, kv, ranks, r.stdout[-500:], r.stderr[-3000:])


_BASE = dict(num_layer=2, hidden_size=256, head_num=4, kv_head_num=2, size_per_head=64, inter_size=512, vocab_size=300,
             max_pos_seq_len=512, activation_type="silu", weight_data_type="bf16", start_id=1, end_id=2)
_FAMILIES = {
    "llama": {}, "yarn_llama": {}, "gemma": dict(activation_type="gelu"), "qwen": dict(seq_length=16), "qwen2": {},
    "qwen3": dict(do_qk_norm=True), "baichuan": {}, "baichuan-alibi": dict(max_pos_seq_len=0), "chatglm2": {},
    "chatglm3": dict(kv_head_num=1), "chatglm4": {}, "gpt": dict(kv_head_num=4, activation_type="relu"),
    "telechat": dict(kv_head_num=4), "chatglm": dict(kv_head_num=4, activation_type="gelu"),
    "mixtral": dict(sparse_experts=4, num_experts_per_tok=2),
    "qwen3_moe": dict(sparse_experts=6, num_experts_per_tok=3, moe_intermediate_size=128, do_qk_norm=True),
}
_DENSE = [f for f in _FAMILIES if f not in ("mixtral", "qwen3_moe")]


def _config_dir(tmp_path, fam):
    kw = dict(_BASE, model_type=fam.split("-")[0])
    kw.update(_FAMILIES[fam])
    cfg = ModelConfig(**kw)
    if fam == "yarn_llama":
        cfg.rope.scaling_type, cfg.rope.scaling_factor, cfg.rope.original_max_pos = "yarn", 4.0, 128
    d = str(tmp_path / fam)
    cfg.to_ini(d)
    return d


@pytest.mark.parametrize("fam", sorted(_FAMILIES))
def test_engine_host_side_every_family(hostcheck, fam, tmp_path):
    d = _config_dir(tmp_path, fam)
    _run(hostcheck, d, "bf16", "fp16", 1)
    # two thread ranks: tensor-parallel attention and FFN; whole experts per rank for the routed families
    _run(hostcheck, d, "bf16", "int8" if fam != "chatglm" else "fp16", 2)
    if fam == "qwen3_moe":
        _run(hostcheck, d, "bf16", "fp16", 4)                                          # 6 experts over 4 ranks: 2, 2, 1, 1


@pytest.mark.parametrize("fam", ["llama", "chatglm2", "gpt"])
@pytest.mark.parametrize("dtype", ["int8", "w8a8", "int4", "nf4", "bf16_int8", "w8a8_nf4"])
def test_engine_host_side_weight_types(hostcheck, fam, dtype, tmp_path):
    d = _config_dir(tmp_path, fam)
    _run(hostcheck, d, dtype, "fp16", 1)
    if dtype in ("int8", "w8a8_nf4"):
        _run(hostcheck, d, dtype, "int8", 3)                                           # three ranks: uneven ranges


def _deepseek_config(**kw):
    base = dict(model_type="deepseek_moe", num_layer=3, hidden_size=256, head_num=4, kv_head_num=4, size_per_head=128,
                inter_size=512, vocab_size=300, max_pos_seq_len=4096, q_lora_rank=64, kv_lora_rank=512,
                qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, moe_intermediate_size=128,
                first_k_dense_replace=1, dense_experts=1, sparse_experts=8, routed_scaling_factor=2.5,
                topk_method="noaux_tc", n_group=1, topk_group=1, num_experts_per_tok=8, norm_topk_prob=True,
                scoring_func="sigmoid", activation_type="silu", weight_data_type="bf16", start_id=0, end_id=1,
                rope=RopeConfig(theta=10000, scaling_type="yarn", scaling_factor=40, original_max_pos=4096,
                                beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0))
    base.update(kw)
    return ModelConfig(**base)


@pytest.mark.parametrize("fam", ["mixtral", "qwen3_moe"])
@pytest.mark.parametrize("dtype", ["int8", "w8a8", "nf4", "int4", "bf16_int8", "w8a8_nf4"])
def test_engine_host_side_quantised_expert_families(hostcheck, fam, dtype, tmp_path):
    d = _config_dir(tmp_path, fam)
    _run(hostcheck, d, dtype, "int8", 1)
    _run(hostcheck, d, dtype, "fp16", 2)


def test_engine_host_side_deepseek(hostcheck, tmp_path):
    cfg = ModelConfig(model_type="deepseek_moe", num_layer=3, hidden_size=256, head_num=4, kv_head_num=4, size_per_head=128,
                      inter_size=512, vocab_size=300, max_pos_seq_len=4096, q_lora_rank=64, kv_lora_rank=512,
                      qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, moe_intermediate_size=64,
                      first_k_dense_replace=1, dense_experts=1, sparse_experts=8, routed_scaling_factor=2.5,
                      topk_method="noaux_tc", n_group=4, topk_group=2, num_experts_per_tok=3, norm_topk_prob=True,
                      scoring_func="sigmoid", activation_type="silu", weight_data_type="bf16", start_id=0, end_id=1,
                      rope=RopeConfig(theta=10000, scaling_type="yarn", scaling_factor=40, original_max_pos=4096,
                                      beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0))
    d = str(tmp_path / "deepseek_moe")
    cfg.to_ini(d)
    _run(hostcheck, d, "bf16", "fp16", 1)
    _run(hostcheck, d, "bf16", "fp16", 2)                       # heads, dense FFN, shared experts and experts split
    _run(hostcheck, d, "bf16", "fp16", 4)                       # one head per rank; the narrow shared expert leaves ranks empty
    cfg.q_lora_rank = 0                                                                # no query compression
    d2 = str(tmp_path / "deepseek_moe_noq")
    cfg.to_ini(d2)
    _run(hostcheck, d2, "bf16", "fp16", 1)
    _run(hostcheck, d2, "bf16", "fp16", 3)


@pytest.mark.parametrize("qt,dtype", [("int8", "int8"), ("int8", "w8a8"), ("uint4", "int4"), ("uint4", "bf16_int8")])
def test_engine_host_side_gptq_checkpoint(hostcheck, qt, dtype, tmp_path):
    """Real files: a GPTQ-converted directory (codes + scales + zeros), on one rank and sliced over two."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from gptq_util import make_gptq_dir
    cfg = ModelConfig(**dict(_BASE, model_type="llama"))
    d = make_gptq_dir(str(tmp_path / "gptq"), cfg, qt, seed=1)
    _run(hostcheck, d, dtype, "fp16", 1, fake=False)
    _run(hostcheck, d, dtype, "fp16", 2, fake=False)


# ------------------------------------------------------------------------------------------------------------------
# numerics: the C++ engine over the arithmetic stand-in against the package's fp32 PyTorch path

def _engine_logits(exe, d, ranks, prompt, steps, kv="fp16", wdt="bf16", stages=1, micro=1, extra_env=None, expect_stderr=None):
    B, P = prompt.shape
    idf, outf = os.path.join(d, "ids.txt"), os.path.join(d, "logits.%d.bin" % ranks)
    with open(idf, "w") as f:
        f.write("%d %d %d\n" % (B, P, steps) + " ".join(str(int(x)) for x in prompt.flatten().tolist()) + "\n")
    env = dict(os.environ, XFT_MOCK_MATH="1", XFT_ARENA_EXACT="1", ASAN_OPTIONS="detect_leaks=1", XFT_PIPELINE_STAGE=str(stages),
               XFT_MAX_REQUEST_NUM=str(micro))
    env.pop("XFT_FAKE_MODEL", None)
    env.update(extra_env or {})
    r = subprocess.run([exe, "logits", d, wdt, kv, str(ranks), idf, outf], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "hostcheck logits ok" in r.stdout, (d, ranks, r.stdout[-500:], r.stderr[-3000:])
    if expect_stderr is not None:
        assert (expect_stderr[0] in r.stderr) == expect_stderr[1], r.stderr[-1000:]
    raw = open(outf, "rb").read()
    b, v, n = struct.unpack("iii", raw[:12])
    lg = np.frombuffer(raw, dtype=np.float32, count=n * b * v, offset=12).reshape(n, b, v)
    tk = np.frombuffer(raw, dtype=np.int32, count=n * b, offset=12 + 4 * n * b * v).reshape(n, b)
    return torch.from_numpy(lg.copy()), torch.from_numpy(tk.copy())


def _oracle_logits(d, prompt, tokens, monkeypatch):
    """Teacher-forced logits [steps + 1, B, V] of the PyTorch path: the prompt, then the engine's tokens one at a time."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.parallel.dist import DistContext
    from xfastertransformer_b200.utils.flags import Env
    monkeypatch.setenv("XFT_ENGINE", "CPU")
    Env._inst = None
    DistContext.reset()
    try:
        m = xft.AutoModel.from_pretrained(d, dtype="bf16")
        P, steps = prompt.shape[1], tokens.shape[0] - 1
        sid = m.set_input_cb(prompt.tolist(), None, P + steps + 2)
        rows = [m.forward_cb().float()]
        for s in range(steps):
            m.set_input_cb(tokens[s].tolist(), sid, P + steps + 2)
            rows.append(m.forward_cb().float())
        m.free_seqs(sid)
        return torch.stack(rows, 0)
    finally:
        monkeypatch.delenv("XFT_ENGINE")
        Env._inst = None
        DistContext.reset()


_NUMERIC = dict(_FAMILIES)
# every expert selected: no discrete routing decision that a last-bit difference could flip
_NUMERIC["mixtral"] = dict(sparse_experts=4, num_experts_per_tok=4)
_NUMERIC["qwen3_moe"] = dict(sparse_experts=4, num_experts_per_tok=4, moe_intermediate_size=128, do_qk_norm=True)
_NUMERIC["mixtral-top2"] = dict(sparse_experts=6, num_experts_per_tok=2)


def _synthetic_dir(tmp_path, fam, extra):
    from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint
    kw = dict(_BASE, model_type=fam.split("-")[0])
    kw.update(extra)
    cfg = ModelConfig(**kw)
    if fam == "yarn_llama":
        cfg.rope.scaling_type, cfg.rope.scaling_factor, cfg.rope.original_max_pos = "yarn", 4.0, 128
    d = str(tmp_path / fam)
    write_synthetic_checkpoint(d, cfg, seed=3, dtype="bf16", std=0.08)
    return d


@pytest.mark.parametrize("fam", sorted(_NUMERIC))
def test_engine_logits_match_pytorch(hostcheck, fam, tmp_path, monkeypatch):
    """Prompt pass and four decode steps of every family: logits of the C++ engine (bf16 roundings where the kernels round)
    within a bf16 tolerance of the fp32 PyTorch path, on one rank and on tensor-parallel thread ranks; ranks among
    themselves must agree bit for bit (the harness checks that)."""
    d = _synthetic_dir(tmp_path, fam, _NUMERIC[fam])
    prompt = torch.randint(5, 290, (2, 20), generator=torch.Generator().manual_seed(4))
    steps = 4
    plans = ((1, "fp16"), (2, "fp16"), (3 if fam in ("llama", "chatglm4", "gpt") else 2, "int8"))
    for ranks, kv in plans:
        got, tokens = _engine_logits(hostcheck, d, ranks, prompt, steps, kv=kv)
        want = _oracle_logits(d, prompt, tokens, monkeypatch)
        top = max(1.0, want.abs().max().item())
        err = (got - want).abs().amax(-1)                   # [steps + 1, B]
        if fam == "mixtral-top2":
            # a near-tie may send a token to another expert: most rows must agree tightly
            assert (err < 0.04 * top).float().mean().item() >= 0.7, (fam, ranks, err.tolist(), top)
        elif fam in ("mixtral", "qwen3_moe"):
            # the expert layers of these random models amplify rounding differences on some rows (the same rows move by
            # as much when the stand-in rounds differently), so: most rows tight, every row bounded
            assert err.median().item() < 0.03 * top and err.max().item() < 0.15 * top, (fam, ranks, err.tolist(), top)
        else:
            assert err.max().item() < (0.04 if kv == "fp16" else 0.08) * top, (fam, ranks, kv, err.tolist(), top)


@pytest.mark.parametrize("case", ["bf16", "fp8_e4m3", "no-q-lora", "grouped"])
def test_engine_logits_match_pytorch_deepseek(hostcheck, case, tmp_path, monkeypatch):
    """DeepSeek (latent attention, YaRN table, dense first layer, shared + routed experts; e4m3 files dequantised at load)
    on 1, 2 and 3 or 4 thread ranks against the fp32 PyTorch path.  "grouped" routes 4 of 16 experts out of the 2 best of
    4 groups: a near-tie may pick another expert for a token, so there most rows must agree tightly."""
    from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint
    kw = {}
    if case == "fp8_e4m3":
        kw["weight_data_type"] = "fp8_e4m3"
    if case == "no-q-lora":
        kw["q_lora_rank"] = 0
    if case == "grouped":
        kw.update(sparse_experts=16, n_group=4, topk_group=2, num_experts_per_tok=4)
    cfg = _deepseek_config(**kw)
    d = str(tmp_path / "ds")
    write_synthetic_checkpoint(d, cfg, seed=0, dtype=cfg.weight_data_type, std=0.05)
    prompt = torch.randint(0, 300, (2, 20), generator=torch.Generator().manual_seed(3))
    ran = "mock device: grouped e4m3 gemm ran"
    for ranks in (1, 2, 3 if case == "no-q-lora" else 4):
        # e4m3 files keep the experts in e4m3 on the device (the grouped e4m3 GEMM runs); bf16 files never reach it
        got, tokens = _engine_logits(hostcheck, d, ranks, prompt, 3, extra_env={"XFT_MOCK_REPORT": "1"},
                                     expect_stderr=(ran, case == "fp8_e4m3"))
        want = _oracle_logits(d, prompt, tokens, monkeypatch)
        top = max(1.0, want.abs().max().item())
        err = (got - want).abs().amax(-1)
        if case == "grouped":
            assert (err < 0.04 * top).float().mean().item() >= 0.6, (case, ranks, err.tolist(), top)
        else:
            assert err.max().item() < 0.04 * top, (case, ranks, err.tolist(), top)
    if case == "fp8_e4m3":
        # XFT_FP8_EXPERTS=0: the experts are dequantised like every other tensor; same logits
        got2, _ = _engine_logits(hostcheck, d, 1, prompt, 3, extra_env={"XFT_MOCK_REPORT": "1", "XFT_FP8_EXPERTS": "0"},
                                 expect_stderr=(ran, False))
        got1, _ = _engine_logits(hostcheck, d, 1, prompt, 3)
        assert (got1 - got2).abs().max().item() < 0.02 * top


@pytest.mark.parametrize("beams,eos", [(1, -1), (3, 299), (4, 17)])
def test_engine_generation_matches_pytorch(hostcheck, beams, eos, tmp_path, monkeypatch):
    """config / input / generate / finalize of the C++ engine (greedy; beam search with the host scorer, beams forking
    and reordering block tables, an eos that ends hypotheses early) against generate() of the package's PyTorch path on
    one and two thread ranks.  Greedy tokens must be equal; beams amplify last-bit differences (a flipped near-tie changes
    which hypotheses survive), so there the sequence log-probability under the fp32 model is compared."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.parallel.dist import DistContext
    from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint
    from xfastertransformer_b200.utils.flags import Env
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", vocab_size=300), seed=5, dtype="bf16", std=0.15)
    prompt = torch.tensor([[5, 17, 99, 200, 3, 42, 7], [9, 8, 250, 6, 5, 4, 3]])
    P, new = prompt.shape[1], 10
    monkeypatch.setenv("XFT_ENGINE", "CPU")
    Env._inst = None
    DistContext.reset()
    try:
        py = xft.AutoModel.from_pretrained(d, dtype="bf16")
        want = py.generate(prompt, max_length=P + new, num_beams=beams, eos_token_id=eos if eos >= 0 else 100000, pad_token_id=0)

        def seq_logprob(row):
            n = len(row)
            while n > P and row[n - 1] == 0:      # padding
                n -= 1
            ids = torch.tensor([row[:n]])
            lp = torch.log_softmax(py(ids[:, :-1]).float()[0], -1)
            return sum(float(lp[t - 1, ids[0, t]]) for t in range(P, n)) / max(n - P, 1)

        for ranks in (1, 2):
            idf, outf = os.path.join(d, "ids.txt"), os.path.join(d, "gen.bin")
            with open(idf, "w") as f:
                f.write("2 %d %d\n" % (P, new) + " ".join(str(int(x)) for x in prompt.flatten().tolist()) + "\n")
            env = dict(os.environ, XFT_MOCK_MATH="1", XFT_ARENA_EXACT="1", ASAN_OPTIONS="detect_leaks=1")
            r = subprocess.run([hostcheck, "generate", d, "bf16", "fp16", str(ranks), idf, outf, str(beams), str(eos)], env=env,
                               capture_output=True, text=True, timeout=900)
            assert r.returncode == 0 and "hostcheck generate ok" in r.stdout, (r.stdout[-500:], r.stderr[-3000:])
            raw = open(outf, "rb").read()
            b, n = struct.unpack("ii", raw[:8])
            got = torch.from_numpy(np.frombuffer(raw, dtype=np.int32, offset=8).reshape(b, n).copy()).long()
            assert b == 2 and torch.equal(got[:, :P], prompt)
            if beams == 1:
                assert torch.equal(got, want[:, :n].long()), (got.tolist(), want.tolist())
                continue
            for row in range(2):
                g, w = seq_logprob(got[row].tolist()), seq_logprob(want[row].tolist())
                assert g >= w - max(0.25, 0.1 * abs(w)), (beams, ranks, row, g, w, got[row].tolist(), want[row].tolist())
    finally:
        monkeypatch.delenv("XFT_ENGINE")
        Env._inst = None
        DistContext.reset()


def _same_dtype_oracle(d, dtype, prompt, tokens, monkeypatch):
    """Teacher-forced logits of the package's PyTorch path with the same weight type (the same quantisation formulas)."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.parallel.dist import DistContext
    from xfastertransformer_b200.utils.flags import Env
    monkeypatch.setenv("XFT_ENGINE", "CPU")
    Env._inst = None
    DistContext.reset()
    try:
        m = xft.AutoModel.from_pretrained(d, dtype=dtype)
        P, steps = prompt.shape[1], tokens.shape[0] - 1
        sid = m.set_input_cb(prompt.tolist(), None, P + steps + 2)
        rows = [m.forward_cb().float()]
        for s in range(steps):
            m.set_input_cb(tokens[s].tolist(), sid, P + steps + 2)
            rows.append(m.forward_cb().float())
        m.free_seqs(sid)
        return torch.stack(rows, 0)
    finally:
        monkeypatch.delenv("XFT_ENGINE")
        Env._inst = None
        DistContext.reset()


@pytest.mark.parametrize("dtype", ["int8", "w8a8", "int4", "nf4", "bf16_int8", "w8a8_nf4"])
def test_engine_logits_quantised_weights(hostcheck, dtype, tmp_path, monkeypatch):
    """Quantise-at-load in the C++ engine (the stand-in follows the quantiser's and the quantised GEMMs' formulas) against
    the PyTorch path with the same weight type: the codes are the same, so the logits agree within bf16 roundings
    (int8 x int8: within the difference between quantising bf16 and fp32 activations).  On two ranks a row-parallel slice
    gets its own per-channel range, so only int8 — whose quantisation error is small — is compared there."""
    d = _synthetic_dir(tmp_path, "llama", {})
    prompt = torch.randint(5, 290, (2, 20), generator=torch.Generator().manual_seed(4))
    for ranks in (1, 2) if dtype in ("int8", "bf16_int8") else (1,):
        got, tokens = _engine_logits(hostcheck, d, ranks, prompt, 3, wdt=dtype)
        want = _same_dtype_oracle(d, dtype, prompt, tokens, monkeypatch)
        top = max(1.0, want.abs().max().item())
        err = (got - want).abs().amax(-1)
        tol = (0.1 if dtype.startswith("w8a8") else 0.04) * (1.5 if ranks > 1 else 1.0)
        assert err.max().item() < tol * top, (dtype, ranks, err.tolist(), top)


@pytest.mark.parametrize("qt,dtype", [("int8", "int8"), ("int8", "w8a8"), ("int8", "bf16"), ("uint4", "int4"), ("uint4", "bf16_int8")])
def test_engine_logits_gptq_checkpoint(hostcheck, qt, dtype, tmp_path, monkeypatch):
    """A GPTQ-converted directory through the C++ engine (codes kept when the weight type matches, dequantised and
    requantised otherwise; code tensors sliced for two ranks) against the Python loader on the same files.  Per-channel
    scales do not change with the slicing, so two ranks are held to the same tolerance as one."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from gptq_util import make_gptq_dir
    d = make_gptq_dir(str(tmp_path / "gptq"), ModelConfig(**dict(_BASE, model_type="llama")), qt, seed=1)
    prompt = torch.randint(5, 290, (2, 20), generator=torch.Generator().manual_seed(4))
    for ranks in (1, 2):
        got, tokens = _engine_logits(hostcheck, d, ranks, prompt, 3, wdt=dtype)
        want = _same_dtype_oracle(d, dtype, prompt, tokens, monkeypatch)
        top = max(1.0, want.abs().max().item())
        err = (got - want).abs().amax(-1)
        assert err.max().item() < (0.1 if dtype == "w8a8" else 0.04) * top, (qt, dtype, ranks, err.tolist(), top)


@pytest.mark.parametrize("fam", ["mixtral", "qwen3_moe"])
@pytest.mark.parametrize("dtype", ["int8", "w8a8", "nf4", "bf16_int8", "w8a8_nf4"])
def test_engine_logits_quantised_expert_families(hostcheck, fam, dtype, tmp_path, monkeypatch):
    """Expert families with a quantised weight type: the attention projections are quantised for real, the experts take
    the values of the quantised weights and stay bf16 on the device — what the Python engine does, against which the
    logits are held (every expert selected, so no routing decision can flip).  A hybrid type keeps two expert stacks:
    the first type's for the prompt pass, the second's for the decode steps."""
    d = _synthetic_dir(tmp_path, fam, _NUMERIC[fam])
    prompt = torch.randint(5, 290, (2, 20), generator=torch.Generator().manual_seed(4))
    got, tokens = _engine_logits(hostcheck, d, 1, prompt, 3, wdt=dtype)
    want = _same_dtype_oracle(d, dtype, prompt, tokens, monkeypatch)
    top = max(1.0, want.abs().max().item())
    err = (got - want).abs().amax(-1)
    assert err.median().item() < (0.06 if dtype.startswith("w8a8") else 0.03) * top and err.max().item() < 0.15 * top, \
        (fam, dtype, err.tolist(), top)


# ------------------------------------------------------------------------------------------------------------------
# pipeline stages (XFT_PIPELINE_STAGE): world = stages x tensor-parallel ranks

@pytest.mark.parametrize("fam,stages,ranks", [("llama", 2, 2), ("llama", 2, 4), ("llama", 3, 3), ("chatglm", 2, 2), ("gpt", 2, 4),
                                              ("mixtral", 2, 4), ("qwen3_moe", 4, 4)])
def test_engine_host_side_pipeline_stages(hostcheck, fam, stages, ranks, tmp_path):
    """Every request shape (batch generation, sampling, beams, continuous batching, prefix sharing) with the layers cut
    into pipeline stages: each stage keeps the KV cache of its own layers, the hidden state crosses the stage borders,
    the logits come back from the last stage, and every rank must end with the same tokens."""
    kw = dict(_BASE, model_type=fam, num_layer=4)
    kw.update(_FAMILIES[fam])
    d = str(tmp_path / fam)
    ModelConfig(**kw).to_ini(d)
    _run(hostcheck, d, "bf16", "int8" if fam == "llama" else "fp16", ranks, stages=stages)


@pytest.mark.parametrize("fam,stages,ranks", [("llama", 2, 2), ("llama", 2, 4), ("llama", 3, 6), ("chatglm", 2, 2), ("telechat", 4, 4),
                                              ("mixtral", 2, 4)])
def test_engine_logits_pipeline_stages(hostcheck, fam, stages, ranks, tmp_path, monkeypatch):
    """Logits of a model cut into pipeline stages (with tensor-parallel groups inside the stages where ranks > stages; four
    layers over three stages: 2 + 1 + 1) against the fp32 PyTorch path."""
    d = _synthetic_dir(tmp_path, fam, dict(_NUMERIC[fam], num_layer=4))
    prompt = torch.randint(5, 290, (2, 20), generator=torch.Generator().manual_seed(4))
    got, tokens = _engine_logits(hostcheck, d, ranks, prompt, 3, stages=stages)
    want = _oracle_logits(d, prompt, tokens, monkeypatch)
    top = max(1.0, want.abs().max().item())
    err = (got - want).abs().amax(-1)
    if fam == "mixtral":
        assert err.median().item() < 0.03 * top and err.max().item() < 0.15 * top, (fam, stages, ranks, err.tolist(), top)
    else:
        assert err.max().item() < 0.04 * top, (fam, stages, ranks, err.tolist(), top)


def test_engine_logits_pipeline_stages_deepseek(hostcheck, tmp_path, monkeypatch):
    """DeepSeek over three stages (the dense first layer alone on stage 0) and over two stages of two ranks each."""
    from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint
    cfg = _deepseek_config()
    d = str(tmp_path / "ds")
    write_synthetic_checkpoint(d, cfg, seed=0, dtype="bf16", std=0.05)
    prompt = torch.randint(0, 300, (2, 20), generator=torch.Generator().manual_seed(3))
    for stages, ranks in ((3, 3), (2, 4)):
        got, tokens = _engine_logits(hostcheck, d, ranks, prompt, 3, stages=stages)
        want = _oracle_logits(d, prompt, tokens, monkeypatch)
        top = max(1.0, want.abs().max().item())
        err = (got - want).abs().amax(-1)
        assert err.max().item() < 0.04 * top, (stages, ranks, err.tolist(), top)


def test_example_programs_over_the_stand_in(hostcheck, tmp_path):
    """examples/cpp/cb_check.cpp (sequences decoded alone and inside a staggered continuous batch must agree) and
    examples/cpp/tp_check.cpp (thread ranks — tensor-parallel, or pipeline stages with -s — against a single rank), built
    over the arithmetic stand-in and run on a CPU box."""
    d = _synthetic_dir(tmp_path, "llama", dict(num_layer=4))
    here = os.path.dirname(hostcheck)
    env = dict(os.environ, XFT_MOCK_MATH="1", XFT_ARENA_EXACT="1", ASAN_OPTIONS="detect_leaks=1")
    env.pop("XFT_FAKE_MODEL", None)
    r = subprocess.run([os.path.join(here, "cb_check"), "-m", d, "-n", "5", "-o", "6", "--stride", "2", "--min_len", "4", "--max_len", "70"],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-1500:])
    # a quantised weight type by name, and a prompt given as ids (the reference's -i)
    r = subprocess.run([os.path.join(here, "cb_check"), "-m", d, "-d", "w8a8", "-n", "3", "-o", "4", "-i", "5 6 7 8 9 10 11", "--tolerate", "1"],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-1500:])
    assert subprocess.run([os.path.join(here, "cb_check"), "-m", d, "-d", "int3"], env=env, capture_output=True, text=True,
                          timeout=60).returncode == 2
    assert subprocess.run([os.path.join(here, "cb_check"), "-m", d, "-i", "some text"], env=env, capture_output=True, text=True,
                          timeout=60).returncode == 2                     # text needs -t
    for extra in (["-n", "2"], ["-n", "3", "-d", "int8", "--kv_cache_dtype", "int8"], ["-n", "4", "-s", "2"], ["-n", "2", "-s", "2"]):
        r = subprocess.run([os.path.join(here, "tp_check"), "-m", d, "-o", "3"] + extra, env=env, capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, (extra, r.stdout[-1500:], r.stderr[-1500:])


def test_engine_pipeline_micro_batches(hostcheck, tmp_path, monkeypatch):
    """XFT_MAX_REQUEST_NUM cuts the sequences of a forward pass into micro-batches that travel through the stages one
    after the other; the logits are collected on the last stage and shared once.  Every request shape with 2 and 3
    micro-batches, and the logits of three sequences in two micro-batches (2 + 1) against the fp32 PyTorch path."""
    kw = dict(_BASE, model_type="llama", num_layer=4)
    d = str(tmp_path / "cfg")
    ModelConfig(**kw).to_ini(d)
    _run(hostcheck, d, "bf16", "fp16", 2, stages=2, micro=2)
    _run(hostcheck, d, "bf16", "int8", 4, stages=2, micro=3)
    d2 = _synthetic_dir(tmp_path, "llama", dict(num_layer=4))
    prompt = torch.randint(5, 290, (3, 20), generator=torch.Generator().manual_seed(4))
    got, tokens = _engine_logits(hostcheck, d2, 4, prompt, 3, stages=2, micro=2)
    want = _oracle_logits(d2, prompt, tokens, monkeypatch)
    top = max(1.0, want.abs().max().item())
    assert (got - want).abs().max().item() < 0.04 * top


@pytest.mark.parametrize("fam,world,stages", [("llama", 2, 1), ("llama", 4, 2), ("chatglm2", 3, 1), ("mixtral", 2, 1), ("llama", 2, 2)])
def test_engine_process_ranks_over_stand_in_nccl(hostcheck, fam, world, stages, tmp_path, monkeypatch):
    """The engine as REAL processes, one per rank, that find their rank in the launcher's variables and meet through the
    NCCL communicator (csrc/core/comm.cc: library opened with dlopen, id through a file, bf16 sums, gathers, host
    broadcasts, and for pipeline stages send / receive and the split into tensor-parallel groups) — against a stand-in
    NCCL over shared memory and the arithmetic stand-in of the device library.  Rank 0 writes the logits, which are
    compared with the fp32 PyTorch path."""
    d = _synthetic_dir(tmp_path, fam, dict(_NUMERIC[fam], num_layer=4))
    prompt = torch.randint(5, 290, (2, 20), generator=torch.Generator().manual_seed(4))
    steps = 3
    idf, outf = os.path.join(d, "ids.txt"), os.path.join(d, "logits.procs.bin")
    with open(idf, "w") as f:
        f.write("2 20 %d\n" % steps + " ".join(str(int(x)) for x in prompt.flatten().tolist()) + "\n")
    here = os.path.dirname(hostcheck)
    procs = []
    for r in range(world):
        env = dict(os.environ, XFT_MOCK_MATH="1", XFT_ARENA_EXACT="1", ASAN_OPTIONS="detect_leaks=1", RANK=str(r), WORLD_SIZE=str(world),
                   LOCAL_RANK=str(r), XFT_NCCL_LIB=os.path.join(here, "libfake_nccl.so"), XFT_COMM_ID_FILE=str(tmp_path / "nccl_id"),
                   XFT_DIST_TIMEOUT_S="60", XFT_PIPELINE_STAGE=str(stages))
        for k in ("XFT_FAKE_MODEL", "SINGLE_INSTANCE", "OMPI_COMM_WORLD_RANK", "PMI_RANK"):
            env.pop(k, None)
        procs.append(subprocess.Popen([hostcheck, "logits", d, "bf16", "fp16", "env", idf, outf], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=600) for p in procs]
    for r, (p, (so, se)) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, (r, so[-500:], se[-3000:])
    assert "hostcheck logits ok" in outs[0][0]
    raw = open(outf, "rb").read()
    b, v, n = struct.unpack("iii", raw[:12])
    got = torch.from_numpy(np.frombuffer(raw, dtype=np.float32, count=n * b * v, offset=12).reshape(n, b, v).copy())
    tokens = torch.from_numpy(np.frombuffer(raw, dtype=np.int32, count=n * b, offset=12 + 4 * n * b * v).reshape(n, b).copy())
    want = _oracle_logits(d, prompt, tokens, monkeypatch)
    top = max(1.0, want.abs().max().item())
    err = (got - want).abs().amax(-1)
    if fam == "mixtral":
        assert err.median().item() < 0.03 * top and err.max().item() < 0.15 * top, (fam, world, err.tolist(), top)
    else:
        assert err.max().item() < 0.04 * top, (fam, world, stages, err.tolist(), top)


def test_gpu_rank_cases_over_the_stand_in(hostcheck, tmp_path):
    """The cases of tests/test_zzz_cpp_ranks_gpu.py (tp_check on expert families, DeepSeek, pipeline stages) with the same
    checkpoints and tolerances, over the arithmetic stand-in: what runs there on a GPU has run here first."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("cpp_ranks_gpu", os.path.join(ROOT, "tests", "test_zzz_cpp_ranks_gpu.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    exe = os.path.join(os.path.dirname(hostcheck), "tp_check")
    env = dict(os.environ, XFT_MOCK_MATH="1", XFT_ARENA_EXACT="1", ASAN_OPTIONS="detect_leaks=1")
    for k in ("XFT_FAKE_MODEL", "XFT_PIPELINE_STAGE"):
        env.pop(k, None)
    for i, case in enumerate(sorted(mod.CASES)):
        sub = tmp_path / ("c%d" % i)
        sub.mkdir()
        mod.tp_check_case(exe, case, sub, env=env)
    for i, (ranks, dtype) in enumerate(((["-n", "2"], "bf16"), (["-n", "4", "-s", "2"], "bf16"), (["-n", "2"], "fp8_e4m3"))):
        sub = tmp_path / ("d%d" % i)
        sub.mkdir()
        mod.deepseek_case(exe, ranks, sub, env=env, dtype=dtype)


@pytest.mark.parametrize("fam", ["llama", "chatglm", "mixtral"])
def test_engine_debug_dumps_match_python_layer_by_layer(hostcheck, fam, tmp_path, monkeypatch):
    """XFT_DEBUG_DIR: the C++ engine writes the hidden state after the embedding and after every attention and FFN block
    under the names the Python engine uses, so the two can be compared layer by layer — done here for the prompt pass
    (the C++ side over the arithmetic stand-in, the Python side on its fp32 path)."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.parallel.dist import DistContext
    from xfastertransformer_b200.utils import debugger
    from xfastertransformer_b200.utils.flags import Env
    d = _synthetic_dir(tmp_path, fam, _NUMERIC[fam])
    prompt = torch.randint(5, 290, (2, 20), generator=torch.Generator().manual_seed(4))
    cpp_dir, py_dir = str(tmp_path / "cpp_dump"), str(tmp_path / "py_dump")
    os.makedirs(cpp_dir)
    _engine_logits(hostcheck, d, 1, prompt, 0, extra_env={"XFT_DEBUG_DIR": cpp_dir})
    monkeypatch.setenv("XFT_ENGINE", "CPU")
    monkeypatch.setenv("XFT_DEBUG_DIR", py_dir)
    Env._inst = None
    DistContext.reset()
    try:
        m = xft.AutoModel.from_pretrained(d, dtype="bf16")
        first = debugger._step + 1
        sid = m.set_input_cb(prompt.tolist(), None, 30)
        m.forward_cb()
        m.free_seqs(sid)
    finally:
        monkeypatch.delenv("XFT_ENGINE")
        monkeypatch.delenv("XFT_DEBUG_DIR")
        Env._inst = None
        DistContext.reset()
    names = ["embedding"] + ["layer%d_%s_out" % (l, w) for l in range(2) for w in ("attn", "ffn")]
    log = open(os.path.join(cpp_dir, "rank0.log")).read()
    for name in names:
        got = torch.from_numpy(np.fromfile(os.path.join(cpp_dir, "rank0_step1_%s.bin" % name), dtype=np.float32).reshape(-1, 256))
        want = torch.load(os.path.join(py_dir, "rank0_step%d_%s.pt" % (first, name)))
        assert got.shape == want.shape == (40, 256), (name, got.shape, want.shape)
        scale = max(1.0, want.abs().max().item())
        # (the expert layers of the random Mixtral amplify rounding differences on single elements; see the logits test)
        diff = (got - want).abs()
        assert diff.max().item() < (0.06 if fam == "mixtral" else 0.03) * scale and diff.mean().item() < 0.005 * scale, \
            (fam, name, diff.max().item(), diff.mean().item(), scale)
        assert ("step 1 %s: shape (40, 256) dtype bf16" % name) in log


def test_engine_fake_load_info(hostcheck, tmp_path):
    """XFT_FAKE_LOAD_INFO with XFT_FAKE_MODEL: the engine names every tensor a real load would have read."""
    d = _config_dir(tmp_path, "llama")
    env = dict(os.environ, XFT_FAKE_MODEL="2", XFT_FAKE_LOAD_INFO="1", XFT_ARENA_EXACT="1")
    r = subprocess.run([hostcheck, d, "bf16", "fp16", "1"], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "hostcheck ok" in r.stdout, r.stderr[-2000:]
    for name in ("model.wte.bin", "model.lm_head.weight.bin", "model.layers.1.attention.query_key_value.weight.0.bin",
                 "model.layers.0.mlp.down_proj.weight.0.bin", "model.final_layernorm.weight.bin"):
        assert "[fake load] " + name in r.stdout, name


def test_engine_verbose_lines(hostcheck, tmp_path):
    """XFT_VERBOSE=1: one line per GEMM-shaped call in the reference's format, with the shapes of the call."""
    d = _config_dir(tmp_path, "llama")
    with open(os.path.join(d, "ids.txt"), "w") as f:
        f.write("1 4 0\n5 6 7 8\n")
    env = dict(os.environ, XFT_FAKE_MODEL="2", XFT_VERBOSE="1")
    r = subprocess.run([hostcheck, "logits", d, "int8", "fp16", "1", os.path.join(d, "ids.txt"), os.path.join(d, "o.bin")], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("xft_verbose,exec,gpu,api,")]
    # per layer: qkv, o, gate‖up, down (int8 weights), and the bf16 lm_head on the last row
    assert "xft_verbose,exec,gpu,api,gemm_int8,m4n512k256," in r.stdout                 # QKV: (4 + 2 * 2) heads of 64
    assert "xft_verbose,exec,gpu,api,gemm_int8,m4n1024k256," in r.stdout                # gate and up: 2 x 512
    assert "xft_verbose,exec,gpu,api,gemm_bf16,m1n300k256," in r.stdout                 # lm_head
    assert len(lines) == 2 * 4 + 1 and all(float(l.rsplit(",", 1)[1]) >= 0 for l in lines), lines


@pytest.mark.parametrize("fam,ranks,stages", [("llama", 1, 1), ("chatglm", 2, 1), ("llama", 2, 2)])
def test_engine_token_budget_groups(hostcheck, fam, ranks, stages, tmp_path):
    """XFT_MAX_BATCH_TOKENS: three prompts of 20 tokens under a budget of 25 run as three groups (45 under a budget of 45:
    two groups), the logits are put together in the order of the sequences — the same numbers as in one pass, since a
    sequence never shares arithmetic with its neighbours; every request shape also runs under a small budget."""
    d = _synthetic_dir(tmp_path, fam, dict(_NUMERIC[fam], num_layer=2))
    prompt = torch.randint(5, 290, (3, 20), generator=torch.Generator().manual_seed(4))
    whole, tok0 = _engine_logits(hostcheck, d, ranks, prompt, 2, stages=stages)
    for budget in ("25", "45"):
        got, tok = _engine_logits(hostcheck, d, ranks, prompt, 2, stages=stages, extra_env={"XFT_MAX_BATCH_TOKENS": budget})
        assert torch.equal(tok, tok0) and torch.equal(got, whole), (budget, (got - whole).abs().max().item())
    cfg = str(tmp_path / "cfg")
    ModelConfig(**dict(_BASE, model_type=fam.split("-")[0], **_FAMILIES[fam])).to_ini(cfg)
    env = dict(os.environ, XFT_FAKE_MODEL="2", XFT_ARENA_EXACT="1", ASAN_OPTIONS="detect_leaks=1", XFT_MAX_BATCH_TOKENS="70",
               XFT_PIPELINE_STAGE=str(stages))
    r = subprocess.run([hostcheck, cfg, "bf16", "fp16", str(ranks)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "hostcheck ok" in r.stdout, (r.stdout[-500:], r.stderr[-3000:])


@pytest.mark.parametrize("dtype,ranks", [("bf16", 5), ("w8a8", 8), ("nf4", 3)])
def test_engine_host_side_odd_sizes_and_rank_counts(hostcheck, dtype, ranks, tmp_path):
    """Sizes that do not divide: 8 query heads over 2 KV heads, an FFN of 1408 (22 x 64), an odd vocabulary (4003), on 3, 5
    and 8 ranks — ranks share KV heads, the FFN and vocabulary slices differ in width."""
    cfg = ModelConfig(**dict(_BASE, model_type="llama", hidden_size=512, head_num=8, kv_head_num=2, inter_size=1408, vocab_size=4003))
    d = str(tmp_path / "odd")
    cfg.to_ini(d)
    _run(hostcheck, d, dtype, "int8", ranks)


def test_engine_logits_odd_sizes_on_many_ranks(hostcheck, tmp_path, monkeypatch):
    """The logits of a model whose sizes do not divide (8 query heads over 2 KV heads, FFN 1408, vocabulary 1003) on 5 and
    8 tensor-parallel ranks against the fp32 PyTorch path."""
    d = _synthetic_dir(tmp_path, "llama", dict(hidden_size=512, head_num=8, kv_head_num=2, inter_size=1408, vocab_size=1003))
    prompt = torch.randint(5, 990, (2, 20), generator=torch.Generator().manual_seed(4))
    for ranks in (5, 8):
        got, tokens = _engine_logits(hostcheck, d, ranks, prompt, 2)
        want = _oracle_logits(d, prompt, tokens, monkeypatch)
        top = max(1.0, want.abs().max().item())
        assert (got - want).abs().max().item() < 0.04 * top, (ranks, (got - want).abs().max().item(), top)


def test_engine_thread_ranks_under_thread_sanitizer(tmp_path):
    """Race detection: the whole engine as thread ranks under ThreadSanitizer — the ranks share process-wide state (the
    device arena, the flags, cached tables), which is safe only because one rank runs at a time.  Tensor-parallel ranks
    with int8 KV, pipeline stages with micro-batches, expert-parallel ranks: no report."""
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    flags = ["-O1", "-g", "-std=c++17", "-fsanitize=thread", "-I", os.path.join(ROOT, "csrc", "api"), "-I", os.path.join(ROOT, "csrc", "core"),
             "-I", "/usr/local/cuda/include"]
    srcs = [os.path.join(ROOT, "csrc", "tests", "engine_hostcheck.cc"), os.path.join(ROOT, "csrc", "tests", "mock_device.cc")] + \
           [os.path.join(ROOT, "csrc", "core", f) for f in CORE]
    jobs = []
    for src in srcs:
        obj = str(tmp_path / (os.path.basename(src) + ".o"))
        jobs.append((obj, subprocess.Popen(["g++"] + flags + ["-c", src, "-o", obj], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for obj, job in jobs:
        log = job.communicate(timeout=900)[0]
        assert job.returncode == 0, log[-4000:]
    exe = str(tmp_path / "hostcheck_tsan")
    b = subprocess.run(["g++", "-fsanitize=thread"] + [o for o, _ in jobs] + ["-o", exe, "-ldl", "-lpthread"], capture_output=True, text=True,
                       timeout=900)
    assert b.returncode == 0, b.stderr[-4000:]
    for fam, dtype, kv, ranks, extra in (("llama", "bf16", "int8", 4, {}), ("llama", "w8a8", "fp16", 4, dict(XFT_PIPELINE_STAGE="2", XFT_MAX_REQUEST_NUM="2")),
                                         ("qwen3_moe", "bf16", "fp16", 4, {})):
        d = _config_dir(tmp_path, fam)
        env = dict(os.environ, XFT_FAKE_MODEL="2", **extra)
        r = subprocess.run([exe, d, dtype, kv, str(ranks)], env=env, capture_output=True, text=True, timeout=900)
        assert r.returncode == 0 and "hostcheck ok" in r.stdout and "ThreadSanitizer" not in r.stderr, (fam, r.stdout[-300:], r.stderr[-3000:])
