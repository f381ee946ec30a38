"""The C++ engine's host side on a CPU box: csrc/tests/engine_hostcheck.cc drives xft::AutoModel through every request
shape over a host stand-in of the device library (csrc/tests/mock_device.cc) whose kernels touch exactly the memory the
real ones read and write; AddressSanitizer + UndefinedBehaviorSanitizer + exact-size buffers (XFT_ARENA_EXACT) then check
buffer sizes, strides, slot / block arithmetic and tensor-parallel ranges for every family, weight type and rank count,
and that thread ranks produce the same tokens."""
import os
import shutil
import subprocess
import sys

import pytest

from xfastertransformer_b200.config import ModelConfig, RopeConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CORE = ["engine.cc", "comm.cc", "runtime.cc", "ini.cc", "beam.cc", "env.cc", "arena.cc", "rope_tables.cc", "gptq.cc"]


@pytest.fixture(scope="module")
def hostcheck(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = str(tmp_path_factory.mktemp("hostcheck") / "engine_hostcheck")
    cmd = ["g++", "-O1", "-g", "-std=c++17", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
           "-fno-omit-frame-pointer", "-I", os.path.join(ROOT, "csrc", "api"), "-I", os.path.join(ROOT, "csrc", "core"),
           "-I", "/usr/local/cuda/include", os.path.join(ROOT, "csrc", "tests", "engine_hostcheck.cc"),
           os.path.join(ROOT, "csrc", "tests", "mock_device.cc")] + [os.path.join(ROOT, "csrc", "core", f) for f in CORE] + \
          ["-o", exe, "-ldl", "-lpthread"]
    b = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert b.returncode == 0, b.stderr[-4000:]
    return exe


def _run(exe, d, dtype, kv, ranks, fake=True):
    env = dict(os.environ, XFT_ARENA_EXACT="1", ASAN_OPTIONS="detect_leaks=1", UBSAN_OPTIONS="print_stacktrace=1")
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
    if fam in _DENSE:
        _run(hostcheck, d, "bf16", "int8" if fam != "chatglm" else "fp16", 2)          # tensor parallel, two thread ranks


@pytest.mark.parametrize("fam", ["llama", "chatglm2", "gpt"])
@pytest.mark.parametrize("dtype", ["int8", "w8a8", "int4", "nf4", "bf16_int8", "w8a8_nf4"])
def test_engine_host_side_weight_types(hostcheck, fam, dtype, tmp_path):
    d = _config_dir(tmp_path, fam)
    _run(hostcheck, d, dtype, "fp16", 1)
    if dtype in ("int8", "w8a8_nf4"):
        _run(hostcheck, d, dtype, "int8", 3)                                           # three ranks: uneven ranges


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
    cfg.q_lora_rank = 0                                                                # no query compression
    d2 = str(tmp_path / "deepseek_moe_noq")
    cfg.to_ini(d2)
    _run(hostcheck, d2, "bf16", "fp16", 1)


@pytest.mark.parametrize("qt,dtype", [("int8", "int8"), ("int8", "w8a8"), ("uint4", "int4"), ("uint4", "bf16_int8")])
def test_engine_host_side_gptq_checkpoint(hostcheck, qt, dtype, tmp_path):
    """Real files: a GPTQ-converted directory (codes + scales + zeros), on one rank and sliced over two."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from gptq_util import make_gptq_dir
    cfg = ModelConfig(**dict(_BASE, model_type="llama"))
    d = make_gptq_dir(str(tmp_path / "gptq"), cfg, qt, seed=1)
    _run(hostcheck, d, dtype, "fp16", 1, fake=False)
    _run(hostcheck, d, dtype, "fp16", 2, fake=False)
