"""The C++ engine's newer rank layouts on ONE GPU, as thread ranks (examples/cpp/tp_check.cpp: N ranks as threads of one
process against the single-rank engine, logits of the prompt pass and of teacher-forced decode steps): routed experts
as whole experts per rank, DeepSeek's latent attention split by query head, pipeline stages with tensor-parallel groups
inside.  The same cases run on a CPU box over the stand-in device library (tests/test_cpp_engine_host.py)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# (family, extra config, tp_check arguments, tolerance).  The expert families select every expert: no routing decision
# that a different summation order could flip.
CASES = {
    "llama-2-stages": ("llama", dict(num_layer=4), ["-n", "2", "-s", "2"], 0.05),
    "llama-2x2-stages": ("llama", dict(num_layer=4), ["-n", "4", "-s", "2"], 0.05),
    "chatglm-3-stages": ("chatglm", dict(num_layer=4, kv_head_num=4, activation_type="gelu"), ["-n", "3", "-s", "3"], 0.05),
    "mixtral-2": ("mixtral", dict(sparse_experts=4, num_experts_per_tok=4), ["-n", "2"], 0.15),
    "qwen3_moe-4": ("qwen3_moe", dict(sparse_experts=6, num_experts_per_tok=6, moe_intermediate_size=128, do_qk_norm=True,
                                      kv_head_num=4), ["-n", "4"], 0.15),
    "mixtral-2x2-stages": ("mixtral", dict(sparse_experts=4, num_experts_per_tok=4), ["-n", "4", "-s", "2"], 0.15),
}


def tp_check_case(exe, case, tmp_path, env=None):
    from xfastertransformer_b200.config import ModelConfig
    from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint
    fam, extra, args, tol = CASES[case]
    kw = dict(model_type=fam, num_layer=2, hidden_size=256, head_num=4, kv_head_num=2, size_per_head=64, inter_size=512,
              vocab_size=2000, max_pos_seq_len=512, activation_type="silu", weight_data_type="bf16", start_id=1, end_id=2)
    kw.update(extra)
    d = str(tmp_path / "m")
    write_synthetic_checkpoint(d, ModelConfig(**kw), seed=8, dtype="bf16", std=0.08)
    r = subprocess.run([exe, "-m", d, "-o", "4", "--tol", str(tol)] + args, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "tensor-parallel ranks agree" in r.stdout, r.stdout


def deepseek_case(exe, ranks, tmp_path, env=None, dtype="bf16"):
    from xfastertransformer_b200.config import ModelConfig, RopeConfig
    from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint
    cfg = ModelConfig(model_type="deepseek_moe", num_layer=3, hidden_size=512, head_num=8, kv_head_num=8, size_per_head=128,
                      inter_size=1024, vocab_size=1024, max_pos_seq_len=4096, q_lora_rank=256, kv_lora_rank=512,
                      qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, moe_intermediate_size=256,
                      first_k_dense_replace=1, dense_experts=1, routed_scaling_factor=2.5, topk_method="noaux_tc",
                      norm_topk_prob=True, scoring_func="sigmoid", activation_type="silu", weight_data_type=dtype,
                      start_id=0, end_id=1, sparse_experts=8, n_group=1, topk_group=1, num_experts_per_tok=8,
                      rope=RopeConfig(theta=10000, scaling_type="yarn", scaling_factor=40, original_max_pos=4096,
                                      beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0))
    d = str(tmp_path / "ds")
    write_synthetic_checkpoint(d, cfg, seed=0, dtype=dtype, std=0.05)
    r = subprocess.run([exe, "-m", d, "-o", "3", "--tol", "0.1"] + ranks, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "tensor-parallel ranks agree" in r.stdout, r.stdout


def _exe():
    exe = os.path.join(ROOT, "xfastertransformer_b200", "lib", "xft_tp_check")
    if not os.path.exists(exe):
        pytest.skip("tp_check not built")
    return exe


@pytest.mark.parametrize("case", sorted(CASES))
def test_cpp_thread_ranks_experts_and_stages(case, tmp_path):
    tp_check_case(_exe(), case, tmp_path)


@pytest.mark.parametrize("ranks,dtype", [(["-n", "2"], "bf16"), (["-n", "4", "-s", "2"], "bf16"), (["-n", "2"], "fp8_e4m3")])
def test_cpp_thread_ranks_deepseek(ranks, dtype, tmp_path):
    """DeepSeek on two ranks (query heads, dense FFN, shared experts and routed experts split), as two pipeline stages of
    two ranks, and from an e4m3 checkpoint (routed experts kept in e4m3 on the device, a run of them per rank)."""
    deepseek_case(_exe(), ranks, tmp_path, dtype=dtype)
