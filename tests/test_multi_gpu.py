"""Multi-GPU tests (one process per GPU over NCCL + peer memory).  Skipped with fewer than two GPUs:
kernels that wait on a peer are never emulated as several launches on one device."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

from eager_llama import EagerLlama
from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_peer_comm_and_model(world, tmp_path):
    if _ngpu() < world:
        pytest.skip(f"needs {world} GPUs")
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama", head_num=8, kv_head_num=8, size_per_head=64, hidden_size=512,
                                         inter_size=1408), seed=0, dtype="bf16", std=0.05)
    out = str(tmp_path / "out.pt")
    env = dict(os.environ, XFT_DIST_TIMEOUT_S="120", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29700 + world), os.path.join(ROOT, "tests", "mgpu_worker.py"), d, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-4000:]
    got = torch.load(out)
    assert got["res"]["allreduce"] == "ok" and got["res"]["gemm_ar"] == "ok"
    assert got["res"]["fused_calls"] > 0, "decode did not use the fused GEMM+all-reduce kernel"
    assert got["res"]["graph_launches"] > 0
    tokens = got["tokens"]
    ref = EagerLlama(d)
    # tensor-parallel logits against the fp32 eager model, within what bf16 activations allow: the prompt's last
    # position (prefill path) and the step after it (decode graph with the fused GEMM + all-reduce kernels)
    prompt = tokens[:, :32]
    want0 = ref.logits(prompt)[:, -1]
    scale = want0.abs().max().item()
    assert (got["logits0"] - want0).abs().max().item() < 4e-2 * scale
    want1 = ref.logits(torch.cat([prompt, got["next"][:, None]], 1))[:, -1]
    assert (got["logits1"] - want1).abs().max().item() < 4e-2 * scale
    full = ref.logits(tokens[:, :-1])
    for b in range(tokens.shape[0]):
        for t in range(32, tokens.shape[1]):
            row = full[b, t - 1]
            assert row[tokens[b, t]] >= row.max() - 0.05 * max(1.0, row.abs().max().item()), (b, t)


def test_pipeline_parallel_two_gpus(tmp_path):
    """Two pipeline stages on two GPUs (NCCL send/recv of the hidden state, logits broadcast back): every generated
    token is (near-)argmax of the fp32 eager model's logits."""
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama"), seed=0, dtype="bf16", std=0.05)
    out = str(tmp_path / "pp.pt")
    env = dict(os.environ, XFT_DIST_TIMEOUT_S="120", XFT_PIPELINE_STAGE="2", NCCL_NVLS_ENABLE="0",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29731", os.path.join(ROOT, "tests", "pp_worker.py"), d, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-4000:]
    got = torch.load(out)
    assert sorted(got["layers"]) == [(0, 1, 0, 0), (1, 2, 1, 0)]
    tokens = got["tokens"]
    ref = EagerLlama(d)
    full = ref.logits(tokens[:, :-1])
    for b in range(tokens.shape[0]):
        for t in range(32, tokens.shape[1]):
            row = full[b, t - 1]
            assert row[tokens[b, t]] >= row.max() - 0.1 * max(1.0, row.abs().max().item()), (b, t)
