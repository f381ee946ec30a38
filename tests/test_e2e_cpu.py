"""Tiny-Llama end to end on CPU, world_size 1 and 2 (gloo): logits and greedy tokens against an
independent PyTorch-eager model reading the same converted checkpoint."""
import os
import subprocess
import sys

import pytest
import torch

from eager_llama import EagerLlama
from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("tiny_llama"))
    write_synthetic_checkpoint(d, preset("tiny-llama"), seed=0, dtype="bf16")
    return d


def _prompt():
    g = torch.Generator().manual_seed(1)
    return torch.randint(0, 32000, (2, 32), generator=g)


def test_logits_and_greedy_ws1(tiny, monkeypatch):
    monkeypatch.setenv("XFT_ENGINE", "CPU")
    import xfastertransformer_b200 as xft
    model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    ids = _prompt()
    ref = EagerLlama(tiny)
    # prefill logits through the continuous-batching API
    sid = model.set_input_cb(ids.tolist(), None, 64)
    logits = model.forward_cb()
    want = ref.logits(ids)[:, -1]
    assert torch.allclose(logits, want, atol=2e-3, rtol=2e-3), (logits - want).abs().max()
    model.free_seqs(sid)
    # all-position logits
    full = model(ids)
    assert torch.allclose(full, ref.logits(ids), atol=2e-3, rtol=2e-3)
    # greedy decode of 16 tokens
    out = model.generate(ids, max_length=48)
    assert out.shape == (2, 48)
    assert torch.equal(out, ref.greedy(ids, 16))


@pytest.mark.parametrize("spec,overlap", [(0, 0), (4, 0), (0, 1)])
def test_ws2_gloo(tiny, tmp_path, spec, overlap):
    """Two tensor-parallel gloo ranks against the eager reference; spec = 4: the same with n-gram speculative decoding
    (every rank derives the same drafts from the token stream, so the ranks stay in step); overlap = 1: the prefill of
    the two prompts interleaved block by block with asynchronous all-reduces (XFT_PREFILL_OVERLAP)."""
    out = str(tmp_path / "ws2.pt")
    env = dict(os.environ, XFT_ENGINE="CPU", XFT_SPEC_NGRAM=str(spec), XFT_PREFILL_OVERLAP=str(overlap),
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29611 + 50 * (spec > 0) + 90 * overlap),
           os.path.join(ROOT, "tests", "ws2_worker.py"), tiny, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    ids = _prompt()
    ref = EagerLlama(tiny)
    assert torch.allclose(got["logits"], ref.logits(ids)[:, -1], atol=2e-3, rtol=2e-3)
    assert torch.equal(got["tokens"], ref.greedy(ids, 16))
    # TP really split the work: FFN 688 over 2 ranks -> 352 + 336, two allreduces per layer per step
    assert got["ffn"] == [352, 336]
    assert got["all_reduce"] > 0
    assert got["pairs"] == (2 if overlap else 0)          # the forward_cb prefill and generate's prefill, both as a pair


def test_pipeline_parallel_two_stages_gloo(tiny, tmp_path):
    """XFT_PIPELINE_STAGE=2 on two gloo ranks: stage 0 owns layer 0, stage 1 layer 1 and the head; the hidden state
    crosses by send/recv and the logits come back to every stage; tokens equal the single-process greedy result."""
    out = str(tmp_path / "pp2.pt")
    env = dict(os.environ, XFT_ENGINE="CPU", XFT_PIPELINE_STAGE="2",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29613", os.path.join(ROOT, "tests", "pp_worker.py"), tiny, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    ids = _prompt()
    ref = EagerLlama(tiny)
    assert torch.allclose(got["logits"], ref.logits(ids)[:, -1], atol=2e-3, rtol=2e-3)
    assert torch.equal(got["tokens"], ref.greedy(ids, 16))
    assert sorted(got["layers"]) == [(0, 1, 0, 0), (1, 2, 1, 0)]


@pytest.mark.parametrize("dp", [0, 1])
def test_cb_follower_loop_and_greedy_fast_path(tiny, tmp_path, dp):
    """Two gloo ranks: rank 1 only runs follow_cb(); rank 0 mixes forward_cb_greedy and forward_cb steps.  Tokens equal
    the single-process greedy continuation and the follower exits on shutdown.  dp = 1: the same under
    XFT_ATTENTION_DP=1 (a dense model: each rank serves its own sequences with the full weights)."""
    out = str(tmp_path / "cbf.pt")
    env = dict(os.environ, XFT_ENGINE="CPU", XFT_ATTENTION_DP=str(dp),
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29615 + 40 * dp), os.path.join(ROOT, "tests", "cb_follow_worker.py"), tiny, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)["tokens"]
    ids = _prompt()
    ref = EagerLlama(tiny)
    assert torch.equal(got, ref.greedy(ids, 7)[:, ids.shape[1]:])


def test_lost_rank_raises_comm_error_not_hang(tiny, tmp_path):
    """Failure detection on the host: a rank that leaves between requests makes the driver's next request fail with
    CommError within XFT_DIST_TIMEOUT_S."""
    out = str(tmp_path / "lost.txt")
    env = dict(os.environ, XFT_ENGINE="CPU", XFT_DIST_TIMEOUT_S="8",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29617", os.path.join(ROOT, "tests", "lost_rank_worker.py"), tiny, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert os.path.exists(out), r.stdout[-2000:] + r.stderr[-2000:]
    res, secs, width = open(out).read().split("\n")[:3]
    assert res == "CommError", (res, r.stderr[-1500:])
    assert float(secs) < 60 and int(width) == 12


@pytest.mark.parametrize("mt,ep", [("mixtral", 0), ("mixtral", 1), ("deepseek_moe", 1), ("qwen3_moe", 0),
                                   ("mixtral", 2), ("deepseek_moe", 2), ("mixtral", 3), ("deepseek_moe", 4)])
def test_moe_two_ranks_sliced_and_expert_parallel(mt, ep, tmp_path):
    """MoE across two gloo ranks against the single-rank engine on the same files: XFT_EXPERT_PARALLEL=0 slices every
    expert's intermediate dimension (the reference's only mode, src/layers/moe_deepseek.h / mlp_llama.h:70-79), =1
    places whole experts on ranks (each rank runs its own experts on the replicated tokens; the row-parallel reduction
    combines).  ep = 2 stands for XFT_ATTENTION_DP=1: no tensor parallelism, every rank runs attention for its own
    sequences (3 prompts over 2 ranks: 2 + 1) and tokens travel to their experts' ranks and back by all-to-all.
    Prefill and one decode step."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.config import ModelConfig, RopeConfig
    from xfastertransformer_b200.parallel.dist import DistContext
    from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint
    if mt == "deepseek_moe":
        cfg = ModelConfig(model_type=mt, head_num=4, kv_head_num=4, size_per_head=32, hidden_size=128, inter_size=256,
                          num_layer=2, vocab_size=1000, max_pos_seq_len=512, weight_data_type="bf16", q_lora_rank=64,
                          kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                          moe_intermediate_size=64, sparse_experts=8, dense_experts=1, num_experts_per_tok=2, n_group=4,
                          topk_group=2, first_k_dense_replace=1, routed_scaling_factor=2.5, topk_method="noaux_tc",
                          scoring_func="sigmoid", norm_topk_prob=True, activation_type="silu", start_id=1, end_id=2,
                          rope=RopeConfig(theta=10000))
    else:
        cfg = ModelConfig(model_type=mt, num_layer=2, hidden_size=128, head_num=4, kv_head_num=2, size_per_head=32,
                          inter_size=128, moe_intermediate_size=128, vocab_size=1000, max_pos_seq_len=512,
                          sparse_experts=8, num_experts_per_tok=2, norm_topk_prob=True, activation_type="silu",
                          weight_data_type="bf16", do_qk_norm=(mt == "qwen3_moe"), start_id=1, end_id=2)
    d = str(tmp_path / "m")
    write_synthetic_checkpoint(d, cfg, seed=0, dtype="bf16", std=0.05)
    out = str(tmp_path / "moe.pt")
    # ep = 3 / 4: sliced / whole experts with the prefill of the three prompts interleaved (XFT_PREFILL_OVERLAP=1)
    overlap, ep = int(ep >= 3), {3: 0, 4: 1}.get(ep, ep)
    env = dict(os.environ, XFT_ENGINE="CPU", XFT_EXPERT_PARALLEL=str(int(ep == 1)), XFT_ATTENTION_DP=str(int(ep == 2)),
               XFT_PREFILL_OVERLAP=str(overlap), PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    port = 29621 + 2 * (ep + 2 * ["mixtral", "deepseek_moe", "qwen3_moe"].index(mt)) + 100 * overlap
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "moe_tp_worker.py"), d, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    # single rank, same files
    os.environ["XFT_ENGINE"] = "CPU"
    DistContext.reset()
    m = xft.AutoModel.from_pretrained(d, dtype="bf16")
    ids = torch.randint(0, 1000, (3, 20), generator=torch.Generator().manual_seed(2))
    sid = m.set_input_cb(ids.tolist(), None, 64)
    want = m.forward_cb()
    m.set_input_cb(want.argmax(-1).tolist(), sid, 64)
    want2 = m.forward_cb()
    m.free_seqs(sid)
    scale = want.abs().max().item()
    assert (got["logits"] - want).abs().max().item() < 2e-3 * max(scale, 1.0)
    assert (got["logits2"] - want2).abs().max().item() < 2e-3 * max(scale, 1.0)
    I = cfg.moe_intermediate_size if mt != "mixtral" else cfg.inter_size
    if ep:
        assert got["held"] == [(4, 0, I), (4, 4, I)]              # whole experts, half of them each
    else:
        assert [h[0] for h in got["held"]] == [8, 8] and sum(h[2] for h in got["held"]) == I     # every expert, sliced


def test_pipeline_parallel_microbatches_gloo(tiny, tmp_path):
    """XFT_MAX_REQUEST_NUM=2 with two pipeline stages: every forward of a 4-sequence batch is cut into two micro-batches
    that the stages process one behind the other; results equal the single-process greedy decode."""
    out = str(tmp_path / "pp2mb.pt")
    env = dict(os.environ, XFT_ENGINE="CPU", XFT_PIPELINE_STAGE="2", XFT_MAX_REQUEST_NUM="2",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29619", os.path.join(ROOT, "tests", "pp_worker.py"), tiny, out, "4"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    ids = torch.randint(0, 32000, (4, 32), generator=torch.Generator().manual_seed(1))
    ref = EagerLlama(tiny)
    assert torch.allclose(got["logits"], ref.logits(ids)[:, -1], atol=2e-3, rtol=2e-3)
    assert torch.equal(got["tokens"], ref.greedy(ids, 16))
    assert got["microbatches"] == 2 * 17      # forward_cb, then a prefill and 15 decode steps: two micro-batches each


def test_data_parallel_attention_scenarios(tmp_path):
    """XFT_ATTENTION_DP=1 on two gloo ranks against the single-rank engine: a batch of one (rank 1 owns no sequence and
    only serves its experts), prompts whose prefill needs more passes on one rank than on the other
    (XFT_MAX_BATCH_TOKENS=32), beam search (beams stay on their request's rank) and all-position logits."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.config import ModelConfig
    from xfastertransformer_b200.parallel.dist import DistContext
    from xfastertransformer_b200.utils.flags import Env
    cfg = ModelConfig(model_type="mixtral", num_layer=2, hidden_size=128, head_num=4, kv_head_num=2, size_per_head=32,
                      inter_size=128, moe_intermediate_size=128, vocab_size=1000, max_pos_seq_len=512, sparse_experts=8,
                      num_experts_per_tok=2, norm_topk_prob=True, activation_type="silu", weight_data_type="bf16",
                      start_id=1, end_id=2)
    d = str(tmp_path / "m")
    write_synthetic_checkpoint(d, cfg, seed=0, dtype="bf16", std=0.05)
    out = str(tmp_path / "dp.pt")
    env = dict(os.environ, XFT_ENGINE="CPU", XFT_ATTENTION_DP="1", XFT_MAX_BATCH_TOKENS="32",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29641", os.path.join(ROOT, "tests", "dp_worker.py"), d, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    os.environ["XFT_ENGINE"] = "CPU"
    DistContext.reset()
    Env.get().reload()
    m = xft.AutoModel.from_pretrained(d, dtype="bf16")
    g = torch.Generator().manual_seed(4)
    one = torch.randint(0, 1000, (1, 9), generator=g)
    three = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (40, 7, 33)]
    two = torch.randint(0, 1000, (2, 11), generator=g)
    assert torch.equal(got["one"], m.generate(one, max_length=15))
    sid = m.set_input_cb(three, None, 64)
    want = m.forward_cb()
    m.free_seqs(sid)
    assert torch.allclose(got["three"], want, atol=2e-3 * max(1.0, want.abs().max().item()))
    assert torch.equal(got["beams"], m.generate(two, max_length=16, num_beams=2))
    full = m(two)
    assert torch.allclose(got["all"], full, atol=2e-3 * max(1.0, full.abs().max().item()))
    # no tensor parallelism (o_proj sees all 4 heads), both ranks took part in the expert exchange
    assert [i[:2] for i in got["info"]] == [(2, 1), (2, 1)] and all(i[2] > 0 and i[3] == 128 for i in got["info"])
    assert got["info"][0][2] == got["info"][1][2]


def test_general_follower_loop_gloo(tiny, tmp_path):
    """Rank 1 only runs model.follow(); rank 0 mixes generate (greedy, beams), config + input + forward, continuous
    batching and all-position logits.  Everything equals the single-process results and the follower exits on shutdown."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.parallel.dist import DistContext
    from xfastertransformer_b200.utils.flags import Env
    out = str(tmp_path / "follow.pt")
    env = dict(os.environ, XFT_ENGINE="CPU", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29671", os.path.join(ROOT, "tests", "follow_worker.py"), tiny, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    ids = _prompt()
    ref = EagerLlama(tiny)
    assert torch.equal(got["greedy"], ref.greedy(ids, 8))
    assert torch.equal(got["stepwise"], ref.greedy(ids, 4))
    assert torch.allclose(got["cb_logits"], ref.logits(ids)[:, -1], atol=2e-3, rtol=2e-3)
    assert torch.allclose(got["all"], ref.logits(ids[:, :16]), atol=2e-3, rtol=2e-3)
    os.environ["XFT_ENGINE"] = "CPU"
    DistContext.reset()
    Env.get().reload()
    m = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    assert torch.equal(got["beams"], m.generate(ids[:, :12], max_length=18, num_beams=2))


def test_prefix_reuse_under_tensor_parallelism_gloo(tiny, tmp_path):
    """XFT_PREFIX_CACHE=1 on two tensor-parallel gloo ranks: both ranks adopt the same cached blocks (the index is a
    pure function of the token stream), results equal the single-process engine without reuse."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.parallel.dist import DistContext
    from xfastertransformer_b200.utils.flags import Env
    out = str(tmp_path / "prefix.pt")
    env = dict(os.environ, XFT_ENGINE="CPU", XFT_PREFIX_CACHE="1",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29681", os.path.join(ROOT, "tests", "prefix_worker.py"), tiny, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    os.environ["XFT_ENGINE"] = "CPU"
    os.environ.pop("XFT_PREFIX_CACHE", None)
    DistContext.reset()
    Env.get().reload()
    m = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    g = torch.Generator().manual_seed(11)
    common = torch.randint(5, 900, (150,), generator=g).tolist()
    p2 = common + torch.randint(5, 900, (20,), generator=g).tolist()
    sid = m.set_input_cb([p2], None, 256)
    want = m.forward_cb()
    m.free_seqs(sid)
    assert torch.allclose(got["logits"], want, atol=2e-3, rtol=2e-3)
    assert torch.equal(got["tokens"], m.generate(torch.tensor([p2]), max_length=len(p2) + 5))
    assert got["stats"][0] == got["stats"][1] and got["stats"][0][0] == 4          # 2 blocks reused, twice


def test_data_parallel_decode_runner_logic_gloo(tmp_path):
    """The decode runner's data-parallel step (each rank decodes its own sequences, a rank without sequences serves its
    experts, tokens are exchanged on the host) with eager stand-ins for the CUDA-graph parts, on two gloo ranks."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.config import ModelConfig
    from xfastertransformer_b200.parallel.dist import DistContext
    from xfastertransformer_b200.utils.flags import Env
    cfg = ModelConfig(model_type="mixtral", num_layer=2, hidden_size=128, head_num=4, kv_head_num=2, size_per_head=32,
                      inter_size=128, moe_intermediate_size=128, vocab_size=1000, max_pos_seq_len=512, sparse_experts=8,
                      num_experts_per_tok=2, norm_topk_prob=True, activation_type="silu", weight_data_type="bf16",
                      start_id=1, end_id=2)
    d = str(tmp_path / "m")
    write_synthetic_checkpoint(d, cfg, seed=0, dtype="bf16", std=0.05)
    out = str(tmp_path / "dpr.pt")
    env = dict(os.environ, XFT_ENGINE="CPU", XFT_ATTENTION_DP="1",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29695", os.path.join(ROOT, "tests", "dp_runner_worker.py"), d, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    os.environ["XFT_ENGINE"] = "CPU"
    DistContext.reset()
    Env.get().reload()
    m = xft.AutoModel.from_pretrained(d, dtype="bf16")
    g = torch.Generator().manual_seed(4)
    one = torch.randint(0, 1000, (1, 9), generator=g)
    three = torch.randint(0, 1000, (3, 11), generator=g)
    assert torch.equal(got["one"], m.generate(one, max_length=15))
    assert torch.equal(got["three"], m.generate(three, max_length=17))
    # 5 + 5 decode steps after the prefills; rank 1 owns nothing in the first request and one sequence in the second
    assert got["stats"] == [(10, 0), (5, 5)]
