"""MoE kernels (routers, dispatch plan, grouped tcgen05 GEMM, combine) and the MoE model families on one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from xfastertransformer_b200.ops import reference as R
from xfastertransformer_b200.runtime.loader import make_linear


@pytest.mark.parametrize("kind,E,k", [("mixtral", 8, 2), ("softmax_topk", 128, 8), ("deepseek", 256, 8), ("deepseek", 64, 6)])
def test_routers(kind, E, k):
    from xfastertransformer_b200.ops import native as Nat
    g = torch.Generator().manual_seed(E)
    logits = torch.randn(37, E, generator=g)
    bias = torch.randn(E, generator=g) * 0.1 if kind == "deepseek" else None
    ng, tg = (8, 4) if kind == "deepseek" else (1, 1)
    if kind == "mixtral":
        wi, ww = R.route_mixtral(logits, k)
    elif kind == "softmax_topk":
        wi, ww = R.route_softmax_topk(logits, k, True)
    else:
        wi, ww = R.route_deepseek(logits, bias, k, ng, tg, 2.5, True, "sigmoid")
    gi, gw = Nat.route(logits.cuda(), kind, k, None if bias is None else bias.cuda(), ng, tg, 2.5, True, "sigmoid")
    # same expert sets and weights (order inside the k slots may differ on ties only)
    gi, gw = gi.cpu().long(), gw.cpu()
    for t in range(logits.shape[0]):
        assert sorted(gi[t].tolist()) == sorted(wi[t].tolist()), (t, gi[t], wi[t])
        a = dict(zip(gi[t].tolist(), gw[t].tolist()))
        b = dict(zip(wi[t].tolist(), ww[t].tolist()))
        for e in a:
            assert abs(a[e] - b[e]) < 1e-4 * max(1.0, abs(b[e])), (t, e, a[e], b[e])


@pytest.mark.parametrize("T,E,k,I,H", [(5, 8, 2, 256, 512), (64, 8, 2, 352, 256), (33, 32, 4, 128, 1024), (300, 16, 2, 256, 512)])
def test_moe_experts_grouped(T, E, k, I, H):
    from xfastertransformer_b200.ops import native as Nat
    g = torch.Generator().manual_seed(T + E)
    x = (torch.randn(T, H, generator=g) * 0.5).bfloat16()
    experts = []
    for _ in range(E):
        gu = make_linear(torch.randn(2 * I, H, generator=g) * 0.05, "bf16")
        dn = make_linear(torch.randn(H, I, generator=g) * 0.05, "bf16")
        experts.append((gu, dn))
    logits = torch.randn(T, E, generator=g)
    idx, w = R.route_mixtral(logits, k)
    want = R.moe_experts(x.float(), idx, w, experts, "silu")
    # only experts 2.. are "local" in a second run (expert-parallel shard)
    cuda_experts = [(a.to("cuda"), b.to("cuda")) for a, b in experts]
    got = Nat.moe_experts(x.cuda(), idx.cuda().int(), w.cuda(), cuda_experts, "silu")
    Nat.Workspace.get(torch.device("cuda", 0)).check_status()
    err = (got.cpu() - want).abs().max().item()
    assert err < 3e-2 * max(1.0, want.abs().max().item()), err
    lo = 2
    want2 = R.moe_experts(x.float(), idx, w, experts[lo:], "silu", expert_offset=lo)
    shard = cuda_experts[lo:]
    got2 = Nat.moe_experts(x.cuda(), idx.cuda().int(), w.cuda(), shard, "silu", expert_offset=lo)
    err2 = (got2.cpu() - want2).abs().max().item()
    assert err2 < 3e-2 * max(1.0, want2.abs().max().item()), err2


@pytest.mark.parametrize("mt", ["mixtral", "qwen3_moe"])
def test_tiny_moe_models(mt, tmp_path):
    """Tiny MoE checkpoints: GPU logits vs the CPU engine (pure PyTorch path) on the same files."""
    import subprocess, sys, os
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.config import ModelConfig
    from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint
    cfg = ModelConfig(model_type=mt, num_layer=2, hidden_size=256, head_num=4, kv_head_num=2, size_per_head=64,
                      inter_size=384, moe_intermediate_size=384, vocab_size=1024, max_pos_seq_len=512,
                      sparse_experts=8, num_experts_per_tok=2, norm_topk_prob=True, activation_type="silu",
                      weight_data_type="bf16", do_qk_norm=(mt == "qwen3_moe"), start_id=1, end_id=2)
    d = str(tmp_path / mt)
    write_synthetic_checkpoint(d, cfg, seed=0, dtype="bf16", std=0.05)
    ids = torch.randint(0, 1024, (3, 20), generator=torch.Generator().manual_seed(2))
    m = xft.AutoModel.from_pretrained(d, dtype="bf16")
    sid = m.set_input_cb(ids.tolist(), None, 64)
    got = m.forward_cb().cpu()
    m.free_seqs(sid)
    out = m.generate(ids, max_length=28)
    assert out.shape == (3, 28)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import sys,torch; sys.path.insert(0, %r); import xfastertransformer_b200 as xft;"
            "m = xft.AutoModel.from_pretrained(%r, dtype='bf16'); ids = torch.load(%r);"
            "sid = m.set_input_cb(ids.tolist(), None, 64); torch.save(m.forward_cb(), %r)")
    torch.save(ids, str(tmp_path / "ids.pt"))
    r = subprocess.run([sys.executable, "-c", code % (root, d, str(tmp_path / "ids.pt"), str(tmp_path / "cpu.pt"))],
                       env=dict(os.environ, XFT_ENGINE="CPU"), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    want = torch.load(str(tmp_path / "cpu.pt"))
    rel = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-6)
    assert rel < 0.08, rel


@pytest.mark.parametrize("T,E,k,I,H", [(5, 8, 2, 256, 512), (70, 8, 4, 128, 256), (300, 16, 2, 256, 512)])
def test_moe_experts_fp8_grouped(T, E, k, I, H):
    """fp8 block-scaled experts run through the grouped fp8 GEMM (weights stay e4m3 on the device)."""
    from xfastertransformer_b200.ops import native as Nat
    from xfastertransformer_b200.ops import native_moe
    g = torch.Generator().manual_seed(T + E + 1)
    x = (torch.randn(T, H, generator=g) * 0.5).bfloat16()
    experts = []
    for _ in range(E):
        gu = make_linear(torch.randn(2 * I, H, generator=g) * 0.05, "fp8")
        dn = make_linear(torch.randn(H, I, generator=g) * 0.05, "fp8")
        experts.append((gu, dn))
    logits = torch.randn(T, E, generator=g)
    idx, w = R.route_mixtral(logits, k)
    want = R.moe_experts(x.float(), idx, w, experts, "silu")
    cuda_experts = [(a.to("cuda"), b.to("cuda")) for a, b in experts]
    pk = native_moe.pack_experts(cuda_experts)
    assert pk.get("fp8") and pk["gu"].dtype == torch.uint8
    got = Nat.moe_experts(x.cuda(), idx.cuda().int(), w.cuda(), cuda_experts, "silu", packed=pk)
    Nat.Workspace.get(torch.device("cuda", 0)).check_status()
    err = (got.cpu() - want).abs().max().item()
    assert err < 3e-2 * max(1.0, want.abs().max().item()), err
    lo = 3
    want2 = R.moe_experts(x.float(), idx, w, experts[lo:], "silu", expert_offset=lo)
    got2 = Nat.moe_experts(x.cuda(), idx.cuda().int(), w.cuda(), cuda_experts[lo:], "silu", expert_offset=lo)
    assert (got2.cpu() - want2).abs().max().item() < 3e-2 * max(1.0, want2.abs().max().item())
