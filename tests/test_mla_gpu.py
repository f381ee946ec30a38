"""MLA latent-cache attention kernel + absorb GEMMs against the fp32 oracle, and a tiny DeepSeek model."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from xfastertransformer_b200.ops import reference as R


@pytest.mark.parametrize("Hl", [16, 8, 40])
@pytest.mark.parametrize("mode", ["decode", "prefill"])
def test_mla_attention(Hl, mode):
    from xfastertransformer_b200.ops import native as Nat
    g = torch.Generator().manual_seed(Hl)
    nope, rope, L, vd, bs = 128, 64, 512, 128, 64
    if mode == "decode":
        q_lens, past = [1, 1, 1, 1], [0, 63, 200, 1500]
    else:
        q_lens, past = [1, 7, 70], [5, 0, 64]
    kv_lens = [a + b for a, b in zip(q_lens, past)]
    B = len(q_lens)
    nbs = [(n + bs - 1) // bs for n in kv_lens]
    nb = sum(nbs) + 1
    perm = torch.randperm(nb, generator=g).tolist()
    bt = torch.zeros(B, max(nbs), dtype=torch.int32)
    off = 0
    for b in range(B):
        for j in range(nbs[b]):
            bt[b, j] = perm[off]; off += 1
    cache = (torch.randn(nb, 1, bs, L + rope, generator=g) * 0.5).bfloat16()
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    qn = (torch.randn(T, Hl, nope, generator=g) * 0.5).bfloat16()
    qr = (torch.randn(T, Hl, rope, generator=g) * 0.5).bfloat16()
    w_uk = (torch.randn(Hl, nope, L, generator=g) * 0.06).bfloat16()
    w_uv = (torch.randn(Hl, vd, L, generator=g) * 0.06).bfloat16()
    scale = 1 / math.sqrt(nope + rope)
    want = R.mla_attention(qn.float(), qr.float(), cache, bt, cu, kv_lens, w_uk, w_uv, scale, absorbed=True)
    want2 = R.mla_attention(qn.float(), qr.float(), cache, bt, cu, kv_lens, w_uk, w_uv, scale, absorbed=False)
    assert torch.allclose(want, want2, atol=1e-3, rtol=1e-3), "absorbed and materialised forms must agree"
    got = Nat.mla_attention(qn.cuda(), qr.cuda(), cache.cuda(), bt.cuda(), cu, kv_lens, w_uk.cuda(), w_uv.cuda(), scale)
    Nat.Workspace.get(torch.device("cuda", 0)).check_status()
    err = (got.float().cpu() - want).abs().max().item()
    assert err < 4e-2 * max(1.0, want.abs().max().item()), err


@pytest.mark.parametrize("dtype", ["bf16", "fp8_e4m3"])
def test_tiny_deepseek(dtype, tmp_path):
    import os, subprocess, sys
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.config import ModelConfig, RopeConfig
    from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint
    cfg = ModelConfig(model_type="deepseek_moe", num_layer=3, hidden_size=512, head_num=8, kv_head_num=8,
                      size_per_head=128, inter_size=1024, vocab_size=1024, max_pos_seq_len=4096, q_lora_rank=256,
                      kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                      moe_intermediate_size=256, first_k_dense_replace=1, dense_experts=1, sparse_experts=16,
                      routed_scaling_factor=2.5, topk_method="noaux_tc", n_group=4, topk_group=2, num_experts_per_tok=4,
                      norm_topk_prob=True, scoring_func="sigmoid", activation_type="silu", weight_data_type=dtype,
                      start_id=0, end_id=1,
                      rope=RopeConfig(theta=10000, scaling_type="yarn", scaling_factor=40, original_max_pos=4096,
                                      beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0))
    d = str(tmp_path / "ds")
    write_synthetic_checkpoint(d, cfg, seed=0, dtype=dtype, std=0.05)
    ids = torch.randint(0, 1024, (2, 24), generator=torch.Generator().manual_seed(3))
    m = xft.AutoModel.from_pretrained(d, dtype=dtype, kv_cache_dtype="bf16")
    sid = m.set_input_cb(ids.tolist(), None, 64)
    got = m.forward_cb().cpu()
    m.free_seqs(sid)
    out = m.generate(ids, max_length=32)
    assert out.shape == (2, 32)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import sys,torch; sys.path.insert(0, %r); import xfastertransformer_b200 as xft;"
            "m = xft.AutoModel.from_pretrained(%r, dtype=%r, kv_cache_dtype='bf16'); ids = torch.load(%r);"
            "sid = m.set_input_cb(ids.tolist(), None, 64); torch.save(m.forward_cb(), %r)")
    torch.save(ids, str(tmp_path / "ids.pt"))
    r = subprocess.run([sys.executable, "-c", code % (root, d, dtype, str(tmp_path / "ids.pt"), str(tmp_path / "cpu.pt"))],
                       env=dict(os.environ, XFT_ENGINE="CPU"), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    want = torch.load(str(tmp_path / "cpu.pt"))
    rel = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-6)
    assert rel < 0.1, rel


@pytest.mark.parametrize("Hl,nope,rope,kvl,ql", [(16, 128, 64, 512, 1536), (5, 32, 16, 64, 0)])
def test_mla_prep_splits_rotates_normalises_and_appends(Hl, nope, rope, kvl, ql):
    """The one launch between the MLA projections and the MLA attention against the composed fp32 steps; q and kv are
    column views of wider projection outputs, as the decoder passes them."""
    from xfastertransformer_b200 import ops
    g = torch.Generator().manual_seed(Hl + kvl)
    T, bs, nb = 21, 64, 3
    qfull = (torch.randn(T, Hl * (nope + rope) + 8, generator=g) * 0.7).bfloat16()
    kvfull = (torch.randn(T, ql + kvl + rope, generator=g) * 0.7).bfloat16()
    pos = torch.randint(0, 400, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(nb * bs, generator=g)[:T].int()
    table = R.rope_table(512, rope)
    w = 1 + 0.1 * torch.randn(kvl, generator=g)
    c_cpu = torch.zeros(nb, 1, bs, kvl + rope, dtype=torch.bfloat16)
    c_gpu = torch.zeros_like(c_cpu).cuda()
    wn, wr = ops.mla_prep(qfull[:, : Hl * (nope + rope)].float(), kvfull[:, ql:].float(), Hl, nope, rope, kvl, pos, table,
                          w, 1e-6, c_cpu, slots)
    qg, kvg = qfull.cuda(), kvfull.cuda()
    gn, gr = ops.mla_prep(qg[:, : Hl * (nope + rope)], kvg[:, ql:], Hl, nope, rope, kvl, pos.cuda(), table.cuda(),
                          w.cuda(), 1e-6, c_gpu, slots.cuda())
    from xfastertransformer_b200.ops import native as Nat
    Nat.Workspace.get(gn.device).check_status()
    assert torch.equal(gn.cpu().float(), wn.float().bfloat16().float())
    torch.testing.assert_close(gr.cpu().float(), wr.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(c_gpu.cpu().float(), c_cpu.float(), rtol=2e-2, atol=2e-2)
