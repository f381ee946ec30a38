"""Tiny-Llama end to end on one B200: the CUDA path (tcgen05 GEMMs, paged attention, CUDA-graph decode)
against the eager fp32 oracle."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from eager_llama import EagerLlama
from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("tiny_llama_gpu"))
    write_synthetic_checkpoint(d, preset("tiny-llama"), seed=0, dtype="bf16", std=0.05)
    return d


@pytest.mark.parametrize("kv", ["fp16", "int8"])
def test_tiny_llama_gpu(tiny, kv):
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.ops import native as N
    model = xft.AutoModel.from_pretrained(tiny, dtype="bf16", kv_cache_dtype=kv)
    assert model.model.ctx.device.type == "cuda"
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 32000, (2, 32), generator=g)
    ref = EagerLlama(tiny)
    sid = model.set_input_cb(ids.tolist(), None, 64)
    logits = model.forward_cb().cpu()
    model.free_seqs(sid)
    want = ref.logits(ids)[:, -1]
    err = (logits - want).abs().max().item()
    tol = 0.08 if kv == "fp16" else 0.15
    assert err < tol * max(1.0, want.abs().max().item()), f"prefill logits err {err}"
    # greedy decode through the CUDA-graph runner; compare against teacher-forced oracle logits:
    # every emitted token must be (near-)argmax of the oracle at that position
    out = model.generate(ids, max_length=48)
    N.Workspace.get(model.model.ctx.device).check_status()
    assert out.shape == (2, 48)
    assert torch.equal(out[:, :32], ids)
    full = ref.logits(out[:, :-1])
    for b in range(2):
        for t in range(32, 48):
            row = full[b, t - 1]
            assert row[out[b, t]] >= row.max() - tol * max(1.0, row.abs().max().item()), (b, t)
    assert model.model.runner.graph_launches > 0, "decode did not run through the CUDA graph"
    assert N.launches() > 0


def test_forward_cb_greedy_replays_the_decode_graph(tiny):
    """Continuous batching with on-device token selection: decode steps go through the CUDA-graph runner and yield
    the tokens of generate()."""
    import xfastertransformer_b200 as xft
    model = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 32000, (3, 20), generator=g)
    want = model.generate(ids, max_length=30)[:, 20:]
    runner = model.model.runner
    assert runner is not None
    g0 = runner.graph_launches
    sids = model.set_input_cb(ids.tolist(), None, 40, greedy=True)
    toks = [model.forward_cb_greedy()]
    for _ in range(9):
        model.set_input_cb([[int(t)] for t in toks[-1]], sids, None, greedy=True)
        toks.append(model.forward_cb_greedy())
    model.free_seqs(sids)
    got = torch.stack(toks, 1)
    # the eager step and the captured step plan their split-KV differently, so sums differ in the last bits and a
    # near-tie may flip: every token must be (near-)argmax of the fp32 oracle given its own history
    full_ids = torch.cat([ids, got], 1)
    oracle = EagerLlama(tiny).logits(full_ids[:, :-1])
    for b in range(full_ids.shape[0]):
        for t in range(20, full_ids.shape[1]):
            row = oracle[b, t - 1]
            assert row[full_ids[b, t]] >= row.max() - 0.1 * max(1.0, row.abs().max().item()), (b, t)
    assert (got == want).float().mean() > 0.5
    assert runner.graph_launches - g0 >= 6      # first decode step eager, second captures, the rest replay


def test_mixed_prefill_and_decode_step_on_gpu(tiny):
    """One forward carrying a new prompt and running sequences (set_input_cb hold / append) on the CUDA path: the ragged
    attention kernel serves rows of length 20 and 1 together; logits match the separate forwards."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.ops import native as N
    m = xft.AutoModel.from_pretrained(tiny, dtype="bf16")
    g = torch.Generator().manual_seed(3)
    p1 = torch.randint(5, 30000, (2, 12), generator=g).tolist()
    p2 = torch.randint(5, 30000, (1, 20), generator=g).tolist()
    s1 = m.set_input_cb(p1, None, 40)
    t1 = m.forward_cb().argmax(-1).tolist()
    m.set_input_cb([[t] for t in t1], s1, None)
    want_dec = m.forward_cb().clone()
    s2 = m.set_input_cb(p2, None, 40)
    want_pre = m.forward_cb().clone()
    m.free_seqs(torch.cat([s1, s2]))
    s1 = m.set_input_cb(p1, None, 40)
    m.forward_cb()
    s2 = m.set_input_cb(p2, None, 40, hold=True)
    m.set_input_cb([[t] for t in t1], s1, None, append=True)
    both = m.forward_cb()
    N.Workspace.get(m.model.ctx.device).check_status()
    assert both.shape[0] == 3
    scale = max(1.0, want_pre.abs().max().item())
    assert (both[:1] - want_pre).abs().max().item() < 0.05 * scale
    assert (both[1:] - want_dec).abs().max().item() < 0.05 * scale
    m.free_seqs(torch.cat([s1, s2]))
