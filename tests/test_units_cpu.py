"""Host-side units on CPU: layout arithmetic, paged KV bookkeeping, checkpoint files, config.ini, timeline, rotary and
ALiBi tables, batch buckets.  (The reference tests the corresponding C++ units one gtest binary each: kv_reorder_test,
alibi_embedding_test, rotary_embedding_test, timeline_test, transpose_test.)"""
import json
import math
import os

import pytest
import torch

from xfastertransformer_b200.config import ModelConfig, RopeConfig
from xfastertransformer_b200.ops import reference as R
from xfastertransformer_b200.parallel import partition as P
from xfastertransformer_b200.runtime.kv_cache import PagedKVCache
from xfastertransformer_b200.runtime.loader import read_bin, write_bin


# ------------------------------------------------------------------------------------------- partition
def test_task_range_granularity_and_coverage():
    # the reference's SplitUtil: 64-granular when it divides, else 16, else 2 (split_util.h:8-50)
    assert [P.task_range(11008, 8, r) for r in range(8)] == \
        [(0, 1408), (1408, 2816), (2816, 4224), (4224, 5632), (5632, 6976), (6976, 8320), (8320, 9664), (9664, 11008)]
    assert [P.task_range(688, 2, r) for r in range(2)] == [(0, 352), (352, 688)]
    for n in (64, 688, 1000, 4096, 11008, 28672, 13696):
        for s in (1, 2, 3, 4, 8):
            spans = [P.task_range(n, s, r) for r in range(s)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(b >= a for a, b in spans)


def test_head_range_gqa_cover_and_vocab_split():
    # 64 q heads / 8 kv heads over 8 ranks: 8 q heads and exactly their kv head each
    for r in range(8):
        (q0, q1), (k0, k1) = P.head_range(64, 8, 8, r)
        assert (q0, q1) == (8 * r, 8 * r + 8) and (k0, k1) == (r, r + 1)
    # more ranks than kv heads: several ranks share one kv head
    seen = []
    for r in range(4):
        (q0, q1), (k0, k1) = P.head_range(32, 2, 4, r)
        assert k1 - k0 == 1 and k0 == q0 // 16
        seen += list(range(q0, q1))
    assert seen == list(range(32))
    spans = [P.vocab_range(32000, 8, r) for r in range(8)]
    assert spans[0][0] == 0 and spans[-1][1] == 32000 and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def test_pp_layers_and_expert_owner():
    assert [P.pp_layer_range(80, 4, s) for s in range(4)] == [(0, 20), (20, 40), (40, 60), (60, 80)]
    owners = [P.expert_owner(e, 256, 8) for e in range(256)]
    assert owners[0] == 0 and owners[-1] == 7 and sorted(set(owners)) == list(range(8))
    for r in range(8):
        e0, e1 = P.expert_range(256, 8, r)
        assert all(owners[e] == r for e in range(e0, e1)) and e1 - e0 == 32


# ------------------------------------------------------------------------------------------- paged KV cache
def _cache(blocks=0):
    c = PagedKVCache(2, 2, 8, 8, "fp16", torch.device("cpu"), 64)
    if blocks:
        c.ensure_blocks(blocks)
    return c


def test_kv_fork_copy_on_write_and_free():
    c = _cache()
    c.reserve(4)
    c.add_sequence(1)
    slots = c.append_slots(1, 70)                       # two blocks, the second partially filled
    assert len(slots) == 70 and len(c.tables[1]) == 2
    c.k[0].view(-1, 2, 8)                               # layout sanity: [blocks, heads, 64, d]
    c.k[0][c.tables[1][1], :, 5] = 7.0                  # token 69 of the sequence
    c.fork(1, 2)
    assert c.tables[2] == c.tables[1] and all(c.alloc.ref[b] == 2 for b in c.tables[1])
    s2 = c.append_slots(2, 1)                           # writing into the shared tail block copies it first
    assert c.tables[2][0] == c.tables[1][0] and c.tables[2][1] != c.tables[1][1]
    assert float(c.k[0][c.tables[2][1], 0, 5, 0]) == 7.0          # the copy carries the history
    assert s2[0] == c.tables[2][1] * 64 + 6
    free_before = c.alloc.num_free
    c.free_sequence(2)
    assert c.alloc.num_free == free_before + 1 and c.alloc.ref[c.tables[1][0]] == 1
    c.free_sequence(1)
    assert c.alloc.num_free == c.alloc.num_blocks


def test_kv_reorder_is_a_permutation_of_tables():
    c = _cache()
    c.reserve(8)
    for s in (10, 11, 12):
        c.add_sequence(s)
        c.append_slots(s, 64 + s)
    before = {s: list(c.tables[s]) for s in (10, 11, 12)}
    lens = {s: c.lens[s] for s in (10, 11, 12)}
    c.reorder([10, 11, 12], [2, 2, 0])                  # beams 0 and 1 continue beam 2, beam 2 continues beam 0
    assert c.tables[10] == before[12] and c.tables[11] == before[12] and c.tables[12] == before[10]
    assert c.lens[10] == lens[12] and c.lens[12] == lens[10]
    assert all(c.alloc.ref[b] == 2 for b in before[12]) and all(c.alloc.ref[b] == 0 for b in before[11])
    c.truncate(10, 3)
    assert c.lens[10] == 3 and len(c.tables[10]) == 1


def test_kv_pools_grow_without_losing_contents():
    c = _cache(2)
    c.add_sequence(0)
    c.append_slots(0, 100)
    c.k[1][c.tables[0][1], 1, 3] = 5.0
    v0 = c.version
    c.reserve(50)
    assert c.version > v0 and c.alloc.num_blocks >= 52
    assert float(c.k[1][c.tables[0][1], 1, 3, 0]) == 5.0
    bt = c.block_table([0], 8)
    assert bt.shape == (1, 8) and bt[0, :2].tolist() == c.tables[0]


# ------------------------------------------------------------------------------------------- files and config
@pytest.mark.parametrize("dtype,tol", [("fp32", 0.0), ("fp16", 1e-3), ("bf16", 8e-3)])
def test_bin_round_trip_and_slices(tmp_path, dtype, tol):
    t = torch.randn(6, 10)
    f = str(tmp_path / "w.bin")
    write_bin(f, t, dtype)
    assert os.path.getsize(f) == 60 * (4 if dtype == "fp32" else 2)
    back = read_bin(f, dtype, (6, 10)).float()
    assert torch.allclose(back, t, atol=tol, rtol=tol)
    rows = read_bin(f, dtype, (6, 10), rows=(2, 5)).float()
    assert torch.allclose(rows, t[2:5], atol=tol, rtol=tol)


def test_config_ini_round_trip_with_rope_and_moe_keys(tmp_path):
    cfg = ModelConfig(model_type="deepseek_moe", head_num=16, kv_head_num=16, size_per_head=128, hidden_size=1024,
                      inter_size=2048, num_layer=4, vocab_size=1000, max_pos_seq_len=4096, weight_data_type="fp8_e4m3",
                      q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                      moe_intermediate_size=256, sparse_experts=16, num_experts_per_tok=4, n_group=4, topk_group=2,
                      first_k_dense_replace=1, routed_scaling_factor=2.5, topk_method="noaux_tc", scoring_func="sigmoid",
                      norm_topk_prob=True,
                      rope=RopeConfig(theta=10000, scaling_type="yarn", scaling_factor=40, original_max_pos=4096, mscale=1.0,
                                      mscale_all_dim=1.0))
    d = str(tmp_path / "m")
    os.makedirs(d)
    cfg.to_ini(d)
    back = ModelConfig.from_ini(d)
    for k in ("model_type", "head_num", "hidden_size", "num_layer", "kv_lora_rank", "qk_rope_head_dim", "sparse_experts",
              "num_experts_per_tok", "n_group", "topk_group", "first_k_dense_replace", "topk_method", "weight_data_type"):
        assert getattr(back, k) == getattr(cfg, k), k
    assert back.rope.scaling_type == "yarn" and back.rope.scaling_factor == 40 and back.routed_scaling_factor == 2.5
    assert back.attn_scale == pytest.approx(cfg.attn_scale)


# ------------------------------------------------------------------------------------------- tables
def test_rope_table_values_and_half_rotation():
    tab = R.rope_table(16, 8, 10000.0)
    assert tab.shape == (16, 8)
    for pos in (0, 3, 15):
        for i in range(4):
            inv = 10000.0 ** (-2.0 * i / 8)
            assert tab[pos, i].item() == pytest.approx(math.cos(pos * inv), abs=1e-5)
            assert tab[pos, 4 + i].item() == pytest.approx(math.sin(pos * inv), abs=1e-5)
    q = torch.randn(3, 2, 8)
    k = torch.randn(3, 1, 8)
    pos = torch.tensor([0, 5, 9])
    q2, k2 = R.rope_apply(q, k, pos, tab, 8, "half")
    assert torch.allclose(q2[0], q[0]) and torch.allclose(k2[0], k[0])          # position 0 is the identity
    # rotation preserves the norm of every (i, i + half) pair
    assert torch.allclose((q2 ** 2).sum(-1), (q ** 2).sum(-1), atol=1e-4)
    x, y = q[1, 0, 1].item(), q[1, 0, 5].item()
    c, s = tab[5, 1].item(), tab[5, 5].item()
    assert q2[1, 0, 1].item() == pytest.approx(x * c - y * s, abs=1e-5)
    assert q2[1, 0, 5].item() == pytest.approx(y * c + x * s, abs=1e-5)


def test_alibi_slopes_powers_of_two_and_odd_counts():
    s8 = R.alibi_slopes(8)
    assert torch.allclose(s8, torch.tensor([2.0 ** (-(i + 1)) for i in range(8)]))
    s12 = R.alibi_slopes(12)                          # 8 regular slopes + 4 interleaved from the next power of two
    assert s12.shape == (12,) and torch.allclose(s12[:8], s8)
    assert torch.allclose(s12[8:], torch.tensor([2.0 ** (-(2 * i + 1) / 2) for i in range(4)]))


# ------------------------------------------------------------------------------------------- timeline, buckets
def test_python_timeline_whitelist_and_dump(tmp_path, monkeypatch):
    from xfastertransformer_b200.utils import trace
    from xfastertransformer_b200.utils.flags import Env
    monkeypatch.setenv("XFT_TIMELINE_WHITELIST", "A,B")
    monkeypatch.chdir(tmp_path)
    Env.get().reload()
    trace.enable(True)
    try:
        with trace.TimeLine("A"):
            pass
        with trace.TimeLine("not listed"):
            pass
        with trace.TimeLine("B"):
            pass
        path = trace.dump()
    finally:
        trace.enable(False)
        monkeypatch.delenv("XFT_TIMELINE_WHITELIST")
        Env.get().reload()
    ev = json.load(open(path))
    ev = ev["traceEvents"] if isinstance(ev, dict) else ev
    assert [e["name"] for e in ev] == ["A", "B"] and all(e["ph"] == "X" for e in ev)


def test_runner_batch_buckets():
    from xfastertransformer_b200.runtime.cuda_runner import CudaRunner
    b = [CudaRunner.bucket(n) for n in range(1, 300)]
    assert all(x >= n for n, x in zip(range(1, 300), b))
    assert b == sorted(b) and len(set(b)) <= 24                 # a handful of graphs covers every batch size
    assert CudaRunner.bucket(16) == 16 and CudaRunner.bucket(17) == 24 and CudaRunner.bucket(64) == 64
    assert max(x / n for n, x in zip(range(9, 300), b[8:])) <= 1.5     # padding waste is bounded


@pytest.mark.parametrize("mask_tok", [130001, 130000])
def test_chatglm_2d_positions_honour_both_mask_tokens(mask_tok):
    """ChatGLM-1 positions: index up to the [gMASK] / [MASK] slot, frozen there from bos on; block positions count from
    bos.  The reference only ever detects gMASK (a comparison where an assignment was meant); here both work."""
    from types import SimpleNamespace as NS
    from xfastertransformer_b200.runtime.engine import Model
    BOS = 130004
    prompt = [11, 12, mask_tok, BOS]                 # context of 3 tokens, mask at index 2, then bos
    stub = NS(ctx=NS(device=torch.device("cpu")))
    # prefill of the whole prompt
    b = NS()
    Model._chatglm_positions(stub, b, [NS(prompt=prompt, past_len=0, pending=prompt)])
    assert b.positions.tolist() == [0, 1, 2, 2] and b.positions2.tolist() == [0, 0, 0, 1] and b.prefix_lm_lens == [3]
    # two decode steps later
    b = NS()
    Model._chatglm_positions(stub, b, [NS(prompt=prompt, past_len=5, pending=[99])])
    assert b.positions.tolist() == [2] and b.positions2.tolist() == [3]
    # no mask token at all: the position freezes at the end of the context
    b = NS()
    Model._chatglm_positions(stub, b, [NS(prompt=[11, 12, 13, BOS], past_len=0, pending=[11, 12, 13, BOS])])
    assert b.positions.tolist() == [0, 1, 2, 3]


def test_runner_staging_buffer_layout_with_padding_rows():
    """The decode runner's per-step staging buffer: [ids | positions | slots | kv lengths | cu_q | block table], real rows
    first, padding rows of the bucket pointing at the runner's scratch block with a context of one token."""
    from types import SimpleNamespace
    from xfastertransformer_b200.runtime.cuda_runner import CudaRunner, _Graph
    cache = PagedKVCache(1, 1, 8, 8, "bf16", torch.device("cpu"), block_size=4)
    r = CudaRunner.__new__(CudaRunner)
    r.m = SimpleNamespace(cache=cache)
    r._scratch_block = None
    sb = r._scratch()
    seqs = []
    for sid, past in ((10, 5), (11, 9), (12, 2)):
        cache.add_sequence(sid, 16)
        cache.append_slots(sid, past)
        seqs.append(SimpleNamespace(seq_id=sid, pending=[100 + sid], past_len=past, max_len=16))
    slots = r._reserve_slots(seqs)
    B, W = 4, 8
    g = _Graph()
    g.B, g.W = B, W
    o_ids, o_pos, o_slot, o_kv, o_cu, o_bt, total = r._layout(B, W)
    g.host = torch.full((total,), -7, dtype=torch.int32)
    r._fill(g, seqs, slots)
    h = g.host
    assert h[o_ids:o_ids + B].tolist() == [110, 111, 112, 0]
    assert h[o_pos:o_pos + B].tolist() == [5, 9, 2, 0]
    assert h[o_kv:o_kv + B].tolist() == [6, 10, 3, 1]
    assert h[o_slot:o_slot + B].tolist() == slots + [sb * cache.block]
    for i, s in enumerate(seqs):
        tab = cache.tables[s.seq_id]
        assert slots[i] == tab[s.past_len // 4] * 4 + s.past_len % 4
        row = h[o_bt + i * W:o_bt + (i + 1) * W].tolist()
        assert row[:len(tab)] == tab and row[len(tab):] == [0] * (W - len(tab))
    assert h[o_bt + 3 * W:o_bt + 4 * W].tolist() == [sb] * W
    assert o_bt % 4 == 0 and sb not in sum((cache.tables[s.seq_id] for s in seqs), [])


def test_progress_bar_draws_on_request_only(monkeypatch):
    import io
    from xfastertransformer_b200.utils.progress import ProgressBar
    buf = io.StringIO()
    out = list(ProgressBar.wrap(range(4), "Loading layers", width=8, stream=buf, enabled=True))
    text = buf.getvalue()
    assert out == [0, 1, 2, 3] and "Loading layers [####....] 2/4" in text and text.rstrip().endswith("s")
    assert "[########] 4/4" in text and text.endswith("\n")
    quiet = io.StringIO()                                 # not a terminal, not forced: silent
    monkeypatch.delenv("XFT_PROGRESS", raising=False)
    assert list(ProgressBar.wrap(range(3), "x", stream=quiet)) == [0, 1, 2] and quiet.getvalue() == ""
    monkeypatch.setenv("XFT_PROGRESS", "1")
    monkeypatch.setenv("RANK", "1")                       # follower ranks never draw
    assert list(ProgressBar.wrap(range(3), "x", stream=quiet)) == [0, 1, 2] and quiet.getvalue() == ""
    monkeypatch.setenv("RANK", "0")
    list(ProgressBar.wrap(range(3), "x", stream=quiet))
    assert "3/3" in quiet.getvalue()


def _simulate_fused_prefill(num_blocks, n_tiles, world, ctas, lag):
    """Discrete simulation of the fused prefill GEMM + all-reduce schedule: every rank has `ctas` persistent CTAs that
    take work items round-robin from the rank's visiting order; a tile of a block the rank does not own completes at
    once (it only sends), a tile of an owned block completes when every other rank has completed the same tile.
    Returns the number of sweeps until everything is done, or -1 if the system stops making progress."""
    orders = [P.block_visit_order(num_blocks, world, r, lag) for r in range(world)]
    items = [[(b, nt) for b in orders[r] for nt in range(n_tiles)] for r in range(world)]
    queues = [[items[r][c::ctas] for c in range(ctas)] for r in range(world)]
    heads = [[0] * ctas for _ in range(world)]
    sent = [set() for _ in range(world)]           # (block, tile) whose partial rank r has delivered
    sweeps = 0
    while True:
        progressed, pending = False, False
        for r in range(world):
            for c in range(ctas):
                h = heads[r][c]
                if h >= len(queues[r][c]):
                    continue
                pending = True
                b, nt = queues[r][c][h]
                if P.block_owner(b, world) != r:
                    sent[r].add((b, nt))
                elif not all((b, nt) in sent[s] for s in range(world) if s != r):
                    continue                         # the owner waits for its peers' partial sums
                heads[r][c] = h + 1
                progressed = True
        sweeps += 1
        if not pending:
            return sweeps
        if not progressed:
            return -1


def test_fused_prefill_visit_order_is_a_live_permutation():
    import random
    for world in (2, 3, 4, 8):
        for nb in (1, 2, 7, 32, 33):
            for lag in (-1, 0, 1, 5):
                for r in range(world):
                    o = P.block_visit_order(nb, world, r, lag)
                    assert sorted(o) == list(range(nb))
                    eff = world if lag < 0 else lag
                    for j in range(nb):
                        if P.block_owner(j, world) == r:
                            # an owned block comes after every foreign block up to j + lag (those it may wait for)
                            later = [b for b in o[o.index(j) + 1:] if P.block_owner(b, world) != r]
                            assert all(b > j + eff for b in later), (world, nb, lag, r, j)
    rng = random.Random(0)
    for _ in range(60):
        world = rng.choice((2, 4, 8))
        nb, nt, ctas = rng.randint(1, 40), rng.randint(1, 5), rng.randint(1, 9)
        lag = rng.choice((-1, 0, 2, 8))
        assert _simulate_fused_prefill(nb, nt, world, ctas, lag) > 0, (world, nb, nt, ctas, lag)


@pytest.mark.parametrize("world,T,N", [(2, 300, 256), (4, 1000, 1000), (8, 2048, 384), (3, 130, 128)])
def test_fused_prefill_allreduce_addressing_emulated(world, T, N):
    """The addressing of the fused prefill GEMM + all-reduce, replayed on the CPU with the kernel's own formulas
    (csrc/kernels/gemm_prefill_sm100.cu): partial tiles go to slot `rank` of the owner's partial area at row
    (block / world) * BN + t, flags live at [(block / world) * n_tiles + tile][source], finished tiles are stored into
    every rank's output and flagged at [block * n_tiles + tile].  Every offset must stay inside the sizes that
    xft_prefill_ar_sizes reports, no two writers may touch the same element, and all ranks end with the same sum."""
    import ctypes as C
    from xfastertransformer_b200.ops import native as N_
    lib = C.CDLL(N_.lib_path())
    pe, nfp, nfr = C.c_longlong(), C.c_longlong(), C.c_longlong()
    lib.xft_prefill_ar_sizes(T, N, world, C.byref(pe), C.byref(nfp), C.byref(nfr))
    pe, nfp, nfr = pe.value, nfp.value, nfr.value
    BN = 256 if T > 128 else 128
    t_tiles, n_tiles = (T + BN - 1) // BN, (N + 127) // 128
    g = torch.Generator().manual_seed(world * 1000 + T)
    partial = [torch.randn(T, N, generator=g) for _ in range(world)]       # each rank's local product
    part = [torch.zeros(world * pe) for _ in range(world)]
    part_writes = [torch.zeros(world * pe, dtype=torch.int32) for _ in range(world)]
    flag_part = [torch.zeros(nfp, dtype=torch.int64) for _ in range(world)]
    flag_res = [torch.zeros(nfr, dtype=torch.int64) for _ in range(world)]
    out = [torch.full((T * N,), float("nan")) for _ in range(world)]
    epoch = 1
    orders = [P.block_visit_order(t_tiles, world, r) for r in range(world)]
    todo = [[(b, nt) for b in orders[r] for nt in range(n_tiles)] for r in range(world)]
    head = [0] * world
    while any(head[r] < len(todo[r]) for r in range(world)):
        moved = False
        for r in range(world):
            if head[r] >= len(todo[r]):
                continue
            blk, nt = todo[r][head[r]]
            owner, own_idx = blk % world, blk // world
            t0, n0 = blk * BN, nt * 128
            rows = torch.arange(t0, min(t0 + BN, T))
            cols = torch.arange(n0, min(n0 + 128, N))
            if owner != r:
                off = r * pe + ((own_idx * BN + (rows - t0))[:, None] * N + cols[None, :]).reshape(-1)
                assert int(off.max()) < (r + 1) * pe and int(off.min()) >= r * pe      # stays inside its slot
                part[owner][off] = partial[r][rows][:, cols].reshape(-1)
                part_writes[owner][off] += 1
                f = (own_idx * n_tiles + nt) * world + r
                assert f < nfp
                flag_part[owner][f] = epoch
            else:
                fl = [(own_idx * n_tiles + nt) * world + s for s in range(world) if s != r]
                if not all(int(flag_part[r][f]) == epoch for f in fl):
                    continue                                     # peers have not delivered yet: wait
                acc = torch.zeros(len(rows), len(cols))
                for s in range(world):                           # rank order
                    if s == r:
                        acc += partial[r][rows][:, cols]
                    else:
                        off = s * pe + ((own_idx * BN + (rows - t0))[:, None] * N + cols[None, :]).reshape(-1)
                        acc += part[r][off].view(len(rows), len(cols))
                dst = (rows[:, None] * N + cols[None, :]).reshape(-1)
                for s in range(world):
                    assert bool(torch.isnan(out[s][dst]).all())  # nobody wrote these before
                    out[s][dst] = acc.reshape(-1)
                    if s != r:
                        assert blk * n_tiles + nt < nfr
                        flag_res[s][blk * n_tiles + nt] = epoch
            head[r] += 1
            moved = True
        assert moved, "schedule stopped making progress"
    want = sum(partial).reshape(-1)
    for r in range(world):
        assert int(part_writes[r].max()) <= 1                  # no element of the partial area has two writers
        assert torch.allclose(out[r], want, atol=1e-5)
        for blk in range(t_tiles):
            for nt in range(n_tiles):
                assert (int(flag_res[r][blk * n_tiles + nt]) == epoch) == (blk % world != r)


@pytest.mark.parametrize("world,E,k", [(2, 8, 2), (4, 8, 2), (8, 60, 4), (3, 8, 3)])
def test_expert_exchange_addressing_emulated(world, E, k):
    """The peer-memory expert exchange (csrc/kernels/ep_comm.cu) replayed on the CPU with the kernels' formulas: a pair
    goes to slot [source][p] of the owner's receive area with {expert id, pair index}, comes back to the source's
    return area at the pair index, and the weighted sum at home equals the dense reference.  Ranks may have no tokens."""
    g = torch.Generator().manual_seed(world * 100 + E)
    H, max_tokens = 16, 6
    cap = pairs_cap = max_tokens * k
    Ts = [int(torch.randint(0, max_tokens + 1, (1,), generator=g)) for _ in range(world)]
    Ts[0] = 0                                                  # an idle rank
    Ts[-1] = max_tokens
    h = [torch.randn(T, H, generator=g) for T in Ts]
    idx = [torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]) if T else torch.zeros(0, k, dtype=torch.long)
           for T in Ts]
    w = [torch.rand(T, k, generator=g) for T in Ts]
    expert = [torch.randn(H, H, generator=g) * 0.3 for _ in range(E)]        # expert e: y = x @ M_e
    owner = [P.expert_owner(e, E, world) for e in range(E)]
    rx_tok = [torch.full((world * cap, H), float("nan")) for _ in range(world)]
    rx_meta = [torch.full((world * cap, 2), -7, dtype=torch.long) for _ in range(world)]
    rx_cnt = [[None] * world for _ in range(world)]
    ret = [torch.full((pairs_cap, H), float("nan")) for _ in range(world)]
    dest, slot = [], []
    # plan + dispatch on every home rank
    for r in range(world):
        cnt = [0] * world
        d_r, s_r = [], []
        for i in range(Ts[r] * k):
            e = int(idx[r].reshape(-1)[i])
            d = owner[e]
            p = cnt[d]
            cnt[d] += 1
            assert p < cap and i < pairs_cap
            d_r.append(d)
            s_r.append(p)
            row = r * cap + p
            assert bool(torch.isnan(rx_tok[d][row]).all())          # nobody else writes this slot
            rx_tok[d][row] = h[r][i // k]
            rx_meta[d][row, 0], rx_meta[d][row, 1] = e, i
        for d in range(world):
            rx_cnt[d][r] = cnt[d]
        dest.append(d_r)
        slot.append(s_r)
    # receive + experts + return on every expert rank
    for d in range(world):
        e0, e1 = P.expert_range(E, world, d)
        for j in range(world * cap):
            s, q = j // cap, j % cap
            if q >= rx_cnt[d][s]:
                continue
            e, pair = int(rx_meta[d][j, 0]), int(rx_meta[d][j, 1])
            assert e0 <= e < e1 and 0 <= pair < pairs_cap             # only this rank's experts arrive here
            assert bool(torch.isnan(ret[s][pair]).all())
            ret[s][pair] = rx_tok[d][j] @ expert[e]
    # combine at home
    for r in range(world):
        for t in range(Ts[r]):
            got = sum(w[r][t, j] * ret[r][t * k + j] for j in range(k))
            want = sum(w[r][t, j] * (h[r][t] @ expert[int(idx[r][t, j])]) for j in range(k))
            assert torch.allclose(got, want, atol=1e-5)


def test_expert_exchange_plan_drops_take_no_slot():
    """Plan rule of csrc/kernels/ep_comm.cu (ep_plan_kernel) replayed on the CPU for the overflow cases: a pair beyond
    the return area (index >= pairs_cap) or with a bad expert id is dropped BEFORE a receive slot is taken, so every
    slot below a destination's published count holds exactly one dispatched pair and the receiver never reads a slot
    that nothing wrote; a pair that finds its destination's receive area full is dropped too and the count is capped."""
    E, world, k, cap, pairs_cap = 8, 2, 2, 5, 9
    g = torch.Generator().manual_seed(3)
    idx = torch.randint(0, E, (14,), generator=g).tolist()
    idx[4] = E + 3                                               # a bad expert id
    s_cnt, dest, slot, status = [0] * world, [], [], 0
    for i, e in enumerate(idx):
        d = s = -1
        if 0 <= e < E and i < pairs_cap:
            d = P.expert_owner(e, E, world)
            s = s_cnt[d]
            s_cnt[d] += 1
            if s >= cap:
                status, d = 5, -1
        else:
            status = 5
        dest.append(d)
        slot.append(s)
    cnt = [min(c, cap) for c in s_cnt]
    assert status == 5 and all(d == -1 for d in dest[pairs_cap:]) and dest[4] == -1
    for d in range(world):
        filled = sorted(slot[i] for i in range(len(idx)) if dest[i] == d)
        assert filled == list(range(cnt[d]))                    # no published slot is empty, none is written twice


def test_persistent_gemm_barrier_protocol_model():
    """Model check of the persistent prefill kernel's synchronisation (csrc/kernels/gemm_prefill_sm100.cu): three
    actors (TMA producer, MMA issuer, epilogue) over a ring of `stages` shared-memory stages and two TMEM accumulators,
    with mbarrier semantics (a phase completes after `count` arrivals; waiting on parity P succeeds once the phase of
    that parity has completed, and a fresh barrier counts as having completed the phase of parity 1).  The parities are
    the kernel's: producer waits empty[s] on ((it / stages) & 1) ^ 1, the MMA issuer waits full[s] on (it / stages) & 1
    and tmem_empty[a] on ((tile >> 1) & 1) ^ 1, the epilogue waits tmem_full[a] on (tile >> 1) & 1.  Under random
    interleavings nothing deadlocks, no stage is overwritten before it was consumed and no accumulator is reused before
    it was drained."""
    import random

    class Bar:
        def __init__(self, count):
            self.count, self.pending, self.phase = count, count, 0

        def arrive(self):
            self.pending -= 1
            if self.pending == 0:
                self.pending, self.phase = self.count, self.phase ^ 1

        def done(self, parity):            # try_wait.parity
            return self.phase != parity

    for trial in range(40):
        rng = random.Random(trial)
        stages, num_kb, tiles = rng.choice((2, 3, 4, 6)), rng.randint(1, 7), rng.randint(1, 9)
        full = [Bar(1) for _ in range(stages)]
        empty = [Bar(1) for _ in range(stages)]
        tmem_full, tmem_empty = [Bar(1), Bar(1)], [Bar(4), Bar(4)]
        stage_data = [None] * stages            # (tile, kb) held by the stage, None = free
        acc = [None, None]                      # None = free, else [tile, k-blocks accumulated]
        P_ = dict(tile=0, kb=0, it=0)
        M_ = dict(tile=0, kb=0, it=0, started=False)
        E_ = dict(tile=0, warps_left=0)
        drained = []

        def producer():
            if P_["tile"] >= tiles:
                return False
            s, ph = P_["it"] % stages, (P_["it"] // stages) & 1
            if not empty[s].done(ph ^ 1):
                return False
            assert stage_data[s] is None, "stage overwritten before it was consumed"
            stage_data[s] = (P_["tile"], P_["kb"])
            full[s].arrive()                    # the TMA transaction completes
            P_["it"] += 1
            P_["kb"] += 1
            if P_["kb"] == num_kb:
                P_["kb"], P_["tile"] = 0, P_["tile"] + 1
            return True

        def mma():
            if M_["tile"] >= tiles:
                return False
            a, aph = M_["tile"] & 1, (M_["tile"] >> 1) & 1
            if not M_["started"]:
                if not tmem_empty[a].done(aph ^ 1):
                    return False
                assert acc[a] is None, "accumulator reused before it was drained"
                acc[a] = [M_["tile"], 0]
                M_["started"] = True
                return True
            s, ph = M_["it"] % stages, (M_["it"] // stages) & 1
            if not full[s].done(ph):
                return False
            assert stage_data[s] == (M_["tile"], M_["kb"]), "MMA read a stage that holds another k-block"
            acc[a][1] += 1
            stage_data[s] = None
            empty[s].arrive()                   # tcgen05.commit on the stage
            M_["it"] += 1
            M_["kb"] += 1
            if M_["kb"] == num_kb:
                tmem_full[a].arrive()           # tcgen05.commit on the accumulator
                M_["kb"], M_["tile"], M_["started"] = 0, M_["tile"] + 1, False
            return True

        def epilogue():
            if E_["tile"] >= tiles:
                return False
            a, aph = E_["tile"] & 1, (E_["tile"] >> 1) & 1
            if E_["warps_left"] == 0:
                if not tmem_full[a].done(aph):
                    return False
                assert acc[a] == [E_["tile"], num_kb], "epilogue read an incomplete or foreign accumulator"
                E_["warps_left"] = 4
                return True
            E_["warps_left"] -= 1               # one epilogue warp finished its TMEM loads and arrives
            if E_["warps_left"] == 0:
                drained.append(acc[a][0])
                acc[a] = None
            tmem_empty[a].arrive()
            if E_["warps_left"] == 0:
                E_["tile"] += 1
            return True

        actors = [producer, mma, epilogue]
        while E_["tile"] < tiles:
            order = actors[:]
            rng.shuffle(order)
            assert any(f() for f in order), f"deadlock: stages={stages} kb={num_kb} tiles={tiles} P={P_} M={M_} E={E_}"
        assert drained == list(range(tiles))


def test_expert_exchange_protocol_model_over_consecutive_layers():
    """Model check of the peer-memory expert exchange across consecutive exchanges (csrc/kernels/ep_comm.cu): ranks run
    dispatch -> receive -> experts -> return -> combine at independent speeds, with one receive area per (destination,
    source), one return area per source and {payload, epoch} words.  No buffer is double-buffered, so the check is that
    a rank never overwrites data its peer has not consumed yet and never reads data of another exchange."""
    import random
    for trial in range(30):
        rng = random.Random(trial)
        world, rounds = rng.choice((2, 3, 4)), 4
        rx = [[dict(epoch=0, consumed=True) for _ in range(world)] for _ in range(world)]       # rx[dest][src]
        rx_cnt = [[0] * world for _ in range(world)]
        ret = [[dict(epoch=0, consumed=True) for _ in range(world)] for _ in range(world)]      # ret[home][expert rank]
        ret_flag = [[0] * world for _ in range(world)]
        epoch = [0] * world                       # completed exchanges per rank
        stage = [0] * world                       # 0 dispatch, 1 receive, 2 return, 3 combine
        done_rounds = [0] * world

        def step(r):
            e = epoch[r] + 1
            if done_rounds[r] == rounds:
                return False
            if stage[r] == 0:                     # dispatch: rows, then the count words
                for d in range(world):
                    assert rx[d][r]["consumed"], f"rank {r} overwrites rows rank {d} has not read (exchange {e})"
                    rx[d][r] = dict(epoch=e, consumed=False)
                    rx_cnt[d][r] = e
                stage[r] = 1
                return True
            if stage[r] == 1:                     # receive: wait for every source's count word of this exchange
                if any(rx_cnt[r][s] != e for s in range(world)):
                    return False
                stage[r] = 2
                return True
            if stage[r] == 2:                     # experts read the receive area, outputs go back, then the flags
                for s in range(world):
                    assert rx[r][s]["epoch"] == e and not rx[r][s]["consumed"]
                    rx[r][s]["consumed"] = True
                    assert ret[s][r]["consumed"], f"rank {r} overwrites a return row rank {s} has not combined"
                    ret[s][r] = dict(epoch=e, consumed=False)
                    ret_flag[s][r] = e
                stage[r] = 3
                return True
            if any(ret_flag[r][d] != e for d in range(world)):     # combine: wait for every expert rank
                return False
            for d in range(world):
                assert ret[r][d]["epoch"] == e
                ret[r][d]["consumed"] = True
            epoch[r] += 1
            done_rounds[r] += 1
            stage[r] = 0
            return True

        while any(n < rounds for n in done_rounds):
            order = list(range(world))
            rng.shuffle(order)
            # a random subset runs in each sweep: ranks drift apart as far as the protocol lets them
            progressed = [step(r) for r in order if rng.random() < 0.6]
            if not any(progressed):
                assert any(step(r) for r in order), "deadlock"


def test_fused_prefill_protocol_model_over_consecutive_launches():
    """Model check of the fused prefill GEMM + all-reduce across consecutive launches (the decoder's chain: the output of
    one launch is the residual of the next, two output buffers alternate).  Ranks walk their tiles at independent
    speeds.  Checked: a partial slot is never overwritten before its owner has reduced it, an output buffer is never
    written while its rank still reads it as the residual of the previous launch, every read sees the data of the
    launch it belongs to, and nothing deadlocks."""
    import random
    for trial in range(25):
        rng = random.Random(100 + trial)
        world, nb, launches = rng.choice((2, 3, 4)), rng.randint(1, 7), 4
        orders = [P.block_visit_order(nb, world, r) for r in range(world)]
        part = [[[dict(epoch=0, consumed=True) for _ in range(world)] for _ in range(nb)] for _ in range(world)]
        flag_part = [[[0] * world for _ in range(nb)] for _ in range(world)]        # [owner][block][src]
        out = [[[0] * nb for _ in range(2)] for _ in range(world)]                  # [rank][buffer][block] = epoch held
        reading = [[False, False] for _ in range(world)]                            # rank still reads buffer as residual
        flag_res = [[0] * nb for _ in range(world)]
        launch = [1] * world
        pos = [0] * world                                                           # next position in the visiting order

        def step(r):
            e = launch[r]
            if e > launches:
                return False
            w, prev = e % 2, (e - 1) % 2
            if pos[r] == 0:
                reading[r][prev] = e > 1           # the launch reads the previous output as its residual
            if pos[r] < nb:
                b = orders[r][pos[r]]
                owner = b % world
                if owner != r:
                    slot = part[owner][b][r]
                    assert slot["consumed"], f"rank {r} overwrites a partial rank {owner} has not reduced (launch {e})"
                    part[owner][b][r] = dict(epoch=e, consumed=False)
                    flag_part[owner][b][r] = e
                else:
                    if any(flag_part[r][b][s] != e for s in range(world) if s != r):
                        return False
                    for s in range(world):
                        if s != r:
                            assert part[r][b][s]["epoch"] == e and not part[r][b][s]["consumed"]
                            part[r][b][s]["consumed"] = True
                    if e > 1:
                        assert out[r][prev][b] == e - 1, "residual of another launch"
                    for s in range(world):
                        assert not reading[s][w], f"rank {r} writes buffer {w} of rank {s} while {s} still reads it"
                        out[s][w][b] = e
                        if s != r:
                            flag_res[s][b] = e
                pos[r] += 1
                return True
            if any(flag_res[r][b] != e for b in range(nb) if b % world != r):      # the launch's last CTA
                return False
            assert all(out[r][w][b] == e for b in range(nb))
            reading[r][prev] = False
            launch[r] += 1
            pos[r] = 0
            return True

        while any(l <= launches for l in launch):
            order = list(range(world))
            rng.shuffle(order)
            progressed = [step(r) for r in order if rng.random() < 0.6]
            if not any(progressed):
                assert any(step(r) for r in order), f"deadlock world={world} nb={nb} launch={launch} pos={pos}"


def test_prefix_index_shares_full_blocks_and_evicts_lru():
    """Automatic prefix reuse at the block level: a chain of digests over full token blocks, one reference per remembered
    block, longest-prefix lookup that always leaves a token to run, LRU eviction of blocks nobody else holds."""
    from xfastertransformer_b200.runtime.kv_cache import PrefixIndex
    cache = PagedKVCache(1, 1, 8, 8, "bf16", torch.device("cpu"), block_size=4)
    cache.ensure_blocks(12)
    idx = PrefixIndex(cache)
    cache.prefix_index = idx
    a = list(range(100, 111))                      # 11 tokens: two full blocks + 3
    cache.add_sequence(1)
    cache.append_slots(1, len(a))
    assert idx.insert(a, cache.tables[1]) == 2 and idx.insert(a, cache.tables[1]) == 0
    full = cache.tables[1][:2]
    assert [cache.alloc.ref[b] for b in cache.tables[1]] == [2, 2, 1]
    # same first block, different second block: one hit; a prompt that IS the remembered prefix keeps a token to run
    assert idx.lookup(a[:4] + [7, 7, 7, 7, 7]) == full[:1]
    assert idx.lookup(a[:8]) == full[:1] and idx.lookup(a[:9]) == full and idx.lookup([1, 2, 3, 4, 5]) == []
    cache.add_sequence(2)
    assert cache.adopt(2, idx.lookup(a[:8] + [5, 6])) == 8 and cache.tables[2] == full
    slots = cache.append_slots(2, 2)               # continues in a fresh block, the shared ones stay untouched
    assert cache.tables[2][:2] == full and slots[0] // 4 == cache.tables[2][2] and cache.tables[2][2] not in cache.tables[1]
    cache.free_sequence(1)
    cache.free_sequence(2)
    assert [cache.alloc.ref[b] for b in full] == [1, 1] and cache.alloc.num_free == 10      # only the index holds them
    # a second chain; then pressure: the least recently used chain goes first, children before parents
    b = list(range(200, 209))
    cache.add_sequence(3)
    cache.append_slots(3, len(b))
    idx.insert(b, cache.tables[3])
    tab_b = list(cache.tables[3][:2])
    cache.free_sequence(3)
    idx.lookup(a + [0])                            # chain a is now the most recently used one
    assert cache.alloc.num_free == 8
    cache.reserve(10)                              # needs two more blocks: both come from chain b, nothing grows
    assert cache.alloc.num_blocks == 12 and cache.alloc.num_free == 10 and idx.evicted == 2
    assert idx.lookup(b + [0]) == [] and idx.lookup(a + [0]) == full
    assert all(cache.alloc.ref[x] == 0 for x in tab_b)
    cache.add_sequence(4)
    cache.adopt(4, idx.lookup(a + [0]))
    cache.reserve(12)                              # blocks held by a live sequence are never evicted: the pools grow
    assert cache.alloc.num_blocks > 12 and idx.lookup(a + [0]) == full
    cache.free_sequence(4)
    idx.clear()
    assert cache.alloc.num_free == cache.alloc.num_blocks
