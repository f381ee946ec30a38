"""The C++ runtime twins (libxft_b200_core.so: layout arithmetic, block tables, samplers) against the Python
implementations, through the C ABI.  No GPU needed."""
import ctypes as C
import os
import random

import pytest
import torch

from xfastertransformer_b200.ops import reference as R
from xfastertransformer_b200.parallel import partition as P
from xfastertransformer_b200.runtime.kv_cache import PagedKVCache

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "xfastertransformer_b200", "lib",
                   "libxft_b200_core.so")


@pytest.fixture(scope="module")
def core():
    if not os.path.exists(LIB):
        import importlib.util
        spec = importlib.util.spec_from_file_location("b", os.path.join(os.path.dirname(LIB), "..", "..", "csrc", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    lib = C.CDLL(LIB)
    lib.xftc_tables_new.restype = C.c_void_p
    return lib


def test_split_util_matches_python(core):
    out = (C.c_int * 4)()
    for n in (688, 11008, 28672, 4096, 32000, 14336, 130, 64):
        for splits in (1, 2, 3, 4, 8):
            for i in range(splits):
                core.xftc_task_range(n, splits, i, out)
                assert (out[0], out[1]) == P.task_range(n, splits, i), (n, splits, i)
    assert [P.task_range(11008, 8, i)[1] - P.task_range(11008, 8, i)[0] for i in range(8)] == [1408] * 4 + [1344] * 4
    assert [P.task_range(688, 2, i) for i in range(2)] == [(0, 352), (352, 688)]
    for q, kv in ((64, 8), (32, 32), (40, 40), (28, 4), (12, 2)):
        for splits in (1, 2, 3, 4, 8):
            for i in range(splits):
                core.xftc_head_range(q, kv, splits, i, out)
                (a, b), (c, d) = P.head_range(q, kv, splits, i)
                assert tuple(out) == (a, b, c, d)


def test_block_tables_match_python(core):
    rng = random.Random(0)
    t = C.c_void_p(core.xftc_tables_new(64, 40))
    py = PagedKVCache(1, 1, 8, 8, "fp16", torch.device("cpu"), 64, torch.float32)
    py.ensure_blocks(40)
    slots = (C.c_int * 512)()
    cow = (C.c_int * 2)()
    tab = (C.c_int * 64)()
    live = []
    for step in range(300):
        op = rng.choice(["add", "append", "append", "fork", "free", "truncate", "reorder"])
        if op == "add" and len(live) < 6:
            sid = step
            assert core.xftc_tables_add(t, sid) == 0
            py.add_sequence(sid)
            live.append(sid)
        elif op == "append" and live:
            sid = rng.choice(live)
            n = rng.randint(1, 90)
            if py.alloc.num_free < (n + 63) // 64 + 1:
                continue
            got = core.xftc_tables_append(t, sid, n, slots, cow)
            want = py.append_slots(sid, n)
            assert got == n and list(slots[:n]) == want
        elif op == "fork" and live and len(live) < 6:
            src, dst = rng.choice(live), 1000 + step
            assert core.xftc_tables_fork(t, src, dst) == 0
            py.tables[dst] = []
            py.lens[dst] = 0
            py.fork(src, dst)
            live.append(dst)
        elif op == "free" and live:
            sid = live.pop(rng.randrange(len(live)))
            core.xftc_tables_free(t, sid)
            py.free_sequence(sid)
        elif op == "truncate" and live:
            sid = rng.choice(live)
            new_len = rng.randint(0, py.lens[sid])
            assert core.xftc_tables_truncate(t, sid, new_len) == 0
            py.truncate(sid, new_len)
        elif op == "reorder" and len(live) >= 2:
            group = rng.sample(live, rng.randint(2, min(4, len(live))))
            src = [rng.randrange(len(group)) for _ in group]              # beam i continues from beam src[i]
            assert core.xftc_tables_reorder(t, (C.c_int * len(group))(*group), (C.c_int * len(group))(*src), len(group)) == 0
            py.reorder(group, src)
        assert core.xftc_tables_num_free(t) == py.alloc.num_free
        refs = {}
        for sid in live:
            n = core.xftc_tables_table(t, sid, tab, 64)
            assert list(tab[:n]) == py.tables[sid] and core.xftc_tables_len(t, sid) == py.lens[sid]
            assert len(py.tables[sid]) == (py.lens[sid] + 63) // 64            # no block beyond the length
            for b in py.tables[sid]:
                refs[b] = refs.get(b, 0) + 1
        # reference counts equal the number of tables that hold the block; every other block is free
        assert all(core.xftc_tables_refs(t, b) == n for b, n in refs.items())
        assert len(refs) + py.alloc.num_free == 40
    core.xftc_tables_delete(t)


def test_samplers_match_reference(core):
    g = torch.Generator().manual_seed(0)
    for _ in range(20):
        l = torch.randn(500, generator=g) * 3
        arr = (C.c_float * 500)(*l.tolist())
        assert core.xftc_argmax(arr, 500) == int(l.argmax())
        u = float(torch.rand(1, generator=g))
        want = int(R.sample_top_k_top_p(l[None], 40, 0.9, 0.8, torch.tensor([u]))[0])
        got = core.xftc_sample(arr, 500, 40, C.c_float(0.9), C.c_float(0.8), C.c_float(u))
        assert got == want
    l = torch.tensor([2.0, -2.0, 1.0, 0.5])
    arr = (C.c_float * 4)(*l.tolist())
    toks = (C.c_int * 4)(0, 1, 1, 9)
    core.xftc_repetition_penalty(arr, 4, toks, 4, C.c_float(2.0), 0)
    assert list(arr) == [1.0, -4.0, 1.0, 0.5]


def test_split_k_planner_choices():
    """The GEMM's split-K planner is host arithmetic: its choices for the 70B decode shapes must land on
    single-wave grids (tiles x splits <= 296 resident CTAs) and leave full grids unsplit."""
    import ctypes
    import os
    import xfastertransformer_b200 as pkg
    path = os.path.join(os.path.dirname(pkg.__file__), "lib", "libxft_b200_kernels.so")
    if not os.path.exists(path):
        pytest.skip("kernel library not built")
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:
        pytest.skip(f"kernel library does not load here: {e}")
    lib.xft_plan_splits.argtypes = [ctypes.c_int] * 4 + [ctypes.c_size_t, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                                         ctypes.POINTER(ctypes.c_int)]
    lib.xft_plan_splits.restype = None

    def plan(tiles, num_kb, bn=16, nacc=1):
        s, per = ctypes.c_int(), ctypes.c_int()
        lib.xft_plan_splits(tiles, num_kb, bn, nacc, 96 << 20, 1024, ctypes.byref(s), ctypes.byref(per))
        assert (s.value - 1) * per.value < num_kb <= s.value * per.value
        return s.value

    assert plan(80, 128) == 3           # qkv 10240 x 8192
    assert plan(64, 128) in (3, 4)      # o_proj
    assert plan(64, 448) == 4           # down 8192 x 28672
    assert plan(224, 128, nacc=2) == 1  # gate|up already fills the machine
    assert plan(250, 128) == 1          # lm_head
    assert plan(400, 128) == 1          # more tiles than slots: never split
    assert 8 <= plan(10, 128) <= 16     # a TP=8 slice needs many splits to reach the HBM rate
    assert plan(28, 128, bn=64, nacc=2) <= 3   # wide token tiles pay for the reduction


def test_cpp_env_flags_and_timeline(core, tmp_path, monkeypatch):
    """csrc/core/env.cc: the Env singleton reads the same variables as the Python package; TimeLine scopes honour the
    whitelist and dump a chrome trace."""
    import ctypes
    import json
    core.xftc_env_int.argtypes = [ctypes.c_char_p]
    monkeypatch.setenv("XFT_VERBOSE", "2")
    monkeypatch.setenv("XFT_PIPELINE_STAGE", "3")
    monkeypatch.setenv("XFT_TIMELINE", "1")
    monkeypatch.setenv("XFT_TIMELINE_WHITELIST", "A.scope,B.scope")
    monkeypatch.setenv("XFT_MAX_BATCH_TOKENS", "4096")
    core.xftc_env_reload()
    assert core.xftc_env_int(b"verbose") == 2
    assert core.xftc_env_int(b"pipeline_stage") == 3
    assert core.xftc_env_int(b"timeline") == 1
    assert core.xftc_env_int(b"whitelist_size") == 2
    assert core.xftc_env_int(b"max_batch_tokens") == 4096
    assert core.xftc_env_int(b"kv_block_size") == 64
    core.xftc_timeline_scope.argtypes = [ctypes.c_char_p, ctypes.c_int]
    core.xftc_timeline_scope(b"A.scope", 200)
    core.xftc_timeline_scope(b"not.listed", 10)
    core.xftc_timeline_scope(b"B.scope", 100)
    assert core.xftc_timeline_pending() == 2
    path = str(tmp_path / "trace.json").encode()
    buf = ctypes.create_string_buffer(512)
    core.xftc_timeline_dump.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]
    assert core.xftc_timeline_dump(path, buf, 512) > 0
    ev = json.load(open(path.decode()))["traceEvents"]
    assert [e["name"] for e in ev] == ["A.scope", "B.scope"] and ev[0]["dur"] >= 200 and ev[0]["ph"] == "X"
    assert core.xftc_timeline_pending() == 0
    monkeypatch.delenv("XFT_TIMELINE")
    monkeypatch.delenv("XFT_TIMELINE_WHITELIST")
    core.xftc_env_reload()
    core.xftc_timeline_scope(b"A.scope", 10)
    assert core.xftc_timeline_pending() == 0


def test_cpp_arena_reuses_blocks(core):
    """csrc/core/arena.cc over malloc/free: size classes, reuse from the free list (no backend call in steady state),
    trim."""
    import ctypes
    c = core
    c.xftc_arena_new_host.restype = ctypes.c_void_p
    c.xftc_arena_alloc.restype = ctypes.c_void_p
    c.xftc_arena_alloc.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
    c.xftc_arena_release.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    c.xftc_arena_trim.argtypes = [ctypes.c_void_p]
    c.xftc_arena_delete.argtypes = [ctypes.c_void_p]
    c.xftc_arena_stat.restype = ctypes.c_size_t
    c.xftc_arena_stat.argtypes = [ctypes.c_void_p, ctypes.c_int]
    c.xftc_arena_round.restype = ctypes.c_size_t
    c.xftc_arena_round.argtypes = [ctypes.c_size_t]
    assert c.xftc_arena_round(1) == 512 and c.xftc_arena_round(513) == 1024
    assert c.xftc_arena_round((1 << 20) + 1) == 2 << 20 and c.xftc_arena_round(3 << 20) == 4 << 20
    a = c.xftc_arena_new_host()
    p1 = c.xftc_arena_alloc(a, 1000)
    p2 = c.xftc_arena_alloc(a, 3 << 20)
    assert p1 and p2 and c.xftc_arena_stat(a, 0) == 1024 + (4 << 20) and c.xftc_arena_stat(a, 2) == 2
    c.xftc_arena_release(a, p1)
    assert c.xftc_arena_stat(a, 1) == 1024
    p3 = c.xftc_arena_alloc(a, 900)                 # same class: comes from the free list
    assert p3 == p1 and c.xftc_arena_stat(a, 2) == 2 and c.xftc_arena_stat(a, 1) == 0
    for _ in range(50):                             # a steady loop allocates nothing new
        q = c.xftc_arena_alloc(a, 2 << 20)
        c.xftc_arena_release(a, q)
    assert c.xftc_arena_stat(a, 2) == 3
    c.xftc_arena_release(a, p2)
    c.xftc_arena_release(a, p3)
    c.xftc_arena_release(a, 12345)                  # unknown pointer: ignored
    assert c.xftc_arena_stat(a, 0) == 0 and c.xftc_arena_stat(a, 1) > 0
    c.xftc_arena_trim(a)
    assert c.xftc_arena_stat(a, 1) == 0
    c.xftc_arena_delete(a)


@pytest.mark.parametrize("early,lp,eos", [(False, 1.0, 3), (True, 0.7, 3), (False, 1.3, -1)])
def test_cpp_beam_scorer_matches_python(core, early, lp, eos):
    """csrc/core/beam.cc against runtime/sampler.py on random log-probabilities: same tokens, source beams, done flag
    at every step and the same final hypotheses."""
    import ctypes
    import torch
    from xfastertransformer_b200.runtime.sampler import BeamSearchScorer
    from xfastertransformer_b200.runtime.sequence import SamplingMeta
    c = core
    c.xftc_beam_new.restype = ctypes.c_void_p
    c.xftc_beam_new.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    c.xftc_beam_process.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
    c.xftc_beam_done.argtypes = [ctypes.c_void_p]
    c.xftc_beam_delete.argtypes = [ctypes.c_void_p]
    c.xftc_beam_finalize.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
    bs, nb, V, steps, P = 3, 4, 23, 9, 5
    cfg = SamplingMeta(max_length=P + steps, num_beams=nb, num_return_sequences=2, length_penalty=lp, early_stopping=early,
                       eos_token_id=eos, pad_token_id=0)
    plens = [P, P + 7, P + 2]                                   # the length that normalises scores includes the prompt
    py = BeamSearchScorer(bs, cfg, plens)
    cc = c.xftc_beam_new(bs, nb, lp, int(early), eos, 0, 2)
    c.xftc_beam_set_prompt_lens(ctypes.c_void_p(cc), (ctypes.c_int * bs)(*plens), bs)
    g = torch.Generator().manual_seed(int(lp * 10) + eos + 5)
    for step in range(steps):
        lp_t = torch.log_softmax(torch.randn(bs * nb, V, generator=g) * 2.0, -1).contiguous()
        want_tok, want_src = py.process(lp_t.clone())
        tok = torch.zeros(bs * nb, dtype=torch.int32)
        src = torch.zeros(bs * nb, dtype=torch.int32)
        c.xftc_beam_process(cc, lp_t.data_ptr(), V, tok.data_ptr(), src.data_ptr(), bs * nb)
        live = [b for b in range(bs) if not py.done[b]]          # rows of finished requests carry padding
        for b in live:
            sl = slice(b * nb, (b + 1) * nb)
            assert tok[sl].tolist() == want_tok[sl].tolist(), (step, b)
            assert src[sl].tolist() == want_src[sl].tolist(), (step, b)
        assert bool(c.xftc_beam_done(cc)) == py.is_done, step
        if py.is_done:
            break
    prompts = torch.arange(bs * P, dtype=torch.int32).view(bs, P) + 100
    want = py.finalize(prompts.tolist(), P + steps)
    out = torch.zeros(bs * 2 * (P + steps + 2), dtype=torch.int32)
    rw = c.xftc_beam_finalize(cc, prompts.data_ptr(), bs, P, P + steps, out.data_ptr(), out.numel())
    rows, width = rw >> 16, rw & 0xFFFF
    assert rows == len(want) and width == len(want[0])
    assert out[:rows * width].view(rows, width).tolist() == want
    c.xftc_beam_delete(cc)
    # log-softmax helper
    x = torch.randn(50)
    y = x.clone()
    c.xftc_log_softmax.argtypes = [ctypes.c_void_p, ctypes.c_int]
    c.xftc_log_softmax(y.data_ptr(), 50)
    assert torch.allclose(y, torch.log_softmax(x, -1), atol=1e-5)


def test_native_selftest_under_sanitizers(tmp_path):
    """The C++ runtime's own unit-test program (csrc/tests/runtime_selftest.cc), built together with the runtime sources
    with -fsanitize=address,undefined -Wall -Wextra -Werror: every expectation holds and neither sanitizer reports."""
    import importlib.util
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("xft_build", os.path.join(root, "csrc", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    exe = mod.build_selftest()
    r = subprocess.run([exe, str(tmp_path)], capture_output=True, text=True, timeout=120,
                       env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1", UBSAN_OPTIONS="print_stacktrace=1"))
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failed" in r.stdout and "runtime error" not in r.stderr and "AddressSanitizer" not in r.stderr


def test_example_cli_flags_follow_the_reference(core):
    """examples/cpp/example.cpp takes the reference's flag names (-m -t -i -d --kv_cache_dtype -l -o --prefix_len -n -b
    --loop --topK --temperature --topP --repetPen --no_stream --do_sample); argument errors are reported before any
    device work."""
    import subprocess
    exe = os.path.join(os.path.dirname(LIB), "xft_example")
    if not os.path.exists(exe):
        pytest.skip("example not built")
    run = lambda *a: subprocess.run([exe, *a], capture_output=True, text=True, timeout=60)
    assert run().returncode == 2
    assert run("-m", "/nonexistent", "--bogus").returncode == 2
    r = run("-m", "/nonexistent", "-t", "/nonexistent/tokenizer.model", "-i", "1 2 3")
    assert r.returncode == 1 and "cannot open tokenizer model" in r.stderr
    r = run("-m", "/nonexistent", "-i", "1 2 3", "-d", "bf16", "--kv_cache_dtype", "int8", "-l", "2", "-o", "4",
            "--prefix_len", "0", "-n", "2", "-b", "2", "--loop", "1", "--topK", "4", "--temperature", "0.7", "--topP", "0.9",
            "--repetPen", "1.1", "--no_stream", "--do_sample")
    assert r.returncode == 1 and "config.ini" in r.stderr and "input_len 2 is not longer" in r.stderr
    assert run("-m", "/nonexistent", "-i", "hello").returncode == 2           # text needs -t <tokenizer.model>
    assert run("-m", "/nonexistent", "-i", "1 2 3", "--prefix_len", "3").returncode == 2
    r = run("--model=/nonexistent", "--input=1 2 3", "--output_len=4", "--num_beams", "2")    # the reference's long forms
    assert r.returncode == 1 and "config.ini" in r.stderr
    r = run("-m", "/nonexistent", "-i", "1 2 3", "-d", "int3")               # weight types: the package's dtype strings
    assert r.returncode == 2 and "unknown weight type int3" in r.stderr
    for dt in ("int8", "w8a8", "int4", "nf4", "bf16_int8", "w8a8_nf4"):
        r = run("-m", "/nonexistent", "-i", "1 2 3", "-d", dt)
        assert r.returncode == 1 and "config.ini" in r.stderr, (dt, r.stderr)
    tp = os.path.join(os.path.dirname(LIB), "xft_tp_check")
    if os.path.exists(tp):
        assert subprocess.run([tp], capture_output=True, text=True, timeout=60).returncode == 2
        assert subprocess.run([tp, "-m", "/nonexistent", "-n", "1"], capture_output=True, text=True, timeout=60).returncode == 2
        r = subprocess.run([tp, "-m", "/nonexistent", "-n", "2"], capture_output=True, text=True, timeout=60)
        assert r.returncode == 1 and "config.ini" in r.stderr
        assert subprocess.run([tp, "-m", "/nonexistent", "-n", "4", "-s", "3"], capture_output=True, text=True, timeout=60).returncode == 2
        r = subprocess.run([tp, "-m", "/nonexistent", "-n", "4", "-s", "2"], capture_output=True, text=True, timeout=60)
        assert r.returncode == 1 and "config.ini" in r.stderr


def test_rope_and_alibi_tables_match_python(core):
    """csrc/core/rope_tables.cc against ops/reference.py: plain, linear, YaRN (DeepSeek's mscale ratio and Llama-YaRN's
    table scale), Qwen's dynamic-NTK base, ALiBi slopes for power-of-two and other head counts."""
    import math
    core.xftc_qwen_ntk_theta.restype = C.c_double
    D = C.c_double
    cases = [(0, "", dict()), (1, "linear", dict(factor=4.0)),
             (2, "yarn", dict(factor=40.0, original_max_pos=4096, beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0)),
             (2, "yarn", dict(factor=16.0, original_max_pos=2048, mscale=0.707, mscale_all_dim=0.0)),
             (2, "yarn", dict(factor=8.0, original_max_pos=512, table_scale=R.yarn_mscale(8.0, 1.0)))]
    for code, name, kw in cases:
        for rot, theta in ((64, 10000.0), (128, 1e6)):
            max_pos = 600
            want = R.rope_table(max_pos, rot, theta, name, **kw)
            out = (C.c_float * (max_pos * rot))()
            core.xftc_rope_table(max_pos, rot, D(theta), code, D(kw.get("factor", 1.0)), kw.get("original_max_pos", 2048),
                                 D(kw.get("beta_fast", 32)), D(kw.get("beta_slow", 1)), D(kw.get("mscale", 1.0)),
                                 D(kw.get("mscale_all_dim", 0.0)), D(kw.get("table_scale", -1.0)), out)
            got = torch.tensor(list(out)).view(max_pos, rot)
            assert torch.allclose(got, want, atol=3e-4), (name, kw, rot, (got - want).abs().max())
    for max_kv, seq in ((4096, 8192), (8193, 8192), (40000, 8192), (3000, 2048)):
        want = 10000.0
        if max_kv > seq:
            alpha = max(2 ** math.ceil(math.log(max_kv / seq, 2) + 1) - 1, 1)
            want = 10000.0 * alpha ** (128 / 126)
        assert abs(core.xftc_qwen_ntk_theta(D(10000.0), 128, max_kv, seq) - want) < 1e-6 * want
    core.xftc_telechat_ntk_theta.restype = C.c_double
    core.xftc_telechat_mscale.restype = C.c_double
    for kv, train in ((100, 4096), (100, 8192), (9000, 8192), (70000, 8192), (5000, 2048)):
        want = 10000.0 * R.telechat_ntk_alpha(max(kv, train)) ** (128 / 126)
        assert abs(core.xftc_telechat_ntk_theta(D(10000.0), 128, kv, train) - want) < 1e-6 * want
    assert core.xftc_telechat_mscale(100, 8192) == 1.0
    assert abs(core.xftc_telechat_mscale(20000, 8192) - (0.1 * math.log(20000 / 8192) + 1)) < 1e-12
    for n in (1, 8, 12, 32, 40, 52, 64):
        out = (C.c_float * n)()
        core.xftc_alibi_slopes(n, out)
        assert torch.allclose(torch.tensor(list(out)), R.alibi_slopes(n), rtol=1e-6), n


def test_parallel_layout_twins_match_python(core):
    """Pipeline stage ranges, the MoE slice rotation, expert placement and the fused prefill kernel's visiting order:
    C++ (csrc/core/runtime.cc) against parallel/partition.py."""
    out = (C.c_int * 2)()
    for layers in (1, 7, 32, 61, 80):
        for pp in (1, 2, 3, 8):
            for r in range(pp):
                core.xftc_pp_layer_range(layers, pp, r, out)
                assert (out[0], out[1]) == P.pp_layer_range(layers, pp, r)
    for E in (8, 60, 128, 256):
        for ep in (1, 2, 3, 8):
            owners = []
            for r in range(ep):
                core.xftc_expert_range(E, ep, r, out)
                assert (out[0], out[1]) == P.expert_range(E, ep, r)
                owners += [r] * (out[1] - out[0])
            assert [core.xftc_expert_owner(e, E, ep) for e in range(E)] == owners == [P.expert_owner(e, E, ep) for e in range(E)]
    for tp in (2, 8):
        for dim in (0, 1):
            assert all(core.xftc_moe_slice_index(r, tp, l, e, dim) == P.moe_slice_index(r, tp, l, e, dim)
                       for r in range(tp) for l in (0, 3, 9) for e in (0, 5))
    buf = (C.c_int * 64)()
    for world in (2, 4, 8):
        for nb in (1, 5, 33):
            for lag in (-1, 0, 3):
                for r in range(world):
                    n = core.xftc_block_visit_order(nb, world, r, lag, buf)
                    assert list(buf[:n]) == P.block_visit_order(nb, world, r, lag)


def test_host_numeric_conversions_match_torch(core):
    """csrc/core/dtypes.h (float <-> fp16 / bf16 on the host, used while loading checkpoints) against torch's casts:
    random values over many magnitudes, subnormals, ties and overflow."""
    g = torch.Generator().manual_seed(0)
    x = torch.cat([torch.randn(4000, generator=g) * 10 ** torch.randint(-9, 6, (4000,), generator=g).float(),
                   torch.tensor([0.0, -0.0, 1.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 5.96e-8, 2.9e-8, 3.1e-8, 6.1e-5,
                                 1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11, 1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8])]).float()
    n = x.numel()
    src = (C.c_float * n)(*x.tolist())
    for kind, dt in ((1, torch.float16), (2, torch.bfloat16)):
        out = (C.c_uint16 * n)()
        core.xftc_convert_from_float(src, out, n, kind)
        want = x.to(dt).view(torch.int16).to(torch.int32) & 0xffff
        got = torch.tensor(list(out), dtype=torch.int32)
        assert torch.equal(got, want), (kind, x[(got != want).nonzero()[:5, 0]])
        back = (C.c_float * n)()
        core.xftc_convert_to_float(out, back, n, kind)
        ref = x.to(dt).float()
        assert torch.equal(torch.tensor(list(back)), ref)


def test_cmake_tree_configures_and_runs_the_native_tests(tmp_path):
    """CMakeLists.txt: the tree configures for sm_100a, the native unit-test targets (the runtime's unit tests, the engine
    over the stand-in device library) build and pass under ctest (the
    kernel and core libraries are built the same way; that takes minutes and is left to `cmake --build`)."""
    import shutil
    import subprocess
    if shutil.which("cmake") is None:
        pytest.skip("cmake not installed")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    b = str(tmp_path / "b")
    env = dict(os.environ, CXX="/usr/bin/g++") if os.path.exists("/usr/bin/g++") else dict(os.environ)
    r = subprocess.run(["cmake", "-S", root, "-B", b, "-DXFT_BUILD_TESTS=ON", f"-DXFT_OUT={b}/out"], capture_output=True,
                       text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    flags = open(os.path.join(b, "CMakeFiles", "xft_b200_kernels.dir", "flags.make")).read()
    assert "compute_100a" in flags and "sm_100a" in flags                  # Blackwell's architecture-specific target
    r = subprocess.run(["cmake", "--build", b, "--target", "xft_runtime_selftest", "xft_engine_hostcheck", "-j", "8"],
                       capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    r = subprocess.run(["ctest", "--output-on-failure"], cwd=b, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "100% tests passed" in r.stdout, r.stdout[-2000:]


def test_ctypes_mirrors_of_kernel_parameter_structs_have_the_c_layout():
    """Each struct that Python fills and a kernel reads by value: the ctypes mirror has the size and the field offsets
    the compiler gave the C struct (the library reports them)."""
    import xfastertransformer_b200 as pkg
    from xfastertransformer_b200.parallel import fused_comm as F
    path = os.path.join(os.path.dirname(pkg.__file__), "lib", "libxft_b200_kernels.so")
    if not os.path.exists(path):
        pytest.skip("kernel library not built")
    try:
        lib = C.CDLL(path)
    except OSError as e:
        pytest.skip(f"kernel library does not load here: {e}")
    from xfastertransformer_b200.ops import native as NAT
    for fn, mirror in (("xft_comm_params_layout", F.CommParams), ("xft_ar_params_layout", F.ArParams),
                       ("xft_bulk_ar_layout", F.BulkArParams), ("xft_ep_layout", F.EpParams),
                       ("xft_sk_qkv_layout", NAT.SkQkv)):
        out = (C.c_longlong * 32)()
        f = getattr(lib, fn)
        f.restype = C.c_int
        n = f(out, 32)
        names = [name for name, _ in mirror._fields_]
        assert n == 1 + len(names), fn
        assert out[0] == C.sizeof(mirror), fn
        assert [out[1 + i] for i in range(len(names))] == [getattr(mirror, name).offset for name in names], fn


def test_decode_gemm_work_decomposition_covers_every_unit_once():
    """The balanced decode GEMM (csrc/kernels/gemm_decode_sm100.cu) deals n_tiles x num_kb weight blocks to G CTAs as
    contiguous runs.  With the library's own arithmetic: the runs partition the units; the CTAs that share a tile are
    exactly c_lo..c_hi as the kernel computes them; a CTA leaves at most two partial tiles, and the scratch slot rule
    (2 * cta + 0 for the CTA's first tile, + 1 otherwise) gives every partial its own slot and lets the reducer find it;
    the all-reduce ownership formula cuts the output into `world` contiguous ranges that match the owners' bounds."""
    import xfastertransformer_b200 as pkg
    path = os.path.join(os.path.dirname(pkg.__file__), "lib", "libxft_b200_kernels.so")
    if not os.path.exists(path):
        pytest.skip("kernel library not built")
    try:
        lib = C.CDLL(path)
    except OSError as e:
        pytest.skip(f"kernel library does not load here: {e}")
    lib.xft_sk_cta_of.restype = C.c_int
    lib.xft_sk_first_unit.restype = C.c_longlong
    cta_of = lambda u, U, G: lib.xft_sk_cta_of(C.c_longlong(u), C.c_longlong(U), G)
    first = lambda c, U, G: lib.xft_sk_first_unit(c, C.c_longlong(U), G)
    for n_tiles, num_kb, G in ((10, 128, 148), (64, 16, 148), (28, 128, 148), (250, 128, 148), (6, 4, 12), (3, 7, 10),
                               (1, 9, 4), (80, 128, 148), (5, 2, 5), (64, 56, 148), (7, 3, 1)):
        U = n_tiles * num_kb
        assert G <= max(1, U // 2) or G == 1
        bounds = [first(c, U, G) for c in range(G + 1)]
        assert bounds[0] == 0 and bounds[-1] == U and all(b1 > b0 for b0, b1 in zip(bounds, bounds[1:]))
        for u in range(U):
            c = cta_of(u, U, G)
            assert bounds[c] <= u < bounds[c + 1]
        slots = {}
        arrivals = [0] * n_tiles
        for c in range(G):
            u, seg, partial = bounds[c], 0, 0
            while u < bounds[c + 1]:
                tile, kb0 = divmod(u, num_kb)
                kb1 = min(num_kb, kb0 + bounds[c + 1] - u)
                if not (kb0 == 0 and kb1 == num_kb):
                    partial += 1
                    slot = 2 * c + (0 if seg == 0 else 1)
                    assert slot not in slots
                    slots[slot] = tile
                    arrivals[tile] += 1
                u += kb1 - kb0
                seg += 1
            assert partial <= 2
        # the list of split tiles every CTA builds: CTA c >= 1 names the tile its first unit falls into when that unit is
        # not the tile's first and CTA c - 1 holds the tile's first unit
        named = []
        for c in range(1, G):
            b = bounds[c]
            t = b // num_kb
            if b % num_kb != 0 and cta_of(t * num_kb, U, G) == c - 1:
                named.append(t)
        assert named == [t for t in range(n_tiles) if cta_of(t * num_kb, U, G) != cta_of((t + 1) * num_kb - 1, U, G)]
        for tile in range(n_tiles):
            lo, hi = cta_of(tile * num_kb, U, G), cta_of((tile + 1) * num_kb - 1, U, G)
            if lo == hi:
                assert arrivals[tile] == 0
                continue
            assert arrivals[tile] == hi - lo + 1
            for c in range(lo, hi + 1):                  # the reducer's slot rule finds the writer's slot
                sl = 2 * c + (0 if first(c, U, G) // num_kb == tile else 1)
                assert slots.get(sl) == tile
    for E2, world in ((32768, 8), (1000, 3), (7, 8), (4096, 2), (131072, 4)):
        owner = [(i * world) // E2 for i in range(E2)]
        for r in range(world):
            r0, r1 = (r * E2 + world - 1) // world, ((r + 1) * E2 + world - 1) // world
            assert all(owner[i] == r for i in range(r0, r1))
            assert owner.count(r) == r1 - r0


@pytest.mark.parametrize("model_type,byte_fallback", [("bpe", True), ("bpe", False), ("unigram", False), ("unigram", True)])
def test_cpp_sentencepiece_reader_matches_the_library(core, tmp_path, model_type, byte_fallback):
    """csrc/core/tokenizer.cc reads a SentencePiece model file and segments text with the file's own algorithm; ids
    and the decoded text equal the sentencepiece library's on a model trained here (BPE as in Llama / Mistral, unigram as
    in ChatGLM), with and without byte fallback, including characters outside the vocabulary and repeated spaces."""
    spm = pytest.importorskip("sentencepiece")
    words = ("the quick brown fox jumps over the lazy dog while seven wizards quietly mix potions under a pale moon "
             "tensor kernels stream weights through shared memory and the decoder appends a token to every sequence "
             "Paris London Tokyo Berlin 2023 2024 3.14159 hello world foo bar baz café naïve über").split()
    rng = random.Random(0)
    corpus = tmp_path / "corpus.txt"
    corpus.write_text("\n".join(" ".join(rng.choice(words) for _ in range(rng.randint(4, 14))) for _ in range(600)))
    prefix = str(tmp_path / f"tok_{model_type}_{int(byte_fallback)}")
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=prefix, vocab_size=420 if byte_fallback else 180, model_type=model_type,
                                   byte_fallback=byte_fallback, character_coverage=0.98, normalization_rule_name="identity",
                                   remove_extra_whitespaces=(model_type == "unigram"), hard_vocab_limit=False, minloglevel=2)
    sp = spm.SentencePieceProcessor(model_file=prefix + ".model")
    core.xftc_tok_load.restype = C.c_void_p
    h = core.xftc_tok_load((prefix + ".model").encode())
    assert h
    info = lambda w: core.xftc_tok_info(C.c_void_p(h), w)
    assert info(0) == sp.get_piece_size() and info(1) == sp.bos_id() and info(2) == sp.eos_id() and info(3) == sp.unk_id()
    assert info(4) == (1 if model_type == "bpe" else 0)
    texts = ["the quick brown fox", "hello world", "seven wizards quietly mix potions", "Tokyo 2024  and   Berlin",
             "unseen zebra xylophone", "café über naïve", "日本語 text with 😀 emoji", "", "a", " leading and trailing "]
    for t in texts:
        want = sp.encode(t)
        out = (C.c_int * 512)()
        n = core.xftc_tok_encode(C.c_void_p(h), t.encode(), 0, 0, out, 512)
        got = list(out[:n])
        assert got == want, (model_type, byte_fallback, t, got, want)
        buf = C.create_string_buffer(2048)
        ids = (C.c_int * max(1, len(want)))(*want)
        core.xftc_tok_decode(C.c_void_p(h), ids, len(want), buf, 2048)
        assert buf.value.decode("utf-8", "replace") == sp.decode(want), (t, buf.value, sp.decode(want))
    out = (C.c_int * 16)()
    n = core.xftc_tok_encode(C.c_void_p(h), b"hello", 1, 1, out, 16)
    assert out[0] == sp.bos_id() and out[n - 1] == sp.eos_id()
    core.xftc_tok_free(C.c_void_p(h))
    assert not core.xftc_tok_load(str(tmp_path / "missing.model").encode())


@pytest.mark.parametrize("ranks", [1, 2, 3, 8])
def test_thread_rank_communicator_protocol(ranks, tmp_path):
    """The in-process tensor-parallel communicator of the C++ engine (csrc/core/comm.cc, thread ranks that take turns):
    built with ThreadSanitizer against host stand-ins for the CUDA calls (csrc/tests/comm_selftest.cc), 200 rounds of
    all-reduce / all-gather / broadcast / barrier per rank; a rank that leaves early fails the others."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "comm_selftest")
    cmd = ["g++", "-O1", "-g", "-std=c++17", "-fsanitize=thread", "-I", os.path.join(ROOT, "csrc", "core"), "-I",
           os.path.join(ROOT, "csrc", "api"), "-I", "/usr/local/cuda/include",
           os.path.join(ROOT, "csrc", "tests", "comm_selftest.cc"), os.path.join(ROOT, "csrc", "core", "comm.cc"), "-o", exe,
           "-ldl", "-lpthread"]
    b = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert b.returncode == 0, b.stderr[-3000:]
    r = subprocess.run([exe, str(ranks)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert f"{ranks}/{ranks} ranks ok, overlap=0" in r.stdout
    assert "rank0 failed as expected" in r.stdout
    assert "ThreadSanitizer" not in r.stderr


def test_weight_type_names_and_launcher_ranks(core, monkeypatch):
    """dataTypeFromName (csrc/api/xft/dtype.h) maps the package's dtype strings to the reference's enum values, and
    rankFromEnv reads torchrun / Open MPI / MPICH variables (the first complete pair wins, none means one rank)."""
    names = ["fp32", "bf16", "fp16", "int8", "w8a8", "int4", "nf4", "bf16_fp16", "bf16_int8", "bf16_w8a8", "bf16_int4",
             "bf16_nf4", "w8a8_int8", "w8a8_int4", "w8a8_nf4", "fp8_e4m3"]
    for i, n in enumerate(names):
        assert core.xftc_dtype_from_name(n.encode()) == i, n
    for bad in ("", "bf", "bf16_", "int8x", "BF16"):
        assert core.xftc_dtype_from_name(bad.encode()) == len(names), bad       # DataType::unknown

    def ranks():
        r, w = C.c_int(-1), C.c_int(-1)
        core.xftc_rank_from_env(C.byref(r), C.byref(w))
        return r.value, w.value
    for k in ("RANK", "WORLD_SIZE", "OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "PMI_RANK", "PMI_SIZE", "SINGLE_INSTANCE"):
        monkeypatch.delenv(k, raising=False)
    assert ranks() == (0, 1)
    monkeypatch.setenv("PMI_RANK", "3"); monkeypatch.setenv("PMI_SIZE", "4")
    assert ranks() == (3, 4)
    monkeypatch.setenv("OMPI_COMM_WORLD_RANK", "1"); monkeypatch.setenv("OMPI_COMM_WORLD_SIZE", "2")
    assert ranks() == (1, 2)
    monkeypatch.setenv("RANK", "5")                      # incomplete pair: ignored
    assert ranks() == (1, 2)
    monkeypatch.setenv("WORLD_SIZE", "8")
    assert ranks() == (5, 8)
    monkeypatch.setenv("SINGLE_INSTANCE", "1")           # a model per process, whatever launched it
    assert ranks() == (0, 1)


@pytest.mark.parametrize("uint4", [False, True])
def test_gptq_repack_matches_the_python_loader(core, uint4, tmp_path):
    """csrc/core/gptq.cc against runtime/loader.py:gptq_linear on the same files: the [out, in] codes (uint4: repacked
    along `in`), a tensor-parallel slice of them, the dequantised values and the per-row code sums."""
    from xfastertransformer_b200.runtime.loader import WeightSource, write_bin
    g = torch.Generator().manual_seed(13)
    in_f, out_f = 48, 40
    if uint4:
        q = torch.randint(0, 16, (in_f, out_f), generator=g, dtype=torch.uint8)
        disk = (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()
        (tmp_path / "w.qweight.0.bin").write_bytes(disk.numpy().tobytes())
    else:
        q = torch.randint(-128, 128, (in_f, out_f), generator=g, dtype=torch.int8)
        disk = q
        (tmp_path / "w.qweight.0.bin").write_bytes(q.numpy().tobytes())
    scale = torch.rand(out_f, generator=g) * 0.01 + 0.001
    zero = torch.randn(out_f, generator=g) * 0.01
    write_bin(str(tmp_path / "w.scales.0.bin"), scale, "fp32")
    write_bin(str(tmp_path / "w.zeros.0.bin"), zero, "fp32")
    src = WeightSource(str(tmp_path), "fp16", torch.device("cpu"))
    raw = (C.c_uint8 * disk.numel()).from_buffer_copy(disk.numpy().tobytes())
    for (i0, i1, o0, o1) in [(0, in_f, 0, out_f), (16, 48, 0, out_f), (0, in_f, 10, 30)]:
        W = src.gptq_linear("w", in_f, out_f, "uint4" if uint4 else "int8", "int4" if uint4 else "int8",
                            in_rng=(i0, i1), out_rng=(o0, o1))
        K, rows = i1 - i0, o1 - o0
        row_bytes = K // 2 if uint4 else K
        pitch = (row_bytes + 15) // 16 * 16
        out = (C.c_uint8 * (rows * pitch))()
        core.xftc_gptq_repack(raw, in_f, out_f, int(uint4), i0, i1, o0, o1, pitch, out)
        got = torch.frombuffer(bytearray(out), dtype=torch.uint8).view(rows, pitch)
        want = W.w.view(torch.uint8) if not uint4 else W.w
        assert torch.equal(got[:, :row_bytes], want.reshape(rows, row_bytes)), (uint4, i0, i1, o0, o1)
        assert int(got[:, row_bytes:].sum()) == 0
        deq = (C.c_float * (rows * K))()
        sc = (C.c_float * out_f)(*scale.tolist())
        zp = (C.c_float * out_f)(*zero.tolist())
        core.xftc_gptq_dequant(raw, in_f, out_f, int(uint4), i0, i1, o0, o1, sc, zp, deq)
        torch.testing.assert_close(torch.tensor(list(deq)).view(rows, K), R.dequant_weight(W), rtol=1e-6, atol=1e-7)
        sums = (C.c_float * rows)()
        core.xftc_gptq_row_sums(raw, in_f, out_f, int(uint4), i0, i1, o0, o1, sums)
        codes = q[i0:i1, o0:o1].t().float()
        assert list(sums) == codes.sum(1).tolist()


def test_reference_call_forms_compile():
    """Every call form of the reference's C++ Model API resolves against csrc/api/xft/models.h (a compile-only
    translation unit, csrc/tests/api_signatures.cc)."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-Wall", "-I", os.path.join(root, "csrc", "api"), "-I",
                        "/usr/local/cuda/include", os.path.join(root, "csrc", "tests", "api_signatures.cc")],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]


def test_reference_header_names(tmp_path):
    """`#include "xfastertransformer.h"` (and the other header names of the reference's include/ directory) resolve from
    csrc/api/include; its host-side bf16 value type rounds to nearest even."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "include_names")
    r = subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(root, "csrc", "api", "include"), "-I",
                        "/usr/local/cuda/include", os.path.join(root, "csrc", "tests", "include_names.cc"), "-o", exe],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    out = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0 and out.stdout.split()[:2] == ["1", "3"], out.stdout
    for name in ("abstract_decoder", "abstract_searcher", "bfloat16", "bit_cast", "dtype", "layers_attention", "layers_decoder",
                 "layers_gemm", "layers_mlp", "layers_norm", "layers_rotary_embedding", "layers_token_embedding", "models",
                 "xfastertransformer"):
        assert os.path.exists(os.path.join(root, "csrc", "api", "include", name + ".h")), name


def test_process_rank_communicator_with_a_stand_in_nccl(tmp_path):
    """The NCCL communicator of the C++ engine (csrc/core/comm.cc: library opened with dlopen, unique id handed over
    through a file, host broadcasts in pieces through a staging buffer, bf16 sums, gathers) as 1 to 4 real processes,
    against a stand-in NCCL over shared memory (csrc/tests/fake_nccl.cc) and host stand-ins for the CUDA calls; a rank
    whose rank 0 never comes gives up after XFT_DIST_TIMEOUT_S with an error, and so does a rank whose collective never
    finishes or for which NCCL reports an asynchronous error (bounded wait, communicator aborted)."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    fake = str(tmp_path / "libfake_nccl.so")
    exe = str(tmp_path / "comm_selftest")
    inc = ["-I", os.path.join(root, "csrc", "core"), "-I", os.path.join(root, "csrc", "api"), "-I", "/usr/local/cuda/include"]
    for cmd in (["g++", "-O1", "-std=c++17", "-shared", "-fPIC", os.path.join(root, "csrc", "tests", "fake_nccl.cc"), "-o", fake,
                 "-lrt", "-lpthread"],
                ["g++", "-O1", "-std=c++17"] + inc + [os.path.join(root, "csrc", "tests", "comm_selftest.cc"),
                                                     os.path.join(root, "csrc", "core", "comm.cc"), "-o", exe, "-ldl", "-lpthread"]):
        b = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        assert b.returncode == 0, b.stderr[-3000:]
    env = dict(os.environ, XFT_NCCL_LIB=fake, XFT_DIST_TIMEOUT_S="30")
    for world in (2, 4):
        idf = str(tmp_path / f"id{world}")
        procs = [subprocess.Popen([exe, "process", str(r), str(world), idf], env=env, stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True) for r in reversed(range(world))]   # rank 0 starts last
        outs = [p.communicate(timeout=120)[0] for p in procs]
        assert all(p.returncode == 0 for p in procs), outs
        assert sorted(o.strip() for o in outs) == sorted(f"rank {r} of {world} ok" for r in range(world))
        assert not os.path.exists(idf) and not os.path.exists(idf + ".ready")          # rank 0 removed the hand-over files
    lone = subprocess.run([exe, "process", "1", "2", str(tmp_path / "never")], env=dict(env, XFT_DIST_TIMEOUT_S="1"),
                          capture_output=True, text=True, timeout=60)
    assert lone.returncode == 1 and "did not arrive" in lone.stdout
    # a collective that never finishes (the stream stays busy: what a lost rank looks like): the wait gives up after
    # XFT_DIST_TIMEOUT_S, the communicator is aborted, the rank reports instead of waiting for ever ...
    for extra, words in ((dict(XFT_DIST_TIMEOUT_S="3"), "did not finish within 3 s"),
                         # ... and at once when NCCL itself reports an asynchronous error
                         (dict(XFT_DIST_TIMEOUT_S="60", XFT_FAKE_NCCL_ASYNC_ERROR="1"), "asynchronous error")):
        idf = str(tmp_path / "id_lost")
        e2 = dict(env, XFT_STUB_STREAM_BUSY="1", **extra)
        procs = [subprocess.Popen([exe, "process", str(r), "2", idf], env=e2, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                 for r in (1, 0)]
        outs = [p.communicate(timeout=60)[0] for p in procs]
        assert all(p.returncode == 1 for p in procs) and all(words in o for o in outs), outs
        for f in (idf, idf + ".ready"):
            if os.path.exists(f):
                os.remove(f)


_BPE_CORPUS = [
    "The quick brown fox jumps over the lazy dog. It's 2024, isn't it? We'll see; they've gone, I'm here, he'd say.",
    "def tokenize(text: str) -> list[int]:\n    return [ord(c) for c in text]  # 123456 items, 3.14159 pi\n\n\n",
    "Prices: $1,234.56 (approx.)   spaced    out\ttabs\there \n new lines \r\n and more... END!!! ???",
    "naïve café déjà vu — über straße; 你好世界 这是一个测试 こんにちは 안녕하세요 Привет мир",
    "email@example.com http://example.org/path?q=1&r=2 #hashtag @user 100% 50/50 a_b_c x-y-z",
    "I'M SHOUTING, YOU'RE NOT. WE'VE 12345678 numbers 007 and 42nd Street's 'quoted' words",
]


def _train_bpe(tmp_path, style):
    """A byte-level BPE tokenizer.json made with the `tokenizers` library: GPT-2 pre-tokenizer, or the regex split of
    Llama-3 / Qwen2 in front of a plain byte-level mapping."""
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    if style == "gpt2":
        tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    else:
        digits = r"\p{N}{1,3}" if style == "llama3" else r"\p{N}"
        pat = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|" + digits +
               r"| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")
        tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated"),
                                                     pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|endoftext|>", "<|im_start|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train_from_iterator(_BPE_CORPUS * 3, trainer)
    path = str(tmp_path / f"{style}.json")
    tok.save(path)
    return tok, path


@pytest.mark.parametrize("style", ["gpt2", "llama3", "qwen2"])
def test_bpe_tokenizer_matches_the_tokenizers_library(core, style, tmp_path):
    """csrc/core/bpe_tokenizer.cc (tokenizer.json reader, pre-tokenizer patterns, byte-level BPE) against the Hugging
    Face `tokenizers` library on the same file: ids of ASCII, accented, CJK / Hangul / Cyrillic text, code, numbers,
    contractions in both cases, runs of spaces / tabs / newlines, added tokens in the text; decoding round-trips."""
    tok, path = _train_bpe(tmp_path, style)
    core.xftc_bpe_load.restype = C.c_void_p
    core.xftc_bpe_pattern.restype = C.c_char_p
    core.xftc_bpe_error.restype = C.c_char_p
    h = core.xftc_bpe_load(path.encode())
    assert h, core.xftc_bpe_error()
    h = C.c_void_p(h)
    try:
        assert core.xftc_bpe_pattern(h).decode() == style
        assert core.xftc_bpe_vocab_size(h) == tok.get_vocab_size()
        assert core.xftc_bpe_special_id(h, b"<|im_start|>") == tok.token_to_id("<|im_start|>")
        texts = _BPE_CORPUS + ["", " ", "  leading and trailing  ", "a", "\n", "x\n\n  y", "tab\t\tsep", "it'S Don'T we'Re",
                               "<|im_start|>user\nhello<|endoftext|>", "12 345 6789012", "mixed123abc456", "...!!!\n\nnext"]
        for t in texts:
            want = tok.encode(t).ids
            buf = (C.c_int * 4096)()
            n = core.xftc_bpe_encode(h, t.encode(), buf, 4096)
            got = list(buf[:n])
            assert got == want, (style, t, got, want)
            out = C.create_string_buffer(8192)
            core.xftc_bpe_decode(h, (C.c_int * n)(*got), n, out, 8192)
            assert out.value.decode() == t, (style, t)
    finally:
        core.xftc_bpe_free(h)
    assert not core.xftc_bpe_load(str(tmp_path / "missing.json").encode())
    assert b"cannot open tokenizer" in core.xftc_bpe_error()
    if style == "gpt2":
        # the older pair of files (vocab.json + merges.txt) in a directory gives the same ids
        d = tmp_path / "pair"
        d.mkdir()
        tok.model.save(str(d))
        h2 = C.c_void_p(core.xftc_bpe_load(str(d).encode()))
        assert h2.value, core.xftc_bpe_error()
        for t in _BPE_CORPUS:
            buf = (C.c_int * 4096)()
            n = core.xftc_bpe_encode(h2, t.encode(), buf, 4096)
            assert list(buf[:n]) == tok.encode(t).ids
        core.xftc_bpe_free(h2)
        # the example CLI takes the file for -t: text is tokenised before the model is opened
        import subprocess
        exe = os.path.join(os.path.dirname(LIB), "xft_example")
        if os.path.exists(exe):
            r = subprocess.run([exe, "-m", "/nonexistent", "-t", path, "-i", "The quick brown fox", "--bos", "2"],
                               capture_output=True, text=True, timeout=60)
            assert r.returncode == 1 and "config.ini" in r.stderr          # got past the tokenizer, failed at the model
            (tmp_path / "bad.json").write_text("{\"model\": {\"type\": \"Unigram\"}}")
            r = subprocess.run([exe, "-m", "/nonexistent", "-t", str(tmp_path / "bad.json"), "-i", "hi"],
                               capture_output=True, text=True, timeout=60)
            assert r.returncode == 1 and "not a BPE tokenizer.json" in r.stderr
