"""sm_100a kernels against the plain-PyTorch fp32 oracle (`ops.reference`) on small shapes."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from xfastertransformer_b200.ops import reference as R
from xfastertransformer_b200.runtime.loader import make_linear


def _dev():
    return torch.device("cuda", 0)


def _ws():
    from xfastertransformer_b200.ops import native as N
    return N.Workspace.get(_dev())


def _close(got, want, atol, rtol, what=""):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    assert bool((err <= tol).all()), f"{what}: max err {err.max().item():.4g} (tol {atol}+{rtol}*|x|), " \
                                     f"bad {(err > tol).sum().item()}/{err.numel()}"


@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (16, 256, 512), (7, 1000, 328), (33, 384, 1024), (64, 4096, 4096),
                                   (100, 512, 256), (130, 640, 512), (300, 1280, 768), (1024, 2048, 1024)])
def test_gemm_bf16(T, N, K):
    from xfastertransformer_b200.ops import native as N_
    g = torch.Generator(device="cpu").manual_seed(T * 131 + N)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    want = x.float() @ w.float().t()
    got = N_.gemm_bf16(x.cuda(), w.cuda(), N)
    _ws().check_status()
    _close(got, want, 2e-2, 2e-2, f"gemm {T}x{N}x{K}")


@pytest.mark.parametrize("T,N,K", [(4096, 2560, 512), (2500, 3968, 256)])
def test_gemm_pair_mode(T, N, K):
    """Compute-bound shapes take the paired-tile path (two 128-feature tiles per CTA); N = 3968 leaves the last
    pair half empty."""
    from xfastertransformer_b200.ops import native as N_
    g = torch.Generator().manual_seed(N)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    bias = torch.randn(N, generator=g) * 0.1
    res = torch.randn(T, N, generator=g).bfloat16()
    W = make_linear(w, "bf16")
    want = R.linear(x.float(), W, bias, "gelu", res.float(), 1.0, out_dtype=torch.float32)
    got = N_.linear(x.cuda(), W.to("cuda"), bias.cuda(), "gelu", res.cuda(), 1.0)
    _ws().check_status()
    _close(got, want, 3e-2, 2e-2, "pair mode")


@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (16, 256, 8192), (7, 1000, 328), (33, 384, 1024), (64, 4096, 4096),
                                   (16, 1408, 4096), (200, 512, 256)])
def test_gemm_with_fused_rmsnorm(T, N, K, gated):
    """RMSNorm folded into the GEMM: gain pre-multiplied into W's columns, 1/rms per token computed by the kernel
    (split-K slices add their sums of squares).  T = 200 takes the unfused route (norm kernel + GEMM)."""
    from xfastertransformer_b200.ops import native as N_
    g = torch.Generator().manual_seed(T + N + K)
    x = (torch.randn(T, K, generator=g) * 3.0).bfloat16()
    rows = 2 * N if gated else N
    w = (torch.randn(rows, K, generator=g) * 0.05).bfloat16()
    gain = 1.0 + 0.2 * torch.randn(K, generator=g)
    bias = torch.randn(rows, generator=g) * 0.1
    eps = 1e-5
    h = R.rmsnorm(x.float(), gain, eps)
    Wref = make_linear(w, "bf16")
    if gated:
        want = R.linear_gated(h, Wref, "silu", bias)
    else:
        want = R.linear(h, Wref, bias, "gelu", None, 1.0, out_dtype=torch.float32)
    Wf = make_linear((w.float() * gain[None, :]).bfloat16(), "bf16").to("cuda")
    got = N_.linear_rms(x.cuda(), Wf, eps, bias.cuda(), "silu" if gated else "gelu", gated=gated)
    _ws().check_status()
    # the folded weight is rounded to bf16 once more, so the tolerance follows the output's scale
    scale = float(want.abs().max())
    _close(got, want, 1.5e-2 * scale, 3e-2, f"rms-fused gemm {T}x{N}x{K} gated={gated}")
    rel = float((got.float().cpu() - want).norm() / want.norm())
    assert rel < 1e-2, rel


@pytest.mark.parametrize("splits", [2, 3, 8])
def test_gemm_split_k(splits):
    from xfastertransformer_b200.ops import native as N_
    T, N, K = 16, 256, 2048
    g = torch.Generator().manual_seed(splits)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    want = x.float() @ w.float().t()
    a = N_.gemm_bf16(x.cuda(), w.cuda(), N, force_splits=splits, out_dtype=torch.float32)
    b = N_.gemm_bf16(x.cuda(), w.cuda(), N, force_splits=splits, out_dtype=torch.float32)
    _ws().check_status()
    _close(a, want, 5e-3, 5e-3, f"split-k {splits}")
    assert torch.equal(a, b), "split-K reduction must be deterministic"
    assert int(_ws().counters.abs().sum().item()) == 0, "tile counters must return to zero"


@pytest.mark.parametrize("T", [3, 48, 200])
@pytest.mark.parametrize("act", ["silu", "gelu", "relu", None])
def test_gemm_epilogues(T, act):
    from xfastertransformer_b200.ops import native as N_
    N, K = 384, 512
    g = torch.Generator().manual_seed(7)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    bias = torch.randn(N, generator=g) * 0.1
    res = torch.randn(T, N, generator=g).bfloat16()
    W = make_linear(w, "bf16")
    want = R.linear(x.float(), W, bias, act, res.float(), 0.5, out_dtype=torch.float32)
    got = N_.linear(x.cuda(), W.to("cuda"), bias.cuda(), act, res.cuda(), 0.5)
    _ws().check_status()
    _close(got, want, 3e-2, 2e-2, f"epilogue act={act}")
    got32 = N_.linear(x.cuda(), W.to("cuda"), None, None, None, 1.0, torch.float32)
    assert got32.dtype == torch.float32
    _close(got32, x.float() @ w.float().t(), 5e-3, 5e-3, "fp32 out")


@pytest.mark.parametrize("T,I", [(5, 352), (64, 1408), (256, 512)])
def test_gemm_gated(T, I):
    from xfastertransformer_b200.ops import native as N_
    K = 256
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(2 * I, K, generator=g) * 0.08).bfloat16()
    W = make_linear(w, "bf16")
    want = R.linear_gated(x.float(), W, "silu")
    got = N_.linear_gated(x.cuda(), W.to("cuda"), "silu")
    _ws().check_status()
    _close(got, want, 2e-2, 2e-2, "gated")


def test_norms_and_embedding():
    from xfastertransformer_b200.ops import native as N_
    g = torch.Generator().manual_seed(3)
    for T, H in [(1, 256), (9, 4096), (33, 8192), (4, 1536)]:
        x = torch.randn(T, H, generator=g).bfloat16()
        w = 1 + 0.1 * torch.randn(H, generator=g)
        b = 0.1 * torch.randn(H, generator=g)
        _close(N_.rmsnorm(x.cuda(), w.cuda(), 1e-6), R.rmsnorm(x.float(), w, 1e-6), 2e-2, 1e-2, "rmsnorm")
        _close(N_.layernorm(x.cuda(), w.cuda(), b.cuda(), 1e-5), R.layernorm(x.float(), w, b, 1e-5), 2e-2, 1e-2, "ln")
        r = torch.randn(T, H, generator=g).bfloat16()
        y, h = N_.rmsnorm(x.cuda(), w.cuda(), 1e-6, r.cuda())
        yr, hr = R.rmsnorm(x, w, 1e-6, r)
        _close(h, hr, 2e-2, 1e-2, "add")
        _close(y, yr, 3e-2, 2e-2, "add+rmsnorm")
    table = torch.randn(1000, 512, generator=g).bfloat16()
    ids = torch.randint(0, 1000, (37,), generator=g, dtype=torch.int32)
    got = N_.embedding(ids.cuda(), table.cuda(), 2.0, torch.bfloat16)
    _close(got, R.embedding(ids, table, 2.0, torch.float32), 2e-2, 1e-2, "embedding")
    _ws().check_status()


def _mk_cache(nb, hkv, bs, D, int8, dev):
    if int8:
        kc = torch.zeros(nb, hkv, bs, D, dtype=torch.int8, device=dev)
        vc = torch.zeros_like(kc)
        ks = torch.zeros(nb, hkv, bs, dtype=torch.float32, device=dev)
        return kc, vc, ks, torch.zeros_like(ks)
    kc = torch.zeros(nb, hkv, bs, D, dtype=torch.bfloat16, device=dev)
    return kc, torch.zeros_like(kc), None, None


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("style,rot_frac", [("half", 1.0), ("interleaved", 0.5)])
def test_qkv_rope_cache(int8, style, rot_frac):
    from xfastertransformer_b200.ops import native as N_
    from xfastertransformer_b200 import ops
    T, hq, hkv, D, bs, nb = 19, 8, 2, 128, 64, 6
    rot = int(D * rot_frac)
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(T, (hq + 2 * hkv) * D, generator=g).bfloat16()
    pos = torch.randint(0, 500, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(nb * bs, generator=g)[:T].int()
    table = R.rope_table(512, rot)
    qn = 1 + 0.1 * torch.randn(D, generator=g)
    kn = 1 + 0.1 * torch.randn(D, generator=g)
    cpu = _mk_cache(nb, hkv, bs, D, int8, "cpu")
    gpu = _mk_cache(nb, hkv, bs, D, int8, "cuda")
    want = ops.qkv_rope_cache(qkv.float(), hq, hkv, D, pos, table, rot, style, *cpu, slots, None, qn, kn, 1e-6)
    got = N_.qkv_rope_cache(qkv.cuda(), hq, hkv, D, pos.cuda(), table.cuda(), rot, style, *gpu, slots.cuda(), None,
                            qn.cuda(), kn.cuda(), 1e-6)
    _ws().check_status()
    _close(got, want, 5e-2, 2e-2, "q")
    if int8:
        for c, gq, s_c, s_g in ((cpu[0], gpu[0], cpu[2], gpu[2]), (cpu[1], gpu[1], cpu[3], gpu[3])):
            _close(gq.float() * s_g[..., None], c.float() * s_c[..., None], 6e-2, 3e-2, "int8 cache")
    else:
        _close(gpu[0], cpu[0], 5e-2, 2e-2, "k cache")
        _close(gpu[1], cpu[1], 5e-2, 2e-2, "v cache")


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("D", [128, 64])
def test_qkv_rope2d_cache(int8, D):
    """ChatGLM-1: both position streams, the split and the cache append in one launch, against two fp32 rotations."""
    from xfastertransformer_b200 import ops
    T, hq, hkv, bs, nb = 23, 4, 4, 64, 5
    g = torch.Generator().manual_seed(9)
    qkv = torch.randn(T, (hq + 2 * hkv) * D, generator=g).bfloat16()
    pos = torch.randint(0, 300, (T,), generator=g, dtype=torch.int32)
    pos2 = torch.randint(0, 40, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(nb * bs, generator=g)[:T].int()
    table = R.rope_table(512, D // 2)
    cpu = _mk_cache(nb, hkv, bs, D, int8, "cpu")
    gpu = _mk_cache(nb, hkv, bs, D, int8, "cuda")
    want = ops.qkv_rope2d_cache(qkv.float(), hq, hkv, D, pos, pos2, table, *cpu, slots)
    got = ops.qkv_rope2d_cache(qkv.cuda(), hq, hkv, D, pos.cuda(), pos2.cuda(), table.cuda(), *gpu, slots.cuda())
    _ws().check_status()
    _close(got, want, 5e-2, 2e-2, "q")
    if int8:
        for c, gq, s_c, s_g in ((cpu[0], gpu[0], cpu[2], gpu[2]), (cpu[1], gpu[1], cpu[3], gpu[3])):
            _close(gq.float() * s_g[..., None], c.float() * s_c[..., None], 6e-2, 3e-2, "int8 cache")
    else:
        _close(gpu[0], cpu[0], 5e-2, 2e-2, "k cache")
        _close(gpu[1], cpu[1], 5e-2, 2e-2, "v cache")


def _fill_paged(B, kv_lens, hkv, D, bs, int8, g):
    nb_per = [(n + bs - 1) // bs for n in kv_lens]
    nb = sum(nb_per) + 2
    perm = torch.randperm(nb, generator=g).tolist()
    W = max(nb_per)
    bt = torch.zeros(B, W, dtype=torch.int32)
    k = torch.randn(nb, hkv, bs, D, generator=g)
    v = torch.randn(nb, hkv, bs, D, generator=g)
    off = 0
    for b in range(B):
        for j in range(nb_per[b]):
            bt[b, j] = perm[off]
            off += 1
    if int8:
        kq, ks = R.quantize_kv_int8(k.permute(0, 2, 1, 3).reshape(-1, hkv, D))
        vq, vs = R.quantize_kv_int8(v.permute(0, 2, 1, 3).reshape(-1, hkv, D))
        kc = kq.view(nb, bs, hkv, D).permute(0, 2, 1, 3).contiguous()
        vc = vq.view(nb, bs, hkv, D).permute(0, 2, 1, 3).contiguous()
        ks = ks.view(nb, bs, hkv).permute(0, 2, 1).contiguous()
        vs = vs.view(nb, bs, hkv).permute(0, 2, 1).contiguous()
        return kc, vc, ks, vs, bt
    return k.bfloat16(), v.bfloat16(), None, None, bt


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("D,hq,hkv", [(128, 8, 1), (128, 8, 8), (64, 4, 4), (128, 32, 8), (256, 4, 1)])
def test_attention_decode(int8, D, hq, hkv):
    from xfastertransformer_b200.ops import native as N_
    g = torch.Generator().manual_seed(D + hq)
    kv_lens = [1, 7, 64, 65, 300, 1000]
    B, bs = len(kv_lens), 64
    kc, vc, ks, vs, bt = _fill_paged(B, kv_lens, hkv, D, bs, int8, g)
    q = torch.randn(B, hq, D, generator=g).bfloat16()
    cu = list(range(B + 1))
    scale = 1 / math.sqrt(D)
    want = R.paged_attention(q.float(), kc, vc, bt, cu, kv_lens, scale, ks, vs)
    c = lambda t: None if t is None else t.cuda()
    got = N_.paged_attention(q.cuda(), c(kc), c(vc), bt.cuda(), cu, kv_lens, scale, c(ks), c(vs))
    _ws().check_status()
    _close(got, want, 2e-2, 2e-2, "decode attention")

    class M:  # force the split-KV path + merge kernel
        cu_q_dev = torch.tensor(cu, dtype=torch.int32, device="cuda")
        kv_lens_dev = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
        is_decode, max_q, max_kv = True, 1, max(kv_lens)
        meta = {"nsplit": 4}
    got = N_.paged_attention(q.cuda(), c(kc), c(vc), bt.cuda(), cu, kv_lens, scale, c(ks), c(vs), meta=M)
    _ws().check_status()
    _close(got, want, 2e-2, 2e-2, "split-KV decode attention")


@pytest.mark.parametrize("tma", [True, False])
@pytest.mark.parametrize("alibi", [False, True])
def test_attention_decode_long_context_both_kernels(tma, alibi):
    """bf16 decode through the TMA-ring kernel and through the cp.async kernel: long ragged contexts (ring wraps
    several times, last tile partial), GQA group 8, ALiBi, planned and forced split counts."""
    from xfastertransformer_b200.ops import native as N_
    from xfastertransformer_b200.utils.flags import Env
    g = torch.Generator().manual_seed(11)
    D, hq, hkv = 128, 16, 2
    kv_lens = [2060, 4097, 130, 33, 3000]
    B, bs = len(kv_lens), 64
    kc, vc, _, _, bt = _fill_paged(B, kv_lens, hkv, D, bs, False, g)
    q = torch.randn(B, hq, D, generator=g).bfloat16()
    cu = list(range(B + 1))
    scale = 1 / math.sqrt(D)
    sl = R.alibi_slopes(hq) if alibi else None
    want = R.paged_attention(q.float(), kc, vc, bt, cu, kv_lens, scale, None, None, sl)
    env = Env.get()
    old = env.attn_tma
    env.attn_tma = tma
    try:
        for ns in (None, 1, 2, 3, 7):
            class M:
                cu_q_dev = torch.tensor(cu, dtype=torch.int32, device="cuda")
                kv_lens_dev = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
                is_decode, max_q, max_kv = True, 1, max(kv_lens)
                meta = {} if ns is None else {"nsplit": ns}
            got = N_.paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cu, kv_lens, scale,
                                     slopes=None if sl is None else sl.cuda(), meta=M)
            _ws().check_status()
            _close(got, want, 4e-3, 1e-2, f"decode tma={tma} alibi={alibi} nsplit={ns}")
    finally:
        env.attn_tma = old


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("D,hq,hkv", [(128, 8, 2), (64, 4, 4), (256, 2, 1)])
def test_attention_prefill(int8, D, hq, hkv):
    from xfastertransformer_b200.ops import native as N_
    g = torch.Generator().manual_seed(D)
    q_lens = [1, 7, 33, 128, 200]
    past = [0, 64, 5, 0, 100]                   # chunked / prefix prefill: keys already in the cache
    kv_lens = [a + b for a, b in zip(q_lens, past)]
    B, bs = len(q_lens), 64
    kc, vc, ks, vs, bt = _fill_paged(B, kv_lens, hkv, D, bs, int8, g)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    q = torch.randn(cu[-1], hq, D, generator=g).bfloat16()
    scale = 1 / math.sqrt(D)
    slopes = R.alibi_slopes(hq)
    c = lambda t: None if t is None else t.cuda()
    for sl in (None, slopes):
        want = R.paged_attention(q.float(), kc, vc, bt, cu, kv_lens, scale, ks, vs, sl)
        got = N_.paged_attention(q.cuda(), c(kc), c(vc), bt.cuda(), cu, kv_lens, scale, c(ks), c(vs), c(sl))
        _ws().check_status()
        _close(got, want, 2e-2, 2e-2, f"prefill attention alibi={sl is not None}")


def test_argmax_first_max_wins():
    from xfastertransformer_b200.ops import native as N_
    x = torch.randn(5, 32000)
    x[1, 100] = x[1, 31999] = 50.0
    x[3, 0] = 99.0
    v, i = N_.argmax_rows(x.cuda())
    wv, wi = R.argmax_rows(x)
    assert torch.equal(i.cpu().long(), wi)
    assert int(i[1]) == 100
    assert torch.allclose(v.cpu(), wv)


def test_bounded_wait_reports_bad_index_without_faulting():
    """A slot outside the cache is skipped and reported through the status word; the context
    stays usable (no trap, no out-of-bounds access)."""
    from xfastertransformer_b200.ops import native as N_
    T, hq, hkv, D, bs, nb = 4, 2, 1, 64, 64, 2
    qkv = torch.randn(T, (hq + 2 * hkv) * D).bfloat16().cuda()
    kc, vc, _, _ = _mk_cache(nb, hkv, bs, D, False, "cuda")
    slots = torch.tensor([0, 1, nb * bs + 5, 2], dtype=torch.int32).cuda()
    pos = torch.arange(T, dtype=torch.int32).cuda()
    N_.qkv_rope_cache(qkv, hq, hkv, D, pos, None, 0, "half", kc, vc, None, None, slots)
    with pytest.raises(N_.KernelError):
        _ws().check_status()
    _ws().check_status()            # cleared
    assert torch.isfinite(N_.rmsnorm(qkv, torch.ones(qkv.shape[1]).cuda(), 1e-6).float()).all()


@pytest.mark.parametrize("T,N,K,gated", [(16, 1280, 8192, False), (16, 8192, 1024, False), (5, 896, 2048, True),
                                         (64, 1024, 3584, False), (33, 640, 512, True), (2, 130, 72, False),
                                         # the planner's balanced-stream mode (few tiles, > 32 MB of weights): tiles shared
                                         # by more than four CTAs, added up by all CTAs behind the grid-wide wait
                                         (16, 2560, 8192, False), (7, 1536, 8192, True), (40, 3072, 8192, False)])
def test_decode_gemm_balanced_stream(T, N, K, gated):
    """Decode-size GEMM whose weight blocks are dealt to the CTAs in equal runs: runs that end inside a tile leave
    partials, the last arriver adds them in CTA order.  Same answer twice (deterministic), counters back at zero, and
    the result equals the tile-per-CTA kernel's within rounding."""
    from xfastertransformer_b200.ops import native as N_
    from xfastertransformer_b200.utils.flags import Env
    g = torch.Generator().manual_seed(T + N + K)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16().cuda()
    rows = 2 * N if gated else N
    w = (torch.randn(rows, K, generator=g) * 0.05).bfloat16().cuda()
    bias = (torch.randn(rows, generator=g) * 0.1).cuda()
    res = None if gated else torch.randn(T, N, generator=g).bfloat16().cuda()
    y = x.float() @ w.float().t() + bias
    want = torch.nn.functional.silu(y[:, :N]) * y[:, N:] if gated else y + 0.5 * res.float()
    assert Env.get().gemm_streamk
    kw = dict(gated=gated, dual_off=N if gated else 0, bias=bias, act="silu" if gated else None, residual=res,
              res_scale=0.5)
    a = N_.gemm_bf16(x, w, N, **kw)
    b = N_.gemm_bf16(x, w, N, **kw)
    _ws().check_status()
    _close(a, want, 3e-2, 2e-2, f"balanced decode gemm {T}x{N}x{K}")
    assert torch.equal(a, b)
    assert int(_ws().counters.abs().sum().item()) == 0
    a32 = N_.gemm_bf16(x, w[:N], N, out_dtype=torch.float32)
    _close(a32, x.float() @ w[:N].float().t(), 5e-3, 5e-3, "fp32 out")


@pytest.mark.parametrize("style,rot_frac,fold", [("half", 1.0, True), ("interleaved", 0.5, False), ("half", 0.5, False)])
@pytest.mark.parametrize("T", [1, 16, 37])
@pytest.mark.parametrize("hq,hkv,K", [(8, 2, 1024), (16, 2, 8192)])      # cluster mode; balanced stream + grid-wide fixup
def test_qkv_product_with_rope_and_cache_append_epilogue(style, rot_frac, fold, T, hq, hkv, K):
    """QKV product + split + RoPE + paged cache append as one kernel against the three separate steps of the oracle."""
    from xfastertransformer_b200.ops import native as N_
    from xfastertransformer_b200 import ops
    D, bs, nb = 128, 64, 6
    rot = int(D * rot_frac)
    g = torch.Generator().manual_seed(T)
    x = (torch.randn(T, K, generator=g) * (3.0 if fold else 0.5)).bfloat16()
    w = (torch.randn((hq + 2 * hkv) * D, K, generator=g) * (0.05 if K <= 1024 else 0.02)).bfloat16()
    bias = torch.randn((hq + 2 * hkv) * D, generator=g) * 0.1
    pos = torch.randint(0, 500, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(nb * bs, generator=g)[:T].int()
    table = R.rope_table(512, rot)
    qs = 1.0 + torch.rand(T, generator=g)
    eps = 1e-5
    h = R.rmsnorm(x.float(), torch.ones(K), eps) if fold else x.float()
    qkv = (h @ w.float().t() + bias).bfloat16()
    cpu = _mk_cache(nb, hkv, bs, D, False, "cpu")
    gpu = _mk_cache(nb, hkv, bs, D, False, "cuda")
    want = ops.qkv_rope_cache(qkv.float(), hq, hkv, D, pos, table, rot, style, *cpu, slots, qs, None, None, eps)
    W = make_linear(w, "bf16").to("cuda")
    assert N_.can_fuse_qkv_rope(W, T, D, gpu[0], None, None, None, style)
    got = N_.qkv_linear_rope_cache(x.cuda(), W, bias.cuda(), eps if fold else None, hq, hkv, pos.cuda(), table.cuda(),
                                   rot, style, gpu[0], gpu[1], slots.cuda(), qs.cuda())
    _ws().check_status()
    scale = float(want.abs().max())
    _close(got, want, 2e-2 * scale, 3e-2, "q")
    _close(gpu[0], cpu[0], 2e-2 * scale, 3e-2, "k cache")
    _close(gpu[1], cpu[1], 2e-2 * scale, 3e-2, "v cache")
