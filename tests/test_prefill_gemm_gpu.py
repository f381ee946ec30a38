"""The persistent prefill GEMM (csrc/kernels/gemm_prefill_sm100.cu): on one GPU against the fp32 product, and on 2+
GPUs with the all-reduce fused in (XFT_GEMM_PERSISTENT / XFT_PREFILL_FUSED_AR), and its token-major form, the default
for prompt-size products."""
import ctypes as C
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _call(x, w, N, bias=None, act=None, residual=None, res_scale=1.0, order=None, ctas=0):
    from xfastertransformer_b200.ops import native as N_
    T, K = x.shape
    out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    ws = N_.Workspace.get(x.device)
    lib = N_.lib()
    lib.xft_gemm_bf16_prefill.restype = C.c_int
    rc = lib.xft_gemm_bf16_prefill(N_._p(x), x.stride(0), N_._p(w), w.shape[0], w.stride(0), N_._p(out), N, T, N, K,
                                   N_._p(bias), N_._p(residual), residual.stride(0) if residual is not None else 0,
                                   C.c_float(res_scale), N_._ACT[act], N_._p(order), N_._p(ws.status), C.c_void_p(0),
                                   ctas, N_._stream())
    assert rc == 0, rc
    torch.cuda.synchronize()
    ws.check_status()
    return out


@pytest.mark.parametrize("T,N,K", [(100, 256, 128), (260, 200, 64), (130, 640, 512), (300, 1280, 768), (1024, 2048, 1024),
                                   (2500, 3968, 256), (8192, 1024, 512)])
def test_persistent_gemm_matches_fp32(T, N, K):
    g = torch.Generator().manual_seed(T + N)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    bias = (torch.randn(N, generator=g) * 0.1).cuda()
    res = torch.randn(T, N, generator=g).bfloat16().cuda()
    want = torch.nn.functional.gelu(x.float() @ w.float().t() + bias, approximate="tanh") + 0.5 * res.float()
    got = _call(x, w, N, bias, "gelu", res, 0.5)
    err = (got.float() - want).abs()
    assert bool((err <= 3e-2 + 2e-2 * want.abs()).all()), err.max().item()
    # plain product, few CTAs (every CTA walks many tiles: both accumulators and all ring phases are reused) and a
    # reversed visiting order
    bn = 256 if T > 128 else 128
    nb = (T + bn - 1) // bn
    order = torch.arange(nb - 1, -1, -1, dtype=torch.int32, device="cuda")
    got2 = _call(x, w, N, order=order, ctas=5)
    want2 = x.float() @ w.float().t()
    err2 = (got2.float() - want2).abs()
    assert bool((err2 <= 3e-2 + 2e-2 * want2.abs()).all()), err2.max().item()
    assert torch.equal(got2, _call(x, w, N))       # the schedule does not change the numbers


@pytest.mark.parametrize("T,N,K", [(130, 256, 128), (1000, 1408, 512), (4096, 3584, 1024)])
def test_persistent_gated_gemm_matches_fp32(T, N, K):
    """Gated form: silu(x Wg^T + bg) * (x Wu^T + bu) with gate rows [0, N) and up rows [N, 2N) of one weight."""
    from xfastertransformer_b200.ops import native as N_
    g = torch.Generator().manual_seed(T + N)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16().cuda()
    w = (torch.randn(2 * N, K, generator=g) * 0.05).bfloat16().cuda()
    bias = (torch.randn(2 * N, generator=g) * 0.1).cuda()
    out = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
    ws = N_.Workspace.get(x.device)
    lib = N_.lib()
    lib.xft_gemm_bf16_prefill_gated.restype = C.c_int
    rc = lib.xft_gemm_bf16_prefill_gated(N_._p(x), K, N_._p(w), 2 * N, K, N_._p(out), N, T, N, K, N, N_._p(bias),
                                         N_._ACT["silu"], N_._p(ws.status), 0, N_._stream())
    assert rc == 0, rc
    torch.cuda.synchronize()
    ws.check_status()
    y = x.float() @ w.float().t() + bias
    want = torch.nn.functional.silu(y[:, :N]) * y[:, N:]
    err = (out.float() - want).abs()
    assert bool((err <= 3e-2 + 2e-2 * want.abs()).all()), err.max().item()


def test_linear_takes_the_persistent_kernel_when_asked(monkeypatch):
    from xfastertransformer_b200.ops import native as N_
    from xfastertransformer_b200.utils.flags import Env
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(600, 512, generator=g) * 0.5).bfloat16().cuda()
    w = (torch.randn(768, 512, generator=g) * 0.05).bfloat16().cuda()
    a = N_.gemm_bf16(x, w, 768)
    monkeypatch.setenv("XFT_GEMM_PERSISTENT", "1")
    Env.get().reload()
    try:
        b = N_.gemm_bf16(x, w, 768)
    finally:
        monkeypatch.delenv("XFT_GEMM_PERSISTENT")
        Env.get().reload()
    torch.cuda.synchronize()
    assert (a.float() - b.float()).abs().max().item() < 2e-2


def test_persistent_gemm_with_wide_stores():
    """The same single-GPU cases with XFT_PREFILL_WIDE_STORES=1 (rows leave through shared memory as 256-byte runs); the
    switch is read once per process, hence the child process."""
    if os.environ.get("XFT_PREFILL_WIDE_STORES") == "1":
        pytest.skip("already the wide-store run")
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-q", "-x", "-k", "matches_fp32"],
                       env=dict(os.environ, XFT_PREFILL_WIDE_STORES="1"), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


@pytest.mark.parametrize("wide", [0, 1])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_prefill_gemm_allreduce(world, wide, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = str(tmp_path / "r.pt")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", XFT_PREFILL_WIDE_STORES=str(wide),
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29700 + 2 * world + wide), os.path.join(ROOT, "tests", "prefill_ar_worker.py"), out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    assert got["calls"] >= 12 and got["worst"] < 6e-2


@pytest.mark.parametrize("T,N,K,gated", [(130, 256, 128, False), (260, 200, 64, False), (300, 1288, 768, False),
                                         (8192, 1024, 512, False), (1000, 1408, 512, True), (4096, 3584, 1024, True),
                                         (257, 136, 72, True)])
def test_token_major_prefill_gemm_matches_fp32(T, N, K, gated):
    """Token-major persistent kernel (the default for more than 128 tokens): tokens on the MMA rows, features on its
    columns, vector epilogue; partial token blocks, feature tiles that are not full, N not a multiple of 16."""
    from xfastertransformer_b200.ops import native as N_
    g = torch.Generator().manual_seed(T + N + K)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16().cuda()
    rows = 2 * N if gated else N
    w = (torch.randn(rows, K, generator=g) * 0.05).bfloat16().cuda()
    bias = (torch.randn(rows, generator=g) * 0.1).cuda()
    res = None if gated else torch.randn(T, N, generator=g).bfloat16().cuda()
    y = x.float() @ w.float().t() + bias
    if gated:
        want = torch.nn.functional.silu(y[:, :N]) * y[:, N:]
    else:
        want = torch.nn.functional.gelu(y, approximate="tanh") + 0.5 * res.float()
    N_._ENV().gemm_prefill_tm, N_._ENV().gemm_prefill_tm_all = True, True      # every shape through the token-major kernel
    got = N_.gemm_bf16(x, w, N, gated=gated, dual_off=N if gated else 0, bias=bias, act="silu" if gated else "gelu",
                       residual=res, res_scale=0.5)
    torch.cuda.synchronize()
    N_.Workspace.get(x.device).check_status()
    err = (got.float() - want).abs()
    assert bool((err <= 3e-2 + 2e-2 * want.abs()).all()), err.max().item()
    assert torch.equal(got, N_.gemm_bf16(x, w, N, gated=gated, dual_off=N if gated else 0, bias=bias,
                                         act="silu" if gated else "gelu", residual=res, res_scale=0.5))
