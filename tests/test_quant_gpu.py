"""Quantised GEMM kernels (weight-only int8/uint4/nf4/fp8 dequant-GEMM, W8A8) against the fp32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from xfastertransformer_b200.ops import reference as R
from xfastertransformer_b200.runtime.loader import make_linear


def _close(got, want, atol, rtol, what):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    assert bool((err <= tol).all()), f"{what}: max err {err.max().item():.4g}, bad {(err > tol).sum().item()}/{err.numel()}"


@pytest.mark.parametrize("kind", ["int8", "int4", "nf4", "fp8", "w8a8"])
@pytest.mark.parametrize("T,N,K", [(5, 384, 512), (48, 256, 1024), (130, 640, 256), (16, 1024, 4096), (7, 200, 328)])
def test_quant_linear(kind, T, N, K):
    from xfastertransformer_b200.ops import native as Nat
    if kind == "w8a8" and K % 16:
        pytest.skip("the int8 tensor path needs K % 16 == 0")
    g = torch.Generator().manual_seed(T + N + len(kind))
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16()
    w = torch.randn(N, K, generator=g) * 0.05
    bias = torch.randn(N, generator=g) * 0.1
    res = torch.randn(T, N, generator=g).bfloat16()
    W = make_linear(w, kind)
    want = R.linear(x.float(), W, bias, "silu", res.float(), 0.5, out_dtype=torch.float32)
    got = Nat.linear(x.cuda(), W.to("cuda"), bias.cuda(), "silu", res.cuda(), 0.5)
    Nat.Workspace.get(torch.device("cuda", 0)).check_status()
    tol = 6e-2 if kind == "w8a8" else 3e-2
    _close(got, want, tol, tol, f"{kind} linear {T}x{N}x{K}")


@pytest.mark.parametrize("kind", ["int8", "int4", "nf4", "fp8", "w8a8"])
@pytest.mark.parametrize("T,I,K", [(7, 384, 512), (64, 1408, 256)])
def test_quant_gated(kind, T, I, K):
    from xfastertransformer_b200.ops import native as Nat
    g = torch.Generator().manual_seed(I + len(kind))
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16()
    w = torch.randn(2 * I, K, generator=g) * 0.08
    W = make_linear(w, kind)
    want = R.linear_gated(x.float(), W, "silu")
    got = Nat.linear_gated(x.cuda(), W.to("cuda"), "silu")
    Nat.Workspace.get(torch.device("cuda", 0)).check_status()
    tol = 6e-2 if kind == "w8a8" else 3e-2
    _close(got, want, tol, tol, f"{kind} gated")


@pytest.mark.parametrize("dtype", ["int8", "w8a8", "int4", "nf4", "bf16_int8", "w8a8_int4"])
def test_tiny_llama_quant_dtypes(dtype, tmp_path):
    """Model-level smoke over the weight dtypes (reference ci/test_case matrix): logits stay close to the bf16
    model's and decoding runs through the CUDA graph."""
    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.tools.synthetic import preset, write_synthetic_checkpoint
    d = str(tmp_path / "tiny")
    write_synthetic_checkpoint(d, preset("tiny-llama"), seed=0, dtype="bf16", std=0.05)
    ids = torch.randint(0, 32000, (2, 32), generator=torch.Generator().manual_seed(1))
    base = xft.AutoModel.from_pretrained(d, dtype="bf16")
    sid = base.set_input_cb(ids.tolist(), None, 64)
    want = base.forward_cb().cpu()
    base.free_seqs(sid)
    m = xft.AutoModel.from_pretrained(d, dtype=dtype, kv_cache_dtype="int8")
    sid = m.set_input_cb(ids.tolist(), None, 64)
    got = m.forward_cb().cpu()
    m.free_seqs(sid)
    rel = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-6)
    assert rel < (0.6 if "4" in dtype else 0.15), rel   # per-channel 4-bit noise on random weights
    out = m.generate(ids, max_length=40)
    assert out.shape == (2, 40)


@pytest.mark.parametrize("kind", ["int8", "w8a8", "int4", "nf4"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_quantize_at_load_kernel_matches_pytorch_formulation(kind, dtype):
    """The load-time quantiser (one kernel per matrix) against the PyTorch formulation of the same arithmetic: scales and
    zero points bit-equal, codes equal (a code may differ by one where the quotient sits on a rounding boundary)."""
    from xfastertransformer_b200.ops import native_quant
    g = torch.Generator().manual_seed(17)
    for rows, K in [(70, 1000), (9, 4096), (3, 34)]:
        w = (torch.randn(rows, K, generator=g) * 0.05).to(dtype)
        w[0] = 0                                            # a constant row: scale clamps, codes stay finite
        q, s, z, ws = native_quant.quantize_rows(w.cuda(), kind)
        if kind in ("int8", "w8a8"):
            wq, wsc, wz = R.quantize_int8_per_channel(w)
        elif kind == "int4":
            wq, wsc, wz = R.quantize_uint4_per_channel(w)
        else:
            wq, wsc, wz = R.quantize_nf4_per_channel(w)
        assert torch.equal(s.cpu(), wsc) and torch.equal(z.cpu(), wz), (kind, dtype, rows, K)
        if kind in ("int8", "w8a8"):
            d = (q.cpu().int() - wq.int()).abs()
        else:
            d = (R.unpack_nibbles(q.cpu()).int() - R.unpack_nibbles(wq).int()).abs()
        assert d.max().item() <= 1 and (d != 0).float().mean().item() < 1e-3, (kind, dtype, d.max().item())
        if kind == "w8a8":
            assert torch.equal(ws.cpu(), q.cpu().float().sum(1))
        else:
            assert ws is None
