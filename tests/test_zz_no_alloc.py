"""The allocation-free GEMM entry point, called through its exported C symbol.

It serves callers that cannot allocate device memory (graph capture, a host process that already owns
all GPU memory, raw-pointer C callers): its split-K scratch is a static device array inside the
library.  The result must match the regular entry point (which takes caller-provided scratch) on two
calls in a row — the second call sees the scratch exactly as the first one left it.
Collected last on purpose, so a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from xfastertransformer_b200.ops import native as N
    lib = C.CDLL(N.lib_path())
    lib.xft_gemm_bf16_noalloc.restype = C.c_int
    lib.xft_gemm_bf16_noalloc_status.restype = C.c_int
    lib.xft_gemm_bf16_noalloc_strerror.restype = C.c_char_p
    return lib


def _call(lib, x, w, y, bias, res, res_scale, act):
    T, K = x.shape
    N = w.shape[0]
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)
    return lib.xft_gemm_bf16_noalloc(p(x), x.stride(0), p(w), w.stride(0), p(y), y.stride(0),
                                     int(y.dtype == torch.float32), T, N, K, p(bias), p(res),
                                     0 if res is None else res.stride(0), C.c_float(res_scale), act, st)


@pytest.mark.parametrize("T,N,K", [(16, 1024, 4096), (3, 384, 1024)])
def test_no_alloc_matches_regular_entry_point_twice(T, N, K):
    from xfastertransformer_b200.ops import native as Nat
    lib = _lib()
    # both shapes must plan a split-K launch, otherwise the static scratch would never be touched: ask the planner
    # with the entry point's own scratch size and tile limit
    bn = 16
    tiles = (N + 127) // 128
    splits, per = C.c_int(0), C.c_int(0)
    lib.xft_plan_splits(tiles, (K + 63) // 64, bn, 1, C.c_size_t(8 << 20), 1024, C.byref(splits), C.byref(per))
    assert splits.value > 1, "shape no longer exercises the static split-K scratch"
    g = torch.Generator().manual_seed(T + N)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    bias = (torch.randn(N, generator=g) * 0.1).cuda()
    res = torch.randn(T, N, generator=g).bfloat16().cuda()
    want = Nat.gemm_bf16(x, w, N, bias=bias, act="silu", residual=res, res_scale=0.5)
    want32 = Nat.gemm_bf16(x, w, N, out_dtype=torch.float32)
    torch.cuda.synchronize()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        y = torch.zeros(T, N, dtype=torch.bfloat16, device="cuda")
        rc = _call(lib, x, w, y, bias, res, 0.5, 2)
        assert rc == 0, lib.xft_gemm_bf16_noalloc_strerror(rc)
        assert lib.xft_gemm_bf16_noalloc_status(st) == 0
        assert torch.allclose(y.float(), want.float(), atol=2e-2, rtol=2e-2), f"call {call}"
        y32 = torch.zeros(T, N, dtype=torch.float32, device="cuda")
        rc = _call(lib, x, w, y32, None, None, 1.0, 0)
        assert rc == 0, lib.xft_gemm_bf16_noalloc_strerror(rc)
        assert lib.xft_gemm_bf16_noalloc_status(st) == 0
        assert torch.allclose(y32, want32, atol=5e-3, rtol=5e-3), f"fp32 call {call}"


def test_no_alloc_rejects_sizes_beyond_its_scratch():
    lib = _lib()
    x = torch.zeros(300, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(300, 128, dtype=torch.bfloat16, device="cuda")
    rc = _call(lib, x, w, y, None, None, 1.0, 0)
    assert rc == -100
    assert b"256" in lib.xft_gemm_bf16_noalloc_strerror(rc)


def test_no_alloc_rejects_short_leading_dimensions():
    lib = _lib()
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda")
    T, K, N = 4, 64, 128
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)
    # ldo < N, then a residual with ldr < N: refused before anything is launched
    assert lib.xft_gemm_bf16_noalloc(p(x), K, p(w), K, p(y), 64, 0, T, N, K, p(None), p(None), 0, C.c_float(1.0), 0, st) == -103
    assert lib.xft_gemm_bf16_noalloc(p(x), K, p(w), K, p(y), N, 0, T, N, K, p(None), p(y), 64, C.c_float(1.0), 0, st) == -103
