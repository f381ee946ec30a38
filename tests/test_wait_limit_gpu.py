"""Failure detection on the device without a fault: a kernel that waits for a peer's word gives up after its limit,
records a code in the status word and returns, and the context stays usable.  The peer-memory all-reduce is launched
as rank 0 of 2 on ONE GPU with both receive areas in local memory, so rank 1's words never arrive (nothing sets them)
and the wait, limited to about a millisecond here, runs out."""
import ctypes as C
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_wait_runs_out_and_reports_through_the_status_word():
    from xfastertransformer_b200.ops import native as N
    from xfastertransformer_b200.parallel.fused_comm import ArParams
    dev = torch.device("cuda", 0)
    lib = N.lib()
    lib.xft_allreduce_oneshot.restype = C.c_int
    ws = N.Workspace.get(dev)
    ws.check_status()
    n, cap = 1024, 4096
    recv = [torch.zeros(2 * 2 * cap, dtype=torch.int64, device=dev) for _ in range(2)]    # [parity][source][cap] words
    counters = torch.zeros(4, dtype=torch.int32, device=dev)                              # [epoch, done]
    p = ArParams()
    p.world, p.rank = 2, 0
    p.recv[0], p.recv[1] = recv[0].data_ptr(), recv[1].data_ptr()
    p.epoch, p.done = counters.data_ptr(), counters.data_ptr() + 4
    p.cap = cap
    p.wait_cycles = 2_000_000                    # about a millisecond
    p.status = ws.status.data_ptr()
    x = torch.ones(n, dtype=torch.float32, device=dev)
    out = torch.full((n,), -1.0, dtype=torch.float32, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    rc = lib.xft_allreduce_oneshot(N._p(x), N._p(out), N._p(None), C.c_longlong(n), 0, C.byref(p), 4, 0, N._stream())
    e1.record()
    assert rc == 0
    torch.cuda.synchronize()
    assert e0.elapsed_time(e1) < 1000.0          # it returned by itself, in about the limit
    with pytest.raises(N.KernelError, match="status 4"):
        ws.check_status()
    ws.check_status()                            # the word was cleared: the next check passes
    c = counters.tolist()
    assert c[0] == 1 and c[1] == 0               # the launch still closed its epoch and reset its CTA counter
    # rank 0's own words did arrive in both receive areas
    # (epoch 1 selects parity 1: words [parity 1][source 0][i])
    assert int((recv[1][2 * cap:2 * cap + n] >> 32).min()) == 1 and int((recv[0][2 * cap:2 * cap + n] >> 32).min()) == 1
    # the context is usable: an ordinary kernel of the library and a torch op run afterwards
    w = torch.ones(64, dtype=torch.float32, device=dev)
    y = N.rmsnorm(torch.ones(4, 64, dtype=torch.bfloat16, device=dev), w, 1e-6)
    assert torch.allclose(y.float(), torch.ones(4, 64, device=dev), atol=1e-2)
    assert float((x + 1).sum()) == 2 * n
