"""torchrun worker (one process per GPU) for the fused prefill GEMM + all-reduce: several shapes against the fp32
product of the full operands, repeated calls (both output buffers, growing epochs), bit-identical results on all ranks."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from xfastertransformer_b200.ops import native as N
from xfastertransformer_b200.parallel.dist import DistContext
from xfastertransformer_b200.parallel.fused_comm import PeerComm
from xfastertransformer_b200.runtime.loader import make_linear

out = sys.argv[1]


def stage(msg):
    print(f"[rank {os.environ.get('RANK')}] {msg}", file=sys.stderr, flush=True)


os.environ["XFT_PREFILL_FUSED_AR"] = "1"
os.environ.setdefault("XFT_MAX_BATCH_TOKENS", "2048")
ctx = DistContext.get()
rank, world, dev = ctx.rank, ctx.world, ctx.device
peer = PeerComm(ctx, n_max=2048, wait_ms=1000.0)
stage("peer comm up")
worst = 0.0
for T, Nf, K in ((300, 256, 512), (1024, 1024, 2048), (2048, 2048, 1024), (777, 1000, 512)):
    g = torch.Generator().manual_seed(T + Nf)
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(Nf, K, generator=g) * 0.05).bfloat16()
    bias = torch.randn(Nf, generator=g) * 0.1
    resid = torch.randn(T, Nf, generator=g).bfloat16()
    ks = K // world
    xs = x[:, rank * ks:(rank + 1) * ks].contiguous().to(dev)
    W = make_linear(w[:, rank * ks:(rank + 1) * ks].contiguous().to(dev), "bf16")
    want = x.float() @ w.float().t() + bias + 0.5 * resid.float()
    assert peer.can_fuse_bulk(T, Nf, ks, "bf16")
    last = None
    for it in range(3):
        y = peer.gemm_ar_bulk(xs, W, bias.to(dev), None, resid.to(dev), 0.5)
        torch.cuda.synchronize()
        N.Workspace.get(dev).check_status()
        last = y.float().cpu()
        err = (last - want).abs().max().item()
        worst = max(worst, err)
        assert err < 6e-2, (T, Nf, K, it, err)
    gathered = [None] * world
    dist.all_gather_object(gathered, last, group=ctx.ctrl_group)
    assert all(torch.equal(gathered[0], t) for t in gathered), "ranks must hold bit-identical results"
    stage(f"{T}x{Nf}x{K} ok")
# chained calls: the output of one call is the residual of the next (the decoder's pattern)
T, Nf, K = 512, 1024, 1024
g = torch.Generator().manual_seed(5)
x = (torch.randn(T, K, generator=g) * 0.5).bfloat16()
w = (torch.randn(Nf, K, generator=g) * 0.03).bfloat16()
ks = K // world
xs = x[:, rank * ks:(rank + 1) * ks].contiguous().to(dev)
W = make_linear(w[:, rank * ks:(rank + 1) * ks].contiguous().to(dev), "bf16")
prod = x.float() @ w.float().t()
y = peer.gemm_ar_bulk(xs, W)
ref = prod.clone()
for it in range(4):
    y = peer.gemm_ar_bulk(xs, W, None, None, y, 1.0)
    ref = prod + ref.bfloat16().float()
torch.cuda.synchronize()
N.Workspace.get(dev).check_status()
err = (y.float().cpu() - ref).abs().max().item()
assert err < 0.25, err
stage("chained ok")
if rank == 0:
    torch.save({"worst": worst, "calls": peer.bulk_calls}, out)
dist.barrier(group=ctx.ctrl_group)
peer.close()
