"""torchrun worker for the multi-GPU tests (one process per GPU)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import xfastertransformer_b200 as xft
from xfastertransformer_b200.ops import native as N
from xfastertransformer_b200.parallel.dist import DistContext
from xfastertransformer_b200.parallel.fused_comm import PeerComm
from xfastertransformer_b200.runtime.loader import make_linear

path, out = sys.argv[1], sys.argv[2]


def stage(msg):
    print(f"[rank {os.environ.get('RANK')}] {msg}", file=sys.stderr, flush=True)


stage("start")
ctx = DistContext.get()
rank, world = ctx.rank, ctx.world
dev = ctx.device
res = {}
stage("dist up")

# --- 1. one-shot all-reduce: each rank contributes rank+1, expect n(n+1)/2; odd size hits the tail -------
peer = PeerComm(ctx, n_max=8192)
ctx.peer = peer
stage("peer comm up")
for n in (128 * 5120, 1024 * 4096 + 1 if 1024 * 4096 + 1 <= peer.slot else peer.slot - 1, 7):
    n = min(n, peer.slot)
    for dt in (torch.float32, torch.bfloat16):
        t = torch.full((n,), float(rank + 1), dtype=dt, device=dev)
        o = peer.all_reduce(t)
        torch.cuda.synchronize()
        want = world * (world + 1) / 2
        assert bool((o.float() == want).all()), (n, dt, o[:4])
res["allreduce"] = "ok"
stage("allreduce ok")
g2 = peer.all_gather(torch.full((5, 2), float(rank), device=dev))
torch.cuda.synchronize()
assert all(bool((g2[r] == r).all()) for r in range(world))
stage("allgather ok")

# --- 2. fused GEMM + all-reduce vs fp32 reference ---------------------------------------------------------
for T in (16, 33):                              # 33 tokens: odd tail of the two-tokens-per-word packing; two-shot from 4 ranks
    g = torch.Generator().manual_seed(T)
    Nf, K = 1024, 2048                          # K is the full reduction dim; each rank owns K/world of it
    x = (torch.randn(T, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(Nf, K, generator=g) * 0.05).bfloat16()
    bias = torch.randn(Nf, generator=g) * 0.1
    resid = torch.randn(T, Nf, generator=g).bfloat16()
    ks = K // world
    xs, ws_ = x[:, rank * ks:(rank + 1) * ks].contiguous().to(dev), w[:, rank * ks:(rank + 1) * ks].contiguous().to(dev)
    W = make_linear(ws_, "bf16")
    want = x.float() @ w.float().t() + bias + 0.5 * resid.float()
    outs = []
    for it in range(3):                         # several calls: exercises both buffer parities
        y = peer.gemm_ar(xs, W, bias.to(dev), None, resid.to(dev), 0.5)
        torch.cuda.synchronize()
        outs.append(y.float().cpu())
        err = (outs[-1] - want).abs().max().item()
        assert err < 5e-2, (T, it, err)
    gathered = [torch.empty_like(outs[0]) for _ in range(world)]
    dist.all_gather_object(gathered, outs[-1], group=ctx.ctrl_group)
    assert all(torch.equal(gathered[0], t) for t in gathered), "ranks must hold bit-identical results"
N.Workspace.get(dev).check_status()
res["gemm_ar"] = "ok"
stage("gemm_ar ok")

# --- 3. tiny Llama, tensor parallel over the GPUs, CUDA-graph decode with the fused kernels -----------------
model = xft.AutoModel.from_pretrained(path, dtype="bf16")
stage("model loaded")
gi = torch.Generator().manual_seed(1)
ids = torch.randint(0, 32000, (2, 32), generator=gi)
# prompt logits of the last position, then one decode step through the CUDA-graph runner: both go to the fp32 oracle
if rank == 0:
    sid = model.set_input_cb(ids.tolist(), None, 64)
    logits0 = model.forward_cb().float().cpu()
    nxt = logits0.argmax(-1)
    model.set_input_cb([[int(t)] for t in nxt], sid, 64)
    logits1 = model.forward_cb().float().cpu()
    model.free_seqs(sid)
else:
    model.set_input_cb()
    model.forward_cb()
    model.set_input_cb()
    model.forward_cb()
    model.free_seqs()
stage("logits done")
tokens = model.generate(ids, max_length=48) if rank == 0 else model.generate()
stage("generate done")
N.Workspace.get(dev).check_status()
m = model.model
res["fused_calls"] = m.ctx.peer.fused_calls
res["graph_launches"] = m.runner.graph_launches
if rank == 0:
    torch.save({"tokens": tokens, "res": res, "logits0": logits0, "logits1": logits1, "next": nxt}, out)
m._closed = True
dist.barrier(group=ctx.ctrl_group)
