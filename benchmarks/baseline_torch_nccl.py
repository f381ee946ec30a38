#!/usr/bin/env python
"""GPU baseline: the same Llama architecture and decode workload in plain PyTorch — cuBLAS GEMMs (torch.matmul),
scaled_dot_product_attention over a contiguous KV cache, NCCL all-reduce for tensor parallelism — with random
weights and synthetic ids.  No kernel of this repository is used.  Prints one JSON line with the same metric as
bench.py (decode tokens/s, device-timed, max over ranks) so the two can be put side by side.

    python benchmarks/baseline_torch_nccl.py --steps 32 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29520 \
        benchmarks/baseline_torch_nccl.py --steps 32 --warmup 3
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from xfastertransformer_b200.tools.synthetic import PRESETS  # noqa: E402  (architecture table only)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-2-70b")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--input-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0)
    a = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    c = PRESETS[a.model]
    H, nh, nkv, D, I, V = c["hidden_size"], c["head_num"], c["kv_head_num"], c["size_per_head"], c["inter_size"], c["vocab_size"]
    L = a.layers or c["num_layer"]
    hq, hkv, Il, Vl = nh // world, max(nkv // world, 1), I // world, V // world
    B, S = a.batch, a.input_len
    total = S + 1 + a.warmup + a.steps
    bf = torch.bfloat16
    rnd = lambda *s: torch.empty(*s, dtype=bf, device=dev).normal_(0, 0.02)
    E, topk = int(c.get("sparse_experts", 0) or 0), int(c.get("num_experts_per_tok", 2) or 2)
    mlp_w = (lambda: dict(router=rnd(E, H), gu=rnd(E, 2 * Il, H), dn=rnd(E, H, Il))) if E else \
        (lambda: dict(gu=rnd(2 * Il, H), dn=rnd(H, Il)))
    layers = [dict(qkv=rnd((hq + 2 * hkv) * D, H), o=rnd(H, hq * D), **mlp_w(), n1=torch.ones(H, dtype=bf, device=dev),
                   n2=torch.ones(H, dtype=bf, device=dev), k=torch.zeros(B, hkv, total, D, dtype=bf, device=dev),
                   v=torch.zeros(B, hkv, total, D, dtype=bf, device=dev)) for _ in range(L)]
    wte, head, fn = rnd(V, H), rnd(Vl, H), torch.ones(H, dtype=bf, device=dev)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=dev).float() / D))

    def rms(x, w):
        return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(bf) * w

    def rope(x, pos):          # x [B, h, T, D]
        f = pos[:, None].float() * inv[None]
        cos, sin = f.cos()[None, None].to(bf), f.sin()[None, None].to(bf)
        x1, x2 = x[..., : D // 2], x[..., D // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    def step(ids, p0):         # ids [B, T]
        T = ids.shape[1]
        pos = torch.arange(p0, p0 + T, device=dev)
        x = wte[ids]
        for l in layers:
            h = rms(x, l["n1"])
            qkv = h @ l["qkv"].t()
            q = qkv[..., : hq * D].view(B, T, hq, D).transpose(1, 2)
            k = qkv[..., hq * D:(hq + hkv) * D].view(B, T, hkv, D).transpose(1, 2)
            v = qkv[..., (hq + hkv) * D:].view(B, T, hkv, D).transpose(1, 2)
            q, k = rope(q, pos), rope(k, pos)
            l["k"][:, :, p0:p0 + T] = k
            l["v"][:, :, p0:p0 + T] = v
            att = F.scaled_dot_product_attention(q, l["k"][:, :, : p0 + T], l["v"][:, :, : p0 + T], is_causal=T > 1,
                                                 enable_gqa=hq != hkv)
            o = att.transpose(1, 2).reshape(B, T, hq * D) @ l["o"].t()
            if world > 1:
                dist.all_reduce(o)
            x = x + o
            h = rms(x, l["n2"])
            if E:
                # Mixtral-style MoE the eager way: every rank holds a slice of every expert; tokens are gathered per
                # expert, run through its two matmuls and scattered back with the routing weight
                flat = h.reshape(-1, H)
                wts, sel = torch.topk(flat.float() @ l["router"].float().t(), topk, dim=-1)
                wts = torch.softmax(wts, -1).to(bf)
                y = torch.zeros_like(flat)
                for e in range(E):
                    tok, slot = (sel == e).nonzero(as_tuple=True)
                    if tok.numel():
                        g = flat[tok] @ l["gu"][e].t()
                        y.index_add_(0, tok, ((F.silu(g[:, :Il]) * g[:, Il:]) @ l["dn"][e].t()) * wts[tok, slot, None])
                y = y.view_as(h)
            else:
                gu = h @ l["gu"].t()
                y = (F.silu(gu[..., :Il]) * gu[..., Il:]) @ l["dn"].t()
            if world > 1:
                dist.all_reduce(y)
            x = x + y
        logits = rms(x[:, -1], fn) @ head.t()
        v_, i_ = logits.float().max(-1)
        if world > 1:
            pair = torch.stack([v_, (i_ + rank * Vl).float()], -1)
            allp = [torch.empty_like(pair) for _ in range(world)]
            dist.all_gather(allp, pair)
            allp = torch.stack(allp)
            return allp[..., 1].gather(0, allp[..., 0].argmax(0)[None])[0].long()
        return i_

    ids = torch.randint(0, V, (B, S), generator=torch.Generator().manual_seed(1)).to(dev)
    with torch.no_grad():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ttfts = []
        for _ in range(2):             # the first prefill is the warm-up (cold: first use of every kernel and of NCCL)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0.record()
            # prefill in chunks of 4 sequences to bound activations
            nxt = step(ids, 0)
            e1.record()
            torch.cuda.synchronize()
            ttfts.append(e0.elapsed_time(e1))
        ttft_cold, ttft = ttfts
        p = S
        for _ in range(a.warmup):
            nxt = step(nxt[:, None], p)
            p += 1
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.steps):
            nxt = step(nxt[:, None], p)
            p += 1
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    t = torch.tensor([ms, ttft, ttft_cold], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"impl": "torch cuBLAS + SDPA + NCCL (eager)", "metric": "decode_tokens_per_s",
                          "value": round(B * a.steps / (t[0].item() / 1e3), 2), "ms_per_step": round(t[0].item() / a.steps, 4),
                          "ttft_ms": round(t[1].item(), 2), "ttft_cold_ms": round(t[2].item(), 2), "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
                          "config": {"model": a.model, "global_batch": B, "seq_len": S, "layers": L}}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
