#!/usr/bin/env python
"""GPU baseline: the same Llama architecture and decode workload in plain PyTorch — cuBLAS GEMMs (torch.matmul),
scaled_dot_product_attention over a contiguous KV cache, NCCL all-reduce for tensor parallelism — with random
weights and synthetic ids.  No kernel of this repository is used.  Prints one JSON line with the same metric as
bench.py (decode tokens/s, device-timed, max over ranks) so the two can be put side by side.

It is meant as a fair library arm, not a straw man: decode attention treats the query heads of one KV head as the
query rows of that head, so SDPA runs its fused backend without the GQA expansion; the prompt is prefilled in chunks of
sequences like the engine does; on one GPU (no NCCL in the step) the decode step is captured in a CUDA graph
(`--graph 0` turns that off); with several ranks the step runs eagerly with NCCL all-reduces, never captured.

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
    ap.add_argument("--graph", type=int, default=-1, help="1: CUDA-graph the decode step (default on one GPU, dense models)")
    ap.add_argument("--prefill-chunk", type=int, default=4, help="sequences per prefill pass")
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

    def attention(l, q, k, v, b0, Bc, T, p0, pos_dev):
        """q [Bc, hq, T, D]; appends k, v [Bc, hkv, T, D] to the cache and attends over it."""
        kc, vc = l["k"][b0:b0 + Bc], l["v"][b0:b0 + Bc]
        if pos_dev is not None:
            # graph-safe decode: the position lives on the device, the whole cache is attended under a mask
            kc.index_copy_(2, pos_dev, k)
            vc.index_copy_(2, pos_dev, v)
            mask = (torch.arange(total, device=dev) <= pos_dev)[None, None, None, :]
            g = hq // hkv
            o = F.scaled_dot_product_attention(q.view(Bc, hkv, g, D), kc, vc, attn_mask=mask)
            return o.view(Bc, hq, 1, D)
        kc[:, :, p0:p0 + T] = k
        vc[:, :, p0:p0 + T] = v
        if T == 1:
            g = hq // hkv          # the g query heads of a KV head are g query rows of that head: no causal mask needed
            o = F.scaled_dot_product_attention(q.view(Bc, hkv, g, D), kc[:, :, : p0 + 1], vc[:, :, : p0 + 1])
            return o.view(Bc, hq, 1, D)
        return F.scaled_dot_product_attention(q, kc[:, :, : p0 + T], vc[:, :, : p0 + T], is_causal=True,
                                              enable_gqa=hq != hkv)

    def step(ids, p0, b0=0, pos_dev=None):         # ids [Bc, T]; sequences b0 .. b0 + Bc of the batch
        Bc, T = ids.shape
        pos = pos_dev if pos_dev is not None else torch.arange(p0, p0 + T, device=dev)
        x = wte[ids]
        for l in layers:
            h = rms(x, l["n1"])
            qkv = h @ l["qkv"].t()
            q = qkv[..., : hq * D].view(Bc, T, hq, D).transpose(1, 2)
            k = qkv[..., hq * D:(hq + hkv) * D].view(Bc, T, hkv, D).transpose(1, 2)
            v = qkv[..., (hq + hkv) * D:].view(Bc, T, hkv, D).transpose(1, 2)
            q, k = rope(q, pos), rope(k, pos)
            att = attention(l, q, k, v, b0, Bc, T, p0, pos_dev)
            o = att.transpose(1, 2).reshape(Bc, T, hq * D) @ l["o"].t()
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

    def prefill(ids):
        outs = []
        for b0 in range(0, B, max(1, a.prefill_chunk)):
            outs.append(step(ids[b0:b0 + a.prefill_chunk], 0, b0))
        return torch.cat(outs)

    ids = torch.randint(0, V, (B, S), generator=torch.Generator().manual_seed(1)).to(dev)
    with torch.no_grad():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ttfts = []
        for _ in range(2):             # the first prefill is the warm-up (cold: first use of every kernel and of NCCL)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0.record()
            nxt = prefill(ids)
            e1.record()
            torch.cuda.synchronize()
            ttfts.append(e0.elapsed_time(e1))
        ttft_cold, ttft = ttfts
        p = S
        use_graph = (a.graph == 1 or (a.graph < 0 and world == 1)) and world == 1 and not E
        if use_graph:
            # one captured decode step, replayed with the position and the input ids updated in place
            pos_dev = torch.tensor([p], device=dev, dtype=torch.long)
            ids_in = nxt[:, None].clone()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step(ids_in, p, 0, pos_dev)            # warm the kernels outside capture
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    out_ids = step(ids_in, p, 0, pos_dev)
            torch.cuda.current_stream().wait_stream(side)

            def decode_once():
                nonlocal p
                graph.replay()
                ids_in.copy_(out_ids[:, None])
                pos_dev.add_(1)
                p += 1
        else:
            def decode_once():
                nonlocal p, nxt
                nxt = step(nxt[:, None], p)
                p += 1
        for _ in range(a.warmup):
            decode_once()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.steps):
            decode_once()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    t = torch.tensor([ms, ttft, ttft_cold], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"impl": "torch cuBLAS + SDPA" + (" (decode step in a CUDA graph)" if use_graph else " + NCCL (eager)"), "metric": "decode_tokens_per_s",
                          "value": round(B * a.steps / (t[0].item() / 1e3), 2), "ms_per_step": round(t[0].item() / a.steps, 4),
                          "ttft_ms": round(t[1].item(), 2), "ttft_cold_ms": round(t[2].item(), 2), "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
                          "config": {"model": a.model, "global_batch": B, "seq_len": S, "layers": L, "graph": bool(use_graph)}}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
