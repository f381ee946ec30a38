#!/usr/bin/env python
"""Fused GEMM + one-shot all-reduce against its parts, on N GPUs (one process per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29510 benchmarks/bench_fused_comm.py

For the row-parallel shapes of Llama-2-70B at TP=N (o_proj, down_proj; T = 16 and 64 tokens) it times, as CUDA
graphs of 16 back-to-back calls over distinct weight copies (so weights stream from HBM), max over ranks:
  gemm          the local partial GEMM alone (no communication)
  fused         GEMM with the all-reduce in its epilogue over peer memory (xft_gemm_bf16_ar)
  gemm+ar       the partial GEMM followed by the stand-alone peer-memory one-shot all-reduce kernel
  nccl          the partial GEMM followed by an NCCL all-reduce (eager launches; the PyTorch baseline)
and reports the fused kernel against its roofline: the slower of (weight bytes / measured HBM rate) and
(bytes that must cross NVLink per GPU / 770 GB/s).

`--prefill [tokens]` times the prefill-size kernel instead (persistent GEMM with reduce-scatter + all-gather fused in,
opt-in path of the engine) against GEMM + NCCL all-reduce.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from xfastertransformer_b200.ops import native as N  # noqa: E402
from xfastertransformer_b200.parallel.dist import DistContext  # noqa: E402
from xfastertransformer_b200.parallel.fused_comm import PeerComm  # noqa: E402
from xfastertransformer_b200.runtime.loader import make_linear  # noqa: E402


def graph_time(fn, n_calls, iters=20):
    for i in range(n_calls):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for i in range(n_calls):
                fn(i)
        for _ in range(3):
            g.replay()
        s.synchronize()
        ts = []
        for _ in range(iters):
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(s)
            g.replay()
            b.record(s)
            s.synchronize()
            ts.append(a.elapsed_time(b) / n_calls)
    ts.sort()
    return ts[len(ts) // 2]


def eager_time(fn, n_calls, iters=10):
    for i in range(n_calls):
        fn(i)
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n_calls):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) / n_calls)
    ts.sort()
    return ts[len(ts) // 2]


def prefill(ctx, peaks, tokens):
    """Prefill sizes (`--prefill`): the row-parallel GEMMs of Llama-2-70B over `tokens` rows, eager launches, max over
    ranks: the partial GEMM alone, the persistent kernel with reduce-scatter + all-gather fused in
    (PeerComm.gemm_ar_bulk), and GEMM followed by an NCCL all-reduce.  Roofline of the fused kernel: the slower of
    FLOPs / measured bf16 rate and the bytes a GPU must send, 2 (w-1)/w T N 2 B, over 770 GB/s."""
    world, rank, dev = ctx.world, ctx.rank, ctx.device
    os.environ["XFT_PREFILL_FUSED_AR"] = "1"
    os.environ["XFT_MAX_BATCH_TOKENS"] = str(tokens)
    peer = PeerComm(ctx, n_max=8192)
    H = 8192
    for name, K in (("o_proj", 8192 // world), ("down_proj", 28672 // world)):
        K = (K + 63) // 64 * 64
        W = make_linear((torch.randn(H, K, device=dev, dtype=torch.bfloat16) * 0.02), "bf16")
        x = torch.randn(tokens, K, device=dev, dtype=torch.bfloat16)
        resid = torch.randn(tokens, H, device=dev, dtype=torch.bfloat16)
        t_gemm = eager_time(lambda i: N.gemm_bf16(x, W.w, H, residual=resid), 4)
        t_fused = eager_time(lambda i: peer.gemm_ar_bulk(x, W, None, None, resid, 1.0), 4)

        def nccl(i):
            y = N.gemm_bf16(x, W.w, H, residual=resid)
            dist.all_reduce(y)
        t_nccl = eager_time(nccl, 4)
        t = torch.tensor([t_gemm, t_fused, t_nccl], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_gemm, t_fused, t_nccl = t.tolist()
        flops = 2.0 * tokens * H * K
        link_bytes = 2.0 * (world - 1) / world * tokens * H * 2
        roof_ms = max(flops / (peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops", 1400.0)) * 1e12),
                      link_bytes / 770e9) * 1e3
        if rank == 0:
            print(json.dumps({"shape": f"{name} T={tokens} N={H} K={K}", "world": world, "gemm_us": round(t_gemm * 1e3, 1),
                              "fused_us": round(t_fused * 1e3, 1), "gemm_plus_nccl_us": round(t_nccl * 1e3, 1),
                              "roofline_us": round(roof_ms * 1e3, 1), "fused_frac_of_roofline": round(roof_ms / t_fused, 3),
                              "fused_vs_nccl": round(t_nccl / t_fused, 2),
                              "wide_stores": os.environ.get("XFT_PREFILL_WIDE_STORES", "0")}), flush=True)
    N.Workspace.get(dev).check_status()
    dist.barrier()
    peer.close()
    dist.destroy_process_group()


def main():
    ctx = DistContext.get()
    world, rank, dev = ctx.world, ctx.rank, ctx.device
    if "--prefill" in sys.argv:
        peaks = {"hbm_gbs": 6459.6, "bf16_tflops": 1590.0}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        i = sys.argv.index("--prefill")
        tokens = int(sys.argv[i + 1]) if len(sys.argv) > i + 1 and sys.argv[i + 1].isdigit() else 8192
        return prefill(ctx, peaks, tokens)
    peer = PeerComm(ctx, n_max=8192)
    peaks = {"hbm_gbs": 6459.6}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    H = 8192
    shapes = [("o_proj", 16, H, 8192 // world), ("down_proj", 16, H, 28672 // world),
              ("o_proj", 64, H, 8192 // world), ("down_proj", 64, H, 28672 // world)]
    copies = 16
    for name, T, Nf, K in shapes:
        K = (K + 63) // 64 * 64
        ws = [make_linear((torch.randn(Nf, K, device=dev, dtype=torch.bfloat16) * 0.02), "bf16") for _ in range(copies)]
        x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        resid = torch.randn(T, Nf, device=dev, dtype=torch.bfloat16)
        t_gemm = graph_time(lambda i: N.gemm_bf16(x, ws[i].w, Nf, residual=resid), copies)
        t_fused = graph_time(lambda i: peer.gemm_ar(x, ws[i], None, None, resid, 1.0), copies)
        t_two = graph_time(lambda i: peer.all_reduce(N.gemm_bf16(x, ws[i].w, Nf, out_dtype=torch.float32)), copies)

        def nccl(i):
            y = N.gemm_bf16(x, ws[i].w, Nf, residual=resid)
            dist.all_reduce(y)
        t_nccl = eager_time(nccl, copies)
        t = torch.tensor([t_gemm, t_fused, t_two, t_nccl], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_gemm, t_fused, t_two, t_nccl = t.tolist()
        wbytes = Nf * K * 2
        link_bytes = (world - 1) * T * Nf * 4               # fp32 partial tile pushed to every peer
        roof_ms = max(wbytes / (peaks["hbm_gbs"] * 1e9), link_bytes / 770e9) * 1e3
        if rank == 0:
            print(json.dumps({"shape": f"{name} T={T} N={Nf} K={K}", "world": world, "gemm_us": round(t_gemm * 1e3, 2),
                              "fused_us": round(t_fused * 1e3, 2), "gemm_plus_peer_ar_us": round(t_two * 1e3, 2),
                              "gemm_plus_nccl_us": round(t_nccl * 1e3, 2), "roofline_us": round(roof_ms * 1e3, 2),
                              "fused_frac_of_roofline": round(roof_ms / t_fused, 3),
                              "fused_vs_nccl": round(t_nccl / t_fused, 2)}), flush=True)
    N.Workspace.get(dev).check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
