#!/usr/bin/env python
"""Kernel micro-benchmark: the tcgen05 GEMM of this library against torch.matmul (cuBLAS) on the
per-GPU shapes of the BASELINE configs.  CUDA-event timing on the launching stream, warm-up, and a
rotation over enough distinct weight copies that every timed launch streams its weight from HBM
(working set > the 126 MB L2).  Prints achieved GB/s (decode shapes are bandwidth-bound) and TFLOP/s,
and the fraction of the measured peaks in MEASURED_PEAKS.json.

    python benchmarks/bench_gemm.py [--shapes decode|prefill|all] [--iters 20] [--one T,N,K[,gated]]
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from xfastertransformer_b200.ops import native as N  # noqa: E402

# (name, T, N, K, gated)  — Llama-2-70B at TP=1 and TP=8, decode batch 16/64 and a prefill chunk
DECODE = [
    ("70b tp1 qkv   b16", 16, 10240, 8192, False), ("70b tp1 o     b16", 16, 8192, 8192, False),
    ("70b tp1 gateup b16", 16, 28672, 8192, True), ("70b tp1 down  b16", 16, 8192, 28672, False),
    ("70b tp1 lmhead b16", 16, 32000, 8192, False),
    ("70b tp8 qkv   b16", 16, 1280, 8192, False), ("70b tp8 o     b16", 16, 8192, 1024, False),
    ("70b tp8 gateup b16", 16, 3584, 8192, True), ("70b tp8 down  b16", 16, 8192, 3584, False),
    ("70b tp8 gateup b64", 64, 3584, 8192, True), ("70b tp1 gateup b64", 64, 28672, 8192, True),
    ("70b tp2 qkv   b16", 16, 5120, 8192, False), ("70b tp2 o     b16", 16, 8192, 4096, False),
    ("70b tp2 gateup b16", 16, 14336, 8192, True), ("70b tp2 down  b16", 16, 8192, 14336, False),
    ("70b tp4 gateup b16", 16, 7168, 8192, True), ("70b tp4 down  b16", 16, 8192, 7168, False),
    ("70b tp8 lmhead b16", 16, 4000, 8192, False), ("7b  tp1 qkv   b16", 16, 12288, 4096, False),
    ("7b  tp1 gateup b16", 16, 11008, 4096, True), ("7b  tp1 down  b16", 16, 4096, 11008, False),
]
PREFILL = [
    ("70b tp1 qkv   t8192", 8192, 10240, 8192, False), ("70b tp1 gateup t8192", 8192, 28672, 8192, True),
    ("70b tp1 down  t8192", 8192, 8192, 28672, False), ("70b tp8 gateup t8192", 8192, 3584, 8192, True),
    ("7b  tp1 qkv   t4096", 4096, 12288, 4096, False),
    # tensor-parallel slices: the row-parallel products have a short reduction, so the epilogue weighs most
    ("70b tp8 qkv   t8192", 8192, 1280, 8192, False), ("70b tp8 o     t8192", 8192, 8192, 1024, False),
    ("70b tp8 down  t8192", 8192, 8192, 3584, False), ("70b tp2 o     t8192", 8192, 8192, 4096, False),
    ("70b tp2 down  t8192", 8192, 8192, 14336, False), ("70b tp4 down  t8192", 8192, 8192, 7168, False),
]


def time_fn(fn, n_variants, iters):
    """Median time per launch.  Each timed sample is one CUDA-graph replay of `n_variants` launches (one per
    weight copy), so short kernels are not measured through host launch gaps."""
    for i in range(n_variants):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for i in range(n_variants):
                fn(i)
        for _ in range(3):
            g.replay()
        s.synchronize()
        evs = []
        for i in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(s)
            g.replay()
            b.record(s)
            evs.append((a, b))
        s.synchronize()
    ts = sorted(a.elapsed_time(b) / n_variants for a, b in evs)
    return ts[len(ts) // 2]


def kernel_timeline(fn, copies):
    """Time line of one launch of the decode GEMM (csrc/kernels/gemm_decode_sm100.cu) inside an eager chain of launches
    over distinct weights: the kernel stamps the GPU's global timer at eight points per CTA (xft_gemm_sk_set_trace);
    returned are min / median / max over the CTAs in microseconds after the first CTA's entry, plus the exit of the
    launch in front.  Empty when the product did not go through that kernel."""
    import ctypes as C
    lib = N.lib()
    max_ctas = 320
    buf = torch.zeros(copies, max_ctas * 8, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    for i in range(copies):
        lib.xft_gemm_sk_set_trace(C.c_void_p(buf[i].data_ptr()))
        fn(i)
    lib.xft_gemm_sk_set_trace(C.c_void_p(0))
    torch.cuda.synchronize()
    b = buf.cpu().view(copies, max_ctas, 8)
    i = copies - 2
    live = b[i][:, 0] > 0
    if int(live.sum()) == 0:
        return {}
    t = b[i][live].double()
    prev = b[i - 1][b[i - 1][:, 0] > 0]
    t0 = t[:, 0].min().item()
    names = ["entry", "setup_done", "dependency_resolved", "first_block_landed", "last_mma_issued", "last_accumulator_ready",
             "epilogue_done", "exit"]
    out = {n: [round((f(t[:, k]).item() - t0) / 1e3, 2) for f in (torch.min, torch.median, torch.max)]
           for k, n in enumerate(names)}
    out["ctas"] = int(live.sum())
    if prev.numel():
        out["previous_exit"] = round((prev[:, 7].max().item() - t0) / 1e3, 2)
    return out


def run(name, T, Nf, K, gated, iters, peaks, timeline=False):
    rows = 2 * Nf if gated else Nf
    wbytes = rows * K * 2
    copies = max(4, min(24, (400 << 20) // wbytes + 1))
    ws = [(torch.randn(rows, K, device="cuda", dtype=torch.bfloat16) * 0.02) for _ in range(copies)]
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, Nf, device="cuda", dtype=torch.bfloat16)

    def ours(i):
        N.gemm_bf16(x, ws[i], Nf, gated=gated, dual_off=Nf, act="silu" if gated else None, out=out)

    def cublas(i):
        y = torch.matmul(x, ws[i].t())
        if gated:
            torch.nn.functional.silu(y[:, :Nf]).mul_(y[:, Nf:])

    t_ours = time_fn(ours, copies, iters)
    t_ref = time_fn(cublas, copies, iters)
    byts = wbytes + T * K * 2 + T * Nf * 2
    flops = 2.0 * T * rows * K
    gbs = byts / t_ours / 1e6
    tf = flops / t_ours / 1e9
    rec = {"shape": name, "T": T, "N": Nf, "K": K, "gated": gated, "ours_us": round(t_ours * 1e3, 2),
           "cublas_us": round(t_ref * 1e3, 2), "speedup_vs_cublas": round(t_ref / t_ours, 3), "GBps": round(gbs, 1),
           "TFLOPs": round(tf, 1)}
    if peaks:
        rec["hbm_frac_of_measured"] = round(gbs / peaks["hbm_gbs"], 3)
        rec["mma_frac_of_measured"] = round(tf / peaks["bf16_tflops"], 3)
    if timeline and T <= 64:
        rec["timeline_us"] = kernel_timeline(ours, copies)
    print(json.dumps(rec), flush=True)
    N.Workspace.get(torch.device("cuda", 0)).check_status()


def sweep(name, T, Nf, K, gated, iters):
    """Time every split-K factor of one shape (force_splits) next to the planner's own choice (0)."""
    rows = 2 * Nf if gated else Nf
    wbytes = rows * K * 2
    copies = max(4, min(24, (400 << 20) // wbytes + 1))
    ws = [(torch.randn(rows, K, device="cuda", dtype=torch.bfloat16) * 0.02) for _ in range(copies)]
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, Nf, device="cuda", dtype=torch.bfloat16)
    res = {}
    for s in (0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 12, 14, 16, 20, 24, 32):
        if s > max(1, K // 128):
            break

        def f(i):
            N.gemm_bf16(x, ws[i], Nf, gated=gated, dual_off=Nf, act="silu" if gated else None, out=out, force_splits=s)
        res[s] = round(time_fn(f, copies, iters) * 1e3, 2)
    best = min((v, k) for k, v in res.items() if k)[1]
    print(json.dumps({"shape": name, "T": T, "N": Nf, "K": K, "gated": gated, "planner_us": res[0], "best_split": best,
                      "best_us": res[best], "us_by_split": {str(k): v for k, v in res.items() if k}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep-splits", action="store_true", help="time each split-K factor per shape")
    ap.add_argument("--shapes", default="all")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--one", default="")
    ap.add_argument("--timeline", action="store_true", help="decode shapes: per-CTA time line of one launch")
    a = ap.parse_args()
    peaks = None
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    if a.one:
        f = a.one.split(",")
        shapes = [("custom", int(f[0]), int(f[1]), int(f[2]), len(f) > 3 and f[3] == "gated")]
    else:
        shapes = (DECODE if a.shapes in ("decode", "all") else []) + (PREFILL if a.shapes in ("prefill", "all") else [])
    for s in shapes:
        if a.sweep_splits:
            sweep(*s, a.iters)
        else:
            run(*s, a.iters, peaks, a.timeline)


if __name__ == "__main__":
    main()
