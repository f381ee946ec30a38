#!/usr/bin/env python
"""Headline benchmark: Llama-2-70B (bf16) decode tokens/s and first-token latency on N B200s.

Metric definitions are the reference's (``benchmark/benchmark.py:303-357``): first-token latency =
time of the first ``forward()`` after ``set_input`` (prefill + first token); next-token latency =
time of each later ``forward()``; throughput = 1000 / mean(next_token_ms) * batch_size.

    python bench.py --gpus 1 --steps 32 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 32 --warmup 3

A step is one decode step of the whole batch through the public API (`AutoModel.set_input` +
`forward()`), tensor-parallel over the N GPUs (strong scaling: the job is the same at every N).
Weights are random N(0, 0.02) of the named architecture drawn on the device
(``XFT_FAKE_MODEL=2``), token ids are synthetic.  Two numbers are reported:

* ``value``      — device time of the K timed steps (CUDA events around each step's graph launch on
                   the launching stream), max over ranks;
* ``e2e.value``  — the same K steps timed end to end around ``forward()``: every step includes the
                   host->device copy of that step's inputs from pinned memory and the device->host read
                   of the chosen tokens.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _clock_sampler():
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
    try:
        p = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "200"],
                             stdout=f, stderr=subprocess.DEVNULL)
    except Exception:
        return None, f.name
    return p, f.name


def _clock_summary(proc, path, dev_index):
    if proc is None:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    proc.terminate()
    try:
        proc.wait(timeout=5)
    except Exception:
        proc.kill()
    sm, mx, reasons = [], [], set()
    try:
        lines = open(path).read().splitlines()
        if not any(l.strip() for l in lines):
            # region shorter than one sampling period: take one reading now
            q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
                 "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                 "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
            try:
                lines = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                                       capture_output=True, text=True, timeout=20).stdout.splitlines()
            except Exception:
                lines = []
        for line in lines:
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9 or not c[0].isdigit() or int(c[0]) != dev_index:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
    finally:
        try:
            os.unlink(path)
        except OSError:
            pass
    return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons), "samples": len(sm)}


def run_reference(args):
    """The reference (intel/xFasterTransformer) is a Xeon engine: its CMake build needs AVX512-BF16/AMX and
    downloads xDNN, oneDNN, oneCCL and MKL at configure time, so the one offline install attempt failed."""
    why = ("reference cannot be installed offline: pip --no-deps build of the unmodified tree stops in CMake "
           "(\"Your compiler has issues to support avx512bf16\"; it would next download xDNN/oneDNN/oneCCL/MKL); "
           "it has no CUDA path at all")
    if int(os.environ.get("RANK", "0")) == 0:            # one line per job, also under torchrun
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def _vs_baseline(model, batch, input_len, n_gpus, dtype, value):
    """value / the decode tokens/s of the plain PyTorch (cuBLAS + SDPA + NCCL) arm measured on this pool for the same
    model, batch, prompt length and GPU count (benchmarks/baseline_results.json, written from runs of
    benchmarks/baseline_torch_nccl.py; the reference itself publishes no number).  None when no such row exists."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "benchmarks", "baseline_results.json")
    try:
        with open(path) as f:
            rows = json.load(f)["rows"]
    except (OSError, ValueError, KeyError):
        return None
    for r in rows:
        c = r.get("config", {})
        if (c.get("model") == model and c.get("global_batch") == batch and c.get("seq_len") == input_len
                and r.get("n_gpus") == n_gpus and r.get("dtype", "bf16") == dtype and r.get("value")):
            return round(value / float(r["value"]), 3)
    return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-2-70b")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--input-len", type=int, default=2048)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--kv-dtype", default="bf16")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (result is flagged invalid)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.warmup < 3:
        args.warmup = 3

    os.environ["XFT_FAKE_MODEL"] = "2"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    import torch
    import torch.distributed as dist

    import xfastertransformer_b200 as xft
    from xfastertransformer_b200.ops import native as N
    from xfastertransformer_b200.tools.synthetic import config_only, preset

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run",
                  file=sys.stderr)
        if world == 1 and args.gpus > 1:
            return 2
    over = {"num_layer": args.layers} if args.layers else {}
    cfg = preset(args.model, **over)
    cfg.max_pos_seq_len = max(cfg.max_pos_seq_len, args.input_len + args.steps + args.warmup + 8)
    tmp = tempfile.mkdtemp(prefix="xft_bench_")
    config_only(tmp, cfg)

    t_load = time.time()
    model = xft.AutoModel.from_pretrained(tmp, dtype=args.dtype, kv_cache_dtype=args.kv_dtype)
    m = model.model
    dev = m.ctx.device
    torch.cuda.synchronize()
    t_load = time.time() - t_load

    B, L = args.batch, args.input_len
    total_new = 1 + args.warmup + args.steps
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (B, L), generator=g).pin_memory()

    def sync_all():
        if world > 1:
            dist.barrier(group=m.ctx.ctrl_group)
        torch.cuda.synchronize()

    # eos = -2 never matches: all sequences decode the full length.  The first pass is the warm-up of the prefill (first
    # use of every kernel, the allocator's first blocks, NCCL's channels); the reference's benchmark also reports
    # first-token latency of warmed iterations (benchmark/benchmark.py: --warmup).  A new set_input releases the first
    # pass's sequences, so the second pass prefills the same prompts from an empty cache.
    ttft = []
    for _ in range(2):
        model.set_input(ids, max_length=L + total_new + 1, eos_token_id=-2, pad_token_id=0)
        sync_all()
        t0 = time.perf_counter()
        model.forward()                          # prefill + first token
        torch.cuda.synchronize()
        ttft.append((time.perf_counter() - t0) * 1e3)
    ttft_cold_ms, ttft_ms = ttft
    for _ in range(args.warmup):
        model.forward()
    runner = m.runner
    ws = N.Workspace.get(dev)
    runner.timing = True
    runner.step_events = []
    launches0 = runner.kernel_launches
    h2d0, d2h0 = runner.h2d_bytes, runner.d2h_bytes
    sampler, spath = _clock_sampler() if rank == 0 else (None, None)
    sync_all()
    wall0 = time.perf_counter()
    step_ms = []
    eager_events = []            # steps that do not go through the graph runner (pipeline stages, data-parallel attention)
    launches_ws0 = ws.launches
    for _ in range(args.steps):
        t1 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        model.forward()
        e1.record()
        eager_events.append((e0, e1))
        step_ms.append((time.perf_counter() - t1) * 1e3)
    sync_all()
    wall = time.perf_counter() - wall0
    clocks = _clock_summary(sampler, spath, dev.index or 0) if rank == 0 else None
    if len(runner.step_events) == args.steps:
        dev_ms = sum(a.elapsed_time(b) for a, b in runner.step_events)
        n_launch = runner.kernel_launches - launches0
    else:
        dev_ms = sum(a.elapsed_time(b) for a, b in eager_events)
        n_launch = ws.launches - launches_ws0
    runner.timing = False
    ws.check_status()
    t = torch.tensor([dev_ms, wall * 1e3, ttft_ms, ttft_cold_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms, ttft_ms, ttft_cold_ms = t.tolist()
    if rank == 0:
        K = args.steps
        value = B * K / (dev_ms / 1e3)
        e2e = B * K / (wall_ms / 1e3)
        wbytes = m.decoder.weight_bytes()
        out = {
            "metric": "decode_tokens_per_s", "value": round(value, 2), "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": args.warmup, "ms_per_step": round(dev_ms / K, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": _vs_baseline(args.model, B, L, world, args.dtype, value), "dtype": args.dtype,
            "data": "synthetic token ids; random-init N(0,0.02) weights of the named architecture",
            "config": {"model": args.model, "global_batch": B, "seq_len": L, "output_len": total_new,
                       "parallelism": (f"dp{world}+ep{world}" if m.ctx.dp_size > 1 else
                                       f"pp{m.ctx.pp_size}xtp{m.ctx.tp_size}" if m.ctx.pp_size > 1 else
                                       f"tp{world}+ep{world}" if m.ctx.ep_size > 1 else f"tp{world}"),
                       "kv_cache": f"paged-64 {args.kv_dtype}",
                       "l2": "inputs larger than L2 (each step streams %.1f GB of weights per GPU)" % (wbytes / 1e9),
                       "layers": cfg.num_layer,
                       # every XFT_* variable that was set for this run (opt-in kernels and modes change what is timed)
                       "env": {k: v for k, v in sorted(os.environ.items())
                               if k.startswith("XFT_") and k != "XFT_FAKE_MODEL"}},
            "ttft_ms": round(ttft_ms, 2), "ttft_cold_ms": round(ttft_cold_ms, 2),
            "next_token_ms": {"avg": round(statistics.mean(step_ms), 4), "min": round(min(step_ms), 4),
                              "max": round(max(step_ms), 4),
                              "p90": round(sorted(step_ms)[int(0.9 * (len(step_ms) - 1))], 4)},
            "e2e": {"value": round(e2e, 2), "unit": "tokens/s",
                    "h2d_bytes_per_step": (runner.h2d_bytes - h2d0) // K,
                    "d2h_bytes_per_step": (runner.d2h_bytes - d2h0) // K},
            "gpu_launches": int(n_launch),
            "clocks": clocks,
            "hbm_fraction_of_measured": None,
            "load_s": round(t_load, 1),
        }
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
            kvb = sum(2 * (L + 1 + args.warmup + K // 2) * m.decoder.hkv * m.decoder.D * 2 for _ in range(B)) * \
                len(m.decoder.layers)
            out["hbm_fraction_of_measured"] = round((wbytes + kvb) / (dev_ms / K / 1e3) / (peaks["hbm_gbs"] * 1e9), 3)
        except Exception:
            pass
        if args.layers:
            out["invalid"] = "debug run with fewer layers"
        print(json.dumps(out))
    model.finalize()
    m._closed = True          # every rank runs this script to the end: nobody sits in a serving loop to be released
    if world > 1:
        dist.barrier(group=m.ctx.ctrl_group)
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
