"""Tensor dumps for debugging (reference: ``src/utils/debugger.h`` — ``dumpMatrix`` calls compiled in with ``-DDEBUG`` that
write intermediate activations of every layer to files).  Here it is a run-time switch: with ``XFT_DEBUG_DIR=<dir>`` set,
the decoder writes the hidden state after each attention and FFN block of every forward to
``<dir>/rank<r>_step<k>_<name>.pt`` (fp32 on the host) and a one-line summary (shape, mean, abs-max, first values) to
``<dir>/rank<r>.log``.  Dumping synchronises the device and disables CUDA-graph capture; it is off by default.
"""
from __future__ import annotations

import os
import threading
from typing import Optional

import torch

from .flags import Env

_lock = threading.Lock()
_step = 0


def enabled() -> bool:
    return bool(Env.get().debug_dir)


def next_step() -> int:
    global _step
    with _lock:
        _step += 1
        return _step


def dump(name: str, t: Optional[torch.Tensor], rank: int = 0, step: Optional[int] = None, max_rows: int = 64) -> None:
    """Write `t` (first `max_rows` rows) and a summary line; no-op unless XFT_DEBUG_DIR is set."""
    d = Env.get().debug_dir
    if not d or t is None:
        return
    os.makedirs(d, exist_ok=True)
    k = _step if step is None else step
    x = t.detach()
    x2 = x.reshape(-1, x.shape[-1]) if x.dim() > 1 else x.reshape(1, -1)
    host = x2[:max_rows].float().cpu()
    torch.save(host, os.path.join(d, f"rank{rank}_step{k}_{name}.pt"))
    with _lock, open(os.path.join(d, f"rank{rank}.log"), "a") as f:
        flat = host.flatten()
        f.write(f"step {k} {name}: shape {tuple(x.shape)} dtype {x.dtype} mean {float(flat.mean()):.6g} "
                f"absmax {float(flat.abs().max()):.6g} first {[round(float(v), 5) for v in flat[:6]]}\n")
