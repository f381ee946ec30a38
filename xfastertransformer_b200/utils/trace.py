"""Chrome-trace timeline (reference ``src/utils/timeline.h``): RAII-style scopes that record
``{ph:"X", name, pid, tid, ts, dur}`` events, filtered by ``XFT_TIMELINE_WHITELIST`` and
dumped to ``timeline_<YYYYmmdd_HHMMSS>.json`` under a file lock at ``finalize()``/``free_seqs()``.

On CUDA a scope also records a pair of CUDA events so the dumped duration is device time,
and pushes an NVTX range with the same name.
"""
from __future__ import annotations

import fcntl
import json
import os
import threading
import time
from typing import List, Optional

from .flags import Env

_events: List[dict] = []
_pending: List[tuple] = []
_lock = threading.Lock()
_enabled: Optional[bool] = None


def enabled() -> bool:
    global _enabled
    if _enabled is None:
        _enabled = Env.get().timeline
    return _enabled


def enable(flag: bool = True) -> None:
    global _enabled
    _enabled = flag


class TimeLine:
    """``with TimeLine("Decoder.forward"):`` — no-op unless tracing is enabled."""

    __slots__ = ("name", "t0", "ev0", "ev1", "on")

    def __init__(self, name: str):
        self.name = name
        self.on = enabled() and self._allowed(name)
        self.ev0 = self.ev1 = None

    @staticmethod
    def _allowed(name: str) -> bool:
        wl = Env.get().timeline_whitelist
        return not wl or name in wl

    def __enter__(self):
        if self.on:
            self.t0 = time.perf_counter_ns()
            try:
                import torch
                if torch.cuda.is_available() and torch.cuda.is_initialized():
                    torch.cuda.nvtx.range_push(self.name)
                    self.ev0 = torch.cuda.Event(enable_timing=True)
                    self.ev1 = torch.cuda.Event(enable_timing=True)
                    self.ev0.record()
            except Exception:
                self.ev0 = None
        return self

    def __exit__(self, *exc):
        if not self.on:
            return False
        t1 = time.perf_counter_ns()
        ev = {"ph": "X", "name": self.name, "pid": os.getpid(), "tid": threading.get_ident() % 100000,
              "ts": self.t0 / 1000.0, "dur": (t1 - self.t0) / 1000.0}
        if self.ev0 is not None:
            import torch
            self.ev1.record()
            torch.cuda.nvtx.range_pop()
            with _lock:
                _pending.append((ev, self.ev0, self.ev1))
        else:
            with _lock:
                _events.append(ev)
        return False


def _resolve_pending() -> None:
    if not _pending:
        return
    import torch
    torch.cuda.synchronize()
    for ev, e0, e1 in _pending:
        ev["dur"] = e0.elapsed_time(e1) * 1000.0
        ev["args"] = {"clock": "cuda_event"}
        _events.append(ev)
    _pending.clear()


def dump(path: Optional[str] = None) -> Optional[str]:
    """Append-safe dump; returns the file written (None if nothing recorded)."""
    with _lock:
        _resolve_pending()
        if not _events:
            return None
        if path is None:
            path = time.strftime("timeline_%Y%m%d_%H%M%S.json")
        with open(path, "a+") as f:
            fcntl.flock(f, fcntl.LOCK_EX)
            f.seek(0)
            txt = f.read()
            old = []
            if txt.strip():
                try:
                    old = json.loads(txt).get("traceEvents", [])
                except Exception:
                    old = []
            f.seek(0)
            f.truncate()
            json.dump({"traceEvents": old + _events}, f)
            fcntl.flock(f, fcntl.LOCK_UN)
        _events.clear()
        return path


def events() -> List[dict]:
    with _lock:
        _resolve_pending()
        return list(_events)
