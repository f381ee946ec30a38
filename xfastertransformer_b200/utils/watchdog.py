"""Host-side watchdog on step latency.

The reference has no failure detection: a rank that dies leaves the others blocked in a collective for ever
(``src/comm_helper/comm_helper.cpp:94-113``, the spins of ``src/utils/shm_ccl.h:60-70``).  Here every device-side wait is
bounded and every host collective has a time-out; this module is the last line: a monitor thread that notices when one
engine step (a prefill or a decode step, including its collectives and the copy of the chosen tokens) takes longer
than ``XFT_STEP_TIMEOUT_S`` seconds.  A blocked CUDA call cannot be interrupted from Python, so the watchdog

* logs the overdue step (what it was, for how long) and dumps every thread's Python stack to stderr
  (``faulthandler``), which is what an operator needs to see where a rank is stuck,
* calls an optional hook (the serving layer uses it to fail its health check; multi-rank launchers can use it to tell
  the other ranks through the store before their next launch),
* and makes the step raise :class:`StepTimeout` when (if) it returns, so the caller does not continue with a result
  that arrived after the peers may have given up.

With the limit at 0 (the default) ``StepWatchdog.scope`` is a no-op context manager and no thread is started.
"""
from __future__ import annotations

import contextlib
import faulthandler
import sys
import threading
import time
from typing import Callable, Optional

from . import log


class StepTimeout(RuntimeError):
    """An engine step ran longer than XFT_STEP_TIMEOUT_S."""


class StepWatchdog:
    def __init__(self, limit_s: float, on_timeout: Optional[Callable[[str, float], None]] = None,
                 dump_stacks: bool = True):
        self.limit_s = float(limit_s)
        self.on_timeout = on_timeout
        self.dump_stacks = dump_stacks
        self.trips = 0                      # steps that ran over, since construction
        self.last_overdue: Optional[str] = None
        self._cv = threading.Condition()
        self._armed_at: Optional[float] = None
        self._what = ""
        self._tripped = False
        self._stop = False
        self._thread: Optional[threading.Thread] = None

    # ------------------------------------------------------------------------------------
    def _ensure_thread(self) -> None:
        if self._thread is None or not self._thread.is_alive():
            self._stop = False
            self._thread = threading.Thread(target=self._monitor, name="xft-step-watchdog", daemon=True)
            self._thread.start()

    def _monitor(self) -> None:
        with self._cv:
            while not self._stop:
                if self._armed_at is None or self._tripped:
                    self._cv.wait(1.0)
                    continue
                left = self._armed_at + self.limit_s - time.monotonic()
                if left > 0:
                    self._cv.wait(left)
                    continue
                # overdue: report once per step, outside the lock-free fast path of the engine thread
                self._tripped = True
                self.trips += 1
                what, late = self._what, time.monotonic() - self._armed_at
                self.last_overdue = what
                self._cv.release()
                try:
                    self._report(what, late)
                finally:
                    self._cv.acquire()

    def _report(self, what: str, late: float) -> None:
        log.error(f"step watchdog: '{what}' has been running for {late:.1f} s (limit {self.limit_s:g} s)")
        if self.dump_stacks:
            try:
                faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
            except Exception:
                pass
        if self.on_timeout is not None:
            try:
                self.on_timeout(what, late)
            except Exception as e:          # a failing hook must not kill the monitor
                log.error(f"step watchdog: hook raised {e!r}")

    # ------------------------------------------------------------------------------------
    @contextlib.contextmanager
    def scope(self, what: str):
        """Guard one step.  Raises StepTimeout on exit if the step ran over the limit."""
        if self.limit_s <= 0:
            yield
            return
        self._ensure_thread()
        with self._cv:
            self._armed_at = time.monotonic()
            self._what = what
            self._tripped = False
            self._cv.notify()
        try:
            yield
        finally:
            with self._cv:
                tripped, t0 = self._tripped, self._armed_at
                self._armed_at = None
                self._tripped = False
        if tripped:
            raise StepTimeout(f"'{what}' took {time.monotonic() - t0:.1f} s, over the limit of {self.limit_s:g} s "
                              f"(XFT_STEP_TIMEOUT_S)")

    @property
    def overdue(self) -> bool:
        """True while a guarded step is still running past its limit (a health check can fail on it)."""
        return self._tripped and self._armed_at is not None

    def close(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
            self._thread = None
