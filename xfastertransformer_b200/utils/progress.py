"""Text progress bar for weight loading (reference: ``src/utils/progress_bar.h``, used by ``DecoderBlock``'s
constructor at ``src/layers/decoder_block.h:45,66-68`` to show one tick per loaded layer).

Drawn on rank 0 only, and only when the stream is a terminal or ``XFT_PROGRESS=1`` is set, so logs of batch jobs and of
the follower ranks stay clean.  ``for i in ProgressBar.wrap(range(n), "Loading layers"): ...``
"""
from __future__ import annotations

import os
import sys
import time
from typing import Iterable, Iterator, Optional, TextIO


class ProgressBar:
    def __init__(self, total: int, title: str = "", width: int = 40, stream: Optional[TextIO] = None,
                 enabled: Optional[bool] = None):
        self.total = max(int(total), 0)
        self.title = title
        self.width = width
        self.stream = stream if stream is not None else sys.stderr
        if enabled is None:
            forced = os.environ.get("XFT_PROGRESS")
            rank0 = int(os.environ.get("RANK", os.environ.get("PMI_RANK", "0")) or 0) == 0
            enabled = rank0 and (forced == "1" or (forced is None and hasattr(self.stream, "isatty") and self.stream.isatty()))
        self.enabled = bool(enabled) and self.total > 0
        self.done = 0
        self.t0 = time.perf_counter()
        self._draw()

    def _draw(self) -> None:
        if not self.enabled:
            return
        frac = self.done / self.total
        fill = int(round(frac * self.width))
        dt = time.perf_counter() - self.t0
        self.stream.write(f"\r{self.title} [{'#' * fill}{'.' * (self.width - fill)}] {self.done}/{self.total} "
                          f"{dt:5.1f}s")
        if self.done >= self.total:
            self.stream.write("\n")
        self.stream.flush()

    def update(self, n: int = 1) -> None:
        self.done = min(self.done + n, self.total)
        self._draw()

    @classmethod
    def wrap(cls, it: Iterable, title: str = "", **kw) -> Iterator:
        items = list(it)
        bar = cls(len(items), title, **kw)
        for x in items:
            yield x
            bar.update()
