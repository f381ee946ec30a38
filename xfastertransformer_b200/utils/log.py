"""Leveled logger (reference ``src/utils/logger.h:25-89``) and the per-kernel verbose line
(``src/utils/verbose.h:24-83``: ``xft_verbose,exec,<dev>,api,<kernel>,m<M>n<N>k<K>,<ms>``)."""
from __future__ import annotations

import sys
import time

DEBUG, INFO, WARNING, ERROR = 0, 1, 2, 3
_level = INFO
_names = {DEBUG: "DEBUG", INFO: "INFO", WARNING: "WARNING", ERROR: "ERROR"}
_colors = {DEBUG: "\033[36m", INFO: "\033[32m", WARNING: "\033[33m", ERROR: "\033[31m"}


def set_level(level: int) -> None:
    global _level
    _level = level


def _emit(level: int, msg: str) -> None:
    if level < _level:
        return
    ts = time.strftime("%Y-%m-%d %H:%M:%S")
    tty = sys.stdout.isatty()
    c, r = (_colors[level], "\033[0m") if tty else ("", "")
    print(f"{c}[{ts}] [{_names[level]}] {msg}{r}", flush=True)


def debug(msg: str) -> None: _emit(DEBUG, msg)
def info(msg: str) -> None: _emit(INFO, msg)
def warning(msg: str) -> None: _emit(WARNING, msg)
def error(msg: str) -> None: _emit(ERROR, msg)


def verbose_line(device: str, kernel: str, m: int, n: int, k: int, ms: float) -> None:
    print(f"xft_verbose,exec,{device},api,{kernel},m{m}n{n}k{k},{ms:.6f}", flush=True)
