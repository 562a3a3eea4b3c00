"""Opt-in timing log, counters and profiler ranges.

The reference logs every stage of every collective to a file unconditionally
(``python/bitscom/api.py:25-58``, ``cpp/src/process_group_lowbit.cc:74-91``).  Here the
log is off unless ``BITSCOM_TIMING=1``; ranges are always emitted as
``torch.profiler.record_function`` (free when no profiler is attached) and as NVTX
ranges when ``BITSCOM_NVTX=1``.  Counters are plain Python integers that a trainer can
read at any time through :func:`counters`.
"""

from __future__ import annotations

import contextlib
import os
import threading
import time
from collections import defaultdict
from typing import Dict, Iterator

import torch

_lock = threading.Lock()
_counters: Dict[str, float] = defaultdict(float)
_TRUE = {"1", "true", "yes", "on"}


def _flag(name: str) -> bool:
    return os.environ.get(name, "0").strip().lower() in _TRUE


def timing_enabled() -> bool:
    return _flag("BITSCOM_TIMING")


def log_dir() -> str:
    root = os.environ.get("BITSCOM_TIMING_DIR") or os.path.join(os.getcwd(), "debug_logs", "timing")
    os.makedirs(root, exist_ok=True)
    return root


def _rank() -> int:
    try:
        import torch.distributed as dist

        return dist.get_rank() if dist.is_initialized() else -1
    except Exception:
        return -1


def log(message: str) -> None:
    if not timing_enabled():
        return
    rank = _rank()
    line = f"[bitscom-timing rank={rank} t={time.time():.6f}] {message}\n"
    with _lock, open(os.path.join(log_dir(), f"bitscom_rank{rank}.log"), "a",
                     encoding="utf-8") as f:
        f.write(line)


def add(name: str, value: float = 1.0) -> None:
    with _lock:
        _counters[name] += value


def counters() -> Dict[str, float]:
    with _lock:
        return dict(_counters)


def reset_counters() -> None:
    with _lock:
        _counters.clear()


@contextlib.contextmanager
def span(name: str) -> Iterator[None]:
    """Named host-side range: profiler range, optional NVTX range, optional log line."""
    nvtx = _flag("BITSCOM_NVTX") and torch.cuda.is_available()
    t0 = time.perf_counter()
    if nvtx:
        torch.cuda.nvtx.range_push(f"bitscom:{name}")
    try:
        with torch.profiler.record_function(f"bitscom:{name}"):
            yield
    finally:
        if nvtx:
            torch.cuda.nvtx.range_pop()
        if timing_enabled():
            log(f"{name} elapsed_ms={(time.perf_counter() - t0) * 1e3:.3f}")


class DeviceTimer:
    """CUDA-event stopwatch for phases enqueued on one stream."""

    def __init__(self):
        self._pairs = []

    @contextlib.contextmanager
    def measure(self, name: str, stream=None):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        try:
            yield
        finally:
            b.record(stream)
            self._pairs.append((name, a, b))

    def results_ms(self) -> Dict[str, float]:
        out: Dict[str, float] = defaultdict(float)
        for name, a, b in self._pairs:
            b.synchronize()
            out[name] += a.elapsed_time(b)
        return dict(out)
