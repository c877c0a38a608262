"""Lightweight tracing: NVTX ranges and CUDA-event timers around the framework's device stages.

The reference has no tracing beyond samples-per-second estimates and the server's ``StatsReporter``
(hivemind/utils/performance_ema.py:7-70, hivemind/moe/server/runtime.py:161-199). Here every device stage of a round
(butterfly send / reduce / apply, expert dispatch / FFN / combine, multi-tensor optimizer and gradient kernels,
PowerSGD compress / orthogonalise / reconstruct) can be wrapped in
``device_range(name)``: with ``HIVEMIND_B200_NVTX=1`` it pushes an NVTX range (visible in profiler timelines); with
``HIVEMIND_B200_TIMING=1`` it also brackets the stage with CUDA events on the current stream and accumulates the
elapsed device time per name, readable with ``timing_summary()``. With neither variable set the context manager
costs one dictionary lookup.
"""
from __future__ import annotations

import contextlib
import functools
import os
import threading
from collections import defaultdict
from typing import Dict, List, Optional, Tuple

import torch

_NVTX = os.environ.get("HIVEMIND_B200_NVTX", "0") == "1"
_TIMING = os.environ.get("HIVEMIND_B200_TIMING", "0") == "1"
_lock = threading.Lock()
_pending: List[Tuple[str, "torch.cuda.Event", "torch.cuda.Event"]] = []
_totals: Dict[str, List[float]] = defaultdict(lambda: [0, 0.0])  # name -> [count, milliseconds]


def enable(nvtx: Optional[bool] = None, timing: Optional[bool] = None) -> None:
    """Switch tracing on or off at run time (overrides the environment variables)."""
    global _NVTX, _TIMING
    if nvtx is not None:
        _NVTX = bool(nvtx)
    if timing is not None:
        _TIMING = bool(timing)


@contextlib.contextmanager
def device_range(name: str, stream: Optional["torch.cuda.Stream"] = None):
    """Mark a stage of device work; see the module docstring for what is recorded."""
    if not (_NVTX or _TIMING) or not torch.cuda.is_available():
        yield
        return
    if _NVTX:
        torch.cuda.nvtx.range_push(name)
    events = None
    if _TIMING:
        stream = stream if stream is not None else torch.cuda.current_stream()
        events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        events[0].record(stream)
    try:
        yield
    finally:
        if events is not None:
            events[1].record(stream)
            with _lock:
                _pending.append((name, events[0], events[1]))
        if _NVTX:
            torch.cuda.nvtx.range_pop()


def traced(name: str):
    """Decorator form of ``device_range`` for functions that enqueue one stage of device work."""

    def wrap(fn):
        @functools.wraps(fn)
        def inner(*args, **kwargs):
            if not (_NVTX or _TIMING):
                return fn(*args, **kwargs)
            with device_range(name):
                return fn(*args, **kwargs)

        return inner

    return wrap


def _collect(wait: bool) -> None:
    with _lock:
        remaining = []
        for name, start, stop in _pending:
            if wait:
                stop.synchronize()
            if stop.query():
                entry = _totals[name]
                entry[0] += 1
                entry[1] += start.elapsed_time(stop)
            else:
                remaining.append((name, start, stop))
        _pending[:] = remaining


def timing_summary(wait: bool = True, reset: bool = False) -> Dict[str, Dict[str, float]]:
    """Device time per stage name: ``{name: {"count": n, "total_ms": t, "mean_ms": t / n}}``."""
    _collect(wait)
    with _lock:
        summary = {name: {"count": count, "total_ms": ms, "mean_ms": ms / max(count, 1)}
                   for name, (count, ms) in _totals.items()}
        if reset:
            _totals.clear()
    return summary
