"""Exponential moving average of throughput (samples per second), with bias correction.

Used by the progress tracker and the optimizer to predict when the swarm reaches its target batch
(reference: hivemind/utils/performance_ema.py:7-70).
"""
from __future__ import annotations

import time
from contextlib import contextmanager
from threading import Lock


class PerformanceEMA:
    def __init__(self, alpha: float = 0.1, eps: float = 1e-20, paused: bool = False):
        self.alpha, self.eps = alpha, eps
        self.num_updates = 0
        self.ema_seconds_per_sample = 0.0
        self.samples_per_second = eps
        self.timestamp = time.perf_counter()
        self.paused = paused
        self.lock = Lock()

    def update(self, task_size: float, interval: float = None) -> float:
        """Register ``task_size`` samples done since the last update (or in ``interval`` seconds)."""
        assert task_size > 0, f"task size must be positive, got {task_size}"
        if not self.paused:
            self.timestamp, previous = time.perf_counter(), self.timestamp
            interval = interval if interval is not None else self.timestamp - previous
        else:
            assert interval is not None, "a paused EMA needs explicit intervals"
        self.ema_seconds_per_sample = self.alpha * interval / task_size + (1 - self.alpha) * self.ema_seconds_per_sample
        self.num_updates += 1
        correction = 1 - (1 - self.alpha) ** self.num_updates
        self.samples_per_second = 1 / max(self.ema_seconds_per_sample / correction, self.eps)
        return self.samples_per_second

    def reset_timer(self) -> None:
        self.timestamp = time.perf_counter()

    @contextmanager
    def pause(self):
        """Do not count the time spent inside the block."""
        self.paused, was = True, self.paused
        try:
            yield
        finally:
            self.paused = was
            self.reset_timer()

    @contextmanager
    def update_threadsafe(self, task_size: float):
        """Time the block and register it as one task; safe to enter from several threads."""
        start = time.perf_counter()
        yield
        with self.lock:
            self.update(task_size, interval=time.perf_counter() - max(start, self.timestamp))
            self.reset_timer()
