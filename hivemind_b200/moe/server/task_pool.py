"""``TaskPool``: gathers single requests for one expert function into batches for the ``Runtime``.

The reference forks one process per pool and ships batches through pipes and shared memory
(hivemind/moe/server/task_pool.py:25-256). Here a pool is a thread-safe queue inside the server process: connection
handlers call ``submit_task`` from their event loops and await the returned future; the ``Runtime`` thread asks the
pool with the oldest waiting task for a batch (``load_batch_to_runtime``), runs it on the device and hands the outputs
back (``send_outputs_from_runtime``), which resolves the futures row-slice by row-slice. Batching rules are the
reference's: at most ``max_batch_size`` rows per batch, tasks are never split, a batch is released only when at least
``min_batch_size`` rows are waiting (or ``timeout`` has passed since the oldest task arrived).
"""
from __future__ import annotations

import threading
import time
from abc import ABCMeta, abstractmethod
from collections import deque
from concurrent.futures import Future
from typing import Any, Callable, Deque, List, NamedTuple, Optional, Tuple

import torch

from hivemind_b200.utils import MPFuture, get_logger

logger = get_logger(__name__)


class Task(NamedTuple):
    future: MPFuture
    args: Tuple[torch.Tensor, ...]
    timestamp: float

    @property
    def size(self) -> int:
        return len(self.args[0]) if self.args else 0


class TaskPoolBase(metaclass=ABCMeta):
    """A source of batches for the Runtime; ``priority`` orders pools (smaller = more urgent)."""

    def __init__(self, process_func: Callable, daemon: bool = True, **kwargs):
        self.process_func = process_func
        self._priority = float("inf")

    @abstractmethod
    def submit_task(self, *args: torch.Tensor) -> Future:
        ...

    @abstractmethod
    def load_batch_to_runtime(self, timeout=None, device=None) -> Tuple[Any, List[torch.Tensor]]:
        ...

    @abstractmethod
    def send_outputs_from_runtime(self, uid: int, batch_outputs: List[torch.Tensor]):
        ...

    @property
    def priority(self) -> float:
        return self._priority

    @property
    @abstractmethod
    def empty(self) -> bool:
        ...


class TaskPool(TaskPoolBase):
    """
    :param process_func: ``(*batched inputs) -> batched outputs``, run by the Runtime
    :param max_batch_size: rows per batch (a single task may not exceed it)
    :param min_batch_size: do not release a batch with fewer rows, unless ``timeout`` ran out
    :param timeout: seconds after which waiting tasks are released regardless of ``min_batch_size``
    :param pool_size: kept for interface parity (the queue is unbounded)
    """

    def __init__(self, process_func: Callable, max_batch_size: int, name: str, min_batch_size: int = 1,
                 timeout: Optional[float] = None, pool_size: Optional[int] = None, prefetch_batches: int = 1,
                 daemon: bool = True, start: bool = False):
        super().__init__(process_func, daemon=daemon)
        self.name = name
        self.min_batch_size, self.max_batch_size, self.timeout = min_batch_size, max_batch_size, timeout
        self.prefetch_batches = prefetch_batches
        self._tasks: Deque[Task] = deque()
        self._queued_rows = 0
        self._lock = threading.Lock()
        self._in_flight = {}
        self._next_batch_id = 0
        self._listeners: List[threading.Condition] = []
        self._alive = True

    # the Runtime registers a condition variable that is notified whenever new work arrives
    def attach_listener(self, condition: threading.Condition) -> None:
        self._listeners.append(condition)

    def start(self) -> None:
        self._alive = True

    def run(self) -> None:  # interface parity: pools do not own threads here
        self._alive = True

    def is_alive(self) -> bool:
        return self._alive

    def shutdown(self, timeout: float = 3) -> None:
        self._alive = False
        with self._lock:
            tasks, self._tasks, self._queued_rows = list(self._tasks), deque(), 0
        for task in tasks:
            if not task.future.done():
                task.future.set_exception(RuntimeError(f"{self.name} was shut down"))

    def submit_task(self, *args: torch.Tensor) -> MPFuture:
        """Queue one request (tensors with a common first dimension); the future resolves to its outputs."""
        task = Task(MPFuture(), args, time.monotonic())
        if task.size > self.max_batch_size:
            exc = ValueError(f"Task size greater than max_batch_size ({self.max_batch_size}), it can't be processed")
            task.future.set_exception(exc)
            return task.future
        if not self._alive:
            task.future.set_exception(RuntimeError(f"{self.name} is not running"))
            return task.future
        with self._lock:
            self._tasks.append(task)
            self._queued_rows += task.size
            self._priority = self._tasks[0].timestamp
        for condition in self._listeners:
            with condition:
                condition.notify_all()
        return task.future

    @property
    def empty(self) -> bool:
        return not self._tasks

    @property
    def priority(self) -> float:
        """Arrival time of the oldest task that may be dispatched now; +inf if nothing is ready."""
        with self._lock:
            if not self._tasks:
                return float("inf")
            oldest = self._tasks[0].timestamp
            if self._queued_rows >= self.min_batch_size:
                return oldest
            if self.timeout is not None and time.monotonic() - oldest >= self.timeout:
                return oldest
            return float("inf")

    def next_ready_time(self) -> float:
        """When the oldest waiting task becomes dispatchable because of ``timeout`` (monotonic clock; inf if never)."""
        with self._lock:
            if not self._tasks or self.timeout is None:
                return float("inf")
            return self._tasks[0].timestamp + self.timeout

    def load_batch_to_runtime(self, timeout: Optional[float] = None, device: Optional[torch.device] = None
                              ) -> Tuple[Any, List[torch.Tensor]]:
        """Take as many whole tasks as fit into ``max_batch_size`` rows, concatenate them and move to ``device``."""
        with self._lock:
            batch_tasks: List[Task] = []
            rows = 0
            while self._tasks and rows + self._tasks[0].size <= self.max_batch_size:
                task = self._tasks.popleft()
                if task.future.cancelled():
                    self._queued_rows -= task.size
                    continue
                batch_tasks.append(task)
                rows += task.size
            self._queued_rows -= rows
            self._priority = self._tasks[0].timestamp if self._tasks else float("inf")
            batch_id = self._next_batch_id
            self._next_batch_id += 1
            self._in_flight[batch_id] = batch_tasks
        if not batch_tasks:
            return batch_id, []
        for task in batch_tasks:
            task.future.set_running_or_notify_cancel()
        num_inputs = len(batch_tasks[0].args)
        batch_inputs = []
        for i in range(num_inputs):
            parts = [task.args[i] for task in batch_tasks]
            to_cuda = device is not None and device.type == "cuda" and parts[0].device.type == "cpu"
            if len(parts) == 1:
                merged = parts[0].detach()
                if to_cuda and not merged.is_pinned():
                    merged = merged.pin_memory()
            elif to_cuda:  # concatenate straight into page-locked memory: one host copy instead of two
                merged = torch.empty((rows, *parts[0].shape[1:]), dtype=parts[0].dtype, pin_memory=True)
                torch.cat([p.detach() for p in parts], dim=0, out=merged)
            else:
                merged = torch.cat(parts, dim=0)
            if device is not None and merged.device != device:
                merged = merged.to(device, non_blocking=True)
            batch_inputs.append(merged)
        return batch_id, batch_inputs

    def send_outputs_from_runtime(self, uid: int, batch_outputs: List[torch.Tensor]) -> None:
        """Split the batched outputs by task and resolve the tasks' futures (with CPU tensors)."""
        batch_tasks = self._in_flight.pop(uid, [])
        sizes = [task.size for task in batch_tasks]
        outputs_cpu = [out.detach().to("cpu", non_blocking=False) if isinstance(out, torch.Tensor) else out
                       for out in batch_outputs]
        split = [out.split_with_sizes(sizes, dim=0) for out in outputs_cpu]
        for i, task in enumerate(batch_tasks):
            if not task.future.done():
                task.future.set_result(tuple(parts[i] for parts in split))

    def send_exception_from_runtime(self, uid: int, exception: BaseException) -> None:
        for task in self._in_flight.pop(uid, []):
            if not task.future.done():
                task.future.set_exception(exception)

    def get_task_size(self, task: Task) -> int:
        return task.size
