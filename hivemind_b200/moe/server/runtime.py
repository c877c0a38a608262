"""``Runtime``: the one thread of a server that runs expert computations on the device.

It waits until some pool has a dispatchable batch, picks the pool whose oldest task has waited longest, runs the
pool's function on the batch and returns the outputs; an exception in one batch is delivered to that batch's
callers and the loop goes on (reference: hivemind/moe/server/runtime.py:22-199). An optional ``StatsReporter``
logs batches/s and examples/s per pool.
"""
from __future__ import annotations

import queue
import threading
import time
from collections import defaultdict
from typing import Dict, NamedTuple, Optional

import torch

from hivemind_b200.moe.server.module_backend import ModuleBackend
from hivemind_b200.utils import get_logger

logger = get_logger(__name__)


class Runtime(threading.Thread):
    """
    :param module_backends: experts served by this runtime, by uid
    :param prefetch_batches: kept for interface parity (batches are formed on demand here)
    :param device: where experts live; batches are moved there
    :param stats_report_interval: seconds between performance reports (None = off)
    """

    SHUTDOWN_TRIGGER = "RUNTIME SHUTDOWN TRIGGERED"

    def __init__(self, module_backends: Dict[str, ModuleBackend], prefetch_batches: int = 64, sender_threads: int = 1,
                 device: torch.device = None, stats_report_interval: Optional[int] = None):
        super().__init__(daemon=True, name="Runtime")
        self.module_backends = module_backends
        self.pools = tuple(pool for backend in module_backends.values() for pool in backend.get_pools())
        self.device = torch.device(device) if device is not None else None
        self.prefetch_batches = prefetch_batches
        self.shutdown_trigger = threading.Event()
        self.ready = threading.Event()
        self._work_available = threading.Condition()
        for pool in self.pools:
            pool.attach_listener(self._work_available)
        self.stats_report_interval = stats_report_interval
        self.stats_reporter = StatsReporter(stats_report_interval) if stats_report_interval is not None else None

    def run(self) -> None:
        for pool in self.pools:
            pool.start()
        if self.device is not None:
            if self.device.type == "cuda":
                if self.device.index is None:  # "cuda" means the current device; pools and tensors need an index
                    self.device = torch.device("cuda", torch.cuda.current_device())
                torch.cuda.set_device(self.device)
            for backend in self.module_backends.values():
                backend.module.to(self.device)
        if self.stats_reporter is not None:
            self.stats_reporter.start()
        use_cuda = self.device is not None and self.device.type == "cuda"
        sender = None
        if use_cuda:
            # three streams: inputs are uploaded while the previous batch computes, results are downloaded (and the
            # callers' futures resolved) by a helper thread while the next batch computes
            self._h2d_stream = torch.cuda.Stream(self.device)
            self._d2h_stream = torch.cuda.Stream(self.device)
            self._finished: "queue.Queue" = queue.Queue(maxsize=max(2, min(self.prefetch_batches, 8)))
            sender = threading.Thread(target=self._deliver_outputs, name="Runtime.sender", daemon=True)
            sender.start()
        self.ready.set()
        logger.info("Started")
        try:
            while not self.shutdown_trigger.is_set():
                pool = self._wait_for_ready_pool()
                if pool is None:
                    continue
                start = time.perf_counter()
                if use_cuda:
                    compute = torch.cuda.current_stream(self.device)
                    with torch.cuda.stream(self._h2d_stream):
                        batch_index, batch = pool.load_batch_to_runtime(device=self.device)
                    compute.wait_stream(self._h2d_stream)
                    for tensor in batch:
                        tensor.record_stream(compute)
                else:
                    batch_index, batch = pool.load_batch_to_runtime(device=self.device)
                if not batch:
                    continue
                try:
                    outputs = pool.process_func(*batch)
                    batch_size = outputs[0].size(0) if outputs else batch[0].size(0)
                    if use_cuda:
                        done = torch.cuda.Event()
                        done.record(torch.cuda.current_stream(self.device))
                        self._finished.put((pool, batch_index, list(outputs), done, batch_size, start))
                    else:
                        pool.send_outputs_from_runtime(batch_index, list(outputs))
                        if self.stats_reporter is not None:
                            self.stats_reporter.report_stats(pool.name, batch_size, time.perf_counter() - start)
                except KeyboardInterrupt:
                    raise
                except BaseException as exception:
                    logger.exception(f"Caught {exception!r}, attempting to recover")
                    pool.send_exception_from_runtime(batch_index, exception)
        finally:
            if sender is not None:
                self._finished.put(None)
                sender.join(timeout=10)
            if not self.shutdown_trigger.is_set():
                self.shutdown()

    def _deliver_outputs(self) -> None:
        """Helper thread of a CUDA runtime: wait for a batch, copy its outputs to page-locked memory, resolve futures."""
        torch.cuda.set_device(self.device)
        while True:
            item = self._finished.get()
            if item is None:
                return
            pool, batch_index, outputs, done, batch_size, start = item
            try:
                done.synchronize()
                with torch.cuda.stream(self._d2h_stream):
                    host = []
                    for out in outputs:
                        if isinstance(out, torch.Tensor) and out.is_cuda:
                            page_locked = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
                            page_locked.copy_(out.detach(), non_blocking=True)
                            host.append(page_locked)
                        else:
                            host.append(out)
                self._d2h_stream.synchronize()
                pool.send_outputs_from_runtime(batch_index, host)
                if self.stats_reporter is not None:
                    self.stats_reporter.report_stats(pool.name, batch_size, time.perf_counter() - start)
            except BaseException as exception:
                logger.exception(f"Caught {exception!r} while returning outputs")
                pool.send_exception_from_runtime(batch_index, exception)

    def _wait_for_ready_pool(self):
        """Block until a pool has a batch to run (or a batching timeout is about to make one ready)."""
        with self._work_available:
            while not self.shutdown_trigger.is_set():
                best, best_priority = None, float("inf")
                for pool in self.pools:
                    priority = pool.priority
                    if priority < best_priority:
                        best, best_priority = pool, priority
                if best is not None:
                    return best
                wake = min((pool.next_ready_time() for pool in self.pools), default=float("inf"))
                wait = 0.5 if wake == float("inf") else max(0.0, min(0.5, wake - time.monotonic()))
                self._work_available.wait(wait)
        return None

    def shutdown(self) -> None:
        """Stop the loop; pending tasks are failed by their pools."""
        logger.info("Shutting down")
        self.ready.clear()
        if self.stats_reporter is not None:
            self.stats_reporter.stop.set()
        self.shutdown_trigger.set()
        with self._work_available:
            self._work_available.notify_all()
        for pool in self.pools:
            pool.shutdown()


class BatchStats(NamedTuple):
    batch_size: int
    processing_time: float


class StatsReporter(threading.Thread):
    """Periodically logs, for each pool, how many batches and examples it processed and how fast."""

    def __init__(self, report_interval: int):
        super().__init__(daemon=True)
        self.report_interval = report_interval
        self.stop = threading.Event()
        self._lock = threading.Lock()
        self._stats = defaultdict(list)

    def run(self) -> None:
        while not self.stop.wait(self.report_interval):
            with self._lock:
                stats, self._stats = self._stats, defaultdict(list)
            for pool_uid, batches in stats.items():
                total_examples = sum(b.batch_size for b in batches)
                total_time = sum(b.processing_time for b in batches)
                logger.info(f"{pool_uid}: {len(batches)} batches ({len(batches) / max(total_time, 1e-9):.2f} batches/s), "
                            f"{total_examples} examples ({total_examples / max(total_time, 1e-9):.2f} examples/s), "
                            f"avg batch size {total_examples / max(len(batches), 1):.2f}")

    def report_stats(self, pool_uid: str, batch_size: int, processing_time: float) -> None:
        with self._lock:
            self._stats[pool_uid].append(BatchStats(batch_size, processing_time))
