"""One background event loop per process for all client-side expert calls.

``RemoteExpert.forward`` is a blocking autograd function, but the RPCs behind it are coroutines; this helper owns
a daemon loop thread, started lazily and re-created after ``fork`` (reference:
hivemind/moe/client/remote_expert_worker.py:11-36).
"""
from __future__ import annotations

import os
import threading
from concurrent.futures import Future
from typing import Awaitable, Optional

from hivemind_b200.utils.asyncio import LoopThread


class RemoteExpertWorker:
    _lock = threading.Lock()
    _worker: Optional[LoopThread] = None
    _pid: Optional[int] = None

    @classmethod
    def _ensure_started(cls) -> LoopThread:
        with cls._lock:
            if cls._worker is None or cls._pid != os.getpid() or not cls._worker.is_alive:
                cls._worker = LoopThread("RemoteExpertWorker").start()
                cls._pid = os.getpid()
            return cls._worker

    @classmethod
    def run_coroutine(cls, coro: Awaitable, return_future: bool = False):
        """Run ``coro`` on the shared loop; block for the result unless ``return_future``."""
        future: Future = cls._ensure_started().submit(coro)
        return future if return_future else future.result()
