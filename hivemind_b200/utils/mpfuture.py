"""``MPFuture``: a future that can be completed from any thread and awaited from any event loop.

The reference runs the DHT, every averager and every MoE handler in forked processes and ships results through
shared memory and pipes (hivemind/utils/mpfuture.py:65-328). Forking does not mix with CUDA, so in this framework
those components are threads of one process per GPU and ``MPFuture`` is an in-process primitive with the same
interface: ``set_result`` / ``set_exception`` / ``cancel`` / ``result(timeout)`` / ``done`` / callbacks / ``await``.
"""
from __future__ import annotations

import asyncio
import concurrent.futures as base
import threading
from typing import Generic, Optional, TypeVar

ResultType = TypeVar("ResultType")

# the reference exposes these names on the module; keep them importable
InvalidStateError = base.InvalidStateError
CancelledError = base.CancelledError
TimeoutError = base.TimeoutError


class MPFuture(base.Future, Generic[ResultType]):
    """Thread-safe, awaitable future. Setting a result twice raises ``InvalidStateError`` as in the reference."""

    def __init__(self, *, use_lock: bool = True):
        super().__init__()
        self._state_lock = threading.RLock() if use_lock else None
        self._running = False

    # -- producer side -------------------------------------------------------------------------------------
    def set_result(self, result: ResultType) -> None:
        if self.done():
            raise InvalidStateError(f"cannot set_result: future is already {self._state}")
        super().set_result(result)

    def set_exception(self, exception: Optional[BaseException]) -> None:
        if self.done():
            raise InvalidStateError(f"cannot set_exception: future is already {self._state}")
        super().set_exception(exception)

    def set_running_or_notify_cancel(self) -> bool:
        if self.cancelled():
            return False
        if self.done():
            raise InvalidStateError(f"future is already {self._state}")
        if not self._running:
            self._running = True
            return super().set_running_or_notify_cancel()
        return True

    def cancel(self) -> bool:
        """Cancel unless finished. Unlike ``concurrent.futures``, a running future can be cancelled too."""
        with self._condition:
            if self._state in (base._base.FINISHED,):
                return False
            if self._state in (base._base.CANCELLED, base._base.CANCELLED_AND_NOTIFIED):
                return True
            self._state = base._base.CANCELLED
            self._condition.notify_all()
        self._invoke_callbacks()
        return True

    # -- consumer side -------------------------------------------------------------------------------------
    def __await__(self):
        loop = asyncio.get_event_loop()
        aio_future = loop.create_future()

        def _transfer(fut: "MPFuture"):
            def _apply():
                if aio_future.done():
                    return
                if fut.cancelled():
                    aio_future.cancel()
                elif fut.exception() is not None:
                    aio_future.set_exception(fut.exception())
                else:
                    aio_future.set_result(fut.result())

            try:
                loop.call_soon_threadsafe(_apply)
            except RuntimeError:
                pass  # the awaiting loop was closed in the meantime

        self.add_done_callback(_transfer)
        try:
            return (yield from aio_future.__await__())
        except asyncio.CancelledError:
            self.cancel()
            raise

    def __repr__(self) -> str:
        return f"<{type(self).__name__} at {hex(id(self))} state={self._state.lower()}>"

    @classmethod
    def reset_backend(cls) -> None:
        """Kept for interface parity with the reference's process-based backend; nothing to reset here."""
