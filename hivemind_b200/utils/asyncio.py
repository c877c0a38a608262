"""asyncio helpers used across the control plane (same names as hivemind/utils/asyncio.py:16-210)."""
from __future__ import annotations

import asyncio
import concurrent.futures
import os
import threading
from concurrent.futures import ThreadPoolExecutor
from contextlib import AbstractAsyncContextManager, AbstractContextManager
from typing import AsyncIterable, AsyncIterator, Awaitable, Callable, Coroutine, Iterable, Optional, Tuple, TypeVar

from hivemind_b200.utils.logging import get_logger

try:
    import uvloop
except ImportError:  # pragma: no cover
    uvloop = None

T = TypeVar("T")
logger = get_logger(__name__)


def new_event_loop() -> asyncio.AbstractEventLoop:
    """
    A fresh event loop that is not yet bound to any thread.

    Components are threads of one process here, each with its own loop. uvloop finalises its handles in whichever
    thread happens to run the garbage collector, which is not safe while the handle's own loop is running in
    another thread, so the default is the standard library's loop. ``HIVEMIND_B200_UVLOOP=1`` opts into uvloop
    (about 20 % more RPC throughput) for processes that accept that risk, e.g. benchmark clients.
    """
    if uvloop is not None and os.getenv("HIVEMIND_B200_UVLOOP", "0") == "1":
        return uvloop.new_event_loop()
    return asyncio.new_event_loop()


def switch_to_uvloop() -> asyncio.AbstractEventLoop:
    """Create a new loop, make it current for this thread and return it."""
    loop = new_event_loop()
    asyncio.set_event_loop(loop)
    return loop


class LoopThread:
    """A daemon thread that owns one event loop; the home of a component that the reference ran as a process."""

    def __init__(self, name: str):
        self.name = name
        self.loop: Optional[asyncio.AbstractEventLoop] = None
        self._thread: Optional[threading.Thread] = None
        self._started = threading.Event()
        self._outstanding: set = set()  # strong references to submitted work, see submit()

    def start(self) -> "LoopThread":
        if self._thread is not None:
            return self
        self._thread = threading.Thread(target=self._main, name=self.name, daemon=True)
        self._thread.start()
        self._started.wait()
        return self

    def _main(self) -> None:
        self.loop = switch_to_uvloop()
        self.loop.call_soon(self._started.set)
        try:
            self.loop.run_forever()
        finally:
            try:
                pending = [t for t in asyncio.all_tasks(self.loop) if not t.done()]
                for t in pending:
                    t.cancel()
                if pending:
                    self.loop.run_until_complete(asyncio.gather(*pending, return_exceptions=True))
                self.loop.run_until_complete(self.loop.shutdown_asyncgens())
            except Exception:
                pass
            # the loop object is deliberately not closed: late call_soon_threadsafe calls from other threads
            # (future callbacks, destructors) must find a stopped loop, not a freed one

    @property
    def is_alive(self) -> bool:
        return self._thread is not None and self._thread.is_alive()

    def submit(self, coro: Coroutine) -> concurrent.futures.Future:
        """Schedule ``coro`` on the loop; returns a ``concurrent.futures.Future``."""
        assert self.loop is not None, "loop thread is not running"
        future = asyncio.run_coroutine_threadsafe(coro, self.loop)
        # The event loop keeps only weak references to its tasks. A caller that drops the returned future leaves
        # the task reachable only through whatever it is awaiting; if that is itself reachable only from the task
        # (objects created inside the coroutine), the garbage collector destroys the pending task in mid-flight.
        # Holding the future here keeps the task alive until it is done.
        self._outstanding.add(future)
        future.add_done_callback(self._outstanding.discard)
        return future

    def run(self, coro: Coroutine, timeout: Optional[float] = None):
        """Run ``coro`` on the loop and wait for its result from a foreign thread."""
        if threading.current_thread() is self._thread:
            raise RuntimeError("LoopThread.run called from its own loop thread: await the coroutine instead")
        return self.submit(coro).result(timeout)

    def stop(self, join_timeout: float = 5.0) -> None:
        if self.loop is not None and self._thread is not None and self._thread.is_alive():
            self.loop.call_soon_threadsafe(self.loop.stop)
            if threading.current_thread() is not self._thread:
                self._thread.join(join_timeout)
        self._thread = None


_background_tasks: set = set()


def spawn(coro: Coroutine) -> "asyncio.Task":
    """``asyncio.create_task`` for work whose result nobody awaits: the task is kept alive until it is done (the
    event loop itself only holds weak references to its tasks)."""
    task = asyncio.create_task(coro)
    _background_tasks.add(task)
    task.add_done_callback(_background_tasks.discard)
    return task


async def anext(aiter: AsyncIterator[T]) -> T:
    return await aiter.__anext__()


async def iter_as_aiter(iterable: Iterable[T]) -> AsyncIterator[T]:
    for elem in iterable:
        yield elem


async def as_aiter(*args: T) -> AsyncIterator[T]:
    for arg in args:
        yield arg


async def azip(*iterables: AsyncIterable[T]) -> AsyncIterator[Tuple[T, ...]]:
    iterators = [it.__aiter__() for it in iterables]
    while True:
        try:
            yield tuple(await asyncio.gather(*(it.__anext__() for it in iterators)))
        except StopAsyncIteration:
            break


async def achain(*async_iters: AsyncIterable[T]) -> AsyncIterator[T]:
    for aiter in async_iters:
        async for elem in aiter:
            yield elem


async def aenumerate(aiterable: AsyncIterable[T]) -> AsyncIterator[Tuple[int, T]]:
    index = 0
    async for elem in aiterable:
        yield index, elem
        index += 1


async def asingle(aiter: AsyncIterable[T]) -> T:
    """The only item of an async iterable; ValueError if there are none or several."""
    count, result = 0, None
    async for item in aiter:
        count += 1
        if count > 1:
            raise ValueError("asingle() expected an iterable with exactly one item, but got two or more items")
        result = item
    if count == 0:
        raise ValueError("asingle() expected an iterable with exactly one item, but got an empty iterable")
    return result


async def await_cancelled(awaitable: Awaitable) -> bool:
    try:
        await awaitable
        return False
    except (asyncio.CancelledError, concurrent.futures.CancelledError):
        return True
    except BaseException:
        logger.exception(f"exception while waiting for a cancelled {awaitable}")
        return False


async def cancel_and_wait(awaitable: Awaitable) -> bool:
    """Cancel a task/future and wait until it has really finished; True if it ended cancelled."""
    awaitable.cancel()
    return await await_cancelled(awaitable)


async def amap_in_executor(func: Callable[..., T], *iterables: AsyncIterable, max_prefetch: int = 1,
                           executor: Optional[ThreadPoolExecutor] = None,
                           inline: Optional[Callable[..., bool]] = None) -> AsyncIterator[T]:
    """Map ``func`` over async iterables in a thread pool, keeping at most ``max_prefetch`` results in flight.

    :param inline: if given and ``inline(*args)`` is true, ``func(*args)`` runs in the event loop itself: handing an
      item to a thread and waking the loop again costs more than, say, viewing half a megabyte as a tensor
    """
    assert max_prefetch > 0, "max_prefetch must be positive"
    loop = asyncio.get_event_loop()
    queue: asyncio.Queue = asyncio.Queue(max_prefetch)

    def _computed_here(args) -> asyncio.Future:
        done = loop.create_future()
        try:
            done.set_result(func(*args))
        except Exception as e:
            done.set_exception(e)
        return done

    async def _produce():
        try:
            async for args in azip(*iterables):
                if inline is not None and inline(*args):
                    await queue.put(_computed_here(args))
                else:
                    await queue.put(loop.run_in_executor(executor, func, *args))
            await queue.put(None)
        except asyncio.CancelledError:
            raise  # the consumer is gone (it cancels the producer on its way out): nobody is left to tell
        except BaseException as e:
            # an error of the source belongs to the consumer: it travels through the queue as a failed future and is
            # raised where the consumer awaits it. The producer itself ends quietly.
            failed = loop.create_future()
            failed.set_exception(e)
            try:
                await queue.put(failed)
            except BaseException:
                failed.exception()  # undeliverable: mark it as seen, so that the loop does not report it at collection
                raise

    producer = asyncio.create_task(_produce())
    try:
        while True:
            fut = await queue.get()
            if fut is None:
                break
            yield await fut
    finally:
        await cancel_and_wait(producer)
        while not queue.empty():
            fut = queue.get_nowait()
            if fut is not None:
                fut.cancel() if not fut.done() else fut.exception() if not fut.cancelled() else None


async def aiter_with_timeout(iterable: AsyncIterable[T], timeout: Optional[float]) -> AsyncIterator[T]:
    """Iterate, raising ``asyncio.TimeoutError`` if the next item takes longer than ``timeout`` seconds."""
    iterator = iterable.__aiter__()
    while True:
        try:
            yield await asyncio.wait_for(iterator.__anext__(), timeout=timeout)
        except StopAsyncIteration:
            break


async def attach_event_on_finished(iterable: AsyncIterable[T], event: asyncio.Event) -> AsyncIterator[T]:
    """Iterate and set ``event`` when iteration ends for any reason."""
    try:
        async for item in iterable:
            yield item
    finally:
        event.set()


class _AsyncContextWrapper(AbstractAsyncContextManager):
    """Enter a blocking context manager in a worker thread so that the event loop stays responsive."""

    # every coroutine that waits for a blocking context holds one worker thread, and a waiter that never gets a thread
    # can never be woken; the pool therefore has to be far larger than the default (cpu count + 4)
    MAX_WAITERS = 4096
    EXECUTOR_PID = None
    CONTEXT_EXECUTOR = None
    EXECUTOR_LOCK = threading.Lock()

    def __init__(self, context: AbstractContextManager):
        self._context = context

    @classmethod
    def get_process_wide_executor(cls) -> ThreadPoolExecutor:
        if os.getpid() != cls.EXECUTOR_PID:
            with cls.EXECUTOR_LOCK:
                if os.getpid() != cls.EXECUTOR_PID:
                    cls.CONTEXT_EXECUTOR = ThreadPoolExecutor(max_workers=cls.MAX_WAITERS)
                    cls.EXECUTOR_PID = os.getpid()
        return cls.CONTEXT_EXECUTOR

    async def __aenter__(self):
        loop = asyncio.get_event_loop()
        return await loop.run_in_executor(self.get_process_wide_executor(), self._context.__enter__)

    async def __aexit__(self, exc_type, exc_value, traceback):
        return self._context.__exit__(exc_type, exc_value, traceback)


def enter_asynchronously(context: AbstractContextManager) -> AbstractAsyncContextManager:
    """``async with enter_asynchronously(lock):`` acquires a threading lock without blocking the loop."""
    return _AsyncContextWrapper(context)


def cancel_task_if_running(task: Optional[asyncio.Task]) -> None:
    if task is not None and not task.done():
        task.get_loop().call_soon_threadsafe(task.cancel)
