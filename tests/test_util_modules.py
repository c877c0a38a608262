"""Runtime utilities: futures, serializer, nested structures, asyncio helpers, timed storage, EMA, descriptors,
multiaddr (modelled on the reference's tests/test_util_modules.py and tests/test_multiaddr.py)."""
import asyncio
import concurrent.futures
import os
import threading
import time

import pytest
import torch

from hivemind_b200.utils import (BatchTensorDescriptor, MPFuture, MSGPackSerializer, PerformanceEMA, TensorDescriptor,
                                 TimedStorage, ValueWithExpiration, get_dht_time, nested_compare, nested_flatten,
                                 nested_map, nested_pack)
from hivemind_b200.utils.asyncio import (LoopThread, achain, aenumerate, aiter_with_timeout, amap_in_executor, anext,
                                         as_aiter, asingle, attach_event_on_finished, azip, cancel_and_wait,
                                         enter_asynchronously)
from hivemind_b200.utils.multiaddr import Multiaddr
from hivemind_b200.proto.runtime_pb2 import CompressionType


def test_mpfuture_result_exception_cancel_and_callbacks():
    future = MPFuture()
    seen = []
    future.add_done_callback(lambda f: seen.append(f.result()))
    threading.Timer(0.05, lambda: future.set_result(123)).start()
    assert future.result(timeout=2) == 123 and future.done() and not future.cancelled()
    time.sleep(0.05)
    assert seen == [123]
    with pytest.raises(concurrent.futures.InvalidStateError):
        future.set_result(5)

    failing = MPFuture()
    failing.set_exception(ValueError("boom"))
    with pytest.raises(ValueError):
        failing.result()
    assert isinstance(failing.exception(), ValueError)

    cancelled = MPFuture()
    assert cancelled.cancel() and cancelled.cancelled() and cancelled.done()
    with pytest.raises(concurrent.futures.CancelledError):
        cancelled.result()
    assert not cancelled.set_running_or_notify_cancel()

    pending = MPFuture()
    with pytest.raises(concurrent.futures.TimeoutError):
        pending.result(timeout=0.05)
    assert pending.set_running_or_notify_cancel() and pending.running()
    assert pending.cancel() and pending.cancelled()  # unlike concurrent.futures, a running future can still be cancelled


def test_mpfuture_is_awaitable_from_other_loops():
    future = MPFuture()

    async def waiter():
        return await future

    worker = LoopThread("test-waiter").start()
    try:
        pending = worker.submit(waiter())
        time.sleep(0.05)
        assert not pending.done()
        future.set_result("done")
        assert pending.result(2) == "done"
        failed = MPFuture()
        pending = worker.submit(asyncio.wait_for(_await(failed), 2))
        failed.set_exception(KeyError("k"))
        with pytest.raises(KeyError):
            pending.result(2)
    finally:
        worker.stop()


async def _await(future):
    return await future


def test_serializer_round_trips_and_extensions():
    for value in (1, 1.5, "text", b"bytes", None, True, [1, "a", None], (1, (2, 3)), {"k": (1, 2), 5: [b"x"]}):
        assert MSGPackSerializer.loads(MSGPackSerializer.dumps(value)) == value
    restored = MSGPackSerializer.loads(MSGPackSerializer.dumps((1, [2, (3,)])))
    assert isinstance(restored, tuple) and isinstance(restored[1][1], tuple)  # tuples survive (ext type 0x40)

    @MSGPackSerializer.ext_serializable(0x3F)
    class Pair:
        def __init__(self, a, b):
            self.a, self.b = a, b

        def packb(self) -> bytes:
            return MSGPackSerializer.dumps([self.a, self.b])

        @classmethod
        def unpackb(cls, raw: bytes):
            return cls(*MSGPackSerializer.loads(raw))

    nested = MSGPackSerializer.loads(MSGPackSerializer.dumps({"p": Pair(1, (2, 3))}))
    assert isinstance(nested["p"], Pair) and nested["p"].b == (2, 3)
    descr = BatchTensorDescriptor(3, 4, dtype=torch.float16, compression=CompressionType.FLOAT16)
    back = MSGPackSerializer.loads(MSGPackSerializer.dumps(descr))
    assert isinstance(back, BatchTensorDescriptor) and back.dtype == torch.float16 and back.compression == CompressionType.FLOAT16


def test_nested_structures():
    structure = {"b": [1, (2, 3)], "a": 4, "c": {"z": 5, "y": 6}}
    flat = list(nested_flatten(structure))
    assert flat == [4, 1, 2, 3, 6, 5]  # dictionaries are walked in sorted key order
    assert nested_pack(flat, structure) == structure
    assert nested_map(lambda v: v * 10, structure)["b"][1] == (20, 30)
    assert nested_compare(structure, nested_map(str, structure))
    assert not nested_compare(structure, {"b": [1, (2,)], "a": 4, "c": {"z": 5, "y": 6}})
    assert not nested_compare((1, 2), [1, 2])
    summed = nested_map(lambda x, y: x + y, (1, {"k": 2}), (10, {"k": 20}))
    assert summed == (11, {"k": 22})


def test_tensor_descriptors():
    tensor = torch.randn(5, 7, dtype=torch.float64, requires_grad=True)
    descr = TensorDescriptor.from_tensor(tensor)
    assert descr.shape == (5, 7) and descr.dtype == torch.float64 and descr.requires_grad and descr.numel() == 35
    zeros = descr.make_zeros()
    assert zeros.shape == (5, 7) and zeros.dtype == torch.float64 and not zeros.any()
    batch = BatchTensorDescriptor.from_tensor(torch.zeros(9, 3, 2), compression=CompressionType.UNIFORM_8BIT)
    assert batch.shape[0] is None and tuple(batch.shape[1:]) == (3, 2)
    made = batch.make_zeros(4)
    assert made.shape == (4, 3, 2)
    assert batch.make_zeros(2, 6).shape == (2, 6, 3, 2)


def test_asyncio_helpers():
    async def scenario():
        assert [x async for x in as_aiter(1, 2, 3)] == [1, 2, 3]
        assert [x async for x in azip(as_aiter(1, 2, 3), as_aiter("a", "b"))] == [(1, "a"), (2, "b")]
        assert [x async for x in achain(as_aiter(1), as_aiter(2, 3))] == [1, 2, 3]
        assert [x async for x in aenumerate(as_aiter("x", "y"))] == [(0, "x"), (1, "y")]
        assert await asingle(as_aiter(7)) == 7
        with pytest.raises(ValueError):
            await asingle(as_aiter(1, 2))
        with pytest.raises(ValueError):
            await asingle(as_aiter())
        it = as_aiter(1, 2).__aiter__()
        assert await anext(it) == 1 and await anext(it) == 2
        squares = [x async for x in amap_in_executor(lambda v: v * v, as_aiter(*range(20)), max_prefetch=3)]
        assert squares == [v * v for v in range(20)]
        pairs = [x async for x in amap_in_executor(lambda a, b: a + b, as_aiter(1, 2), as_aiter(10, 20))]
        assert pairs == [11, 22]

        async def slow():
            yield 1
            await asyncio.sleep(1.0)
            yield 2

        with pytest.raises(asyncio.TimeoutError):
            [x async for x in aiter_with_timeout(slow(), timeout=0.1)]
        finished = asyncio.Event()
        assert [x async for x in attach_event_on_finished(as_aiter(1, 2), finished)] == [1, 2] and finished.is_set()

        sleeper = asyncio.create_task(asyncio.sleep(10))
        assert await cancel_and_wait(sleeper) and sleeper.cancelled()
        done = asyncio.create_task(asyncio.sleep(0))
        await done
        assert not await cancel_and_wait(done)

        lock = threading.Lock()
        async with enter_asynchronously(lock):
            assert lock.locked()
        assert not lock.locked()

    asyncio.new_event_loop().run_until_complete(scenario())


def test_enter_asynchronously_survives_a_flood_of_waiters():
    """Far more coroutines than a default thread pool has workers queue on two locks taken in nested order; with too
    few worker threads the holder of the first lock could never get a thread for the second and all would stall
    (the case of hivemind tests/test_util_modules.py::test_async_context_flooding)."""
    outer, inner = threading.Lock(), threading.Lock()
    entered = []

    async def visitor(index):
        async with enter_asynchronously(outer):
            await asyncio.sleep(0)
            async with enter_asynchronously(inner):
                assert outer.locked() and inner.locked()
                entered.append(index)
                await asyncio.sleep(0)

    async def scenario():
        n_visitors = 8 * (os.cpu_count() or 1) + 200
        ticks = 0

        async def heartbeat():
            nonlocal ticks
            while True:
                ticks += 1
                await asyncio.sleep(0.005)

        beat = asyncio.create_task(heartbeat())
        await asyncio.wait_for(asyncio.gather(*(visitor(i) for i in range(n_visitors))), timeout=60)
        beat.cancel()
        assert sorted(entered) == list(range(n_visitors))
        assert ticks > 1, "the event loop was blocked while the visitors waited for the locks"
        assert not outer.locked() and not inner.locked()

    asyncio.new_event_loop().run_until_complete(scenario())


def test_timed_storage_expiration_order_and_freeze():
    storage = TimedStorage(maxsize=3)
    now = get_dht_time()
    assert storage.store("a", 1, now + 0.2) and storage.store("b", 2, now + 10)
    assert not storage.store("b", 0, now + 5)  # an older expiration never replaces a newer one
    assert storage.get("b") == ValueWithExpiration(2, now + 10)
    storage.store("c", 3, now + 20)
    storage.store("d", 4, now + 30)  # over maxsize: the entry that expires first goes
    assert "a" not in storage and len(storage) == 3
    assert storage.top()[0] == "b"
    short = TimedStorage()
    short.store("x", 1, get_dht_time() + 0.1)
    with short.freeze():
        time.sleep(0.15)
        assert "x" in short  # frozen storages do not drop expired entries
    assert "x" not in short


def test_performance_ema():
    ema = PerformanceEMA(alpha=0.5)
    ema.update(100, interval=1.0)
    assert abs(ema.samples_per_second - 100) < 1e-6  # the first update is not biased towards zero
    ema.update(300, interval=1.0)
    assert 100 < ema.samples_per_second < 300
    paused = PerformanceEMA(alpha=0.5, paused=True)
    with paused.pause():
        pass
    before = paused.samples_per_second
    with paused.update_threadsafe(10):
        time.sleep(0.01)
    assert paused.samples_per_second != before or paused.samples_per_second > 0


def test_multiaddr_text_binary_and_manipulation():
    text = "/ip4/127.0.0.1/tcp/31337/p2p/QmYyQSo1c1Ym7orWxLYvCrM2EmxFTANf8wXmmE7DWjhx5N"
    addr = Multiaddr(text)
    assert str(addr) == text and Multiaddr(addr.to_bytes()) == addr and Multiaddr(bytes(addr)) == addr
    assert addr["ip4"] == "127.0.0.1" and addr["tcp"] == "31337" and "p2p" in addr and "udp" not in addr
    assert [p.name for p in addr.protocols()] == ["ip4", "tcp", "p2p"]
    assert addr.value_for_protocol("p2p").startswith("Qm")
    transport = addr.decapsulate("/p2p/QmYyQSo1c1Ym7orWxLYvCrM2EmxFTANf8wXmmE7DWjhx5N")
    assert str(transport) == "/ip4/127.0.0.1/tcp/31337"
    assert transport.encapsulate("/p2p/QmYyQSo1c1Ym7orWxLYvCrM2EmxFTANf8wXmmE7DWjhx5N") == addr
    assert [str(part) for part in addr.split()][:2] == ["/ip4/127.0.0.1", "/tcp/31337"]
    assert Multiaddr.join("/ip4/10.0.0.1", "/tcp/80") == Multiaddr("/ip4/10.0.0.1/tcp/80")
    assert {Multiaddr("/ip4/1.2.3.4/tcp/5"): 1}[Multiaddr("/ip4/1.2.3.4/tcp/5")] == 1
    unix = Multiaddr("/unix/tmp/hivemind.sock")
    assert unix["unix"].endswith("tmp/hivemind.sock") and Multiaddr(unix.to_bytes()) == unix
    six = Multiaddr("/ip6/::1/tcp/4001")
    assert Multiaddr(six.to_bytes()) == six
    for bad in ("ip4/1.2.3.4", "/ip4/999.1.1.1/tcp/1", "/tcp/70000", "/nosuchproto/1", "/ip4"):
        with pytest.raises(Exception):
            Multiaddr(bad)


def test_device_range_is_a_no_op_without_a_gpu_or_when_disabled():
    from hivemind_b200.utils import profiling

    profiling.enable(nvtx=False, timing=False)
    with profiling.device_range("anything"):
        pass
    assert "anything" not in profiling.timing_summary()

    @profiling.traced("stage.name")
    def add(a, b=1):
        """doc"""
        return a + b

    assert add(2, b=3) == 5 and add.__name__ == "add" and add.__doc__ == "doc"
    profiling.enable(timing=True)  # without a GPU the range stays a no-op even when switched on
    try:
        assert add(1) == 2
        if not __import__("torch").cuda.is_available():
            assert "stage.name" not in profiling.timing_summary()
    finally:
        profiling.enable(timing=False)


def test_small_parity_helpers():
    import collections
    import logging

    import torch

    from hivemind_b200.compression.floating import get_num_bits
    from hivemind_b200.optim.training_averager import initialize_optimizer_state
    from hivemind_b200.utils import MAX_DHT_TIME_DISCREPANCY_SECONDS
    from hivemind_b200.utils.logging import golog_level_to_python, in_ipython, python_level_to_golog
    from hivemind_b200.utils.nested import is_namedtuple

    assert MAX_DHT_TIME_DISCREPANCY_SECONDS > 0
    assert get_num_bits(torch.bool) == 8 and get_num_bits(torch.bfloat16) == 16 and get_num_bits(torch.int64) == 64
    point = collections.namedtuple("point", "x y")(1, 2)
    assert is_namedtuple(point) and not is_namedtuple((1, 2))
    assert golog_level_to_python("warn") == logging.WARNING and golog_level_to_python("PANIC") == logging.CRITICAL
    assert python_level_to_golog(logging.WARNING) == "WARN" and python_level_to_golog("debug") == "DEBUG"
    assert in_ipython() is False
    layer = torch.nn.Linear(3, 2)
    before = layer.weight.detach().clone()
    opt = torch.optim.Adam(layer.parameters(), lr=0.1)
    initialize_optimizer_state(opt)
    assert len(opt.state) == 2 and torch.equal(layer.weight, before)


def test_reference_import_paths_of_the_daemon_bindings():
    import hivemind_b200.p2p as p2p
    from hivemind_b200.p2p.p2p_daemon_bindings.control import ControlClient
    from hivemind_b200.p2p.p2p_daemon_bindings.datastructures import PeerID, PeerInfo, StreamInfo
    from hivemind_b200.p2p.p2p_daemon_bindings.p2pclient import Client
    from hivemind_b200.p2p.p2p_daemon_bindings.utils import ControlFailure, P2PDaemonError, P2PHandlerError

    assert PeerID is p2p.PeerID and Client is ControlClient
    assert issubclass(ControlFailure, P2PDaemonError) and P2PHandlerError is p2p.P2PHandlerError
    assert PeerInfo is not None and StreamInfo is not None


def test_a_thousand_futures_between_threads():
    """Many futures set from worker threads and awaited from an event loop in another thread, with cancellations and
    exceptions mixed in (the shape of the reference's stress test, tests/test_util_modules.py:285-331)."""
    import concurrent.futures
    import random

    from hivemind_b200.utils import MPFuture

    count = 1000
    futures = [MPFuture() for _ in range(count)]
    rng = random.Random(0)
    plan = [rng.choice(("result", "exception", "cancel")) for _ in range(count)]

    def producer(chunk):
        for i in chunk:
            if plan[i] == "result":
                futures[i].set_result(i * i)
            elif plan[i] == "exception":
                futures[i].set_exception(ValueError(str(i)))
            else:
                futures[i].cancel()

    async def consumer():
        seen = []
        for i, future in enumerate(futures):
            try:
                seen.append(("result", await future))
            except ValueError as e:
                seen.append(("exception", int(str(e))))
            except (asyncio.CancelledError, concurrent.futures.CancelledError):
                seen.append(("cancel", i))
        return seen

    with concurrent.futures.ThreadPoolExecutor(8) as pool:
        loop_result = pool.submit(lambda: asyncio.new_event_loop().run_until_complete(consumer()))
        time.sleep(0.05)  # the consumer is already waiting when the first futures are resolved
        indices = list(range(count))
        rng.shuffle(indices)
        for k in range(8):
            pool.submit(producer, indices[k::8])
        seen = loop_result.result(timeout=60)
    for i, (kind, value) in enumerate(seen):
        assert kind == plan[i]
        assert value == (i * i if kind == "result" else i)
    assert all(f.done() for f in futures)


def test_amap_in_executor_mixes_inline_and_threaded_items_in_order():
    """Items that ``inline`` picks are computed in the loop's own thread, the others in the pool; results come out in
    input order either way, and an exception of either kind is raised at its position."""
    async def scenario():
        loop_thread = threading.get_ident()
        where = {}

        def work(x):
            where[x] = threading.get_ident()
            if x == 7:
                raise ValueError("seven")
            time.sleep(0.01 if x % 2 else 0)
            return x * x

        results = [r async for r in amap_in_executor(work, as_aiter(*range(6)), max_prefetch=3,
                                                      inline=lambda x: x % 2 == 0)]
        assert results == [x * x for x in range(6)]
        assert all(where[x] == loop_thread for x in (0, 2, 4)) and all(where[x] != loop_thread for x in (1, 3, 5))

        for failing_inline in (True, False):
            seen = []
            with pytest.raises(ValueError, match="seven"):
                async for r in amap_in_executor(work, as_aiter(5, 6, 7, 8), inline=lambda x: failing_inline):
                    seen.append(r)
            assert seen == [25, 36]

    asyncio.new_event_loop().run_until_complete(scenario())
