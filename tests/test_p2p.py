"""Transport daemon + P2P wrapper + servicer reflection (cases modelled on the reference's tests/test_p2p_daemon.py
and tests/test_p2p_servicer.py: unary and streaming handlers, errors, cancellation, replicas, balanced handlers)."""
import asyncio
import contextlib
from typing import AsyncIterator

import pytest

from hivemind_b200.p2p import P2P, P2PContext, P2PDaemonError, P2PHandlerError, PeerID, ServicerBase
from hivemind_b200.proto import test_pb2


def run(coro):
    loop = asyncio.new_event_loop()
    try:
        return loop.run_until_complete(asyncio.wait_for(coro, 60))
    finally:
        loop.close()


async def _pair():
    server = await P2P.create()
    client = await P2P.create(initial_peers=await server.get_visible_maddrs())
    return server, client


def test_daemon_start_identity_and_peers(tmp_path):
    async def main():
        ident = str(tmp_path / "id.key")
        a = await P2P.create(identity_path=ident)
        pid = a.peer_id
        maddrs = await a.get_visible_maddrs()
        assert maddrs and str(maddrs[0]).endswith(pid.to_base58())
        b = await P2P.create(initial_peers=maddrs)
        await b.wait_for_at_least_n_peers(1)
        assert any(p.peer_id == pid for p in await b.list_peers())
        await a.shutdown()
        a2 = await P2P.create(identity_path=ident)
        assert a2.peer_id == pid  # identity files make the id deterministic
        await a2.shutdown()
        await b.shutdown()
        assert not a.is_alive and not b.is_alive

    run(main())


def test_unary_and_errors_and_cancel():
    async def main():
        server, client = await _pair()
        cancelled = asyncio.Event()

        async def square(request: test_pb2.TestRequest, context: P2PContext) -> test_pb2.TestResponse:
            assert context.remote_id == client.peer_id
            return test_pb2.TestResponse(number=request.number ** 2)

        async def fail(request, context):
            raise ValueError("boom")

        async def slow(request, context):
            try:
                await asyncio.sleep(30)
            except asyncio.CancelledError:
                cancelled.set()
                raise
            return test_pb2.TestResponse(number=0)

        await server.add_protobuf_handler("square", square, test_pb2.TestRequest)
        await server.add_protobuf_handler("fail", fail, test_pb2.TestRequest)
        await server.add_protobuf_handler("slow", slow, test_pb2.TestRequest)
        out = await client.call_protobuf_handler(server.peer_id, "square", test_pb2.TestRequest(number=12), test_pb2.TestResponse)
        assert out.number == 144
        results = await asyncio.gather(*[client.call_protobuf_handler(server.peer_id, "square", test_pb2.TestRequest(number=i),
                                                                     test_pb2.TestResponse) for i in range(50)])
        assert [r.number for r in results] == [i * i for i in range(50)]
        with pytest.raises(P2PHandlerError, match="boom"):
            await client.call_protobuf_handler(server.peer_id, "fail", test_pb2.TestRequest(number=1), test_pb2.TestResponse)
        with pytest.raises(P2PHandlerError):
            await client.call_protobuf_handler(server.peer_id, "missing", test_pb2.TestRequest(number=1), test_pb2.TestResponse)
        task = asyncio.create_task(client.call_protobuf_handler(server.peer_id, "slow", test_pb2.TestRequest(number=1),
                                                                test_pb2.TestResponse))
        await asyncio.sleep(0.3)
        task.cancel()
        await asyncio.wait_for(cancelled.wait(), 5)  # the cancel reaches the remote handler
        # a handler that was withdrawn is gone for callers
        await server.remove_protobuf_handler("square")
        with pytest.raises(P2PHandlerError):
            await client.call_protobuf_handler(server.peer_id, "square", test_pb2.TestRequest(number=7), test_pb2.TestResponse)
        await client.shutdown()
        await server.shutdown()

    run(main())


class ExampleServicer(ServicerBase):
    async def rpc_square(self, request: test_pb2.TestRequest, _context: P2PContext) -> test_pb2.TestResponse:
        return test_pb2.TestResponse(number=request.number ** 2)

    async def rpc_sum(self, stream: AsyncIterator[test_pb2.TestRequest], _context: P2PContext) -> test_pb2.TestResponse:
        total = 0
        async for item in stream:
            total += item.number
        return test_pb2.TestResponse(number=total)

    async def rpc_count(self, request: test_pb2.TestRequest, _context: P2PContext) -> AsyncIterator[test_pb2.TestResponse]:
        for i in range(request.number):
            yield test_pb2.TestResponse(number=i)

    async def rpc_running_sum(self, stream: AsyncIterator[test_pb2.TestRequest], _context: P2PContext
                              ) -> AsyncIterator[test_pb2.TestResponse]:
        total = 0
        async for item in stream:
            total += item.number
            yield test_pb2.TestResponse(number=total)

    async def rpc_fail_midway(self, request: test_pb2.TestRequest, _context: P2PContext) -> AsyncIterator[test_pb2.TestResponse]:
        yield test_pb2.TestResponse(number=1)
        raise RuntimeError("midway failure")


def test_servicer_four_combinations():
    async def main():
        server, client = await _pair()
        servicer = ExampleServicer()
        await servicer.add_p2p_handlers(server, namespace="ns")
        stub = ExampleServicer.get_stub(client, server.peer_id, namespace="ns")
        assert (await stub.rpc_square(test_pb2.TestRequest(number=9), timeout=10)).number == 81

        async def numbers(n):
            for i in range(n):
                yield test_pb2.TestRequest(number=i)

        assert (await stub.rpc_sum(numbers(10))).number == 45
        got = [r.number async for r in await stub.rpc_count(test_pb2.TestRequest(number=5))]
        assert got == list(range(5))
        got = [r.number async for r in await stub.rpc_running_sum(numbers(5))]
        assert got == [0, 1, 3, 6, 10]
        with pytest.raises(P2PHandlerError, match="midway failure"):
            async for _ in await stub.rpc_fail_midway(test_pb2.TestRequest(number=1)):
                pass
        # wrong namespace is not served
        other = ExampleServicer.get_stub(client, server.peer_id, namespace="other")
        with pytest.raises(P2PHandlerError):
            await other.rpc_square(test_pb2.TestRequest(number=2), timeout=10)
        await servicer.remove_p2p_handlers(server, namespace="ns")
        with pytest.raises(P2PHandlerError):
            await stub.rpc_square(test_pb2.TestRequest(number=2), timeout=10)
        await client.shutdown()
        await server.shutdown()

    run(main())


def test_large_stream_and_binary_handlers():
    async def main():
        server, client = await _pair()

        async def echo(info, reader, writer):
            data = await P2P.receive_raw_data(reader)
            await P2P.send_raw_data(data[::-1], writer)

        await server.add_binary_stream_handler("echo", echo)
        payload = bytes(range(256)) * (20 * 1024)  # 5 MiB, more than one socket buffer
        _, reader, writer = await client.call_binary_stream_handler(server.peer_id, "echo")
        await P2P.send_raw_data(payload, writer)
        assert await P2P.receive_raw_data(reader) == payload[::-1]
        writer.close()
        with pytest.raises(P2PHandlerError):
            await client.call_binary_stream_handler(server.peer_id, "nope")
        await client.shutdown()
        await server.shutdown()

    run(main())


def test_replicas_balanced_and_third_party_discovery():
    async def main():
        server = await P2P.create()
        replica = await P2P.replicate(server.daemon_listen_maddr)
        assert replica.peer_id == server.peer_id
        hits = {"a": 0, "b": 0}

        def make(tag):
            async def handler(request: test_pb2.TestRequest, context: P2PContext) -> test_pb2.TestResponse:
                hits[tag] += 1
                return test_pb2.TestResponse(number=request.number)
            return handler

        await server.add_protobuf_handler("bal", make("a"), test_pb2.TestRequest, balanced=True)
        await replica.add_protobuf_handler("bal", make("b"), test_pb2.TestRequest, balanced=True)
        with pytest.raises(P2PDaemonError):
            await replica.add_protobuf_handler("bal2", make("a"), test_pb2.TestRequest)
            await server.add_protobuf_handler("bal2", make("b"), test_pb2.TestRequest)  # not balanced: second one refused
        client = await P2P.create(initial_peers=await server.get_visible_maddrs())
        for i in range(10):
            await client.call_protobuf_handler(server.peer_id, "bal", test_pb2.TestRequest(number=i), test_pb2.TestResponse)
        assert hits["a"] == 5 and hits["b"] == 5
        # a third peer that only knows the server can reach `client` through address gossip / who-has
        third = await P2P.create(initial_peers=await server.get_visible_maddrs())

        async def hello(request: test_pb2.TestRequest, context: P2PContext) -> test_pb2.TestResponse:
            return test_pb2.TestResponse(number=request.number + 1)

        await client.add_protobuf_handler("hello", hello, test_pb2.TestRequest)
        out = await third.call_protobuf_handler(client.peer_id, "hello", test_pb2.TestRequest(number=1), test_pb2.TestResponse)
        assert out.number == 2
        # calling oneself works too
        out = await client.call_protobuf_handler(client.peer_id, "hello", test_pb2.TestRequest(number=5), test_pb2.TestResponse)
        assert out.number == 6
        for p in (third, client, replica, server):
            await p.shutdown()

    run(main())


def test_peer_id_derivation_is_stable():
    from cryptography.hazmat.primitives.asymmetric import rsa

    key = rsa.generate_private_key(public_exponent=65537, key_size=2048)
    a, b = PeerID.from_private_key(key), PeerID.from_private_key(key)
    assert a == b and a.to_base58().startswith("Qm") and PeerID.from_base58(a.to_base58()) == a


class _EndlessServicer(ServicerBase):
    def __init__(self):
        self.started, self.cancelled = asyncio.Event(), asyncio.Event()

    async def rpc_ticks(self, request: test_pb2.TestRequest, _context: P2PContext) -> AsyncIterator[test_pb2.TestResponse]:
        self.started.set()
        try:
            i = 0
            while True:
                yield test_pb2.TestResponse(number=i)
                i += 1
                await asyncio.sleep(0.05)
        except (asyncio.CancelledError, GeneratorExit):
            self.cancelled.set()
            raise
        finally:
            self.cancelled.set()


def test_streaming_handler_stops_when_the_caller_walks_away():
    """A client that abandons a response stream (reference: test_unary_stream_cancel in tests/test_p2p_servicer.py):
    the server-side generator is closed instead of producing forever."""
    async def main():
        server, client = await _pair()
        servicer = _EndlessServicer()
        await servicer.add_p2p_handlers(server)
        stub = _EndlessServicer.get_stub(client, server.peer_id)

        async def consume_three():
            received = []
            async with contextlib.aclosing(await stub.rpc_ticks(test_pb2.TestRequest(number=0))) as ticks:
                async for item in ticks:
                    received.append(item.number)
                    if len(received) == 3:
                        break
            return received

        assert await consume_three() == [0, 1, 2]
        await asyncio.wait_for(servicer.started.wait(), 5)
        await asyncio.wait_for(servicer.cancelled.wait(), 10)
        # the connection pair stays usable afterwards
        servicer.started.clear()
        servicer.cancelled.clear()
        assert (await consume_three()) == [0, 1, 2]
        await client.shutdown()
        await server.shutdown()

    run(main())


def test_dead_daemon_is_reported_and_shutdown_is_idempotent():
    async def main():
        node = await P2P.create()
        assert node.is_alive
        await node.shutdown()
        await node.shutdown()  # second call is a no-op
        assert not node.is_alive

    run(main())


def test_start_up_failures_say_why():
    """Reference cases test_startup_error_message (tests/test_p2p_daemon.py:44-56): unreachable bootstrap peers and an
    impossible start-up time limit end in P2PDaemonError with a message that names the cause."""
    async def main():
        import socket

        with socket.socket() as probe:  # a port that nobody listens on
            probe.bind(("127.0.0.1", 0))
            port = probe.getsockname()[1]
        nobody = f"/ip4/127.0.0.1/tcp/{port}/p2p/QmdaK4LUeQaKhqSFPRu9N7MvXUEWDxWwtCvPrS444tCgd1"
        with pytest.raises(P2PDaemonError, match=r"(?i)failed to connect to bootstrap peers"):
            await P2P.create(initial_peers=[nobody])
        with pytest.raises(P2PDaemonError, match=r"Daemon failed to start in .+ seconds"):
            await P2P.create(startup_timeout=0.0001)

    run(main())


def test_daemon_dies_with_its_owner_and_identities_are_exclusive(tmp_path):
    """Reference cases test_daemon_killed_on_del and test_check_if_identity_free (tests/test_p2p_daemon.py:28-42,
    64-86): dropping the last reference to a P2P instance ends its daemon process; an identity that answers on the
    network cannot be used by a second peer, a fresh one can."""
    async def main():
        import gc
        import os

        instance = await P2P.create()
        pid = instance._child.pid
        os.kill(pid, 0)  # alive
        del instance
        gc.collect()
        for _ in range(50):
            await asyncio.sleep(0.1)
            try:
                os.kill(pid, 0)
                with open(f"/proc/{pid}/stat") as f:
                    if f.read().split()[2] == "Z":  # a zombie counts as dead: nobody will wait for it after __del__
                        break
            except (ProcessLookupError, FileNotFoundError):
                break
        else:
            raise AssertionError("the daemon outlived its owner")

        taken, free = str(tmp_path / "taken.key"), str(tmp_path / "free.key")
        P2P.generate_identity(taken)
        P2P.generate_identity(free)
        first = await P2P.create(identity_path=taken)
        maddrs = await first.get_visible_maddrs()
        assert await P2P.is_identity_taken(first.peer_id, maddrs)
        with pytest.raises(P2PDaemonError, match="already in use"):
            await P2P.create(identity_path=taken, initial_peers=maddrs)
        other = await P2P.create(identity_path=free, initial_peers=maddrs)
        assert other.peer_id != first.peer_id and not await P2P.is_identity_taken(PeerID.from_base58(
            "QmdaK4LUeQaKhqSFPRu9N7MvXUEWDxWwtCvPrS444tCgd1"), maddrs)
        await other.shutdown()
        await first.shutdown()

    run(main())


def test_removed_handlers_stop_answering():
    """Reference cases test_removing_unary_handlers / test_removing_stream_handlers (tests/test_p2p_daemon.py:362-420)."""
    async def main():
        server, client = await _pair()

        async def double(request: test_pb2.TestRequest, context: P2PContext) -> test_pb2.TestResponse:
            return test_pb2.TestResponse(number=2 * request.number)

        async def count(request: test_pb2.TestRequest, context: P2PContext) -> AsyncIterator[test_pb2.TestResponse]:
            for i in range(request.number):
                yield test_pb2.TestResponse(number=i)

        await server.add_protobuf_handler("double", double, test_pb2.TestRequest)
        await server.add_protobuf_handler("count", count, test_pb2.TestRequest, stream_output=True)
        reply = await client.call_protobuf_handler(server.peer_id, "double", test_pb2.TestRequest(number=21), test_pb2.TestResponse)
        assert reply.number == 42
        stream = await client.iterate_protobuf_handler(server.peer_id, "count", test_pb2.TestRequest(number=3), test_pb2.TestResponse)
        assert [item.number async for item in stream] == [0, 1, 2]

        await server.remove_protobuf_handler("double")
        await server.remove_protobuf_handler("count", stream_output=True)
        with pytest.raises((P2PHandlerError, P2PDaemonError)):
            await client.call_protobuf_handler(server.peer_id, "double", test_pb2.TestRequest(number=1), test_pb2.TestResponse)
        with pytest.raises((P2PHandlerError, P2PDaemonError)):
            stream = await client.iterate_protobuf_handler(server.peer_id, "count", test_pb2.TestRequest(number=3), test_pb2.TestResponse)
            async for _ in stream:
                pass
        # a handler can be registered again under the same name
        await server.add_protobuf_handler("double", double, test_pb2.TestRequest)
        reply = await client.call_protobuf_handler(server.peer_id, "double", test_pb2.TestRequest(number=4), test_pb2.TestResponse)
        assert reply.number == 8
        await client.shutdown()
        await server.shutdown()

    run(main())


def _serve_in_child(addresses, stop) -> None:
    """Body of a child process: one peer with a unary and a binary stream handler, until ``stop`` is set."""
    async def main():
        server = await P2P.create()

        async def double(request: test_pb2.TestRequest, context: P2PContext) -> test_pb2.TestResponse:
            return test_pb2.TestResponse(number=2 * request.number)

        async def upper(info, reader, writer):
            await P2P.send_raw_data((await P2P.receive_raw_data(reader)).upper(), writer)

        await server.add_protobuf_handler("double", double, test_pb2.TestRequest)
        await server.add_binary_stream_handler("upper", upper)
        addresses.put(([str(m) for m in await server.get_visible_maddrs()], server.peer_id.to_base58()))
        while not stop.is_set():
            await asyncio.sleep(0.05)
        await server.shutdown()

    asyncio.new_event_loop().run_until_complete(main())


def test_calls_between_processes_and_a_peer_that_disappears():
    """Reference cases test_call_peer_different_processes / test_error_closes_connection (tests/test_p2p_daemon.py):
    handlers in another process answer; once that process is gone (killed, so it says no goodbye) a call ends in an
    error within its time limit instead of hanging, and the caller's own daemon keeps serving other peers."""
    import multiprocessing as mp
    import os
    import signal

    ctx = mp.get_context("spawn")
    addresses, stop = ctx.Queue(), ctx.Event()
    child = ctx.Process(target=_serve_in_child, args=(addresses, stop), daemon=True)
    child.start()
    maddrs, peer_text = addresses.get(timeout=120)
    remote = PeerID.from_base58(peer_text)

    async def main():
        client = await P2P.create(initial_peers=maddrs)
        out = await client.call_protobuf_handler(remote, "double", test_pb2.TestRequest(number=21), test_pb2.TestResponse)
        assert out.number == 42
        _, reader, writer = await client.call_binary_stream_handler(remote, "upper")
        await P2P.send_raw_data(b"between processes", writer)
        assert await P2P.receive_raw_data(reader) == b"BETWEEN PROCESSES"
        writer.close()

        os.kill(child.pid, signal.SIGKILL)  # the exact process started above
        child.join(timeout=30)
        with pytest.raises((P2PHandlerError, P2PDaemonError, asyncio.TimeoutError, ConnectionError)):
            await asyncio.wait_for(client.call_protobuf_handler(remote, "double", test_pb2.TestRequest(number=1),
                                                                test_pb2.TestResponse), timeout=15)

        bystander = await P2P.create(initial_peers=await client.get_visible_maddrs())

        async def hello(request: test_pb2.TestRequest, context: P2PContext) -> test_pb2.TestResponse:
            return test_pb2.TestResponse(number=request.number + 1)

        await client.add_protobuf_handler("hello", hello, test_pb2.TestRequest)
        out = await bystander.call_protobuf_handler(client.peer_id, "hello", test_pb2.TestRequest(number=1),
                                                    test_pb2.TestResponse)
        assert out.number == 2
        await bystander.shutdown()
        await client.shutdown()

    try:
        run(main())
    finally:
        stop.set()
        if child.is_alive():
            child.join(timeout=10)


def test_handlers_on_different_replicas_and_a_replica_that_leaves():
    """Reference cases test_handlers_on_different_replicas and test_daemon_replica_does_not_affect_primary: each
    replica of one daemon serves the handlers that it registered; shutting a replica down removes its handlers only."""
    async def main():
        primary = await P2P.create()
        replica = await P2P.replicate(primary.daemon_listen_maddr)
        client = await P2P.create(initial_peers=await primary.get_visible_maddrs())

        def answer(offset):
            async def handler(request: test_pb2.TestRequest, context: P2PContext) -> test_pb2.TestResponse:
                return test_pb2.TestResponse(number=request.number + offset)
            return handler

        async def echo(tag):
            async def handler(info, reader, writer):
                await P2P.send_raw_data(tag + await P2P.receive_raw_data(reader), writer)
            return handler

        await primary.add_protobuf_handler("plus_one", answer(1), test_pb2.TestRequest)
        await replica.add_protobuf_handler("plus_ten", answer(10), test_pb2.TestRequest)
        await primary.add_binary_stream_handler("tag_p", await echo(b"p:"))
        await replica.add_binary_stream_handler("tag_r", await echo(b"r:"))

        async def call(name):
            return (await client.call_protobuf_handler(primary.peer_id, name, test_pb2.TestRequest(number=1),
                                                       test_pb2.TestResponse)).number

        async def stream(name):
            _, reader, writer = await client.call_binary_stream_handler(primary.peer_id, name)
            await P2P.send_raw_data(b"x", writer)
            try:
                return await P2P.receive_raw_data(reader)
            finally:
                writer.close()

        assert await call("plus_one") == 2 and await call("plus_ten") == 11
        assert await stream("tag_p") == b"p:x" and await stream("tag_r") == b"r:x"

        await replica.shutdown()
        assert primary.is_alive
        assert await call("plus_one") == 2 and await stream("tag_p") == b"p:x"
        with pytest.raises((P2PHandlerError, P2PDaemonError)):
            await call("plus_ten")
        with pytest.raises((P2PHandlerError, P2PDaemonError, asyncio.IncompleteReadError, ConnectionError)):
            await stream("tag_r")
        # the name is free again for whoever is still there
        await primary.add_protobuf_handler("plus_ten", answer(100), test_pb2.TestRequest)
        assert await call("plus_ten") == 101
        await client.shutdown()
        await primary.shutdown()

    run(main())
