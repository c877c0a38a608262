"""The wire framing between the Python client and the transport daemon, exercised against in-memory streams and a
scripted fake daemon on a Unix socket (no real daemon process). Frames are ``u32 length | u8 type | fields``, fields
being u8, big-endian u32 or length-prefixed blobs (``hivemind_b200/p2p/control.py``). The reference tests its own
(varint / protobuf) framing the same way (tests/test_p2p_daemon_bindings.py:83-371)."""
import asyncio
import os
import struct

import pytest

from hivemind_b200.p2p import control
from hivemind_b200.p2p.control import DaemonClient, P2PDaemonError, _Reader, _Writer, read_frame
from hivemind_b200.p2p.datastructures import PeerID


def run(coro, timeout=30):
    loop = asyncio.new_event_loop()
    try:
        return loop.run_until_complete(asyncio.wait_for(coro, timeout))
    finally:
        loop.close()


def _stream_with(data: bytes, eof: bool = True) -> asyncio.StreamReader:
    reader = asyncio.StreamReader()
    reader.feed_data(data)
    if eof:
        reader.feed_eof()
    return reader


def test_writer_layout_is_length_type_fields():
    frame = _Writer(7).u8(3).u32(0x01020304).blob(b"abc").blob(b"").finish()
    assert frame == struct.pack(">I", 1 + 1 + 4 + 4 + 3 + 4) + bytes([7, 3]) + b"\x01\x02\x03\x04" + \
        struct.pack(">I", 3) + b"abc" + struct.pack(">I", 0)
    fields = _Reader(frame[5:])
    assert (fields.u8(), fields.u32(), fields.blob(), fields.blob()) == (3, 0x01020304, b"abc", b"")


@pytest.mark.parametrize("payload", [b"", b"x", os.urandom(70000)])
def test_frames_round_trip_through_a_stream(payload):
    async def main():
        first = _Writer(control.R_OK).blob(payload).u32(len(payload)).finish()
        second = _Writer(control.R_ERR).blob(b"boom").finish()
        reader = _stream_with(first + second)
        msg_type, body = await read_frame(reader)
        assert msg_type == control.R_OK and body.blob() == payload and body.u32() == len(payload)
        msg_type, body = await read_frame(reader)
        assert msg_type == control.R_ERR and body.blob() == b"boom"
        with pytest.raises(asyncio.IncompleteReadError):
            await read_frame(reader)  # clean end of stream between frames

    run(main())


def test_frames_that_arrive_in_pieces_are_reassembled():
    async def main():
        frame = _Writer(control.P_RESPONSE).blob(b"call-id-0123456").blob(b"y" * 1000).finish()
        reader = asyncio.StreamReader()

        async def feed():
            for i in range(0, len(frame), 7):
                reader.feed_data(frame[i:i + 7])
                await asyncio.sleep(0)
            reader.feed_eof()

        feeder = asyncio.create_task(feed())
        msg_type, body = await read_frame(reader)
        await feeder
        assert msg_type == control.P_RESPONSE and body.blob() == b"call-id-0123456" and body.blob() == b"y" * 1000

    run(main())


def test_truncated_frames_and_fields_are_errors():
    async def main():
        whole = _Writer(control.R_OK).blob(b"0123456789").finish()
        with pytest.raises(asyncio.IncompleteReadError):
            await read_frame(_stream_with(whole[:-3]))  # the stream ends inside the body
        with pytest.raises(asyncio.IncompleteReadError):
            await read_frame(_stream_with(whole[:2]))  # ... inside the length word
        # a blob whose declared length exceeds what the frame holds
        lying = bytes([control.R_OK]) + struct.pack(">I", 50) + b"short"
        _, body = await read_frame(_stream_with(struct.pack(">I", len(lying)) + lying))
        with pytest.raises(P2PDaemonError):
            body.blob()

    run(main())


def test_client_commands_against_a_scripted_daemon(tmp_path):
    """``DaemonClient`` talking to a fake daemon that records the request frames and answers with canned replies."""
    async def main():
        control_path, listen_path = str(tmp_path / "control.sock"), str(tmp_path / "listen.sock")
        me = PeerID(b"\x12\x20" + bytes(range(32)))
        requests = []

        async def fake_daemon(reader, writer):
            msg_type, body = await read_frame(reader)
            requests.append(msg_type)
            if msg_type == control.C_PERSISTENT:
                writer.write(_Writer(control.R_OK).finish())
                await writer.drain()
                await reader.read()  # the persistent link just stays open
            elif msg_type == control.C_IDENTIFY:
                writer.write(_Writer(control.R_OK).blob(me.to_base58().encode()).u32(1).blob(b"/ip4/127.0.0.1/tcp/4001").finish())
            elif msg_type == control.C_DISCONNECT:
                requests.append(body.blob())
                writer.write(_Writer(control.R_ERR).blob("no such peer".encode()).finish())
            else:
                writer.write(_Writer(99).finish())  # a reply type the client does not know
            await writer.drain()
            writer.close()

        server = await asyncio.start_unix_server(fake_daemon, path=control_path)
        client = await DaemonClient.create(control_path, listen_path)
        try:
            peer_id, maddrs = await client.identify()
            assert peer_id == me and [str(m) for m in maddrs] == ["/ip4/127.0.0.1/tcp/4001"]
            with pytest.raises(P2PDaemonError, match="no such peer"):
                await client.disconnect(me)
            assert me.to_base58().encode() in requests  # the peer id travelled as a base58 blob
            with pytest.raises(P2PDaemonError, match="unexpected reply type 99"):
                await client.list_peers()
            assert requests[0] == control.C_PERSISTENT and control.C_IDENTIFY in requests
        finally:
            await client.close()
            server.close()
            await server.wait_closed()

    run(main())


def test_chunked_stream_reader_matches_the_standard_reader_on_random_traffic():
    """Blocks of random sizes go in, reads of random sizes come out: same bytes, same EOF behaviour as
    ``asyncio.StreamReader`` (whose interface it keeps for ``read`` / ``readexactly`` / ``at_eof``)."""
    import asyncio
    import random

    from hivemind_b200.p2p.chunked_reader import ChunkedStreamReader

    async def scenario():
        rng = random.Random(0)
        payload = bytes(rng.getrandbits(8) for _ in range(200_000))
        for trial in range(20):
            ours, theirs = ChunkedStreamReader(limit=4096), asyncio.StreamReader(limit=4096)
            cursor = 0
            while cursor < len(payload):
                step = rng.choice([1, 7, 100, 4096, 65536])
                for reader in (ours, theirs):
                    reader.feed_data(payload[cursor:cursor + step])
                cursor += step
            for reader in (ours, theirs):
                reader.feed_eof()
            collected = []
            while True:
                if rng.random() < 0.5:
                    n = rng.choice([1, 2, 9, 1000, 50_000])
                    a, b = await ours.read(n), await theirs.read(n)
                else:
                    n = rng.choice([1, 8, 333, 70_000])
                    results = []
                    for reader in (ours, theirs):
                        try:
                            results.append(await reader.readexactly(n))
                        except asyncio.IncompleteReadError as e:
                            results.append(("incomplete", e.partial, e.expected))
                    a, b = results
                assert a == b
                collected.append(a if isinstance(a, bytes) else a[1])
                assert ours.at_eof() == theirs.at_eof()
                if ours.at_eof():
                    break
            assert b"".join(collected) == payload
            assert await ours.read(10) == b"" and await ours.read() == b""
        assert await ChunkedStreamReader().read(0) == b"" and await ChunkedStreamReader().readexactly(0) == b""
        with pytest.raises(ValueError):
            await ChunkedStreamReader().readexactly(-1)
        with pytest.raises(NotImplementedError):
            await ChunkedStreamReader().readline()

    asyncio.new_event_loop().run_until_complete(scenario())


def test_chunked_stream_reader_waits_pauses_and_reports_errors():
    import asyncio

    from hivemind_b200.p2p.chunked_reader import ChunkedStreamReader

    class FakeTransport:
        def __init__(self):
            self.paused, self.events = False, []

        def pause_reading(self):
            self.paused = True
            self.events.append("pause")

        def resume_reading(self):
            self.paused = False
            self.events.append("resume")

    async def scenario():
        reader, transport = ChunkedStreamReader(limit=100), FakeTransport()
        reader.set_transport(transport)
        pending = asyncio.ensure_future(reader.readexactly(250))  # larger than twice the limit
        await asyncio.sleep(0)
        for _ in range(5):
            reader.feed_data(b"x" * 60)  # the third block crosses the high-water mark and pauses the transport
            await asyncio.sleep(0)  # ... the waiting read resumes it: it still needs bytes
        assert await asyncio.wait_for(pending, 1) == b"x" * 250
        assert transport.events[:2] == ["pause", "resume"] and not transport.paused
        assert await reader.read(1000) == b"x" * 50

        reader.feed_data(b"y" * 300)
        assert transport.paused
        assert await reader.read(250) == b"y" * 250 and not transport.paused, "draining below the limit resumes"

        waiting = asyncio.ensure_future(reader.read(10))
        await asyncio.sleep(0)
        reader.feed_data(b"tail")
        assert await asyncio.wait_for(waiting, 1) == b"yyyyyyyyyy"

        broken = ChunkedStreamReader()
        waiter = asyncio.ensure_future(broken.readexactly(4))
        await asyncio.sleep(0)
        broken.set_exception(ConnectionResetError("peer went away"))
        with pytest.raises(ConnectionResetError):
            await waiter
        with pytest.raises(ConnectionResetError):
            await broken.read(1)

    asyncio.new_event_loop().run_until_complete(scenario())
