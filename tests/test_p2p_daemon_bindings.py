"""Framing helpers and message schema of the libp2p daemon's control protocol, and the data types that convert to and
from its messages (the unit tier of the reference's tests/test_p2p_daemon_bindings.py: varints, length-prefixed
protobufs against in-memory streams, PeerID / PeerInfo / StreamInfo)."""
import asyncio
import io

import pytest

from hivemind_b200.p2p.p2p_daemon_bindings.datastructures import PeerID, PeerInfo, StreamInfo
from hivemind_b200.p2p.p2p_daemon_bindings.utils import (ControlFailure, P2PDaemonError, raise_if_failed,
                                                         read_pbmsg_safe, read_unsigned_varint, write_pbmsg,
                                                         write_unsigned_varint)
from hivemind_b200.proto import p2pd_pb2
from hivemind_b200.utils.multiaddr import Multiaddr


def run(coro):
    loop = asyncio.new_event_loop()
    try:
        return loop.run_until_complete(asyncio.wait_for(coro, 30))
    finally:
        loop.close()


class MemoryStream(io.BytesIO):
    """Stands in for both ends of an asyncio stream pair."""

    async def readexactly(self, n: int) -> bytes:
        await asyncio.sleep(0)
        data = self.read(n)
        if len(data) != n:
            raise asyncio.IncompleteReadError(data, n)
        return data

    async def drain(self) -> None:
        pass


VARINTS = [(0, "00"), (1, "01"), (127, "7f"), (128, "8001"), (150, "9601"), (300, "ac02"), (16384, "808001"),
           (2 ** 32 - 1, "ffffffff0f"), (2 ** 63, "80" * 9 + "01"), (2 ** 64 - 1, "ff" * 9 + "01")]
TOO_LARGE = [(2 ** 64, "80" * 9 + "02"), (2 ** 64 + 1, "81" + "80" * 8 + "02"), (2 ** 70 - 1, "ff" * 10),
             (2 ** 128, "80" * 18 + "04")]


@pytest.mark.parametrize("number,encoded", VARINTS)
def test_varints_both_ways(number, encoded):
    out = MemoryStream()
    run(write_unsigned_varint(out, number))
    assert out.getvalue().hex() == encoded
    assert run(read_unsigned_varint(MemoryStream(bytes.fromhex(encoded) + b"\xff trailing"))) == number


@pytest.mark.parametrize("number,encoded", TOO_LARGE)
def test_varints_that_do_not_fit_are_refused(number, encoded):
    with pytest.raises(ValueError):
        run(write_unsigned_varint(MemoryStream(), number))
    with pytest.raises(ValueError):
        run(read_unsigned_varint(MemoryStream(bytes.fromhex(encoded))))


@pytest.mark.parametrize("number", [-1, -(2 ** 32), -(2 ** 64), -(2 ** 128)])
def test_negative_numbers_are_refused(number):
    with pytest.raises(ValueError):
        run(write_unsigned_varint(MemoryStream(), number))


@pytest.mark.parametrize("max_bits", [2, 7, 8, 31, 32, 63, 64, 127, 128])
def test_varint_bit_limits(max_bits):
    for number in (2 ** max_bits - 3, 2 ** max_bits - 2, 2 ** max_bits - 1):
        stream = MemoryStream()
        run(write_unsigned_varint(stream, number, max_bits=max_bits))
        stream.seek(0)
        assert run(read_unsigned_varint(stream, max_bits=max_bits)) == number
    with pytest.raises(ValueError):
        run(write_unsigned_varint(MemoryStream(), 2 ** max_bits, max_bits=max_bits))
    oversize = MemoryStream()
    run(write_unsigned_varint(oversize, 2 ** max_bits, max_bits=max_bits + 8))
    oversize.seek(0)
    with pytest.raises(ValueError):
        run(read_unsigned_varint(oversize, max_bits=max_bits))


def test_a_stream_that_ends_inside_a_number_or_a_message():
    with pytest.raises(asyncio.IncompleteReadError):
        run(read_unsigned_varint(MemoryStream(b"\x80\x80")))
    with pytest.raises(asyncio.IncompleteReadError):
        run(read_pbmsg_safe(MemoryStream(b"\x05\x08\x01"), p2pd_pb2.Response()))


PEER_TEXT = "QmS5QmciTXXnCUCyxud5eWFenUMAmvAWSDa1c7dvdXRMZ7"
PEER_BYTES = PeerID.from_base58(PEER_TEXT).to_bytes()  # a sha2-256 multihash: 0x12, 0x20, then 32 digest bytes
ADDR = Multiaddr("/ip4/127.0.0.1/tcp/4001")


def test_messages_have_the_wire_format_of_the_schema():
    # field 1 varint (type), then length-delimited sub-messages under the schema's field numbers
    request = p2pd_pb2.Request(type=p2pd_pb2.Request.STREAM_OPEN,
                               streamOpen=p2pd_pb2.StreamOpenRequest(peer=b"abc", proto=["/x/1"], timeout=5))
    assert request.SerializeToString().hex() == "0802" + "1a0d" + "0a03616263" + "1204" + b"/x/1".hex() + "1805"
    error = p2pd_pb2.Response(type=p2pd_pb2.Response.ERROR, error=p2pd_pb2.ErrorResponse(msg="x"))
    assert error.SerializeToString().hex() == "0801" + "1203" + "0a0178"
    assert p2pd_pb2.Request.Type.Name(10) == "REMOVE_STREAM_HANDLER" and p2pd_pb2.Request.PERSISTENT_CONN_UPGRADE == 9
    assert p2pd_pb2.DHTRequest.GET_CLOSEST_PEERS == 3 and p2pd_pb2.PSRequest.Type.Value("SUBSCRIBE") == 3
    with pytest.raises(Exception):
        p2pd_pb2.Response().SerializeToString()  # `type` is a required field
    call = p2pd_pb2.PersistentConnectionRequest(callId=b"i" * 16, callUnary=p2pd_pb2.CallUnaryRequest(
        peer=b"p", proto="q", data=b"d"))
    assert call.WhichOneof("message") == "callUnary"
    call.cancel.SetInParent()
    assert call.WhichOneof("message") == "cancel" and not call.HasField("callUnary")
    answer = p2pd_pb2.CallUnaryResponse(response=b"ok")
    answer.error = b"failed"
    assert answer.WhichOneof("result") == "error" and not answer.HasField("response")
    parsed = p2pd_pb2.PersistentConnectionResponse.FromString(p2pd_pb2.PersistentConnectionResponse(
        callId=b"i" * 16, daemonError=p2pd_pb2.DaemonError(message="gone")).SerializeToString())
    assert parsed.WhichOneof("message") == "daemonError" and parsed.daemonError.message == "gone"


def test_length_prefixed_messages_over_memory_and_real_streams():
    messages = [
        p2pd_pb2.Request(type=p2pd_pb2.Request.IDENTIFY),
        p2pd_pb2.Request(type=p2pd_pb2.Request.CONNECT, connect=p2pd_pb2.ConnectRequest(
            peer=PEER_BYTES, addrs=[ADDR.to_bytes()], timeout=3)),
        p2pd_pb2.Request(type=p2pd_pb2.Request.STREAM_HANDLER, streamHandler=p2pd_pb2.StreamHandlerRequest(
            addr=Multiaddr("/unix/tmp/handler.sock").to_bytes(), proto=["/a/1", "/b/2"], balanced=True)),
        p2pd_pb2.Request(type=p2pd_pb2.Request.DHT, dht=p2pd_pb2.DHTRequest(
            type=p2pd_pb2.DHTRequest.PUT_VALUE, key=b"k" * 300, value=b"v" * 70000)),  # multi-byte length prefixes
    ]
    stream = MemoryStream()
    for message in messages:
        run(write_pbmsg(stream, message))
    assert stream.getvalue()[:3] == b"\x02\x08\x00"
    stream.seek(0)
    for message in messages:
        received = p2pd_pb2.Request(type=p2pd_pb2.Request.PUBSUB, pubsub=p2pd_pb2.PSRequest(type=0, topic="stale"))
        run(read_pbmsg_safe(stream, received))
        assert received == message and not received.HasField("pubsub"), "earlier content must be replaced"

    async def over_a_socket():
        arrived = asyncio.Queue()

        async def serve(reader, writer):
            request = p2pd_pb2.Request()
            await read_pbmsg_safe(reader, request)
            await arrived.put(request)
            response = p2pd_pb2.Response(type=p2pd_pb2.Response.OK, identify=p2pd_pb2.IdentifyResponse(
                id=PEER_BYTES, addrs=[ADDR.to_bytes()]))
            await write_pbmsg(writer, response)
            await writer.drain()
            writer.close()

        server = await asyncio.start_server(serve, "127.0.0.1", 0)
        port = server.sockets[0].getsockname()[1]
        reader, writer = await asyncio.open_connection("127.0.0.1", port)
        await write_pbmsg(writer, messages[1])
        await writer.drain()
        response = p2pd_pb2.Response()
        await read_pbmsg_safe(reader, response)
        writer.close()
        server.close()
        await server.wait_closed()
        return await arrived.get(), response

    request, response = run(over_a_socket())
    assert request == messages[1]
    raise_if_failed(response)
    assert PeerID(response.identify.id).to_base58() == PEER_TEXT and Multiaddr(response.identify.addrs[0]) == ADDR


def test_error_responses_become_control_failures():
    raise_if_failed(p2pd_pb2.Response(type=p2pd_pb2.Response.OK))
    with pytest.raises(ControlFailure, match="no route") as failure:
        raise_if_failed(p2pd_pb2.Response(type=p2pd_pb2.Response.ERROR, error=p2pd_pb2.ErrorResponse(msg="no route")))
    assert isinstance(failure.value, P2PDaemonError)


def test_peer_ids_and_infos_convert_to_and_from_messages():
    peer_id = PeerID.from_base58(PEER_TEXT)
    assert PEER_BYTES[:2] == b"\x12\x20" and len(PEER_BYTES) == 34
    assert peer_id.to_bytes() == PEER_BYTES and peer_id.to_string() == peer_id.pretty() == str(peer_id) == PEER_TEXT
    assert repr(peer_id) == f"<PeerID {PEER_TEXT}>"
    assert peer_id == PeerID(PEER_BYTES) and peer_id == PEER_TEXT and peer_id == PEER_BYTES and peer_id != 1
    assert peer_id != PeerID.from_base58("QmcgpsyWgH8Y8ajJz1Cu72KnS5uo2Aa2LpzU7kinSupNK1")
    assert hash(peer_id) == hash(PeerID(PEER_BYTES)) and len({peer_id, PeerID(PEER_BYTES)}) == 1
    assert sorted([PeerID(b"\x12\x01b"), PeerID(b"\x12\x01a")])[0] == PeerID(b"\x12\x01a")
    with pytest.raises(TypeError):
        peer_id < PEER_TEXT
    import copy
    import pickle
    for twin in (pickle.loads(pickle.dumps(peer_id)), copy.copy(peer_id), copy.deepcopy(peer_id), PeerID(PEER_BYTES)):
        assert twin == peer_id and twin.to_base58() == PEER_TEXT and hash(twin) == hash(peer_id)

    info = PeerInfo(peer_id, [ADDR, Multiaddr("/ip6/::1/udp/9/quic")])
    message = info.to_protobuf()
    assert isinstance(message, p2pd_pb2.PeerInfo) and message.id == PEER_BYTES and len(message.addrs) == 2
    assert PeerInfo.from_protobuf(p2pd_pb2.PeerInfo.FromString(message.SerializeToString())) == info
    assert info != PeerInfo(peer_id, [ADDR]) and "PeerInfo" in repr(info)

    stream_info = StreamInfo(peer_id=peer_id, addr=ADDR, proto="/hivemind/test/1")
    message = stream_info.to_protobuf()
    assert (message.peer, message.addr, message.proto) == (PEER_BYTES, ADDR.to_bytes(), "/hivemind/test/1")
    assert StreamInfo.from_protobuf(message) == stream_info and PEER_TEXT in repr(stream_info)
