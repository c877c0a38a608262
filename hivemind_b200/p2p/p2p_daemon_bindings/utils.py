"""Framing of the libp2p daemon's control protocol and the error types of the bindings
(same names as hivemind/p2p/p2p_daemon_bindings/utils.py:16-87).

A control message is a protobuf (``hivemind_b200.proto.p2pd_pb2``) prefixed with its length as an unsigned varint.
This package's own transport daemon uses a different framing (``hivemind_b200/p2p/control.py``); these helpers serve
code that talks to a libp2p daemon and pin the wire format for both directions.
"""
from __future__ import annotations

import asyncio

from google.protobuf.message import Message as PBMessage

from hivemind_b200.p2p.control import DispatchFailure, P2PDaemonError, P2PHandlerError  # noqa: F401
from hivemind_b200.proto import p2pd_pb2

DEFAULT_MAX_BITS: int = 64


class ControlFailure(P2PDaemonError):
    """The daemon answered a control request with an error."""


async def write_unsigned_varint(stream: asyncio.StreamWriter, integer: int, max_bits: int = DEFAULT_MAX_BITS) -> None:
    """Write ``integer`` in LEB128: seven bits per byte, least significant group first, high bit = "more follows"."""
    if not 0 <= integer < (1 << max_bits):
        raise ValueError(f"{integer} does not fit an unsigned varint of at most {max_bits} bits")
    encoded = bytearray()
    while True:
        low, integer = integer & 0x7F, integer >> 7
        if integer:
            encoded.append(low | 0x80)
        else:
            encoded.append(low)
            break
    stream.write(bytes(encoded))


async def read_unsigned_varint(stream: asyncio.StreamReader, max_bits: int = DEFAULT_MAX_BITS) -> int:
    """Read one LEB128 number; ``ValueError`` if it does not end within ``max_bits`` bits,
    ``asyncio.IncompleteReadError`` if the stream ends first."""
    max_bytes = (max_bits + 6) // 7
    value = 0
    for index in range(max_bytes):
        (byte,) = await stream.readexactly(1)
        value |= (byte & 0x7F) << (7 * index)
        if not byte & 0x80:
            if value >> max_bits:
                break
            return value
    raise ValueError(f"varint overflowed {max_bits} bits")


def raise_if_failed(response: p2pd_pb2.Response) -> None:
    """Turn an ERROR response of the daemon into ``ControlFailure``."""
    if response.type == p2pd_pb2.Response.ERROR:
        raise ControlFailure(f"Connect failed. msg={response.error.msg}")


async def write_pbmsg(stream: asyncio.StreamWriter, pbmsg: PBMessage) -> None:
    """Send one message: varint length, then the serialized bytes."""
    payload = pbmsg.SerializeToString()
    await write_unsigned_varint(stream, len(payload))
    stream.write(payload)


async def read_pbmsg_safe(stream: asyncio.StreamReader, pbmsg: PBMessage) -> None:
    """Receive one message into ``pbmsg`` (its previous content is replaced)."""
    length = await read_unsigned_varint(stream)
    pbmsg.ParseFromString(await stream.readexactly(length))
